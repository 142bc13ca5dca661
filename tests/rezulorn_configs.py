"""Small Rezulorn configurations for the tests.  They differ from one another in every size and option: the order of
the three kinds of layer, head counts (query heads that share key heads two, three and four to one, and one to one),
key and value sizes that differ and are no power of two, rotation over all of a head, over part of it and none, with and
without a divisor on the frequencies, windows (1, shorter than a page, a page exactly, a page and one, several pages,
none) with kept first tokens (none, one, fewer and more than a window, more than a page), decays from 0 over weak and
strong to 1, convolutions of 1 to 4 taps and none, layers without feed-forward, constants on the branches and on the
logits that are 1 and that are not, widths that are no power of two."""


def _rot(dims, base=10000.0, factor=None):
    rot = {"base": base, "dims": dims}
    if factor is not None:
        rot["scaling"] = {"factor": factor}
    return rot


def _decayed(heads, dim, vdim, decay, rot=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}
    if rot:
        m["rot"] = rot
    return m


def _scored(heads, kv_heads, dim, vdim, scale, window=None, keep_first=None, rot=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot:
        m["rot"] = rot
    if window:
        m["mask"] = {"size": window}
        if keep_first is not None:
            m["mask"]["keep_first"] = keep_first
    return m


def _pair(left, right, left_scale=None, right_scale=None):
    m = {"left": left, "right": right}
    if left_scale is not None:
        m["left_scale"] = left_scale
    if right_scale is not None:
        m["right_scale"] = right_scale
    return m


def _layer(kind, mixer, ff):
    return {"type": kind, "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


REZ_A = {
    "architecture": "Rezulorn", "vocab": 300, "width": 88, "norm": {"eps": 1e-5}, "canon": {"taps": 4}, "residual_mult": 0.7,
    "logit_scale": 0.4,
    "layers": [
        _layer("lightning", _decayed(3, 24, 40, [0.5, 0.93, 0.999]), 120),
        _layer("attention", _scored(6, 2, 16, 24, 0.3, window=17, keep_first=3), 72),
        _layer("parallel", _pair(_scored(4, 1, 24, 16, 0.22, rot=_rot(16, 100.0, 4.0)),
                                 _decayed(2, 40, 24, [0.97, 0.8], rot=_rot(40, 5000.0)), 0.8, 1.3), None),
        _layer("attention", _scored(2, 2, 40, 8, 0.15, window=70, keep_first=0), 96),
    ],
}

REZ_B = {
    "architecture": "Rezulorn", "vocab": 210, "width": 72, "norm": {"eps": 1e-6}, "canon": {"taps": 2},
    "layers": [
        _layer("parallel", _pair(_scored(3, 3, 8, 24, 0.35, rot=_rot(8, 500000.0)),
                                 _decayed(3, 12, 20, [1.0, 0.0, 0.9], rot=_rot(4, 30.0, 0.5))), 64),
        _layer("attention", _scored(4, 1, 32, 32, 0.18, window=64, keep_first=70), None),
        _layer("lightning", _decayed(5, 8, 8, [0.99, 0.98, 0.6, 0.9995, 0.3]), 40),
        _layer("attention", _scored(3, 1, 24, 40, 0.2), 56),
        _layer("attention", _scored(2, 1, 16, 16, 0.25, window=1, keep_first=1), None),
    ],
}

# No convolutions; windows a page and one and several pages long; more kept first tokens than a page holds.
REZ_C = {
    "architecture": "Rezulorn", "vocab": 256, "width": 128, "norm": {"eps": 1e-6}, "residual_mult": 1.0, "logit_scale": 1.0,
    "layers": [
        _layer("attention", _scored(4, 2, 64, 64, 0.125, window=65, keep_first=66), 160),
        _layer("lightning", _decayed(2, 64, 128, [0.995, 0.9]), 128),
        _layer("parallel", _pair(_scored(2, 1, 128, 64, 0.09, window=130, keep_first=5, rot=_rot(64, 1000.0)),
                                 _decayed(1, 128, 64, [0.98], rot=_rot(128, 10000.0, 8.0)), 1.0, 0.5), 96),
        _layer("attention", _scored(8, 2, 32, 64, 0.2, window=32, keep_first=33), None),
    ],
}

# One tap: the convolution multiplies the present input only and keeps nothing.
REZ_D = {
    "architecture": "Rezulorn", "vocab": 150, "width": 48, "norm": {"eps": 1e-4}, "canon": {"taps": 1}, "residual_mult": 1.5,
    "logit_scale": 2.0,
    "layers": [
        _layer("lightning", _decayed(1, 16, 48, [0.9]), None),
        _layer("parallel", _pair(_scored(2, 2, 16, 8, 0.4), _decayed(4, 4, 12, [0.2, 0.7, 0.95, 0.99]), 2.0, 0.25), 80),
        _layer("lightning", _decayed(2, 132, 20, [0.9, 0.999]), 24),
    ],
}

# Heads of 64 and 128 entries for keys and values alike: what the tensor-core attention takes in bfloat16.
REZ_E = {
    "architecture": "Rezulorn", "vocab": 200, "width": 96, "norm": {"eps": 1e-5}, "canon": {"taps": 3}, "residual_mult": 0.8,
    "logit_scale": 0.5,
    "layers": [
        _layer("parallel", _pair(_scored(2, 1, 128, 128, 0.09, rot=_rot(32, 1000.0, 2.0)),
                                 _decayed(2, 16, 32, [0.9, 0.99], rot=_rot(16, 800.0)), 0.7, 1.1), 64),
        _layer("attention", _scored(4, 2, 64, 64, 0.125, window=40, keep_first=5), None),
        _layer("attention", _scored(3, 3, 128, 128, 0.09, window=100, keep_first=64), 80),
        _layer("attention", _scored(6, 1, 64, 64, 0.125), 48),
    ],
}

# Head sizes that are no multiple of 8 or of 4 (rows of keys and states that start on no 16-byte border), a width that is
# no multiple of 8, five taps, an odd vocabulary.
REZ_F = {
    "architecture": "Rezulorn", "vocab": 131, "width": 52, "norm": {"eps": 1e-5}, "canon": {"taps": 5}, "residual_mult": 0.9,
    "logit_scale": 0.7,
    "layers": [
        _layer("attention", _scored(4, 2, 20, 12, 0.22, window=9, keep_first=2), 44),
        _layer("parallel", _pair(_scored(3, 1, 10, 6, 0.3, rot=_rot(6, 3000.0, 3.0)),
                                 _decayed(2, 6, 10, [0.9, 0.99], rot=_rot(2, 50.0)), 1.1, 0.9), 36),
        _layer("lightning", _decayed(3, 10, 6, [0.8, 0.95, 0.999]), None),
    ],
}

REZ_CONFIGS = {"rez_a": REZ_A, "rez_b": REZ_B, "rez_c": REZ_C, "rez_d": REZ_D, "rez_e": REZ_E, "rez_f": REZ_F}
