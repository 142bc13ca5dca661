"""Small Zasorax configurations for the tests.  They differ from one another in every size and option: the order of the
two kinds of layer, head counts (query heads that share key heads two, three and four to one, and one to one), key and
value sizes that differ, are odd multiples and are no power of two (and 64 and 128 both, which the tensor-core kernels
take), chunks of 1, shorter than a page, a page exactly, a page and one and several pages, distance tables of 2 to 16 rows
(odd counts too) that end before, at and beyond the chunk, layers that read an earlier layer's keys and values with a
shorter and with a longer chunk than that layer's own, rotation over all of a head and over part of it, dense, routed and
no feed-forward, routers that choose one expert, some and all, an embedding constant that is 1 and that is not, widths
that are no power of two.  The two configurations that the tensor-core attention takes route every token to all of their
experts: no rounding can change a choice there, so their bfloat16 logits are checked at every position (see the helpers'
rule for the others)."""


def _chunked(heads, kv_heads, dim, vdim, scale, chunk, far, rows, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "bias_max": far, "mask": {"size": chunk},
         "bias_rows": rows}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _turned(heads, kv_heads, dim, vdim, scale, dims, base, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": {"base": base, "dims": dims}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(ff, experts, top):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def _layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


ZAS_A = {
    "architecture": "Zasorax", "vocab": 300, "width": 88, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.0},
    "layers": [
        _layer("attention", _chunked(6, 2, 16, 24, 0.3, chunk=17, far=40, rows=10), _dense(120)),
        _layer("attention_2", _turned(4, 1, 24, 16, 0.22, dims=16, base=100.0), _moe(32, 6, 2)),
        _layer("attention", _chunked(6, 2, 16, 24, 0.4, chunk=33, far=50.5, rows=12, kv_from=0), None),
        _layer("attention_2", _turned(2, 2, 40, 8, 0.15, dims=40, base=5000.0), _moe(24, 3, 1)),
    ],
}

# keys and values of 64: the tensor-core attention in bfloat16; a chunk of a page exactly
ZAS_B = {
    "architecture": "Zasorax", "vocab": 257, "width": 64, "norm": {"eps": 1e-6},
    "layers": [
        _layer("attention_2", _turned(4, 4, 64, 64, 0.125, dims=32, base=10000.0), _dense(96)),
        _layer("attention", _chunked(4, 2, 64, 64, 0.11, chunk=64, far=64, rows=16), _moe(40, 4, 4)),
        _layer("attention", _chunked(4, 2, 64, 64, 0.09, chunk=40, far=30, rows=8, kv_from=1), _dense(72)),
        _layer("attention_2", _turned(4, 4, 64, 64, 0.1, dims=32, base=10000.0, kv_from=0), None),
    ],
}

# keys and values of 128; a chunk of a page and one; a table with an odd number of rows that widens beyond the chunk
ZAS_C = {
    "architecture": "Zasorax", "vocab": 190, "width": 96, "norm": {"eps": 1e-5}, "embedding": {"scale": 0.5},
    "layers": [
        _layer("attention", _chunked(2, 1, 128, 128, 0.07, chunk=65, far=200, rows=7), _moe(48, 2, 2)),
        _layer("attention_2", _turned(3, 1, 128, 128, 0.09, dims=128, base=1.0e6), _dense(80)),
        _layer("attention", _chunked(4, 1, 128, 128, 0.06, chunk=150, far=90, rows=16, kv_from=0), _moe(16, 3, 3)),
    ],
}

# a chunk of one position (a token sees itself and the sink only), a table of two rows, sizes that are no multiple of 8 or 4
ZAS_D = {
    "architecture": "Zasorax", "vocab": 120, "width": 40, "norm": {"eps": 1e-4}, "embedding": {"scale": 6.3},
    "layers": [
        _layer("attention", _chunked(3, 3, 12, 10, 0.5, chunk=1, far=3, rows=2), None),
        _layer("attention", _chunked(2, 1, 20, 6, 0.35, chunk=200, far=128, rows=9), _dense(56)),
        _layer("attention_2", _turned(5, 5, 10, 14, 0.4, dims=6, base=37.0), _moe(8, 7, 3)),
        _layer("attention", _chunked(4, 1, 20, 6, 0.3, chunk=5, far=6, rows=5, kv_from=1), _dense(24)),
        # a reader whose own row (5 query heads of 10 and 5 gates) is narrower than the keys and values it reads
        _layer("attention_2", _turned(5, 5, 10, 14, 0.25, dims=6, base=37.0, kv_from=2), None),
    ],
}

ZAS_CONFIGS = {"zas_a": ZAS_A, "zas_b": ZAS_B, "zas_c": ZAS_C, "zas_d": ZAS_D}
