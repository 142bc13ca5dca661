"""Rezulorn without a GPU: the configuration and its errors, the plan's tensors and cache requests, the cache's pages
under a window that keeps the first tokens, and the plain implementation's own mechanisms on cases small enough to work
out by hand."""

import copy
import math

import pytest
import torch

from tests.plain import rezulorn as plain
from tests.rezulorn_configs import REZ_A, REZ_B, REZ_C, REZ_CONFIGS, REZ_D


def _model(raw, dtype=torch.float32):
    from gtar_kimik3_public_b200.models.model import Model
    from gtar_kimik3_public_b200.registry import architecture, config_from_dict

    config = config_from_dict(raw)
    return Model(architecture("Rezulorn").build_plan(config), config, dtype, "cpu")


@pytest.mark.parametrize("tag", sorted(REZ_CONFIGS))
def test_configurations_are_read_and_give_their_tensors(tag):
    raw = REZ_CONFIGS[tag]
    W = raw["width"]
    model = _model(raw)
    specs = model.tensor_specs()
    assert specs["embed"].shape == (raw["vocab"], W) and specs["head"].shape == (raw["vocab"], W)
    assert specs["final.norm"].shape == (W,)
    taps = (raw.get("canon") or {}).get("taps", 0)
    for i, layer in enumerate(raw["layers"]):
        m = layer["mixer"]
        assert specs[f"l{i}.norm1"].shape == (W,)
        assert (f"l{i}.canon1" in specs) == bool(taps)
        if taps:
            assert specs[f"l{i}.canon1"].shape == (W, taps)
        if layer["type"] == "lightning":
            assert specs[f"l{i}.mix.k"].shape == (m["heads"] * m["dim"], W)
            assert specs[f"l{i}.mix.g"].shape == (m["heads"] * m["vdim"], W)
            assert specs[f"l{i}.mix.norm"].shape == (m["heads"] * m["vdim"],)
        elif layer["type"] == "attention":
            assert specs[f"l{i}.mix.q"].shape == (m["heads"] * m["dim"], W)
            assert specs[f"l{i}.mix.v"].shape == (m["kv_heads"] * m["vdim"], W)
            assert specs[f"l{i}.mix.o"].shape == (W, m["heads"] * m["vdim"])
            assert specs[f"l{i}.mix.r1"].shape == (m["heads"],) and specs[f"l{i}.mix.r2"].shape == (m["heads"],)
            assert f"l{i}.mix.pb" not in specs
        else:
            left, right = m["left"], m["right"]
            assert specs[f"l{i}.mix.left.k"].shape == (left["kv_heads"] * left["dim"], W)
            assert specs[f"l{i}.mix.left.pb"].shape == (left["heads"],)
            assert f"l{i}.mix.left.r1" not in specs and f"l{i}.mix.right.norm" not in specs
            assert specs[f"l{i}.mix.right.g"].shape == (right["heads"] * right["vdim"], W)
            assert specs[f"l{i}.mix.right.o"].shape == (W, right["heads"] * right["vdim"])
        if layer["mlp"] is None:
            assert not any(name.startswith(f"l{i}.mlp.") or name in (f"l{i}.norm2", f"l{i}.canon2") for name in specs)
        else:
            assert specs[f"l{i}.mlp.up"].shape == (layer["mlp"]["ff"], W)
            assert specs[f"l{i}.mlp.down"].shape == (W, layer["mlp"]["ff"])
            assert (f"l{i}.canon2" in specs) == bool(taps)
    assert model.graph_safe()


def test_cache_requests_follow_the_layers():
    from gtar_kimik3_public_b200.parts.base import KVRequest, StateRequest

    conv = StateRequest((3, 88), torch.float32)
    requests = _model(REZ_A).cache_layout().requests
    assert requests[0] == [StateRequest((3, 24, 40), torch.float32), conv, conv]
    assert requests[1] == [KVRequest(2, 16, 17, value_dim=24, keep_first=3), conv, conv]
    assert requests[2] == [KVRequest(1, 24, None, value_dim=16), StateRequest((2, 40, 24), torch.float32), conv]
    assert requests[3] == [KVRequest(2, 40, 70, value_dim=8), conv, conv]
    # no convolutions, or one tap: nothing kept beside the mixer's own
    assert _model(REZ_C).cache_layout().requests[1] == StateRequest((2, 64, 128), torch.float32)
    assert _model(REZ_D).cache_layout().requests[0] == StateRequest((1, 16, 48), torch.float32)
    assert _model(REZ_B).cache_layout().requests[3] == [KVRequest(1, 24, None, value_dim=40), StateRequest((1, 72), torch.float32),
                                                        StateRequest((1, 72), torch.float32)]


def test_layers_with_equal_rotations_share_a_table():
    raw = copy.deepcopy(REZ_A)
    raw["layers"].append(copy.deepcopy(raw["layers"][2]))
    raw["layers"][4]["mixer"]["right"]["rot"]["base"] = 7.0
    plan = _model(raw).plan
    assert len(plan.positions) == 3
    assert plan.layers[2].mixer.left.position is plan.layers[4].mixer.left.position
    assert plan.layers[2].mixer.right.position is not plan.layers[4].mixer.right.position


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].update(type="rnn"), "not a mixer"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=4), "multiple of kv_heads"),
    (lambda c: c["layers"][2]["mixer"]["left"]["rot"].update(dims=26), "rot.dims"),
    (lambda c: c["layers"][2]["mixer"]["left"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"].update(decay=[0.5, 0.9]), "one number per head"),
    (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "not a feed-forward"),
    (lambda c: c["layers"][0]["mixer"].pop("vdim"), "missing keys"),
    (lambda c: c["layers"][2]["mixer"].pop("right"), "missing keys"),
    (lambda c: c["layers"][1]["mixer"].update(bias=True), "unknown keys"),
    (lambda c: c["layers"][1]["mixer"]["mask"].update(size=0), "mask.size"),
    (lambda c: c["norm"].pop("eps"), "missing keys"),
    (lambda c: c.update(width=0), "width"),
    (lambda c: c["canon"].update(taps=-1), "canon.taps"),
])
def test_configuration_errors_name_the_key(change, message):
    from gtar_kimik3_public_b200.config.base import ConfigError
    from gtar_kimik3_public_b200.registry import config_from_dict

    raw = copy.deepcopy(REZ_A)
    change(raw)
    with pytest.raises(ConfigError, match=message):
        config_from_dict(raw)


def test_a_configuration_survives_its_own_file(tmp_path):
    """What the random-weights mode writes as config.json reads back as the same configuration."""
    import json

    from gtar_kimik3_public_b200.registry import config_from_dict

    for raw in REZ_CONFIGS.values():
        config = config_from_dict(raw)
        again = config_from_dict(json.loads(json.dumps(config.to_dict())))
        assert again == config and again.taps == (raw.get("canon") or {}).get("taps", 0)


def test_pages_of_kept_first_tokens_stay_when_the_window_leaves_them():
    """A window of 17 with 3 kept first tokens in pages of 64: while a sequence grows to five pages, the page of the
    first tokens and the pages that the window touches stay, the ones between go back to the pool."""
    from gtar_kimik3_public_b200.cache import Cache

    model = _model(REZ_A)
    cache = Cache(model.cache_layout(), max_tokens=640, max_seqs=2, dtype=torch.float32, device="cpu")
    group = next(g for g in cache.kv_groups if g.request.window == 17)
    slot = cache.open()
    length = 0
    for step in (100, 1, 1, 90, 1, 60, 1, 130):
        cache.grow(slot, step)
        length += step
        owned = sorted(group.owned[slot])
        assert 0 in owned, f"the kept first tokens' page was given back at length {length}"
        assert (length - 1) // 64 in owned
        cache.check_invariants()
    assert sorted(group.owned[slot]) == [0, 3, 4, 5]  # the last step read from position 238 on and wrote up to 383
    cache.grow(slot, 1)
    assert sorted(group.owned[slot]) == [0, 5, 6]
    cache.close(slot)
    assert group.pages.n_used == 0


def test_plain_decayed_sum_by_hand():
    """d = 1, dv = 1: S_t = g S + k v, o = S q."""
    q = torch.tensor([[1.0], [2.0], [-1.0]], dtype=torch.float64)
    k = torch.tensor([[1.0], [0.5], [2.0]], dtype=torch.float64)
    v = torch.tensor([[3.0], [-1.0], [0.25]], dtype=torch.float64)
    s1 = 3.0
    s2 = 0.5 * s1 - 0.5
    s3 = 0.5 * s2 + 0.5
    out = plain.decayed_sum(q, k, v, 0.5)
    assert torch.allclose(out, torch.tensor([[s1], [2.0 * s2], [-s3]], dtype=torch.float64))
    # the closed form: o_t = sum_{j <= t} g^(t - j) (q_t . k_j) v_j
    gen = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(9, n, generator=gen, dtype=torch.float64) for n in (5, 5, 3))
    want = torch.stack([sum(0.8 ** (t - j) * (q[t] @ k[j]) * v[j] for j in range(t + 1)) for t in range(9)])
    assert torch.allclose(plain.decayed_sum(q, k, v, 0.8), want, atol=1e-12)


def test_plain_window_keeps_the_first_tokens():
    seen = plain.visible(8, {"size": 3, "keep_first": 2})
    assert seen[7].tolist() == [True, True, False, False, False, True, True, True]
    assert seen[3].tolist() == [True, True, True, True, False, False, False, False]
    assert plain.visible(4, None).tolist() == torch.ones(4, 4).tril().bool().tolist()
    assert plain.visible(5, {"size": 2})[4].tolist() == [False, False, False, True, True]


def test_plain_distance_term_and_softmax_by_hand():
    """One head, keys that are all equal: the weights are the softmax of the distance term alone."""
    T, d = 5, 4
    q = torch.ones(T, 1, d, dtype=torch.float64)
    k = torch.ones(T, 1, d, dtype=torch.float64)
    v = torch.eye(T, dtype=torch.float64)[:, None, :]
    r1, r2 = torch.tensor([0.7], dtype=torch.float64), torch.tensor([1.5], dtype=torch.float64)
    out = plain.softmax_core(q, k, v, 0.3, {"size": 3, "keep_first": 1}, r1, r2)
    i = 4
    seen = [0, 2, 3, 4]
    e = torch.tensor([(1.0 + 1.5 * (i - j)) ** -0.7 for j in seen], dtype=torch.float64)
    want = torch.zeros(T, dtype=torch.float64)
    want[seen] = e / e.sum()
    assert torch.allclose(out[i, 0], want, atol=1e-12)


def test_plain_sigmoid_weights_do_not_share_a_sum():
    T, d = 4, 2
    q = torch.tensor([[[1.0, 0.0]]] * T, dtype=torch.float64)
    k = torch.tensor([[[2.0, 0.0]], [[-1.0, 5.0]], [[0.0, 0.0]], [[4.0, 1.0]]], dtype=torch.float64)
    v = torch.eye(T, dtype=torch.float64)[:, None, :]
    out = plain.sigmoid_core(q, k, v, 0.5, None, torch.tensor([-1.0], dtype=torch.float64))
    want = torch.tensor([1 / (1 + math.exp(-(0.5 * s - 1.0))) for s in (2.0, -1.0, 0.0, 4.0)], dtype=torch.float64)
    assert torch.allclose(out[3, 0], want, atol=1e-12)
    assert torch.allclose(out[1, 0], torch.cat([want[:2], torch.zeros(2, dtype=torch.float64)]), atol=1e-12)


def test_plain_rotation_by_hand():
    """Entry i turns with entry i + dims/2 by position * base^(-2i/dims) / factor; entries beyond dims pass."""
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0, 5.0, 6.0]]] * 3, dtype=torch.float64)
    out = plain.turn(x, {"base": 100.0, "dims": 4, "scaling": {"factor": 2.0}})
    assert torch.allclose(out[0], x[0])
    for p in (1, 2):
        a0, a1 = p * 1.0 / 2.0, p * 100.0 ** (-0.5) / 2.0
        want = [1.0 * math.cos(a0) - 3.0 * math.sin(a0), 2.0 * math.cos(a1) - 4.0 * math.sin(a1),
                3.0 * math.cos(a0) + 1.0 * math.sin(a0), 4.0 * math.cos(a1) + 2.0 * math.sin(a1), 5.0, 6.0]
        assert torch.allclose(out[p, 0], torch.tensor(want, dtype=torch.float64), atol=1e-12)


def test_plain_convolution_and_norm_by_hand():
    h = torch.tensor([[1.0, 10.0], [2.0, 20.0], [3.0, 30.0], [4.0, 40.0]], dtype=torch.float64)
    w = torch.tensor([[0.5, 0.0, 2.0], [0.0, 1.0, 0.0]], dtype=torch.float64)  # the last tap multiplies the present input
    out = plain.with_time_conv(h, w)
    assert out[:, 0].tolist() == [1.0 + 2.0, 2.0 + 4.0, 3.0 + 6.0 + 0.5, 4.0 + 8.0 + 1.0]
    assert out[:, 1].tolist() == [10.0, 20.0 + 10.0, 30.0 + 20.0, 40.0 + 30.0]
    x = torch.tensor([[1.0, 2.0, 3.0, 6.0]], dtype=torch.float64)
    wn = torch.tensor([1.0, 2.0, 1.0, 0.5], dtype=torch.float64)
    dev = x - 3.0
    want = dev / math.sqrt(float(dev.pow(2).mean()) + 0.1) * wn
    assert torch.allclose(plain.layer_norm(x, wn, 0.1), want, atol=1e-12)
    assert torch.allclose(plain.rms(x, 0.1), x / math.sqrt(12.5 + 0.1), atol=1e-12)
