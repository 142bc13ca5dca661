"""Zasorax without a GPU: the configuration and its errors, the plan's tensors, cache requests and shared storage, the
rows of the distance table, the cache's pages under a chunk that a reader looks further back than, and the plain
implementation's own mechanisms on cases small enough to work out by hand."""

import copy
import math

import pytest
import torch

from tests.plain import zasorax as plain
from tests.zasorax_configs import ZAS_A, ZAS_B, ZAS_C, ZAS_CONFIGS, ZAS_D


def _model(raw, dtype=torch.float32):
    from gtar_kimik3_public_b200.models.model import Model
    from gtar_kimik3_public_b200.registry import architecture, config_from_dict

    config = config_from_dict(raw)
    return Model(architecture("Zasorax").build_plan(config), config, dtype, "cpu")


@pytest.mark.parametrize("tag", sorted(ZAS_CONFIGS))
def test_configurations_are_read_and_give_their_tensors(tag):
    raw = ZAS_CONFIGS[tag]
    W = raw["width"]
    model = _model(raw)
    specs = model.tensor_specs()
    assert specs["embed"].shape == (raw["vocab"], W) and specs["head"].shape == (raw["vocab"], W)
    assert specs["final.norm"].shape == (W,)
    for i, layer in enumerate(raw["layers"]):
        m = layer["mixer"]
        own = m.get("kv_from") is None
        assert specs[f"l{i}.norm1"].shape == (W,)
        assert specs[f"l{i}.mix.q"].shape == (m["heads"] * m["dim"], W)
        assert specs[f"l{i}.mix.o"].shape == (W, m["heads"] * m["vdim"])
        assert (f"l{i}.mix.k" in specs) == own and (f"l{i}.mix.v" in specs) == own
        if own:
            assert specs[f"l{i}.mix.k"].shape == (m["kv_heads"] * m["dim"], W)
            assert specs[f"l{i}.mix.v"].shape == (m["kv_heads"] * m["vdim"], W)
        if layer["type"] == "attention":
            assert specs[f"l{i}.mix.q.norm"].shape == (m["heads"] * m["dim"],)
            assert (f"l{i}.mix.k.norm" in specs) == own
            assert specs[f"l{i}.mix.rel"].shape == (m["bias_rows"], m["heads"]) and specs[f"l{i}.mix.rel"].free == (0,)
            assert specs[f"l{i}.mix.temp"].shape == (m["heads"],) and specs[f"l{i}.mix.sink"].shape == (m["heads"],)
            assert f"l{i}.mix.g" not in specs
        else:
            assert specs[f"l{i}.mix.g"].shape == (m["heads"], W)
            assert not any(f"l{i}.mix.{name}" in specs for name in ("q.norm", "k.norm", "rel", "temp", "sink"))
        mlp = layer["mlp"]
        if mlp is None:
            assert not any(name.startswith(f"l{i}.mlp.") or name == f"l{i}.norm2" for name in specs)
        elif mlp["kind"] == "dense":
            assert specs[f"l{i}.mlp.up"].shape == (mlp["ff"], W) and specs[f"l{i}.mlp.down"].shape == (W, mlp["ff"])
            assert specs[f"l{i}.mlp.act"].shape == (2,) and specs[f"l{i}.norm2"].shape == (W,)
        else:
            n, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
            assert specs[f"l{i}.mlp.router"].shape == (n, W) and specs[f"l{i}.mlp.router.b"].shape == (n,)
            assert specs[f"l{i}.mlp.e{n - 1}.gate"].shape == (ff, W) and specs[f"l{i}.mlp.e0.down"].shape == (W, ff)
            assert f"l{i}.mlp.e{n}.up" not in specs
    assert model.graph_safe()


def test_cache_requests_and_shared_storage():
    from gtar_kimik3_public_b200.parts.base import KVRequest

    layout = _model(ZAS_A).cache_layout()
    # the owner's pages reach as far back as its furthest reader looks (33), not only as far as its own chunk (17)
    assert layout.requests[0] == KVRequest(2, 16, 33, value_dim=24)
    assert layout.requests[1] == KVRequest(1, 24, None, value_dim=16)
    assert layout.shared_with == {2: 0}
    layout = _model(ZAS_B).cache_layout()
    assert layout.shared_with == {2: 1, 3: 0}
    assert layout.requests[1] == KVRequest(2, 64, 64) and layout.requests[0] == KVRequest(4, 64, None)
    layout = _model(ZAS_D).cache_layout()
    assert layout.requests[0] == KVRequest(3, 12, 1, value_dim=10) and layout.requests[1] == KVRequest(1, 20, 200, value_dim=6)


def test_layers_with_equal_rotations_share_a_table():
    plan = _model(ZAS_B).plan
    # q/k over 32 entries and values over 64, both of base 10000, shared by the two layers that have them
    assert len(plan.positions) == 2
    assert plan.layers[0].mixer.position is plan.layers[3].mixer.position
    assert plan.layers[0].mixer.value_position is plan.layers[3].mixer.value_position
    assert len(_model(ZAS_A).plan.positions) == 3  # one layer turns its values as it turns 16 entries of its keys


@pytest.mark.parametrize("rows,far", [(10, 40), (12, 50.5), (16, 64), (8, 30), (7, 200), (2, 3), (9, 128), (5, 6), (32, 4096)])
def test_distance_rows_follow_the_rule(rows, far):
    from gtar_kimik3_public_b200.parts.scored_attention import distance_rows

    got = distance_rows(rows, far)
    assert got == [plain.distance_bucket(n, rows, far) for n in range(len(got))]
    assert got[-1] == rows - 1 and len(got) == math.ceil(far) + 1
    assert all(plain.distance_bucket(n, rows, far) == rows - 1 for n in (len(got), 3 * len(got), 10**6))
    assert got[:rows // 2] == list(range(rows // 2)) and all(b >= a for a, b in zip(got, got[1:]))


def _changed(path, value):
    raw = copy.deepcopy(ZAS_A)
    at = raw
    for key in path[:-1]:
        at = at[key]
    if value is KeyError:
        del at[path[-1]]
    else:
        at[path[-1]] = value
    return raw


@pytest.mark.parametrize("change,message", [
    ((("layers", 0, "type"), "lightning"), "not a mixer"),
    ((("layers", 0, "mixer", "mask"), {}), "missing keys ['size']"),
    ((("layers", 0, "mixer", "bias_max"), 0), "bias_max"),
    ((("layers", 1, "mixer", "rot"), KeyError), "missing keys ['rot']"),
    ((("layers", 1, "mixer", "rot", "dims"), 26), "rot.dims"),
    ((("layers", 1, "mixer", "vdim"), 15), "vdim"),
    ((("layers", 1, "mixer", "window"), 4), "unknown keys ['window']"),
    ((("layers", 0, "mixer", "heads"), 5), "multiple of kv_heads"),
    ((("layers", 2, "mixer", "kv_from"), 2), "earlier layer"),
    ((("layers", 2, "mixer", "kv_from"), 1), "must be that layer's"),
    ((("layers", 2, "mixer", "vdim"), 16), "must be that layer's"),
    ((("layers", 0, "mlp", "kind"), "swiglu"), "mlp.kind"),
    ((("layers", 1, "mlp", "router", "top"), 7), "cannot be chosen"),
    ((("norm",), {}), "missing keys ['eps']"),
    ((("depth",), 3), "unknown keys ['depth']"),
])
def test_configuration_errors_name_the_key(change, message):
    from gtar_kimik3_public_b200.config.base import ConfigError
    from gtar_kimik3_public_b200.registry import config_from_dict

    with pytest.raises(ConfigError) as caught:
        config_from_dict(_changed(*change))
    assert message in str(caught.value)


def test_a_layer_without_chunks_sees_everything_and_keeps_every_page():
    raw = copy.deepcopy(ZAS_A)
    del raw["layers"][2]["mixer"]["mask"]  # the reader of layer 0's pages
    model = _model(raw)
    assert model.plan.layers[2].mixer.chunk is None and model.plan.layers[0].mixer.chunk == 17
    assert model.cache_layout().requests[0].window is None, "the owner must keep what its reader may look back at"


def test_a_reader_of_a_reader_is_refused():
    from gtar_kimik3_public_b200.config.base import ConfigError
    from gtar_kimik3_public_b200.registry import config_from_dict

    raw = copy.deepcopy(ZAS_A)
    raw["layers"].append(copy.deepcopy(raw["layers"][2]))
    raw["layers"][4]["mixer"]["kv_from"] = 2
    with pytest.raises(ConfigError, match="no keys and values of its own"):
        config_from_dict(raw)


def test_a_configuration_survives_its_own_file(tmp_path):
    import json

    from gtar_kimik3_public_b200.registry import config_from_dict, config_from_file

    config = config_from_dict(ZAS_C)
    (tmp_path / "config.json").write_text(json.dumps(config.to_dict()))
    again = config_from_file(tmp_path)
    assert again == config and again.embedding_scale == 0.5 and config_from_dict(ZAS_B).embedding_scale == 1.0


def test_a_file_without_row_counts_loads_tables_of_any_height(tmp_path):
    """The rows of a distance table are the tensor's: a config that does not name them still takes the file."""
    from gtar_kimik3_public_b200.registry import config_from_dict
    from gtar_kimik3_public_b200.weights.loader import check_tensors

    raw = copy.deepcopy(ZAS_D)
    for layer in raw["layers"]:
        layer["mixer"].pop("bias_rows", None)
    specs = _model(raw).tensor_specs()
    have = {name: tuple(spec.shape) for name, spec in specs.items()}
    have["l1.mix.rel"] = (9, 2)
    check_tensors(tmp_path, specs, have, {})
    have["l1.mix.rel"] = (9, 3)
    from gtar_kimik3_public_b200.weights.loader import WeightsError

    with pytest.raises(WeightsError):
        check_tensors(tmp_path, specs, have, {})


def test_pages_behind_every_readers_chunk_go_back_to_the_pool():
    """Layer 0 of the first configuration owns pages that a later layer reads 33 positions back: a page returns to the
    pool only when it lies wholly behind that, and a sequence that ends returns all."""
    from gtar_kimik3_public_b200.cache import Cache

    cache = Cache(_model(ZAS_A).cache_layout(), 64 * 12, torch.float32, "cpu", max_seqs=2)
    chunked = next(g for g in cache.kv_groups if g.request.window == 33)
    slot = cache.open()
    cache.grow(slot, 130)  # pages 0, 1, 2
    assert sorted(chunked.owned[slot]) == [0, 1, 2]
    cache.grow(slot, 1)  # position 130 is read from 98 on: page 0 (positions 0..63) has left
    assert sorted(chunked.owned[slot]) == [1, 2]
    cache.grow(slot, 30)  # the step's first position, 131, is read from 99 on: page 1 (64..127) stays for this step
    assert sorted(chunked.owned[slot]) == [1, 2]
    cache.grow(slot, 1)  # position 161 is read from 129 on: page 1 has left
    assert sorted(chunked.owned[slot]) == [2]
    cache.check_invariants()
    cache.close(slot)
    assert chunked.pages.n_used == 0


# ------------------------------------------------------------------ the plain implementation by hand
def test_plain_softmax_with_sink_by_hand():
    s = torch.tensor([[0.0, 1.0, 5.0]], dtype=torch.float64)
    seen = torch.tensor([[True, True, False]])
    got = plain.softmax_with_sink(s, seen, math.log(2.0))
    denom = 2.0 + 1.0 + math.e
    assert torch.allclose(got, torch.tensor([[1.0 / denom, math.e / denom, 0.0]], dtype=torch.float64))
    # a sink far above every score takes nearly all the weight; far below, the rows sum to one
    assert plain.softmax_with_sink(s, seen, 50.0).sum().item() < 1e-20
    assert abs(plain.softmax_with_sink(s, seen, -50.0).sum().item() - 1.0) < 1e-12


def test_plain_distance_bucket_by_hand():
    # 8 rows up to distance 64: rows 0..3 one distance each, then ln(n / 4) / ln(16) * 4 rows further
    assert [plain.distance_bucket(n, 8, 64) for n in (0, 3, 4, 7, 8, 15, 16, 31, 32, 63, 64, 1000)] == [0, 3, 4, 4, 5, 5, 6, 6, 7, 7, 7, 7]


def test_plain_rotation_and_its_way_back():
    x = torch.randn(9, 2, 10, dtype=torch.float64, generator=torch.Generator().manual_seed(1))
    there = plain.turn(x, 6, 37.0)
    assert torch.equal(there[..., 6:], x[..., 6:]) and torch.equal(there[0], x[0])
    assert torch.allclose(plain.turn(there, 6, 37.0, backwards=True), x, atol=1e-12)
    a = 4 * 37.0 ** (-2.0 / 6)  # position 4, pair 1 (entries 1 and 4)
    assert math.isclose(there[4, 0, 1].item(), x[4, 0, 1].item() * math.cos(a) - x[4, 0, 4].item() * math.sin(a), abs_tol=1e-12)
    assert math.isclose(there[4, 0, 4].item(), x[4, 0, 4].item() * math.cos(a) + x[4, 0, 1].item() * math.sin(a), abs_tol=1e-12)


def test_plain_activation_by_hand():
    numbers = torch.tensor([0.3, -0.2], dtype=torch.float64)
    up, down = math.log1p(math.exp(0.3)), 0.5 + math.log1p(math.exp(-0.2))
    z = torch.tensor([2.0, 0.0, -1.5], dtype=torch.float64)
    want = [up * 4.0 + 1.0, 0.0, down * (math.exp(-1.5) - 1.0 + 1.5) - 0.75]
    assert torch.allclose(plain.xielu(z, numbers), torch.tensor(want, dtype=torch.float64), atol=1e-12)


def test_plain_router_by_hand():
    h = torch.tensor([[1.0, 0.0], [0.0, 1.0]], dtype=torch.float64)
    w = {"r.router": torch.tensor([[2.0, 0.0], [1.0, 3.0], [0.0, 1.0]], dtype=torch.float64), "r.router.b": torch.tensor([0.0, 0.5, 2.5], dtype=torch.float64)}
    for e in range(3):  # expert e multiplies its input by e + 1: gate so large that silu(g) = g, up = 1 / g ... kept linear by hand below
        w[f"r.e{e}.gate"] = torch.eye(2, dtype=torch.float64) * 50.0
        w[f"r.e{e}.up"] = torch.eye(2, dtype=torch.float64) / 50.0
        w[f"r.e{e}.down"] = torch.eye(2, dtype=torch.float64) * (e + 1)
    got = plain.routed_ff(h, w, "r.", {"router": {"experts": 3, "top": 2}})
    # token 0: logits 2, 1.5, 2.5 -> experts 2 and 0 with softmax(2.5, 2); token 1: 0, 3.5, 3.5 -> experts 1 and 2, equal shares
    a = math.exp(2.5) / (math.exp(2.5) + math.exp(2.0))
    assert math.isclose(got[0, 0].item(), a * 3 + (1 - a) * 1, rel_tol=1e-9)
    assert math.isclose(got[1, 1].item(), 0.5 * 2 + 0.5 * 3, rel_tol=1e-9)
