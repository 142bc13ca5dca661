"""The Zasorax engine against the plain implementation on configurations and schedules drawn from a seed: two to five
layers of either kind in any order, readers of earlier layers' pages with chunks of their own, head counts, key and value
sizes (64 and 128 among them, which bfloat16 runs take to the tensor cores), chunks from 1 position to several pages,
distance tables of 2 to 33 rows that end before and beyond the chunk, partial and whole rotations with several bases,
dense, routed and no feed-forwards, widths that are no power of two; batches of one to six requests whose prompts end on,
before and after the edges of a cache page, decoded one token a step for 0 to 70 steps (a request that is through leaves
its batch), and a second batch that takes the first one's slots.  Every page starts as NaN.

float32 runs are compared everywhere, within 2e-4 of the float64 oracle.  bfloat16 runs draw routers that choose every
expert (one token sent to another expert would change every later logit by order one, see the helpers of the fixed
configurations) and may err three times as much as the plain implementation with bfloat16 products and storage."""

import math
import random
import tempfile

import pytest
import torch

from tests.plain import zasorax as plain
from tests.plain.weights import read_safetensors

pytestmark = pytest.mark.gpu

LENGTHS = [1, 2, 3, 15, 17, 31, 33, 63, 64, 65, 100, 127, 128, 129, 191, 200, 257, 300]


def drawn_config(rng: random.Random, all_chosen: bool) -> dict:
    width = rng.choice([40, 72, 96, 136, 264])
    layers = []
    for i in range(rng.choice([2, 3, 4, 5])):
        kind = rng.choice(["attention", "attention", "attention_2"])
        earlier = [j for j, other in enumerate(layers) if other["type"] == kind and "kv_from" not in other["mixer"]]
        if earlier and rng.random() < 0.4:
            source = rng.choice(earlier)
            m = {k: layers[source]["mixer"][k] for k in ("kv_heads", "dim", "vdim")}
            m["kv_from"] = source
            if kind == "attention_2":
                m["rot"] = dict(layers[source]["mixer"]["rot"])
        else:
            dim = rng.choice([8, 12, 16, 24, 40, 64, 64, 128])
            vdim = dim if rng.random() < 0.5 else rng.choice([6, 10, 16, 24, 48, 80])
            m = {"kv_heads": rng.choice([1, 2, 3]), "dim": dim, "vdim": vdim}
            if kind == "attention_2":
                m["rot"] = {"base": rng.choice([37.0, 1e4, 2.5e5]), "dims": rng.choice([d for d in (2, 4, 6, 8, 16, 32, 64, 128) if d <= dim])}
        m["heads"] = m["kv_heads"] * rng.choice([1, 2, 4, 5])
        m["scale"] = rng.choice([1.0, 2.0, 0.5]) * m["dim"] ** -0.5
        if kind == "attention":
            m["mask"] = {"size": rng.choice([1, 2, 7, 31, 64, 65, 100, 128, 190, 500])}
            rows = rng.choice([2, 3, 8, 16, 33])
            m["bias_rows"] = rows
            m["bias_max"] = rng.choice([rows // 2 + 1, rows // 2 + 0.5, 20, 64, 120.5, 700])
            if not m["bias_max"] > rows // 2:
                m["bias_max"] = rows
        ff = rng.choice(["dense", "moe", "moe", None])
        if ff == "dense":
            mlp = {"kind": "dense", "ff": rng.choice([24, 56, 200])}
        elif ff == "moe":
            experts = rng.choice([2, 3, 5, 9])
            mlp = {"kind": "moe", "expert": {"ff": rng.choice([8, 24, 40])},
                   "router": {"experts": experts, "top": experts if all_chosen else rng.randrange(1, experts + 1)}}
        else:
            mlp = None
        layers.append({"type": kind, "mixer": m, "mlp": mlp})
    config = {"architecture": "Zasorax", "vocab": rng.choice([100, 257, 1000]), "width": width, "norm": {"eps": rng.choice([1e-6, 1e-5, 3e-4])},
              "layers": layers}
    if rng.random() < 0.7:
        config["embedding"] = {"scale": rng.choice([0.5, 3.0, width ** 0.5])}
    return config


def oracle_and_yardstick(tokens, weights, cfg, with_yardstick):
    ids = torch.tensor(tokens)
    oracle = plain.forward(ids, weights, cfg, torch.float64)
    if not with_yardstick:
        return oracle, 0.0
    plain.LOWP = torch.bfloat16
    try:
        low = plain.forward(ids, weights, cfg, torch.float32).double()
    finally:
        plain.LOWP = None
    return oracle, (low - oracle).abs().max().item()


@pytest.mark.parametrize("seed,dtype", [(s, "float32") for s in (1, 2, 3, 5, 8, 13, 21, 34)] + [(s, "bfloat16") for s in (4, 6, 9, 15, 22, 35, 136)])
def test_drawn_configuration_and_schedule(seed, dtype):
    from gtar_kimik3_public_b200.engine import Engine, StepEntry
    from gtar_kimik3_public_b200.generate import load
    from gtar_kimik3_public_b200.registry import config_from_dict
    from gtar_kimik3_public_b200.weights import write_random_model

    rng = random.Random(seed)
    cfg = drawn_config(rng, all_chosen=dtype == "bfloat16")
    n_req = rng.choice([1, 2, 3, 6])
    batches = [([rng.choice(LENGTHS) for _ in range(n_req)], [rng.choice([0, 1, 2, 5, 33, 70]) for _ in range(n_req)])
               for _ in range(2)]
    room = max(sum(-(-(n + d) // 64) * 64 for n, d in zip(*batch)) for batch in batches)  # one batch at a time
    what = f"seed {seed}: {cfg}, prompts and decoded tokens {batches}"
    with tempfile.TemporaryDirectory(prefix="gtar_test_drawn_") as folder:
        write_random_model(folder, config_from_dict(cfg), seed=seed, std=0.08)
        weights = read_safetensors(folder + "/model.safetensors")
        engine = Engine(load(folder, dtype, "cuda:0"), room, max_seqs=n_req)
        for group in engine.cache.kv_groups:
            group.k.fill_(float("nan"))
            group.v.fill_(float("nan"))
        for number, (prompts, decoded) in enumerate(batches):
            gen = torch.Generator().manual_seed(seed * 10 + number)
            requests = [torch.randint(0, cfg["vocab"], (n + d,), generator=gen).tolist() for n, d in zip(prompts, decoded)]
            checked = [oracle_and_yardstick(tokens, weights, cfg, dtype == "bfloat16") for tokens in requests]
            scale = max(o.abs().max().item() for o, _ in checked)
            limit = 2e-4 * max(1.0, scale) if dtype == "float32" else 3 * max(y for _, y in checked) + 2e-3 + scale / 256
            wants = [sorted({n - 1, rng.randrange(n), rng.randrange(n)}) for n in prompts]
            got = engine.step([StepEntry(i, requests[i][:prompts[i]], wants[i]) for i in range(n_req)]).double().cpu()
            assert torch.isfinite(got).all(), what
            row = 0
            for i in range(n_req):
                for place in wants[i]:
                    err = (got[row] - checked[i][0][place]).abs().max().item()
                    assert err < limit, f"{what}\n{dtype} batch {number} request {i} place {place} of its prompt: {err:.3e} (limit {limit:.3e})"
                    row += 1
            engine.end([i for i in range(n_req) if decoded[i] == 0])
            live = [i for i in range(n_req) if decoded[i] > 0]
            step = 0
            while live:
                got = engine.step([StepEntry(i, [requests[i][prompts[i] + step]], [0]) for i in live]).double().cpu()
                for row, i in enumerate(live):
                    err = (got[row] - checked[i][0][prompts[i] + step]).abs().max().item()
                    assert err < limit, f"{what}\n{dtype} batch {number} request {i} decoded token {step}: {err:.3e} (limit {limit:.3e})"
                step += 1
                engine.end([i for i in live if decoded[i] == step])
                live = [i for i in live if decoded[i] > step]
            engine.cache.check_invariants()
        engine.check()
        assert engine.cache.slots.n_used == 0
