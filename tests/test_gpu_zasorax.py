"""The Zasorax decoder in the engine against the plain implementation: whole prompts, prompts then tokens one by
one, portions down to two tokens, unequal batches against each request alone, slots and pages given back and used
again (pages poisoned first), long decoding across chunks and page borders with pages that left every reader's chunk
going back to the pool, layers that read another layer's pages, in float32 and bfloat16, for small configurations that
differ in every size and option; and greedy generation through the library's entry point."""

import pytest
import torch

from tests.helpers import poison
from tests.zasorax_configs import ZAS_CONFIGS
from tests.zasorax_helpers import zas_check, zas_engine, zas_folder, zas_plain_logits, zas_requests

pytestmark = pytest.mark.gpu

TAGS = ("zas_a", "zas_b", "zas_c", "zas_d")
CASES = [(tag, dtype) for tag in TAGS for dtype in ("float32", "bfloat16")]
LENGTHS = [1, 2, 3, 17, 64, 65, 90, 150]


def _entry(request_id, tokens, want):
    from gtar_kimik3_public_b200.engine import StepEntry

    return StepEntry(request_id, tokens, want)


def spoil(engine) -> None:
    """NaN in every page and in the state rows of every slot that is not in use: a slot that is handed out must be
    cleared by the cache, and nothing may read what no step has written."""
    poison(engine)
    for group in engine.cache.state_groups:
        free = [s for s in range(group.state.shape[1]) if not engine.cache.slots.in_use(s)]
        group.state[:, free] = float("nan")


@pytest.mark.parametrize("tag,dtype", CASES)
def test_whole_prompts(tag, dtype):
    engine = zas_engine(tag, dtype, max_tokens=256)
    spoil(engine)
    for r, tokens in enumerate(zas_requests(tag, LENGTHS)):
        places = list(range(len(tokens)))
        logits = engine.step([_entry(r, tokens, places)])
        engine.end([r])
        assert logits.shape == (len(tokens), ZAS_CONFIGS[tag]["vocab"])
        zas_check(tag, dtype, tokens, places, logits, f"{tag} {dtype} request {r} whole")
        engine.cache.check_invariants()
        spoil(engine)
    assert engine.cache.slots.n_used == 0


@pytest.mark.parametrize("tag,dtype", CASES)
def test_prompt_then_tokens_one_by_one(tag, dtype):
    """Decoding runs past the chunk borders of the configurations and over page borders; in float32 the logits are the
    very numbers of the whole prompt (the 32-bit kernels' order of operations does not depend on the cut)."""
    engine = zas_engine(tag, dtype, max_tokens=512)
    spoil(engine)
    for r, (tokens, head) in enumerate(zip(zas_requests(tag, [150, 100, 40, 230], seed=11), [30, 64, 1, 127])):
        whole = engine.step([_entry(("w", r), tokens, list(range(len(tokens))))])
        engine.end([("w", r)])
        parts = [engine.step([_entry(r, tokens[:head], list(range(head)))])]
        for t in range(head, len(tokens)):
            parts.append(engine.step([_entry(r, [tokens[t]], [0])]))
        engine.end([r])
        stepped = torch.cat(parts)
        zas_check(tag, dtype, tokens, list(range(len(tokens))), stepped, f"{tag} {dtype} request {r} stepped")
        if dtype == "float32":
            assert torch.equal(stepped, whole), f"{tag} request {r}: stepping changed float32 logits"


@pytest.mark.parametrize("tag,dtype", CASES)
@pytest.mark.parametrize("portion", [2, 3, 16, 64, 67])
def test_portions(tag, dtype, portion):
    engine = zas_engine(tag, dtype, max_tokens=256)
    spoil(engine)
    (tokens,) = zas_requests(tag, [141], seed=5)
    parts = []
    for start in range(0, len(tokens), portion):
        piece = tokens[start:start + portion]
        parts.append(engine.step([_entry("p", piece, list(range(len(piece))))]))
    engine.end(["p"])
    zas_check(tag, dtype, tokens, list(range(len(tokens))), torch.cat(parts), f"{tag} {dtype} portions of {portion}")


@pytest.mark.parametrize("tag,dtype", CASES)
def test_unequal_batches_with_slots_used_again(tag, dtype):
    """Requests of unequal lengths start together and are decoded together, the shorter ones ending earlier; then a
    second batch takes the slots, pages and states that the first gave back (all of them poisoned in between)."""
    engine = zas_engine(tag, dtype, max_tokens=640, max_seqs=4)
    for round_, seed in enumerate((3, 4)):
        spoil(engine)
        requests = zas_requests(tag, [1, 70, 140, 33], seed=seed)
        heads = [1, 50, 100, 20]
        got = {i: [] for i in range(4)}
        first = engine.step([_entry((round_, i), requests[i][:heads[i]], list(range(heads[i]))) for i in range(4)])
        at = 0
        for i in range(4):
            got[i].append(first[at:at + heads[i]])
            at += heads[i]
        done = [heads[i] for i in range(4)]
        engine.end([(round_, i) for i in range(4) if done[i] == len(requests[i])])
        while any(done[i] < len(requests[i]) for i in range(4)):
            live = [i for i in range(4) if done[i] < len(requests[i])]
            out = engine.step([_entry((round_, i), [requests[i][done[i]]], [0]) for i in live])
            for row, i in enumerate(live):
                got[i].append(out[row:row + 1])
                done[i] += 1
            engine.end([(round_, i) for i in live if done[i] == len(requests[i])])
            engine.cache.check_invariants()
        for i in range(4):
            zas_check(tag, dtype, requests[i], list(range(len(requests[i]))), torch.cat(got[i]),
                      f"{tag} {dtype} batch {round_} request {i}")
        assert engine.cache.slots.n_used == 0
        assert all(group.pages.n_used == 0 for group in engine.cache.kv_groups)


@pytest.mark.parametrize("tag", TAGS)
def test_batch_equals_alone_in_float32(tag):
    """What a request's logits are does not depend on what else is in the batch: bit-equal in float32."""
    engine = zas_engine(tag, "float32", max_tokens=512, max_seqs=4)
    requests = zas_requests(tag, [80, 9, 131], seed=21)
    alone = []
    for i, tokens in enumerate(requests):
        alone.append(engine.step([_entry(("a", i), tokens, list(range(len(tokens))))]))
        engine.end([("a", i)])
    together = engine.step([_entry(i, tokens, list(range(len(tokens)))) for i, tokens in enumerate(requests)])
    assert torch.equal(together, torch.cat(alone))


@pytest.mark.parametrize("tag,dtype", [("zas_a", "bfloat16"), ("zas_b", "float32"), ("zas_b", "bfloat16"), ("zas_c", "bfloat16"), ("zas_d", "float32")])
def test_graph_replay_matches_launches(tag, dtype):
    """Decode steps replayed from CUDA graphs give what the same steps give launch by launch."""
    (tokens,) = zas_requests(tag, [90], seed=2)
    results = []
    for use_graphs in (True, False):
        engine = zas_engine(tag, dtype, max_tokens=256, use_graphs=use_graphs)
        parts = [engine.step([_entry(0, tokens[:40], [39])])]
        for t in range(40, len(tokens)):
            parts.append(engine.step([_entry(0, [tokens[t]], [0])]))
        results.append(torch.cat(parts))
        engine.check()
    assert torch.equal(results[0], results[1])


@pytest.mark.parametrize("tag,dtype", [("zas_c", "bfloat16"), ("zas_a", "float32"), ("zas_b", "bfloat16"), ("zas_d", "float32")])
def test_long_decoding(tag, dtype):
    """400 tokens one by one from a two-token prompt: every chunk border is crossed by decoded tokens several times, and
    pages that no reader's chunk reaches any more come back into use."""
    engine = zas_engine(tag, dtype, max_tokens=448, max_seqs=1)
    spoil(engine)
    (tokens,) = zas_requests(tag, [402], seed=23)
    parts = [engine.step([_entry(0, tokens[:2], [0, 1])])]
    for t in range(2, len(tokens)):
        parts.append(engine.step([_entry(0, [tokens[t]], [0])]))
    zas_check(tag, dtype, tokens, list(range(len(tokens))), torch.cat(parts), f"{tag} {dtype} long decoding")
    engine.check()


@pytest.mark.parametrize("tag", ["zas_a", "zas_b"])
def test_greedy_generation_through_the_entry_point(tag):
    """``generate`` (scheduler, sampler, cache) in float32 chooses the plain implementation's greedy tokens, for more
    prompts than the batch holds so that slots and states are used again."""
    from gtar_kimik3_public_b200 import generate as g

    model = g.load(zas_folder(tag), dtype="float32")
    prompts = zas_requests(tag, [5, 40, 1, 77, 12], seed=9)
    new = 12
    outputs = g.generate(model, prompts, max_new_tokens=new, temperature=0.0, max_batch=2)
    for prompt, output in zip(prompts, outputs):
        assert len(output) == new
        sequence = list(prompt)
        for token in output:
            logits = zas_plain_logits(tag, sequence, "f64")[-1]
            top = torch.topk(logits, 2).values
            if (top[0] - top[1]).item() > 1e-3:  # a near tie may go either way in 32-bit
                assert int(logits.argmax()) == token, f"{tag}: greedy token differs after {len(sequence)} tokens"
            sequence.append(token)


@pytest.mark.parametrize("tag,dtype", [("zas_a", "float32"), ("zas_c", "bfloat16")])
def test_trace_replay_from_the_command_line(tag, dtype, tmp_path):
    """bin/trace_run chooses the model class by config.json and replays a batch through the engine."""
    import json
    import subprocess
    import sys
    from pathlib import Path

    import numpy as np

    root = Path(__file__).resolve().parents[1]
    vocab = ZAS_CONFIGS[tag]["vocab"]
    a, b = zas_requests(tag, [75, 20], seed=31)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:70], "want": [0, 69]}, {"id": "b", "tokens": b[:18], "want": [17]}],
              "end": []}]
    for i in range(5):
        entries = [{"id": "a", "tokens": [a[70 + i]], "want": [0]}]
        if i < 2:
            entries.append({"id": "b", "tokens": [b[18 + i]], "want": [0]})
        steps.append({"step": i + 1, "entries": entries, "end": (["b"] if i == 1 else []) + (["a"] if i == 4 else [])})
    proc = subprocess.Popen(
        [sys.executable, str(root / "bin" / "trace_run"), "--model", str(zas_folder(tag)), "--dtype", dtype, "--out", str(tmp_path),
         "--max-tokens", "192"], stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, cwd=tmp_path)
    for step in steps:
        proc.stdin.write(json.dumps(step) + "\n")
        proc.stdin.flush()
        assert proc.stdout.readline().strip() == f"done {step['step']}"
    proc.stdin.close()
    assert proc.wait(timeout=120) == 0

    def read(step, n):
        data = np.fromfile(tmp_path / f"{step}.f32", dtype="<f4")
        assert data.size == n * vocab
        return torch.from_numpy(data.reshape(n, vocab))

    first = read(0, 3)
    zas_check(tag, dtype, a, [0, 69], first[:2], "trace step 0, request a")
    zas_check(tag, dtype, b, [17], first[2:], "trace step 0, request b")
    for i in range(5):
        rows = read(i + 1, 2 if i < 2 else 1)
        zas_check(tag, dtype, a, [70 + i], rows[:1], f"trace step {i + 1}, request a")
        if i < 2:
            zas_check(tag, dtype, b, [18 + i], rows[1:], f"trace step {i + 1}, request b")


@pytest.mark.parametrize("tag,dtype", [("zas_c", "bfloat16"), ("zas_b", "float32"), ("zas_a", "float32")])
def test_a_prompt_shape_seen_again_replays_from_a_graph(tag, dtype):
    """A many-token step is captured when its shape comes a second time and replayed from then on: other prompts of the
    same length, in slots and pages that were used before, give the plain implementation's logits each time."""
    engine = zas_engine(tag, dtype, max_tokens=256, max_seqs=2)
    spoil(engine)
    for r, tokens in enumerate(zas_requests(tag, [83, 83, 83, 83], seed=17)):
        logits = engine.step([_entry(r, tokens, [0, 41, 82])])
        engine.end([r])
        zas_check(tag, dtype, tokens, [0, 41, 82], logits, f"{tag} {dtype} prompt {r} of one shape")
        spoil(engine)
    assert engine.graphs is not None and any(key[3] == 83 for key in engine.graphs.graphs)
    engine.check()


def test_command_line_generates_the_greedy_tokens():
    """The generation command line loads the folder by its config.json and prints the plain implementation's greedy tokens."""
    import subprocess
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parents[1]
    (prompt,) = zas_requests("zas_b", [9], seed=13)
    run = subprocess.run(
        [sys.executable, "-m", "gtar_kimik3_public_b200.scripts.generate", "--model", str(zas_folder("zas_b")), "--dtype", "float32",
         "--prompt-ids", ",".join(map(str, prompt)), "--max-new-tokens", "6", "--temperature", "0"],
        capture_output=True, text=True, cwd=root, timeout=300)
    assert run.returncode == 0, run.stderr[-2000:]
    produced = [int(t) for t in run.stdout.strip().splitlines()[0].split(",")]
    assert len(produced) == 6
    sequence = list(prompt)
    for token in produced:
        logits = zas_plain_logits("zas_b", sequence, "f64")[-1]
        top = torch.topk(logits, 2).values
        if (top[0] - top[1]).item() > 1e-3:
            assert int(logits.argmax()) == token
        sequence.append(token)
