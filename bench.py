"""Benchmark of the library's flagship step: decoding with the Qwen3-0.6B layer sizes.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line.  ``value`` is decoded tokens per second at batch 8 after 2,048-token
prompts (device-timed with CUDA events over exactly K decode steps; a step = the model's
forward for one token of every sequence + the greedy token choice, tokens staying on the
device).  ``e2e`` is the same through the Python entry point with host tokens in and out every
step.  ``prefill`` is one 2,048-token prompt in one step; ``points`` holds decoding at batch 1
and 64; ``roofline`` is the decode step's bytes (every weight once + the live requests' keys and
values) over its time, against the measured copy bandwidth.

Weights are random (written as a model folder by the library's random-weights mode and loaded
from there), token ids are seeded uniform-random: there is no network for checkpoints or data.
The library runs on one GPU; with --gpus N > 1 a line says so and the exit code is 2.

``--compare pofadra`` and ``--compare rezulorn`` do the same for the Pofadra and the Rezulorn decoders; ``--compare zasorax`` puts the Zasorax decoder beside the Rezulorn decoder.  ``--compare dasusun`` runs another workload instead and prints its own JSON line: the Dasusun decoder beside the transformer
at equal layer sizes (prefill and decode throughput of both, and the new design's kernels one by one against their rooflines).
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# BASELINE.json configs[2]: the Qwen3-0.6B layer sizes (the reference's configs/transformer_0.6B.json
# plus the vocabulary its tokenizer gives).
BENCH_CONFIG = {
    "arch": "transformer",
    "vocab_size": 151936,
    "hidden_size": 1024,
    "intermediate_size": 3072,
    "num_hidden_layers": 28,
    "num_attention_heads": 16,
    "num_key_value_heads": 8,
    "head_dim": 128,
    "rms_norm_eps": 1e-6,
    "rope_theta": 1000000.0,
    "tie_word_embeddings": True,
    "initializer_range": 0.02,
    "max_position_embeddings": 4096,
}
PROMPT_LEN = 2048
PREFILL_TOKENS = 2048
# BASELINE.json configs[3] and configs[4]: the Qwen3-4B and Qwen3-8B layer sizes, measured as extra points
LARGE_CONFIGS = {
    "qwen3_4b": {"arch": "transformer", "vocab_size": 151936, "hidden_size": 2560, "intermediate_size": 9728,
                 "num_hidden_layers": 36, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
                 "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "tie_word_embeddings": True, "initializer_range": 0.02,
                 "max_position_embeddings": 8192},
    "qwen3_8b": {"arch": "transformer", "vocab_size": 151936, "hidden_size": 4096, "intermediate_size": 12288,
                 "num_hidden_layers": 36, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
                 "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "tie_word_embeddings": False, "initializer_range": 0.02,
                 "max_position_embeddings": 4096},
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            raw = json.loads(path.read_text())
            out = dict(FALLBACK_PEAKS)
            for key in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
                if isinstance(raw.get(key), (int, float)):
                    out[key] = float(raw[key])
            return out, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, sm_max, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for row in self.rows:
            if len(row) < 7:
                continue
            try:
                sm.append(float(row[0]))
                sm_max.append(float(row[1]))
            except ValueError:
                continue
            for name, cell in zip(names, row[3:7]):
                if cell.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(sm_max) if sm_max else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def step_bytes(batch: int, kv_tokens_each: int, layers: int) -> float:
    """Bytes a decode step has to read, from the sizes alone (both arms print it the same way): every
    bfloat16 matrix once, the 32-bit norm weights, and the live requests' keys and values."""
    c = BENCH_CONFIG
    q_width = c["num_attention_heads"] * c["head_dim"]
    kv_width = c["num_key_value_heads"] * c["head_dim"]
    per_layer = 2 * c["hidden_size"] * (2 * q_width + 2 * kv_width + 3 * c["intermediate_size"])
    per_layer += 4 * (2 * c["hidden_size"] + 2 * c["head_dim"])
    head = 2 * c["vocab_size"] * c["hidden_size"] * (1 if c["tie_word_embeddings"] else 2)
    kv = 2 * 2 * kv_width * layers * kv_tokens_each * batch
    return layers * per_layer + head + 4 * c["hidden_size"] + kv


def config_record(batch: int, layers: int, peak_source: str) -> dict:
    """The ``config`` of the JSON line: every size by name, flat.  Both arms build it here."""
    c = BENCH_CONFIG
    return {
        "model": "transformer (Qwen3-0.6B layer sizes)", "global_batch": batch, "seq_len": PROMPT_LEN,
        "context_length": c["max_position_embeddings"], "parallelism": "single GPU",
        "layers": layers, "layers_full_config": c["num_hidden_layers"], "hidden_size": c["hidden_size"],
        "q_heads": c["num_attention_heads"], "kv_heads": c["num_key_value_heads"], "head_dim": c["head_dim"],
        "intermediate_size": c["intermediate_size"], "vocab_size": c["vocab_size"],
        "tied_embeddings": c["tie_word_embeddings"], "prefill_tokens": PREFILL_TOKENS,
        "l2": "no flush: a step reads %.2f GB, far above the 126 MB L2" % (step_bytes(batch, PROMPT_LEN, layers) / 1e9),
        "peaks": peak_source,
    }


def make_model(dtype: str, layers: int | None = None):
    from gtar_kimik3_public_b200.generate import load
    from gtar_kimik3_public_b200.registry import config_from_dict
    from gtar_kimik3_public_b200.weights import write_random_model

    cfg = dict(BENCH_CONFIG)
    if layers:
        cfg["num_hidden_layers"] = layers
    config = config_from_dict(cfg)
    with tempfile.TemporaryDirectory(prefix="gtar_bench_model_") as folder:
        write_random_model(folder, config, seed=0)
        model = load(folder, dtype, "cuda:0")
    return model, config


def random_prompts(batch: int, length: int, vocab: int, seed: int = 0):
    import torch

    gen = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (batch, length), generator=gen).tolist()


def decode_bytes(model, engine, kv_tokens: int) -> float:
    return model.weight_bytes_per_step() + kv_tokens * engine.cache.kv_bytes_per_token()


def time_decode(model, batch: int, steps: int, warmup: int, sample_clocks: bool = False) -> dict:
    """Device-timed decoding: prompts of PROMPT_LEN in one step, then warm-up and K timed steps."""
    import torch

    from gtar_kimik3_public_b200.cache import rounded_tokens
    from gtar_kimik3_public_b200.engine import Engine, StepEntry
    from gtar_kimik3_public_b200.ops import functional as F
    from gtar_kimik3_public_b200.ops import library

    room = rounded_tokens(PROMPT_LEN + warmup + steps + 1)
    engine = Engine(model, batch * room, max_seqs=batch)
    prompts = random_prompts(batch, PROMPT_LEN, model.vocab_size)
    ids = list(range(batch))
    with torch.no_grad():
        logits = None
        for start in range(0, batch, 8):  # prompts in groups of 8 keep the prefill's activations small
            part = engine.step([StepEntry(i, prompts[i], [PROMPT_LEN - 1]) for i in ids[start:start + 8]])
            logits = part if logits is None else torch.cat([logits, part])
        tokens = F.argmax(logits)
        sampler = ClockSampler() if sample_clocks else None
        if sampler:  # started before the warm-up steps: nvidia-smi needs a moment to deliver its first sample
            sampler.start()
        for _ in range(warmup):
            tokens = F.argmax(engine.decode_on_device(ids, tokens))
        torch.cuda.synchronize()
        launches_before = library.launch_count
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        for _ in range(steps):
            tokens = F.argmax(engine.decode_on_device(ids, tokens))
        end.record()
        torch.cuda.synchronize()
        ms = begin.elapsed_time(end)
        launches = library.launch_count - launches_before
        clocks = sampler.stop() if sampler else None
    kv_tokens = sum(engine.cache.length.values()) - batch * (steps // 2)  # mid-point of the timed region
    result = {
        "tokens_per_s": batch * steps / (ms / 1e3), "ms_per_step": ms / steps, "launches": launches,
        "bytes_per_step": decode_bytes(model, engine, kv_tokens), "clocks": clocks,
    }
    engine.end_all()
    del engine
    torch.cuda.empty_cache()
    return result


def time_e2e(model, batch: int, steps: int, warmup: int) -> dict:
    """The same decode through the Python entry point: host token lists in, host token lists out,
    every step a pinned host-to-device copy of its numbers and a device-to-host read of its tokens."""
    import torch

    from gtar_kimik3_public_b200.cache import rounded_tokens
    from gtar_kimik3_public_b200.generate import Generator

    room = rounded_tokens(PROMPT_LEN + warmup + steps + 2)
    generator = Generator(model, max_tokens=batch * room, max_batch=batch)
    prompts = random_prompts(batch, PROMPT_LEN, model.vocab_size)
    stamps = []

    def on_step(live, tokens):
        stamps.append(time.perf_counter())  # the step's tokens are on the host here

    generator.generate(prompts, max_new_tokens=warmup + steps + 1, temperature=0.0, on_step=on_step)
    torch.cuda.synchronize()
    timed = stamps[warmup:warmup + steps + 1]
    seconds = timed[-1] - timed[0]
    # per step: positions + sequence index + starts + slots + lengths + wanted rows in (the token ids a step
    # chose stay on the device for the next step: the loop runs the device one step ahead of the host),
    # tokens out; a sequence's page-table row follows every 64 steps and is not counted
    h2d = 4 * (5 * batch + 1)
    return {"value": batch * steps / seconds, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * batch}


def time_prefill(model, warmup: int, repeats: int = 7) -> dict:
    import torch

    from gtar_kimik3_public_b200.cache import rounded_tokens
    from gtar_kimik3_public_b200.engine import Engine, StepEntry

    engine = Engine(model, rounded_tokens(PREFILL_TOKENS + 1), max_seqs=1)
    prompt = random_prompts(1, PREFILL_TOKENS, model.vocab_size, seed=1)[0]
    times = []
    with torch.no_grad():
        for i in range(warmup + repeats):
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            begin.record()
            engine.step([StepEntry("p", prompt, [PREFILL_TOKENS - 1])])
            end.record()
            torch.cuda.synchronize()
            engine.end(["p"])
            if i >= warmup:
                times.append(begin.elapsed_time(end))
    ms = statistics.median(times)
    c = model.config
    t = PREFILL_TOKENS
    per_layer = 2 * t * c.hidden_size * ((c.num_attention_heads + 2 * c.num_key_value_heads) * c.head_dim
                                         + c.num_attention_heads * c.head_dim + 3 * c.intermediate_size)
    attention = 4 * c.num_attention_heads * c.head_dim * t * t / 2  # QK^T and PV over the causal half
    flops = len(model.plan.run_list) * (per_layer + attention) + 2 * c.hidden_size * c.vocab_size
    del engine
    torch.cuda.empty_cache()
    return {"value": t / (ms / 1e3), "tokens": t, "ms": ms, "flops": flops}


def prefill_flops(config, layers: int, lengths) -> float:
    """Matrix products of every token, attention over the causal half of each prompt, the head for one row each."""
    c = config
    per_token = 2 * c.hidden_size * ((2 * c.num_attention_heads + 2 * c.num_key_value_heads) * c.head_dim + 3 * c.intermediate_size)
    attention = sum(4 * c.num_attention_heads * c.head_dim * t * t / 2 for t in lengths)
    return layers * (per_token * sum(lengths) + attention) + 2 * c.hidden_size * c.vocab_size * len(lengths)


def time_large(name: str, peak: dict, steps: int, warmup: int) -> dict:
    """The 4B and 8B workloads: weights drawn on the device (a folder of these sizes would take minutes to write
    and read), the whole number of layers.  4B: eight prompts of unequal lengths (uniform in [256, 4096], seeded) in
    one step, then decode steps.  8B: 64 prompts of 1,024 tokens, then decode steps; and one 2,048-token prompt."""
    import random

    import torch

    from gtar_kimik3_public_b200.cache import rounded_tokens
    from gtar_kimik3_public_b200.engine import Engine, StepEntry
    from gtar_kimik3_public_b200.models.model import Model
    from gtar_kimik3_public_b200.ops import functional as F
    from gtar_kimik3_public_b200.registry import architecture, config_from_dict
    from gtar_kimik3_public_b200.weights import load_random_weights

    config = config_from_dict(LARGE_CONFIGS[name])
    model = Model(architecture(config.ARCH_NAMES[0]).build_plan(config), config, torch.bfloat16, "cuda:0")
    load_random_weights(model, seed=0)
    layers = len(model.plan.run_list)
    rng = random.Random(0)
    if name == "qwen3_4b":
        lengths, steps, group = [rng.randint(256, 4096) for _ in range(8)], min(steps, 256), 8
    else:
        lengths, steps, group = [1024] * 64, min(steps, 64), 8
    batch = len(lengths)
    engine = Engine(model, sum(rounded_tokens(n + warmup + steps + 1) for n in lengths), max_seqs=batch)
    gen = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, config.vocab_size, (n,), generator=gen).tolist() for n in lengths]
    ids = list(range(batch))
    out = {}
    with torch.no_grad():
        logits = None
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        begin.record()
        for start in range(0, batch, group):
            part = engine.step([StepEntry(i, prompts[i], [lengths[i] - 1]) for i in ids[start:start + group]])
            logits = part if logits is None else torch.cat([logits, part])
        end.record()
        torch.cuda.synchronize()
        if name == "qwen3_4b":  # the unequal prompts in one step (launched kernel by kernel: a first appearance of its shape)
            ms = begin.elapsed_time(end)
            out[f"{name}_prefill_unequal_tokens_per_s"] = round(sum(lengths) / (ms / 1e3), 1)
            out[f"{name}_prefill_unequal_frac"] = round(prefill_flops(config, layers, lengths) / (ms / 1e3) / (peak["bf16_tflops"] * 1e12), 4)
        tokens = F.argmax(logits)
        for _ in range(warmup):
            tokens = F.argmax(engine.decode_on_device(ids, tokens))
        torch.cuda.synchronize()
        begin.record()
        for _ in range(steps):
            tokens = F.argmax(engine.decode_on_device(ids, tokens))
        end.record()
        torch.cuda.synchronize()
        ms = begin.elapsed_time(end) / steps
        kv_tokens = sum(engine.cache.length.values()) - batch * (steps // 2)
        step_bytes_read = decode_bytes(model, engine, kv_tokens)
        tag = f"{name}_decode_b{batch}" + ("_unequal" if name == "qwen3_4b" else "")
        out[tag] = round(batch / (ms / 1e3), 1)
        out[tag + "_ms"] = round(ms, 4)
        out[tag + "_hbm_frac"] = round(step_bytes_read / (ms / 1e3) / 1e9 / peak["hbm_gbs"], 4)
        engine.end_all()
        del engine
        torch.cuda.empty_cache()
        if name == "qwen3_8b":
            engine = Engine(model, rounded_tokens(PREFILL_TOKENS + 1), max_seqs=1)
            prompt = torch.randint(0, config.vocab_size, (PREFILL_TOKENS,), generator=gen).tolist()
            times = []
            for i in range(8):  # the first is the shape's first appearance; the median of the other seven
                torch.cuda.synchronize()
                begin.record()
                engine.step([StepEntry("p", prompt, [PREFILL_TOKENS - 1])])
                end.record()
                torch.cuda.synchronize()
                engine.end(["p"])
                times.append(begin.elapsed_time(end))
            ms = statistics.median(times[1:])
            out[f"{name}_prefill_{PREFILL_TOKENS}_tokens_per_s"] = round(PREFILL_TOKENS / (ms / 1e3), 1)
            out[f"{name}_prefill_{PREFILL_TOKENS}_frac"] = round(prefill_flops(config, layers, [PREFILL_TOKENS]) / (ms / 1e3) / (peak["bf16_tflops"] * 1e12), 4)
            del engine
    out[f"{name}_layers"] = layers
    del model
    torch.cuda.empty_cache()
    return out


def run_ours(args) -> dict:
    import torch

    from gtar_kimik3_public_b200.ops.library import require_device

    require_device(torch.device("cuda:0"))
    peak, peak_source = peaks()
    model, config = make_model("bfloat16", args.layers)
    layers_run = len(model.plan.run_list)
    batch = args.batch
    main = time_decode(model, batch, args.steps, args.warmup, sample_clocks=True)
    e2e = time_e2e(model, batch, args.steps, args.warmup)
    prefill = time_prefill(model, max(1, min(args.warmup, 3)))
    points = {}
    for b in (1, 64):
        points[f"decode_b{b}"] = round(time_decode(model, b, min(args.steps, 64), args.warmup)["tokens_per_s"], 1)
    del model
    import gc

    gc.collect()
    torch.cuda.empty_cache()
    if not args.no_large:
        for name in LARGE_CONFIGS:
            points.update(time_large(name, peak, args.steps, args.warmup))
    achieved = main["bytes_per_step"] / (main["ms_per_step"] / 1e3) / 1e9
    prefill_peak = peak["bf16_tflops"] * 1e12
    return {
        "metric": "decode tokens/s (Qwen3-0.6B layer sizes, batch 8, after 2,048-token prompts)",
        "value": round(main["tokens_per_s"], 1),
        "unit": "tokens/s",
        "n_gpus": 1,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": round(main["ms_per_step"], 4),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic: seeded uniform-random token ids, random weights (N(0, 0.02)) of the named architecture",
        "impl": "ours",
        "config": config_record(batch, layers_run, peak_source),
        "e2e": {k: (round(v, 1) if isinstance(v, float) else v) for k, v in e2e.items()},
        "gpu_launches": main["launches"],
        "clocks": main["clocks"],
        "prefill": {"value": round(prefill["value"], 1), "tokens": prefill["tokens"], "ms": round(prefill["ms"], 3),
                    "frac": round(prefill["flops"] / (prefill["ms"] / 1e3) / prefill_peak, 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peak["hbm_gbs"], 4)},
        "points": points,
    }


def reference_folder() -> Path | None:
    """Where the unmodified reference lies: ``baseline/_ref`` beside this file (a plain copy of the
    reference's folder; it is a folder of scripts that runs from ``sys.path``), or the folder that the
    environment variable GTAR_REFERENCE_DIR names."""
    for folder in (os.environ.get("GTAR_REFERENCE_DIR"), ROOT / "baseline" / "_ref"):
        if folder and (Path(folder) / "src" / "engine.py").exists():
            return Path(folder)
    return None


class ReferenceArm:
    """The reference's own generation, untouched: ``Engine(TransformerForCausalLM).generate`` (src/engine.py:22-46)
    on the model that configs/transformer_0.6B.json describes, with the reference's own random initialisation.
    Nothing of this repository's package is imported here."""

    def __init__(self, folder: Path, device: str, layers: int | None, sizes: dict | None = None):
        import torch

        sys.path.insert(0, str(folder))
        from src.engine import Engine
        from src.models import ARCHITECTURES

        file = json.loads((folder / "configs" / "transformer_0.6B.json").read_text())
        config_class, model_class = ARCHITECTURES[file["arch"]]
        fields = dict(file["model"], vocab_size=BENCH_CONFIG["vocab_size"])
        for key, value in fields.items():  # the reference's file and the benchmark's sizes are the same model
            assert BENCH_CONFIG[key] == value, f"{key}: the reference's config has {value}, the benchmark {BENCH_CONFIG[key]}"
        if layers:
            fields["num_hidden_layers"] = layers
        if sizes:  # only the tests shrink the model (they run this arm on the CPU)
            fields.update(sizes)
        self.torch, self.device, self.fields = torch, device, fields
        torch.manual_seed(0)
        with torch.device(device):
            model = model_class(config_class(**fields))
        self.engine = Engine(model)
        self.eos = fields["vocab_size"] - 1  # the command line always passes a stop token (scripts/generate.py:40,44)

    def generate_seconds(self, prompts, new_tokens: int) -> float:
        """Wall clock of one call of the public API between synchronisations, as the reference times generation
        (scripts/benchmark_speculative.py:107-117): host token ids in, host token ids out."""
        torch = self.torch
        cuda = self.device.startswith("cuda")
        if cuda:
            torch.cuda.synchronize()
        begin = time.perf_counter()
        out = self.engine.generate(prompts, max_new_tokens=new_tokens, temperature=0.0, eos_token_id=self.eos).cpu()
        if cuda:
            torch.cuda.synchronize()
        seconds = time.perf_counter() - begin
        if out.shape[1] != new_tokens:  # every sequence chose the stop token: the run was cut short
            raise RuntimeError(f"the reference stopped after {out.shape[1]} of {new_tokens} tokens")
        return seconds

    def decode(self, batch: int, prompt_len: int, steps: int, warmup: int, repeats: int = 3) -> dict:
        """Seconds per decode step: a call that decodes warm-up + K steps minus a call that decodes warm-up steps,
        so that the prompts' step and the set-up cancel.  (A call for n new tokens runs n - 1 decode steps.)"""
        torch = self.torch
        gen = torch.Generator().manual_seed(0)
        prompts = torch.randint(0, self.fields["vocab_size"] - 1, (batch, prompt_len), generator=gen)
        self.generate_seconds(prompts, warmup + 1)  # untimed: compiles the attention kernel, loads the libraries
        short = [self.generate_seconds(prompts, warmup + 1) for _ in range(repeats)]
        long = [self.generate_seconds(prompts, warmup + steps + 1) for _ in range(repeats)]
        seconds = statistics.median(long) - statistics.median(short)
        return {"tokens_per_s": batch * steps / seconds, "ms_per_step": seconds / steps * 1e3,
                "h2d_bytes_per_step": batch * prompt_len * 8 // steps, "d2h_bytes_per_step": batch * 8}

    def prefill(self, tokens: int, repeats: int = 3) -> float:
        """Milliseconds of one prompt through the public API (one new token: the prompt's step and nothing else)."""
        torch = self.torch
        gen = torch.Generator().manual_seed(1)
        prompt = torch.randint(0, self.fields["vocab_size"] - 1, (1, tokens), generator=gen)
        self.generate_seconds(prompt, 1)
        return statistics.median(self.generate_seconds(prompt, 1) for _ in range(repeats)) * 1e3


def run_reference(args, device: str = "cuda:0", sizes: dict | None = None, prompt_len: int = PROMPT_LEN,
                  prefill_tokens: int = PREFILL_TOKENS, batches: tuple = (1, 64)) -> dict:
    """The reference arm: the same metric on the same configuration from the unmodified reference."""
    folder = reference_folder()
    if folder is None:
        return {"impl": "reference", "unavailable": "no copy of the reference under baseline/_ref (it is not part of "
                                                    "the repository's history) and GTAR_REFERENCE_DIR names none"}
    import torch

    if device.startswith("cuda") and not torch.cuda.is_available():
        return {"impl": "reference", "unavailable": "no CUDA device here: the arm is timed on a GPU only"}
    peak, peak_source = peaks()
    try:
        arm = ReferenceArm(folder, device, args.layers, sizes)
        sampler = ClockSampler()
        sampler.start()
        main = arm.decode(args.batch, prompt_len, args.steps, args.warmup)
        clocks = sampler.stop()
        prefill_ms = arm.prefill(prefill_tokens)
        points = {f"decode_b{b}": round(arm.decode(b, prompt_len, min(args.steps, 64), args.warmup, repeats=1)["tokens_per_s"], 1)
                  for b in batches}
    except Exception as error:  # the line says why; the trace goes to standard error
        import traceback

        traceback.print_exc()
        return {"impl": "reference", "unavailable": ("the reference failed here: %s: %s" % (type(error).__name__, error)).replace("\n", " ")[:300]}
    layers = arm.fields["num_hidden_layers"]
    achieved = step_bytes(args.batch, prompt_len + args.warmup + args.steps // 2, layers) / (main["ms_per_step"] / 1e3) / 1e9
    c = BENCH_CONFIG
    t = prefill_tokens
    per_layer = 2 * t * c["hidden_size"] * ((2 * c["num_attention_heads"] + 2 * c["num_key_value_heads"]) * c["head_dim"] + 3 * c["intermediate_size"])
    attention = 4 * c["num_attention_heads"] * c["head_dim"] * t * t / 2
    flops = layers * (per_layer + attention) + 2 * c["hidden_size"] * c["vocab_size"]  # counted as for the own arm: the wanted row only
    rate = round(main["tokens_per_s"], 1)
    return {
        "metric": "decode tokens/s (Qwen3-0.6B layer sizes, batch 8, after 2,048-token prompts)",
        "value": rate, "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(main["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic: seeded uniform-random token ids, random weights of the named architecture (the reference's own init_weights)",
        "impl": "reference",
        "timing": "wall clock around Engine.generate between synchronisations, long call minus short call (the "
                  "reference has no device-timed loop; value and e2e are the same measurement)",
        "config": config_record(args.batch, layers, peak_source),
        "e2e": {"value": rate, "unit": "tokens/s", "h2d_bytes_per_step": main["h2d_bytes_per_step"],
                "d2h_bytes_per_step": main["d2h_bytes_per_step"]},
        "gpu_launches": None,
        "clocks": clocks,
        "prefill": {"value": round(t / (prefill_ms / 1e3), 1), "tokens": t, "ms": round(prefill_ms, 3),
                    "frac": round(flops / (prefill_ms / 1e3) / (peak["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peak["hbm_gbs"], 4)},
        "points": points,
    }


# ---------------------------------------------------------------------------------------------------------------------
# --compare dasusun: the Dasusun decoder beside the dense transformer at equal layer sizes (random weights drawn on the
# device, the same prompts, the same engine): prefill and decode throughput, and the new design's kernels one by one
# against their rooflines beside the like kernels of the transformer.
def _dasusun_config(width, layers, heads, dim, rot, vdim, q_rank, kv_rank, window, ff, vocab):
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
             "scale": (dim + rot) ** -0.5, "mask": {"size": window},
             "rot": {"base": 10000.0, "dims": rot, "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}
    layer = {"type": "latent_attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": ff}}
    return {"architecture": "Dasusun", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "canon": {"taps": 4},
            "layers": [layer] * layers, "initializer_range": 0.02, "max_position_embeddings": 4096}


def _transformer_config(hidden, layers, heads, kv_heads, head_dim, ff, vocab):
    return {"arch": "transformer", "vocab_size": vocab, "hidden_size": hidden, "intermediate_size": ff, "num_hidden_layers": layers,
            "num_attention_heads": heads, "num_key_value_heads": kv_heads, "head_dim": head_dim, "rms_norm_eps": 1e-6,
            "rope_theta": 1000000.0, "tie_word_embeddings": True, "initializer_range": 0.02, "max_position_embeddings": 4096}


COMPARE_SIZES = {
    # name: (Dasusun sizes, transformer sizes); 8 layers each, vocabulary 32,768
    "width1024": (dict(width=1024, layers=8, heads=16, dim=64, rot=32, vdim=64, q_rank=512, kv_rank=256, window=1024, ff=4096, vocab=32768),
                  dict(hidden=1024, layers=8, heads=16, kv_heads=8, head_dim=128, ff=3072, vocab=32768)),
    "width2048": (dict(width=2048, layers=8, heads=16, dim=128, rot=64, vdim=128, q_rank=768, kv_rank=512, window=2048, ff=8192, vocab=32768),
                  dict(hidden=2048, layers=8, heads=16, kv_heads=8, head_dim=128, ff=6144, vocab=32768)),
}


def _device_model(raw: dict):
    import torch

    from gtar_kimik3_public_b200.models.model import Model
    from gtar_kimik3_public_b200.registry import architecture, config_from_dict
    from gtar_kimik3_public_b200.weights import load_random_weights

    config = config_from_dict(raw)
    model = Model(architecture(config.ARCH_NAMES[0]).build_plan(config), config, torch.bfloat16, "cuda:0")
    load_random_weights(model, seed=0, std=0.02)
    return model


def _time_prefill_ms(model, tokens: int, warmup: int = 3, repeats: int = 5) -> float:
    import torch

    from gtar_kimik3_public_b200.cache import rounded_tokens
    from gtar_kimik3_public_b200.engine import Engine, StepEntry

    engine = Engine(model, rounded_tokens(tokens + 1), max_seqs=1)
    prompt = random_prompts(1, tokens, model.vocab_size, seed=1)[0]
    times = []
    with torch.no_grad():
        for i in range(warmup + repeats):
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            begin.record()
            engine.step([StepEntry("p", prompt, [tokens - 1])])
            end.record()
            torch.cuda.synchronize()
            engine.end(["p"])
            if i >= warmup:
                times.append(begin.elapsed_time(end))
    del engine
    torch.cuda.empty_cache()
    return statistics.median(times)


def _dasusun_prefill_flops(d: dict, tokens: int) -> float:
    w, h = d["width"], d["heads"]
    per_token = 2 * (w * (d["q_rank"] + d["kv_rank"] + d["rot"]) + d["q_rank"] * h * (d["dim"] + d["rot"]) + h * d["dim"] * d["kv_rank"]
                     + h * d["kv_rank"] * d["vdim"] + h * d["vdim"] * w + 2 * w * d["ff"])
    seen = sum(min(t + 1, d["window"]) for t in range(tokens))
    attention = h * seen * (2 * (d["kv_rank"] + d["rot"]) + 2 * d["kv_rank"])
    return d["layers"] * (per_token * tokens + attention) + 2 * w * d["vocab"]


def _transformer_prefill_flops(t: dict, tokens: int) -> float:
    per_token = 2 * t["hidden"] * ((2 * t["heads"] + 2 * t["kv_heads"]) * t["head_dim"] + 3 * t["ff"])
    attention = 4 * t["heads"] * t["head_dim"] * tokens * tokens / 2
    return t["layers"] * (per_token * tokens + attention) + 2 * t["hidden"] * t["vocab"]


def _event_ms(fn, warmup: int = 3, repeats: int = 10, flush=None, inner: int = 1) -> float:
    """Median device time of one call.  ``flush``: a buffer larger than the L2 is written between the timed calls
    (many-token kernels).  ``inner`` > 1: that many calls back to back in one timed region, replayed from a CUDA graph so
    that the host's launch cost is not what is measured (few-token kernels, whose operands a step finds in the L2
    anyway)."""
    import torch

    graph = None
    if inner > 1:
        fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(inner):
                fn()
    times = []
    for i in range(warmup + repeats):
        if flush is not None and graph is None:
            flush.add_(1.0)
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        begin.record()
        if graph is None:
            fn()
        else:
            graph.replay()
        end.record()
        torch.cuda.synchronize()
        if i >= warmup:
            times.append(begin.elapsed_time(end) / inner)
    return statistics.median(times)


def _kernel_table(d: dict, t: dict, peak: dict) -> dict:
    """The new design's kernels alone, and the like kernels of the transformer, each with its share of its roofline
    (bytes over the measured copy bandwidth, or FLOPs over the measured bfloat16 product rate, whichever is larger)."""
    import torch

    from gtar_kimik3_public_b200.ops import functional as F

    dev = torch.device("cuda:0")
    flush = torch.zeros(48 << 20, dtype=torch.float32, device=dev)  # 192 MB: larger than the 126 MB L2
    hbm, tflops = peak["hbm_gbs"] * 1e9, peak["bf16_tflops"] * 1e12
    out = {}

    def record(name, ms, n_bytes, flops=0.0):
        floor = max(n_bytes / hbm, flops / tflops) * 1e3
        out[name] = {"us": round(ms * 1e3, 2), "roofline_us": round(floor * 1e3, 2), "frac": round(floor / ms, 4),
                     "bound": "hbm" if n_bytes / hbm >= flops / tflops else "tensor"}

    def tables(n, half):
        angle = torch.arange(n, dtype=torch.float32, device=dev)[:, None] * torch.rand(half, device=dev)[None, :]
        return angle.cos().contiguous(), angle.sin().contiguous()

    for label, tokens, n_seqs in (("prefill_2048", 2048, 1), ("decode_b8_ctx2048", 8, 8)):
        each = tokens // n_seqs
        inner = 1 if n_seqs == 1 else 20
        past = 0 if n_seqs == 1 else 2047
        length = past + each
        pages_each = -(-length // 64)
        table = torch.arange(n_seqs * pages_each, dtype=torch.int32, device=dev).view(n_seqs, pages_each)
        tok_seq = torch.arange(n_seqs, dtype=torch.int32, device=dev).repeat_interleave(each)
        tok_pos = (torch.arange(each, dtype=torch.int32, device=dev) + past).repeat(n_seqs)
        cu_q = torch.arange(n_seqs + 1, dtype=torch.int32, device=dev) * each
        slots = torch.arange(n_seqs, dtype=torch.int32, device=dev)
        kv_len = torch.full((n_seqs,), length, dtype=torch.int32, device=dev)
        # ---- the new design
        w, h, r, rot, dn = d["width"], d["heads"], d["kv_rank"], d["rot"], d["dim"]
        rows = F.PagedRows(torch.randn(n_seqs * pages_each, 64, r + rot, device=dev).bfloat16() * 0.1, table)
        cos, sin = tables(length, rot // 2)
        carried = torch.randn(h, tokens, r, device=dev).bfloat16()
        q_raw = torch.randn(tokens, h, dn + rot, device=dev).bfloat16()
        mixed = torch.empty(h, tokens, r, dtype=torch.bfloat16, device=dev)
        splits = 1 if n_seqs == 1 else F.latent_splits(n_seqs, h, length, d["window"], F.sm_count(dev))
        seen = sum(min(p + 1, d["window"]) for p in range(past, length)) * n_seqs
        flops = h * seen * (4 * r + 2 * rot)
        n_bytes = 2 * (tokens * h * (2 * r + dn + rot) + n_seqs * min(length, d["window"] + each) * (r + rot))
        ms = _event_ms(lambda: F.attention_latent_tiled(carried.transpose(0, 1), q_raw, dn, rot, rot, cos, sin, rows, tok_pos, cu_q,
                                                         slots, d["scale_"], d["window"], mixed.transpose(0, 1), n_seqs, each, splits),
                       flush=flush, inner=inner)
        record(f"dasusun latent attention, {label}", ms, n_bytes, flops)
        x = torch.randn(tokens, w, device=dev)
        y = torch.randn(tokens, w, device=dev).bfloat16()
        kept = torch.randn(d["layers"] + 1, tokens, w, device=dev)
        mix = torch.rand(d["layers"] // 2 + 1, device=dev)
        ones = torch.ones(w, device=dev)
        ms = _event_ms(lambda: F.branch_merge(x, y, ones, 1e-6, ones, kept=kept, n_kept=d["layers"] // 2, mix=mix, next_weight=ones,
                                               next_eps=1e-6, next_dtype=torch.float32), flush=flush, inner=inner)
        record(f"dasusun branch merge with depth mix of {d['layers'] // 2 + 1} streams and next norm, {label}", ms,
               tokens * w * (4 + 2 + 4 * (d["layers"] // 2) + 4 + 4 + 4))
        ms = _event_ms(lambda: F.branch_merge(x, y, ones, 1e-6, ones, next_weight=ones, next_eps=1e-6, next_dtype=torch.bfloat16), flush=flush, inner=inner)
        record(f"dasusun branch merge with next norm, {label}", ms, tokens * w * (4 + 2 + 4 + 2))
        state = torch.zeros(n_seqs, 3, w, device=dev)
        conv_w = torch.randn(4, w, device=dev)
        ms = _event_ms(lambda: F.causal_conv(x, conv_w, state, tok_pos, tok_seq, cu_q, slots, torch.bfloat16), flush=flush, inner=inner)
        record(f"dasusun causal convolution (4 taps), {label}", ms, tokens * w * (4 + 2))
        proj = torch.randn(tokens, d["q_rank"] + r + rot, device=dev).bfloat16()
        ms = _event_ms(lambda: F.latent_prepare(proj, d["q_rank"], r, rot, rot, torch.ones(d["q_rank"], device=dev), torch.ones(r, device=dev),
                                                 1e-6, cos, sin, tok_pos, tok_seq, slots, rows, length - 1), flush=flush, inner=inner)
        record(f"dasusun latent norms, rotation and cache write, {label}", ms, tokens * (d["q_rank"] + r + rot) * 2 * 2)
        act = torch.randn(tokens, d["ff"], device=dev).bfloat16()
        ms = _event_ms(lambda: F.gelu_tanh(act), flush=flush, inner=inner)
        record(f"dasusun GELU, {label}", ms, tokens * d["ff"] * 4)
        # ---- the transformer's like kernels
        hq, hk, hd = t["heads"], t["kv_heads"], t["head_dim"]
        kv = F.PagedKV(torch.randn(n_seqs * pages_each, hk, 64, hd, device=dev).bfloat16() * 0.1,
                       torch.randn(n_seqs * pages_each, hk, 64, hd, device=dev).bfloat16() * 0.1, table, F.DecodeWork(dev))
        q = torch.randn(tokens, hq, hd, device=dev).bfloat16()
        if n_seqs == 1:
            ms = _event_ms(lambda: F.attention_prefill(q, kv, cu_q, kv_len, slots, each, hd ** -0.5, 0), flush=flush, inner=inner)
            record(f"transformer attention, {label}", ms, 2 * (2 * tokens * hq * hd + 2 * length * hk * hd), 4 * hq * hd * tokens * tokens / 2)
        else:
            sp = F.decode_splits(n_seqs, hk, length, 64, F.sm_count(dev), F.decode_cluster_places(hd, F.sm_count(dev)))
            ms = _event_ms(lambda: F.attention_decode(q, kv, kv_len, slots, hd ** -0.5, 0, sp), flush=flush, inner=inner)
            record(f"transformer attention, {label}", ms, 2 * (2 * tokens * hq * hd + 2 * n_seqs * length * hk * hd), 4 * hq * hd * tokens * length)
        hs = torch.randn(tokens, t["hidden"], device=dev)
        delta = torch.randn(tokens, t["hidden"], device=dev).bfloat16()
        wn = torch.ones(t["hidden"], device=dev)
        ms = _event_ms(lambda: F.add_rmsnorm(hs, delta, wn, 1e-6, torch.bfloat16), flush=flush, inner=inner)
        record(f"transformer residual add with next norm, {label}", ms, tokens * t["hidden"] * (4 + 2 + 4 + 2))
        gu = torch.randn(tokens, 2 * t["ff"], device=dev).bfloat16()
        ms = _event_ms(lambda: F.swiglu(gu, interleaved=True), flush=flush, inner=inner)
        record(f"transformer SwiGLU, {label}", ms, tokens * t["ff"] * 6)
    return out


def run_compare(args) -> dict:
    import gc

    import torch

    from gtar_kimik3_public_b200.ops.library import require_device

    require_device(torch.device("cuda:0"))
    peak, peak_source = peaks()
    global PROMPT_LEN
    results = {}
    for name, (d, t) in COMPARE_SIZES.items():
        entry = {}
        for arch, raw, flops in (("dasusun", _dasusun_config(**d), _dasusun_prefill_flops(d, PREFILL_TOKENS)),
                                 ("transformer", _transformer_config(**t), _transformer_prefill_flops(t, PREFILL_TOKENS))):
            model = _device_model(raw)
            ms = _time_prefill_ms(model, PREFILL_TOKENS)
            decode = time_decode(model, args.batch, min(args.steps, 64), args.warmup)
            entry[arch] = {
                "weight_bytes_per_step": model.weight_bytes_per_step(),
                "prefill_tokens_per_s": round(PREFILL_TOKENS / (ms / 1e3), 1), "prefill_ms": round(ms, 3),
                "prefill_frac_of_bf16_peak": round(flops / (ms / 1e3) / (peak["bf16_tflops"] * 1e12), 4),
                "decode_tokens_per_s": round(decode["tokens_per_s"], 1), "decode_ms_per_step": round(decode["ms_per_step"], 4),
                "decode_frac_of_hbm_peak": round(decode["bytes_per_step"] / (decode["ms_per_step"] / 1e3) / 1e9 / peak["hbm_gbs"], 4),
                "decode_launches_per_step": decode["launches"] // max(1, min(args.steps, 64)),
            }
            del model
            gc.collect()
            torch.cuda.empty_cache()
        d_k = dict(d, scale_=(d["dim"] + d["rot"]) ** -0.5)
        entry["kernels"] = _kernel_table(d_k, t, peak)
        results[name] = {"sizes": {"dasusun": d, "transformer": t}, **entry}
    return {"compare": "dasusun beside transformer at equal layer sizes", "batch": args.batch, "prompt_tokens": PROMPT_LEN,
            "prefill_tokens": PREFILL_TOKENS, "dtype": "bf16", "data": "synthetic: random token ids, random weights drawn on the device",
            "peaks": dict(peak, source=peak_source), "l2": "single kernels: a 192 MB buffer is written between the timed calls of the 2,048-token cases; the 8-token cases are 20 calls back to back from a CUDA graph",
            "results": results}


# ---------------------------------------------------------------------------------------------------------------------
# --compare pofadra: the Pofadra decoder (delta-rule layers with one windowed attention layer in four, routed experts)
# beside the dense transformer at equal width and equal bytes of weights read per token, and its kernels one by one.
def _pofadra_config(width, layers, heads, kv_heads, dim, vdim, conv, rank, a_heads, a_kv, a_dim, window, rot, experts, top, ff,
                    groups, keep, vocab):
    delta = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv, "decay_rank": rank, "gate_rank": rank}
    attention = {"heads": a_heads, "kv_heads": a_kv, "dim": a_dim, "vdim": a_dim, "scale": a_dim ** -0.5, "mask": {"size": window},
                 "rot": {"base": 10000.0, "dims": rot}}
    mlp = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": 1.0, "groups": {"count": groups, "keep": keep}}}
    stack = [{"type": "attention" if i % 4 == 3 else "channel_delta", "mixer": attention if i % 4 == 3 else delta, "mlp": mlp}
             for i in range(layers)]
    return {"architecture": "Pofadra", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
            "logit_softcap": 40.0, "layers": stack, "initializer_range": 0.02, "max_position_embeddings": 4096}


POFADRA_SIZES = {
    # name: (Pofadra sizes, transformer sizes); 8 layers each, vocabulary 32,768; a token's experts hold what the dense
    # feed-forward of the transformer beside it holds (top * expert ff = the dense ff)
    "width1024": (dict(width=1024, layers=8, heads=8, kv_heads=8, dim=128, vdim=128, conv=4, rank=64, a_heads=16, a_kv=4, a_dim=64,
                       window=1024, rot=32, experts=32, top=4, ff=768, groups=4, keep=2, vocab=32768),
                  dict(hidden=1024, layers=8, heads=16, kv_heads=8, head_dim=128, ff=3072, vocab=32768)),
    "width2048": (dict(width=2048, layers=8, heads=16, kv_heads=16, dim=128, vdim=128, conv=4, rank=128, a_heads=16, a_kv=4, a_dim=128,
                       window=2048, rot=64, experts=64, top=6, ff=1024, groups=8, keep=4, vocab=32768),
                  dict(hidden=2048, layers=8, heads=16, kv_heads=8, head_dim=128, ff=6144, vocab=32768)),
}


def _pofadra_prefill_flops(d: dict, tokens: int) -> float:
    w, H, G, dk, dv = d["width"], d["heads"], d["kv_heads"], d["dim"], d["vdim"]
    n_attn = d["layers"] // 4
    n_delta = d["layers"] - n_attn
    delta = 2 * (w * (2 * G * dk + H * dv + H + 2 * d["rank"]) + 2 * d["rank"] * H * (dk + dv) // 2 + H * dv * w) + H * dv * 6 * dk
    aq, ak, ad = d["a_heads"], d["a_kv"], d["a_dim"]
    seen = sum(min(t + 1, d["window"]) for t in range(tokens))
    attention = 2 * w * ((2 * aq + ak) * ad) + 2 * aq * ad * w
    experts = 2 * w * d["experts"] + d["top"] * 6 * w * d["ff"]
    return (n_delta * delta + n_attn * attention + d["layers"] * experts) * tokens + n_attn * aq * seen * 4 * ad + 2 * w * d["vocab"]


def _pofadra_kernel_table(d: dict, t: dict, peak: dict) -> dict:
    """The new design's kernels alone and the like kernels of the transformer, each with its share of its roofline."""
    import torch

    from gtar_kimik3_public_b200.ops import functional as F
    from gtar_kimik3_public_b200.ops.linear import linear_grouped

    dev = torch.device("cuda:0")
    flush = torch.zeros(48 << 20, dtype=torch.float32, device=dev)  # 192 MB: larger than the 126 MB L2
    hbm, tflops = peak["hbm_gbs"] * 1e9, peak["bf16_tflops"] * 1e12
    out = {}

    def record(name, ms, n_bytes, flops=0.0):
        floor = max(n_bytes / hbm, flops / tflops) * 1e3
        out[name] = {"us": round(ms * 1e3, 2), "roofline_us": round(floor * 1e3, 2), "frac": round(floor / ms, 4),
                     "bound": "hbm" if n_bytes / hbm >= flops / tflops else "tensor"}

    w, H, G, dk, dv, taps = d["width"], d["heads"], d["kv_heads"], d["dim"], d["vdim"], d["conv"]
    aq, ak, ad, window = d["a_heads"], d["a_kv"], d["a_dim"], d["window"]
    E, top, ff = d["experts"], d["top"], d["ff"]
    C = 2 * G * dk + H * dv
    for label, tokens, n_seqs in (("prefill_2048", 2048, 1), ("decode_b8_ctx2048", 8, 8)):
        each = tokens // n_seqs
        inner = 1 if n_seqs == 1 else 20
        past = 0 if n_seqs == 1 else 2047
        length = past + each
        pages_each = -(-length // 64)
        table = torch.arange(n_seqs * pages_each, dtype=torch.int32, device=dev).view(n_seqs, pages_each)
        tok_seq = torch.arange(n_seqs, dtype=torch.int32, device=dev).repeat_interleave(each)
        tok_pos = (torch.arange(each, dtype=torch.int32, device=dev) + past).repeat(n_seqs)
        cu_q = torch.arange(n_seqs + 1, dtype=torch.int32, device=dev) * each
        slots = torch.arange(n_seqs, dtype=torch.int32, device=dev)
        kv_len = torch.full((n_seqs,), length, dtype=torch.int32, device=dev)
        # ---- the delta rule
        proj = (torch.randn(tokens, C + H + (-(C + H)) % 8, device=dev) * 0.5).bfloat16()
        low = torch.randn(tokens, H * (dk + dv), device=dev)
        conv_w, conv_state = torch.randn(C, taps, device=dev) * 0.3, torch.zeros(n_seqs, taps - 1, C, device=dev)
        a_log, dt_bias = torch.randn(H, device=dev) - 1, torch.randn(H * dk, device=dev) - 1
        ms = _event_ms(lambda: F.delta_prepare(proj, low, conv_w, conv_state, a_log, dt_bias, tok_pos, tok_seq, cu_q, slots, H, G, dk, dv, taps),
                       flush=flush, inner=inner)
        record(f"pofadra convolutions, unit lengths, decays and beta, {label}", ms, tokens * (2 * (C + H) + 4 * H * dk + 4 * (C + H * dk + H)))
        q, k, v, g, beta = F.delta_prepare(proj, low, conv_w, conv_state, a_log, dt_bias, tok_pos, tok_seq, cu_q, slots, H, G, dk, dv, taps)
        state = torch.zeros(n_seqs, H, dk, dv, device=dev)
        ms = _event_ms(lambda: F.delta_scan(q, k, v, g, beta, state, cu_q, slots, n_seqs), flush=flush, inner=inner)
        record(f"pofadra delta rule recurrence, {label}", ms, 4 * (tokens * (2 * G * dk + H * dk + 2 * H * dv + H) + 2 * n_seqs * H * dk * dv))
        o = torch.randn(tokens, H, dv, device=dev)
        norm_w = torch.ones(dv, device=dev)
        ms = _event_ms(lambda: F.head_norm_gate(o, norm_w, low, H * dk, 1e-6, torch.bfloat16), flush=flush, inner=inner)
        record(f"pofadra head norm and gate, {label}", ms, tokens * H * dv * (4 + 4 + 2))
        # ---- attention with wide norms and a sink, beside the transformer's
        kv = F.PagedKV(torch.randn(n_seqs * pages_each, ak, 64, ad, device=dev).bfloat16() * 0.1,
                       torch.randn(n_seqs * pages_each, ak, 64, ad, device=dev).bfloat16() * 0.1, table, F.DecodeWork(dev))
        wide = (torch.randn(tokens, (2 * aq + ak) * ad, device=dev)).bfloat16()
        angle = torch.arange(length, dtype=torch.float32, device=dev)[:, None] * torch.rand(d["rot"] // 2, device=dev)[None, :]
        cos, sin = angle.cos().contiguous(), angle.sin().contiguous()
        wq, wk = torch.ones(aq * ad, device=dev), torch.ones(ak * ad, device=dev)
        ms = _event_ms(lambda: F.wide_norm_rope_write(wide, aq, ak, ad, wq, wk, 1e-6, cos, sin, d["rot"], tok_pos, tok_seq, slots, kv, length - 1),
                       flush=flush, inner=inner)
        record(f"pofadra wide norms, rotation and cache write, {label}", ms, tokens * 2 * ((aq + ak) * ad + aq * ad + 2 * ak * ad))
        qa = torch.randn(tokens, aq, ad, device=dev).bfloat16()
        seen = sum(min(p + 1, window) for p in range(past, length)) * n_seqs
        if n_seqs == 1:
            ms = _event_ms(lambda: F.attention_prefill(qa, kv, cu_q, kv_len, slots, each, ad ** -0.5, window, sink=True), flush=flush, inner=inner)
        else:
            sp = F.decode_splits(n_seqs, ak, length, 64, F.sm_count(dev), F.decode_cluster_places(ad, F.sm_count(dev)))
            ms = _event_ms(lambda: F.attention_decode(qa, kv, kv_len, slots, ad ** -0.5, window, sp, sink=True), flush=flush, inner=inner)
        record(f"pofadra window attention with sink, {label}", ms, 2 * (2 * tokens * aq * ad + 2 * n_seqs * min(length, window + each) * ak * ad),
               4 * aq * ad * seen)
        gate_src = torch.randn(tokens, aq * ad, device=dev).bfloat16()
        ms = _event_ms(lambda: F.sigmoid_gate(qa.view(tokens, aq * ad), gate_src, 0), flush=flush, inner=inner)
        record(f"pofadra output gate, {label}", ms, tokens * aq * ad * 6)
        # ---- routed experts
        x = torch.randn(tokens, w, device=dev).bfloat16()
        router, correction = torch.randn(E, w, device=dev) * 0.05, torch.randn(E, device=dev) * 0.1
        ms = _event_ms(lambda: F.route_groups(x, router, correction, top, d["groups"], d["keep"], 1.0), flush=flush, inner=inner)
        record(f"pofadra router, {label}", ms, tokens * w * 2 + E * w * 4)
        ids, weights = F.route_groups(x, router, correction, top, d["groups"], d["keep"], 1.0)
        gate_up = (torch.randn(E, 2, ff, w, device=dev) * 0.02).bfloat16()
        down = (torch.randn(E, w, ff, device=dev) * 0.02).bfloat16()
        used = int(torch.unique(ids).numel())
        expert_bytes = used * 3 * ff * w * 2
        if n_seqs == 1:
            def grouped():
                ends, place_of, pair_at = F.experts_sort(ids, E)
                rows = F.gather_rows(x, pair_at, top)
                act = F.swiglu(linear_grouped(rows, gate_up.view(E, 2 * ff, w), ends))
                return F.experts_combine(linear_grouped(act, down, ends), place_of, weights, x)
            ms = _event_ms(grouped, flush=flush, inner=inner)
            record(f"pofadra experts (sorted, grouped products), {label}", ms, expert_bytes + tokens * top * (w * 4 + ff * 6), tokens * top * 6 * w * ff)
        else:
            ms = _event_ms(lambda: F.experts_pairwise(x, gate_up, down, ids, weights, x), flush=flush, inner=inner)
            record(f"pofadra experts (pair by pair), {label}", ms, expert_bytes, tokens * top * 6 * w * ff)
        # ---- the transformer's like kernels
        hq, hk, hd = t["heads"], t["kv_heads"], t["head_dim"]
        kvt = F.PagedKV(torch.randn(n_seqs * pages_each, hk, 64, hd, device=dev).bfloat16() * 0.1,
                        torch.randn(n_seqs * pages_each, hk, 64, hd, device=dev).bfloat16() * 0.1, table, F.DecodeWork(dev))
        qt = torch.randn(tokens, hq, hd, device=dev).bfloat16()
        if n_seqs == 1:
            ms = _event_ms(lambda: F.attention_prefill(qt, kvt, cu_q, kv_len, slots, each, hd ** -0.5, 0), flush=flush, inner=inner)
            record(f"transformer attention, {label}", ms, 2 * (2 * tokens * hq * hd + 2 * length * hk * hd), 4 * hq * hd * tokens * tokens / 2)
            ms = _event_ms(lambda: F.attention_prefill(qt, kvt, cu_q, kv_len, slots, each, hd ** -0.5, window, tensor_cores="mma"), flush=flush, inner=inner)
            record(f"transformer attention on the warp-level kernel with the same window, {label}", ms,
                   2 * (2 * tokens * hq * hd + 2 * length * hk * hd), 4 * hq * hd * seen)
        else:
            sp = F.decode_splits(n_seqs, hk, length, 64, F.sm_count(dev), F.decode_cluster_places(hd, F.sm_count(dev)))
            ms = _event_ms(lambda: F.attention_decode(qt, kvt, kv_len, slots, hd ** -0.5, 0, sp), flush=flush, inner=inner)
            record(f"transformer attention, {label}", ms, 2 * (2 * tokens * hq * hd + 2 * n_seqs * length * hk * hd), 4 * hq * hd * tokens * length)
        qkv = torch.randn(tokens, (hq + 2 * hk) * hd, device=dev).bfloat16()
        anglet = torch.arange(length, dtype=torch.float32, device=dev)[:, None] * torch.rand(hd // 2, device=dev)[None, :]
        ones = torch.ones(hd, device=dev)
        ms = _event_ms(lambda: F.qk_norm_rope_write(qkv, hq, hk, hd, ones, ones, 1e-6, anglet.cos().contiguous(), anglet.sin().contiguous(), tok_pos,
                                                     tok_seq, slots, kvt, length - 1), flush=flush, inner=inner)
        record(f"transformer q/k norm, rotation and cache write, {label}", ms, tokens * 2 * ((hq + 2 * hk) * hd + hq * hd + 2 * hk * hd))
        hs = torch.randn(tokens, t["hidden"], device=dev)
        delta = torch.randn(tokens, t["hidden"], device=dev).bfloat16()
        wn = torch.ones(t["hidden"], device=dev)
        ms = _event_ms(lambda: F.add_rmsnorm(hs, delta, wn, 1e-6, torch.bfloat16), flush=flush, inner=inner)
        record(f"transformer residual add with next norm, {label}", ms, tokens * t["hidden"] * (4 + 2 + 4 + 2))
        gu = torch.randn(tokens, 2 * t["ff"], device=dev).bfloat16()
        ms = _event_ms(lambda: F.swiglu(gu, interleaved=True), flush=flush, inner=inner)
        record(f"transformer SwiGLU, {label}", ms, tokens * t["ff"] * 6)
    return out


def run_compare_pofadra(args) -> dict:
    import gc

    import torch

    from gtar_kimik3_public_b200.ops.library import require_device

    require_device(torch.device("cuda:0"))
    peak, peak_source = peaks()
    results = {}
    for name, (d, t) in POFADRA_SIZES.items():
        entry = {}
        for arch, raw, flops in (("pofadra", _pofadra_config(**d), _pofadra_prefill_flops(d, PREFILL_TOKENS)),
                                 ("transformer", _transformer_config(**t), _transformer_prefill_flops(t, PREFILL_TOKENS))):
            model = _device_model(raw)
            ms = _time_prefill_ms(model, PREFILL_TOKENS)
            decode = time_decode(model, args.batch, min(args.steps, 64), args.warmup)
            entry[arch] = {
                "weight_bytes_per_step": model.weight_bytes_per_step(),
                "prefill_tokens_per_s": round(PREFILL_TOKENS / (ms / 1e3), 1), "prefill_ms": round(ms, 3),
                "prefill_frac_of_bf16_peak": round(flops / (ms / 1e3) / (peak["bf16_tflops"] * 1e12), 4),
                "decode_tokens_per_s": round(decode["tokens_per_s"], 1), "decode_ms_per_step": round(decode["ms_per_step"], 4),
                "decode_frac_of_hbm_peak": round(decode["bytes_per_step"] / (decode["ms_per_step"] / 1e3) / 1e9 / peak["hbm_gbs"], 4),
                "decode_launches_per_step": decode["launches"] // max(1, min(args.steps, 64)),
            }
            del model
            gc.collect()
            torch.cuda.empty_cache()
        entry["kernels"] = _pofadra_kernel_table(d, t, peak)
        results[name] = {"sizes": {"pofadra": d, "transformer": t}, **entry}
    return {"compare": "pofadra beside transformer at equal width", "batch": args.batch, "prompt_tokens": PROMPT_LEN,
            "prefill_tokens": PREFILL_TOKENS, "dtype": "bf16", "data": "synthetic: random token ids, random weights drawn on the device",
            "peaks": dict(peak, source=peak_source), "l2": "single kernels: a 192 MB buffer is written between the timed calls of the 2,048-token cases; the 8-token cases are 20 calls back to back from a CUDA graph",
            "results": results}


# --compare rezulorn: the Rezulorn decoder (decayed linear attention, scored attention with a distance term and a window
# that keeps the first tokens, pairs of sigmoid-weighted attention and retention; squared-relu feed-forwards) beside the
# dense transformer at equal width, and its kernels one by one beside the like kernels of the models that were here.
def _rezulorn_config(width, layers, heads, kv_heads, dim, window, keep, l_heads, l_dim, l_vdim, p_heads, p_kv, r_heads, r_dim, rot, ff,
                     vocab):
    def decays(n):
        return [1.0 - 2.0 ** (-3 - 6 * i / max(1, n - 1)) for i in range(n)]

    lightning = {"heads": l_heads, "dim": l_dim, "vdim": l_vdim, "decay": decays(l_heads)}
    attention = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5,
                 "mask": {"size": window, "keep_first": keep}}
    pair = {"left": {"heads": p_heads, "kv_heads": p_kv, "dim": dim, "vdim": dim, "scale": dim ** -0.5,
                     "rot": {"base": 500000.0, "dims": rot, "scaling": {"factor": 2.0}}},
            "right": {"heads": r_heads, "dim": r_dim, "vdim": r_dim, "decay": decays(r_heads), "rot": {"base": 10000.0, "dims": rot // 2}},
            "left_scale": 0.6, "right_scale": 0.9}
    kinds = {"parallel": pair, "lightning": lightning, "attention": attention}
    order = ["parallel", "lightning", "attention", "parallel"]
    stack = [{"type": order[i % 4], "mixer": kinds[order[i % 4]], "mlp": {"kind": "dense", "ff": ff}} for i in range(layers)]
    return {"architecture": "Rezulorn", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "canon": {"taps": 4}, "residual_mult": 0.5,
            "logit_scale": 0.25, "layers": stack, "initializer_range": 0.02, "max_position_embeddings": 4096}


REZULORN_SIZES = {
    # name: (Rezulorn sizes, transformer sizes); 8 layers each, vocabulary 32,768; the two matrices of a squared-relu
    # feed-forward hold about what the three of the transformer's gated one hold
    "width1024": (dict(width=1024, layers=8, heads=16, kv_heads=4, dim=64, window=1024, keep=64, l_heads=8, l_dim=128, l_vdim=128,
                       p_heads=8, p_kv=2, r_heads=8, r_dim=64, rot=64, ff=4096, vocab=32768),
                  dict(hidden=1024, layers=8, heads=16, kv_heads=8, head_dim=128, ff=3072, vocab=32768)),
    "width2048": (dict(width=2048, layers=8, heads=16, kv_heads=4, dim=128, window=1024, keep=64, l_heads=16, l_dim=128, l_vdim=128,
                       p_heads=8, p_kv=2, r_heads=8, r_dim=128, rot=64, ff=8192, vocab=32768),
                  dict(hidden=2048, layers=8, heads=16, kv_heads=8, head_dim=128, ff=6144, vocab=32768)),
}


def _rezulorn_prefill_flops(d: dict, tokens: int) -> float:
    w, dim = d["width"], d["dim"]
    windowed = sum(min(t + 1, d["window"] + d["keep"]) for t in range(tokens))
    causal = tokens * (tokens + 1) // 2
    ff = 4 * w * d["ff"]
    lightning = 2 * w * d["l_heads"] * (2 * d["l_dim"] + 2 * d["l_vdim"]) + 2 * d["l_heads"] * d["l_vdim"] * w + 4 * d["l_heads"] * d["l_dim"] * d["l_vdim"]
    attention = 2 * w * (d["heads"] + 2 * d["kv_heads"]) * dim + 2 * d["heads"] * dim * w
    left = 2 * w * (d["p_heads"] + 2 * d["p_kv"]) * dim + 2 * d["p_heads"] * dim * w
    right = 2 * w * d["r_heads"] * 4 * d["r_dim"] + 2 * d["r_heads"] * d["r_dim"] * w + 4 * d["r_heads"] * d["r_dim"] ** 2
    total = 0.0
    for i in range(d["layers"]):
        kind = ("parallel", "lightning", "attention", "parallel")[i % 4]
        if kind == "lightning":
            total += (lightning + ff) * tokens
        elif kind == "attention":
            total += (attention + ff) * tokens + 4 * d["heads"] * dim * windowed
        else:
            total += (left + right + ff) * tokens + 4 * d["p_heads"] * dim * causal
    return total + 2 * w * d["vocab"]

def _rezulorn_kernel_table(d: dict, t: dict, peak: dict) -> dict:
    """The new design's kernels alone and the like kernels of the transformer (attention, norms) and of the delta-rule
    decoder (the recurrence and the norm behind it), each with its share of its roofline."""
    import torch

    from gtar_kimik3_public_b200.ops import functional as F

    dev = torch.device("cuda:0")
    flush = torch.zeros(48 << 20, dtype=torch.float32, device=dev)  # 192 MB: larger than the 126 MB L2
    hbm, tflops = peak["hbm_gbs"] * 1e9, peak["bf16_tflops"] * 1e12
    out = {}

    def record(name, ms, n_bytes, flops=0.0):
        floor = max(n_bytes / hbm, flops / tflops) * 1e3
        out[name] = {"us": round(ms * 1e3, 2), "roofline_us": round(floor * 1e3, 2), "frac": round(floor / ms, 4),
                     "bound": "hbm" if n_bytes / hbm >= flops / tflops else "tensor"}

    w, dim, window, keep = d["width"], d["dim"], d["window"], d["keep"]
    aq, ak, pq, pk = d["heads"], d["kv_heads"], d["p_heads"], d["p_kv"]
    H, dk, dv = d["l_heads"], d["l_dim"], d["l_vdim"]
    bf = torch.bfloat16
    for label, tokens, n_seqs in (("prefill_2048", 2048, 1), ("decode_b8_ctx2048", 8, 8)):
        each = tokens // n_seqs
        inner = 1 if n_seqs == 1 else 20
        past = 0 if n_seqs == 1 else 2047
        length = past + each
        pages_each = -(-length // 64)
        table = torch.arange(n_seqs * pages_each, dtype=torch.int32, device=dev).view(n_seqs, pages_each)
        tok_seq = torch.arange(n_seqs, dtype=torch.int32, device=dev).repeat_interleave(each)
        tok_pos = (torch.arange(each, dtype=torch.int32, device=dev) + past).repeat(n_seqs)
        cu_q = torch.arange(n_seqs + 1, dtype=torch.int32, device=dev) * each
        slots = torch.arange(n_seqs, dtype=torch.int32, device=dev)
        kv_len = torch.full((n_seqs,), length, dtype=torch.int32, device=dev)
        # ---- the stream: layer norm with the pending branch, the convolution over time, the sum of a pair
        hs = torch.randn(tokens, w, device=dev)
        branch = torch.randn(tokens, w, device=dev).to(bf)
        wn = torch.ones(w, device=dev)
        ms = _event_ms(lambda: F.add_layernorm(hs, branch, wn, 1e-5, torch.float32, delta_scale=0.5), flush=flush, inner=inner)
        record(f"rezulorn residual add with layer norm, {label}", ms, tokens * w * (4 + 2 + 4 + 4))
        ms = _event_ms(lambda: F.add_rmsnorm(hs, branch, wn, 1e-6, bf), flush=flush, inner=inner)
        record(f"transformer residual add with next norm, {label}", ms, tokens * w * (4 + 2 + 4 + 2))
        normed = torch.randn(tokens, w, device=dev)
        conv_w, conv_state = torch.randn(4, w, device=dev) * 0.3, torch.zeros(n_seqs, 3, w, device=dev)
        ms = _event_ms(lambda: F.causal_conv(normed, conv_w, conv_state, tok_pos, tok_seq, cu_q, slots, bf, update_single_token_state=n_seqs > 1),
                       flush=flush, inner=inner)
        record(f"rezulorn convolution over time, {label}", ms, tokens * w * (4 + 2) + (n_seqs * 3 * w * 8 if n_seqs > 1 else 0))
        if n_seqs > 1:  # what single-token steps run instead of the two above
            ms = _event_ms(lambda: F.add_layernorm_conv_single(hs, branch, wn, 1e-5, conv_w, conv_state, tok_pos, tok_seq, slots, bf,
                                                               delta_scale=0.5), flush=flush, inner=inner)
            record(f"rezulorn residual add, layer norm and convolution in one kernel, {label}", ms,
                   tokens * w * (4 + 2 + 4 + 2) + n_seqs * 3 * w * 8)
        ms = _event_ms(lambda: F.scaled_sum(branch, 0.6, branch, 0.9), flush=flush, inner=inner)
        record(f"rezulorn sum of a pair's branches, {label}", ms, tokens * w * (2 + 2 + 4))
        # ---- the recurrence with a fixed decay, beside the delta rule at the same heads
        proj = (torch.randn(tokens, H * (2 * dk + 2 * dv), device=dev) * 0.5).to(bf)
        ms = _event_ms(lambda: F.heads_prepare(proj, 0, H * dk, 2 * H * dk, H, H, dk, dv, tok_pos, tok_seq, slots, silu_qk=True, silu_v=True),
                       flush=flush, inner=inner)
        record(f"rezulorn SiLU of q, k, v into 32-bit arrays, {label}", ms, tokens * H * (2 * dk + dv) * (2 + 4))
        q, k, v = F.heads_prepare(proj, 0, H * dk, 2 * H * dk, H, H, dk, dv, tok_pos, tok_seq, slots, silu_qk=True, silu_v=True)
        q *= dk ** -0.5
        decay = torch.linspace(0.9, 0.999, H, device=dev)
        state = torch.zeros(n_seqs, H, dk, dv, device=dev)
        ms = _event_ms(lambda: F.decay_scan(q, k, v, decay, state, cu_q, slots, n_seqs), flush=flush, inner=inner)
        scan_bytes = 4 * (tokens * H * (2 * dk + 2 * dv) + 2 * n_seqs * H * dk * dv)
        record(f"rezulorn recurrence with a fixed decay, token by token, {label}", ms, scan_bytes)
        if tokens // n_seqs >= 64:
            ms = _event_ms(lambda: F.decay_scan_chunked(q, k, v, decay, state, cu_q, slots, n_seqs, tokens // n_seqs), flush=flush, inner=inner)
            chunk_flops = 2.0 * tokens * H * (2 * dk * dv + 64 * dk // 2 + 64 * dv // 2)
            record(f"rezulorn recurrence with a fixed decay, in chunks of 64 (32-bit pipe: {chunk_flops / 1e9:.2f} GFLOP), {label}", ms, scan_bytes)
        g, beta = torch.exp(-torch.rand(tokens, H, dk, device=dev) * 0.1), torch.rand(tokens, H, device=dev)
        kn = torch.nn.functional.normalize(k, dim=-1)
        ms = _event_ms(lambda: F.delta_scan(q, kn, v, g, beta, state, cu_q, slots, n_seqs), flush=flush, inner=inner)
        record(f"delta-rule decoder recurrence at the same heads, {label}", ms, scan_bytes + 4 * tokens * H * (dk + 1))
        o = torch.randn(tokens, H * dv, device=dev)
        norm_w = torch.ones(H * dv, device=dev)
        ms = _event_ms(lambda: F.group_norm_gate(o, H * dv, norm_w, proj, 2 * H * dk + H * dv, 1e-5, bf, "sigmoid"), flush=flush, inner=inner)
        record(f"rezulorn norm over all heads with sigmoid gate, {label}", ms, tokens * H * dv * (4 + 2 + 2))
        ms = _event_ms(lambda: F.group_norm_gate(o, dv, None, proj, 2 * H * dk + H * dv, 1e-5, bf, "silu"), flush=flush, inner=inner)
        record(f"rezulorn unit heads with SiLU gate, {label}", ms, tokens * H * dv * (4 + 2 + 2))
        head_w = torch.ones(dv, device=dev)
        gate32 = torch.randn(tokens, H * dv, device=dev)
        ms = _event_ms(lambda: F.head_norm_gate(o.view(tokens, H, dv), head_w, gate32, 0, 1e-6, bf), flush=flush, inner=inner)
        record(f"delta-rule decoder head norm and gate, {label}", ms, tokens * H * dv * (4 + 4 + 2))
        # ---- scored attention beside the transformer's
        def pages(n_heads, size):
            return F.PagedKV(torch.randn(n_seqs * pages_each, n_heads, 64, size, device=dev).to(bf) * 0.1,
                             torch.randn(n_seqs * pages_each, n_heads, 64, size, device=dev).to(bf) * 0.1, table, F.DecodeWork(dev))

        kv = pages(ak, dim)
        wide = torch.randn(tokens, (aq + 2 * ak) * dim, device=dev).to(bf)
        ms = _event_ms(lambda: F.heads_prepare(wide, 0, aq * dim, (aq + ak) * dim, aq, ak, dim, dim, tok_pos, tok_seq, slots, kv=kv,
                                               max_position=length - 1), flush=flush, inner=inner)
        record(f"rezulorn cache write (no rotation), {label}", ms, tokens * 2 * ((aq + 2 * ak) * dim + aq * dim + 2 * ak * dim))
        angle = torch.arange(length, dtype=torch.float32, device=dev)[:, None] * torch.rand(d["rot"] // 2, device=dev)[None, :]
        cos, sin = angle.cos().contiguous(), angle.sin().contiguous()
        kvp = pages(pk, dim)
        widep = torch.randn(tokens, (pq + 2 * pk) * dim, device=dev).to(bf)
        ms = _event_ms(lambda: F.heads_prepare(widep, 0, pq * dim, (pq + pk) * dim, pq, pk, dim, dim, tok_pos, tok_seq, slots, rot=d["rot"],
                                               cos=cos, sin=sin, unit_eps=1e-5, kv=kvp, max_position=length - 1), flush=flush, inner=inner)
        record(f"rezulorn rotation, unit q and k, cache write, {label}", ms, tokens * 2 * ((pq + 2 * pk) * dim + pq * dim + 2 * pk * dim))
        qa = torch.randn(tokens, aq, dim, device=dev).to(bf)
        r1, r2 = torch.full((aq,), 0.3, device=dev), torch.full((aq,), 0.5, device=dev)
        seen = sum(min(p + 1, window) + min(keep, max(0, p + 1 - window)) for p in range(past, length)) * n_seqs
        parts = F.scored_attention_parts(n_seqs, aq, ak, each, -(-(window + keep) // 64) + 2, F.sm_count(dev))
        ms = _event_ms(lambda: F.attention_scored(qa, kv, cu_q, kv_len, slots, each, dim ** -0.5, window, keep, r1, r2, None, "softmax", parts),
                       flush=flush, inner=inner)
        attn_bytes = 2 * (2 * tokens * aq * dim + 2 * n_seqs * min(length, window + keep + each) * ak * dim)
        record(f"rezulorn attention: distance term, window {window} keeping {keep}, softmax, {label}", ms, attn_bytes, 4 * aq * dim * seen)
        ms = _event_ms(lambda: F.attention_scored_exact(qa, kv, tok_pos, tok_seq, slots, dim ** -0.5, window, keep, r1, r2, None, "softmax"),
                       flush=flush, inner=inner, repeats=3)
        record(f"rezulorn attention, the same on the exact kernel (what 32-bit runs use), {label}", ms, attn_bytes, 4 * aq * dim * seen)
        qp = torch.randn(tokens, pq, dim, device=dev).to(bf)
        pb = torch.full((pq,), -4.0, device=dev)
        causal = sum(p + 1 for p in range(past, length)) * n_seqs
        parts = F.scored_attention_parts(n_seqs, pq, pk, each, pages_each, F.sm_count(dev))
        ms = _event_ms(lambda: F.attention_scored(qp, kvp, cu_q, kv_len, slots, each, dim ** -0.5, 0, 0, None, None, pb, "sigmoid", parts),
                       flush=flush, inner=inner)
        record(f"rezulorn attention: causal, sigmoid weights, {label}", ms, 2 * (2 * tokens * pq * dim + 2 * n_seqs * length * pk * dim),
               4 * pq * dim * causal)
        hq, hk, hd = t["heads"], t["kv_heads"], t["head_dim"]
        kvt = pages(hk, hd)
        qt = torch.randn(tokens, hq, hd, device=dev).to(bf)
        if n_seqs == 1:
            ms = _event_ms(lambda: F.attention_prefill(qt, kvt, cu_q, kv_len, slots, each, hd ** -0.5, 0), flush=flush, inner=inner)
            record(f"transformer attention, {label}", ms, 2 * (2 * tokens * hq * hd + 2 * length * hk * hd), 4 * hq * hd * causal)
            ms = _event_ms(lambda: F.attention_prefill(qt, kvt, cu_q, kv_len, slots, each, hd ** -0.5, 0, tensor_cores="mma"), flush=flush, inner=inner)
            record(f"transformer attention on the warp-level kernel, {label}", ms, 2 * (2 * tokens * hq * hd + 2 * length * hk * hd),
                   4 * hq * hd * causal)
            ms = _event_ms(lambda: F.attention_prefill(qt, kvt, cu_q, kv_len, slots, each, hd ** -0.5, window, tensor_cores="mma"), flush=flush,
                           inner=inner)
            record(f"transformer attention on the warp-level kernel with window {window}, {label}", ms,
                   2 * (2 * tokens * hq * hd + 2 * length * hk * hd), 4 * hq * hd * sum(min(p + 1, window) for p in range(length)))
        else:
            sp = F.decode_splits(n_seqs, hk, length, 64, F.sm_count(dev), F.decode_cluster_places(hd, F.sm_count(dev)))
            ms = _event_ms(lambda: F.attention_decode(qt, kvt, kv_len, slots, hd ** -0.5, 0, sp), flush=flush, inner=inner)
            record(f"transformer attention, {label}", ms, 2 * (2 * tokens * hq * hd + 2 * n_seqs * length * hk * hd), 4 * hq * hd * tokens * length)
            sp = F.decode_splits(n_seqs, hk, window, 64, F.sm_count(dev), F.decode_cluster_places(hd, F.sm_count(dev)))
            ms = _event_ms(lambda: F.attention_decode(qt, kvt, kv_len, slots, hd ** -0.5, window, sp), flush=flush, inner=inner)
            record(f"transformer attention with window {window}, {label}", ms, 2 * (2 * tokens * hq * hd + 2 * n_seqs * window * hk * hd),
                   4 * hq * hd * tokens * window)
        qkv = torch.randn(tokens, (hq + 2 * hk) * hd, device=dev).to(bf)
        anglet = torch.arange(length, dtype=torch.float32, device=dev)[:, None] * torch.rand(hd // 2, device=dev)[None, :]
        cost, sint = anglet.cos().contiguous(), anglet.sin().contiguous()
        ones = torch.ones(hd, device=dev)
        ms = _event_ms(lambda: F.qk_norm_rope_write(qkv, hq, hk, hd, ones, ones, 1e-6, cost, sint, tok_pos, tok_seq, slots, kvt, length - 1),
                       flush=flush, inner=inner)
        record(f"transformer q/k norm, rotation and cache write, {label}", ms, tokens * 2 * ((hq + 2 * hk) * hd + hq * hd + 2 * hk * hd))
    return out


def run_compare_rezulorn(args) -> dict:
    import gc

    import torch

    from gtar_kimik3_public_b200.ops.library import require_device

    require_device(torch.device("cuda:0"))
    peak, peak_source = peaks()
    results = {}
    for name, (d, t) in REZULORN_SIZES.items():
        entry = {}
        for arch, raw, flops in (("rezulorn", _rezulorn_config(**d), _rezulorn_prefill_flops(d, PREFILL_TOKENS)),
                                 ("transformer", _transformer_config(**t), _transformer_prefill_flops(t, PREFILL_TOKENS))):
            model = _device_model(raw)
            ms = _time_prefill_ms(model, PREFILL_TOKENS)
            decode = time_decode(model, args.batch, min(args.steps, 64), args.warmup)
            entry[arch] = {
                "weight_bytes_per_step": model.weight_bytes_per_step(),
                "prefill_tokens_per_s": round(PREFILL_TOKENS / (ms / 1e3), 1), "prefill_ms": round(ms, 3),
                "prefill_frac_of_bf16_peak": round(flops / (ms / 1e3) / (peak["bf16_tflops"] * 1e12), 4),
                "decode_tokens_per_s": round(decode["tokens_per_s"], 1), "decode_ms_per_step": round(decode["ms_per_step"], 4),
                "decode_frac_of_hbm_peak": round(decode["bytes_per_step"] / (decode["ms_per_step"] / 1e3) / 1e9 / peak["hbm_gbs"], 4),
                "decode_launches_per_step": decode["launches"] // max(1, min(args.steps, 64)),
            }
            del model
            gc.collect()
            torch.cuda.empty_cache()
        entry["kernels"] = _rezulorn_kernel_table(d, t, peak)
        results[name] = {"sizes": {"rezulorn": d, "transformer": t}, **entry}
    return {"compare": "rezulorn beside transformer at equal width", "batch": args.batch, "prompt_tokens": PROMPT_LEN,
            "prefill_tokens": PREFILL_TOKENS, "dtype": "bf16", "data": "synthetic: random token ids, random weights drawn on the device",
            "peaks": dict(peak, source=peak_source), "l2": "single kernels: a 192 MB buffer is written between the timed calls of the 2,048-token cases; the 8-token cases are 20 calls back to back from a CUDA graph",
            "results": results}

# --compare zasorax: the Zasorax decoder (sublayers that read the stream itself and are normed on their way out; scored
# attention in chunks with a distance table, head temperatures and learned sinks, some layers reading an earlier layer's
# pages; causal attention with turned values, a fixed sink and a gate per head; dense xIELU and routed feed-forwards)
# beside the Rezulorn decoder, whose attention kernels it shares, at equal width, and its kernels one by one beside the
# like kernels of the models that were here.
def _zasorax_config(width, layers, heads, kv_heads, dim, chunk, far, rows, t_heads, t_kv, rot, ff, experts, top, expert_ff, vocab):
    chunked = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "bias_max": far, "mask": {"size": chunk},
               "bias_rows": rows}
    turned = {"heads": t_heads, "kv_heads": t_kv, "dim": dim, "vdim": dim, "scale": 0.3, "rot": {"base": 500000.0, "dims": rot}}
    dense = {"kind": "dense", "ff": ff}
    moe = {"kind": "moe", "expert": {"ff": expert_ff}, "router": {"experts": experts, "top": top}}
    stack = []
    for i in range(layers):
        place = i % 4
        if place == 2:
            stack.append({"type": "attention_2", "mixer": turned, "mlp": moe})
        else:  # the fourth layer of every four reads the pages of the second
            mixer = dict(chunked, kv_from=i - 2) if place == 3 else chunked
            stack.append({"type": "attention", "mixer": mixer, "mlp": dense if place == 0 else moe})
    return {"architecture": "Zasorax", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "embedding": {"scale": width ** 0.5},
            "layers": stack, "initializer_range": 0.02, "max_position_embeddings": 4096}


ZASORAX_SIZES = {
    # name: (Zasorax sizes, Rezulorn sizes); 8 layers each, vocabulary 32,768; a routed layer's chosen experts hold what
    # a dense feed-forward of the other design holds
    "width1024": (dict(width=1024, layers=8, heads=16, kv_heads=4, dim=64, chunk=1024, far=1024, rows=32, t_heads=16, t_kv=4, rot=32,
                       ff=4096, experts=32, top=4, expert_ff=704, vocab=32768),
                  REZULORN_SIZES["width1024"][0]),
    "width2048": (dict(width=2048, layers=8, heads=16, kv_heads=4, dim=128, chunk=1024, far=1024, rows=32, t_heads=16, t_kv=4, rot=64,
                       ff=8192, experts=32, top=4, expert_ff=1408, vocab=32768),
                  REZULORN_SIZES["width2048"][0]),
}


def _zasorax_prefill_flops(d: dict, tokens: int) -> float:
    w, dim = d["width"], d["dim"]
    in_chunk = sum(t % d["chunk"] + 1 for t in range(tokens))
    causal = tokens * (tokens + 1) // 2
    dense = 4 * w * d["ff"]
    routed = 6 * w * d["expert_ff"] * d["top"] + 2 * w * d["experts"]
    own = 2 * w * (d["heads"] + 2 * d["kv_heads"]) * dim + 2 * d["heads"] * dim * w
    reader = 2 * w * d["heads"] * dim + 2 * d["heads"] * dim * w
    turned = 2 * w * ((d["t_heads"] + 2 * d["t_kv"]) * dim + d["t_heads"]) + 2 * d["t_heads"] * dim * w
    total = 0.0
    for i in range(d["layers"]):
        place = i % 4
        if place == 2:
            total += (turned + routed) * tokens + 4 * d["t_heads"] * dim * causal
        else:
            total += ((reader if place == 3 else own) + (dense if place == 0 else routed)) * tokens + 4 * d["heads"] * dim * in_chunk
    return total + 2 * w * d["vocab"]


def _zasorax_kernel_table(d: dict, r: dict, peak: dict) -> dict:
    """The new design's kernels alone and the like kernels of the models that were here (the Rezulorn decoder's scored
    attention and cache writes, the transformer's residual add, the Pofadra decoder's whole-row norms, gate and router),
    each with its share of its roofline."""
    import torch

    from gtar_kimik3_public_b200.ops import functional as F
    from gtar_kimik3_public_b200.parts.scored_attention import distance_rows

    dev = torch.device("cuda:0")
    flush = torch.zeros(48 << 20, dtype=torch.float32, device=dev)  # 192 MB: larger than the 126 MB L2
    hbm, tflops = peak["hbm_gbs"] * 1e9, peak["bf16_tflops"] * 1e12
    out = {}

    def record(name, ms, n_bytes, flops=0.0):
        floor = max(n_bytes / hbm, flops / tflops) * 1e3
        out[name] = {"us": round(ms * 1e3, 2), "roofline_us": round(floor * 1e3, 2), "frac": round(floor / ms, 4),
                     "bound": "hbm" if n_bytes / hbm >= flops / tflops else "tensor"}

    w, dim, chunk = d["width"], d["dim"], d["chunk"]
    aq, ak, tq, tk = d["heads"], d["kv_heads"], d["t_heads"], d["t_kv"]
    window, keep = r["window"], r["keep"]
    bf = torch.bfloat16
    for label, tokens, n_seqs in (("prefill_2048", 2048, 1), ("decode_b8_ctx2048", 8, 8)):
        each = tokens // n_seqs
        inner = 1 if n_seqs == 1 else 20
        past = 0 if n_seqs == 1 else 2047
        length = past + each
        pages_each = -(-length // 64)
        table = torch.arange(n_seqs * pages_each, dtype=torch.int32, device=dev).view(n_seqs, pages_each)
        tok_seq = torch.arange(n_seqs, dtype=torch.int32, device=dev).repeat_interleave(each)
        tok_pos = (torch.arange(each, dtype=torch.int32, device=dev) + past).repeat(n_seqs)
        cu_q = torch.arange(n_seqs + 1, dtype=torch.int32, device=dev) * each
        slots = torch.arange(n_seqs, dtype=torch.int32, device=dev)
        kv_len = torch.full((n_seqs,), length, dtype=torch.int32, device=dev)

        def pages(n_heads, size):
            return F.PagedKV(torch.randn(n_seqs * pages_each, n_heads, 64, size, device=dev).to(bf) * 0.1,
                             torch.randn(n_seqs * pages_each, n_heads, 64, size, device=dev).to(bf) * 0.1, table, F.DecodeWork(dev))

        # ---- the stream: a branch's norm, its add and the stream's copy, beside the add with the next norm
        hs = torch.randn(tokens, w, device=dev)
        branch = torch.randn(tokens, w, device=dev).to(bf)
        wn = torch.ones(w, device=dev)
        ms = _event_ms(lambda: F.branch_merge(hs, branch, wn, 1e-6, copy_dtype=bf), flush=flush, inner=inner)
        record(f"zasorax branch norm, add and copy of the stream, {label}", ms, tokens * w * (4 + 2 + 4 + 2))
        ms = _event_ms(lambda: F.add_rmsnorm(hs, branch, wn, 1e-6, bf), flush=flush, inner=inner)
        record(f"transformer residual add with next norm, {label}", ms, tokens * w * (4 + 2 + 4 + 2))
        ms = _event_ms(lambda: F.add_layernorm(hs, branch, wn, 1e-5, torch.float32, delta_scale=0.5), flush=flush, inner=inner)
        record(f"rezulorn residual add with layer norm, {label}", ms, tokens * w * (4 + 2 + 4 + 4))
        # ---- activations behind the first product of a dense feed-forward
        wide_ff = torch.randn(tokens, d["ff"], device=dev).to(bf)
        ms = _event_ms(lambda: F.xielu(wide_ff, 0.8, 1.2), flush=flush, inner=inner)
        record(f"zasorax xIELU, {label}", ms, tokens * d["ff"] * 4)
        ms = _event_ms(lambda: F.relu_squared(wide_ff), flush=flush, inner=inner)
        record(f"rezulorn squared relu, {label}", ms, tokens * d["ff"] * 4)
        # ---- routers
        hb = torch.randn(tokens, w, device=dev).to(bf)
        w_r, bias = torch.randn(d["experts"], w, device=dev) * 0.5, torch.randn(d["experts"], device=dev)
        route_bytes = tokens * w * 2 + d["experts"] * w * 4 + tokens * d["top"] * 8
        ms = _event_ms(lambda: F.route_groups(hb, w_r, bias, d["top"], 1, 1, 1.0, logits=True), flush=flush, inner=inner)
        record(f"zasorax router (softmax over the chosen logits), {label}", ms, route_bytes)
        ms = _event_ms(lambda: F.route_groups(hb, w_r, bias, d["top"], 4, 2, 2.5), flush=flush, inner=inner)
        record(f"pofadra router (sigmoid scores, groups), {label}", ms, route_bytes)
        # ---- between the projection and attention
        kv = pages(ak, dim)
        wide = torch.randn(tokens, (aq + 2 * ak) * dim, device=dev).to(bf)
        wq, wk = torch.ones(aq * dim, device=dev), torch.ones(ak * dim, device=dev)
        prep_bytes = tokens * 2 * ((aq + 2 * ak) * dim + aq * dim + 2 * ak * dim)
        ms = _event_ms(lambda: F.wide_norm_rope_write(wide, aq, ak, dim, wq, wk, 1e-6, None, None, 0, tok_pos, tok_seq, slots, kv, length - 1,
                                                      v_at=(aq + ak) * dim), flush=flush, inner=inner)
        record(f"zasorax whole-row norms and cache write (own values), {label}", ms, prep_bytes)
        ms = _event_ms(lambda: F.wide_norm_rope_write(wide, aq, ak, dim, wq, wk, 1e-6, None, None, 0, tok_pos, tok_seq, slots, kv, length - 1),
                       flush=flush, inner=inner)
        record(f"pofadra whole-row norms and cache write (values are the keys), {label}", ms, tokens * 2 * ((aq + ak) * dim + aq * dim + 2 * ak * dim))
        ms = _event_ms(lambda: F.heads_prepare(wide, 0, aq * dim, (aq + ak) * dim, aq, ak, dim, dim, tok_pos, tok_seq, slots, kv=kv,
                                               max_position=length - 1), flush=flush, inner=inner)
        record(f"rezulorn cache write (no rotation), {label}", ms, prep_bytes)
        angle = torch.arange(length, dtype=torch.float32, device=dev)[:, None] * torch.rand(d["rot"] // 2, device=dev)[None, :]
        cos, sin = angle.cos().contiguous(), angle.sin().contiguous()
        v_angle = torch.arange(length, dtype=torch.float32, device=dev)[:, None] * torch.rand(dim // 2, device=dev)[None, :]
        v_cos, v_sin = v_angle.cos().contiguous(), v_angle.sin().contiguous()
        kvt = pages(tk, dim)
        widet = torch.randn(tokens, (tq + 2 * tk) * dim + 8 * -(-tq // 8), device=dev).to(bf)
        prep_t = tokens * 2 * ((tq + 2 * tk) * dim + tq * dim + 2 * tk * dim)
        ms = _event_ms(lambda: F.heads_prepare(widet, 0, tq * dim, (tq + tk) * dim, tq, tk, dim, dim, tok_pos, tok_seq, slots, rot=d["rot"],
                                               cos=cos, sin=sin, unit_eps=1e-6, kv=kvt, max_position=length - 1, v_cos=v_cos, v_sin=v_sin),
                       flush=flush, inner=inner)
        record(f"zasorax rotation, unit q and k, turned values, cache write, {label}", ms, prep_t)
        ms = _event_ms(lambda: F.heads_prepare(widet, 0, tq * dim, (tq + tk) * dim, tq, tk, dim, dim, tok_pos, tok_seq, slots, rot=d["rot"],
                                               cos=cos, sin=sin, unit_eps=1e-6, kv=kvt, max_position=length - 1), flush=flush, inner=inner)
        record(f"rezulorn rotation, unit q and k, cache write, {label}", ms, prep_t)
        # ---- attention
        qa = torch.randn(tokens, aq, dim, device=dev).to(bf)
        rel = torch.randn(d["rows"], aq, device=dev)
        dist = rel[torch.tensor(distance_rows(d["rows"], d["far"]), device=dev)].contiguous()
        temp, sink = torch.full((aq,), 0.9, device=dev), torch.full((aq,), 0.5, device=dev)
        seen = sum(p % chunk + 1 for p in range(past, length)) * n_seqs
        longest = min(length, chunk + each)
        parts = F.scored_attention_parts(n_seqs, aq, ak, each, -(-chunk // 64) + 2, F.sm_count(dev))
        ms = _event_ms(lambda: F.attention_scored(qa, kv, cu_q, kv_len, slots, each, dim ** -0.5, n_parts=parts, chunk=chunk, temp=temp,
                                                  dist_bias=dist, sink=sink), flush=flush, inner=inner)
        attn_bytes = 2 * (2 * tokens * aq * dim + 2 * n_seqs * longest * ak * dim)
        record(f"zasorax attention: chunks of {chunk}, distance table, head temperature, learned sink, {label}", ms, attn_bytes,
               4 * aq * dim * seen)
        ms = _event_ms(lambda: F.attention_scored_exact(qa, kv, tok_pos, tok_seq, slots, dim ** -0.5, chunk=chunk, temp=temp, dist_bias=dist,
                                                        sink=sink), flush=flush, inner=inner, repeats=3)
        record(f"zasorax attention, the same on the exact kernel (what 32-bit runs use), {label}", ms, attn_bytes, 4 * aq * dim * seen)
        r1, r2 = torch.full((aq,), 0.3, device=dev), torch.full((aq,), 0.5, device=dev)
        seen_r = sum(min(p + 1, window) + min(keep, max(0, p + 1 - window)) for p in range(past, length)) * n_seqs
        parts = F.scored_attention_parts(n_seqs, aq, ak, each, -(-(window + keep) // 64) + 2, F.sm_count(dev))
        ms = _event_ms(lambda: F.attention_scored(qa, kv, cu_q, kv_len, slots, each, dim ** -0.5, window, keep, r1, r2, None, "softmax", parts),
                       flush=flush, inner=inner)
        record(f"rezulorn attention: distance term, window {window} keeping {keep}, softmax, {label}", ms,
               2 * (2 * tokens * aq * dim + 2 * n_seqs * min(length, window + keep + each) * ak * dim), 4 * aq * dim * seen_r)
        qt = torch.randn(tokens, tq, dim, device=dev).to(bf)
        zero = torch.zeros(tq, device=dev)
        causal = sum(p + 1 for p in range(past, length)) * n_seqs
        parts = F.scored_attention_parts(n_seqs, tq, tk, each, pages_each, F.sm_count(dev))
        causal_bytes = 2 * (2 * tokens * tq * dim + 2 * n_seqs * length * tk * dim)
        ms = _event_ms(lambda: F.attention_scored(qt, kvt, cu_q, kv_len, slots, each, 0.3, n_parts=parts, sink=zero), flush=flush, inner=inner)
        record(f"zasorax attention: causal, one added to the denominator, {label}", ms, causal_bytes, 4 * tq * dim * causal)
        pb = torch.full((tq,), -4.0, device=dev)
        ms = _event_ms(lambda: F.attention_scored(qt, kvt, cu_q, kv_len, slots, each, 0.3, 0, 0, None, None, pb, "sigmoid", parts),
                       flush=flush, inner=inner)
        record(f"rezulorn attention: causal, sigmoid weights, {label}", ms, causal_bytes, 4 * tq * dim * causal)
        # ---- behind attention
        gate_at = (tq + 2 * tk) * dim
        ms = _event_ms(lambda: F.turn_back_gate(qt, v_cos, v_sin, tok_pos, length - 1, widet, gate_at), flush=flush, inner=inner)
        record(f"zasorax read-outs turned back, gate per head, {label}", ms, tokens * tq * dim * 4)
        flat = qt.view(tokens, tq * dim)
        gates = torch.randn(tokens, tq * dim, device=dev).to(bf)
        ms = _event_ms(lambda: F.sigmoid_gate(flat, gates, 0), flush=flush, inner=inner)
        record(f"pofadra gate per entry, {label}", ms, tokens * tq * dim * 6)
    return out


def run_compare_zasorax(args) -> dict:
    import gc

    import torch

    from gtar_kimik3_public_b200.ops.library import require_device

    require_device(torch.device("cuda:0"))
    peak, peak_source = peaks()
    results = {}
    for name, (d, r) in ZASORAX_SIZES.items():
        entry = {}
        for arch, raw, flops in (("zasorax", _zasorax_config(**d), _zasorax_prefill_flops(d, PREFILL_TOKENS)),
                                 ("rezulorn", _rezulorn_config(**r), _rezulorn_prefill_flops(r, PREFILL_TOKENS))):
            model = _device_model(raw)
            ms = _time_prefill_ms(model, PREFILL_TOKENS)
            decode = time_decode(model, args.batch, min(args.steps, 64), args.warmup)
            entry[arch] = {
                "weight_bytes_per_step": model.weight_bytes_per_step(),
                "prefill_tokens_per_s": round(PREFILL_TOKENS / (ms / 1e3), 1), "prefill_ms": round(ms, 3),
                "prefill_frac_of_bf16_peak": round(flops / (ms / 1e3) / (peak["bf16_tflops"] * 1e12), 4),
                "decode_tokens_per_s": round(decode["tokens_per_s"], 1), "decode_ms_per_step": round(decode["ms_per_step"], 4),
                "decode_frac_of_hbm_peak": round(decode["bytes_per_step"] / (decode["ms_per_step"] / 1e3) / 1e9 / peak["hbm_gbs"], 4),
                "decode_launches_per_step": decode["launches"] // max(1, min(args.steps, 64)),
            }
            if arch == "zasorax":
                # a step's weight bytes count the experts ONE token reads; a batch reads every distinct expert its tokens
                # choose: with uniform choices E (1 - (1 - top / E)^batch) of them in every routed layer
                distinct = d["experts"] * (1.0 - (1.0 - d["top"] / d["experts"]) ** args.batch)
                routed_layers = sum(1 for i in range(d["layers"]) if i % 4 != 0)
                more = routed_layers * (distinct - d["top"]) * 3 * d["expert_ff"] * d["width"] * 2
                entry[arch]["decode_expected_distinct_experts"] = round(distinct, 1)
                entry[arch]["decode_frac_of_hbm_peak_with_distinct_experts"] = round(
                    (decode["bytes_per_step"] + more) / (decode["ms_per_step"] / 1e3) / 1e9 / peak["hbm_gbs"], 4)
            del model
            gc.collect()
            torch.cuda.empty_cache()
        entry["kernels"] = _zasorax_kernel_table(d, r, peak)
        results[name] = {"sizes": {"zasorax": d, "rezulorn": r}, **entry}
    return {"compare": "zasorax beside rezulorn at equal width", "batch": args.batch, "prompt_tokens": PROMPT_LEN,
            "prefill_tokens": PREFILL_TOKENS, "dtype": "bf16", "data": "synthetic: random token ids, random weights drawn on the device",
            "peaks": dict(peak, source=peak_source), "l2": "single kernels: a 192 MB buffer is written between the timed calls of the 2,048-token cases; the 8-token cases are 20 calls back to back from a CUDA graph",
            "results": results}


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=256)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration (named in config)")
    parser.add_argument("--no-large", action="store_true", help="leave out the points at the 4B and 8B layer sizes")
    parser.add_argument("--compare", default=None, choices=["dasusun", "pofadra", "rezulorn", "zasorax"],
                        help="instead of the default workload: this architecture beside the transformer at equal layer sizes")
    args = parser.parse_args()
    if args.compare:
        if args.warmup < 3:
            args.warmup = 3
        runner = {"pofadra": run_compare_pofadra, "rezulorn": run_compare_rezulorn, "zasorax": run_compare_zasorax, "dasusun": run_compare}[args.compare]
        print(json.dumps(runner(args)))
        return 0
    if args.impl == "reference":
        if args.warmup < 3:
            args.warmup = 3
        print(json.dumps(run_reference(args)))
        return 0
    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) != 1:
        if int(os.environ.get("RANK", "0")) == 0:
            print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not supported (no distributed path is built)")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    print(json.dumps(run_ours(args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
