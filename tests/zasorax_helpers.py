"""Shared pieces of the Zasorax tests: tiny model folders written by the library's random-weights mode, the plain
implementation's logits for a request, and the error rules."""

from __future__ import annotations

import tempfile
from pathlib import Path

import torch

from tests.plain import zasorax as plain
from tests.plain.weights import read_safetensors
from tests.zasorax_configs import ZAS_CONFIGS

WEIGHT_STD = 0.08
_folders: dict = {}
_weights: dict = {}
_logits: dict = {}


def zas_folder(tag: str, seed: int = 0) -> Path:
    key = (tag, seed)
    if key not in _folders:
        from gtar_kimik3_public_b200.registry import config_from_dict
        from gtar_kimik3_public_b200.weights import write_random_model

        holder = tempfile.TemporaryDirectory(prefix=f"gtar_test_{tag}_")
        write_random_model(holder.name, config_from_dict(ZAS_CONFIGS[tag]), seed, std=WEIGHT_STD)
        _folders[key] = holder
    return Path(_folders[key].name)


def zas_weights(tag: str, seed: int = 0) -> dict:
    key = (tag, seed)
    if key not in _weights:
        _weights[key] = read_safetensors(zas_folder(tag, seed) / "model.safetensors")
    return _weights[key]


def zas_requests(tag: str, lengths, seed: int = 7) -> list[list[int]]:
    gen = torch.Generator().manual_seed(seed)
    return [torch.randint(0, ZAS_CONFIGS[tag]["vocab"], (n,), generator=gen).tolist() for n in lengths]


def zas_plain_logits(tag: str, tokens, mode: str = "f64", seed: int = 0) -> torch.Tensor:
    key = (tag, tuple(tokens), mode, seed)
    if key not in _logits:
        ids = torch.tensor(list(tokens))
        if mode == "lowp":
            plain.LOWP = torch.bfloat16
            try:
                out = plain.forward(ids, zas_weights(tag, seed), ZAS_CONFIGS[tag], torch.float32)
            finally:
                plain.LOWP = None
        else:
            out = plain.forward(ids, zas_weights(tag, seed), ZAS_CONFIGS[tag], torch.float64 if mode == "f64" else torch.float32)
        _logits[key] = out
    return _logits[key]


CLOSE_CALL = 0.03  # of the router logits' spread
ALL_CHOSEN = ("zas_b", "zas_c")  # configurations whose routers choose every expert
_safe: dict = {}


def zas_safe_prefix(tag: str, tokens, seed: int = 0) -> int:
    """How many leading positions of the request are free of close routing calls in the oracle.  A layer of this design
    norms its feed-forward's result before the add, so ONE token that bfloat16 rounding sends to another expert changes
    that token's stream by order one, and through attention every later token's: from the first close call on, a
    bfloat16 run is not comparable with the oracle position by position.  (float32 runs are checked everywhere.)"""
    key = (tag, tuple(tokens), seed)
    if key not in _safe:
        calls: list = []
        plain.forward(torch.tensor(list(tokens)), zas_weights(tag, seed), ZAS_CONFIGS[tag], torch.float64, calls=calls)
        close = torch.zeros(len(tokens), dtype=torch.bool)
        for margins in calls:
            close |= margins < CLOSE_CALL
        hits = close.nonzero()
        _safe[key] = int(hits[0]) if hits.numel() else len(tokens)
    return _safe[key]


def zas_engine(tag: str, dtype: str, max_tokens: int, seed: int = 0, max_seqs: int | None = None, **options):
    from gtar_kimik3_public_b200.engine import Engine
    from gtar_kimik3_public_b200.generate import load

    return Engine(load(zas_folder(tag, seed), dtype, "cuda:0"), max_tokens, max_seqs=max_seqs, **options)


def zas_check(tag: str, dtype: str, tokens, places, got: torch.Tensor, what: str) -> None:
    """float32: within 1e-4 of the float64 oracle on logits of size O(1).  bfloat16: against the error of the plain
    implementation with bfloat16 matrix products and bfloat16 storage between them, the largest error over the positions
    may be at most three times the yardstick's largest and (over eight positions or more) the mean error at most one and a half
    times its mean, each plus
    2e-3 and half a bfloat16 step at the largest logit.  (Every branch of this design is normed before its add, so a
    position where a branch nearly cancels is sensitive, and how large its error comes out depends on the order of the
    roundings: the largest error is one sample, the mean is the measure of a systematic loss.)  Only positions before the
    request's first close routing call are compared in bfloat16 (``zas_safe_prefix``)."""
    got = got.detach().double().cpu()
    assert torch.isfinite(got).all(), f"{what}: logits are not finite"
    if dtype != "float32":
        safe = zas_safe_prefix(tag, tokens)
        assert tag not in ALL_CHOSEN or safe == len(tokens)
        keep = [k for k, place in enumerate(places) if place < safe]
        if not keep:
            return
        places, got = [places[k] for k in keep], got[keep]
    oracle = zas_plain_logits(tag, tokens, "f64")[places]
    err = (got - oracle).abs().amax(-1)
    if dtype == "float32":
        assert err.max().item() < 1e-4, f"{what}: float32 logits differ from the oracle by {err.max().item():.3e}"
    else:
        yard = (zas_plain_logits(tag, tokens, "lowp")[places].double() - oracle).abs().amax(-1)
        slack = 2e-3 + oracle.abs().max().item() / 256
        assert err.max().item() <= 3 * yard.max().item() + slack, \
            f"{what}: bfloat16 error {err.max().item():.3e} exceeds three times the yardstick {yard.max().item():.3e}"
        assert len(places) < 8 or err.mean().item() <= 1.5 * yard.mean().item() + slack, \
            f"{what}: mean bfloat16 error {err.mean().item():.3e} exceeds one and a half times the yardstick's {yard.mean().item():.3e}"
