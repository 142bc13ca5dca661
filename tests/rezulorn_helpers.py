"""Shared pieces of the Rezulorn tests: tiny model folders written by the library's random-weights mode, the plain
implementation's logits for a request, and the error rules."""

from __future__ import annotations

import tempfile
from pathlib import Path

import torch

from tests.plain import rezulorn as plain
from tests.plain.weights import read_safetensors
from tests.rezulorn_configs import REZ_CONFIGS

WEIGHT_STD = 0.08
_folders: dict = {}
_weights: dict = {}
_logits: dict = {}


def rez_folder(tag: str, seed: int = 0) -> Path:
    key = (tag, seed)
    if key not in _folders:
        from gtar_kimik3_public_b200.registry import config_from_dict
        from gtar_kimik3_public_b200.weights import write_random_model

        holder = tempfile.TemporaryDirectory(prefix=f"gtar_test_{tag}_")
        write_random_model(holder.name, config_from_dict(REZ_CONFIGS[tag]), seed, std=WEIGHT_STD)
        _folders[key] = holder
    return Path(_folders[key].name)


def rez_weights(tag: str, seed: int = 0) -> dict:
    key = (tag, seed)
    if key not in _weights:
        _weights[key] = read_safetensors(rez_folder(tag, seed) / "model.safetensors")
    return _weights[key]


def rez_requests(tag: str, lengths, seed: int = 7) -> list[list[int]]:
    gen = torch.Generator().manual_seed(seed)
    return [torch.randint(0, REZ_CONFIGS[tag]["vocab"], (n,), generator=gen).tolist() for n in lengths]


def rez_plain_logits(tag: str, tokens, mode: str = "f64", seed: int = 0) -> torch.Tensor:
    key = (tag, tuple(tokens), mode, seed)
    if key not in _logits:
        ids = torch.tensor(list(tokens))
        if mode == "lowp":
            plain.LOWP = torch.bfloat16
            try:
                out = plain.forward(ids, rez_weights(tag, seed), REZ_CONFIGS[tag], torch.float32)
            finally:
                plain.LOWP = None
        else:
            out = plain.forward(ids, rez_weights(tag, seed), REZ_CONFIGS[tag], torch.float64 if mode == "f64" else torch.float32)
        _logits[key] = out
    return _logits[key]


def rez_engine(tag: str, dtype: str, max_tokens: int, seed: int = 0, max_seqs: int | None = None, **options):
    from gtar_kimik3_public_b200.engine import Engine
    from gtar_kimik3_public_b200.generate import load

    return Engine(load(rez_folder(tag, seed), dtype, "cuda:0"), max_tokens, max_seqs=max_seqs, **options)


def rez_check(tag: str, dtype: str, tokens, places, got: torch.Tensor, what: str) -> None:
    """float32: within 1e-4 of the float64 oracle on logits of size O(1).  bfloat16: the error against the oracle may be at
    most twice that of the plain implementation with bfloat16 matrix products, plus 2e-3 and half a bfloat16 step at the
    largest logit (for a request of one token the yardstick is a single sample of such steps)."""
    got = got.detach().double().cpu()
    assert torch.isfinite(got).all(), f"{what}: logits are not finite"
    oracle = rez_plain_logits(tag, tokens, "f64")[places]
    err = (got - oracle).abs().amax(-1)
    if dtype == "float32":
        assert err.max().item() < 1e-4, f"{what}: float32 logits differ from the oracle by {err.max().item():.3e}"
    else:
        yard = (rez_plain_logits(tag, tokens, "lowp")[places].double() - oracle).abs().amax(-1)
        assert err.max().item() <= 2 * yard.max().item() + 2e-3 + oracle.abs().max().item() / 256, \
            f"{what}: bfloat16 error {err.max().item():.3e} exceeds twice the yardstick {yard.max().item():.3e}"
