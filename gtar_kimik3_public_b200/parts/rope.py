"""Rotary position encoding: tables of cos and sin of ``position * inv_freq``.

``inv_freq[i] = 1 / base^(2i/dim)`` is built in float32 by the reference's own expression and
the angle is a float32 product (src/layers/rope.py:8,11-14); the rotation pairs element ``i``
with ``i + dim/2`` (rope.py:17-19).  The tables hold the ``dim/2`` distinct angles per position
and are made on the device once, for as many positions as the cache can hold.
"""

from __future__ import annotations

import math

import torch

from .base import PositionEncoding, register_part


class RotaryEncoding(PositionEncoding):
    graph_safe = True

    def __init__(self, dim: int, base: float, precise: bool = False, divisor: float = 1.0):
        """``precise``: frequencies, angles, cosines and sines are formed in 64-bit and rounded once to the 32-bit
        tables (the default forms them in 32-bit, as the reference does).  ``divisor``: every frequency is divided by
        it (linear scaling of positions; 1 leaves them as they are)."""
        if dim % 2:
            raise ValueError(f"rotary dimension must be even, got {dim}")
        self.dim = int(dim)
        self.base = float(base)
        self.precise = bool(precise)
        self.divisor = float(divisor)
        if not self.divisor > 0:
            raise ValueError("the frequency divisor must be positive")
        self.cos: torch.Tensor | None = None
        self.sin: torch.Tensor | None = None
        self._replaced: list[torch.Tensor] = []  # shorter tables of before: captured launches may still read them

    def inv_freq(self) -> torch.Tensor:
        plain = 1.0 / (self.base ** (torch.arange(0, self.dim, 2, dtype=torch.float32) / self.dim))
        return plain / self.divisor if self.divisor != 1.0 else plain

    def magnitude(self) -> float:
        """A factor on every cosine and sine (1 for the plain rotation)."""
        return 1.0

    def prepare(self, max_position: int, device: torch.device) -> None:
        have = 0 if self.cos is None else self.cos.shape[0]
        if self.cos is not None and self.cos.device == device and have > max_position:
            return
        if self.cos is not None:
            # A CUDA graph captured earlier holds the old tables' addresses.  Their rows stay right (a row depends
            # on its position only), so they are kept instead of freed.
            self._replaced += [self.cos, self.sin]
        n = max(max_position + 1, 2 * have, 64)
        if self.precise:
            inv = self.base ** (-torch.arange(0, self.dim, 2, dtype=torch.float64) / self.dim) / self.divisor
            freqs = torch.arange(n, dtype=torch.float64)[:, None] * inv[None, :]
            self.cos = (freqs.cos() * self.magnitude()).float().to(device).contiguous()
            self.sin = (freqs.sin() * self.magnitude()).float().to(device).contiguous()
            return
        positions = torch.arange(n, dtype=torch.float32, device=device)
        freqs = positions[:, None] * self.inv_freq().to(device)[None, :]
        magnitude = self.magnitude()
        self.cos = (freqs.cos() * magnitude).contiguous() if magnitude != 1.0 else freqs.cos().contiguous()
        self.sin = (freqs.sin() * magnitude).contiguous() if magnitude != 1.0 else freqs.sin().contiguous()


class ScaledRotaryEncoding(RotaryEncoding):
    """Rotation whose slow frequencies are stretched for contexts longer than the ``original`` one (the YaRN rule).

    With ``d(t) = dim * ln(original / (2 pi t)) / (2 ln base)`` the index of the frequency that makes ``t`` turns over
    the original context, ``lo = max(floor(d(fast)), 0)``, ``hi = min(ceil(d(slow)), dim - 1)`` and ``ramp_i =
    clamp((i - lo) / max(hi - lo, 0.001), 0, 1)``, frequency ``i`` becomes ``f_i / factor * ramp_i + f_i * (1 - ramp_i)``:
    fast frequencies stay, slow ones are divided by ``factor``, a linear blend between.  Every cosine and sine is
    multiplied by ``0.1 ln(factor) + 1``.
    """

    def __init__(self, dim: int, base: float, factor: float, original: float, fast: float, slow: float):
        super().__init__(dim, base)
        if not factor > 0 or not original > 0 or not fast > 0 or not slow > 0:
            raise ValueError("scaling factor, original context and the two turn counts must be positive")
        self.factor, self.original, self.fast, self.slow = float(factor), float(original), float(fast), float(slow)

    def _turn_index(self, turns: float) -> float:
        return self.dim * math.log(self.original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.base))

    def inv_freq(self) -> torch.Tensor:
        plain = super().inv_freq()
        lo = max(math.floor(self._turn_index(self.fast)), 0)
        hi = min(math.ceil(self._turn_index(self.slow)), self.dim - 1)
        ramp = ((torch.arange(self.dim // 2, dtype=torch.float32) - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
        return plain / self.factor * ramp + plain * (1.0 - ramp)

    def magnitude(self) -> float:
        return 0.1 * math.log(self.factor) + 1.0


register_part("position", "rope", RotaryEncoding)
register_part("position", "rope_scaled", ScaledRotaryEncoding)
