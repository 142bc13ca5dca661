"""Grouped-query attention with a rule for the scores and a rule for the weights.

``q = W_q x`` (``n_q_heads`` heads of ``key_dim``), ``k = W_k x`` and ``v = W_v x`` (``n_kv_heads`` heads of ``key_dim``
and ``value_dim``; query head ``h`` reads key/value head ``h // (n_q_heads / n_kv_heads)``), no biases.  The builder
chooses what happens around the scores:

* ``position``: the first ``position.dim`` entries of every q and k head are rotated by position (entry ``i`` paired with
  ``i + dim/2``), the rest pass; without it positions enter only through the rules below;
* ``unit_qk``: after the rotation every q and k head is divided by its root mean square (eps inside the root, no weight);
* the score of key ``j`` for the token at ``i`` is ``q . k * scale``; with ``distance_bias`` the term
  ``r1_h * ln(1 + r2_h * (i - j))`` is taken off, ``r1`` and ``r2`` being a number per query head (tensors ``r1``, ``r2``);
* visible keys: ``j <= i``, and with a ``window`` only those with ``i - j < window`` or ``j < keep_first``: the first
  tokens stay visible, at their true positions, after the window has left them;
* ``weights="softmax"``: the ordinary softmax over the visible keys; ``weights="sigmoid"``: a key's weight is
  ``sigmoid(score + pb_h)`` with a number per query head (tensor ``pb``, with ``head_bias``), and no sum over keys divides.

Scores, weights and the sums over keys are 32-bit.  A step's kernels: the packed projection q | k | v; one kernel for
rotation, unit lengths and the cache write; attention over the pages (on the tensor cores in bfloat16 with keys and
values of 64 or 128 entries, where steps of few tokens are cut over the keys into parts; else the exact kernel); the
output projection.
"""

from __future__ import annotations

import torch

from ..ops import functional as F
from ..ops.linear import linear
from .base import KVRequest, Mixer, PositionEncoding, StepContext, TensorSpec, register_part
from .delta_rule import _pad_rows

_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "r1": "r1", "r2": "r2", "pb": "pb"}


class ScoredAttention(Mixer):
    graph_safe = True

    def __init__(self, hidden_size: int, n_q_heads: int, n_kv_heads: int, key_dim: int, value_dim: int, scale: float,
                 norm_eps: float, position: PositionEncoding | None = None, unit_qk: bool = False, window: int | None = None,
                 keep_first: int = 0, distance_bias: bool = False, weights: str = "softmax", head_bias: bool = False,
                 names: dict[str, str] | None = None):
        if n_q_heads % n_kv_heads:
            raise ValueError("query heads must be a multiple of key heads")
        if weights not in ("softmax", "sigmoid"):
            raise ValueError(f"weights are 'softmax' or 'sigmoid', not {weights!r}")
        self.hidden_size, self.n_q, self.n_kv = int(hidden_size), int(n_q_heads), int(n_kv_heads)
        self.d, self.dv, self.scale, self.norm_eps = int(key_dim), int(value_dim), float(scale), float(norm_eps)
        self.position, self.unit_qk = position, bool(unit_qk)
        self.window = None if not window else int(window)
        self.keep_first = int(keep_first) if self.window else 0
        self.distance_bias, self.weights, self.head_bias = bool(distance_bias), weights, bool(head_bias)
        self.rot = 0 if position is None else int(position.dim)
        if self.rot > self.d:
            raise ValueError(f"{self.rot} rotated entries in heads of {self.d}")
        self.names = {**_NAMES, **(names or {})}
        self.w_in = self.w_o = self.r1 = self.r2 = self.pb = None

    def tensor_specs(self):
        n, W = self.names, self.hidden_size
        specs = {n["q"]: TensorSpec((self.n_q * self.d, W)), n["k"]: TensorSpec((self.n_kv * self.d, W)),
                 n["v"]: TensorSpec((self.n_kv * self.dv, W)), n["o"]: TensorSpec((W, self.n_q * self.dv))}
        if self.distance_bias:
            specs[n["r1"]] = TensorSpec((self.n_q,), "vector", init=(0.3, 0.1))
            specs[n["r2"]] = TensorSpec((self.n_q,), "vector", init=(0.5, 0.1))
        if self.head_bias:
            specs[n["pb"]] = TensorSpec((self.n_q,), "vector", init=(-2.0, 0.5))
        return specs

    def load(self, tensors):
        n = self.names
        mats = [tensors[n[key]] for key in ("q", "k", "v")]
        if len({m.dtype for m in mats}) != 1:
            mats = [m.float() for m in mats]
        self.w_in = _pad_rows(torch.cat(mats, dim=0)).contiguous()
        self.w_o = tensors[n["o"]].contiguous()
        if self.distance_bias:
            self.r1, self.r2 = tensors[n["r1"]].float().contiguous(), tensors[n["r2"]].float().contiguous()
        if self.head_bias:
            self.pb = tensors[n["pb"]].float().contiguous()

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.w_o))

    def cache_request(self):
        return KVRequest(self.n_kv, self.d, self.window, value_dim=None if self.dv == self.d else self.dv, keep_first=self.keep_first)

    def forward(self, x, ctx: StepContext, cache: F.PagedKV) -> torch.Tensor:
        cos = sin = None
        if self.rot:
            cos, sin = self.position.cos, self.position.sin
        write = not ctx.extras.get("cache_read_only", False)
        nq, nk = self.n_q * self.d, self.n_kv * self.d
        proj = linear(x, self.w_in)
        q = F.heads_prepare(proj, 0, nq, nq + nk, self.n_q, self.n_kv, self.d, self.dv, ctx.tok_pos, ctx.tok_seq, ctx.slots,
                            rot=self.rot, cos=cos, sin=sin, unit_eps=self.norm_eps if self.unit_qk else None, kv=cache,
                            write_kv=write, max_position=ctx.max_position)
        if q.dtype == torch.bfloat16 and self.d == self.dv and self.d in (64, 128) and cache.page_size == 64:
            # what a row can see at most, whatever the lengths of later steps that replay this one from a graph
            seen = -(-(self.window + self.keep_first) // 64) + 2 if self.window else cache.max_pages
            parts = F.scored_attention_parts(ctx.n_seqs, self.n_q, self.n_kv, ctx.max_q_len, min(seen, cache.max_pages),
                                             F.sm_count(q.device))
            o = F.attention_scored(q, cache, ctx.cu_q, ctx.kv_len, ctx.slots, ctx.max_q_len, self.scale, self.window or 0,
                                   self.keep_first, self.r1, self.r2, self.pb, self.weights, parts)
        else:  # 32-bit runs and other head sizes
            o = F.attention_scored_exact(q, cache, ctx.tok_pos, ctx.tok_seq, ctx.slots, self.scale, self.window or 0,
                                         self.keep_first, self.r1, self.r2, self.pb, self.weights)
        return linear(o.view(ctx.n_tokens, self.n_q * self.dv), self.w_o)


register_part("mixer", "scored_attention", ScoredAttention)
