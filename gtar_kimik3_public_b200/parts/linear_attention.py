"""A recurrent mixer: linear attention with a fixed decay per head.

Per head a state ``S [d, dv]`` of 32-bit floats, zero at the start of a sequence, is carried from token to token:

    S <- decay_h * S + k_t v_t^T ;   o_t = S^T q_t

with no softmax, no denominator and no other scale.  ``q_t, k_t`` (``n_heads`` heads of ``key_dim``) and ``v_t`` (heads
of ``value_dim``) are projections of the layer's input.  What stands between the projections and the recurrence, and
between the recurrence and the output projection, is chosen by the builder:

* ``activation="silu"``: SiLU on q, k and v;
* ``position``: the first ``position.dim`` entries of every q and k head are rotated by position (entry ``i`` paired
  with ``i + dim/2``), the rest pass;
* ``k_scale``: a constant on k (after the rotation);
* ``read_norm="all"``: the concatenated read-outs of all heads are divided by their common root mean square and
  multiplied by a weight of ``n_heads * value_dim`` entries (tensor ``norm``); ``read_norm="head"``: every head's
  read-out is divided by its own root mean square, no weight;
* ``gate="sigmoid"`` or ``"silu"``: the normed read-outs are multiplied by that function of a gate projection.

Everything from the activations to the gate is 32-bit.  What a sequence keeps between steps: the states of all heads.

A step's kernels: the packed projection q | k | v | gate; one kernel for activation, rotation and scale; the recurrence;
norm and gate; the output projection.  The recurrence runs token by token where a step brings few tokens a sequence
and in 32-bit runs (there a token's sums have the same order however a prompt is cut), and in chunks of 64 tokens whose
inner work is matrix products in bfloat16 runs with many tokens (the same numbers within 32-bit rounding).
"""

from __future__ import annotations

import torch

from ..ops import functional as F
from ..ops.linear import linear
from .base import Mixer, PositionEncoding, StateRequest, StepContext, TensorSpec, register_part
from .delta_rule import _pad_rows

_NAMES = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "norm": "norm"}


class DecayLinearAttention(Mixer):
    graph_safe = True  # kernels only; starts and slots are read from device memory
    chunked_from = 48  # steps whose longest sequence brings this many tokens take the chunked kernels (bfloat16 runs)

    def __init__(self, hidden_size: int, n_heads: int, key_dim: int, value_dim: int, decay, norm_eps: float,
                 activation: str | None = None, position: PositionEncoding | None = None, k_scale: float = 1.0,
                 read_norm: str = "head", gate: str = "sigmoid", names: dict[str, str] | None = None):
        self.hidden_size, self.n_heads, self.d, self.dv = int(hidden_size), int(n_heads), int(key_dim), int(value_dim)
        if min(self.hidden_size, self.n_heads, self.d, self.dv) <= 0:
            raise ValueError("linear attention sizes must be positive")
        self.decay_values = [float(g) for g in decay]
        if len(self.decay_values) != self.n_heads:
            raise ValueError(f"{len(self.decay_values)} decays for {self.n_heads} heads")
        if activation not in (None, "silu"):
            raise ValueError(f"activation is None or 'silu', not {activation!r}")
        if read_norm not in ("all", "head") or gate not in ("sigmoid", "silu"):
            raise ValueError("read_norm is 'all' or 'head', gate 'sigmoid' or 'silu'")
        self.norm_eps, self.activation, self.position, self.k_scale = float(norm_eps), activation, position, float(k_scale)
        self.read_norm, self.gate = read_norm, gate
        self.rot = 0 if position is None else int(position.dim)
        if self.rot > self.d:
            raise ValueError(f"{self.rot} rotated entries in heads of {self.d}")
        self.names = {**_NAMES, **(names or {})}
        self.w_in = self.w_o = self.norm_w = self.decay = None

    def tensor_specs(self):
        n, W, H, d, dv = self.names, self.hidden_size, self.n_heads, self.d, self.dv
        specs = {n["q"]: TensorSpec((H * d, W)), n["k"]: TensorSpec((H * d, W)), n["v"]: TensorSpec((H * dv, W)),
                 n["g"]: TensorSpec((H * dv, W)), n["o"]: TensorSpec((W, H * dv))}
        if self.read_norm == "all":
            specs[n["norm"]] = TensorSpec((H * dv,), "vector")
        return specs

    def load(self, tensors):
        n = self.names
        mats = [tensors[n[key]] for key in ("q", "k", "v", "g")]
        if len({m.dtype for m in mats}) != 1:
            mats = [m.float() for m in mats]
        self.w_in = _pad_rows(torch.cat(mats, dim=0)).contiguous()
        self.w_o = tensors[n["o"]].contiguous()
        self.norm_w = tensors[n["norm"]].float().contiguous() if self.read_norm == "all" else None
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=self.w_in.device)

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.w_o))

    def cache_request(self):
        return StateRequest((self.n_heads, self.d, self.dv), torch.float32)

    def forward(self, x, ctx: StepContext, cache) -> torch.Tensor:
        if ctx.extras.get("cache_read_only", False):
            raise ValueError("a recurrent mixer advances its state at every step: it cannot run on another entry's storage")
        H, d, dv = self.n_heads, self.d, self.dv
        cos = sin = None
        if self.rot:
            cos, sin = self.position.cos, self.position.sin
        silu = self.activation == "silu"
        proj = linear(x, self.w_in)
        q, k, v = F.heads_prepare(proj, 0, H * d, 2 * H * d, H, H, d, dv, ctx.tok_pos, ctx.tok_seq, ctx.slots, silu_qk=silu,
                                  silu_v=silu, rot=self.rot, cos=cos, sin=sin, k_scale=self.k_scale, max_position=ctx.max_position)
        if ctx.dtype == torch.bfloat16 and ctx.max_q_len >= self.chunked_from and F.decay_scan_chunked_fits(d, dv):
            o = F.decay_scan_chunked(q, k, v, self.decay, cache, ctx.cu_q, ctx.slots, ctx.n_seqs, ctx.max_q_len)
        else:  # few tokens a sequence, and 32-bit runs (whose numbers do not depend on how a prompt is cut)
            o = F.decay_scan(q, k, v, self.decay, cache, ctx.cu_q, ctx.slots, ctx.n_seqs)
        group = H * dv if self.read_norm == "all" else dv
        y = F.group_norm_gate(o.view(ctx.n_tokens, H * dv), group, self.norm_w, proj, 2 * H * d + H * dv, self.norm_eps, ctx.dtype,
                              self.gate)
        return linear(y, self.w_o)


register_part("mixer", "decay_linear_attention", DecayLinearAttention)
