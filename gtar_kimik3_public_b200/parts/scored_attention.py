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

Further rules, each switched on by the builder:

* ``wide_norm``: before anything else the whole query row (all heads at once) is divided by its root mean square and
  multiplied by a weight per entry (tensor ``q.norm``), and so is the whole key row (``k.norm``);
* ``temperature``: the product is multiplied by a number per query head (tensor ``temp``), ``q . k * scale * temp_h``;
* ``distance_table = (rows, far)``: a learned term per query head and distance is ADDED to the score (the scale does not
  touch it), read from ``rel [rows, heads]`` (a model file's tensor chooses ``rows``) at row ``bucket(i - j)``: ``bucket(n) = n`` below ``rows // 2``, then
  ``min(rows - 1, rows // 2 + floor(ln(n / (rows // 2)) / ln(far / (rows // 2)) * (rows - rows // 2)))``, so the rows'
  distances widen logarithmically up to ``far``;
* ``chunk``: a key is visible only from positions of its own chunk, ``i // chunk == j // chunk``, chunks counted from the
  sequence's first position (never from where a prompt was cut);
* ``sink``: the softmax's denominator holds one more term that has no key and no value: ``exp(sink_h)`` with a learned
  number per query head (``"learned"``, tensor ``sink``), or 1 (``"zero"``);
* ``value_position``: every value head is turned by ITS position over all of its entries (entry ``m`` paired with
  ``m + vdim/2``, frequencies ``base^(-2m/vdim)``) and cached so; every head's read-out is turned back by the READING
  position, so that a value enters a read-out turned by the distance between the two;
* ``head_gate``: every head's read-out is multiplied by the sigmoid of one number per head, ``W_g x`` (tensor ``g``
  ``[heads, hidden]``, packed behind the other input projections), before the output projection;
* ``own_kv`` False: the layer has no key and value tensors and reads the pages of an earlier layer (the model's run
  list names it), with its own queries and rules; ``cache_span`` is then, for the layer that owns the pages, how far
  back any of their readers look (None: every page is kept; by default the layer's own window or chunk).

Scores, weights and the sums over keys are 32-bit.  A step's kernels: the packed projection q | k | v | g; one kernel for
norms, rotation, unit lengths and the cache write; attention over the pages (on the tensor cores in bfloat16 with keys and
values of 64 or 128 entries, where steps of few tokens are cut over the keys into parts; else the exact kernel); the
read-outs' turn back and gate; the output projection.
"""

from __future__ import annotations

import math

import torch

from ..ops import functional as F
from ..ops.linear import linear
from .base import KVRequest, Mixer, PositionEncoding, StepContext, TensorSpec, register_part
from .delta_rule import _pad_rows

_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "r1": "r1", "r2": "r2", "pb": "pb", "q_norm": "q.norm", "k_norm": "k.norm",
          "temp": "temp", "rel": "rel", "sink": "sink", "g": "g"}


def distance_rows(rows: int, far: float) -> list[int]:
    """Which row of a distance table of ``rows`` rows each distance ``0 .. ceil(far)`` reads (every distance beyond reads
    the last row, as the last entry of the list does): a row a distance below ``rows // 2``, then logarithmically wider."""
    half = rows // 2
    if half < 1 or not far > half:
        raise ValueError(f"a distance table of {rows} rows cannot widen up to distance {far}")
    out = []
    for n in range(int(math.ceil(far)) + 1):
        out.append(n if n < half else min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half)))))
    return out


class ScoredAttention(Mixer):
    graph_safe = True

    def __init__(self, hidden_size: int, n_q_heads: int, n_kv_heads: int, key_dim: int, value_dim: int, scale: float,
                 norm_eps: float, position: PositionEncoding | None = None, unit_qk: bool = False, window: int | None = None,
                 keep_first: int = 0, distance_bias: bool = False, weights: str = "softmax", head_bias: bool = False,
                 names: dict[str, str] | None = None, wide_norm: bool = False, temperature: bool = False,
                 distance_table: tuple[int, float] | None = None, chunk: int | None = None, sink: str | None = None,
                 value_position: PositionEncoding | None = None, head_gate: bool = False, own_kv: bool = True,
                 cache_span: int | None | str = "own"):
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
        if sink not in (None, "learned", "zero"):
            raise ValueError(f"a sink is 'learned' or 'zero', not {sink!r}")
        if sink and weights != "softmax":
            raise ValueError("a sink belongs to the softmax")
        self.wide_norm, self.temperature, self.sink_kind = bool(wide_norm), bool(temperature), sink
        if self.wide_norm and (self.rot or self.unit_qk):
            raise ValueError("norms over whole rows come without rotation and unit lengths")
        self.distance_table = None if distance_table is None else (int(distance_table[0]), float(distance_table[1]))
        self.dist_rows = None  # formed at load: the table's height is the tensor's
        self.chunk = None if not chunk else int(chunk)
        self.value_position, self.head_gate, self.own_kv = value_position, bool(head_gate), bool(own_kv)
        if value_position is not None and (int(value_position.dim) != self.dv or self.dv % 2):
            raise ValueError(f"values of {self.dv} entries turn over all of them: the tables must have {self.dv} / 2 angles")
        # how far back the pages must reach: the layer's own window or chunk, or what the builder says their readers need
        spans = [s for s in (self.window, self.chunk) if s]
        if cache_span == "own":
            self.cache_span = min(spans) if spans else None
        else:  # the builder's word: a number of positions, or None for all
            self.cache_span = int(cache_span) if cache_span else None
        self.names = {**_NAMES, **(names or {})}
        self.w_in = self.w_o = self.r1 = self.r2 = self.pb = None
        self.q_norm = self.k_norm = self.temp = self.dist_bias = self.sink = None

    def tensor_specs(self):
        n, W = self.names, self.hidden_size
        specs = {n["q"]: TensorSpec((self.n_q * self.d, W))}
        if self.own_kv:
            specs[n["k"]] = TensorSpec((self.n_kv * self.d, W))
            specs[n["v"]] = TensorSpec((self.n_kv * self.dv, W))
        specs[n["o"]] = TensorSpec((W, self.n_q * self.dv))
        if self.distance_bias:
            specs[n["r1"]] = TensorSpec((self.n_q,), "vector", init=(0.3, 0.1))
            specs[n["r2"]] = TensorSpec((self.n_q,), "vector", init=(0.5, 0.1))
        if self.head_bias:
            specs[n["pb"]] = TensorSpec((self.n_q,), "vector", init=(-2.0, 0.5))
        if self.wide_norm:
            specs[n["q_norm"]] = TensorSpec((self.n_q * self.d,), "vector")
            if self.own_kv:
                specs[n["k_norm"]] = TensorSpec((self.n_kv * self.d,), "vector")
        if self.temperature:
            specs[n["temp"]] = TensorSpec((self.n_q,), "vector", init=(1.0, 0.3))
        if self.distance_table is not None:
            specs[n["rel"]] = TensorSpec((self.distance_table[0], self.n_q), "vector", init=(0.0, 0.5), free=(0,))
        if self.sink_kind == "learned":
            specs[n["sink"]] = TensorSpec((self.n_q,), "vector", init=(0.0, 1.0))
        if self.head_gate:
            specs[n["g"]] = TensorSpec((self.n_q, W), init=(0.0, 0.3))
        return specs

    def load(self, tensors):
        n = self.names
        mats = [tensors[n[key]] for key in (("q", "k", "v") if self.own_kv else ("q",))]
        self.gate_at = sum(m.shape[0] for m in mats)
        if self.head_gate:
            mats.append(tensors[n["g"]])
        if len({m.dtype for m in mats}) != 1:
            mats = [m.float() for m in mats]
        self.w_in = _pad_rows(torch.cat(mats, dim=0)).contiguous()
        self.w_o = tensors[n["o"]].contiguous()
        if self.distance_bias:
            self.r1, self.r2 = tensors[n["r1"]].float().contiguous(), tensors[n["r2"]].float().contiguous()
        if self.head_bias:
            self.pb = tensors[n["pb"]].float().contiguous()
        if self.wide_norm:
            self.q_norm = tensors[n["q_norm"]].float().contiguous()
            self.k_norm = tensors[n["k_norm"]].float().contiguous() if self.own_kv else self.q_norm
        if self.temperature:
            self.temp = tensors[n["temp"]].float().contiguous()
        if self.distance_table is not None:
            # one row a distance: the kernels read the term at min(distance, rows - 1) without forming the bucket
            rel = tensors[n["rel"]].float()
            self.distance_table = (int(rel.shape[0]), self.distance_table[1])
            self.dist_rows = distance_rows(*self.distance_table)
            reach = min(s for s in (self.window, self.chunk, len(self.dist_rows)) if s)
            if reach < len(self.dist_rows) and not self.keep_first:
                self.dist_rows = self.dist_rows[:reach]  # no visible key is further back than the chunk or window is long
            self.dist_bias = rel[torch.tensor(self.dist_rows, device=rel.device)].contiguous()
        if self.sink_kind == "learned":
            self.sink = tensors[n["sink"]].float().contiguous()
        elif self.sink_kind == "zero":
            self.sink = torch.zeros(self.n_q, dtype=torch.float32, device=self.w_o.device)

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.w_o))

    def cache_request(self):
        return KVRequest(self.n_kv, self.d, self.cache_span, value_dim=None if self.dv == self.d else self.dv,
                         keep_first=self.keep_first if self.cache_span == self.window else 0)

    def forward(self, x, ctx: StepContext, cache: F.PagedKV) -> torch.Tensor:
        cos = sin = v_cos = v_sin = None
        if self.rot:
            cos, sin = self.position.cos, self.position.sin
        if self.value_position is not None:
            v_cos, v_sin = self.value_position.cos, self.value_position.sin
        write = self.own_kv and not ctx.extras.get("cache_read_only", False)
        nq, nk = self.n_q * self.d, self.n_kv * self.d
        proj = linear(x, self.w_in)
        if self.wide_norm:
            q = F.wide_norm_rope_write(proj, self.n_q, self.n_kv, self.d, self.q_norm, self.k_norm, self.norm_eps, None, None, 0,
                                       ctx.tok_pos, ctx.tok_seq, ctx.slots, cache, ctx.max_position, write,
                                       v_at=nq + nk if self.own_kv else None, has_k=self.own_kv)
        else:
            k_at, v_at = (nq, nq + nk) if self.own_kv else (0, 0)
            q = F.heads_prepare(proj, 0, k_at, v_at, self.n_q, self.n_kv, self.d, self.dv, ctx.tok_pos, ctx.tok_seq, ctx.slots,
                                rot=self.rot, cos=cos, sin=sin, unit_eps=self.norm_eps if self.unit_qk else None, kv=cache,
                                write_kv=write, max_position=ctx.max_position, v_cos=v_cos if self.own_kv else None,
                                v_sin=v_sin if self.own_kv else None)
        rules = dict(chunk=self.chunk or 0, temp=self.temp, dist_bias=self.dist_bias, sink=self.sink)
        if q.dtype == torch.bfloat16 and self.d == self.dv and self.d in (64, 128) and cache.page_size == 64:
            # what a row can see at most, whatever the lengths of later steps that replay this one from a graph
            spans = [s for s in (self.window + self.keep_first if self.window else None, self.chunk) if s]
            seen = -(-min(spans) // 64) + 2 if spans else cache.max_pages
            parts = F.scored_attention_parts(ctx.n_seqs, self.n_q, self.n_kv, ctx.max_q_len, min(seen, cache.max_pages),
                                             F.sm_count(q.device))
            o = F.attention_scored(q, cache, ctx.cu_q, ctx.kv_len, ctx.slots, ctx.max_q_len, self.scale, self.window or 0,
                                   self.keep_first, self.r1, self.r2, self.pb, self.weights, parts, **rules)
        else:  # 32-bit runs and other head sizes
            o = F.attention_scored_exact(q, cache, ctx.tok_pos, ctx.tok_seq, ctx.slots, self.scale, self.window or 0,
                                         self.keep_first, self.r1, self.r2, self.pb, self.weights, **rules)
        if self.value_position is not None or self.head_gate:
            o = F.turn_back_gate(o, v_cos, v_sin, ctx.tok_pos, ctx.max_position, proj if self.head_gate else None, self.gate_at)
        return linear(o.view(ctx.n_tokens, self.n_q * self.dv), self.w_o)


register_part("mixer", "scored_attention", ScoredAttention)
