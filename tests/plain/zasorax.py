"""A plain, slow implementation of the Zasorax decoder, written from the design's equations.

Whole sequences, no cache, one function per mechanism, PyTorch in one working precision
(float64 for the oracle).  It shares no code with the library under test: it reads a dict of
tensors keyed by the model file's names and the config as a plain dict.

Notation: T tokens, W the model width; a mixer has H query heads and G key/value heads (query head
``h`` reads key/value head ``h // (H / G)``), ``d`` key entries and ``dv`` value entries per head.
A layer adds the NORMED result of each sublayer to the stream; the sublayers read the stream itself.
"""

from __future__ import annotations

import math

import torch

# When set to torch.bfloat16 every matrix product rounds its operands and its result to that type, while norms,
# angles, scores, weights, routers and the residual sums stay in the working precision: the "standard low-precision
# implementation" that the bfloat16 tests measure the library against.
LOWP: torch.dtype | None = None


def mm(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    if LOWP is None:
        return a @ b
    wide = a.dtype
    return (a.to(LOWP).to(wide) @ b.to(LOWP).to(wide)).to(LOWP).to(wide)


def kept(x: torch.Tensor) -> torch.Tensor:
    """What a low-precision run stores between two products (queries, cached keys and values, read-outs): rounded to the
    low precision; unchanged for the oracle."""
    return x if LOWP is None else x.to(LOWP).to(x.dtype)


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps): eps inside the root."""
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.log1p(torch.exp(-z.abs())) + z.clamp_min(0.0)


def distance_bucket(n: int, rows: int, far: float) -> int:
    """Row of the distance table for a key ``n`` back: one row a distance for the first half of the rows, then rows that
    widen logarithmically until distance ``far``, which (and everything beyond) reads the last row."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def turn(x: torch.Tensor, dims: int, base: float, backwards: bool = False) -> torch.Tensor:
    """x [T, heads, n]: the first ``dims`` entries of each head turn by position * f_i, entry i paired with i + dims/2,
    f_i = base^(-2i/dims); the rest pass.  ``backwards`` turns by minus the angle."""
    half = dims // 2
    f = base ** (-2.0 * torch.arange(half, dtype=x.dtype) / dims)
    a = torch.arange(x.shape[0], dtype=x.dtype)[:, None] * f[None, :]
    cos, sin = a.cos()[:, None, :], a.sin()[:, None, :]
    if backwards:
        sin = -sin
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], -1)


def softmax_with_sink(s: torch.Tensor, seen: torch.Tensor, sink: torch.Tensor | float) -> torch.Tensor:
    """Rows of weights exp(s_j) / (exp(sink) + sum over the seen keys of exp(s)): the sink adds to the denominator only."""
    s = s.masked_fill(~seen, -math.inf)
    sink = torch.as_tensor(sink, dtype=s.dtype)
    top = torch.maximum(s.amax(-1, keepdim=True), sink)
    e = torch.exp(s - top)
    return e / (e.sum(-1, keepdim=True) + torch.exp(sink - top))


def chunk_attention(h: torch.Tensor, w: dict, p: str, m: dict, eps: float, kv: tuple | None):
    """Attention without rotation: one RMS norm with a weight over the whole query row and one over the whole key row,
    a number per head on the scores, a table of distance terms, keys of the token's own chunk only, a learned sink per
    head.  ``kv``: keys and values of another layer to read instead of own ones.  Returns (branch, (k, v))."""
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = kept(rms(mm(h, w[p + "q"].T), eps) * w[p + "q.norm"]).view(T, H, d)
    if kv is None:
        k = kept(rms(mm(h, w[p + "k"].T), eps) * w[p + "k.norm"]).view(T, G, d)
        v = mm(h, w[p + "v"].T).view(T, G, dv)
    else:
        k, v = kv
    rel = w[p + "rel"]
    rows, far, size = rel.shape[0], m["bias_max"], m["mask"]["size"]
    i = torch.arange(T)
    seen = (i[:, None] >= i[None, :]) & ((i[:, None] // size) == (i[None, :] // size))
    row_of = torch.tensor([distance_bucket(n, rows, far) for n in range(T)])[(i[:, None] - i[None, :]).clamp_min(0)]
    outs = []
    for head in range(H):
        kh = head // (H // G)
        s = (q[:, head] @ k[:, kh].T) * m["scale"] * w[p + "temp"][head] + rel[:, head][row_of]
        outs.append(softmax_with_sink(s, seen, w[p + "sink"][head]) @ v[:, kh])
    o = kept(torch.stack(outs, 1)).reshape(T, H * dv)
    return mm(o, w[p + "o"].T), (k, v)


def turned_value_attention(h: torch.Tensor, w: dict, p: str, m: dict, eps: float, kv: tuple | None):
    """Causal attention with turned q and k, each head of both divided by its root mean square afterwards; values turned
    by their own position over all of their entries and every head's read-out turned back by the reading position; a
    softmax with one added to the denominator; a sigmoid gate per head."""
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    rot = m["rot"]
    q = kept(rms(turn(mm(h, w[p + "q"].T).view(T, H, d), rot["dims"], rot["base"]), eps))
    if kv is None:
        k = kept(rms(turn(mm(h, w[p + "k"].T).view(T, G, d), rot["dims"], rot["base"]), eps))
        v = kept(turn(mm(h, w[p + "v"].T).view(T, G, dv), dv, rot["base"]))
    else:
        k, v = kv
    i = torch.arange(T)
    seen = i[:, None] >= i[None, :]
    outs = []
    for head in range(H):
        kh = head // (H // G)
        s = (q[:, head] @ k[:, kh].T) * m["scale"]
        outs.append(softmax_with_sink(s, seen, 0.0) @ v[:, kh])
    o = turn(kept(torch.stack(outs, 1)), dv, rot["base"], backwards=True)
    gate = torch.sigmoid(mm(h, w[p + "g"].T))  # [T, H]
    return mm((o * gate[:, :, None]).reshape(T, H * dv), w[p + "o"].T), (k, v)


def xielu(z: torch.Tensor, numbers: torch.Tensor) -> torch.Tensor:
    """z > 0: softplus(p) z^2 + z/2;  z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2."""
    up, down = softplus(numbers[0]), 0.5 + softplus(numbers[1])
    return torch.where(z > 0, up * z * z + 0.5 * z, down * (torch.expm1(z.clamp_max(0.0)) - z) + 0.5 * z)


def dense_ff(h: torch.Tensor, w: dict, p: str) -> torch.Tensor:
    return mm(xielu(mm(h, w[p + "up"].T), w[p + "act"]), w[p + "down"].T)


def routed_ff(h: torch.Tensor, w: dict, p: str, mlp: dict, calls: list | None = None) -> torch.Tensor:
    """Router logits W_r h + b; the ``top`` largest are chosen and weighted by the softmax over the chosen logits alone.
    ``calls`` receives, per token, how far the last chosen logit lies above the first one not chosen, in units of the
    logits' spread (infinite where every expert is chosen): a small number is a close call that rounding may decide."""
    n, top = mlp["router"]["experts"], mlp["router"]["top"]
    seen = h if LOWP is None else h.to(LOWP).to(h.dtype)  # the router may read the rounding that the experts read
    z = seen @ w[p + "router"].T + w[p + "router.b"]
    if calls is not None:
        ranked = z.sort(-1, descending=True).values
        calls.append((ranked[:, top - 1] - ranked[:, top]) / z.std() if top < n else torch.full_like(z[:, 0], math.inf))
    best, ids = z.topk(top, dim=-1)
    share = torch.softmax(best, -1)
    out = torch.zeros_like(h)
    for e in range(n):
        rows, place = (ids == e).nonzero(as_tuple=True)
        if rows.numel() == 0:
            continue
        x = h[rows]
        g = mm(x, w[f"{p}e{e}.gate"].T)
        y = mm(g * torch.sigmoid(g) * mm(x, w[f"{p}e{e}.up"].T), w[f"{p}e{e}.down"].T)
        out[rows] += share[rows, place][:, None] * y
    return out


MIXERS = {"attention": chunk_attention, "attention_2": turned_value_attention}


def forward(tokens: torch.Tensor, weights: dict, config: dict, dtype=torch.float64, keep_layers: list | None = None,
            calls: list | None = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence.  ``keep_layers``: a list that receives the stream after every layer; ``calls``:
    a list that receives every routed layer's margins (see ``routed_ff``)."""
    w = {name: (t.to(dtype) if t.is_floating_point() else t) for name, t in weights.items()}
    eps = config["norm"]["eps"]
    x = w["embed"][tokens] * (config.get("embedding") or {"scale": 1.0})["scale"]
    kept: dict = {}
    for i, layer in enumerate(config["layers"]):
        m = layer["mixer"]
        source = m.get("kv_from")
        branch, kept[i] = MIXERS[layer["type"]](x, w, f"l{i}.mix.", m, eps, None if source is None else kept[source])
        x = x + rms(branch, eps) * w[f"l{i}.norm1"]
        mlp = layer.get("mlp")
        if mlp is not None:
            branch = dense_ff(x, w, f"l{i}.mlp.") if mlp["kind"] == "dense" else routed_ff(x, w, f"l{i}.mlp.", mlp, calls)
            x = x + rms(branch, eps) * w[f"l{i}.norm2"]
        if keep_layers is not None:
            keep_layers.append(x)
    return mm(rms(x, eps) * w["final.norm"], w["head"].T)
