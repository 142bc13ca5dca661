"""A plain, slow implementation of the Rezulorn decoder, written from the design's equations.

Whole sequences, no cache, one function per mechanism, PyTorch in one working precision
(float64 for the oracle).  It shares no code with the library under test: it reads a dict of
tensors keyed by the model file's names and the config as a plain dict.

Notation: T tokens, W the model width; a mixer has H heads (G key/value heads where they are
fewer; query head ``h`` reads key/value head ``h // (H / G)``), ``d`` key entries and ``dv``
value entries per head.
"""

from __future__ import annotations

import math

import torch

# When set to torch.bfloat16 every matrix product rounds its operands and its result to that type, while
# norms, angles, scores, weights, the recurrences and the residual sums stay in the working precision: the
# "standard low-precision implementation" that the bfloat16 tests measure the library against.
LOWP: torch.dtype | None = None


def mm(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    if LOWP is None:
        return a @ b
    wide = a.dtype
    return (a.to(LOWP).to(wide) @ b.to(LOWP).to(wide)).to(LOWP).to(wide)


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps): eps inside the root."""
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def layer_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """(x - mean) / sqrt(var + eps) * weight, var the mean of squared deviations; no bias."""
    mean = x.mean(-1, keepdim=True)
    dev = x - mean
    return dev / torch.sqrt(dev.pow(2).mean(-1, keepdim=True) + eps) * weight


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def with_time_conv(h: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """h [T, W], w [W, taps]: h_t + sum_j w[:, j] * h_(t - taps + 1 + j), zeros before the start."""
    taps = w.shape[1]
    y = h.clone()
    for j in range(taps):
        back = taps - 1 - j
        if back == 0:
            y = y + w[:, j] * h
        elif back < h.shape[0]:
            y[back:] = y[back:] + w[:, j] * h[:-back]
    return y


def turn(x: torch.Tensor, rot: dict | None) -> torch.Tensor:
    """x [T, heads, d]: the first rot.dims entries of each head turn by position * f_i, entry i paired with
    i + dims/2, f_i = base^(-2i/dims) / scaling.factor; the rest pass."""
    if not rot:
        return x
    dims, half = rot["dims"], rot["dims"] // 2
    f = rot["base"] ** (-2.0 * torch.arange(half, dtype=x.dtype) / dims)
    f = f / (rot.get("scaling") or {"factor": 1.0})["factor"]
    a = torch.arange(x.shape[0], dtype=x.dtype)[:, None] * f[None, :]
    cos, sin = a.cos()[:, None, :], a.sin()[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], -1)


def decayed_sum(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: float) -> torch.Tensor:
    """One head.  q, k [T, d]; v [T, dv].  S [d, dv] starts at zero; S = decay * S + k v^T; o = S^T q."""
    S = torch.zeros(q.shape[1], v.shape[1], dtype=q.dtype)
    out = []
    for t in range(q.shape[0]):
        S = decay * S + torch.outer(k[t], v[t])
        out.append(S.T @ q[t])
    return torch.stack(out)


def lightning(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    """Linear attention with SiLU on q, k and v, a decay per head, one RMS norm over all heads and a sigmoid gate."""
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = silu(mm(h, w[p + "q"].T)).view(T, H, d)
    k = silu(mm(h, w[p + "k"].T)).view(T, H, d)
    v = silu(mm(h, w[p + "v"].T)).view(T, H, dv)
    o = torch.stack([decayed_sum(q[:, i], k[:, i], v[:, i], m["decay"][i]) for i in range(H)], 1).reshape(T, H * dv)
    o = rms(o, eps) * w[p + "norm"] * torch.sigmoid(mm(h, w[p + "g"].T))
    return mm(o, w[p + "o"].T)


def retention(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    """Linear attention with turned q and k, k times d^-1/2, a decay per head, each head divided by its root mean
    square, a SiLU gate."""
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = turn(mm(h, w[p + "q"].T).view(T, H, d), m.get("rot"))
    k = turn(mm(h, w[p + "k"].T).view(T, H, d), m.get("rot")) * d ** -0.5
    v = mm(h, w[p + "v"].T).view(T, H, dv)
    o = torch.stack([rms(decayed_sum(q[:, i], k[:, i], v[:, i], m["decay"][i]), eps) for i in range(H)], 1).reshape(T, H * dv)
    return mm(o * silu(mm(h, w[p + "g"].T)), w[p + "o"].T)


def _visible(T: int, mask: dict | None) -> torch.Tensor:
    i = torch.arange(T)
    seen = i[:, None] >= i[None, :]
    if mask:
        near = (i[:, None] - i[None, :]) < mask["size"]
        seen &= near | (i[None, :] < mask.get("keep_first", 0))
    return seen


def visible(T: int, mask: dict | None) -> torch.Tensor:
    return _visible(T, mask)


def softmax_core(q, k, v, scale: float, mask: dict | None, r1=None, r2=None) -> torch.Tensor:
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H, dv]: softmax over the visible keys of
    q . k * scale - r1_h ln(1 + r2_h (i - j))."""
    T, H, G = q.shape[0], q.shape[1], k.shape[1]
    seen = _visible(T, mask)
    i = torch.arange(T, dtype=q.dtype)
    gap = (i[:, None] - i[None, :]).clamp_min(0.0)
    outs = []
    for head in range(H):
        kh = head // (H // G)
        s = (q[:, head] @ k[:, kh].T) * scale
        if r1 is not None:
            s = s - r1[head] * torch.log1p(r2[head] * gap)
        s = s.masked_fill(~seen, -math.inf)
        outs.append(torch.softmax(s, -1) @ v[:, kh])
    return torch.stack(outs, 1)


def sigmoid_core(q, k, v, scale: float, mask: dict | None, pb) -> torch.Tensor:
    """The same shapes: a visible key's weight is sigmoid(q . k * scale + pb_h); nothing divides."""
    T, H, G = q.shape[0], q.shape[1], k.shape[1]
    seen = _visible(T, mask)
    outs = []
    for head in range(H):
        kh = head // (H // G)
        s = (q[:, head] @ k[:, kh].T) * scale + pb[head]
        outs.append(torch.sigmoid(s).masked_fill(~seen, 0.0) @ v[:, kh])
    return torch.stack(outs, 1)


def biased_attention(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    """Softmax attention without rotation: score minus r1 ln(1 + r2 (i - j)); a sliding window that keeps the
    first tokens."""
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = turn(mm(h, w[p + "q"].T).view(T, H, d), m.get("rot"))
    k = turn(mm(h, w[p + "k"].T).view(T, G, d), m.get("rot"))
    v = mm(h, w[p + "v"].T).view(T, G, dv)
    o = softmax_core(q, k, v, m["scale"], m.get("mask"), w.get(p + "r1"), w.get(p + "r2"))
    return mm(o.reshape(T, H * dv), w[p + "o"].T)


def sigmoid_attention(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    """Causal attention whose weights are sigmoid(score + a number per head), not normalised; q and k turned by
    position and then divided by their root mean square."""
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = rms(turn(mm(h, w[p + "q"].T).view(T, H, d), m.get("rot")), eps)
    k = rms(turn(mm(h, w[p + "k"].T).view(T, G, d), m.get("rot")), eps)
    v = mm(h, w[p + "v"].T).view(T, G, dv)
    o = sigmoid_core(q, k, v, m["scale"], m.get("mask"), w[p + "pb"])
    return mm(o.reshape(T, H * dv), w[p + "o"].T)


def side_by_side(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    left = sigmoid_attention(h, w, p + "left.", m["left"], eps)
    right = retention(h, w, p + "right.", m["right"], eps)
    return m.get("left_scale", 1.0) * left + m.get("right_scale", 1.0) * right


def relu_squared_ff(h: torch.Tensor, w: dict, p: str) -> torch.Tensor:
    return mm(torch.relu(mm(h, w[p + "up"].T)).pow(2), w[p + "down"].T)


MIXERS = {"lightning": lightning, "attention": biased_attention, "parallel": side_by_side}


def forward(tokens: torch.Tensor, weights: dict, config: dict, dtype=torch.float64, keep_layers: list | None = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence.  ``keep_layers``: a list that receives the stream after every layer."""
    w = {name: (t.to(dtype) if t.is_floating_point() else t) for name, t in weights.items()}
    eps, mult = config["norm"]["eps"], config.get("residual_mult", 1.0)
    x = w["embed"][tokens]
    for i, layer in enumerate(config["layers"]):
        h = layer_norm(x, w[f"l{i}.norm1"], eps)
        if f"l{i}.canon1" in w:
            h = with_time_conv(h, w[f"l{i}.canon1"])
        x = x + mult * MIXERS[layer["type"]](h, w, f"l{i}.mix.", layer["mixer"], eps)
        if layer.get("mlp") is not None:
            h = layer_norm(x, w[f"l{i}.norm2"], eps)
            if f"l{i}.canon2" in w:
                h = with_time_conv(h, w[f"l{i}.canon2"])
            x = x + mult * relu_squared_ff(h, w, f"l{i}.mlp.")
        if keep_layers is not None:
            keep_layers.append(x)
    return mm(layer_norm(x, w["final.norm"], eps), w["head"].T) * config.get("logit_scale", 1.0)
