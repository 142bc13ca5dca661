"""Zasorax's mechanisms one at a time on the GPU, each against the plain implementation's function for it: the norm of a
branch with its add and the copy of the stream, the activation of the dense feed-forward, the router that weights by the
softmax over the chosen logits (alone and inside the routed feed-forward, few and many tokens), the norms over whole rows
with values of their own, values turned into the cache and read-outs turned back and gated, and scored attention under
the rules of both mixers (chunks, the table by distance, a number per head on the product, learned and fixed sinks) with
keys that stand out far away, at page borders and on both sides of every chunk's edge, on the exact kernel and on the
tensor cores."""

import math

import pytest
import torch

from tests.plain import zasorax as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
PAGE = 64


def F():
    from gtar_kimik3_public_b200.ops import functional

    return functional


def _i32(values):
    return torch.tensor(list(values), dtype=torch.int32, device=DEV)


def _layout(lengths, starts=None):
    """tok_pos, tok_seq, cu_q for sequences that bring ``lengths`` tokens from positions ``starts`` on."""
    starts = starts or [0] * len(lengths)
    pos, seq, cu = [], [], [0]
    for s, (n, at) in enumerate(zip(lengths, starts)):
        pos += list(range(at, at + n))
        seq += [s] * n
        cu.append(cu[-1] + n)
    return _i32(pos), _i32(seq), _i32(cu)


def _paged(ks, vs, dtype, seed=0):
    """Pages that hold the sequences' keys ``ks[s] [L, G, d]`` and values ``vs[s] [L, G, dv]`` in a scrambled order, the
    rest NaN; slot of sequence ``s`` is ``n - 1 - s``."""
    n = len(ks)
    G, d, dv = ks[0].shape[1], ks[0].shape[2], vs[0].shape[2]
    per_seq = max(-(-k.shape[0] // PAGE) for k in ks)
    n_pages = n * per_seq + 3
    order = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed)).tolist()
    k_pages = torch.full((n_pages, G, PAGE, d), float("nan"), dtype=dtype, device=DEV)
    v_pages = torch.full((n_pages, G, PAGE, dv), float("nan"), dtype=dtype, device=DEV)
    table = torch.zeros(n, per_seq, dtype=torch.int32)
    slots = [n - 1 - s for s in range(n)]
    for s, (k, v) in enumerate(zip(ks, vs)):
        for i in range(-(-k.shape[0] // PAGE)):
            page = order.pop()
            table[slots[s], i] = page
            rows = slice(i * PAGE, min((i + 1) * PAGE, k.shape[0]))
            count = rows.stop - rows.start
            k_pages[page, :, :count] = k[rows].transpose(0, 1).to(dtype)
            v_pages[page, :, :count] = v[rows].transpose(0, 1).to(dtype)
    return F().PagedKV(k_pages, v_pages, table.to(DEV)), _i32(slots)


# ------------------------------------------------------------------ the norm of a branch, its add, the stream's copy
@pytest.mark.parametrize("width,branch_dtype,copy_dtype", [(88, torch.bfloat16, torch.bfloat16), (40, torch.float32, None),
                                                           (1027, torch.float32, torch.bfloat16), (2048, torch.bfloat16, torch.bfloat16)])
def test_branch_norm_add_and_copy(width, branch_dtype, copy_dtype):
    gen = torch.Generator(device=DEV).manual_seed(width)
    x = torch.randn(29, width, generator=gen, device=DEV) * 2.0
    y = (torch.randn(29, width, generator=gen, device=DEV) * 5.0 + 1.0).to(branch_dtype)
    weight = 1.0 + 0.2 * torch.randn(width, generator=gen, device=DEV)
    want = x.double().cpu() + plain.rms(y.double().cpu(), 1e-5) * weight.double().cpu()
    stream = x.clone()
    _, copy = F().branch_merge(stream, y, weight, 1e-5, copy_dtype=copy_dtype)
    assert (stream.double().cpu() - want).abs().max().item() < 2e-5
    if copy_dtype is None:
        assert copy is None
    else:
        assert copy.dtype == copy_dtype and torch.equal(copy, stream.to(copy_dtype)), "the copy is not the new stream's rounding"
    assert torch.equal(F().stream_cast(stream, torch.bfloat16), stream.to(torch.bfloat16))
    assert F().stream_cast(stream, torch.float32) is stream


# ------------------------------------------------------------------ the dense feed-forward's activation
@pytest.mark.parametrize("dtype,n", [(torch.float32, 1001), (torch.bfloat16, 4096), (torch.bfloat16, 77)])
def test_activation(dtype, n):
    gen = torch.Generator(device=DEV).manual_seed(n)
    z = (torch.randn(n, generator=gen, device=DEV) * 3.0).to(dtype)
    z[:3] = torch.tensor([0.0, -20.0, 20.0], device=DEV).to(dtype)
    numbers = torch.tensor([0.3, -0.7], dtype=torch.float64)
    up, down = plain.softplus(numbers[0]).item(), 0.5 + plain.softplus(numbers[1]).item()
    got = F().xielu(z, up, down)
    want = plain.xielu(z.double().cpu(), numbers)
    err = ((got.double().cpu() - want).abs() / (1.0 + want.abs())).max().item()
    assert err < (2e-6 if dtype == torch.float32 else 5e-3)


# ------------------------------------------------------------------ the router
@pytest.mark.parametrize("n_experts,top,T,W", [(6, 2, 50, 88), (3, 1, 7, 40), (4, 4, 33, 64), (40, 5, 130, 96)])
def test_router_weights_are_the_softmax_over_the_chosen_logits(n_experts, top, T, W):
    gen = torch.Generator(device=DEV).manual_seed(n_experts * T)
    h = torch.randn(T, W, generator=gen, device=DEV)
    w_r = torch.randn(n_experts, W, generator=gen, device=DEV) * 0.5
    bias = torch.randn(n_experts, generator=gen, device=DEV) * 2.0  # large enough to change choices
    ids, weights = F().route_groups(h, w_r, bias, top, 1, 1, 1.0, logits=True)
    z = h.double().cpu() @ w_r.double().cpu().T + bias.double().cpu()
    best, want_ids = z.topk(top, dim=-1)
    assert torch.equal(ids.cpu().long(), want_ids), "other experts than the largest logits (bias included)"
    assert (weights.double().cpu() - torch.softmax(best, -1)).abs().max().item() < 1e-5
    assert (weights.sum(-1) - 1.0).abs().max().item() < 1e-5
    without = (h.double().cpu() @ w_r.double().cpu().T).topk(top, dim=-1).indices
    assert n_experts == top or not torch.equal(without, want_ids), "the bias changes no choice: the test would not see it dropped"


@pytest.mark.parametrize("dtype,T", [(torch.float32, 9), (torch.bfloat16, 5), (torch.bfloat16, 300)])
def test_routed_feed_forward_against_the_plain_one(dtype, T):
    """Few tokens (every pair by itself) and many (pairs sorted by expert through grouped products)."""
    from gtar_kimik3_public_b200.parts.base import build_part

    W, ff, n, top = 64, 24, 5, 2
    gen = torch.Generator().manual_seed(T)
    w = {f"e{e}.{k}": (torch.randn(*(shape), generator=gen) * 0.1).to(torch.bfloat16).float()
         for e in range(n) for k, shape in (("gate", (ff, W)), ("up", (ff, W)), ("down", (W, ff)))}
    w["router"] = torch.randn(n, W, generator=gen) * 0.5
    w["router.b"] = torch.randn(n, generator=gen)
    part = build_part("feed_forward", "routed_experts", hidden_size=W, expert_size=ff, n_experts=n, top=top, logit_weights=True,
                      bias_name="router.b")
    part.load({name: t.to(DEV).to(torch.float32 if name.startswith("router") else dtype) for name, t in w.items()})
    h = (torch.randn(T, W, generator=gen) * 1.5).to(dtype)
    got = part.forward(h.to(DEV), None)
    plain.LOWP = None if dtype == torch.float32 else torch.bfloat16
    try:
        want = plain.routed_ff(h.double(), {"m." + k: t.double() for k, t in w.items()}, "m.", {"router": {"experts": n, "top": top}})
    finally:
        plain.LOWP = None
    assert got.dtype == torch.float32
    assert (got.double().cpu() - want).abs().max().item() < (2e-5 if dtype == torch.float32 else 3e-2)


# ------------------------------------------------------------------ norms over whole rows, values of their own
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,dv", [(6, 2, 16, 24), (3, 3, 12, 10), (4, 1, 64, 64)])
def test_whole_row_norms_write_keys_and_own_values(dtype, H, G, d, dv):
    gen = torch.Generator(device=DEV).manual_seed(H * d)
    lengths, starts = [70, 3], [60, 0]  # the first sequence's tokens cross a page border
    pos, seq, _ = _layout(lengths, starts)
    T = sum(lengths)
    nq, nk = H * d, G * d
    proj = (torch.randn(T, nq + nk + G * dv + 8, generator=gen, device=DEV) * 2.0).to(dtype)
    w_q = 1.0 + 0.2 * torch.randn(nq, generator=gen, device=DEV)
    w_k = 1.0 + 0.2 * torch.randn(nk, generator=gen, device=DEV)
    ks = [torch.zeros(a + n, G, d) for n, a in zip(lengths, starts)]
    vs = [torch.zeros(a + n, G, dv) for n, a in zip(lengths, starts)]
    kv, slots = _paged(ks, vs, dtype)
    q = F().wide_norm_rope_write(proj, H, G, d, w_q, w_k, 1e-5, None, None, 0, pos, seq, slots, kv, 200, True, v_at=nq + nk)
    p = proj.double().cpu()
    want_q = plain.rms(p[:, :nq], 1e-5) * w_q.double().cpu()
    want_k = plain.rms(p[:, nq:nq + nk], 1e-5) * w_k.double().cpu()
    tol = 1e-5 if dtype == torch.float32 else 3e-2
    assert (q.double().cpu().view(T, nq) - want_q).abs().max().item() < tol
    table = kv.block_table.cpu()
    for t in range(T):
        s, at = int(seq[t]), int(pos[t])
        page = int(table[int(slots[s]), at // PAGE])
        got_k = kv.k[page, :, at % PAGE].double().cpu().reshape(nk)
        got_v = kv.v[page, :, at % PAGE].double().cpu().reshape(G * dv)
        assert (got_k - want_k[t]).abs().max().item() < tol
        assert torch.equal(got_v, p[t, nq + nk:nq + nk + G * dv]), "values go into the pages as projected"
    # a row of queries only: the same queries, and no page is touched
    before_k, before_v = kv.k.clone(), kv.v.clone()
    alone = F().wide_norm_rope_write(proj[:, :nq].contiguous(), H, G, d, w_q, w_k, 1e-5, None, None, 0, pos, seq, slots, kv, 200,
                                     has_k=False)
    assert (alone.double() - q.double()).abs().max().item() < tol  # rows of other widths may take another form of the kernel
    assert torch.equal(kv.k.nan_to_num(), before_k.nan_to_num()) and torch.equal(kv.v.nan_to_num(), before_v.nan_to_num())


# ------------------------------------------------------------------ values turned into the cache, read-outs turned back
def _tables(dims, base, n=400):
    inv = base ** (-torch.arange(0, dims, 2, dtype=torch.float64) / dims)
    a = torch.arange(n, dtype=torch.float64)[:, None] * inv[None, :]
    return a.cos().float().to(DEV), a.sin().float().to(DEV)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,dv,rot", [(4, 1, 24, 16, 16), (5, 5, 10, 14, 6), (2, 2, 64, 64, 32)])
def test_values_are_cached_turned_by_their_position(dtype, H, G, d, dv, rot):
    gen = torch.Generator(device=DEV).manual_seed(H + dv)
    lengths, starts = [9, 70], [0, 120]
    pos, seq, _ = _layout(lengths, starts)
    T = sum(lengths)
    nq, nk = H * d, G * d
    proj = torch.randn(T, nq + nk + G * dv, generator=gen, device=DEV).to(dtype)
    cos, sin = _tables(rot, 37.0)
    v_cos, v_sin = _tables(dv, 37.0)
    ks = [torch.zeros(a + n, G, d) for n, a in zip(lengths, starts)]
    vs = [torch.zeros(a + n, G, dv) for n, a in zip(lengths, starts)]
    kv, slots = _paged(ks, vs, dtype)
    q = F().heads_prepare(proj, 0, nq, nq + nk, H, G, d, dv, pos, seq, slots, rot=rot, cos=cos, sin=sin, unit_eps=1e-5, kv=kv,
                          max_position=300, v_cos=v_cos, v_sin=v_sin)
    p = proj.double().cpu()
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    table = kv.block_table.cpu()
    for s, (n, a) in enumerate(zip(lengths, starts)):
        rows = slice(sum(lengths[:s]), sum(lengths[:s]) + n)
        pad = torch.zeros(a, 1, 1, dtype=torch.float64)
        whole_q = torch.cat([pad.expand(a, H, d), p[rows, :nq].view(n, H, d)])
        whole_k = torch.cat([pad.expand(a, G, d), p[rows, nq:nq + nk].view(n, G, d)])
        whole_v = torch.cat([pad.expand(a, G, dv), p[rows, nq + nk:].view(n, G, dv)])
        want_q = plain.rms(plain.turn(whole_q, rot, 37.0), 1e-5)[a:]
        want_k = plain.rms(plain.turn(whole_k, rot, 37.0), 1e-5)[a:]
        want_v = plain.turn(whole_v, dv, 37.0)[a:]
        assert (q[rows].double().cpu() - want_q).abs().max().item() < tol
        for t in range(n):
            at = a + t
            page = int(table[int(slots[s]), at // PAGE])
            assert (kv.k[page, :, at % PAGE].double().cpu() - want_k[t]).abs().max().item() < tol
            assert (kv.v[page, :, at % PAGE].double().cpu() - want_v[t]).abs().max().item() < tol
    if dv > 2:
        assert not torch.allclose(want_v, whole_v[a:]), "the turn changes nothing: the test would not see it dropped"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,dv,turned,gated", [(4, 16, True, True), (5, 14, True, False), (3, 64, False, True), (2, 128, True, True)])
def test_read_outs_turn_back_and_take_one_gate_a_head(dtype, H, dv, turned, gated):
    gen = torch.Generator(device=DEV).manual_seed(H * dv)
    lengths, starts = [5, 40], [0, 250]
    pos, _, _ = _layout(lengths, starts)
    T = sum(lengths)
    o = torch.randn(T, H, dv, generator=gen, device=DEV).to(dtype)
    wide = torch.randn(T, 11 + H, generator=gen, device=DEV).to(dtype) * 2.0
    cos, sin = _tables(dv, 5000.0) if turned else (None, None)
    got = F().turn_back_gate(o, cos, sin, pos, 300, wide if gated else None, 11)
    want = o.double().cpu()
    if turned:
        for (n, a), rows in zip(zip(lengths, starts), (slice(0, 5), slice(5, 45))):
            padded = torch.cat([torch.zeros(a, H, dv, dtype=torch.float64), want[rows]])
            want[rows] = plain.turn(padded, dv, 5000.0, backwards=True)[a:]
    if gated:
        want = want * torch.sigmoid(wide.double().cpu()[:, 11:])[:, :, None]
    assert (got.double().cpu() - want).abs().max().item() < (1e-5 if dtype == torch.float32 else 3e-2)


def test_turning_values_and_turning_back_gives_the_distance():
    """What the two turns are for: a value written at ``j`` and read at ``i`` has turned by ``j - i``."""
    dv, base = 8, 37.0
    v = torch.randn(50, 1, dv, dtype=torch.float64, generator=torch.Generator().manual_seed(3))
    there = plain.turn(v, dv, base)
    j, i = 13, 41
    one = torch.zeros(50, 1, dv, dtype=torch.float64)
    one[i] = there[j]  # the read-out at i is the cached value of j alone
    back = plain.turn(one, dv, base, backwards=True)[i, 0]
    for m in range(dv // 2):
        a = (j - i) * base ** (-2.0 * m / dv)
        assert math.isclose(back[m].item(), v[j, 0, m].item() * math.cos(a) - v[j, 0, m + dv // 2].item() * math.sin(a), abs_tol=1e-12)


# ------------------------------------------------------------------ scored attention under the two mixers' rules
def _plain_rules(q, k, v, scale, chunk, temp, rel, far, sink):
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H, dv] by the plain implementation's pieces."""
    q, k, v = q.double().cpu(), k.double().cpu(), v.double().cpu()
    T, H, G = q.shape[0], q.shape[1], k.shape[1]
    i = torch.arange(T)
    seen = i[:, None] >= i[None, :]
    if chunk:
        seen &= (i[:, None] // chunk) == (i[None, :] // chunk)
    outs = []
    for head in range(H):
        s = (q[:, head] @ k[:, head // (H // G)].T) * scale
        if temp is not None:
            s = s * temp[head].item()
        if rel is not None:
            rows = torch.tensor([plain.distance_bucket(n, rel.shape[0], far) for n in range(T)])
            s = s + rel.double().cpu()[:, head][rows[(i[:, None] - i[None, :]).clamp_min(0)]]
        if sink is None:
            weights = torch.softmax(s.masked_fill(~seen, -math.inf), -1)
        else:
            weights = plain.softmax_with_sink(s, seen, sink[head].item())
        outs.append(weights @ v[:, head // (H // G)])
    return torch.stack(outs, 1)


def _rules(H, rel, far, temp, sink, gen):
    """The kernels' arguments for a layer's learned numbers (the table by distance as the part lays it out)."""
    from gtar_kimik3_public_b200.parts.scored_attention import distance_rows

    dist = None if rel is None else rel[torch.tensor(distance_rows(rel.shape[0], far), device=DEV)].contiguous()
    return dict(temp=temp, dist_bias=dist, sink=sink)


RULES = [
    # H, G, d, dv, chunk, table rows, far, temp, sink
    (6, 2, 16, 24, 17, 10, 40, True, "learned"),
    (4, 2, 64, 64, 64, 16, 64, True, "learned"),
    (2, 1, 128, 128, 65, 7, 200, True, "learned"),
    (3, 3, 12, 10, 1, 2, 3, True, "learned"),
    (2, 1, 20, 6, 200, 9, 128, True, "learned"),
    (4, 1, 20, 6, 5, 5, 6, False, "learned"),
    (4, 1, 24, 16, 0, 0, 0, False, "zero"),
    (4, 4, 64, 64, 0, 0, 0, False, "zero"),
    (3, 1, 128, 128, 0, 0, 0, False, "zero"),
    (5, 5, 10, 14, 0, 0, 0, False, None),
    (4, 2, 64, 64, 100, 0, 0, False, None),
]


def _learned(H, rows, temp, sink, gen):
    rel = torch.randn(rows, H, generator=gen, device=DEV) * 1.5 if rows else None
    t = (1.0 + 0.5 * torch.randn(H, generator=gen, device=DEV)).abs() + 0.2 if temp else None
    if sink == "learned":
        s = torch.randn(H, generator=gen, device=DEV) * 2.0
    else:
        s = torch.zeros(H, device=DEV) if sink == "zero" else None
    return rel, t, s


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,dv,chunk,rows,far,temp,sink", RULES)
def test_rules_prompts_portions_and_single_tokens(dtype, H, G, d, dv, chunk, rows, far, temp, sink):
    """Two sequences of unequal length in one launch: all their tokens; the last portion of each; their last tokens alone.
    Every row equals the plain implementation's, on the exact kernel and, where the sizes allow, on the tensor cores with
    the walk over the keys whole and in parts."""
    gen = torch.Generator(device=DEV).manual_seed(H * d + chunk)
    lengths = [201, 77]
    qs = [torch.randn(L, H, d, generator=gen, device=DEV).to(dtype) for L in lengths]
    ks = [torch.randn(L, G, d, generator=gen, device=DEV).to(dtype) for L in lengths]
    vs = [torch.randn(L, G, dv, generator=gen, device=DEV).to(dtype) for L in lengths]
    rel, t, s = _learned(H, rows, temp, sink, gen)
    scale = d ** -0.5
    kv, slots = _paged(ks, vs, dtype)
    want = [_plain_rules(q, k, v, scale, chunk, t, rel, far, s) for q, k, v in zip(qs, ks, vs)]
    rules = _rules(H, rel, far, t, s, gen)
    tol = 3e-5 if dtype == torch.float32 else 4e-2
    exact = []
    for starts in ([0, 0], [139, 70], [200, 76]):
        pos, seq, cu = _layout([L - a for L, a in zip(lengths, starts)], starts)
        q = torch.cat([q[a:] for q, a in zip(qs, starts)]).contiguous()
        ref = torch.cat([w[a:] for w, a in zip(want, starts)])
        got = F().attention_scored_exact(q, kv, pos, seq, slots, scale, chunk=chunk, **rules)
        assert torch.isfinite(got).all()
        assert (got.double().cpu() - ref).abs().max().item() < tol, f"queries from {starts}"
        exact.append(got)
        if dtype == torch.bfloat16 and d == dv and d in (64, 128):
            for parts in (1, 2, 5):
                fast = F().attention_scored(q, kv, cu, _i32(lengths), slots, max(L - a for L, a in zip(lengths, starts)), scale,
                                            n_parts=parts, chunk=chunk, **rules)
                assert (fast.double().cpu() - ref).abs().max().item() < tol, f"tensor cores, queries from {starts}, {parts} parts"
    whole = exact[0]
    assert torch.equal(exact[1], torch.cat([whole[139:201], whole[201 + 70:]])), "a portion's rows are not the whole prompt's"
    assert torch.equal(exact[2], torch.stack([whole[200], whole[201 + 76]])), "a single token's row is not the whole prompt's"


def test_a_sink_takes_its_share_and_nothing_else():
    """One token that sees itself alone (a chunk of one): the read-out is its value times 1 / (1 + exp(sink - score))."""
    H, d, dv = 2, 16, 8
    q = torch.zeros(3, H, d, device=DEV)
    k = torch.zeros(3, 1, d, device=DEV)
    v = torch.ones(3, 1, dv, device=DEV) * 4.0
    q[:, :, 0], k[:, :, 0] = 2.0, 1.5  # every score: 3 * scale
    sink = torch.tensor([math.log(3.0), -1.0], device=DEV)
    kv, slots = _paged([k], [v], torch.float32)
    pos, seq, _ = _layout([3])
    got = F().attention_scored_exact(q, kv, pos, seq, slots, 0.5, chunk=1, sink=sink)
    for head in range(H):
        share = math.exp(1.5) / (math.exp(1.5) + math.exp(sink[head].item()))
        assert torch.allclose(got[:, head], torch.full((3, dv), 4.0 * share, device=DEV), atol=1e-5)
    none = F().attention_scored_exact(q, kv, pos, seq, slots, 0.5, chunk=1)
    assert torch.allclose(none, torch.full((3, H, dv), 4.0, device=DEV), atol=1e-6), "without a sink the weights sum to one"


def _standout(L, H, G, d, dv, dtype, seed):
    gen = torch.Generator(device=DEV).manual_seed(seed)
    q = (torch.randn(L, H, d, generator=gen, device=DEV) * 0.05).to(dtype)
    k = (torch.randn(L, G, d, generator=gen, device=DEV) * 0.05).to(dtype)
    v = (torch.randn(L, G, dv, generator=gen, device=DEV) * 0.05).to(dtype)
    return q, k, v


EDGES = [
    # chunk, reader i, key j, seen
    (0, 700, 3, True),         # far back, no chunk
    (0, 700, 63, True),        # the last place of the first page
    (0, 700, 64, True),        # the first place of the second
    (0, 700, 700, True),       # the token itself
    (120, 700, 600, True),     # the first key of the reader's chunk
    (120, 700, 599, False),    # the last key of the chunk before, 101 back: nearer than a chunk's length, still hidden
    (120, 719, 600, True),     # from the chunk's last position
    (120, 720, 719, False),    # the first position of a chunk sees nothing of the one before, not even its neighbour
    (120, 720, 720, True),
    (64, 200, 192, True),      # a chunk of a page: its first key
    (64, 200, 191, False),
    (64, 191, 128, True),
    (65, 200, 195, True),      # a chunk of a page and one
    (65, 200, 194, False),
    (33, 127, 99, True),       # an edge in the middle of a block of 32 keys
    (33, 127, 98, False),
    (32, 128, 128, True),      # an edge on a block's border
    (32, 128, 127, False),
    (1, 300, 300, True),       # a chunk of the token itself
    (1, 300, 299, False),
    (500, 40, 1, True),        # a chunk longer than the sequence
    (7, 3, 0, True),           # the first tokens of a sequence
    (300, 650, 600, True),     # several pages inside a chunk
    (300, 650, 599, False),
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("chunk,i,j,seen", EDGES)
def test_rules_see_one_key_or_not(dtype, chunk, i, j, seen):
    """Among hundreds of small keys one is made to stand out for the query at ``i`` (its score is large, its value is 100
    in one entry).  If ``j`` is visible from ``i`` that entry of the output is near 100, else near 0: in a whole prompt,
    and for the token at ``i`` alone over the cache.  The distance table, the numbers on the products and the sinks are
    small beside the score that stands out."""
    H, G, d, dv = 4, 2, 16, 24
    L = i + 5
    q, k, v = _standout(L, H, G, d, dv, dtype, i + j)
    head, kv_head = 3, 1
    q[i, head] = 0.0
    q[i, head, 2] = 8.0
    k[j, kv_head, 2] = 8.0
    v[j, kv_head] = 0.0
    v[j, kv_head, 7] = 100.0
    gen = torch.Generator(device=DEV).manual_seed(i)
    rel = torch.randn(12, H, generator=gen, device=DEV)
    temp = torch.full((H,), 0.8, device=DEV)
    sink = torch.full((H,), 2.0, device=DEV)
    rules = _rules(H, rel, 90.0, temp, sink, gen)
    kv, slots = _paged([k], [v], dtype, seed=j)
    want = _plain_rules(q, k, v, 0.5, chunk, temp, rel, 90.0, sink)
    for first in (0, i):
        pos, seq, _ = _layout([L - first if first == 0 else 1], [first])
        rows = q[first:] if first == 0 else q[i:i + 1]
        got = F().attention_scored_exact(rows.contiguous(), kv, pos, seq, slots, 0.5, chunk=chunk, **rules)
        at = i - first
        value = got[at, head, 7].item()
        assert (value > 90.0) == seen and (abs(value) < 2.0) != seen, f"key {j} from {i}: {value}"
        ref = want[first:] if first == 0 else want[i:i + 1]
        assert (got.double().cpu() - ref).abs().max().item() < (2e-4 if dtype == torch.float32 else 0.4)


@pytest.mark.parametrize("parts", [1, 4])
@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("chunk,i,j,seen", EDGES)
def test_tensor_core_rules_see_one_key_or_not(parts, d, chunk, i, j, seen):
    """The key that stands out through the tensor-core kernel: in a whole prompt, in a portion that starts in the middle of
    a tile of rows, and for the token at ``i`` alone; the walk over the keys whole and in parts (the sink counts once)."""
    H, G = 4, 2
    L = i + 5
    dtype = torch.bfloat16
    q, k, v = _standout(L, H, G, d, d, dtype, i + j)
    head, kv_head = 3, 1
    q[i, head] = 0.0
    q[i, head, 2] = 8.0
    k[j, kv_head, 2] = 8.0
    v[j, kv_head] = 0.0
    v[j, kv_head, 7] = 100.0
    gen = torch.Generator(device=DEV).manual_seed(i)
    rel = torch.randn(12, H, generator=gen, device=DEV)
    temp = torch.full((H,), 0.8, device=DEV)
    sink = torch.full((H,), 2.0, device=DEV)
    rules = _rules(H, rel, 90.0, temp, sink, gen)
    kv, slots = _paged([k], [v], dtype, seed=j)
    want = _plain_rules(q, k, v, 0.5, chunk, temp, rel, 90.0, sink)
    for first in sorted({0, max(0, i - 37), i}):
        rows = q[first:].contiguous() if first < i else q[i:i + 1].contiguous()
        lengths = [L if first < i else i + 1]
        _, _, cu = _layout([lengths[0] - first], [first])
        got = F().attention_scored(rows, kv, cu, _i32(lengths), slots, lengths[0] - first, 0.5, n_parts=parts, chunk=chunk, **rules)
        value = got[i - first, head, 7].item()
        assert (value > 90.0) == seen and (abs(value) < 2.0) != seen, f"key {j} from {i} (rows from {first}): {value}"
        ref = want[first:] if first < i else want[i:i + 1]
        assert (got.double().cpu() - ref).abs().max().item() < 0.4


def test_a_sink_weighs_in_when_no_key_stands_out():
    """Small scores everywhere and a large sink: the read-outs shrink by the sink's share, on both kernels and however the
    walk over the keys is cut (the sink must count once, not once a part)."""
    H, G, d = 4, 2, 64
    L = 300
    q, k, v = _standout(L, H, G, d, d, torch.bfloat16, 5)
    v = v + 1.0
    sink = torch.tensor([0.0, 3.0, 6.0, -40.0], device=DEV)
    kv, slots = _paged([k], [v], torch.bfloat16)
    want = _plain_rules(q, k, v, 0.5, 0, None, None, 0, sink)
    pos, seq, cu = _layout([L])
    exact = F().attention_scored_exact(q, kv, pos, seq, slots, 0.5, sink=sink)
    assert (exact.double().cpu() - want).abs().max().item() < 2e-2
    for parts in (1, 2, 5):
        fast = F().attention_scored(q, kv, cu, _i32([L]), slots, L, 0.5, n_parts=parts, sink=sink)
        assert (fast.double().cpu() - want).abs().max().item() < 2e-2, f"{parts} parts"
    # position 0 sees one key: shares 1/2, 1/(1 + e^3), 1/(1 + e^6), 1
    shares = [1 / (1 + math.exp(s)) for s in (0.0, 3.0, 6.0, -40.0)]
    for head, share in enumerate(shares):
        assert abs(exact[0, head, 0].item() / v[0, head // 2, 0].item() - share) < 2e-2
