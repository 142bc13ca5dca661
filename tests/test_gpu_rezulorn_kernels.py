"""Rezulorn's mechanisms one at a time on the GPU, each against the plain implementation's function for it: the layer
norm with the pending add, the step between a packed projection and a mixer's core (SiLU, rotation, unit lengths, the
constant on keys, the cache write), the decayed recurrence (whole, in portions, batched, from slots used before), the
norm and gate behind it, and scored attention (distance term, window with kept first tokens, softmax and sigmoid
weights) with keys that stand out far away, at page borders and on both sides of every edge."""

import math

import pytest
import torch

from tests.plain import rezulorn as plain

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


# ------------------------------------------------------------------ layer norm
@pytest.mark.parametrize("width,out_dtype", [(88, torch.float32), (72, torch.bfloat16), (320, torch.float32), (1, torch.float32),
                                             (2048, torch.bfloat16), (4100, torch.float32)])
def test_layer_norm_with_pending_add(width, out_dtype):
    gen = torch.Generator(device=DEV).manual_seed(width)
    h = torch.randn(37, width, generator=gen, device=DEV) * 3.0 + 1.5  # a mean that is not zero
    delta = torch.randn(37, width, generator=gen, device=DEV).to(out_dtype)
    weight = 1.0 + 0.2 * torch.randn(width, generator=gen, device=DEV)
    summed = h.double() + 0.35 * delta.double()
    want = plain.layer_norm(summed.cpu(), weight.double().cpu(), 1e-5)
    stream = h.clone()
    got = F().add_layernorm(stream, delta, weight, 1e-5, out_dtype, delta_scale=0.35)
    assert torch.allclose(stream.double(), summed, atol=1e-6), "the stream does not hold the sum"
    tol = 2e-5 if out_dtype == torch.float32 else 2e-2
    assert (got.double().cpu() - want).abs().max().item() < tol
    # no pending branch; chosen rows only, the stream untouched
    rows = _i32([5, 0, 36])
    before = stream.clone()
    got = F().add_layernorm(stream, None, weight, 1e-5, torch.float32, rows=rows)
    assert torch.equal(stream, before)
    want = plain.layer_norm(before.double().cpu()[[5, 0, 36]], weight.double().cpu(), 1e-5)
    assert (got.double().cpu() - want).abs().max().item() < 2e-5


def test_layer_norm_is_not_an_rms_norm():
    """A row with a large mean: dividing by the root mean square instead of the deviation would be off by far."""
    h = torch.full((1, 64), 100.0, device=DEV)
    h[0, ::2] += 1.0
    got = F().add_layernorm(h, None, torch.ones(64, device=DEV), 1e-6, torch.float32)
    assert torch.allclose(got[0, ::2], torch.full((32,), 1.0, device=DEV), atol=1e-3)
    assert torch.allclose(got[0, 1::2], torch.full((32,), -1.0, device=DEV), atol=1e-3)


# ------------------------------------------------------------------ convolution in front of a sublayer
@pytest.mark.parametrize("taps,cuts", [(4, [50]), (4, [1, 1, 2, 3, 43]), (2, [7, 43]), (3, [2] * 25), (1, [20, 30])])
def test_time_convolution_in_portions(taps, cuts):
    width = 40
    gen = torch.Generator(device=DEV).manual_seed(taps)
    a = torch.randn(50, width, generator=gen, device=DEV)
    w = torch.randn(width, taps, generator=gen, device=DEV) * 0.5
    want = plain.with_time_conv(a.double().cpu(), w.double().cpu())
    weight = w.t().contiguous()
    state = torch.full((3, max(taps - 1, 0), width), float("nan"), device=DEV) if taps > 1 else None
    slot = 2
    if state is not None:
        state[slot] = 0.0
    got, at = [], 0
    for n in cuts:
        pos, seq, cu = _layout([n], [at])
        piece = a[at:at + n].contiguous()
        single = n == 1
        got.append(F().causal_conv(piece, weight, state, pos, seq, cu, _i32([slot]), torch.float32,
                                   update_single_token_state=single and state is not None))
        if state is not None and not single:
            F().conv_state(piece, state, cu, _i32([slot]), 1)
        at += n
    assert (torch.cat(got).double().cpu() - want).abs().max().item() < 1e-5


@pytest.mark.parametrize("taps,width,out_dtype", [(4, 40, torch.float32), (2, 72, torch.bfloat16), (1, 24, torch.float32),
                                                  (5, 2056, torch.float32)])
def test_norm_and_time_convolution_in_one_kernel_token_by_token(taps, width, out_dtype):
    """Three sequences of unequal age, one token each a step, in slots that are not in order: the stream gets the scaled
    branch, and what comes out is the plain norm through the plain convolution over each sequence's whole past."""
    steps, starts, slots = 9, [0, 2, 5], [3, 0, 2]
    gen = torch.Generator(device=DEV).manual_seed(taps * 100 + width)
    norm_w = 1.0 + 0.2 * torch.randn(width, generator=gen, device=DEV)
    w = torch.randn(width, taps, generator=gen, device=DEV) * 0.5
    weight = w.t().contiguous()
    state = torch.full((4, taps - 1, width), float("nan"), device=DEV) if taps > 1 else None
    # the rows every sequence has seen before its first step here, through the unfused kernels
    past = [torch.randn(n, width, generator=gen, device=DEV) * 2.0 + 0.5 for n in starts]
    normed = [[] for _ in starts]
    for s, rows in enumerate(past):
        if state is not None:
            state[slots[s]] = 0.0
        if rows.shape[0]:
            y = F().add_layernorm(rows.clone(), None, norm_w, 1e-5, torch.float32)
            normed[s].append(y)
            if state is not None:
                F().conv_state(y, state, _i32([0, rows.shape[0]]), _i32([slots[s]]), 1)
    outs = [[] for _ in starts]
    for step in range(steps):
        h = torch.randn(len(starts), width, generator=gen, device=DEV) * 2.0 + 0.5
        delta = torch.randn(len(starts), width, generator=gen, device=DEV).to(out_dtype)
        summed = h.double() + 0.4 * delta.double()
        pos, seq, _ = _layout([1] * len(starts), [at + step for at in starts])
        frozen = state.clone() if state is not None else None
        peek = F().add_layernorm_conv_single(h.clone(), delta, norm_w, 1e-5, weight, state, pos, seq, _i32(slots), out_dtype,
                                             delta_scale=0.4, update_state=False)
        if state is not None:
            assert torch.equal(state[slots], frozen[slots]), "a read-only step moved the states"
        stream = h.clone()
        got = F().add_layernorm_conv_single(stream, delta, norm_w, 1e-5, weight, state, pos, seq, _i32(slots), out_dtype,
                                            delta_scale=0.4)
        assert torch.equal(got, peek)
        assert torch.allclose(stream.double(), summed, atol=1e-6), "the stream does not hold the sum"
        for s in range(len(starts)):
            normed[s].append(plain.layer_norm(summed[s:s + 1].cpu(), norm_w.double().cpu(), 1e-5).to(DEV))
            outs[s].append(got[s])
    tol = 3e-5 if out_dtype == torch.float32 else 4e-2
    for s in range(len(starts)):
        want = plain.with_time_conv(torch.cat(normed[s]).double().cpu(), w.double().cpu())[starts[s]:]
        assert (torch.stack(outs[s]).double().cpu() - want).abs().max().item() < tol, f"sequence {s}"


# ------------------------------------------------------------------ between the projection and the core
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n_q,n_k,d,dv,rot,divisor,silu,unit,k_scale", [
    (4, 4, 24, 40, 0, 1.0, True, False, 1.0),        # SiLU on q, k and v, nothing else
    (2, 2, 40, 24, 40, 1.0, False, False, 40 ** -0.5),  # the whole head rotated, a constant on k
    (3, 3, 12, 20, 4, 0.5, False, False, 0.3),      # part of the head rotated, frequencies divided
    (6, 2, 16, 8, 8, 4.0, False, True, 1.0),        # rotation, then unit length
    (1, 1, 132, 260, 0, 1.0, True, True, 2.0),      # heads wider than a warp's first round
])
def test_heads_prepare_to_arrays(dtype, n_q, n_k, d, dv, rot, divisor, silu, unit, k_scale):
    from gtar_kimik3_public_b200.parts.base import build_part

    T = 23
    gen = torch.Generator(device=DEV).manual_seed(d)
    pad = 5
    proj = torch.randn(T, pad + n_q * d + n_k * d + n_k * dv + 3, generator=gen, device=DEV).to(dtype)
    starts = [0, 100]
    pos, seq, _ = _layout([10, 13], starts)
    cos = sin = None
    rot_cfg = None
    if rot:
        part = build_part("position", "rope", dim=rot, base=300.0, precise=True, divisor=divisor)
        part.prepare(256, torch.device(DEV))
        cos, sin = part.cos, part.sin
        rot_cfg = {"base": 300.0, "dims": rot, "scaling": {"factor": divisor}}
    q_at, k_at, v_at = pad, pad + n_q * d, pad + n_q * d + n_k * d
    q, k, v = F().heads_prepare(proj, q_at, k_at, v_at, n_q, n_k, d, dv, pos, seq, _i32([0, 1]), silu_qk=silu, silu_v=silu,
                                rot=rot, cos=cos, sin=sin, unit_eps=1e-5 if unit else None, k_scale=k_scale, max_position=112)
    p64 = proj.double().cpu()
    for got, at, n, width, is_k in ((q, q_at, n_q, d, False), (k, k_at, n_k, d, True), (v, v_at, n_k, dv, False)):
        x = p64[:, at:at + n * width].reshape(T, n, width).clone()
        if silu:
            x = plain.silu(x)
        if width == d and got is not v:
            for lo, n_tok, start in ((0, 10, 0), (10, 13, 100)):
                # positions are the tokens' own: the second sequence starts far from 0
                whole = torch.zeros(start + n_tok, n, width, dtype=torch.float64)
                whole[start:] = x[lo:lo + n_tok]
                x[lo:lo + n_tok] = plain.turn(whole, rot_cfg)[start:]
            if unit:
                x = plain.rms(x, 1e-5)
            if is_k:
                x = x * k_scale
        assert got.dtype == torch.float32
        assert (got.double().cpu() - x).abs().max().item() < 2e-5, "q" if got is q else "k" if got is k else "v"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_heads_prepare_writes_the_pages(dtype):
    """Keys and values land at their positions' places in the sequences' pages (page borders included), queries come back
    in the run's type; with ``write_kv=False`` the pages are left alone."""
    n_q, n_k, d, dv = 4, 2, 16, 24
    gen = torch.Generator(device=DEV).manual_seed(3)
    lengths, starts = [70, 3], [60, 127]
    T = sum(lengths)
    proj = torch.randn(T, n_q * d + n_k * d + n_k * dv, generator=gen, device=DEV).to(dtype)
    pos, seq, _ = _layout(lengths, starts)
    k_pages = torch.zeros(9, n_k, PAGE, d, dtype=dtype, device=DEV)
    v_pages = torch.zeros(9, n_k, PAGE, dv, dtype=dtype, device=DEV)
    table = _i32([7, 2, 5, 0, 4, 8, 1, 3, 6]).view(3, 3)
    kv = F().PagedKV(k_pages, v_pages, table)
    slots = _i32([2, 0])
    q = F().heads_prepare(proj, 0, n_q * d, n_q * d + n_k * d, n_q, n_k, d, dv, pos, seq, slots, kv=kv, write_kv=False)
    assert not k_pages.any() and not v_pages.any()
    q = F().heads_prepare(proj, 0, n_q * d, n_q * d + n_k * d, n_q, n_k, d, dv, pos, seq, slots, kv=kv)
    assert q.dtype == dtype and torch.equal(q.view(T, -1), proj[:, :n_q * d])
    written = 0
    for t in range(T):
        slot, p = int(slots[int(seq[t])]), int(pos[t])
        page = int(table[slot, p // PAGE])
        assert torch.equal(k_pages[page, :, p % PAGE].reshape(-1), proj[t, n_q * d:n_q * d + n_k * d])
        assert torch.equal(v_pages[page, :, p % PAGE].reshape(-1), proj[t, n_q * d + n_k * d:])
        written += 1
    assert int((k_pages != 0).any(-1).sum()) == written * n_k


# ------------------------------------------------------------------ the decayed recurrence
def _scan_whole(q, k, v, decay):
    return torch.stack([plain.decayed_sum(q[:, h].double().cpu(), k[:, h].double().cpu(), v[:, h].double().cpu(), float(decay[h]))
                        for h in range(q.shape[1])], 1)


@pytest.mark.parametrize("H,d,dv,T", [(3, 24, 40, 90), (2, 64, 128, 70), (1, 132, 20, 40), (5, 8, 8, 150), (4, 4, 12, 33),
                                      (1, 256, 36, 20), (2, 32, 33, 64)])
def test_decay_scan_whole_and_in_portions(H, d, dv, T):
    gen = torch.Generator(device=DEV).manual_seed(H * d)
    q, k = (torch.randn(T, H, d, generator=gen, device=DEV) for _ in range(2))
    v = torch.randn(T, H, dv, generator=gen, device=DEV)
    decay = torch.tensor(([1.0, 0.0, 0.9, 0.999, 0.5] * 2)[:H], device=DEV)
    want = _scan_whole(q, k, v, decay)
    scale = want.abs().max().item()
    state = torch.full((4, H, d, dv), float("nan"), device=DEV)
    results = []
    for cuts in ([T], [1] * 5 + [2, 3, 16, T - 26], [T - 7] + [1] * 7):
        state[1] = 0.0
        got, at = [], 0
        for n in cuts:
            _, _, cu = _layout([n])
            got.append(F().decay_scan(q[at:at + n].contiguous(), k[at:at + n].contiguous(), v[at:at + n].contiguous(), decay, state,
                                      cu, _i32([1]), 1))
            at += n
        results.append(torch.cat(got))
        assert (results[-1].double().cpu() - want).abs().max().item() < 2e-5 * max(scale, 1.0), f"cuts {cuts[:6]}"
    assert torch.equal(results[0], results[1]) and torch.equal(results[0], results[2]), "a cut changed 32-bit sums"
    assert torch.isnan(state[[0, 2, 3]]).all(), "another slot's state was written"


def test_decay_scan_batch_of_unequal_sequences_from_kept_states():
    """Three sequences of 1, 40 and 17 tokens in one launch, each going on from the state its slot holds, give what each
    gives alone; the states afterwards are the recurrences' own."""
    H, d, dv = 2, 40, 24
    gen = torch.Generator(device=DEV).manual_seed(1)
    lengths = [1, 40, 17]
    T = sum(lengths)
    q, k = (torch.randn(T, H, d, generator=gen, device=DEV) for _ in range(2))
    v = torch.randn(T, H, dv, generator=gen, device=DEV)
    decay = torch.tensor([0.97, 0.8], device=DEV)
    begin = torch.randn(5, H, d, dv, generator=gen, device=DEV)
    slots = [4, 0, 2]
    state = begin.clone()
    _, _, cu = _layout(lengths)
    together = F().decay_scan(q, k, v, decay, state, cu, _i32(slots), 3)
    at = 0
    for n, slot in zip(lengths, slots):
        S = begin[slot].double().cpu()
        for t in range(at, at + n):
            for h in range(H):
                S[h] = float(decay[h]) * S[h] + torch.outer(k[t, h].double().cpu(), v[t, h].double().cpu())
                want = S[h].T @ q[t, h].double().cpu()
                assert (together[t, h].double().cpu() - want).abs().max().item() < 1e-4
        assert (state[slot].double().cpu() - S).abs().max().item() < 1e-4
        at += n
    assert torch.equal(state[[1, 3]], begin[[1, 3]])


def test_decay_scan_remembers_a_far_token():
    """A decay near 1 carries one large key-value pair over 600 tokens, a small decay forgets it: the read-out of the
    last token holds the pair's value, weakened by decay^distance, in the first head and nothing of it in the second."""
    H, d, dv, T = 2, 16, 8, 601
    gen = torch.Generator(device=DEV).manual_seed(2)
    q, k = (torch.randn(T, H, d, generator=gen, device=DEV) * 0.01 for _ in range(2))
    v = torch.randn(T, H, dv, generator=gen, device=DEV) * 0.01
    k[0, :, 3], v[0, :, 5], q[T - 1, :, 3] = 10.0, 10.0, 10.0
    decay = torch.tensor([0.999, 0.9], device=DEV)
    state = torch.zeros(1, H, d, dv, device=DEV)
    _, _, cu = _layout([T])
    out = F().decay_scan(q, k, v, decay, state, cu, _i32([0]), 1)
    assert abs(out[T - 1, 0, 5].item() - 1000.0 * 0.999 ** 600) < 1.0
    assert abs(out[T - 1, 1, 5].item()) < 0.1
    want = _scan_whole(q, k, v, decay)
    assert (out.double().cpu() - want).abs().max().item() < 1e-3


@pytest.mark.parametrize("H,d,dv,lengths", [(3, 24, 40, [90]), (2, 64, 128, [200, 64, 1]), (1, 132, 20, [63, 65, 128]),
                                            (5, 8, 8, [150, 2]), (2, 4, 12, [129]), (1, 256, 36, [70]), (2, 128, 68, [300, 17])])
def test_decay_scan_in_chunks_against_token_by_token(H, d, dv, lengths):
    """The chunked kernels on batches of unequal sequences that go on from kept states, with chunk borders inside, at and
    one off the ends, against the recurrence in float64 and against the token-by-token kernel; decays of 1 and 0 too."""
    gen = torch.Generator(device=DEV).manual_seed(H * d + dv)
    T, n = sum(lengths), len(lengths)
    q, k = (torch.randn(T, H, d, generator=gen, device=DEV) for _ in range(2))
    v = torch.randn(T, H, dv, generator=gen, device=DEV)
    decay = torch.tensor(([1.0, 0.0, 0.9, 0.999, 0.5] * 2)[:H], device=DEV)
    begin = torch.randn(n + 2, H, d, dv, generator=gen, device=DEV)
    slots = list(range(n, 0, -1))
    _, _, cu = _layout(lengths)
    assert F().decay_scan_chunked_fits(d, dv)
    for wave_floats in (1 << 26, 1):  # all chunks in one wave, and one chunk a wave
        state = begin.clone()
        before = F().DECAY_WORKSPACE_FLOATS
        F().DECAY_WORKSPACE_FLOATS = wave_floats
        try:
            got = F().decay_scan_chunked(q, k, v, decay, state, cu, _i32(slots), n, max(lengths))
        finally:
            F().DECAY_WORKSPACE_FLOATS = before
        stepped_state = begin.clone()
        stepped = F().decay_scan(q, k, v, decay, stepped_state, cu, _i32(slots), n)
        at = 0
        for length, slot in zip(lengths, slots):
            S = begin[slot].double().cpu()
            want = torch.empty(length, H, dv, dtype=torch.float64)
            for t in range(length):
                S = decay.double().cpu()[:, None, None] * S + torch.einsum("hd,he->hde", k[at + t].double().cpu(), v[at + t].double().cpu())
                want[t] = torch.einsum("hde,hd->he", S, q[at + t].double().cpu())
            scale = max(1.0, want.abs().max().item())
            assert (got[at:at + length].double().cpu() - want).abs().max().item() < 2e-5 * scale, f"read-outs, wave {wave_floats}"
            assert (state[slot].double().cpu() - S).abs().max().item() < 2e-5 * max(1.0, S.abs().max().item()), "state behind the step"
            at += length
        assert (got - stepped).abs().max().item() < 4e-5 * max(1.0, stepped.abs().max().item())
        assert torch.equal(state[[0, n + 1]], begin[[0, n + 1]]), "another slot's state was written"


def test_decay_scan_in_chunks_remembers_a_far_token():
    """One large key-value pair at the first token, read by the last token 600 tokens later, through nine chunk borders."""
    H, d, dv, T = 2, 16, 8, 601
    gen = torch.Generator(device=DEV).manual_seed(2)
    q, k = (torch.randn(T, H, d, generator=gen, device=DEV) * 0.01 for _ in range(2))
    v = torch.randn(T, H, dv, generator=gen, device=DEV) * 0.01
    k[0, :, 3], v[0, :, 5], q[T - 1, :, 3] = 10.0, 10.0, 10.0
    decay = torch.tensor([0.999, 0.9], device=DEV)
    state = torch.zeros(1, H, d, dv, device=DEV)
    _, _, cu = _layout([T])
    out = F().decay_scan_chunked(q, k, v, decay, state, cu, _i32([0]), 1, T)
    assert abs(out[T - 1, 0, 5].item() - 1000.0 * 0.999 ** 600) < 1.0
    assert abs(out[T - 1, 1, 5].item()) < 0.1
    assert (out.double().cpu() - _scan_whole(q, k, v, decay)).abs().max().item() < 1e-3


# ------------------------------------------------------------------ norm and gate behind the recurrence
@pytest.mark.parametrize("H,dv,whole,gate_kind,out_dtype", [(3, 40, True, "sigmoid", torch.float32), (2, 24, False, "silu", torch.bfloat16),
                                                            (5, 8, False, "silu", torch.float32), (1, 260, True, "sigmoid", torch.bfloat16),
                                                            (4, 160, True, "sigmoid", torch.bfloat16), (2, 516, False, "silu", torch.float32)])
def test_group_norm_gate(H, dv, whole, gate_kind, out_dtype):
    T, width = 19, H * dv
    gen = torch.Generator(device=DEV).manual_seed(dv)
    x = torch.randn(T, width, generator=gen, device=DEV) * 4.0
    gate_at = 11
    proj = torch.randn(T, gate_at + width + 2, generator=gen, device=DEV).to(out_dtype)
    weight = (1.0 + 0.3 * torch.randn(width, generator=gen, device=DEV)) if whole else None
    got = F().group_norm_gate(x, width if whole else dv, weight, proj, gate_at, 1e-5, out_dtype, gate_kind)
    x64, g64 = x.double().cpu(), proj.double().cpu()[:, gate_at:gate_at + width]
    if whole:
        normed = plain.rms(x64, 1e-5) * weight.double().cpu()
    else:
        normed = plain.rms(x64.view(T, H, dv), 1e-5).reshape(T, width)
    want = normed * (torch.sigmoid(g64) if gate_kind == "sigmoid" else plain.silu(g64))
    tol = 2e-5 if out_dtype == torch.float32 else 3e-2
    assert (got.double().cpu() - want).abs().max().item() < tol


def test_scaled_sum_and_squared_relu():
    gen = torch.Generator(device=DEV).manual_seed(0)
    a, b = (torch.randn(33, 50, generator=gen, device=DEV).to(torch.bfloat16) for _ in range(2))
    got = F().scaled_sum(a, 0.6, b, -1.3)
    assert got.dtype == torch.float32
    assert (got.double() - (0.6 * a.double() - 1.3 * b.double())).abs().max().item() < 1e-6
    x = torch.randn(40, 70, generator=gen, device=DEV)
    assert torch.allclose(F().relu_squared(x), torch.relu(x) ** 2)
    from gtar_kimik3_public_b200.ops.linear import linear

    for dtype, n_tokens in ((torch.float32, 3), (torch.bfloat16, 5), (torch.bfloat16, 200), (torch.float32, 130)):
        w = (torch.randn(96, 64, generator=gen, device=DEV) * 0.2).to(dtype)
        h = torch.randn(n_tokens, 64, generator=gen, device=DEV).to(dtype)
        want = torch.relu(h.double() @ w.double().T) ** 2
        got = linear(h, w, relu_squared=True)
        err = ((got.double() - want).abs() / (1.0 + want)).max().item()  # a squared value carries twice the relative rounding
        assert err < (1e-5 if dtype == torch.float32 else 3e-2)


# ------------------------------------------------------------------ scored attention
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


def _plain_attention(q, k, v, scale, window, keep_first, r1, r2, pb, weights):
    mask = {"size": window, "keep_first": keep_first} if window else None
    q, k, v = q.double().cpu(), k.double().cpu(), v.double().cpu()
    if weights == "sigmoid":
        return plain.sigmoid_core(q, k, v, scale, mask, pb.double().cpu())
    return plain.softmax_core(q, k, v, scale, mask, None if r1 is None else r1.double().cpu(), None if r2 is None else r2.double().cpu())


RULES = [
    # H, G, d, dv, window, keep_first, distance term, weights
    (6, 2, 16, 24, 17, 3, True, "softmax"),
    (4, 1, 32, 32, 64, 70, True, "softmax"),
    (2, 2, 40, 8, 70, 0, True, "softmax"),
    (3, 1, 24, 40, 0, 0, True, "softmax"),
    (2, 1, 16, 16, 1, 1, True, "softmax"),
    (8, 2, 32, 64, 32, 33, False, "softmax"),
    (4, 2, 64, 64, 65, 66, True, "softmax"),
    (4, 1, 24, 16, 0, 0, False, "sigmoid"),
    (3, 3, 8, 24, 0, 0, False, "sigmoid"),
    (2, 1, 128, 64, 130, 5, False, "sigmoid"),
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,dv,window,keep_first,biased,weights", RULES)
def test_scored_attention_prompts_portions_and_single_tokens(dtype, H, G, d, dv, window, keep_first, biased, weights):
    """Two sequences of unequal length in one launch: all their tokens; the last portion of each (from a position that
    is no multiple of anything); their last tokens alone.  Every row equals the plain implementation's."""
    gen = torch.Generator(device=DEV).manual_seed(H * d + window)
    lengths = [201, 77]
    qs = [torch.randn(L, H, d, generator=gen, device=DEV).to(dtype) for L in lengths]
    ks = [torch.randn(L, G, d, generator=gen, device=DEV).to(dtype) for L in lengths]
    vs = [torch.randn(L, G, dv, generator=gen, device=DEV).to(dtype) for L in lengths]
    r1 = (0.3 + 0.1 * torch.randn(H, generator=gen, device=DEV)) if biased else None
    r2 = (0.5 + 0.1 * torch.randn(H, generator=gen, device=DEV)).abs() if biased else None
    pb = (-2.0 + 0.5 * torch.randn(H, generator=gen, device=DEV)) if weights == "sigmoid" else None
    scale = d ** -0.5
    kv, slots = _paged(ks, vs, dtype)
    want = [_plain_attention(q, k, v, scale, window, keep_first, r1, r2, pb, weights) for q, k, v in zip(qs, ks, vs)]
    tol = 3e-5 if dtype == torch.float32 else 4e-2
    if weights == "sigmoid":
        tol *= 4  # sums of up to 200 weights that nothing divides
    exact = []
    for starts in ([0, 0], [139, 70], [200, 76]):
        pos, seq, _ = _layout([L - a for L, a in zip(lengths, starts)], starts)
        q = torch.cat([q[a:] for q, a in zip(qs, starts)]).contiguous()
        got = F().attention_scored_exact(q, kv, pos, seq, slots, scale, window, keep_first, r1, r2, pb, weights)
        ref = torch.cat([w[a:] for w, a in zip(want, starts)])
        assert torch.isfinite(got).all()
        assert (got.double().cpu() - ref).abs().max().item() < tol, f"queries from {starts}"
        exact.append(got)
    whole = exact[0]
    assert torch.equal(exact[1], torch.cat([whole[139:201], whole[201 + 70:]])), "a portion's rows are not the whole prompt's"
    assert torch.equal(exact[2], torch.stack([whole[200], whole[201 + 76]])), "a single token's row is not the whole prompt's"


def _standout(L, H, G, d, dv, dtype, seed):
    """Small random queries, keys and values; the caller makes one key stand out for one query."""
    gen = torch.Generator(device=DEV).manual_seed(seed)
    q = (torch.randn(L, H, d, generator=gen, device=DEV) * 0.05).to(dtype)
    k = (torch.randn(L, G, d, generator=gen, device=DEV) * 0.05).to(dtype)
    v = (torch.randn(L, G, dv, generator=gen, device=DEV) * 0.05).to(dtype)
    return q, k, v


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("weights", ["softmax", "sigmoid"])
@pytest.mark.parametrize("window,keep_first,i,j,seen", [
    (0, 0, 700, 3, True),        # far back, no window
    (0, 0, 700, 63, True),       # the last place of the first page
    (0, 0, 700, 64, True),       # the first place of the second
    (0, 0, 700, 700, True),      # the token itself
    (96, 20, 700, 605, True),    # just inside the window
    (96, 20, 700, 604, False),   # just outside
    (96, 20, 700, 19, True),     # the last kept first token
    (96, 20, 700, 20, False),    # the first that is not kept
    (96, 20, 700, 0, True),
    (64, 65, 200, 64, True),     # more kept tokens than a page: the second page's first place
    (64, 65, 200, 65, False),
    (64, 65, 200, 137, True),
    (64, 65, 200, 136, False),
    (33, 1, 127, 95, True),      # an edge in the middle of a block of 32 keys
    (33, 1, 127, 94, False),
    (32, 0, 128, 97, True),      # an edge on a block's border
    (32, 0, 128, 96, False),
    (1, 0, 300, 300, True),      # a window of the token itself
    (1, 0, 300, 299, False),
    (5, 2, 3, 0, True),          # the first tokens of a sequence: the window has not left anything yet
    (500, 0, 40, 1, True),       # a window longer than the sequence
])
def test_scored_attention_sees_one_key_or_not(dtype, weights, window, keep_first, i, j, seen):
    """Among hundreds of small keys one is made to stand out for the query at ``i`` (its score is large, its value is 100
    in one entry).  If ``j`` is visible from ``i`` that entry of the output is near 100, else near 0: in a whole prompt,
    and for the token at ``i`` alone over the cache."""
    H, G, d, dv = 4, 2, 16, 24
    L = i + 5
    q, k, v = _standout(L, H, G, d, dv, dtype, i + j)
    head, kv_head = 3, 1
    q[i, head] = 0.0
    q[i, head, 2] = 8.0
    k[j, kv_head, 2] = 8.0
    v[j, kv_head] = 0.0
    v[j, kv_head, 7] = 100.0
    r1 = torch.full((H,), 0.3, device=DEV) if weights == "softmax" else None
    r2 = torch.full((H,), 0.5, device=DEV) if weights == "softmax" else None
    pb = torch.full((H,), -9.0, device=DEV) if weights == "sigmoid" else None
    scale = 0.5  # the score that stands out: 32, minus at most 0.3 ln(1 + 350) < 2
    kv, slots = _paged([k], [v], dtype, seed=j)
    want = _plain_attention(q, k, v, scale, window, keep_first, r1, r2, pb, weights)
    for first in (0, i):
        pos, seq, _ = _layout([L - first if first == 0 else 1], [first])
        rows = q[first:] if first == 0 else q[i:i + 1]
        got = F().attention_scored_exact(rows.contiguous(), kv, pos, seq, slots, scale, window, keep_first, r1, r2, pb, weights)
        at = i - first
        value = got[at, head, 7].item()
        assert (value > 90.0) == seen and (abs(value) < 2.0) != seen, f"key {j} from {i}: {value}"
        ref = want[first:] if first == 0 else want[i:i + 1]
        assert (got.double().cpu() - ref).abs().max().item() < (2e-4 if dtype == torch.float32 else 0.4)
        if window == 0 and j < i - 100:  # the other query head of the same key head did not ask for it
            assert abs(got[at, 2, 7].item()) < 2.0


# ------------------------------------------------------------------ scored attention on the tensor cores
def _fast(q, kv, lengths, starts, slots, scale, window, keep_first, r1, r2, pb, weights, parts):
    _, _, cu = _layout([L - a for L, a in zip(lengths, starts)], starts)
    longest = max(L - a for L, a in zip(lengths, starts))
    return F().attention_scored(q, kv, cu, _i32(lengths), slots, longest, scale, window, keep_first, r1, r2, pb, weights, parts)


FAST_RULES = [
    # H, G, d, window, keep_first, distance term, weights
    (4, 2, 64, 0, 0, True, "softmax"),
    (6, 2, 64, 17, 3, True, "softmax"),
    (4, 1, 128, 64, 70, True, "softmax"),
    (2, 2, 128, 70, 0, False, "softmax"),
    (8, 2, 64, 32, 33, False, "softmax"),
    (2, 1, 64, 1, 1, True, "softmax"),
    (5, 1, 64, 130, 129, True, "softmax"),
    (4, 1, 64, 0, 0, False, "sigmoid"),
    (3, 3, 128, 0, 0, False, "sigmoid"),
    (2, 1, 128, 130, 5, False, "sigmoid"),
]


@pytest.mark.parametrize("H,G,d,window,keep_first,biased,weights", FAST_RULES)
def test_tensor_core_scored_attention_prompts_portions_and_single_tokens(H, G, d, window, keep_first, biased, weights):
    """Three sequences of unequal length in one launch: all their tokens, the last portion of each, their last tokens
    alone; the walk over the keys whole and cut into 2, 3 and more parts than there are pages."""
    gen = torch.Generator(device=DEV).manual_seed(H * d + window)
    lengths = [333, 77, 1]
    dtype = torch.bfloat16
    qs = [torch.randn(L, H, d, generator=gen, device=DEV).to(dtype) for L in lengths]
    ks = [torch.randn(L, G, d, generator=gen, device=DEV).to(dtype) for L in lengths]
    vs = [torch.randn(L, G, d, generator=gen, device=DEV).to(dtype) for L in lengths]
    r1 = (0.3 + 0.1 * torch.randn(H, generator=gen, device=DEV)) if biased else None
    r2 = (0.5 + 0.1 * torch.randn(H, generator=gen, device=DEV)).abs() if biased else None
    pb = (-2.0 + 0.5 * torch.randn(H, generator=gen, device=DEV)) if weights == "sigmoid" else None
    scale = d ** -0.5
    kv, slots = _paged(ks, vs, dtype)
    want = [_plain_attention(q, k, v, scale, window, keep_first, r1, r2, pb, weights) for q, k, v in zip(qs, ks, vs)]
    tol = 4e-2 * (4 if weights == "sigmoid" else 1)
    for starts in ([0, 0, 0], [139, 70, 0], [332, 76, 0]):
        q = torch.cat([q[a:] for q, a in zip(qs, starts)]).contiguous()
        ref = torch.cat([w[a:] for w, a in zip(want, starts)])
        for parts in (1, 2, 3, 9):
            got = _fast(q, kv, lengths, starts, slots, scale, window, keep_first, r1, r2, pb, weights, parts)
            assert torch.isfinite(got).all()
            assert (got.double().cpu() - ref).abs().max().item() < tol, f"queries from {starts}, {parts} parts"


@pytest.mark.parametrize("parts", [1, 4])
@pytest.mark.parametrize("weights", ["softmax", "sigmoid"])
@pytest.mark.parametrize("window,keep_first,i,j,seen", [
    (0, 0, 700, 3, True), (0, 0, 700, 63, True), (0, 0, 700, 64, True), (0, 0, 700, 700, True),
    (96, 20, 700, 605, True), (96, 20, 700, 604, False), (96, 20, 700, 19, True), (96, 20, 700, 20, False), (96, 20, 700, 0, True),
    (64, 65, 200, 64, True), (64, 65, 200, 65, False), (64, 65, 200, 137, True), (64, 65, 200, 136, False),
    (33, 1, 127, 95, True), (33, 1, 127, 94, False), (32, 0, 128, 97, True), (32, 0, 128, 96, False),
    (1, 0, 300, 300, True), (1, 0, 300, 299, False), (5, 2, 3, 0, True), (500, 0, 40, 1, True),
    (128, 64, 640, 513, True), (128, 64, 640, 512, False), (128, 64, 640, 63, True), (128, 64, 640, 64, False),
])
def test_tensor_core_scored_attention_sees_one_key_or_not(parts, weights, window, keep_first, i, j, seen):
    """The key that stands out (see above) through the tensor-core kernel: in a whole prompt, in a portion that starts
    in the middle of a tile of rows, and for the token at ``i`` alone."""
    H, G, d = 4, 2, 64
    L = i + 5
    dtype = torch.bfloat16
    q, k, v = _standout(L, H, G, d, d, dtype, i + j)
    head, kv_head = 3, 1
    q[i, head] = 0.0
    q[i, head, 2] = 8.0
    k[j, kv_head, 2] = 8.0
    v[j, kv_head] = 0.0
    v[j, kv_head, 7] = 100.0
    r1 = torch.full((H,), 0.3, device=DEV) if weights == "softmax" else None
    r2 = torch.full((H,), 0.5, device=DEV) if weights == "softmax" else None
    pb = torch.full((H,), -9.0, device=DEV) if weights == "sigmoid" else None
    kv, slots = _paged([k], [v], dtype, seed=j)
    want = _plain_attention(q, k, v, 0.5, window, keep_first, r1, r2, pb, weights)
    for first in sorted({0, max(0, i - 37), i}):
        got = _fast(q[first:].contiguous() if first < i else q[i:i + 1].contiguous(), kv, [L if first < i else i + 1], [first], slots, 0.5,
                    window, keep_first, r1, r2, pb, weights, parts)
        value = got[i - first, head, 7].item()
        assert (value > 90.0) == seen and (abs(value) < 2.0) != seen, f"key {j} from {i} (rows from {first}): {value}"
        ref = want[first:] if first < i else want[i:i + 1]
        assert (got.double().cpu() - ref).abs().max().item() < 0.4


def test_scored_attention_parts_rule():
    parts = F().scored_attention_parts
    assert parts(1, 16, 4, 2048, 32, 148) == 1            # a long prompt fills the GPU by its rows
    assert parts(8, 16, 4, 1, 33, 148) > 1                # single tokens do not
    assert parts(8, 16, 4, 1, 1, 148) == 1                # never more parts than pages
    assert parts(1, 2, 1, 1, 1000, 148) <= 32
    assert 8 * 4 * parts(8, 16, 4, 1, 33, 148) <= 2 * 148  # the blocks stay within two a multiprocessor
