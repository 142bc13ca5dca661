"""Python faces of the kernels: argument checks, then one call into the kernel library.

Every function works on CUDA tensors on the current stream and allocates at most its own
output.  Shapes follow the packed ("varlen") convention of the step function: activations are
``[n_tokens, width]`` with the tokens of all sequences of a step one after another.
"""

from __future__ import annotations

import functools
from dataclasses import dataclass

import torch

from .library import KernelError, call, dtype_code, ptr, require_device, stream_ptr


def _check(tensor: torch.Tensor, name: str, dtype=None, dims: int | None = None) -> None:
    if not tensor.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor")
    if not tensor.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and tensor.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {tensor.dtype}")
    if dims is not None and tensor.dim() != dims:
        raise KernelError(f"{name} must have {dims} dimensions, got shape {tuple(tensor.shape)}")


@dataclass
class PagedKV:
    """One layer's keys and values in pages, and the table that maps a sequence's pages.

    ``k``, ``v``: ``[n_pages, n_kv_heads, page_size, head_dim]``; ``block_table``:
    ``[n_slots, max_pages]`` int32, entry ``[slot, i]`` = page that holds positions
    ``i*page_size .. (i+1)*page_size-1`` of the sequence in ``slot``.
    """

    k: torch.Tensor
    v: torch.Tensor
    block_table: torch.Tensor
    work: "DecodeWork | None" = None  # what decode attention keeps between launches; the cache group owns it

    @property
    def page_size(self) -> int:
        return self.k.shape[2]

    @property
    def max_pages(self) -> int:
        return self.block_table.shape[1]


class DecodeWork:
    """Scratch memory that decode attention keeps between launches, one per cache group (its layers run one after
    another on one stream): the partial results of sequences whose pages are shared by several blocks, and a ticket
    counter per (sequence, kv head), zero between launches (the kernel sets back what it counts up).  Buffers that
    are outgrown stay alive: a captured graph may still name them."""

    MIN_FLOATS, MIN_PAIRS = 1 << 18, 1024  # the least that is asked of the allocator, so that growth is rare

    def __init__(self, device: torch.device):
        self.device = device
        self.part: torch.Tensor | None = None
        self.tickets: torch.Tensor | None = None
        self.outgrown: list[torch.Tensor] = []

    def get(self, n_floats: int, n_pairs: int) -> tuple[torch.Tensor, torch.Tensor]:
        if self.part is None or self.part.numel() < n_floats:
            if self.part is not None:
                self.outgrown.append(self.part)
            self.part = torch.empty((max(n_floats, self.MIN_FLOATS),), dtype=torch.float32, device=self.device)
        if self.tickets is None or self.tickets.numel() < n_pairs:
            if self.tickets is not None:
                self.outgrown.append(self.tickets)
            self.tickets = torch.zeros((max(n_pairs, self.MIN_PAIRS),), dtype=torch.int32, device=self.device)
        return self.part, self.tickets


def embed_rows(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor | None = None, scale: float = 1.0) -> torch.Tensor:
    """``out[t] = table[ids[t]] * scale`` widened to float32 (the residual stream's type) before the product."""
    require_device(table.device)
    _check(table, "table", dims=2)
    _check(ids, "ids", torch.int32, 1)
    n, hidden = ids.shape[0], table.shape[1]
    if out is None:
        out = torch.empty((n, hidden), dtype=torch.float32, device=table.device)
    _check(out, "out", torch.float32, 2)
    call("gk_embed_rows", ptr(table), dtype_code(table.dtype), ptr(ids), ptr(out), n, hidden, float(scale), stream_ptr())
    return out


def add_rmsnorm(
    h: torch.Tensor,
    delta: torch.Tensor | None,
    weight: torch.Tensor,
    eps: float,
    out_dtype: torch.dtype,
    rows: torch.Tensor | None = None,
    out: torch.Tensor | None = None,
) -> torch.Tensor:
    """``h += delta`` (in place, skipped when ``delta`` is None), then RMSNorm of ``h`` times ``weight``.

    With ``rows`` (int32 indices) only those rows are normalised and ``h`` is not written: the
    sum ``h + delta`` of such a row is formed on the fly.
    """
    require_device(h.device)
    _check(h, "h", torch.float32, 2)
    _check(weight, "weight", dims=1)
    hidden = h.shape[1]
    if weight.shape[0] != hidden:
        raise KernelError(f"norm weight has {weight.shape[0]} entries for rows of {hidden}")
    delta_code = 0
    if delta is not None:
        _check(delta, "delta", dims=2)
        if delta.shape != h.shape:
            raise KernelError(f"delta {tuple(delta.shape)} does not match h {tuple(h.shape)}")
        delta_code = dtype_code(delta.dtype)
    n_out = h.shape[0]
    if rows is not None:
        _check(rows, "rows", torch.int32, 1)
        n_out = rows.shape[0]
    if out is None:
        out = torch.empty((n_out, hidden), dtype=out_dtype, device=h.device)
    _check(out, "out", out_dtype, 2)
    call(
        "gk_add_rmsnorm", ptr(h), ptr(delta), delta_code, ptr(weight), dtype_code(weight.dtype), ptr(out),
        dtype_code(out_dtype), ptr(rows), n_out, hidden, float(eps), stream_ptr(),
    )
    return out


def swiglu(gate_up: torch.Tensor, out: torch.Tensor | None = None, interleaved: bool = False) -> torch.Tensor:
    """``silu(gate) * up`` for rows packed as ``[gate (I) | up (I)]``, or with ``interleaved`` as
    ``g0 u0 g1 u1 ...``."""
    require_device(gate_up.device)
    _check(gate_up, "gate_up", dims=2)
    n, two_i = gate_up.shape
    if two_i % 2:
        raise KernelError("gate_up rows must hold gate and up halves of equal width")
    inter = two_i // 2
    if out is None:
        out = torch.empty((n, inter), dtype=gate_up.dtype, device=gate_up.device)
    _check(out, "out", gate_up.dtype, 2)
    call("gk_swiglu", ptr(gate_up), ptr(out), dtype_code(gate_up.dtype), n, inter, int(interleaved), stream_ptr())
    return out


def qk_norm_rope_write(
    qkv: torch.Tensor,
    n_q: int,
    n_kv: int,
    head_dim: int,
    q_weight: torch.Tensor | None,
    k_weight: torch.Tensor | None,
    eps: float,
    cos: torch.Tensor | None,
    sin: torch.Tensor | None,
    tok_pos: torch.Tensor,
    tok_seq: torch.Tensor,
    slots: torch.Tensor,
    kv: PagedKV,
    max_position: int,
    q_out: torch.Tensor | None = None,
    write_kv: bool = True,
) -> torch.Tensor:
    """Per-head RMSNorm of q and k, rotation by position, and the write of k and v into the pages.

    ``qkv``: ``[n_tokens, (n_q + 2 n_kv) * head_dim]``.  Returns the finished queries
    ``[n_tokens, n_q, head_dim]``.  ``max_position`` is the largest entry of ``tok_pos`` (known on
    the host) and is checked against the rotary table.  ``write_kv=False`` leaves the pages alone
    (a layer that attends over keys and values written by another layer).
    """
    require_device(qkv.device)
    _check(qkv, "qkv", dims=2)
    n = qkv.shape[0]
    if qkv.shape[1] != (n_q + 2 * n_kv) * head_dim:
        raise KernelError(f"qkv rows are {qkv.shape[1]} wide, expected {(n_q + 2 * n_kv) * head_dim}")
    cache_dtype = qkv.dtype
    for name, t in (("tok_pos", tok_pos), ("tok_seq", tok_seq), ("slots", slots)):
        _check(t, name, torch.int32, 1)
    _check(kv.block_table, "block_table", torch.int32, 2)
    _check(kv.k, "k pages", cache_dtype, 4)
    _check(kv.v, "v pages", cache_dtype, 4)
    if kv.k.shape[1] != n_kv or kv.k.shape[3] != head_dim or kv.v.shape != kv.k.shape:
        raise KernelError(f"pages {tuple(kv.k.shape)} do not fit n_kv={n_kv}, head_dim={head_dim}")
    use_norm = q_weight is not None
    weight_code = 0
    if use_norm:
        _check(q_weight, "q_weight", dims=1)
        _check(k_weight, "k_weight", q_weight.dtype, 1)
        if q_weight.shape[0] != head_dim or k_weight.shape[0] != head_dim:
            raise KernelError("q/k norm weights must have head_dim entries")
        weight_code = dtype_code(q_weight.dtype)
    table_positions = 0
    if cos is not None:
        _check(cos, "cos", torch.float32, 2)
        _check(sin, "sin", torch.float32, 2)
        if cos.shape[1] != head_dim // 2 or sin.shape != cos.shape:
            raise KernelError("rotary tables must be [positions, head_dim / 2]")
        table_positions = cos.shape[0]
    if q_out is None:
        q_out = torch.empty((n, n_q, head_dim), dtype=cache_dtype, device=qkv.device)
    _check(q_out, "q_out", cache_dtype, 3)
    call(
        "gk_qk_norm_rope_write", ptr(qkv), dtype_code(qkv.dtype), ptr(q_weight), ptr(k_weight), weight_code, ptr(cos),
        ptr(sin), table_positions, ptr(tok_pos), ptr(tok_seq), ptr(slots), ptr(kv.block_table), ptr(q_out),
        ptr(kv.k) if write_kv else None, ptr(kv.v) if write_kv else None, n, n_q, n_kv, head_dim, kv.max_pages, kv.page_size, float(eps), int(use_norm), int(max_position),
        stream_ptr(),
    )
    return q_out


# Tiles of 128 x 256 from which the q|k|v product does its output stage itself.  Below, the library product and the
# stage as a kernel of its own are faster (1,024 tokens x 4,096 columns = 128 tiles: 16.2 against 17.7 us; 2,048
# tokens = 256 tiles: 26.7 against 25.9): the persistent kernel leaves SMs idle and its last tile's stage exposed.
QKV_FUSED_FROM_TILES = 200


def qkv_fused_ok(x: torch.Tensor, weight: torch.Tensor, head_dim: int, kv: PagedKV) -> bool:
    """Whether the q|k|v projection of this step can do the attention input stage in its epilogue:
    bfloat16, enough tokens for the many-token orientation and its wide tiles, head size 64 or 128."""
    m, k = x.shape
    n = weight.shape[0]
    return (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and kv.k.dtype == torch.bfloat16
            and m > SKINNY_M and k % 8 == 0 and head_dim in (64, 128)
            and n >= PREFILL_BN and -(-m // 128) * -(-n // PREFILL_BN) >= QKV_FUSED_FROM_TILES)


def gemm_tc_qkv(
    x: torch.Tensor,
    weight: torch.Tensor,
    n_q: int,
    n_kv: int,
    head_dim: int,
    q_weight: torch.Tensor | None,
    k_weight: torch.Tensor | None,
    eps: float,
    cos: torch.Tensor | None,
    sin: torch.Tensor | None,
    tok_pos: torch.Tensor,
    tok_seq: torch.Tensor,
    slots: torch.Tensor,
    kv: PagedKV,
    max_position: int,
    write_kv: bool = True,
) -> torch.Tensor:
    """``x @ weight.T`` for the packed q|k|v weight with per-head q/k RMSNorm, rotation and the write of
    k and v into the pages done in the product's epilogue.  Returns the queries ``[n_tokens, n_q, head_dim]``."""
    require_device(x.device)
    _check(x, "x", torch.bfloat16, 2)
    _check(weight, "weight", torch.bfloat16, 2)
    n, k = x.shape
    if weight.shape != ((n_q + 2 * n_kv) * head_dim, k):
        raise KernelError(f"weight is {tuple(weight.shape)}, expected {((n_q + 2 * n_kv) * head_dim, k)}")
    for name, t in (("tok_pos", tok_pos), ("tok_seq", tok_seq), ("slots", slots)):
        _check(t, name, torch.int32, 1)
    _check(kv.k, "k pages", torch.bfloat16, 4)
    _check(kv.v, "v pages", torch.bfloat16, 4)
    if kv.k.shape[1] != n_kv or kv.k.shape[3] != head_dim:
        raise KernelError(f"pages {tuple(kv.k.shape)} do not fit n_kv={n_kv}, head_dim={head_dim}")
    use_norm = q_weight is not None
    weight_code = 0
    if use_norm:
        _check(q_weight, "q_weight", dims=1)
        _check(k_weight, "k_weight", q_weight.dtype, 1)
        weight_code = dtype_code(q_weight.dtype)
    table_positions = 0
    if cos is not None:
        _check(cos, "cos", torch.float32, 2)
        _check(sin, "sin", torch.float32, 2)
        table_positions = cos.shape[0]
    q_out = torch.empty((n, n_q, head_dim), dtype=torch.bfloat16, device=x.device)
    call(
        "gk_gemm_bf16_tc_qkv", ptr(x), n, ptr(weight), k, n_q, n_kv, head_dim, ptr(q_weight), ptr(k_weight), weight_code,
        int(use_norm), float(eps), ptr(cos), ptr(sin), table_positions, int(max_position), ptr(tok_pos), ptr(tok_seq),
        ptr(slots), ptr(kv.block_table), kv.max_pages, kv.page_size, ptr(q_out), ptr(kv.k) if write_kv else None,
        ptr(kv.v) if write_kv else None, ptr(error_flag(x.device)), stream_ptr(),
    )
    return q_out


def linear_f32(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype = torch.float32,
               out: torch.Tensor | None = None) -> torch.Tensor:
    """``x @ weight.T`` on the FP32 pipes: ``weight`` float32 ``[N, K]``, ``x`` float32 or bfloat16 ``[M, K]``."""
    require_device(x.device)
    _check(x, "x", dims=2)
    _check(weight, "weight", torch.float32, 2)
    m, k = x.shape
    n = weight.shape[0]
    if weight.shape[1] != k:
        raise KernelError(f"x is [{m}, {k}] but weight is {tuple(weight.shape)}")
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype, device=x.device)
    _check(out, "out", out_dtype, 2)
    call("gk_gemm_f32", ptr(x), dtype_code(x.dtype), ptr(weight), ptr(out), dtype_code(out_dtype), m, n, k, k, k, n,
         stream_ptr())
    return out


def attention_exact(
    q: torch.Tensor,
    kv: PagedKV,
    tok_pos: torch.Tensor,
    tok_seq: torch.Tensor,
    slots: torch.Tensor,
    scale: float,
    window: int = 0,
    out: torch.Tensor | None = None,
    sink: bool = False,
) -> torch.Tensor:
    """Causal grouped-query attention of ``q [n_tokens, n_q, d]`` over the pages (exact kernel).  ``sink``: the
    softmax's denominator has one more term, a key of score 0 without a value."""
    require_device(q.device)
    _check(q, "q", dims=3)
    n, n_q, d = q.shape
    _check(kv.k, "k pages", q.dtype, 4)
    _check(kv.v, "v pages", q.dtype, 4)
    n_kv = kv.k.shape[1]
    if kv.k.shape[3] != d:
        raise KernelError(f"pages have head_dim {kv.k.shape[3]}, queries {d}")
    for name, t in (("tok_pos", tok_pos), ("tok_seq", tok_seq), ("slots", slots)):
        _check(t, name, torch.int32, 1)
    if out is None:
        out = torch.empty_like(q)
    call(
        "gk_attention_exact", ptr(q), ptr(kv.k), ptr(kv.v), ptr(out), dtype_code(q.dtype), ptr(tok_pos), ptr(tok_seq),
        ptr(slots), ptr(kv.block_table), n, n_q, n_kv, d, kv.max_pages, kv.page_size, float(scale), int(window),
        int(sink), stream_ptr(),
    )
    return out


_error_flags: dict[int, torch.Tensor] = {}


def error_flag(device: torch.device) -> torch.Tensor:
    """The device int that kernels with bounded waits set when a wait gives up (0 = all well)."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    if index not in _error_flags:
        _error_flags[index] = torch.zeros(1, dtype=torch.int32, device=device)
    return _error_flags[index]


def check_kernel_errors(device: torch.device | str = "cuda:0") -> None:
    """Raises if a kernel gave up a wait since the last check (synchronises the device)."""
    flag = error_flag(torch.device(device))
    code = int(flag.item())
    if code:
        flag.zero_()
        raise KernelError(f"a kernel gave up waiting on a barrier (code {code}); its output is not valid")


EPI_STORE, EPI_SWIGLU_A, EPI_SWIGLU_B = 0, 1, 2
SKINNY_M = 64  # up to this many tokens the weights take the MMA's 128 rows (swap-AB)


SPLIT_TARGET_BLOCKS = 128
PREFILL_BN = 256  # 128 x 256 tiles, walked by one persistent block per SM
SCRATCH_SPLITS_FROM = 17
SKINNY_BN_MAX = 64
SPLIT_MIN_K_BLOCKS = 4


_sm_counts: dict[int, int] = {}


def sm_count(device: torch.device | None = None) -> int:
    """Multiprocessors of the device (asked once per device)."""
    index = torch.cuda.current_device() if device is None or device.index is None else device.index
    if index not in _sm_counts:
        _sm_counts[index] = torch.cuda.get_device_properties(index).multi_processor_count
    return _sm_counts[index]


def split_k_for(m: int, n: int, k: int) -> int:
    """How many blocks share the K range of one output tile of a skinny product (m <= SKINNY_M).
    More blocks stream weights from more SMs: about 64 blocks in all, at least four k-blocks of 64
    each, and 1, 2, 4 or 8 ways (the blocks of a tile form one cluster)."""
    if m > SKINNY_M:
        return 1
    tiles = -(-n // 128) * -(-m // min(SKINNY_BN_MAX, 16 if m <= 16 else 32 if m <= 32 else 64))
    by_blocks = SPLIT_TARGET_BLOCKS // tiles
    if tiles * 8 <= SPLIT_TARGET_BLOCKS + 32:
        by_blocks = 8  # 17 to 20 tiles: eight ways (up to 160 blocks) beat four (2,560 rows of 9,728: 14.0 against 17.2 us)
    limit = min(by_blocks, (k // 64) // SPLIT_MIN_K_BLOCKS, 8)
    return 8 if limit >= 8 else 4 if limit >= 4 else 2 if limit >= 2 else 1


def set_pdl(on: bool) -> bool:
    """Switches programmatic dependent launch for all later kernel launches; returns the old setting."""
    from .library import library

    return bool(library().gk_set_pdl(int(on)))


GEMV_MAX_TOKENS = 16
GEMV_MAX_TOKENS_SHORT_K = 32  # with the activations of all tokens in registers (see gemv_suits)


def gemv_max_rows(device: torch.device) -> int:
    """Most weight rows ``gemv`` takes: one block per SM, each with up to eight groups of eight rows."""
    return sm_count(device) * 64



def set_gemm_pairs(mode: int) -> int:
    """How many-token products with wide tiles are run: 1 as pairs of blocks on one 256 x 256 tile (tcgen05
    cta_group::2), 0 as single blocks on 128 x 256 tiles, 2 (the default) pairs where the product is large
    enough for them to be the faster choice.  Returns the old setting."""
    from .library import library

    return int(library().gk_set_gemm_pairs(int(mode)))


def gemv_suits(m: int, n: int, k: int, device: torch.device) -> bool:
    """Whether ``gemv`` is the kernel for ``[m, k] @ [n, k].T``: few tokens, few enough weight rows, and
    activations that fit in shared memory beside a block's weights (it takes longer K too, in rounds, but
    there the tensor-memory product is the better choice).  17 to 32 tokens only where the activations of
    all of them stay in registers: K of 257 to 1,024 and a block's weights in shared memory at once."""
    if n > gemv_max_rows(device):
        return False
    if m <= GEMV_MAX_TOKENS:
        rows = 8 if m <= 8 else 16
        return k <= 1024 or rows * k * 2 <= 96 * 1024
    if m <= GEMV_MAX_TOKENS_SHORT_K:
        per_warp = -(-(-(-k // 32)) // 8)  # 32-wide chunks of K a warp takes per group of eight weight rows
        groups = -(-n // 8)
        per_block = -(-groups // min(groups, gemv_max_rows(device) // 64))
        return 2 <= per_warp <= 4 and per_block * per_warp <= 24
    return False


def gemv(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16, swiglu: bool = False,
         out: torch.Tensor | None = None, gelu: bool = False, relu_squared: bool = False,
         xielu: tuple[float, float] | None = None) -> torch.Tensor:
    """``x [M, K] @ weight[N, K].T`` for up to 16 tokens (32 where ``gemv_suits`` says so): weights go from memory straight into registers and
    through ``mma.sync`` with 32-bit accumulation; made for the latency of a decode step, where a projection
    is a few megabytes of weights and next to no arithmetic.  ``swiglu`` as in ``gemm_tc``; ``gelu`` stores the tanh form
    of GELU of every result (the 32-bit sums go through it before they are rounded), ``relu_squared`` the square of its
    relu, ``xielu = (up, down)`` the activation ``up z^2 + z/2`` above zero and ``down (exp(z) - 1 - z) + z/2`` below."""
    require_device(x.device)
    _check(x, "x", torch.bfloat16, 2)
    _check(weight, "weight", torch.bfloat16, 2)
    m, k = x.shape
    n = weight.shape[0]
    if weight.shape[1] != k:
        raise KernelError(f"x is {tuple(x.shape)} but weight is {tuple(weight.shape)}")
    if m > GEMV_MAX_TOKENS_SHORT_K:
        raise KernelError(f"gemv takes up to {GEMV_MAX_TOKENS_SHORT_K} tokens, got {m}")
    if swiglu and n % 2:
        raise KernelError("the SwiGLU epilogue needs an even number of weight rows")
    if swiglu + gelu + relu_squared + (xielu is not None) > 1:
        raise KernelError("one output stage at a time: SwiGLU, GELU, squared relu or xIELU")
    n_out = n // 2 if swiglu else n
    if out is None:
        out = torch.empty((m, n_out), dtype=out_dtype, device=x.device)
    _check(out, "out", out_dtype, 2)
    if tuple(out.shape) != (m, n_out):
        raise KernelError(f"out has shape {tuple(out.shape)}, expected {(m, n_out)}")
    call("gk_gemv_bf16", ptr(weight), n, k, k, ptr(x), m, k, ptr(out), dtype_code(out_dtype),
         4 if xielu is not None else 3 if relu_squared else 2 if gelu else int(swiglu), float(xielu[0]) if xielu else 0.0,
         float(xielu[1]) if xielu else 0.0, stream_ptr())
    return out


def gemv_normed_suits(m: int, n: int, k: int, device: torch.device) -> bool:
    """Whether ``gemv_stream`` can form its activations as the RMSNorm of a 32-bit stream itself: up to 16 tokens whose
    rows (up to 1,024 long) a block's threads hold whole, and a block's weights in shared memory at once."""
    if m > GEMV_MAX_TOKENS or k > 1024 or k % 8 or n > gemv_max_rows(device):
        return False
    per_warp = -(-(-(-k // 32)) // 8)
    groups = -(-n // 8)
    per_block = -(-groups // min(groups, gemv_max_rows(device) // 64))
    return per_block * per_warp <= 24


def gemv_stream(weight: torch.Tensor, x: torch.Tensor | None = None, norm: tuple | None = None, resid: torch.Tensor | None = None,
                swiglu: bool = False, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor | None:
    """The few-token product with the residual stream at either end.

    ``norm = (h, norm_weight, eps)``: the activations are the RMSNorm of the rows of the 32-bit stream ``h [tokens, k]``,
    formed inside the kernel (no norm kernel in front).  ``resid``: the 32-bit stream ``[tokens, n]`` that the result,
    rounded to bfloat16 as a projection's output is, is added to in place (no add in the norm kernel behind); nothing
    is returned then.  Otherwise as ``gemv``."""
    require_device(weight.device)
    _check(weight, "weight", torch.bfloat16, 2)
    n, k = weight.shape
    if norm is not None:
        h, norm_weight, eps = norm
        _check(h, "h", torch.float32, 2)
        _check(norm_weight, "norm weight", dims=1)
        m = h.shape[0]
        if h.shape[1] != k or norm_weight.shape[0] != k:
            raise KernelError(f"the stream is {tuple(h.shape)} and the norm's weight {tuple(norm_weight.shape)} for rows of {k}")
        if not gemv_normed_suits(m, n, k, weight.device):
            raise KernelError(f"the norm on load does not take {m} tokens of {k} with {n} weight rows")
    else:
        _check(x, "x", torch.bfloat16, 2)
        m = x.shape[0]
        if x.shape[1] != k:
            raise KernelError(f"x is {tuple(x.shape)} but weight is {tuple(weight.shape)}")
        h, norm_weight, eps = None, None, 1.0
    out = None
    if resid is not None:
        _check(resid, "resid", torch.float32, 2)
        if tuple(resid.shape) != (m, n) or swiglu:
            raise KernelError(f"the residual stream must be {(m, n)} (and no SwiGLU), got {tuple(resid.shape)}")
    else:
        out = torch.empty((m, n // 2 if swiglu else n), dtype=out_dtype, device=weight.device)
    call("gk_gemv_bf16_stream", ptr(weight), n, k, k, ptr(x), m, k, ptr(out), dtype_code(out_dtype), int(swiglu), ptr(h), k,
         ptr(norm_weight), int(norm_weight is not None and norm_weight.dtype == torch.bfloat16), float(eps), ptr(resid), n, stream_ptr())
    return out


def gemm_tc(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16, swiglu: bool = False,
            splits: int = 1, out: torch.Tensor | None = None) -> torch.Tensor:
    """``x [M, K] @ weight[N, K].T`` in bfloat16 on the tcgen05 tensor cores, float32 accumulation.

    ``swiglu=True``: the rows of ``weight`` alternate gate, up, gate, up, ...; the result is
    ``silu(gate) * up`` of width ``N / 2``.  ``splits > 1`` shares the K range of every output tile
    among 2, 4 or 8 blocks (a skinny product then streams weights from more SMs); the blocks form a
    cluster and add their partial tiles through distributed shared memory in a fixed order.
    """
    require_device(x.device)
    _check(x, "x", torch.bfloat16, 2)
    _check(weight, "weight", torch.bfloat16, 2)
    m, k = x.shape
    n = weight.shape[0]
    if weight.shape[1] != k:
        raise KernelError(f"x is {tuple(x.shape)} but weight is {tuple(weight.shape)}")
    if swiglu and n % 2:
        raise KernelError("the SwiGLU epilogue needs an even number of weight rows")
    n_out = n // 2 if swiglu else n
    if out is None:
        out = torch.empty((m, n_out), dtype=out_dtype, device=x.device)
    _check(out, "out", out_dtype, 2)
    if tuple(out.shape) != (m, n_out):
        raise KernelError(f"out has shape {tuple(out.shape)}, expected {(m, n_out)}")
    flag = error_flag(x.device)
    if m <= SKINNY_M:
        bn = 16 if m <= 16 else 32 if m <= 32 else 64
        bn = min(bn, SKINNY_BN_MAX)
        call("gk_gemm_bf16_tc", ptr(weight), n, k, ptr(x), m, k, k, ptr(out), dtype_code(out_dtype), 1, n_out,
             EPI_SWIGLU_A if swiglu else EPI_STORE, bn, splits, 1, 0, ptr(flag), stream_ptr())
    else:
        wide = n >= PREFILL_BN and -(-m // 128) * -(-n // PREFILL_BN) >= 120  # enough wide tiles to fill the GPU
        bn = PREFILL_BN if wide else 128 if n >= 128 else 64 if n >= 64 else 32 if n >= 32 else 16
        call("gk_gemm_bf16_tc", ptr(x), m, k, ptr(weight), n, k, k, ptr(out), dtype_code(out_dtype), n_out, 1,
             EPI_SWIGLU_B if swiglu else EPI_STORE, bn, splits, 0, 1, ptr(flag), stream_ptr())
    return out


@functools.lru_cache(maxsize=None)
def decode_cluster_places(head_dim: int, sm_count: int) -> tuple[int, int, int, int]:
    """How many clusters of 1, 2, 4 and 8 blocks of the decode attention kernel the device holds at once.  Asked of the
    device where there is one (clusters are placed inside a GPC, so eight-block clusters fill fewer of the SMs' places
    than single blocks do); two blocks an SM otherwise."""
    if torch.cuda.is_available():
        from .library import library

        got = [library().gk_attention_decode_resident_clusters(int(head_dim), c) for c in (1, 2, 4, 8)]
        if all(g > 0 for g in got):
            return tuple(got)
    return tuple(2 * sm_count // c for c in (1, 2, 4, 8))


@functools.lru_cache(maxsize=4096)
def decode_splits(n_seqs: int, n_kv: int, max_kv_len: int, page_size: int, sm_count: int,
                  cluster_places: tuple[int, int, int, int] | None = None) -> int:
    """How many blocks share a sequence's pages in decode attention.

    Two blocks fit an SM.  With few (sequence, kv head) pairs and a long context, as many splits as fill those
    places go through scratch and a second kernel.  Otherwise 1, 2, 4 or 8 splits merge inside the kernel (a
    cluster per pair, which then does the q/k preparation too), and the number is the one with the lowest
    estimate of  waves of clusters x (pages a block streams + 8 pages' worth of time for what a block does
    besides); ``cluster_places`` says how many clusters of 1, 2, 4 and 8 blocks run at once (default: two blocks
    an SM, whatever the cluster).  It agrees with step times measured at batch 1 to 64 with 2,048-token contexts;
    against the old "fill the places once" rule it gains 7 to 13% at batch 12, 40 and 48 (clusters of three place
    badly: two splits are faster; 320 or 384 pairs are better cut in two than run as one and a bit waves)."""
    pairs = max(1, n_seqs * n_kv)
    pages = max(1, -(-max_kv_len // page_size))
    places = 2 * sm_count
    fill = max(1, min(places // pairs, pages, 64))
    # (one and two sequences of 8,192 tokens are faster as clusters of eight, 0.83 and 0.91 ms a step against 0.85 and 0.98
    # through scratch; of 16,384 tokens slower, 1.18 and 1.45 against 1.03 and 1.32)
    if fill >= SCRATCH_SPLITS_FROM and max_kv_len >= 12288:
        return fill
    if cluster_places is None:
        cluster_places = tuple(places // c for c in (1, 2, 4, 8))
    at_once = dict(zip((1, 2, 4, 8), cluster_places))

    def estimate(splits: int) -> float:
        # clusters of eight that have to share SMs cost more besides their pages than the eight say, the more of the SMs
        # hold two of their blocks (four sequences of 2,048 tokens: 0.73 ms a step with four splits, 0.76 with eight; three
        # sequences: 0.70 with four, 0.65 with eight; one and two sequences are faster with eight)
        besides = 8.0
        if splits == 8 and pairs * splits > sm_count:
            besides = 13.0 if pairs * splits > 1.5 * sm_count else 10.0
        return -(-pairs // max(1, at_once[splits])) * (pages / splits + besides)

    return min((s for s in (1, 2, 4, 8) if s <= pages), key=lambda s: (estimate(s), s))


def decode_flat_wins(n_seqs: int, n_kv: int, kv_len: int, page_size: int, sm_count: int,
                     cluster_places: tuple[int, int, int, int] | None, flat_places: int) -> bool:
    """Whether dealing the step's pages out evenly among all blocks is expected to beat the best equal cut.

    The evenly dealt kernel costs some 7 us more than the equal cut where that fits the device (partial results
    through scratch, a ticket per part, a merge by whoever comes last), so it is chosen where the equal cut fits
    badly.  Measured, 28 layers of the 0.6B sizes, ms a step with the equal cut against dealt evenly:

    * blocks that come in two waves of which the second is thin: contexts of 2,048, 40 sequences (320 pairs on 296
      places) 2.86 / 2.57, 44: 2.88 / 2.78, but 48: 2.89 / 2.91, 52: 3.00 / 3.05, 56: 3.13 / 3.21, 60: 3.17 / 3.33; contexts
      of 512, 40: 1.57 / 1.53; of 1,024, 40: 2.05 / 1.91 but 56: 2.16 / 2.26;
    * three and more waves of clusters: contexts of 4,096, 40 sequences (five waves of clusters of four) 4.13 / 3.90; of
      8,192, 40: 6.67 / 6.61;
    * whole sequences a block that fill little more than half of the places and are long: 20 sequences of 4,096
      2.57 / 2.34, of 8,192 4.06 / 3.70, but of 2,048 1.66 / 1.70; 24 of 2,048 1.71 / 1.83, of 4,096 2.72 / 2.70;
    * clusters of eight that share SMs on long contexts: 32,768 tokens, 3 sequences 2.66 / 2.42, 4: 3.17 / 2.92; 16,384, 4:
      2.09 / 2.05 but 3: 1.34 / 1.64, 6 (cut in four): 2.37 / 2.63; 8,192, 4: 1.19 / 1.45.

    Elsewhere the equal cut is ahead: 8 sequences of 2,048 tokens 0.82 / 1.1, 12: 1.11 / 1.21, 16: 1.25 / 1.5, 32: 1.98 / 2.2,
    64: 3.26 / 3.5; 12 of 8,192 (cut in two): 2.33 / 2.48."""
    splits = decode_splits(n_seqs, n_kv, kv_len, page_size, sm_count, cluster_places)
    if splits > 8:
        return False
    pairs = max(1, n_seqs * n_kv)
    pages = max(1, -(-kv_len // page_size))
    if cluster_places is None:
        cluster_places = tuple(2 * sm_count // c for c in (1, 2, 4, 8))
    at_once = max(1, dict(zip((1, 2, 4, 8), cluster_places))[splits])
    waves = -(-pairs // at_once)
    fill = pairs / (waves * at_once)
    per_block = pairs * pages / flat_places  # pages a block streams when they are dealt evenly
    if waves == 1:
        if splits == 8 and pairs * 8 > sm_count:
            # the more of the SMs hold two blocks of a cluster of eight, the sooner
            return per_block >= (24 if pairs * 8 > 1.5 * sm_count else 30)
        return splits == 1 and fill < 0.66 and per_block >= 28
    return fill < (0.62 if waves == 2 else 0.92)


def attention_decode(
    q: torch.Tensor,
    kv: PagedKV,
    kv_len: torch.Tensor,
    slots: torch.Tensor,
    scale: float,
    window: int = 0,
    n_splits: int = 1,
    out: torch.Tensor | None = None,
    use_scratch: bool = False,
    sink: bool = False,
) -> torch.Tensor:
    """(``sink``: one more term in the softmax's denominator, a key of score 0 without a value.)
    Attention of one new token per sequence (``q [n_seqs, n_q, d]`` bfloat16, ``d`` 64 or 128) over
    the pages; ``kv_len[i]`` counts the sequence's cached tokens including the new one.  Up to eight
    splits merge inside one kernel (a cluster per sequence and kv head); more, or ``use_scratch``, go
    through scratch memory allocated here and a second kernel."""
    require_device(q.device)
    _check(q, "q", torch.bfloat16, 3)
    n, n_q, d = q.shape
    _check(kv.k, "k pages", torch.bfloat16, 4)
    _check(kv.v, "v pages", torch.bfloat16, 4)
    _check(kv_len, "kv_len", torch.int32, 1)
    _check(slots, "slots", torch.int32, 1)
    if kv_len.shape[0] != n or slots.shape[0] != n:
        raise KernelError("kv_len and slots need one entry per sequence")
    n_kv = kv.k.shape[1]
    if kv.k.shape[3] != d:
        raise KernelError(f"pages have head_dim {kv.k.shape[3]}, queries {d}")
    if out is None:
        out = torch.empty_like(q)
    part_o = part_ml = None
    if n_splits > 8 or (n_splits > 1 and use_scratch):
        part_o = torch.empty((n * n_q * n_splits * d,), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((n * n_q * n_splits * 2,), dtype=torch.float32, device=q.device)
    call(
        "gk_attention_decode_bf16", ptr(q), ptr(kv.k), ptr(kv.v), ptr(out), ptr(part_o), ptr(part_ml), ptr(kv_len),
        ptr(slots), ptr(kv.block_table), n, n_q, n_kv, d, kv.max_pages, kv.page_size, float(scale), int(window),
        int(n_splits), int(sink), stream_ptr(),
    )
    return out


def attention_decode_fused(
    qkv: torch.Tensor,
    n_q: int,
    n_kv: int,
    head_dim: int,
    q_weight: torch.Tensor | None,
    k_weight: torch.Tensor | None,
    eps: float,
    cos: torch.Tensor | None,
    sin: torch.Tensor | None,
    kv: PagedKV,
    kv_len: torch.Tensor,
    slots: torch.Tensor,
    max_position: int,
    scale: float,
    window: int = 0,
    n_splits: int = 1,
    write_kv: bool = True,
) -> torch.Tensor:
    """Decode attention straight from the packed projection of the new tokens: per-head q/k RMSNorm,
    rotation, the write of the new key and value into the pages and the attention itself in one kernel
    (bfloat16, head size 64 or 128, at most 8 splits).  Returns ``[n_seqs, n_q, head_dim]``."""
    require_device(qkv.device)
    _check(qkv, "qkv", torch.bfloat16, 2)
    n = qkv.shape[0]
    if qkv.shape[1] != (n_q + 2 * n_kv) * head_dim:
        raise KernelError(f"qkv rows are {qkv.shape[1]} wide, expected {(n_q + 2 * n_kv) * head_dim}")
    _check(kv.k, "k pages", torch.bfloat16, 4)
    _check(kv.v, "v pages", torch.bfloat16, 4)
    _check(kv_len, "kv_len", torch.int32, 1)
    _check(slots, "slots", torch.int32, 1)
    if kv.k.shape[1] != n_kv or kv.k.shape[3] != head_dim:
        raise KernelError(f"pages {tuple(kv.k.shape)} do not fit n_kv={n_kv}, head_dim={head_dim}")
    if n_splits > 8:
        raise KernelError("the fused decode attention takes at most 8 splits")
    use_norm = q_weight is not None
    weight_code = 0
    if use_norm:
        _check(q_weight, "q_weight", dims=1)
        _check(k_weight, "k_weight", q_weight.dtype, 1)
        weight_code = dtype_code(q_weight.dtype)
    table_positions = 0
    if cos is not None:
        _check(cos, "cos", torch.float32, 2)
        _check(sin, "sin", torch.float32, 2)
        if cos.shape[1] != head_dim // 2 or sin.shape != cos.shape:
            raise KernelError("rotary tables must be [positions, head_dim / 2]")
        table_positions = cos.shape[0]
    out = torch.empty((n, n_q, head_dim), dtype=torch.bfloat16, device=qkv.device)
    call(
        "gk_attention_decode_fused_bf16", ptr(qkv), ptr(q_weight), ptr(k_weight), weight_code, int(use_norm), float(eps),
        ptr(cos), ptr(sin), table_positions, int(max_position), int(write_kv), ptr(kv.k), ptr(kv.v), ptr(out), None, None,
        ptr(kv_len), ptr(slots), ptr(kv.block_table), n, n_q, n_kv, head_dim, kv.max_pages, kv.page_size, float(scale),
        int(window), int(n_splits), stream_ptr(),
    )
    return out


@functools.lru_cache(maxsize=None)
def decode_flat_places(head_dim: int, sm_count: int) -> int:
    """How many blocks of the evenly dealt decode attention kernel the device holds at once: the most pieces that
    the step's pages are cut into.  Asked of the device where there is one; two blocks an SM otherwise."""
    if torch.cuda.is_available():
        from .library import library

        got = library().gk_attention_decode_flat_resident_blocks(int(head_dim))
        if got > 0:
            return got
    return 2 * sm_count


def attention_decode_flat(
    q: torch.Tensor | None,
    qkv: torch.Tensor | None,
    n_q: int,
    n_kv: int,
    head_dim: int,
    q_weight: torch.Tensor | None,
    k_weight: torch.Tensor | None,
    eps: float,
    cos: torch.Tensor | None,
    sin: torch.Tensor | None,
    kv: PagedKV,
    kv_len: torch.Tensor,
    slots: torch.Tensor,
    max_position: int,
    scale: float,
    window: int = 0,
    n_blocks: int = 0,
    write_kv: bool = True,
) -> torch.Tensor:
    """Decode attention with the pages of all sequences dealt out evenly among ``n_blocks`` blocks (0: as many
    as the device holds at once), whatever the sequences' lengths.  Either ``q [n_seqs, n_q, head_dim]`` (keys and
    values are in the pages) or the packed projection ``qkv [n_seqs, (n_q + 2 n_kv) * head_dim]`` of the new tokens,
    which the kernel then norms, rotates and writes itself as ``attention_decode_fused`` does.  Returns
    ``[n_seqs, n_q, head_dim]`` bfloat16."""
    if (q is None) == (qkv is None):
        raise KernelError("either q or qkv")
    given = q if qkv is None else qkv
    require_device(given.device)
    if qkv is None:
        _check(q, "q", torch.bfloat16, 3)
        if q.shape[1] != n_q or q.shape[2] != head_dim:
            raise KernelError(f"q is {tuple(q.shape)}, expected [n, {n_q}, {head_dim}]")
    else:
        _check(qkv, "qkv", torch.bfloat16, 2)
        if qkv.shape[1] != (n_q + 2 * n_kv) * head_dim:
            raise KernelError(f"qkv rows are {qkv.shape[1]} wide, expected {(n_q + 2 * n_kv) * head_dim}")
    n = given.shape[0]
    _check(kv.k, "k pages", torch.bfloat16, 4)
    _check(kv.v, "v pages", torch.bfloat16, 4)
    _check(kv_len, "kv_len", torch.int32, 1)
    _check(slots, "slots", torch.int32, 1)
    if kv_len.shape[0] != n or slots.shape[0] != n:
        raise KernelError("kv_len and slots need one entry per sequence")
    if kv.k.shape[1] != n_kv or kv.k.shape[3] != head_dim:
        raise KernelError(f"pages {tuple(kv.k.shape)} do not fit n_kv={n_kv}, head_dim={head_dim}")
    use_norm = qkv is not None and q_weight is not None
    weight_code = 0
    if use_norm:
        _check(q_weight, "q_weight", dims=1)
        _check(k_weight, "k_weight", q_weight.dtype, 1)
        weight_code = dtype_code(q_weight.dtype)
    table_positions = 0
    if qkv is not None and cos is not None:
        _check(cos, "cos", torch.float32, 2)
        _check(sin, "sin", torch.float32, 2)
        if cos.shape[1] != head_dim // 2 or sin.shape != cos.shape:
            raise KernelError("rotary tables must be [positions, head_dim / 2]")
        table_positions = cos.shape[0]
    else:
        cos = sin = None
    if n_blocks <= 0:
        n_blocks = decode_flat_places(head_dim, sm_count(given.device))
    work = kv.work if kv.work is not None else DecodeWork(given.device)
    part, tickets = work.get((n_blocks + n * n_kv) * (n_q // n_kv) * (head_dim + 2), n * n_kv)
    out = torch.empty((n, n_q, head_dim), dtype=torch.bfloat16, device=given.device)
    call(
        "gk_attention_decode_flat_bf16", ptr(q), ptr(qkv), ptr(q_weight) if use_norm else None,
        ptr(k_weight) if use_norm else None, weight_code, int(use_norm), float(eps), ptr(cos), ptr(sin), table_positions,
        int(max_position), int(write_kv), ptr(kv.k), ptr(kv.v), ptr(out), ptr(part), ptr(tickets), ptr(kv_len), ptr(slots),
        ptr(kv.block_table), n, n_q, n_kv, head_dim, kv.max_pages, kv.page_size, float(scale), int(window), int(n_blocks),
        stream_ptr(),
    )
    return out


def attention_prefill(
    q: torch.Tensor,
    kv: PagedKV,
    cu_q: torch.Tensor,
    kv_len: torch.Tensor,
    slots: torch.Tensor,
    max_q_len: int,
    scale: float,
    window: int = 0,
    out: torch.Tensor | None = None,
    tensor_cores: str = "auto",
    sink: bool = False,
) -> torch.Tensor:
    """Causal attention of the packed new tokens ``q [n_tokens, n_q, d]`` (bfloat16, ``d`` 64 or 128) of
    ``n_seqs`` sequences over the pages.  Sequence ``i`` owns tokens ``cu_q[i] .. cu_q[i+1]-1``, which
    are its last positions: ``kv_len[i]`` counts its cached tokens including them.  ``tensor_cores``:
    ``"tcgen05"`` (head size 128 only), ``"mma"`` (the warp-level kernel), or ``"auto"``.  ``sink``: one more term in
    the softmax's denominator, a key of score 0 without a value."""
    require_device(q.device)
    _check(q, "q", torch.bfloat16, 3)
    n, n_q, d = q.shape
    _check(kv.k, "k pages", torch.bfloat16, 4)
    _check(kv.v, "v pages", torch.bfloat16, 4)
    for name, t in (("cu_q", cu_q), ("kv_len", kv_len), ("slots", slots)):
        _check(t, name, torch.int32, 1)
    n_seqs = kv_len.shape[0]
    if cu_q.shape[0] != n_seqs + 1 or slots.shape[0] != n_seqs:
        raise KernelError("cu_q needs n_seqs + 1 entries, slots and kv_len n_seqs")
    n_kv = kv.k.shape[1]
    if kv.k.shape[3] != d:
        raise KernelError(f"pages have head_dim {kv.k.shape[3]}, queries {d}")
    if out is None:
        out = torch.empty_like(q)
    if tensor_cores not in ("auto", "tcgen05", "mma"):
        raise KernelError(f"tensor_cores must be auto, tcgen05 or mma, got {tensor_cores!r}")
    if tensor_cores == "tcgen05" and d != 128:
        raise KernelError("the tcgen05 prefill attention takes head size 128 only")
    if tensor_cores == "tcgen05" or (tensor_cores == "auto" and d == 128):
        call(
            "gk_attention_prefill_tc_tokens_bf16", ptr(q), ptr(kv.k), ptr(kv.v), ptr(out), ptr(cu_q), ptr(kv_len), ptr(slots),
            ptr(kv.block_table), n_seqs, int(max_q_len), n_q, n_kv, d, kv.max_pages, kv.page_size, kv.k.shape[0],
            float(scale), int(window), ptr(error_flag(q.device)), stream_ptr(), int(q.shape[0]), int(sink),
        )
        return out
    call(
        "gk_attention_prefill_bf16", ptr(q), ptr(kv.k), ptr(kv.v), ptr(out), ptr(cu_q), ptr(kv_len), ptr(slots),
        ptr(kv.block_table), n_seqs, int(max_q_len), n_q, n_kv, d, kv.max_pages, kv.page_size, float(scale), int(window),
        int(sink), stream_ptr(),
    )
    return out


def set_attention_prefill_keys(keys: int) -> int:
    """Keys per step of the tcgen05 prefill attention: 128 (the default: one block per SM, two score buffers,
    two threads a row, a heavy and a light query tile per block) or 64 (two blocks per SM, one query tile
    each).  Returns the old setting."""
    from .library import library

    return int(library().gk_set_attention_prefill_keys(int(keys)))


def set_attention_prefill_stay(mode: int) -> int:
    """Whether the tcgen05 prefill attention (128 keys a step) runs as blocks that stay, one an SM, and take query tiles
    from the launch's list with the next tile's queries and first scores under the tile in hand: 1 = always, 2 (the
    default) = where the launch has more tiles than the device SMs, 0 = never (a block a tile).  Returns the old setting."""
    from .library import library

    return int(library().gk_set_attention_prefill_stay(int(mode)))


def set_attention_prefill_one_tile(mode: int) -> int:
    """How the tcgen05 prefill attention (128 keys a step) deals out its query tiles: 1 (the default) = a tile a
    block with the heaviest first, 0 = a heavy and a light tile a block.  Returns the old setting."""
    from .library import library

    return int(library().gk_set_attention_prefill_one_tile(int(mode)))


def row_parts(n_rows: int, vocab: int, device: torch.device) -> int:
    """Blocks that share a row of logits in the token choice: about eight blocks per multiprocessor in all, slices
    of at least 4,096 entries, at most 64 a row."""
    return max(1, min(8 * sm_count(device) // max(n_rows, 1), vocab // 4096, 64))


def argmax(logits: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """Index of the largest logit of each row (lowest index on ties), int32."""
    require_device(logits.device)
    _check(logits, "logits", torch.float32, 2)
    n, vocab = logits.shape
    if out is None:
        out = torch.empty((n,), dtype=torch.int32, device=logits.device)
    _check(out, "out", torch.int32, 1)
    # few rows of a wide vocabulary: several blocks share a row so that the scan uses the whole GPU
    parts = row_parts(n, vocab, logits.device)
    scratch = torch.empty((n * parts * 2,), dtype=torch.int32, device=logits.device) if parts > 1 else None
    call("gk_argmax", ptr(logits), vocab, n, vocab, ptr(out), parts, ptr(scratch), stream_ptr())
    return out


def sample(
    logits: torch.Tensor,
    temperature: float,
    top_k: int,
    seed: int,
    request_ids: torch.Tensor,
    steps: torch.Tensor,
    advance_steps: bool = False,
    out: torch.Tensor | None = None,
) -> torch.Tensor:
    """Temperature (+ top-k) sampling by the Gumbel-max rule with counter-based uniforms.

    Row ``r`` draws with the key ``(seed, request_ids[r], steps[r])``; with ``advance_steps`` the
    kernel adds one to ``steps[r]`` afterwards, so a loop replayed from a CUDA graph needs no host
    work between tokens.
    """
    require_device(logits.device)
    _check(logits, "logits", torch.float32, 2)
    n, vocab = logits.shape
    _check(request_ids, "request_ids", torch.int32, 1)
    _check(steps, "steps", torch.int32, 1)
    if out is None:
        out = torch.empty((n,), dtype=torch.int32, device=logits.device)
    _check(out, "out", torch.int32, 1)
    # as for argmax: several blocks share a row; eight bytes of scratch per row for the top-k thresholds (four
    # used) and eight per row and part for the parts' results
    parts = row_parts(n, vocab, logits.device)
    scratch = torch.empty((2 * ((n + 1) // 2) + 2 * n * parts,), dtype=torch.int32, device=logits.device)
    call(
        "gk_sample", ptr(logits), vocab, n, vocab, float(temperature), int(top_k or 0), int(seed) & (2**64 - 1),
        ptr(request_ids), ptr(steps), int(advance_steps), ptr(out), parts, ptr(scratch), stream_ptr(),
    )
    return out


def linear_bf16(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """``x @ weight.T`` for bfloat16 operands with 32-bit accumulation (library matrix product,
    as the reference's nn.Linear under autocast is: src/engine.py:35)."""
    require_device(x.device)
    _check(x, "x", torch.bfloat16, 2)
    _check(weight, "weight", torch.bfloat16, 2)
    if weight.shape[1] != x.shape[1]:
        raise KernelError(f"x is {tuple(x.shape)} but weight is {tuple(weight.shape)}")
    y = torch.mm(x, weight.t())
    return y if out_dtype == torch.bfloat16 else y.to(out_dtype)


# ------------------------------------------------------------------ a run of layers of a decode step as one kernel
DECODE_LAYERS_MAX_SEQS = 8


def decode_layers_work_sizes(n_seqs: int, hidden: int, n_q: int, n_kv: int, head_dim: int, inter: int, max_kv_len: int,
                             page_size: int) -> tuple[int, int] | None:
    """(floats of partial results, 32-bit words of counters) that ``decode_layers`` needs for these sizes, or None if
    the kernel does not take them (the library's message says why: ``library().gk_last_error()``)."""
    import ctypes

    from .library import library

    out = (ctypes.c_longlong * 2)()
    status = library().gk_decode_layers_plan(n_seqs, hidden, n_q, n_kv, head_dim, inter, max_kv_len, page_size, out)
    return (int(out[0]), int(out[1])) if status == 0 else None


def decode_layers(layer_table: torch.Tensor, n_layers: int, h: torch.Tensor, n_q: int, n_kv: int, head_dim: int, inter: int,
                  qkv: torch.Tensor, att: torch.Tensor, act: torch.Tensor, part: torch.Tensor, words: torch.Tensor,
                  kv_len: torch.Tensor, slots: torch.Tensor, block_table: torch.Tensor, max_kv_len: int,
                  cos: torch.Tensor | None, sin: torch.Tensor | None, norm_bf16: bool, qk_bf16: bool, scale: float,
                  stamps: torch.Tensor | None = None) -> None:
    """Runs ``n_layers`` pre-norm layers (RMSNorm, grouped-query attention with per-head q/k norm and rotation over
    the paged cache, RMSNorm, SwiGLU) of a decode step on the stream ``h [n_seqs, hidden]`` (float32, updated in
    place) as one persistent kernel.  ``layer_table``: the layers' pointers and constants as the kernel's records (96
    bytes each, see ``models/persistent_decode.py``); ``qkv``, ``att``, ``act``, ``part``, ``words``: work areas
    (``words`` zero before the first call; the kernel leaves it zero).  ``stamps`` (int64 ``[blocks, 5 n_layers, 2]``,
    for measurements): every block's clock readings, in nanoseconds, at its arrival at and release from each barrier."""
    require_device(h.device)
    _check(h, "h", torch.float32, 2)
    _check(layer_table, "layer_table", torch.uint8, 1)
    n_seqs, hidden = h.shape
    if layer_table.shape[0] < 96 * n_layers:
        raise KernelError("the layer table is shorter than its layers")
    for name, t, dtype in (("qkv", qkv, torch.bfloat16), ("att", att, torch.bfloat16), ("act", act, torch.bfloat16),
                           ("part", part, torch.float32), ("words", words, torch.int32), ("kv_len", kv_len, torch.int32),
                           ("slots", slots, torch.int32)):
        _check(t, name, dtype)
    _check(block_table, "block_table", torch.int32, 2)
    if qkv.numel() < n_seqs * (n_q + 2 * n_kv) * head_dim or att.numel() < n_seqs * n_q * head_dim or act.numel() < n_seqs * inter:
        raise KernelError("a work area is smaller than the step needs")
    if words.numel() < 8 + n_seqs * n_kv or kv_len.shape[0] != n_seqs or slots.shape[0] != n_seqs:
        raise KernelError("counters, lengths and slots need one entry per sequence (and kv head)")
    table_positions = 0
    if cos is not None:
        _check(cos, "cos", torch.float32, 2)
        _check(sin, "sin", torch.float32, 2)
        if cos.shape[1] != head_dim // 2 or sin.shape != cos.shape:
            raise KernelError("rotary tables must be [positions, head_dim / 2]")
        table_positions = cos.shape[0]
    call("gk_decode_layers", ptr(layer_table), n_layers, n_seqs, hidden, n_q, n_kv, head_dim, inter, ptr(h), ptr(qkv), ptr(att),
         ptr(act), ptr(part), part.numel(), ptr(words), ptr(kv_len), ptr(slots), ptr(block_table), block_table.shape[1],
         int(max_kv_len), ptr(cos), ptr(sin), table_positions, int(norm_bf16), int(qk_bf16), float(scale),
         ptr(error_flag(h.device)), ptr(stamps), stream_ptr())


# ------------------------------------------------------------------ rows in pages, and attention through a latent
@dataclass
class PagedRows:
    """One layer's per-position rows in pages: ``rows [n_pages, page_size, width]`` and the table that maps a
    sequence's pages (as in ``PagedKV``).  A latent-attention layer keeps one such row per position for all heads."""

    rows: torch.Tensor
    block_table: torch.Tensor

    @property
    def page_size(self) -> int:
        return self.rows.shape[1]

    @property
    def max_pages(self) -> int:
        return self.block_table.shape[1]


def branch_merge(x: torch.Tensor, y: torch.Tensor, norm_weight: torch.Tensor, eps: float, scale: torch.Tensor | None = None,
                 kept: torch.Tensor | None = None, n_kept: int = 0, mix: torch.Tensor | None = None,
                 next_weight: torch.Tensor | None = None, next_eps: float = 0.0, next_dtype: torch.dtype = torch.float32,
                 x_out: torch.Tensor | None = None, copy_dtype: torch.dtype | None = None):
    """``v = x + scale * rmsnorm(y) * norm_weight``; with ``kept`` ``[n, rows, width]``: ``kept[n_kept] = v`` and
    ``v = sum_{j <= n_kept} mix[j] * kept[j]``; the new stream goes to ``x_out`` (default: ``x`` itself); with
    ``next_weight`` also returns ``rmsnorm(v) * next_weight`` in ``next_dtype``; with ``copy_dtype`` instead, the new
    stream itself in that type (for a sublayer that reads the stream without a norm).  All weights are 32-bit effective
    weights.  Returns ``(stream, normed or copy or None)``."""
    require_device(x.device)
    _check(x, "x", torch.float32, 2)
    _check(y, "y", dims=2)
    rows, width = x.shape
    if y.shape != x.shape:
        raise KernelError(f"branch {tuple(y.shape)} does not match the stream {tuple(x.shape)}")
    for name, t in (("norm_weight", norm_weight), ("scale", scale), ("next_weight", next_weight)):
        if t is not None:
            _check(t, name, torch.float32, 1)
            if t.shape[0] != width:
                raise KernelError(f"{name} has {t.shape[0]} entries for rows of {width}")
    stride = 0
    if kept is not None:
        _check(kept, "kept", torch.float32, 3)
        _check(mix, "mix", torch.float32, 1)
        if kept.shape[1:] != x.shape or not 0 <= n_kept < kept.shape[0] or mix.shape[0] != n_kept + 1:
            raise KernelError(f"history {tuple(kept.shape)} / mixing weights {tuple(mix.shape)} do not fit entry {n_kept} of a "
                              f"stream {tuple(x.shape)}")
        stride = kept.stride(0)
    if x_out is None:
        x_out = x
    _check(x_out, "x_out", torch.float32, 2)
    z = None
    if next_weight is not None:
        z = torch.empty((rows, width), dtype=next_dtype, device=x.device)
    elif copy_dtype is not None:
        next_dtype = copy_dtype
        z = torch.empty((rows, width), dtype=copy_dtype, device=x.device)
    call("gk_branch_merge", ptr(x), ptr(y), dtype_code(y.dtype), ptr(norm_weight), ptr(scale), float(eps), ptr(kept), stride,
         int(n_kept), ptr(mix), ptr(x_out), ptr(next_weight), float(next_eps), ptr(z), dtype_code(next_dtype), rows, width,
         stream_ptr())
    return x_out, z


def causal_conv(a: torch.Tensor, weight: torch.Tensor, state: torch.Tensor | None, tok_pos: torch.Tensor, tok_seq: torch.Tensor,
                cu_q: torch.Tensor, slots: torch.Tensor, out_dtype: torch.dtype, update_single_token_state: bool = False) -> torch.Tensor:
    """``a + conv(a)`` over time on each channel: ``a [n_tokens, width]`` 32-bit, ``weight [taps, width]`` 32-bit (tap by tap, so
    that neighbouring channels' weights lie side by side),
    ``state [n_slots, taps - 1, width]`` the sequences' inputs of before (read only; ``conv_state`` brings it up to date
    afterwards).  ``update_single_token_state``: every sequence of the step brings exactly one token, and the kernel moves
    the states on itself."""
    require_device(a.device)
    _check(a, "a", torch.float32, 2)
    _check(weight, "weight", torch.float32, 2)
    n, width = a.shape
    taps = weight.shape[0]
    if weight.shape[1] != width:
        raise KernelError(f"convolution weights {tuple(weight.shape)} for rows of {width}")
    if taps > 1:
        _check(state, "state", torch.float32, 3)
        if tuple(state.shape[1:]) != (taps - 1, width):
            raise KernelError(f"state {tuple(state.shape)} does not hold {taps - 1} inputs of width {width}")
    out = torch.empty((n, width), dtype=out_dtype, device=a.device)
    call("gk_causal_conv", ptr(a), ptr(weight), ptr(state) if taps > 1 else None, ptr(tok_pos), ptr(tok_seq), ptr(cu_q),
         ptr(slots), ptr(out), dtype_code(out_dtype), n, width, taps, int(bool(update_single_token_state)), stream_ptr())
    return out


def conv_state(a: torch.Tensor, state: torch.Tensor, cu_q: torch.Tensor, slots: torch.Tensor, n_seqs: int) -> None:
    """Brings the sequences' convolution states up to date after ``causal_conv`` has read them: each holds its
    sequence's last ``taps - 1`` inputs."""
    _check(a, "a", torch.float32, 2)
    _check(state, "state", torch.float32, 3)
    call("gk_conv_state", ptr(a), ptr(state), ptr(cu_q), ptr(slots), int(n_seqs), a.shape[1], state.shape[1] + 1, stream_ptr())


def gelu_tanh(x: torch.Tensor) -> torch.Tensor:
    """``0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))`` in 32-bit, element by element."""
    require_device(x.device)
    _check(x, "x")
    out = torch.empty_like(x)
    call("gk_gelu_tanh", ptr(x), ptr(out), dtype_code(x.dtype), x.numel(), stream_ptr())
    return out


def latent_prepare(proj: torch.Tensor, q_rank: int, rank: int, rot: int, rot_dims: int, w_q: torch.Tensor, w_kv: torch.Tensor,
                   eps: float, cos: torch.Tensor | None, sin: torch.Tensor | None, tok_pos: torch.Tensor, tok_seq: torch.Tensor,
                   slots: torch.Tensor, cache: PagedRows, max_position: int, write: bool = True) -> torch.Tensor:
    """From the packed projection rows ``[q latent | kv latent | shared key part]``: returns the normed q latent
    ``[n, q_rank]`` and writes each position's cache row (normed kv latent, rotated shared key part)."""
    require_device(proj.device)
    _check(proj, "proj", dims=2)
    n = proj.shape[0]
    if proj.shape[1] != q_rank + rank + rot:
        raise KernelError(f"projection rows of {proj.shape[1]} are not {q_rank} + {rank} + {rot}")
    _check(w_q, "w_q", torch.float32, 1)
    _check(w_kv, "w_kv", torch.float32, 1)
    _check(cache.rows, "cache rows", proj.dtype, 3)
    if cache.rows.shape[2] != rank + rot:
        raise KernelError(f"cache rows of {cache.rows.shape[2]} are not {rank} + {rot}")
    table_rows = 0
    if rot_dims:
        _check(cos, "cos", torch.float32, 2)
        _check(sin, "sin", torch.float32, 2)
        if cos.shape[1] != rot_dims // 2 or sin.shape != cos.shape:
            raise KernelError(f"rotation tables {tuple(cos.shape)} do not hold {rot_dims // 2} angles a position")
        table_rows = cos.shape[0]
    out = torch.empty((n, q_rank), dtype=proj.dtype, device=proj.device)
    call("gk_latent_prepare", ptr(proj), dtype_code(proj.dtype), ptr(w_q), ptr(w_kv), float(eps), ptr(cos), ptr(sin),
         ptr(tok_pos), ptr(tok_seq), ptr(slots), ptr(cache.block_table), ptr(out), ptr(cache.rows) if write else None, n, q_rank,
         rank, rot, rot_dims, cache.max_pages, cache.page_size, int(max_position), table_rows, stream_ptr())
    return out


def attention_latent_exact(q_carried: torch.Tensor, q_raw: torch.Tensor, q_rot_at: int, rot: int, rot_dims: int,
                           cos: torch.Tensor | None, sin: torch.Tensor | None, cache: PagedRows, tok_pos: torch.Tensor,
                           tok_seq: torch.Tensor, slots: torch.Tensor, scale: float, window: int, out: torch.Tensor) -> torch.Tensor:
    """Attention of ``[q_carried (rank) | rotated part of q_raw]`` over the cached rows; the value of a row is its
    first ``rank`` entries.  ``q_carried`` and ``out`` are ``[n_tokens, n_heads, rank]`` views with any token and
    head strides (innermost contiguous); ``q_raw [n_tokens, n_heads, d]`` holds each head's part to rotate at
    ``q_rot_at``."""
    require_device(q_raw.device)
    _check(q_raw, "q_raw", dims=3)
    n, heads, raw_dim = q_raw.shape
    rank = q_carried.shape[2]
    for name, t in (("q_carried", q_carried), ("out", out)):
        if t.dtype != q_raw.dtype or tuple(t.shape) != (n, heads, rank) or t.stride(2) != 1:
            raise KernelError(f"{name} must be {q_raw.dtype} [{n}, {heads}, {rank}] with a contiguous last axis")
    _check(cache.rows, "cache rows", q_raw.dtype, 3)
    if cache.rows.shape[2] != rank + rot:
        raise KernelError(f"cache rows of {cache.rows.shape[2]} are not {rank} + {rot}")
    call("gk_attention_latent_exact", ptr(q_carried), q_carried.stride(0), q_carried.stride(1), ptr(q_raw), raw_dim, int(q_rot_at),
         ptr(cos), ptr(sin), ptr(cache.rows), ptr(out), out.stride(0), out.stride(1), dtype_code(q_raw.dtype), ptr(tok_pos),
         ptr(tok_seq), ptr(slots), ptr(cache.block_table), n, heads, rank, rot, rot_dims, cache.max_pages, cache.page_size,
         float(scale), int(window), stream_ptr())
    return out


def linear_batched(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """``out[b] = x[b] @ weight[b].T`` for a batch of products (one per head): ``x [B, M, K]`` and ``out [B, M, N]`` may be
    views with any batch and row strides (innermost contiguous), ``weight [B, N, K]`` is contiguous.  float32 weights go
    through the FP32-pipe kernel; bfloat16 ones through this library's small-product kernel for a few tokens (as the
    few-token product serves the projections) and through the library's batched product for many, both with 32-bit sums."""
    require_device(x.device)
    b, m, k = x.shape
    n = weight.shape[1]
    _check(weight, "weight", dims=3)
    if weight.shape[0] != b or weight.shape[2] != k or tuple(out.shape) != (b, m, n) or x.stride(2) != 1 or out.stride(2) != 1:
        raise KernelError(f"batched product of {tuple(x.shape)} with {tuple(weight.shape)} into {tuple(out.shape)}")
    if weight.dtype == torch.float32:
        call("gk_gemm_f32_batched", ptr(x), dtype_code(x.dtype), ptr(weight), ptr(out), dtype_code(out.dtype), b, m, n, k,
             x.stride(1), k, out.stride(1), x.stride(0), n * k, out.stride(0), stream_ptr())
        return out
    if weight.dtype != torch.bfloat16 or x.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("a bfloat16 batched product needs bfloat16 operands and output")
    if m <= GEMV_MAX_TOKENS:
        call("gk_heads_product_bf16", ptr(x), x.stride(0), x.stride(1), ptr(weight), ptr(out), out.stride(0), out.stride(1), b, m, n, k,
             stream_ptr())
        return out
    torch.bmm(x, weight.transpose(1, 2), out=out)
    return out


LATENT_TILED_MAX_SPLITS = 16


def latent_tiled_ok(n_heads: int, rank: int, rot: int, cache: PagedRows) -> bool:
    """Whether the tensor-core kernel takes the layer: bfloat16 rows in pages of 64, the latent a multiple of 64 up to
    512, the rotated part a multiple of 16 (other sizes run on the exact kernel)."""
    return (cache.rows.dtype == torch.bfloat16 and cache.page_size == 64 and rank % 64 == 0 and 0 < rank <= 512 and rot % 16 == 0
            and (16 + 128) * (rank + rot + 8) * 2 + 4096 <= 200 * 1024)


def latent_splits(n_seqs: int, n_heads: int, kv_len: int, window: int, sms: int) -> int:
    """Into how many blocks a tile's pages are cut in a single-token step: enough blocks for the device, at most one
    per page and ``LATENT_TILED_MAX_SPLITS``."""
    tiles = n_seqs * -(-n_heads // 16)
    span = min(kv_len, window) if window else kv_len
    pages = span // 64 + 1
    return max(1, min(pages, (2 * sms) // max(tiles, 1), LATENT_TILED_MAX_SPLITS))


def attention_latent_tiled(q_carried: torch.Tensor, q_raw: torch.Tensor, q_rot_at: int, rot: int, rot_dims: int,
                           cos: torch.Tensor | None, sin: torch.Tensor | None, cache: PagedRows, tok_pos: torch.Tensor,
                           cu_q: torch.Tensor, slots: torch.Tensor, scale: float, window: int, out: torch.Tensor, n_seqs: int,
                           max_q_len: int, splits: int = 1) -> torch.Tensor:
    """As ``attention_latent_exact``, on the tensor cores (bfloat16).  A sequence's tokens of the step must be at
    consecutive rows in rising positions.  ``splits`` > 1 cuts every tile's pages among that many blocks (steps of few
    tokens); the partial results go through scratch made here."""
    require_device(q_raw.device)
    _check(q_raw, "q_raw", torch.bfloat16, 3)
    n, heads, raw_dim = q_raw.shape
    rank = q_carried.shape[2]
    for name, t in (("q_carried", q_carried), ("out", out)):
        if t.dtype != torch.bfloat16 or tuple(t.shape) != (n, heads, rank) or t.stride(2) != 1:
            raise KernelError(f"{name} must be bfloat16 [{n}, {heads}, {rank}] with a contiguous last axis")
    _check(cache.rows, "cache rows", torch.bfloat16, 3)
    if cache.rows.shape[2] != rank + rot:
        raise KernelError(f"cache rows of {cache.rows.shape[2]} are not {rank} + {rot}")
    part_o = part_ml = None
    if splits > 1:
        part_o = torch.empty((splits, n * heads, rank), dtype=torch.float32, device=q_raw.device)
        part_ml = torch.empty((splits, n * heads, 2), dtype=torch.float32, device=q_raw.device)
    call("gk_attention_latent_tiled", ptr(q_carried), q_carried.stride(0), q_carried.stride(1), ptr(q_raw), raw_dim, int(q_rot_at),
         ptr(cos), ptr(sin), ptr(cache.rows), ptr(out), out.stride(0), out.stride(1), ptr(part_o), ptr(part_ml), ptr(tok_pos),
         ptr(cu_q), ptr(slots), ptr(cache.block_table), n, int(n_seqs), int(max_q_len), heads, rank, rot, rot_dims,
         cache.max_pages, cache.page_size, float(scale), int(window), int(splits), stream_ptr())
    return out


# ------------------------------------------------------------------ the delta rule as a recurrent mixer
def delta_prepare(proj: torch.Tensor, low: torch.Tensor, conv_w: torch.Tensor, conv_state: torch.Tensor | None, a_log: torch.Tensor,
                  dt_bias: torch.Tensor, tok_pos: torch.Tensor, tok_seq: torch.Tensor, cu_q: torch.Tensor, slots: torch.Tensor,
                  n_heads: int, n_kv: int, d: int, dv: int, taps: int, roll_single: bool = False):
    """Everything between the input projections and the recurrence, in 32-bit.  ``proj [T, >= 2 n_kv d + n_heads dv + n_heads]``
    holds q | k | v | b of every token, ``low [T, >= n_heads d + n_heads dv]`` the decay's and the gate's second
    projections; ``conv_w [channels, taps]``; ``conv_state [slots, taps - 1, channels]`` the inputs before the step.
    ``roll_single``: every sequence of the step brings ONE token and the kernel moves the convolution state on itself
    (otherwise ``conv_roll`` follows).
    Returns q, k ``[T, n_kv, d]`` (unit length; q also times ``d ** -0.5``), v ``[T, n_heads, dv]``, the decays
    ``[T, n_heads, d]`` and beta ``[T, n_heads]``."""
    require_device(proj.device)
    _check(proj, "proj", dims=2)
    _check(low, "low", dims=2)
    T = proj.shape[0]
    channels = 2 * n_kv * d + n_heads * dv
    if proj.shape[1] < channels + n_heads or low.shape[1] < n_heads * (d + dv) or low.shape[0] != T:
        raise KernelError(f"projections {tuple(proj.shape)} / {tuple(low.shape)} are too narrow for these sizes")
    _check(conv_w, "conv_w", torch.float32, 2)
    if tuple(conv_w.shape) != (channels, taps):
        raise KernelError(f"conv_w is {tuple(conv_w.shape)}, expected {(channels, taps)}")
    if taps > 1:
        _check(conv_state, "conv_state", torch.float32, 3)
        if tuple(conv_state.shape[1:]) != (taps - 1, channels):
            raise KernelError(f"conv_state is {tuple(conv_state.shape)}, expected [slots, {taps - 1}, {channels}]")
    _check(a_log, "a_log", torch.float32, 1)
    _check(dt_bias, "dt_bias", torch.float32, 1)
    for name, t in (("tok_pos", tok_pos), ("tok_seq", tok_seq), ("cu_q", cu_q), ("slots", slots)):
        _check(t, name, torch.int32, 1)
    dev = proj.device
    q = torch.empty((T, n_kv, d), dtype=torch.float32, device=dev)
    k = torch.empty((T, n_kv, d), dtype=torch.float32, device=dev)
    v = torch.empty((T, n_heads, dv), dtype=torch.float32, device=dev)
    g = torch.empty((T, n_heads, d), dtype=torch.float32, device=dev)
    beta = torch.empty((T, n_heads), dtype=torch.float32, device=dev)
    call("gk_delta_prepare", ptr(proj), dtype_code(proj.dtype), proj.shape[1], ptr(low), dtype_code(low.dtype), low.shape[1],
         ptr(conv_w), ptr(conv_state) if taps > 1 else None, ptr(a_log), ptr(dt_bias), ptr(tok_pos), ptr(tok_seq), ptr(cu_q),
         ptr(slots), ptr(q), ptr(k), ptr(v), ptr(g), ptr(beta), T, n_heads, n_kv, d, dv, taps, int(roll_single and taps > 1), stream_ptr())
    return q, k, v, g, beta


def conv_roll(proj: torch.Tensor, state: torch.Tensor, cu_q: torch.Tensor, slots: torch.Tensor, n_seqs: int, channels: int) -> None:
    """Moves every sequence's convolution state ``[slots, taps - 1, channels]`` on by the step's inputs (the first
    ``channels`` columns of ``proj``)."""
    _check(proj, "proj", dims=2)
    _check(state, "state", torch.float32, 3)
    call("gk_conv_roll", ptr(proj), dtype_code(proj.dtype), proj.shape[1], ptr(state), ptr(cu_q), ptr(slots), n_seqs, channels,
         state.shape[1] + 1, stream_ptr())


# lanes that share a column of the state in the recurrence: 0 = the kernel's own choice by the key size; 8, 16 or 32 for
# measurements (environment variable GTAR_B200_SCAN_LANES)
DELTA_SCAN_LANES = int(__import__("os").environ.get("GTAR_B200_SCAN_LANES", "0"))
DELTA_SCAN_COLS = int(__import__("os").environ.get("GTAR_B200_SCAN_COLS", "0"))  # columns a block, 0 = the kernel's choice


def delta_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, beta: torch.Tensor, state: torch.Tensor,
               cu_q: torch.Tensor, slots: torch.Tensor, n_seqs: int) -> torch.Tensor:
    """The recurrence ``S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q`` over the step's tokens of every
    sequence, from and to ``state [slots, n_heads, d, dv]`` (32-bit).  Returns ``o [T, n_heads, dv]`` (32-bit)."""
    require_device(q.device)
    for name, t in (("q", q), ("k", k), ("v", v), ("g", g)):
        _check(t, name, torch.float32, 3)
    _check(beta, "beta", torch.float32, 2)
    _check(state, "state", torch.float32, 4)
    T, n_kv, d = q.shape
    n_heads, dv = v.shape[1], v.shape[2]
    if tuple(state.shape[1:]) != (n_heads, d, dv) or tuple(g.shape) != (T, n_heads, d) or k.shape != q.shape:
        raise KernelError("delta_scan: the state or the inputs have other sizes than the heads")
    out = torch.empty((T, n_heads, dv), dtype=torch.float32, device=q.device)
    call("gk_delta_scan", ptr(q), ptr(k), ptr(v), ptr(g), ptr(beta), ptr(state), ptr(out), ptr(cu_q), ptr(slots), n_seqs, n_heads,
         n_kv, d, dv, DELTA_SCAN_LANES, DELTA_SCAN_COLS, stream_ptr())
    return out


def head_norm_gate(o: torch.Tensor, weight: torch.Tensor, gate: torch.Tensor, gate_at: int, eps: float, out_dtype: torch.dtype) -> torch.Tensor:
    """``o [T, H, dv]`` (32-bit) divided by each head's root mean square, times ``weight [dv]``, times the sigmoid of
    ``gate[:, gate_at : gate_at + H dv]``.  Returns ``[T, H dv]`` in ``out_dtype``."""
    _check(o, "o", torch.float32, 3)
    _check(weight, "weight", torch.float32, 1)
    _check(gate, "gate", dims=2)
    T, H, dv = o.shape
    if gate.shape[1] < gate_at + H * dv or weight.shape[0] != dv:
        raise KernelError("head_norm_gate: gate or weight do not fit the heads")
    out = torch.empty((T, H * dv), dtype=out_dtype, device=o.device)
    call("gk_head_norm_gate", ptr(o), ptr(weight), gate.data_ptr() + gate_at * gate.element_size(), dtype_code(gate.dtype),
         gate.shape[1], ptr(out), dtype_code(out_dtype), T, H, dv, float(eps), stream_ptr())
    return out


# ------------------------------------------------------------------ routed experts
def route_groups(h: torch.Tensor, w_router: torch.Tensor, correction: torch.Tensor, top: int, n_groups: int, keep: int,
                 scale: float, logits: bool = False) -> tuple[torch.Tensor, torch.Tensor]:
    """Chosen experts ``[T, top]`` (int32) and their weights (float32): sigmoid scores, choice by score plus
    ``correction`` among the experts of the best ``keep`` of ``n_groups`` groups, weight = score times ``scale``.
    ``logits``: the score is the logit plus ``correction`` (a bias), the choice goes by it, and the weights are the
    softmax over the chosen scores alone, times ``scale``."""
    require_device(h.device)
    _check(h, "h", dims=2)
    _check(w_router, "w_router", torch.float32, 2)
    _check(correction, "correction", torch.float32, 1)
    T, width = h.shape
    n_experts = w_router.shape[0]
    if w_router.shape[1] != width or correction.shape[0] != n_experts:
        raise KernelError("route_groups: router sizes do not fit")
    ids = torch.empty((T, top), dtype=torch.int32, device=h.device)
    weights = torch.empty((T, top), dtype=torch.float32, device=h.device)
    z = torch.empty((T, n_experts), dtype=torch.float32, device=h.device)
    call("gk_route_groups", ptr(h), dtype_code(h.dtype), ptr(w_router), ptr(correction), ptr(z), ptr(ids), ptr(weights), T, width, n_experts,
         top, n_groups, keep, float(scale), int(bool(logits)), stream_ptr())
    return ids, weights


def experts_pairwise(h: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor,
                     add: torch.Tensor | None = None) -> torch.Tensor:
    """``add + sum_k weights[t, k] * down_e(silu(gate_e h_t) * up_e h_t)`` with ``e = ids[t, k]``, a (token, expert) pair
    at a time.  ``w_gate_up [E, 2, ff, width]``, ``w_down [E, width, ff]``.  Returns 32-bit ``[T, width]``."""
    require_device(h.device)
    _check(h, "h", dims=2)
    _check(w_gate_up, "w_gate_up", dims=4)
    _check(w_down, "w_down", w_gate_up.dtype, 3)
    _check(ids, "ids", torch.int32, 2)
    _check(weights, "weights", torch.float32, 2)
    T, width = h.shape
    E, _, ff, _ = w_gate_up.shape
    top = ids.shape[1]
    if tuple(w_gate_up.shape) != (E, 2, ff, width) or tuple(w_down.shape) != (E, width, ff):
        raise KernelError("experts: weight shapes do not fit")
    if add is not None:
        _check(add, "add", h.dtype, 2)
    act = torch.empty((T * top, ff), dtype=h.dtype, device=h.device)
    out = torch.empty((T, width), dtype=torch.float32, device=h.device)
    call("gk_experts_up", ptr(h), dtype_code(h.dtype), ptr(w_gate_up), dtype_code(w_gate_up.dtype), ptr(ids), ptr(act), T, width, ff,
         top, stream_ptr())
    call("gk_experts_down", ptr(act), dtype_code(h.dtype), ptr(w_down), dtype_code(w_down.dtype), ptr(ids), ptr(weights), ptr(add),
         ptr(out), T, width, ff, top, stream_ptr())
    return out


# ------------------------------------------------------------------ attention with norms over whole projections
def wide_norm_rope_write(proj: torch.Tensor, n_q: int, n_kv: int, d: int, w_q: torch.Tensor, w_k: torch.Tensor, eps: float,
                         cos: torch.Tensor | None, sin: torch.Tensor | None, rot: int, tok_pos: torch.Tensor, tok_seq: torch.Tensor,
                         slots: torch.Tensor, kv: PagedKV, max_position: int, write_kv: bool = True, v_at: int | None = None,
                         has_k: bool = True) -> torch.Tensor:
    """RMS norm of the whole query row and of the whole key row of every token (``proj [T, >= (n_q + n_kv) d]`` holds
    q | k), rotation of the first ``rot`` entries of every head, the finished keys into the key pages and the keys as
    projected into the value pages.  With ``v_at`` the values are a projection of their own, from that column of the
    row on, as wide as the value pages say.  ``has_k`` False: the row holds queries only and nothing is written (a
    layer that reads another layer's pages).  Returns the finished queries ``[T, n_q, d]``."""
    require_device(proj.device)
    _check(proj, "proj", dims=2)
    _check(w_q, "w_q", torch.float32, 1)
    _check(w_k, "w_k", torch.float32, 1)
    T = proj.shape[0]
    dv = kv.v.shape[3]
    if not has_k:
        write_kv, v_at = False, None
    if proj.shape[1] < (n_q + (n_kv if has_k else 0)) * d or w_q.shape[0] != n_q * d or (has_k and w_k.shape[0] != n_kv * d):
        raise KernelError("wide_norm_rope_write: sizes do not fit")
    if v_at is not None and (v_at < (n_q + n_kv) * d or proj.shape[1] < v_at + n_kv * dv):
        raise KernelError("wide_norm_rope_write: the values do not lie behind the keys inside the row")
    if kv.k.shape[1] != n_kv or kv.k.shape[3] != d or (has_k and v_at is None and kv.v.shape != kv.k.shape) or kv.v.shape[:3] != kv.k.shape[:3]:
        raise KernelError(f"pages {tuple(kv.k.shape)} / {tuple(kv.v.shape)} do not fit n_kv={n_kv}, head_dim={d}")
    positions = 0
    if rot:
        _check(cos, "cos", torch.float32, 2)
        _check(sin, "sin", torch.float32, 2)
        if cos.shape[1] != rot // 2 or sin.shape != cos.shape:
            raise KernelError("rotary tables must be [positions, rot / 2]")
        positions = cos.shape[0]
    q = torch.empty((T, n_q, d), dtype=proj.dtype, device=proj.device)
    call("gk_wide_norm_rope_write", ptr(proj), dtype_code(proj.dtype), proj.shape[1], ptr(w_q), ptr(w_k), ptr(cos) if rot else None,
         ptr(sin) if rot else None, positions, ptr(tok_pos), ptr(tok_seq), ptr(slots), ptr(kv.block_table), ptr(q),
         ptr(kv.k) if write_kv else None, ptr(kv.v) if write_kv else None, dtype_code(kv.k.dtype), T, n_q, n_kv, d, int(rot),
         kv.max_pages, kv.page_size, float(eps), int(max_position), -1 if v_at is None else int(v_at), int(dv), int(bool(has_k)),
         stream_ptr())
    return q


def turn_back_gate(o: torch.Tensor, cos: torch.Tensor | None, sin: torch.Tensor | None, tok_pos: torch.Tensor, max_position: int,
                   gate: torch.Tensor | None = None, gate_at: int = 0) -> torch.Tensor:
    """Every head's read-out ``o [T, n_heads, dv]`` turned by minus its token's position over all ``dv`` entries (entry
    ``m`` paired with ``m + dv/2``; ``cos``, ``sin`` ``[positions, dv/2]``; None: no turn), then times the sigmoid of one
    number per head, ``gate[:, gate_at + h]`` (None: no gate)."""
    require_device(o.device)
    _check(o, "o", dims=3)
    T, n_heads, dv = o.shape
    positions = 0
    if cos is not None:
        _check(cos, "cos", torch.float32, 2)
        _check(sin, "sin", torch.float32, 2)
        _check(tok_pos, "tok_pos", torch.int32, 1)
        if cos.shape[1] != dv // 2 or sin.shape != cos.shape or dv % 2:
            raise KernelError(f"turn_back_gate: tables of {cos.shape[1]} angles for read-outs of {dv}")
        positions = cos.shape[0]
    gate_ptr, ld = None, 0
    if gate is not None:
        _check(gate, "gate", o.dtype, 2)
        if gate.shape[0] != T or gate.shape[1] < gate_at + n_heads:
            raise KernelError("turn_back_gate: the gate is narrower than the heads")
        gate_ptr, ld = gate.data_ptr() + gate_at * gate.element_size(), gate.shape[1]
    out = torch.empty_like(o)
    call("gk_turn_back_gate", ptr(o), ptr(cos), ptr(sin), positions, int(max_position), ptr(tok_pos), gate_ptr, ld, ptr(out),
         dtype_code(o.dtype), T, n_heads, dv, stream_ptr())
    return out


def xielu(x: torch.Tensor, up: float, down: float) -> torch.Tensor:
    """``up z^2 + z/2`` above zero, ``down (exp(z) - 1 - z) + z/2`` at and below, element by element (32-bit arithmetic)."""
    require_device(x.device)
    _check(x, "x")
    out = torch.empty_like(x)
    call("gk_xielu", ptr(x), ptr(out), dtype_code(x.dtype), x.numel(), float(up), float(down), stream_ptr())
    return out


def stream_cast(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """The 32-bit stream in the run's type (the stream itself where that is 32-bit)."""
    _check(x, "x", torch.float32)
    if dtype == torch.float32:
        return x
    require_device(x.device)
    out = torch.empty(x.shape, dtype=dtype, device=x.device)
    call("gk_stream_cast", ptr(x), ptr(out), dtype_code(dtype), x.numel(), stream_ptr())
    return out


def sigmoid_gate(o: torch.Tensor, gate: torch.Tensor, gate_at: int) -> torch.Tensor:
    """``o [T, n] * sigmoid(gate[:, gate_at : gate_at + n])``."""
    _check(o, "o", dims=2)
    _check(gate, "gate", o.dtype, 2)
    T, n = o.shape
    if gate.shape[1] < gate_at + n or gate.shape[0] != T:
        raise KernelError("sigmoid_gate: the gate is narrower than the rows")
    out = torch.empty_like(o)
    call("gk_sigmoid_gate", ptr(o), gate.data_ptr() + gate_at * gate.element_size(), gate.shape[1], ptr(out), dtype_code(o.dtype), T, n,
         stream_ptr())
    return out


def softcap_(x: torch.Tensor, cap: float) -> torch.Tensor:
    """``x <- cap * tanh(x / cap)`` in place (32-bit)."""
    _check(x, "x", torch.float32)
    call("gk_softcap", ptr(x), x.numel(), float(cap), stream_ptr())
    return x


def experts_sort(ids: torch.Tensor, n_experts: int) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """The (token, chosen expert) pairs ``ids [T, top]`` put in the order of their experts: ``ends [E]`` (one past each
    expert's last place), ``place_of [T, top]`` and ``pair_at [T * top]``, all int32."""
    _check(ids, "ids", torch.int32, 2)
    n = ids.numel()
    ends = torch.empty((n_experts,), dtype=torch.int32, device=ids.device)
    place_of = torch.empty_like(ids)
    pair_at = torch.empty((n,), dtype=torch.int32, device=ids.device)
    call("gk_experts_sort", ptr(ids), n, n_experts, ptr(ends), ptr(place_of), ptr(pair_at), stream_ptr())
    return ends, place_of, pair_at


def gather_rows(x: torch.Tensor, pair_at: torch.Tensor, top: int) -> torch.Tensor:
    """``out[place] = x[pair_at[place] // top]``."""
    _check(x, "x", dims=2)
    _check(pair_at, "pair_at", torch.int32, 1)
    out = torch.empty((pair_at.shape[0], x.shape[1]), dtype=x.dtype, device=x.device)
    call("gk_gather_rows", ptr(x), dtype_code(x.dtype), ptr(pair_at), ptr(out), pair_at.shape[0], x.shape[1], top, stream_ptr())
    return out


def experts_combine(y: torch.Tensor, place_of: torch.Tensor, weights: torch.Tensor, add: torch.Tensor | None) -> torch.Tensor:
    """``add[t] + sum_k weights[t, k] * y[place_of[t, k]]`` in the order of ``k``, 32-bit ``[T, width]``."""
    _check(y, "y", dims=2)
    _check(place_of, "place_of", torch.int32, 2)
    _check(weights, "weights", torch.float32, 2)
    T, top = place_of.shape
    if add is not None:
        _check(add, "add", y.dtype, 2)
    out = torch.empty((T, y.shape[1]), dtype=torch.float32, device=y.device)
    call("gk_experts_combine", ptr(y), dtype_code(y.dtype), ptr(place_of), ptr(weights), ptr(add), ptr(out), T, y.shape[1], top,
         stream_ptr())
    return out


# ------------------------------------------------------------------ layer norm, scored attention, linear attention with a fixed decay
def add_layernorm(h: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
                  rows: torch.Tensor | None = None, delta_scale: float = 1.0) -> torch.Tensor:
    """``h += delta_scale * delta`` (in place, skipped when ``delta`` is None), then the layer norm of ``h`` with a weight
    and no bias: ``(h - mean) / sqrt(mean((h - mean)^2) + eps) * weight``.  With ``rows`` (int32 indices) only those rows
    are normed and ``h`` is not written."""
    require_device(h.device)
    _check(h, "h", torch.float32, 2)
    _check(weight, "weight", dims=1)
    hidden = h.shape[1]
    if weight.shape[0] != hidden:
        raise KernelError(f"norm weight has {weight.shape[0]} entries for rows of {hidden}")
    delta_code = 0
    if delta is not None:
        _check(delta, "delta", dims=2)
        if delta.shape != h.shape:
            raise KernelError(f"delta {tuple(delta.shape)} does not match h {tuple(h.shape)}")
        delta_code = dtype_code(delta.dtype)
    n_out = h.shape[0]
    if rows is not None:
        _check(rows, "rows", torch.int32, 1)
        n_out = rows.shape[0]
    out = torch.empty((n_out, hidden), dtype=out_dtype, device=h.device)
    call("gk_add_layernorm", ptr(h), ptr(delta), delta_code, float(delta_scale), ptr(weight), dtype_code(weight.dtype), ptr(out),
         dtype_code(out_dtype), ptr(rows), n_out, hidden, float(eps), stream_ptr())
    return out


def add_layernorm_conv_single_fits(hidden: int, taps: int) -> bool:
    """Whether :func:`add_layernorm_conv_single` takes rows of this width: the row, its ``taps - 1`` earlier inputs and the
    weights of the norm and of the taps within 200 KB of shared memory (the kernel's own rule)."""
    return hidden > 0 and taps >= 1 and hidden * (2 * taps + 1) * 4 <= 200 * 1024


def add_layernorm_conv_single(h: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, eps: float, conv_weight: torch.Tensor,
                              state: torch.Tensor | None, tok_pos: torch.Tensor, tok_seq: torch.Tensor, slots: torch.Tensor,
                              out_dtype: torch.dtype, delta_scale: float = 1.0, update_state: bool = True) -> torch.Tensor:
    """:func:`add_layernorm` and :func:`causal_conv` behind it in one kernel, for steps in which every sequence brings one
    token (row ``t`` belongs to sequence ``tok_seq[t]``): ``h += delta_scale * delta``, ``y = layernorm(h)``, returns
    ``y + conv(y)`` with the earlier inputs from ``state [n_slots, taps - 1, width]``, which is moved on by ``y`` when
    ``update_state``.  The same numbers as the two kernels one after the other."""
    require_device(h.device)
    _check(h, "h", torch.float32, 2)
    _check(weight, "weight", torch.float32, 1)
    _check(conv_weight, "conv_weight", torch.float32, 2)
    n, hidden = h.shape
    taps = conv_weight.shape[0]
    if weight.shape[0] != hidden or conv_weight.shape[1] != hidden:
        raise KernelError(f"norm weight of {weight.shape[0]} and convolution weights {tuple(conv_weight.shape)} for rows of {hidden}")
    delta_code = 0
    if delta is not None:
        _check(delta, "delta", dims=2)
        if delta.shape != h.shape:
            raise KernelError(f"delta {tuple(delta.shape)} does not match h {tuple(h.shape)}")
        delta_code = dtype_code(delta.dtype)
    if taps > 1:
        _check(state, "state", torch.float32, 3)
        if tuple(state.shape[1:]) != (taps - 1, hidden):
            raise KernelError(f"state {tuple(state.shape)} does not hold {taps - 1} inputs of width {hidden}")
    for name, t in (("tok_pos", tok_pos), ("tok_seq", tok_seq), ("slots", slots)):
        _check(t, name, torch.int32, 1)
    if tok_pos.shape[0] < n or tok_seq.shape[0] < n:
        raise KernelError("add_layernorm_conv_single: fewer positions than rows")
    out = torch.empty((n, hidden), dtype=out_dtype, device=h.device)
    call("gk_add_layernorm_conv_single", ptr(h), ptr(delta), delta_code, float(delta_scale), ptr(weight), ptr(conv_weight),
         ptr(state) if taps > 1 else None, ptr(tok_pos), ptr(tok_seq), ptr(slots), ptr(out), dtype_code(out_dtype), n, hidden, taps,
         float(eps), int(bool(update_state)), stream_ptr())
    return out


def scaled_sum(a: torch.Tensor, scale_a: float, b: torch.Tensor, scale_b: float) -> torch.Tensor:
    """``scale_a * a + scale_b * b`` in 32-bit, element by element."""
    require_device(a.device)
    _check(a, "a")
    _check(b, "b", a.dtype)
    if a.shape != b.shape:
        raise KernelError(f"scaled_sum: {tuple(a.shape)} and {tuple(b.shape)}")
    out = torch.empty(a.shape, dtype=torch.float32, device=a.device)
    call("gk_scaled_sum", ptr(a), float(scale_a), ptr(b), float(scale_b), dtype_code(a.dtype), ptr(out), a.numel(), stream_ptr())
    return out


def scale_(x: torch.Tensor, factor: float) -> torch.Tensor:
    """``x <- factor * x`` in place (32-bit)."""
    _check(x, "x", torch.float32)
    call("gk_scale", ptr(x), x.numel(), float(factor), stream_ptr())
    return x


def relu_squared(x: torch.Tensor) -> torch.Tensor:
    """``max(x, 0)^2``, element by element."""
    require_device(x.device)
    _check(x, "x")
    out = torch.empty_like(x)
    call("gk_relu_squared", ptr(x), ptr(out), dtype_code(x.dtype), x.numel(), stream_ptr())
    return out


PREPARE_SILU_QK, PREPARE_SILU_V, PREPARE_UNIT_RMS, PREPARE_TURN_V = 1, 2, 4, 8


def heads_prepare(proj: torch.Tensor, q_at: int, k_at: int, v_at: int, n_q: int, n_k: int, d: int, dv: int, tok_pos: torch.Tensor,
                  tok_seq: torch.Tensor, slots: torch.Tensor, *, silu_qk: bool = False, silu_v: bool = False, rot: int = 0,
                  cos: torch.Tensor | None = None, sin: torch.Tensor | None = None, unit_eps: float | None = None,
                  k_scale: float = 1.0, kv: PagedKV | None = None, write_kv: bool = True, max_position: int | None = None,
                  v_cos: torch.Tensor | None = None, v_sin: torch.Tensor | None = None):
    """What stands between a packed projection and a mixer's core.  ``proj [T, >= ...]`` holds ``n_q`` query heads of ``d``
    from column ``q_at``, ``n_k`` key heads of ``d`` from ``k_at`` and ``n_k`` value heads of ``dv`` from ``v_at``.  In this
    order: SiLU (``silu_qk`` on q and k, ``silu_v`` on v); rotation of the first ``rot`` entries of every q and k head by
    the token's position (entry ``i`` with ``i + rot/2``; ``cos``, ``sin`` ``[positions, rot/2]``); with ``unit_eps`` every q
    and k head divided by its root mean square; ``k_scale`` on k; with ``v_cos``, ``v_sin`` ``[positions, dv/2]`` every
    value head turned by its token's position over all of its entries (entry ``m`` with ``m + dv/2``).  With ``kv`` the keys and values are written into the
    cache's pages and q ``[T, n_q, d]`` comes back in the projection's type; without, q, k ``[T, n, d]`` and v ``[T, n_k,
    dv]`` come back as 32-bit arrays."""
    require_device(proj.device)
    _check(proj, "proj", dims=2)
    T = proj.shape[0]
    reads_kv = kv is None or write_kv  # a step that writes no pages reads the queries alone (a layer that reads another's pages)
    if max(q_at + n_q * d, (k_at + n_k * d) if reads_kv else 0, (v_at + n_k * dv) if reads_kv else 0) > proj.shape[1]:
        raise KernelError(f"heads_prepare: a projection of {proj.shape[1]} columns is too narrow for these heads")
    for name, t in (("tok_pos", tok_pos), ("tok_seq", tok_seq), ("slots", slots)):
        _check(t, name, torch.int32, 1)
    if rot:
        _check(cos, "cos", torch.float32, 2)
        _check(sin, "sin", torch.float32, 2)
        if cos.shape[1] != rot // 2 or sin.shape != cos.shape:
            raise KernelError(f"heads_prepare: tables of {cos.shape[1]} angles for {rot} rotated entries")
        if max_position is not None and cos.shape[0] <= max_position:
            raise KernelError(f"heads_prepare: tables hold {cos.shape[0]} positions, the step reaches {max_position}")
    flags = (PREPARE_SILU_QK if silu_qk else 0) | (PREPARE_SILU_V if silu_v else 0) | (PREPARE_UNIT_RMS if unit_eps is not None else 0)
    if v_cos is not None:
        _check(v_cos, "v_cos", torch.float32, 2)
        _check(v_sin, "v_sin", torch.float32, 2)
        if dv % 2 or v_cos.shape[1] != dv // 2 or v_sin.shape != v_cos.shape:
            raise KernelError(f"heads_prepare: tables of {v_cos.shape[1]} angles for values of {dv}")
        if max_position is not None and v_cos.shape[0] <= max_position:
            raise KernelError(f"heads_prepare: value tables hold {v_cos.shape[0]} positions, the step reaches {max_position}")
        flags |= PREPARE_TURN_V
    dev = proj.device
    if kv is not None:
        _check(kv.k, "k pages", proj.dtype, 4)
        _check(kv.v, "v pages", proj.dtype, 4)
        if tuple(kv.k.shape[1:]) != (n_k, kv.page_size, d) or tuple(kv.v.shape[1:]) != (n_k, kv.page_size, dv):
            raise KernelError(f"heads_prepare: pages {tuple(kv.k.shape)} / {tuple(kv.v.shape)} do not hold {n_k} heads of {d} / {dv}")
        q = torch.empty((T, n_q, d), dtype=proj.dtype, device=dev)
        call("gk_heads_prepare", ptr(proj), dtype_code(proj.dtype), proj.shape[1], q_at, k_at, v_at, n_q, n_k, d, dv, flags, rot,
             ptr(cos) if rot else None, ptr(sin) if rot else None, ptr(v_cos), ptr(v_sin), float(unit_eps or 0.0), float(k_scale),
             ptr(tok_pos), ptr(tok_seq), ptr(slots), ptr(q), dtype_code(q.dtype), None, None, ptr(kv.k), ptr(kv.v), ptr(kv.block_table), kv.max_pages,
             kv.page_size, int(write_kv), T, stream_ptr())
        return q
    q = torch.empty((T, n_q, d), dtype=torch.float32, device=dev)
    k = torch.empty((T, n_k, d), dtype=torch.float32, device=dev)
    v = torch.empty((T, n_k, dv), dtype=torch.float32, device=dev)
    call("gk_heads_prepare", ptr(proj), dtype_code(proj.dtype), proj.shape[1], q_at, k_at, v_at, n_q, n_k, d, dv, flags, rot,
         ptr(cos) if rot else None, ptr(sin) if rot else None, ptr(v_cos), ptr(v_sin), float(unit_eps or 0.0), float(k_scale),
         ptr(tok_pos), ptr(tok_seq), ptr(slots), ptr(q), dtype_code(q.dtype), ptr(k), ptr(v), None, None, None, 0, 0, 0, T, stream_ptr())
    return q, k, v


def decay_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor, state: torch.Tensor, cu_q: torch.Tensor,
               slots: torch.Tensor, n_seqs: int) -> torch.Tensor:
    """The recurrence ``S <- decay_h S + k v^T; o = S^T q`` over the step's tokens of every sequence, from and to
    ``state [slots, heads, d, dv]`` (32-bit).  q, k ``[T, heads, d]``, v ``[T, heads, dv]``, ``decay [heads]``, all 32-bit.
    Returns ``o [T, heads, dv]`` (32-bit)."""
    require_device(q.device)
    for name, t in (("q", q), ("k", k), ("v", v)):
        _check(t, name, torch.float32, 3)
    _check(decay, "decay", torch.float32, 1)
    _check(state, "state", torch.float32, 4)
    T, n_heads, d = q.shape
    dv = v.shape[2]
    if k.shape != q.shape or tuple(v.shape[:2]) != (T, n_heads) or tuple(state.shape[1:]) != (n_heads, d, dv) or decay.shape[0] != n_heads:
        raise KernelError("decay_scan: the state, the decays or the inputs have other sizes than the heads")
    out = torch.empty((T, n_heads, dv), dtype=torch.float32, device=q.device)
    call("gk_decay_scan", ptr(q), ptr(k), ptr(v), ptr(decay), ptr(state), ptr(out), ptr(cu_q), ptr(slots), int(n_seqs), n_heads, d, dv,
         stream_ptr())
    return out


DECAY_CHUNK = 64                 # tokens a chunk of decay_scan_chunked
DECAY_WORKSPACE_FLOATS = 1 << 26  # at most this many 32-bit numbers of chunk states in flight (256 MB)


def decay_scan_chunked_fits(d: int, dv: int) -> bool:
    """Whether :func:`decay_scan_chunked` takes heads of these sizes: rows of 16-byte vectors, and the transposed q and k
    tiles, a tile of values and a tile of weights within 200 KB of shared memory (the kernel's own rule)."""
    return d > 0 and dv > 0 and d % 4 == 0 and dv % 4 == 0 and (2 * d * 68 + 64 * 64 + 64 * 68 + 68) * 4 <= 200 * 1024


def decay_scan_chunked(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor, state: torch.Tensor, cu_q: torch.Tensor,
                       slots: torch.Tensor, n_seqs: int, max_q_len: int) -> torch.Tensor:
    """:func:`decay_scan` for steps of many tokens: the tokens of every sequence are cut into chunks of 64 whose inner
    work is matrix products that run side by side, with one short pass over the chunks in sequence between them.  32-bit
    throughout; the sums have another order than token by token, so the two agree within rounding.  ``max_q_len`` bounds
    the sequences' token counts in this step."""
    require_device(q.device)
    for name, t in (("q", q), ("k", k), ("v", v)):
        _check(t, name, torch.float32, 3)
    _check(decay, "decay", torch.float32, 1)
    _check(state, "state", torch.float32, 4)
    T, n_heads, d = q.shape
    dv = v.shape[2]
    if k.shape != q.shape or tuple(v.shape[:2]) != (T, n_heads) or tuple(state.shape[1:]) != (n_heads, d, dv) or decay.shape[0] != n_heads:
        raise KernelError("decay_scan_chunked: the state, the decays or the inputs have other sizes than the heads")
    out = torch.empty((T, n_heads, dv), dtype=torch.float32, device=q.device)
    chunks = max(1, -(-int(max_q_len) // DECAY_CHUNK))
    wave = max(1, min(chunks, DECAY_WORKSPACE_FLOATS // max(1, n_seqs * n_heads * d * dv)))
    ws = torch.empty((max(1, n_seqs) * wave * n_heads * d * dv,), dtype=torch.float32, device=q.device)
    call("gk_decay_scan_chunked", ptr(q), ptr(k), ptr(v), ptr(decay), ptr(state), ptr(out), ptr(ws), ptr(cu_q), ptr(slots), int(n_seqs),
         n_heads, d, dv, int(max_q_len), wave, stream_ptr())
    return out


def group_norm_gate(x: torch.Tensor, group: int, weight: torch.Tensor | None, gate: torch.Tensor, gate_at: int, eps: float,
                    out_dtype: torch.dtype, gate_kind: str = "sigmoid") -> torch.Tensor:
    """Rows of ``x [T, width]`` (32-bit) cut into groups of ``group`` entries; every group divided by its root mean square
    (eps inside the root), multiplied by ``weight [group]`` (if given) and by sigmoid or SiLU of
    ``gate[:, gate_at : gate_at + width]``.  Returns ``[T, width]`` in ``out_dtype``."""
    require_device(x.device)
    _check(x, "x", torch.float32, 2)
    _check(gate, "gate", dims=2)
    T, width = x.shape
    if width % group or gate.shape[1] < gate_at + width or gate.shape[0] != T:
        raise KernelError("group_norm_gate: the groups or the gate do not fit the rows")
    if weight is not None:
        _check(weight, "weight", torch.float32, 1)
        if weight.shape[0] != group:
            raise KernelError(f"group_norm_gate: a weight of {weight.shape[0]} for groups of {group}")
    kinds = {"sigmoid": 0, "silu": 1}
    out = torch.empty((T, width), dtype=out_dtype, device=x.device)
    call("gk_group_norm_gate", ptr(x), ptr(weight), gate.data_ptr() + gate_at * gate.element_size(), dtype_code(gate.dtype),
         gate.shape[1], ptr(out), dtype_code(out_dtype), T, width // group, group, float(eps), kinds[gate_kind], stream_ptr())
    return out


def attention_scored_exact(q: torch.Tensor, kv: PagedKV, tok_pos: torch.Tensor, tok_seq: torch.Tensor, slots: torch.Tensor,
                           scale: float, window: int = 0, keep_first: int = 0, r1: torch.Tensor | None = None,
                           r2: torch.Tensor | None = None, head_bias: torch.Tensor | None = None,
                           weights: str = "softmax", chunk: int = 0, temp: torch.Tensor | None = None,
                           dist_bias: torch.Tensor | None = None, sink: torch.Tensor | None = None) -> torch.Tensor:
    """Causal grouped-query attention of ``q [T, n_q, d]`` over pages of keys ``[.., d]`` and values ``[.., dv]`` (exact
    kernel): a key at ``j`` is seen from ``i`` if ``i - j < window`` or ``j < keep_first``; the score is ``q . k * scale -
    r1_h ln(1 + r2_h (i - j))``; the weights are the softmax over the seen keys, or ``sigmoid(score + head_bias_h)``
    without a sum that divides.  ``chunk``: only keys of the token's own chunk of that many positions are seen; ``temp``
    ``[n_q]`` multiplies the product per head; ``dist_bias [n_dist, n_q]`` is added by distance (the last row for
    every distance beyond); ``sink [n_q]`` joins the softmax's denominator as ``exp(sink_h)``.  Returns ``[T, n_q, dv]``."""
    require_device(q.device)
    _check(q, "q", dims=3)
    n, n_q, d = q.shape
    _check_score_rules(n_q, temp, dist_bias, sink)
    _check(kv.k, "k pages", q.dtype, 4)
    _check(kv.v, "v pages", q.dtype, 4)
    n_kv, dv = kv.k.shape[1], kv.v.shape[3]
    if kv.k.shape[3] != d:
        raise KernelError(f"pages have keys of {kv.k.shape[3]}, queries of {d}")
    for name, t in (("tok_pos", tok_pos), ("tok_seq", tok_seq), ("slots", slots)):
        _check(t, name, torch.int32, 1)
    for name, t in (("r1", r1), ("r2", r2), ("head_bias", head_bias)):
        if t is not None:
            _check(t, name, torch.float32, 1)
            if t.shape[0] != n_q:
                raise KernelError(f"{name} has {t.shape[0]} entries for {n_q} query heads")
    out = torch.empty((n, n_q, dv), dtype=q.dtype, device=q.device)
    call("gk_attention_scored_exact", ptr(q), ptr(kv.k), ptr(kv.v), ptr(out), dtype_code(q.dtype), ptr(tok_pos), ptr(tok_seq),
         ptr(slots), ptr(kv.block_table), n, n_q, n_kv, d, dv, kv.max_pages, kv.page_size, float(scale), int(window),
         int(keep_first), ptr(r1), ptr(r2), ptr(head_bias), {"softmax": 0, "sigmoid": 1}[weights], int(chunk), ptr(temp),
         ptr(dist_bias), 0 if dist_bias is None else dist_bias.shape[0], ptr(sink), stream_ptr())
    return out


def _check_score_rules(n_q: int, temp, dist_bias, sink) -> None:
    for name, t in (("temp", temp), ("sink", sink)):
        if t is not None:
            _check(t, name, torch.float32, 1)
            if t.shape[0] != n_q:
                raise KernelError(f"{name} has {t.shape[0]} entries for {n_q} query heads")
    if dist_bias is not None:
        _check(dist_bias, "dist_bias", torch.float32, 2)
        if dist_bias.shape[1] != n_q or dist_bias.shape[0] < 1:
            raise KernelError(f"a distance table {tuple(dist_bias.shape)} for {n_q} query heads")


def scored_attention_parts(n_seqs: int, n_q: int, n_kv: int, max_q_len: int, visible_pages: int, n_sms: int) -> int:
    """Into how many parts :func:`attention_scored` cuts the walk over a block's pages: one where the rows alone fill the
    GPU twice over, else as many as bring the blocks to two a multiprocessor, and never more than the pages that a row can
    see.  Steps of few tokens have blocks of equal length: the count is rounded down, for heads of 128 fit two blocks a
    multiprocessor and a few blocks over make a second wave (14 us against 19).  A prompt's blocks differ in length, the
    short ones fill in behind the long ones, and rounding up is the faster (78 us against 102)."""
    row_blocks = -(-max_q_len * (n_q // n_kv) // 64)
    blocks = max(1, n_seqs * n_kv * row_blocks)
    if blocks >= 2 * n_sms:
        return 1
    wanted = 2 * n_sms // blocks if row_blocks == 1 else -(-2 * n_sms // blocks)
    return max(1, min(wanted, visible_pages, 32))


def attention_scored(q: torch.Tensor, kv: PagedKV, cu_q: torch.Tensor, kv_len: torch.Tensor, slots: torch.Tensor, max_q_len: int,
                     scale: float, window: int = 0, keep_first: int = 0, r1: torch.Tensor | None = None,
                     r2: torch.Tensor | None = None, head_bias: torch.Tensor | None = None, weights: str = "softmax",
                     n_parts: int = 1, chunk: int = 0, temp: torch.Tensor | None = None, dist_bias: torch.Tensor | None = None,
                     sink: torch.Tensor | None = None) -> torch.Tensor:
    """:func:`attention_scored_exact` on the tensor cores: bfloat16, keys and values of 64 or 128 entries both, pages of 64
    keys.  The new tokens ``q [n_tokens, n_q, d]`` are packed by sequence (``cu_q``), ``kv_len`` counts each sequence's
    cached tokens including them.  ``n_parts`` > 1 cuts every block's keys into that many blocks whose sums a second
    kernel adds (steps of few tokens)."""
    require_device(q.device)
    _check(q, "q", torch.bfloat16, 3)
    n, n_q, d = q.shape
    _check(kv.k, "k pages", torch.bfloat16, 4)
    _check(kv.v, "v pages", torch.bfloat16, 4)
    if kv.k.shape[3] != d or kv.v.shape[3] != d:
        raise KernelError(f"attention_scored: pages of {kv.k.shape[3]} / {kv.v.shape[3]} for queries of {d} (use the exact kernel)")
    for name, t in (("cu_q", cu_q), ("kv_len", kv_len), ("slots", slots)):
        _check(t, name, torch.int32, 1)
    n_seqs = kv_len.shape[0]
    if cu_q.shape[0] != n_seqs + 1 or slots.shape[0] != n_seqs:
        raise KernelError("cu_q needs n_seqs + 1 entries, slots and kv_len n_seqs")
    for name, t in (("r1", r1), ("r2", r2), ("head_bias", head_bias)):
        if t is not None:
            _check(t, name, torch.float32, 1)
            if t.shape[0] != n_q:
                raise KernelError(f"{name} has {t.shape[0]} entries for {n_q} query heads")
    _check_score_rules(n_q, temp, dist_bias, sink)
    sigmoid = {"softmax": 0, "sigmoid": 1}[weights]
    out = torch.empty_like(q)
    part_o = part_ml = None
    if n_parts > 1:
        part_o = torch.empty((n_parts, n, n_q, d), dtype=torch.float32, device=q.device)
        if not sigmoid:
            part_ml = torch.empty((n_parts, n, n_q, 2), dtype=torch.float32, device=q.device)
    call("gk_attention_scored_bf16", ptr(q), ptr(kv.k), ptr(kv.v), ptr(out), ptr(part_o), ptr(part_ml), ptr(cu_q), ptr(kv_len),
         ptr(slots), ptr(kv.block_table), n_seqs, int(max_q_len), n, n_q, kv.k.shape[1], d, kv.max_pages, kv.page_size, float(scale),
         int(window), int(keep_first), ptr(r1), ptr(r2), ptr(head_bias), sigmoid, int(n_parts), int(chunk), ptr(temp),
         ptr(dist_bias), 0 if dist_bias is None else dist_bias.shape[0], ptr(sink), stream_ptr())
    return out
