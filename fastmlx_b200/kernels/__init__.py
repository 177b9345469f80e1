"""The kernel namespace that parts call: tensors in, tensors out, CUDA underneath.

Every function launches hand-written sm_100a kernels from `csrc/` on the current stream.
Matrix products of the bfloat16 path go to cuBLAS through `torch.mm`, where tamnd/fastmlx
calls its library's matmul (compute/models/qwen3_forward.go:111-115 -> mlxgo/binding_cgo.go:
324-328); the 32-bit path uses its own fixed-order kernel and never a reduced-precision
matrix mode.  Nothing here runs on the CPU.
"""
from __future__ import annotations

import torch

from . import lib as _lib
from .lib import KernelError, call, load, loaded_libraries


def launch_count() -> int:
    """Calls into the package's CUDA libraries so far (a graph replay is counted by its owner)."""
    return _lib.launches

F32, BF16 = 0, 1
BAD_TOKEN, BAD_SLOT, BAD_PAGE, BAD_ROW = 1, 2, 3, 4


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16, got {t.dtype}")


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise KernelError("kernels run on CUDA tensors only; there is no CPU path")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream():
    """The current stream's handle.  A step makes a hundred and more launches, and building a
    torch.cuda.Stream object for each cost about 5 us of host time per launch."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _ptr(t):
    return None if t is None else t.data_ptr()


# ----------------------------------------------------------------------------- rows
def gather_rows(table: torch.Tensor, ids: torch.Tensor, status, code: int = BAD_ROW) -> torch.Tensor:
    _need_cuda(table, ids)
    assert ids.dtype == torch.int32 and table.dim() == 2 and table.is_contiguous()
    n, d = ids.numel(), table.shape[1]
    out = torch.empty((n, d), dtype=table.dtype, device=table.device)
    call("common", "fmx_gather_rows", table.data_ptr(), ids.data_ptr(), out.data_ptr(), n, d, table.shape[0],
         _dt(table), _ptr(status), code, _stream())
    return out


def embedding(ids: torch.Tensor, table: torch.Tensor, status, out_dtype=None) -> torch.Tensor:
    """Rows of the table; a table stored in 32-bit can feed bfloat16 activations (rounded here)."""
    if out_dtype == torch.bfloat16 and table.dtype == torch.float32:
        _need_cuda(table, ids)
        assert ids.dtype == torch.int32 and table.dim() == 2 and table.is_contiguous()
        n, d = ids.numel(), table.shape[1]
        out = torch.empty((n, d), dtype=torch.bfloat16, device=table.device)
        call("common", "fmx_gather_rows_f32_to_bf16", table.data_ptr(), ids.data_ptr(), out.data_ptr(), n, d,
             table.shape[0], _ptr(status), BAD_TOKEN, _stream())
        return out
    return gather_rows(table, ids, status, BAD_TOKEN)


def add_rmsnorm(x, residual, weight: torch.Tensor, eps: float, stream_dtype=None, out_dtype=None):
    """-> (norm(residual + x) * weight, residual + x); the sum replaces `residual` in place.
    Without a residual, x is the stream's first value: it is returned as the stream, as it is or,
    when `stream_dtype` is float32 beside bfloat16 activations, as a 32-bit copy that the later
    sums then never round.  x may be None when there is a residual (the stream itself is
    normalised; `out_dtype` then names the activations' type)."""
    _need_cuda(x, residual, weight)
    assert weight.dtype == torch.float32
    ref = x if x is not None else residual
    assert ref is not None and ref.dim() == 2 and ref.is_contiguous()
    act = x.dtype if x is not None else (out_dtype or residual.dtype)
    init = 0
    if residual is None and stream_dtype is not None and stream_dtype != act:
        residual = torch.empty(ref.shape, dtype=stream_dtype, device=ref.device)
        init = 1
    assert residual is None or (residual.shape == ref.shape and residual.is_contiguous())
    out = torch.empty(ref.shape, dtype=act, device=ref.device)
    call("common", "fmx_add_rmsnorm", _ptr(x), _ptr(residual), weight.data_ptr(), out.data_ptr(), ref.shape[0], ref.shape[1],
         float(eps), _dt(out), _dt(residual) if residual is not None else _dt(out), init, _stream())
    return out, (residual if residual is not None else x)


def silu_mul(gate_up: torch.Tensor, block: int | None = None) -> torch.Tensor:
    """silu(gate) * up over rows of 2 I values laid out in blocks of `block` gates followed by
    their `block` ups (block = I, the default: all gates, then all ups)."""
    _need_cuda(gate_up)
    assert gate_up.dim() == 2 and gate_up.is_contiguous() and gate_up.shape[1] % 2 == 0
    rows, inter = gate_up.shape[0], gate_up.shape[1] // 2
    out = torch.empty((rows, inter), dtype=gate_up.dtype, device=gate_up.device)
    call("common", "fmx_silu_mul", gate_up.data_ptr(), out.data_ptr(), rows, inter, int(block or inter), _dt(gate_up),
         _stream())
    return out


# ----------------------------------------------------------------------------- matrix products
def gemm_simple(x, w, bias, out_dtype) -> torch.Tensor:
    M, K = x.shape
    N = w.shape[0]
    out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    call("common", "fmx_gemm_simple", x.data_ptr(), w.data_ptr(), _ptr(bias), out.data_ptr(), M, N, K,
         x.stride(0), w.stride(0), out.stride(0), _dt(x), _dt(w), _dt(out), _stream())
    return out


_tc_status: dict = {}
_props: dict = {}


def _dev_index(device) -> int:
    device = torch.device(device)
    return device.index if device.index is not None else torch.cuda.current_device()


def num_sms(device=None) -> int:
    """Multiprocessors of the device (148 on a B200; fewer under a partition), read once per
    device.  Where no device is visible (host-side arithmetic in tests) a B200's count."""
    if not torch.cuda.is_available():
        return 148
    i = _dev_index(device if device is not None else "cuda")
    n = _props.get(i)
    if n is None:
        n = _props[i] = torch.cuda.get_device_properties(i).multi_processor_count
    return n


def set_status_word(device, status: torch.Tensor) -> None:
    """The word in which kernels called through `linear` report trouble (a bounded wait that
    ran out): the engine registers its own, so that one read after a step covers them."""
    _tc_status[_dev_index(device)] = status


def _status_word(device):
    st = _tc_status.get(_dev_index(device))
    if st is None:
        st = _tc_status[_dev_index(device)] = torch.zeros(4, dtype=torch.int32, device=device)
    return st


# Which kernel multiplies, by the rows M of x (one path per class, no switch):
#   M <= 16                    whole-K weight-streaming kernel (`gemv`), except the vocabulary-sized head
#   M >= 128, full rounds      tcgen05 kernel (`gemm_tcgen05`)
#   everything else in bf16    the library (cuBLAS through torch.mm), as tamnd/fastmlx calls its library's matmul
#   32-bit or mixed types      fixed-order FMA kernel (`gemm_simple`)
GEMV_MAX_ROWS = 16
LIBRARY_MIN_FEATURES = 65536     # from this many output features on (the vocabulary) the library's product streams best
TC_MIN_ROWS = 128
GATE_UP_BLOCK = 128              # gate/up rows of a fused weight alternate in blocks of this many
EPI_PLAIN, EPI_SILU_MUL, EPI_RESIDUAL = 0, 1, 2


def _bf16_operands(x, w) -> bool:
    """bfloat16 operands laid out as the tensor-core kernels read them (16-byte rows)."""
    return (x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[0] > 0
            and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and x.stride(1) == 1 and w.stride(1) == 1
            and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def can_gemv(x, w) -> bool:
    """May this product run on the whole-K kernel of decode steps?"""
    return _bf16_operands(x, w) and x.shape[0] <= GEMV_MAX_ROWS


def gemv(x, w, bias=None, out_dtype=torch.bfloat16, residual=None, block: int = 0, out=None, wide=None, warps=None):
    """x[M <= 16, K] @ w[N, K]^T, one block per `wide` (8, 16, 32) output features and the whole of K:
    nothing is summed across blocks.  residual [M, n_out] is added to the product (out may be
    the residual itself).  block > 0: w's rows alternate in blocks of `block` gate rows and
    their up rows, and the result is silu(gate) * up, [M, N/2]."""
    M, K = x.shape
    N = w.shape[0]
    n_out = N // 2 if block else N
    if out is None:
        out = torch.empty((M, n_out), dtype=out_dtype, device=x.device)
    # wide / warps left open: the library plans them (`fmx_gemv_plan_width`, `fmx_gemv_plan_warps`)
    call("bf16", "fmx_gemv", x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), _ptr(bias), _ptr(residual),
         residual.stride(0) if residual is not None else 0, out.data_ptr(), out.stride(0), M, N, K, _dt(out), int(block),
         int(wide or 0), int(warps or 0), _stream())
    return out


_greedy_ws: dict = {}


def greedy_workspace(device):
    """The greedy head's 16 best-so-far words and its ticket, one pair per device, made once
    (captured graphs hold their addresses); zero between launches."""
    ws = _greedy_ws.get(_dev_index(device))
    if ws is None:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("the greedy head's workspace must exist before a CUDA graph is captured")
        ws = _greedy_ws[_dev_index(device)] = (torch.zeros(16, dtype=torch.int64, device=device),
                                               torch.zeros(1, dtype=torch.int32, device=device))
    return ws


GREEDY_HEAD_MAX_ROWS = 8      # beyond, the library's product followed by the split argmax is the faster head


def can_greedy_head(x, w) -> bool:
    """Should the output head choose greedily in the same pass (no logits written)?  Up to 8
    rows (128,256 x 2,048: 84 us against 86 for the library's product and the argmax kernel; at
    16 rows 101 against 88)."""
    return _bf16_operands(x, w) and x.shape[0] <= GREEDY_HEAD_MAX_ROWS


def greedy_head(x, w) -> torch.Tensor:
    """argmax over n of x[m] . w[n]^T for at most 16 rows, the lowest index on ties: the head of
    a decode step whose rows all choose greedily.  The weight streams once; every block keeps the
    best of its 32 logits per row, and the rows' bests meet in one 64-bit atomicMax each.
    -> int32 [M]."""
    M, K = x.shape
    ids = torch.empty(M, dtype=torch.int32, device=x.device)
    best, ticket = greedy_workspace(x.device)
    call("bf16", "fmx_gemv_argmax", x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), ids.data_ptr(), best.data_ptr(),
         ticket.data_ptr(), M, w.shape[0], K, _stream())
    return ids


def tile_width(M: int, N: int, sms: int = 148) -> int:
    """The tile width (of 128, 192, 256) whose tiles fill the SMs' rounds best, as the
    tensor-core library plans it (`fmx_gemm_tcgen05_plan_width`)."""
    return int(load("tc").fmx_gemm_tcgen05_plan_width(int(M), int(N), int(sms)))


def tc_fills_the_gpu(M: int, N: int, sms: int = 148) -> bool:
    """Does a product of these sizes fill the GPU on the tensor-memory kernel (else the
    library's product, which splits K, is the faster one)?  The library's own plan
    (`fmx_gemm_tcgen05_plan_fills`)."""
    return bool(load("tc").fmx_gemm_tcgen05_plan_fills(int(M), int(N), int(sms)))


def can_tc(x, w, bias=None, out_dtype=torch.bfloat16, epilogue: int = EPI_PLAIN) -> bool:
    """Does this product go to the tcgen05 kernel?  Only with an epilogue of its own (SiLU-mul over
    blocks of gate and up rows, or a residual), bfloat16 operands, at least 128 rows and tiles
    that fill the GPU.  A plain product runs in the library: with the weights coming from HBM it
    is ahead of the one-CTA kernel at every size measured (2048 x 2048 x 8192: 47 us against 52)."""
    return (epilogue != EPI_PLAIN and _bf16_operands(x, w) and bias is None and out_dtype == torch.bfloat16
            and x.shape[0] >= TC_MIN_ROWS and (epilogue != EPI_SILU_MUL or w.shape[0] % (2 * GATE_UP_BLOCK) == 0)
            and tc_fills_the_gpu(x.shape[0], w.shape[0], num_sms(x.device)))


def gemm_tcgen05(x, w, status=None, epilogue: int = EPI_PLAIN, residual=None, bn: int | None = None) -> torch.Tensor:
    """x[M, K] @ w[N, K]^T on the tcgen05 tensor cores (TMA-fed, accumulators in tensor memory).
    epilogue EPI_SILU_MUL: w's rows come in blocks of bn/2 gate rows then bn/2 up rows, and the
    result is silu(gate) * up, [M, N/2]; EPI_RESIDUAL: residual + product."""
    M, K = x.shape
    N = w.shape[0]
    sms = num_sms(x.device)
    out = torch.empty((M, N // 2 if epilogue == EPI_SILU_MUL else N), dtype=torch.bfloat16, device=x.device)
    call("tc", "fmx_gemm_tcgen05", x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(), out.stride(0),
         _ptr(residual), residual.stride(0) if residual is not None else 0, M, N, K, int(bn or 0), epilogue, sms,
         _ptr(status if status is not None else _status_word(x.device)), _stream())
    return out


def linear(x: torch.Tensor, w: torch.Tensor, bias, out_dtype) -> torch.Tensor:
    """x[M, K] @ w[N, K]^T (+ bias) -> [M, N] in `out_dtype`, accumulated in 32-bit."""
    _need_cuda(x, w, bias)
    assert x.dim() == 2 and w.dim() == 2 and x.shape[1] == w.shape[1], (x.shape, w.shape)
    assert x.stride(1) == 1 and w.stride(1) == 1
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x.shape[0] == 0:
        return gemm_simple(x, w, bias, out_dtype)
    if can_gemv(x, w) and (w.shape[0] < LIBRARY_MIN_FEATURES or bias is not None):
        return gemv(x, w, bias, out_dtype)
    wt = w.t()
    if bias is not None:
        if out_dtype == torch.bfloat16:
            return torch.addmm(bias.to(torch.bfloat16), x, wt)
        return gemm_simple(x, w, bias, out_dtype)
    return torch.mm(x, wt) if out_dtype == torch.bfloat16 else torch.mm(x, wt, out_dtype=out_dtype)


# ----------------------------------------------------------------------------- positions and cache
def rope_kv_write(qkv, positions, inv_freq, rotary_dim, traditional, slot_mapping, kv, nh, nkv, hd, status) -> None:
    """Rotate q and k of qkv[T, (nh + 2 nkv) hd] in place and store k, v at slot_mapping."""
    _need_cuda(qkv, positions, inv_freq, slot_mapping, kv)
    assert qkv.dim() == 2 and qkv.stride(1) == 1 and positions.dtype == torch.int32
    if kv is not None:
        assert kv.is_contiguous() and kv.dtype == qkv.dtype and kv.shape[1] == 2 and kv.shape[2] == nkv \
            and kv.shape[4] == hd and slot_mapping is not None and slot_mapping.dtype == torch.int64
        num_pages, page_size = kv.shape[0], kv.shape[3]
    else:
        num_pages, page_size = 0, 1
    call("common", "fmx_rope_kv_write", qkv.data_ptr(), positions.data_ptr(), _ptr(inv_freq), _ptr(slot_mapping),
         _ptr(kv), qkv.shape[0], nh, nkv, hd, int(rotary_dim), int(bool(traditional)), page_size, num_pages,
         qkv.stride(0), _dt(qkv), _ptr(status), _stream())


def paged_attention_simple(qkv, kv, ctx, group, nh, nkv, hd, scale, window) -> torch.Tensor:
    T = qkv.shape[0]
    out = torch.empty((T, nh * hd), dtype=qkv.dtype, device=qkv.device)
    bt = group.block_tables
    call("common", "fmx_paged_attention_simple", qkv.data_ptr(), qkv.stride(0), kv.data_ptr(), bt.data_ptr(),
         bt.stride(0), ctx.token_row.data_ptr(), ctx.positions.data_ptr(), out.data_ptr(), T, nh, nkv, hd,
         kv.shape[3], kv.shape[0], float(scale), int(window), bt.shape[0], _dt(qkv), _ptr(ctx.status), _stream())
    return out


MAX_SPLITS = 64
ATTN_SCRATCH_FLOATS = 8 << 20        # 32 MiB of split partials per device
_scratch: dict = {}


def attention_scratch(device, floats: int = 0) -> torch.Tensor:
    """The workspace of the split decode attention (partial outputs, maxima and sums): one per
    device, made once at a fixed size and never replaced, since captured graphs hold its
    address.  The engine's own split counts keep rows * kv heads * splits within a round of
    resident blocks, which needs at most 12 MB; a call that asks for more than the buffer
    holds is refused."""
    i = _dev_index(device)
    buf = _scratch.get(i)
    if buf is None:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("the attention workspace must exist before a CUDA graph is captured")
        buf = _scratch[i] = torch.empty(ATTN_SCRATCH_FLOATS, dtype=torch.float32, device=device)
    if floats > buf.numel():
        raise KernelError(f"the split decode attention's workspace holds {buf.numel()} floats, {floats} asked for: "
                          "use fewer splits")
    return buf


ATTN_TICKETS = 1 << 16
_tickets: dict = {}


def attention_tickets(device) -> torch.Tensor:
    """Tickets of the split decode attention (one per row and kv head), zero between launches."""
    t = _tickets.get(_dev_index(device))
    if t is None:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("the attention tickets must exist before a CUDA graph is captured")
        t = _tickets[_dev_index(device)] = torch.zeros(ATTN_TICKETS, dtype=torch.int32, device=device)
    return t


def decode_splits(rows: int, nkv: int, max_ctx: int, hd: int = 64, device=None) -> int:
    """Splits over the keys of a decode step, as the attention library of this head size plans
    them from its own tile and shared-memory sizes (`fmx_attn_decode_plan`)."""
    lib = load(f"attn_hd{hd}")
    return int(lib.fmx_attn_decode_plan(int(rows), int(nkv), int(max_ctx), num_sms(device)))


def attn_decode_scratch_floats(rows: int, nkv: int, splits: int, hd: int) -> int:
    return 0 if splits <= 1 else rows * nkv * splits * 16 * (hd + 2)


def paged_attention_decode(qkv, kv, ctx, group, nh, nkv, hd, scale, window, splits=None, rope=None, out=None) -> torch.Tensor:
    """Every row brings one token: split over the keys, all query heads of a kv head together.
    rope = (inv_freq or None, rotary_dim, traditional, store): qkv is as the projection left it;
    the kernel rotates the queries itself and, if `store`, rotates each row's new key and puts
    it and its value into the cache (what rope_kv_write does in a kernel of its own)."""
    T = qkv.shape[0]
    R = ctx.R
    if out is None:
        out = torch.empty((T, nh * hd), dtype=qkv.dtype, device=qkv.device)
    if splits is None:
        splits = getattr(ctx, "n_splits", 0) or decode_splits(R, nkv, max(1, ctx.max_ctx_after), hd, qkv.device)
    need = attn_decode_scratch_floats(R, nkv, splits, hd)
    scratch = attention_scratch(qkv.device, need) if need else None
    tickets = attention_tickets(qkv.device) if need and R * nkv <= ATTN_TICKETS else None
    bt = group.block_tables
    inv_freq, rot, trad, mode = None, 0, False, 0
    if rope is not None:
        inv_freq, rot, trad, store = rope
        mode = 1 if store else 2
    call(f"attn_hd{hd}", "fmx_attn_decode", qkv.data_ptr(), qkv.stride(0), kv.data_ptr(), bt.data_ptr(), bt.stride(0),
         ctx.row_start.data_ptr(), ctx.positions.data_ptr(), out.data_ptr(), _ptr(scratch),
         scratch.numel() if scratch is not None else 0, _ptr(tickets), R, splits, nh, nkv, kv.shape[3], kv.shape[0],
         float(scale), int(window), _ptr(ctx.status), _ptr(inv_freq), int(rot), 1 if trad else 0, mode, _stream())
    return out


def paged_attention_prefill(qkv, kv, ctx, group, nh, nkv, hd, scale, window, out=None) -> torch.Tensor:
    """Any mix of rows, tiled over 64 packed query rows and 64 keys."""
    T = qkv.shape[0]
    if out is None:
        out = torch.empty((T, nh * hd), dtype=qkv.dtype, device=qkv.device)
    bt = group.block_tables
    call(f"attn_hd{hd}", "fmx_attn_prefill", qkv.data_ptr(), qkv.stride(0), kv.data_ptr(), bt.data_ptr(), bt.stride(0),
         ctx.row_start.data_ptr(), ctx.row_ctx.data_ptr(), out.data_ptr(), ctx.R, int(ctx.max_q_len), nh, nkv,
         kv.shape[3], kv.shape[0], float(scale), int(window), _ptr(ctx.status), _stream())
    return out


TC_ATTN_MIN_TOKENS = 64       # portions at least this long attend on the tensor-memory kernel


def tc_attention_ok(nh: int, nkv: int, hd: int, page_size: int, window: int) -> bool:
    """Sizes the tensor-memory attention kernel takes: head size 64 or 128, at most 16 query
    heads per kv head, a page size that divides 128 (at least 8), no window."""
    rep = nh // nkv
    return (hd in (64, 128) and window <= 0 and rep <= 16
            and page_size >= 8 and 128 % page_size == 0)


def paged_attention_prefill_tc(qkv, kv, ctx, group, nh, nkv, hd, scale, variant: int = 0, out=None, ksplits=None) -> torch.Tensor:
    """Causal attention of prompt portions on the tcgen05 tensor cores (TMA-fed, scores and
    outputs in tensor memory).  variant 0: the library's choice of kernel, 1: one query tile per
    CTA, 2: two.  ksplits: how many CTAs share the keys of a pair of query tiles (the two-tile
    kernel; None: as many as the library plans for a grid that would leave most SMs idle)."""
    T = qkv.shape[0]
    if out is None:
        out = torch.empty((T, nh * hd), dtype=qkv.dtype, device=qkv.device)
    bt = group.block_tables
    lib = load(f"attn_hd{hd}")
    if ksplits is None:
        ksplits = 1
        if variant != 1 and (128 if hd == 64 else 64) % kv.shape[3] == 0:
            ksplits = int(lib.fmx_attn_prefill_tc_plan_splits(int(ctx.R), int(ctx.max_q_len), int(ctx.max_ctx_after), nh, nkv,
                                                               num_sms(qkv.device)))
            if ksplits > 1 and int(lib.fmx_attn_prefill_tc_scratch_floats(T, nh, ksplits)) > ATTN_SCRATCH_FLOATS:
                ksplits = 1
    scratch = attention_scratch(qkv.device, int(lib.fmx_attn_prefill_tc_scratch_floats(T, nh, ksplits))) if ksplits > 1 else None
    call(f"attn_hd{hd}", "fmx_attn_prefill_tc", qkv.data_ptr(), qkv.stride(0), T, kv.data_ptr(), bt.data_ptr(),
         bt.stride(0), ctx.row_start.data_ptr(), ctx.row_ctx.data_ptr(), out.data_ptr(), ctx.R, int(ctx.max_q_len), nh,
         nkv, kv.shape[3], kv.shape[0], float(scale), int(2 if ksplits > 1 else variant), _ptr(ctx.status), int(ksplits),
         _ptr(scratch), scratch.numel() if scratch is not None else 0, _stream())
    return out


def decode_attention_clusters(hd: int, allow: bool) -> bool:
    """Let the split decode attention of head size `hd` combine a row's splits inside a thread-block
    cluster (the default) or make it take the path through L2 and tickets; -> the old setting."""
    return bool(load(f"attn_hd{hd}").fmx_attn_decode_allow_clusters(int(bool(allow))))


def decode_attention_fuses_rope(qkv, kv, ctx, nh, nkv, hd) -> bool:
    """Will `paged_attention` take this step on the split decode kernel, which can rotate q and
    k and store k and v itself?"""
    return (qkv.is_cuda and qkv.dtype == torch.bfloat16 and kv is not None and kv.dtype == qkv.dtype
            and hd % 16 == 0 and hd <= 256 and qkv.stride(0) % 2 == 0 and ctx.all_decode and nh // nkv <= 16)


def _rows_of(ctx, group, a: int, b: int, max_q_len: int, max_ctx_after: int):
    """The rows [a, b) of a step as a step of their own for the attention kernels: the arrays per
    row start at row a, token indices and positions stay those of the whole step."""
    from types import SimpleNamespace
    sub = SimpleNamespace(positions=ctx.positions, status=ctx.status, row_start=ctx.row_start[a:], row_ctx=ctx.row_ctx[a:],
                          R=b - a, max_q_len=max_q_len, max_ctx_after=max_ctx_after, all_decode=max_q_len == 1, n_splits=0)
    return sub, SimpleNamespace(block_tables=group.block_tables[a:b])


def paged_attention(qkv, kv, ctx, group, nh, nkv, hd, scale, window, rope=None) -> torch.Tensor:
    """Attention of every token of the step over the pages of its own request.
    qkv[T, >= nh*hd] holds the (rotated) queries first; -> [T, nh*hd].  bfloat16 with a head
    size in steps of 16 (at most 256) runs on the tensor cores; everything else, and all
    of the 32-bit path, on the one-warp-per-query kernel.  In a mixed step the decoding rows at
    its head go to the split decode kernel and the portions behind them to the tiled one: alone
    on a tile, a decoding row would walk its whole context in one block."""
    _need_cuda(qkv, kv)
    assert kv.is_contiguous() and kv.dtype == qkv.dtype and qkv.stride(1) == 1
    tiled = qkv.dtype == torch.bfloat16 and hd % 16 == 0 and hd <= 256 and qkv.stride(0) % 2 == 0
    if tiled and ctx.all_decode and nh // nkv <= 16:
        return paged_attention_decode(qkv, kv, ctx, group, nh, nkv, hd, scale, window, rope=rope)
    if rope is not None:
        raise KernelError("only the split decode kernel rotates by itself: ask decode_attention_fuses_rope first")
    if not tiled:
        return paged_attention_simple(qkv, kv, ctx, group, nh, nkv, hd, scale, window)
    out = None
    d = getattr(ctx, "decode_rows", 0)
    if d > 0 and nh // nkv <= 16:
        key = ("attention rows", id(group))
        views = ctx.scratch.get(key)
        if views is None:
            views = ctx.scratch[key] = (_rows_of(ctx, group, 0, d, 1, ctx.decode_max_ctx),
                                        _rows_of(ctx, group, d, ctx.R, ctx.rest_max_q_len, ctx.rest_max_ctx))
        (dctx, dgroup), (ctx, group) = views
        out = torch.empty((qkv.shape[0], nh * hd), dtype=qkv.dtype, device=qkv.device)
        paged_attention_decode(qkv, kv, dctx, dgroup, nh, nkv, hd, scale, window, out=out)
    if ctx.max_q_len >= TC_ATTN_MIN_TOKENS and tc_attention_ok(nh, nkv, hd, kv.shape[3], window) \
            and qkv.stride(0) % 8 == 0 and qkv.data_ptr() % 16 == 0:
        return paged_attention_prefill_tc(qkv, kv, ctx, group, nh, nkv, hd, scale, out=out)
    return paged_attention_prefill(qkv, kv, ctx, group, nh, nkv, hd, scale, window, out=out)


# ----------------------------------------------------------------------------- sampling
ARGMAX_ROWS, ARGMAX_CHUNKS = 1024, 32      # the split greedy choice's workspace: rows x chunks pairs
ARGMAX_MIN_CHUNK = 4096                    # logits per block at least
_argmax_ws: dict = {}


def argmax_workspace(device):
    """Chunk results and tickets of the split greedy choice, one pair per device, made once;
    the tickets are zero between launches."""
    ws = _argmax_ws.get(_dev_index(device))
    if ws is None:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("the greedy choice's workspace must exist before a CUDA graph is captured")
        ws = (torch.empty(ARGMAX_ROWS * ARGMAX_CHUNKS * 2, dtype=torch.int32, device=device),
              torch.zeros(ARGMAX_ROWS, dtype=torch.int32, device=device))
        _argmax_ws[_dev_index(device)] = ws
    return ws


def argmax_chunks(rows: int, V: int) -> int:
    """Blocks per row of the greedy choice: enough to fill the SMs about once, each with at
    least ARGMAX_MIN_CHUNK logits; 1 = the one-block kernel."""
    if rows > ARGMAX_ROWS:
        return 1
    return max(1, min(ARGMAX_CHUNKS, V // ARGMAX_MIN_CHUNK, -(-num_sms() // max(rows, 1))))


def sample(logits: torch.Tensor, temperature=None, uniform=None, keep=None) -> torch.Tensor:
    """Row-wise token choice: argmax where temperature <= 0 (or None), else a draw from
    softmax(logits / temperature) among keep != 0 by the given uniform numbers."""
    _need_cuda(logits, temperature, uniform, keep)
    assert logits.dim() == 2 and logits.dtype == torch.float32 and logits.stride(1) == 1
    rows, V = logits.shape
    out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    if keep is not None:
        assert keep.dtype == torch.uint8 and keep.shape == logits.shape and keep.stride(1) == 1
    chunks = argmax_chunks(rows, V) if temperature is None and keep is None else 1
    partial, tickets = argmax_workspace(logits.device) if chunks > 1 else (None, None)
    call("common", "fmx_sample", logits.data_ptr(), logits.stride(0), rows, V, _ptr(temperature), _ptr(uniform),
         _ptr(keep), keep.stride(0) if keep is not None else 0, out.data_ptr(), chunks, _ptr(partial), ARGMAX_CHUNKS,
         _ptr(tickets), ARGMAX_ROWS, _stream())
    return out


def argmax(logits: torch.Tensor) -> torch.Tensor:
    return sample(logits)


def filter_mask(logits, top_p=None, min_p=None, top_k=None, min_keep=None) -> torch.Tensor:
    """uint8 [rows, V]: 1 where the row's filters (top-p, then min-p, then top-k) keep the token.
    Each argument is a per-row tensor (float32 / int32) or None for "off"."""
    _need_cuda(logits, top_p, min_p, top_k, min_keep)
    assert logits.dim() == 2 and logits.dtype == torch.float32 and logits.stride(1) == 1
    rows, V = logits.shape
    keep = torch.empty((rows, V), dtype=torch.uint8, device=logits.device)
    call("common", "fmx_filter_mask", logits.data_ptr(), logits.stride(0), rows, V, _ptr(top_p), _ptr(min_p),
         _ptr(top_k), _ptr(min_keep), keep.data_ptr(), keep.stride(0), _stream())
    return keep


def filter_sample_takes(V: int) -> bool:
    """Rows of this width can be filtered and sampled by one kernel (`filter_sample`)."""
    return bool(load("common").fmx_filter_sample_takes(int(V)))


def filter_sample(logits, temperature, uniform, top_p=None, min_p=None, top_k=None, min_keep=None) -> torch.Tensor:
    """The token of each row after its filters, in one kernel and without a keep mask in memory:
    what `sample(logits, temperature, uniform, filter_mask(logits, ...))` gives.  A row is spread
    over a thread-block cluster with its logits in registers."""
    _need_cuda(logits, temperature, uniform, top_p, min_p, top_k, min_keep)
    assert logits.dim() == 2 and logits.dtype == torch.float32 and logits.stride(1) == 1
    rows, V = logits.shape
    out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    call("common", "fmx_filter_sample", logits.data_ptr(), logits.stride(0), rows, V, _ptr(temperature), _ptr(uniform),
         _ptr(top_p), _ptr(min_p), _ptr(top_k), _ptr(min_keep), out.data_ptr(), _stream())
    return out


def penalties(logits, history, repetition, presence, frequency, windows) -> None:
    """In place on float32 logits [rows, V].  history int32 [rows, H] (oldest first, -1 padded
    in front); repetition/presence/frequency float32 [rows] or None; windows int32 [rows, 3]."""
    _need_cuda(logits, history, repetition, presence, frequency, windows)
    assert logits.dtype == torch.float32 and history.dtype == torch.int32 and windows.dtype == torch.int32
    call("common", "fmx_penalties", logits.data_ptr(), logits.stride(0), logits.shape[0], logits.shape[1],
         history.data_ptr(), history.shape[1], _ptr(repetition), _ptr(presence), _ptr(frequency),
         windows.data_ptr(), _stream())


def logit_bias(logits, rows, ids, values) -> None:
    """logits[rows[i], ids[i]] += values[i], in place."""
    _need_cuda(logits, rows, ids, values)
    call("common", "fmx_logit_bias", logits.data_ptr(), logits.stride(0), logits.shape[1], rows.data_ptr(),
         ids.data_ptr(), values.data_ptr(), rows.numel(), _stream())
