"""The decode attention entry point for callers that cannot allocate device memory
(csrc/attn/attention_noalloc.h), called through its exported C symbol.

Such callers are embedders that own every allocation themselves, or code that runs where
allocating is not allowed (during a stream capture, under a memory pool that must not be
disturbed): they hand the library inputs and an output and nothing else.  The entry point
keeps its workspace in a fixed array of the loaded module.  Here it is checked against the
ordinary entry point (which is given a workspace) and against the plain statement of the
operation, on calls in a row, because the array keeps the earlier call's contents; with a
padding row, a window, and more splits than the context has key tiles; and its size limit and
its refusal of a first call under stream capture are checked.

This file sorts last on purpose: a run that stops at the first failure has then run every
other test already.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _lib(hd):
    from fastmlx_b200.kernels import lib as klib
    lib = klib.load(f"attn_hd{hd}")
    c_p, c_i, c_l, c_f = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
    fn = lib.fmx_attn_decode_noalloc
    fn.argtypes = [c_p, c_l, c_p, c_p, c_i, c_p, c_p, c_p, c_i, c_i, c_i, c_i, c_i, c_l, c_f, c_i, c_p, c_p]
    fn.restype = c_i
    lib.fmx_attn_decode_noalloc_floats.argtypes = [c_i, c_i, c_i]
    lib.fmx_attn_decode_noalloc_floats.restype = c_l
    lib.fmx_attn_decode_noalloc_max_floats.restype = c_l
    return lib


def _case(rows, ctx_lens, nh, nkv, hd, page, seed):
    g = torch.Generator().manual_seed(seed)
    blocks = [-(-(c + 1) // page) for c in ctx_lens]
    num_pages = sum(blocks) + 2
    perm = torch.randperm(num_pages, generator=g).tolist()
    bt = torch.full((rows, max(blocks)), -1, dtype=torch.int32)
    for r, n in enumerate(blocks):
        for b in range(n):
            bt[r, b] = perm.pop()
    kv = torch.randn(num_pages, 2, nkv, page, hd, generator=g).to(torch.bfloat16)
    q = torch.randn(rows, (nh + 2 * nkv) * hd, generator=g).to(torch.bfloat16)
    return (q.to(DEV), kv.to(DEV), bt.to(DEV), torch.arange(rows + 1, dtype=torch.int32, device=DEV),
            torch.tensor(ctx_lens, dtype=torch.int32, device=DEV))


def _noalloc(lib, q, kv, bt, row_start, positions, nh, nkv, hd, splits, window=0):
    rows = positions.numel()
    out = torch.full((rows, nh * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    rc = lib.fmx_attn_decode_noalloc(q.data_ptr(), q.stride(0), kv.data_ptr(), bt.data_ptr(), bt.stride(0),
                                     row_start.data_ptr(), positions.data_ptr(), out.data_ptr(), rows, splits, nh, nkv,
                                     kv.shape[3], kv.shape[0], hd ** -0.5, window, status.data_ptr(),
                                     torch.cuda.current_stream().cuda_stream)
    return rc, out, status


def _ordinary(q, kv, bt, row_start, positions, nh, nkv, hd, splits, window=0):
    from types import SimpleNamespace
    import fastmlx_b200.kernels as k
    ctx = SimpleNamespace(R=positions.numel(), row_start=row_start, positions=positions, max_ctx_after=int(positions.max()) + 1,
                          status=torch.zeros(4, dtype=torch.int32, device=DEV), n_splits=0)
    return k.paged_attention_decode(q, kv, ctx, SimpleNamespace(block_tables=bt), nh, nkv, hd, hd ** -0.5, window, splits=splits)


def _plain(q, kv, bt, row_start, positions, nh, nkv, hd, window=0):
    from types import SimpleNamespace
    import plain_ops
    ctx = SimpleNamespace(positions=positions.cpu(), token_row=torch.arange(positions.numel(), dtype=torch.int32),
                          status=torch.zeros(4, dtype=torch.int32))
    return plain_ops.paged_attention(q.cpu(), kv.cpu(), ctx, SimpleNamespace(block_tables=bt.cpu()), nh, nkv, hd, hd ** -0.5, window)


def _close(got, want, extra=0.0):
    """One bfloat16 unit in the last place (2^-7 relative at worst) plus a floor."""
    diff = (got.float().cpu() - want.float().cpu()).abs()
    assert (diff <= 2.0 ** -7 * want.float().cpu().abs() + 1e-3 + extra).all(), diff.max().item()


def test_a_first_call_under_stream_capture_is_refused():
    """The set-up of a device's first call asks the runtime for the array's address, which a
    capturing stream must not see: the call says so instead of breaking the capture.  A head
    size that no other test loads, so that this is its library's first call in any order of
    the tests."""
    hd, nh, nkv, page = 240, 2, 1, 16
    lib = _lib(hd)
    case = _case(2, [40, 3], nh, nkv, hd, page, seed=5)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        rc, _, _ = _noalloc(lib, *case, nh, nkv, hd, 2)
    assert rc != 0 and "before any stream capture" in lib.fmx_last_error().decode()
    rc, got, _ = _noalloc(lib, *case, nh, nkv, hd, 2)                  # outside a capture it sets up and runs
    assert rc == 0, lib.fmx_last_error().decode()
    _close(got, _plain(*case, nh, nkv, hd), extra=2.0 ** -9 * 5)


@pytest.mark.parametrize("nh,nkv,hd,page", [(32, 8, 64, 16), (8, 2, 128, 32)])
def test_no_alloc_entry_matches_the_ordinary_one_twice_in_a_row(nh, nkv, hd, page):
    lib = _lib(hd)
    first = _case(5, [700, 64, 0, 333, 1500], nh, nkv, hd, page, seed=1)
    second = _case(3, [90, 1023, 17], nh, nkv, hd, page, seed=2)      # other sizes over the same array
    padded = _case(3, [70, 5, 69], nh, nkv, hd, page, seed=4)         # row 1 is a padding row: position -1, no pages;
    #                                                                   32 splits over 70 keys: most splits hold no key
    padded[4][1] = -1
    padded[2][1] = -1
    for case, splits, window in ((first, 6, 0), (second, 3, 0), (first, 1, 0), (padded, 32, 0), (first, 5, 100),
                                 (second, 2, 24)):
        rc, got, status = _noalloc(lib, *case, nh, nkv, hd, splits, window)
        assert rc == 0, lib.fmx_last_error().decode()
        want = _ordinary(*case, nh, nkv, hd, splits, window)
        torch.cuda.synchronize()
        assert status.tolist()[0] == 0
        assert torch.isfinite(got.float()).all()
        # the same partial results, combined by another kernel (a product with 1/L here, a
        # division by L there): equal to one unit in the last place
        _close(got, want)
        # and against the plain statement, with the 2^-9 rounding of the probabilities handed to
        # the tensor cores on top
        _close(got, _plain(*case, nh, nkv, hd, window), extra=2.0 ** -9 * float(case[1].float().abs().max()))
    assert float(got.float().abs().sum()) > 0
    rc, got, _ = _noalloc(lib, *padded, nh, nkv, hd, 32)
    assert rc == 0 and float(got[1].float().abs().sum()) == 0.0        # the padding row reads nothing


def test_no_alloc_entry_refuses_what_its_array_cannot_hold():
    lib = _lib(64)
    limit = lib.fmx_attn_decode_noalloc_max_floats()
    assert limit == 1 << 20
    assert lib.fmx_attn_decode_noalloc_floats(8, 8, 4) == 8 * 8 * 4 * 16 * 66
    assert lib.fmx_attn_decode_noalloc_floats(8, 8, 1) == 0
    rows, nh, nkv, hd, page = 64, 32, 8, 64, 16
    assert lib.fmx_attn_decode_noalloc_floats(rows, nkv, 8) > limit
    case = _case(rows, [40] * rows, nh, nkv, hd, page, seed=3)
    rc, out, _ = _noalloc(lib, *case, nh, nkv, hd, 8)
    assert rc != 0
    msg = lib.fmx_last_error().decode()
    assert "floats of workspace" in msg and "holds" in msg
    torch.cuda.synchronize()
    assert torch.isnan(out.float()).all()                              # nothing was launched
    rc, out, _ = _noalloc(lib, *case, nh, nkv, hd, 1)                  # one split needs no workspace at all
    assert rc == 0
    _close(out, _ordinary(*case, nh, nkv, hd, 1))
