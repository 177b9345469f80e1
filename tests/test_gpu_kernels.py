"""Each CUDA kernel alone against its plain statement (tests/plain_ops.py), at sizes other
than the engine's, in 32-bit and in bfloat16."""
from types import SimpleNamespace

import pytest
import torch

import plain_ops

pytestmark = pytest.mark.gpu

DEV = "cuda"
DTYPES = [torch.float32, torch.bfloat16]


def k():
    import fastmlx_b200.kernels as kern
    return kern


def status():
    return torch.zeros(4, dtype=torch.int32, device=DEV)


def close(got, ref, dtype, what="", scale=None, extra=0.0):
    """32-bit: a few units of float32 rounding of the result's scale.  bfloat16: the same
    value may round to the neighbouring bfloat16 (one unit in the last place = 2^-7
    relative at worst) when 32-bit and 64-bit arithmetic land on different sides."""
    got, ref = got.detach().double().cpu(), ref.detach().double().cpu()
    s = ref.abs().max().item() if scale is None else scale
    s = max(s, 1e-30)
    if dtype == torch.float32:
        tol = 2e-6 * s
        bad = (got - ref).abs() > tol + 2e-6 * ref.abs()
    else:
        bad = (got - ref).abs() > 2.0 ** -7 * ref.abs() + 1e-3 * s + extra
    assert not bad.any(), f"{what} (extra {extra:.2e}): {int(bad.sum())} of {bad.numel()} off, worst {(got - ref).abs().max().item():.3e} (scale {s:.3e})"


def rnd(*shape, dtype=torch.float32, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


# ----------------------------------------------------------------------------- rows
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("V,d,n", [(131, 80, 7), (320, 2048, 33), (50, 100, 5), (17, 3, 4)])
def test_embedding(dtype, V, d, n):
    table = rnd(V, d, dtype=dtype)
    ids = torch.randint(0, V, (n,), dtype=torch.int32)
    st = status()
    out = k().embedding(ids.to(DEV), table.to(DEV), st)
    assert torch.equal(out.cpu(), table[ids.long()])
    assert st.tolist()[0] == 0


def test_embedding_bad_id_leaves_code_not_fault():
    table = rnd(10, 16).to(DEV)
    st = status()
    out = k().embedding(torch.tensor([1, 10, 2], dtype=torch.int32, device=DEV), table, st)
    assert st.tolist()[0] == k().BAD_TOKEN and st.tolist()[1] == 10
    assert torch.equal(out[0].cpu(), table[1].cpu()) and float(out[1].abs().sum()) == 0.0


# ----------------------------------------------------------------------------- norm
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,d,eps", [(1, 64, 1e-5), (5, 192, 1e-6), (33, 80, 1e-3), (4, 2048, 1e-5), (3, 1000, 1e-5), (2, 5, 0.0)])
@pytest.mark.parametrize("with_residual", [False, True])
def test_add_rmsnorm(dtype, rows, d, eps, with_residual):
    x = rnd(rows, d, dtype=dtype, seed=1, scale=3.0)
    res = rnd(rows, d, dtype=dtype, seed=2, scale=5.0) if with_residual else None
    w = 1 + rnd(d, seed=3, scale=0.1)
    ref_out, ref_res = plain_ops.add_rmsnorm(x.clone(), res.clone() if with_residual else None, w, eps)
    xd = x.to(DEV)
    rd = res.to(DEV) if with_residual else None
    out, res_out = k().add_rmsnorm(xd, rd, w.to(DEV), eps)
    close(out, ref_out, dtype, "norm")
    if with_residual:
        assert res_out.data_ptr() == rd.data_ptr()
        close(res_out, ref_res, dtype, "residual")
    else:
        assert res_out.data_ptr() == xd.data_ptr()


@pytest.mark.parametrize("rows,d,eps", [(1, 64, 1e-5), (5, 192, 1e-6), (33, 80, 1e-3), (4, 2048, 1e-5), (3, 1000, 1e-5), (2, 5, 0.0),
                                        (8, 8192, 1e-5), (3, 8200, 1e-5)])
def test_add_rmsnorm_with_a_32_bit_stream(rows, d, eps):
    """bfloat16 activations beside a stream kept in 32-bit: the first call makes the stream from
    x, later calls add to it without rounding it, and the stream alone can be normalised."""
    x = rnd(rows, d, dtype=torch.bfloat16, seed=1, scale=3.0)
    y = rnd(rows, d, dtype=torch.bfloat16, seed=2, scale=0.01)          # small against the stream, as a layer's output is
    w = 1 + rnd(d, seed=3, scale=0.1)
    wd = w.to(DEV)
    ref0, ref_stream = plain_ops.add_rmsnorm(x.clone(), None, w, eps, stream_dtype=torch.float32)
    out0, stream = k().add_rmsnorm(x.to(DEV), None, wd, eps, stream_dtype=torch.float32)
    assert stream.dtype == torch.float32 and out0.dtype == torch.bfloat16
    assert torch.equal(stream.cpu(), x.float())
    close(out0, ref0, torch.bfloat16, "norm of the first value")
    for i in range(3):
        ref1, ref_stream = plain_ops.add_rmsnorm(y.clone(), ref_stream, w, eps)
        out1, stream2 = k().add_rmsnorm(y.to(DEV), stream, wd, eps)
        assert stream2.data_ptr() == stream.data_ptr()
        close(stream, ref_stream, torch.float32, "32-bit stream")
        close(out1, ref1, torch.bfloat16, "norm over a 32-bit stream")
    # three additions of a value that bfloat16 would have lost against the stream
    assert (stream.cpu() - x.float() - 3 * y.float()).abs().max() < 1e-5 * x.float().abs().max()
    ref2, _ = plain_ops.add_rmsnorm(None, ref_stream.clone(), w, eps, out_dtype=torch.bfloat16)
    out2, _ = k().add_rmsnorm(None, stream, wd, eps, out_dtype=torch.bfloat16)
    close(out2, ref2, torch.bfloat16, "norm of the stream alone")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,I", [(1, 176), (7, 512), (3, 200), (65, 8192), (2, 1)])
def test_silu_mul(dtype, rows, I):
    gu = rnd(rows, 2 * I, dtype=dtype, seed=4, scale=4.0)
    close(k().silu_mul(gu.to(DEV)), plain_ops.silu_mul(gu), dtype, "silu_mul")


# ----------------------------------------------------------------------------- matrix products
@pytest.mark.parametrize("M,N,K", [(1, 64, 64), (7, 131, 80), (65, 192, 500), (130, 70, 33), (3, 320, 192), (64, 64, 16)])
@pytest.mark.parametrize("bias", [False, True])
def test_gemm_f32_fixed_order(M, N, K, bias):
    x, w = rnd(M, K, seed=5), rnd(N, K, seed=6)
    b = rnd(N, seed=7) if bias else None
    ref = plain_ops.linear(x, w, b, torch.float64)
    got = k().linear(x.to(DEV), w.to(DEV), b.to(DEV) if bias else None, torch.float32)
    bound = (x.abs().double() @ w.abs().double().t()) * 1.2e-7 * 4 + 1e-30   # a few roundings of the running sum
    assert ((got.cpu().double() - ref).abs() <= bound * (K ** 0.5 + 2)).all()


def test_gemm_f32_result_does_not_depend_on_the_batch():
    """A row's product is bit-identical whether it runs alone or among 100 others."""
    x, w = rnd(101, 300, seed=8).to(DEV), rnd(77, 300, seed=9).to(DEV)
    full = k().linear(x, w, None, torch.float32)
    for r in (0, 50, 100):
        alone = k().linear(x[r:r + 1].contiguous(), w, None, torch.float32)
        assert torch.equal(alone[0], full[r])
    part = k().linear(x[37:90], w, None, torch.float32)       # a strided view of rows
    assert torch.equal(part, full[37:90])


@pytest.mark.parametrize("M,N,K", [(1, 64, 64), (9, 136, 80), (70, 192, 512), (2048, 320, 192)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("bias", [False, True])
def test_linear_bf16(M, N, K, out_dtype, bias):
    x, w = rnd(M, K, dtype=torch.bfloat16, seed=5), rnd(N, K, dtype=torch.bfloat16, seed=6)
    b = rnd(N, seed=7).bfloat16().float() if bias else None
    ref = plain_ops.linear(x, w, b, torch.float64)
    got = k().linear(x.to(DEV), w.to(DEV), b.to(DEV) if bias else None, out_dtype)
    assert got.dtype == out_dtype
    close(got, ref, out_dtype if out_dtype == torch.bfloat16 else torch.float32, "linear", scale=ref.abs().max().item() * 8)


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (128, 256, 64), (256, 256, 512), (2048, 3072, 2048), (300, 200, 136),
                                   (1, 320, 192), (100, 8, 8), (129, 385, 72), (640, 2048, 8192)])
@pytest.mark.parametrize("bn", [128, 192, 256])
def test_gemm_tcgen05(M, N, K, bn):
    """The tensor-memory product against the plain one: tiles cut by every edge (rows, columns
    and k that are no multiples of 128 / bn / 64), all three tile widths."""
    x, w = rnd(M, K, dtype=torch.bfloat16, seed=21), rnd(N, K, dtype=torch.bfloat16, seed=22, scale=0.05)
    st = status()
    got = k().gemm_tcgen05(x.to(DEV), w.to(DEV), st, bn=bn)
    assert st.tolist()[0] == 0
    close(got, plain_ops.linear(x, w, None, torch.float64), torch.bfloat16, f"tcgen05 product, tile width {bn}")


@pytest.mark.parametrize("M,I,K", [(128, 128, 64), (300, 384, 136), (2048, 1024, 512), (5, 256, 64)])
def test_gemm_tcgen05_epilogues(M, I, K):
    x = rnd(M, K, dtype=torch.bfloat16, seed=31)
    wg, wu = rnd(I, K, dtype=torch.bfloat16, seed=32, scale=0.1), rnd(I, K, dtype=torch.bfloat16, seed=33, scale=0.1)
    blk = k().GATE_UP_BLOCK
    w = torch.stack([wg.view(-1, blk, K), wu.view(-1, blk, K)], dim=1).reshape(2 * I, K).contiguous()
    st = status()
    got = k().gemm_tcgen05(x.to(DEV), w.to(DEV), st, epilogue=k().EPI_SILU_MUL)
    # as the unfused path: both products rounded to bfloat16, then silu(gate) * up
    g = plain_ops.linear(x, wg, None, torch.bfloat16)
    u = plain_ops.linear(x, wu, None, torch.bfloat16)
    ref = plain_ops.silu_mul(torch.cat([g, u], dim=1))
    assert got.shape == (M, I) and st.tolist()[0] == 0
    close(got, ref, torch.bfloat16, "fused SiLU-mul epilogue", extra=2.0 ** -8 * ref.abs().max().item())
    # the same weight through the unfused kernels
    gu = k().linear(x.to(DEV), w.to(DEV), None, torch.bfloat16)
    close(k().silu_mul(gu, blk), ref, torch.bfloat16, "blocked SiLU-mul", extra=2.0 ** -8 * ref.abs().max().item())
    res = rnd(M, 2 * I, dtype=torch.bfloat16, seed=34)
    got = k().gemm_tcgen05(x.to(DEV), w.to(DEV), st, epilogue=k().EPI_RESIDUAL, residual=res.to(DEV))
    ref = (plain_ops.linear(x, w, None, torch.bfloat16).double() + res.double())
    close(got, ref, torch.bfloat16, "residual epilogue", extra=2.0 ** -8 * ref.abs().max().item())


@pytest.mark.parametrize("M", [1, 2, 7, 8, 9, 16])
@pytest.mark.parametrize("N,K", [(16, 32), (64, 64), (131, 80), (3072, 2048), (2048, 8192), (50, 8), (320, 192), (17, 1000)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemv(M, N, K, out_dtype):
    """The product with the whole of K in one block: every row count up to 16, widths that are
    no multiple of the 32-wide k block or of the 8-feature tile, bias, residual in place, both
    tile widths."""
    x, w = rnd(M, K, dtype=torch.bfloat16, seed=11), rnd(N, K, dtype=torch.bfloat16, seed=12, scale=0.05)
    b = rnd(N, seed=13) if N % 2 else None
    ref = plain_ops.linear(x, w, b, torch.float64)
    scale = ref.abs().max().item() * 8 if out_dtype == torch.float32 else None
    xd, wd, bd = x.to(DEV), w.to(DEV), b.to(DEV) if b is not None else None
    for wide, warps in ((8, 8), (16, 8), (32, 8), (8, 16), (16, 16)):
        got = k().gemv(xd, wd, bd, out_dtype, wide=wide, warps=warps)
        close(got, ref, out_dtype, "gemv", scale=scale)
        alone = k().gemv(xd[M - 1:].contiguous(), wd, bd, out_dtype, wide=wide, warps=warps)
        if M <= 8:                                       # rows 8..15 sit in another accumulator half
            assert torch.equal(alone[0], got[M - 1])     # a row's result does not depend on its companions
    if out_dtype == torch.bfloat16:
        res = rnd(M, N, dtype=torch.bfloat16, seed=44)
        stream = res.clone().to(DEV)
        out = k().gemv(xd, wd, residual=stream, out=stream)
        assert out.data_ptr() == stream.data_ptr()
        want = plain_ops.linear(x, w, None, torch.bfloat16).double() + res.double()
        close(stream, want, torch.bfloat16, "gemv residual epilogue", extra=2.0 ** -8 * want.abs().max().item())


@pytest.mark.parametrize("M", [1, 8, 13])
@pytest.mark.parametrize("I,K,blk", [(128, 64, 128), (8192, 2048, 128), (384, 200, 128), (64, 72, 32), (48, 40, 16)])
def test_gemv_gate_up(M, I, K, blk):
    x = rnd(M, K, dtype=torch.bfloat16, seed=51, scale=2.0)
    wg, wu = rnd(I, K, dtype=torch.bfloat16, seed=52, scale=0.1), rnd(I, K, dtype=torch.bfloat16, seed=53, scale=0.1)
    w = torch.stack([wg.view(-1, blk, K), wu.view(-1, blk, K)], dim=1).reshape(2 * I, K).contiguous()
    g = plain_ops.linear(x, wg, None, torch.bfloat16)
    u = plain_ops.linear(x, wu, None, torch.bfloat16)
    ref = plain_ops.silu_mul(torch.cat([g, u], dim=1))
    for wide in (8, 16, 32):
        if blk % wide:
            continue
        got = k().gemv(x.to(DEV), w.to(DEV), block=blk, wide=wide)
        assert got.shape == (M, I)
        close(got, ref, torch.bfloat16, "gemv gate/up with SiLU-mul", extra=2.0 ** -7 * ref.abs().max().item())


@pytest.mark.parametrize("ta,tw,tc", [(torch.bfloat16, torch.float32, torch.bfloat16), (torch.bfloat16, torch.float32, torch.float32),
                                      (torch.bfloat16, torch.bfloat16, torch.float32), (torch.bfloat16, torch.bfloat16, torch.bfloat16)])
def test_gemm_simple_mixed_types(ta, tw, tc):
    x, w = rnd(19, 70, dtype=ta, seed=1), rnd(45, 70, dtype=tw, seed=2)
    got = k().gemm_simple(x.to(DEV), w.to(DEV), None, tc)
    close(got, plain_ops.linear(x, w, None, torch.float64), tc, "gemm_simple", scale=None)


# ----------------------------------------------------------------------------- rope + cache write
def _paged(n_rows, lens, page_size, num_pages, seed=0):
    """Block tables that scatter each row's pages over the pool in a shuffled order."""
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(num_pages, generator=g).tolist()
    max_blocks = max(-(-n // page_size) for n in lens)
    bt = torch.full((n_rows, max_blocks + 1), -1, dtype=torch.int32)
    for r, n in enumerate(lens):
        for b in range(-(-n // page_size)):
            bt[r, b] = perm.pop()
    return bt


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd,rot,trad", [(4, 2, 16, 16, False), (6, 3, 32, 32, False), (5, 1, 48, 48, True),
                                                 (8, 2, 64, 32, False), (3, 3, 128, 128, False), (2, 1, 80, 40, True),
                                                 (4, 0, 32, 32, False), (4, 2, 32, 0, False)])
def test_rope_kv_write(dtype, nh, nkv, hd, rot, trad):
    T, page_size, num_pages = 23, 8, 9
    qkv = rnd(T, (nh + 2 * nkv) * hd, dtype=dtype, seed=1)
    positions = torch.tensor([0, 1, 2, 3, 63, 64, 65, 500, 8191, 8192, 100000, 131071] + list(range(7, 18)), dtype=torch.int32)
    inv_freq = (10000.0 ** (-torch.arange(0, max(rot, 2), 2, dtype=torch.float64) / max(rot, 2))).float()
    slots = torch.randperm(num_pages * page_size, generator=torch.Generator().manual_seed(2))[:T].long()
    slots[5] = -1                                                # a padding token is stored nowhere
    kv_ref = torch.zeros(num_pages, 2, max(nkv, 1), page_size, hd, dtype=dtype)
    kv_dev = kv_ref.clone().to(DEV)
    q_ref = qkv.clone()
    st_ref = torch.zeros(4, dtype=torch.int32)
    plain_ops.rope_kv_write(q_ref, positions, inv_freq, rot, trad, slots, kv_ref if nkv else None, nh, nkv, hd, st_ref)
    q_dev = qkv.clone().to(DEV)
    st = status()
    k().rope_kv_write(q_dev, positions.to(DEV), inv_freq.to(DEV), rot, trad, slots.to(DEV), kv_dev if nkv else None,
                      nh, nkv, hd, st)
    assert st.tolist()[0] == 0
    close(q_dev, q_ref, dtype, "rotated qkv")
    close(kv_dev, kv_ref, dtype, "pages", scale=1.0)


def test_rope_bad_slot_leaves_code():
    qkv = rnd(2, 4 * 16).to(DEV)
    kv = torch.zeros(2, 2, 1, 4, 16, device=DEV)
    st = status()
    k().rope_kv_write(qkv, torch.zeros(2, dtype=torch.int32, device=DEV), torch.ones(8, device=DEV), 16, False,
                      torch.tensor([0, 99], device=DEV), kv, 2, 1, 16, st)
    assert st.tolist()[:2] == [k().BAD_SLOT, 99]


# ----------------------------------------------------------------------------- attention over pages
def _attention_case(dtype, nh, nkv, hd, page_size, rows, window=0, seed=0, spike=None):
    """rows: list of (ctx_before, q_len).  Pages are filled for every position < ctx+q."""
    lens = [c + q for c, q in rows]
    num_pages = sum(-(-n // page_size) for n in lens) + 3
    bt = _paged(len(rows), lens, page_size, num_pages, seed)
    g = torch.Generator().manual_seed(seed + 1)
    kv = torch.randn(num_pages, 2, nkv, page_size, hd, generator=g).to(dtype)
    T = sum(q for _, q in rows)
    q = torch.randn(T, nh * hd, generator=g).to(dtype)
    pos, trow = [], []
    for r, (c, ql) in enumerate(rows):
        pos += list(range(c, c + ql))
        trow += [r] * ql
    if spike is not None:
        # One far key is made to stand out for one query: the query and that key are scaled
        # along a common direction so its score dominates, and its value row is marked.
        t, key_pos, head = spike
        r = trow[t]
        page = int(bt[r, key_pos // page_size])
        gk = head // (nh // nkv)
        d = torch.randn(hd, generator=g)
        d = d / d.norm()
        q[t, head * hd:(head + 1) * hd] = (d * 12.0).to(dtype)
        kv[page, 0, gk, key_pos % page_size] = (d * 12.0).to(dtype)
        kv[page, 1, gk, key_pos % page_size] = torch.full((hd,), 7.0).to(dtype)
    ctx = SimpleNamespace(positions=torch.tensor(pos, dtype=torch.int32), token_row=torch.tensor(trow, dtype=torch.int32),
                          status=torch.zeros(4, dtype=torch.int32))
    grp = SimpleNamespace(block_tables=bt)
    return q, kv, ctx, grp


def _to_dev(ctx, grp):
    return (SimpleNamespace(positions=ctx.positions.to(DEV), token_row=ctx.token_row.to(DEV), status=status(),
                            all_decode=False, max_q_len=0, max_ctx_after=0, row_start=None, row_ctx=None, R=grp.block_tables.shape[0], scratch={}),
            SimpleNamespace(block_tables=grp.block_tables.to(DEV), page_size=None))


ATT_SHAPES = [(4, 2, 16, 16), (6, 3, 32, 16), (5, 1, 48, 8), (8, 8, 64, 32), (12, 4, 128, 64), (3, 3, 80, 16), (2, 1, 256, 16)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd,page_size", ATT_SHAPES)
@pytest.mark.parametrize("window", [0, 24])
def test_paged_attention_simple_mixed_rows(dtype, nh, nkv, hd, page_size, window):
    rows = [(0, 37), (90, 1), (31, 2), (0, 1), (15, 17), (64, 1)]
    q, kv, ctx, grp = _attention_case(dtype, nh, nkv, hd, page_size, rows, window)
    ref = plain_ops.paged_attention(q, kv, ctx, grp, nh, nkv, hd, hd ** -0.5, window)
    dctx, dgrp = _to_dev(ctx, grp)
    got = k().paged_attention_simple(q.to(DEV), kv.to(DEV), dctx, dgrp, nh, nkv, hd, hd ** -0.5, window)
    assert dctx.status.tolist()[0] == 0
    close(got, ref, dtype, "attention", scale=1.0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("key_pos", [0, 15, 16, 17, 31, 32, 63, 64, 511, 512, 700])
def test_paged_attention_simple_far_key_stands_out(dtype, key_pos):
    """Among 701 keys one is made dominant; a kernel that misses it (a page's edge, a
    chunk's edge) returns something far from its marked value."""
    nh, nkv, hd, page_size = 4, 2, 32, 16
    rows = [(700, 1), (0, 5)]
    q, kv, ctx, grp = _attention_case(dtype, nh, nkv, hd, page_size, rows, spike=(0, key_pos, 3))
    dctx, dgrp = _to_dev(ctx, grp)
    got = k().paged_attention_simple(q.to(DEV), kv.to(DEV), dctx, dgrp, nh, nkv, hd, 1.0, 0)
    ref = plain_ops.paged_attention(q, kv, ctx, grp, nh, nkv, hd, 1.0, 0)
    assert (ref[0, 3 * hd:4 * hd].float() - 7.0).abs().max() < 0.1
    close(got, ref, dtype, "attention with a dominant key", scale=7.0)


@pytest.mark.parametrize("dtype", DTYPES)
def test_paged_attention_simple_window_edge(dtype):
    """The key just outside a window must not count even when it would dominate; the one
    just inside must."""
    nh, nkv, hd, page_size, window = 2, 1, 32, 16, 40
    for key_pos, inside in ((100 - 40, False), (100 - 39, True)):
        rows = [(100, 1)]
        q, kv, ctx, grp = _attention_case(dtype, nh, nkv, hd, page_size, rows, window, spike=(0, key_pos, 1))
        dctx, dgrp = _to_dev(ctx, grp)
        got = k().paged_attention_simple(q.to(DEV), kv.to(DEV), dctx, dgrp, nh, nkv, hd, 1.0, window)
        ref = plain_ops.paged_attention(q, kv, ctx, grp, nh, nkv, hd, 1.0, window)
        assert ((ref[0, hd:].float() - 7.0).abs().max() < 0.1) == inside
        close(got, ref, dtype, "window edge", scale=7.0)


def test_paged_attention_never_reads_unseen_keys():
    """Pages hold NaN wherever a key is not visible: the result must stay finite."""
    nh, nkv, hd, page_size = 4, 2, 32, 16
    rows = [(20, 3), (0, 9)]
    q, kv, ctx, grp = _attention_case(torch.float32, nh, nkv, hd, page_size, rows)
    lens = [c + ql for c, ql in rows]
    poisoned = torch.full_like(kv, float("nan"))
    for r, n in enumerate(lens):
        for j in range(n):
            p = int(grp.block_tables[r, j // page_size])
            poisoned[p, :, :, j % page_size] = kv[p, :, :, j % page_size]
    dctx, dgrp = _to_dev(ctx, grp)
    got = k().paged_attention_simple(q.to(DEV), poisoned.to(DEV), dctx, dgrp, nh, nkv, hd, hd ** -0.5, 0)
    ref = plain_ops.paged_attention(q, kv, ctx, grp, nh, nkv, hd, hd ** -0.5, 0)
    assert torch.isfinite(got).all()
    close(got, ref, torch.float32, "attention", scale=1.0)


def _full_ctx(rows, ctx, grp):
    """A device step context with the row arrays the tiled kernels read."""
    starts, at = [], 0
    for _, ql in rows:
        starts.append(at)
        at += ql
    starts.append(at)
    d, g = _to_dev(ctx, grp)
    d.row_start = torch.tensor(starts, dtype=torch.int32, device=DEV)
    d.row_ctx = torch.tensor([c for c, _ in rows], dtype=torch.int32, device=DEV)
    d.max_q_len = max(ql for _, ql in rows)
    d.max_ctx_after = max(c + ql for c, ql in rows)
    d.all_decode = all(ql == 1 for _, ql in rows)
    d.R = len(rows)
    d.n_splits = 0
    return d, g


# The tiled kernels hand the probabilities to the tensor cores in bfloat16: each p_j carries a
# relative error of 2^-9, so sum_j p_j v_j is off by at most 2^-9 * max|v| on top of the
# rounding of the result itself.
P_ROUNDING = 2.0 ** -9

TILED_SHAPES = [(4, 2, 16, 16), (6, 3, 32, 16), (5, 1, 48, 8), (8, 8, 64, 32), (32, 8, 64, 16), (12, 4, 128, 64),
                (24, 8, 128, 16), (3, 3, 80, 16), (2, 1, 256, 16), (16, 1, 96, 128),
                (12, 1, 64, 16),      # more than 8 query heads to a kv head at a head size with both decode tiles
                (6, 2, 32, 12)]       # pages of no power of two


@pytest.mark.parametrize("nh,nkv,hd,page_size", TILED_SHAPES)
@pytest.mark.parametrize("window", [0, 24, 100])
def test_tiled_prefill_attention_mixed_rows(nh, nkv, hd, page_size, window):
    """Portions of prompts with and without earlier context, single tokens, tiles that end in
    the middle of a portion, rows that span several 64-row and 64-key tiles."""
    rows = [(0, 37), (90, 1), (31, 2), (0, 1), (15, 17), (64, 1), (200, 130), (0, 64), (63, 65)]
    q, kv, ctx, grp = _attention_case(torch.bfloat16, nh, nkv, hd, page_size, rows, window)
    ref = plain_ops.paged_attention(q, kv, ctx, grp, nh, nkv, hd, hd ** -0.5, window)
    dctx, dgrp = _full_ctx(rows, ctx, grp)
    got = k().paged_attention_prefill(q.to(DEV), kv.to(DEV), dctx, dgrp, nh, nkv, hd, hd ** -0.5, window)
    assert dctx.status.tolist()[0] == 0
    close(got, ref, torch.bfloat16, "tiled prefill attention", scale=1.0, extra=P_ROUNDING * kv.abs().max().item())


@pytest.mark.parametrize("nh,nkv,hd,page_size", TILED_SHAPES + [(8, 2, 64, 16), (8, 2, 128, 16)])
@pytest.mark.parametrize("window", [0, 70])
@pytest.mark.parametrize("portion", [17, 130])
def test_mixed_step_attention_takes_two_kernels(nh, nkv, hd, page_size, window, portion):
    """A step whose first rows decode and whose last rows are portions: the dispatch hands the
    decoding rows to the split kernel and the rest to a tiled one (the tensor-memory kernel for
    the 130-token portion where it takes the sizes), into one output, and a single token among
    the portions stays with them."""
    from fastmlx_b200.engine.batch import leading_decode_rows
    rows = [(300, 1), (1000, 1), (63, 1), (0, 1), (0, portion), (90, 1), (31, 2), (200, portion)]
    q, kv, ctx, grp = _attention_case(torch.bfloat16, nh, nkv, hd, page_size, rows, window)
    ref = plain_ops.paged_attention(q, kv, ctx, grp, nh, nkv, hd, hd ** -0.5, window)
    dctx, dgrp = _full_ctx(rows, ctx, grp)
    for name, value in leading_decode_rows([ql for _, ql in rows], [c for c, _ in rows]).items():
        setattr(dctx, name, value)
    assert dctx.decode_rows == 4 and dctx.decode_max_ctx == 1001 and dctx.rest_max_q_len == portion \
        and dctx.rest_max_ctx == 200 + portion
    dctx.scratch = {}
    before = k().launch_count()
    got = k().paged_attention(q.to(DEV), kv.to(DEV), dctx, dgrp, nh, nkv, hd, hd ** -0.5, window)
    assert k().launch_count() - before == 2 and dctx.status.tolist()[0] == 0
    close(got, ref, torch.bfloat16, "mixed step attention", scale=1.0, extra=P_ROUNDING * kv.abs().max().item())


@pytest.mark.parametrize("nh,nkv,hd,page_size", TILED_SHAPES)
@pytest.mark.parametrize("window", [0, 70])
@pytest.mark.parametrize("splits", [1, 2, 5, 8, 9, 32])
def test_split_decode_attention(nh, nkv, hd, page_size, window, splits):
    rows = [(0, 1), (1, 1), (63, 1), (64, 1), (65, 1), (300, 1), (1000, 1), (127, 1)]
    q, kv, ctx, grp = _attention_case(torch.bfloat16, nh, nkv, hd, page_size, rows, window)
    ref = plain_ops.paged_attention(q, kv, ctx, grp, nh, nkv, hd, hd ** -0.5, window)
    dctx, dgrp = _full_ctx(rows, ctx, grp)
    got = k().paged_attention_decode(q.to(DEV), kv.to(DEV), dctx, dgrp, nh, nkv, hd, hd ** -0.5, window, splits=splits)
    assert dctx.status.tolist()[0] == 0
    close(got, ref, torch.bfloat16, "split decode attention", scale=1.0, extra=P_ROUNDING * kv.abs().max().item())
    # up to 8 splits are one thread-block cluster; the same through L2 and tickets, as where no cluster fits
    was = k().decode_attention_clusters(hd, False)
    try:
        again = k().paged_attention_decode(q.to(DEV), kv.to(DEV), dctx, dgrp, nh, nkv, hd, hd ** -0.5, window, splits=splits)
    finally:
        k().decode_attention_clusters(hd, was)
    assert was and dctx.status.tolist()[0] == 0
    close(again, ref, torch.bfloat16, "split decode attention through tickets", scale=1.0, extra=P_ROUNDING * kv.abs().max().item())
    if splits <= 8:
        assert torch.equal(again, got)          # both sum the splits in split order


@pytest.mark.parametrize("seed", range(24))
def test_split_decode_attention_on_random_shapes(seed):
    """Shapes drawn at random: head sizes, heads per kv head up to 16, pages of any size, rows of
    any length with and without a window, every way of splitting (one block, a cluster of up to 8,
    tickets), and the planner's own choice."""
    import random
    rng = random.Random(1000 + seed)
    hd = rng.choice([16, 32, 48, 64, 64, 80, 96, 128, 128])
    nkv = rng.choice([1, 2, 3, 8])
    rep = rng.choice([1, 2, 4, 4, 5, 8, 9, 16])
    nh = nkv * rep
    page_size = rng.choice([4, 8, 12, 16, 16, 32, 64])
    rows = [(rng.choice([0, 1, 15, 16, 17, 63, 64, 65, rng.randrange(100, 3000)]), 1) for _ in range(rng.randint(1, 6))]
    window = rng.choice([0, 0, rng.randrange(1, 200)])
    q, kv, ctx, grp = _attention_case(torch.bfloat16, nh, nkv, hd, page_size, rows, window, seed=seed)
    ref = plain_ops.paged_attention(q, kv, ctx, grp, nh, nkv, hd, hd ** -0.5, window)
    dctx, dgrp = _full_ctx(rows, ctx, grp)
    for splits in (None, 1, rng.randint(2, 8), rng.randint(9, 40)):
        got = k().paged_attention_decode(q.to(DEV), kv.to(DEV), dctx, dgrp, nh, nkv, hd, hd ** -0.5, window, splits=splits)
        assert dctx.status.tolist()[0] == 0
        close(got, ref, torch.bfloat16, f"decode attention nh={nh} nkv={nkv} hd={hd} page={page_size} window={window} "
              f"rows={rows} splits={splits}", scale=1.0, extra=P_ROUNDING * kv.abs().max().item())


@pytest.mark.parametrize("nh,nkv,hd,page_size", TILED_SHAPES)
@pytest.mark.parametrize("rot_frac,traditional", [(1.0, False), (0.5, False), (1.0, True), (0.0, False)])
@pytest.mark.parametrize("splits", [1, 3])
def test_decode_attention_rotates_and_stores_by_itself(nh, nkv, hd, page_size, rot_frac, traditional, splits):
    """The decode kernel given q, k, v as the projection left them: the same bits, in its
    output and in the cache, as the rotary kernel followed by the decode kernel."""
    rows = [(0, 1), (1, 1), (63, 1), (64, 1), (65, 1), (300, 1), (1000, 1), (127, 1)]
    _, kv, ctx, grp = _attention_case(torch.bfloat16, nh, nkv, hd, page_size, rows, 0)
    rot = int(hd * rot_frac) // 2 * 2
    inv = (10000.0 ** (-torch.arange(0, rot, 2, dtype=torch.float64) / max(rot, 1))).float().to(DEV) if rot else None
    qkv = rnd(len(rows), (nh + 2 * nkv) * hd, dtype=torch.bfloat16, seed=77).to(DEV)
    dctx, dgrp = _full_ctx(rows, ctx, grp)
    bt = grp.block_tables
    slots = torch.tensor([int(bt[r, c // page_size]) * page_size + c % page_size for r, (c, _) in enumerate(rows)],
                         dtype=torch.int64, device=DEV)
    # the two kernels
    qkv_a, kv_a = qkv.clone(), kv.to(DEV).clone()
    k().rope_kv_write(qkv_a, dctx.positions, inv, rot, traditional, slots, kv_a, nh, nkv, hd, dctx.status)
    want = k().paged_attention_decode(qkv_a, kv_a, dctx, dgrp, nh, nkv, hd, hd ** -0.5, 0, splits=splits)
    # the one
    qkv_b, kv_b = qkv.clone(), kv.to(DEV).clone()
    got = k().paged_attention_decode(qkv_b, kv_b, dctx, dgrp, nh, nkv, hd, hd ** -0.5, 0, splits=splits,
                                     rope=(inv, rot, traditional, True))
    assert dctx.status.tolist()[0] == 0
    assert torch.equal(kv_a, kv_b), "the cache holds other bits"
    assert torch.equal(got, want)
    assert torch.equal(qkv_b, qkv), "the fused kernel must leave qkv alone"
    # queries only (a layer that reads another layer's cache): the cache stays as it is
    kv_c = kv_a.clone()
    got_q = k().paged_attention_decode(qkv.clone(), kv_c, dctx, dgrp, nh, nkv, hd, hd ** -0.5, 0, splits=splits,
                                       rope=(inv, rot, traditional, False))
    assert torch.equal(kv_c, kv_a) and torch.equal(got_q, want)


TC_SHAPES = [(4, 1, 64, 16), (8, 2, 64, 16), (32, 8, 64, 16), (8, 8, 64, 32), (16, 1, 64, 128), (8, 2, 128, 16),
             (24, 24, 128, 64), (16, 2, 128, 8), (24, 8, 128, 16), (6, 2, 64, 16), (5, 1, 64, 32), (7, 1, 128, 16)]


@pytest.mark.parametrize("variant", [0, 1, 2])
@pytest.mark.parametrize("nh,nkv,hd,page_size", TC_SHAPES)
def test_tensor_memory_prefill_attention(nh, nkv, hd, page_size, variant):
    """The tcgen05 attention kernel on portions with and without earlier context, single
    tokens, rows that end inside a 128-row tile and inside a 128-key tile."""
    rows = [(0, 37), (90, 1), (31, 2), (0, 1), (15, 17), (64, 1), (200, 130), (0, 128), (127, 129), (0, 300)]
    q, kv, ctx, grp = _attention_case(torch.bfloat16, nh, nkv, hd, page_size, rows)
    ref = plain_ops.paged_attention(q, kv, ctx, grp, nh, nkv, hd, hd ** -0.5, 0)
    dctx, dgrp = _full_ctx(rows, ctx, grp)
    assert k().tc_attention_ok(nh, nkv, hd, page_size, 0)
    # variant 0: the library's choice; 1: one query tile per CTA; 2: two where the page size allows that kernel
    got = k().paged_attention_prefill_tc(q.to(DEV), kv.to(DEV), dctx, dgrp, nh, nkv, hd, hd ** -0.5, variant=variant)
    assert dctx.status.tolist()[0] == 0
    close(got, ref, torch.bfloat16, "tensor-memory attention", scale=1.0, extra=P_ROUNDING * kv.abs().max().item())


@pytest.mark.parametrize("ksplits", [2, 3, 4])
@pytest.mark.parametrize("nh,nkv,hd,page_size", [s for s in TC_SHAPES if (128 if s[2] == 64 else 64) % s[3] == 0])
def test_tensor_memory_attention_shares_keys_out(nh, nkv, hd, page_size, ksplits):
    """The keys of a pair of query tiles shared out over several CTAs and combined by a second
    kernel: rows whose keys end in the first share (the others then bring nothing), rows that
    reach into every share, a portion behind a long context, single tokens."""
    rows = [(0, 37), (1500, 130), (90, 1), (700, 2), (0, 300), (2000, 64), (64, 1)]
    q, kv, ctx, grp = _attention_case(torch.bfloat16, nh, nkv, hd, page_size, rows)
    ref = plain_ops.paged_attention(q, kv, ctx, grp, nh, nkv, hd, hd ** -0.5, 0)
    dctx, dgrp = _full_ctx(rows, ctx, grp)
    got = k().paged_attention_prefill_tc(q.to(DEV), kv.to(DEV), dctx, dgrp, nh, nkv, hd, hd ** -0.5, variant=2, ksplits=ksplits)
    assert dctx.status.tolist()[0] == 0
    close(got, ref, torch.bfloat16, f"tensor-memory attention, keys in {ksplits} shares", scale=1.0,
          extra=P_ROUNDING * kv.abs().max().item())
    # one long portion alone: the library plans the shares itself
    rows = [(3000, 200)]
    q, kv, ctx, grp = _attention_case(torch.bfloat16, nh, nkv, hd, page_size, rows, seed=3, spike=(150, 40, nh - 1))
    ref = plain_ops.paged_attention(q, kv, ctx, grp, nh, nkv, hd, hd ** -0.5, 0)
    dctx, dgrp = _full_ctx(rows, ctx, grp)
    from fastmlx_b200.kernels.lib import load
    planned = load(f"attn_hd{hd}").fmx_attn_prefill_tc_plan_splits(1, 200, 3200, nh, nkv, k().num_sms())
    assert planned > 1
    got = k().paged_attention_prefill_tc(q.to(DEV), kv.to(DEV), dctx, dgrp, nh, nkv, hd, hd ** -0.5)
    assert dctx.status.tolist()[0] == 0
    close(got, ref, torch.bfloat16, "tensor-memory attention, planned shares, a far key that stands out", scale=1.0,
          extra=P_ROUNDING * kv.abs().max().item())


@pytest.mark.parametrize("variant", [1, 2])
@pytest.mark.parametrize("key_pos", [0, 15, 16, 127, 128, 129, 255, 256, 511, 700])
def test_tensor_memory_attention_far_key_and_unseen_keys(key_pos, variant):
    """One key among 701 dominates for one head (a tile edge or a page edge that loses it shows
    at once); pages hold NaN wherever a key is out of sight."""
    nh, nkv, hd, page_size = 8, 2, 64, 16
    rows = [(636, 65), (0, 70)]
    q, kv, ctx, grp = _attention_case(torch.bfloat16, nh, nkv, hd, page_size, rows, spike=(64, key_pos, 5))
    ref = plain_ops.paged_attention(q, kv, ctx, grp, nh, nkv, hd, 1.0, 0)
    assert (ref[64, 5 * hd:6 * hd].float() - 7.0).abs().max() < 0.1
    poisoned = torch.full_like(kv, float("nan"))
    for r, (c, ql) in enumerate(rows):
        for j in range(c + ql):
            p = int(grp.block_tables[r, j // page_size])
            poisoned[p, :, :, j % page_size] = kv[p, :, :, j % page_size]
    dctx, dgrp = _full_ctx(rows, ctx, grp)
    got = k().paged_attention_prefill_tc(q.to(DEV), poisoned.to(DEV), dctx, dgrp, nh, nkv, hd, 1.0, variant=variant)
    assert torch.isfinite(got).all()
    close(got, ref, torch.bfloat16, "dominant key", scale=7.0)


def test_decode_padding_rows_read_nothing():
    """A padding row (position -1, block table of -1) gives zeros and no status code."""
    nh, nkv, hd, page_size = 8, 2, 64, 16
    rows = [(100, 1), (0, 1)]
    q, kv, ctx, grp = _attention_case(torch.bfloat16, nh, nkv, hd, page_size, rows)
    ctx.positions[1] = -1
    grp.block_tables[1] = -1
    dctx, dgrp = _full_ctx(rows, ctx, grp)
    got = k().paged_attention_decode(q.to(DEV), kv.to(DEV), dctx, dgrp, nh, nkv, hd, hd ** -0.5, 0, splits=3)
    assert dctx.status.tolist()[0] == 0 and float(got[1].abs().sum()) == 0.0 and torch.isfinite(got).all()


@pytest.mark.parametrize("kernel", ["prefill", "decode"])
@pytest.mark.parametrize("key_pos", [0, 15, 16, 63, 64, 65, 127, 128, 511, 512, 700])
def test_tiled_attention_far_key_stands_out(kernel, key_pos):
    """One key among 701 dominates for one head: a tile edge, a page edge or a split edge
    that loses it shows at once."""
    nh, nkv, hd, page_size = 8, 2, 64, 16
    rows = [(700, 1), (0, 5)] if kernel == "prefill" else [(700, 1), (4, 1)]
    q, kv, ctx, grp = _attention_case(torch.bfloat16, nh, nkv, hd, page_size, rows, spike=(0, key_pos, 5))
    ref = plain_ops.paged_attention(q, kv, ctx, grp, nh, nkv, hd, 1.0, 0)
    assert (ref[0, 5 * hd:6 * hd].float() - 7.0).abs().max() < 0.1
    dctx, dgrp = _full_ctx(rows, ctx, grp)
    if kernel == "prefill":
        got = k().paged_attention_prefill(q.to(DEV), kv.to(DEV), dctx, dgrp, nh, nkv, hd, 1.0, 0)
    else:
        got = k().paged_attention_decode(q.to(DEV), kv.to(DEV), dctx, dgrp, nh, nkv, hd, 1.0, 0, splits=4)
    close(got, ref, torch.bfloat16, "dominant key", scale=7.0)


@pytest.mark.parametrize("kernel", ["prefill", "decode"])
def test_tiled_attention_window_edge_and_unseen_keys(kernel):
    """The key just outside the window must not count, the one just inside must; and pages
    hold NaN wherever a key is out of sight."""
    nh, nkv, hd, page_size, window = 4, 1, 64, 16, 40
    for key_pos, inside in ((100 - 40, False), (100 - 39, True)):
        rows = [(100, 1), (7, 1)]
        q, kv, ctx, grp = _attention_case(torch.bfloat16, nh, nkv, hd, page_size, rows, window, spike=(0, key_pos, 1))
        ref = plain_ops.paged_attention(q, kv, ctx, grp, nh, nkv, hd, 1.0, window)
        assert ((ref[0, hd:2 * hd].float() - 7.0).abs().max() < 0.1) == inside
        poisoned = torch.full_like(kv, float("nan"))
        for r, (c, ql) in enumerate(rows):
            for j in range(max(0, c - window + 1), c + ql):
                p = int(grp.block_tables[r, j // page_size])
                poisoned[p, :, :, j % page_size] = kv[p, :, :, j % page_size]
        dctx, dgrp = _full_ctx(rows, ctx, grp)
        fn = k().paged_attention_prefill if kernel == "prefill" else k().paged_attention_decode
        got = fn(q.to(DEV), poisoned.to(DEV), dctx, dgrp, nh, nkv, hd, 1.0, window)
        assert torch.isfinite(got).all()
        close(got, ref, torch.bfloat16, "window edge", scale=7.0)


# ----------------------------------------------------------------------------- sampling
@pytest.mark.parametrize("V", [131, 320, 1000, 128256])
def test_argmax_first_index_on_ties(V):
    logits = rnd(5, V, seed=3)
    logits[1, 7] = logits[1, V - 2] = 50.0
    logits[2, :] = 0.0
    logits[3, V - 1] = 60.0
    got = k().argmax(logits.to(DEV)).cpu()
    assert got.tolist() == plain_ops.argmax(logits).tolist()
    assert got[1] == 7 and got[2] == 0 and got[3] == V - 1


@pytest.mark.parametrize("rows,V,pad", [(1, 128256, 0), (8, 128256, 0), (3, 50001, 0), (64, 32003, 1), (100, 20000, 3),
                                        (2, 8192, 0)])
def test_argmax_in_chunks(rows, V, pad):
    """Large vocabularies: a row is cut over several blocks.  Equal maxima on both sides of every
    chunk border, rows that do not start on 16 bytes (pad), a width that is no multiple of 4."""
    kk = k()
    chunks = kk.argmax_chunks(rows, V)
    assert chunks > 1
    chunk = ((V + chunks - 1) // chunks + 3) // 4 * 4
    buf = rnd(rows, V + pad, seed=11)
    logits = buf[:, :V]
    for r in range(rows):
        border = chunk * (1 + r % (chunks - 1))
        if r % 3 == 0 and border < V:
            logits[r, border - 1] = logits[r, border] = 70.0          # a tie across a border
        elif r % 3 == 1:
            logits[r, V - 1] = 70.0                                   # the ragged end
        else:
            logits[r, min(V - 1, border + 1)] = 70.0
    dev = buf.to(DEV)[:, :V]
    for _ in range(3):                                                # the tickets come back to zero
        got = kk.argmax(dev).cpu()
        assert got.tolist() == plain_ops.argmax(logits).tolist()
    assert int(kk.argmax_workspace(dev.device)[1].abs().sum()) == 0


@pytest.mark.parametrize("V", [131, 320, 5000, 128256])
def test_temperature_sampling_matches_inverse_cdf(V):
    rows = 24
    logits = rnd(rows, V, seed=5, scale=3.0)
    temps = torch.tensor([0.0, 0.7, 1.0, 1.5] * (rows // 4))
    u = torch.rand(rows, generator=torch.Generator().manual_seed(6))
    u[1], u[2] = 0.0, 0.99999994
    got = k().sample(logits.to(DEV), temps.to(DEV), u.to(DEV)).cpu()
    for r in range(rows):
        if temps[r] == 0:
            assert got[r] == int(torch.argmax(logits[r]))
            continue
        w = torch.softmax(logits[r].double() / temps[r].double(), 0)
        c = torch.cumsum(w, 0)
        i = int(got[r])
        lo, hi = (c[i - 1].item() if i > 0 else 0.0), c[i].item()
        # the chosen token's interval of the CDF holds u, up to 32-bit rounding of the running sum
        assert lo - 1e-4 <= u[r].item() <= hi + 1e-4, (r, i, lo, u[r].item(), hi)


def test_sampling_keep_mask():
    V = 300
    logits = rnd(6, V, seed=8)
    keep = torch.zeros(6, V, dtype=torch.uint8)
    keep[:, 100:110] = 1
    temps = torch.tensor([0.0, 1.0, 1.0, 2.0, 0.5, 1.0])
    u = torch.tensor([0.1, 0.0, 0.999, 0.5, 0.3, 0.7])
    got = k().sample(logits.to(DEV), temps.to(DEV), u.to(DEV), keep.to(DEV)).cpu()
    assert ((got >= 100) & (got < 110)).all()
    assert got.tolist() == plain_ops.sample(logits, temps, u, keep).tolist()


# ----------------------------------------------------------------------------- a wait that runs out
def test_a_wait_that_runs_out_leaves_a_code_and_a_usable_stream():
    """Every wait on a barrier in the tensor-core kernels is bounded.  The library `tc_expiry` is
    the product kernel's source built with a limit of 100,000 clocks and a producer that never
    brings its last block: the issuing thread and the epilogue warps wait for what never comes,
    give up, leave code 5 in the status word, wait for the products already issued, free their
    tensor memory and return.  Nothing faults and nothing is in flight; the next ordinary
    product on the same stream is right."""
    from fastmlx_b200.kernels.lib import call
    M, N, K = 256, 512, 512
    x, w = rnd(M, K, dtype=torch.bfloat16, seed=1).to(DEV), rnd(N, K, dtype=torch.bfloat16, seed=2, scale=0.1).to(DEV)
    out = torch.zeros(M, N, dtype=torch.bfloat16, device=DEV)
    st = status()
    call("tc_expiry", "fmx_gemm_tcgen05", x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(), out.stride(0),
         None, 0, M, N, K, 256, 0, 0, st.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()                               # returns: the kernel ended by itself
    code, role, block = st.tolist()[:3]
    assert code == 5 and role in (2, 3), (code, role, block)
    st2 = status()
    got = k().gemm_tcgen05(x, w, st2, bn=256)
    torch.cuda.synchronize()
    assert st2.tolist()[0] == 0
    close(got, plain_ops.linear(x.cpu(), w.cpu(), None, torch.bfloat16), torch.bfloat16, "the product after an expired wait")


# ----------------------------------------------------------------------------- the greedy head
@pytest.mark.parametrize("M", [1, 5, 8, 9, 16])
@pytest.mark.parametrize("V,K", [(256, 64), (320, 192), (131, 80), (128256, 2048), (50001, 136)])
def test_greedy_head_chooses_the_largest_logit(M, V, K):
    """The head's product with the greedy choice inside against the logits' argmax; twice in a row
    (its words go back to zero by themselves), and with ties, where the lowest index wins."""
    x = rnd(M, K, dtype=torch.bfloat16, seed=M).to(DEV)
    w = rnd(V, K, dtype=torch.bfloat16, seed=V, scale=0.05).to(DEV)
    w[V - 1] = w[3]                                          # rows 3 and V-1 give equal logits everywhere
    if V > 40:
        x[0] = (w[3].float() * 40).to(torch.bfloat16)        # ... and row 0's largest logit is that pair's
    logits = k().gemv(x, w, out_dtype=torch.float32) if V < 65536 else None
    ref = plain_ops.linear(x.cpu(), w.cpu(), None, torch.float64)
    for _ in range(2):
        ids = k().greedy_head(x, w).cpu()
        for r in range(M):
            got = int(ids[r])
            assert 0 <= got < V
            best = float(ref[r].max())
            assert float(ref[r, got]) >= best - 1e-3 * max(1.0, abs(best)), (r, got, int(ref[r].argmax()))
        if logits is not None:                               # the same sums: the same choice, the first index on ties
            assert ids.tolist() == k().argmax(logits).cpu().tolist()
        if V > 40:
            assert int(ids[0]) == 3
    best_words, ticket = k().greedy_workspace(DEV)
    assert int(ticket) == 0 and int(best_words.abs().sum()) == 0
