"""Times one kernel alone on synthetic inputs (CUDA events around a captured graph of
launches), for tuning and for profiler captures on a small case.

    python -m fastmlx_b200.kernels.microbench --kernel attn_decode --batch 8 --ctx 8192
    python -m fastmlx_b200.kernels.microbench --kernel attn_prefill --batch 1 --qlen 2048
    python -m fastmlx_b200.kernels.microbench --kernel gemv --M 8 --N 2048 --K 8192
    python -m fastmlx_b200.kernels.microbench --kernel gemm --M 2048 --N 16384 --K 2048
    python -m fastmlx_b200.kernels.microbench --kernel sample --batch 8 --N 128256
"""
from __future__ import annotations

import argparse
from types import SimpleNamespace

import torch

from .. import kernels as k

DEV = "cuda"


def _time_graph(fn, launches: int, replays: int) -> float:
    """Microseconds per call of fn, from a CUDA graph holding `launches` calls."""
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(launches):
            fn()
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(replays):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / (replays * launches) * 1e3


def _attention_inputs(a, qlen):
    B, ctx_len, nh, nkv, hd, ps = a.batch, a.ctx, a.nh, a.nkv, a.hd, a.page
    per = -(-(ctx_len + qlen) // ps)
    num_pages = B * per + 8
    kv = torch.randn(num_pages, 2, nkv, ps, hd, device=DEV, dtype=torch.bfloat16)
    bt = torch.randperm(num_pages, device=DEV)[:B * per].int().view(B, per).contiguous()
    T = B * qlen
    qkv = torch.randn(T, (nh + 2 * nkv) * hd, device=DEV, dtype=torch.bfloat16)
    pos = torch.cat([torch.arange(ctx_len, ctx_len + qlen) for _ in range(B)]).int().to(DEV)
    ctx = SimpleNamespace(positions=pos, token_row=torch.arange(B).repeat_interleave(qlen).int().to(DEV),
                          status=torch.zeros(4, dtype=torch.int32, device=DEV),
                          row_start=(torch.arange(B + 1) * qlen).int().to(DEV),
                          row_ctx=torch.full((B,), ctx_len, dtype=torch.int32, device=DEV), R=B, max_q_len=qlen,
                          max_ctx_after=ctx_len + qlen, all_decode=qlen == 1, n_splits=0, scratch={})
    return qkv, kv, ctx, SimpleNamespace(block_tables=bt)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--kernel", required=True, choices=["attn_decode", "attn_prefill", "gemv", "gemm", "sample"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--ctx", type=int, default=8192, help="tokens already in the cache")
    ap.add_argument("--qlen", type=int, default=2048, help="tokens per row (attn_prefill)")
    ap.add_argument("--nh", type=int, default=32)
    ap.add_argument("--nkv", type=int, default=8)
    ap.add_argument("--hd", type=int, default=64)
    ap.add_argument("--page", type=int, default=16)
    ap.add_argument("--splits", type=int, default=0, help="0: the engine's own choice")
    ap.add_argument("--M", type=int, default=8)
    ap.add_argument("--N", type=int, default=2048)
    ap.add_argument("--K", type=int, default=8192)
    ap.add_argument("--dual", action="store_true", help="gemv: the gate/up product with SiLU-mul")
    ap.add_argument("--resident", action="store_true", help="one weight matrix, reused (it may stay in L2)")
    ap.add_argument("--only", default="", help="time only the implementations whose name starts so")
    ap.add_argument("--launches", type=int, default=10, help="kernel launches per graph")
    ap.add_argument("--replays", type=int, default=5)
    a = ap.parse_args(argv)
    if a.kernel == "attn_decode":
        qkv, kv, ctx, grp = _attention_inputs(a, 1)
        splits = a.splits or k.decode_splits(a.batch, a.nkv, a.ctx + 1, a.hd)
        # as in a model, where every layer has a cache of its own: more K and V than L2 holds
        copies = 1 if a.resident else max(1, int(400e6 // kv.numel() // 2) + 1)
        kvs = [kv] + [torch.randn_like(kv) for _ in range(copies - 1)]
        at = [0]

        def f():
            at[0] = (at[0] + 1) % copies
            return k.paged_attention_decode(qkv, kvs[at[0]], ctx, grp, a.nh, a.nkv, a.hd, a.hd ** -0.5, 0, splits=splits)
        us = _time_graph(f, a.launches, a.replays)
        nbytes = a.batch * (a.ctx + 1) * a.nkv * a.hd * 2 * 2
        print(f"attn_decode B={a.batch} ctx={a.ctx} nh={a.nh} nkv={a.nkv} hd={a.hd} page={a.page} splits={splits}: "
              f"{us:.1f} us, {nbytes / us / 1e3:.0f} GB/s of K and V")
    elif a.kernel == "attn_prefill":
        a.ctx = a.ctx if a.ctx != 8192 else 0
        qkv, kv, ctx, grp = _attention_inputs(a, a.qlen)
        flops = 4 * a.nh * a.hd * a.batch * (a.qlen * a.ctx + a.qlen * (a.qlen + 1) / 2)
        impls = [("mma.sync", lambda: k.paged_attention_prefill(qkv, kv, ctx, grp, a.nh, a.nkv, a.hd, a.hd ** -0.5, 0))]
        if k.tc_attention_ok(a.nh, a.nkv, a.hd, a.page, 0):
            impls.append(("tcgen05, one query tile per CTA",
                          lambda: k.paged_attention_prefill_tc(qkv, kv, ctx, grp, a.nh, a.nkv, a.hd, a.hd ** -0.5, variant=1)))
            if (128 if a.hd == 64 else 64) % a.page == 0:
                impls.append(("tcgen05, two query tiles per CTA",
                              lambda: k.paged_attention_prefill_tc(qkv, kv, ctx, grp, a.nh, a.nkv, a.hd, a.hd ** -0.5, variant=2, ksplits=1)))
                for ks in (2, 4):
                    if ks * qkv.shape[0] * a.nh * (a.hd + 2) > k.ATTN_SCRATCH_FLOATS:
                        continue
                    impls.append((f"tcgen05, two query tiles per CTA, keys in {ks} shares", (lambda ks: lambda: k.paged_attention_prefill_tc(
                        qkv, kv, ctx, grp, a.nh, a.nkv, a.hd, a.hd ** -0.5, variant=2, ksplits=ks))(ks)))
                impls.append(("tcgen05, the library's choice", lambda: k.paged_attention_prefill_tc(
                    qkv, kv, ctx, grp, a.nh, a.nkv, a.hd, a.hd ** -0.5)))
        for name, f in impls:
            us = _time_graph(f, a.launches, a.replays)
            print(f"attn_prefill {name} B={a.batch} ctx={a.ctx} qlen={a.qlen} nh={a.nh} nkv={a.nkv} hd={a.hd}: {us:.1f} us, "
                  f"{flops / us / 1e6:.0f} TFLOP/s")
        print("status", ctx.status.tolist())
    elif a.kernel == "sample":
        # filters and draw over --batch rows of --N logits: the reference's default (top_p 0.95), top_p with top_k, none
        rows, V = a.batch, a.N
        logits = torch.randn(rows, V, device=DEV) * 2
        f = lambda v, dt=torch.float32: torch.full((rows,), v, dtype=dt, device=DEV)
        T, u = f(1.0), torch.rand(rows, device=DEV)
        cases = [("no filter", ()), ("top_p 0.95", (f(0.95), f(0.0), f(0, torch.int32), f(1, torch.int32))),
                 ("top_p 0.9, top_k 50", (f(0.9), f(0.0), f(50, torch.int32), f(1, torch.int32)))]
        for name, args in cases:
            if not name.startswith(a.only):
                continue
            if k.filter_sample_takes(V):
                us = _time_graph(lambda: k.filter_sample(logits, T, u, *args), a.launches, a.replays)
                print(f"sample rows={rows} V={V} {name}, one kernel on a cluster per row: {us:.1f} us")
            us = _time_graph(lambda: k.sample(logits, T, u, k.filter_mask(logits, *args) if args else None), a.launches, a.replays)
            print(f"sample rows={rows} V={V} {name}, filter kernel then sampling kernel: {us:.1f} us")
    elif a.kernel == "gemm":
        copies = 1 if a.resident else max(1, int(300e6 // (a.N * a.K * 2)) + 1)        # more weight than L2 holds
        ws = [torch.randn(a.N, a.K, device=DEV, dtype=torch.bfloat16) * 0.02 for _ in range(copies)]
        x = torch.randn(a.M, a.K, device=DEV, dtype=torch.bfloat16)
        st = torch.zeros(4, dtype=torch.int32, device=DEV)
        flops = 2.0 * a.M * a.N * a.K
        at = [0]

        def rotating(fn):
            def f():
                at[0] = (at[0] + 1) % copies
                return fn(ws[at[0]])
            return f
        impls = [("cublas", lambda w: torch.mm(x, w.t())),
                 ("tcgen05 bn128", lambda w: k.gemm_tcgen05(x, w, st, bn=128)),
                 ("tcgen05 bn256", lambda w: k.gemm_tcgen05(x, w, st, bn=256))]
        for name, fn in impls:
            if not name.startswith(a.only):
                continue
            us = _time_graph(rotating(fn), a.launches, a.replays)
            print(f"gemm M={a.M} N={a.N} K={a.K} {name}: {us:.1f} us, {flops / us / 1e6:.0f} TFLOP/s")
        print("status", st.tolist())
    else:
        copies = 1 if a.resident else max(1, int(300e6 // (a.N * a.K * 2)) + 1)        # more weight than L2 holds
        ws = [torch.randn(a.N, a.K, device=DEV, dtype=torch.bfloat16) * 0.02 for _ in range(copies)]
        x = torch.randn(a.M, a.K, device=DEV, dtype=torch.bfloat16)
        st = torch.zeros(4, dtype=torch.int32, device=DEV)
        k.set_status_word(x.device, st)
        at = [0]

        def rotating(fn):
            def f():
                at[0] = (at[0] + 1) % copies
                return fn(ws[at[0]])
            return f
        impls = [("cublas", lambda w: torch.mm(x, w.t()))]
        if a.M <= 16:
            impls.append(("gemv 8 features", lambda w: k.gemv(x, w, wide=8, warps=8)))
            impls.append(("gemv 16 features", lambda w: k.gemv(x, w, wide=16, warps=8)))
            impls.append(("gemv 32 features", lambda w: k.gemv(x, w, wide=32, warps=8)))
            impls.append(("gemv 8 features, 16 warps", lambda w: k.gemv(x, w, wide=8, warps=16)))
            impls.append(("gemv 16 features, 16 warps", lambda w: k.gemv(x, w, wide=16, warps=16)))
        if a.dual:                      # N rows of gate and up in blocks of 128, SiLU-mul in the epilogue
            impls = [(f"gemv gate/up {wd} features", (lambda wd: lambda w: k.gemv(x, w, block=128, wide=wd))(wd))
                     for wd in (8, 16, 32) if a.M <= 16]
            impls.append(("library product, then SiLU-mul", lambda w: k.silu_mul(torch.mm(x, w.t()), 128)))
        for name, fn in impls:
            if not name.startswith(a.only):
                continue
            us = _time_graph(rotating(fn), a.launches, a.replays)
            print(f"gemv M={a.M} N={a.N} K={a.K} {name}: {us:.1f} us, {a.N * a.K * 2 / us / 1e3:.0f} GB/s of weights")
        print("status", st.tolist())
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
