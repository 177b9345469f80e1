"""The compiled batch layout (csrc/host/step_executor.cu, `fmx_exec_layout`) against the Python one
(`engine/batch.py:build_context`) without a GPU: the library is host code, and given no device buffer
it leaves the description's pointers pointing into the host buffer it filled."""
import ctypes
import random

import numpy as np
import pytest
import torch


def _host_lib():
    from fastmlx_b200.csrc import build
    from fastmlx_b200.engine import native as nat
    try:
        build.find_nvcc()
    except build.BuildError:
        pytest.skip("nvcc is not installed: the host library cannot be built")
    return nat, nat.host_library()


@pytest.mark.parametrize("seed", [1, 2, 3])
def test_native_layout_matches_build_context_on_the_cpu(seed):
    from fastmlx_b200.cache import CacheManager
    from fastmlx_b200.engine.batch import StepEntry, build_context
    from fastmlx_b200.parts import PagedKVSpec
    nat, lib = _host_lib()
    rng = random.Random(seed)
    ps = rng.choice([4, 8, 16])
    needs = [(PagedKVSpec(2, 16, 0), None, None), (PagedKVSpec(1, 32, 3 * ps + 1), None, None)]
    m = CacheManager(needs, page_size=ps, num_pages=400, max_requests=12, dtype=torch.float32, allocate=False)
    status = torch.zeros(4, dtype=torch.int32)
    live = {}
    compared = 0
    for step in range(40):
        while len(live) < 8 and rng.random() < 0.6:
            rid = f"r{step}-{len(live)}"
            live[rid] = m.add_request(rid)
        if not live:
            continue
        entries = []
        for rid in rng.sample(sorted(live), rng.randint(1, len(live))):
            q = 1 if rng.random() < 0.5 else rng.randint(2, 3 * ps + 5)
            entries.append(StepEntry(live[rid], [rng.randrange(1000) for _ in range(q)],
                                     sorted(rng.sample(range(q), rng.randint(0, min(q, 3))))))
            m.reserve(live[rid], q)
        one_each = all(len(e.tokens) == 1 for e in entries)
        pad_rows = rng.choice([0, 8, 16]) if one_each else 0
        pad_blocks = rng.choice([0, 16, 64])
        ctx = build_context(entries, m, None, status, pad_rows=pad_rows, pad_blocks=pad_blocks)
        R = len(entries)
        want, off = [], 0
        for e in entries:
            want += [off + w for w in e.want]
            off += len(e.tokens)
        flat = np.array([len(e.tokens) for e in entries] + [e.request.length for e in entries] + [e.request.slot for e in entries]
                        + want + [t for e in entries for t in e.tokens], dtype=np.int32)
        inp = nat.FmxBatchIn()
        base = flat.ctypes.data
        inp.R, inp.n_want = R, len(want)
        inp.q_lens, inp.ctx_lens, inp.slots = base, base + 4 * R, base + 8 * R
        inp.want, inp.tokens = base + 12 * R, base + 12 * R + 4 * len(want)
        inp.pad_rows, inp.pad_blocks, inp.page_size, inp.n_groups = pad_rows, pad_blocks, ps, 2
        for g, mir in enumerate(m.table_mirror):
            inp.mirror[g], inp.mirror_cols[g] = mir.ctypes.data, mir.shape[1]
        ints = lib.fmx_exec_layout_ints(ctypes.byref(inp))
        assert ints > 0 and ints % 4 == 0
        host = np.zeros(ints, dtype=np.int32)
        d = nat.FmxStepDesc()
        assert lib.fmx_exec_layout(ctypes.byref(inp), host.ctypes.data, None, ints, ctypes.byref(d), None) == 0, \
            lib.fmx_last_error().decode()

        def arr(ptr, n, dtype=np.int32):
            o = (ptr - host.ctypes.data) // 4
            return host[o: o + n * (2 if dtype == np.int64 else 1)].view(dtype)
        assert (d.T, d.R, d.n_want, d.max_q_len, d.max_ctx_after, d.all_decode) == \
            (ctx.T, ctx.R, len(want), ctx.max_q_len, ctx.max_ctx_after, int(ctx.all_decode))
        assert (d.decode_rows, d.decode_max_ctx, d.rest_max_q_len, d.rest_max_ctx) == \
            (ctx.decode_rows, ctx.decode_max_ctx, ctx.rest_max_q_len, ctx.rest_max_ctx)
        for name, n in (("tokens", d.T), ("positions", d.T), ("token_row", d.T), ("row_start", d.R + 1), ("row_ctx", d.R),
                        ("row_slot", d.R)):
            assert np.array_equal(arr(getattr(d, name), n), getattr(ctx, name).numpy()), (step, name)
        if want:
            assert np.array_equal(arr(d.want, len(want)), ctx.logit_rows.numpy())
        for g in range(2):
            bt = ctx.groups[g].block_tables.numpy()
            assert d.bt_stride[g] == bt.shape[1]
            assert np.array_equal(arr(d.block_tables[g], bt.size).reshape(bt.shape), bt), (step, g)
            assert np.array_equal(arr(d.slot_mapping[g], d.T, np.int64), ctx.groups[g].slot_mapping.numpy()), (step, g)
        compared += 1
        for e in entries:
            m.commit(e.request)
        m.check()
        for rid in [r for r in sorted(live) if rng.random() < 0.15]:
            m.free(rid)
            del live[rid]
    assert compared > 20


def test_native_layout_refuses_what_it_cannot_lay_out():
    nat, lib = _host_lib()
    flat = np.array([0, 5, 0, 1], dtype=np.int32)            # an entry that brings no token
    inp = nat.FmxBatchIn()
    inp.R, inp.n_want = 1, 0
    inp.q_lens, inp.ctx_lens, inp.slots, inp.want, inp.tokens = (flat.ctypes.data + 4 * i for i in (0, 1, 2, 3, 3))
    inp.page_size, inp.n_groups = 16, 0
    assert lib.fmx_exec_layout_ints(ctypes.byref(inp)) < 0
    assert b"brings 0 tokens" in lib.fmx_last_error()
