"""The native step executor (csrc/host/step_executor.cu) against the Python path it stands for
and against the plain model: the same parts, the same kernels, the same choices, so in 32-bit
the logits are equal to the bit; in bfloat16 they are equal wherever both paths take this
package's kernels and within rounding where a library product's algorithm may differ."""
import numpy as np
import pytest
import torch

import plain_llama
import tiny
import traces

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    root = tmp_path_factory.mktemp("models")
    return {n: tiny.make_model_dir(root, c, seed=13) for n, c in tiny.CONFIGS.items()}


def _replay(d, dtype, steps, native, page=16, max_tokens=768):
    from fastmlx_b200.engine.replay import Replayer
    rp = Replayer(d, dtype, max_tokens, page_size=page, native=native)
    assert (rp.step_fn.native is not None) == native
    outs = []
    for s in steps:
        outs.append(rp.step(s))
        rp.manager.check()
    return outs, rp


@pytest.mark.parametrize("name", ["A", "B", "C"])
@pytest.mark.parametrize("cut", ["portions", "mixed"])
def test_native_and_python_paths_agree_to_the_bit_in_32_bit(dirs, name, cut):
    cfg = tiny.CONFIGS[name]
    prompts = {f"r{i}": tiny.rand_tokens(n, cfg["vocab_size"], 40 + i) for i, n in enumerate([7, 64, 100, 33, 2, 130, 61])}
    steps = {"portions": traces.portions, "mixed": traces.mixed}[cut](prompts)
    a, rp = _replay(dirs[name], "float32", steps, True)
    b, _ = _replay(dirs[name], "float32", steps, False)
    assert rp.step_fn.native.lib.fmx_exec_launches(rp.step_fn.native.handle) > 0
    for x, y in zip(a, b):
        assert (x is None) == (y is None)
        if x is not None:
            assert np.array_equal(x, y)


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_native_path_in_bfloat16_against_the_plain_model_and_the_python_path(dirs, name):
    cfg = tiny.CONFIGS[name]
    W = tiny.load_plain_weights(dirs[name])
    prompts = {f"r{i}": tiny.rand_tokens(n, cfg["vocab_size"], 70 + i) for i, n in enumerate([7, 64, 100, 33, 2, 130, 61])}
    steps = traces.mixed(prompts)
    a, _ = _replay(dirs[name], "bfloat16", steps, True)
    b, _ = _replay(dirs[name], "bfloat16", steps, False)
    rows_a, rows_b = traces.collect(steps, a), traces.collect(steps, b)
    for rid, toks in prompts.items():
        ref = plain_llama.forward(cfg, W, toks, round_to=torch.bfloat16)
        scale = ref.abs().max().item()
        for pos in range(len(toks)):
            assert np.abs(rows_a[rid][pos] - ref[pos].numpy()).max() / scale < 2e-2, (rid, pos)
            assert np.abs(rows_a[rid][pos] - rows_b[rid][pos]).max() / scale < 1e-2, (rid, pos)


def test_generation_is_the_same_with_and_without_the_native_executor(dirs):
    """Scheduler, graphs and one step ahead over the native executor (whose captured decode steps
    run its program too) and over the Python path: the same tokens in 32-bit."""
    from fastmlx_b200 import Engine, SamplingParams
    cfg = tiny.TINY_B
    prompts = [tiny.rand_tokens(n, cfg["vocab_size"], 90 + n) for n in (5, 33, 70, 12, 150)]
    sps = [SamplingParams(max_tokens=20, temperature=0.0 if i % 2 else 0.8, seed=5 + i) for i in range(5)]
    got = {}
    for native in (True, False):
        eng = Engine(dirs["B"], dtype="float32", block_size=16, max_cache_tokens=2048, max_concurrent_requests=4,
                     prefill_chunk=32, native_executor=native)
        assert eng.stats()["native_executor"] == native
        got[native] = [o.output_token_ids for o in eng.generate(prompts, sps)]
        assert eng.stats()["graph_replays"] > 0 and eng.stats()["pages_used"] == 0
    assert got[True] == got[False]


def test_a_model_with_a_python_part_stays_on_the_python_path(tmp_path):
    """A mixer defined outside the package has no `emit`: the step function keeps `Model.forward`."""
    from fastmlx_b200 import registry, write_random_model
    from fastmlx_b200.engine.replay import Replayer
    from test_gpu_parts import make_toy
    ToyCfg, build = make_toy()
    registry.register(["toy_decay_n"], ToyCfg.from_dict, build, replace=True)
    try:
        d = write_random_model(str(tmp_path / "toy"), {"model_type": "toy_decay_n", "vocab_size": 77, "width": 40, "decay": 0.9}, seed=4)
        rp = Replayer(d, "float32", 256, page_size=8)
        assert rp.step_fn.native is None
        out = rp.step({"step": 0, "entries": [{"id": "a", "tokens": [1, 2, 3], "want": [2]}], "end": ["a"]})
        assert out.shape == (1, 77)
    finally:
        registry.unregister(["toy_decay_n"])


def test_the_native_layout_is_the_python_layout():
    """`fmx_exec_layout` against `build_context` on the same entries: every array of the packed
    description, padding rows and a windowed group's -1 holes included."""
    import ctypes
    from fastmlx_b200.cache import CacheManager
    from fastmlx_b200.engine import native as nat
    from fastmlx_b200.engine.batch import StepEntry, build_context
    from fastmlx_b200.parts import PagedKVSpec
    needs = [(PagedKVSpec(2, 16, 0), None, None), (PagedKVSpec(2, 16, 9), None, None)]
    m = CacheManager(needs, page_size=8, num_pages=64, max_requests=6, dtype=torch.float32, device="cuda")
    reqs = [m.add_request(i) for i in range(4)]
    for r, n in zip(reqs, (37, 5, 0, 20)):
        if n:
            m.reserve(r, n)
            m.commit(r)
    entries = [StepEntry(reqs[0], [3], [0]), StepEntry(reqs[1], [4, 5, 6, 7, 8], [1, 4]), StepEntry(reqs[2], list(range(11)), []),
               StepEntry(reqs[3], [9, 9], [1])]
    for e in entries:
        m.reserve(e.request, len(e.tokens))
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    for pad_rows, pad_blocks in ((0, 0), (8, 16)):
        ctx = build_context(entries, m, "cuda", status, pad_rows=pad_rows, pad_blocks=pad_blocks)
        lib = nat.host_library()
        flat = np.array([len(e.tokens) for e in entries] + [e.request.length for e in entries] + [e.request.slot for e in entries]
                        + [0, 2, 5, 18] + [t for e in entries for t in e.tokens], dtype=np.int32)
        inp = nat.FmxBatchIn()
        R = len(entries)
        base = flat.ctypes.data
        inp.R, inp.n_want = R, 4
        inp.q_lens, inp.ctx_lens, inp.slots, inp.want, inp.tokens = base, base + 4 * R, base + 8 * R, base + 12 * R, base + 12 * R + 16
        inp.pad_rows, inp.pad_blocks, inp.page_size, inp.n_groups = pad_rows, pad_blocks, 8, 2
        for g, mir in enumerate(m.table_mirror):
            inp.mirror[g], inp.mirror_cols[g] = mir.ctypes.data, mir.shape[1]
        ints = lib.fmx_exec_layout_ints(ctypes.byref(inp))
        host = torch.zeros(ints, dtype=torch.int32).pin_memory()
        dev = torch.zeros(ints, dtype=torch.int32, device="cuda")
        d = nat.FmxStepDesc()
        assert lib.fmx_exec_layout(ctypes.byref(inp), host.data_ptr(), dev.data_ptr(), ints, ctypes.byref(d),
                                   torch.cuda.current_stream().cuda_stream) == 0
        torch.cuda.synchronize()
        assert (d.T, d.R, d.n_want, d.max_q_len, d.max_ctx_after, d.all_decode) == \
            (ctx.T, ctx.R, 4, ctx.max_q_len, ctx.max_ctx_after, int(ctx.all_decode))
        assert (d.decode_rows, d.decode_max_ctx, d.rest_max_q_len, d.rest_max_ctx) == \
            (ctx.decode_rows, ctx.decode_max_ctx, ctx.rest_max_q_len, ctx.rest_max_ctx)

        def arr(ptr, n, dtype=torch.int32):
            off = (ptr - dev.data_ptr()) // 4
            t = dev[off: off + n * (2 if dtype == torch.int64 else 1)]
            return t.view(dtype).cpu()
        assert torch.equal(arr(d.tokens, d.T), ctx.tokens.cpu())
        assert torch.equal(arr(d.positions, d.T), ctx.positions.cpu())
        assert torch.equal(arr(d.token_row, d.T), ctx.token_row.cpu())
        assert torch.equal(arr(d.row_start, d.R + 1), ctx.row_start.cpu())
        assert torch.equal(arr(d.row_ctx, d.R), ctx.row_ctx.cpu())
        assert torch.equal(arr(d.row_slot, d.R), ctx.row_slot.cpu())
        assert torch.equal(arr(d.want, 4), ctx.logit_rows.cpu())
        for g in range(2):
            bt = ctx.groups[g].block_tables.cpu()
            assert d.bt_stride[g] == bt.shape[1]
            assert torch.equal(arr(d.block_tables[g], bt.numel()).view(bt.shape), bt)
            assert torch.equal(arr(d.slot_mapping[g], d.T, torch.int64), ctx.groups[g].slot_mapping.cpu())


@pytest.mark.parametrize("seed", [1, 2, 3, 4])
def test_the_native_layout_is_the_python_layout_on_random_steps(seed):
    """Random live requests in two cache groups (one with a window, so its tables have -1 holes),
    random mixes of portions and single tokens, random padding: `fmx_exec_layout` and
    `build_context` describe every step alike."""
    import ctypes
    import random
    from fastmlx_b200.cache import CacheManager
    from fastmlx_b200.engine import native as nat
    from fastmlx_b200.engine.batch import StepEntry, build_context
    from fastmlx_b200.parts import PagedKVSpec
    rng = random.Random(seed)
    ps = rng.choice([4, 8, 16])
    needs = [(PagedKVSpec(2, 16, 0), None, None), (PagedKVSpec(1, 32, 3 * ps + 1), None, None)]
    m = CacheManager(needs, page_size=ps, num_pages=400, max_requests=12, dtype=torch.float32, device="cuda")
    lib = nat.host_library()
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    live = {}
    for step in range(30):
        while len(live) < 8 and rng.random() < 0.6:
            rid = f"r{step}-{len(live)}-{rng.random()}"
            live[rid] = m.add_request(rid)
        if not live:
            continue
        chosen = rng.sample(sorted(live), rng.randint(1, len(live)))
        entries = []
        for rid in chosen:
            q = 1 if rng.random() < 0.5 else rng.randint(2, 3 * ps + 5)
            toks = [rng.randrange(1000) for _ in range(q)]
            entries.append(StepEntry(live[rid], toks, sorted(rng.sample(range(q), rng.randint(0, min(q, 3))))))
            m.reserve(live[rid], q)
        pad_rows = rng.choice([0, 0, 8, 16])
        pad_blocks = rng.choice([0, 0, 16, 64])
        if pad_rows and any(len(e.tokens) != 1 for e in entries):
            pad_rows = 0                                    # the Python layout pads one-token steps only
        ctx = build_context(entries, m, "cuda", status, pad_rows=pad_rows, pad_blocks=pad_blocks)
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
        host = torch.zeros(ints, dtype=torch.int32).pin_memory()
        dev = torch.zeros(ints, dtype=torch.int32, device="cuda")
        d = nat.FmxStepDesc()
        assert lib.fmx_exec_layout(ctypes.byref(inp), host.data_ptr(), dev.data_ptr(), ints, ctypes.byref(d),
                                   torch.cuda.current_stream().cuda_stream) == 0
        torch.cuda.synchronize()

        def arr(ptr, n, dtype=torch.int32):
            o = (ptr - dev.data_ptr()) // 4
            return dev[o: o + n * (2 if dtype == torch.int64 else 1)].view(dtype).cpu()
        assert (d.T, d.R, d.max_q_len, d.max_ctx_after, d.all_decode) == (ctx.T, ctx.R, ctx.max_q_len, ctx.max_ctx_after, int(ctx.all_decode))
        assert (d.decode_rows, d.decode_max_ctx, d.rest_max_q_len, d.rest_max_ctx) == \
            (ctx.decode_rows, ctx.decode_max_ctx, ctx.rest_max_q_len, ctx.rest_max_ctx)
        for name, n in (("tokens", d.T), ("positions", d.T), ("token_row", d.T), ("row_start", d.R + 1), ("row_ctx", d.R),
                        ("row_slot", d.R)):
            assert torch.equal(arr(getattr(d, name), n), getattr(ctx, name).cpu()), (step, name)
        if want:
            assert torch.equal(arr(d.want, len(want)), ctx.logit_rows.cpu())
        for g in range(2):
            bt = ctx.groups[g].block_tables.cpu()
            assert torch.equal(arr(d.block_tables[g], bt.numel()).view(bt.shape), bt), (step, g)
            assert torch.equal(arr(d.slot_mapping[g], d.T, torch.int64), ctx.groups[g].slot_mapping.cpu()), (step, g)
        for e in entries:
            m.commit(e.request)
        m.check()
        for rid in [r for r in sorted(live) if rng.random() < 0.15]:
            m.free(rid)
            del live[rid]
