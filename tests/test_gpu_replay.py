"""Replay on the GPU: the same requests whole, with the tail decoded token by token, in
portions of changing size, and mixed with other requests over a pool so small that pages
are used again; in 32-bit and in bfloat16; against the plain model."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_llama
import tiny
import traces

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# Largest |difference| allowed, as a fraction of the largest |logit| of the reference.
# 32-bit: sums of a few hundred terms in float32 against float64.  bfloat16: against the
# plain model rounding to bfloat16 at the same places; what is left are values that land on
# the other side of a rounding boundary (2^-8 relative each) and what they stir up later.
TOL = {"float32": 1e-5, "bfloat16": 2e-2}

CASES = {
    "A": dict(lens=[7, 13, 29, 40, 64, 65, 3, 100, 90, 77, 50], page=16, max_tokens=512),
    "B": dict(lens=[1, 17, 64, 100, 200, 33, 2, 130, 150, 61], page=16, max_tokens=768),
    "C": dict(lens=[5, 33, 70, 128, 31, 100, 60], page=32, max_tokens=448),
}


def _prompts(name):
    cfg = tiny.CONFIGS[name]
    return {f"r{i}": tiny.rand_tokens(n, cfg["vocab_size"], 100 + i) for i, n in enumerate(CASES[name]["lens"])}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("models")
    out = {}
    for name, cfg in tiny.CONFIGS.items():
        d = tiny.make_model_dir(root, cfg, seed=11)
        W = tiny.load_plain_weights(d)
        prompts = _prompts(name)
        ref = {"float32": {r: plain_llama.forward(cfg, W, t) for r, t in prompts.items()},
               "bfloat16": {r: plain_llama.forward(cfg, W, t, round_to=torch.bfloat16) for r, t in prompts.items()}}
        out[name] = (d, prompts, ref)
    return out


def _run(model_dir, dtype, steps, max_tokens, page, native=True):
    from fastmlx_b200.engine.replay import Replayer
    rp = Replayer(model_dir, dtype, max_tokens, page_size=page, native=native)
    assert (rp.step_fn.native is not None) == native
    outs = []
    for st in steps:
        outs.append(rp.step(st))
        rp.manager.check()
    assert not rp.manager.requests and all(g.pool.used_pages == 0 for g in rp.manager.groups)
    return outs, rp


def _compare(steps, outs, prompts, ref, tol):
    rows = traces.collect(steps, outs)
    worst = 0.0
    for rid, toks in prompts.items():
        assert sorted(rows[rid]) == list(range(len(toks)))
        got = torch.from_numpy(np.stack([rows[rid][i] for i in range(len(toks))])).double()
        scale = ref[rid].abs().max().item()
        err = (got - ref[rid]).abs().max(dim=1).values / scale
        first_bad = torch.nonzero(err > tol)
        assert first_bad.numel() == 0, (f"request {rid}: first wrong position {int(first_bad[0])} of {len(toks)}, "
                                        f"error {err[int(first_bad[0])].item():.3e} (allowed {tol:.1e})")
        worst = max(worst, err.max().item())
    return worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
@pytest.mark.parametrize("cut", ["whole", "tail", "portions", "mixed"])
@pytest.mark.parametrize("native", [True, False], ids=["native", "python"])
def test_replay(models, name, dtype, cut, native):
    """native: the step's host work in the compiled executor; python: through `Model.forward`."""
    d, prompts, ref = models[name]
    case = CASES[name]
    steps = {"whole": traces.whole, "tail": traces.tail_decoded, "portions": traces.portions,
             "mixed": traces.mixed}[cut](prompts)
    outs, rp = _run(d, dtype, steps, case["max_tokens"], case["page"], native)
    _compare(steps, outs, prompts, ref[dtype], TOL[dtype])
    if cut == "mixed":
        total_pages = sum(-(-len(t) // case["page"]) for t in prompts.values())
        assert total_pages > rp.manager.groups[0].pool.num_pages, "the pool is too large for pages to be used again"


@pytest.mark.parametrize("name", ["A", "B"])
def test_cuts_agree_in_32_bit_to_rounding(models, name):
    """The logits at a position do not depend on the cut, far below the tolerance against
    the plain model: the 32-bit kernels sum in an order that the cut does not change."""
    d, prompts, ref = models[name]
    case = CASES[name]
    base_steps = traces.whole(prompts)
    base = traces.collect(base_steps, _run(d, "float32", base_steps, case["max_tokens"], case["page"])[0])
    for cut in (traces.tail_decoded, traces.portions, traces.mixed):
        steps = cut(prompts)
        rows = traces.collect(steps, _run(d, "float32", steps, case["max_tokens"], case["page"])[0])
        for rid in prompts:
            for i, row in rows[rid].items():
                assert np.array_equal(row, base[rid][i]), (cut.__name__, rid, i, np.abs(row - base[rid][i]).max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(models, tmp_path, dtype):
    """bin/trace_run as a user runs it: JSON lines in, `done <step>` lines out, .f32 files."""
    d, prompts, ref = models["B"]
    sub = {r: prompts[r] for r in ("r1", "r2", "r5", "r6")}
    steps = traces.mixed(sub)
    out = tmp_path / "out"
    proc = subprocess.Popen([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", dtype,
                             "--out", str(out), "--max-tokens", "256"], stdin=subprocess.PIPE, stdout=subprocess.PIPE,
                            text=True)
    outs = []
    for st in steps:
        proc.stdin.write(json.dumps(st) + "\n")
        proc.stdin.flush()
        assert proc.stdout.readline().strip() == f"done {st['step']}"
        f = out / f"{st['step']}.f32"
        outs.append(np.fromfile(f, dtype="<f4").reshape(-1, tiny.TINY_B["vocab_size"]) if f.exists() else None)
    proc.stdin.close()
    assert proc.wait(timeout=60) == 0
    _compare(steps, outs, sub, ref[dtype], TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(models, dtype):
    """Three tokens of prompt, then 250 tokens one by one, across many page edges."""
    d, _, _ = models["B"]
    cfg = tiny.TINY_B
    toks = tiny.rand_tokens(253, cfg["vocab_size"], 77)
    W = tiny.load_plain_weights(d)
    ref = plain_llama.forward(cfg, W, toks, round_to=torch.bfloat16 if dtype == "bfloat16" else None)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": toks[:3], "want": [0, 1, 2]}], "end": []}]
    steps += [{"step": i - 2, "entries": [{"id": "x", "tokens": [toks[i]], "want": [0]}], "end": []} for i in range(3, 253)]
    steps[-1]["end"] = ["x"]
    outs, _ = _run(d, dtype, steps, 256, 16)
    _compare(steps, outs, {"x": toks}, {"x": ref}, TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_runs_past_max_position_embeddings(models, dtype):
    """Replay feeds what the trace says: a sequence longer than the configuration's
    max_position_embeddings is run (rotary positions have no table to run out of); serving
    refuses such a request in the scheduler instead."""
    d, _, _ = models["A"]
    cfg = tiny.TINY_A
    n = cfg["max_position_embeddings"] + 40
    toks = tiny.rand_tokens(n, cfg["vocab_size"], 78)
    W = tiny.load_plain_weights(d)
    ref = plain_llama.forward(cfg, W, toks, round_to=torch.bfloat16 if dtype == "bfloat16" else None)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": toks[:n - 20], "want": list(range(n - 20))}], "end": []}]
    steps += [{"step": i - (n - 21), "entries": [{"id": "x", "tokens": [toks[i]], "want": [0]}], "end": []} for i in range(n - 20, n)]
    steps[-1]["end"] = ["x"]
    outs, _ = _run(d, dtype, steps, 256, 16)
    _compare(steps, outs, {"x": toks}, {"x": ref}, TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_first_tokens(models, name, dtype):
    """Sequences of one and two tokens, and a first step of a single token."""
    d, _, _ = models[name]
    cfg = tiny.CONFIGS[name]
    W = tiny.load_plain_weights(d)
    prompts = {"one": tiny.rand_tokens(1, cfg["vocab_size"], 5), "two": tiny.rand_tokens(2, cfg["vocab_size"], 6),
               "three": tiny.rand_tokens(3, cfg["vocab_size"], 7)}
    ref = {r: plain_llama.forward(cfg, W, t, round_to=torch.bfloat16 if dtype == "bfloat16" else None) for r, t in prompts.items()}
    steps = traces.tail_decoded(prompts, tail=2)
    outs, _ = _run(d, dtype, steps, 256, 16)
    _compare(steps, outs, prompts, ref, TOL[dtype])


@pytest.mark.parametrize("name", ["A", "B"])
def test_weights_stored_in_32_bit_under_bfloat16(tmp_path, name):
    """A folder whose tensors are all float32, run with bfloat16 activations: the tensors stay
    32-bit (products take 32-bit weights), activations and cache are bfloat16."""
    cfg = tiny.CONFIGS[name]
    d = tiny.make_model_dir(tmp_path, cfg, seed=17, dtype=torch.float32)
    W = tiny.load_plain_weights(d)
    assert all(t.dtype == torch.float32 for t in W.values())
    prompts = {"p": tiny.rand_tokens(70, cfg["vocab_size"], 3), "q": tiny.rand_tokens(9, cfg["vocab_size"], 4)}
    ref = {r: plain_llama.forward(cfg, W, t, round_to=torch.bfloat16) for r, t in prompts.items()}
    for cut in (traces.whole, traces.mixed):
        steps = cut(prompts)
        outs, rp = _run(d, "bfloat16", steps, 256, 16)
        assert rp.model.layers[0].mixer.qkv.weight.dtype == torch.float32
        _compare(steps, outs, prompts, ref, TOL["bfloat16"])
