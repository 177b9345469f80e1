"""Generation through the Python entry point and the command line, on the GPU, against the
plain model; what happens when pages run out; sampling with a fixed seed."""
import json
import os
import subprocess
import sys

import pytest
import torch

import plain_llama
import tiny

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    root = tmp_path_factory.mktemp("models")
    return {n: tiny.make_model_dir(root, c, seed=21) for n, c in tiny.CONFIGS.items()}


def _plain_greedy_with_margins(cfg, W, prompt, n, round_to):
    """Tokens of the plain model, and for each the gap between its two best logits."""
    seq, margins = list(prompt), []
    for _ in range(n):
        row = plain_llama.forward(cfg, W, seq, round_to)[-1]
        top = torch.topk(row, 2).values
        margins.append((top[0] - top[1]).item() / row.abs().max().item())
        seq.append(int(torch.argmax(row)))
    return seq[len(prompt):], margins


def _agree(got, want, margins, slack):
    """Equal token by token; where the plain model's two best logits are closer than the
    dtype's tolerance either may win, and the sequences part ways legitimately."""
    for i, (g, w) in enumerate(zip(got, want)):
        if g != w:
            assert margins[i] < slack, f"token {i}: engine {g}, plain {w}, margin {margins[i]:.2e}"
            return
    assert len(got) == len(want)


@pytest.mark.parametrize("dtype,slack", [("float32", 1e-5), ("bfloat16", 2e-2)])
@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_generation_matches_plain(dirs, dtype, slack, graphs):
    from fastmlx_b200 import Engine, SamplingParams
    cfg = tiny.TINY_A
    W = tiny.load_plain_weights(dirs["A"])
    prompts = [tiny.rand_tokens(n, cfg["vocab_size"], 40 + n) for n in (7, 13, 29)]
    eng = Engine(dirs["A"], dtype=dtype, block_size=16, max_cache_tokens=512, max_concurrent_requests=4,
                 cuda_graphs=graphs)
    outs = eng.generate(prompts, SamplingParams(max_tokens=16, temperature=0.0))
    rt = torch.bfloat16 if dtype == "bfloat16" else None
    for p, out in zip(prompts, outs):
        assert out.finished and out.finish_reason == "length" and out.completion_tokens == 16
        want, margins = _plain_greedy_with_margins(cfg, W, p, 16, rt)
        _agree(out.output_token_ids, want, margins, slack)
    st = eng.stats()
    assert st["pages_used"] == 0 and st["generated_tokens"] == 48 and st["prompt_tokens"] == 49
    if graphs:
        assert st["graph_replays"] > 0


def test_mixed_batch_with_temperature_is_reproducible_and_cut_invariant(dirs):
    """Five prompts of 1..200 tokens, 32-token portions, 24 decoded tokens each, temperature
    0.7 from a fixed seed, page size 16: the tokens do not depend on the token budget, on the
    number of sequences that run together, or on whether a request runs alone."""
    from fastmlx_b200 import Engine, SamplingParams
    cfg = tiny.TINY_B
    prompts = [tiny.rand_tokens(n, cfg["vocab_size"], 60 + n) for n in (1, 17, 64, 100, 200)]
    sps = [SamplingParams(max_tokens=24, temperature=0.7, seed=1234 + i) for i in range(5)]

    def run(**kw):
        eng = Engine(dirs["B"], dtype="float32", block_size=16, max_cache_tokens=2048, **kw)
        return [o.output_token_ids for o in eng.generate(prompts, sps)], eng.stats()

    base, st = run(max_concurrent_requests=8, max_num_batched_tokens=64, prefill_chunk=32)
    assert all(len(t) == 24 for t in base) and st["pages_used"] == 0
    assert len({tuple(t) for t in base}) == 5
    other, _ = run(max_concurrent_requests=2, max_num_batched_tokens=4096)
    assert other == base
    third, _ = run(max_concurrent_requests=3, max_num_batched_tokens=7, prefill_chunk=5, cuda_graphs=False)
    assert third == base
    eng = Engine(dirs["B"], dtype="float32", block_size=16, max_cache_tokens=2048)
    for p, sp, want in zip(prompts, sps, base):
        assert eng.generate([p], sp)[0].output_token_ids == want
    # the plain model, fed the engine's own tokens, gives each of them a fair probability
    W = tiny.load_plain_weights(dirs["B"])
    logits = plain_llama.forward(cfg, W, prompts[1] + base[1])
    probs = torch.softmax(logits[len(prompts[1]) - 1: -1] / 0.7, dim=-1)
    assert all(probs[i, t] > 1e-4 for i, t in enumerate(base[1]))


def test_sampling_over_a_wide_vocabulary_is_reproducible(tmp_path):
    """A vocabulary of 16,640: the filters and the draw of a row run in one kernel on a cluster of
    blocks.  With the reference's default filter (top_p 0.95) and with top-k and min-p, the
    tokens of a request do not depend on what runs beside it or on how its prompt is cut, and the
    plain model, fed the engine's tokens, gives each of them a probability that the filters keep."""
    from fastmlx_b200 import Engine, SamplingParams
    cfg = dict(tiny.TINY_A, vocab_size=16640)
    path = tiny.make_model_dir(tmp_path, cfg, seed=5)
    prompts = [tiny.rand_tokens(n, cfg["vocab_size"], 70 + n) for n in (3, 40, 90)]
    sps = [SamplingParams(max_tokens=12, temperature=1.0, seed=1),                               # top_p 0.95 by default
           SamplingParams(max_tokens=12, temperature=0.8, top_p=0.9, top_k=50, seed=2),
           SamplingParams(max_tokens=12, temperature=1.3, top_p=1.0, min_p=0.01, seed=3)]

    def run(**kw):
        eng = Engine(path, dtype="float32", block_size=16, max_cache_tokens=1024, **kw)
        return [o.output_token_ids for o in eng.generate(prompts, sps)]

    base = run(max_concurrent_requests=4)
    assert all(len(t) == 12 for t in base)
    assert run(max_concurrent_requests=1, max_num_batched_tokens=16, prefill_chunk=7, cuda_graphs=False) == base
    eng = Engine(path, dtype="float32", block_size=16, max_cache_tokens=1024)
    for p, sp, want in zip(prompts, sps, base):
        assert eng.generate([p], sp)[0].output_token_ids == want
    W = tiny.load_plain_weights(path)
    logits = plain_llama.forward(cfg, W, prompts[1] + base[1])[len(prompts[1]) - 1: -1]
    for i, t in enumerate(base[1]):                       # top-k 50: the token is among the 50 most likely
        assert t in torch.topk(logits[i], 50).indices.tolist()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_preemption_changes_no_token(dirs, dtype):
    """With a pool of 18 pages three requests cannot all grow: the newest is preempted and
    recomputed, and still every request produces what it produces alone (32-bit: the same
    tokens to the last; bfloat16: each token the plain model's choice at its place, or as good
    within the rounding margin, since the kernels of a recomputed prompt round differently)."""
    from fastmlx_b200 import Engine, SamplingParams
    cfg = tiny.TINY_A
    prompts = [tiny.rand_tokens(n, cfg["vocab_size"], 80 + n) for n in (30, 28, 25)]
    sp = SamplingParams(max_tokens=40, temperature=0.0)
    tight = Engine(dirs["A"], dtype=dtype, block_size=8, initial_cache_blocks=18, max_concurrent_requests=4)
    outs = tight.generate(prompts, sp)
    assert tight.stats()["preemptions"] > 0
    W = tiny.load_plain_weights(dirs["A"])
    if dtype == "float32":
        roomy = Engine(dirs["A"], dtype="float32", block_size=8, initial_cache_blocks=64, max_concurrent_requests=4)
        assert [o.output_token_ids for o in outs] == [o.output_token_ids for o in roomy.generate(prompts, sp)]
    for p, o in zip(prompts, outs):
        assert o.finish_reason == "length" and len(o.output_token_ids) == 40
        tiny.check_greedy(cfg, W, p, o.output_token_ids, torch.bfloat16 if dtype == "bfloat16" else None,
                          2e-2 if dtype == "bfloat16" else 1e-5)
    assert tight.stats()["pages_used"] == 0
    tight.manager.check()


def test_errors_are_reported_per_request(dirs):
    from fastmlx_b200 import Engine, SamplingParams
    eng = Engine(dirs["A"], dtype="float32", block_size=16, max_cache_tokens=256)
    outs = eng.generate([[], [1, 2, 999999], [3, 4, 5]], SamplingParams(max_tokens=2, temperature=0.0))
    assert outs[0].finish_reason == "error" and "empty" in outs[0].err
    assert outs[1].finish_reason == "error" and "vocabulary" in outs[1].err
    # the bad token's step took its neighbours down with it, as a backend error does in the
    # reference; a later request runs normally
    ok = eng.generate([[3, 4, 5]], SamplingParams(max_tokens=2, temperature=0.0))[0]
    assert ok.finish_reason == "length" and ok.completion_tokens == 2
    assert eng.stats()["pages_used"] == 0


def test_abort_and_eos(dirs):
    from fastmlx_b200 import Engine, SamplingParams
    cfg = tiny.TINY_A
    W = tiny.load_plain_weights(dirs["A"])
    prompt = tiny.rand_tokens(9, cfg["vocab_size"], 5)
    want = plain_llama.greedy_generate(cfg, W, prompt, 6)
    eng = Engine(dirs["A"], dtype="float32", block_size=16, max_cache_tokens=256)
    out = eng.generate([prompt], SamplingParams(max_tokens=20, temperature=0.0, stop_token_ids=[want[3]]))[0]
    assert out.finish_reason == "stop" and out.output_token_ids == want[:want.index(want[3]) + 1]
    rid = eng.submit(prompt, SamplingParams(max_tokens=1000, temperature=0.0))
    eng.step()
    eng.abort(rid)
    outs = []
    while eng.has_unfinished():
        outs += eng.step()
    assert outs[-1].request_id == rid and outs[-1].finish_reason == "abort"
    assert eng.stats()["pages_used"] == 0


def test_command_line_generate(dirs, tmp_path):
    cfg = tiny.TINY_A
    W = tiny.load_plain_weights(dirs["A"])
    prompt = tiny.rand_tokens(11, cfg["vocab_size"], 9)
    want = plain_llama.greedy_generate(cfg, W, prompt, 5)
    cmd = [sys.executable, "-m", "fastmlx_b200", "generate", "--model-dir", dirs["A"], "--dtype", "float32",
           "--prompt-ids", ",".join(map(str, prompt)), "--max-tokens", "5", "--temperature", "0",
           "--max-cache-tokens", "256"]
    res = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stderr[-2000:]
    out = json.loads(res.stdout.strip().splitlines()[-1])
    assert out["output_token_ids"] == want and out["finish_reason"] == "length"
    # a folder written by the command line's random-model runs too
    cpath = tmp_path / "c.json"
    cpath.write_text(json.dumps(tiny.TINY_C))
    made = subprocess.run([sys.executable, "-m", "fastmlx_b200", "random-model", "--config", str(cpath), "--out",
                           str(tmp_path / "m"), "--seed", "3"], cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert made.returncode == 0, made.stderr[-2000:]
    res = subprocess.run([sys.executable, "-m", "fastmlx_b200", "generate", "--model-dir", str(tmp_path / "m"),
                          "--prompt-ids", "1,2,3;4,5", "--max-tokens", "3", "--seed", "7", "--max-cache-tokens", "256"],
                         cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [json.loads(l) for l in res.stdout.strip().splitlines()]
    assert len(lines) == 2 and all(l["completion_tokens"] == 3 for l in lines)


def test_running_one_step_ahead_changes_no_token(dirs):
    """The engine launches a decode step before it has read the ids of the one before (they
    are fed on the device).  Tokens, finish reasons and counts must be those of the engine
    that waits every step: with temperature sampling, with a request that stops on a token in
    mid-flight (its look-ahead step is thrown away), with one that ends by length, and with
    requests that arrive while others decode."""
    from fastmlx_b200 import Engine, SamplingParams
    cfg = tiny.TINY_B
    prompts = [tiny.rand_tokens(n, cfg["vocab_size"], 300 + n) for n in (5, 33, 70, 12)]

    def run(lookahead, stop_on=None):
        eng = Engine(dirs["B"], dtype="float32", block_size=16, max_cache_tokens=2048, max_concurrent_requests=4,
                     lookahead=lookahead)
        sps = [SamplingParams(max_tokens=30, temperature=0.8, seed=7),
               SamplingParams(max_tokens=40, temperature=0.0, stop_token_ids=[stop_on] if stop_on is not None else []),
               SamplingParams(max_tokens=9, temperature=1.0, top_p=0.9, seed=9),
               SamplingParams(max_tokens=25, temperature=0.0)]
        ids = [eng.submit(p, sp) for p, sp in zip(prompts[:3], sps[:3])]
        final, steps = {}, 0
        while eng.has_unfinished():
            steps += 1
            if steps == 6:
                ids.append(eng.submit(prompts[3], sps[3]))          # arrives while the others decode
            for o in eng.step():
                if o.finished:
                    final[o.request_id] = o
        assert eng.stats()["pages_used"] == 0
        eng.manager.check()
        return [(final[i].output_token_ids, final[i].finish_reason) for i in ids], eng.stats()

    base, st0 = run(False)
    stop_token = base[1][0][10]                                     # greedy request: stop it in mid-flight
    want, _ = run(False, stop_token)
    got, st1 = run(True, stop_token)
    assert got == want
    assert want[1][1] == "stop" and want[0][1] == "length" and want[2][1] == "length"
    assert st1["graph_replays"] > 0
    assert run(True)[0] == base


@pytest.mark.parametrize("seed", [1, 2, 3])
def test_random_arrivals_aborts_and_a_tight_pool(dirs, seed):
    """Requests of random lengths arrive while others decode, some are aborted midway, the pool is
    too small for all of them (so some are preempted and recomputed) and prompts are cut into
    portions: every request that finishes produces what it produces alone, greedy or sampled
    from its own seed, and at the end no page is held."""
    import random
    from fastmlx_b200 import Engine, SamplingParams
    rng = random.Random(seed)
    cfg = tiny.TINY_B
    n_req = 10
    prompts = [tiny.rand_tokens(rng.randint(1, 90), cfg["vocab_size"], 500 + 17 * seed + i) for i in range(n_req)]
    sps = [SamplingParams(max_tokens=rng.randint(3, 30), temperature=0.0 if i % 3 else 0.8, seed=77 + i)
           for i in range(n_req)]
    alone = Engine(dirs["B"], dtype="float32", block_size=16, max_cache_tokens=1024)
    want = [alone.generate([p], sp)[0].output_token_ids for p, sp in zip(prompts, sps)]

    eng = Engine(dirs["B"], dtype="float32", block_size=8, initial_cache_blocks=40, max_concurrent_requests=4,
                 max_num_batched_tokens=48, prefill_chunk=rng.choice([5, 16, 32]))
    arrive = sorted(rng.randint(0, 40) for _ in range(n_req))
    abort_at = {i: arrive[i] + rng.randint(1, 12) for i in rng.sample(range(n_req), 3)}
    ids, final, got = {}, {}, {}
    step = 0
    while step < 2000 and (len(ids) < n_req or eng.has_unfinished()):
        for i in range(n_req):
            if i not in ids and arrive[i] <= step:
                ids[i] = eng.submit(prompts[i], sps[i])
        for i, at in abort_at.items():
            if at == step and i in ids and ids[i] not in final:
                eng.abort(ids[i])
        for out in eng.step():
            got.setdefault(out.request_id, []).extend(out.new_token_ids)
            if out.finished:
                final[out.request_id] = out
        step += 1
    for out in eng.flush():
        got.setdefault(out.request_id, []).extend(out.new_token_ids)
        if out.finished:
            final[out.request_id] = out
    assert len(final) == n_req
    finished_normally = 0
    for i in range(n_req):
        out = final[ids[i]]
        assert out.err == ""
        if out.finish_reason == "abort":
            assert i in abort_at
            assert out.output_token_ids == want[i][:len(out.output_token_ids)]
        else:
            finished_normally += 1
            assert out.finish_reason == "length" and out.output_token_ids == want[i]
            assert got[ids[i]] == want[i]                 # the increments add up to the whole
    # and what "alone" produced is the plain model's choice, token by token (the greedy requests)
    W = tiny.load_plain_weights(dirs["B"])
    for i in range(n_req):
        if sps[i].temperature == 0.0:
            tiny.check_greedy(cfg, W, prompts[i], want[i], None, 1e-5)
    assert finished_normally >= n_req - 3
    assert eng.stats()["pages_used"] == 0
    eng.manager.check()


def test_bad_token_in_an_early_portion_is_reported(dirs):
    """A portion of a prompt that asks for no token is not waited for; the status it leaves is
    read with the next step's ids, while the request still runs.  An aborted request's status
    falls on nobody."""
    from fastmlx_b200 import Engine, SamplingParams
    cfg = tiny.TINY_A
    sp = SamplingParams(max_tokens=2, temperature=0.0)
    eng = Engine(dirs["A"], dtype="float32", block_size=16, max_cache_tokens=256, prefill_chunk=8,
                 max_num_batched_tokens=8)
    bad = tiny.rand_tokens(30, cfg["vocab_size"], 3)
    bad[2] = 999999
    out = eng.generate([bad], sp)[0]
    assert out.finish_reason == "error" and "vocabulary" in out.err
    good = tiny.rand_tokens(30, cfg["vocab_size"], 4)
    ok = eng.generate([good], sp)[0]
    assert ok.finish_reason == "length" and ok.completion_tokens == 2
    rid = eng.submit(bad, sp)
    eng.step()                                           # the first portion, with the bad token
    eng.abort(rid)
    while eng.has_unfinished():
        eng.step()
    eng.step()
    ok2 = eng.generate([good], sp)[0]
    assert ok2.finish_reason == "length" and ok2.output_token_ids == ok.output_token_ids
    assert eng.stats()["pages_used"] == 0


def test_running_one_step_ahead_in_bfloat16(dirs):
    """The bfloat16 decode path (weight-streaming products with fused SiLU-mul, attention that
    rotates and stores by itself, dependent launches) under graphs and one step ahead of the
    host: a request stopped by a token in mid-flight, one that ends by length, one that
    arrives while the others decode.  Every token is the plain model's choice at its place."""
    from fastmlx_b200 import Engine, SamplingParams
    cfg = tiny.TINY_B
    W = tiny.load_plain_weights(dirs["B"])
    prompts = [tiny.rand_tokens(n, cfg["vocab_size"], 300 + n) for n in (5, 33, 70, 12)]
    plain1, margins = _plain_greedy_with_margins(cfg, W, prompts[1], 40, torch.bfloat16)
    at = next(i for i in range(8, 40) if plain1[i] not in plain1[:i])
    sps = [SamplingParams(max_tokens=30, temperature=0.0),
           SamplingParams(max_tokens=40, temperature=0.0, stop_token_ids=[plain1[at]]),
           SamplingParams(max_tokens=9, temperature=0.0),
           SamplingParams(max_tokens=25, temperature=0.0)]
    for lookahead in (True, False):
        eng = Engine(dirs["B"], dtype="bfloat16", block_size=16, max_cache_tokens=2048, max_concurrent_requests=4,
                     lookahead=lookahead)
        ids = [eng.submit(p, sp) for p, sp in zip(prompts[:3], sps[:3])]
        final, steps = {}, 0
        while eng.has_unfinished():
            steps += 1
            if steps == 6:
                ids.append(eng.submit(prompts[3], sps[3]))
            for o in eng.step():
                if o.finished:
                    final[o.request_id] = o
        assert eng.stats()["pages_used"] == 0 and eng.stats()["graph_replays"] > 0
        eng.manager.check()
        for i, (p, sp) in enumerate(zip(prompts, sps)):
            out = final[ids[i]]
            tiny.check_greedy(cfg, W, p, out.output_token_ids, torch.bfloat16, 2e-2)
            if i != 1:
                assert out.finish_reason == "length" and len(out.output_token_ids) == sp.max_tokens
        got1 = final[ids[1]].output_token_ids
        if got1[:at + 1] == plain1[:at + 1]:
            assert final[ids[1]].finish_reason == "stop" and len(got1) == at + 1
        else:                                   # parted ways with the plain model at a thin margin, legitimately
            first = next(i for i, (g, w) in enumerate(zip(got1, plain1)) if g != w)
            assert margins[first] < 2e-2


def test_random_arrivals_aborts_and_a_tight_pool_in_bfloat16(dirs):
    """The schedule of `test_random_arrivals_aborts_and_a_tight_pool` (arrivals while others
    decode, aborts, preemption, portions) with bfloat16 kernels and greedy choices: what a
    request produced, whole or up to its abort, is the plain model's choice token by token."""
    import random
    from fastmlx_b200 import Engine, SamplingParams
    rng = random.Random(1)
    cfg = tiny.TINY_B
    W = tiny.load_plain_weights(dirs["B"])
    n_req = 10
    prompts = [tiny.rand_tokens(rng.randint(1, 90), cfg["vocab_size"], 900 + i) for i in range(n_req)]
    sps = [SamplingParams(max_tokens=rng.randint(3, 30), temperature=0.0) for i in range(n_req)]
    eng = Engine(dirs["B"], dtype="bfloat16", block_size=8, initial_cache_blocks=40, max_concurrent_requests=4,
                 max_num_batched_tokens=48, prefill_chunk=16)
    arrive = sorted(rng.randint(0, 40) for _ in range(n_req))
    abort_at = {i: arrive[i] + rng.randint(1, 12) for i in rng.sample(range(n_req), 3)}
    ids, final = {}, {}
    step = 0
    while step < 2000 and (len(ids) < n_req or eng.has_unfinished()):
        for i in range(n_req):
            if i not in ids and arrive[i] <= step:
                ids[i] = eng.submit(prompts[i], sps[i])
        for i, at in abort_at.items():
            if at == step and i in ids and ids[i] not in final:
                eng.abort(ids[i])
        for out in eng.step():
            if out.finished:
                final[out.request_id] = out
        step += 1
    for out in eng.flush():
        if out.finished:
            final[out.request_id] = out
    assert len(final) == n_req
    for i in range(n_req):
        out = final[ids[i]]
        assert out.err == ""
        if out.finish_reason != "abort":
            assert out.finish_reason == "length" and len(out.output_token_ids) == sps[i].max_tokens
        if out.output_token_ids:
            tiny.check_greedy(cfg, W, prompts[i], out.output_token_ids, torch.bfloat16, 2e-2)
    assert eng.stats()["pages_used"] == 0
    eng.manager.check()


LONG_B = dict(tiny.TINY_B, max_position_embeddings=2048)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_graphs_across_block_table_widths_and_batch_sizes(tmp_path, dtype):
    """Decode graphs are captured per (rows rounded up to a power of two, block-table width
    rounded up to a power of two, at least 16 pages).  Here contexts grow across 256 and 512
    tokens at page size 16 (widths 16 -> 32 -> 64) while a step runs ahead of the host, a long
    prompt arrives in between, and the batch shrinks from 5 (8 rows) to 4, 2 and 1 as requests
    end: each change meets a new graph whose token ids come from the graph before.  32-bit: the same tokens as without
    graphs.  Both: every token the plain model's choice at its place."""
    from fastmlx_b200 import Engine, SamplingParams
    cfg = LONG_B
    d = tiny.make_model_dir(tmp_path, cfg, seed=31)
    W = tiny.load_plain_weights(d)
    lens_new = [(100, 170), (30, 12), (200, 100), (60, 20), (10, 8), (500, 40)]
    prompts = [tiny.rand_tokens(n, cfg["vocab_size"], 700 + n) for n, _ in lens_new]
    sps = [SamplingParams(max_tokens=m, temperature=0.0) for _, m in lens_new]

    def run(graphs):
        eng = Engine(d, dtype=dtype, block_size=16, max_cache_tokens=4096, max_concurrent_requests=8,
                     cuda_graphs=graphs, lookahead=graphs)
        ids = [eng.submit(p, sp) for p, sp in zip(prompts[:5], sps[:5])]      # five short ones: 8 rows, 16 pages wide
        final, steps = {}, 0
        while eng.has_unfinished():
            steps += 1
            if steps == 30:
                ids.append(eng.submit(prompts[5], sps[5]))                   # 500 tokens: 32 pages, 64 from its 13th token on
            for o in eng.step():
                if o.finished:
                    final[o.request_id] = o
        assert eng.stats()["pages_used"] == 0
        return [final[i].output_token_ids for i in ids], eng

    got, eng = run(True)
    keys = set(eng.step_fn.graphs)
    assert {k[1] for k in keys} >= {16, 32, 64}, keys
    assert {k[0] for k in keys} >= {8, 4, 2, 1}, keys
    for (n, m), p, toks in zip(lens_new, prompts, got):
        assert len(toks) == m
        tiny.check_greedy(cfg, W, p, toks, torch.bfloat16 if dtype == "bfloat16" else None,
                          2e-2 if dtype == "bfloat16" else 1e-5)
    if dtype == "float32":
        assert run(False)[0] == got


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("live", [32, 64])
def test_many_live_requests(dirs, dtype, live):
    """32 and 64 requests decode together (in bfloat16: library products for more than 16
    rows, attention with few splits, a graph of that many rows); prompts of 1 to 90 tokens."""
    from fastmlx_b200 import Engine, SamplingParams
    cfg = tiny.TINY_B
    W = tiny.load_plain_weights(dirs["B"])
    prompts = [tiny.rand_tokens(1 + (37 * i) % 90, cfg["vocab_size"], 1200 + i) for i in range(live)]
    eng = Engine(dirs["B"], dtype=dtype, block_size=16, max_cache_tokens=live * 128, max_concurrent_requests=live,
                 max_num_batched_tokens=4096)
    outs = eng.generate(prompts, SamplingParams(max_tokens=6, temperature=0.0))
    assert max(k[0] for k in eng.step_fn.graphs) == live
    for p, o in zip(prompts, outs):
        assert o.finish_reason == "length" and len(o.output_token_ids) == 6
        tiny.check_greedy(cfg, W, p, o.output_token_ids, torch.bfloat16 if dtype == "bfloat16" else None,
                          2e-2 if dtype == "bfloat16" else 1e-5)
    assert eng.stats()["pages_used"] == 0
