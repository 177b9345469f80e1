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


def test_preemption_changes_no_token(dirs):
    """With a pool of 12 pages three requests cannot all grow: the newest is preempted and
    recomputed, and still every request produces what it produces alone."""
    from fastmlx_b200 import Engine, SamplingParams
    cfg = tiny.TINY_A
    prompts = [tiny.rand_tokens(n, cfg["vocab_size"], 80 + n) for n in (30, 28, 25)]
    sp = SamplingParams(max_tokens=40, temperature=0.0)
    roomy = Engine(dirs["A"], dtype="float32", block_size=8, initial_cache_blocks=64, max_concurrent_requests=4)
    want = [o.output_token_ids for o in roomy.generate(prompts, sp)]
    tight = Engine(dirs["A"], dtype="float32", block_size=8, initial_cache_blocks=18, max_concurrent_requests=4)
    outs = tight.generate(prompts, sp)
    assert tight.stats()["preemptions"] > 0
    assert [o.output_token_ids for o in outs] == want
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


def test_real_layer_sizes_bfloat16_against_32_bit(tmp_path):
    """Two layers with the layer sizes of Llama-3.2-1B (width 2048, 32/8 heads of 64, 8192
    intermediate, llama3-scaled rotary) and a vocabulary cut to 4,000: the bfloat16 engine
    (tensor-memory products for the prompt, weight-streaming products and split attention
    for the decoded tokens, CUDA graphs) against the 32-bit engine, on a prompt of 300
    tokens fed in portions beside another request's decoded tokens."""
    from fastmlx_b200.engine.replay import Replayer
    import traces
    cfg = {"model_type": "llama", "num_hidden_layers": 2, "hidden_size": 2048, "num_attention_heads": 32,
           "num_key_value_heads": 8, "head_dim": 64, "intermediate_size": 8192, "vocab_size": 4000,
           "rope_theta": 500000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 4096,
           "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                            "original_max_position_embeddings": 8192}}
    d = tiny.make_model_dir(tmp_path, cfg, seed=5)
    prompts = {"long": tiny.rand_tokens(300, 4000, 1), "short": tiny.rand_tokens(40, 4000, 2),
               "mid": tiny.rand_tokens(150, 4000, 3)}
    steps = traces.mixed(prompts, chunk=(129, 64, 33, 2, 128), decode_after=0.8)
    want_last = [dict(s, entries=[dict(e, want=e["want"][-1:]) for e in s["entries"]]) for s in steps]
    outs = {}
    for dtype in ("float32", "bfloat16"):
        rp = Replayer(d, dtype, 1024, page_size=16)
        outs[dtype] = traces.collect(want_last, [rp.step(s) for s in want_last])
        rp.manager.check()
    import numpy as np
    worst = 0.0
    for rid in prompts:
        for pos, ref in outs["float32"][rid].items():
            got = outs["bfloat16"][rid][pos]
            worst = max(worst, float(np.abs(got - ref).max() / np.abs(ref).max()))
    assert worst < 3e-2, worst


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
