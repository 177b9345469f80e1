"""The scheduler's decisions, on the CPU, over a cache manager that holds no tensors and a
fake step that returns scripted tokens (as tamnd/fastmlx tests its generator with a fake
model, compute/batch_generator_test.go:13-127)."""
import random

import pytest

from fastmlx_b200.cache import CacheManager, OutOfPages
from fastmlx_b200.engine.request import Request, RequestStatus
from fastmlx_b200.engine.scheduler import Scheduler, SchedulerConfig
from fastmlx_b200.parts import PagedKVSpec
from fastmlx_b200.sampling import SamplingParams

NEEDS = [(PagedKVSpec(2, 16), None, None), (PagedKVSpec(2, 16), None, None)]


def make(num_pages=16, page=4, max_seqs=4, budget=32, chunk=0, eos=(), max_pos=0, needs=NEEDS):
    m = CacheManager(needs, page_size=page, num_pages=num_pages, max_requests=max_seqs, allocate=False)
    return m, Scheduler(m, SchedulerConfig(max_seqs, budget, chunk), eos_token_ids=eos, max_positions=max_pos)


def req(rid, n, max_tokens=4, **kw):
    return Request(rid, list(range(1, n + 1)), SamplingParams(max_tokens=max_tokens, temperature=0.0, **kw))


def drive(m, s, script=lambda r, i: 100 + i, limit=1000):
    """Run to the end; -> (final outputs by id, log of plans)."""
    final, log = {}, []
    for _ in range(limit):
        if not s.has_unfinished():
            break
        plan = s.schedule()
        m.check()
        for r in plan.finished:
            final[r.request_id] = s._output(r, [])
        log.append([(r.request_id, len(e.tokens), smp) for r, e, smp in zip(plan.requests, plan.entries, plan.samples)])
        toks = [script(r, len(r.output_token_ids)) for r, smp in zip(plan.requests, plan.samples) if smp]
        for out in s.step_done(plan, toks):
            if out.finished:
                final[out.request_id] = out
        m.check()
    assert not s.has_unfinished()
    return final, log


def test_prompt_is_fed_whole_then_one_token_per_step():
    m, s = make()
    assert s.add_request(req("a", 5, max_tokens=3)) is None
    final, log = drive(m, s)
    assert log == [[("a", 5, True)], [("a", 1, True)], [("a", 1, True)]]
    assert final["a"].output_token_ids == [100, 101, 102] and final["a"].finish_reason == "length"
    assert m.free_pages == 16 and not m.requests


def test_prompt_is_cut_into_portions_under_the_budget():
    m, s = make(num_pages=64, budget=8)
    s.add_request(req("a", 19, max_tokens=2))
    final, log = drive(m, s)
    assert log == [[("a", 8, False)], [("a", 8, False)], [("a", 3, True)], [("a", 1, True)]]
    assert final["a"].completion_tokens == 2


def test_prefill_chunk_caps_one_prompts_share():
    m, s = make(num_pages=64, budget=16, chunk=6)
    s.add_request(req("a", 10, max_tokens=1))
    s.add_request(req("b", 4, max_tokens=1))
    _, log = drive(m, s)
    assert log[0] == [("a", 6, False), ("b", 4, True)]
    assert log[1] == [("a", 4, True)]


def test_decodes_come_first_and_portions_fill_the_rest():
    m, s = make(num_pages=64, budget=10)
    s.add_request(req("a", 3, max_tokens=5))
    plan = s.schedule()
    s.step_done(plan, [7])
    s.add_request(req("b", 30, max_tokens=2))
    plan = s.schedule()
    assert [(r.request_id, len(e.tokens)) for r, e in zip(plan.requests, plan.entries)] == [("a", 1), ("b", 9)]
    assert plan.entries[0].tokens == [7]
    assert plan.entries[0].want == [0] and plan.entries[1].want == []


def test_first_come_first_served_and_max_num_seqs():
    m, s = make(num_pages=64, max_seqs=2, budget=64)
    for i, n in enumerate([4, 4, 4]):
        s.add_request(req(f"r{i}", n, max_tokens=2))
    plan = s.schedule()
    assert [r.request_id for r in plan.requests] == ["r0", "r1"]
    assert [r.request_id for r in s.waiting] == ["r2"]
    s.step_done(plan, [1, 1])
    final, _ = drive(m, s)
    assert set(final) == {"r0", "r1", "r2"}


def test_eos_and_stop_ids_finish_with_stop():
    m, s = make(eos=[9])
    s.add_request(req("a", 3, max_tokens=10))
    s.add_request(req("b", 3, max_tokens=10, stop_token_ids=[55]))
    s.add_request(req("c", 3, max_tokens=10, ignore_eos=True))
    script = lambda r, i: {"a": [1, 9], "b": [1, 2, 55], "c": [9, 9, 9, 9, 9, 9, 9, 9, 9, 9]}[r.request_id][i]
    final, _ = drive(m, s, script)
    assert final["a"].finish_reason == "stop" and final["a"].output_token_ids == [1, 9]
    assert final["b"].finish_reason == "stop" and final["b"].output_token_ids == [1, 2, 55]
    assert final["c"].finish_reason == "length" and final["c"].completion_tokens == 10


def test_empty_and_oversized_prompts_fail_at_admission():
    m, s = make(num_pages=4, page=4, max_pos=64)
    out = s.add_request(req("e", 0))
    assert out.finished and out.finish_reason == "error" and "empty" in out.err
    out = s.add_request(req("big", 17))
    assert out.finished and out.finish_reason == "error" and "pool" in out.err
    out = s.add_request(req("long", 64))
    assert out.finish_reason == "error" and "max_position_embeddings" in out.err
    assert not s.has_unfinished()


def test_abort_waiting_and_running():
    m, s = make(max_seqs=1)
    s.add_request(req("a", 3, max_tokens=50))
    s.add_request(req("b", 3, max_tokens=50))
    s.step_done(s.schedule(), [1])
    s.abort("a")
    s.abort("b")
    plan = s.schedule()
    assert sorted(r.request_id for r in plan.finished) == ["a", "b"]
    assert all(r.status == RequestStatus.FINISHED_ABORTED for r in plan.finished)
    assert not s.has_unfinished() and m.free_pages == 16
    m.check()


def test_when_pages_run_out_the_newest_request_is_preempted_and_later_recomputed():
    # 6 pages of 4 tokens.  a and b take 2 pages each for their prompts (8 tokens) and
    # one more each when they pass 8; the pool is dry when either passes 12.
    m, s = make(num_pages=6, page=4, max_seqs=2, budget=64)
    s.add_request(req("a", 8, max_tokens=9))
    s.add_request(req("b", 8, max_tokens=9))
    final, log = drive(m, s)
    assert s.num_preemptions >= 1
    # the victim is the newer request; the older one is never preempted
    assert final["a"].completion_tokens == 9 and final["b"].completion_tokens == 9
    flat = [x for step in log for x in step]
    # after the preemption b's prompt and its generated tokens are fed again; a's never
    assert sum(n for rid, n, _ in flat if rid == "a") == 8 + 8
    assert sum(n for rid, n, _ in flat if rid == "b") > 8 + 8
    # tokens are the scripted ones, in order, with none lost or doubled by the recomputation
    assert final["b"].output_token_ids == [100 + i for i in range(9)]
    assert m.free_pages == 6


def test_a_request_too_long_for_the_pool_alone_ends_with_length():
    m, s = make(num_pages=3, page=4, max_seqs=2)
    s.add_request(req("a", 10, max_tokens=100))
    final, _ = drive(m, s)
    assert final["a"].finish_reason == "length"
    assert final["a"].completion_tokens == 3            # 12 places: 10 prompt + 2 fed back; the third token is drawn, then no page
    assert m.free_pages == 3


def test_two_half_prefilled_prompts_do_not_deadlock():
    m, s = make(num_pages=6, page=4, max_seqs=2, budget=8)
    s.add_request(req("a", 20, max_tokens=1))
    s.add_request(req("b", 20, max_tokens=1))
    final, _ = drive(m, s)
    assert final["a"].completion_tokens == 1 and final["b"].completion_tokens == 1


def test_backend_error_ends_the_steps_requests():
    m, s = make()
    s.add_request(req("a", 3))
    plan = s.schedule()
    outs = s.step_failed(plan, "boom")
    assert outs[0].finish_reason == "error" and outs[0].err == "boom"
    assert m.free_pages == 16 and not s.has_unfinished()
    m.check()


@pytest.mark.parametrize("seed", range(8))
def test_random_workloads_keep_every_invariant(seed):
    rng = random.Random(seed)
    m, s = make(num_pages=rng.choice([8, 12, 20]), page=rng.choice([2, 4, 8]), max_seqs=rng.choice([1, 2, 4]),
                budget=rng.choice([4, 16, 64]), chunk=rng.choice([0, 3, 8]), eos=[7])
    pool = m.groups[0].pool.num_pages * m.page_size
    want = {}
    pending = [(f"r{i}", rng.randint(1, pool), rng.randint(1, 12)) for i in range(12)]
    final = {}
    steps = 0
    while pending or s.has_unfinished():
        steps += 1
        assert steps < 5000
        if pending and rng.random() < 0.4:
            rid, n, mt = pending.pop()
            out = s.add_request(req(rid, n, max_tokens=mt))
            want[rid] = mt
            if out is not None:
                final[rid] = out
        if rng.random() < 0.05 and s.running:
            s.abort(rng.choice(s.running).request_id)
        if not s.has_unfinished():
            continue
        plan = s.schedule()
        m.check()
        assert plan.num_tokens <= s.cfg.max_num_batched_tokens
        assert len(s.running) <= s.cfg.max_num_seqs
        assert len({id(r) for r in plan.requests}) == len(plan.requests)
        for r in plan.finished:
            final[r.request_id] = s._output(r, [])
        toks = [rng.choice([7, 50, 51]) if rng.random() < 0.2 else 60 for smp in plan.samples if smp]
        for out in s.step_done(plan, toks):
            if out.finished:
                final[out.request_id] = out
        m.check()
    assert set(final) == set(want)
    assert m.free_pages == m.groups[0].pool.num_pages and not m.requests
    for rid, out in final.items():
        assert out.finished and out.finish_reason in ("stop", "length", "abort", "error")
        assert out.completion_tokens <= want[rid]
