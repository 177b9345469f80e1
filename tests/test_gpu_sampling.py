"""Sampling filters and logits processors on the GPU against the plain statements and
against the cases of tamnd/fastmlx's own fixtures (kept as data in tests/data/sampling_cases.json)."""
import json
import os

import pytest

import tiny
import torch

import plain_sampling as ps

pytestmark = pytest.mark.gpu
DEV = "cuda"
with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "data", "sampling_cases.json")) as _f:
    CASES = json.load(_f)


def k():
    import fastmlx_b200.kernels as kern
    return kern


def _mask(logits, top_p=0.0, min_p=0.0, top_k=0, min_keep=1):
    rows = logits.shape[0]
    f = lambda v: torch.full((rows,), float(v), device=DEV)
    i = lambda v: torch.full((rows,), int(v), dtype=torch.int32, device=DEV)
    return k().filter_mask(logits.to(DEV), f(top_p), f(min_p), i(top_k), i(min_keep)).cpu()


def test_filters_match_the_reference_fixture():
    for case in CASES["filters"]:
        lp = torch.tensor([ps.log_softmax(case["logits"])], dtype=torch.float32)
        p = case["params"]
        if case["op"] == "apply_top_p":
            got = _mask(lp, top_p=p["top_p"])
        elif case["op"] == "apply_min_p":
            got = _mask(lp, min_p=p["min_p"], min_keep=p.get("min_tokens_to_keep", 1))
        elif case["op"] == "apply_top_k":
            got = _mask(lp, top_k=p["top_k"])
        else:
            continue
        assert got[0].tolist() == case["kept"], case["label"]


@pytest.mark.parametrize("V", [12, 131, 1000, 5000, 16385, 40000, 128256])     # above 16,384: a cluster of blocks per row
@pytest.mark.parametrize("params", [dict(top_p=0.9), dict(top_p=0.3), dict(min_p=0.05), dict(min_p=0.5, min_keep=7),
                                     dict(top_k=1), dict(top_k=40), dict(top_p=0.95, min_p=0.02, top_k=50),
                                     dict(top_p=0.5, top_k=3, min_p=0.9, min_keep=5)])
def test_filters_match_plain(V, params):
    g = torch.Generator().manual_seed(V)
    logits = torch.randn(3, V, generator=g) * 3
    logits[1, : V // 2] = logits[1, V // 2: 2 * (V // 2)]           # many equal values: ties at every threshold
    logits[2] = torch.round(logits[2])
    got = _mask(logits, **params)
    for r in range(3):
        want = ps.apply_filters(logits[r].tolist(), **params)
        diff = [i for i in range(V) if bool(got[r, i]) != want[i]]
        if diff and "top_p" in params:
            # the running mass is summed in 32-bit here and in 64-bit there: a token whose
            # mass lands within rounding of the threshold may fall on either side
            lp = ps.log_softmax(logits[r].tolist())
            order = sorted(range(V), key=lambda i: lp[i])
            run, cum = 0.0, {}
            import math
            for i in order:
                run += math.exp(lp[i])
                cum[i] = run
            assert all(abs(cum[i] - (1 - params["top_p"])) < 1e-5 for i in diff) and "top_k" not in params, (r, diff[:5])
        else:
            assert not diff, (r, diff[:5])


def test_large_vocabulary_top_k_and_top_p():
    V = 128256
    logits = torch.randn(2, V, generator=torch.Generator().manual_seed(1)) * 2
    got = _mask(logits, top_k=50)
    for r in range(2):
        assert sorted(torch.nonzero(got[r]).flatten().tolist()) == sorted(torch.topk(logits[r], 50).indices.tolist())
    got = _mask(logits, top_p=0.9)
    for r in range(2):
        p = torch.softmax(logits[r].double(), 0)
        kept = p[got[r].bool()]
        assert kept.sum() >= 0.9 - 1e-4 and kept.sum() - kept.min() <= 0.9 + 1e-4      # the smallest set reaching top_p
        assert p[~got[r].bool()].max() <= kept.min()


@pytest.mark.parametrize("V", [16385, 50001, 128256])
@pytest.mark.parametrize("params", [dict(), dict(top_p=0.9), dict(top_k=40), dict(min_p=0.05, min_keep=3),
                                     dict(top_p=0.95, min_p=0.02, top_k=50)])
def test_filters_and_draw_in_one_kernel(V, params):
    """Wide rows: one kernel filters and draws, a row on a cluster of blocks.  Its token lies in the
    set that the filter kernel alone keeps, its interval of the kept tokens' CDF holds the uniform
    number, a row at temperature 0 takes the first largest logit, and a row's token does not
    depend on the rows beside it."""
    rows = 12
    g = torch.Generator().manual_seed(V + len(params))
    logits = torch.randn(rows, V, generator=g) * 3
    logits[3, 100] = logits[3, 7] = logits[3].max() + 1.0              # a tie for the largest: the lower index
    temps = torch.tensor([0.0, 0.7, 1.0, 1.5] * (rows // 4))
    u = torch.rand(rows, generator=g)
    u[1], u[2] = 0.0, 0.99999994
    f = lambda name, dt: torch.full((rows,), params.get(name, 0 if name != "min_keep" else 1), dtype=dt, device=DEV)
    args = (f("top_p", torch.float32), f("min_p", torch.float32), f("top_k", torch.int32), f("min_keep", torch.int32))
    dev = logits.to(DEV)
    assert k().filter_sample_takes(V)
    got = k().filter_sample(dev, temps.to(DEV), u.to(DEV), *(args if params else ())).cpu()
    keep = k().filter_mask(dev, *args).cpu().bool() if params else torch.ones(rows, V, dtype=torch.bool)
    for r in range(rows):
        i = int(got[r])
        assert keep[r, i], (r, i)
        if temps[r] == 0:
            assert i == int(torch.argmax(logits[r])) and (r != 3 or i == 7)
            continue
        w = torch.softmax(torch.where(keep[r], logits[r].double(), torch.tensor(-float("inf"), dtype=torch.float64))
                          / temps[r].double(), 0)
        c = torch.cumsum(w, 0)
        lo, hi = (c[i - 1].item() if i > 0 else 0.0), c[i].item()
        assert lo - 1e-4 <= u[r].item() <= hi + 1e-4 and w[i] > 0, (r, i, lo, u[r].item(), hi)
    alone = k().filter_sample(dev[5:6].contiguous(), temps[5:6].to(DEV), u[5:6].to(DEV), *((a[5:6] for a in args) if params else ()))
    assert int(alone[0]) == int(got[5])


def test_processors_match_the_reference_fixture():
    cases = CASES["processors"]
    from fastmlx_b200.engine.loading import make_runtime
    from fastmlx_b200.sampling import Sampler, SamplingParams
    sampler = Sampler(make_runtime("float32"))
    for case in cases:
        p = case["params"]
        sp = SamplingParams(temperature=0.0, logit_bias={int(a): b for a, b in (p.get("logit_bias") or {}).items()},
                            repetition_penalty=p.get("repetition_penalty", 1.0),
                            presence_penalty=p.get("presence_penalty", 0.0),
                            frequency_penalty=p.get("frequency_penalty", 0.0),
                            repetition_context_size=p.get("repetition_context_size", 20),
                            presence_context_size=p.get("presence_context_size", 20),
                            frequency_context_size=p.get("frequency_context_size", 20))
        logits = torch.tensor([case["logits"]], dtype=torch.float32, device=DEV)
        tok = sampler.sample(logits, [(sp, 0, 0, case["history"])])
        assert logits[0].cpu().tolist() == pytest.approx(case["expected"], abs=1e-6), case["label"]
        assert int(tok[0]) == max(range(len(case["expected"])), key=lambda i: (case["expected"][i], -i)), case["label"]


def test_processors_match_plain_on_random_rows():
    from fastmlx_b200.engine.loading import make_runtime
    from fastmlx_b200.sampling import Sampler, SamplingParams
    sampler = Sampler(make_runtime("float32"))
    g = torch.Generator().manual_seed(3)
    V = 97
    logits = torch.randn(4, V, generator=g) * 2
    hist = [torch.randint(0, 12, (n,), generator=g).tolist() for n in (0, 5, 30, 64)]
    sps = [SamplingParams(temperature=0.0, repetition_penalty=1.3),
           SamplingParams(temperature=0.0, presence_penalty=0.5, frequency_penalty=0.25, frequency_context_size=3),
           SamplingParams(temperature=0.0, repetition_penalty=0.8, presence_penalty=-0.2, frequency_penalty=0.1,
                          repetition_context_size=7, presence_context_size=40, logit_bias={3: 2.0, 96: -1.0}),
           SamplingParams(temperature=0.0)]
    dev = logits.clone().to(DEV)
    sampler.sample(dev, [(sp, 0, 0, h) for sp, h in zip(sps, hist)])
    for r, (sp, h) in enumerate(zip(sps, hist)):
        want = ps.apply_processors(h, logits[r].tolist(), sp.logit_bias, sp.repetition_penalty if sp.repetition_penalty != 1 else None,
                                   sp.presence_penalty, sp.frequency_penalty, sp.repetition_context_size,
                                   sp.presence_context_size, sp.frequency_context_size)
        assert dev[r].cpu().tolist() == pytest.approx(want, abs=1e-6), r


def test_draws_depend_on_the_seed_and_index_not_on_the_batch():
    from fastmlx_b200.engine.loading import make_runtime
    from fastmlx_b200.sampling import Sampler, SamplingParams
    sampler = Sampler(make_runtime("float32"))
    V = 320
    logits = (torch.randn(5, V, generator=torch.Generator().manual_seed(4)) * 2).to(DEV)
    sp = SamplingParams(temperature=0.7, top_p=0.9, top_k=20)
    rows = [(sp, 11 + r, 3 * r, []) for r in range(5)]
    together = sampler.sample(logits.clone(), rows).tolist()
    alone = [int(sampler.sample(logits[r:r + 1].clone(), [rows[r]])[0]) for r in range(5)]
    reordered = sampler.sample(logits.flip(0).contiguous(), rows[::-1]).tolist()[::-1]
    assert together == alone == reordered
    mixed = sampler.sample(logits.clone(), [(SamplingParams(temperature=0.0), 0, 0, [])] + rows[1:]).tolist()
    assert mixed[0] == int(torch.argmax(logits[0])) and mixed[1:] == together[1:]
