"""The plain sampling statements against the cases of tamnd/fastmlx's own fixtures (kept as
data in tests/data/sampling_cases.json and, when that checkout is present, compared with the
files they come from), and the engine's uniform numbers."""
import json
import os

import pytest

import tiny

import plain_sampling as ps
from fastmlx_b200.sampling import SamplingParams, uniform_for

REF = tiny.reference_dir()
needs_ref = pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "compute", "testdata")),
                               reason="the reference checkout is not present")


with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "data", "sampling_cases.json")) as _f:
    CASES = json.load(_f)


@needs_ref
def test_the_kept_cases_are_the_reference_fixtures():
    with open(os.path.join(REF, "compute", "testdata", "sampler_filters.json")) as f:
        fx = [c for c in json.load(f)["cases"] if c["op"] in ("apply_top_p", "apply_min_p", "apply_top_k")]
    assert [(c["label"], c["op"], c["params"], c["logits"], [int(x) for x in c["kept"]]) for c in fx] == \
        [(c["label"], c["op"], c["params"], c["logits"], c["kept"]) for c in CASES["filters"]]
    with open(os.path.join(REF, "compute", "testdata", "logits_processors.json")) as f:
        pc = json.load(f)
    assert [(c["label"], c["params"], c["tokens"], c["logits"], c["expected"]) for c in pc] == \
        [(c["label"], c["params"], c["history"], c["logits"], c["expected"]) for c in CASES["processors"]]


def test_plain_filters_match_the_reference_fixture():
    for case in CASES["filters"]:
        lp = ps.log_softmax(case["logits"])
        p = case["params"]
        if case["op"] == "apply_top_p":
            keep = ps.top_p_keep(lp, p["top_p"])
        elif case["op"] == "apply_min_p":
            keep = ps.min_p_keep(lp, p["min_p"], p.get("min_tokens_to_keep", 1))
        elif case["op"] == "apply_top_k":
            keep = ps.top_k_keep(lp, p["top_k"])
        else:
            continue
        assert [int(x) for x in keep] == case["kept"], case["label"]


def test_plain_processors_match_the_reference_fixture():
    for case in CASES["processors"]:
        p = case["params"]
        got = ps.apply_processors(case["history"], case["logits"], p.get("logit_bias"), p.get("repetition_penalty"),
                                  p.get("presence_penalty"), p.get("frequency_penalty"),
                                  p.get("repetition_context_size") or 20, p.get("presence_context_size") or 20,
                                  p.get("frequency_context_size") or 20)
        assert got == pytest.approx(case["expected"], abs=1e-6), case["label"]


def test_uniform_numbers_depend_on_seed_and_index_only():
    a = [uniform_for(5, i) for i in range(1000)]
    assert a == [uniform_for(5, i) for i in range(1000)]
    assert all(0.0 <= u < 1.0 for u in a)
    assert abs(sum(a) / 1000 - 0.5) < 0.05
    assert a != [uniform_for(6, i) for i in range(1000)]
    assert len(set(a)) > 990


def test_sampling_params_defaults_are_the_references():
    sp = SamplingParams()
    assert (sp.max_tokens, sp.temperature, sp.top_p, sp.top_k, sp.repetition_penalty) == (32768, 1.0, 0.95, 0, 1.0)
    assert SamplingParams(max_tokens=0).max_tokens == 32768
    assert SamplingParams(temperature=0).greedy and not SamplingParams(temperature=0).filters_on
    assert SamplingParams().filters_on and not SamplingParams(top_p=1.0).filters_on
    assert SamplingParams(repetition_context_size=0).repetition_context_size == 20
