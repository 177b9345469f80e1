"""Two layers with the layer sizes of Llama-3.2-1B, Llama-3.2-3B and Llama-3.1-8B (vocabulary cut
to 4,000) against the plain model: the sizes at which the engine picks its tensor-memory
attention with two score buffers (head size 128, three and four query heads per kv head), the
192- and 256-wide product tiles and the 16-warp weight-streaming product.

32-bit engine against the plain model in float64; bfloat16 engine against the plain model that
rounds to bfloat16 where the engine does.  The prompts are cut as the mixed replay cuts them:
portions of three requests beside each other's decoded tokens.
"""
import os
import tempfile

import numpy as np
import pytest
import torch

import plain_llama
import tiny
import traces

pytestmark = pytest.mark.gpu

_ROPE = {"rope_type": "llama3", "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 8192}
SHAPES = {
    "1b": dict(hidden_size=2048, num_attention_heads=32, num_key_value_heads=8, head_dim=64, intermediate_size=8192,
               tie_word_embeddings=True, rope_scaling=dict(_ROPE, factor=32.0)),
    "3b": dict(hidden_size=3072, num_attention_heads=24, num_key_value_heads=8, head_dim=128, intermediate_size=8192,
               tie_word_embeddings=True, rope_scaling=dict(_ROPE, factor=32.0)),
    "8b": dict(hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=14336,
               tie_word_embeddings=False, rope_scaling=dict(_ROPE, factor=8.0)),
}

# The tolerances of the replay tests at the tiny sizes (measured here: 3e-6 to 6e-6 in 32-bit,
# 8e-3 to 9e-3 in bfloat16, of the largest logit).
TOL = {"float32": 1e-5, "bfloat16": 2e-2}


def _config(shape):
    return dict({"model_type": "llama", "num_hidden_layers": 2, "vocab_size": 4000, "rope_theta": 500000.0,
                 "rms_norm_eps": 1e-5, "max_position_embeddings": 4096}, **SHAPES[shape])


@pytest.fixture(scope="module", params=list(SHAPES))
def case(request):
    cfg = _config(request.param)
    # up to 0.9 GB of weights: a memory-backed temporary folder where there is one
    with tempfile.TemporaryDirectory(dir="/dev/shm" if os.access("/dev/shm", os.W_OK) else None) as tmp:
        d = tiny.make_model_dir(tmp, cfg, seed=5)
        W = {n: t.clone() for n, t in tiny.load_plain_weights(d).items()}
        prompts = {"long": tiny.rand_tokens(300, 4000, 1), "short": tiny.rand_tokens(40, 4000, 2),
                   "mid": tiny.rand_tokens(150, 4000, 3)}
        yield request.param, cfg, d, W, prompts


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_real_layer_sizes_against_the_plain_model(case, dtype):
    from fastmlx_b200.engine.replay import Replayer
    shape, cfg, d, W, prompts = case
    steps = traces.mixed(prompts, chunk=(129, 64, 33, 2, 128), decode_after=0.8)
    # logits at the last place of every entry: the head is not what is tested here
    steps = [dict(s, entries=[dict(e, want=e["want"][-1:]) for e in s["entries"]]) for s in steps]
    rp = Replayer(d, dtype, 1024, page_size=16)
    rows = traces.collect(steps, [rp.step(s) for s in steps])
    rp.manager.check()
    rt = torch.bfloat16 if dtype == "bfloat16" else None
    worst = 0.0
    for rid, toks in prompts.items():
        ref = plain_llama.forward(cfg, W, toks, round_to=rt)
        scale = ref.abs().max().item()
        assert len(toks) - 1 in rows[rid]
        for pos, got in sorted(rows[rid].items()):
            err = float(np.abs(got.astype(np.float64) - ref[pos].numpy()).max()) / scale
            assert err < TOL[dtype], f"{shape} {dtype}: request {rid}, position {pos}: error {err:.3e} (allowed {TOL[dtype]:.0e})"
            worst = max(worst, err)
    print(f"real layer sizes {shape} {dtype}: worst error {worst:.3e} of the largest logit")


def test_bfloat16_generation_at_real_layer_sizes(case):
    """Greedy generation through the engine (scheduler, graphs, one step ahead) at these sizes:
    every token is the plain model's choice at its place, or as good within the bfloat16 margin."""
    from fastmlx_b200 import Engine, SamplingParams
    shape, cfg, d, W, prompts = case
    eng = Engine(d, dtype="bfloat16", block_size=16, max_cache_tokens=2048, max_concurrent_requests=4, prefill_chunk=128)
    plist = [prompts["long"], prompts["short"], prompts["mid"]]
    outs = eng.generate(plist, SamplingParams(max_tokens=12, temperature=0.0))
    for p, out in zip(plist, outs):
        assert out.finish_reason == "length" and len(out.output_token_ids) == 12
        tiny.check_greedy(cfg, W, p, out.output_token_ids, torch.bfloat16, 3e-2)
    assert eng.stats()["graph_replays"] > 0 and eng.stats()["pages_used"] == 0
