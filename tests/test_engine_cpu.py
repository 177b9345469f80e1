"""The host side of the engine (cache manager, batch layout, step function, replay), run
on the CPU with the plain statements of the kernels in their place, against the plain
model.  What it proves is the book-keeping; the kernels have their own GPU tests."""
import pytest
import torch

import plain_llama
import plain_ops
import tiny
import traces
from fastmlx_b200.engine.replay import Replayer


def _prompts(vocab, lens, seed=1):
    return {f"r{i}": tiny.rand_tokens(n, vocab, seed + i) for i, n in enumerate(lens)}


def _reference(cfg, W, prompts, round_to=None):
    return {rid: plain_llama.forward(cfg, W, toks, round_to) for rid, toks in prompts.items()}


@pytest.mark.parametrize("name,lens,page,max_tokens", [
    ("A", [7, 13, 29, 40], 16, 256), ("B", [1, 17, 64, 100], 16, 256), ("C", [5, 33], 32, 128)])
@pytest.mark.parametrize("cut", ["whole", "tail", "portions", "mixed"])
def test_replay_cuts_match_plain(tmp_path, name, lens, page, max_tokens, cut):
    cfg = tiny.CONFIGS[name]
    d = tiny.make_model_dir(tmp_path, cfg, seed=3)
    W = tiny.load_plain_weights(d)
    prompts = _prompts(cfg["vocab_size"], lens)
    ref = _reference(cfg, W, prompts)
    steps = {"whole": traces.whole, "tail": lambda p: traces.tail_decoded(p, 8), "portions": traces.portions,
             "mixed": traces.mixed}[cut](prompts)
    rp = Replayer(d, "float32", max_tokens, page_size=page, device="cpu", kernels=plain_ops)
    outs = []
    for st in steps:
        outs.append(rp.step(st))
        rp.manager.check()
    rows = traces.collect(steps, outs)
    for rid, toks in prompts.items():
        assert sorted(rows[rid]) == list(range(len(toks)))
        got = torch.tensor([rows[rid][i] for i in range(len(toks))], dtype=torch.float64)
        err = (got - ref[rid]).abs().max().item() / ref[rid].abs().max().item()
        assert err < 2e-6, (rid, err)
    assert not rp.manager.requests
    assert all(g.pool.used_pages == 0 for g in rp.manager.groups)
