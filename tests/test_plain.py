"""The plain implementation checked against itself: properties that hold for any correct
statement of the formulas, so that the oracle is not trusted blindly."""
import json
import math
import subprocess
import sys
import os

import pytest
import torch

import plain_llama as pl
import tiny

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _weights(cfg, seed=0):
    g = torch.Generator().manual_seed(seed)
    c = pl.derive(cfg)
    d, nh, nkv, hd, I, V = (c["hidden_size"], c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"],
                            c["intermediate_size"], c["vocab_size"])
    r = lambda *s: torch.randn(*s, generator=g) * 0.05
    W = {"model.embed_tokens.weight": r(V, d), "model.norm.weight": 1 + r(d)}
    for i in range(c["num_hidden_layers"]):
        p = f"model.layers.{i}."
        W.update({p + "input_layernorm.weight": 1 + r(d), p + "post_attention_layernorm.weight": 1 + r(d),
                  p + "self_attn.q_proj.weight": r(nh * hd, d), p + "self_attn.k_proj.weight": r(nkv * hd, d),
                  p + "self_attn.v_proj.weight": r(nkv * hd, d), p + "self_attn.o_proj.weight": r(d, nh * hd),
                  p + "mlp.gate_proj.weight": r(I, d), p + "mlp.up_proj.weight": r(I, d), p + "mlp.down_proj.weight": r(d, I)})
        if c["attention_bias"]:
            W.update({p + "self_attn.q_proj.bias": r(nh * hd), p + "self_attn.k_proj.bias": r(nkv * hd),
                      p + "self_attn.v_proj.bias": r(nkv * hd), p + "self_attn.o_proj.bias": r(d)})
        if c["mlp_bias"]:
            W.update({p + "mlp.gate_proj.bias": r(I), p + "mlp.up_proj.bias": r(I), p + "mlp.down_proj.bias": r(d)})
    if not c["tie_word_embeddings"]:
        W["lm_head.weight"] = r(V, d)
    return W


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_a_position_does_not_see_later_tokens(name):
    cfg = tiny.CONFIGS[name]
    W = _weights(cfg)
    toks = tiny.rand_tokens(40, cfg["vocab_size"], 1)
    full = pl.forward(cfg, W, toks)
    for n in (1, 2, 17, 39):
        part = pl.forward(cfg, W, toks[:n])
        assert torch.allclose(part, full[:n], rtol=0, atol=1e-12)
    other = toks[:20] + tiny.rand_tokens(20, cfg["vocab_size"], 2)
    assert torch.allclose(pl.forward(cfg, W, other)[:20], full[:20], rtol=0, atol=1e-12)
    assert not torch.allclose(pl.forward(cfg, W, other)[20:], full[20:], atol=1e-6)


def test_grouped_queries_equal_full_heads_with_repeated_kv():
    g = torch.Generator().manual_seed(0)
    q, k, v = torch.randn(9, 6, 8, generator=g), torch.randn(9, 2, 8, generator=g), torch.randn(9, 2, 8, generator=g)
    grouped = pl.attention(q, k, v, 0.3)
    full = pl.attention(q, k.repeat_interleave(3, dim=1), v.repeat_interleave(3, dim=1), 0.3)
    assert torch.allclose(grouped, full, atol=1e-14)
    # a window of w keys equals full attention while the sequence is no longer than w
    assert torch.allclose(pl.attention(q, k, v, 0.3, window=9), grouped, atol=1e-14)
    w4 = pl.attention(q, k, v, 0.3, window=4)
    assert torch.allclose(w4[:4], grouped[:4], atol=1e-14) and not torch.allclose(w4[8], grouped[8], atol=1e-6)
    # the first row attends to its own key only
    assert torch.allclose(grouped[0, 4], v[0, 1].double(), atol=1e-14)


def test_rotation_keeps_norms_and_relative_angles():
    inv = pl.rope_inv_freq(16, 10000.0, None)
    assert inv[0] == 1.0 and abs(inv[-1].item() - 10000.0 ** (-14 / 16)) < 1e-15
    g = torch.Generator().manual_seed(1)
    x, y = torch.randn(1, 1, 16, generator=g).double(), torch.randn(1, 1, 16, generator=g).double()
    for trad in (False, True):
        xr = pl.apply_rope(x.expand(6, 1, 16), torch.arange(6), inv, trad)
        yr = pl.apply_rope(y.expand(6, 1, 16), torch.arange(6), inv, trad)
        assert torch.allclose(xr.norm(dim=-1), x.norm().expand(6, 1), atol=1e-6)
        assert torch.allclose(xr[0], x[0], atol=1e-15)                       # position 0 rotates by nothing
        dots = [(xr[i + 2] * yr[i]).sum().item() for i in range(4)]           # depends on the distance only
        assert max(dots) - min(dots) < 1e-5
    half = pl.apply_rope(x.expand(3, 1, 16), torch.arange(3), pl.rope_inv_freq(8, 10000.0, None), False)
    assert torch.equal(half[..., 8:], x.expand(3, 1, 16)[..., 8:])            # a partial rotation leaves the rest


def test_llama3_scaling_has_three_bands():
    sc = tiny.TINY_B["rope_scaling"]
    base = pl.rope_inv_freq(32, 500000.0, None)
    scaled = pl.rope_inv_freq(32, 500000.0, sc)
    ratio = scaled / base
    wavelen = 2 * math.pi / base
    orig = sc["original_max_position_embeddings"]
    for i in range(16):
        if wavelen[i] < orig / sc["high_freq_factor"]:
            assert ratio[i] == 1.0
        elif wavelen[i] > orig / sc["low_freq_factor"]:
            assert abs(ratio[i].item() - 1 / sc["factor"]) < 1e-15
        else:
            assert 1 / sc["factor"] < ratio[i] < 1.0
    assert (ratio == 1).any() and ((ratio > 0.126) & (ratio < 1)).any() and (ratio < 0.126).any()


def test_norm_and_activation_definitions():
    x = torch.tensor([[3.0, 4.0]])
    assert torch.allclose(pl.rms_norm(x, torch.tensor([1.0, 2.0]), 0.0), torch.tensor([[3.0, 8.0]]).double() / math.sqrt(12.5))
    assert abs(pl.silu(torch.tensor([1.0]))[0].item() - 1 / (1 + math.exp(-1))) < 1e-15
    assert pl.argmax([1.0, 3.0, 3.0, 2.0]) == 1 and pl.argmax([]) == -1


def test_rounding_mode_rounds_where_bfloat16_activations_round():
    cfg = tiny.TINY_A
    W = {n: t.to(torch.bfloat16) for n, t in _weights(cfg).items()}
    toks = tiny.rand_tokens(12, cfg["vocab_size"], 3)
    exact, rounded = pl.forward(cfg, W, toks), pl.forward(cfg, W, toks, round_to=torch.bfloat16)
    rel = ((exact - rounded).abs().max() / exact.abs().max()).item()
    assert 1e-5 < rel < 3e-2
    # the stream itself (the sum of every layer's rounded output) is not rounded
    _, hidden = pl.forward(cfg, W, toks, round_to=torch.bfloat16, return_hidden=True)
    assert not torch.equal(hidden, hidden.to(torch.bfloat16).to(hidden.dtype))


def test_greedy_generation_feeds_its_own_tokens():
    cfg = tiny.TINY_A
    W = _weights(cfg, 2)
    prompt = tiny.rand_tokens(5, cfg["vocab_size"], 4)
    out = pl.greedy_generate(cfg, W, prompt, 4)
    seq = list(prompt)
    for tok in out:
        assert tok == int(torch.argmax(pl.forward(cfg, W, seq)[-1]))
        seq.append(tok)


def test_command_line_writes_a_model_folder_and_reports_its_version(tmp_path):
    cpath = tmp_path / "c.json"
    cpath.write_text(json.dumps(tiny.TINY_C))
    env = dict(os.environ, PYTHONPATH=ROOT)
    res = subprocess.run([sys.executable, "-m", "fastmlx_b200", "random-model", "--config", str(cpath), "--out",
                          str(tmp_path / "m"), "--seed", "3", "--max-shard-mb", "1"], cwd=ROOT, env=env,
                         capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stderr[-1000:]
    from fastmlx_b200.weights import load_checkpoint
    cfg, tensors = load_checkpoint(str(tmp_path / "m"))
    assert cfg == tiny.TINY_C and "model.layers.0.mlp.down_proj.bias" in tensors
    res = subprocess.run([sys.executable, "-m", "fastmlx_b200", "version"], cwd=ROOT, env=env, capture_output=True, text=True)
    assert res.returncode == 0 and res.stdout.strip()
