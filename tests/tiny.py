"""Tiny Llama configurations for the tests.  A and B differ in every size and option;
C adds what neither has: projection biases, the traditional rotary pairing, one kv head,
a head size that is not hidden/heads, an odd vocabulary."""
import json
import os
import tempfile

import torch

TINY_A = {
    "model_type": "llama", "architectures": ["LlamaForCausalLM"],
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 16, "intermediate_size": 176, "vocab_size": 256, "rope_theta": 10000.0,
    "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 128,
}
TINY_B = {
    "model_type": "llama", "architectures": ["LlamaForCausalLM"],
    "num_hidden_layers": 3, "hidden_size": 192, "num_attention_heads": 6, "num_key_value_heads": 3,
    "head_dim": 32, "intermediate_size": 512, "vocab_size": 320, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 64},
    "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "max_position_embeddings": 512,
}
TINY_C = {
    "model_type": "llama",
    "num_hidden_layers": 1, "hidden_size": 80, "num_attention_heads": 5, "num_key_value_heads": 1,
    "head_dim": 48, "intermediate_size": 200, "vocab_size": 131, "rope_theta": 1000.0,
    "rope_traditional": True, "attention_bias": True, "mlp_bias": True,
    "rms_norm_eps": 1e-3, "tie_word_embeddings": False, "max_position_embeddings": 300,
}
CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C}


def make_model_dir(tmp_path, config, seed=0, **kw):
    from fastmlx_b200.weights import write_random_model
    d = os.path.join(str(tmp_path), f"model_{abs(hash(json.dumps(config, sort_keys=True))) % 10**8}_{seed}")
    write_random_model(d, config, seed, **kw)
    return d


def load_plain_weights(model_dir):
    """Tensors of a folder for the plain model, read with the safetensors library (not with
    the package's reader)."""
    from safetensors.torch import load_file
    out = {}
    for f in sorted(os.listdir(model_dir)):
        if f.endswith(".safetensors"):
            out.update(load_file(os.path.join(model_dir, f)))
    return out


def rand_tokens(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def reference_dir() -> str:
    """Where tamnd/fastmlx's checkout lies, if anywhere: $FASTMLX_REFERENCE, or a folder
    `reference` beside this repository.  Its test data are golden vectors for a few tests,
    which are skipped without it."""
    import os
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    return os.environ.get("FASTMLX_REFERENCE") or os.path.join(os.path.dirname(here), "reference")


def check_greedy(cfg, W, prompt, got, round_to, slack):
    """Every generated token is the plain model's best at its place, given the tokens before it
    (one forward over prompt + generated: the model is causal), or falls short of the best
    by less than `slack` of the largest logit (where two logits are that close, rounding
    decides, and either choice is right)."""
    import plain_llama
    logits = plain_llama.forward(cfg, W, list(prompt) + list(got), round_to)[len(prompt) - 1: -1]
    assert logits.shape[0] == len(got)
    for i, tok in enumerate(got):
        row = logits[i]
        best = int(torch.argmax(row))
        if best != tok:
            gap = float(row[best] - row[tok]) / float(row.abs().max())
            assert gap < slack, f"token {i}: engine chose {tok}, plain model {best}, gap {gap:.2e} (allowed {slack:.0e})"
