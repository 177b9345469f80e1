"""Plain, slow Llama 3 dense model: the oracle every engine test compares with.

It rests on the formulas of tamnd/fastmlx's Go sources, not on running them: that
project's tensor backend (cgo over mlx-c) is not buildable from its repository and its
default build returns ErrMLXUnavailable at the first op (mlxgo/binding_stub.go:169-180),
so no golden output of its model code can be produced on any host.  Each function cites
the file:line it restates.

Whole sequences only, no cache, one function per part, float64 arithmetic by default.
It shares no code with the package under test (it does not import it).

`round_to=torch.bfloat16` rounds the result of every part to bfloat16, which is where
an engine whose activations are bfloat16 rounds too; the arithmetic inside a part stays
in the wide type, as the engine's kernels keep it in 32-bit.
"""
from __future__ import annotations

import math

import torch

WIDE = torch.float64


def _rnd(x: torch.Tensor, round_to):
    if round_to is None:
        return x
    return x.to(round_to).to(x.dtype)


# ----------------------------------------------------------------------------- config
def derive(cfg: dict) -> dict:
    """Defaults of compute/models/llama.go:69-120: head_dim = hidden/heads, kv heads =
    heads, rope_theta = 10000, tied embeddings unless the config says otherwise."""
    c = dict(cfg)
    c.setdefault("num_key_value_heads", c["num_attention_heads"])
    c.setdefault("head_dim", c["hidden_size"] // c["num_attention_heads"])
    c.setdefault("rope_theta", 10000.0)
    c.setdefault("tie_word_embeddings", True)
    c.setdefault("attention_bias", False)
    c.setdefault("mlp_bias", False)
    c.setdefault("rope_traditional", False)
    c.setdefault("rope_scaling", None)
    return c


# ----------------------------------------------------------------------------- parts
def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """h[t,:] = E[id_t,:], no scaling (compute/models/llama.go:385-390,
    compute/models/quant.go:117-125)."""
    return table.to(WIDE)[ids.long()]


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """x * rsqrt(mean(x^2) + eps) * w, the weight a plain multiplier
    (compute/models/llama.go:402,425,432; mlxgo/binding_cgo.go:382-396)."""
    x = x.to(WIDE)
    var = (x * x).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(var + eps) * w.to(WIDE)


def linear(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor | None = None) -> torch.Tensor:
    """x @ W^T (+ b), W stored [out, in] (compute/models/qwen3_forward.go:111-115,
    compute/models/llama.go:335-342)."""
    y = x.to(WIDE) @ w.to(WIDE).t()
    if b is not None:
        y = y + b.to(WIDE)
    return y


def rope_inv_freq(head_dim: int, theta: float, scaling: dict | None) -> torch.Tensor:
    """Inverse frequencies theta^(-2j/hd) (base = rope_theta, dims = head_dim, position
    scale 1: compute/models/llama.go:377,411-412, compute/models/qwen3_forward.go:153-172).

    The llama3 scaling is named by the config fixture the reference parses
    (compute/testdata/llama_args.json:161-183) but is never applied by its forward; the
    definition used here is the one the config keys spell out: wavelengths shorter than
    orig/high_freq_factor keep their frequency, longer than orig/low_freq_factor are
    divided by factor, and the band between is interpolated linearly in orig/wavelength.
    """
    j = torch.arange(0, head_dim, 2, dtype=WIDE)
    f = theta ** (-j / head_dim)
    if not scaling:
        return f
    kind = scaling.get("rope_type", scaling.get("type"))
    if kind in (None, "default"):
        return f
    assert kind == "llama3", kind
    factor = float(scaling["factor"])
    lo = float(scaling["low_freq_factor"])
    hi = float(scaling["high_freq_factor"])
    orig = float(scaling["original_max_position_embeddings"])
    wavelen = 2 * math.pi / f
    out = f.clone()
    for i in range(f.numel()):
        lam = wavelen[i].item()
        if lam < orig / hi:
            continue
        if lam > orig / lo:
            out[i] = f[i] / factor
        else:
            s = (orig / lam - lo) / (hi - lo)
            out[i] = (1 - s) * f[i] / factor + s * f[i]
    return out


def apply_rope(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor,
               traditional: bool = False) -> torch.Tensor:
    """Rotate x[T, n, hd] by angle p * f_j.  Non-traditional pairing joins element j
    with j + hd/2; traditional joins 2j with 2j+1 (compute/models/qwen3_forward.go:153-172).
    The angle is formed in 32-bit (table and product), as the engine forms it; its sine
    and cosine are then taken in the wide type."""
    T, n, hd = x.shape
    x = x.to(WIDE)
    ang = (positions.to(torch.float32)[:, None] * inv_freq.to(torch.float32)[None, :]).to(WIDE)
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    rot = 2 * inv_freq.numel()
    out = x.clone()
    if traditional:
        a, b = x[..., 0:rot:2], x[..., 1:rot:2]
        out[..., 0:rot:2] = a * cos - b * sin
        out[..., 1:rot:2] = b * cos + a * sin
    else:
        a, b = x[..., : rot // 2], x[..., rot // 2: rot]
        out[..., : rot // 2] = a * cos - b * sin
        out[..., rot // 2: rot] = b * cos + a * sin
    return out


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
              window: int | None = None) -> torch.Tensor:
    """softmax_j(scale * q.k_j + mask) . v with a causal mask (query i sees keys j <= i,
    compute/models/batch_mask.go:33-41, compute/models/cache.go:134-139) and grouped
    queries: query head h uses kv head h // (nh / nkv) (compute/models/llama.go:420,
    mlxgo/binding_cgo.go:619-634).  q [T, nh, hd]; k, v [T, nkv, hd].  `window` keeps
    only the last `window` keys (j > i - window); Llama 3 has none."""
    T, nh, hd = q.shape
    nkv = k.shape[1]
    rep = nh // nkv
    q, k, v = q.to(WIDE), k.to(WIDE), v.to(WIDE)
    out = torch.zeros(T, nh, v.shape[-1], dtype=WIDE)
    i = torch.arange(T)
    visible = i[None, :] <= i[:, None]
    if window is not None and window > 0:
        visible &= i[None, :] > (i[:, None] - window)
    for h in range(nh):
        g = h // rep
        s = (q[:, h, :] @ k[:, g, :].t()) * scale
        s = s.masked_fill(~visible, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, h, :] = p @ v[:, g, :]
    return out


def silu(x: torch.Tensor) -> torch.Tensor:
    """x * sigmoid(x) (compute/models/qwen3_forward.go:229-239)."""
    x = x.to(WIDE)
    return x * torch.sigmoid(x)


def swiglu(y, wg, wu, wd, bg=None, bu=None, bd=None, round_to=None) -> torch.Tensor:
    """(silu(y Wg^T) * (y Wu^T)) Wd^T (compute/models/llama.go:426-428)."""
    g = _rnd(linear(y, wg, bg), round_to)
    u = _rnd(linear(y, wu, bu), round_to)
    z = _rnd(silu(g) * u, round_to)
    return _rnd(linear(z, wd, bd), round_to)


def attention_block(x, W, p, cfg, positions, inv_freq, round_to=None, window=None):
    """Projections, head split, rotary positions on q and k, attention, output
    projection (compute/models/llama.go:403-422)."""
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    T = x.shape[0]
    bias = (lambda n: W.get(p + n + ".bias")) if cfg["attention_bias"] else (lambda n: None)
    q = _rnd(linear(x, W[p + "self_attn.q_proj.weight"], bias("self_attn.q_proj")), round_to)
    k = _rnd(linear(x, W[p + "self_attn.k_proj.weight"], bias("self_attn.k_proj")), round_to)
    v = _rnd(linear(x, W[p + "self_attn.v_proj.weight"], bias("self_attn.v_proj")), round_to)
    q = _rnd(apply_rope(q.view(T, nh, hd), positions, inv_freq, cfg["rope_traditional"]), round_to)
    k = _rnd(apply_rope(k.view(T, nkv, hd), positions, inv_freq, cfg["rope_traditional"]), round_to)
    a = attention(q, k, v.view(T, nkv, hd), hd ** -0.5, window)
    a = _rnd(a.reshape(T, nh * hd), round_to)
    return _rnd(linear(a, W[p + "self_attn.o_proj.weight"], bias("self_attn.o_proj")), round_to)


def forward(cfg: dict, W: dict, tokens, round_to=None, return_hidden: bool = False):
    """Logits [T, V] of one whole sequence (compute/models/llama.go:371-442)."""
    cfg = derive(cfg)
    ids = torch.as_tensor(tokens, dtype=torch.long)
    T = ids.numel()
    positions = torch.arange(T)
    inv_freq = rope_inv_freq(cfg["head_dim"], cfg["rope_theta"], cfg["rope_scaling"])
    eps = cfg["rms_norm_eps"]
    h = embedding(ids, W["model.embed_tokens.weight"])
    mbias = (lambda p, n: W.get(p + n + ".bias")) if cfg["mlp_bias"] else (lambda p, n: None)
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        x = _rnd(rms_norm(h, W[p + "input_layernorm.weight"], eps), round_to)
        h = h + attention_block(x, W, p, cfg, positions, inv_freq, round_to)      # the stream itself is never rounded
        y = _rnd(rms_norm(h, W[p + "post_attention_layernorm.weight"], eps), round_to)
        y = swiglu(y, W[p + "mlp.gate_proj.weight"], W[p + "mlp.up_proj.weight"],
                   W[p + "mlp.down_proj.weight"], mbias(p, "mlp.gate_proj"),
                   mbias(p, "mlp.up_proj"), mbias(p, "mlp.down_proj"), round_to)
        h = h + y
    hn = _rnd(rms_norm(h, W["model.norm.weight"], eps), round_to)
    head = W["model.embed_tokens.weight"] if cfg["tie_word_embeddings"] else W["lm_head.weight"]
    logits = linear(hn, head)
    return (logits, h) if return_hidden else logits


# ----------------------------------------------------------------------------- sampling
def argmax(row) -> int:
    """Index of the highest logit, the first one on ties (compute/sampler.go:61-72)."""
    best, val = -1, None
    for i, v in enumerate(row):
        if best == -1 or v > val:
            best, val = i, v
    return best


def greedy_generate(cfg: dict, W: dict, prompt, n: int, round_to=None) -> list[int]:
    """Feed the whole sequence again for every new token: no cache to get wrong."""
    seq = list(prompt)
    for _ in range(n):
        logits = forward(cfg, W, seq, round_to)
        seq.append(int(torch.argmax(logits[-1]).item()))
    return seq[len(prompt):]
