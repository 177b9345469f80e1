"""Rotary position encoding, fused with the write of k and v into the layer's pages."""
from __future__ import annotations

import math

import torch

from .base import PositionEncoding, Runtime


def inverse_frequencies(rotary_dim: int, theta: float, scaling=None) -> torch.Tensor:
    """f_j = theta^(-2j/dims), j < dims/2, in float64 (tamnd/fastmlx passes base=rope_theta,
    dims=head_dim, scale=1 to the fused rope: compute/models/llama.go:377,411-412,
    compute/models/qwen3_forward.go:153-172).

    `scaling` (a config.llama.RopeScaling of type llama3; the reference parses the block,
    compute/testdata/llama_args.json:161-183, and never applies it) rescales by wavelength
    l_j = 2 pi / f_j: shorter than orig/high_freq_factor keeps f_j; longer than
    orig/low_freq_factor gives f_j/factor; between, with s = (orig/l_j - low)/(high - low),
    (1 - s) f_j/factor + s f_j."""
    j = torch.arange(0, rotary_dim, 2, dtype=torch.float64)
    f = torch.pow(torch.tensor(float(theta), dtype=torch.float64), -j / rotary_dim)
    if scaling is None:
        return f
    orig = float(scaling.original_max_position_embeddings)
    lo, hi, factor = scaling.low_freq_factor, scaling.high_freq_factor, scaling.factor
    lam = 2 * math.pi / f
    s = (orig / lam - lo) / (hi - lo)
    mid = (1 - s) * f / factor + s * f
    return torch.where(lam < orig / hi, f, torch.where(lam > orig / lo, f / factor, mid))


class RotaryEmbedding(PositionEncoding):
    """Rotates pairs of q and k by position * f_j (angle, sine and cosine in 32-bit).
    `traditional` pairs (2j, 2j+1), otherwise (j, j + rotary_dim/2).  It has no tensors in
    the checkpoint; the table is built once, in float64, and held in 32-bit."""

    def __init__(self, head_dim: int, theta: float, scaling=None, traditional: bool = False,
                 rotary_dim: int | None = None):
        self.head_dim = int(head_dim)
        self.rotary_dim = int(rotary_dim if rotary_dim is not None else head_dim)
        if self.rotary_dim % 2 or not 0 <= self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {self.head_dim}")
        self.theta, self.scaling, self.traditional = float(theta), scaling, bool(traditional)
        self.inv_freq = None

    def bind_own(self, tensors, rt: Runtime):
        self.inv_freq = inverse_frequencies(self.rotary_dim, self.theta, self.scaling) \
            .to(torch.float32).to(rt.device).contiguous()

    def apply_and_store(self, qkv, ctx, cache, nh, nkv, hd):
        g = ctx.groups[cache.group] if cache.kv is not None else None
        self.rt.k.rope_kv_write(
            qkv, ctx.positions, self.inv_freq, self.rotary_dim, self.traditional,
            g.slot_mapping if (g is not None and cache.writable) else None,
            cache.kv if cache.writable else None,
            nh, nkv, hd, ctx.status)


    def fused_args(self, cache):
        """What a mixer kernel needs to rotate and store by itself: (frequencies, rotated
        width, pairing, whether to store k and v)."""
        return (self.inv_freq, self.rotary_dim, self.traditional, bool(cache.kv is not None and cache.writable))

    def native_args(self):
        return (self.inv_freq, self.rotary_dim, self.traditional)


class NoPositionEncoding(PositionEncoding):
    """Stores k and v unrotated (a mixer whose positions come from elsewhere)."""

    def apply_and_store(self, qkv, ctx, cache, nh, nkv, hd):
        g = ctx.groups[cache.group] if cache.kv is not None else None
        self.rt.k.rope_kv_write(
            qkv, ctx.positions, None, 0, False,
            g.slot_mapping if (g is not None and cache.writable) else None,
            cache.kv if cache.writable else None,
            nh, nkv, hd, ctx.status)

    def fused_args(self, cache):
        return (None, 0, False, bool(cache.kv is not None and cache.writable))

    def native_args(self):
        return (None, 0, False)
