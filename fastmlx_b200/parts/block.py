"""The arrangement of norm, mixer and feed-forward in one layer."""
from __future__ import annotations

from .base import FeedForward, Mixer, Norm, Part


class PreNormBlock(Part):
    """h += mixer(norm1(h)); h += ffn(norm2(h)) (tamnd/fastmlx compute/models/llama.go:402-429).
    The stream is carried as (delta, residual): each norm first adds the delta to the
    residual in 32-bit, then normalises the sum, so the add costs no pass of its own."""

    def __init__(self, mixer: Mixer, ffn: FeedForward, norm1: Norm, norm2: Norm):
        self.mixer, self.ffn, self.norm1, self.norm2 = mixer, ffn, norm1, norm2

    def children(self):
        return (self.norm1, self.mixer, self.norm2, self.ffn)

    def cache_spec(self):
        return self.mixer.cache_spec()

    def state_spec(self):
        return self.mixer.state_spec()

    @property
    def supports_cuda_graph(self):
        return bool(getattr(self.mixer, "supports_cuda_graph", False)) and \
            bool(getattr(self.ffn, "supports_cuda_graph", True))

    def forward(self, delta, residual, ctx, cache):
        delta, residual = self.mixer.forward_in_block(delta, residual, self.norm1, ctx, cache)
        return self.ffn.forward_in_block(delta, residual, self.norm2, ctx)

    def emit(self, b, delta, stream, pos):
        """Native program: (delta register, stream register or None) -> (delta', stream)."""
        x, stream = self.norm1.emit(b, delta, stream)
        y = self.mixer.emit(b, x, pos)
        b.release(x)
        x, stream = self.norm2.emit(b, y, stream)
        z = self.ffn.emit(b, x)
        b.release(x)
        return z, stream
