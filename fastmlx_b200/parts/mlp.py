"""Dense gated feed-forward."""
from __future__ import annotations

from .base import FeedForward
from .linear import Linear


class SwiGLU(FeedForward):
    """down(silu(gate(x)) * up(x)), silu(g) = g * sigmoid(g) in 32-bit (tamnd/fastmlx
    compute/models/llama.go:426-428, compute/models/qwen3_forward.go:229-239).  gate and
    up run as one product whose output is [gate | up]."""

    def __init__(self, width: int, intermediate: int, name: str, bias: bool = False,
                 proj_names=("gate_proj", "up_proj", "down_proj")):
        self.width, self.intermediate = int(width), int(intermediate)
        g, u, d = (f"{name}.{p}" for p in proj_names)
        self.gate_up = Linear(width, [(g, intermediate), (u, intermediate)], bias)
        self.down = Linear(intermediate, [(d, width)], bias)

    def children(self):
        return (self.gate_up, self.down)

    def forward(self, x, ctx):
        gu = self.gate_up.forward(x)
        return self.down.forward(self.rt.k.silu_mul(gu))
