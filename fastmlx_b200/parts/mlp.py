"""Dense gated feed-forward."""
from __future__ import annotations

import torch

from .base import FeedForward
from .linear import Linear


class SwiGLU(FeedForward):
    """down(silu(gate(x)) * up(x)), silu(g) = g * sigmoid(g) in 32-bit (tamnd/fastmlx
    compute/models/llama.go:426-428, compute/models/qwen3_forward.go:229-239).  gate and
    up run as one product whose output is [gate | up]."""

    BLOCK = 128          # gate and up rows alternate in blocks of this many when the width allows

    def __init__(self, width: int, intermediate: int, name: str, bias: bool = False,
                 proj_names=("gate_proj", "up_proj", "down_proj")):
        self.width, self.intermediate = int(width), int(intermediate)
        g, u, d = (f"{name}.{p}" for p in proj_names)
        # In blocks, a 256-wide tile of the product holds 128 gates and their 128 ups: the
        # tensor-core kernel then applies SiLU-and-multiply in its epilogue and the [T, 2I]
        # intermediate is never written.
        self.block = self.BLOCK if intermediate % self.BLOCK == 0 else 0
        self.gate_up = Linear(width, [(g, intermediate), (u, intermediate)], bias, interleave=self.block)
        self.down = Linear(intermediate, [(d, width)], bias)

    def children(self):
        return (self.gate_up, self.down)

    def forward(self, x, ctx):
        k, w = self.rt.k, self.gate_up.weight
        fused = self.block and self.gate_up.bias is None and hasattr(k, "can_tc")
        if fused and k.can_tc(x, w, None, x.dtype, k.EPI_SILU_MUL):
            # prompt portions: a 256-wide tile holds 128 gates and their ups, SiLU-mul in the epilogue
            act = k.gemm_tcgen05(x, w, ctx.status if ctx is not None else None, epilogue=k.EPI_SILU_MUL)
        elif fused and self.block % 16 == 0 and k.can_gemv(x, w):
            # decode steps: a block owns some gate rows and their up rows, SiLU-mul in its epilogue
            act = k.gemv(x, w, block=self.block)
        else:
            act = k.silu_mul(self.gate_up.forward(x), self.block or None)
        return self.down.forward(act)

    def emit(self, b, x):
        from ..engine.native import OP_GATE_UP, _dt
        act = b.reg(self.intermediate)
        both = b.reg(2 * self.intermediate)              # gate and up side by side, where no kernel fuses SiLU-mul in
        w = self.gate_up.weight
        b.op(OP_GATE_UP, in0=x, out0=act, out1=both, w=b.ptr(w), bias=b.ptr(self.gate_up.bias), w_dtype=_dt(w.dtype),
             ldw=w.stride(0), n=2 * self.intermediate, k=self.width, block=self.block, out_dtype=b.act)
        b.release(both)
        out = self.down.emit(b, act)
        b.release(act)
        return out
