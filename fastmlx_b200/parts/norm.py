"""RMSNorm with the residual sum fused in front of it."""
from __future__ import annotations

import torch

from .base import Norm, Runtime, WeightSpec, to_f32_vector


class RMSNorm(Norm):
    """x * rsqrt(mean(x^2) + eps) * w; the weight is a plain multiplier
    (tamnd/fastmlx compute/models/llama.go:402,425,432 -> mlxgo/binding_cgo.go:382-396).
    Sum of squares, rsqrt and the residual sum are 32-bit."""

    def __init__(self, width: int, eps: float, name: str):
        self.width, self.eps, self.name = int(width), float(eps), name

    def own_weight_specs(self):
        return [WeightSpec(self.name + ".weight", (self.width,), "norm")]

    def bind_own(self, tensors, rt: Runtime):
        self.weight = to_f32_vector(tensors[self.name + ".weight"], rt)

    def weight_bytes(self):
        return self.weight.numel() * 4

    def forward(self, x, residual):
        # Beside bfloat16 activations the stream (the running sum of every layer's output) is kept
        # in 32-bit: each layer's contribution is small against it, and rounding the sum to
        # bfloat16 twice a layer is what a deep model's logits would feel most.
        return self.rt.k.add_rmsnorm(x, residual, self.weight, self.eps, stream_dtype=torch.float32,
                                     out_dtype=self.rt.dtype)

    def emit(self, b, x, stream):
        from ..engine.native import BF16, F32, OP_ADD_RMSNORM
        out = b.reg(self.width)
        args = dict(out0=out, vec=b.ptr(self.weight), n=self.width, eps=self.eps)
        if stream is None and b.act == BF16:
            # the stream's first value, widened into a 32-bit register of its own
            stream = b.reg(self.width, F32)
            b.op(OP_ADD_RMSNORM, in0=x, in1=stream, init=1, **args)
            b.release(x)
        elif stream is None:
            b.op(OP_ADD_RMSNORM, in0=x, **args)          # x itself is the stream from here on
            stream = x
        else:
            b.op(OP_ADD_RMSNORM, in0=-1 if x is None else x, in1=stream, **args)
            b.release(x)
        return out, stream

    def fold(self):
        """(weight, eps) for a kernel that normalises its input rows itself."""
        return (self.weight, self.eps)
