"""y = x W^T (+ b), W stored [out, in]."""
from __future__ import annotations

import torch

from .base import Part, Runtime, WeightSpec, to_compute, to_f32_vector


class Linear(Part):
    """One or several checkpoint matrices applied as a single product: `names` lists
    (tensor name prefix, out features); their rows are stacked at bind time, so q/k/v or
    gate/up run as one matrix product (tamnd/fastmlx runs them one by one,
    compute/models/llama.go:403-405,426-427, through compute/models/qwen3_forward.go:111-115)."""

    def __init__(self, in_features: int, names, bias: bool = False, interleave: int = 0):
        """`interleave` = b > 0 (two matrices of equal height, a multiple of b): their rows are
        stacked in alternating blocks of b, so that a tile of 2b output columns holds b rows
        of the first and the matching b rows of the second."""
        self.in_features = int(in_features)
        self.names = [(n, int(o)) for n, o in names]
        self.out_features = sum(o for _, o in self.names)
        self.has_bias = bool(bias)
        self.interleave = int(interleave)
        if self.interleave and (len(self.names) != 2 or self.names[0][1] != self.names[1][1]
                                or self.names[0][1] % self.interleave):
            raise ValueError("interleaving takes two matrices of equal height, a multiple of the block")
        self.weight = None
        self.bias = None

    def own_weight_specs(self):
        specs = [WeightSpec(n + ".weight", (o, self.in_features), "matrix") for n, o in self.names]
        if self.has_bias:
            specs += [WeightSpec(n + ".bias", (o,), "bias") for n, o in self.names]
        return specs

    def bind_own(self, tensors, rt: Runtime):
        ws = [to_compute(tensors[n + ".weight"], rt) for n, _ in self.names]
        if len({w.dtype for w in ws}) > 1:
            ws = [w.float() for w in ws]
        bs = [to_f32_vector(tensors[n + ".bias"], rt) for n, _ in self.names] if self.has_bias else None
        if self.interleave:
            b = self.interleave
            ws = [torch.stack([w.view(-1, b, self.in_features) for w in ws], dim=1).reshape(-1, self.in_features)]
            if bs is not None:
                bs = [torch.stack([v.view(-1, b) for v in bs], dim=1).reshape(-1)]
        self.weight = ws[0].contiguous() if len(ws) == 1 else torch.cat(ws, dim=0).contiguous()
        if bs is not None:
            self.bias = torch.cat(bs).contiguous()

    def weight_bytes(self):
        return self.weight.numel() * self.weight.element_size()

    def forward(self, x, out_dtype=None):
        return self.rt.k.linear(x, self.weight, self.bias, out_dtype or self.rt.dtype)

    def emit(self, b, x: int, out_dtype=None, out: int | None = None) -> int:
        """Native program: out = x . W^T (+ b) into a new register (or into `out`)."""
        from ..engine.native import OP_LINEAR, _dt
        dt = _dt(out_dtype or self.rt.dtype)
        if out is None:
            out = b.reg(self.out_features, dt)
        b.op(OP_LINEAR, in0=x, out0=out, w=b.ptr(self.weight), bias=b.ptr(self.bias), w_dtype=_dt(self.weight.dtype),
             ldw=self.weight.stride(0), n=self.out_features, k=self.in_features, out_dtype=dt)
        return out
