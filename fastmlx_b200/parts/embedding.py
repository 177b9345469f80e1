"""Token embedding and output head."""
from __future__ import annotations

import torch

from .base import Part, Runtime, WeightSpec, to_compute


class Embedding(Part):
    """h[t] = E[id_t], no scaling (tamnd/fastmlx compute/models/llama.go:385-390)."""

    def __init__(self, vocab: int, width: int, name: str):
        self.vocab, self.width, self.name = int(vocab), int(width), name
        self.weight = None

    def own_weight_specs(self):
        return [WeightSpec(self.name + ".weight", (self.vocab, self.width), "embedding")]

    def bind_own(self, tensors, rt: Runtime):
        self.weight = to_compute(tensors[self.name + ".weight"], rt)

    def weight_bytes(self):
        return 0          # a step reads T rows, not the table

    def forward(self, ids, ctx):
        if self.weight.dtype != self.rt.dtype:          # a table stored in 32-bit under bfloat16 activations
            return self.rt.k.embedding(ids, self.weight, ctx.status, self.rt.dtype)
        return self.rt.k.embedding(ids, self.weight, ctx.status)


    def emit(self, b) -> int:
        from ..engine.native import OP_EMBED, _dt
        out = b.reg(self.width)
        b.op(OP_EMBED, out0=out, w=b.ptr(self.weight), w_dtype=_dt(self.weight.dtype), n=self.width, table_rows=self.vocab)
        return out


class LMHead(Part):
    """logits = x W^T in 32-bit, no bias, cap or scale; W is the embedding table when the
    model ties them (tamnd/fastmlx compute/models/llama.go:433-437).  Only the rows whose
    logits are wanted reach it."""

    def __init__(self, vocab: int, width: int, name: str | None, tied: Embedding | None = None):
        if (name is None) == (tied is None):
            raise ValueError("LMHead takes either a tensor name or an embedding to tie to")
        self.vocab, self.width, self.name, self.tied = int(vocab), int(width), name, tied
        self.weight = None

    def own_weight_specs(self):
        return [] if self.tied is not None else [WeightSpec(self.name + ".weight", (self.vocab, self.width), "matrix")]

    def bind_own(self, tensors, rt: Runtime):
        if self.tied is None:
            self.weight = to_compute(tensors[self.name + ".weight"], rt)

    def weight_bytes(self):
        w = self.tied.weight if self.tied is not None else self.weight
        return w.numel() * w.element_size()

    def forward(self, x):
        w = self.tied.weight if self.tied is not None else self.weight
        return self.rt.k.linear(x, w, None, torch.float32)

    def forward_after(self, delta, residual, norm, greedy: bool = False):
        """Final norm, then logits; `greedy`: the index of each row's largest logit instead
        (int32), chosen inside the head's product where its kernel can (no logits written)."""
        x, _ = norm.forward(delta, residual)
        if not greedy:
            return self.forward(x)
        k = self.rt.k
        w = self.tied.weight if self.tied is not None else self.weight
        if hasattr(k, "can_greedy_head") and k.can_greedy_head(x, w):
            return k.greedy_head(x, w)
        return k.argmax(self.forward(x))

    def emit_after(self, b, delta, stream, norm) -> None:
        """Native program: final norm, then the step's logits."""
        from ..engine.native import F32, LOGITS, OP_LINEAR, _dt
        x, _ = norm.emit(b, delta, stream)
        w = self.tied.weight if self.tied is not None else self.weight
        b.op(OP_LINEAR, in0=x, out0=LOGITS, w=b.ptr(w), w_dtype=_dt(w.dtype), ldw=w.stride(0), n=self.vocab, k=self.width,
             out_dtype=F32)
        # the greedy choice inside the product takes bfloat16 operands in 16-byte rows
        b.greedy_head_ok = bool(w.dtype == torch.bfloat16 and b.act == _dt(torch.bfloat16) and self.width % 8 == 0
                                and w.stride(0) % 8 == 0 and w.data_ptr() % 16 == 0)
