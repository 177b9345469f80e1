"""Interfaces of the parts a model is assembled from.

A part owns its sizes and constants as constructor parameters, declares the checkpoint
tensors it binds (`weight_specs`) and what it needs from the cache manager, and runs on
a flat batch of T tokens.  No part knows which model it is in: names of tensors are
handed to it by the architecture's builder.

tamnd/fastmlx hard-wires these choices inside one forward function
(compute/models/llama.go:371-442) and models per-layer cache kinds as a list behind one
interface (compute/kvcache.go:41-53) with two fixed-size state fields on the tensor cache
(compute/models/cache.go:28-34); the split into parts below keeps that generality and
makes the choice a per-layer datum.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Sequence

import torch


@dataclass(frozen=True)
class WeightSpec:
    """One checkpoint tensor: `kind` picks the random init (matrix, embedding and bias
    N(0, 0.02); norm 1 + N(0, 0.02))."""
    name: str
    shape: tuple[int, ...]
    kind: str = "matrix"


@dataclass(frozen=True)
class PagedKVSpec:
    """A mixer that keeps keys and values of earlier tokens in pages.  `window` = 0
    keeps every key; w > 0 only the last w (the page manager gives older pages back)."""
    num_kv_heads: int
    head_dim: int
    window: int = 0


@dataclass(frozen=True)
class StateSpec:
    """Per-request state of fixed size, kept in a slot (zero when a request starts)."""
    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class Runtime:
    """Where and how parts compute: the device, the activation dtype (bfloat16 or
    float32) and the kernel namespace every part calls."""
    device: torch.device
    dtype: torch.dtype
    k: Any                       # fastmlx_b200.kernels, or a stand-in with its functions

    @property
    def is_fp32(self) -> bool:
        return self.dtype == torch.float32


class Part:
    """Base of all parts: a tree whose leaves declare tensors.

    A part may also describe what it does to the native step executor (`emit`, writing
    operations over numbered activation buffers to an `engine.native.ProgramBuilder`); a part
    without it keeps its model on the Python path, where `forward` runs."""

    def children(self) -> Sequence["Part"]:
        return ()

    def own_weight_specs(self) -> list[WeightSpec]:
        return []

    def weight_specs(self) -> list[WeightSpec]:
        specs = list(self.own_weight_specs())
        for c in self.children():
            specs.extend(c.weight_specs())
        return specs

    def bind(self, tensors: dict[str, torch.Tensor], rt: Runtime) -> None:
        """Take this part's tensors (already checked for presence and shape) onto the
        device in the layout its kernels want."""
        self.rt = rt
        self.bind_own(tensors, rt)
        for c in self.children():
            c.bind(tensors, rt)

    def bind_own(self, tensors: dict[str, torch.Tensor], rt: Runtime) -> None:
        pass

    def weight_bytes(self) -> int:
        """Bytes of device weights one step reads (for the roofline)."""
        return sum(c.weight_bytes() for c in self.children())


def to_compute(t: torch.Tensor, rt: Runtime) -> torch.Tensor:
    """A matrix for the compute path.  bfloat16 tensors widen exactly on the 32-bit path;
    a tensor stored in 32-bit stays in 32-bit on either path."""
    if t.dtype == torch.float32:
        return t.to(rt.device).contiguous()
    return t.to(device=rt.device, dtype=rt.dtype).contiguous()


def to_f32_vector(t: torch.Tensor, rt: Runtime) -> torch.Tensor:
    """Norm weights and biases are held in 32-bit (exact for either stored dtype)."""
    return t.to(device=rt.device, dtype=torch.float32).contiguous()


class Mixer(Part):
    """Token mixer of a block (attention here).  forward(x[T, d], ctx, cache) -> [T, d_out]."""

    # A mixer whose forward only launches kernels that read the step's device arrays may be
    # captured in a CUDA graph; one that loops over rows on the host may not.
    supports_cuda_graph = False

    def cache_spec(self) -> PagedKVSpec | None:
        return None

    def state_spec(self) -> StateSpec | None:
        return None

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:  # pragma: no cover
        raise NotImplementedError

    def emit(self, b, x: int, pos: int) -> int:
        """Native program: register x[T, d] in, a new register [T, d_out] out; `pos` is the
        schedule position whose cache this run uses."""
        from ..engine.native import NotNative
        raise NotNative(f"{type(self).__name__} runs in Python only")

    def forward_in_block(self, delta, residual, norm: "Norm", ctx, cache):
        """What a block calls: (delta, residual) in, (delta', residual') out, where the stream
        is residual + delta (either may be None).  The default normalises and calls `forward`;
        a part whose kernels fold the norm or the residual sum in overrides this and returns
        (None, stream)."""
        x, residual = norm.forward(delta, residual)
        return self.forward(x, ctx, cache), residual


class FeedForward(Part):
    """forward(x[T, d], ctx) -> [T, d]; dense here, a routed one has the same face."""

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:  # pragma: no cover
        raise NotImplementedError

    def emit(self, b, x: int) -> int:
        """Native program: register x[T, d] in, a new register [T, d] out."""
        from ..engine.native import NotNative
        raise NotNative(f"{type(self).__name__} runs in Python only")

    def forward_in_block(self, delta, residual, norm: "Norm", ctx):
        """See Mixer.forward_in_block."""
        x, residual = norm.forward(delta, residual)
        return self.forward(x, ctx), residual


class Norm(Part):
    """forward(x, residual) -> (normed, residual'): residual' = residual + x (or whichever of
    the two is given when the other is None), summed in 32-bit and rounded once; normed =
    norm(residual')."""

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None):  # pragma: no cover
        raise NotImplementedError

    def emit(self, b, x: int | None, stream: int | None) -> tuple[int, int]:
        """Native program: (register x or None, stream register or None) -> (normed, stream);
        x is given back to the builder once the stream holds its value."""
        from ..engine.native import NotNative
        raise NotNative(f"{type(self).__name__} runs in Python only")


class PositionEncoding(Part):
    """Puts positions into the projected q and k of an attention mixer and stores k and v
    in the layer's pages (one fused kernel)."""

    def apply_and_store(self, qkv, ctx, cache, nh: int, nkv: int, hd: int) -> None:  # pragma: no cover
        raise NotImplementedError

    def fused_args(self, cache):
        """If a mixer's kernel may do this part's work itself: (frequencies or None, rotated
        width, traditional pairing, whether to store k and v); else None."""
        return None

    def native_args(self):
        """For the native executor's attention operation, which rotates and stores itself:
        (inverse frequencies or None, rotated width, traditional pairing)."""
        from ..engine.native import NotNative
        raise NotNative(f"{type(self).__name__} runs in Python only")


class StreamEncoding(Part):
    """Puts positions into the embedding stream itself (learned absolute positions, a sinusoid
    added to the token embeddings): forward(h[T, d], ctx) -> h', applied once, after the
    embedding and before the first layer.  `ctx.positions` holds every token's position.  A
    model whose mixers use it passes them a `NoPositionEncoding`, which only stores k and v."""

    def forward(self, h: torch.Tensor, ctx) -> torch.Tensor:  # pragma: no cover
        raise NotImplementedError


@dataclass(frozen=True)
class Run:
    """One entry of a model's schedule: run `layer`; `cache_from` names an earlier
    schedule entry whose cache this run reads instead of owning one."""
    layer: int
    cache_from: int | None = None
