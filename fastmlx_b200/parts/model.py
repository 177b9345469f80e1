"""A model: embedding, a list of blocks, the order they run in, final norm, head."""
from __future__ import annotations

from typing import Sequence

import torch

from ..weights.loader import WeightError
from .base import Norm, Part, Run, Runtime
from .embedding import Embedding, LMHead


class Model(Part):
    """`layers` are the distinct blocks; `schedule` says in which order they run, as a
    list of Run entries: a layer may be named twice (it then has a cache per entry), and
    an entry may read the cache of an earlier entry instead of owning one.  Cache needs
    are indexed by schedule position.

    `drop` lists name fragments of checkpoint tensors that are ignored when present
    (tamnd/fastmlx drops rotary inv_freq buffers and a tied checkpoint's lm_head.weight,
    compute/models/llama.go:206-216)."""

    def __init__(self, embed: Embedding, layers: Sequence[Part], final_norm: Norm, head: LMHead,
                 schedule: Sequence[Run] | None = None, drop: Sequence[str] = (), vocab_size: int | None = None,
                 max_positions: int = 0, eos_token_ids: Sequence[int] = (), stream_encoding: Part | None = None):
        """`stream_encoding`: an optional `StreamEncoding` that puts positions into the embedding
        stream (architectures whose positions are not applied to q and k)."""
        self.embed, self.layers, self.final_norm, self.head = embed, list(layers), final_norm, head
        self.stream_encoding = stream_encoding
        self.schedule = list(schedule) if schedule is not None else [Run(i) for i in range(len(self.layers))]
        for pos, run in enumerate(self.schedule):
            if not 0 <= run.layer < len(self.layers):
                raise ValueError(f"schedule[{pos}] names layer {run.layer}, the model has {len(self.layers)}")
            if run.cache_from is not None:
                if not 0 <= run.cache_from < pos or self.schedule[run.cache_from].cache_from is not None:
                    raise ValueError(f"schedule[{pos}] must read the cache of an earlier entry that owns one")
        self.drop = tuple(drop)
        self.vocab_size = int(vocab_size if vocab_size is not None else embed.vocab)
        self.max_positions = int(max_positions)
        self.eos_token_ids = tuple(eos_token_ids)

    def children(self):
        extra = (self.stream_encoding,) if self.stream_encoding is not None else ()
        return (self.embed, *extra, *self.layers, self.final_norm, self.head)

    # ---- what the cache manager must provide, by schedule position
    def cache_needs(self):
        """[(PagedKVSpec | None, StateSpec | None, cache_from | None)] per schedule entry."""
        out = []
        for run in self.schedule:
            layer = self.layers[run.layer]
            kv = layer.cache_spec() if run.cache_from is None else None
            out.append((kv, layer.state_spec(), run.cache_from))
        return out

    @property
    def graph_safe(self) -> bool:
        """May a decode step of this model be captured in a CUDA graph?"""
        return all(getattr(layer, "supports_cuda_graph", False) for layer in self.layers) and \
            bool(getattr(self.stream_encoding, "supports_cuda_graph", True))

    # ---- weights
    def check_weights(self, tensors: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
        """One error that lists every missing tensor, every unexpected one and every wrong
        shape.  (The reference reports the first missing name, ignores extras and checks
        no shape: compute/models/llama.go:246-333.)"""
        specs = {s.name: s for s in self.weight_specs()}
        kept = {n: t for n, t in tensors.items() if not any(d in n for d in self.drop)}
        missing = sorted(n for n in specs if n not in kept)
        unexpected = sorted(n for n in kept if n not in specs)
        wrong = sorted((n, tuple(kept[n].shape), specs[n].shape) for n in specs
                       if n in kept and tuple(kept[n].shape) != tuple(specs[n].shape))
        if missing or unexpected or wrong:
            lines = ["checkpoint does not match the configuration:"]
            if missing:
                lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
            if unexpected:
                lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
            if wrong:
                lines.append(f"  wrong shape ({len(wrong)}): " +
                             ", ".join(f"{n} has {list(g)}, want {list(w)}" for n, g, w in wrong))
            err = WeightError("\n".join(lines))
            err.missing, err.unexpected, err.wrong_shape = missing, unexpected, wrong
            raise err
        return kept

    def load_weights(self, tensors: dict[str, torch.Tensor], rt: Runtime) -> "Model":
        self.bind(self.check_weights(tensors), rt)
        return self

    # ---- one step over a flat batch
    def forward(self, ctx, greedy: bool = False) -> torch.Tensor:
        """Logits [len(ctx.logit_rows), vocab] in 32-bit for the batch that `ctx` describes;
        `greedy`: each wanted row's greedy choice instead, int32 [len(ctx.logit_rows)]."""
        delta = self.embed.forward(ctx.tokens, ctx)
        if self.stream_encoding is not None:
            delta = self.stream_encoding.forward(delta, ctx)
        residual = None
        for pos, run in enumerate(self.schedule):
            delta, residual = self.layers[run.layer].forward(delta, residual, ctx, ctx.caches[pos])
        k = self.rt.k
        if ctx.logit_rows is not None:
            if delta is not None:
                delta = k.gather_rows(delta, ctx.logit_rows, ctx.status)
            if residual is not None:
                residual = k.gather_rows(residual, ctx.logit_rows, ctx.status)
        return self.head.forward_after(delta, residual, self.final_norm, greedy)

    def emit(self, b) -> None:
        """The step as a program of the native executor (engine/native.py): what `forward` does,
        said once.  Raises NotNative where a part has no `emit`."""
        from ..engine.native import NotNative, OP_GATHER_ROWS
        for part in (self.embed, self.final_norm, self.head, *self.layers):
            if not hasattr(part, "emit") and not hasattr(part, "emit_after"):
                raise NotNative(f"{type(part).__name__} runs in Python only")
        if self.stream_encoding is not None:
            if not hasattr(self.stream_encoding, "emit"):
                raise NotNative(f"{type(self.stream_encoding).__name__} runs in Python only")
            delta, stream = self.stream_encoding.emit(b, self.embed.emit(b)), None
        else:
            delta, stream = self.embed.emit(b), None
        for pos, run in enumerate(self.schedule):
            delta, stream = self.layers[run.layer].emit(b, delta, stream, pos)
        b.wanted = True                                   # from here on: the wanted rows only
        picked = b.reg(b.cols(delta), b.dtype_of(delta))
        b.op(OP_GATHER_ROWS, in0=delta, out0=picked)
        picked_stream = None
        if stream is not None and stream != delta:
            picked_stream = b.reg(b.cols(stream), b.dtype_of(stream))
            b.op(OP_GATHER_ROWS, in0=stream, out0=picked_stream)
        self.head.emit_after(b, picked, picked_stream, self.final_norm)
