"""Grouped-query attention over a paged cache."""
from __future__ import annotations

from .base import Mixer, PagedKVSpec, PositionEncoding, Runtime
from .linear import Linear


class GQAAttention(Mixer):
    """softmax(scale * q k^T + causal mask) v with nh query heads sharing nkv key/value
    heads: query head h reads kv head h // (nh / nkv) (tamnd/fastmlx
    compute/models/llama.go:403-422; the grouping happens inside its fused call,
    mlxgo/binding_cgo.go:619-634).  Every query token sees the keys of its own request at
    positions <= its own (compute/models/batch_mask.go:33-41), or only the last `window`.

    The step writes this step's k and v into the pages first and then attends from the
    pages alone, so a token's result does not depend on how the tokens were cut into steps.
    With `share_kv=True` the part has no k/v projections and reads the cache of the
    schedule entry it is pointed at.
    """

    supports_cuda_graph = True

    def __init__(self, width: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 pos: PositionEncoding, name: str, bias: bool = False, scale: float | None = None,
                 window: int = 0, share_kv: bool = False,
                 proj_names=("q_proj", "k_proj", "v_proj", "o_proj")):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} query heads are no multiple of {num_kv_heads} kv heads")
        self.nh, self.nkv, self.hd = int(num_heads), int(num_kv_heads), int(head_dim)
        self.scale = float(scale) if scale is not None else float(head_dim) ** -0.5
        self.window = int(window)
        self.share_kv = bool(share_kv)
        self.pos = pos
        qn, kn, vn, on = (f"{name}.{p}" for p in proj_names)
        outs = [(qn, self.nh * self.hd)]
        if not share_kv:
            outs += [(kn, self.nkv * self.hd), (vn, self.nkv * self.hd)]
        self.qkv = Linear(width, outs, bias)
        self.o = Linear(self.nh * self.hd, [(on, width)], bias)

    def children(self):
        return (self.qkv, self.o, self.pos)

    def cache_spec(self):
        return PagedKVSpec(self.nkv, self.hd, self.window)

    def forward(self, x, ctx, cache):
        return self.o.forward(self._attend(self.qkv.forward(x), ctx, cache))

    def _attend(self, qkv, ctx, cache):
        k = self.rt.k
        fuses = getattr(k, "decode_attention_fuses_rope", None)
        rope = None
        if fuses is not None and fuses(qkv, cache.kv, ctx, self.nh, self.nkv, self.hd):
            rope = self.pos.fused_args(cache)
        if rope is not None:
            # decode steps: the attention kernel rotates q and the new k and stores k and v itself
            if self.share_kv:
                rope = rope[:3] + (False,)
            return k.paged_attention(qkv, cache.kv, ctx, ctx.groups[cache.group], self.nh, self.nkv, self.hd,
                                     self.scale, self.window, rope=rope)
        self.pos.apply_and_store(qkv, ctx, cache, self.nh, 0 if self.share_kv else self.nkv, self.hd)
        return self.rt.k.paged_attention(qkv, cache.kv, ctx, ctx.groups[cache.group],
                                         self.nh, self.nkv, self.hd, self.scale, self.window)

    def emit(self, b, x, pos):
        from ..engine.native import BF16, NotNative, OP_ATTENTION, _fn
        from ..kernels import lib as klib
        cache = b.manager.entries[pos]
        if cache.kv is None:
            raise NotNative("an attention layer without pages")
        inv_freq, rot, trad = self.pos.native_args()
        qkv = self.qkv.emit(b, x)
        out = b.reg(self.nh * self.hd)
        kv = cache.kv
        num_pages, page_size = kv.shape[0], kv.shape[3]
        fns = {}
        tc_ok = 0
        if b.act == BF16 and kv.dtype == self.rt.dtype and self.hd % 16 == 0 and self.hd <= 256:
            lib = klib.load(f"attn_hd{self.hd}")
            fns = dict(fn_attn_decode=_fn(lib, "fmx_attn_decode"), fn_attn_prefill=_fn(lib, "fmx_attn_prefill"),
                       fn_attn_prefill_tc=_fn(lib, "fmx_attn_prefill_tc"), fn_attn_plan=_fn(lib, "fmx_attn_decode_plan"),
                       fn_attn_prefill_tc_plan=_fn(lib, "fmx_attn_prefill_tc_plan_splits"))
            tc_ok = int(bool(lib.fmx_attn_prefill_tc_available())
                        and self.rt.k.tc_attention_ok(self.nh, self.nkv, self.hd, page_size, self.window))
        b.op(OP_ATTENTION, in0=qkv, out0=out, vec=b.ptr(inv_freq), nh=self.nh, nkv=self.nkv, hd=self.hd, window=self.window,
             rot=int(rot), trad=int(bool(trad)), store=int(bool(cache.writable and not self.share_kv)),
             share_kv=int(self.share_kv), group=cache.group, kv=b.ptr(kv), page_size=page_size, num_pages=num_pages,
             scale=self.scale, tc_attention_ok=tc_ok, **fns)
        b.release(qkv)
        o = self.o.emit(b, out)
        b.release(out)
        return o
