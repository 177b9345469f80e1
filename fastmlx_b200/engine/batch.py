"""The flat, ragged batch one step runs, and its device-side description."""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch


@dataclass
class StepEntry:
    """One request's share of a step: its next tokens (a portion of its prompt, or one
    decoded token) and the places among them whose logits are wanted."""
    request: object                    # cache.RequestCache
    tokens: list[int]
    want: list[int] = field(default_factory=list)


@dataclass
class GroupMeta:
    """Per cache group: where each token of the step is stored and where each row's
    pages are."""
    page_size: int
    block_tables: torch.Tensor         # int32 [R, max_blocks]; -1 = page given back / not there
    slot_mapping: torch.Tensor         # int64 [T]: page * page_size + offset of each token
    window: int = 0


@dataclass
class StepContext:
    """Everything the parts may read about the step.  Rows are requests; row r owns the
    tokens [row_start[r], row_start[r+1]) at positions row_ctx[r] ... ."""
    T: int
    R: int
    tokens: torch.Tensor               # int32 [T]
    positions: torch.Tensor            # int32 [T]
    token_row: torch.Tensor            # int32 [T]
    row_start: torch.Tensor            # int32 [R+1]
    row_ctx: torch.Tensor              # int32 [R]   tokens in the cache before this step
    row_slot: torch.Tensor             # int32 [R]   state slot of the row's request
    logit_rows: torch.Tensor | None    # int32 [n]   token indices whose logits are wanted
    status: torch.Tensor               # int32 [4]   kernels flag a bad id, slot or page here
    groups: list[GroupMeta]
    caches: list                       # cache.EntryCache per schedule entry
    # host copies, for mixers written in Python and for kernel dispatch
    h_row_start: list[int] = field(default_factory=list)
    h_row_ctx: list[int] = field(default_factory=list)
    h_row_slot: list[int] = field(default_factory=list)
    max_q_len: int = 0
    max_ctx_after: int = 0
    all_decode: bool = False           # every row brings exactly one token
    # a mixed step whose first rows bring one token each (the scheduler puts decoding requests first): how many,
    # the longest context among them, and the longest portion among the rest; 0 where the step is not mixed so
    decode_rows: int = 0
    decode_max_ctx: int = 0
    rest_max_q_len: int = 0
    rest_max_ctx: int = 0
    n_splits: int = 0                  # decode attention: fixed split count (0 = kernel's choice)
    scratch: dict = field(default_factory=dict)


class StaticBuffers:
    """The fixed device buffer of a captured decode graph (the same layout every step, so the
    graph's kernels always read the same addresses) and a small ring of pinned host buffers
    that feed it.  The host may run several steps ahead of the device: a host buffer is
    written again only after the copy that last read it has finished."""

    def __init__(self, ints: int, device, ring: int = 4):
        self.dev = torch.zeros(ints, dtype=torch.int32, device=device)
        self.hosts = [torch.zeros(ints, dtype=torch.int32).pin_memory() for _ in range(ring)]
        self.events = [None] * ring
        self.at = 0

    def next_host(self) -> torch.Tensor:
        self.at = (self.at + 1) % len(self.hosts)
        ev = self.events[self.at]
        if ev is not None:
            ev.synchronize()
        return self.hosts[self.at]

    def upload(self) -> torch.Tensor:
        self.dev.copy_(self.hosts[self.at], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self.events[self.at] = ev
        return self.dev


def leading_decode_rows(q_lens, ctxs) -> dict:
    """The one-token rows at the head of a mixed step, which attend on the split decode kernel
    while the portions behind them take the tiled one."""
    d = 0
    while d < len(q_lens) and q_lens[d] == 1:
        d += 1
    if d == 0 or d == len(q_lens):
        return {}
    return {"decode_rows": d, "decode_max_ctx": max(c + 1 for c in ctxs[:d]), "rest_max_q_len": max(q_lens[d:]),
            "rest_max_ctx": max(c + q for c, q in zip(ctxs[d:], q_lens[d:]))}


def build_context(entries, manager, device, status, *, pad_rows: int = 0, pad_blocks: int = 0,
                  pad_want: bool = False, static: StaticBuffers | None = None, pinned: bool = True) -> StepContext:
    """Lay the entries out as one flat batch.  Pages for the new tokens must have been
    reserved already.  One host buffer carries every integer array to the device.

    `pad_rows` / `pad_blocks` / `pad_want` fix the sizes (rows, block-table width, one
    wanted place per row) for a captured graph: padding rows bring one token at position
    -1 that is stored nowhere and sees no key, and their state slot is -1 (a mixer with
    state of its own skips them as attention skips position -1)."""
    R = len(entries)
    q_lens = [len(e.tokens) for e in entries]
    T = sum(q_lens)
    Rp = max(R, pad_rows)
    ngroups = len(manager.groups)
    ps = manager.page_size
    ctxs = [e.request.length for e in entries]
    max_blocks = max([1] + [-(-(c + q) // ps) for c, q in zip(ctxs, q_lens)] + [pad_blocks])
    Tp = T + (Rp - R)                  # padded rows bring one dummy token each

    want = []
    off = 0
    for e, q in zip(entries, q_lens):
        for w in e.want:
            if not 0 <= w < q:
                raise ValueError(f"wanted place {w} lies outside the {q} tokens of the entry")
            want.append(off + w)
        off += q
    if pad_want:
        if any(q != 1 for q in q_lens):
            raise ValueError("a padded batch holds one token per row")
        want = list(range(Tp))

    # layout of the packed int32 buffer
    sizes = {"tokens": Tp, "positions": Tp, "token_row": Tp, "row_start": Rp + 1, "row_ctx": Rp,
             "row_slot": Rp, "want": len(want)}
    for g in range(ngroups):
        sizes[f"bt{g}"] = Rp * max_blocks
        sizes[f"sm{g}"] = 2 * Tp       # int64 as two int32
    offs, total = {}, 0
    for k, n in sizes.items():
        total = (total + 3) // 4 * 4   # 16-byte alignment of every array
        offs[k] = total
        total += n
    if static is not None:
        if static.dev.numel() != total:
            raise ValueError("the static buffers were made for another layout")
        host = static.next_host().numpy()
        host[:] = 0
    else:
        host = np.zeros(total, dtype=np.int32)

    def view(k):
        return host[offs[k]: offs[k] + sizes[k]]

    tok, pos, trow = view("tokens"), view("positions"), view("token_row")
    rstart, rctx, rslot = view("row_start"), view("row_ctx"), view("row_slot")
    one_each = T == R
    slots = [e.request.slot for e in entries]
    if one_each:
        # one token per row: no per-row loop, the block tables come from the manager's mirror
        tok[:R] = [e.tokens[0] for e in entries]
        pos[:R] = ctxs
        trow[:Rp] = np.arange(Rp, dtype=np.int32)
        pos[R:Rp] = -1
        rstart[:Rp + 1] = np.arange(Rp + 1, dtype=np.int32)
        rctx[:R] = ctxs
        rslot[:R] = slots
        rslot[R:Rp] = -1
        view("want")[:] = want
        ctx_np = np.asarray(ctxs, dtype=np.int64)
        for g in range(ngroups):
            mirror = manager.table_mirror[g]
            w = min(max_blocks, mirror.shape[1])
            bt = view(f"bt{g}").reshape(Rp, max_blocks)
            bt[:] = -1
            bt[:R, :w] = mirror[slots, :w]
            sm = view(f"sm{g}").view(np.int64)
            sm[:] = -1
            sm[:R] = bt[np.arange(R), ctx_np // ps].astype(np.int64) * ps + ctx_np % ps
    off = 0
    for r, (e, q, c) in enumerate(zip(entries, q_lens, ctxs) if not one_each else ()):
        tok[off: off + q] = e.tokens
        pos[off: off + q] = np.arange(c, c + q, dtype=np.int32)
        trow[off: off + q] = r
        rstart[r], rctx[r], rslot[r] = off, c, e.request.slot
        off += q
    for r in range(R, Rp) if not one_each else ():   # padding rows: one token, no context, stored nowhere
        trow[off] = r
        pos[off] = -1
        rstart[r], rctx[r], rslot[r] = off, 0, -1
        off += 1
    if not one_each:
        rstart[Rp] = off
        view("want")[:] = want
    for g in range(ngroups) if not one_each else ():
        bt = view(f"bt{g}").reshape(Rp, max_blocks)
        bt[:] = -1
        sm = view(f"sm{g}").view(np.int64)
        sm[:] = -1
        off = 0
        for r, (e, q, c) in enumerate(zip(entries, q_lens, ctxs)):
            pages = e.request.tables[g].pages
            bt[r, :len(pages)] = pages
            p = np.arange(c, c + q)
            sm[off: off + q] = np.asarray(pages, dtype=np.int64)[p // ps] * ps + p % ps
            off += q

    if static is not None:
        dev = static.upload()
    else:
        t = torch.from_numpy(host)
        if device is not None and torch.device(device).type == "cuda":
            if pinned:
                t = t.pin_memory()
            dev = t.to(device, non_blocking=True)
        else:
            dev = t

    def dview(k):
        return dev[offs[k]: offs[k] + sizes[k]]

    groups = []
    for g in range(ngroups):
        groups.append(GroupMeta(ps, dview(f"bt{g}").view(Rp, max_blocks),
                                dview(f"sm{g}").view(torch.int64), manager.groups[g].spec.window))
    return StepContext(
        T=Tp, R=Rp, tokens=dview("tokens"), positions=dview("positions"), token_row=dview("token_row"),
        row_start=dview("row_start"), row_ctx=dview("row_ctx"), row_slot=dview("row_slot"),
        logit_rows=dview("want"), status=status, groups=groups, caches=manager.entries,
        h_row_start=rstart.tolist(), h_row_ctx=rctx.tolist(), h_row_slot=rslot.tolist(),
        max_q_len=max(q_lens + [1]), max_ctx_after=max([c + q for c, q in zip(ctxs, q_lens)] + [1]),
        all_decode=all(q == 1 for q in q_lens), scratch={"h2d_bytes": host.nbytes, "layout_ints": total},
        **leading_decode_rows(q_lens, ctxs))
