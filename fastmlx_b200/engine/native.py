"""The native step executor's Python side: a model's parts describe themselves once as a
program, and a step then costs one call into compiled code.

tamnd/fastmlx's loop is compiled code (enginecore/core.go:134-171, scheduler/scheduler.go:126-154).
Here the scheduler stays in Python, but what runs per step on the host (the batch layout, one
host-to-device copy, the choice of kernel for every operation and a hundred and more launches)
is `csrc/host/step_executor.cu`.  A model takes this path when every one of its parts has an
`emit` method (the stock parts have); a model with a part that has none (a part written in Python
against the interfaces of `parts/base.py`) runs through `Model.forward` as before.

`ProgramBuilder` is what `emit` methods write to: numbered activation buffers ("registers",
each a number of columns and a type; the rows are the step's tokens) and operations over them.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_longlong, c_void_p

import numpy as np
import torch

from ..kernels import lib as _klib

MAX_GROUPS = 8
OP_EMBED, OP_ADD_RMSNORM, OP_LINEAR, OP_GATE_UP, OP_ATTENTION, OP_GATHER_ROWS = range(6)
LOGITS = -2                 # an operation's out0: the step's logits
F32, BF16 = 0, 1


class NotNative(Exception):
    """A part cannot describe itself to the native executor: the model runs through Python."""


class FmxReg(Structure):
    _fields_ = [("cols", c_int), ("dtype", c_int)]


class FmxOp(Structure):
    _fields_ = [("kind", c_int), ("in0", c_int), ("in1", c_int), ("out0", c_int), ("out1", c_int),
                ("wanted_rows", c_int), ("w", c_void_p), ("bias", c_void_p), ("vec", c_void_p), ("w_dtype", c_int),
                ("ldw", c_longlong), ("n", c_int), ("k", c_int), ("out_dtype", c_int), ("block", c_int),
                ("eps", c_float), ("scale", c_float), ("table_rows", c_longlong), ("init", c_int),
                ("nh", c_int), ("nkv", c_int), ("hd", c_int), ("window", c_int), ("rot", c_int), ("trad", c_int),
                ("store", c_int), ("group", c_int), ("share_kv", c_int), ("kv", c_void_p), ("page_size", c_int),
                ("num_pages", c_longlong), ("fn_attn_decode", c_void_p), ("fn_attn_prefill", c_void_p),
                ("fn_attn_prefill_tc", c_void_p), ("fn_attn_plan", c_void_p), ("fn_attn_prefill_tc_plan", c_void_p),
                ("tc_attention_ok", c_int)]


class FmxKernelTable(Structure):
    _fields_ = [(n, c_void_p) for n in ("gather_rows", "gather_rows_f32_to_bf16", "add_rmsnorm", "silu_mul", "gemm_simple",
                                        "rope_kv_write", "paged_attention_simple", "fill_rows", "gemv", "gemm_tcgen05",
                                        "gemm_tcgen05_plan_fills", "gemv_argmax")]


class FmxStepDesc(Structure):
    _fields_ = [("T", c_int), ("R", c_int), ("n_want", c_int), ("max_q_len", c_int), ("max_ctx_after", c_int),
                ("all_decode", c_int), ("n_splits", c_int), ("n_groups", c_int),
                ("decode_rows", c_int), ("decode_max_ctx", c_int), ("rest_max_q_len", c_int), ("rest_max_ctx", c_int),
                ("tokens", c_void_p), ("positions", c_void_p), ("token_row", c_void_p), ("row_start", c_void_p),
                ("row_ctx", c_void_p), ("row_slot", c_void_p), ("want", c_void_p),
                ("block_tables", c_void_p * MAX_GROUPS), ("bt_stride", c_int * MAX_GROUPS),
                ("slot_mapping", c_void_p * MAX_GROUPS), ("status", c_void_p), ("arena", c_void_p),
                ("arena_bytes", c_longlong), ("logits", c_void_p), ("attn_scratch", c_void_p),
                ("attn_scratch_floats", c_longlong), ("attn_tickets", c_void_p), ("attn_tickets_n", c_int),
                ("greedy_ids", c_void_p), ("greedy_best", c_void_p), ("greedy_ticket", c_void_p)]


class FmxBatchIn(Structure):
    _fields_ = [("R", c_int), ("q_lens", c_void_p), ("ctx_lens", c_void_p), ("slots", c_void_p), ("tokens", c_void_p),
                ("n_want", c_int), ("want", c_void_p), ("pad_rows", c_int), ("pad_blocks", c_int), ("page_size", c_int),
                ("n_groups", c_int), ("mirror", c_void_p * MAX_GROUPS), ("mirror_cols", c_int * MAX_GROUPS)]


def _fn(lib, name):
    return ctypes.cast(getattr(lib, name), c_void_p).value


def _dt(dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise NotNative(f"the native executor computes in float32 or bfloat16, not {dtype}")


_host_lib = None


def host_library():
    """libfmx_host.so with its entry points declared."""
    global _host_lib
    if _host_lib is None:
        lib = _klib.load("host")
        lib.fmx_exec_create.argtypes = [POINTER(FmxOp), c_int, POINTER(FmxReg), c_int, POINTER(FmxKernelTable), c_int,
                                        c_char_p, c_void_p, c_longlong]
        lib.fmx_exec_create.restype = c_void_p
        lib.fmx_exec_destroy.argtypes = [c_void_p]
        lib.fmx_exec_destroy.restype = None
        lib.fmx_exec_arena_bytes.argtypes = [c_void_p, c_int]
        lib.fmx_exec_arena_bytes.restype = c_longlong
        lib.fmx_exec_layout_ints.argtypes = [POINTER(FmxBatchIn)]
        lib.fmx_exec_layout_ints.restype = c_longlong
        lib.fmx_exec_layout.argtypes = [POINTER(FmxBatchIn), c_void_p, c_void_p, c_longlong, POINTER(FmxStepDesc), c_void_p]
        lib.fmx_exec_layout.restype = c_int
        lib.fmx_exec_forward.argtypes = [c_void_p, POINTER(FmxStepDesc), c_void_p]
        lib.fmx_exec_forward.restype = c_int
        lib.fmx_exec_launches.argtypes = [c_void_p]
        lib.fmx_exec_launches.restype = c_longlong
        sizes = (c_int * 5)()
        lib.fmx_exec_struct_sizes(sizes)
        mine = [ctypes.sizeof(t) for t in (FmxOp, FmxStepDesc, FmxBatchIn, FmxKernelTable, FmxReg)]
        if list(sizes) != mine:
            raise _klib.KernelError(f"the step executor's structures measure {list(sizes)} bytes, their mirrors here {mine}")
        _host_lib = lib
    return _host_lib


class ProgramBuilder:
    """What the parts' `emit` methods write to.  `reg` hands out a register of so many columns
    (one that an earlier `release` gave back, where one fits), `op` appends an operation."""

    def __init__(self, rt, manager):
        self.rt, self.manager = rt, manager
        self.act = _dt(rt.dtype)
        self.regs: list[tuple[int, int]] = []
        self.ops: list[FmxOp] = []
        self.keep: list = []                       # tensors whose addresses the program holds
        self._free: dict[tuple[int, int], list[int]] = {}
        self.wanted = False                        # operations from here on run over the wanted rows only
        self.greedy_head_ok = False                # the head may choose greedily inside its product

    def reg(self, cols: int, dtype=None) -> int:
        key = (int(cols), self.act if dtype is None else _dt(dtype) if not isinstance(dtype, int) else dtype)
        free = self._free.get(key)
        if free:
            return free.pop()
        self.regs.append(key)
        return len(self.regs) - 1

    def release(self, r: int) -> None:
        if r is not None and r >= 0:
            self._free.setdefault(self.regs[r], []).append(r)

    def cols(self, r: int) -> int:
        return self.regs[r][0]

    def dtype_of(self, r: int) -> int:
        return self.regs[r][1]

    def ptr(self, t):
        """The address of a device tensor the program will read every step."""
        if t is None:
            return None
        if not t.is_cuda or not t.is_contiguous():
            raise NotNative("the native executor reads contiguous device tensors")
        self.keep.append(t)
        return t.data_ptr()

    def op(self, kind: int, **fields) -> FmxOp:
        o = FmxOp()
        o.kind, o.in0, o.in1, o.out0, o.out1 = kind, -1, -1, -1, -1
        o.wanted_rows = 1 if self.wanted else 0
        o.group = -1
        for name, value in fields.items():
            setattr(o, name, value)
        self.ops.append(o)
        return o


class _Buffers:
    """Pinned host buffers in a ring and one device buffer for the packed description of a
    step; a host buffer is written again only after the copy that last read it has finished."""

    def __init__(self, ints: int, device, ring: int = 4):
        self.ints = ints
        self.dev = torch.empty(ints, dtype=torch.int32, device=device)
        self.hosts = [torch.empty(ints, dtype=torch.int32).pin_memory() for _ in range(ring)]
        self.events = [None] * ring
        self.at = 0

    def next_host(self) -> torch.Tensor:
        self.at = (self.at + 1) % len(self.hosts)
        ev = self.events[self.at]
        if ev is not None:
            ev.synchronize()
        return self.hosts[self.at]

    def mark(self) -> None:
        ev = self.events[self.at]
        if ev is None:
            ev = self.events[self.at] = torch.cuda.Event()
        ev.record()


class StepInfo:
    """What the step function keeps of a step that the native executor ran."""

    def __init__(self, T: int, h2d_bytes: int):
        self.T = T
        self.scratch = {"h2d_bytes": h2d_bytes}


class NativeProgram:
    """A model's step as a program of the native executor, with the buffers it runs in."""

    CUBLAS_WORKSPACE = 32 << 20
    GRAPH_ROWS = 256                 # the fixed arena of captured steps holds this many tokens

    def __init__(self, model, manager, rt, status: torch.Tensor, graph_rows: int = 256):
        if rt.device.type != "cuda":
            raise NotNative("the native executor drives CUDA kernels")
        if len(manager.groups) > MAX_GROUPS:
            raise NotNative(f"the native executor takes up to {MAX_GROUPS} cache groups")
        self.model, self.manager, self.rt, self.status = model, manager, rt, status
        self.lib = host_library()
        b = ProgramBuilder(rt, manager)
        model.emit(b)                                  # raises NotNative where a part cannot describe itself
        self.builder = b
        k = rt.k
        table = FmxKernelTable()
        common = _klib.load("common")
        for name in ("gather_rows", "gather_rows_f32_to_bf16", "add_rmsnorm", "silu_mul", "gemm_simple", "rope_kv_write",
                     "paged_attention_simple", "fill_rows"):
            setattr(table, name, _fn(common, "fmx_" + name))
        if rt.dtype == torch.bfloat16:
            setattr(table, "gemv", _fn(_klib.load("bf16"), "fmx_gemv"))
            table.gemv_argmax = _fn(_klib.load("bf16"), "fmx_gemv_argmax")
            tc = _klib.load("tc")
            table.gemm_tcgen05 = _fn(tc, "fmx_gemm_tcgen05")
            table.gemm_tcgen05_plan_fills = _fn(tc, "fmx_gemm_tcgen05_plan_fills")
        self._ops = (FmxOp * len(b.ops))(*b.ops)
        self._regs = (FmxReg * len(b.regs))(*[FmxReg(c, d) for c, d in b.regs])
        self._blas_ws = torch.empty(self.CUBLAS_WORKSPACE, dtype=torch.uint8, device=rt.device)
        path = os.path.join(os.path.dirname(torch.__file__), "..", "nvidia", "cublas", "lib", "libcublas.so.12")
        self.handle = self.lib.fmx_exec_create(self._ops, len(b.ops), self._regs, len(b.regs), ctypes.byref(table),
                                               k.num_sms(rt.device), os.path.normpath(path).encode(),
                                               self._blas_ws.data_ptr(), self._blas_ws.numel())
        if not self.handle:
            raise _klib.KernelError(self.lib.fmx_last_error().decode(errors="replace"))
        self.vocab = model.vocab_size
        self.greedy_ok = bool(b.greedy_head_ok and rt.dtype == torch.bfloat16)
        self.greedy_ws = k.greedy_workspace(rt.device) if self.greedy_ok else None
        self.scratch = k.attention_scratch(rt.device)
        self.tickets = k.attention_tickets(rt.device)
        self.graph_rows = int(graph_rows)
        self.graph_arena = self._arena(self.graph_rows)       # captured steps hold its address: never replaced
        self.arena_tokens = max(self.graph_rows, 2048)
        self.arena = self._arena(self.arena_tokens)
        self.buffers = None
        self._counted = 0

    def __del__(self):
        try:
            if getattr(self, "handle", None):
                self.lib.fmx_exec_destroy(self.handle)
                self.handle = None
        except Exception:
            pass

    def _arena(self, tokens: int) -> torch.Tensor:
        return torch.empty(self.lib.fmx_exec_arena_bytes(self.handle, int(tokens)), dtype=torch.uint8, device=self.rt.device)

    def _count(self) -> None:
        n = self.lib.fmx_exec_launches(self.handle)
        _klib.launches += n - self._counted
        self._counted = n

    def _check(self, rc: int) -> None:
        if rc != 0:
            raise _klib.KernelError(self.lib.fmx_last_error().decode(errors="replace"))

    def _finish_desc(self, d: FmxStepDesc, arena: torch.Tensor, n_want: int, greedy: bool = False):
        """-> (the step's result tensor, whether the ids still have to be chosen from it)."""
        fused = greedy and self.greedy_ok and 0 < n_want <= getattr(self.rt.k, "GREEDY_HEAD_MAX_ROWS", 8)
        if fused:
            result = torch.empty(n_want, dtype=torch.int32, device=self.rt.device)
            d.greedy_ids = result.data_ptr()
            d.greedy_best, d.greedy_ticket = self.greedy_ws[0].data_ptr(), self.greedy_ws[1].data_ptr()
        else:
            result = torch.empty((n_want, self.vocab), dtype=torch.float32, device=self.rt.device)
            d.logits = result.data_ptr()
        d.status = self.status.data_ptr()
        d.arena, d.arena_bytes = arena.data_ptr(), arena.numel()
        d.attn_scratch, d.attn_scratch_floats = self.scratch.data_ptr(), self.scratch.numel()
        d.attn_tickets, d.attn_tickets_n = self.tickets.data_ptr(), self.tickets.numel()
        return result, greedy and not fused

    def _result(self, result, choose: bool):
        return self.rt.k.argmax(result) if choose and result.shape[0] else \
            (torch.empty(0, dtype=torch.int32, device=self.rt.device) if choose else result)

    # ------------------------------------------------------------------ a step the Python side has laid out
    def forward_context(self, ctx, greedy: bool = False) -> torch.Tensor:
        """Run the program over a `StepContext` (the captured decode steps are laid out by
        `build_context` into their graph's fixed buffers).  `greedy`: -> the wanted rows' greedy
        choices (int32) instead of their logits."""
        d = FmxStepDesc()
        n_want = int(ctx.logit_rows.numel()) if ctx.logit_rows is not None else 0
        d.T, d.R, d.n_want = ctx.T, ctx.R, n_want
        d.max_q_len, d.max_ctx_after = int(ctx.max_q_len), int(ctx.max_ctx_after)
        d.all_decode, d.n_splits, d.n_groups = int(bool(ctx.all_decode)), int(ctx.n_splits), len(ctx.groups)
        d.decode_rows, d.decode_max_ctx, d.rest_max_q_len = (int(getattr(ctx, "decode_rows", 0)), int(getattr(ctx, "decode_max_ctx", 0)),
                                                             int(getattr(ctx, "rest_max_q_len", 0)))
        d.rest_max_ctx = int(getattr(ctx, "rest_max_ctx", 0))
        d.tokens, d.positions, d.token_row = ctx.tokens.data_ptr(), ctx.positions.data_ptr(), ctx.token_row.data_ptr()
        d.row_start, d.row_ctx, d.row_slot = ctx.row_start.data_ptr(), ctx.row_ctx.data_ptr(), ctx.row_slot.data_ptr()
        d.want = ctx.logit_rows.data_ptr() if n_want else None
        for g, meta in enumerate(ctx.groups):
            d.block_tables[g] = meta.block_tables.data_ptr()
            d.bt_stride[g] = meta.block_tables.stride(0)
            d.slot_mapping[g] = meta.slot_mapping.data_ptr()
        capturing = torch.cuda.is_current_stream_capturing()
        if ctx.T <= self.graph_rows:
            arena = self.graph_arena
        elif capturing:
            raise _klib.KernelError(f"a captured step holds at most {self.graph_rows} tokens")
        else:
            arena = self._big_arena(ctx.T)
        result, choose = self._finish_desc(d, arena, n_want, greedy)
        self._check(self.lib.fmx_exec_forward(self.handle, ctypes.byref(d), torch.cuda.current_stream().cuda_stream))
        self._count()
        return self._result(result, choose)

    def _big_arena(self, T: int) -> torch.Tensor:
        if T > self.arena_tokens:
            # nothing holds the old one's address once its steps have run: the allocator hands its
            # memory on only to work that comes after them on this stream
            self.arena_tokens = max(int(T), 2 * self.arena_tokens)
            self.arena = self._arena(self.arena_tokens)
        return self.arena

    # ------------------------------------------------------------------ a step from its entries
    def step(self, entries, greedy: bool = False) -> tuple[torch.Tensor, StepInfo]:
        """Lay the entries out, copy the description to the device and run the program: one
        call into compiled code.  Pages for the new tokens must have been reserved."""
        R = len(entries)
        q_lens = [len(e.tokens) for e in entries]
        head = q_lens + [e.request.length for e in entries] + [e.request.slot for e in entries]
        want, off = [], 0
        for e, q in zip(entries, q_lens):
            for w in e.want:
                if not 0 <= w < q:
                    raise ValueError(f"wanted place {w} lies outside the {q} tokens of the entry")
                want.append(off + w)
            off += q
        flat = np.empty(3 * R + len(want) + off, dtype=np.int32)
        flat[:3 * R] = head
        flat[3 * R: 3 * R + len(want)] = want
        at = 3 * R + len(want)
        for e, q in zip(entries, q_lens):
            flat[at: at + q] = e.tokens
            at += q
        base = flat.ctypes.data
        inp = FmxBatchIn()
        inp.R, inp.n_want = R, len(want)
        inp.q_lens, inp.ctx_lens, inp.slots = base, base + 4 * R, base + 8 * R
        inp.want, inp.tokens = base + 12 * R, base + 4 * (3 * R + len(want))
        inp.pad_rows = inp.pad_blocks = 0
        inp.page_size, inp.n_groups = self.manager.page_size, len(self.manager.groups)
        for g, m in enumerate(self.manager.table_mirror):
            inp.mirror[g], inp.mirror_cols[g] = m.ctypes.data, m.shape[1]
        ints = self.lib.fmx_exec_layout_ints(ctypes.byref(inp))
        if ints < 0:
            self._check(1)
        if self.buffers is None or self.buffers.ints < ints:
            if self.buffers is not None:
                torch.cuda.current_stream().synchronize()        # copies out of the old pinned buffers have landed
            self.buffers = _Buffers(max(2 * int(ints), 1 << 14), self.rt.device)
        host = self.buffers.next_host()
        d = FmxStepDesc()
        stream = torch.cuda.current_stream().cuda_stream
        self._check(self.lib.fmx_exec_layout(ctypes.byref(inp), host.data_ptr(), self.buffers.dev.data_ptr(),
                                             self.buffers.ints, ctypes.byref(d), stream))
        self.buffers.mark()
        result, choose = self._finish_desc(d, self._big_arena(d.T), len(want), greedy)
        self._check(self.lib.fmx_exec_forward(self.handle, ctypes.byref(d), stream))
        self._count()
        return self._result(result, choose), StepInfo(d.T, int(ints) * 4)


def build_program(model, manager, rt, status, graph_rows: int = 256):
    """-> a NativeProgram, or None when the model has a part that only Python can run."""
    if not hasattr(model, "emit"):
        return None
    try:
        return NativeProgram(model, manager, rt, status, graph_rows)
    except NotNative:
        return None
