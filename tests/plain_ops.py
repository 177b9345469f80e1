"""Plain PyTorch statements of every kernel, with the kernels' own signatures.

Two uses.  The GPU tests run each CUDA kernel alone against the function of the same name
here.  The CPU tests put this module in the place of `fastmlx_b200.kernels`, so that the
cache manager, the step function, the scheduler and the replay program can be checked
against the plain model without a GPU.  It is test code: nothing in the package imports it.
"""
from __future__ import annotations

import torch

F64 = torch.float64


def gather_rows(table, ids, status, code=4):
    return table[ids.long()].clone()


def embedding(ids, table, status, out_dtype=None):
    if ((ids < 0) | (ids >= table.shape[0])).any():
        status[0] = 1
        ids = ids.clamp(0, table.shape[0] - 1)
    out = table[ids.long()].clone()
    return out.to(out_dtype) if out_dtype is not None else out


def add_rmsnorm(x, residual, weight, eps, stream_dtype=None, out_dtype=None):
    act = x.dtype if x is not None else (out_dtype or residual.dtype)
    if residual is not None:
        h = residual.to(F64) if x is None else (x.to(F64) + residual.to(F64))
        residual.copy_(h.to(residual.dtype))
    elif stream_dtype is not None and stream_dtype != act:
        residual = x.to(stream_dtype)
    else:
        residual = x
    h = residual.to(F64)
    out = h * torch.rsqrt((h * h).mean(-1, keepdim=True) + eps) * weight.to(F64)
    return out.to(act), residual


def silu_mul(gate_up, block=None):
    inter = gate_up.shape[1] // 2
    b = block or inter
    v = gate_up.reshape(gate_up.shape[0], inter // b, 2, b).to(F64)
    g, u = v[:, :, 0, :].reshape(-1, inter), v[:, :, 1, :].reshape(-1, inter)
    return (g * torch.sigmoid(g) * u).to(gate_up.dtype)


def linear(x, w, bias, out_dtype):
    y = x.to(F64) @ w.to(F64).t()
    if bias is not None:
        y = y + bias.to(F64)
    return y.to(out_dtype)


gemm_simple = linear


def rope_kv_write(qkv, positions, inv_freq, rotary_dim, traditional, slot_mapping, kv, nh, nkv, hd, status):
    T = qkv.shape[0]
    if rotary_dim > 0:
        ang = (positions.to(torch.float32)[:, None] * inv_freq.to(torch.float32)[None, :]).to(F64)
        cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        heads = qkv[:, :(nh + nkv) * hd].reshape(T, nh + nkv, hd).to(F64)
        out = heads.clone()
        r = rotary_dim
        if traditional:
            a, b = heads[..., 0:r:2], heads[..., 1:r:2]
            out[..., 0:r:2] = a * cos - b * sin
            out[..., 1:r:2] = b * cos + a * sin
        else:
            a, b = heads[..., :r // 2], heads[..., r // 2:r]
            out[..., :r // 2] = a * cos - b * sin
            out[..., r // 2:r] = b * cos + a * sin
        qkv[:, :(nh + nkv) * hd] = out.reshape(T, -1).to(qkv.dtype)
    if kv is None or slot_mapping is None or nkv == 0:
        return
    page_size = kv.shape[3]
    k = qkv[:, nh * hd:(nh + nkv) * hd].reshape(T, nkv, hd)
    v = qkv[:, (nh + nkv) * hd:(nh + 2 * nkv) * hd].reshape(T, nkv, hd)
    for t in range(T):
        s = int(slot_mapping[t])
        if s < 0:
            continue
        if s >= kv.shape[0] * page_size:
            status[0] = 2
            continue
        kv[s // page_size, 0, :, s % page_size, :] = k[t]
        kv[s // page_size, 1, :, s % page_size, :] = v[t]


def paged_attention(qkv, kv, ctx, group, nh, nkv, hd, scale, window):
    """Each token attends over the pages of its own row, keys lo..position."""
    T = qkv.shape[0]
    page_size = kv.shape[3]
    out = torch.zeros(T, nh * hd, dtype=F64)
    q = qkv[:, :nh * hd].reshape(T, nh, hd).to(F64)
    rep = nh // nkv
    for t in range(T):
        pos = int(ctx.positions[t])
        if pos < 0:
            continue
        bt = group.block_tables[int(ctx.token_row[t])]
        lo = max(0, pos - window + 1) if window > 0 else 0
        js = torch.arange(lo, pos + 1)
        pages = bt[(js // page_size).long()].long()
        if (pages < 0).any():
            ctx.status[0] = 3
            continue
        K = kv[pages, 0, :, (js % page_size).long(), :].to(F64)       # [n, nkv, hd]
        V = kv[pages, 1, :, (js % page_size).long(), :].to(F64)
        for h in range(nh):
            s = (K[:, h // rep, :] @ q[t, h]) * scale
            p = torch.softmax(s, dim=0)
            out[t, h * hd:(h + 1) * hd] = p @ V[:, h // rep, :]
    return out.to(qkv.dtype)


paged_attention_simple = paged_attention


def sample(logits, temperature=None, uniform=None, keep=None):
    rows, V = logits.shape
    out = torch.empty(rows, dtype=torch.int32)
    for r in range(rows):
        row = logits[r].to(F64).clone()
        if keep is not None:
            row[keep[r] == 0] = float("-inf")
        T = float(temperature[r]) if temperature is not None else 0.0
        top = int(torch.argmax(row))          # torch returns the first maximal index
        if not T > 0:
            out[r] = top
            continue
        w = torch.exp((row - row[top]) / T)
        c = torch.cumsum(w, 0)
        target = float(uniform[r]) * float(c[-1])
        idx = int(torch.searchsorted(c, torch.tensor(target, dtype=F64), right=True))
        out[r] = min(idx, V - 1)
    return out


def argmax(logits):
    return sample(logits)


def paged_attention_by_rows(q, kv, rows, block_tables, nh, nkv, hd, scale, window=0):
    """The same statement as `paged_attention`, one request at a time instead of one token at a
    time, for contexts of thousands of keys.  rows: (keys before this step, tokens of this
    step) per request; q [T, nh*hd] holds the steps' tokens in row order.  float64 on the CPU."""
    page_size = kv.shape[3]
    out = torch.zeros(q.shape[0], nh * hd, dtype=F64)
    rep = nh // nkv
    at = 0
    for r, (c, ql) in enumerate(rows):
        n = c + ql
        js = torch.arange(n)
        pages = block_tables[r][(js // page_size).long()].long()
        assert (pages >= 0).all()
        K = kv[pages, 0, :, (js % page_size).long(), :].to(F64)       # [n, nkv, hd]
        V = kv[pages, 1, :, (js % page_size).long(), :].to(F64)
        qi = torch.arange(c, n)
        visible = js[None, :] <= qi[:, None]
        if window > 0:
            visible &= js[None, :] > (qi[:, None] - window)
        qr = q[at:at + ql].reshape(ql, nh, hd).to(F64)
        for h in range(nh):
            s = (qr[:, h, :] @ K[:, h // rep, :].t()) * scale
            s = s.masked_fill(~visible, float("-inf"))
            out[at:at + ql, h * hd:(h + 1) * hd] = torch.softmax(s, dim=-1) @ V[:, h // rep, :]
        at += ql
    return out.to(q.dtype)
