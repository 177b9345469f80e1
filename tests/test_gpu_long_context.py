"""The attention kernels over contexts of 4,096 to 8,192 keys, where the tile, page and split
index arithmetic, the order in which heavy tiles start and the lazy rescaling of the
tensor-memory kernel matter: each against the plain statement, with three kinds of input.

random      normal q, k, v: the ordinary tolerance of the kernel tests;
far key     one query and one key among thousands are scaled along a common direction so that
            this key's score dominates and its value row (all 7) is the answer: a tile, page or
            split edge that loses it shows at once;
counting    q = 0, so every visible key weighs 1/n exactly, and v marks the 64-key tile a key
            lies in: a tile that is dropped, counted twice or cut at the wrong causal edge
            changes an output by a large fraction of itself, and the tolerance is relative.
"""
import pytest
import torch

import plain_ops
from test_gpu_kernels import DEV, P_ROUNDING, _attention_case, _full_ctx, close, k

pytestmark = pytest.mark.gpu

# (query heads, kv heads, head size, page size): head sizes 64 and 128, four and three query heads per kv head
SHAPES = [(8, 2, 64, 16), (6, 2, 128, 16), (4, 1, 128, 64)]
DECODE_ROWS = [(8191, 1), (4095, 1), (4096, 1), (100, 1), (5000, 1)]
PREFILL_ROWS = [(4000, 130), (0, 2100), (8000, 70), (0, 1)]


def _ref(q, kv, rows, grp, nh, nkv, hd, scale):
    return plain_ops.paged_attention_by_rows(q, kv, rows, grp.block_tables, nh, nkv, hd, scale)


def _counting_inputs(dtype, nh, nkv, hd, page_size, rows):
    """q = 0 and v[j, :] = one-hot of (j // 64) % hd: an output holds, per 64-key tile class,
    the share of the visible keys that lie in it."""
    q, kv, ctx, grp = _attention_case(dtype, nh, nkv, hd, page_size, rows, seed=3)
    q.zero_()
    kv[:, 1] = 0
    for r, (c, ql) in enumerate(rows):
        for j0 in range(0, c + ql, page_size):
            page = int(grp.block_tables[r, j0 // page_size])
            for j in range(j0, min(j0 + page_size, c + ql)):
                kv[page, 1, :, j % page_size, (j // 64) % hd] = 1.0
    return q, kv, ctx, grp


def _run(kernel, q, kv, rows, ctx, grp, nh, nkv, hd, scale, **kw):
    dctx, dgrp = _full_ctx(rows, ctx, grp)
    kern = k()
    qd, kvd = q.to(DEV), kv.to(DEV)
    if kernel == "decode":
        got = kern.paged_attention_decode(qd, kvd, dctx, dgrp, nh, nkv, hd, scale, 0, **kw)
    elif kernel == "tc":
        assert kern.tc_attention_ok(nh, nkv, hd, kv.shape[3], 0)
        got = kern.paged_attention_prefill_tc(qd, kvd, dctx, dgrp, nh, nkv, hd, scale, **kw)
    elif kernel == "mma":
        got = kern.paged_attention_prefill(qd, kvd, dctx, dgrp, nh, nkv, hd, scale, 0)
    else:
        got = kern.paged_attention_simple(qd, kvd, dctx, dgrp, nh, nkv, hd, scale, 0)
    assert dctx.status.tolist()[0] == 0
    assert torch.isfinite(got).all()
    return got


# ----------------------------------------------------------------------------- decode
@pytest.mark.parametrize("nh,nkv,hd,page_size", SHAPES)
@pytest.mark.parametrize("splits", [None, 1, 7, 32])
def test_decode_random(nh, nkv, hd, page_size, splits):
    q, kv, ctx, grp = _attention_case(torch.bfloat16, nh, nkv, hd, page_size, DECODE_ROWS)
    ref = _ref(q, kv, DECODE_ROWS, grp, nh, nkv, hd, hd ** -0.5)
    got = _run("decode", q, kv, DECODE_ROWS, ctx, grp, nh, nkv, hd, hd ** -0.5, splits=splits)
    close(got, ref, torch.bfloat16, "decode over 8k keys", scale=1.0, extra=P_ROUNDING * kv.abs().max().item())


@pytest.mark.parametrize("nh,nkv,hd,page_size", SHAPES)
@pytest.mark.parametrize("key_pos", [0, 63, 4095, 4096, 8127, 8128, 8190, 8191])
def test_decode_far_key(nh, nkv, hd, page_size, key_pos):
    q, kv, ctx, grp = _attention_case(torch.bfloat16, nh, nkv, hd, page_size, DECODE_ROWS, spike=(0, key_pos, nh - 1))
    ref = _ref(q, kv, DECODE_ROWS, grp, nh, nkv, hd, 1.0)
    assert (ref[0, (nh - 1) * hd:].float() - 7.0).abs().max() < 0.1
    for splits in (None, 32):
        got = _run("decode", q, kv, DECODE_ROWS, ctx, grp, nh, nkv, hd, 1.0, splits=splits)
        close(got[:1], ref[:1], torch.bfloat16, f"far key {key_pos}, splits {splits}", scale=7.0)


@pytest.mark.parametrize("nh,nkv,hd,page_size", SHAPES)
@pytest.mark.parametrize("splits", [None, 5, 32])
def test_decode_counts_every_key_once(nh, nkv, hd, page_size, splits):
    q, kv, ctx, grp = _counting_inputs(torch.bfloat16, nh, nkv, hd, page_size, DECODE_ROWS)
    ref = _ref(q, kv, DECODE_ROWS, grp, nh, nkv, hd, hd ** -0.5)
    got = _run("decode", q, kv, DECODE_ROWS, ctx, grp, nh, nkv, hd, hd ** -0.5, splits=splits)
    close(got, ref, torch.bfloat16, "counting", scale=ref.abs().max().item())


def test_decode_32_bit_kernel():
    nh, nkv, hd, page_size = 4, 2, 32, 16
    q, kv, ctx, grp = _attention_case(torch.float32, nh, nkv, hd, page_size, DECODE_ROWS, spike=(0, 4096, 1))
    ref = _ref(q, kv, DECODE_ROWS, grp, nh, nkv, hd, 1.0)
    got = _run("simple", q, kv, DECODE_ROWS, ctx, grp, nh, nkv, hd, 1.0)
    close(got, ref, torch.float32, "32-bit attention over 8k keys", scale=7.0)


# ----------------------------------------------------------------------------- prompt portions
@pytest.mark.parametrize("nh,nkv,hd,page_size", SHAPES)
@pytest.mark.parametrize("kernel", ["tc2", "tc1", "mma"])
def test_prefill_random(nh, nkv, hd, page_size, kernel):
    q, kv, ctx, grp = _attention_case(torch.bfloat16, nh, nkv, hd, page_size, PREFILL_ROWS)
    ref = _ref(q, kv, PREFILL_ROWS, grp, nh, nkv, hd, hd ** -0.5)
    kw = {"variant": int(kernel[2])} if kernel.startswith("tc") else {}
    got = _run(kernel[:2] if kernel.startswith("tc") else kernel, q, kv, PREFILL_ROWS, ctx, grp, nh, nkv, hd, hd ** -0.5, **kw)
    close(got, ref, torch.bfloat16, "portions over 4k-8k keys", scale=1.0, extra=P_ROUNDING * kv.abs().max().item())


@pytest.mark.parametrize("nh,nkv,hd,page_size", SHAPES)
@pytest.mark.parametrize("kernel", ["tc2", "tc1", "mma"])
@pytest.mark.parametrize("token,key_pos", [(129, 0), (129, 4000), (129, 4129), (0, 4000), (130 + 2099, 1),
                                            (130 + 2099, 2048), (2230, 8000), (2299, 64)])
def test_prefill_far_key(nh, nkv, hd, page_size, kernel, token, key_pos):
    q, kv, ctx, grp = _attention_case(torch.bfloat16, nh, nkv, hd, page_size, PREFILL_ROWS, spike=(token, key_pos, 1))
    ref = _ref(q, kv, PREFILL_ROWS, grp, nh, nkv, hd, 1.0)
    assert (ref[token, hd:2 * hd].float() - 7.0).abs().max() < 0.1
    kw = {"variant": int(kernel[2])} if kernel.startswith("tc") else {}
    got = _run(kernel[:2] if kernel.startswith("tc") else kernel, q, kv, PREFILL_ROWS, ctx, grp, nh, nkv, hd, 1.0, **kw)
    close(got[token:token + 1], ref[token:token + 1], torch.bfloat16, f"far key {key_pos} for token {token}", scale=7.0)


@pytest.mark.parametrize("nh,nkv,hd,page_size", SHAPES)
@pytest.mark.parametrize("kernel", ["tc2", "tc1", "mma"])
def test_prefill_counts_every_key_once(nh, nkv, hd, page_size, kernel):
    q, kv, ctx, grp = _counting_inputs(torch.bfloat16, nh, nkv, hd, page_size, PREFILL_ROWS)
    ref = _ref(q, kv, PREFILL_ROWS, grp, nh, nkv, hd, hd ** -0.5)
    kw = {"variant": int(kernel[2])} if kernel.startswith("tc") else {}
    got = _run(kernel[:2] if kernel.startswith("tc") else kernel, q, kv, PREFILL_ROWS, ctx, grp, nh, nkv, hd, hd ** -0.5, **kw)
    # every row of the result is compared at its own scale: early tokens of a prompt see few keys
    # and their shares are large, late ones see thousands
    for t in range(0, ref.shape[0], 97):
        close(got[t:t + 1], ref[t:t + 1], torch.bfloat16, f"counting, token {t}", scale=ref[t].abs().max().item())
    close(got, ref, torch.bfloat16, "counting", scale=1.0)


def test_prefill_32_bit_kernel():
    nh, nkv, hd, page_size = 2, 1, 32, 16
    rows = [(4000, 40), (0, 300)]
    q, kv, ctx, grp = _attention_case(torch.float32, nh, nkv, hd, page_size, rows, spike=(39, 3999, 1))
    ref = _ref(q, kv, rows, grp, nh, nkv, hd, 1.0)
    got = _run("simple", q, kv, rows, ctx, grp, nh, nkv, hd, 1.0)
    close(got, ref, torch.float32, "32-bit attention, portions over 4k keys", scale=7.0)
