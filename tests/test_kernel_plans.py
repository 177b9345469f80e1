"""Host-side arithmetic of the kernels' work division, checked without a GPU."""


def test_stream_plan_covers_every_unit_once():
    """The arithmetic that cuts units into CTA ranges and finds a tile's contributors, redone
    on the host for shapes where ranges start and end inside tiles."""
    from fastmlx_b200 import kernels as k
    assert k.stream_plan(8, 2048, 2048, False) == (148, 3, 148 * 2 * 8 * 128, 16)
    assert k.stream_plan(8, 16384, 2048, True) == (148, 3, 148 * 2 * 2 * 8 * 128, 64)
    assert k.stream_plan(64, 256, 64, False)[0] == 2
    for tiles, kb, ctas in [(16, 32, 148), (64, 32, 148), (1, 3, 2), (7, 5, 4), (1002, 32, 148), (3, 1, 3), (5, 128, 148)]:
        total = tiles * kb
        ctas = min(ctas, total)
        start = lambda c: c * total // ctas
        owner = []
        for c in range(ctas):
            owner += [c] * (start(c + 1) - start(c))
        assert len(owner) == total and all(start(c + 1) > start(c) for c in range(ctas))
        for t in range(tiles):
            t0, t1 = t * kb, t * kb + kb - 1
            c_lo, c_hi = min((t0 + 1) * ctas // total, ctas - 1), min((t1 + 1) * ctas // total, ctas - 1)
            while c_lo > 0 and start(c_lo) > t0: c_lo -= 1
            while c_lo + 1 < ctas and start(c_lo + 1) <= t0: c_lo += 1
            while c_hi > 0 and start(c_hi) > t1: c_hi -= 1
            while c_hi + 1 < ctas and start(c_hi + 1) <= t1: c_hi += 1
            assert (c_lo, c_hi) == (owner[t0], owner[t1])
            assert sorted(set(owner[t0:t1 + 1])) == list(range(c_lo, c_hi + 1))


def test_short_prompts_go_to_the_library_product():
    """Fewer tiles than about a round of the SMs: the whole-tile kernel would leave most idle."""
    from fastmlx_b200 import kernels as k
    assert k.tc_fills_the_gpu(2048, 2048) and k.tc_fills_the_gpu(8192, 3072) and k.tc_fills_the_gpu(512, 16384)
    assert k.tc_fills_the_gpu(2048, 6144) and not k.tc_fills_the_gpu(2048, 3072)       # 192 tiles: 65 % of two rounds
    assert not k.tc_fills_the_gpu(512, 2048) and not k.tc_fills_the_gpu(1024, 3072) and not k.tc_fills_the_gpu(128, 8192)
