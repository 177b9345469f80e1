"""Host-side arithmetic of the kernels' work division, checked without a GPU."""


def test_short_prompts_go_to_the_library_product():
    """Fewer tiles than about a round of the SMs: the whole-tile kernel would leave most idle."""
    from fastmlx_b200 import kernels as k
    assert k.tc_fills_the_gpu(2048, 2048) and k.tc_fills_the_gpu(8192, 3072) and k.tc_fills_the_gpu(512, 16384)
    assert k.tc_fills_the_gpu(2048, 6144) and not k.tc_fills_the_gpu(2048, 3072)       # 192 tiles: 65 % of two rounds
    assert not k.tc_fills_the_gpu(512, 2048) and not k.tc_fills_the_gpu(1024, 3072) and not k.tc_fills_the_gpu(128, 8192)
