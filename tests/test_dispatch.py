"""Host-side choices of the kernel dispatcher that need no GPU."""

from mlx_omnia_b200.kernels import ops


def test_width_bucket_keeps_three_bits_and_is_its_own_fixed_point():
    assert [ops.width_bucket(n) for n in (0, 1, 8, 9, 16, 17, 100, 256, 257, 5000)] == \
        [8, 8, 8, 10, 16, 20, 112, 256, 320, 5120]
    for n in range(1, 3000, 7):
        b = ops.width_bucket(n)
        assert n <= b <= max(8, n + n // 4) and ops.width_bucket(b) == b


def test_decode_plan_is_a_tile_multiple_within_bounds_and_the_same_for_a_bucket():
    for requests in (1, 3, 8, 17, 64, 100, 512):
        for nkv in (1, 3, 8):
            for longest in (1, 90, 128, 1000, 4096, 5000, 100000):
                chunk, warps = ops.decode_plan(requests, nkv, longest)
                assert 128 <= chunk <= 1024 and chunk % 64 == 0 and warps in (1, 4)
                # A captured graph's batch is a power of two: same plan.
                assert (chunk, warps) == ops.decode_plan(1 << (requests - 1).bit_length(), nkv, longest)


def test_decode_plan_grows_with_the_work():
    """Few pairs: short chunks and four warps a block, so that enough warps run; more pairs: one
    warp a block and the shortest chunk whose blocks the GPU holds at a time."""
    assert ops.decode_plan(1, 8, 4096) == (256, 4)
    assert ops.decode_plan(2, 8, 4096) == (256, 4)
    assert ops.decode_plan(4, 8, 4096) == (192, 1)
    assert ops.decode_plan(8, 8, 4096) == (320, 1)
    assert ops.decode_plan(8, 8, 5120) == (448, 1)
    assert ops.decode_plan(16, 8, 4096) == (704, 1)
    assert ops.decode_plan(64, 8, 8192) == (1024, 1)
    # One long request: four warps a block, chunks so long that two blocks an SM hold them all.
    chunk, warps = ops.decode_plan(1, 8, 32768)
    assert warps == 4 and 8 * -(-32768 // chunk) <= 2 * 148


def test_timeline_groups_a_step_s_kernels_by_their_place_in_a_layer():
    from mlx_omnia_b200.kernels import timeline

    layer = [("gemv", 7, 10.0), ("attention", 9, 27.0), ("gemv", 7, 3.0), ("gemv", 7, 12.0), ("gemv", 7, 6.0)]
    kernels = [("elementwise", 1, 5.0), ("elementwise", 2, 6.0)] + layer * 4 + [("elementwise", 3, 2.0)]
    lines = timeline.by_layer(kernels, "attention")
    assert len(lines) == 2 + 5 + 1 + 1
    assert lines[0].startswith("before the layers") and lines[-1].startswith("after the layers")
    assert "attention:9" in lines[3] and "27.00 us" in lines[3] and "4 layers" in lines[3]
    assert lines[7].split()[2] == "58.00"
    assert timeline.by_layer(layer, "attention") == [f"{lib}:{line} {us:8.2f} us" for lib, line, us in layer]
