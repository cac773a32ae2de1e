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
