"""Host-side choices of the kernel dispatcher that need no GPU."""

from mlx_omnia_b200.kernels import ops


def test_decode_chunk_is_a_tile_multiple_within_bounds_and_the_same_for_a_bucket():
    for pairs in (1, 3, 8, 17, 64, 100, 512, 4096):
        for longest in (1, 90, 128, 1000, 4096, 5000, 100000):
            chunk = ops.decode_chunk(pairs, longest)
            assert 128 <= chunk <= 1024 and chunk % 64 == 0
            # A captured graph is sized for bounds that are powers of two: same chunk.
            up = lambda n: 1 << (n - 1).bit_length()
            assert chunk == ops.decode_chunk(up(pairs), up(longest))


def test_decode_plan_grows_with_the_work():
    """Few pairs: short chunks and four warps a block, so that enough warps run; many pairs:
    long chunks walked by one warp."""
    chunk, warps = ops.decode_plan(8, 4096)
    assert chunk <= 256 and warps == 4
    assert ops.decode_plan(64, 4096) == (512, 1)
    assert ops.decode_plan(512, 8192) == (1024, 1)
