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
                chunk, warps = ops.decode_plan(requests, nkv, longest, 148)
                assert 128 <= chunk <= 1024 and chunk % 64 == 0 and warps in (1, 4)
                # A captured graph's batch is a power of two: same plan.
                assert (chunk, warps) == ops.decode_plan(1 << (requests - 1).bit_length(), nkv, longest, 148)


def test_decode_plan_grows_with_the_work():
    """Few pairs: short chunks and four warps a block, so that enough warps run; more pairs: one
    warp a block and the shortest chunk whose blocks the GPU holds at a time."""
    assert ops.decode_plan(1, 8, 4096, 148) == (256, 4)
    assert ops.decode_plan(2, 8, 4096, 148) == (256, 4)
    assert ops.decode_plan(4, 8, 4096, 148) == (192, 1)
    assert ops.decode_plan(8, 8, 4096, 148) == (320, 1)
    assert ops.decode_plan(8, 8, 5120, 148) == (448, 1)
    assert ops.decode_plan(16, 8, 4096, 148) == (704, 1)
    assert ops.decode_plan(64, 8, 8192, 148) == (1024, 1)
    # One long request: four warps a block, chunks so long that two blocks an SM hold them all.
    chunk, warps = ops.decode_plan(1, 8, 32768, 148)
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


def test_a_pending_residual_step_is_settled_once_and_says_when_it_was_consumed(cpu_ops):
    """Without a GPU no product runs a pending step itself (the blocks then make none): settling one
    runs the residual kernel (here its plain reference) in place; asking again gives the same
    activations; a step that a product consumed keeps no activations and says so."""
    import pytest
    import torch

    import kernel_refs

    ops = cpu_ops
    x, branch = torch.randn(3, 16), torch.randn(3, 16).bfloat16()
    wb, wo = torch.rand(16) + 0.5, torch.rand(16) + 0.5
    expect_x = x.clone()
    expect_h = kernel_refs.add_rmsnorm(expect_x, branch, wb, 1e-6, wo, 1e-5)
    step = ops.PendingStep(x, branch, wb, 1e-6, wo, 1e-5)
    assert not ops.pending_supported(x, branch)
    assert torch.equal(ops.settle(step), expect_h)
    assert step.x_new is x and torch.equal(x, expect_x) and ops.residual_after(step, torch.zeros(1)) is x
    assert torch.equal(ops.settle(step), expect_h) and ops.settle(expect_h) is expect_h
    assert ops.residual_after(expect_h, x) is x
    consumed = ops.PendingStep(x, branch, wb, 1e-6, wo, 1e-5, x_new=torch.zeros_like(x))
    with pytest.raises(RuntimeError, match="already consumed"):
        ops.settle(consumed)


def test_prefill_blocks_are_listed_longest_first_heads_innermost(monkeypatch):
    """The tcgen05 prefill kernel's block list: every block of tokens of every multi-token request
    once per key/value head, ordered by the key tiles it sees (most first), ties in the order
    request, first token, head; requests that bring one token are left to the decode kernel."""
    from types import SimpleNamespace

    def expected(q_lens, seq_lens, tokens_per_block, tile, nkv, window):
        items = []
        for s, n in enumerate(q_lens):
            if n <= 1:
                continue
            for t0 in range(0, n, tokens_per_block):
                pos0 = seq_lens[s] - n + t0
                last = pos0 + min(tokens_per_block, n - t0) - 1
                first = max(0, pos0 - window + 1) if window else 0
                items += [(last // tile - first // tile + 1, s, t0, h) for h in range(nkv)]
        items.sort(key=lambda item: -item[0])
        return [list(item[1:]) for item in items]

    monkeypatch.setattr(ops, "_ints_to_device", lambda values, device: values)
    for q_lens, seq_lens, per_block, tile, nkv, window in [([2048], [2048], 64, 64, 8, 0),
                                                            ([7, 1, 300, 40], [7, 90, 1000, 45], 64, 64, 3, 0),
                                                            ([500, 33], [900, 33], 32, 64, 2, 130), ([1, 1], [5, 9], 64, 64, 2, 0)]:
        step = SimpleNamespace(workspace=None, q_lens=q_lens, seq_lens_host=seq_lens)
        work = ops._prefill_work_flat(step, per_block, tile, nkv, window, None)
        assert work.tolist() == expected(q_lens, seq_lens, per_block, tile, nkv, window)
        assert ops._prefill_work_flat(step, per_block, tile, nkv, window, None) is work  # built once per step
