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


def test_prefill_blocks_are_listed_longest_first_and_cut_into_parts(monkeypatch):
    """The tcgen05 prefill kernel's list: every block of tokens of every multi-token request once per
    key/value head (requests that bring one token are left to the decode kernel); a block that alone
    would run longer than the device's share of all key tiles is listed as parts whose runs of tiles
    cover the block's tiles once and in order; the items with the most tiles come first; parts of one
    block share a place in the workspace and a ticket that no other block has."""
    from types import SimpleNamespace
    import numpy as np

    def blocks_of(q_lens, seq_lens, tokens_per_block, tile, nkv, window):
        items = {}
        for s, n in enumerate(q_lens):
            if n <= 1:
                continue
            for t0 in range(0, n, tokens_per_block):
                pos0 = seq_lens[s] - n + t0
                last = pos0 + min(tokens_per_block, n - t0) - 1
                first = max(0, pos0 - window + 1) if window else 0
                for h in range(nkv):
                    items[(s, t0, h)] = last // tile - first // tile + 1
        return items

    slots = 222  # one and a half places per SM of a 148-SM device
    cases = [([2048], [2048], 64, 64, 8, 0), ([7, 1, 300, 40], [7, 90, 1000, 45], 64, 64, 3, 0),
             ([500, 33], [900, 33], 32, 64, 2, 130), ([1, 1], [5, 9], 64, 64, 2, 0),
             ([256] + [1] * 8, [8000] + [4096] * 8, 64, 64, 8, 0), ([512], [40000], 64, 64, 8, 0),
             ([64], [40000], 64, 64, 8, 0)]
    for q_lens, seq_lens, per_block, tile, nkv, window in cases:
        table = ops.prefill_work_table(q_lens, seq_lens, per_block, tile, nkv, window, slots)
        want = blocks_of(q_lens, seq_lens, per_block, tile, nkv, window)
        assert table.shape == (table.shape[0], 8) and table.dtype == np.int32
        assert table.shape[0] <= len(want) + slots
        seen, places, tickets, lengths = {}, {}, {}, []
        for s, t0, h, lo, count, packed, slot0, unit in table.tolist():
            parts, part = packed & 255, packed >> 8
            tiles = want[(s, t0, h)]
            if parts == 1:
                assert (lo, count, part) == (0, -1, 0)
                count = tiles
            else:
                assert 1 < parts <= ops.PREFILL_MAX_PARTS and 0 <= part < parts and count >= 1
                places.setdefault((slot0, parts), set()).add((s, t0, h))
                tickets.setdefault(unit, set()).add((s, t0, h))
            seen.setdefault((s, t0, h), []).append((part, lo, count, parts))
            lengths.append(count)
        assert lengths == sorted(lengths, reverse=True)
        assert set(seen) == set(want)
        for key, runs in seen.items():
            runs.sort()
            assert [r[0] for r in runs] == list(range(runs[0][3]))  # every part once
            assert runs[0][1] == 0 and all(a[1] + a[2] == b[1] for a, b in zip(runs, runs[1:]))  # in order, no gap
            assert runs[-1][1] + runs[-1][2] == want[key]
        assert all(len(v) == 1 for v in places.values()) and all(len(v) == 1 for v in tickets.values())
        spans = sorted((slot0, slot0 + parts) for slot0, parts in places)
        assert all(a[1] <= b[0] for a, b in zip(spans, spans[1:]))  # no two blocks share a place
        assert sorted(tickets) == list(range(len(tickets)))
        # A long block over few blocks is cut; a step with many blocks of its own is cut less or not at all.
        if q_lens == [512]:  # 64 blocks of 618 to 625 tiles on 222 places: four parts each
            assert {r[3] for runs in seen.values() for r in runs} == {4}
        if q_lens == [64]:
            assert {r[3] for runs in seen.values() for r in runs} == {ops.PREFILL_MAX_PARTS}
        if q_lens == [2048]:  # a whole prompt has blocks enough of its own: none is cut
            assert {r[3] for runs in seen.values() for r in runs} == {1}
        if q_lens == [1, 1]:
            assert table.shape[0] == 0
        padded = ops.prefill_work_table(q_lens, seq_lens, per_block, tile, nkv, window, slots, capacity=len(want) + slots)
        assert padded.shape[0] == len(want) + slots and (padded[: table.shape[0]] == table).all()
        assert (padded[table.shape[0]:, 0] == -1).all()

    monkeypatch.setattr(ops, "_ints_to_device", lambda values, device: values)
    monkeypatch.setattr(ops, "sm_count", lambda device=None: 148)
    step = SimpleNamespace(workspace=None, q_lens=[300, 1], seq_lens_host=[5000, 77])
    work = ops._prefill_work_flat(step, 64, 64, 8, 0, None, 222)
    assert (work == ops.prefill_work_table([300, 1], [5000, 77], 64, 64, 8, 0, 222)).all()
    assert ops._prefill_work_flat(step, 64, 64, 8, 0, None, 222) is work  # built once per step


def test_which_prefill_kernel_a_step_takes():
    """One block to an SM pays for prompts from their first token, each at least 512 tokens long, that
    make at most two blocks to an SM; every other step takes the kernel with two blocks to an SM."""
    pays = lambda q, held, window=0: ops.wide_prefill_pays(q, held, 64, 8, window, 148)
    assert pays([512], [512]) and pays([1024], [1024]) and pays([2048], [2048]) and pays([2304], [2304])
    assert pays([512] * 4, [512] * 4) and pays([1024, 1024], [1024, 1024])
    assert pays([1, 2048, 1], [300, 2048, 77])                # requests that decode beside the prompt do not matter
    assert not pays([2432], [2432]) and not pays([4096], [4096]) and not pays([1536, 1536], [1536, 1536])  # too many blocks
    assert not pays([1024], [4096]) and not pays([512], [8192])  # portions of prompts under way
    assert not pays([256] * 8, [256] * 8) and not pays([2048, 300], [2048, 300])  # short prompts: short chains of tiles
    assert not pays([2048], [2048], window=600) and pays([2048], [2048], window=1024)
    assert not pays([1, 1], [50, 60]) and not pays([2048], None)
    assert ops.wide_prefill_pays([2048], [2048], 32, 8, 0, 148) is False  # groups of four: 512 blocks


def test_which_tcgen05_kernel_takes_gate_up_with_swiglu():
    """One SM to a 128-row tile or two SMs to a 256-row tile: the one that runs fewer waves of tiles
    (12,288 weight rows: 48 tiles of 128 output columns per tile of rows, 148 SMs or 74 pairs)."""
    pair = lambda rows, n=12288: ops._pair_pays(rows, n, 2048, 1, 148)
    assert not pair(264) and not pair(384)          # 144 tiles: one wave of SMs against two of pairs
    assert pair(385) and pair(512) and pair(768)    # two waves either way, and a pair's wave is the shorter
    assert pair(896) and pair(2048) and pair(8192)
    assert not pair(200)                            # under a pair's 256 rows
    assert not pair(896, 24576)                     # twice the columns: five waves of SMs against six of pairs
    assert ops.FUSED_GATE_ROWS <= 384
