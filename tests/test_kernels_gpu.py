"""Each CUDA kernel alone against its plain PyTorch reference, at sizes that are not
the engine's: widths and vocabularies that are no power of two, head sizes in steps
of 8, odd page sizes, in float32 and in bfloat16."""

from __future__ import annotations

import pytest
import torch

import kernel_refs
from mlx_omnia_b200.parts.base import KVView, StepContext

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return 1e-5 if dtype == torch.float32 else 1e-2


def close(a, b, dtype, scale=1.0):
    a, b = a.float(), b.float()
    bound = tol(dtype) * scale * max(1.0, float(b.abs().max()))
    assert float((a - b).abs().max()) <= bound, (float((a - b).abs().max()), bound)


@pytest.fixture
def ops():
    from mlx_omnia_b200.kernels import ops as module
    return module


def rand(*shape, dtype=torch.float32, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, generator=g, device="cuda") * scale).to(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden,vocab,eps", [(72, 301, 1e-6), (2048, 1000, 1e-5), (100, 50, None)])
def test_embed_rmsnorm(ops, dtype, hidden, vocab, eps):
    table = rand(vocab, hidden, dtype=dtype, scale=0.02)
    ids = torch.randint(0, vocab, (37,), device="cuda", dtype=torch.int32)
    close(ops.embed_rmsnorm(ids, table, eps), kernel_refs.embed_rmsnorm(ids, table, eps), torch.float32)


def test_embed_flags_bad_token(ops):
    table = rand(10, 16)
    ids = torch.tensor([3, 11], device="cuda", dtype=torch.int32)
    ops.embed_rmsnorm(ids, table, 1e-6)
    with pytest.raises(ops.KernelError, match="token id"):
        ops.raise_on_error(table.device)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,hidden", [(5, 72), (33, 2048), (3, 5120), (2, 13000)])
def test_rmsnorm_and_add_rmsnorm(ops, dtype, rows, hidden):
    x = rand(rows, hidden, scale=3.0, seed=1)
    w = 1 + rand(hidden, scale=0.1, seed=2)
    close(ops.rmsnorm(x, w, 1e-5, dtype), kernel_refs.rmsnorm(x, w, 1e-5, dtype), dtype)
    close(ops.rmsnorm(x, None, 1e-6, dtype), kernel_refs.rmsnorm(x, None, 1e-6, dtype), dtype)
    branch = rand(rows, hidden, dtype=dtype, scale=0.3, seed=3)
    wb, wo = 1 + rand(hidden, scale=0.1, seed=4), 1 + rand(hidden, scale=0.1, seed=5)
    for args in [(wb, 1e-6, wo, 1e-5), (None, None, wo, 1e-5), (wb, 1e-6, None, None), (None, 1e-6, None, 1e-5)]:
        x1, x2 = x.clone(), x.clone()
        h1 = ops.add_rmsnorm(x1, branch, *args)
        h2 = kernel_refs.add_rmsnorm(x2, branch, *args)
        close(x1, x2, torch.float32)
        assert (h1 is None) == (h2 is None)
        if h1 is not None:
            close(h1, h2, dtype)


def make_kv(tokens, nkv, d, page_size, dtype, num_pages, seed=0):
    """A cache view with one request per row of `tokens` (a list of lengths): random page
    placement, every other page poisoned with huge values."""
    g = torch.Generator().manual_seed(seed)
    pages = torch.full((num_pages, 2, nkv, page_size, d), 1e4, dtype=dtype, device="cuda")
    order = torch.randperm(num_pages, generator=g).tolist()
    tables, width = [], max(-(-n // page_size) for n in tokens)
    for n in tokens:
        need = -(-n // page_size)
        tables.append([order.pop() for _ in range(need)] + [-1] * (width - need))
    return pages, torch.tensor(tables, dtype=torch.int32, device="cuda")


def step_of(q_lens, seq_lens):
    cu = [0]
    positions = []
    for q, s in zip(q_lens, seq_lens):
        cu.append(cu[-1] + q)
        positions += list(range(s - q, s))
    dev = lambda v, dt=torch.int32: torch.tensor(v, dtype=dt, device="cuda")
    return StepContext(num_tokens=cu[-1], num_seqs=len(q_lens), token_ids=dev([0] * cu[-1]), positions=dev(positions),
                       cu_seqlens=dev(cu), seq_lens=dev(seq_lens), state_slots=dev([0] * len(q_lens)),
                       fresh=dev([0] * len(q_lens)), logit_rows=dev([]), q_lens=q_lens, seq_lens_host=seq_lens,
                       max_q_len=max(q_lens), max_seq_len=max(seq_lens), decode_only=all(q == 1 for q in q_lens),
                       groups={})


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,d,page,rot", [(4, 2, 16, 4, 16), (8, 1, 24, 8, 24), (6, 3, 128, 16, 128),
                                                (5, 5, 40, 3, 0), (2, 2, 256, 16, 64)])
def test_qk_norm_rope_store(ops, dtype, nq, nkv, d, page, rot):
    q_lens, seq_lens = [5, 1, 9], [12, 30, 9]
    step = step_of(q_lens, seq_lens)
    pages, table = make_kv(seq_lens, nkv, d, page, dtype, 40)
    slots = []
    for s, (q, n) in enumerate(zip(q_lens, seq_lens)):
        for pos in range(n - q, n):
            slots.append(int(table[s, pos // page]) * page + pos % page)
    slots[3] = -1  # a padded token stores nothing
    width = (2 * nq + 2 * nkv) * d + 8
    proj = rand(step.num_tokens, width, dtype=dtype, seed=7)
    inv_freq = None if rot == 0 else (10000.0 ** (-torch.arange(rot // 2, dtype=torch.float64) * 2 / rot)).float().cuda()
    q_col, k_col, v_col = 0, 2 * nq * d, 2 * nq * d + nkv * d
    view1 = KVView(pages.clone(), table, torch.tensor(slots, device="cuda"), page, None)
    view2 = KVView(pages.clone(), table, torch.tensor(slots, device="cuda"), page, None)
    for eps in (1e-6, None):
        q1 = ops.qk_norm_rope_store(proj, q_col, k_col, v_col, nq, nkv, d, eps, inv_freq, step.positions, view1)
        q2 = kernel_refs.qk_norm_rope_store(proj, q_col, k_col, v_col, nq, nkv, d, eps, inv_freq, step.positions, view2)
        close(q1, q2, dtype)
        close(view1.pages, view2.pages, dtype, scale=1e-4 if dtype == torch.float32 else 1e-4)
    ops.raise_on_error(proj.device)


@pytest.mark.parametrize("nq,nkv,d,page,rotated,gated,hidden", [(4, 2, 128, 16, True, True, 192), (6, 3, 64, 32, True, False, 136),
                                                                 (3, 1, 128, 16, False, True, 64), (4, 0, 64, 16, True, True, 72)])
def test_input_projection_with_norm_rotation_and_cache_write_in_its_epilogue(ops, nq, nkv, d, page, rotated, gated, hidden):
    """From some 1,300 rows on the attention input projection does in its epilogue what a kernel of
    its own does for fewer rows: against the plain product followed by that kernel's reference,
    with rows in two requests at positions far from zero, a row that stores nothing, a last tile
    of rows that is not full, and pages that hold NaN wherever nothing is to be written (nkv 0: a
    layer that reads another layer's cache writes none)."""
    dtype = torch.bfloat16
    q_lens, seq_lens = [900, 750], [5000, 750]
    step = step_of(q_lens, seq_lens)
    store = nkv > 0
    pages, table = make_kv(seq_lens, max(nkv, 1), d, page, dtype, 4 + sum(-(-n // page) for n in seq_lens), seed=5)
    pages.fill_(float("nan"))
    slots = []
    for s, (q, n) in enumerate(zip(q_lens, seq_lens)):
        slots += [int(table[s, pos // page]) * page + pos % page for pos in range(n - q, n)]
    slots[1000] = -1  # a padded token stores nothing
    q_cols, kv_cols = nq * d, nkv * d
    q_col, gate_col = 0, q_cols
    k_col = q_cols * (2 if gated else 1)
    v_col = k_col + kv_cols
    weight = rand(v_col + kv_cols, hidden, dtype=dtype, scale=hidden ** -0.5, seed=61)
    x = rand(step.num_tokens, hidden, dtype=dtype, seed=62)
    inv_freq = (10000.0 ** (-torch.arange(d // 2, dtype=torch.float64) * 2 / d)).float().cuda() if rotated else None
    for eps in (1e-6, None):
        mine = KVView(pages.clone(), table, torch.tensor(slots, device="cuda"), page, None) if store else None
        theirs = KVView(pages.clone(), table, torch.tensor(slots, device="cuda"), page, None) if store else None
        made = ops.linear_qkv(x, weight, q_col, k_col, v_col, nq, nkv, d, eps, inv_freq, step, mine)
        assert made is not None
        proj, q = made
        plain = (x.float() @ weight.float().t()).to(dtype)
        want = kernel_refs.qk_norm_rope_store(plain, q_col, k_col, v_col, nq, nkv, d, eps, inv_freq, step.positions, theirs)
        close(q, want, dtype)
        if gated:
            close(proj[:, gate_col: gate_col + q_cols], plain[:, gate_col: gate_col + q_cols], dtype)
        if store:
            written = ~torch.isnan(theirs.pages)
            assert torch.equal(written, ~torch.isnan(mine.pages))  # the same places, no other
            close(torch.nan_to_num(mine.pages), torch.nan_to_num(theirs.pages), dtype)
    assert ops.linear_qkv(x[:1000], weight, q_col, k_col, v_col, nq, nkv, d, 1e-6, inv_freq, step, None) is None  # few rows
    ops.raise_on_error(x.device)
    if store:
        # A slot past the pool is reported, and nothing is written for it.
        beyond = list(slots)
        beyond[7] = pages.shape[0] * page + 3
        view = KVView(pages.clone(), table, torch.tensor(beyond, device="cuda"), page, None)
        ops.linear_qkv(x, weight, q_col, k_col, v_col, nq, nkv, d, 1e-6, inv_freq, step, view)
        with pytest.raises(ops.KernelError, match="cache slot"):
            ops.raise_on_error(x.device)
        assert int((~torch.isnan(view.pages)).sum()) == (len(slots) - 2) * 2 * nkv * d  # all rows but that one and the padded one


def prefill_kernels(ops, dtype, nq, nkv, d, page):
    """The choices of prefill kernel to run a case with: the dispatcher's own, and, where the tcgen05
    kernels take the case, each of the two by name (False: two blocks to an SM; True: one)."""
    return (None, False, True) if ops.tcgen05_attention_supported(dtype, nq, nkv, d, page) else (None,)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,d,page,window", [(4, 2, 16, 4, None), (8, 1, 24, 8, 16), (6, 3, 128, 16, None),
                                                   (5, 5, 40, 3, 7), (2, 1, 256, 16, 33), (16, 8, 64, 16, None)])
def test_paged_attention(ops, dtype, nq, nkv, d, page, window):
    q_lens, seq_lens = [7, 1, 40, 1, 2], [7, 61, 75, 1, 130]
    step = step_of(q_lens, seq_lens)
    pages, table = make_kv(seq_lens, nkv, d, page, dtype, 140, seed=3)
    for s, n in enumerate(seq_lens):  # fill the live positions with ordinary values
        for pos in range(n):
            p = int(table[s, pos // page])
            pages[p, :, :, pos % page, :] = rand(2, nkv, d, dtype=dtype, seed=1000 * s + pos)
    q = rand(step.num_tokens, nq, d, dtype=dtype, seed=11)
    gate = rand(step.num_tokens, nq * d + 24, dtype=dtype, seed=12)
    view = KVView(pages, table, torch.zeros(step.num_tokens, dtype=torch.int64, device="cuda"), page, window)
    scale = 1.3 * d ** -0.5
    for wide in prefill_kernels(ops, dtype, nq, nkv, d, page):
        close(ops.paged_attention(q, view, step, scale, wide=wide), kernel_refs.paged_attention(q, view, step, scale), dtype)
        close(ops.paged_attention(q, view, step, scale, gate=gate, gate_col=24, wide=wide),
              kernel_refs.paged_attention(q, view, step, scale, gate=gate, gate_col=24), dtype)
    ops.raise_on_error(q.device)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,d,page,window", [(6, 3, 128, 16, 33), (16, 8, 64, 16, 20), (6, 3, 128, 16, None),
                                                   (4, 2, 128, 32, 100), (8, 1, 24, 8, 16), (5, 5, 40, 4, 70)])
def test_prefill_attention_at_a_window_s_edge_with_nan_elsewhere(ops, dtype, nq, nkv, d, page, window):
    """Prompt portions that start at, inside and past a 64-key tile edge, with a window whose
    first key falls inside a tile and inside a page. Everything a request may not read holds
    NaN: free pages, the unwritten tail of each request's last page, and the pages wholly
    behind the window, whose block-table entries are -1 as the cache manager leaves them. One
    key too many at either edge of the window is a NaN in the output."""
    q_lens, seq_lens = [40, 30, 50, 2, 64, 1, 17], [104, 100, 180, 67, 64, 90, 33]
    step = step_of(q_lens, seq_lens)
    pages, table = make_kv(seq_lens, nkv, d, page, dtype, 8 + sum(-(-n // page) for n in seq_lens), seed=21)
    pages.fill_(float("nan"))
    for s, (q, n) in enumerate(zip(q_lens, seq_lens)):
        dead_below = n - q - window + 1 if window else 0  # no token of this step sees positions below this
        for first in range(0, n, page):
            if first + page <= dead_below:
                table[s, first // page] = -1
                continue
            count = min(page, n - first)
            pages[int(table[s, first // page]), :, :, :count, :] = rand(2, nkv, count, d, dtype=dtype, seed=100 * s + first)
    q = rand(step.num_tokens, nq, d, dtype=dtype, seed=31)
    gate = rand(step.num_tokens, nq * d, dtype=dtype, seed=32)
    view = KVView(pages, table, torch.zeros(step.num_tokens, dtype=torch.int64, device="cuda"), page, window)
    scale = 1.1 * d ** -0.5
    want = kernel_refs.paged_attention(q, view, step, scale, gate=gate)
    for wide in prefill_kernels(ops, dtype, nq, nkv, d, page):
        got = ops.paged_attention(q, view, step, scale, gate=gate, wide=wide)
        assert not torch.isnan(got).any()
        close(got, want, dtype)
    ops.raise_on_error(q.device)


@pytest.mark.parametrize("nq,nkv,d,page,window", [(4, 2, 128, 16, None), (8, 2, 64, 16, None), (6, 3, 128, 32, 1500),
                                                   (2, 1, 128, 16, 700)])
def test_prefill_attention_in_parts(ops, nq, nkv, d, page, window):
    """Portions of prompts over long contexts: few blocks that each see dozens of key tiles, which the
    tcgen05 kernel lists as parts and merges (the list says so). Everything a request may not read
    holds NaN; a far key that matches one query stands out against hundreds of others; a second
    launch finds the tickets as the first one left them."""
    dtype = torch.bfloat16
    q_lens, seq_lens = [70, 130, 1, 33], [2900, 1700, 300, 1203]
    step = step_of(q_lens, seq_lens)
    work = ops.prefill_work_table(q_lens, seq_lens, 128 // (nq // nkv), 64, nkv, window or 0, ops.prefill_places(ops.sm_count()))
    assert ((work[:, 5] & 255) > 1).any()
    pages, table = make_kv(seq_lens, nkv, d, page, dtype, 8 + sum(-(-n // page) for n in seq_lens), seed=41)
    pages.fill_(float("nan"))
    for s, (q, n) in enumerate(zip(q_lens, seq_lens)):
        dead_below = n - q - window + 1 if window else 0
        for first in range(0, n, page):
            if first + page <= dead_below:
                table[s, first // page] = -1
                continue
            count = min(page, n - first)
            pages[int(table[s, first // page]), :, :, :count, :] = rand(2, nkv, count, d, dtype=dtype, scale=0.3, seed=100 * s + first)
    q = rand(step.num_tokens, nq, d, dtype=dtype, scale=0.3, seed=51)
    # Request 0's last token looks for the key at position 2,000 (visible whatever the window is here).
    far = 2000 if not window or window > 900 else 2500
    slot = int(table[0, far // page])
    pages[slot, 0, :, far % page, :] = 0.0
    pages[slot, 0, :, far % page, 0] = 8.0
    q[q_lens[0] - 1] = 0.0
    q[q_lens[0] - 1, :, 0] = 50.0
    gate = rand(step.num_tokens, nq * d, dtype=dtype, seed=52)
    view = KVView(pages, table, torch.zeros(step.num_tokens, dtype=torch.int64, device="cuda"), page, window)
    scale = 1.2 * d ** -0.5
    want = kernel_refs.paged_attention(q, view, step, scale, gate=gate)
    for _ in range(2):
        got = ops.paged_attention(q, view, step, scale, gate=gate)
        assert not torch.isnan(got).any()
        close(got, want, dtype)
    value = pages[slot, 1, :, far % page, :].float()  # [nkv, d]: the far key's value, what the last token must return
    for wide in (None, True):
        plain = ops.paged_attention(q, view, step, scale, wide=wide)
        close(plain[q_lens[0] - 1].view(nq, d), value.repeat_interleave(nq // nkv, dim=0), dtype, scale=3)
    # The kernel that gives a block its SM walks the same long runs of keys whole, two teams taking
    # turns with the tiles, the score buffers coming round many times.
    got = ops.paged_attention(q, view, step, scale, gate=gate, wide=True)
    assert not torch.isnan(got).any()
    close(got, want, dtype)
    ops.raise_on_error(q.device)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,d,page,window", [(4, 2, 16, 4, None), (8, 1, 24, 8, 16), (6, 3, 128, 16, None),
                                                   (6, 3, 128, 16, 200), (5, 5, 40, 3, 130), (16, 8, 64, 16, None),
                                                   (10, 2, 96, 16, None), (16, 1, 128, 32, 300), (4, 4, 64, 64, 70),
                                                   (8, 4, 128, 16, 64)])
def test_paged_attention_decode_only(ops, dtype, nq, nkv, d, page, window):
    """Every request brings one token: the split-key kernel, at lengths around its chunk
    and tile edges. Unused places of the cache hold NaN."""
    seq_lens = [1, 31, 32, 33, 127, 128, 129, 257, 700]
    q_lens = [1] * len(seq_lens)
    step = step_of(q_lens, seq_lens)
    pages, table = make_kv(seq_lens, nkv, d, page, dtype, 1 + sum(-(-n // page) for n in seq_lens), seed=6)
    pages.fill_(float("nan"))
    for s, n in enumerate(seq_lens):
        for first in range(0, n, page):
            p = int(table[s, first // page])
            count = min(page, n - first)
            pages[p, :, :, :count, :] = rand(2, nkv, count, d, dtype=dtype, seed=100 * s + first)
    q = rand(step.num_tokens, nq, d, dtype=dtype, seed=13)
    gate = rand(step.num_tokens, nq * d, dtype=dtype, seed=14)
    view = KVView(pages, table, torch.zeros(step.num_tokens, dtype=torch.int64, device="cuda"), page, window)
    scale = 0.9 * d ** -0.5
    close(ops.paged_attention(q, view, step, scale, gate=gate), kernel_refs.paged_attention(q, view, step, scale, gate=gate),
          dtype)
    ops.raise_on_error(q.device)


@pytest.mark.parametrize("rotated", [True, False])
@pytest.mark.parametrize("nq,nkv,d,page,window", [(6, 3, 128, 16, None), (6, 3, 128, 16, 200), (16, 8, 64, 16, None),
                                                   (10, 2, 96, 16, None), (16, 1, 128, 32, 300), (4, 4, 64, 64, 70),
                                                   (2, 1, 32, 16, 40)])
def test_decode_attention_from_projected_rows(ops, nq, nkv, d, page, window, rotated):
    """The decode kernel's fused mode: QK-norm, rotation and the cache write happen inside it.
    The place of the new token holds NaN beforehand, so a kernel that attended what the cache
    held there instead of its own key and value would show; lengths sit around tile and chunk edges."""
    dtype = torch.bfloat16
    seq_lens = [1, 31, 32, 33, 127, 128, 129, 257, 700]
    step = step_of([1] * len(seq_lens), seq_lens)
    pages, table = make_kv(seq_lens, nkv, d, page, dtype, 1 + sum(-(-n // page) for n in seq_lens), seed=8)
    pages.fill_(float("nan"))
    slots = []
    for s, n in enumerate(seq_lens):
        for first in range(0, n - 1, page):
            count = min(page, n - 1 - first)
            pages[int(table[s, first // page]), :, :, :count, :] = rand(2, nkv, count, d, dtype=dtype, seed=100 * s + first)
        slots.append(int(table[s, (n - 1) // page]) * page + (n - 1) % page)
    slots = torch.tensor(slots, device="cuda")
    width = (2 * nq + 2 * nkv) * d + 8
    proj = rand(step.num_tokens, width, dtype=dtype, seed=17)
    inv_freq = (10000.0 ** (-torch.arange(d // 2, dtype=torch.float64) * 2 / d)).float().cuda() if rotated else None
    q_col, k_col, v_col, gate_col = 8, 8 + 2 * nq * d, 8 + 2 * nq * d + nkv * d, 8 + nq * d
    scale = 0.9 * d ** -0.5
    for eps in (1e-6, None):
        fused = KVView(pages.clone(), table, slots, page, window)
        plain = KVView(pages.clone(), table, slots, page, window)
        assert ops.decode_fusable(proj, nq, nkv, d, inv_freq, fused, step)
        rows = ops.Projection(proj, q_col, k_col, v_col, nq, d, eps, inv_freq)
        got = ops.paged_attention(None, fused, step, scale, gate=proj, gate_col=gate_col, projection=rows)
        q = kernel_refs.qk_norm_rope_store(proj, q_col, k_col, v_col, nq, nkv, d, eps, inv_freq, step.positions, plain)
        want = kernel_refs.paged_attention(q, plain, step, scale, gate=proj, gate_col=gate_col)
        close(got, want, dtype)
        written = ~torch.isnan(plain.pages)
        assert torch.equal(written, ~torch.isnan(fused.pages))
        close(fused.pages[written], plain.pages[written], dtype)
    ops.raise_on_error(proj.device)


@pytest.mark.parametrize("dtype", DTYPES)
def test_paged_attention_finds_a_far_key(ops, dtype):
    """One key among hundreds matches the query: the output must be its value."""
    nq, nkv, d, page = 4, 2, 64, 16
    seq_lens, q_lens = [700], [1]
    step = step_of(q_lens, seq_lens)
    pages, table = make_kv(seq_lens, nkv, d, page, dtype, 50, seed=4)
    for pos in range(700):
        pages[int(table[0, pos // page]), :, :, pos % page, :] = rand(2, nkv, d, dtype=dtype, scale=0.1, seed=pos)
    far = 37
    q = rand(1, nq, d, dtype=dtype, seed=5)
    p, off = int(table[0, far // page]), far % page
    for h in range(nkv):
        pages[p, 0, h, off] = q[0, h * 2] * 8  # both heads of a group share the key; match the first
        pages[p, 1, h, off] = 5.0
    view = KVView(pages, table, torch.zeros(1, dtype=torch.int64, device="cuda"), page, None)
    out = ops.paged_attention(q, view, step, 1.0).float().reshape(nq, d)
    close(out, kernel_refs.paged_attention(q, view, step, 1.0).float().reshape(nq, d), dtype)
    assert float(out[0].mean()) > 4.9 and float(out[2].mean()) > 4.9


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu_softcap_gather(ops, dtype):
    gu = rand(19, 2 * 321, dtype=dtype, scale=3.0)
    close(ops.swiglu(gu), kernel_refs.swiglu(gu), dtype)
    z = rand(7, 1001, dtype=dtype, scale=30.0)
    close(ops.softcap(z, 0.5, 20.0), kernel_refs.softcap(z, 0.5, 20.0), torch.float32, scale=10)
    close(ops.softcap(z, 2.0, None), kernel_refs.softcap(z, 2.0, None), torch.float32)
    rows = torch.tensor([6, 0, 3, 3], dtype=torch.int32, device="cuda")
    assert torch.equal(ops.gather_rows(z, rows), kernel_refs.gather_rows(z, rows))


def test_linear_is_true_float32(ops):
    a, w = rand(33, 517, seed=1), rand(129, 517, seed=2)
    expect = (a.double() @ w.double().t()).float()
    close(ops.linear(a, w), expect, torch.float32, scale=3)
    ab, wb = a.bfloat16(), w.bfloat16()
    close(ops.linear(ab, wb), (ab.double() @ wb.double().t()).float(), torch.bfloat16, scale=3)


@pytest.mark.parametrize("m", [1, 3, 8, 11, 16])
@pytest.mark.parametrize("n,k", [(2048, 2048), (6144, 2048), (2048, 6144), (1000, 96), (777, 160), (50, 8), (5000, 520)])
def test_streamed_products(ops, m, n, k):
    """The weight-streaming kernel and its fused epilogues against float64 products of the same
    bfloat16 operands, at sizes with ragged edges in every dimension."""
    a = rand(m, k, dtype=torch.bfloat16, seed=m)
    w = rand(n, k, dtype=torch.bfloat16, scale=0.05, seed=n + k)
    exact = a.double() @ w.double().t()
    z = exact.float().bfloat16().double()
    def streamed(epilogue, multiplier=1.0, cap=0.0):
        out = torch.empty(m, n // 2 if epilogue == 1 else n, dtype=torch.float32 if epilogue == 2 else torch.bfloat16,
                          device="cuda")
        return ops._gemv_stream(a, w, out, epilogue, multiplier, cap)

    close(streamed(0), exact, torch.bfloat16)
    close(streamed(2, 3.0, 7.0), 7.0 * torch.tanh(z * 3.0 / 7.0), torch.bfloat16)
    close(streamed(2, 0.5, 0.0), z * 0.5, torch.bfloat16)
    if n % 2 == 0:
        g, u = z[:, : n // 2], z[:, n // 2:]
        close(streamed(1), g * torch.sigmoid(g) * u, torch.bfloat16)
    close(ops.linear(a, w), exact, torch.bfloat16)
    ops.raise_on_error(a.device)


@pytest.mark.parametrize("m", [1, 3, 5, 8])
@pytest.mark.parametrize("n,k", [(6144, 2048), (3072, 2048), (1000, 520), (600, 264), (48, 8)])
def test_product_runs_a_pending_residual_step(ops, m, n, k):
    """The ring-fed kernel with a residual step in front (x_new = x + norm(branch), h = norm(x_new),
    out = h w^T) against the residual kernel's reference followed by a float64 product; with and
    without weights and branch norm; the old residual stays as it was."""
    x = rand(m, k, scale=2.0, seed=m + k)
    branch = rand(m, k, dtype=torch.bfloat16, scale=0.7, seed=n)
    w = rand(n, k, dtype=torch.bfloat16, scale=0.05, seed=n + k)
    wb, wo = 1 + rand(k, scale=0.1, seed=4), 1 + rand(k, scale=0.1, seed=5)
    for args in [(wb, 1e-6, wo, 1e-5), (None, None, wo, 1e-5), (wb, 1e-6, None, 1e-6), (None, 1e-6, None, 1e-5)]:
        for gated in (False, True):
            kept, x_ref = x.clone(), x.clone()
            step = ops.PendingStep(kept, branch, *args)
            assert ops.pending_supported(kept, branch)
            got = ops.linear_swiglu(step, w) if gated else ops.linear(step, w)
            h = kernel_refs.add_rmsnorm(x_ref, branch, *args)
            z = (h.double() @ w.double().t()).float().bfloat16().double()
            want = z[:, : n // 2] * torch.sigmoid(z[:, : n // 2]) * z[:, n // 2:] if gated else z
            assert step.x_new is not None and step.x_new.data_ptr() != kept.data_ptr() and step.h is None
            assert torch.equal(kept, x)
            close(step.x_new, x_ref, torch.float32)
            close(got, want, torch.bfloat16)
            assert ops.residual_after(step, kept) is step.x_new
    # Wider than the kernel holds in registers: the step is settled by its own kernel, in place.
    wide = ops.PENDING_MAX_WIDTH + 64
    x, branch = rand(2, wide, seed=1), rand(2, wide, dtype=torch.bfloat16, seed=2)
    assert not ops.pending_supported(x, branch)
    step = ops.PendingStep(x, branch, None, 1e-6, None, 1e-6)
    w = rand(40, wide, dtype=torch.bfloat16, scale=0.05, seed=3)
    x_ref = x.clone()
    h = kernel_refs.add_rmsnorm(x_ref, branch, None, 1e-6, None, 1e-6)
    close(ops.linear(step, w), h.double() @ w.double().t(), torch.bfloat16)
    assert step.x_new is x
    close(x, x_ref, torch.float32)
    ops.raise_on_error(x.device)


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (128, 128, 128), (129, 1000, 96), (200, 300, 136), (300, 778, 160),
                                   (2048, 2048, 2048), (1000, 6144, 2048), (260, 2048, 6144), (130, 12288, 512),
                                   (2048, 6144, 2048), (777, 1000, 520), (2048, 12288, 2048)])
@pytest.mark.parametrize("kernel", ["one_sm", "two_sm", "dispatch"])
def test_tcgen05_products(ops, kernel, m, n, k):
    """The tcgen05/TMA kernels (one SM to a tile; two SMs to a tile, cta_group::2) and their
    epilogues against float64 products of the same bfloat16 operands: whole tiles, ragged edges
    in m, n and k, wide and narrow tilings; and whichever of them `linear` picks."""
    a = rand(m, k, dtype=torch.bfloat16, seed=m)
    w = rand(n, k, dtype=torch.bfloat16, scale=0.05, seed=n + k)
    exact = a.double() @ w.double().t()
    z = exact.float().bfloat16().double()
    g, u = z[:, : n // 2], z[:, n // 2:]
    if kernel == "dispatch":
        plain, capped, gated = ops.linear(a, w), ops.linear_softcap(a, w, 3.0, 7.0), ops.linear_swiglu(a, w)
    else:
        pair = kernel == "two_sm"
        plain = ops._gemm_tcgen05(a, w, torch.empty(m, n, dtype=torch.bfloat16, device="cuda"), 0, pair=pair)
        capped = ops._gemm_tcgen05(a, w, torch.empty(m, n, dtype=torch.float32, device="cuda"), 2, 3.0, 7.0, pair=pair)
        gated = ops._gemm_tcgen05(a, w, torch.empty(m, n // 2, dtype=torch.bfloat16, device="cuda"), 1, pair=pair)
    close(plain, exact, torch.bfloat16)
    close(capped, 7.0 * torch.tanh(z * 3.0 / 7.0), torch.bfloat16)
    close(gated, g * torch.sigmoid(g) * u, torch.bfloat16)
    ops.raise_on_error(a.device)


def test_sampling(ops):
    vocab, rows = 1531, 6
    logits = rand(rows, vocab, scale=2.0, seed=9)
    logits[1, 77] = logits[1, 1200] = logits[1].max() + 1  # a tie: greedy takes the first
    dev = lambda v, dt: torch.tensor(v, dtype=dt, device="cuda")
    temperature = dev([0.0, 0.0, 0.8, 1.0, 1.3, 0.7], torch.float32)
    top_k = dev([0, 0, 0, 5, 50, 0], torch.int32)
    top_p = dev([1.0, 1.0, 1.0, 1.0, 0.9, 0.5], torch.float32)
    min_p = dev([0.0, 0.0, 0.0, 0.0, 0.0, 0.05], torch.float32)
    seeds = dev([1, 2, 3, 4, 5, 6], torch.int64)
    for draw in range(4):
        draws = dev([draw] * rows, torch.int64)
        got = ops.sample(logits.clone(), temperature, top_k, top_p, min_p, seeds, draws)
        expect = kernel_refs.sample(logits.clone(), temperature, top_k, top_p, min_p, seeds, draws)
        assert got.tolist() == expect.tolist(), (draw, got.tolist(), expect.tolist())
        assert got[1].item() == 77
    # With a penalty, the recently seen ids are pushed down before anything else.
    history = dev([[int(logits[0].argmax()), -1, -1]] + [[-1, -1, -1]] * (rows - 1), torch.int32)
    penalty = dev([100.0] + [1.0] * (rows - 1), torch.float32)
    draws = dev([0] * rows, torch.int64)
    got = ops.sample(logits.clone(), temperature, top_k, top_p, min_p, seeds, draws, penalty, history)
    expect = kernel_refs.sample(logits.clone(), temperature, top_k, top_p, min_p, seeds, draws, penalty, history)
    assert got.tolist() == expect.tolist() and got[0].item() != int(logits[0].argmax())


def test_argmax_takes_the_first_of_a_tie(ops):
    logits = rand(9, 151936 // 8 + 3, scale=2.0, seed=3)
    logits[2, 5] = logits[2, 18000] = 50.0
    logits[4, -1] = 60.0
    got = ops.argmax(logits)
    assert got.tolist() == torch.argmax(logits, dim=-1).tolist() and got[2].item() == 5


def test_sampling_keeps_exactly_the_filtered_set(ops):
    """Many draws never leave the set that top_k/top_p/min_p keep, and reach all of it."""
    vocab = 300
    logits = rand(1, vocab, scale=3.0, seed=21)
    keep = kernel_refs.kept_mask(logits[0].cpu(), 0.9, 12, 0.8, 0.02)
    dev = lambda v, dt: torch.tensor(v, dtype=dt, device="cuda")
    seen = set()
    rows = 256
    big = logits.expand(rows, vocab).contiguous()
    for block in range(4):
        got = ops.sample(big.clone(), dev([0.9] * rows, torch.float32), dev([12] * rows, torch.int32),
                         dev([0.8] * rows, torch.float32), dev([0.02] * rows, torch.float32),
                         dev([7] * rows, torch.int64), dev(list(range(block * rows, (block + 1) * rows)), torch.int64))
        seen |= set(got.tolist())
    allowed = set(torch.nonzero(keep).flatten().tolist())
    assert seen <= allowed and len(seen) >= min(len(allowed), 3)


def test_tracing_build_marks_every_kernel_s_wait():
    """With OMNIA_TIMELINE=1 the libraries are built with clock stamps around each kernel's wait
    for the kernel before it: three launches leave three pairs of marks, in order, the second of
    a pair no earlier than the first, and reading the marks empties them."""
    import os
    import subprocess
    import sys
    from pathlib import Path

    script = """
import torch
from mlx_omnia_b200.csrc import build
from mlx_omnia_b200.kernels import ops
x = torch.randn(5, 256, device="cuda")
for _ in range(3):
    ops.rmsnorm(x, None, 1e-6, torch.bfloat16)
torch.cuda.synchronize()
marks = build.timeline()
assert [m[3] for m in marks if m[1] == "elementwise"] == [0, 1] * 3, marks
times = [m[0] for m in marks]
assert times == sorted(times) and len({m[2] for m in marks}) == 1
assert build.timeline() == []
print("marks ok")
"""
    root = Path(__file__).resolve().parent.parent
    env = dict(os.environ, OMNIA_TIMELINE="1", PYTHONPATH=str(root))
    done = subprocess.run([sys.executable, "-c", script], capture_output=True, text=True, env=env, timeout=600)
    assert done.returncode == 0 and "marks ok" in done.stdout, done.stderr[-2000:]
