"""The decode-attention entry point that allocates nothing (csrc/attention_static.h).

Some users of the compiled library cannot allocate device memory when they call it: the
host program has given all free GPU memory to its own pool, or cannot afford the
device-wide synchronisation of cudaMalloc on its critical path, or is inside a stream
capture. For them `omnia_attention_decode_tc_static` keeps its scratch in an array inside
the library. This test calls that function through its exported C symbol, twice in a row
(the second call meets the first call's leftovers in the shared scratch), and compares the
output with the ordinary entry point's, which takes caller-allocated scratch. It also
checks that a call too large for the array is refused with a message and launches nothing.

The file is named to be collected last, so a run that stops at the first failure has
already run every other test. It builds its own inputs and passes alone in a fresh
process as well as after the others.
"""

from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

HEAD_DIM, GROUP = 128, 2


def test_static_scratch_entry_point_matches_the_allocating_one(monkeypatch):
    from mlx_omnia_b200.csrc.build import load_library
    from mlx_omnia_b200.kernels import ops
    from mlx_omnia_b200.parts.base import KVView, StepContext

    # The ordinary entry point picks its chunk and warps per block from the batch; held to the
    # chunk and the single warp that this test gives the static one, the two add in the same order.
    monkeypatch.setattr(ops, "decode_plan", lambda requests, nkv, longest, sms: (ops.DECODE_CHUNK, 1))

    device = torch.device("cuda:0")
    torch.cuda.set_device(device)
    library = load_library("attention_tc", {"HEAD_DIM": HEAD_DIM, "GROUP": GROUP})
    entry = library.omnia_attention_decode_tc_static
    entry.restype = c_int
    entry.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int,
                      c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p]
    reason = library.omnia_attention_static_error
    reason.restype = c_char_p

    nq, nkv, page = 6, 3, 16
    generator = torch.Generator(device="cuda").manual_seed(77)

    def rand(*shape, scale=1.0):
        return (torch.randn(*shape, generator=generator, device=device) * scale).bfloat16()

    def int32(values):
        return torch.tensor(values, dtype=torch.int32, device=device)

    # Two calls in a row, of different shapes; the second with a window of 200 positions.
    for seq_lens, window in (([1, 130, 700, 257], None), ([513, 64, 5, 129, 1000], 200)):
        batch = len(seq_lens)
        need = [-(-n // page) for n in seq_lens]
        num_pages = sum(need) + 3
        order = torch.randperm(num_pages).tolist()
        table = torch.full((batch, max(need)), -1, dtype=torch.int32)
        for s, count in enumerate(need):
            table[s, :count] = torch.tensor([order.pop() for _ in range(count)], dtype=torch.int32)
        table = table.to(device)
        pages = rand(num_pages, 2, nkv, page, HEAD_DIM)
        q, gate = rand(batch, nq, HEAD_DIM), rand(batch, nq * HEAD_DIM)
        step = StepContext(num_tokens=batch, num_seqs=batch, token_ids=int32([0] * batch),
                           positions=int32([n - 1 for n in seq_lens]), cu_seqlens=int32(list(range(batch + 1))),
                           seq_lens=int32(seq_lens), state_slots=int32([0] * batch), fresh=int32([0] * batch),
                           logit_rows=int32([]), q_lens=[1] * batch, seq_lens_host=seq_lens, max_q_len=1,
                           max_seq_len=max(seq_lens), decode_only=True, groups={})
        view = KVView(pages, table, torch.zeros(batch, dtype=torch.int64, device=device), page, window)
        scale = 0.7 * HEAD_DIM ** -0.5
        expect = ops.paged_attention(q, view, step, scale, gate=gate)  # the entry point with caller scratch
        max_chunks = -(-max(seq_lens) // ops.DECODE_CHUNK)
        out = torch.full_like(expect, float("nan"))
        stream = torch.cuda.current_stream().cuda_stream
        code = entry(q.data_ptr(), pages.data_ptr(), table.data_ptr(), step.cu_seqlens.data_ptr(),
                     step.seq_lens.data_ptr(), None, batch, ops.DECODE_CHUNK, max_chunks, gate.data_ptr(),
                     gate.shape[1], out.data_ptr(), table.shape[1], num_pages, nq, nkv, page, window or 0, scale,
                     ops.error_word(device).data_ptr(), stream)
        assert code == 0, reason().decode()
        torch.cuda.synchronize()
        ops.raise_on_error(device)
        # Same kernel, same order of additions: the two entry points agree to the tolerance of the
        # kernel tests (1e-2 of the largest value in bfloat16), and in fact bit for bit.
        difference = float((out.float() - expect.float()).abs().max())
        assert difference <= 1e-2 * max(1.0, float(expect.float().abs().max())), difference
        assert torch.equal(out, expect)

    # A call beyond the array's size is refused, says why, and touches nothing.
    out = torch.zeros(4, nq * HEAD_DIM, dtype=torch.bfloat16, device=device)
    code = entry(q.data_ptr(), pages.data_ptr(), table.data_ptr(), step.cu_seqlens.data_ptr(),
                 step.seq_lens.data_ptr(), None, 4096, ops.DECODE_CHUNK, 64, None, 0, out.data_ptr(),
                 table.shape[1], num_pages, nq, nkv, page, 0, scale, ops.error_word(device).data_ptr(),
                 torch.cuda.current_stream().cuda_stream)
    assert code == -2 and b"static scratch holds" in reason()
    torch.cuda.synchronize()
    assert float(out.abs().max()) == 0.0

    # Arguments that would make the kernel divide by zero or index before its buffers are
    # refused with a reason, and nothing is launched.
    for requests, chunk in ((-1, ops.DECODE_CHUNK), (batch, 0), (batch, -128), (batch, 100)):
        code = entry(q.data_ptr(), pages.data_ptr(), table.data_ptr(), step.cu_seqlens.data_ptr(),
                     step.seq_lens.data_ptr(), None, requests, chunk, 8, None, 0, out.data_ptr(),
                     table.shape[1], num_pages, nq, nkv, page, 0, scale, ops.error_word(device).data_ptr(),
                     torch.cuda.current_stream().cuda_stream)
        assert code == 1 and reason(), (requests, chunk)  # cudaErrorInvalidValue
    torch.cuda.synchronize()
    assert float(out.abs().max()) == 0.0
