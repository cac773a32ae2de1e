"""The operations the parts are written in, each one a launch of this package's own
CUDA kernels (sources under `csrc/`). There is no other implementation behind these
functions: on a machine without a CUDA device or without nvcc they raise.

Conventions: tensors are contiguous CUDA tensors; `dtype` is float32 or bfloat16 and
names the element type of activations, matrices and cache pages; the residual stream
`x` and all logits are float32; integer metadata is int32 except `slot_mapping`
(int64). Functions return new tensors unless they say "in place".
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

from dataclasses import dataclass

import numpy as np
import torch

from mlx_omnia_b200.csrc.build import load_library
from mlx_omnia_b200.parts.base import KVView, StepContext

_DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}

ERROR_BITS = {1: "a token id outside the embedding table", 2: "a cache slot outside the page pool",
              4: "a block-table entry outside the page pool", 8: "a bounded wait inside a kernel ran out",
              16: "a work list asked a kernel for what it does not do"}


class KernelError(RuntimeError):
    """A kernel launch failed, or a kernel reported bad indices."""


_functions: dict[str, ctypes._CFuncPtr] = {}
_error_words: dict[int, torch.Tensor] = {}


def _function(library: str, name: str, argtypes: list, defines: dict | None = None):
    key = f"{library}:{name}:{sorted((defines or {}).items())}"
    fn = _functions.get(key)
    if fn is None:
        fn = getattr(load_library(library, defines), name)
        fn.argtypes = argtypes
        fn.restype = c_int
        _functions[key] = fn
    return fn


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _stream() -> int:
    """The current stream's handle (the raw query: `torch.cuda.current_stream()` builds a Python
    object and costs 3 us, which a step of 230 launches pays 230 times)."""
    return torch._C._cuda_getCurrentRawStream(torch.cuda.current_device())


launches = 0
"""How many launches of this package's own kernels this process has issued (a call that
launches two kernels counts once; replayed CUDA graphs add what their capture recorded)."""


def _check(code: int, what: str) -> None:
    global launches
    launches += 1
    if code != 0:
        raise KernelError(f"{what}: CUDA error {code} at launch (bad sizes for this kernel, or an earlier fault)")


def _code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"kernels take float32 or bfloat16, not {dtype}") from None


def error_word(device: torch.device) -> torch.Tensor:
    """The int32 word that kernels OR their index-check failures into."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    word = _error_words.get(index)
    if word is None:
        word = torch.zeros(1, dtype=torch.int32, device=device)
        _error_words[index] = word
    return word


def raise_on_error(device: torch.device) -> None:
    """Read the error word (a device sync) and raise if any kernel flagged bad indices."""
    word = error_word(device)
    bits = int(word.item())
    if bits:
        word.zero_()
        # A kernel that gave up may have left its tickets half drawn: the buffers that their users
        # are to leave zero are zero again for the next launch.
        for key in _zeroed:
            if key[0] == (device.index or 0):
                _scratch[key].zero_()
        raise KernelError("kernel index check failed: " + "; ".join(m for b, m in ERROR_BITS.items() if bits & b))


def require_cuda() -> None:
    if not torch.cuda.is_available():
        raise KernelError("mlx_omnia_b200 runs on a CUDA device (sm_100a) only; none is visible")


_sm_counts: dict[int, int] = {}


def sm_count(device: torch.device | None = None) -> int:
    """How many SMs `device` (the current one when None) has; asked once per device. Plans that
    count waves or shares of the GPU are made from this."""
    index = torch.cuda.current_device() if device is None or device.index is None else device.index
    count = _sm_counts.get(index)
    if count is None:
        count = _sm_counts[index] = torch.cuda.get_device_properties(index).multi_processor_count
    return count


# ------------------------------------------------------------------------------------


def embed_rmsnorm(ids: torch.Tensor, table: torch.Tensor, eps: float | None) -> torch.Tensor:
    """x[t] = table[ids[t]], RMS-normalised without a weight when `eps` is given. -> float32."""
    tokens, (vocab, hidden) = ids.shape[0], table.shape
    x = torch.empty(tokens, hidden, dtype=torch.float32, device=table.device)
    fn = _function("elementwise", "omnia_embed_rmsnorm",
                   [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p])
    _check(fn(_ptr(ids), _ptr(table), _ptr(x), tokens, hidden, vocab, 0.0 if eps is None else eps,
              int(eps is not None), _code(table.dtype), _ptr(error_word(table.device)), _stream()), "embed_rmsnorm")
    return x


def rmsnorm(x: torch.Tensor, weight: torch.Tensor | None, eps: float, dtype: torch.dtype) -> torch.Tensor:
    """h = x * rsqrt(mean x^2 + eps) * weight, x float32 [rows, hidden] -> `dtype`."""
    rows, hidden = x.shape
    h = torch.empty(rows, hidden, dtype=dtype, device=x.device)
    fn = _function("elementwise", "omnia_rmsnorm", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_void_p])
    _check(fn(_ptr(x), _ptr(weight), _ptr(h), rows, hidden, eps, _code(dtype), _stream()), "rmsnorm")
    return h


def add_rmsnorm(x: torch.Tensor, branch: torch.Tensor, branch_weight: torch.Tensor | None,
                branch_eps: float | None, out_weight: torch.Tensor | None, out_eps: float | None) -> torch.Tensor | None:
    """x += norm_b(branch) in place (float32), then h = norm_o(x) in branch's dtype.
    `branch_eps is None` adds the branch as it is; `out_eps is None` returns no h."""
    rows, hidden = x.shape
    h = torch.empty_like(branch) if out_eps is not None else None
    fn = _function("elementwise", "omnia_add_rmsnorm",
                   [c_void_p, c_void_p, c_void_p, c_float, c_int, c_void_p, c_float, c_int, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(x), _ptr(branch), _ptr(branch_weight), branch_eps or 0.0, int(branch_eps is not None),
              _ptr(out_weight), out_eps or 0.0, int(out_eps is not None), _ptr(h), rows, hidden,
              _code(branch.dtype), _stream()), "add_rmsnorm")
    return h


def qk_norm_rope_store(proj: torch.Tensor, q_col: int, k_col: int, v_col: int, nq: int, nkv: int, d: int,
                       eps: float | None, inv_freq: torch.Tensor | None, positions: torch.Tensor,
                       kv: KVView | None) -> torch.Tensor:
    """Per head of the projected rows: weightless RMS (q, k), rotation of the first
    2 * len(inv_freq) dims, q out as [tokens, nq, d], k and v into the cache pages.
    With `kv` None or not writing, only q is produced."""
    tokens, stride = proj.shape
    q = torch.empty(tokens, nq, d, dtype=proj.dtype, device=proj.device)
    store = kv is not None and kv.writes
    rot = 0 if inv_freq is None else 2 * inv_freq.shape[0]
    fn = _function("elementwise", "omnia_qk_norm_rope_store",
                   [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_int, c_void_p,
                    c_void_p, c_void_p, c_void_p, c_int, c_longlong, c_int, c_int, c_void_p, c_void_p])
    _check(fn(_ptr(proj), stride, q_col, k_col, v_col, nq, nkv if store else 0, d, -1.0 if eps is None else eps,
              _ptr(inv_freq), rot, _ptr(positions), _ptr(kv.slot_mapping) if store else None, _ptr(q),
              _ptr(kv.pages) if store else None, kv.page_size if store else 1,
              kv.pages.shape[0] * kv.page_size if store else 0, tokens, _code(proj.dtype),
              _ptr(error_word(proj.device)), _stream()), "qk_norm_rope_store")
    return q


DECODE_CHUNK = 128
"""Keys per split of the decode attention kernel (chunks are aligned to absolute positions)."""

_scratch: dict[tuple[int, str], torch.Tensor] = {}
_zeroed: set[tuple[int, str]] = set()  # the scratch buffers that are zero between launches


def scratch(device: torch.device, name: str, numel: int, dtype: torch.dtype = torch.float32,
            zeroed: bool = False) -> torch.Tensor:
    """A reusable buffer of at least `numel` elements. Its contents are undefined unless
    `zeroed`, in which case it is zero when created and its users leave it zero."""
    key = (device.index or 0, name)
    held = _scratch.get(key)
    if held is None or held.numel() < numel or held.dtype != dtype:
        make = torch.zeros if zeroed else torch.empty
        held = _scratch[key] = make(max(numel, 1), dtype=dtype, device=device)
        if zeroed:
            _zeroed.add(key)
    return held


def _step_buffers(step: StepContext, device: torch.device, wanted: dict) -> list[torch.Tensor]:
    """Scratch buffers `name -> (elements, dtype, zeroed)` for a kernel of this step. A step whose
    workspace says `private` (a step captured into a graph, which must keep its buffers for as
    long as the graph lives) gets buffers of its own, kept in the workspace; any other step
    shares the process-wide ones. A zeroed buffer is zero when created and its users leave it zero."""
    held = step.workspace if isinstance(step.workspace, dict) else None
    private = held is not None and held.get("private", False)
    buffers = []
    for name, (numel, dtype, zeroed) in wanted.items():
        if private:
            t = held.get(name)
            if t is None or t.numel() < numel or t.dtype != dtype:
                t = held[name] = (torch.zeros if zeroed else torch.empty)(max(numel, 1), dtype=dtype, device=device)
        else:
            t = scratch(device, name, numel, dtype, zeroed)
        buffers.append(t)
    return buffers


def width_bucket(pages: int) -> int:
    """`pages` (of the longest block table of a step) rounded up to three significant bits, at
    least 8: the widths that captured decode graphs are made for, and the bound that the decode
    attention kernel's plan is made from, so that a step takes the same plan whether it runs on
    its own or from a captured graph. Rounding to powers of two would be fewer graphs, but a
    request just past 4,096 tokens would then run the grid of one of 8,192."""
    pages = max(pages, 8)
    step = 1 << max(pages.bit_length() - 3, 0)
    return -(-pages // step) * step


def decode_plan(requests: int, nkv: int, longest: int, sms: int) -> tuple[int, int]:
    """(keys per block, warps per block) of the decode attention kernel for `requests` requests
    (rounded up to a power of two, as a captured graph's batch is) of `nkv` key/value heads whose
    longest holds `longest` positions. A block of one warp walks its chunk's 32-key tiles one after
    the other, a chain of memory round trips; the GPU holds six such blocks per SM at a time, and
    measured inside whole decode steps the best plan is the one with the most blocks that still
    run in one wave: enough loads in flight to fill the memory's bandwidth, short chains, and SMs
    that all get their share. With one or two requests (at most an eighth as many (request, head)
    pairs as SMs) a block has four warps that take the chunk's tiles in turn, without a ring (a
    tile counts one and a half); at some 244 registers a thread two such blocks fit an SM (plans
    made for three ran in one and a half waves, and badly). The cost of a plan, in tile times:
    waves x (4 for a block's start and its partial result + tiles per warp), for four-warp blocks
    divided by the share of the SMs' places that they fill, + a round trip of the merge per eight
    chunks; the plan is the cheapest chunk (a multiple of 64 keys, 128 to 1024), the shorter on a
    tie. Its pick was the best or within 2 % of the best of the plans tried at 4,096 positions
    (batches 1 to 16) and at 16,000 and 32,000 (batches 1 and 2), on a GPU of 148 SMs (`sms`)."""
    pairs = (1 << max(requests - 1, 0).bit_length()) * max(nkv, 1)
    longest = max(longest, 1)
    warps, per_sm, tile = (4, 2, 1.5) if pairs * 8 <= sms else (1, 6, 1.0)
    best, best_cost = (DECODE_CHUNK, warps), None
    for chunk in range(DECODE_CHUNK, 1024 + 1, 64):
        chunks = -(-longest // chunk)
        blocks = pairs * chunks
        waves = -(-blocks // (per_sm * sms))
        filled = blocks / (min(per_sm, -(-blocks // sms)) * sms) if waves == 1 and warps == 4 else 1.0
        cost = waves * (4 + tile * -(-(chunk // 32) // warps)) / filled + -(-chunks // 8)
        if best_cost is None or cost < best_cost:
            best, best_cost = (chunk, warps), cost
    return best


def tiled_attention_supported(dtype: torch.dtype, nq: int, nkv: int, d: int) -> bool:
    """The tensor-core kernels take bfloat16, head sizes in steps of 8 up to 256 and up to
    16 query heads per key/value head; everything else runs on the generic kernel."""
    return dtype == torch.bfloat16 and d % 8 == 0 and d <= 256 and nq % nkv == 0 and nq // nkv <= 16


# The small index lists below go to the device through a ring of pinned slots that is made once:
# pinning a fresh buffer for every list cost a prefill step 0.15 ms with the GPU idle.
_STAGING_SLOTS, _STAGING_INTS = 16, 16384
_staging: dict[int, list] = {}


def _ints_to_device(values, device: torch.device) -> torch.Tensor:
    """`values` (ints, possibly nested evenly) as an int32 tensor on `device`, copied without
    blocking from a pinned slot; a slot is written again only after its last copy has finished."""
    host = torch.from_numpy(np.ascontiguousarray(values, dtype=np.int32)) if isinstance(values, np.ndarray) \
        else torch.tensor(values, dtype=torch.int32)
    if host.numel() > _STAGING_INTS:
        return host.to(device, non_blocking=True)
    index = device.index if device.index is not None else torch.cuda.current_device()
    ring = _staging.get(index)
    if ring is None:
        ring = _staging[index] = [torch.empty(_STAGING_SLOTS, _STAGING_INTS, dtype=torch.int32).pin_memory(),
                                  [None] * _STAGING_SLOTS, 0]
    slots, events, at = ring
    ring[2] = (at + 1) % _STAGING_SLOTS
    if events[at] is not None:
        events[at].synchronize()
    else:
        events[at] = torch.cuda.Event()
    pinned = slots[at, : host.numel()].view(host.shape)
    pinned.copy_(host)
    out = pinned.to(device, non_blocking=True)
    events[at].record()
    return out


def _step_list(step: StepContext, key, build, device: torch.device) -> torch.Tensor:
    """A small list of ints that a kernel of this step reads (`build(step)` makes it on the host),
    made once per step and shared by the layers. A step that is to be captured into a graph (its
    workspace says `private`) runs once uncaptured first: the list then gets a place of its own
    and its builder is kept, and the runner fills the list again before every replay of the graph
    (`fill_step_lists`): a copy made during a capture would be replayed with whatever its staging
    memory holds by then."""
    if step.workspace is None:
        step.workspace = {}
    held = step.workspace.get(key)
    if held is None:
        if step.workspace.get("private"):
            if torch.cuda.is_current_stream_capturing():
                raise KernelError(f"the list {key} of a captured step was not made before the capture")
            held = _ints_to_device(build(step), device).clone()  # a place of its own, kept with the graph
            step.workspace.setdefault("lists", {})[key] = build
        else:
            held = _ints_to_device(build(step), device)
        step.workspace[key] = held
    return held


def fill_step_lists(step: StepContext) -> None:
    """Bring the lists of a captured step up to date with the step's host-side numbers (see
    `_step_list`); each goes to the device from a pinned buffer of its own."""
    workspace = step.workspace
    pinned = workspace.setdefault("pinned", {})
    for key, build in workspace.get("lists", {}).items():
        values = np.ascontiguousarray(build(step), dtype=np.int32)
        target = workspace[key]
        if tuple(values.shape) != tuple(target.shape):
            raise KernelError(f"the list {key} changed its shape between replays of one captured step")
        host = pinned.get(key)
        if host is None:
            host = pinned[key] = torch.empty(values.shape, dtype=torch.int32).pin_memory()
        host.numpy()[...] = values
        target.copy_(host, non_blocking=True)


def _prefill_work(step: StepContext, tokens_per_block: int, device: torch.device) -> torch.Tensor:
    """(request, first token) of every block of `tokens_per_block` query tokens, the blocks
    that see the most keys first (they run longest)."""
    def build(step: StepContext) -> np.ndarray:
        items = [(s, t0) for s, n in enumerate(step.q_lens) if n > 1 for t0 in range(0, n, tokens_per_block)]
        if step.seq_lens_host:
            items.sort(key=lambda item: -(step.seq_lens_host[item[0]] - step.q_lens[item[0]] + item[1]))
        return np.asarray(items, dtype=np.int32).reshape(-1, 2)

    return _step_list(step, ("prefill_work", tokens_per_block), build, device)


PREFILL_MAX_PARTS = 16
PREFILL_MIN_PART_TILES = 12
"""The tcgen05 prefill kernel's blocks may be listed in parts (runs of a block's key tiles, merged by
the part that finishes last): at most this many parts a block, none shorter than this many tiles,
and only in steps with at most one block per SM (portions of prompts over long contexts), whose
tiles are then shared out over one and a half places per SM. Measured on B200 with the headline
model (`bench.py --only portions`, `--only mixed`), whole blocks against parts: a prompt of 8,192
tokens read in portions of 512: 68 and 53 ms, in portions of 256: 119 and 84; 32,768 tokens in
portions of 512: 586 and 328; a step of 8 decoding requests beside a 512-token portion: 6.1 and 4.9
ms. Parts of at least 4, 8, 12, 16, 24 tiles: 4.00, 3.92, 3.83, 4.23, 4.01 ms for such a step with a
256-token portion. A whole prompt has blocks enough of its own: cut, its 2,048-token attention
takes 47 us a layer against 44 (a part pays for its start, for writing its 64 KB and for the merge)."""


def prefill_places(sms: int) -> int:
    """Over how many places the tiles of a step's blocks are shared out when blocks are cut."""
    return sms + sms // 2


def prefill_blocks(step: StepContext, tokens_per_block: int, nkv: int) -> int:
    """How many blocks of query tokens (each once per key/value head) the step's prompts' portions make."""
    return sum(-(-n // tokens_per_block) for n in step.q_lens if n > 1) * nkv


def prefill_work_table(q_lens, seq_lens, tokens_per_block: int, tile: int, nkv: int, window: int, places: int,
                       capacity: int | None = None) -> np.ndarray:
    """The tcgen05 prefill kernel's list, int32 [blocks, 8]: (request, first token, key/value head, first
    key tile of the part, tiles of the part (-1: all), parts + 256 * part, place of the block's first
    part in the workspace, number of the block among the split ones), the longest first: blocks are
    handed to SMs in this order as others finish, so the long ones start early and the short ones
    fill the gaps (measured: 30 % off a 4,096-token prefill against an order that keeps a head's
    blocks together).

    In a step of at most two thirds of `places` blocks, a block is cut into parts when it alone would
    run longer than a place's share of all tiles: into runs of max(that share, PREFILL_MIN_PART_TILES)
    tiles, so splitting adds at most `places` items. With `capacity` the list has
    exactly that many items, the unused ones marked with request -1 (a captured step's list keeps
    its shape from replay to replay while the contexts grow)."""
    blocks = []
    for s, n in enumerate(q_lens):
        if n <= 1:
            continue
        t0 = np.arange(0, n, tokens_per_block, dtype=np.int64)
        tiles = np.full_like(t0, -1)
        if seq_lens:
            pos0 = seq_lens[s] - n + t0
            last = pos0 + np.minimum(tokens_per_block, n - t0) - 1
            first = np.maximum(0, pos0 - window + 1) if window else np.zeros_like(t0)
            tiles = last // tile - first // tile + 1
        # Every block of tokens once per key/value head, heads innermost.
        blocks.append(np.stack([np.repeat(tiles, nkv), np.full(t0.size * nkv, s), np.repeat(t0, nkv),
                                np.tile(np.arange(nkv), t0.size)], axis=1))
    table = np.concatenate(blocks) if blocks else np.zeros((0, 4), dtype=np.int64)
    tiles = table[:, 0]
    out = np.zeros((table.shape[0], 9), dtype=np.int64)  # column 0: the sort key
    out[:, 0], out[:, 1:4], out[:, 5], out[:, 6] = tiles, table[:, 1:4], -1, 1
    if table.shape[0] and tiles.min() > 0 and table.shape[0] * 3 <= places * 2:
        share = max(PREFILL_MIN_PART_TILES, -(-int(tiles.sum()) // places))
        wanted = np.minimum(PREFILL_MAX_PARTS, -(-tiles // share))
        per = -(-tiles // wanted)
        parts = -(-tiles // per)
        if (parts > 1).any():
            split = parts > 1
            unit = np.cumsum(split) - 1
            slot0 = np.concatenate([[0], np.cumsum(np.where(split, parts, 0))[:-1]])
            index = np.repeat(np.arange(table.shape[0]), parts)
            part = np.arange(index.size) - np.repeat(np.cumsum(parts) - parts, parts)
            rows = np.zeros((index.size, 9), dtype=np.int64)
            rows[:, 1:4] = table[index, 1:4]
            rows[:, 4] = part * per[index]
            rows[:, 5] = np.minimum(per[index], tiles[index] - rows[:, 4])
            rows[:, 6] = parts[index] + 256 * part
            rows[:, 7], rows[:, 8] = slot0[index], unit[index]
            rows[:, 0] = rows[:, 5]
            whole = ~split[index]
            rows[whole, 4], rows[whole, 5], rows[whole, 6], rows[whole, 0] = 0, -1, 1, tiles[index][whole]
            out = rows
    order = np.argsort(-out[:, 0], kind="stable")
    out = out[order, 1:].astype(np.int32)
    if capacity is not None:
        if out.shape[0] > capacity:
            raise KernelError(f"the prefill kernel's list has {out.shape[0]} items, its place holds {capacity}")
        padded = np.full((capacity, 8), -1, dtype=np.int32)
        padded[: out.shape[0]] = out
        out = padded
    return out


WIDE_MIN_TOKENS = 512
WIDE_MIN_WINDOW = 1024


def wide_prefill_pays(q_lens, seq_lens, tokens_per_block: int, nkv: int, window: int, sms: int) -> bool:
    """Which of the two tcgen05 prefill kernels a step's prompts take: True for the one that gives a
    block an SM of its own (attention_tcgen05_wide.cu), False for the one that runs two blocks to an
    SM and cuts long blocks into parts (attention_tcgen05.cu).

    Measured on a B200 (16 query and 8 key/value heads of 128, with the gate; us, wide against two to
    an SM; a prompt of n tokens makes n / 64 blocks per key/value head): one whole prompt of 512 / 1,024
    / 2,048 / 2,304 tokens 17 / 19 / 37 / 42 against 22 / 24 / 44 / 52 (few blocks, each a long chain of
    tiles, which a block alone on its SM walks at 1.16 us for 128 keys against 1.06 us for 64), of
    2,560 / 2,816 / 3,072: 53 / 61 / 68 against 57 / 60 / 65, of 4,096 / 8,192: 101 / 323 against 88 / 290
    (a block's 7 us of start and epilogue overlap nothing when it has its SM alone); 2 prompts of 768
    or of 1,024, 4 of 512: even; 2 of 1,536, 3 of 1,024 (384 blocks): 48 / 40 against 39 / 31; 8
    portions of 256 over 1,024: 36 against 31; 512 over 8,192 cut into parts: 75 against 57. So:
    prompts from their first token, each of at least WIDE_MIN_TOKENS tokens, at most two blocks to an
    SM, and no window shorter than WIDE_MIN_WINDOW. The answer depends on the step's lengths and on
    whether its prompts start at zero, both of which a captured step's key holds."""
    prompts = [(n, held) for n, held in zip(q_lens, seq_lens or ()) if n > 1]
    if not prompts or any(held != n or n < WIDE_MIN_TOKENS for n, held in prompts):
        return False
    blocks = sum(-(-n // tokens_per_block) for n, _ in prompts) * nkv
    return blocks <= 2 * sms and (not window or window >= WIDE_MIN_WINDOW)


def _prefill_work_flat(step: StepContext, tokens_per_block: int, tile: int, nkv: int, window: int,
                       device: torch.device, places: int) -> torch.Tensor:
    """The list of `prefill_work_table` for this step, made once and shared by the layers of equal window."""
    capacity = prefill_blocks(step, tokens_per_block, nkv) + places if (step.workspace or {}).get("private") else None
    build = lambda st: prefill_work_table(st.q_lens, st.seq_lens_host, tokens_per_block, tile, nkv, window, places, capacity)
    return _step_list(step, ("prefill_work_flat", tokens_per_block, tile, nkv, window, places), build, device)


def single_token_longest(step: StepContext) -> int:
    """The longest of the requests that bring one token to a mixed step (they take the decode kernel)."""
    return max((n for q, n in zip(step.q_lens, step.seq_lens_host) if q == 1), default=0)


def _single_token_requests(step: StepContext, device: torch.device) -> tuple[torch.Tensor | None, int]:
    """Indices of the requests that bring one token to a mixed step, and the longest of them."""
    ids = [s for s, n in enumerate(step.q_lens) if n == 1]
    if not ids:
        return None, 0
    return _step_list(step, "single_token_requests", lambda _: np.asarray(ids, dtype=np.int32), device), \
        single_token_longest(step)


def tcgen05_attention_supported(dtype: torch.dtype, nq: int, nkv: int, d: int, page_size: int) -> bool:
    """The tcgen05 prefill kernel takes bfloat16, head sizes 64 and 128, pages of a multiple
    of 16 tokens and up to 16 query heads per key/value head."""
    return (dtype == torch.bfloat16 and d in (64, 128) and page_size % 16 == 0 and nq % nkv == 0
            and nq // nkv <= 16)


@dataclass
class Projection:
    """A decode step's projected rows, for the decode attention kernel to normalise, rotate and
    store by itself (what `qk_norm_rope_store` would do in a kernel of its own)."""
    rows: torch.Tensor  # [tokens, stride]
    q_col: int
    k_col: int
    v_col: int
    nq: int
    d: int
    eps: float | None
    inv_freq: torch.Tensor | None


def decode_fusable(proj: torch.Tensor, nq: int, nkv: int, d: int, inv_freq: torch.Tensor | None,
                   kv: KVView, step: StepContext) -> bool:
    """Whether the decode attention kernel can take the projected rows as they are: a step of
    single tokens, bfloat16, a head size that is a multiple of 32, rotated whole or not at all,
    and a cache entry that this layer writes."""
    return (step.decode_only and proj.is_cuda and kv.writes and d % 32 == 0
            and (inv_freq is None or 2 * inv_freq.shape[0] == d) and proj.shape[1] % 2 == 0
            and tiled_attention_supported(proj.dtype, nq, nkv, d))


def paged_attention(q: torch.Tensor | None, kv: KVView, step: StepContext, scale: float,
                    gate: torch.Tensor | None = None, gate_col: int = 0,
                    projection: Projection | None = None, wide: bool | None = None) -> torch.Tensor:
    """Causal (windowed) attention of this step's queries over the paged cache, the
    output multiplied by sigmoid(gate) when `gate` (the projected rows; the gate's
    columns start at `gate_col`) is given.  -> [tokens, nq * d]

    With `projection` (only where `decode_fusable` holds) q is not given: the kernel makes the
    queries and the new keys and values from the projected rows, and writes the latter to the cache.

    bfloat16 with a supported head size runs on the tensor-core kernels: the split-key
    decode kernel when every request brings one token; otherwise the tcgen05 prefill kernel
    (head sizes 64 and 128, pages of a multiple of 16) or the mma.sync prefill kernel. Other
    cases (the 32-bit path among them) run on the generic kernel."""
    if projection is not None:
        tokens, nq, d = projection.rows.shape[0], projection.nq, projection.d
        q = projection.rows  # for its dtype and device only
    else:
        tokens, nq, d = q.shape
    nkv = kv.pages.shape[2]
    out = torch.empty(tokens, nq * d, dtype=q.dtype, device=q.device)
    gate_ptr = None if gate is None else gate.data_ptr() + gate_col * gate.element_size()
    gate_stride = 0 if gate is None else gate.shape[1]
    err = _ptr(error_word(q.device))
    max_pages, num_pages = kv.block_table.shape[1], kv.pages.shape[0]
    if not tiled_attention_supported(q.dtype, nq, nkv, d):
        fn = _function("attention_generic", "omnia_paged_attention_generic",
                       [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int,
                        c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p])
        _check(fn(_ptr(q), _ptr(kv.pages), _ptr(kv.block_table), _ptr(step.cu_seqlens), _ptr(step.positions),
                  gate_ptr, gate_stride, _ptr(out), tokens, step.num_seqs, max_pages, num_pages, nq, nkv, d,
                  kv.page_size, kv.window or 0, scale, _code(q.dtype), err, _stream()), "paged_attention")
        return out
    defines = {"HEAD_DIM": d, "GROUP": nq // nkv}
    # Requests that bring a single token take the split-key decode kernel, in a decode-only step
    # (all of them, no index list: the shape a captured graph replays) and in a mixed step alike.
    single, longest = (None, step.max_seq_len) if step.decode_only else _single_token_requests(step, q.device)
    if step.decode_only or single is not None:
        count = step.num_seqs if step.decode_only else single.shape[0]
        longest = width_bucket(-(-longest // kv.page_size)) * kv.page_size
        chunk, warps = decode_plan(count, nkv, longest, sm_count(q.device))
        max_chunks = -(-longest // chunk)
        part_o, part_ml, tickets = _step_buffers(step, q.device, {
            "attention_part_o": (count * nq * max_chunks * d, torch.float32, False),
            "attention_part_ml": (count * nq * max_chunks * 2, torch.float32, False),
            "attention_tickets": (count * nkv, torch.int32, True)})
        fn = _function("attention_tc", "omnia_attention_decode_tc",
                       [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                        c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                        c_float, c_int, c_void_p, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p,
                        c_int, c_void_p, c_void_p], defines)
        p = projection
        fused = (None, 0, 0, 0, 0, -1.0, None, None) if p is None else (
            _ptr(p.rows), p.rows.shape[1], p.q_col, p.k_col, p.v_col, -1.0 if p.eps is None else p.eps,
            _ptr(p.inv_freq), _ptr(kv.slot_mapping))
        _check(fn(None if p is not None else _ptr(q), _ptr(kv.pages), _ptr(kv.block_table), _ptr(step.cu_seqlens),
                  _ptr(step.seq_lens), _ptr(single), count, _ptr(part_o), _ptr(part_ml), _ptr(tickets), chunk,
                  max_chunks, gate_ptr, gate_stride, _ptr(out), max_pages, num_pages, nq, nkv, kv.page_size,
                  kv.window or 0, scale, warps, *fused, 1, err, _stream()), "attention_decode")
        if step.decode_only or all(n == 1 for n in step.q_lens):
            return out
    if tcgen05_attention_supported(q.dtype, nq, nkv, d, kv.page_size):
        per_block = 128 // (nq // nkv)
        sms = sm_count(q.device)
        if wide is None:
            wide = wide_prefill_pays(step.q_lens, step.seq_lens_host, per_block, nkv, kv.window or 0, sms)
        if wide:
            # Every block whole (no places to share tiles over), an SM to a block.
            work = _prefill_work_flat(step, per_block, 64, nkv, kv.window or 0, q.device, 0)
            fn = _function("attention_tcgen05_wide", "omnia_attention_prefill_tcgen05_wide",
                           [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
                            c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p], defines)
            _check(fn(_ptr(q), tokens, _ptr(kv.pages), _ptr(kv.block_table), _ptr(step.cu_seqlens), _ptr(step.seq_lens),
                      _ptr(work), work.shape[0], gate_ptr, gate_stride, _ptr(out), max_pages, num_pages, nq, nkv,
                      kv.page_size, kv.window or 0, scale, err, _stream()), "attention_prefill_tcgen05_wide")
            return out
        work = _prefill_work_flat(step, per_block, 64, nkv, kv.window or 0, q.device, prefill_places(sms))
        # Room for the parts of blocks that are cut (at most one more item per block the device runs at
        # a time) and a ticket per block; the sizes do not depend on the contexts' lengths.
        part_floats = _function("attention_tcgen05", "omnia_attention_tcgen05_part_floats", [], defines)()
        base = prefill_blocks(step, per_block, nkv)
        partial, tickets = _step_buffers(step, q.device, {
            "prefill_parts": ((base + prefill_places(sms)) * part_floats, torch.float32, False),
            "prefill_tickets": (base, torch.int32, True)})
        fn = _function("attention_tcgen05", "omnia_attention_prefill_tcgen05",
                       [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
                        c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p],
                       defines)
        _check(fn(_ptr(q), tokens, _ptr(kv.pages), _ptr(kv.block_table), _ptr(step.cu_seqlens), _ptr(step.seq_lens),
                  _ptr(work), work.shape[0], gate_ptr, gate_stride, _ptr(out), _ptr(partial), _ptr(tickets), max_pages,
                  num_pages, nq, nkv, kv.page_size, kv.window or 0, scale, err, _stream()), "attention_prefill_tcgen05")
        return out
    tokens_per_block = 64 // (nq // nkv)
    work = _prefill_work(step, tokens_per_block, q.device)
    fn = _function("attention_tc", "omnia_attention_prefill_tc",
                   [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p,
                    c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p], defines)
    _check(fn(_ptr(q), _ptr(kv.pages), _ptr(kv.block_table), _ptr(step.cu_seqlens), _ptr(step.seq_lens), _ptr(work),
              work.shape[0], gate_ptr, gate_stride, _ptr(out), max_pages, num_pages, nq, nkv, kv.page_size,
              kv.window or 0, scale, err, _stream()), "attention_prefill")
    return out


def swiglu(gu: torch.Tensor) -> torch.Tensor:
    """act = silu(gu[:, :inner]) * gu[:, inner:]"""
    rows, two_inner = gu.shape
    inner = two_inner // 2
    act = torch.empty(rows, inner, dtype=gu.dtype, device=gu.device)
    fn = _function("elementwise", "omnia_swiglu", [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(gu), _ptr(act), rows, inner, _code(gu.dtype), _stream()), "swiglu")
    return act


def softcap(z: torch.Tensor, multiplier: float, cap: float | None) -> torch.Tensor:
    """float32 logits = cap * tanh(z * multiplier / cap); no cap when `cap` is None."""
    out = torch.empty(z.shape, dtype=torch.float32, device=z.device)
    fn = _function("elementwise", "omnia_softcap", [c_void_p, c_void_p, c_longlong, c_float, c_float, c_int, c_void_p])
    _check(fn(_ptr(z), _ptr(out), z.numel(), multiplier, cap or 0.0, _code(z.dtype), _stream()), "softcap")
    return out


def gather_rows(src: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
    """out[r] = src[rows[r]]"""
    count, width = rows.shape[0], src.shape[1]
    out = torch.empty(count, width, dtype=src.dtype, device=src.device)
    fn = _function("elementwise", "omnia_gather_rows", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(src), _ptr(rows), _ptr(out), count, width, _code(src.dtype), _stream()), "gather_rows")
    return out


SKINNY_ROWS = 16
"""Up to this many activation rows, bfloat16 products run on the weight-streaming kernel."""

FUSED_GATE_ROWS = 320
FUSED_CAP_ROWS = 129
"""From these many rows on, the products that have an epilogue fused into them (gate‖up with SwiGLU;
the head with its soft cap) run on this package's tcgen05 kernels. Measured on B200 inside replayed
graphs (weights of 8 to 50 MB, fresh for every launch): gate‖up with SwiGLU takes 46.7 us at 1,024
rows, 87.5 at 2,048 and 305 at 8,192, against 58.7, 112 and 408 for the vendor library's product
followed by the SwiGLU kernel; at 384 / 512 / 640 / 768 / 896 rows 24.3 / 31.0 / 34.6 / 35.0 / 46.3
against 26.7 / 33.8 / 41.5 / 43.0 / 55.5 (the kernel with one SM or two to a tile, whichever runs fewer
waves: `_pair_pays`); at 264 rows the library's pair is the faster one (23.3 against 24.1 us).

A product with nothing fused into it is the vendor library's above the streaming kernel's rows, as the
reference's is MLX's. The tcgen05 kernels take the same products (`_gemm_tcgen05`, tested), but the
library is ahead at every size measured: by 3 to 10 % at 2,048 to 4,096 rows (38.5 against 39.6 us
for 2,048 x 6,144 x 2,048), by 1.3 to 2.8 times between 129 and 1,024 rows, where 128 x 256 tiles
are too few for the SMs (12.1 against 33.8 us for 264 x 2,048 x 6,144), and by 10 to 28 % at 8,192.
Two kernels of this package's own for the rows in between were built, right and deterministic, and
not kept: the weights as the 128-row operand of tcgen05.mma with the few activation rows as its
columns (a tcgen05.mma with M = 128 occupies the tensor core for some 80 ns however few columns it
has, so the weights stream at half the rate of 256-column tiles), and the k range of a 128 x 256 tile
cut over a thread-block cluster (the exchange of partial sums, 128 KB a block, costs what the cut
saves: 10.6 to 32 us against the library's 8 to 12)."""

PENDING_MAX_ROWS = 8
PENDING_MAX_WIDTH = 2048
"""The most rows and the widest residual stream whose pending step the weight-streaming kernel runs itself."""

def _skinny(a: torch.Tensor, weight: torch.Tensor) -> bool:
    return (a.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and 0 < a.shape[0] <= SKINNY_ROWS
            and a.shape[1] % 8 == 0 and a.is_cuda and a.is_contiguous() and weight.is_contiguous()
            and a.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


def _tensor_core(a: torch.Tensor, weight: torch.Tensor, rows: int) -> bool:
    """Whether a product with a fused epilogue runs on the tcgen05 kernels (from `rows` rows on)."""
    return (a.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and a.is_cuda
            and a.shape[0] >= rows and a.shape[1] % 8 == 0 and a.is_contiguous()
            and weight.is_contiguous())


def _pair_pays(rows: int, n: int, k: int, epilogue: int, sms: int) -> bool:
    """Whether the two-SM kernel is the faster one: it brings in a third less per step of k, but
    has half as many (twice as large) tiles to hand out and a longer start. Measured on a GPU of
    148 SMs it wins by 4 to 13 % where a pair of SMs gets at least 64 steps of k of a 256 x 256
    tile to do (2,048 rows of 2,048 columns times 6,144 or more; 8,192 rows: all), and loses where
    the work is less (2,048 x 2,048 x 2,048; 512 rows)."""
    if rows < 256:
        return False
    if epilogue == 1:
        # gate|up with SwiGLU: tiles of 128 output columns, 128 rows to an SM or 256 to a pair. What
        # decides is how many waves of tiles each kernel runs (measured, 12,288 weight rows of 2,048:
        # some 10 us and 14 a wave for one SM, 8 and 13 a wave for a pair; 264 / 512 / 768 / 896 rows:
        # 24 / 38 / 38 / 51 us against 30 / 31 / 35 / 46).
        tiles = -(-(n // 2) // 128)
        one = -(-(-(-rows // 128) * tiles) // sms)
        two = -(-(-(-rows // 256) * tiles) // (sms // 2))
        return 8 + 13 * two < 10 + 14 * one
    tiles = -(-rows // 256) * -(-n // 256)
    return tiles * -(-k // 64) >= 64 * (sms // 2)


def _gemm_tcgen05(a: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, epilogue: int, multiplier: float = 1.0,
                  cap: float = 0.0, pair: bool | None = None) -> torch.Tensor:
    """The product on one of the two tcgen05 kernels: two SMs to a tile where that pays (`pair` None),
    or the one the caller names."""
    if pair is None:
        pair = _pair_pays(a.shape[0], weight.shape[0], a.shape[1], epilogue, sm_count(a.device))
    library, name = ("gemm_tcgen05_pair", "omnia_gemm_tcgen05_pair") if pair else ("gemm_tcgen05", "omnia_gemm_tcgen05")
    fn = _function(library, name,
                   [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_float, c_void_p, c_void_p])
    _check(fn(_ptr(a), _ptr(weight), _ptr(out), a.shape[0], weight.shape[0], a.shape[1], epilogue, multiplier, cap,
              _ptr(error_word(a.device)), _stream()), library)
    return out


def begin_pass(step: StepContext) -> None:
    """A pass over the model's layers begins: what kernels keep for the length of one pass (tables
    made from the step's positions, shared by the layers) is made afresh. A captured step is the
    same object from replay to replay, and its capture must hold the kernels that make them."""
    if isinstance(step.workspace, dict):
        step.workspace.pop("pass", None)


def rope_angles(step: StepContext, inv_freq: torch.Tensor) -> torch.Tensor:
    """(cos, sin)(position * inv_freq) for every token of the step, float32 [len(inv_freq), tokens, 2],
    made once per pass and per table of frequencies (layers of one base share it)."""
    if step.workspace is None:
        step.workspace = {}
    made = step.workspace.setdefault("pass", {})
    key = ("rope_angles", inv_freq.data_ptr())
    table = made.get(key)
    if table is None:
        half = inv_freq.shape[0]
        (table,) = _step_buffers(step, inv_freq.device,
                                 {f"rope_angles_{inv_freq.data_ptr()}": (step.num_tokens * half * 2, torch.float32, False)})
        fn = _function("elementwise", "omnia_rope_angles", [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p])
        _check(fn(_ptr(step.positions), _ptr(inv_freq), half, step.num_tokens, _ptr(table), _stream()), "rope_angles")
        made[key] = table
    return table


FUSED_QKV_ROWS = 1280
"""From how many rows on the attention input projection runs on the two-SM tcgen05 kernel with the
head norms, the rotation and the cache write in its epilogue, instead of the library's product and
the kernel that reads its result back. B200, rows x 2,048 -> 6,144, us for the two against the one
(without the 3 us of the angles' table, which a pass makes once for all its layers): 768 rows 22.7
against 23.2, 1,024: 29.4 against 29.7, 1,280: 34.8 against 31.2, 1,536: 37.2 against 31.7, 2,048:
50.7 against 42.9, 4,096: 94.0 against 80.8, 8,192: 182.7 against 154.8 (the bare products at
2,048 rows: 38.8 us for this kernel, 37.3 for the library's)."""


def linear_qkv(x, weight: torch.Tensor, q_col: int, k_col: int, v_col: int, nq: int, nkv: int, d: int,
               eps: float | None, inv_freq: torch.Tensor | None, step: StepContext,
               kv: KVView | None) -> tuple[torch.Tensor, torch.Tensor] | None:
    """x @ weight.T for weight = [q | (gate) | k | v] rows, with `qk_norm_rope_store` done in the
    product's epilogue: -> (the projected rows, of which only the columns that are neither q, k nor
    v are written; q as [tokens, nq, d]), k and v in the cache pages. None where this does not
    apply (few rows, another dtype, a head size other than 64 or 128, a rotation of part of the
    head): the caller then takes the product and `qk_norm_rope_store` one after the other."""
    store = kv is not None and kv.writes
    if not (isinstance(x, torch.Tensor) and _tensor_core(x, weight, FUSED_QKV_ROWS) and d in (64, 128)
            and (inv_freq is None or 2 * inv_freq.shape[0] == d) and weight.shape[0] % d == 0
            and q_col % d == 0 and (not store or (k_col % d == 0 and v_col % d == 0 and kv.pages.dtype == torch.bfloat16))):
        return None
    rows, n = x.shape[0], weight.shape[0]
    proj = torch.empty(rows, n, dtype=x.dtype, device=x.device)
    q = torch.empty(rows, nq, d, dtype=x.dtype, device=x.device)
    angles = None if inv_freq is None else rope_angles(step, inv_freq)
    fn = _function("gemm_tcgen05_pair", "omnia_gemm_tcgen05_pair_qkv",
                   [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                    c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_void_p])
    _check(fn(_ptr(x), _ptr(weight), _ptr(proj), rows, n, x.shape[1], d, q_col, k_col if store else 0, v_col if store else 0,
              nq, nkv if store else 0, -1.0 if eps is None else eps, _ptr(angles), _ptr(kv.slot_mapping) if store else None,
              _ptr(q), _ptr(kv.pages) if store else None, kv.page_size if store else 1,
              kv.pages.shape[0] * kv.page_size if store else 0, _ptr(error_word(x.device)), _stream()), "gemm_tcgen05_pair_qkv")
    return proj, q


def _library_mm(a: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    if a.dtype == torch.float32 and (torch.backends.cuda.matmul.allow_tf32
                                      or torch.get_float32_matmul_precision() != "highest"):
        raise KernelError("the 32-bit path needs true float32 matrix products; TF32 is switched on")
    return torch.mm(a, weight.t())


def _gemv_stream(a: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, epilogue: int, multiplier: float = 1.0,
                 cap: float = 0.0) -> torch.Tensor:
    """The product of up to 16 rows on the weight-streaming kernel (epilogue 0 store, 1 SwiGLU, 2 soft cap)."""
    fn = _function("gemv_stream", "omnia_gemv_stream",
                   [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_float, c_void_p, c_void_p])
    _check(fn(_ptr(a), _ptr(weight), _ptr(out), a.shape[0], weight.shape[0], a.shape[1], epilogue, multiplier, cap,
              _ptr(error_word(a.device)), _stream()), "gemv_stream")
    return out


@dataclass
class PendingStep:
    """A residual step that has not run yet: x_new = x + norm_b(branch), h = norm_o(x_new). The
    product that takes h (`linear`, `linear_swiglu`) runs it in its own kernel where it can, and
    anything else settles it first with `settle`. Either way `x_new` then holds the new residual
    (a buffer of its own when a product ran the step, since a kernel whose blocks all read x
    cannot update it in place; x itself otherwise)."""

    x: torch.Tensor
    branch: torch.Tensor
    branch_weight: torch.Tensor | None
    branch_eps: float | None
    out_weight: torch.Tensor | None
    out_eps: float
    x_new: torch.Tensor | None = None
    h: torch.Tensor | None = None


def pending_supported(x: torch.Tensor, branch: torch.Tensor) -> bool:
    """Whether a product of this step's rows could run the residual step itself."""
    return (x.is_cuda and branch.dtype == torch.bfloat16 and 0 < x.shape[0] <= PENDING_MAX_ROWS
            and x.shape[1] % 8 == 0 and x.shape[1] <= PENDING_MAX_WIDTH and x.is_contiguous()
            and branch.is_contiguous())


def settle(h):
    """The activations of `h`; a pending step is run now, by the kernel of its own."""
    if not isinstance(h, PendingStep):
        return h
    if h.x_new is None:
        h.h = add_rmsnorm(h.x, h.branch, h.branch_weight, h.branch_eps, h.out_weight, h.out_eps)
        h.x_new = h.x
    if h.h is None:
        raise RuntimeError("a pending residual step was already consumed by a product; its activations were not kept")
    return h.h


def residual_after(h, x: torch.Tensor) -> torch.Tensor:
    """The residual stream after whatever took `h` has run: `x` itself, or the new residual of a
    pending step (settled now if nothing took it)."""
    if not isinstance(h, PendingStep):
        return x
    if h.x_new is None:
        settle(h)
    return h.x_new


def _pending_product(step: PendingStep, weight: torch.Tensor, epilogue: int) -> torch.Tensor | None:
    """The product with the pending step in front, or None where the kernel does not take it."""
    if step.x_new is not None or not (weight.dtype == torch.bfloat16 and weight.shape[1] == step.x.shape[1]
                                      and weight.data_ptr() % 16 == 0 and weight.is_contiguous()
                                      and pending_supported(step.x, step.branch)):
        return None
    rows, n = step.x.shape[0], weight.shape[0]
    out = torch.empty(rows, n // 2 if epilogue == 1 else n, dtype=torch.bfloat16, device=step.x.device)
    x_new = torch.empty_like(step.x)
    fn = _function("gemv_stream", "omnia_gemv_stream_pending",
                   [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_int, c_void_p, c_float, c_void_p, c_void_p,
                    c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(fn(_ptr(step.x), _ptr(x_new), _ptr(step.branch), _ptr(step.branch_weight), step.branch_eps or 0.0,
              int(step.branch_eps is not None), _ptr(step.out_weight), step.out_eps, _ptr(weight), _ptr(out), rows, n,
              weight.shape[1], epilogue, _ptr(error_word(step.x.device)), _stream()), "gemv_stream_pending")
    step.x_new = x_new
    return out


def linear(a, weight: torch.Tensor) -> torch.Tensor:
    """a [rows, k] times weight [n, k] transposed -> [rows, n], float32 accumulation.
    A few bfloat16 rows (a decode step) run on this package's weight-streaming kernel, with the
    pending residual step fused in front. Otherwise the matrix product is the vendor library's (as
    the reference's is MLX's); on the 32-bit path it runs without any reduced-precision mode.
    `a` may be a PendingStep."""
    if isinstance(a, PendingStep):
        out = _pending_product(a, weight, 0)
        if out is not None:
            return out
        a = settle(a)
    if _skinny(a, weight):
        return _gemv_stream(a, weight, torch.empty(a.shape[0], weight.shape[0], dtype=a.dtype, device=a.device), 0)
    return _library_mm(a, weight)


def linear_swiglu(a, gate_up: torch.Tensor) -> torch.Tensor:
    """silu(a @ gate^T) * (a @ up^T) with gate_up = [gate rows | up rows] -> [rows, inner].
    `a` may be a PendingStep."""
    if isinstance(a, PendingStep):
        out = _pending_product(a, gate_up, 1)
        if out is not None:
            return out
        a = settle(a)
    if _skinny(a, gate_up):
        return _gemv_stream(a, gate_up, torch.empty(a.shape[0], gate_up.shape[0] // 2, dtype=a.dtype, device=a.device), 1)
    if _tensor_core(a, gate_up, FUSED_GATE_ROWS):
        return _gemm_tcgen05(a, gate_up, torch.empty(a.shape[0], gate_up.shape[0] // 2, dtype=a.dtype, device=a.device), 1)
    return swiglu(_library_mm(a, gate_up))


def linear_softcap(a: torch.Tensor, weight: torch.Tensor, multiplier: float, cap: float | None) -> torch.Tensor:
    """float32 logits = cap * tanh((a @ weight^T) * multiplier / cap) -> [rows, n]."""
    if _skinny(a, weight):
        out = torch.empty(a.shape[0], weight.shape[0], dtype=torch.float32, device=a.device)
        return _gemv_stream(a, weight, out, 2, multiplier, cap or 0.0)
    if _tensor_core(a, weight, FUSED_CAP_ROWS):
        out = torch.empty(a.shape[0], weight.shape[0], dtype=torch.float32, device=a.device)
        return _gemm_tcgen05(a, weight, out, 2, multiplier, cap or 0.0)
    return softcap(_library_mm(a, weight), multiplier, cap)


def argmax(logits: torch.Tensor) -> torch.Tensor:
    """The first largest entry of each row of float32 `logits` [rows, vocab]. -> int32 [rows]"""
    rows, vocab = logits.shape
    out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    part_v = scratch(logits.device, "argmax_v", rows * 32)
    part_i = scratch(logits.device, "argmax_i", rows * 32, torch.int32)
    fn = _function("sampling", "omnia_argmax", [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(fn(_ptr(logits), logits.stride(0), rows, vocab, _ptr(part_v), _ptr(part_i), _ptr(out), _stream()), "argmax")
    return out


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           min_p: torch.Tensor, seeds: torch.Tensor, draws: torch.Tensor, penalty: torch.Tensor | None = None,
           history: torch.Tensor | None = None) -> torch.Tensor:
    """One token per row of float32 logits [rows, vocab] (the rows are modified when a
    repetition penalty applies). Per-row parameters: temperature (0 = greedy), top_k
    (0 = off), top_p (1 = off), min_p (0 = off), seed and draw index (int64). -> int32 [rows]"""
    rows, vocab = logits.shape
    out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    fn = _function("sampling", "omnia_sample",
                   [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                    c_int, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(fn(_ptr(logits), logits.stride(0), rows, vocab, _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(min_p),
              _ptr(penalty), _ptr(history), 0 if history is None else history.shape[1], _ptr(seeds), _ptr(draws),
              _ptr(out), _stream()), "sample")
    return out
