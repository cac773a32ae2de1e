"""Plain PyTorch float32 references of the package's kernels, one per function of
`mlx_omnia_b200.kernels.ops`, with the same signatures.

Two uses: the `-m gpu` tests compare each CUDA kernel with its reference here at
sizes of their own; and the CPU tests swap these in for the kernels (the `cpu_ops`
fixture) to exercise the cache manager, the step function and the scheduler's glue
on a machine without a GPU. They are test code: nothing in the package imports them.
"""

from __future__ import annotations

import math

import torch


def _rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    x = x.float()
    return x * torch.rsqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)


def embed_rmsnorm(ids, table, eps):
    x = table[ids.long()].float()
    return x if eps is None else _rms(x, eps)


def rmsnorm(x, weight, eps, dtype):
    h = _rms(x, eps)
    if weight is not None:
        h = h * weight
    return h.to(dtype)


def add_rmsnorm(x, branch, branch_weight, branch_eps, out_weight, out_eps):
    a = branch.float()
    if branch_eps is not None:
        a = _rms(a, branch_eps)
        if branch_weight is not None:
            a = a * branch_weight
    x += a
    if out_eps is None:
        return None
    h = _rms(x, out_eps)
    if out_weight is not None:
        h = h * out_weight
    return h.to(branch.dtype)


def _rotate(v, positions, inv_freq):
    """v: [tokens, heads, d] float32."""
    if inv_freq is None:
        return v
    half = inv_freq.shape[0]
    angle = positions.float()[:, None] * inv_freq.float()[None, :]
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    a, b, rest = v[..., :half], v[..., half: 2 * half], v[..., 2 * half:]
    return torch.cat([a * cos - b * sin, a * sin + b * cos, rest], dim=-1)


def qk_norm_rope_store(proj, q_col, k_col, v_col, nq, nkv, d, eps, inv_freq, positions, kv):
    tokens = proj.shape[0]
    q = proj[:, q_col: q_col + nq * d].float().reshape(tokens, nq, d)
    if eps is not None:
        q = _rms(q, eps)
    q = _rotate(q, positions, inv_freq).to(proj.dtype)
    if kv is not None and kv.writes:
        k = proj[:, k_col: k_col + nkv * d].float().reshape(tokens, nkv, d)
        if eps is not None:
            k = _rms(k, eps)
        k = _rotate(k, positions, inv_freq).to(proj.dtype)
        v = proj[:, v_col: v_col + nkv * d].reshape(tokens, nkv, d)
        slots = kv.slot_mapping.long()
        keep = slots >= 0
        page, off = slots[keep] // kv.page_size, slots[keep] % kv.page_size
        kv.pages[page, 0, :, off, :] = k[keep]
        kv.pages[page, 1, :, off, :] = v[keep]
    return q


def paged_attention(q, kv, step, scale, gate=None, gate_col=0):
    tokens, nq, d = q.shape
    nkv = kv.pages.shape[2]
    out = torch.zeros(tokens, nq * d, dtype=torch.float32, device=q.device)
    cu = step.cu_seqlens.tolist()
    positions = step.positions.tolist()
    for s in range(step.num_seqs):
        table = kv.block_table[s].long()
        for t in range(cu[s], cu[s + 1]):
            pos = positions[t]
            if pos < 0:
                continue
            first = max(0, pos - kv.window + 1) if kv.window else 0
            js = torch.arange(first, pos + 1, device=q.device)
            pages = table[js // kv.page_size]
            assert (pages >= 0).all(), "attention reads a page that was given back"
            k = kv.pages[pages, 0, :, js % kv.page_size, :].float()  # [S, nkv, d]
            v = kv.pages[pages, 1, :, js % kv.page_size, :].float()
            k = k.repeat_interleave(nq // nkv, dim=1)
            v = v.repeat_interleave(nq // nkv, dim=1)
            scores = torch.einsum("hd,shd->hs", q[t].float(), k) * scale
            probs = torch.softmax(scores, dim=-1)
            out[t] = torch.einsum("hs,shd->hd", probs, v).reshape(-1)
    if gate is not None:
        out = out * torch.sigmoid(gate[:, gate_col: gate_col + nq * d].float())
    return out.to(q.dtype)


def swiglu(gu):
    inner = gu.shape[1] // 2
    g, u = gu[:, :inner].float(), gu[:, inner:].float()
    return (g * torch.sigmoid(g) * u).to(gu.dtype)


def softcap(z, multiplier, cap):
    v = z.float() * multiplier
    return v if not cap else cap * torch.tanh(v / cap)


def gather_rows(src, rows):
    return src[rows.long()]


def linear(a, weight):
    return (a.float() @ weight.float().t()).to(a.dtype)


def linear_swiglu(a, gate_up):
    return swiglu(linear(a, gate_up))


def linear_softcap(a, weight, multiplier, cap):
    return softcap(linear(a, weight), multiplier, cap)


# ---- sampling ------------------------------------------------------------------------

_M0, _M1, _W0, _W1 = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85
_MASK = 0xFFFFFFFF


def philox4x32_10(counter: tuple[int, int, int, int], key: tuple[int, int]) -> tuple[int, int, int, int]:
    """The Philox4x32-10 block function (Salmon et al., SC'11), in Python integers."""
    c0, c1, c2, c3 = counter
    k0, k1 = key
    for _ in range(10):
        p0, p1 = _M0 * c0, _M1 * c2
        c0, c1, c2, c3 = ((p1 >> 32) ^ c1 ^ k0) & _MASK, p1 & _MASK, ((p0 >> 32) ^ c3 ^ k1) & _MASK, p0 & _MASK
        k0, k1 = (k0 + _W0) & _MASK, (k1 + _W1) & _MASK
    return c0, c1, c2, c3


def gumbel(seed: int, draw: int, token: int) -> float:
    r = philox4x32_10((token, 0, draw & _MASK, (draw >> 32) & _MASK), (seed & _MASK, (seed >> 32) & _MASK))
    u = ((r[0] >> 8) + 0.5) / 16777216.0
    return -math.log(-math.log(u))


def kept_mask(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, min_p: float) -> torch.Tensor:
    """Which tokens survive temperature -> top_k -> top_p -> min_p (float64 arithmetic)."""
    s = logits.double() / temperature
    keep = torch.ones_like(s, dtype=torch.bool)
    if 0 < top_k < s.shape[0]:
        kth = torch.topk(s, top_k).values.min()
        keep &= s >= kth
    e = torch.where(keep, torch.exp(s - s.max()), torch.zeros_like(s))
    if top_p < 1.0:
        ordered = torch.sort(e, descending=True).values
        covered = torch.cumsum(ordered, 0) - ordered
        cutoff = ordered[covered < top_p * e.sum()].min()
        keep &= e >= cutoff
    if min_p > 0:
        keep &= e >= min_p
    return keep


def argmax(logits):
    return torch.argmax(logits.float(), dim=-1).to(torch.int32)


def sample(logits, temperature, top_k, top_p, min_p, seeds, draws, penalty=None, history=None):
    rows, vocab = logits.shape
    out = torch.empty(rows, dtype=torch.int32)
    for r in range(rows):
        z = logits[r].detach().cpu().float().clone()
        if penalty is not None and history is not None and float(penalty[r]) != 1.0:
            for token in set(int(t) for t in history[r].tolist() if 0 <= int(t) < vocab):
                z[token] = z[token] / float(penalty[r]) if z[token] > 0 else z[token] * float(penalty[r])
        t = float(temperature[r])
        if t <= 0:
            out[r] = int(torch.argmax(z))
            continue
        keep = kept_mask(z, t, int(top_k[r]), float(top_p[r]), float(min_p[r]))
        best, best_score = -1, -math.inf
        for token in torch.nonzero(keep).flatten().tolist():
            score = float(z[token]) / t + gumbel(int(seeds[r]), int(draws[r]), token)
            if score > best_score:
                best, best_score = token, score
        out[r] = best
    return out.to(logits.device)
