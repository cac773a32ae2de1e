"""Plain, slow Muse-Glimmer: whole sequences, no cache, one function per part.

This file is the oracle of the test-suite. It is written from the formulas of
gabfssilva/mlx-omnia (each function cites the file and lines it restates, paths
relative to that project) and shares no code with the `mlx_omnia_b200` package:
it reads a plain ``dict`` of config.json keys and a plain ``dict`` of tensors
under the checkpoint's own names, and runs on the CPU in float32 or float64.

The reference's own model code cannot be imported here (it needs Apple's MLX
and Python >= 3.13), so this implementation rests on the formulas alone.
"""

from __future__ import annotations

import math

import torch

SLIDING = "sliding_attention"  # src/mlx_omnia/engine/core/masks.py:5
FULL = "full_attention"  # src/mlx_omnia/engine/core/masks.py:6

PREFIX = "model.language_model."  # src/mlx_omnia/engine/models/muse_glimmer/checkpoint.py:48-53


class Rounding:
    """Where a reduced-precision run of the reference rounds: every tensor an op hands to the
    next op is stored in `dtype` (MLX keeps activations in the checkpoint's dtype), while
    norms, softmax, rotation angles and the gate's sigmoid work in 32-bit inside the op
    (src/mlx_omnia/engine/core/kernels/add_norm/fused.py:33-46,
    src/mlx_omnia/engine/core/kernels/attention/sink.py:11-25,
    src/mlx_omnia/engine/core/attention.py:673-681). `None` rounds nothing. It exists to measure
    how far a faithful bfloat16 run may drift from the exact result: the tolerance of the
    bfloat16 tests is a multiple of that, not a guess."""

    def __init__(self, dtype: torch.dtype | None = None) -> None:
        self.dtype = dtype

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        return x if self.dtype is None else x.to(self.dtype).to(x.dtype)


EXACT = Rounding(None)


def text_config(config: dict) -> dict:
    """The text trunk's keys live under ``text_config``.
    src/mlx_omnia/engine/models/muse_glimmer/config.py:79-85"""
    return config["text_config"] if "text_config" in config else config


def rms_norm(x: torch.Tensor, weight: torch.Tensor | None, eps: float, r: Rounding = EXACT) -> torch.Tensor:
    """``x * rsqrt(mean(x^2) + eps) * weight``; weightless when ``weight`` is None. The
    normalised value is rounded before the weight multiplies it.
    src/mlx_omnia/engine/models/muse_glimmer/layers/attention.py:8-17 (weightless),
    src/mlx_omnia/engine/core/kernels/add_norm/fused.py:33-46 (the arithmetic)."""
    scale = torch.rsqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)
    y = r(x * scale)
    return y if weight is None else r(y * weight)


def centred(weight: torch.Tensor) -> torch.Tensor:
    """The four block norms store ``w`` and multiply by ``1 + w``.
    src/mlx_omnia/engine/models/muse_glimmer/checkpoint.py:85-93"""
    return weight + 1.0


def embed(ids: torch.Tensor, table: torch.Tensor, eps: float, r: Rounding = EXACT) -> torch.Tensor:
    """Lookup, then a weightless RMS norm over the hidden axis.
    src/mlx_omnia/engine/models/muse_glimmer/model.py:62-63"""
    return rms_norm(table[ids], None, eps, r)


def rope(x: torch.Tensor, positions: torch.Tensor, theta: float, r: Rounding = EXACT) -> torch.Tensor:
    """Half-split rotation of the whole head: pair (i, i + d/2), angle
    ``pos * theta^(-2i/d)``; ``theta == 0`` leaves the head as it is (NoPE).
    x: [tokens, heads, d].
    src/mlx_omnia/engine/core/attention.py:587-599 (traditional=False, scale 1),
    src/mlx_omnia/engine/core/kernels/qkv_rope/epilogue.py:56-63 (pairing, angle),
    src/mlx_omnia/engine/models/muse_glimmer/layers/attention.py:39-40 (0 = NoPE)."""
    if theta == 0:
        return x
    d = x.shape[-1]
    half = d // 2
    exponent = torch.arange(half, dtype=torch.float64) * (2.0 / d)
    inv_freq = torch.pow(torch.tensor(float(theta), dtype=torch.float64), -exponent)
    # The rotation angle is a 32-bit product of the position and the 32-bit frequency
    # unless the whole run is in float64.
    work = torch.float64 if x.dtype == torch.float64 else torch.float32
    angle = positions.to(work)[:, None] * inv_freq.to(work)[None, :]
    cos = torch.cos(angle)[:, None, :].to(x.dtype)  # the rotation itself is 32-bit; its result is rounded
    sin = torch.sin(angle)[:, None, :].to(x.dtype)
    lo, hi = x[..., :half], x[..., half:]
    return r(torch.cat([lo * cos - hi * sin, lo * sin + hi * cos], dim=-1))


def visible(queries: torch.Tensor, keys: torch.Tensor, window: int | None) -> torch.Tensor:
    """Key j is visible to the query at i iff ``j <= i`` and, on a sliding layer,
    ``i < j + window``. Positions are absolute.  -> bool [len(queries), len(keys)]
    src/mlx_omnia/engine/core/masks.py:9-18"""
    rows = queries[:, None]
    cols = keys[None, :]
    within = rows >= cols
    if window is None:
        return within
    return within & (rows < cols + window)


def attention_core(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mask: torch.Tensor, scale: float, r: Rounding = EXACT
) -> torch.Tensor:
    """Grouped-query softmax attention. q: [T, nq, d]; k, v: [S, nkv, d]; query head h
    reads KV head ``h // (nq / nkv)``.  -> [T, nq * d]
    src/mlx_omnia/engine/core/attention.py:661-670; grouping as in
    src/mlx_omnia/engine/core/attend.py:96-107."""
    tokens, heads, d = q.shape
    kv_heads = k.shape[1]
    repeats = heads // kv_heads
    k = k.repeat_interleave(repeats, dim=1)
    v = v.repeat_interleave(repeats, dim=1)
    scores = torch.einsum("thd,shd->hts", q, k) * scale
    scores = scores.masked_fill(~mask[None], float("-inf"))
    probs = torch.softmax(scores, dim=-1)
    out = torch.einsum("hts,shd->thd", probs, v)  # scores, softmax and the sum stay 32-bit; the context is rounded
    return r(out.reshape(tokens, heads * d))


def attention(
    h: torch.Tensor,
    positions: torch.Tensor,
    w: dict[str, torch.Tensor],
    *,
    heads: int,
    kv_heads: int,
    head_dim: int,
    theta: float,
    window: int | None,
    scale: float,
    eps: float,
    shared_kv: tuple[torch.Tensor, torch.Tensor] | None = None,
    r: Rounding = EXACT,
) -> tuple[torch.Tensor, tuple[torch.Tensor, torch.Tensor]]:
    """Project, weightless per-head RMS on q and k, rotate, attend, gate, project out.
    Returns the branch and the (k, v) that a cache would hold.
    src/mlx_omnia/engine/core/attention.py:618-682;
    src/mlx_omnia/engine/models/muse_glimmer/layers/attention.py:20-47."""
    tokens = h.shape[0]
    q = r(h @ w["q_proj.weight"].T).reshape(tokens, heads, head_dim)
    q = rope(rms_norm(q, None, eps, r), positions, theta, r)
    if shared_kv is None:
        k = r(h @ w["k_proj.weight"].T).reshape(tokens, kv_heads, head_dim)
        v = r(h @ w["v_proj.weight"].T).reshape(tokens, kv_heads, head_dim)
        k = rope(rms_norm(k, None, eps, r), positions, theta, r)
    else:
        k, v = shared_kv
    mask = visible(positions, positions, window)
    out = attention_core(q, k, v, mask, scale, r)
    # The gate reads the same normed input as q; sigmoid in 32-bit, full width.
    # src/mlx_omnia/engine/core/attention.py:673-681
    gate = r(torch.sigmoid(r(h @ w["gate_proj.weight"].T)))
    out = r(out * gate)
    return r(out @ w["o_proj.weight"].T), (k, v)


def swiglu(h: torch.Tensor, w: dict[str, torch.Tensor], r: Rounding = EXACT) -> torch.Tensor:
    """``down(silu(gate(h)) * up(h))``.
    src/mlx_omnia/engine/core/layers.py:249-250,253-272"""
    gate = r(h @ w["gate_proj.weight"].T)
    up = r(h @ w["up_proj.weight"].T)
    return r(r(r(gate * torch.sigmoid(gate)) * up) @ w["down_proj.weight"].T)


def trunk_name(name: str) -> str:
    """``model.language_model.X`` and ``model.X`` both name the trunk's ``X``.
    src/mlx_omnia/engine/models/muse_glimmer/checkpoint.py:48-53,72-82"""
    for prefix in (PREFIX, "model."):
        if name.startswith(prefix):
            return name[len(prefix):]
    return name


def sub(weights: dict[str, torch.Tensor], prefix: str) -> dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def block(
    x: torch.Tensor,
    positions: torch.Tensor,
    w: dict[str, torch.Tensor],
    cfg: dict,
    layer_type: str,
    theta: float,
    shared_kv=None,
    r: Rounding = EXACT,
):
    """Sandwich norms: ``x + post_attn(attn(input_ln(x)))`` then
    ``+ post_ff(mlp(pre_ff(.)))``.
    src/mlx_omnia/engine/models/muse_glimmer/layers/block.py:11-26"""
    eps, post_eps = cfg["rms_norm_eps"], cfg["post_norm_eps"]
    d = cfg["head_dim"]
    h1 = rms_norm(x, centred(w["input_layernorm.weight"]), eps, r)
    a, kv = attention(
        h1,
        positions,
        sub(w, "self_attn."),
        heads=cfg["num_attention_heads"],
        kv_heads=cfg["num_key_value_heads"],
        head_dim=d,
        theta=theta,
        window=cfg["sliding_window"] if layer_type == SLIDING else None,
        scale=cfg["qk_scale_factor"] * d**-0.5,
        eps=eps,
        shared_kv=shared_kv,
        r=r,
    )
    x = r(x + rms_norm(a, centred(w["post_attention_layernorm.weight"]), post_eps, r))
    h2 = rms_norm(x, centred(w["pre_feedforward_layernorm.weight"]), eps, r)
    m = swiglu(h2, sub(w, "mlp."), r)
    x = r(x + rms_norm(m, centred(w["post_feedforward_layernorm.weight"]), post_eps, r))
    return x, kv


def head(n: torch.Tensor, lm: torch.Tensor, multiplier: float, cap: float) -> torch.Tensor:
    """``tanh(lm_head(n) * multiplier / cap) * cap``.
    src/mlx_omnia/engine/models/muse_glimmer/model.py:79-82"""
    return torch.tanh((n @ lm.T) * multiplier / cap) * cap


def forward(
    config: dict,
    weights: dict[str, torch.Tensor],
    ids,
    *,
    dtype: torch.dtype = torch.float32,
    schedule: list[tuple[int, int | None]] | None = None,
    taps: dict | None = None,
    activations: torch.dtype | None = None,
    rows=None,
) -> torch.Tensor:
    """Logits at every position of one whole sequence (or at the positions ``rows``, so that a
    wide head need not be applied everywhere).  -> [T or len(rows), vocab]

    ``activations`` (e.g. ``torch.bfloat16``): every tensor handed from one op to the next
    is rounded to that dtype, as in a run of the reference in that precision (see
    ``Rounding``); the logits themselves stay as the head's 32-bit sum gives them.

    ``schedule`` (a test-only generality): a list of ``(layer, reads_entry)``; the
    default is every layer once, each with keys and values of its own. An entry with
    ``reads_entry = j`` attends over the keys and values that entry ``j`` produced.
    src/mlx_omnia/engine/models/muse_glimmer/model.py:89-106"""
    cfg = text_config(config)
    w = {trunk_name(k): v.to(dtype) for k, v in weights.items()}
    ids = torch.as_tensor(ids, dtype=torch.long)
    positions = torch.arange(ids.shape[0])
    r = Rounding(activations)
    x = embed(ids, w["embed_tokens.weight"], cfg["rms_norm_eps"], r)
    if taps is not None:
        taps["embeddings"] = x
        taps["blocks"] = []
    if schedule is None:
        schedule = [(i, None) for i in range(cfg["num_hidden_layers"])]
    produced = []
    for layer, reads in schedule:
        x, kv = block(
            x,
            positions,
            sub(w, f"layers.{layer}."),
            cfg,
            cfg["layer_types"][layer],
            cfg["layer_rope_theta"][layer],
            shared_kv=None if reads is None else produced[reads],
            r=r,
        )
        produced.append(kv)
        if taps is not None:
            taps["blocks"].append(x)
    # The final norm multiplies its weight directly: no +1.
    # src/mlx_omnia/engine/models/muse_glimmer/layers/block.py:39; checkpoint.py:86-91
    if rows is not None:
        x = x[rows]
    n = rms_norm(x, w["norm.weight"], cfg["rms_norm_eps"], r)
    # A tied head reads the embedding table (the house's dense model does so:
    # src/mlx_omnia/engine/core/attention.py:792-796).
    lm = w["embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else w["lm_head.weight"]
    return head(n, lm, cfg["output_multiplier"], cfg["final_logit_softcapping"])


def greedy_generate(config, weights, prompt, steps, *, dtype=torch.float32) -> list[int]:
    """Greedy decoding by re-running the whole sequence every step.
    src/mlx_omnia/engine/generate.py:162-163"""
    ids = list(prompt)
    out = []
    for _ in range(steps):
        logits = forward(config, weights, ids, dtype=dtype)
        token = int(torch.argmax(logits[-1]))
        out.append(token)
        ids.append(token)
    return out


def relative_diff(a: torch.Tensor, b: torch.Tensor) -> float:
    """``max|a - b| / max|b|`` in 64-bit.  tests/conftest.py:49-59 of the reference."""
    a = a.detach().cpu().double()
    b = b.detach().cpu().double()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))


# --- sampling filters -------------------------------------------------------------


def temperature(logits: torch.Tensor, value: float) -> torch.Tensor:
    """src/mlx_omnia/engine/generate.py:166-170"""
    return logits / value


def top_k(logits: torch.Tensor, k: int) -> torch.Tensor:
    """Keeps the k largest; a tie at the k-th value keeps the whole tied block.
    src/mlx_omnia/engine/generate.py:173-183"""
    kth = torch.topk(logits, min(k, logits.shape[-1]), dim=-1).values.min(dim=-1, keepdim=True).values
    return torch.where(logits < kth, torch.full_like(logits, -math.inf), logits)


def top_p(logits: torch.Tensor, p: float) -> torch.Tensor:
    """Keeps the tokens whose strictly-more-probable mass is below p.
    src/mlx_omnia/engine/generate.py:186-201"""
    probs = torch.softmax(logits, dim=-1)
    ordered = torch.sort(probs, dim=-1, descending=True).values
    covered = torch.cumsum(ordered, dim=-1) - ordered
    cutoff = torch.where(covered < p, ordered, torch.full_like(ordered, math.inf)).min(dim=-1, keepdim=True).values
    return torch.where(probs < cutoff, torch.full_like(logits, -math.inf), logits)


def min_p(logits: torch.Tensor, p: float) -> torch.Tensor:
    """Keeps the tokens at least p times as probable as the most probable one.
    src/mlx_omnia/engine/generate.py:204-214"""
    probs = torch.softmax(logits, dim=-1)
    floor = p * probs.max(dim=-1, keepdim=True).values
    return torch.where(probs < floor, torch.full_like(logits, -math.inf), logits)


def repetition_penalty(logits: torch.Tensor, history: list[int], value: float, context: int = 20) -> torch.Tensor:
    """Positive logits of recently seen ids are divided, negative ones multiplied.
    src/mlx_omnia/engine/generate.py:217-233"""
    if not history:
        return logits
    out = logits.clone()
    for token in set(history[-context:]):
        out[token] = out[token] / value if out[token] > 0 else out[token] * value
    return out
