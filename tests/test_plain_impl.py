"""The plain implementation itself: properties its formulas must have, hand-computed
cases for the sampling filters, and its 32-bit noise floor against float64."""

from __future__ import annotations

import math

import torch

import plain_impl
import tiny_configs


def test_mask_is_causal_and_windowed():
    q = torch.arange(5, 9)  # the last four of nine positions
    k = torch.arange(9)
    full = plain_impl.visible(q, k, None)
    assert full.tolist() == [[j <= i for j in range(9)] for i in range(5, 9)]
    win = plain_impl.visible(q, k, 3)
    assert win.tolist() == [[i - 3 < j <= i for j in range(9)] for i in range(5, 9)]
    assert int(win.sum(dim=1).max()) == 3  # the query's own position is one of the window's


def test_rope_rotates_pairs_and_zero_theta_is_identity():
    x = torch.randn(6, 2, 8)
    pos = torch.arange(6)
    assert torch.equal(plain_impl.rope(x, pos, 0.0), x)
    y = plain_impl.rope(x, pos, 100.0)
    assert torch.allclose(y[0], x[0]) and torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-5)
    # pair (0, 4) of position 3 turns by 3 * 100^0 = 3 rad; pair (1, 5) by 3 * 100^(-1/4)
    a, b = x[3, 0, 1], x[3, 0, 5]
    phi = 3 * 100.0 ** (-0.25)
    assert math.isclose(float(y[3, 0, 1]), float(a * math.cos(phi) - b * math.sin(phi)), abs_tol=1e-5)
    assert math.isclose(float(y[3, 0, 5]), float(a * math.sin(phi) + b * math.cos(phi)), abs_tol=1e-5)
    # scores depend on relative position only
    q, k = torch.randn(1, 1, 8), torch.randn(1, 1, 8)
    s1 = (plain_impl.rope(q, torch.tensor([7]), 50.0) * plain_impl.rope(k, torch.tensor([4]), 50.0)).sum()
    s2 = (plain_impl.rope(q, torch.tensor([13]), 50.0) * plain_impl.rope(k, torch.tensor([10]), 50.0)).sum()
    assert math.isclose(float(s1), float(s2), abs_tol=1e-4)


def test_norm_conventions():
    x = torch.randn(3, 16)
    assert torch.allclose(plain_impl.rms_norm(x, None, 0.0).pow(2).mean(-1), torch.ones(3), atol=1e-5)
    w = torch.randn(16) * 0.01
    assert torch.allclose(plain_impl.rms_norm(x, plain_impl.centred(w), 1e-6),
                          plain_impl.rms_norm(x, None, 1e-6) * (1 + w))


def test_logits_are_causal_and_windows_forget():
    raw, weights = tiny_configs.config("B"), tiny_configs.tensors("B")
    ids = tiny_configs.prompt(40, 1000, 0)
    base = plain_impl.forward(raw, weights, ids)
    changed = list(ids)
    changed[30] = (changed[30] + 1) % 1000
    other = plain_impl.forward(raw, weights, changed)
    assert torch.equal(base[:30], other[:30]) and not torch.allclose(base[30:], other[30:])
    # the cap bounds the logits
    assert float(base.abs().max()) <= 20.0
    # a trunk of sliding layers only forgets what lies behind the window (each layer widens the reach)
    raw["text_config"]["layer_types"] = ["sliding_attention"] * 3
    raw["text_config"]["sliding_window"] = 4
    a = plain_impl.forward(raw, weights, ids)
    changed = list(ids)
    changed[5] = (changed[5] + 1) % 1000
    b = plain_impl.forward(raw, weights, changed)
    reach = 5 + 3 * (4 - 1)
    assert not torch.allclose(a[5: reach + 1], b[5: reach + 1]) and torch.equal(a[reach + 1:], b[reach + 1:])


def test_float32_noise_floor():
    for name in ("A", "B"):
        raw, weights = tiny_configs.config(name), tiny_configs.tensors(name)
        ids = tiny_configs.prompt(64, raw["text_config"]["vocab_size"], 1)
        f32 = plain_impl.forward(raw, weights, ids)
        f64 = plain_impl.forward(raw, weights, ids, dtype=torch.float64)
        assert plain_impl.relative_diff(f32, f64) < 5e-6


def test_tied_and_schedule_options():
    raw, weights = tiny_configs.config("A"), tiny_configs.tensors("A")
    ids = tiny_configs.prompt(12, 512, 2)
    base = plain_impl.forward(raw, weights, ids)
    twice = plain_impl.forward(raw, weights, ids, schedule=[(0, None), (1, None), (0, None)])
    shared = plain_impl.forward(raw, weights, ids, schedule=[(0, None), (1, 0)])
    assert not torch.allclose(base, twice) and not torch.allclose(base, shared)
    taps = {}
    plain_impl.forward(raw, weights, ids, taps=taps)
    assert len(taps["blocks"]) == 2 and taps["embeddings"].shape == (12, 64)


def test_sampling_filters_by_hand():
    logits = torch.tensor([2.0, 1.0, 1.0, 0.0, -1.0])
    assert plain_impl.top_k(logits, 1).tolist() == [2.0] + [-math.inf] * 4
    assert plain_impl.top_k(logits, 2).tolist() == [2.0, 1.0, 1.0, -math.inf, -math.inf]  # the tie stays whole
    assert plain_impl.top_k(logits, 9).tolist() == logits.tolist()
    probs = torch.softmax(logits, 0)
    kept = plain_impl.top_p(logits, float(probs[0]) + 1e-3)  # the token that crosses p is kept, ties with it too
    assert kept.tolist() == [2.0, 1.0, 1.0, -math.inf, -math.inf]
    assert plain_impl.top_p(logits, float(probs[0]) - 1e-3).tolist() == [2.0] + [-math.inf] * 4
    assert plain_impl.top_p(logits, 1.0).tolist() == logits.tolist()
    floor = plain_impl.min_p(logits, math.exp(-1.5))
    assert floor.tolist() == [2.0, 1.0, 1.0, -math.inf, -math.inf]
    assert plain_impl.temperature(logits, 0.5).tolist() == [4.0, 2.0, 2.0, 0.0, -2.0]
    pushed = plain_impl.repetition_penalty(logits, [4, 0, 0, 9][:3], 2.0)
    assert pushed.tolist() == [1.0, 1.0, 1.0, 0.0, -2.0]
