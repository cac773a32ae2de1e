"""Each part alone against the plain implementation's function for it, and the
generality of the composition: a schedule that names a layer twice or lets a layer
read another's cache, and a toy mixer with state of its own that is registered, built
and stepped from this file without touching the framework; likewise a toy feed-forward
that routes each token to two of its experts and a toy position encoding."""

from __future__ import annotations

import pytest
import torch

import plain_impl
import tiny_configs
from mlx_omnia_b200.cache import CacheManager
from mlx_omnia_b200.engine.engine import Engine, EngineArgs
from mlx_omnia_b200.engine.step import StepEntry, StepRunner
from mlx_omnia_b200.kernels import ops
from mlx_omnia_b200.parts import (DecoderModel, LayerSpec, ModelSpec, PartSpec, Runtime, ScheduleEntry, StateSpec,
                                  register_mixer)
from mlx_omnia_b200.parts.base import (FEED_FORWARDS, HEADS, EMBEDDINGS, MIXERS, NORMS, POSITIONS, Embedding, FeedForward,
                                       KVSpec, Mixer, Position, TensorSpec, register_embedding, register_feed_forward,
                                       register_position)
from mlx_omnia_b200.architectures.muse_glimmer import model_spec, parse

pytestmark = pytest.mark.gpu
CUDA = torch.device("cuda:0")


def runtime(dtype=torch.float32):
    return Runtime(dtype, CUDA)


def test_norm_part():
    x = torch.randn(7, 96, device=CUDA)
    w = torch.randn(96, device=CUDA) * 0.1
    for convention, expect_w in [("plain", w), ("centred", w + 1), ("none", None)]:
        norm = NORMS.build(PartSpec("rms_norm", {"size": 96, "eps": 1e-5, "weight": convention}))
        assert set(norm.tensors()) == (set() if convention == "none" else {"weight"})
        norm.load({"weight": w} if convention != "none" else {}, runtime())
        assert plain_impl.relative_diff(norm.forward(x), plain_impl.rms_norm(x, expect_w, 1e-5)) < 1e-5


def test_position_part():
    rotary = POSITIONS.build(PartSpec("rotary", {"dims": 24, "theta": 1e6}))
    rotary.load({}, runtime())
    expect = 1e6 ** (-torch.arange(12, dtype=torch.float64) * 2 / 24)
    assert torch.allclose(rotary.table().cpu().double(), expect, rtol=1e-7)
    none = POSITIONS.build(PartSpec("none"))
    none.load({}, runtime())
    assert none.table() is None


def test_feed_forward_part():
    ff = FEED_FORWARDS.build(PartSpec("gated_mlp", {"hidden": 96, "inner": 320}))
    w = {"gate_proj.weight": torch.randn(320, 96, device=CUDA) * 0.1, "up_proj.weight": torch.randn(320, 96, device=CUDA) * 0.1,
         "down_proj.weight": torch.randn(96, 320, device=CUDA) * 0.1}
    assert {k: v.shape for k, v in ff.tensors().items()} == {k: tuple(v.shape) for k, v in w.items()}
    ff.load(w, runtime())
    h = torch.randn(11, 96, device=CUDA)
    assert plain_impl.relative_diff(ff.forward(h, None), plain_impl.swiglu(h, w)) < 1e-5


def test_embedding_and_head_parts():
    table = torch.randn(301, 72, device=CUDA)
    embedding = EMBEDDINGS.build(PartSpec("token_embedding", {"vocab": 301, "hidden": 72, "norm_eps": 1e-6}))
    embedding.load({"weight": table}, runtime())
    ids = torch.randint(0, 301, (9,), device=CUDA, dtype=torch.int32)
    assert plain_impl.relative_diff(embedding.forward(ids), plain_impl.embed(ids.long(), table, 1e-6)) < 1e-6
    for tied in (True, False):
        head = HEADS.build(PartSpec("lm_head", {"vocab": 301, "hidden": 72, "tied": tied, "multiplier": 0.5, "softcap": 20.0}))
        lm = torch.randn(301, 72, device=CUDA)
        head.load({} if tied else {"weight": lm}, runtime())
        head.bind(table)
        n = torch.randn(4, 72, device=CUDA) * 3
        assert plain_impl.relative_diff(head.forward(n), plain_impl.head(n, table if tied else lm, 0.5, 20.0)) < 1e-5


def single_layer_engine(name, layer, schedule=None, dtype="float32"):
    raw, weights = tiny_configs.config(name), tiny_configs.tensors(name)
    engine = Engine.from_tensors(raw, weights, EngineArgs(dtype=dtype, page_size=4, cache_tokens=256, max_requests=2))
    return engine, raw, weights


@pytest.mark.parametrize("name,layer", [("A", 0), ("B", 0), ("B", 1)])
def test_attention_mixer_and_block_alone(name, layer):
    """One block of the loaded model, stepped in two portions, against the plain block."""
    engine, raw, weights = single_layer_engine(name, layer)
    cfg = raw["text_config"]
    block = engine.model.blocks[layer]
    tokens = 29
    x = torch.randn(tokens, cfg["hidden_size"], device=CUDA)
    named = {plain_impl.trunk_name(k): v for k, v in weights.items()}
    w = plain_impl.sub(named, f"layers.{layer}.")
    expect_x, _ = plain_impl.block(x.cpu(), torch.arange(tokens), w, cfg, cfg["layer_types"][layer],
                                   cfg["layer_rope_theta"][layer])
    request = engine.cache.open("r")
    got = []
    for lo, hi in ((0, 18), (18, 29)):
        step = engine.runner.build_context([StepEntry(request, [0] * (hi - lo), [])])
        ctx = engine.runner.layer_contexts(step)[layer]
        part = x[lo:hi].clone()
        h = block.entry_norm.forward(part)
        out, _ = block.forward(part, h, ctx, None)
        got.append(out)
        engine.cache.release_behind_window(request)
    assert plain_impl.relative_diff(torch.cat(got).cpu(), expect_x) < 2e-5


def spec_with_schedule(raw, schedule):
    base = model_spec(parse(raw))
    return ModelSpec(base.embedding, base.layers, tuple(ScheduleEntry(*s) for s in schedule), base.final_norm, base.head)


@pytest.mark.parametrize("schedule", [[(0, None), (1, None), (0, None)], [(0, None), (1, 0)],
                                      [(1, None), (0, None), (1, 1), (0, None)]])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_schedule_is_data(schedule, dtype):
    """A layer may run twice (each run with a cache of its own) and a layer may read the
    cache of an earlier entry; the plain implementation takes the same list."""
    raw, weights = tiny_configs.config("A"), tiny_configs.tensors("A")
    rt = runtime(dtype)
    model = DecoderModel(spec_with_schedule(raw, schedule))
    named = {}
    for k, v in weights.items():
        name = "model." + plain_impl.trunk_name(k) if not k.startswith("lm_head") else k
        kind = model.tensors()[name].kind
        named[name] = v.to(CUDA).to(torch.float32 if kind == "vector" else dtype)
    model.load(named, rt)
    cache = CacheManager(model.cache_needs(), page_size=4, pages_per_group=40, max_requests=2, dtype=dtype, device=CUDA)
    assert len(cache.groups[0].entries) == sum(1 for _, reads in schedule if reads is None)
    runner = StepRunner(model, cache, rt)
    ids = tiny_configs.prompt(33, 512, 8)
    request = cache.open("r")
    got = torch.cat([runner.run([StepEntry(request, ids[:20], list(range(20)))]),
                     runner.run([StepEntry(request, ids[20:31], list(range(11)))]),
                     runner.run([StepEntry(request, ids[31:32], [0])]), runner.run([StepEntry(request, ids[32:], [0])])])
    expect = plain_impl.forward(raw, weights, ids, schedule=schedule)
    assert plain_impl.relative_diff(got, expect) < (1e-4 if dtype == torch.float32 else 3e-2)


# ---- toy parts, defined here: none of them is a change to the framework's files ---------------
# A mixer with state of its own (and a start that is not zero), a mixer that keeps one latent
# row per token in the paged cache instead of keys and values, and an embedding that adds a
# learned absolute position encoding. They never become anyone's model.


@register_mixer("toy_decay_mixer")
class ToyDecayMixer(Mixer):
    """s_t = decay * s_{t-1} + h_t W_in ; out_t = s_t W_out, with s_{-1} = start. Its state is
    one vector per request, kept in a state slot between steps; it keeps no pages. A step of
    single tokens touches no host memory, so it can be captured into a graph."""

    graph_safe = True

    def __init__(self, hidden: int, width: int, decay: float, start: float = 0.0) -> None:
        self.hidden, self.width, self.decay, self.start = hidden, width, decay, start

    def state_spec(self):
        return StateSpec((self.width,), torch.float32)

    def initial_state(self):
        return torch.full((self.width,), self.start) if self.start else None

    def tensors(self):
        return {"in_proj.weight": TensorSpec((self.width, self.hidden)), "out_proj.weight": TensorSpec((self.hidden, self.width))}

    def load(self, tensors, runtime):
        super().load(tensors, runtime)
        self.w_in, self.w_out = tensors["in_proj.weight"], tensors["out_proj.weight"]

    def forward(self, h, ctx):
        u = (h.float() @ self.w_in.float().t())
        if ctx.step.decode_only:
            # One token per request (padding rows of a captured step point at the scratch slot).
            slots = ctx.step.state_slots.long()
            out = self.decay * ctx.state[slots] + u
            ctx.state[slots] = out
        else:
            out = torch.empty_like(u)
            start = 0
            for slot, count in zip(ctx.step.state_slots.tolist(), ctx.step.q_lens):
                state = ctx.state[slot]
                for t in range(start, start + count):
                    state = self.decay * state + u[t]
                    out[t] = state
                ctx.state[slot] = state
                start += count
        return (out @ self.w_out.float().t()).to(h.dtype)


@register_mixer("toy_latent_mixer")
class ToyLatentMixer(Mixer):
    """Keeps ONE row of `latent` numbers per token in the paged cache (no keys and values): c_t =
    h_t W_c; the output at t is softmax_j<=t(q_t . c_j / 4) weighted sum of the c_j, projected."""

    def __init__(self, hidden: int, latent: int) -> None:
        self.hidden, self.latent = hidden, latent

    def kv_spec(self):
        return KVSpec(((1, self.latent),))

    def tensors(self):
        return {"c_proj.weight": TensorSpec((self.latent, self.hidden)), "q_proj.weight": TensorSpec((self.latent, self.hidden)),
                "o_proj.weight": TensorSpec((self.hidden, self.latent))}

    def load(self, tensors, runtime):
        super().load(tensors, runtime)
        self.w = {k: v.float() for k, v in tensors.items()}

    def forward(self, h, ctx):
        kv, step = ctx.kv, ctx.step
        c = h.float() @ self.w["c_proj.weight"].t()
        q = h.float() @ self.w["q_proj.weight"].t()
        rows = kv.row(0)  # [pages, 1, page_size, latent]
        assert kv.pages.shape[1:] == (1, 1, kv.page_size, self.latent)
        flat = rows.reshape(-1, self.latent)  # slot = page * page_size + offset, one head
        flat[kv.slot_mapping] = c.to(flat.dtype)
        out = torch.empty_like(c)
        start = 0
        for s, (count, held) in enumerate(zip(step.q_lens, step.seq_lens_host)):
            table = kv.block_table[s].long()
            js = torch.arange(held, device=h.device)
            cached = flat[table[js // kv.page_size] * kv.page_size + js % kv.page_size].float()
            for t in range(count):
                seen = cached[: held - count + t + 1]
                out[start + t] = torch.softmax(seen @ q[start + t] / 4.0, dim=0) @ seen
            start += count
        return (out @ self.w["o_proj.weight"].t()).to(h.dtype)


@register_embedding("toy_absolute_embedding")
class ToyAbsoluteEmbedding(Embedding):
    """x = table[id] + place[position]: a learned absolute position encoding."""

    def __init__(self, vocab: int, hidden: int, places: int) -> None:
        self.vocab, self.hidden, self.places = vocab, hidden, places

    def tensors(self):
        return {"weight": TensorSpec((self.vocab, self.hidden)), "place": TensorSpec((self.places, self.hidden))}

    def load(self, tensors, runtime):
        super().load(tensors, runtime)
        self.weight, self.place = tensors["weight"], tensors["place"]

    def forward(self, token_ids, positions):
        return self.weight[token_ids.long()].float() + self.place[positions.clamp_min(0).long()].float()


START = 0.25


def toy_spec(hidden=32, vocab=50):
    norm = PartSpec("rms_norm", {"size": hidden, "eps": 1e-6, "weight": "plain"})
    ff = PartSpec("gated_mlp", {"hidden": hidden, "inner": 48})
    norms = {"input_layernorm": norm, "post_attention_layernorm": norm}
    toy = PartSpec("pre_norm", {"mixer": PartSpec("toy_decay_mixer", {"hidden": hidden, "width": 24, "decay": 0.9,
                                                                      "start": START}),
                                "feed_forward": ff, "norms": norms, "mixer_name": "mixer"})
    latent = PartSpec("pre_norm", {"mixer": PartSpec("toy_latent_mixer", {"hidden": hidden, "latent": 12}),
                                   "feed_forward": ff, "norms": norms, "mixer_name": "mixer"})
    attention = PartSpec("pre_norm", {"mixer": PartSpec("gqa_attention", {
        "hidden": hidden, "heads": 2, "kv_heads": 1, "head_dim": 16, "scale": 0.25,
        "position": PartSpec("rotary", {"dims": 8, "theta": 100.0})}), "feed_forward": ff, "norms": norms})
    return ModelSpec(PartSpec("toy_absolute_embedding", {"vocab": vocab, "hidden": hidden, "places": 64}),
                     (LayerSpec(toy, "layers.0"), LayerSpec(latent, "layers.1"), LayerSpec(attention, "layers.2")),
                     (ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(2)), norm,
                     PartSpec("lm_head", {"vocab": vocab, "hidden": hidden}),
                     embedding_prefix="embed", final_norm_prefix="final_norm", head_prefix="head")


def toy_plain(w, ids, layout=(("decay", "layers.0"), ("latent", "layers.1"), ("attention", "layers.2"))):
    """The toy model, whole sequence, plain PyTorch; `layout` lists its layers' mixers in order."""
    positions = torch.arange(len(ids))
    x = w["embed.weight"][ids] + w["embed.place"][positions]
    rms = lambda v, name: plain_impl.rms_norm(v, w[name], 1e-6)
    causal = plain_impl.visible(positions, positions, None)
    for kind, prefix in layout:
        h = rms(x, f"{prefix}.input_layernorm.weight")
        if kind == "decay":
            u = h @ w[f"{prefix}.mixer.in_proj.weight"].t()
            state, rows = torch.full((24,), START), []
            for t in range(len(ids)):
                state = 0.9 * state + u[t]
                rows.append(state)
            x = x + torch.stack(rows) @ w[f"{prefix}.mixer.out_proj.weight"].t()
        elif kind == "latent":
            m = plain_impl.sub(w, f"{prefix}.mixer.")
            c, q = h @ m["c_proj.weight"].t(), h @ m["q_proj.weight"].t()
            scores = (q @ c.t() / 4.0).masked_fill(~causal, float("-inf"))
            x = x + (torch.softmax(scores, dim=-1) @ c) @ m["o_proj.weight"].t()
        else:
            a = plain_impl.sub(w, f"{prefix}.self_attn.")
            q = (h @ a["q_proj.weight"].t()).reshape(-1, 2, 16)
            k = (h @ a["k_proj.weight"].t()).reshape(-1, 1, 16)
            v = (h @ a["v_proj.weight"].t()).reshape(-1, 1, 16)
            rot = lambda z: torch.cat([plain_impl.rope(z[..., :8], positions, 100.0), z[..., 8:]], dim=-1)
            x = x + plain_impl.attention_core(rot(q), rot(k), v, causal, 0.25) @ a["o_proj.weight"].t()
        x = x + plain_impl.swiglu(rms(x, f"{prefix}.post_attention_layernorm.weight"), plain_impl.sub(w, f"{prefix}.mlp."))
    return rms(x, "final_norm.weight") @ w["head.weight"].t()


def toy_model():
    model = DecoderModel(toy_spec())
    g = torch.Generator().manual_seed(4)
    w = {name: (torch.randn(*s.shape, generator=g) * (0.2 if s.kind == "matrix" else 0.1) + (s.kind == "vector"))
         for name, s in model.tensors().items()}
    rt = runtime()
    model.load({k: v.to(CUDA) for k, v in w.items()}, rt)
    return model, w, rt


def test_toy_parts_are_registered_built_and_stepped():
    model, w, rt = toy_model()
    needs = model.cache_needs()
    assert needs[0].kv is None and needs[0].state == StateSpec((24,)) and needs[0].initial_state is not None
    assert needs[1].kv == KVSpec(((1, 12),)) and needs[2].kv == KVSpec.keys_and_values(1, 16)
    cache = CacheManager(needs, page_size=4, pages_per_group=24, max_requests=2, dtype=torch.float32, device=CUDA)
    assert len(cache.groups) == 2  # the latent rows and the keys and values have pages of their own
    assert cache.groups[0].pages.shape == (1, 24, 1, 1, 4, 12) and cache.groups[1].pages.shape == (1, 24, 2, 1, 4, 16)
    runner = StepRunner(model, cache, rt)
    a, b = tiny_configs.prompt(21, 50, 1), tiny_configs.prompt(14, 50, 2)
    ra, rb = cache.open("a"), cache.open("b")
    got_a = [runner.run([StepEntry(ra, a[:9], list(range(9)))])]
    mixed = runner.run([StepEntry(ra, a[9:10], [0]), StepEntry(rb, b[:8], list(range(8)))])
    got_a.append(mixed[:1])
    got_b = [mixed[1:]]
    mixed = runner.run([StepEntry(rb, b[8:], list(range(6))), StepEntry(ra, a[10:], list(range(11)))])
    got_b.append(mixed[:6])
    got_a.append(mixed[6:])
    assert plain_impl.relative_diff(torch.cat(got_a), toy_plain(w, a)) < 2e-5
    assert plain_impl.relative_diff(torch.cat(got_b), toy_plain(w, b)) < 2e-5
    # a slot that is reused starts from the mixer's initial state again
    cache.close("a")
    rc = cache.open("c")
    again = runner.run([StepEntry(rc, a, list(range(21)))])
    assert plain_impl.relative_diff(again, toy_plain(w, a)) < 2e-5
    cache.check()


def test_a_toy_mixer_with_state_decodes_from_a_captured_graph():
    """Three requests decode from a graph made for four: the padding row points at the scratch
    state slot, so no live request's state is touched by it."""
    spec = toy_spec()
    # Without the latent layer, whose toy mixer loops over requests on the host.
    spec = ModelSpec(spec.embedding, (spec.layers[0], spec.layers[2]), (ScheduleEntry(0), ScheduleEntry(1)),
                     spec.final_norm, spec.head, embedding_prefix="embed", final_norm_prefix="final_norm",
                     head_prefix="head")
    model = DecoderModel(spec)
    g = torch.Generator().manual_seed(9)
    w = {name: (torch.randn(*s.shape, generator=g) * (0.2 if s.kind == "matrix" else 0.1) + (s.kind == "vector"))
         for name, s in model.tensors().items()}
    rt = runtime()
    model.load({k: v.to(CUDA) for k, v in w.items()}, rt)

    plain = lambda ids: toy_plain(w, ids, layout=(("decay", "layers.0"), ("attention", "layers.2")))

    cache = CacheManager(model.cache_needs(), page_size=4, pages_per_group=64, max_requests=4, dtype=torch.float32,
                         device=CUDA)
    runner = StepRunner(model, cache, rt, cuda_graphs=True)
    assert runner.graphs is not None
    prompts = [tiny_configs.prompt(n, 50, 20 + n) for n in (17, 30, 9)]
    requests = [cache.open(f"r{i}") for i in range(3)]
    runner.run([StepEntry(r, p[:-5], []) for r, p in zip(requests, prompts)])
    rows = [runner.run([StepEntry(r, [p[len(p) - 5 + k]], [0]) for r, p in zip(requests, prompts)]) for k in range(5)]
    assert runner.graphs.replays == 5
    got = torch.stack(rows)  # [5, 3, vocab]
    for i, p in enumerate(prompts):
        assert plain_impl.relative_diff(got[:, i], plain(p)[-5:]) < 2e-5, i


# ---- a feed-forward with routing and another position encoding, again only here -------------------


@register_feed_forward("toy_routed_experts")
class ToyRoutedExperts(FeedForward):
    """Every token goes to the `top` experts with the largest router logits (float32), weighted by the
    softmax over those logits; an expert is a small gated MLP run on the package's products."""

    def __init__(self, hidden: int, inner: int, experts: int, top: int) -> None:
        self.hidden, self.inner, self.experts, self.top = hidden, inner, experts, top

    def tensors(self):
        out = {"router.weight": TensorSpec((self.experts, self.hidden))}
        for e in range(self.experts):
            out[f"experts.{e}.gate_up.weight"] = TensorSpec((2 * self.inner, self.hidden))
            out[f"experts.{e}.down.weight"] = TensorSpec((self.hidden, self.inner))
        return out

    def load(self, tensors, runtime):
        super().load(tensors, runtime)
        self.w = tensors

    def forward(self, h, ctx):
        logits = h.float() @ self.w["router.weight"].float().t()
        best, chosen = torch.topk(logits, self.top, dim=-1)
        share = torch.softmax(best, dim=-1)
        out = torch.zeros(h.shape[0], self.hidden, dtype=torch.float32, device=h.device)
        for e in range(self.experts):
            rows, place = torch.nonzero(chosen == e, as_tuple=True)
            if rows.numel() == 0:
                continue
            act = ops.linear_swiglu(h[rows].contiguous(), self.w[f"experts.{e}.gate_up.weight"])
            out.index_add_(0, rows, ops.linear(act, self.w[f"experts.{e}.down.weight"]).float() * share[rows, place, None])
        return out.to(h.dtype)


@register_position("toy_interpolated_rotary")
class ToyInterpolatedRotary(Position):
    """Rotary angles of positions divided by `factor` (linear position interpolation)."""

    def __init__(self, dims: int, theta: float, factor: float) -> None:
        self.dims, self.theta, self.factor = dims, theta, factor

    def load(self, tensors, runtime):
        super().load(tensors, runtime)
        exponent = torch.arange(self.dims // 2, dtype=torch.float64) * (2.0 / self.dims)
        self._table = (torch.pow(torch.tensor(self.theta, dtype=torch.float64), -exponent) / self.factor).float().to(runtime.device)

    def table(self):
        return self._table


def test_a_toy_routed_feed_forward_and_a_toy_position_encoding():
    """A layer whose feed-forward routes tokens to two of five experts and whose attention rotates by
    interpolated positions, beside a layer of the architecture's own parts: built from data, stepped
    whole, in portions and token by token, mixed with another request, against plain PyTorch."""
    hidden, vocab, inner, experts, top, factor = 40, 60, 24, 5, 2, 4.0
    norm = PartSpec("rms_norm", {"size": hidden, "eps": 1e-5, "weight": "plain"})
    norms = {"input_layernorm": norm, "post_attention_layernorm": norm}
    attention = lambda position: PartSpec("gqa_attention", {"hidden": hidden, "heads": 4, "kv_heads": 2, "head_dim": 16,
                                                            "scale": 0.25, "position": position})
    routed = PartSpec("pre_norm", {"mixer": attention(PartSpec("toy_interpolated_rotary", {"dims": 16, "theta": 50.0, "factor": factor})),
                                   "feed_forward": PartSpec("toy_routed_experts", {"hidden": hidden, "inner": inner,
                                                                                   "experts": experts, "top": top}),
                                   "norms": norms})
    dense = PartSpec("pre_norm", {"mixer": attention(PartSpec("rotary", {"dims": 16, "theta": 50.0})),
                                  "feed_forward": PartSpec("gated_mlp", {"hidden": hidden, "inner": 56}), "norms": norms})
    spec = ModelSpec(PartSpec("token_embedding", {"vocab": vocab, "hidden": hidden}),
                     (LayerSpec(routed, "layers.0"), LayerSpec(dense, "layers.1")), (ScheduleEntry(0), ScheduleEntry(1)), norm,
                     PartSpec("lm_head", {"vocab": vocab, "hidden": hidden}),
                     embedding_prefix="embed", final_norm_prefix="final_norm", head_prefix="head")
    model = DecoderModel(spec)
    g = torch.Generator().manual_seed(11)
    w = {name: (torch.randn(*s.shape, generator=g) * (0.3 if s.kind == "matrix" else 0.1) + (s.kind == "vector"))
         for name, s in model.tensors().items()}
    rt = runtime()
    model.load({k: v.to(CUDA) for k, v in w.items()}, rt)

    routes = []

    def plain(ids):
        positions = torch.arange(len(ids))
        x = w["embed.weight"][ids]
        rms = lambda v, name: plain_impl.rms_norm(v, w[name], 1e-5)
        causal = plain_impl.visible(positions, positions, None)
        for prefix, scale in (("layers.0", factor), ("layers.1", 1.0)):
            h = rms(x, f"{prefix}.input_layernorm.weight")
            a = plain_impl.sub(w, f"{prefix}.self_attn.")
            q = (h @ a["q_proj.weight"].t()).reshape(-1, 4, 16)
            k = (h @ a["k_proj.weight"].t()).reshape(-1, 2, 16)
            v = (h @ a["v_proj.weight"].t()).reshape(-1, 2, 16)
            rot = lambda z: plain_impl.rope(z, positions / scale, 50.0)
            x = x + plain_impl.attention_core(rot(q), rot(k), v, causal, 0.25) @ a["o_proj.weight"].t()
            h = rms(x, f"{prefix}.post_attention_layernorm.weight")
            if prefix == "layers.1":
                x = x + plain_impl.swiglu(h, plain_impl.sub(w, f"{prefix}.mlp."))
                continue
            m = plain_impl.sub(w, f"{prefix}.mlp.")
            best, chosen = torch.topk(h @ m["router.weight"].t(), top, dim=-1)
            share = torch.softmax(best, dim=-1)
            routes.append(chosen)
            rows = []
            for t in range(len(ids)):
                row = torch.zeros(hidden)
                for j in range(top):
                    e = int(chosen[t, j])
                    gu = h[t] @ m[f"experts.{e}.gate_up.weight"].t()
                    act = torch.nn.functional.silu(gu[:inner]) * gu[inner:]
                    row = row + share[t, j] * (act @ m[f"experts.{e}.down.weight"].t())
                rows.append(row)
            x = x + torch.stack(rows)
        return rms(x, "final_norm.weight") @ w["head.weight"].t()

    cache = CacheManager(model.cache_needs(), page_size=4, pages_per_group=32, max_requests=2, dtype=torch.float32, device=CUDA)
    runner = StepRunner(model, cache, rt)
    a, b = tiny_configs.prompt(23, vocab, 5), tiny_configs.prompt(11, vocab, 6)
    ra, rb = cache.open("a"), cache.open("b")
    got_a = [runner.run([StepEntry(ra, a[:10], list(range(10)))])]
    mixed = runner.run([StepEntry(ra, a[10:12], [0, 1]), StepEntry(rb, b[:7], list(range(7)))])
    got_a.append(mixed[:2])
    got_b = [mixed[2:]]
    for t in range(12, 23):
        step = [StepEntry(ra, a[t:t + 1], [0])] + ([StepEntry(rb, b[7:], list(range(4)))] if t == 12 else [])
        out = runner.run(step)
        got_a.append(out[:1])
        if t == 12:
            got_b.append(out[1:])
    assert plain_impl.relative_diff(torch.cat(got_a), plain(a)) < 2e-5
    assert plain_impl.relative_diff(torch.cat(got_b), plain(b)) < 2e-5
    assert len(set(torch.cat(routes).flatten().tolist())) == experts  # the routing is not trivial: every expert is used
    cache.check()
