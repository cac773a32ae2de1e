"""Generation through the entry point on the GPU: greedy ids equal the plain
implementation's, in 32-bit and bfloat16; sampled ids can be redrawn on the host from
the plain implementation's logits with the same random stream; long decoding and the
first tokens of a sequence; the command line."""

from __future__ import annotations

import subprocess
import sys

import pytest
import torch

import kernel_refs
import plain_impl
import tiny_configs
from mlx_omnia_b200 import GenerationOptions, load, sampler, temperature, top_k, top_p
from trace_tools import ROOT, write_folder

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name,dtype,page", [("A", "float32", 4), ("B", "float32", 8), ("A", "bfloat16", 4),
                                             ("B", "bfloat16", 8)])
def test_greedy_through_the_entry_point(tmp_path, name, dtype, page):
    raw, weights = write_folder(tmp_path / "m", name)
    vocab = raw["text_config"]["vocab_size"]
    lengths = (5, 9, 13) if name == "A" else (3, 17, 31, 40)
    prompts = [tiny_configs.prompt(n, vocab, 40 + n) for n in lengths]
    model = load(tmp_path / "m", dtype=dtype, page_size=page, cache_tokens=512, max_requests=4,
                 max_tokens_per_step=8)
    got = model.generate(prompts, GenerationOptions(max_tokens=8, stop=()))
    if dtype == "float32":
        assert got == [plain_impl.greedy_generate(raw, weights, p, 8) for p in prompts]
    else:
        # In bfloat16 a near-tie may break the other way; every chosen token must be (nearly) the
        # plain implementation's best given the same history.
        for prompt, ids in zip(prompts, got):
            logits = plain_impl.forward(raw, weights, prompt + ids)[len(prompt) - 1: -1]
            chosen = logits[torch.arange(len(ids)), torch.tensor(ids)]
            assert float((logits.max(dim=-1).values - chosen).max()) < 0.03 * float(logits.abs().max())
    streamed = [s.token_id for s in model.stream(prompts[0], GenerationOptions(max_tokens=8, stop=()))]
    assert streamed == got[0]
    assert not model.engine.cache.requests


def test_sampled_ids_can_be_redrawn_on_the_host(tmp_path):
    raw, weights = write_folder(tmp_path / "m", "B")
    model = load(tmp_path / "m", dtype="float32", page_size=8, cache_tokens=512, max_requests=4, max_tokens_per_step=8)
    prompts = [tiny_configs.prompt(n, 1000, 70 + n) for n in (3, 17, 31, 40)]
    chosen = sampler(temperature(0.8), top_k(50), top_p(0.95), seed=1234)
    got = model.generate(prompts, GenerationOptions(max_tokens=6, sampler=chosen, stop=()))
    for prompt, ids in zip(prompts, got):
        for draw, token in enumerate(ids):
            logits = plain_impl.forward(raw, weights, prompt + ids[:draw])[-1]
            keep = kernel_refs.kept_mask(logits, 0.8, 50, 0.95, 0.0)
            scores = {t: float(logits[t]) / 0.8 + kernel_refs.gumbel(1234, draw, t)
                      for t in torch.nonzero(keep).flatten().tolist()}
            assert token in scores and scores[token] >= max(scores.values()) - 1e-3
    again = model.generate(prompts, GenerationOptions(max_tokens=6, sampler=chosen, stop=()))
    assert again == got


def test_long_decoding_and_first_tokens(tmp_path):
    """300 tokens decoded one by one from a two-token prompt stay on the plain
    implementation's logits, across many pages and past the window of B's sliding layers."""
    raw, weights = write_folder(tmp_path / "m", "B")
    model = load(tmp_path / "m", dtype="float32", page_size=8, cache_tokens=1024, max_requests=2)
    prompt = tiny_configs.prompt(2, 1000, 5)
    ids = model.generate([prompt], GenerationOptions(max_tokens=300, stop=()))[0]
    expect = plain_impl.forward(raw, weights, prompt + ids)
    assert ids == expect[1:-1].argmax(dim=-1).tolist()


def test_command_line(tmp_path):
    raw, weights = write_folder(tmp_path / "m", "A")
    prompt = tiny_configs.prompt(7, 512, 3)
    done = subprocess.run([sys.executable, str(ROOT / "bin" / "omnia"), "run", "-m", str(tmp_path / "m"),
                           "--max-tokens", "5", "--temperature", "0", "--dtype", "float32", *map(str, prompt)],
                          capture_output=True, text=True, timeout=300)
    assert done.returncode == 0, done.stderr[-2000:]
    expect = plain_impl.greedy_generate(raw, weights, prompt, 5)
    cut = expect.index(0) if 0 in expect else len(expect)  # token 0 is this configuration's eos
    assert done.stdout.split() == [str(t) for t in expect[:cut]]
    empty = subprocess.run([sys.executable, str(ROOT / "bin" / "omnia"), "run", "-m", str(tmp_path / "m")],
                           capture_output=True, text=True, stdin=subprocess.DEVNULL, timeout=120)
    assert empty.returncode == 2 and "nothing to say" in empty.stderr


@pytest.mark.parametrize("name,dtype", [("B", "float32"), ("C", "bfloat16")])
def test_captured_decode_steps_equal_eager_ones(name, dtype):
    """Single-token steps replayed from a CUDA graph give the logits of the same steps
    launched one kernel at a time, with three requests of different lengths in flight."""
    from mlx_omnia_b200.engine.engine import Engine, EngineArgs
    from mlx_omnia_b200.engine.step import StepEntry

    raw, weights = tiny_configs.config(name), tiny_configs.tensors(name)
    vocab = raw["text_config"]["vocab_size"]
    prompts = [tiny_configs.prompt(n, vocab, 90 + n) for n in (70, 9, 33)]
    results = []
    for graphs in (False, True):
        engine = Engine.from_tensors(raw, weights, EngineArgs(dtype=dtype, page_size=8, cache_tokens=512,
                                                              max_requests=4, cuda_graphs=graphs))
        requests = [engine.cache.open(f"r{i}") for i in range(3)]
        engine.runner.run([StepEntry(r, p[:-20], []) for r, p in zip(requests, prompts) if len(p) > 20])
        rows = []
        for k in range(20):
            live = [(r, p[len(p) - 20 + k]) for r, p in zip(requests, prompts) if len(p) > 20 or k >= 20 - len(p)]
            rows.append(engine.runner.run([StepEntry(r, [t], [0]) for r, t in live]))
        assert (engine.runner.graphs is not None and engine.runner.graphs.replays > 0) == graphs
        results.append(torch.cat(rows))
    assert torch.equal(results[0], results[1])
    expect = plain_impl.forward(raw, weights, prompts[0])[-20:]
    picks, at = [], 0
    for k in range(20):
        live = [i for i, p in enumerate(prompts) if len(p) > 20 or k >= 20 - len(p)]
        picks.append(results[1][at + live.index(0)])
        at += len(live)
    assert plain_impl.relative_diff(torch.stack(picks), expect) < (1e-4 if dtype == "float32" else 3e-2)


def test_pipelined_decoding_gives_the_same_tokens(tmp_path):
    """Launching step n + 1 from the tokens still on the device, before step n's tokens are read,
    changes nothing: greedy and seeded sampling give the ids of the step-by-step loop, stop tokens
    end a request at the same place, and nothing is left in the cache."""
    from mlx_omnia_b200.engine.engine import Engine, EngineArgs
    from mlx_omnia_b200.engine.generate import Generator

    raw, weights = tiny_configs.config("B"), tiny_configs.tensors("B")
    prompts = [tiny_configs.prompt(n, 1000, 300 + n) for n in (5, 19, 33)]
    plain_ids = plain_impl.greedy_generate(raw, weights, prompts[0], 24)
    for options in (GenerationOptions(max_tokens=24, stop=()),
                    GenerationOptions(max_tokens=24, stop=(plain_ids[9],)),
                    GenerationOptions(max_tokens=17, sampler=sampler(temperature(0.9), top_k(30), seed=5), stop=())):
        results = []
        for pipelined in (False, True):
            engine = Engine.from_tensors(raw, weights, EngineArgs(dtype="float32", page_size=8, cache_tokens=512,
                                                                  max_requests=4))
            generator = Generator(engine)
            generator.pipelined = pipelined
            results.append(generator.generate(prompts, options))
            assert not engine.cache.requests and generator._in_flight is None
            assert all(g.pool.free == g.pool.count for g in engine.cache.groups)
        assert results[0] == results[1]
        if options.sampler.greedy:
            cut = plain_ids.index(plain_ids[9]) if options.stop else 24
            assert results[1][0] == plain_ids[:cut]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_preemption_on_the_gpu(dtype):
    """A pool too small for three requests at once: the newest is preempted, gives its pages
    back, and later recomputes its prompt and what it had generated as one long portion beside
    the others' decoded tokens, with captured graphs and pipelined steps on. In 32-bit the
    sampled tokens are those of a roomy pool; in bfloat16 (where a different batch rounds
    differently) every greedy token is the plain implementation's best or nearly so."""
    from mlx_omnia_b200 import repetition_penalty
    from mlx_omnia_b200.engine.engine import Engine, EngineArgs
    from mlx_omnia_b200.engine.generate import Generator

    raw, weights = tiny_configs.config("A"), tiny_configs.tensors("A")
    prompts = [tiny_configs.prompt(n, 512, 60 + n) for n in (17, 9, 12)]
    if dtype == "float32":
        options = GenerationOptions(max_tokens=14, sampler=sampler(temperature(0.9), top_k(20), seed=11), stop=(),
                                    penalty=repetition_penalty(1.3))
    else:
        options = GenerationOptions(max_tokens=14, stop=())
    results = {}
    for pool in (512, 56):
        engine = Engine.from_tensors(raw, weights, EngineArgs(dtype=dtype, page_size=4, cache_tokens=pool, max_requests=4))
        generator = Generator(engine)
        assert generator.pipelined and engine.runner.graphs is not None
        requests = [generator.add(p, options) for p in prompts]
        generator.run()
        results[pool] = [r.generated for r in requests]
        assert (sum(r.preemptions for r in requests) > 0) == (pool == 56)
        assert not engine.cache.requests and all(g.pool.free == g.pool.count for g in engine.cache.groups)
        engine.cache.check()
    if dtype == "float32":
        assert results[56] == results[512]
    else:
        for prompt, ids in zip(prompts, results[56]):
            logits = plain_impl.forward(raw, weights, prompt + ids)[len(prompt) - 1: -1]
            chosen = logits[torch.arange(len(ids)), torch.tensor(ids)]
            assert float((logits.max(dim=-1).values - chosen).max()) < 0.03 * float(logits.abs().max())


def test_command_line_takes_text_and_the_checkpoint_s_defaults(tmp_path):
    """A folder with a tokenizer.json and a generation_config.json: `omnia run -m DIR "hello world"`
    encodes the prompt, decodes greedily because the checkpoint says `do_sample: false`, stops at the
    id the generation config adds, prints text, and with --verbose the request's numbers on stderr."""
    import json

    from test_text import tokenizer_json

    raw, weights = write_folder(tmp_path / "m", "A")
    declared = tokenizer_json()
    known = len(declared["model"]["vocab"]) + len(declared["added_tokens"])
    declared["added_tokens"] += [{"id": i, "content": f"<|{i}|>"} for i in range(known, 512)]
    (tmp_path / "m" / "tokenizer.json").write_text(json.dumps(declared), encoding="utf-8")
    vocab = declared["model"]["vocab"]
    prompt = [vocab["hello"], vocab["Ġworld"]]
    expect = plain_impl.greedy_generate(raw, weights, prompt, 12)
    stop_at = expect[7]
    (tmp_path / "m" / "generation_config.json").write_text(json.dumps({"do_sample": False, "eos_token_id": [stop_at]}))
    done = subprocess.run([sys.executable, str(ROOT / "bin" / "omnia"), "run", "-m", str(tmp_path / "m"),
                           "--max-tokens", "12", "--dtype", "float32", "--verbose", "hello world"],
                          capture_output=True, text=True, timeout=300)
    assert done.returncode == 0, done.stderr[-2000:]
    cut = min(expect.index(t) for t in (stop_at, 0) if t in expect)  # token 0 is config.json's own eos
    from mlx_omnia_b200.text import ByteLevelBPE

    tokenizer = ByteLevelBPE.from_file(tmp_path / "m" / "tokenizer.json")
    assert done.stdout.rstrip("\n") == tokenizer.decode(expect[:cut]).rstrip("\n")
    assert f"prompt 2 tokens, completion {cut} tokens" in done.stderr


@pytest.mark.parametrize("name,dtype,page,portion,steps", [("B", "float32", 8, 48, 7), ("C", "bfloat16", 16, 48, 7),
                                                           ("A", "bfloat16", 4, 48, 7), ("C", "bfloat16", 16, 96, 14)])
def test_captured_mixed_steps_equal_eager_ones(name, dtype, page, portion, steps):
    """Decoding requests beside a long prompt that is read in equal portions: the step's shape comes
    again and again, so it is captured at its third coming and replayed from then on. The logits are
    those of the same steps launched kernel by kernel, the cache is the same afterwards (what is
    decoded later agrees too), and the reader's logits match the plain implementation. In the last
    case the prompt grows to 1,344 tokens: the tcgen05 attention kernel's blocks are then listed in
    parts, more of them from replay to replay, in a list whose place was made before the capture."""
    from floors import Oracle
    from mlx_omnia_b200.engine.engine import Engine, EngineArgs
    from mlx_omnia_b200.engine.step import StepEntry

    raw, weights = tiny_configs.config(name), tiny_configs.tensors(name)
    vocab = raw["text_config"]["vocab_size"]
    decoders = [tiny_configs.prompt(n, vocab, 400 + n) for n in (37, 90, 11)]
    reader = tiny_configs.prompt(steps * portion, vocab, 499)
    results = []
    for graphs in (False, True):
        engine = Engine.from_tensors(raw, weights, EngineArgs(dtype=dtype, page_size=page, cache_tokens=1024 + steps * portion,
                                                              max_requests=4, cuda_graphs=graphs))
        requests = [engine.cache.open(f"d{i}") for i in range(3)]
        long_one = engine.cache.open("reader")
        engine.runner.run([StepEntry(r, p[:-8], []) for r, p in zip(requests, decoders)])
        rows = []
        for k in range(steps):  # mixed steps of one shape: three decoded tokens beside a portion of the prompt
            entries = [StepEntry(r, [p[len(p) - 8 + k % 7]], [0]) for r, p in zip(requests, decoders)] if k < 7 else \
                [StepEntry(r, [1 + k], [0]) for r in requests]
            entries.append(StepEntry(long_one, reader[portion * k: portion * (k + 1)], [0, portion - 1]))
            rows.append(engine.runner.run(entries))
        rows.append(engine.runner.run([StepEntry(r, [p[-1]], [0]) for r, p in zip(requests, decoders)]))
        if graphs:
            # A shape is captured at its third coming; its tables are as wide as the next power of two
            # above the prompt's pages (64 at least), so the longer prompt outgrows its first graph.
            # The step that brings the prompt's first portion has a key of its own (kernels may be chosen by
            # whether a step's prompts start at their first token).
            widths = [(max(64, 1 << (-(-portion * (k + 1) // page) - 1).bit_length()), k == 0) for k in range(steps)]
            comings = {w: widths.count(w) for w in set(widths)}
            assert engine.runner.mixed_graphs.replays == sum(max(0, n - 3) for n in comings.values()) >= 1
            assert len(engine.runner.mixed_graphs.captured) == sum(n >= 3 for n in comings.values())
        ops_check(engine)
        results.append(torch.cat(rows))
    assert torch.equal(results[0], results[1])
    oracle = Oracle(raw, weights, {"reader": reader})
    got = torch.stack([results[1][5 * k + 3 + j] for k in range(steps) for j in range(2)])
    want_rows = [portion * k + w for k in range(steps) for w in (0, portion - 1)]
    assert oracle.diff("reader", got, want_rows) < oracle.tolerance[dtype]


def ops_check(engine):
    from mlx_omnia_b200.kernels import ops

    ops.raise_on_error(engine.runtime.device)
    engine.cache.check()
