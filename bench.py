"""Decode and prefill throughput of the engine on one B200, as one JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

The default run builds the headline model (28 layers, hidden 2048, 16/8 heads
of 128, intermediate 6144, vocabulary 151936, tied head) with random bfloat16 weights,
holds 8 requests whose contexts end at 4096 tokens, and times K decode steps.
`value` is decoded tokens per second timed on the device; `e2e` is the same measured
through the Python entry point's generation loop, which copies every step's inputs
from pinned host memory and reads the chosen tokens back. `prefill` is one step of
2,048 prompt tokens; `roofline` relates the decode step's time to the bytes it must
read (every weight once, and the live requests' cache). `points` holds decode at
batch 1 and 64, two mixed steps (milliseconds a step: eight decoding requests at
4,096 tokens beside a 256-token portion of a prompt, and a lone 128-token portion) and the
time to read a prompt of 8,192 tokens in portions of 512 (a token budget).
`kernels` times each class of kernel alone (operands rotated through more memory than
L2 holds, replayed from a CUDA graph) against the measured peaks: the streamed product
of a decode step, the head, decode attention (GB/s), the prefill product and prefill
attention (TFLOP/s). Data is synthetic: seeded uniform-random token ids.
"""

from __future__ import annotations

import argparse
import json
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

CONFIG2 = {
    "architectures": ["MuseGlimmerForConditionalGeneration"], "model_type": "muse_glimmer",
    "text_config": {
        "hidden_size": 2048, "intermediate_size": 6144, "num_hidden_layers": 28, "num_attention_heads": 16,
        "num_key_value_heads": 8, "head_dim": 128, "vocab_size": 151936, "rms_norm_eps": 1e-6, "post_norm_eps": 1e-6,
        "sliding_window": 4096, "qk_scale_factor": 1.0, "output_multiplier": 1.0, "final_logit_softcapping": 30.0,
        "layer_types": ["full_attention"] * 28, "layer_rope_theta": [1000000.0] * 28,
        "rope_parameters": {"rope_theta": 1000000.0, "rope_type": "default"}, "eos_token_id": [],
        "tie_word_embeddings": True,
    },
}
CONFIG3 = {
    "architectures": ["MuseGlimmerForConditionalGeneration"], "model_type": "muse_glimmer",
    "text_config": {
        "hidden_size": 4096, "intermediate_size": 12288, "num_hidden_layers": 36, "num_attention_heads": 32,
        "num_key_value_heads": 8, "head_dim": 128, "vocab_size": 151936, "rms_norm_eps": 1e-6, "post_norm_eps": 1e-6,
        "sliding_window": 8192, "qk_scale_factor": 1.0, "output_multiplier": 1.0, "final_logit_softcapping": 30.0,
        "layer_types": ["full_attention"] * 36, "layer_rope_theta": [1000000.0] * 36,
        "rope_parameters": {"rope_theta": 1000000.0, "rope_type": "default"}, "eos_token_id": [],
        "tie_word_embeddings": False,
    },
}
CONFIGS = {2: (CONFIG2, 4096), 3: (CONFIG3, 8192)}  # the sizes and the context of a benchmark configuration
SEED = 2
CONTEXT = 4096
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            data = json.loads(path.read_text())
            flat = {}
            for key in FALLBACK_PEAKS:
                value = data.get(key)
                if isinstance(value, dict):
                    value = value.get("value")
                flat[key] = float(value) if value else FALLBACK_PEAKS[key]
            return flat, "measured"
        except (ValueError, TypeError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self) -> None:
        self.rows: list[list[str]] = []
        self.process = None

    def __enter__(self):
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.process = None
        return self

    def _read(self) -> None:
        for line in self.process.stdout:
            self.rows.append([cell.strip() for cell in line.split(",")])

    def __exit__(self, *exc) -> None:
        if self.process is not None:
            self.process.terminate()
            self.thread.join(timeout=2)

    def summary(self) -> dict:
        clocks = [int(r[0]) for r in self.rows if r and r[0].isdigit()]
        peak = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > i + 2 and r[i + 2] == "Active" for r in self.rows)]
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": max(peak) if peak else None,
                "reasons": reasons, "samples": len(clocks)}


def model_bytes(text: dict, layers: int) -> tuple[int, int, int]:
    """(weight bytes a decode step reads, cache bytes per token of context, parameters)."""
    h, i, d = text["hidden_size"], text["intermediate_size"], text["head_dim"]
    q, kv = text["num_attention_heads"] * d, text["num_key_value_heads"] * d
    per_layer = h * (2 * q + 2 * kv) + q * h + 3 * h * i
    head = text["vocab_size"] * h
    params = layers * per_layer + head * (1 if text["tie_word_embeddings"] else 2)
    return 2 * (layers * per_layer + head), 2 * 2 * layers * kv, params


def run(args) -> dict:
    import torch

    from mlx_omnia_b200.engine.decode_graph import capturing
    from mlx_omnia_b200.engine.engine import Engine, EngineArgs
    from mlx_omnia_b200.engine.generate import Generator
    from mlx_omnia_b200.engine.step import StepEntry
    from mlx_omnia_b200.kernels import ops
    from mlx_omnia_b200.sampling import GenerationOptions

    raw = json.loads(json.dumps(CONFIGS[args.config][0]))
    text = raw["text_config"]
    full_layers = text["num_hidden_layers"]
    layers = args.layers or full_layers
    text["num_hidden_layers"] = layers
    text["layer_types"], text["layer_rope_theta"] = text["layer_types"][:layers], text["layer_rope_theta"][:layers]
    vocab = text["vocab_size"]
    measured, peak_source = peaks()
    weight_bytes, kv_per_token, params = model_bytes(text, layers)

    batches = sorted({1, args.batch, 64}) if args.only == "all" else [args.batch]
    cache_tokens = max(batches) * (args.context + 16) + max(PREFILL_TOKENS, args.prefill_tokens,
                                                              32768 + 16 if args.only == "portions" else 8192 + 16,
                                                              (max(args.steps, 8) + max(args.warmup, 3) + 2) * args.portion)
    cache_tokens = max(cache_tokens, args.pool_tokens)
    engine = Engine.from_random(raw, SEED, EngineArgs(dtype="bfloat16", page_size=16, cache_tokens=cache_tokens,
                                                      max_requests=max(batches) + 1))
    g = torch.Generator().manual_seed(SEED)

    def prompts(count: int, length: int) -> list[list[int]]:
        return torch.randint(0, vocab, (count, length), generator=g).tolist()

    def events():
        return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def decode(batch: int, steps: int, warmup: int) -> dict:
        """Fill `batch` requests so that the timed steps end at CONTEXT tokens, then time them."""
        total = warmup + steps
        length = args.context - total - 1
        # One step reads all prompts whole, so every request decodes in lockstep afterwards.
        generator = Generator(engine, max_tokens_per_step=batch * length)
        options = GenerationOptions(max_tokens=total + 1, stop=())
        for p in prompts(batch, length):
            generator.add(p, options)
        assert len(generator.step()) == batch
        for _ in range(warmup):
            generator.step()
        torch.cuda.synchronize()
        start, stop = events()
        launches = ops.launches
        wall = time.perf_counter()
        start.record()
        for _ in range(steps):
            outputs = generator.step()
        stop.record()
        torch.cuda.synchronize()
        wall = time.perf_counter() - wall
        ms = start.elapsed_time(stop) / steps
        assert len(outputs) == batch
        context = generator.scheduler.running[0].computed if generator.scheduler.running else args.context
        generator.run()
        return {"ms": ms, "tokens_per_s": batch * 1000.0 / ms, "wall_tokens_per_s": batch * steps / wall,
                "launches": (ops.launches - launches) // steps, "context": context}

    def prefill(tokens: int, steps: int, warmup: int) -> dict:
        times = []
        for index in range(warmup + steps):
            request = engine.cache.open(f"prefill-{index}")
            ids = prompts(1, tokens)[0]
            torch.cuda.synchronize()
            start, stop = events()
            start.record()
            engine.runner.run([StepEntry(request, ids, [tokens - 1])])
            stop.record()
            torch.cuda.synchronize()
            engine.cache.close(request.request_id)
            if index >= warmup:
                times.append(start.elapsed_time(stop))
        ms = statistics.median(times)
        h, d, nq = text["hidden_size"], text["head_dim"], text["num_attention_heads"]
        matmul = 2 * (weight_bytes // 2 - vocab * h) * tokens + 2 * vocab * h  # the head runs on one row
        attention = layers * 4 * nq * d * tokens * (tokens + 1) // 2
        flops = matmul + attention
        return {"value": tokens * 1000.0 / ms, "tokens": tokens, "ms": ms,
                "frac": flops / (ms / 1000.0) / (measured["bf16_tflops"] * 1e12), "flops": flops}

    def mixed(decoders: int, portion: int, steps: int, warmup: int) -> dict:
        """`decoders` requests at `args.context` tokens decode beside `portion` tokens of a long prompt."""
        requests = [engine.cache.open(f"mixed-{i}") for i in range(decoders)]
        reader = engine.cache.open("mixed-reader")
        if decoders:
            engine.runner.run([StepEntry(r, p, []) for r, p in zip(requests, prompts(decoders, args.context - steps - warmup - 1))])
        times, walls = [], []
        for index in range(warmup + steps):
            entries = [StepEntry(r, [1 + index], [0]) for r in requests] + [StepEntry(reader, prompts(1, portion)[0], [])]
            torch.cuda.synchronize()
            start, stop = events()
            wall = time.perf_counter()
            start.record()
            engine.runner.run(entries)
            stop.record()
            torch.cuda.synchronize()
            wall = time.perf_counter() - wall
            if index >= warmup:
                times.append(start.elapsed_time(stop))
                walls.append(wall * 1e3)
        for r in requests + [reader]:
            engine.cache.close(r.request_id)
        return {"ms": statistics.median(times), "wall_ms": statistics.median(walls)}

    def portions(total: int, portion: int) -> float:
        """Milliseconds to read a prompt of `total` tokens in portions of `portion` (a token budget), warm:
        the best of four prompts (steps whose shape has come three times run from captured graphs)."""
        best = None
        for attempt in range(4):
            request = engine.cache.open(f"portions-{attempt}")
            ids = prompts(1, total)[0]
            torch.cuda.synchronize()
            start, stop = events()
            start.record()
            for at in range(0, total, portion):
                engine.runner.run([StepEntry(request, ids[at:at + portion], [portion - 1] if at + portion >= total else [])])
            stop.record()
            torch.cuda.synchronize()
            engine.cache.close(request.request_id)
            best = start.elapsed_time(stop) if best is None else min(best, start.elapsed_time(stop))
        return best

    def kernel_classes() -> dict:
        """Each class of kernel alone, replayed from a graph over operands that do not fit L2."""
        from mlx_omnia_b200.parts.base import KVView, StepContext

        device = engine.runtime.device
        h, inner, d = text["hidden_size"], text["intermediate_size"], text["head_dim"]
        nq, nkv = text["num_attention_heads"], text["num_key_value_heads"]
        draw = lambda *shape: torch.randn(*shape, device=device, dtype=torch.bfloat16) * 0.05

        def timed(body, sets: int) -> float:
            """Seconds per call of `body(i)`, i cycling through `sets` operand sets."""
            side = torch.cuda.Stream()
            with torch.cuda.stream(side):
                for i in range(sets):
                    body(i)
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                with capturing(graph, stream=side):
                    for i in range(sets):
                        body(i)
            torch.cuda.synchronize()
            for _ in range(3):
                graph.replay()
            start, stop = events()
            start.record()
            for _ in range(5):
                graph.replay()
            stop.record()
            torch.cuda.synchronize()
            return start.elapsed_time(stop) / 1e3 / (5 * sets)

        def record(seconds: float, amount: float, peak: float, unit: str) -> dict:
            achieved = amount / seconds / (1e9 if unit == "GB/s" else 1e12)
            return {"achieved": round(achieved, 1), "unit": unit, "frac": round(achieved / peak, 3), "us": round(seconds * 1e6, 2)}

        out = {}
        hbm, tensor = measured["hbm_gbs"], measured["bf16_tflops"]
        # K3: the streamed product of a decode step (gate|up with SwiGLU, 8 rows).
        weights = [draw(2 * inner, h) for _ in range(6)]
        rows8 = draw(8, h)
        out["k3_streamed_product"] = record(timed(lambda i: ops.linear_swiglu(rows8, weights[i]), 6), 2 * 2 * inner * h, hbm, "GB/s")
        # K10: the head with its soft cap, 8 rows.
        table = engine.model.embedding.weight
        out["k10_head"] = record(timed(lambda i: ops.linear_softcap(rows8, table, 1.0, 30.0), 1), 2 * vocab * h, hbm, "GB/s")
        # K2: a prefill product (2,048 rows, gate|up with SwiGLU).
        rows2k = draw(PREFILL_TOKENS, h)
        out["k2_prefill_product"] = record(timed(lambda i: ops.linear_swiglu(rows2k, weights[i]), 6),
                                           2.0 * PREFILL_TOKENS * 2 * inner * h, tensor, "TFLOP/s")
        del weights
        # K6 / K5: attention over a paged cache of random values, pages in order.
        def attention(batch: int, q_len: int, context: int):
            pages_per = -(-context // 16)
            sets = max(2, int(200e6 // (batch * pages_per * 2 * nkv * 16 * d * 2)) + 1)
            caches = [draw(batch * pages_per, 2, nkv, 16, d) for _ in range(sets)]
            i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=device)
            table = torch.arange(batch * pages_per, dtype=torch.int32, device=device).view(batch, pages_per)
            tokens = batch * q_len
            step = StepContext(
                num_tokens=tokens, num_seqs=batch, token_ids=i32([0] * tokens),
                positions=i32([context - q_len + t for _ in range(batch) for t in range(q_len)]),
                cu_seqlens=i32([q_len * b for b in range(batch + 1)]), seq_lens=i32([context] * batch),
                state_slots=i32([0] * batch), fresh=i32([0] * batch), logit_rows=i32([]), q_lens=[q_len] * batch,
                seq_lens_host=[context] * batch, max_q_len=q_len, max_seq_len=context, decode_only=q_len == 1,
                groups={}, workspace={"private": True})
            q, gate = draw(tokens, nq, d) * 20, draw(tokens, nq * d)
            slots = torch.zeros(tokens, dtype=torch.int64, device=device)
            seconds = timed(lambda i: ops.paged_attention(q, KVView(caches[i], table, slots, 16, None), step,
                                                          d ** -0.5, gate=gate), sets)
            return seconds

        out["k6_decode_attention"] = record(attention(args.batch, 1, args.context),
                                            args.batch * args.context * 2 * nkv * d * 2, hbm, "GB/s")
        out["k5_prefill_attention"] = record(attention(1, PREFILL_TOKENS, PREFILL_TOKENS),
                                             4.0 * nq * d * PREFILL_TOKENS * (PREFILL_TOKENS + 1) / 2, tensor, "TFLOP/s")
        return out

    if args.timeline:
        # One step of a tracing build, kernel by kernel as it runs (set OMNIA_TIMELINE=1): the lines
        # go to stderr, the record says how many kernels were seen.
        from mlx_omnia_b200.kernels import timeline
        if args.only == "prefill":
            prefill(args.prefill_tokens, 1, 2)
            torch.cuda.synchronize()
            timeline.spans()
            prefill(args.prefill_tokens, 1, 0)
            anchor = "attention_tcgen05"
        elif args.only == "mixed":
            # Eager steps (a captured shape would be replayed without passing the host-side marks).
            decoders = [engine.cache.open(f"mixed-{i}") for i in range(args.batch)]
            reader = engine.cache.open("mixed-reader")
            if decoders:
                engine.runner.run([StepEntry(r, p, []) for r, p in zip(decoders, prompts(args.batch, args.context - 4))])
            graphs, engine.runner.mixed_graphs = getattr(engine.runner, "mixed_graphs", None), None
            for index in range(3):
                if index == 2:
                    torch.cuda.synchronize()
                    timeline.spans()
                engine.runner.run([StepEntry(r, [1 + index], [0]) for r in decoders] +
                                  [StepEntry(reader, prompts(1, args.portion)[0], [])])
            engine.runner.mixed_graphs = graphs
            anchor = "attention_tcgen05"
        else:
            length = args.context - 16
            generator = Generator(engine, max_tokens_per_step=args.batch * length)
            for p in prompts(args.batch, length):
                generator.add(p, GenerationOptions(max_tokens=12, stop=()))
            for _ in range(6):
                generator.step()
            torch.cuda.synchronize()
            timeline.spans()
            generator.step()
            anchor = "attention_tc"
        torch.cuda.synchronize()
        kernels = timeline.spans()
        print("\n".join(timeline.by_layer(kernels, anchor)), file=sys.stderr)
        return {"only": args.only, "timeline": True, "kernels": len(kernels), "layers": layers}
    if args.only == "decode":  # a small case for profilers: one batch size, no prefill timing
        part = decode(args.batch, args.steps, args.warmup)
        step_bytes = weight_bytes + args.batch * part["context"] * kv_per_token
        return {"only": "decode", "config": args.config, "batch": args.batch, "layers": layers,
                "ms_per_step": round(part["ms"], 4), "tokens_per_s": round(part["tokens_per_s"], 1),
                "context": part["context"], "step_gb": round(step_bytes / 1e9, 2),
                "hbm_frac": round(step_bytes / (part["ms"] / 1e3) / 1e9 / measured["hbm_gbs"], 3)}
    def replayed(body, sets: int, rounds: int = 10) -> float:
        """Microseconds per call of `body(i)`, i over `sets` operand sets, replayed from a graph."""
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            for i in range(sets):
                body(i)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with capturing(graph, stream=side):
                for i in range(sets):
                    body(i)
        torch.cuda.synchronize()
        graph.replay()
        start, stop = events()
        start.record()
        for _ in range(rounds):
            graph.replay()
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop) * 1e3 / (rounds * sets)

    if args.only == "portions":
        # Prompts read in portions (a token budget): milliseconds for the whole prompt, with the attention
        # kernel's blocks cut into parts as the dispatch cuts them, and whole (no part shorter than a
        # million tiles).
        record = {"only": "portions", "config": args.config, "layers": layers, "unit": "ms"}
        kept = ops.PREFILL_MIN_PART_TILES
        for label, least in (("in_parts", kept), ("whole_blocks", 10 ** 6)):
            ops.PREFILL_MIN_PART_TILES = least
            record[label] = {f"{total}_in_{portion}": round(portions(total, portion), 2)
                             for total, portion in ((8192, 512), (8192, 256), (32768, 1024), (32768, 512))}
        ops.PREFILL_MIN_PART_TILES = kept
        ops.raise_on_error(engine.runtime.device)
        return record
    if args.only == "products":
        # A layer's four products at several row counts: this package's kernels (the streaming kernel up
        # to 16 rows, the one-SM and the two-SM tcgen05 kernels) beside the vendor library's product
        # (followed by the SwiGLU kernel for gate|up); weights fresh for every launch.
        device = engine.runtime.device
        h, inner = text["hidden_size"], text["intermediate_size"]
        q, kv = text["num_attention_heads"] * text["head_dim"], text["num_key_value_heads"] * text["head_dim"]
        shapes = {"qkv": (2 * q + 2 * kv, h, 0), "o": (h, q, 0), "gate_up": (2 * inner, h, 1), "down": (h, inner, 0)}
        draw = lambda *shape: torch.randn(*shape, device=device, dtype=torch.bfloat16) * 0.05
        table = {}
        for rows in (8, 16, 32, 64, 128, 264, 512, 1024, 2048, 4096, 8192):
            for name, (n, k, epilogue) in shapes.items():
                weights, a = [draw(n, k) for _ in range(6)], draw(rows, k) * 20
                out = torch.empty(rows, n // 2 if epilogue else n, dtype=torch.bfloat16, device=device)
                def library(i):
                    z = torch.mm(a, weights[i].t())
                    return ops.swiglu(z) if epilogue else z
                entry = {"library": round(replayed(library, 6), 1)}
                if rows <= 16:
                    entry["streaming"] = round(replayed(lambda i: ops._gemv_stream(a, weights[i], out, epilogue), 6), 1)
                if rows >= 128:
                    entry["one_sm"] = round(replayed(lambda i: ops._gemm_tcgen05(a, weights[i], out, epilogue, pair=False), 6), 1)
                if rows >= 256:
                    entry["two_sm"] = round(replayed(lambda i: ops._gemm_tcgen05(a, weights[i], out, epilogue, pair=True), 6), 1)
                table[f"{name}_{rows}"] = entry
        ops.raise_on_error(device)
        return {"only": "products", "config": args.config, "unit": "us", "products": table}
    if args.only == "elementwise":
        # The prefill step's element-wise kernels alone, buffers fresh for every launch.
        from mlx_omnia_b200.parts.base import KVView
        device = engine.runtime.device
        tokens, h, d = args.prefill_tokens, text["hidden_size"], text["head_dim"]
        nq, nkv = text["num_attention_heads"], text["num_key_value_heads"]
        xs = [torch.randn(tokens, h, device=device) for _ in range(8)]
        branches = [torch.randn(tokens, h, device=device).bfloat16() for _ in range(8)]
        wb, wo = torch.rand(h, device=device) + 0.5, torch.rand(h, device=device) + 0.5
        residual = replayed(lambda i: ops.add_rmsnorm(xs[i], branches[i], wb, 1e-6, wo, 1e-6), 8)
        rows = [torch.randn(tokens, (2 * nq + 2 * nkv) * d, device=device).bfloat16() for _ in range(8)]
        pages = [torch.zeros(-(-tokens // 16), 2, nkv, 16, d, device=device, dtype=torch.bfloat16) for _ in range(8)]
        inv_freq = 1.0 / (1e6 ** (torch.arange(0, d, 2, device=device).float() / d))
        positions = torch.arange(tokens, device=device, dtype=torch.int32)
        slots = torch.arange(tokens, device=device, dtype=torch.int64)
        blocks = torch.arange(-(-tokens // 16), device=device, dtype=torch.int32).view(1, -1)
        rope = replayed(lambda i: ops.qk_norm_rope_store(rows[i], 0, 2 * nq * d, (2 * nq + nkv) * d, nq, nkv, d, 1e-6, inv_freq,
                                                         positions, KVView(pages[i], blocks, slots, 16, None)), 8)
        moved = {"add_rmsnorm": tokens * h * (4 + 2 + 4 + 2), "qk_norm_rope_store": tokens * (nq + 2 * nkv) * d * 2 * 2}
        ops.raise_on_error(device)
        return {"only": "elementwise", "config": args.config, "tokens": tokens,
                "add_rmsnorm": {"us": round(residual, 2), "frac": round(moved["add_rmsnorm"] / residual / 1e3 / measured["hbm_gbs"], 3)},
                "qk_norm_rope_store": {"us": round(rope, 2),
                                       "frac": round(moved["qk_norm_rope_store"] / rope / 1e3 / measured["hbm_gbs"], 3)}}
    if args.only == "sampling":  # temperature, top-k and top-p over the full vocabulary, one row a request
        rows = args.batch
        logits = torch.randn(rows, vocab, device=engine.runtime.device, dtype=torch.float32) * 2.0
        f32 = lambda v: torch.full((rows,), v, dtype=torch.float32, device=logits.device)
        top_k = torch.full((rows,), 50, dtype=torch.int32, device=logits.device)
        seeds = torch.arange(rows, dtype=torch.int64, device=logits.device)
        call = lambda: ops.sample(logits, f32(0.8), top_k, f32(0.95), f32(0.0), seeds, seeds)
        for _ in range(max(args.warmup, 1)):
            call()
        start, stop = events()
        start.record()
        for _ in range(args.steps):
            call()
        stop.record()
        torch.cuda.synchronize()
        return {"only": "sampling", "rows": rows, "vocab": vocab, "us": round(start.elapsed_time(stop) * 1e3 / args.steps, 2)}
    if args.only == "mixed":
        part = mixed(args.batch, args.portion, args.steps, max(args.warmup, 4))
        return {"only": "mixed", "decoders": args.batch, "portion": args.portion, "layers": layers,
                "ms": round(part["ms"], 3), "host_ms": round(part["wall_ms"], 3)}
    if args.only == "prefill":
        part = prefill(args.prefill_tokens, args.steps, args.warmup)
        return {"only": "prefill", "config": args.config, "layers": layers, "tokens": args.prefill_tokens,
                "ms": round(part["ms"], 3), "frac": round(part["frac"], 4)}
    with ClockSampler() as sampler:
        main = decode(args.batch, args.steps, args.warmup)
    clocks = sampler.summary()
    side_steps = max(8, min(args.steps, 32))
    points = {f"decode_b{b}": round(decode(b, side_steps, 3)["tokens_per_s"], 1) for b in (1, 64)}
    pre = prefill(PREFILL_TOKENS, 5, 3)
    for name, (decoders, portion) in {"mixed_b8_ctx4096_portion256": (8, 256), "mixed_portion128": (0, 128)}.items():
        # (Four untimed steps: the prompt's first portion has a shape of its own, the shape of the others
        # is captured at its third coming.)
        part = mixed(decoders, portion, 8 if decoders else 4, 4)  # (a lone prompt of 8 x 128 tokens keeps its table width)
        points[name + "_ms"] = round(part["ms"], 3)
        points[name + "_host_ms"] = round(part["wall_ms"], 3)
    points["prefill_8192_in_portions_of_512_ms"] = round(portions(8192, 512), 2)
    kernels = kernel_classes()
    ops.raise_on_error(engine.runtime.device)

    step_bytes = weight_bytes + args.batch * main["context"] * kv_per_token
    achieved = step_bytes / (main["ms"] / 1000.0) / 1e9
    h2d = 4 * (3 * args.batch + (args.batch + 1) + 2 * args.batch) + 8 * args.batch + \
        4 * args.batch * -(-main["context"] // 16)
    # What a replayed decode step really copies: the whole metadata buffer of its graph, whose block
    # tables are as wide as the graph's bucket, not as the requests' own.
    graphs = getattr(engine.runner, "graphs", None)
    bucket = 1 << max(args.batch - 1, 0).bit_length()
    copied = [c.host_tensor.numel() * 4 for c in graphs.captured.values() if c.layout.seqs == bucket] \
        if graphs is not None else []
    if copied:
        h2d = int(max(copied))
    return {
        "metric": "decode tok/s at batch 8 (configs[2], context 4096)", "value": round(main["tokens_per_s"], 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(main["ms"], 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded uniform-random token ids, random weights N(0, 0.02)",
        "config": {"model": "muse_glimmer configs[2]", "layers": layers, "layers_full": full_layers,
                   "hidden": text["hidden_size"], "heads": text["num_attention_heads"],
                   "kv_heads": text["num_key_value_heads"], "head_dim": text["head_dim"],
                   "intermediate": text["intermediate_size"], "vocab": vocab, "tied": True, "global_batch": args.batch,
                   "seq_len": args.context, "context_at_timed_steps": main["context"], "page_size": 16,
                   "params": params, "parallelism": "single-gpu", "l2": f"weights ({weight_bytes / 1e9:.1f} GB) exceed L2; no flush",
                   "peaks": peak_source},
        "clocks": clocks,
        "e2e": {"value": round(main["wall_tokens_per_s"], 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": 4 * args.batch},
        "gpu_launches": main["launches"] * args.steps,
        "prefill": {"value": round(pre["value"], 1), "tokens": pre["tokens"], "ms": round(pre["ms"], 3),
                    "frac": round(pre["frac"], 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": measured["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / measured["hbm_gbs"], 4)},
        "points": points,
        "kernels": kernels,
    }


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=4)
    parser.add_argument("--impl", choices=["ours", "reference"], default="ours")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--layers", type=int, default=0, help="run fewer layers than configs[2] has (named in config)")
    parser.add_argument("--timeline", action="store_true",
                        help="with --only decode|prefill and OMNIA_TIMELINE=1 in the environment: one step's "
                             "kernels with the time each takes in the stream, on stderr")
    parser.add_argument("--only", choices=["all", "decode", "prefill", "mixed", "portions", "sampling", "products", "elementwise"], default="all",
                        help="time one part only (small cases for profilers); prints a short record")
    parser.add_argument("--config", type=int, choices=sorted(CONFIGS), default=2,
                        help="with --only: the sizes of another benchmark configuration (3: 36 layers, hidden 4096, "
                             "32/8 heads, intermediate 12288, untied head, context 8192)")
    parser.add_argument("--context", type=int, default=0, help="tokens each request holds at the last timed step "
                                                               "(default: the configuration's own)")
    parser.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS)
    parser.add_argument("--pool-tokens", type=int, default=0, help="at least this many tokens of cache pool (default: what the run needs)")
    parser.add_argument("--portion", type=int, default=256,
                        help="--only mixed: tokens of a prompt that run beside --batch decoding requests")
    args = parser.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "gabfssilva/mlx-omnia needs Apple's MLX (Metal) and Python >= 3.13; its offline install "
                          "fails here (no hatchling build backend, no mlx wheel for Linux)"}))
        return 0
    if args.gpus != 1:
        print("bench.py: this engine runs on one GPU; --gpus must be 1")
        return 2
    if args.config != 2 and args.only == "all":
        print("bench.py: the full record is of configuration 2; give --only decode|prefill|mixed with --config")
        return 2
    args.context = args.context or CONFIGS[args.config][1]
    if args.only == "all":
        args.warmup = max(args.warmup, 3)
    print(json.dumps(run(args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
