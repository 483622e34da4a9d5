#!/usr/bin/env python3
"""Benchmark of the engine's decode step (and prefill) at Qwen2-7B layer sizes on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one decode step of a batch of 8 requests whose context ends at 4,096 tokens.
The timed region is K such steps on the device (captured graph: model step, argmax, advance of
positions; no host work), timed with CUDA events; ``value`` is decoded tokens per second.
``e2e`` is the same through ``LLMEngine.step()``: host token lists in, scheduler, pinned
host-to-device copy of the step's inputs, device-to-host read of the sampled tokens.
One line of JSON is printed; see the keys below. Weights are random (seeded), token ids
uniform random, and the cache pages of the device-timed decode runs are filled with random
values instead of being prefilled (the step's time does not depend on the values).
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

# Qwen2-7B layer sizes (the benchmark's named configuration, with random weights)
QWEN2_7B = dict(
    architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=28, hidden_size=3584,
    num_attention_heads=28, num_key_value_heads=4, head_dim=128, intermediate_size=18944, vocab_size=152064,
    rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False, use_sliding_window=False,
    max_position_embeddings=32768,
)
# The two larger shapes that the benchmark's other workloads name (random weights as well)
SHAPES = {
    "0.5b": ("Qwen2-0.5B", dict(QWEN2_7B, num_hidden_layers=24, hidden_size=896, num_attention_heads=14,
                                 num_key_value_heads=2, head_dim=64, intermediate_size=4864, vocab_size=151936,
                                 tie_word_embeddings=True)),
    "1.5b": ("Qwen2-1.5B", dict(QWEN2_7B, num_hidden_layers=28, hidden_size=1536, num_attention_heads=12,
                                 num_key_value_heads=2, head_dim=128, intermediate_size=8960, vocab_size=151936,
                                 tie_word_embeddings=True)),
    "7b": ("Qwen2-7B", QWEN2_7B),
    "14b": ("Qwen2.5-14B", dict(QWEN2_7B, num_hidden_layers=48, hidden_size=5120, num_attention_heads=40,
                                num_key_value_heads=8, intermediate_size=13824, rms_norm_eps=1e-5)),
    "32b": ("Qwen2.5-32B", dict(QWEN2_7B, num_hidden_layers=64, hidden_size=5120, num_attention_heads=40,
                                num_key_value_heads=8, intermediate_size=27648, rms_norm_eps=1e-5)),
}
CONTEXT = 4096
PAGE = 16
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def load_peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            data = json.loads(path.read_text())
            flat = {}

            def walk(obj):
                if isinstance(obj, dict):
                    for key, value in obj.items():
                        if isinstance(value, (int, float)) and key in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
                            flat.setdefault(key, float(value))
                        else:
                            walk(value)
                elif isinstance(obj, list):
                    for item in obj:
                        walk(item)

            walk(data)
            if "hbm_gbs" in flat and "bf16_tflops" in flat:
                flat["source"] = "measured"
                return flat
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self) -> None:
        self.samples: list[list[str]] = []
        self.process = None
        self.thread = None

    def start(self) -> None:
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.process = None
            return

        def reader():
            for line in self.process.stdout:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) == 6:
                    self.samples.append(parts)

        self.thread = threading.Thread(target=reader, daemon=True)
        self.thread.start()

    def mark(self) -> int:
        return len(self.samples)

    def stop(self) -> None:
        if self.process is not None:
            self.process.terminate()
            try:
                self.process.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.process.kill()

    def summary(self, begin: int = 0, end: int | None = None) -> dict:
        rows = self.samples[begin:end] or self.samples
        clocks = [int(r[0]) for r in rows if r[0].isdigit()]
        maxima = [int(r[1]) for r in rows if r[1].isdigit()]
        reasons = [name for i, name in enumerate(self.NAMES) if any(r[2 + i].lower().startswith("active") for r in rows)]
        return {
            "sm_mhz": int(statistics.median(clocks)) if clocks else None,
            "sm_max_mhz": max(maxima) if maxima else None,
            "reasons": reasons,
            "samples": len(rows),
        }


def build_runner(layers: int, max_seqs: int, context: int, seed: int = 0, shape: str = "7b", pages: int | None = None,
                 dtype=None):
    import torch

    from turboserve_b200.config import config_from_dict, lookup
    from turboserve_b200.engine.runner import ModelRunner, make_groups

    raw = shape if isinstance(shape, dict) else dict(SHAPES[shape][1], num_hidden_layers=layers)
    config = config_from_dict(raw)
    model = lookup(config.architecture).build_model(config, dtype or torch.bfloat16, "cuda")
    model.config = config
    model.init_random(seed)
    if pages is None:
        pages = max_seqs * (context // PAGE) + 64
    runner = ModelRunner(model, make_groups(model.cache_plan(), PAGE, pages), max_seqs)
    for cache in runner.storage.run_caches:
        if cache is not None and cache.k_pages is not None and cache.writes:
            cache.k_pages.normal_()
            cache.v_pages.normal_()
    return config, model, runner


def weight_bytes(model) -> int:
    """Bytes a decode step has to read of the weights: everything but the embedding table."""
    total = 0
    for p in model.named_params():
        if model.parts_list[p.owner] is model.embedding and not model.spec.tie_word_embeddings:
            continue  # a decode step reads a few rows of the table
        count = 1
        for s in p.spec.shape:
            count *= s
        total += count * (2 if p.spec.role == "matrix" else 4)
    return total


def decode_on_device(runner, batch: int, context_end: int, steps: int, warmup: int):
    """K decode steps replayed from one graph; returns (seconds, own kernel launches per step, mean context)."""
    import torch

    from turboserve_b200.engine.batch import RequestSlice, StaticBatch
    from turboserve_b200.ops import kernels

    width = context_end // PAGE
    start = context_end - (steps + warmup) - 2
    groups = runner.num_groups
    static = StaticBatch(batch, batch, [width] * groups, runner.device)
    generator = torch.Generator().manual_seed(1)
    ids = torch.randint(0, runner.model.vocab_size, (batch,), generator=generator).tolist()
    slices = [RequestSlice([ids[i]], start, [list(range(i * width, (i + 1) * width))] * groups, i, [0]) for i in range(batch)]
    static.load_decode(slices)
    tokens = torch.empty(batch, dtype=torch.int32, device=runner.device)

    def one_step():
        logits = runner.run(static.batch)
        kernels.argmax(logits, tokens, batch)
        static.batch.token_ids.copy_(tokens)
        static.batch.positions.add_(1)
        static.batch.context_lens.add_(1)

    with torch.inference_mode():
        one_step()
        torch.cuda.synchronize()
        before = kernels.launch_count()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            one_step()
        launches = kernels.launch_count() - before
        for _ in range(warmup):
            graph.replay()
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        for _ in range(steps):
            graph.replay()
        end.record()
        torch.cuda.synchronize()
    runner.check_status()
    mean_context = start + 2 + warmup + steps / 2
    return begin.elapsed_time(end) / 1000.0, launches, mean_context


def decode_end_to_end(runner, config, batch: int, context_end: int, steps: int, warmup: int):
    """The same decode steps through LLMEngine.step(): host tokens in, host tokens out."""
    import torch

    from turboserve_b200 import EngineConfig, LLMEngine, SamplingParams, SchedulerConfig

    # requests finish their prompts some steps apart (a prompt takes several steps under the token
    # budget, one request after the other); leave room so that none reaches the end of its
    # context, and none finishes, inside the timed region
    budget = 2048
    room = batch * -(-context_end // budget) + 8
    prompt_len = context_end - (steps + warmup) - 2 - room
    engine_config = EngineConfig(
        model="(injected)", dtype="bfloat16", max_model_len=context_end,
        scheduler=SchedulerConfig(max_num_seqs=batch, max_num_batched_tokens=budget, block_size=PAGE,
                                  num_blocks=runner.groups[0].num_pages))
    engine = LLMEngine(engine_config, runner=runner)
    generator = torch.Generator().manual_seed(2)
    sampling = SamplingParams(max_tokens=steps + warmup + room, temperature=0.0, ignore_eos=True)
    for i in range(batch):
        prompt = torch.randint(0, config.vocab_size, (prompt_len,), generator=generator).tolist()
        engine.add_request(f"bench-{i}", prompt, sampling)
    while any(seq.num_output_tokens == 0 for seq in engine.scheduler._running) or engine.scheduler.num_waiting:
        engine.step()  # prefill, untimed
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    h2d = runner._graphs[(next(b for b in runner._graph_buckets if b >= batch), 1)][1].nbytes if runner._graph_buckets else 0
    started = time.perf_counter()
    produced = 0
    for _ in range(steps):
        produced += sum(len(o.new_token_ids) for o in engine.step())
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - started
    if produced != batch * steps:
        raise RuntimeError(f"the end-to-end run decoded {produced} tokens in {steps} steps of {batch} requests")
    decode_end_to_end.overlapped = engine.stats()["num_overlapped_steps"]
    engine.close()
    return elapsed, produced, h2d, 4 * runner.token_buffer.numel()


def prefill_end_to_end(runner, config, tokens: int, repeats: int = 5):
    """A prompt of ``tokens`` tokens through ``LLMEngine.step()`` to its first token: host token ids in
    (scheduler, packing, pinned host-to-device copy), one step, the sampled id read back. Median and best, seconds."""
    import torch

    from turboserve_b200 import EngineConfig, LLMEngine, SamplingParams, SchedulerConfig

    engine_config = EngineConfig(
        model="(injected)", dtype="bfloat16", max_model_len=tokens + PAGE,
        scheduler=SchedulerConfig(max_num_seqs=1, max_num_batched_tokens=tokens, block_size=PAGE,
                                  num_blocks=runner.groups[0].num_pages))
    engine = LLMEngine(engine_config, runner=runner)
    generator = torch.Generator().manual_seed(5)
    sampling = SamplingParams(max_tokens=1, temperature=0.0, ignore_eos=True)
    times = []
    for i in range(repeats + 2):
        prompt = torch.randint(0, config.vocab_size, (tokens,), generator=generator).tolist()
        torch.cuda.synchronize()
        started = time.perf_counter()
        engine.add_request(f"prefill-{i}", prompt, sampling)
        outputs = engine.step()
        torch.cuda.synchronize()
        elapsed = time.perf_counter() - started
        if len(outputs) != 1 or not outputs[0].finished:
            raise RuntimeError("the prompt did not run in one step")
        if i >= 2:
            times.append(elapsed)
    engine.close()
    return statistics.median(times), min(times)


def prefill_run(runner, config, tokens: int, repeats: int = 7, warmup: int = 3):
    import torch

    from turboserve_b200.engine.batch import RequestSlice

    generator = torch.Generator().manual_seed(3)
    ids = torch.randint(0, config.vocab_size, (tokens,), generator=generator).tolist()
    table = list(range(-(-tokens // PAGE)))
    batch = runner.build_batch([RequestSlice(ids, 0, [table] * runner.num_groups, 0, [tokens - 1])])
    times = []
    for i in range(warmup + repeats):
        if runner.plan.state_bytes_per_slot():
            runner.reset_state_slot(0)  # a prompt starts from an empty state every time
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        runner.run(batch)
        end.record()
        torch.cuda.synchronize()
        if i >= warmup:
            times.append(begin.elapsed_time(end) / 1000.0)
    runner.check_status()
    return statistics.median(times), min(times)


def prefill_flops(config, tokens: int) -> float:
    h, d = config.hidden_size, config.head_dim
    qkv = (config.num_attention_heads + 2 * config.num_key_value_heads) * d
    per_layer = 2 * tokens * h * (qkv + config.num_attention_heads * d + 3 * config.intermediate_size)
    attention = 2 * tokens * tokens * config.num_attention_heads * d  # QK^T and PV over the causal half
    return config.num_hidden_layers * (per_layer + attention) + 2 * h * config.vocab_size


def one_step(kind: str, layers: int, batch: int, shape: str = "7b", float32: bool = False) -> int:
    """Three eager steps (no graph) of one kind, so that a profiler sees every kernel once per step."""
    import torch

    from turboserve_b200.engine.batch import RequestSlice, StaticBatch

    config, model, runner = build_runner(layers, max(batch, 1), CONTEXT, shape=shape, dtype=torch.float32 if float32 else None)
    width = CONTEXT // PAGE
    if kind == "decode":
        static = StaticBatch(batch, batch, [width], runner.device)
        static.load_decode([RequestSlice([5], CONTEXT - 1, [list(range(i * width, (i + 1) * width))], i, [0])
                            for i in range(batch)])
        batch_obj = static.batch
    else:
        ids = torch.randint(0, config.vocab_size, (2048,), generator=torch.Generator().manual_seed(3)).tolist()
        batch_obj = runner.build_batch([RequestSlice(ids, 0, [list(range(width))], 0, [2047])])
    for _ in range(3):
        runner.run(batch_obj)
    torch.cuda.synchronize()
    runner.check_status()
    print(f"ran three {kind} steps of {layers} layers")
    return 0


def scenario(name: str, shape: str, layers: int, generate: int) -> int:
    """A serving workload through ``LLMEngine``: prompts in, tokens out, the scheduler in between.

    ``mixed``: 32 prompts of 64 to 4,096 tokens (uniform), a token budget of 512 a step (prompts are
    cut into portions beside the decode tokens of the others), contexts up to 8,192, room for all.
    ``preempt``: 16 requests whose contexts end at 16,384 tokens, in a pool that holds their prompts
    and half of what they generate, so that some are preempted and computed again.
    Both generate ``generate`` tokens a request, greedily; one line of JSON with the throughput
    (prompt and generated tokens together) and what the scheduler did.
    """
    import random

    import torch

    from turboserve_b200 import EngineConfig, LLMEngine, SamplingParams, SchedulerConfig

    rng = random.Random(4)
    if name == "mixed":
        batch, context, budget = 32, 8192, 512
        lengths = [rng.randint(64, 4096) for _ in range(batch)]
        pages = sum(-(-(n + generate) // PAGE) for n in lengths) + 64
    else:
        batch, context, budget = 16, 16384, 2048
        lengths = [context - generate] * batch
        pages = batch * -(-(context - generate) // PAGE) + batch * (generate // 2) // PAGE
    config, model, runner = build_runner(layers, batch, context, shape=shape, pages=pages)
    engine_config = EngineConfig(
        model="(injected)", dtype="bfloat16", max_model_len=context,
        scheduler=SchedulerConfig(max_num_seqs=batch, max_num_batched_tokens=budget, block_size=PAGE, num_blocks=pages))
    engine = LLMEngine(engine_config, runner=runner)
    sampling = SamplingParams(max_tokens=generate, temperature=0.0, ignore_eos=True)
    prompts = [[rng.randrange(config.vocab_size) for _ in range(n)] for n in lengths]
    engine.generate([p[:64] for p in prompts[:2]], SamplingParams(max_tokens=4, temperature=0.0, ignore_eos=True))  # warm-up
    before = engine.stats()
    torch.cuda.synchronize()
    started = time.perf_counter()
    outputs = engine.generate(prompts, sampling)
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - started
    after = engine.stats()
    generated = sum(len(o.token_ids) for o in outputs)
    if generated != batch * generate:
        raise RuntimeError(f"{generated} tokens came back, {batch * generate} were asked for")
    engine.scheduler.check_invariants()
    line = {
        "scenario": name, "metric": "prompt + generated tokens/s through LLMEngine.generate",
        "value": round((sum(lengths) + generated) / elapsed, 1), "unit": "tokens/s", "seconds": round(elapsed, 3),
        "prompt_tokens": sum(lengths), "generated_tokens": generated,
        "generated_tokens_per_s": round(generated / elapsed, 1),
        "steps": after["num_steps"] - before["num_steps"],
        "preemptions": after["num_preemptions"] - before["num_preemptions"],
        "recomputed_prompt_tokens": after["num_prefill_tokens"] - before["num_prefill_tokens"] - sum(lengths),
        "config": {"model": f"{SHAPES[shape][0]} shape (random weights)", "layers": layers,
                   "layers_of_model": SHAPES[shape][1]["num_hidden_layers"], "hidden": config.hidden_size,
                   "heads": config.num_attention_heads, "kv_heads": config.num_key_value_heads,
                   "intermediate": config.intermediate_size, "requests": batch, "max_context": context,
                   "token_budget": budget, "pages": pages, "page_size": PAGE, "params": model.num_parameters()},
        "dtype": "bf16", "impl": "ours",
    }
    engine.close()
    print(json.dumps(line))
    return 0


def reference_arm(args, shape_name: str, shape_raw: dict) -> int:
    """The same workload through the unmodified reference engine under ``baseline/_ref``.

    Nothing of this repository's engine is imported on this path. Where the reference cannot be
    imported or run, one line says why and the exit code is still 0.
    """
    sys.path.insert(0, str(ROOT / "baseline"))
    import reference_arm as arm

    try:
        line = arm.run(shape_raw, shape_name, args.layers, args.batch, args.context, PAGE, args.steps, args.warmup,
                       args.skip_points, ClockSampler(), load_peaks(), prefill_flops)
    except arm.UnavailableError as error:
        print(json.dumps({"impl": "reference", "unavailable": str(error)}))
        return 0
    except Exception as error:  # noqa: BLE001 - the reference's own failure is the reason, in its words
        reason = " ".join(f"the reference failed while running: {type(error).__name__}: {error}".split())
        print(json.dumps({"impl": "reference", "unavailable": reason[:500]}))
        return 0
    print(json.dumps(line))
    return 0


def fp32_products(layers: int = 28, steps: int = 8) -> int:
    """The true 32-bit path (FFMA, no tensor cores): its matrix product at the 7B layer's shapes, every
    weight from HBM (copies of a weight taken in turn, 600 MB of them), and one decode step of the
    whole model in float32 at batch 8, context 4,096. One JSON line."""
    import torch

    from turboserve_b200.engine.batch import RequestSlice, StaticBatch
    from turboserve_b200.ops.linear import linear

    shapes = {"qkv": (3584, 4608), "o": (3584, 3584), "gate_up": (3584, 37888), "down": (18944, 3584)}
    line = {"what": "float32 FFMA product (gemm_simt.cu), Qwen2-7B layer shapes", "unit": "TFLOP/s (rows 2048) and GB/s of weights (rows 8)"}
    for name, (k, n) in shapes.items():
        copies = max(2, -(-600_000_000 // (4 * k * n)))
        ws = [torch.randn(n, k, device="cuda") for _ in range(copies)]
        for rows in (2048, 8):
            x = torch.randn(rows, k, device="cuda")
            out = torch.empty(rows, n, device="cuda")
            for w in ws[:2]:
                linear(x, w, out)
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            for w in ws:
                linear(x, w, out)
            end.record()
            torch.cuda.synchronize()
            seconds = begin.elapsed_time(end) / 1e3 / copies
            line[f"{name}_rows{rows}_ms"] = round(seconds * 1e3, 3)
            line[f"{name}_rows{rows}"] = round(2 * rows * k * n / seconds / 1e12, 2) if rows > 8 else round(4 * k * n / seconds / 1e9, 1)
        del ws
    # one decode step of the whole model in float32, launched kernel by kernel (20 ms of device work hide the host)
    batch, context = 8, CONTEXT
    config, model, runner = build_runner(layers, batch, context, dtype=torch.float32)
    width = context // PAGE
    static = StaticBatch(batch, batch, [width], runner.device)
    slices = [RequestSlice([7 + i], context - steps - 4, [list(range(i * width, (i + 1) * width))], i, [0]) for i in range(batch)]
    static.load_decode(slices)
    times = []
    for step in range(steps + 2):
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        runner.run(static.batch)
        end.record()
        torch.cuda.synchronize()
        static.batch.positions.add_(1)
        static.batch.context_lens.add_(1)
        if step >= 2:
            times.append(begin.elapsed_time(end))
    runner.check_status()
    ms = statistics.median(times)
    weights = sum(4 * _count(p.spec.shape) for p in model.named_params() if model.parts_list[p.owner] is not model.embedding)
    cache = batch * (context - 4) * layers * 2 * config.num_key_value_heads * config.head_dim * 4
    line["decode_step"] = {"layers": layers, "layers_of_model": SHAPES["7b"][1]["num_hidden_layers"], "batch": batch, "context": context,
                           "ms": round(ms, 2), "gb_per_s": round((weights + cache) / ms / 1e6, 1),
                           "frac_of_hbm": round((weights + cache) / ms / 1e6 / load_peaks()["hbm_gbs"], 3)}
    print(json.dumps(line))
    return 0


def _count(shape) -> int:
    total = 1
    for s in shape:
        total *= s
    return total


def decode_attention_sweep() -> int:
    """The TMA-fed decode attention kernel alone at a few (requests, keys, parts): µs and TB/s of keys and
    values, CUDA events around a graph of "write 256 MB, run the kernel" with the write alone subtracted."""
    import torch

    from turboserve_b200.ops import attention_bf16 as fa

    nh, nkv, d, page = 28, 4, 128, PAGE
    flush = torch.empty(256 * 1024 * 1024 // 4, device="cuda")
    rows = []

    def timed(graph) -> float:
        graph.replay()
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        for _ in range(20):
            graph.replay()
        end.record()
        torch.cuda.synchronize()
        return begin.elapsed_time(end) / 20 * 1e3

    empty = torch.cuda.CUDAGraph()
    flush.zero_()
    torch.cuda.synchronize()
    with torch.cuda.graph(empty):
        flush.zero_()
    base = timed(empty)
    for batch, ctx, parts in [(8, 4096, 8), (8, 4096, 9), (64, 512, 1), (32, 1024, 1), (32, 1024, 2), (8, 16384, 8),
                              (64, 4096, 1), (1, 4096, 8), (1, 4096, 32)]:
        width = ctx // page + 1
        k_pages = torch.randn(batch * width, page, nkv, d, device="cuda").to(torch.bfloat16)
        v_pages = torch.randn(batch * width, page, nkv, d, device="cuda").to(torch.bfloat16)
        table = torch.arange(batch * width, dtype=torch.int32, device="cuda").view(batch, width)
        q = torch.randn(batch, nh * d, device="cuda").to(torch.bfloat16)
        out = torch.empty_like(q)
        seq = torch.arange(batch, dtype=torch.int32, device="cuda")
        pos = torch.full((batch,), ctx - 1, dtype=torch.int32, device="cuda")
        scratch = torch.empty(max(4, fa.decode_scratch_floats(batch, nh, parts, d)), device="cuda")

        def run():
            fa.flash_decode_tma(q, out, k_pages, v_pages, table, seq, pos, batch, nh, nkv, d, None, d ** -0.5, parts, scratch)

        run()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            flush.zero_()
            run()
        us = timed(graph) - base
        rows.append({"requests": batch, "keys": ctx, "parts": parts, "us": round(us, 1),
                     "tb_per_s": round(batch * ctx * nkv * d * 4 / us / 1e6, 2)})
        del k_pages, v_pages
    print(json.dumps({"what": "flash_decode_tma alone, 28 heads on 4 kv heads of 128, pages of 16", "rows": rows}))
    return 0


def sampling_sweep(context: int = 4096, steps: int = 40) -> int:
    """Decode steps of 8 requests through LLMEngine.step() under a few sets of sampling options: ms a step each."""
    import torch

    from turboserve_b200 import EngineConfig, LLMEngine, SamplingParams, SchedulerConfig

    config, model, runner = build_runner(SHAPES["7b"][1]["num_hidden_layers"], 8, context)
    runner.enable_graphs(8, context, 2048)
    line = {"what": "ms a decode step through LLMEngine.step(), 7B sizes, batch 8", "context": context, "steps": steps}
    for name, options in [("greedy", dict(temperature=0.0)), ("temperature", dict(temperature=0.8, seed=1)),
                          ("top_p", dict(temperature=0.8, top_p=0.9, seed=1)),
                          ("top_k_top_p", dict(temperature=0.8, top_p=0.9, top_k=50, seed=1)),
                          ("penalty", dict(temperature=0.8, top_p=0.9, top_k=50, seed=1, repetition_penalty=1.2)),
                          ("greedy_penalty", dict(temperature=0.0, repetition_penalty=1.2)),
                          ("greedy_logprobs", dict(temperature=0.0, logprobs=True)),
                          ("top_p_penalty_logprobs", dict(temperature=0.8, top_p=0.9, seed=1, repetition_penalty=1.2, logprobs=True)),
                          ("greedy_again", dict(temperature=0.0))]:
        engine = LLMEngine(EngineConfig(model="(injected)", dtype="bfloat16", max_model_len=context, scheduler=SchedulerConfig(
            max_num_seqs=8, max_num_batched_tokens=2048, block_size=PAGE, num_blocks=runner.groups[0].num_pages)), runner=runner)
        generator = torch.Generator().manual_seed(2)
        sampling = SamplingParams(max_tokens=steps + 40, ignore_eos=True, **options)
        for i in range(8):
            engine.add_request(f"r{i}", torch.randint(0, config.vocab_size, (context - steps - 100,), generator=generator).tolist(), sampling)
        while any(seq.num_output_tokens == 0 for seq in engine.scheduler._running) or engine.scheduler.num_waiting:
            engine.step()
        for _ in range(5):
            engine.step()
        torch.cuda.synchronize()
        started = time.perf_counter()
        produced = 0
        for _ in range(steps):
            produced += sum(len(o.new_token_ids) for o in engine.step())
        torch.cuda.synchronize()
        line[name] = round((time.perf_counter() - started) / steps * 1e3, 3)
        if produced != 8 * steps:
            raise RuntimeError(f"{name}: {produced} tokens in {steps} steps")
        engine.close()
    print(json.dumps(line))
    return 0


# ---------------------------------------------------------------------------------------------
# --design baporax: the hybrid design beside the Qwen2 decoder at equal size
# ---------------------------------------------------------------------------------------------

DESIGN_SIZES = {"1k": (1024, 8), "2k": (2048, 12), "4k": (4096, 8)}
DESIGN_WINDOW = 1024
DESIGN_VOCAB = 32000


def baporax_raw(width: int, layers: int) -> dict:
    """Baporax at the sizes of a real model's layers: attention and Mamba-2 layers in turn (a, m, m, a, ...),
    heads of 2 x 64 keys and 128 values, four query heads to a key head, a window of 1,024; Mamba-2
    with an inner width of twice the model's, heads of 64, a state of 128; a feed-forward of 4 x width."""
    heads = max(4, width // 128)
    attention = {"type": "attention", "mlp": {"kind": "dense", "ff": 4 * width},
                 "mixer": dict(heads=heads, kv_heads=heads // 4, dim=64, vdim=128, conv=4, diff=0.5, scale=0.125,
                               mask={"size": DESIGN_WINDOW})}
    mamba = {"type": "mamba2", "mlp": {"kind": "dense", "ff": 4 * width},
             "mixer": dict(heads=2 * width // 64, vdim=64, state=128, groups=1, norm_groups=1, conv=4)}
    pattern = [attention, mamba, mamba, attention]
    return {"architecture": "Baporax", "vocab": DESIGN_VOCAB, "width": width, "logit_scale": 1.0, "norm": {"eps": 1e-6},
            "initializer_range": 0.02, "layers": [pattern[i % 4] for i in range(layers)]}


def qwen2_equal_raw(width: int, layers: int) -> dict:
    """The Qwen2 decoder with as many parameters a layer: the same width and attention widths (heads of 128, four
    to a key head, the same window), and a gated feed-forward of 3.25 x width."""
    heads = max(4, width // 128)
    return dict(QWEN2_7B, num_hidden_layers=layers, hidden_size=width, num_attention_heads=heads,
                num_key_value_heads=heads // 4, head_dim=128, intermediate_size=width * 13 // 4, vocab_size=DESIGN_VOCAB,
                tie_word_embeddings=True, use_sliding_window=True, sliding_window=DESIGN_WINDOW, max_window_layers=0,
                max_position_embeddings=8192)


def filezen_raw(width: int, layers: int) -> dict:
    """Filezen at the sizes of a real model's layers: retention and latent attention in turn (r, l, r, l', ...; l' reads
    the rows the latent layer before it caches). Latent attention: heads of 128 plain and 64 rotated query elements and
    128 values over a latent of 512, a window of 1,024. Retention: heads of 128 keys and 256 values (as wide as the
    model together). The first layer's feed-forward is dense (4 x width); the others are mixtures of 8 experts of
    ``width`` features of which 2 are chosen among the 2 best of 4 groups, beside a shared expert of width / 2."""
    heads = max(4, width // 128)
    r_heads = max(2, width // 256)
    rot = {"base": 10000.0, "dims": 64, "scaling": {"factor": 4.0, "original": 2048, "fast": 16.0, "slow": 2.0}}
    latent = dict(heads=heads, dim=128, rot_dim=64, vdim=128, kv_rank=512, scale=192 ** -0.5, mask={"size": DESIGN_WINDOW}, rot=rot)
    retention = dict(heads=r_heads, dim=128, vdim=256, decay=[1.0 - 2.0 ** (-5 - i * 3 / r_heads) for i in range(r_heads)],
                     rot={"base": 1000000.0, "dims": 128})
    moe = {"kind": "moe", "expert": {"ff": width}, "router": {"experts": 8, "top": 2, "groups": {"count": 4, "keep": 2}},
           "shared": {"ff": width // 2}}
    out = []
    for i in range(layers):
        mlp = {"kind": "dense", "ff": 4 * width} if i == 0 else moe
        if i % 2 == 0:
            out.append({"type": "retention", "mixer": retention, "mlp": mlp})
        elif i % 4 == 1:
            out.append({"type": "latent_attention", "mixer": latent, "mlp": mlp})
        else:
            out.append({"type": "latent_attention", "mixer": dict(latent, kv_from=i - 2), "mlp": mlp})
    return {"architecture": "Filezen", "vocab": DESIGN_VOCAB, "width": width, "embedding": {"scale": 1.0}, "residual_mult": 0.7,
            "norm": {"eps": 1e-6}, "initializer_range": 0.02, "layers": out}


def begovik_raw(width: int, layers: int) -> dict:
    """Begovik at the sizes of a real model's layers: side-by-side layers, the selective scan and wkv time mixing in turn
    (p, m, w, m, ...). Side by side: attention with heads of 128 keys and values, four query heads to a key head, 64
    rotated elements, scores capped at 50, a sink and no window, beside lightning attention with heads of 128 keys and
    values (as wide as the model together). Selective scan: an inner width of twice the model's, a state of 16, step sizes
    of rank width / 16, four taps. wkv: heads of 64, a decay pair of rank 64. Every layer has a clamped feed-forward of
    4 x width."""
    heads = max(4, width // 128)
    left = dict(heads=heads, kv_heads=heads // 4, dim=128, vdim=128, scale=128 ** -0.5, softcap=50.0, rot={"base": 10000.0, "dims": 64})
    r_heads = max(2, width // 128)
    right = dict(heads=r_heads, dim=128, vdim=128, decay=[1.0 - 2.0 ** (-5 - i * 3 / r_heads) for i in range(r_heads)])
    mlp = {"kind": "dense", "ff": 4 * width, "limit": 7.0}
    side = {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": mlp}
    scan = {"type": "mamba1", "mixer": dict(inner=2 * width, state=16, dt_rank=width // 16, conv=4), "mlp": mlp}
    wkv = {"type": "wkv", "mixer": dict(heads=width // 64, dim=64, decay_rank=64), "mlp": mlp}
    pattern = [side, scan, wkv, scan]
    return {"architecture": "Begovik", "vocab": DESIGN_VOCAB, "width": width, "embedding": {"scale": 1.0}, "residual_mult": 0.5,
            "norm": {"eps": 1e-6}, "initializer_range": 0.02, "layers": [pattern[i % 4] for i in range(layers)]}


def lorozen_raw(width: int, layers: int) -> dict:
    """Lorozen at the sizes of a real model's layers, ``layers`` layer runs in all: latent attention, wkv time mixing and
    two layers of attention in turn (l, w, a, a, l, w, ...), of which the second and third are a stretch that runs twice
    (so the model has ``layers - 2`` layers of weights). Latent attention: heads of 128 plain and 64 rotated query
    elements and 128 values over a latent of 512, a window of 1,024, a gate per head. Attention: heads of 128 keys and
    values, four query heads to a key head, 64 rotated elements with stretched long waves, biases, a learned sink, a
    window of 1,024. wkv: heads of 64, a decay pair of rank 64. The first layer's feed-forward is dense (4 x width); the
    others are mixtures of 8 experts of ``width`` features of which 2 are chosen by sigmoid scores, the weight on the
    expert's input, beside a shared expert of width / 2. The logits are capped at 50."""
    heads = max(4, width // 128)
    latent = dict(heads=heads, dim=128, rot_dim=64, vdim=128, kv_rank=512, scale=192 ** -0.5, mask={"size": DESIGN_WINDOW},
                  rot={"base": 10000.0, "dims": 64})
    attention = dict(heads=heads, kv_heads=heads // 4, dim=128, vdim=128, scale=128 ** -0.5, mask={"size": DESIGN_WINDOW},
                     rot={"base": 500000.0, "dims": 64, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}})
    wkv = dict(heads=width // 64, dim=64, decay_rank=64)
    moe = {"kind": "moe", "expert": {"ff": width}, "router": {"experts": 8, "top": 2}, "shared": {"ff": width // 2}}
    pattern = [("latent_attention", latent), ("wkv", wkv), ("attention", attention), ("attention", attention)]
    out = []
    for i in range(layers - 2):
        kind, mixer = pattern[i % 4]
        out.append({"type": kind, "mixer": mixer, "mlp": {"kind": "dense", "ff": 4 * width} if i == 0 else moe})
    return {"architecture": "Lorozen", "vocab": DESIGN_VOCAB, "width": width, "norm": {"eps": 1e-6}, "logit_softcap": 50.0,
            "loop": {"start": 1, "stop": 3, "times": 2}, "initializer_range": 0.02, "layers": out}


class OpTimer:
    """CUDA events around every kernel entry point and matrix product a step calls, summed by name."""

    def __init__(self) -> None:
        self.records: list[tuple[str, object, object]] = []
        self._undo: list[tuple[object, str, object]] = []

    def _wrap(self, owner, attribute: str, name: str) -> None:
        import torch

        original = getattr(owner, attribute)

        def timed(*args, **kwargs):
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            result = original(*args, **kwargs)
            end.record()
            self.records.append((name, begin, end))
            return result

        setattr(owner, attribute, timed)
        self._undo.append((owner, attribute, original))

    def __enter__(self) -> "OpTimer":
        from turboserve_b200.ops import kernels
        from turboserve_b200.parts import (attention, diff_attention, latent_attention, mamba1, mamba2, mlp, moe, retention,
                                           sink_attention, vocabulary, wkv)

        for name in ("embedding", "add_rmsnorm", "stream_norm", "act_mul", "activation", "rope_cache_write", "causal_conv",
                     "diff_attention", "diff_attention_mma", "ssd_scan", "gated_group_norm", "scale_rows", "norm_add",
                     "latent_prepare", "head_linear", "latent_attention", "latent_gather", "latent_softmax", "retention_scan",
                     "head_norm_gate", "head_norm_rope_write", "paged_attention_capped", "paged_attention_capped_mma", "norm_pair_mix",
                     "shift_mix", "selective_scan", "chosen_decay_scan", "part_norm_gate", "norm_add_norm", "softcap_rows", "moe_route", "moe_pair_gate_up", "moe_pair_down", "moe_expert_rows", "moe_sort", "moe_gather", "moe_combine"):
            if hasattr(kernels, name):
                self._wrap(kernels, name, name)
        for module in (attention, diff_attention, mamba2, mlp, vocabulary, latent_attention, retention, sink_attention, wkv, mamba1):
            self._wrap(module, "linear", "linear")
        self._wrap(moe, "linear", "expert_linear")
        self._wrap(latent_attention, "matrix_product", "latent_products")
        self._wrap(mlp, "gated_linear", "gated_linear")
        self._wrap(attention, "paged_attention", "paged_attention")
        return self

    def __exit__(self, *exc) -> None:
        for owner, attribute, original in reversed(self._undo):
            setattr(owner, attribute, original)

    def totals(self) -> dict[str, float]:
        """Microseconds per name over everything recorded (after a synchronize)."""
        out: dict[str, float] = {}
        for name, begin, end in self.records:
            out[name] = out.get(name, 0.0) + begin.elapsed_time(end) * 1e3
        return out


def design_step_ops(runner, batch_obj, repeats: int = 3) -> dict[str, float]:
    """Microseconds by operation of one eager step (the median of ``repeats`` runs)."""
    import torch

    runs = []
    for _ in range(repeats + 1):
        if runner.plan.state_bytes_per_slot() and batch_obj.max_query_len > 1:
            runner.reset_state_slot(0)
        with OpTimer() as timer:
            runner.run(batch_obj)
            torch.cuda.synchronize()
        runs.append(timer.totals())
    runs = runs[1:]
    return {name: round(statistics.median(r.get(name, 0.0) for r in runs), 1) for name in runs[0]}


def visible_pairs(tokens: int, window: int | None) -> int:
    """How many (query, key) pairs a prompt of ``tokens`` positions has under a causal mask and a window."""
    return sum(min(i + 1, window) if window else i + 1 for i in range(tokens))


def design_bench(size: str, steps: int, warmup: int, tokens: int = 2048, context: int = 2048, design: str = "baporax",
                 alone: bool = False) -> int:
    """Prefill and decode throughput of a design (Baporax, or Filezen beside Baporax) at real layer sizes beside Qwen2
    at equal width and depth, and where each model's step spends its time, operation by operation, with the mixers'
    kernels against their rooflines."""
    import torch

    from turboserve_b200.engine.batch import RequestSlice, StaticBatch

    width, layers = DESIGN_SIZES[size]
    peaks = load_peaks()
    of = "of measured" if peaks["source"] == "measured" else "of fallback"
    hbm, tensor = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    titles = {"filezen": "Filezen beside Baporax and Qwen2", "begovik": "Begovik beside Baporax and Qwen2", "baporax": "Baporax beside Qwen2",
              "lorozen": "Lorozen beside Filezen, Begovik and Qwen2"}
    out = {"design": titles[design] + " at equal size",
           "width": width, "layers": layers, "prompt_tokens": tokens,
           "decode_context": context, "window": DESIGN_WINDOW, "dtype": "bf16", "peaks": of, "models": {}}
    heads = max(4, width // 128)
    models = [("baporax", baporax_raw(width, layers)), ("qwen2", qwen2_equal_raw(width, layers))]
    if design == "filezen":
        models.insert(0, ("filezen", filezen_raw(width, layers)))
    if design == "begovik":
        models.insert(0, ("begovik", begovik_raw(width, layers)))
    if design == "lorozen":  # beside the models whose mixers and feed-forwards are nearest to its own
        models = [("lorozen", lorozen_raw(width, layers)), ("filezen", filezen_raw(width, layers)),
                  ("begovik", begovik_raw(width, layers)), ("qwen2", qwen2_equal_raw(width, layers))]
    if alone:
        models = [m for m in models if m[0] == design]
    for name, raw in models:
        config, model, runner = build_runner(layers, 64, context, shape=raw)
        entry = {"params": model.num_parameters()}
        t, best = prefill_run(runner, config, tokens)
        entry["prefill_tokens_per_s"] = round(tokens / t, 1)
        entry["prefill_ms"] = round(t * 1e3, 3)
        table = list(range(-(-tokens // PAGE)))
        generator = torch.Generator().manual_seed(3)
        ids = torch.randint(0, config.vocab_size, (tokens,), generator=generator).tolist()
        prompt = runner.build_batch([RequestSlice(ids, 0, [table] * runner.num_groups, 0, [tokens - 1])])
        entry["prefill_ops_us"] = design_step_ops(runner, prompt)
        pages = context // PAGE
        for batch in (8, 64):
            static = StaticBatch(batch, batch, [pages] * runner.num_groups, runner.device)
            static.load_decode([RequestSlice([5], context - 1, [list(range(i * pages, (i + 1) * pages))] * runner.num_groups, i, [0])
                                for i in range(batch)])
            entry[f"decode_b{batch}_ops_us"] = design_step_ops(runner, static.batch)
        runner.enable_graphs(64, context, tokens)
        for batch in (8, 64):
            seconds, launches, _ = decode_on_device(runner, batch, context, steps, warmup)
            entry[f"decode_b{batch}_tokens_per_s"] = round(batch * steps / seconds, 1)
            entry[f"decode_b{batch}_ms_per_step"] = round(seconds / steps * 1e3, 4)
            entry[f"decode_b{batch}_launches_per_step"] = launches
        # the mixers' kernels against their rooflines (time of all layers of the kind in one step)
        kernels_out = {}
        seen = min(context, DESIGN_WINDOW)
        if name == "lorozen":
            runs = [raw["layers"][run.layer] for run in config.to_model_spec().order]
            entry["layer_runs"] = len(runs)
            attention_runs = sum(1 for layer in runs if layer["type"] == "attention")
            latent_runs = sum(1 for layer in runs if layer["type"] == "latent_attention")
            wkv_runs = len(runs) - attention_runs - latent_runs
            moe_runs = sum(1 for layer in runs if layer["mlp"]["kind"] == "moe")
            w_heads, row = width // 64, 512 + 64
            prefill = entry["prefill_ops_us"]
            flops = attention_runs * visible_pairs(tokens, DESIGN_WINDOW) * heads * 4 * 128
            us = prefill.get("paged_attention_capped_mma", 0.0) + prefill.get("paged_attention_capped", 0.0)
            kernels_out["attention_prefill"] = {"us": us, "tflops": round(flops / us / 1e6, 1), "frac_tensor": round(flops / (us * 1e-6) / tensor, 4)}
            flops = latent_runs * visible_pairs(tokens, DESIGN_WINDOW) * heads * (2 * row + 2 * 512)
            us = sum(prefill.get(k, 0.0) for k in ("latent_attention", "latent_products", "latent_softmax", "latent_gather"))
            kernels_out["latent_prefill"] = {"us": us, "tflops": round(flops / us / 1e6, 1), "frac_tensor": round(flops / (us * 1e-6) / tensor, 4)}
            scan_flops = wkv_runs * tokens * w_heads * 64 * 64 * 6
            us = prefill.get("chosen_decay_scan", 0.0)
            kernels_out["wkv_prefill"] = {"us": us, "fp32_tflops": round(scan_flops / us / 1e6, 2)}
            norm_bytes = 2 * len(runs) * tokens * width * (4 + 4 + 2 + 2)  # residual read and written, an update read, a row written
            us = prefill.get("norm_add_norm", 0.0) + prefill.get("add_rmsnorm", 0.0)
            kernels_out["norms_prefill"] = {"us": us, "gbs": round(norm_bytes / us / 1e3, 1), "frac_hbm": round(norm_bytes / (us * 1e-6) / hbm, 4)}
            entry["active_params_per_token"] = model.num_parameters() - sum(
                1 for layer in raw["layers"] if layer["mlp"]["kind"] == "moe") * 6 * 3 * width * width
            for batch in (8, 64):
                ops = entry[f"decode_b{batch}_ops_us"]
                bytes_read = attention_runs * batch * seen * (heads // 4) * 256 * 2
                us = ops.get("paged_attention_capped", 0.0) + ops.get("paged_attention_capped_mma", 0.0)
                kernels_out[f"attention_decode_b{batch}"] = {"us": us, "gbs": round(bytes_read / us / 1e3, 1), "frac_hbm": round(bytes_read / (us * 1e-6) / hbm, 4)}
                bytes_read = latent_runs * batch * seen * row * 2
                us = ops.get("latent_attention", 0.0)
                kernels_out[f"latent_decode_b{batch}"] = {"us": us, "gbs": round(bytes_read / us / 1e3, 1), "frac_hbm": round(bytes_read / (us * 1e-6) / hbm, 4)}
                state_bytes = wkv_runs * batch * w_heads * 64 * 64 * 4 * 2
                us = ops.get("chosen_decay_scan", 0.0)
                kernels_out[f"wkv_decode_b{batch}"] = {"us": us, "gbs": round(state_bytes / us / 1e3, 1), "frac_hbm": round(state_bytes / (us * 1e-6) / hbm, 4)}
                expert_bytes = moe_runs * min(batch * 2, 8) * 3 * width * width * 2
                us = sum(ops.get(k, 0.0) for k in ("moe_pair_gate_up", "moe_pair_down", "moe_expert_rows"))
                kernels_out[f"experts_decode_b{batch}"] = {"us": us, "gbs": round(expert_bytes / us / 1e3, 1), "frac_hbm": round(expert_bytes / (us * 1e-6) / hbm, 4)}
        elif name == "begovik":
            # attention without a window: a prompt's rows see everything before them, a decoded token its whole context
            side_layers = sum(1 for layer in raw["layers"] if layer["type"] == "parallel")
            scan_layers = sum(1 for layer in raw["layers"] if layer["type"] == "mamba1")
            wkv_layers = layers - side_layers - scan_layers
            r_heads, w_heads, inner, n_state = max(2, width // 128), width // 64, 2 * width, 16
            prefill = entry["prefill_ops_us"]
            flops = side_layers * visible_pairs(tokens, None) * heads * 4 * 128
            us = prefill.get("paged_attention_capped_mma", 0.0) + prefill.get("paged_attention_capped", 0.0)
            kernels_out["attention_prefill"] = {"us": us, "tflops": round(flops / us / 1e6, 1), "frac_tensor": round(flops / (us * 1e-6) / tensor, 4)}
            scan_flops = side_layers * tokens * r_heads * 128 * 128 * 4
            us = prefill.get("retention_scan", 0.0)
            kernels_out["lightning_prefill"] = {"us": us, "fp32_tflops": round(scan_flops / us / 1e6, 2)}
            scan_flops = wkv_layers * tokens * w_heads * 64 * 64 * 6
            us = prefill.get("chosen_decay_scan", 0.0)
            kernels_out["wkv_prefill"] = {"us": us, "fp32_tflops": round(scan_flops / us / 1e6, 2)}
            scan_flops = scan_layers * tokens * inner * n_state * 6
            scan_bytes = scan_layers * tokens * (inner * (2 + 4 + 2 + 2) + 2 * n_state * 2)
            us = prefill.get("selective_scan", 0.0)
            kernels_out["scan_prefill"] = {"us": us, "fp32_tflops": round(scan_flops / us / 1e6, 2), "frac_hbm": round(scan_bytes / (us * 1e-6) / hbm, 4)}
            for batch in (8, 64):
                ops = entry[f"decode_b{batch}_ops_us"]
                bytes_read = side_layers * batch * context * (heads // 4) * 256 * 2
                us = ops.get("paged_attention_capped", 0.0) + ops.get("paged_attention_capped_mma", 0.0)
                kernels_out[f"attention_decode_b{batch}"] = {"us": us, "gbs": round(bytes_read / us / 1e3, 1), "frac_hbm": round(bytes_read / (us * 1e-6) / hbm, 4)}
                for label, key, state_bytes in (
                        ("lightning", "retention_scan", side_layers * batch * r_heads * 128 * 128 * 4 * 2),
                        ("wkv", "chosen_decay_scan", wkv_layers * batch * w_heads * 64 * 64 * 4 * 2),
                        ("scan", "selective_scan", scan_layers * batch * inner * n_state * 4 * 2)):
                    us = ops.get(key, 0.0)
                    kernels_out[f"{label}_decode_b{batch}"] = {"us": us, "gbs": round(state_bytes / us / 1e3, 1), "frac_hbm": round(state_bytes / (us * 1e-6) / hbm, 4)}
        elif name == "filezen":
            latent_layers = sum(1 for layer in raw["layers"] if layer["type"] == "latent_attention")
            owners = sum(1 for layer in raw["layers"] if layer["type"] == "latent_attention" and "kv_from" not in layer["mixer"])
            retention_layers = layers - latent_layers
            moe_layers = sum(1 for layer in raw["layers"] if layer["mlp"]["kind"] == "moe")
            r_heads = max(2, width // 256)
            prefill, row = entry["prefill_ops_us"], 512 + 64
            flops = latent_layers * visible_pairs(tokens, DESIGN_WINDOW) * heads * (2 * row + 2 * 512)
            us = sum(prefill.get(k, 0.0) for k in ("latent_attention", "latent_products", "latent_softmax", "latent_gather"))
            kernels_out["attention_prefill"] = {"us": us, "tflops": round(flops / us / 1e6, 1), "frac_tensor": round(flops / (us * 1e-6) / tensor, 4)}
            scan_flops = retention_layers * tokens * r_heads * 128 * 256 * 4
            us = prefill.get("retention_scan", 0.0)
            kernels_out["scan_prefill"] = {"us": us, "fp32_tflops": round(scan_flops / us / 1e6, 2)}
            entry["active_params_per_token"] = model.num_parameters() - moe_layers * 6 * 3 * width * width
            for batch in (8, 64):
                ops = entry[f"decode_b{batch}_ops_us"]
                bytes_read = latent_layers * batch * seen * row * 2
                us = ops.get("latent_attention", 0.0)
                kernels_out[f"attention_decode_b{batch}"] = {"us": us, "gbs": round(bytes_read / us / 1e3, 1), "frac_hbm": round(bytes_read / (us * 1e-6) / hbm, 4)}
                state_bytes = retention_layers * batch * r_heads * 128 * 256 * 4 * 2
                us = ops.get("retention_scan", 0.0)
                kernels_out[f"scan_decode_b{batch}"] = {"us": us, "gbs": round(state_bytes / us / 1e3, 1), "frac_hbm": round(state_bytes / (us * 1e-6) / hbm, 4)}
                expert_bytes = moe_layers * min(batch * 2, 8) * 3 * width * width * 2
                us = sum(ops.get(k, 0.0) for k in ("moe_pair_gate_up", "moe_pair_down", "moe_expert_rows"))
                kernels_out[f"experts_decode_b{batch}"] = {"us": us, "gbs": round(expert_bytes / us / 1e3, 1), "frac_hbm": round(expert_bytes / (us * 1e-6) / hbm, 4)}
            del owners
        elif name == "baporax":
            attention_layers = sum(1 for layer in raw["layers"] if layer["type"] == "attention")
            mamba_layers = layers - attention_layers
            flops = attention_layers * visible_pairs(tokens, DESIGN_WINDOW) * heads * (4 * 64 + 4 * 128)
            us = entry["prefill_ops_us"].get("diff_attention_mma", 0.0)
            kernels_out["attention_prefill"] = {"us": us, "tflops": round(flops / us / 1e6, 1), "frac_tensor": round(flops / (us * 1e-6) / tensor, 4)}
            for batch in (8, 64):
                bytes_read = attention_layers * batch * seen * (heads // 4) * (128 + 128) * 2
                us = entry[f"decode_b{batch}_ops_us"].get("diff_attention", 0.0)
                kernels_out[f"attention_decode_b{batch}"] = {"us": us, "gbs": round(bytes_read / us / 1e3, 1), "frac_hbm": round(bytes_read / (us * 1e-6) / hbm, 4)}
            m_heads, inner = 2 * width // 64, 2 * width
            scan_flops = mamba_layers * tokens * m_heads * 64 * 128 * 4
            scan_bytes = mamba_layers * tokens * ((inner + 256 + m_heads) * 2 + inner * 4)
            us = entry["prefill_ops_us"].get("ssd_scan", 0.0)
            kernels_out["scan_prefill"] = {"us": us, "fp32_tflops": round(scan_flops / us / 1e6, 2), "frac_hbm": round(scan_bytes / (us * 1e-6) / hbm, 4)}
            for batch in (8, 64):
                state_bytes = mamba_layers * batch * m_heads * 64 * 128 * 4 * 2
                us = entry[f"decode_b{batch}_ops_us"].get("ssd_scan", 0.0)
                kernels_out[f"scan_decode_b{batch}"] = {"us": us, "gbs": round(state_bytes / us / 1e3, 1), "frac_hbm": round(state_bytes / (us * 1e-6) / hbm, 4)}
        else:
            flops = layers * visible_pairs(tokens, DESIGN_WINDOW) * heads * 4 * 128
            us = entry["prefill_ops_us"].get("paged_attention", 0.0)
            kernels_out["attention_prefill"] = {"us": us, "tflops": round(flops / us / 1e6, 1), "frac_tensor": round(flops / (us * 1e-6) / tensor, 4)}
            for batch in (8, 64):
                bytes_read = layers * batch * seen * (heads // 4) * 256 * 2
                us = entry[f"decode_b{batch}_ops_us"].get("paged_attention", 0.0)
                kernels_out[f"attention_decode_b{batch}"] = {"us": us, "gbs": round(bytes_read / us / 1e3, 1), "frac_hbm": round(bytes_read / (us * 1e-6) / hbm, 4)}
        entry["kernels"] = kernels_out
        out["models"][name] = entry
        del runner, model
        torch.cuda.empty_cache()
    print(json.dumps(out))
    return 0


def main() -> int:
    parser = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", choices=["ours", "reference"], default="ours")
    parser.add_argument("--shape", choices=sorted(SHAPES), default="7b",
                        help="layer sizes (the headline is 7b; the others are for the larger workloads)")
    parser.add_argument("--layers", type=int, default=None,
                        help="run fewer layers than the model has (both numbers are reported)")
    parser.add_argument("--scenario", choices=["mixed", "preempt"], default=None,
                        help="run a serving workload through LLMEngine.generate instead (see scenario())")
    parser.add_argument("--generate", type=int, default=128, help="tokens a request generates in a scenario")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--context", type=int, default=CONTEXT,
                        help="context length of the decode runs (the headline is 4096; others are for sweeps)")
    parser.add_argument("--skip-points", action="store_true", help="skip the batch-1 and batch-64 points and the prefill")
    parser.add_argument("--decode-attention-sweep", action="store_true", help="time the decode attention kernel alone at a few sizes and exit")
    parser.add_argument("--sampling-sweep", action="store_true", help="time decode steps through LLMEngine under a few sets of sampling options and exit")
    parser.add_argument("--fp32-products", action="store_true", help="time the float32 path's matrix product at the 7B shapes and exit")
    parser.add_argument("--float32", action="store_true", help="with --one-step: the true 32-bit path")
    parser.add_argument("--design", choices=["baporax", "filezen", "begovik", "lorozen"], default=None,
                        help="measure that design at real layer sizes beside Qwen2 at equal size and exit (see design_bench())")
    parser.add_argument("--design-size", choices=sorted(DESIGN_SIZES), default="2k", help="width and depth for --design")
    parser.add_argument("--design-alone", action="store_true", help="with --design: leave the models beside it out (profiling runs)")
    parser.add_argument("--one-step", choices=["decode", "prefill"], default=None,
                        help="run three eager steps of that kind and exit (a small case for a profiler)")
    args = parser.parse_args()

    if args.gpus != 1:
        print(f"bench.py measures one GPU: this engine runs on a single B200, --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    shape_name, shape_raw = SHAPES[args.shape]
    if args.layers is None:
        args.layers = shape_raw["num_hidden_layers"]
    if args.impl == "reference":
        return reference_arm(args, shape_name, shape_raw)

    import torch

    from turboserve_b200.ops import kernels

    if args.design:
        return design_bench(args.design_size, args.steps, args.warmup, design=args.design, alone=args.design_alone)
    if args.fp32_products:
        return fp32_products()
    if args.decode_attention_sweep:
        return decode_attention_sweep()
    if args.sampling_sweep:
        return sampling_sweep()
    if args.one_step:
        return one_step(args.one_step, args.layers, args.batch, args.shape, args.float32)
    if args.scenario:
        return scenario(args.scenario, args.shape, args.layers, args.generate)
    peaks = load_peaks()
    of = "of measured" if peaks["source"] == "measured" else "of fallback"
    context = args.context
    if context < 256 or context % PAGE:
        print(f"--context must be a multiple of {PAGE} and at least 256")
        return 2
    largest = 64 if not args.skip_points else max(args.batch, 1)
    config, model, runner = build_runner(args.layers, largest, context, shape=args.shape)
    runner.enable_graphs(largest, context, 2048)
    kv_per_token = config.kv_bytes_per_token(2)
    w_bytes = weight_bytes(model)

    sampler = ClockSampler()
    sampler.start()
    time.sleep(0.3)
    mark0 = sampler.mark()
    seconds, launches_per_step, mean_ctx = decode_on_device(runner, args.batch, context, args.steps, args.warmup)
    # the same steps through the entry point, straight after, so that both numbers see the same GPU state
    e2e_seconds, produced, h2d, d2h = decode_end_to_end(runner, config, args.batch, context, args.steps, args.warmup)
    mark1 = sampler.mark()
    value = args.batch * args.steps / seconds
    step_bytes = w_bytes + args.batch * mean_ctx * kv_per_token
    achieved = step_bytes / (seconds / args.steps) / 1e9

    points = {}
    prefill = None
    if not args.skip_points:
        for b in (1, 64):
            s, _, _ = decode_on_device(runner, b, context, args.steps, args.warmup)
            points[f"decode_b{b}"] = round(b * args.steps / s, 1)
            s, n, _, _ = decode_end_to_end(runner, config, b, context, args.steps, args.warmup)
            points[f"e2e_decode_b{b}"] = round(n / s, 1)
        t, best = prefill_run(runner, config, 2048)
        flops = prefill_flops(config, 2048)
        # value, ms and frac are the median of the repeats; best_ms is the fastest of them
        prefill = {"value": round(2048 / t, 1), "tokens": 2048, "ms": round(t * 1e3, 3), "best_ms": round(best * 1e3, 3),
                   "frac": round(flops / t / (peaks["bf16_tflops"] * 1e12), 4), "peak": of}
        if "bf16_tflops_sustained" in peaks:  # the step is long enough to run under the power cap
            prefill["frac_of_sustained"] = round(flops / t / (peaks["bf16_tflops_sustained"] * 1e12), 4)
        e2e_t, e2e_best = prefill_end_to_end(runner, config, 2048)
        prefill["e2e_value"] = round(2048 / e2e_t, 1)
        prefill["e2e_ms"] = round(e2e_t * 1e3, 3)
        prefill["e2e_best_ms"] = round(e2e_best * 1e3, 3)
    # what a batch pays that is the first of its size to be lopsided (decode attention cut finer:
    # another graph): a warm-up step, a synchronisation and the capture. Even batches of every
    # size were captured when the engine was built.
    torch.cuda.synchronize()
    started = time.perf_counter()
    runner._capture(next(b for b in runner._graph_buckets if b >= args.batch), 16)
    torch.cuda.synchronize()
    first_lopsided_ms = (time.perf_counter() - started) * 1e3

    sampler.stop()
    clocks = sampler.summary(mark0, mark1)

    line = {
        "metric": f"decode tokens/s, {shape_name} shape, batch {args.batch}, context {context}",
        "value": round(value, 1),
        "unit": "tokens/s",
        "n_gpus": 1,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": round(seconds / args.steps * 1e3, 4),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic: random weights (seed 0), uniform random token ids, cache pages of the device-timed runs filled with random values",
        "config": {
            "model": f"{shape_name} shape (random weights)", "layers": args.layers, "layers_of_model": shape_raw["num_hidden_layers"],
            "hidden": config.hidden_size, "heads": config.num_attention_heads, "kv_heads": config.num_key_value_heads,
            "head_dim": config.head_dim, "intermediate": config.intermediate_size, "vocab": config.vocab_size,
            "global_batch": args.batch, "seq_len": context, "page_size": PAGE, "parallelism": "single GPU",
            "l2": "inputs larger than L2 (every step reads all weights)", "params": model.num_parameters(),
        },
        "e2e": {"value": round(produced / e2e_seconds, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": round(e2e_seconds / args.steps * 1e3, 4),
                "steps_launched_ahead": getattr(decode_end_to_end, "overlapped", 0)},
        "gpu_launches": launches_per_step * args.steps,
        "clocks": clocks,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4), "peak_source": of,
                     "bytes_per_step": int(step_bytes)},
        "points": points,
        "graphs": {"captured_at_start": runner.num_graph_captures - 1, "first_lopsided_step_extra_ms": round(first_lopsided_ms, 2)},
        "impl": "ours",
    }
    if prefill is not None:
        line["prefill"] = prefill
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
