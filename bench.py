#!/usr/bin/env python3
"""Decode and prefill throughput of metallix_b200 on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W]          the headline line
    python bench.py --shape 8b                                    continuous batching of 64 requests
    python bench.py --shape 32b                                   prefill and decode at 8,192-token contexts
    python bench.py --workload decode|prefill|gemm|attention|pick ...   small fixed workloads for profilers

Default workload: a Qwen3-0.6B-shaped model (28 layers,
hidden 1024, 16 query and 8 key/value heads of 128, SwiGLU 3072, vocabulary
151,936, tied head) with random weights in bfloat16, 8 requests that each hold
a 2,048-token prompt in a cache laid out for 4,096-token contexts (pages of
16), decoding one token per request per step. A "step" is one decode step.

One JSON line is printed:
  value       decoded tokens per second over K device-timed steps (CUDA events
              around K back-to-back steps with given token ids), the median of
              ``--repeats`` such runs of K steps;
  e2e         the same through the Python entry point (scheduler, sampler): host
              token ids in, picked token ids out, every step;
  prefill     one 2,048-token prompt in one step: tokens per second and the
              fraction of the measured bf16 matrix peak its FLOPs reach, for the
              step replayed as a captured graph (``ms``) and for the first
              occurrence of the shape, launched kernel by kernel (``eager_ms``);
  roofline    bytes a decode step must read (every weight once and the cache of
              the live requests) over its time, against the measured copy
              bandwidth;
  points      decode tokens per second at batch 1 and 64.
More than one GPU is outside this engine: --gpus N>1 prints one line and exits 2.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def _qwen3(layers, hidden, heads, kv_heads, inter, tied):
    return dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_act="silu",
                num_hidden_layers=layers, hidden_size=hidden, num_attention_heads=heads,
                num_key_value_heads=kv_heads, head_dim=128, intermediate_size=inter, vocab_size=151936,
                rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=tied,
                max_position_embeddings=40960)


# The three measured shapes, as the config.json of each.
SHAPES = {"0.6b": ("Qwen3-0.6B-shaped", _qwen3(28, 1024, 16, 8, 3072, True)),
          "8b": ("Qwen3-8B-shaped", _qwen3(36, 4096, 32, 8, 12288, False)),
          "32b": ("Qwen3-32B-shaped", _qwen3(64, 5120, 64, 8, 25600, False))}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
REFERENCE_UNAVAILABLE = ("arclabs561/metallix is a Rust workspace on MLX/Metal for Apple Silicon with "
                         "no setup.py or pyproject.toml: pip reports the directory is not installable, "
                         "and neither cargo nor Metal exists on this box")


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as handle:
            raw = json.load(handle)
        out = {k: float(raw[k]) for k in ("hbm_gbs", "bf16_tflops") if k in raw}
        out["bf16_tflops_sustained"] = float(raw.get("bf16_tflops_sustained", out.get("bf16_tflops", 0)))
        if "hbm_gbs" in out and "bf16_tflops" in out:
            return out, "measured"
    except (OSError, ValueError, KeyError, TypeError):
        pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons while a timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.process = None

    def __enter__(self):
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=self.file, stderr=subprocess.DEVNULL)
            time.sleep(0.25)   # the sampler's own start-up stays outside the timed region
        except OSError:
            self.process = None
        return self

    def __exit__(self, *exc):
        if self.process is not None:
            self.process.terminate()
            try:
                self.process.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.process.kill()

    def summary(self):
        self.file.flush()
        self.file.seek(0)
        clocks, peak, reasons = [], 0, set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.file:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                clocks.append(int(float(parts[0])))
                peak = max(peak, int(float(parts[1])))
            except ValueError:
                continue
            for name, value in zip(names, parts[2:6]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        self.file.close()
        os.unlink(self.file.name)
        return {"sm_mhz": int(statistics.median(clocks)) if clocks else None, "sm_max_mhz": peak or None,
                "reasons": sorted(reasons), "samples": len(clocks)}


def prefill_flops(config, tokens, context=0):
    """Multiply-adds times two of one prompt portion of ``tokens`` tokens
    behind ``context`` cached ones: every linear layer on every token, causal
    attention (q k^T and p v over the pairs a causal mask leaves), and the head
    on the one wanted row."""
    h, inter = config.hidden_size, config.intermediate_size
    q = config.num_attention_heads * config.head_dim
    kv = config.num_key_value_heads * config.head_dim
    linear = 2 * tokens * (h * (q + 2 * kv) + q * h + 3 * h * inter)
    pairs = tokens * context + tokens * (tokens + 1) // 2
    attention = 2 * 2 * config.num_attention_heads * config.head_dim * pairs
    return config.num_hidden_layers * (linear + attention) + 2 * h * config.vocab_size


def timed(torch, device, run, count):
    """Milliseconds of ``count`` calls of ``run(index)`` on the device (CUDA events)."""
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(device)
    start.record()
    for index in range(count):
        run(index)
    end.record()
    torch.cuda.synchronize(device)
    return start.elapsed_time(end)


def flat_config(name, config, args, extra):
    out = {"model": name, "layers": config.num_hidden_layers, "layers_of_config": extra.pop("layers_of_config"),
           "hidden": config.hidden_size, "q_heads": config.num_attention_heads,
           "kv_heads": config.num_key_value_heads, "head_dim": config.head_dim,
           "intermediate": config.intermediate_size, "vocab": config.vocab_size,
           "tied_head": bool(config.tie_word_embeddings), "page_tokens": 16, "parallelism": "single GPU",
           "gemm": args.gemm}
    out.update(extra)
    return out


# --------------------------------------------------------------------- headline
def headline(args):
    import numpy as np
    import torch
    from metallix_b200 import ops, parse_config
    from metallix_b200.engine import Engine, StepEntry
    from metallix_b200.engine.generate import Generator
    from metallix_b200.sampling import SamplingParams

    warmup, steps, repeats = max(args.warmup, 3), max(args.steps, 1), max(args.repeats, 1)
    peak, peak_source = peaks()
    name, raw = SHAPES["0.6b"]
    layers_of_config = raw["num_hidden_layers"]
    config = parse_config(dict(raw, num_hidden_layers=args.layers or layers_of_config))
    batches = [args.batch] + ([] if args.no_points else [b for b in (1, 64) if b != args.batch])
    span = args.prompt_len + warmup + repeats * steps + 64   # positions one request may reach here
    if span > args.context:
        raise SystemExit(f"prompt {args.prompt_len} + {warmup} + {repeats} x {steps} steps exceeds the context "
                         f"{args.context}: use fewer --steps or --repeats")
    pages = max(batches) * (-(-span // 16)) + 64
    engine = Engine.from_random(config, seed=0, dtype="bfloat16", page_tokens=16, num_pages=pages,
                                max_requests=max(batches) + 2, max_context=args.context,
                                gemm_backend=args.gemm)
    device = engine.device
    rng = np.random.default_rng(0)
    vocab = config.vocab_size

    # ---------------------------------------------------------------- prefill
    def one_prefill(tokens):
        engine.step([StepEntry("prefill", tokens, [len(tokens) - 1])])
        engine.release("prefill")

    prompt = rng.integers(0, vocab, size=args.prompt_len).tolist()
    # What the first occurrence of a shape costs: every kernel launched from
    # Python (kernels and libraries loaded by the warm-up runs).
    engine.replay_general_steps = False
    for _ in range(3):
        one_prefill(prompt)
    eager_ms = statistics.median(timed(torch, device, lambda _: one_prefill(prompt), 1) for _ in range(5))
    engine.replay_general_steps = True
    for _ in range(3):   # seen, captured, replayed
        one_prefill(prompt)
    prefill_ms = statistics.median(timed(torch, device, lambda _: one_prefill(prompt), 1) for _ in range(5))
    flops = prefill_flops(config, args.prompt_len)
    prefill = {"value": args.prompt_len / prefill_ms * 1e3, "tokens": args.prompt_len, "ms": prefill_ms,
               "frac": flops / (prefill_ms * 1e-3) / (peak["bf16_tflops"] * 1e12), "tflop": flops / 1e12,
               "eager_ms": eager_ms, "eager_value": args.prompt_len / eager_ms * 1e3,
               "eager_frac": flops / (eager_ms * 1e-3) / (peak["bf16_tflops"] * 1e12)}

    # ----------------------------------------------------------------- decode
    def fill(batch):
        engine.release_all()
        names = [f"r{i}" for i in range(batch)]
        for first in range(0, batch, 4):
            engine.step([StepEntry(name, rng.integers(0, vocab, size=args.prompt_len).tolist(), [])
                         for name in names[first:first + 4]])
        return names

    def decode(batch, with_clocks=False):
        """Median over the repeats of K timed steps each: (ms per K steps,
        launches in K steps, clocks, mean context of that repeat)."""
        names = fill(batch)
        feed = rng.integers(0, vocab, size=(warmup + repeats * steps, batch))

        def one(index):
            engine.step([StepEntry(name, [int(feed[index, i])], [0]) for i, name in enumerate(names)])

        for index in range(warmup):
            one(index)
        runs = []

        def all_repeats():
            for repeat in range(repeats):
                first = warmup + repeat * steps
                before = ops.launch_count()
                elapsed = timed(torch, device, lambda index: one(first + index), steps)
                runs.append((elapsed, ops.launch_count() - before,
                             args.prompt_len + first + (steps + 1) / 2))

        clocks = None
        if with_clocks:
            with ClockSampler() as sampler:
                all_repeats()
            clocks = sampler.summary()
        else:
            all_repeats()
        engine.check()
        runs.sort()
        elapsed, launches, mean_context = runs[len(runs) // 2]
        return elapsed, launches, clocks, mean_context

    elapsed, launches, clocks, mean_context = decode(args.batch, with_clocks=True)
    ms_per_step = elapsed / steps
    value = args.batch * steps / elapsed * 1e3
    step_bytes = engine.model.weight_bytes() + args.batch * mean_context * engine.cache.bytes_per_token()
    achieved = step_bytes / (ms_per_step * 1e-3) / 1e9
    points = {}
    for batch in batches[1:]:
        other, _, _, _ = decode(batch)
        points[f"decode_b{batch}"] = batch * steps / other * 1e3

    # The same decode step in an engine that allows the configuration's whole
    # 40,960 positions (what `mxb gen` serves a model folder with): graphs are
    # laid out for the contexts that are live, not for the limit.
    if not args.no_points:
        engine.release_all()
        wide = Engine.from_random(config, seed=0, dtype="bfloat16", page_tokens=16, num_pages=args.batch * (-(-span // 16)) + 64,
                                  max_requests=args.batch + 2, max_context=config.max_position_embeddings,
                                  gemm_backend=args.gemm)
        narrow, engine = engine, wide
        other, _, _, _ = decode(args.batch)
        points[f"decode_b{args.batch}_context_limit_{config.max_position_embeddings}"] = args.batch * steps / other * 1e3
        engine = narrow
        del wide

    # ------------------------------------------- end to end, the entry point
    engine.release_all()
    generator = Generator(engine, max_num_seqs=args.batch, max_tokens_per_step=4 * args.prompt_len)
    total_new = warmup + repeats * steps + 16   # nobody finishes inside the timed steps
    for i in range(args.batch):
        generator.add(rng.integers(0, vocab, size=args.prompt_len).tolist(), total_new,
                      SamplingParams(), eos_ids=(), ignore_eos=True)
    while generator.scheduler.num_waiting() or any(
            len(generator.scheduler.request(r).output) == 0 for r in generator.scheduler.running()):
        generator.step()   # prompts
    for _ in range(warmup):
        generator.step()
    e2e_ms = statistics.median(timed(torch, device, lambda _: generator.step(), steps) for _ in range(repeats))
    e2e_value = args.batch * steps / e2e_ms * 1e3
    h2d = engine.graphs.h2d_bytes if engine.graphs is not None else 0
    generator.run()

    line = {
        "metric": "decode tok/s @ batch 8 (points: batch 1/64; prefill tok/s @ 2048 tokens; % of roofline)",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights N(0, 0.02), uniform-random token ids",
        "impl": "ours", "repeats": repeats,
        "config": flat_config(name, config, args, {
            "layers_of_config": layers_of_config, "global_batch": args.batch, "seq_len": args.context,
            "prompt_len": args.prompt_len, "cuda_graphs": engine.graphs is not None,
            "l2": "inputs larger than L2: every step reads all weights and the live cache",
            "peaks": peak_source, "timing": f"median of {repeats} runs of K steps"}),
        "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": e2e_ms / steps,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * args.batch + 4},
        "gpu_launches": launches,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / peak["hbm_gbs"], "bytes_per_step": step_bytes, "of": peak_source},
        "points": points,
        "clocks": clocks,
    }
    print(json.dumps(line))
    return 0


# ---------------------------------------------------- 8B: continuous batching
def continuous_batching(args):
    """Continuous batching at the 8B layer sizes: 64 requests with uniform-random prompt lengths
    128..2,048 and output lengths 64..512 through the scheduler (continuous
    batching, pages of 16, contexts up to 4,096), as the reference's batched
    decode throughput test and engine loop do
    (crates/models/qwen/src/forward/tests/paged_batch.rs:409-452,
    crates/app/cli/src/engine_loop.rs:618-677)."""
    import numpy as np
    import torch
    from metallix_b200 import ops, parse_config
    from metallix_b200.engine import Engine
    from metallix_b200.engine.generate import Generator
    from metallix_b200.sampling import SamplingParams

    peak, peak_source = peaks()
    name, raw = SHAPES["8b"]
    layers_of_config = raw["num_hidden_layers"]
    config = parse_config(dict(raw, num_hidden_layers=args.layers or layers_of_config))
    rng = np.random.default_rng(4)
    requests = args.requests
    prompts = [int(n) for n in rng.integers(128, 2049, size=requests)]
    outputs = [int(n) for n in rng.integers(64, 513, size=requests)]
    started = time.perf_counter()
    engine = Engine.from_random(config, seed=0, dtype="bfloat16", page_tokens=16, max_requests=requests + 2,
                                max_context=4096, gemm_backend=args.gemm, pool_fraction=args.pool_fraction)
    load_s = time.perf_counter() - started
    device = engine.device
    vocab = config.vocab_size
    bytes_per_token = engine.cache.bytes_per_token()
    weight_bytes = engine.model.weight_bytes()

    def run_once(clocked):
        generator = Generator(engine, max_num_seqs=requests, max_tokens_per_step=args.max_tokens_per_step,
                              prefill_chunk=args.prefill_chunk)
        ids = [generator.add(rng.integers(0, vocab, size=n).tolist(), out, SamplingParams(), eos_ids=(),
                             ignore_eos=True) for n, out in zip(prompts, outputs)]
        step_bytes, decode_steps, live_sum, context_sum = 0.0, 0, 0, 0
        before = ops.launch_count()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize(device)
        wall = time.perf_counter()
        start.record()
        while not generator.idle():
            generator.step()
            running = generator.scheduler.running()
            held = sum(engine.manager.computed(r) for r in running)
            step_bytes += weight_bytes + held * bytes_per_token
            live_sum += len(running)
            context_sum += held
            decode_steps += 1
        end.record()
        torch.cuda.synchronize(device)
        engine.check()
        results = [generator.result(r) for r in ids]
        assert all(not r.failed and len(r.generated_ids) == out for r, out in zip(results, outputs))
        elapsed_ms = start.elapsed_time(end)
        return {"ms": elapsed_ms, "wall_s": time.perf_counter() - wall, "steps": generator.stats.steps,
                "generated": sum(outputs), "prompt_tokens": sum(prompts),
                "preemptions": generator.stats.preemptions, "bytes": step_bytes,
                "mean_live": live_sum / max(decode_steps, 1),
                "mean_context": context_sum / max(live_sum, 1),
                "ahead_kept": generator.stats.ahead_kept, "launches": ops.launch_count() - before}

    run_once(False)    # warm-up: kernels load, graphs of the common shapes are captured
    with ClockSampler() as sampler:
        runs = [run_once(True) for _ in range(max(args.repeats, 1))]
    clocks = sampler.summary()
    runs.sort(key=lambda r: r["ms"])
    run = runs[len(runs) // 2]
    seconds = run["ms"] * 1e-3
    achieved = run["bytes"] / seconds / 1e9
    line = {
        "metric": "generated tok/s, continuous batching of 64 requests (prompts U[128,2048], outputs U[64,512])",
        "value": run["generated"] / seconds, "unit": "tokens/s", "n_gpus": 1, "steps": run["steps"],
        "warmup": 1, "ms_per_step": run["ms"] / run["steps"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights N(0, 0.02), uniform-random token ids and lengths (seeded)",
        "impl": "ours", "repeats": len(runs),
        "config": flat_config(name, config, args, {
            "layers_of_config": layers_of_config, "global_batch": requests, "seq_len": 4096,
            "pool_pages": engine.cache.groups[0].num_pages, "max_tokens_per_step": args.max_tokens_per_step,
            "prefill_chunk": args.prefill_chunk, "peaks": peak_source,
            "timing": "host tokens in and out through Generator; CUDA events around the whole run"}),
        "e2e": {"value": run["generated"] / run["wall_s"], "unit": "tokens/s",
                "total_tok_s": (run["generated"] + run["prompt_tokens"]) / run["wall_s"]},
        "prompt_tok_s": run["prompt_tokens"] / seconds, "total_tok_s": (run["generated"] + run["prompt_tokens"]) / seconds,
        "generated": run["generated"], "prompt_tokens": run["prompt_tokens"], "preemptions": run["preemptions"],
        "mean_live_requests": run["mean_live"], "mean_context": run["mean_context"],
        "steps_launched_ahead": run["ahead_kept"], "gpu_launches": run["launches"], "load_s": load_s,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / peak["hbm_gbs"], "of": peak_source,
                     "bytes": "per step: every weight once and the cache the running requests hold after it"},
        "clocks": clocks,
    }
    print(json.dumps(line))
    return 0


# ------------------------------------------- 32B: prefill and long-context decode
def large_model(args):
    """The 32B layer sizes: prefill of a 2,048-token prompt, then decode at
    batch 1, 8 and 32 with 8,192-token contexts. Weights (65.5 GB) and the
    cache of 32 such requests (68.7 GB) together come close to the device's
    memory: the pool is sized from what is free once the weights are resident."""
    import numpy as np
    import torch
    from metallix_b200 import ops, parse_config
    from metallix_b200.engine import Engine, StepEntry

    warmup, steps, repeats = max(args.warmup, 3), max(args.steps, 1), max(args.repeats, 1)
    peak, peak_source = peaks()
    name, raw = SHAPES["32b"]
    layers_of_config = raw["num_hidden_layers"]
    config = parse_config(dict(raw, num_hidden_layers=args.layers or layers_of_config))
    context = args.context_32b
    batches = [int(b) for b in args.batches.split(",")]
    span = context + len(batches) * (warmup + repeats * steps) + 16   # the first request decodes in every batch size
    started = time.perf_counter()
    engine = Engine.from_random(config, seed=0, dtype="bfloat16", page_tokens=16, max_requests=max(batches) + 2,
                                max_context=-(-span // 256) * 256, gemm_backend=args.gemm,
                                pool_fraction=args.pool_fraction)
    load_s = time.perf_counter() - started
    device = engine.device
    pool_pages = engine.cache.groups[0].num_pages
    need_pages = max(batches) * (-(-span // 16))
    if pool_pages < need_pages:
        raise SystemExit(f"the pool sized from free memory holds {pool_pages} pages, {max(batches)} requests of "
                         f"{span} positions need {need_pages}")
    rng = np.random.default_rng(5)
    vocab = config.vocab_size

    prompt = rng.integers(0, vocab, size=2048).tolist()

    def one_prefill(tokens):
        engine.step([StepEntry("prefill", tokens, [len(tokens) - 1])])
        engine.release("prefill")

    engine.replay_general_steps = False
    for _ in range(2):
        one_prefill(prompt)
    eager_ms = statistics.median(timed(torch, device, lambda _: one_prefill(prompt), 1) for _ in range(3))
    engine.replay_general_steps = True
    for _ in range(3):   # seen, captured, replayed
        one_prefill(prompt)
    prefill_ms = statistics.median(timed(torch, device, lambda _: one_prefill(prompt), 1) for _ in range(3))
    flops = prefill_flops(config, 2048)
    prefill = {"value": 2048 / prefill_ms * 1e3, "tokens": 2048, "ms": prefill_ms, "eager_ms": eager_ms,
               "frac": flops / (prefill_ms * 1e-3) / (peak["bf16_tflops_sustained"] * 1e12), "tflop": flops / 1e12,
               "of": "sustained matrix peak (a step of seconds under the power cap)"}

    names = []
    points = {}
    clocks = None
    for batch in sorted(batches):
        while len(names) < batch:            # another request filled to the context, 2,048 tokens a step
            request = f"r{len(names)}"
            for first in range(0, context, 2048):
                engine.step([StepEntry(request, rng.integers(0, vocab, size=min(2048, context - first)).tolist(), [])])
            names.append(request)
        feed = rng.integers(0, vocab, size=(warmup + repeats * steps, batch))
        done = engine.context_length(names[0]) - context     # steps earlier batches already took

        def one(index):
            engine.step([StepEntry(request, [int(feed[index, i])], [0]) for i, request in enumerate(names[:batch])])

        for index in range(warmup):
            one(index)
        runs = []
        with ClockSampler() as sampler:
            for repeat in range(repeats):
                first = warmup + repeat * steps
                before = ops.launch_count()
                elapsed = timed(torch, device, lambda index: one(first + index), steps)
                contexts = sum(engine.context_length(r) for r in names[:batch]) - batch * (steps - 1) / 2
                runs.append((elapsed, ops.launch_count() - before, contexts))
        clocks = sampler.summary()
        engine.check()
        runs.sort()
        elapsed, launches, contexts = runs[len(runs) // 2]
        step_bytes = engine.model.weight_bytes() + contexts * engine.cache.bytes_per_token()
        ms = elapsed / steps
        points[f"decode_b{batch}"] = {
            "value": batch * steps / elapsed * 1e3, "ms_per_step": ms, "bytes_per_step": step_bytes,
            "achieved_gbs": step_bytes / (ms * 1e-3) / 1e9, "frac": step_bytes / (ms * 1e-3) / 1e9 / peak["hbm_gbs"],
            "gpu_launches": launches, "clocks": clocks}
    top = points[f"decode_b{max(batches)}"]
    free, total = torch.cuda.mem_get_info(device)
    line = {
        "metric": f"decode tok/s @ batch {max(batches)}, {context}-token contexts (points: other batches; prefill tok/s @ 2048)",
        "value": top["value"], "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": top["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights N(0, 0.02), uniform-random token ids",
        "impl": "ours", "repeats": repeats,
        "config": flat_config(name, config, args, {
            "layers_of_config": layers_of_config, "global_batch": max(batches), "seq_len": context,
            "pool_pages": pool_pages, "pool_gb": engine.cache.pool_bytes() / 1e9,
            "weights_gb": engine.model.weight_bytes() / 1e9, "device_free_gb_after": free / 1e9,
            "peaks": peak_source, "timing": f"median of {repeats} runs of K steps"}),
        "gpu_launches": top["gpu_launches"], "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": top["achieved_gbs"], "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": top["frac"], "bytes_per_step": top["bytes_per_step"], "of": peak_source},
        "points": points, "clocks": clocks, "load_s": load_s,
    }
    print(json.dumps(line))
    return 0


# ------------------------------------------------- small workloads for profilers
def workload(args):
    """Small fixed workloads of the 0.6B-shaped layer sizes, for profilers and
    kernel timings. ``decode``: ``--batch`` requests with ``--prompt-len``
    tokens each, then ``--steps`` decode steps (eagerly, so that a profiler
    sees every kernel; ``--graphs`` replays captured graphs and prints the
    time per step; ``--timeline``, with METALLIX_B200_TIMELINE=1 in the
    environment, prints how long each kernel of a layer holds the chain of one
    replayed step). ``prefill``: one prompt of ``--prompt-len`` tokens, three
    times (``--graphs``: then five replays, timed). ``gemm``: the tcgen05
    product against the library's on one shape. ``skinny``: the weight-streaming
    kernels of a decode step on ``--m`` rows against a ``--n`` x ``--k`` weight
    (``--swiglu``: with the activation). ``attention``: the prompt
    attention kernels alone on ``--prompt-len`` tokens behind ``--cached``
    keys. ``pick``: the samplers alone on ``--batch`` rows of logits."""
    import numpy as np
    import torch
    from metallix_b200 import ops, parse_config
    from metallix_b200.engine import Engine, StepEntry

    name, raw = SHAPES[args.shape]
    layers = args.layers or 4

    def event_time(function, count, warm=3):
        for _ in range(warm):
            function()
        return timed(torch, "cuda", lambda _: function(), count) / count

    if args.workload == "gemm":
        from metallix_b200 import tensor_core
        ops.require_cuda()
        a = torch.randn(args.m, args.k, device="cuda").bfloat16()
        w = (torch.randn(args.n, args.k, device="cuda") * 0.05).bfloat16()
        run = (lambda: tensor_core.gemm_swiglu(a, w)) if args.swiglu else (lambda: tensor_core.gemm(a, w))
        for label, function in (("tcgen05", run), ("library", lambda: torch.mm(a, w.t()))):
            microseconds = event_time(function, 10) * 1e3
            print(f"{label}: {microseconds:.1f} us, {2 * args.m * args.n * args.k / microseconds / 1e6:.0f} TFLOP/s"
                  " (launch overhead included)")
        ops.check_status("cuda")
        return 0

    if args.workload == "skinny":
        # The products of a decode step (few rows of x, all of W read once):
        # every kernel that takes the shape, over enough copies of W that none
        # is still in L2 when its turn comes again.
        ops.require_cuda()
        peak, _ = peaks()
        m, n, k = args.m, args.n, args.k
        copies = max(2, int(300e6 // (n * k * 2)) + 1)
        weights = [(torch.randn(n, k, device="cuda") * 0.05).bfloat16() for _ in range(copies)]
        a = torch.randn(m, k, device="cuda").bfloat16()
        kernels = [("stream", lambda w: ops.gemm_skinny(a, w, swiglu=args.swiglu, kernel="stream"),
                    ops.gemm_stream_supported(a, weights[0], args.swiglu)),
                   ("load", lambda w: ops.gemm_skinny(a, w, swiglu=args.swiglu, kernel="load"),
                    ops.gemm_skinny_supported(a, weights[0])),
                   ("library", (lambda w: ops.silu_mul(torch.mm(a, w.t()))) if args.swiglu else (lambda w: torch.mm(a, w.t())),
                    True)]
        for label, function, takes in kernels:
            if not takes:
                print(f"{label}: does not take [{m}, {k}] x [{n}, {k}]^T")
                continue
            for w in weights[:3]:
                function(w)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()   # replayed: the launches from Python do not count
            with torch.cuda.graph(graph):
                for w in weights:
                    function(w)
            graph.replay()
            microseconds = timed(torch, "cuda", lambda _: graph.replay(), 3) / 3 / copies * 1e3
            rate = n * k * 2 / microseconds / 1e3
            print(f"{label}: {microseconds:.2f} us, {rate:.0f} GB/s of W ({rate / peak['hbm_gbs'] * 100:.0f}% of the copy bandwidth)")
        ops.check_status("cuda")
        return 0

    if args.workload == "pick":
        ops.require_cuda()
        rows, vocab = args.batch, raw["vocab_size"]
        generator = torch.Generator(device="cuda").manual_seed(0)
        logits = torch.randn((rows, vocab), device="cuda", generator=generator) * 3.0
        temperature = torch.full((rows,), 0.8, dtype=torch.float64, device="cuda")
        seed = torch.arange(rows, dtype=torch.int64, device="cuda")
        position = torch.arange(rows, dtype=torch.int32, device="cuda")
        top_p = torch.full((rows,), 0.9, dtype=torch.float64, device="cuda")
        top_k = torch.full((rows,), 50, dtype=torch.int32, device="cuda")
        no_k = torch.zeros(rows, dtype=torch.int32, device="cuda")
        picks = (("greedy", lambda: ops.argmax(logits)),
                 ("inverse CDF", lambda: ops.sample_icdf(logits, temperature, seed, seed, position)),
                 ("race", lambda: ops.sample_race(logits, temperature, seed, position)),
                 ("top-k 50 and top-p 0.9 mask", lambda: ops.nucleus_mask(logits, temperature, top_p, top_k)),
                 ("top-p 0.9 mask", lambda: ops.nucleus_mask(logits, temperature, top_p, no_k)))
        for label, function in picks:
            for _ in range(3):
                function()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()   # replayed, so that the launches from Python do not count
            with torch.cuda.graph(graph):
                for _ in range(10):
                    function()
            graph.replay()
            print(f"{label}: {timed(torch, 'cuda', lambda _: graph.replay(), 1) * 100:.1f} us for {rows} rows of "
                  f"{vocab} logits")
        ops.check_status("cuda")
        return 0

    if args.workload == "attention":
        ops.require_cuda()
        heads, kv_heads, head_dim = raw["num_attention_heads"], raw["num_key_value_heads"], raw["head_dim"]
        page_tokens = args.page_tokens
        tokens, total = args.prompt_len, args.cached + args.prompt_len
        pages = -(-total // page_tokens)
        generator = torch.Generator(device="cuda").manual_seed(0)
        cache = torch.randn((pages, 2, kv_heads, page_tokens, head_dim), device="cuda", generator=generator).bfloat16()
        q = torch.randn((tokens, heads, head_dim), device="cuda", generator=generator).bfloat16()
        out = torch.empty_like(q)
        table = torch.randperm(pages, device="cuda", generator=generator).int().view(1, pages)
        tile = ops.flash_prefill_tile()
        starts = list(range(0, tokens, tile))[::-1]   # the tiles with most keys first
        ints = lambda values: torch.tensor(values, dtype=torch.int32, device="cuda")
        tile_request, tile_start = ints([0] * len(starts)), ints(starts)
        tile_length = ints([min(tile, tokens - s) for s in starts])
        positions = torch.arange(args.cached, total, dtype=torch.int32, device="cuda")
        flops = 4.0 * head_dim * heads * sum(args.cached + t + 1 for t in range(tokens))
        for kernel in (("tcgen05", "mma") if args.kernel == "both" else (args.kernel,)):
            run = lambda: ops.flash_prefill(q, cache, out, table, tile_request, tile_start, tile_length, positions,
                                            head_dim ** -0.5, kernel=kernel, longest_context=total)
            microseconds = event_time(run, 10) * 1e3
            print(f"{kernel}: {microseconds:.1f} us, {flops / microseconds / 1e6:.0f} TFLOP/s (causal flops)")
        ops.check_status("cuda")
        return 0

    config = parse_config(dict(raw, num_hidden_layers=layers))
    pages = args.batch * (-(-(args.prompt_len + 64) // args.page_tokens) + 1) + 64 * 16 // args.page_tokens
    engine = Engine.from_random(config, 0, dtype="bfloat16", page_tokens=args.page_tokens, num_pages=pages,
                                max_requests=args.batch + 2, max_context=args.max_context or max(4096, args.prompt_len + 256),
                                cuda_graphs=args.graphs or args.timeline,   # the timeline is of the step as it serves
                                gemm_backend=args.gemm)
    rng = np.random.default_rng(0)
    steps = args.steps if args.steps != 128 else 4
    if args.workload == "prefill":
        ids = rng.integers(0, config.vocab_size, size=args.prompt_len).tolist()
        for _ in range(3):
            engine.step([StepEntry("p", ids, [args.prompt_len - 1])])
            engine.release("p")
        torch.cuda.synchronize()
        if args.graphs:   # the step is replayed as a graph from its second occurrence on
            def once(_):
                engine.step([StepEntry("p", ids, [args.prompt_len - 1])])
                engine.release("p")
            milliseconds = timed(torch, "cuda", once, 5) / 5
            print(f"{milliseconds:.4f} ms per prompt step, {args.prompt_len / milliseconds * 1e3:.0f} tokens/s")
    else:
        names = [f"r{i}" for i in range(args.batch)]
        for first in range(0, args.batch, 4):
            engine.step([StepEntry(n, rng.integers(0, config.vocab_size, size=args.prompt_len).tolist(), [])
                         for n in names[first:first + 4]])
        for _ in range(steps):
            engine.step([StepEntry(n, [int(rng.integers(0, config.vocab_size))], [0]) for n in names])
        torch.cuda.synchronize()
        if args.timeline:
            ops.timeline(reset=True)
            engine.step([StepEntry(n, [5], [0]) for n in names])
            torch.cuda.synchronize()
            events = ops.timeline()
            print(f"{len(events)} chained kernels, {(events[-1][0] - events[0][0]) / 1e3:.1f} us from the first to the last")
            # the kernels of one layer repeat with this period: found from the sources' names
            sources = [source for _, source in events[1:]]
            period = next((p for p in range(2, 40) if sources[:p] == sources[p:2 * p] == sources[2 * p:3 * p]), 9)
            first = 1   # after the embedding
            sums = [0.0] * period
            layer_count = (len(events) - 1 - first) // period
            for layer in range(layer_count):
                for k in range(period):
                    i = first + layer * period + k
                    sums[k] += (events[i + 1][0] - events[i][0]) / 1e3
            print("| kernel of a layer (in launch order) | source | us until the next kernel may go on (mean over layers) |")
            print("|---|---|---|")
            for k in range(period):
                print(f"| {k} | {events[first + k][1]} | {sums[k] / max(layer_count, 1):.2f} |")
            print(f"| a layer | | {sum(sums) / max(layer_count, 1):.2f} |")
        if args.graphs:
            milliseconds = timed(torch, "cuda", lambda _: engine.step([StepEntry(n, [5], [0]) for n in names]), 50) / 50
            print(f"{milliseconds:.4f} ms per decode step")
    engine.check()
    print("ok")
    return 0


def main():
    parser = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=128)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", default="ours", choices=("ours", "reference"))
    parser.add_argument("--shape", default="0.6b", choices=tuple(SHAPES))
    parser.add_argument("--repeats", type=int, default=5, help="runs of K timed steps; the median is reported")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--layers", type=int, default=0, help="fewer layers than the shape has (0: all)")
    parser.add_argument("--prompt-len", type=int, default=2048)
    parser.add_argument("--context", type=int, default=4096)
    parser.add_argument("--gemm", default="auto")
    parser.add_argument("--no-points", action="store_true", help="skip batch 1 and 64")
    parser.add_argument("--decode-many", type=int, default=2048)
    parser.add_argument("--decode-resident", type=int, default=None,
                        help="blocks of the decode attention the GPU is taken to hold at once (0: one block per "
                             "tile always); default: the library's")
    # --shape 8b / 32b
    parser.add_argument("--requests", type=int, default=64)
    parser.add_argument("--max-tokens-per-step", type=int, default=8192)
    parser.add_argument("--prefill-chunk", type=int, default=0)
    parser.add_argument("--pool-fraction", type=float, default=0.9,
                        help="share of the memory free after loading that the cache pool takes")
    parser.add_argument("--batches", default="1,8,32", help="32b: decode batch sizes")
    parser.add_argument("--context-32b", type=int, default=8192)
    # --workload
    parser.add_argument("--workload", choices=("decode", "prefill", "gemm", "skinny", "attention", "pick"))
    parser.add_argument("--graphs", action="store_true")
    parser.add_argument("--timeline", action="store_true")
    parser.add_argument("--m", type=int, default=2048)
    parser.add_argument("--n", type=int, default=4096)
    parser.add_argument("--k", type=int, default=1024)
    parser.add_argument("--swiglu", action="store_true", help="gemm: the fused SwiGLU epilogue (n = 2 * inter)")
    parser.add_argument("--cached", type=int, default=0, help="attention: keys already in the cache")
    parser.add_argument("--kernel", default="both", choices=("both", "tcgen05", "mma"))
    parser.add_argument("--page-tokens", type=int, default=16, help="workloads: tokens per cache page")
    parser.add_argument("--max-context", type=int, default=0, help="workloads: the engine's context limit")
    args = parser.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": REFERENCE_UNAVAILABLE}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU: this engine runs on a single B200, --gpus {args.gpus} is outside it")
        return 2
    if args.decode_resident is not None:
        from metallix_b200 import ops
        ops.set_decode_resident_blocks(args.decode_resident, max(args.decode_many, args.decode_resident))
    if args.workload:
        return workload(args)
    if args.shape == "8b":
        return continuous_batching(args)
    if args.shape == "32b":
        return large_model(args)
    return headline(args)


if __name__ == "__main__":
    sys.exit(main())
