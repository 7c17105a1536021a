#!/usr/bin/env python3
"""Decode and prefill throughput of metallix_b200 on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W]

Default workload: the Qwen3-0.6B-shaped model of BASELINE.json (28 layers,
hidden 1024, 16 query and 8 key/value heads of 128, SwiGLU 3072, vocabulary
151,936, tied head) with random weights in bfloat16, 8 requests that each hold
a 2,048-token prompt in a cache laid out for 4,096-token contexts (pages of
16), decoding one token per request per step. A "step" is one decode step.

One JSON line is printed:
  value       decoded tokens per second over K device-timed steps (CUDA events
              around K back-to-back steps with given token ids);
  e2e         the same through the Python entry point (scheduler, sampler): host
              token ids in, picked token ids out, every step;
  prefill     one 2,048-token prompt in one step: tokens per second and the
              fraction of the measured bf16 matrix peak its FLOPs reach;
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

QWEN3_0_6B = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_act="silu",
                  num_hidden_layers=28, hidden_size=1024, num_attention_heads=16,
                  num_key_value_heads=8, head_dim=128, intermediate_size=3072, vocab_size=151936,
                  rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
                  max_position_embeddings=40960)
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


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
                 "-lms", "25"], stdout=self.file, stderr=subprocess.DEVNULL)
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


def prefill_flops(config, tokens):
    """Multiply-adds times two of one whole prompt: every linear layer on every
    token, causal attention (q k^T and p v over tokens^2 / 2 pairs), and the
    head on the one wanted row."""
    h, inter = config.hidden_size, config.intermediate_size
    q = config.num_attention_heads * config.head_dim
    kv = config.num_key_value_heads * config.head_dim
    linear = 2 * tokens * (h * (q + 2 * kv) + q * h + 3 * h * inter)
    attention = 2 * 2 * config.num_attention_heads * config.head_dim * tokens * (tokens + 1) // 2
    return config.num_hidden_layers * (linear + attention) + 2 * h * config.vocab_size


def main():
    parser = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=128)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", default="ours", choices=("ours", "reference"))
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--layers", type=int, default=QWEN3_0_6B["num_hidden_layers"])
    parser.add_argument("--prompt-len", type=int, default=2048)
    parser.add_argument("--context", type=int, default=4096)
    parser.add_argument("--gemm", default="auto")
    parser.add_argument("--no-points", action="store_true", help="skip batch 1 and 64")
    args = parser.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "arclabs561/metallix is a Rust workspace on MLX/Metal for Apple Silicon with "
                          "no setup.py or pyproject.toml: pip reports the directory is not installable, "
                          "and neither cargo nor Metal exists on this box"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU: this engine runs on a single B200, --gpus {args.gpus} is outside it")
        return 2
    warmup = max(args.warmup, 3)
    steps = max(args.steps, 1)

    import numpy as np
    import torch
    from metallix_b200 import Qwen3Config, ops
    from metallix_b200.engine import Engine, StepEntry
    from metallix_b200.engine.generate import Generator
    from metallix_b200.sampling import SamplingParams

    peak, peak_source = peaks()
    raw = dict(QWEN3_0_6B, num_hidden_layers=args.layers)
    config = Qwen3Config.from_dict(raw)
    batches = [args.batch] + ([] if args.no_points else [b for b in (1, 64) if b != args.batch])
    span = args.prompt_len + warmup + steps + 64   # positions one request may reach here
    if span > args.context:
        raise SystemExit(f"prompt {args.prompt_len} + {warmup + steps} steps exceeds the context {args.context}")
    pages = max(batches) * (-(-span // 16)) + 64
    engine = Engine.from_random(config, seed=0, dtype="bfloat16", page_tokens=16, num_pages=pages,
                                max_requests=max(batches) + 2, max_context=args.context,
                                gemm_backend=args.gemm)
    device = engine.device
    rng = np.random.default_rng(0)
    vocab = config.vocab_size

    def timed(run, count):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize(device)
        start.record()
        for index in range(count):
            run(index)
        end.record()
        torch.cuda.synchronize(device)
        return start.elapsed_time(end)

    # ---------------------------------------------------------------- prefill
    prompt = rng.integers(0, vocab, size=args.prompt_len).tolist()

    def one_prefill(_):
        engine.step([StepEntry("prefill", prompt, [args.prompt_len - 1])])
        engine.release("prefill")

    for _ in range(3):
        one_prefill(0)
    prefill_ms = statistics.median(timed(one_prefill, 1) for _ in range(5))
    flops = prefill_flops(config, args.prompt_len)
    prefill = {"value": args.prompt_len / prefill_ms * 1e3, "tokens": args.prompt_len, "ms": prefill_ms,
               "frac": flops / (prefill_ms * 1e-3) / (peak["bf16_tflops"] * 1e12), "tflop": flops / 1e12}

    # ----------------------------------------------------------------- decode
    def fill(batch):
        engine.release_all()
        names = [f"r{i}" for i in range(batch)]
        for first in range(0, batch, 4):
            engine.step([StepEntry(name, rng.integers(0, vocab, size=args.prompt_len).tolist(), [])
                         for name in names[first:first + 4]])
        return names

    def decode(batch, with_clocks=False):
        names = fill(batch)
        feed = rng.integers(0, vocab, size=(warmup + steps, batch))

        def one(index):
            engine.step([StepEntry(name, [int(feed[index, i])], [0]) for i, name in enumerate(names)])

        for index in range(warmup):
            one(index)
        before = ops.launch_count()
        clocks = None
        if with_clocks:
            with ClockSampler() as sampler:
                elapsed = timed(lambda index: one(warmup + index), steps)
            clocks = sampler.summary()
        else:
            elapsed = timed(lambda index: one(warmup + index), steps)
        launches = ops.launch_count() - before
        engine.check()
        mean_context = args.prompt_len + warmup + (steps + 1) / 2
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

    # ------------------------------------------- end to end, the entry point
    engine.release_all()
    generator = Generator(engine, max_num_seqs=args.batch, max_tokens_per_step=4 * args.prompt_len)
    total_new = warmup + steps + 16   # nobody finishes inside the timed steps
    for i in range(args.batch):
        generator.add(rng.integers(0, vocab, size=args.prompt_len).tolist(), total_new,
                      SamplingParams(), eos_ids=(), ignore_eos=True)
    while generator.scheduler.num_waiting() or any(
            len(generator.scheduler.request(r).output) == 0 for r in generator.scheduler.running()):
        generator.step()   # prompts
    for _ in range(warmup):
        generator.step()
    e2e_ms = timed(lambda _: generator.step(), steps)
    e2e_value = args.batch * steps / e2e_ms * 1e3
    h2d = engine.graphs.h2d_bytes if engine.graphs is not None else 0
    generator.run()

    line = {
        "metric": "decode tok/s @ batch 8 (points: batch 1/64; prefill tok/s @ 2048 tokens; % of roofline)",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights N(0, 0.02), uniform-random token ids",
        "impl": "ours",
        "config": {
            "model": "Qwen3-0.6B-shaped", "layers": args.layers, "layers_of_config": QWEN3_0_6B["num_hidden_layers"],
            "hidden": config.hidden_size, "q_heads": config.num_attention_heads,
            "kv_heads": config.num_key_value_heads, "head_dim": config.head_dim,
            "intermediate": config.intermediate_size, "vocab": config.vocab_size, "tied_head": True,
            "global_batch": args.batch, "seq_len": args.context, "prompt_len": args.prompt_len,
            "page_tokens": 16, "parallelism": "single GPU", "gemm": args.gemm,
            "cuda_graphs": engine.graphs is not None,
            "l2": "inputs larger than L2: every step reads all weights and the live cache",
            "peaks": peak_source,
        },
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


if __name__ == "__main__":
    sys.exit(main())
