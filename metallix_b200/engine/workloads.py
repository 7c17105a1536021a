"""Small fixed workloads of the Qwen3-0.6B-shaped model for profilers.

    python -m metallix_b200.engine.workloads decode --batch 8 --layers 4
    python -m metallix_b200.engine.workloads prefill --layers 4
    python -m metallix_b200.engine.workloads gemm --m 2048 --n 4096 --k 1024
    python -m metallix_b200.engine.workloads attention --prompt-len 2048
    python -m metallix_b200.engine.workloads pick --batch 8

``decode``: ``--batch`` requests with ``--prompt-len`` tokens each, then a few
decode steps (eagerly, so that a profiler sees every kernel; ``--graphs``
replays captured graphs and prints the time per step instead; ``--timeline``,
with METALLIX_B200_TIMELINE=1 in the environment, prints how long each kernel
of a layer holds the chain of one replayed step). ``prefill``:
one prompt of ``--prompt-len`` tokens, three times. ``gemm``: the tcgen05
product against the library's on one shape. ``attention``: the two prompt
attention kernels alone on one prompt of ``--prompt-len`` tokens over
``--context`` cached ones. ``pick``: the samplers alone on ``--batch`` rows of
logits over the model's vocabulary. Random weights, random token ids;
``--layers`` keeps captures small (a profiler replays every kernel many times).
"""
from __future__ import annotations

import argparse
import sys

QWEN3_0_6B = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_act="silu",
                  num_hidden_layers=28, hidden_size=1024, num_attention_heads=16,
                  num_key_value_heads=8, head_dim=128, intermediate_size=3072, vocab_size=151936,
                  rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
                  max_position_embeddings=40960)


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    parser.add_argument("mode", choices=("decode", "prefill", "gemm", "attention", "pick"))
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--layers", type=int, default=4)
    parser.add_argument("--prompt-len", type=int, default=2048)
    parser.add_argument("--steps", type=int, default=4)
    parser.add_argument("--graphs", action="store_true")
    parser.add_argument("--timeline", action="store_true")
    parser.add_argument("--m", type=int, default=2048)
    parser.add_argument("--n", type=int, default=4096)
    parser.add_argument("--k", type=int, default=1024)
    parser.add_argument("--swiglu", action="store_true", help="gemm: the fused SwiGLU epilogue (n = 2 * inter)")
    parser.add_argument("--context", type=int, default=0, help="attention: keys already in the cache")
    parser.add_argument("--kernel", default="both", choices=("both", "tcgen05", "mma"))
    parser.add_argument("--page-tokens", type=int, default=16, help="tokens per cache page")
    args = parser.parse_args(argv)

    import numpy as np
    import torch
    from .. import Qwen3Config, ops
    from .engine import Engine, StepEntry

    if args.mode == "gemm":
        from .. import tensor_core
        ops.require_cuda()
        a = torch.randn(args.m, args.k, device="cuda").bfloat16()
        w = (torch.randn(args.n, args.k, device="cuda") * 0.05).bfloat16()
        run = (lambda: tensor_core.gemm_swiglu(a, w)) if args.swiglu else (lambda: tensor_core.gemm(a, w))
        for name, function in (("tcgen05", run), ("library", lambda: torch.mm(a, w.t()))):
            for _ in range(3):
                function()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for _ in range(10):
                function()
            end.record()
            torch.cuda.synchronize()
            microseconds = start.elapsed_time(end) * 100
            print(f"{name}: {microseconds:.1f} us, {2 * args.m * args.n * args.k / microseconds / 1e6:.0f} TFLOP/s"
                  " (launch overhead included)")
        ops.check_status("cuda")
        return 0

    if args.mode == "pick":
        ops.require_cuda()
        rows, vocab = args.batch, QWEN3_0_6B["vocab_size"]
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
        for name, function in picks:
            for _ in range(3):
                function()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()   # replayed, so that the launches from Python do not count
            with torch.cuda.graph(graph):
                for _ in range(10):
                    function()
            graph.replay()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            graph.replay()
            end.record()
            torch.cuda.synchronize()
            print(f"{name}: {start.elapsed_time(end) * 100:.1f} us for {rows} rows of {vocab} logits")
        ops.check_status("cuda")
        return 0

    if args.mode == "attention":
        ops.require_cuda()
        heads, kv_heads, head_dim, page_tokens = (QWEN3_0_6B["num_attention_heads"], QWEN3_0_6B["num_key_value_heads"],
                                                  QWEN3_0_6B["head_dim"], args.page_tokens)
        tokens, total = args.prompt_len, args.context + args.prompt_len
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
        positions = torch.arange(args.context, total, dtype=torch.int32, device="cuda")
        flops = 4.0 * head_dim * heads * sum(args.context + t + 1 for t in range(tokens))
        for kernel in (("tcgen05", "mma") if args.kernel == "both" else (args.kernel,)):
            run = lambda: ops.flash_prefill(q, cache, out, table, tile_request, tile_start, tile_length, positions,
                                            head_dim ** -0.5, kernel=kernel, longest_context=total)
            for _ in range(3):
                run()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for _ in range(10):
                run()
            end.record()
            torch.cuda.synchronize()
            microseconds = start.elapsed_time(end) * 100
            print(f"{kernel}: {microseconds:.1f} us, {flops / microseconds / 1e6:.0f} TFLOP/s (causal flops)")
        ops.check_status("cuda")
        return 0

    config = Qwen3Config.from_dict(dict(QWEN3_0_6B, num_hidden_layers=args.layers))
    pages = args.batch * (-(-(args.prompt_len + 64) // args.page_tokens) + 1) + 64 * 16 // args.page_tokens
    engine = Engine.from_random(config, 0, dtype="bfloat16", page_tokens=args.page_tokens, num_pages=pages,
                                max_requests=args.batch + 2, max_context=max(4096, args.prompt_len + 256),
                                cuda_graphs=args.graphs or args.timeline)   # the timeline is of the step as it serves
    rng = np.random.default_rng(0)
    if args.mode == "prefill":
        ids = rng.integers(0, config.vocab_size, size=args.prompt_len).tolist()
        for _ in range(3):
            engine.step([StepEntry("p", ids, [args.prompt_len - 1])])
            engine.release("p")
        torch.cuda.synchronize()
        if args.graphs:   # the step is replayed as a graph from its second occurrence on
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for _ in range(5):
                engine.step([StepEntry("p", ids, [args.prompt_len - 1])])
                engine.release("p")
            end.record()
            torch.cuda.synchronize()
            milliseconds = start.elapsed_time(end) / 5
            print(f"{milliseconds:.4f} ms per prompt step, {args.prompt_len / milliseconds * 1e3:.0f} tokens/s")
    else:
        names = [f"r{i}" for i in range(args.batch)]
        for first in range(0, args.batch, 4):
            engine.step([StepEntry(name, rng.integers(0, config.vocab_size, size=args.prompt_len).tolist(), [])
                         for name in names[first:first + 4]])
        for _ in range(args.steps):
            engine.step([StepEntry(name, [int(rng.integers(0, config.vocab_size))], [0]) for name in names])
        torch.cuda.synchronize()
        if args.timeline:
            ops.timeline(reset=True)
            engine.step([StepEntry(name, [5], [0]) for name in names])
            torch.cuda.synchronize()
            events = ops.timeline()
            print(f"{len(events)} chained kernels, {(events[-1][0] - events[0][0]) / 1e3:.1f} us from the first to the last")
            # one layer is nine chained kernels: norm, qkv, q/k norm + rotation, attention, merge, o, norm, gate/up, down
            period = 9
            names_of_layer = ["norm", "qkv product", "q/k norm, rotation, cache", "attention (split keys)",
                              "merge of splits", "o product", "norm", "gate/up product + SwiGLU", "down product"]
            first = 1   # after the embedding
            sums = [0.0] * period
            layers = (len(events) - 1 - first) // period
            for layer in range(layers):
                for k in range(period):
                    i = first + layer * period + k
                    sums[k] += (events[i + 1][0] - events[i][0]) / 1e3
            print("| kernel of a layer | source | us until the next kernel may go on (mean over layers) |")
            print("|---|---|---|")
            for k in range(period):
                print(f"| {names_of_layer[k]} | {events[first + k][1]} | {sums[k] / max(layers, 1):.2f} |")
            print(f"| a layer | | {sum(sums) / max(layers, 1):.2f} |")
        if args.graphs:
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for _ in range(50):
                engine.step([StepEntry(name, [5], [0]) for name in names])
            end.record()
            torch.cuda.synchronize()
            print(f"{start.elapsed_time(end) / 50:.4f} ms per decode step")
    engine.check()
    print("ok")
    return 0


if __name__ == "__main__":
    sys.exit(main())
