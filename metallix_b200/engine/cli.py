"""The command line, after the reference's ``mx gen``
(crates/app/cli/src/cli.rs:318-397): ``--model``, ``--input-ids``,
``--max-tokens``, ``--sample --temperature --seed``, ``--verify-cache``,
``--verbose`` keep their names and meanings; the options a batching engine on
a GPU adds take the names of the reference's serve knobs
(``--max-num-seqs``, ``--prefill-chunk-tokens``, cli.rs:219-284). The receipt
on standard output has the reference's field names
(crates/app/cli/src/qwen_forward.rs:1021-1050).

    mxb gen --model DIR [--input-ids 1,2,3] [--max-tokens 32]
    mxb gen --config config.json --random-weights 0 --input-ids-file prompts.json
    mxb random-weights --config config.json --seed 0 --out DIR
"""
from __future__ import annotations

import argparse
import json
import math
import sys
import time
from typing import List


def _ids(text: str) -> List[int]:
    try:
        return [int(part) for part in text.split(",") if part.strip() != ""]
    except ValueError:
        raise argparse.ArgumentTypeError(f"token ids must be comma-separated integers: {text!r}")


def _temperature(text: str) -> float:
    value = float(text)
    if not math.isfinite(value) or value <= 0.0:  # cli.rs:98-109
        raise argparse.ArgumentTypeError("temperature must be finite and positive")
    return value


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="mxb", description="metallix_b200 command line")
    commands = parser.add_subparsers(dest="command", required=True)

    gen = commands.add_parser("gen", aliases=["generate"], help="generate from token ids")
    source = gen.add_mutually_exclusive_group(required=True)
    source.add_argument("--model", metavar="MODEL_DIR",
                        help="folder with config.json and *.safetensors")
    source.add_argument("--config", metavar="CONFIG_JSON",
                        help="a config.json alone; needs --random-weights")
    gen.add_argument("--random-weights", type=int, metavar="SEED",
                     help="random weights from this seed instead of a checkpoint")
    prompts = gen.add_mutually_exclusive_group()
    prompts.add_argument("--input-ids", type=_ids,
                         help="comma-separated raw token ids; defaults to 1,2,3")
    prompts.add_argument("--input-ids-file",
                         help="JSON file with a list of token-id lists, one request each")
    gen.add_argument("--max-tokens", type=int, default=32, help="generated-token limit per request")
    gen.add_argument("--sample", action="store_true",
                     help="reproducible categorical sampling; requires --temperature and --seed")
    gen.add_argument("--temperature", type=_temperature)
    gen.add_argument("--seed", type=int)
    gen.add_argument("--top-p", type=float, default=1.0)
    gen.add_argument("--top-k", type=int, default=0)
    gen.add_argument("--sampler", choices=("icdf", "race"), default="icdf")
    gen.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16")
    gen.add_argument("--block-size", type=int, default=16, help="positions per cache page")
    gen.add_argument("--num-pages", type=int, help="pages of the cache pool")
    gen.add_argument("--kv-pool-mib", type=int, help="size the cache pool by bytes instead")
    gen.add_argument("--max-num-seqs", type=int, default=8, help="requests decoded together at most")
    gen.add_argument("--max-tokens-per-step", type=int, default=8192)
    gen.add_argument("--prefill-chunk-tokens", type=int, default=0,
                     help="most prompt tokens of one request per step; 0: no cap")
    gen.add_argument("--context-tokens", type=int, default=0,
                     help="the longest context the engine is laid out for; 0: the longest prompt plus --max-tokens")
    gen.add_argument("--generation-timeout-ms", type=float, default=0.0,
                     help="a request leaves with finish_reason 'deadline' this long after it was queued; 0: never")
    gen.add_argument("--eos-ids", type=_ids, help="stop ids; default: the configuration's")
    gen.add_argument("--ignore-eos", action="store_true")
    gen.add_argument("--verify-cache", action="store_true",
                     help="recompute every generated position from the whole sequence and compare")
    gen.add_argument("--gemm", choices=("auto", "tcgen05", "cublas", "simple"), default="auto")
    gen.add_argument("--trace-out", metavar="FILE",
                     help="write a Chrome/Perfetto JSON timeline of the steps (host and device spans)")
    gen.add_argument("-v", "--verbose", "--debug", action="store_true", dest="verbose")

    rnd = commands.add_parser("random-weights", help="write a model folder with random weights")
    rnd.add_argument("--config", required=True)
    rnd.add_argument("--seed", type=int, required=True)
    rnd.add_argument("--out", required=True)
    rnd.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16")
    return parser


VERIFY_BOUNDS = {"float32": (5e-4, 1e-4), "bfloat16": (0.0, 2.5e-2)}   # (absolute, relative to the row's largest |logit|)


def _verify_cache(engine, checker, result, dtype: str) -> dict:
    """Recomputes the logits of every generated position twice over and
    compares them, as the reference's ``--verify-cache`` compares cached and
    uncached logits (crates/app/cli/src/qwen_forward.rs:916-939): once with
    the serving engine from the whole sequence in one step (cache against no
    cache), and once with ``checker``, a second engine over the same weights
    that runs other kernels end to end (no captured graphs, no overlapped
    launches, matrix products on CUDA cores instead of tensor cores or the
    library), so that an error the serving paths share does not hide."""
    import torch
    from .. import ops
    from .engine import StepEntry
    ids = list(result.input_ids) + list(result.generated_ids[:-1])
    first = len(result.input_ids) - 1
    wanted = list(range(first, len(ids)))
    whole = engine.step([StepEntry("verify-cache", ids, wanted)]).clone()
    picked = ops.argmax(whole).tolist()
    engine.check()
    engine.release("verify-cache")
    other = checker.step([StepEntry("verify-cache", ids, wanted)])
    checker.check()
    checker.release("verify-cache")
    absolute, relative = VERIFY_BOUNDS[dtype]
    difference = (whole.double() - other.double()).abs()
    magnitude = other.double().abs().amax(dim=1, keepdim=True)
    bound = absolute + relative * (other.double().abs() if dtype == "float32" else magnitude)
    return {"positions": len(picked), "greedy_tokens_match": picked == list(result.generated_ids),
            "max_abs_logit_difference": float(difference.max()),
            "max_difference_of_row_magnitude": float((difference / magnitude).max()),
            "logits_within_bound": bool((difference <= bound).all()),
            "bound": {"absolute": absolute, "relative": relative},
            "checked_against": "a second engine: eager launches, CUDA-core matrix products"}


def run_gen(args) -> int:
    if args.sample and (args.temperature is None or args.seed is None):
        raise SystemExit("--sample requires --temperature and --seed")
    if (args.temperature is not None or args.seed is not None) and not args.sample:
        raise SystemExit("--temperature and --seed require --sample")
    if args.config and args.random_weights is None:
        raise SystemExit("--config needs --random-weights SEED")
    if args.input_ids_file:
        with open(args.input_ids_file) as handle:
            prompts = json.load(handle)
    else:
        prompts = [args.input_ids or [1, 2, 3]]

    from ..config import parse_config
    from .engine import Engine
    from .generate import generate

    started = time.perf_counter()
    options = dict(dtype=args.dtype, page_tokens=args.block_size, gemm_backend=args.gemm,
                   max_requests=max(args.max_num_seqs, 1) + 1)
    if args.model:
        from ..config import read_config
        config = read_config(args.model)
    else:
        with open(args.config) as handle:
            config = parse_config(json.load(handle))
    if args.num_pages:
        options["num_pages"] = args.num_pages
    elif args.kv_pool_mib:
        # The pool by bytes, as the reference's --kv-pool-mib (cli.rs:219-284): whole pages only.
        options["pool_bytes"] = args.kv_pool_mib * 2 ** 20
    # Rotation tables and graphs are laid out for the contexts this call can reach.
    longest = max(len(prompt) for prompt in prompts) + args.max_tokens
    if args.context_tokens and args.context_tokens < longest:
        raise SystemExit(f"--context-tokens {args.context_tokens} is below the longest prompt plus --max-tokens ({longest})")
    options["max_context"] = max(-(-max(longest, args.context_tokens) // 256) * 256, 256)
    if args.model:
        engine = Engine.from_folder(args.model, **options)
    else:
        engine = Engine.from_random(config, args.random_weights, **options)
    load_ms = (time.perf_counter() - started) * 1e3

    results = generate(engine, prompts, max_new_tokens=args.max_tokens,
                       temperature=args.temperature if args.sample else 0.0,
                       seed=args.seed or 0, top_p=args.top_p, top_k=args.top_k,
                       sampler=args.sampler, eos_ids=args.eos_ids, ignore_eos=args.ignore_eos,
                       max_num_seqs=args.max_num_seqs, max_tokens_per_step=args.max_tokens_per_step,
                       prefill_chunk=args.prefill_chunk_tokens, trace_out=args.trace_out,
                       deadline_s=args.generation_timeout_ms / 1e3 if args.generation_timeout_ms > 0 else None)
    from ..config.registry import resolve
    family = resolve(config.to_dict()).model_type   # "qwen3": the reference's receipts name the family so
    checker, verified = None, True
    if args.verify_cache and not args.sample:
        checker_options = dict(options, cuda_graphs=False, chained_launches=False, gemm_backend="simple")
        longest = max(len(r.input_ids) + len(r.generated_ids) for r in results)
        checker_options["num_pages"] = -(-longest // args.block_size) + 1
        checker_options.pop("pool_bytes", None)
        checker = (Engine.from_folder(args.model, **checker_options) if args.model
                   else Engine.from_random(config, args.random_weights, **checker_options))
    for result in results:
        report = {
            "schema_version": 1,
            "operation": f"{family}_sampled_cached_generation" if args.sample
                         else f"{family}_greedy_cached_generation",
            "backend": f"metallix_b200 sm_100a {args.dtype}",
            "input_ids": result.input_ids,
            "generated_ids": result.generated_ids,
            "finish_reason": result.finish_reason,
            "load_ms": load_ms,
            "prefill_ms": result.prefill_ms,
            "decode_ms": result.decode_ms,
            "cached_tokens": result.cached_tokens,
            "logical_kv_bytes": result.cached_tokens * engine.cache.bytes_per_token(),
            "preemptions": result.preemptions,
        }
        if args.sample:
            report["sampling"] = {"sampler": args.sampler, "algorithm": "Philox4x32-10",
                                  "seed": args.seed, "temperature": args.temperature,
                                  "top_p": args.top_p, "top_k": args.top_k}
        if args.verify_cache and not args.sample and not result.failed:
            report["cache_comparisons"] = _verify_cache(engine, checker, result, args.dtype)
            verified = verified and report["cache_comparisons"]["logits_within_bound"]
        print(json.dumps(report), flush=True)
        if args.verbose:
            print(f"prefill {result.prefill_ms:.2f} ms, {len(result.decode_ms)} decode steps, "
                  f"median {sorted(result.decode_ms)[len(result.decode_ms) // 2] if result.decode_ms else 0:.3f} ms",
                  file=sys.stderr)
    if any(r.failed for r in results):
        return 1
    return 0 if verified else 3


def run_random_weights(args) -> int:
    from ..config import parse_config
    from ..weights import write_model_folder
    with open(args.config) as handle:
        config = parse_config(json.load(handle))
    write_model_folder(args.out, config, args.seed, dtype=args.dtype)
    parameters = sum(math.prod(shape) for shape in config.tensor_shapes().values())
    print(json.dumps({"model": args.out, "seed": args.seed, "dtype": args.dtype, "parameters": parameters}))
    return 0


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    if args.command in ("gen", "generate"):
        return run_gen(args)
    return run_random_weights(args)


if __name__ == "__main__":
    sys.exit(main())
