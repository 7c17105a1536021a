"""Trace replay: feeds given token ids through the model step by step and
writes the logits that are asked for. It samples nothing, and it has no
forward pass, cache or loader of its own: every step is ``Engine.step``.

Input, one JSON object a line on standard input::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step in which something is wanted, ``<out>/<step>.f32`` holds the logits
at the wanted places, in the order of the entries and of ``want``, as
little-endian float32 ``[wanted, vocab]``. After every step a line
``done <step>`` is printed and flushed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

PAGE_TOKENS = 16   # divides the 64-token granularity of --max-tokens
MAX_LIVE = 4       # requests live at a time, at most


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", required=True, choices=("bfloat16", "float32"))
    parser.add_argument("--out", required=True, help="folder for <step>.f32 files")
    parser.add_argument("--max-tokens", type=int, required=True,
                        help="most tokens live requests hold at any time (each rounded up to 64)")
    parser.add_argument("--page-tokens", type=int, default=PAGE_TOKENS)
    args = parser.parse_args(argv)

    from .engine import Engine, StepEntry  # builds the kernels at first use

    os.makedirs(args.out, exist_ok=True)
    pages = -(-args.max_tokens // args.page_tokens)
    engine = Engine.from_folder(args.model, dtype=args.dtype, page_tokens=args.page_tokens,
                                num_pages=pages, max_requests=MAX_LIVE * 2)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step = record["step"]
        entries = [StepEntry(request=e["id"], tokens=e["tokens"], want=e.get("want", ()))
                   for e in record.get("entries", [])]
        if entries:
            logits = engine.step(entries)
            if logits is not None:
                host = logits.detach().to("cpu").contiguous().numpy().astype("<f4", copy=False)
                host.tofile(os.path.join(args.out, f"{step}.f32"))
            engine.check()
        for request in record.get("end", []):
            engine.release(request)
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
