"""The engine against the plain implementation at the layer sizes that are
measured: hidden 1024, 16 query and 8 key/value heads of 128, SwiGLU 3072, a
vocabulary of 151,936, tied head, theta 1e6. Fewer layers than the 28 of the
Qwen3-0.6B shape (two), not smaller ones: every kernel and every launch
choice that the measured step takes runs here inside a model, in every way of
cutting the work, in float32 and in bfloat16.

Bounds. float32: the reference's own bar for the real model, every logit of
a wanted row within 5e-4 + 1e-4 |expected| (crates/app/cli/src/parity.rs:254-297).
bfloat16: relative to the row's largest magnitude; the worst case measured is
printed.
"""
import numpy as np
import pytest

import plain_qwen3 as plain
import replay_helpers as cuts
from conftest import random_ids

pytestmark = pytest.mark.gpu

REAL = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_act="silu",
            num_hidden_layers=2, hidden_size=1024, num_attention_heads=16, num_key_value_heads=8,
            head_dim=128, intermediate_size=3072, vocab_size=151936, rope_theta=1000000.0,
            rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=40960)
PAGE = 16
CONTEXT = 4096
BF16_RELATIVE = 2.5e-2   # of the row's largest |logit|; measured worst case about 1e-2


@pytest.fixture(scope="module")
def real(tmp_path_factory):
    from metallix_b200 import Qwen3Config, write_model_folder
    folder = str(tmp_path_factory.mktemp("real_sizes"))
    write_model_folder(folder, Qwen3Config.from_dict(REAL), 21, dtype="bfloat16", norm_dtype="float32",
                       device="cuda")
    config, tensors = plain.read_model(folder)
    return folder, config, tensors, {}   # the last: plain logits kept from one test to the next


class Expected:
    """Plain logits of chosen positions of named sequences, computed on demand
    and kept: ``expected[name][position]`` is a row of 151,936 values."""

    def __init__(self, config, tensors, sequences, kept):
        self.config, self.tensors, self.sequences = config, tensors, sequences
        self.rows = {name: kept.setdefault(name, {}) for name in sequences}

    def need(self, name, positions):
        missing = sorted(set(p for p in positions if p not in self.rows[name]))
        if missing:
            ids = self.sequences[name][:max(missing) + 1]
            logits = plain.forward_logits(self.config, self.tensors, ids, rows=missing)
            for position, row in zip(missing, logits):
                self.rows[name][position] = row

    def need_steps(self, steps):
        offsets, wanted = {}, {}
        for step in steps:
            for entry in step["entries"]:
                start = offsets.get(entry["id"], 0)
                wanted.setdefault(entry["id"], []).extend(start + i for i in entry["want"])
                offsets[entry["id"]] = start + len(entry["tokens"])
            for name in step["end"]:
                offsets.pop(name, None)
        for name, positions in wanted.items():
            self.need(name, positions)

    def __getitem__(self, name):
        return self.rows[name]


def make_engine(folder, dtype, pages, max_requests=8, **options):
    from metallix_b200.engine import Engine
    return Engine.from_folder(folder, dtype=dtype, page_tokens=PAGE, num_pages=pages,
                              max_requests=max_requests, max_context=CONTEXT, **options)


class Worst:
    def __init__(self, dtype):
        self.dtype, self.absolute, self.relative = dtype, 0.0, 0.0

    def check(self, got, want, label):
        """got, want: [rows, vocab]."""
        got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
        assert got.shape == want.shape, label
        assert np.isfinite(got).all(), label
        difference = np.abs(got - want)
        self.absolute = max(self.absolute, float(difference.max()))
        magnitude = np.abs(want).max(axis=1, keepdims=True)
        self.relative = max(self.relative, float((difference / magnitude).max()))
        if self.dtype == "float32":
            assert (difference <= 5e-4 + 1e-4 * np.abs(want)).all(), f"{label}: {difference.max()}"
        else:
            assert (difference <= BF16_RELATIVE * magnitude).all(), \
                f"{label}: {(difference / magnitude).max()} of the row's magnitude"

    def report(self, label):
        print(f"[real sizes, {self.dtype}] {label}: largest |difference| {self.absolute:.3e}, "
              f"{self.relative:.3e} of the row's largest |logit|")


def run_steps(engine, steps, expected, worst, label):
    from metallix_b200.engine import StepEntry
    expected.need_steps(steps)
    offsets, seen = {}, {}
    for step in steps:
        entries = [StepEntry(e["id"], e["tokens"], e["want"]) for e in step["entries"]]
        for e in step["entries"]:
            offsets.setdefault(e["id"], 0)
        logits = engine.step(entries)
        want = cuts.expected_rows(step, offsets, expected)
        if want is not None:
            got = logits.cpu().numpy()
            worst.check(got, want, f"{label}, step {step['step']}")
            row = 0
            for e in step["entries"]:
                for index in e["want"]:
                    seen[(e["id"], offsets[e["id"]] + index)] = got[row].copy()
                    row += 1
        for e in step["entries"]:
            offsets[e["id"]] += len(e["tokens"])
        for name in step["end"]:
            engine.release(name)
            del offsets[name]
    engine.check()
    return seen


LONG = 2200
# positions looked at in the long sequence: the first ones, the edges of pages
# (16), of query tiles (128) and of key splits (128), and the last 32
LONG_WANT = sorted(set([0, 1, 2, 15, 16, 17, 127, 128, 129, 1023, 1024, 1535, 1536, 2047, 2048, 2111, 2112]
                       + list(range(LONG - 32, LONG))))


def numbered(steps):
    for index, step in enumerate(steps):
        step["step"] = index
    return steps


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_long_prompt_however_it_is_cut(real, dtype):
    """2,200 tokens: whole (the prompt kernels and the products of 1,536 rows
    and more); most in one step and the last 32 one by one; in portions of
    changing size, two of 64 tokens behind 2,048 and more keys (their keys are
    shared out among blocks)."""
    folder, config, tensors, kept = real
    ids = random_ids(5, LONG, config["vocab_size"])
    expected = Expected(config, tensors, {"long": ids}, kept)
    worst = Worst(dtype)
    engine = make_engine(folder, dtype, pages=2 * (-(-LONG // PAGE)) + 8)
    whole = numbered([{"entries": [{"id": "long", "tokens": ids, "want": LONG_WANT}], "end": ["long"]}])
    seen_whole = run_steps(engine, whole, expected, worst, "whole")
    head = LONG - 32
    tail = [{"entries": [{"id": "long", "tokens": ids[:head], "want": [i for i in LONG_WANT if i < head]}], "end": []}]
    tail += [{"entries": [{"id": "long", "tokens": [ids[i]], "want": [0]}], "end": []} for i in range(head, LONG)]
    tail[-1]["end"] = ["long"]
    seen_tail = run_steps(engine, numbered(tail), expected, worst, "the last 32 one by one")
    sizes = [2, 7, 129, 510, 1400, 64, 64, 2, 1, 21]
    assert sum(sizes) == LONG
    ragged, cursor = [], 0
    for size in sizes:
        want = [i - cursor for i in LONG_WANT if cursor <= i < cursor + size]
        ragged.append({"entries": [{"id": "long", "tokens": ids[cursor:cursor + size], "want": want}], "end": []})
        cursor += size
    ragged[-1]["end"] = ["long"]
    seen_ragged = run_steps(engine, numbered(ragged), expected, worst, "portions")
    worst.report("a 2,200-token prompt whole, tail by one, in portions")
    for other in (seen_tail, seen_ragged):
        assert set(other) == set(seen_whole)
    engine.manager.check_invariants()
    assert engine.manager.live_requests() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_batches_over_few_pages(real, dtype):
    """Up to four live requests, portions of prompts beside decoded tokens,
    in a pool so small that pages are used again."""
    folder, config, tensors, kept = real
    lengths = [150, 90, 300, 40, 210, 64, 33]
    requests = {f"m{i}": random_ids(300 + i, n, config["vocab_size"]) for i, n in enumerate(lengths)}
    expected = Expected(config, tensors, requests, kept)
    worst = Worst(dtype)
    for seed in (0, 1):
        steps, peak = cuts.mixed(requests, seed)
        engine = make_engine(folder, dtype, pages=peak // PAGE)
        run_steps(engine, steps, expected, worst, f"mixed, seed {seed}")
        assert any(len(step["entries"]) > 1 for step in steps)
        assert engine.manager.pages_reused() > 0
        engine.manager.check_invariants()
    worst.report("mixed batches")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decoding_with_many_live_requests(real, dtype):
    """Decode steps of 9, 17, 64 and then (after requests have left) 33 live
    requests: the captured graphs of 16, 24, 64 and 48 rows, with padding rows,
    and rows that hold a request in one step and padding in the next."""
    from metallix_b200.engine import StepEntry
    folder, config, tensors, kept = real
    rng = np.random.default_rng(8)
    lengths = [int(n) for n in rng.integers(3, 120, size=64)]
    lengths[0], lengths[5], lengths[40] = 700, 257, 384
    decoded = 10
    requests = {f"d{i}": random_ids(900 + i, n + decoded, config["vocab_size"]) for i, n in enumerate(lengths)}
    expected = Expected(config, tensors, requests, kept)
    worst = Worst(dtype)
    pages = sum(-(-(n + decoded) // PAGE) for n in lengths) + 4
    engine = make_engine(folder, dtype, pages=pages, max_requests=66)
    names = list(requests)
    for first in range(0, 64, 8):     # the prompts, eight requests a step
        engine.step([StepEntry(name, requests[name][:lengths[int(name[1:])]], []) for name in names[first:first + 8]])
    cursor = {name: lengths[int(name[1:])] for name in names}
    for name in names:
        expected.need(name, range(cursor[name], cursor[name] + decoded))

    def decode(live, label):
        logits = engine.step([StepEntry(name, [requests[name][cursor[name]]], [0]) for name in live])
        worst.check(logits.cpu().numpy(), np.stack([expected[name][cursor[name]] for name in live]), label)
        for name in live:
            cursor[name] += 1

    for count in (9, 9, 17, 17, 64, 64, 64):
        decode(names[:count], f"{count} live requests")
    for name in names[20:51]:         # 31 leave: their rows of the next graph are padding
        engine.release(name)
    rest = names[:20] + names[51:]
    decode(rest, "33 live requests")
    decode(rest[::2], "17 live requests after 33")
    engine.check()
    if engine.graphs is not None:
        assert {16, 24, 48, 64} <= set(engine.graphs.sizes_captured())
    worst.report("decode steps with 9, 17, 64, 33 live requests")
    engine.release_all()
    engine.manager.check_invariants()
