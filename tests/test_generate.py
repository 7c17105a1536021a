"""Generation through the Python entry point and the command line against the
plain implementation: greedy, sampled, portions of prompts, a pool so small
that requests are computed again."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import plain_qwen3 as plain
from conftest import ROOT, random_ids

pytestmark = pytest.mark.gpu


def plain_greedy(config, tensors, prompt, count, margin=None):
    """Greedy tokens by recomputing the whole sequence, with the gap between
    the two largest logits at every step."""
    ids, out, gaps = list(prompt), [], []
    for _ in range(count):
        row = plain.forward_logits(config, tensors, ids)[-1]
        order = np.argsort(-row, kind="stable")
        out.append(int(order[0]))
        gaps.append(float(row[order[0]] - row[order[1]]))
        ids.append(out[-1])
    return out, gaps


def test_greedy_workload_a(model_folders):
    """Tiny A, float32: 3 requests, prompts 5/17/31, 16 greedy steps, pages of 4."""
    from metallix_b200.engine import Engine
    from metallix_b200.engine.generate import generate
    folder, config, tensors, page = model_folders["A"]
    prompts = [random_ids(i, n, config["vocab_size"]) for i, n in enumerate((5, 17, 31))]
    engine = Engine.from_folder(folder, dtype="float32", page_tokens=page, num_pages=64)
    results = generate(engine, prompts, max_new_tokens=16, eos_ids=())
    for prompt, result in zip(prompts, results):
        expected, gaps = plain_greedy(config, tensors, prompt, 16)
        assert min(gaps) > 1e-4, "a near tie would make the comparison meaningless"
        assert result.generated_ids == expected and result.finish_reason == "length"
        assert result.cached_tokens == len(prompt) + 15
    assert engine.manager.live_requests() == 0 and engine.manager.free_pages(0) == 64


def test_greedy_bfloat16_agrees_outside_near_ties(model_folders):
    """The reference's rule (crates/models/qwen/tests/bf16_agreement.rs:11-22):
    bfloat16 may leave the float32 tokens only where the two best logits are
    close."""
    from metallix_b200.engine import Engine
    from metallix_b200.engine.generate import generate
    folder, config, tensors, page = model_folders["B"]
    prompts = [random_ids(10 + i, n, config["vocab_size"]) for i, n in enumerate((9, 40, 63))]
    engine = Engine.from_folder(folder, dtype="bfloat16", page_tokens=page, num_pages=64)
    results = generate(engine, prompts, max_new_tokens=12, eos_ids=())
    for prompt, result in zip(prompts, results):
        expected, gaps = plain_greedy(config, tensors, prompt, 12)
        for step, (got, want) in enumerate(zip(result.generated_ids, expected)):
            if got != want:
                assert gaps[step] < 0.05, (step, gaps[step])
                break


def test_sampled_workload_b_with_portions_and_a_small_pool(model_folders):
    """Tiny B: prompts 1/9/40/63, portions of 16, 24 steps at temperature 0.7
    with seed 7, pages of 8. A second run over a pool so small that requests
    lose their pages and are computed again gives the same tokens, and both
    follow the host definition of the sampler on the plain logits."""
    from metallix_b200.engine import Engine
    from metallix_b200.engine.generate import Generator, generate
    from metallix_b200.sampling import SamplingParams
    folder, config, tensors, page = model_folders["B"]
    prompts = [random_ids(20 + i, n, config["vocab_size"]) for i, n in enumerate((1, 9, 40, 63))]
    engine = Engine.from_folder(folder, dtype="float32", page_tokens=page, num_pages=64)
    roomy = generate(engine, prompts, max_new_tokens=24, temperature=0.7, seed=7, eos_ids=(),
                     max_num_seqs=4, prefill_chunk=16, max_tokens_per_step=40)
    for index, (prompt, result) in enumerate(zip(prompts, roomy)):
        ids = list(prompt)
        for position, token in enumerate(result.generated_ids):
            row = plain.forward_logits(config, tensors, ids)[-1].astype(np.float32)
            uniform = plain.request_uniform(7, index, position)
            expected = plain.sample_categorical(row, 0.7, uniform)
            if expected != token:   # only a target within rounding of a boundary may differ
                weights = np.exp((row.astype(np.float64) - row.max()) / 0.7)
                cdf = np.cumsum(weights) / weights.sum()
                assert min(abs(cdf[expected] - uniform), abs(cdf[token] - uniform)) < 1e-5
            ids.append(token)
        assert len(result.generated_ids) == 24
    tight = Engine.from_folder(folder, dtype="float32", page_tokens=page, num_pages=22)
    generator = Generator(tight, max_num_seqs=4, prefill_chunk=16, max_tokens_per_step=40)
    ids = [generator.add(p, 24, SamplingParams(temperature=0.7, seed=7, stream=i)) for i, p in enumerate(prompts)]
    generator.run()
    assert generator.stats.preemptions > 0, "the pool was meant to run out"
    assert [generator.result(r).generated_ids for r in ids] == [r.generated_ids for r in roomy]
    assert tight.manager.free_pages(0) == 22


def test_race_sampler_and_nucleus_through_generate(model_folders):
    from metallix_b200.engine import Engine
    from metallix_b200.engine.generate import generate
    folder, config, tensors, page = model_folders["A"]
    prompt = random_ids(31, 12, config["vocab_size"])
    engine = Engine.from_folder(folder, dtype="float32", page_tokens=page, num_pages=64)
    result = generate(engine, [prompt], max_new_tokens=8, temperature=0.9, seed=5, sampler="race",
                      top_k=20, top_p=0.8, eos_ids=())[0]
    ids = list(prompt)
    for position, token in enumerate(result.generated_ids):
        row = plain.forward_logits(config, tensors, ids)[-1].astype(np.float32)
        legal = plain.nucleus_mask(row, 0.9, 0.8, 20)
        assert legal[token]
        assert token == plain.sample_race(row, 0.9, 5, position, legal=legal)
        ids.append(token)


def test_eos_stops_and_is_reported(model_folders):
    from metallix_b200.engine import Engine
    from metallix_b200.engine.generate import generate
    folder, config, tensors, page = model_folders["A"]
    prompt = random_ids(41, 9, config["vocab_size"])
    engine = Engine.from_folder(folder, dtype="float32", page_tokens=page, num_pages=64)
    free_run = generate(engine, [prompt], max_new_tokens=10, eos_ids=())[0].generated_ids
    stop = free_run[3]
    cut = free_run.index(stop) + 1
    stopped = generate(engine, [prompt], max_new_tokens=10, eos_ids=(stop,))[0]
    assert stopped.generated_ids == free_run[:cut] and stopped.finish_reason == "eos"
    ignored = generate(engine, [prompt], max_new_tokens=10, eos_ids=(stop,), ignore_eos=True)[0]
    assert ignored.generated_ids == free_run and ignored.finish_reason == "length"


def test_a_deadline_ends_generation_and_keeps_what_was_generated(model_folders):
    """A request with a deadline leaves when the deadline has passed (the
    generator's clock is set by hand here), with the tokens it had; the request
    beside it, launched ahead with it until then, goes on to its limit with the
    tokens it would have had alone."""
    from metallix_b200.engine import Engine
    from metallix_b200.engine.generate import Generator, generate
    from metallix_b200.sampling import SamplingParams
    folder, config, tensors, page = model_folders["A"]
    prompts = [random_ids(51, 9, config["vocab_size"]), random_ids(52, 14, config["vocab_size"])]
    engine = Engine.from_folder(folder, dtype="float32", page_tokens=page, num_pages=64)
    alone = [r.generated_ids for r in generate(engine, prompts, max_new_tokens=20, eos_ids=())]
    generator = Generator(engine, max_num_seqs=2)
    now = [100.0]
    generator._clock = lambda: now[0]
    hurried = generator.add(prompts[0], 20, SamplingParams(), eos_ids=(), deadline_s=5.0)
    patient = generator.add(prompts[1], 20, SamplingParams(), eos_ids=())
    for _ in range(6):
        generator.step()
    now[0] = 106.0
    generator.run()
    first, second = generator.result(hurried), generator.result(patient)
    assert first.finish_reason == "deadline" and 0 < len(first.generated_ids) < 20
    assert first.generated_ids == alone[0][:len(first.generated_ids)]
    assert second.finish_reason == "length" and second.generated_ids == alone[1]
    assert engine.manager.live_requests() == 0
    with pytest.raises(ValueError, match="deadline_s"):
        generator.add(prompts[0], 4, SamplingParams(), deadline_s=0.0)


def test_steps_launched_ahead_change_nothing(model_folders):
    """While all requests decode, the generator launches the next step before
    the tokens of this one have reached the host. The tokens are those of a
    generator that never does; a request that stops at an end-of-sequence
    token, one that reaches its limit earlier than the others, one that
    arrives later and a pool that runs out of pages each make it drop or skip
    a step launched ahead."""
    from metallix_b200.engine import Engine
    from metallix_b200.engine.generate import Generator
    from metallix_b200.sampling import SamplingParams
    folder, config, tensors, page = model_folders["B"]
    prompts = [random_ids(60 + i, n, config["vocab_size"]) for i, n in enumerate((9, 40, 21, 5))]
    limits = (30, 17, 30, 24)

    def run(run_ahead, num_pages, stop=(), late=False):
        engine = Engine.from_folder(folder, dtype="bfloat16", page_tokens=page, num_pages=num_pages)
        assert engine.ahead_possible()
        generator = Generator(engine, max_num_seqs=4, run_ahead=run_ahead)
        ids = []
        for index, (prompt, limit) in enumerate(zip(prompts, limits)):
            if late and index == 3:
                continue
            ids.append(generator.add(prompt, limit, SamplingParams(temperature=0.8, seed=3, stream=index),
                                     eos_ids=stop))
        steps = 0
        while not generator.idle():
            generator.step()
            steps += 1
            if late and steps == 9:
                ids.append(generator.add(prompts[3], limits[3], SamplingParams(temperature=0.8, seed=3, stream=3),
                                         eos_ids=stop))
        engine.check()
        assert engine.manager.live_requests() == 0 and engine.manager.free_pages(0) == num_pages
        engine.manager.check_invariants()
        return [generator.result(rid) for rid in ids], generator.stats

    plain_run, plain_stats = run(False, 64)
    assert plain_stats.ahead_kept == 0 and plain_stats.ahead_dropped == 0
    ahead_run, stats = run(True, 64)
    assert [r.generated_ids for r in ahead_run] == [r.generated_ids for r in plain_run]
    assert stats.ahead_kept > 10 and stats.steps == plain_stats.steps
    # an end-of-sequence token in the middle of a request: the step launched ahead is dropped
    stop = (plain_run[0].generated_ids[11],)
    stopped_plain, _ = run(False, 64, stop=stop)
    stopped_ahead, stats = run(True, 64, stop=stop)
    assert [(r.generated_ids, r.finish_reason) for r in stopped_ahead] == \
           [(r.generated_ids, r.finish_reason) for r in stopped_plain]
    assert any(r.finish_reason == "eos" for r in stopped_ahead) and stats.ahead_dropped >= 1
    # a request that arrives while the others decode
    late_plain, _ = run(False, 64, late=True)
    late_ahead, stats = run(True, 64, late=True)
    assert [r.generated_ids for r in late_ahead] == [r.generated_ids for r in late_plain]
    assert stats.ahead_kept > 5
    # so few pages that requests lose theirs while decoding and are computed again
    tight_plain, tight_plain_stats = run(False, 14)
    tight_ahead, stats = run(True, 14)
    assert tight_plain_stats.preemptions > 0 and stats.preemptions > 0
    assert [r.generated_ids for r in tight_ahead] == [r.generated_ids for r in plain_run]
    assert [r.generated_ids for r in tight_plain] == [r.generated_ids for r in plain_run]


def test_command_line(model_folders, tmp_path):
    folder, config, tensors, page = model_folders["A"]
    prompt = random_ids(51, 7, config["vocab_size"])
    expected, gaps = plain_greedy(config, tensors, prompt, 6)
    assert min(gaps) > 1e-4
    result = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "mxb"), "gen", "--model", folder,
                             "--input-ids", ",".join(map(str, prompt)), "--max-tokens", "6",
                             "--dtype", "float32", "--block-size", str(page), "--num-pages", "32",
                             "--context-tokens", "100", "--generation-timeout-ms", "600000",
                             "--verify-cache", "--trace-out", str(tmp_path / "trace.json")],
                            capture_output=True, text=True, timeout=600)
    assert result.returncode == 0, result.stderr[-2000:]
    report = json.loads(result.stdout.strip().splitlines()[-1])
    assert report["generated_ids"] == expected and report["finish_reason"] == "length"
    assert report["input_ids"] == prompt and report["cached_tokens"] == 7 + 5
    assert report["logical_kv_bytes"] == 12 * 2 * 2 * 2 * 16 * 4   # tokens * layers * (K, V) * heads * dim * bytes
    assert report["operation"] == "qwen3_greedy_cached_generation"
    comparison = report["cache_comparisons"]
    assert comparison["greedy_tokens_match"] is True and comparison["logits_within_bound"] is True
    assert comparison["positions"] == 6 and comparison["max_abs_logit_difference"] < 1e-4
    assert len(report["decode_ms"]) == 5
    # the timeline: one host span per step, device spans named by what the step did
    trace = json.load(open(tmp_path / "trace.json"))["traceEvents"]
    host = [e for e in trace if e.get("cat") == "host"]
    device = [e for e in trace if e.get("cat") == "device"]
    assert len(host) == 6 and [e["args"]["step"] for e in host] == list(range(6))
    assert host[0]["args"]["prefill_tokens"] == 7 and host[1]["args"]["decode_tokens"] == 1
    assert device and device[0]["name"] == "engine.prefill" and all(e["dur"] > 0 for e in device)
    assert any(e["name"] == "engine.decode" for e in device)


def test_random_weights_are_the_same_made_in_place_or_written_first(tmp_path):
    """``gen --config X --random-weights S`` and ``random-weights --seed S``
    followed by ``gen --model`` generate from the same tensors."""
    from conftest import TINY_D
    config_path = tmp_path / "config.json"
    config_path.write_text(json.dumps(TINY_D))
    mxb = [sys.executable, os.path.join(ROOT, "bin", "mxb")]
    common = ["--input-ids", "5,9,200,31", "--max-tokens", "12", "--dtype", "bfloat16", "--ignore-eos"]
    direct = subprocess.run(mxb + ["gen", "--config", str(config_path), "--random-weights", "3"] + common,
                            capture_output=True, text=True, timeout=600)
    assert direct.returncode == 0, direct.stderr[-2000:]
    folder = tmp_path / "written"
    made = subprocess.run(mxb + ["random-weights", "--config", str(config_path), "--seed", "3", "--out", str(folder)],
                          capture_output=True, text=True, timeout=600)
    assert made.returncode == 0, made.stderr[-2000:]
    loaded = subprocess.run(mxb + ["gen", "--model", str(folder)] + common, capture_output=True, text=True, timeout=600)
    assert loaded.returncode == 0, loaded.stderr[-2000:]
    first = json.loads(direct.stdout.strip().splitlines()[-1])["generated_ids"]
    second = json.loads(loaded.stdout.strip().splitlines()[-1])["generated_ids"]
    assert len(first) == 12 and first == second
