"""The engine against the plain implementation however the work is cut:
whole requests, the last 32 tokens one by one, portions of changing size, and
mixed batches over so few pages that they are used again; in float32 and in
bfloat16; through Engine.step and through bin/trace_run."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import plain_qwen3 as plain
import replay_helpers as cuts
from conftest import (ROOT, TOL_BF16_VS_EXACT, TOL_BF16_VS_ROUNDED, TOL_CUTS_BF16, TOL_CUTS_F32, TOL_F32,
                      random_ids)

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [5, 17, 31, 70, 100], "B": [1, 9, 40, 63, 130, 97], "C": [3, 50, 200, 33],
           "D": [300, 2, 64, 540, 257]}


@pytest.fixture(scope="module")
def references(model_folders):
    """name -> (requests, exact logits, logits with bfloat16 activation rounding)."""
    out = {}
    for name, (folder, config, tensors, page) in model_folders.items():
        requests = {f"r{i}": random_ids(100 * i + len(name), n, config["vocab_size"])
                    for i, n in enumerate(LENGTHS[name])}
        exact = {k: plain.forward_logits(config, tensors, ids) for k, ids in requests.items()}
        rounded = {k: plain.forward_logits(config, tensors, ids, bf16_activations=True)
                   for k, ids in requests.items()}
        out[name] = (requests, exact, rounded)
    return out


def make_engine(model_folders, name, dtype, pages=None, **options):
    from metallix_b200.engine import Engine
    folder, _, _, page = model_folders[name]
    return Engine.from_folder(folder, dtype=dtype, page_tokens=page, num_pages=pages or 256,
                              max_requests=8, **options)


def bounds(dtype):
    return (TOL_F32, TOL_CUTS_F32) if dtype == "float32" else (TOL_BF16_VS_EXACT, TOL_CUTS_BF16)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_every_cut_matches_the_plain_implementation(model_folders, references, name, dtype):
    from metallix_b200.engine import StepEntry
    requests, exact, rounded = references[name]
    limit, cut_limit = bounds(dtype)
    engine = make_engine(model_folders, name, dtype)
    worst, whole = cuts.replay(engine, cuts.whole(requests), exact, StepEntry)
    assert worst < limit, f"whole requests: {worst}"
    if dtype == "bfloat16":
        against_rounded, _ = cuts.replay(engine, cuts.whole(requests), rounded, StepEntry)
        assert against_rounded < TOL_BF16_VS_ROUNDED
    for label, steps in (("tail", cuts.tail_by_one(requests)), ("ragged", cuts.ragged(requests))):
        worst, seen = cuts.replay(engine, steps, exact, StepEntry)
        assert worst < limit, f"{label}: {worst}"
        drift = max(float(np.abs(row - whole[key]).max()) for key, row in seen.items())
        assert drift < cut_limit, f"{label} against whole: {drift}"
    engine.manager.check_invariants()
    assert engine.manager.live_requests() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_mixed_batches_with_pages_used_again(model_folders, references, name, dtype):
    from metallix_b200.engine import StepEntry
    requests, exact, _ = references[name]
    limit, cut_limit = bounds(dtype)
    page = model_folders[name][3]
    for seed in (0, 1, 2):
        steps, peak = cuts.mixed(requests, seed)
        engine = make_engine(model_folders, name, dtype, pages=peak // page)
        worst, seen = cuts.replay(engine, steps, exact, StepEntry)
        assert worst < limit, f"seed {seed}: {worst}"
        assert any(len(step["entries"]) > 1 for step in steps)
        assert engine.manager.pages_reused() > 0, "the pool was meant to be small enough for reuse"
        assert engine.manager.free_pages(0) == peak // page
        engine.manager.check_invariants()
    # the same places alone and whole
    whole_engine = make_engine(model_folders, name, dtype)
    _, whole = cuts.replay(whole_engine, cuts.whole(requests), exact, StepEntry)
    drift = max(float(np.abs(row - whole[key]).max()) for key, row in seen.items())
    assert drift < cut_limit


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["C", "D"])
def test_long_decoding(model_folders, name, dtype):
    """600 tokens one by one after a short prompt (configurations C and D allow
    that many positions), every tenth compared."""
    from metallix_b200.engine import StepEntry
    folder, config, tensors, page = model_folders[name]
    ids = random_ids(77, 640, config["vocab_size"])
    reference = plain.forward_logits(config, tensors, ids)
    engine = make_engine(model_folders, name, dtype)
    limit, _ = bounds(dtype)
    logits = engine.step([StepEntry("long", ids[:40], [39])])
    assert np.abs(logits.cpu().double().numpy()[0] - reference[39]).max() < limit
    worst = 0.0
    for position in range(40, 640):
        logits = engine.step([StepEntry("long", [ids[position]], [0] if position % 10 == 9 else [])])
        if logits is not None:
            worst = max(worst, float(np.abs(logits.cpu().double().numpy()[0] - reference[position]).max()))
    engine.check()
    assert worst < limit


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["C", "D"])
def test_equal_portions_replay_a_graph(model_folders, name, dtype):
    """A step whose shape has been seen before replays a captured graph with
    the new integers: a prompt in equal portions (each further along, with a
    longer block table), then two requests side by side in portions of two
    sizes, match the plain implementation and what an engine without graphs
    gives."""
    from metallix_b200.engine import StepEntry
    folder, config, tensors, page = model_folders[name]
    ids = [random_ids(90 + i, 480, config["vocab_size"]) for i in range(2)]
    reference = [plain.forward_logits(config, tensors, row) for row in ids]
    limit, cut_limit = bounds(dtype)
    outputs = {}
    for graphs in (True, False):
        engine = make_engine(model_folders, name, dtype, cuda_graphs=graphs)
        seen = []
        for first in range(0, 240, 48):          # five steps of one shape
            logits = engine.step([StepEntry("a", ids[0][first:first + 48], [0, 47])])
            seen.append(logits.cpu().double().numpy())
            assert np.abs(seen[-1] - reference[0][[first, first + 47]]).max() < limit, (graphs, first)
        engine.release("a")
        for first in range(0, 480, 80):          # six steps of another: two requests, 50 and 30 tokens
            a, b = first * 5 // 8, first * 3 // 8
            logits = engine.step([StepEntry("a", ids[0][a:a + 50], [49]), StepEntry("b", ids[1][b:b + 30], [0, 29])])
            seen.append(logits.cpu().double().numpy())
            want = np.stack([reference[0][a + 49], reference[1][b], reference[1][b + 29]])
            assert np.abs(seen[-1] - want).max() < limit, (graphs, first)
        engine.check()
        if graphs:
            # (tokens per request, wanted, context bucket, what the attention says of its launches:
            # no portion behind a long context)
            bound = engine.max_context
            assert set(engine._step_graphs) == {((48,), 2, bound, (False,)), ((50, 30), 3, bound, (False,))}
        outputs[graphs] = seen
        engine.release_all()
        engine.manager.check_invariants()
    drift = max(float(np.abs(x - y).max()) for x, y in zip(outputs[True], outputs[False]))
    assert drift < cut_limit


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,prompt", [("B", 45), ("B", 48), ("D", 270)])
def test_forked_requests_go_their_own_ways(model_folders, name, prompt, dtype):
    """A request is forked after its prompt (in the middle of a page, or at a
    page's edge); parent and child decode different tokens in the same steps;
    the parent ends first and another request takes its pages while the child
    goes on. Every logit matches the plain implementation of the whole
    sequence; with so few pages that the freed ones are used again at once."""
    from metallix_b200.engine import StepEntry
    folder, config, tensors, page = model_folders[name]
    vocab = config["vocab_size"]
    shared = random_ids(5, prompt, vocab)
    ways = {"parent": shared + random_ids(6, 20, vocab), "child": shared + random_ids(7, 40, vocab)}
    other = random_ids(8, 2 * page + 3, vocab)
    expected = {k: plain.forward_logits(config, tensors, ids) for k, ids in ways.items()}
    expected["other"] = plain.forward_logits(config, tensors, other)
    # just enough: the prompt's full pages once and each way's own pages while
    # both live; later the child's whole context beside the newcomer's
    up = lambda tokens: -(-tokens // page)
    pages = max(up(prompt) + 2 * (up(prompt + 20) - prompt // page), up(prompt + 40) + up(len(other)))
    engine = make_engine(model_folders, name, dtype, pages=pages)
    limit, _ = bounds(dtype)
    worst = 0.0

    def compare(logits, pairs):
        nonlocal worst
        got = logits.cpu().double().numpy()
        for row, (key, position) in enumerate(pairs):
            worst = max(worst, float(np.abs(got[row] - expected[key][position]).max()))

    compare(engine.step([StepEntry("parent", shared, [prompt - 1])]), [("parent", prompt - 1)])
    before = engine.manager.free_pages(0)
    engine.fork("parent", "child")
    assert before - engine.manager.free_pages(0) == (1 if prompt % page else 0)   # only a partial page is copied
    assert engine.context_length("child") == prompt
    for position in range(prompt, prompt + 20):
        compare(engine.step([StepEntry("parent", [ways["parent"][position]], [0]),
                             StepEntry("child", [ways["child"][position]], [0])]),
                [("parent", position), ("child", position)])
    engine.release("parent")
    compare(engine.step([StepEntry("child", [ways["child"][prompt + 20]], [0]),
                         StepEntry("other", other, [len(other) - 1])]),
            [("child", prompt + 20), ("other", len(other) - 1)])
    assert engine.manager.pages_reused() > 0
    for position in range(prompt + 21, prompt + 40):
        compare(engine.step([StepEntry("child", [ways["child"][position]], [0])]), [("child", position)])
    engine.check()
    engine.release_all()
    engine.manager.check_invariants()
    assert engine.manager.free_pages(0) == pages
    assert worst < limit


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_first_tokens_of_a_sequence(model_folders, dtype):
    """Position 0 alone, then 1, then 2: no earlier key, a single-token prompt."""
    from metallix_b200.engine import StepEntry
    for name in ("A", "B"):
        _, config, tensors, _ = model_folders[name]
        ids = random_ids(3, 4, config["vocab_size"])
        reference = plain.forward_logits(config, tensors, ids)
        engine = make_engine(model_folders, name, dtype)
        limit, _ = bounds(dtype)
        for position, token in enumerate(ids):
            logits = engine.step([StepEntry("s", [token], [0])])
            assert np.abs(logits.cpu().double().numpy()[0] - reference[position]).max() < limit


def test_refusals_change_nothing(model_folders):
    from metallix_b200.engine import StepEntry, StepError
    engine = make_engine(model_folders, "A", "float32", pages=4)   # 16 positions
    engine.step([StepEntry("a", [1, 2, 3, 4, 5], [4])])
    free = engine.manager.free_pages(0)
    for bad in ([StepEntry("a", [1], [0]), StepEntry("a", [2], [0])],       # twice in one step
                [StepEntry("b", [], [])],                                   # no tokens
                [StepEntry("b", [256], [0])],                               # id outside the vocabulary
                [StepEntry("b", [1, 2], [2])],                              # want outside its tokens
                [StepEntry("a", [1] * 12, [0])],                            # out of pages
                [StepEntry("a", [1], [0]), StepEntry("b", [1] * 12, [0])],  # whole batch or nothing
                []):
        with pytest.raises(StepError):
            engine.step(bad)
        assert engine.manager.free_pages(0) == free and engine.context_length("a") == 5
        assert not engine.live("b")
    engine.manager.check_invariants()
    long_engine = make_engine(model_folders, "A", "float32")
    with pytest.raises(StepError, match="context limit"):
        long_engine.step([StepEntry("x", [1] * 129, [])])   # max_position_embeddings is 128


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(model_folders, references, tmp_path, dtype):
    """bin/trace_run as a user calls it: JSON lines in, 'done <step>' lines and
    <step>.f32 files out."""
    name = "B"
    requests, exact, _ = references[name]
    folder = model_folders[name][0]
    steps, peak = cuts.mixed(requests, 5)
    out = tmp_path / f"out_{dtype}"
    text = "".join(json.dumps(step) + "\n" for step in steps)
    result = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder,
                             "--dtype", dtype, "--out", str(out), "--max-tokens", str(peak)],
                            input=text, capture_output=True, text=True, timeout=600)
    assert result.returncode == 0, result.stderr[-2000:]
    assert [line for line in result.stdout.splitlines() if line.startswith("done")] == \
        [f"done {step['step']}" for step in steps]
    limit, _ = bounds(dtype)
    offsets, vocab = {}, exact["r0"].shape[1]
    for step in steps:
        for e in step["entries"]:
            offsets.setdefault(e["id"], 0)
        want = cuts.expected_rows(step, offsets, exact)
        path = out / f"{step['step']}.f32"
        if want is None:
            assert not path.exists()
        else:
            got = np.fromfile(path, dtype="<f4").reshape(-1, vocab)
            assert got.shape == want.shape
            assert np.abs(got - want).max() < limit, step["step"]
        for e in step["entries"]:
            offsets[e["id"]] += len(e["tokens"])


def test_portions_behind_a_long_context_share_their_keys(tmp_path):
    """A portion of a prompt with 2,048 or more keys in front of it is few
    query tiles with many key tiles each: the prompt kernel then shares a
    tile's keys out among blocks, eagerly and in a captured graph."""
    from metallix_b200 import Qwen3Config, ops, write_model_folder
    from metallix_b200.engine import Engine, StepEntry
    raw = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_act="silu",
               num_hidden_layers=2, hidden_size=128, num_attention_heads=6, num_key_value_heads=2,
               head_dim=64, intermediate_size=192, vocab_size=500, rope_theta=100000.0,
               rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=2560)
    folder = str(tmp_path / "long")
    write_model_folder(folder, Qwen3Config.from_dict(raw), 5, dtype="bfloat16", norm_dtype="float32")
    config, tensors = plain.read_model(folder)
    ids = random_ids(12, 2300, config["vocab_size"])
    wanted = [2099, 2163, 2227, 2299]
    reference = plain.forward_logits(config, tensors, ids)[wanted]
    assert ops.flash_key_shares(6, 2164) == 2
    for graphs in (False, True):
        engine = Engine.from_folder(folder, dtype="bfloat16", page_tokens=16, num_pages=160, max_requests=2,
                                    cuda_graphs=graphs)
        seen = [engine.step([StepEntry("r", ids[:2100], [2099])])]
        for start in (2100, 2164):               # the same shape twice: the second one replays a graph
            seen.append(engine.step([StepEntry("r", ids[start:start + 64], [63])]))
        seen.append(engine.step([StepEntry("r", ids[2228:2300], [71])]))
        engine.check()
        logits = np.concatenate([x.cpu().double().numpy() for x in seen])
        assert np.abs(logits - reference).max() < TOL_BF16_VS_EXACT, graphs
        if graphs:
            assert ((64,), 1, 2560, (True,)) in engine._step_graphs
