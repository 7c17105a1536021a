"""Ways a step can be scheduled that the replay traces do not reach: captured
decode graphs of 16 rows and more with rows that turn into padding, a general
step that holds decoded tokens beside portions replayed as a graph, more
shapes than graphs are kept for, a part that may not ride in a graph, a
window that gives pages back, decode steps captured in several placements; and bit-equality of float32 logits wherever one
kernel family serves both ways of cutting."""
import dataclasses

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
import replay_helpers as cuts
from conftest import TOL_BF16_VS_EXACT, TOL_CUTS_BF16, TOL_CUTS_F32, TOL_F32, random_ids

pytestmark = pytest.mark.gpu


def make_engine(model_folders, name, dtype, pages=256, max_requests=8, **options):
    from metallix_b200.engine import Engine
    folder, _, _, page = model_folders[name]
    return Engine.from_folder(folder, dtype=dtype, page_tokens=page, num_pages=pages,
                              max_requests=max_requests, **options)


def limits(dtype):
    return (TOL_F32, TOL_CUTS_F32) if dtype == "float32" else (TOL_BF16_VS_EXACT, TOL_CUTS_BF16)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "D"])
def test_decode_graphs_of_many_rows(model_folders, name, dtype):
    """9, 17 and 33 live requests (graphs of 16, 24 and 48 rows), then requests
    leave, so that rows which held a request are padding in the next replay of
    the same graph. B decodes through the general attention kernel, D through
    the split-key one."""
    from metallix_b200.engine import StepEntry
    _, config, tensors, page = model_folders[name]
    rng = np.random.default_rng(17)
    lengths = [int(n) for n in rng.integers(2, 60, size=33)]
    decoded = 7
    ids = {f"q{i}": random_ids(500 + i, n + decoded, config["vocab_size"]) for i, n in enumerate(lengths)}
    reference = {k: plain.forward_logits(config, tensors, v) for k, v in ids.items()}
    pages = sum(-(-(n + decoded) // page) for n in lengths) + 8
    engine = make_engine(model_folders, name, dtype, pages=pages, max_requests=40)
    assert engine.graphs is not None
    names = list(ids)
    for first in range(0, 33, 6):
        engine.step([StepEntry(k, ids[k][:lengths[int(k[1:])]], []) for k in names[first:first + 6]])
    cursor = {k: lengths[int(k[1:])] for k in names}
    limit, _ = limits(dtype)

    def decode(live):
        logits = engine.step([StepEntry(k, [ids[k][cursor[k]]], [0]) for k in live]).cpu().double().numpy()
        want = np.stack([reference[k][cursor[k]] for k in live])
        assert np.abs(logits - want).max() < limit, len(live)
        for k in live:
            cursor[k] += 1

    for count in (9, 17, 33, 33):
        decode(names[:count])
    for k in names[10:28]:
        engine.release(k)
    rest = names[:10] + names[28:]          # 15 live: the graph of 16 rows, after its rows 9..14 were padding
    decode(rest)
    decode(names[:9])                       # the graph of 16 again with fewer rows than before
    decode(rest[3:])                        # other requests in the rows
    engine.check()
    assert {16, 24, 48} <= set(engine.graphs.sizes_captured())
    engine.release_all()
    engine.manager.check_invariants()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["C", "D"])
def test_a_mixed_step_replays_a_graph(model_folders, name, dtype):
    """A step with two decoded tokens beside a portion of 24 and one of 9
    tokens, four times: the second occurrence captures a graph and the later
    ones replay it with other positions and block tables."""
    from metallix_b200.engine import StepEntry
    _, config, tensors, _ = model_folders[name]
    ids = [random_ids(700 + i, 200, config["vocab_size"]) for i in range(4)]
    reference = [plain.forward_logits(config, tensors, row) for row in ids]
    limit, cut_limit = limits(dtype)
    outputs = {}
    for graphs in (True, False):
        engine = make_engine(model_folders, name, dtype, cuda_graphs=graphs)
        engine.step([StepEntry("a", ids[0][:30], []), StepEntry("b", ids[1][:5], [])])
        at = [30, 5, 0, 0]
        seen = []
        for _ in range(4):
            logits = engine.step([StepEntry("a", [ids[0][at[0]]], [0]), StepEntry("c", ids[2][at[2]:at[2] + 24], [23]),
                                  StepEntry("b", [ids[1][at[1]]], [0]), StepEntry("d", ids[3][at[3]:at[3] + 9], [0, 8])])
            got = logits.cpu().double().numpy()
            want = np.stack([reference[0][at[0]], reference[2][at[2] + 23], reference[1][at[1]],
                             reference[3][at[3]], reference[3][at[3] + 8]])
            assert np.abs(got - want).max() < limit, (graphs, at)
            seen.append(got)
            at = [at[0] + 1, at[1] + 1, at[2] + 24, at[3] + 9]
        engine.check()
        if graphs:
            assert [key[0] for key in engine._step_graphs] == [(1, 24, 1, 9)]
        outputs[graphs] = seen
    drift = max(float(np.abs(x - y).max()) for x, y in zip(outputs[True], outputs[False]))
    assert drift < cut_limit


def test_more_shapes_than_graphs_are_kept(model_folders):
    """Ten shapes, each stepped twice (the second time captures), then the
    first shape again: its graph has made room meanwhile and is captured
    anew."""
    from metallix_b200.engine import StepEntry
    from metallix_b200.engine.engine import STEP_GRAPHS
    _, config, tensors, _ = model_folders["C"]
    ids = random_ids(31, 400, config["vocab_size"])
    reference = plain.forward_logits(config, tensors, ids)
    engine = make_engine(model_folders, "C", "float32")
    sizes = list(range(3, 3 + STEP_GRAPHS + 2))
    for size in sizes + [sizes[0]]:
        cursor = 0
        for _ in range(3):     # eagerly, captured, replayed
            logits = engine.step([StepEntry("s", ids[cursor:cursor + size], [size - 1])])
            assert np.abs(logits.cpu().double().numpy()[0] - reference[cursor + size - 1]).max() < TOL_F32, size
            cursor += size
        engine.release("s")
        assert len(engine._step_graphs) <= STEP_GRAPHS
    kept = [key[0] for key in engine._step_graphs]
    assert (sizes[0],) in kept and (sizes[1],) not in kept and (sizes[2],) not in kept
    engine.check()


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_float32_cuts_are_bit_equal_within_one_kernel_family(model_folders, name):
    """Head sizes 16, 32 and 48 run every token, however the step is cut,
    through the general attention kernel and the one float32 product, whose
    sums have one order per output: whole requests, portions of changing size
    and single tokens give the same bits."""
    from metallix_b200.engine import StepEntry
    _, config, tensors, _ = model_folders[name]
    lengths = {"A": [31, 100], "B": [63, 130], "C": [200, 33]}[name]
    requests = {f"r{i}": random_ids(40 + i, n, config["vocab_size"]) for i, n in enumerate(lengths)}
    exact = {k: plain.forward_logits(config, tensors, v) for k, v in requests.items()}
    engine = make_engine(model_folders, name, "float32", cuda_graphs=False)
    _, whole = cuts.replay(engine, cuts.whole(requests), exact, StepEntry)
    _, ragged = cuts.replay(engine, cuts.ragged(requests), exact, StepEntry)
    _, tail = cuts.replay(engine, cuts.tail_by_one(requests), exact, StepEntry)
    steps, _ = cuts.mixed(requests, 3)
    _, mixed = cuts.replay(engine, steps, exact, StepEntry)
    for label, seen in (("portions", ragged), ("tail", tail), ("mixed", mixed)):
        for key, row in seen.items():
            assert np.array_equal(row, whole[key]), (label, key)
    graphed = make_engine(model_folders, name, "float32")   # the same kernels inside captured graphs
    _, again = cuts.replay(graphed, cuts.tail_by_one(requests), exact, StepEntry)
    for key, row in again.items():
        assert np.array_equal(row, whole[key]), ("graphs", key)


# ------------------------------------------------ a part that may not ride in a graph
class HostReadingFeedForward:
    """A feed-forward that looks at a device value on the host (it skips its
    work when the input is all zero): it says so, and the engine then runs
    without captured graphs."""

    graph_safe = False

    def __init__(self, spec, weights, runtime):
        self.weight = weights.take(spec["weight"]).to(runtime.device, torch.float32)
        self.dtype = runtime.dtype

    def forward(self, x, ctx):
        if float(x.abs().max()) == 0.0:          # a host read of a device value
            return torch.zeros_like(x)
        assert ctx.request_offsets is not None   # outside a graph the host's lists are there
        return (torch.tanh(x.float() @ self.weight.t())).to(self.dtype)


def test_a_part_that_reads_the_device_on_the_host_turns_graphs_off(model_folders):
    from metallix_b200.config import PartSpec, Qwen3Config
    from metallix_b200.engine import Engine, StepEntry
    from metallix_b200.parts import register_part, unregister_part
    from metallix_b200.weights import load_tensors
    folder, config, tensors, page = model_folders["B"]
    typed = Qwen3Config.from_dict(config)
    register_part("feed_forward", "host_reading", HostReadingFeedForward)
    try:
        base = typed.to_model_spec()
        layers = list(base.layers)
        layers[1] = dataclasses.replace(layers[1], feed_forward=PartSpec("host_reading", {"weight": "toy.ff"}))
        spec = dataclasses.replace(base, layers=tuple(layers))
        loaded = load_tensors(folder, typed, device="cuda:0")
        toy = np.random.default_rng(2).normal(size=(96, 96)) * 0.1
        loaded["toy.ff"] = torch.tensor(toy, dtype=torch.float32, device="cuda:0")
        engine = Engine(typed, loaded, dtype="float32", page_tokens=page, num_pages=32, spec=spec)
        assert engine.graphs is None and engine._step_graphs is None
        plain_engine = Engine(typed, load_tensors(folder, typed, device="cuda:0"), dtype="float32",
                              page_tokens=page, num_pages=32)
        assert plain_engine.graphs is not None
        ids = random_ids(6, 30, config["vocab_size"])
        w = {k: v.astype(np.float64) for k, v in tensors.items()}
        x = plain.embed(w["model.embed_tokens.weight"], ids)
        eps = plain.f32(config["rms_norm_eps"])
        for layer in range(config["num_hidden_layers"]):
            if layer != 1:
                x = plain.decoder_layer(x, np.arange(30), w, layer, config)
                continue
            base_name = f"model.layers.{layer}"
            a = plain.rms_norm(x, w[f"{base_name}.input_layernorm.weight"], eps)
            r = x + plain.attention_block(a, np.arange(30), w, f"{base_name}.self_attn", config)
            x = r + np.tanh(plain.rms_norm(r, w[f"{base_name}.post_attention_layernorm.weight"], eps) @ toy.T)
        reference = plain.rms_norm(x, w["model.norm.weight"], eps) @ w["lm_head.weight"].T
        engine.step([StepEntry("t", ids[:20], [])])
        for position in range(20, 30):      # decode steps, launched kernel by kernel
            logits = engine.step([StepEntry("t", [ids[position]], [0])]).cpu().double().numpy()
            assert np.abs(logits[0] - reference[position]).max() < 5e-5
        engine.check()
    finally:
        unregister_part("feed_forward", "host_reading")


# --------------------------------------------------------------- a window
def plain_with_windows(config, tensors, ids, windows):
    """The plain model with ``windows[layer]`` (None: all keys) as the
    attention window of each layer."""
    w = {k: v.astype(np.float64) for k, v in tensors.items()}
    x = plain.embed(w["model.embed_tokens.weight"], ids)
    eps = plain.f32(config["rms_norm_eps"])
    positions = np.arange(len(ids))
    for layer in range(config["num_hidden_layers"]):
        base = f"model.layers.{layer}"
        a = plain.rms_norm(x, w[f"{base}.input_layernorm.weight"], eps)
        r = x + plain.attention_block(a, positions, w, f"{base}.self_attn", config, window=windows[layer])
        m = plain.rms_norm(r, w[f"{base}.post_attention_layernorm.weight"], eps)
        x = r + plain.swiglu(m, w[f"{base}.mlp.gate_proj.weight"], w[f"{base}.mlp.up_proj.weight"],
                             w[f"{base}.mlp.down_proj.weight"])
    head = w["model.embed_tokens.weight"] if config.get("tie_word_embeddings") else w["lm_head.weight"]
    return plain.rms_norm(x, w["model.norm.weight"], eps) @ head.T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "D"])
def test_a_windowed_layer_beside_full_ones(model_folders, name, dtype):
    """One layer sees the last 24 positions only, the others all: two groups
    of pages. The windowed group gives pages back as the window passes them
    (block tables then hold -1 there) and, in a small pool, another request
    takes them while the first still decodes. Whole, in portions (two tokens
    across the window's edge among them) and token by token through the
    captured graph."""
    from metallix_b200.config import PartSpec, Qwen3Config
    from metallix_b200.engine import Engine, StepEntry
    from metallix_b200.weights import load_tensors
    folder, config, tensors, page = model_folders[name]
    typed = Qwen3Config.from_dict(config)
    base = typed.to_model_spec()
    layers = list(base.layers)
    window = 24
    layers[1] = dataclasses.replace(layers[1], mixer=PartSpec("gqa_attention", dict(layers[1].mixer.params, window=window)))
    spec = dataclasses.replace(base, layers=tuple(layers))
    windows = [window if layer == 1 else None for layer in range(config["num_hidden_layers"])]
    requests = {"u": random_ids(61, 150, config["vocab_size"]), "v": random_ids(62, 90, config["vocab_size"])}
    reference = {k: plain_with_windows(config, tensors, v, windows) for k, v in requests.items()}
    limit, _ = limits(dtype)
    pages = 150 // page + 90 // page + 4
    engine = Engine(typed, load_tensors(folder, typed, device="cuda:0"), dtype=dtype, page_tokens=page,
                    num_pages=pages, max_requests=4, spec=spec)
    assert len(engine.cache.groups) == 2
    windowed = [g.index for g in engine.cache.groups if g.need.window][0]
    worst, _ = cuts.replay(engine, cuts.whole(requests), reference, StepEntry)
    assert worst < limit, f"whole: {worst}"
    # portions: 23 tokens, then two across the window's edge, and on
    worst, _ = cuts.replay(engine, cuts.ragged(requests, sizes=(23, 2, 7, 16, 2, 31, 1, 40)), reference, StepEntry)
    assert worst < limit, f"portions: {worst}"
    # "u" decodes token by token and gives pages of the windowed group back;
    # "v" arrives meanwhile and is handed them
    engine.step([StepEntry("u", requests["u"][:60], [])])
    free_before = engine.manager.free_pages(windowed)
    reused_before = engine.manager.pages_reused()
    for position in range(60, 150):
        entries = [StepEntry("u", [requests["u"][position]], [0])]
        expected = [reference["u"][position]]
        at = position - 100
        if 0 <= at < 45:            # "v": a portion of 2 tokens beside u's decoded token
            entries.append(StepEntry("v", requests["v"][2 * at:2 * at + 2], [1]))
            expected.append(reference["v"][2 * at + 1])
        logits = engine.step(entries).cpu().double().numpy()
        assert np.abs(logits - np.stack(expected)).max() < limit, position
        if position == 99:
            # 40 more positions in the window group cost no page: it gives back what the window has passed
            assert engine.manager.free_pages(windowed) >= free_before - 1
    assert engine.manager.pages_reused() > reused_before
    table = engine.manager.table("u" in engine._ids and engine._ids["u"], windowed)
    assert table[0] == -1 and table[-1] >= 0      # pages behind the window are gone from the table
    engine.check()
    engine.release_all()
    engine.manager.check_invariants()
    assert engine.manager.free_pages(windowed) == pages


def test_a_fork_under_a_window(model_folders):
    """A request forked behind a window: in the windowed group the child
    shares only the pages the window still covers (and copies the partial
    one), in the full group all of them; both go their own ways and match the
    plain implementation; ending the parent leaves the child whole."""
    from metallix_b200.config import PartSpec, Qwen3Config
    from metallix_b200.engine import Engine, StepEntry
    from metallix_b200.weights import load_tensors
    folder, config, tensors, page = model_folders["D"]
    typed = Qwen3Config.from_dict(config)
    base = typed.to_model_spec()
    layers = list(base.layers)
    window = 40
    layers[0] = dataclasses.replace(layers[0], mixer=PartSpec("gqa_attention", dict(layers[0].mixer.params, window=window)))
    spec = dataclasses.replace(base, layers=tuple(layers))
    windows = [window if layer == 0 else None for layer in range(config["num_hidden_layers"])]
    vocab = config["vocab_size"]
    shared = random_ids(71, 107, vocab)                    # 6 pages of 16 and 11 positions of a seventh
    ways = {"parent": shared + random_ids(72, 30, vocab), "child": shared + random_ids(73, 60, vocab)}
    reference = {k: plain_with_windows(config, tensors, v, windows) for k, v in ways.items()}
    engine = Engine(typed, load_tensors(folder, typed, device="cuda:0"), dtype="float32", page_tokens=page,
                    num_pages=24, max_requests=4, spec=spec)
    windowed = [g.index for g in engine.cache.groups if g.need.window][0]
    full = 1 - windowed
    engine.step([StepEntry("parent", shared, [])])
    engine.fork("parent", "child")
    parent_id, child_id = engine._ids["parent"], engine._ids["child"]
    held = engine.manager.table(parent_id, windowed)
    assert held[0] == -1 and engine.manager.table(child_id, windowed)[0] == -1
    assert engine.manager.table(child_id, full)[:6] == engine.manager.table(parent_id, full)[:6]
    assert engine.manager.table(child_id, full)[6] != engine.manager.table(parent_id, full)[6]
    worst = 0.0
    for step in range(30):
        logits = engine.step([StepEntry("parent", [ways["parent"][107 + step]], [0]),
                              StepEntry("child", [ways["child"][107 + step]], [0])]).cpu().double().numpy()
        worst = max(worst, np.abs(logits[0] - reference["parent"][107 + step]).max(),
                    np.abs(logits[1] - reference["child"][107 + step]).max())
    engine.release("parent")
    for step in range(30, 60):
        logits = engine.step([StepEntry("child", [ways["child"][107 + step]], [0])]).cpu().double().numpy()
        worst = max(worst, np.abs(logits[0] - reference["child"][107 + step]).max())
    engine.check()
    engine.manager.check_invariants()
    engine.release_all()
    assert engine.manager.free_pages(windowed) == 24 and engine.manager.free_pages(full) == 24
    assert worst < TOL_F32


def test_a_decode_step_is_captured_in_several_placements(model_folders):
    """The first decode step of a (rows, context) bucket is captured several
    times and the fastest capture kept; each candidate replays the real step,
    which must change nothing: the logits are those of an engine that captures
    once, bit for bit, and the cache goes on from the same state."""
    from metallix_b200.engine import StepEntry
    _, config, tensors, page = model_folders["D"]
    ids = {"a": random_ids(31, 60, config["vocab_size"]), "b": random_ids(32, 45, config["vocab_size"])}
    outputs = []
    for placements in (1, 4):
        engine = make_engine(model_folders, "D", "bfloat16")
        engine.graphs.placements = placements
        engine.step([StepEntry("a", ids["a"][:40], []), StepEntry("b", ids["b"][:25], [])])
        seen = []
        for step in range(20):
            logits = engine.step([StepEntry("a", [ids["a"][40 + step]], [0]), StepEntry("b", [ids["b"][25 + step]], [0])])
            seen.append(logits.cpu().clone())
        engine.check()
        timings = engine.graphs.placement_ms
        assert (len(timings) == 0) if placements == 1 else all(2 <= len(t) <= 4 for t in timings.values()) and timings
        outputs.append(torch.stack(seen))
    assert torch.equal(outputs[0], outputs[1])
    reference = plain.forward_logits(config, tensors, ids["a"])
    assert np.abs(outputs[1][:, 0].double().numpy() - reference[40:60]).max() < TOL_BF16_VS_EXACT
