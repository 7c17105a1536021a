"""Each part alone against the plain implementation, the layer order as data,
and toy parts that are defined here, registered, built and stepped without
any change to the framework's files: a mixer with state of its own, a
feed-forward with routing, a position encoding of another convention."""
import dataclasses

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from conftest import TOL_BF16_VS_EXACT, TOL_F32, random_ids

pytestmark = pytest.mark.gpu


def runtime(dtype, max_positions=512):
    from metallix_b200.parts import Runtime
    return Runtime(device=torch.device("cuda:0"), dtype=dtype, max_positions=max_positions)


def store(tensors):
    from metallix_b200.parts import WeightStore
    return WeightStore({k: torch.tensor(v) for k, v in tensors.items()})


def context(dtype, counts, starts):
    """A StepContext for requests with ``counts`` tokens starting at ``starts``."""
    from metallix_b200.parts import StepContext
    positions, token_request, offsets = [], [], [0]
    for row, (count, start) in enumerate(zip(counts, starts)):
        positions += list(range(start, start + count))
        token_request += [row] * count
        offsets.append(len(positions))
    as_int = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    return StepContext(device=torch.device("cuda:0"), dtype=dtype, num_tokens=len(positions),
                       num_requests=len(counts), positions=as_int(positions),
                       token_request=as_int(token_request), request_slots=as_int(list(range(len(counts)))),
                       request_offsets=offsets, request_positions=list(starts))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_part(dtype):
    from metallix_b200.config import PartSpec
    from metallix_b200.parts import build_part
    rng = np.random.default_rng(0)
    w = (1 + rng.uniform(-0.1, 0.1, size=72)).astype(np.float32)
    norm = build_part("norm", PartSpec("rmsnorm", {"size": 72, "eps": 2e-5, "weight": "n.weight"}),
                      store({"n.weight": w}), runtime(dtype))
    x = rng.normal(size=(5, 72)).astype(np.float32)
    delta = rng.normal(size=(5, 72)).astype(np.float32)
    residual = torch.tensor(x, device="cuda")
    out = norm.add_forward(residual, torch.tensor(delta, device="cuda").to(dtype), dtype)
    total = x.astype(np.float64) + torch.tensor(delta).to(dtype).double().numpy()
    ref = plain.rms_norm(total, w.astype(np.float64), float(np.float32(2e-5)))
    assert np.abs(out.cpu().double().numpy() - ref).max() < (2e-6 if dtype == torch.float32 else 2e-2)
    assert np.abs(residual.cpu().double().numpy() - total).max() < 1e-6
    with pytest.raises(ValueError):
        build_part("norm", PartSpec("rmsnorm", {"size": 71, "eps": 1e-6, "weight": "n.weight"}),
                   store({"n.weight": w}), runtime(dtype))


def test_position_part():
    from metallix_b200.config import PartSpec
    from metallix_b200.parts import build_part
    rope = build_part("position", PartSpec("rope_half", {"theta": 5e4, "rotary_dim": 48, "head_dim": 48}),
                      store({}), runtime(torch.float32, 300))
    rng = np.random.default_rng(1)
    q, k = rng.normal(size=(6, 3 * 48)).astype(np.float32), rng.normal(size=(6, 48)).astype(np.float32)
    positions = [0, 1, 2, 150, 151, 299]
    q_out, k_out = rope.apply(torch.tensor(q, device="cuda"), torch.tensor(k, device="cuda"),
                              torch.tensor(positions, dtype=torch.int32, device="cuda"))
    assert np.abs(q_out.cpu().double().numpy()
                  - plain.rope_half(q.astype(np.float64).reshape(6, 3, 48), positions, 5e4)).max() < 2e-6
    assert np.abs(k_out.cpu().double().numpy()
                  - plain.rope_half(k.astype(np.float64).reshape(6, 1, 48), positions, 5e4)).max() < 2e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_feed_forward_part(dtype):
    from metallix_b200.config import PartSpec
    from metallix_b200.parts import build_part
    rng = np.random.default_rng(2)
    hidden, inter = 72, 200
    weights = {"g": rng.normal(size=(inter, hidden)) * 0.1, "u": rng.normal(size=(inter, hidden)) * 0.1,
               "d": rng.normal(size=(hidden, inter)) * 0.1}
    weights = {k: torch.tensor(v).to(dtype).double().numpy() for k, v in weights.items()}
    part = build_part("feed_forward", PartSpec("swiglu", {
        "hidden_size": hidden, "intermediate_size": inter, "gate_proj": "g", "up_proj": "u",
        "down_proj": "d"}), store(weights), runtime(dtype))
    x = torch.tensor(rng.normal(size=(9, hidden))).to(dtype)
    out = part.forward(x.cuda(), None)
    ref = plain.swiglu(x.double().numpy(), weights["g"], weights["u"], weights["d"])
    assert np.abs(out.cpu().double().numpy() - ref).max() < (1e-5 if dtype == torch.float32 else 3e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_part_with_its_cache(model_folders, dtype):
    """The mixer alone: a prompt portion, then the rest beside another
    request's tokens, against whole-sequence attention."""
    from metallix_b200.config import Qwen3Config
    from metallix_b200.parts import CacheView, build_part
    _, config, tensors, _ = model_folders["B"]
    spec = Qwen3Config.from_dict(config).to_model_spec().layers[1].mixer
    mixer = build_part("mixer", spec, store(tensors), runtime(dtype))
    need = mixer.cache_need()
    assert (need.kind, need.kv_heads, need.head_dim, need.window) == ("kv_pages", 2, 32, None)
    rng = np.random.default_rng(3)
    x = torch.tensor(rng.normal(size=(50, 96))).to(dtype)
    ref = plain.attention_block(x.double().numpy(), np.arange(50), tensors, "model.layers.1.self_attn", config)
    pool = torch.zeros(16, 2, 2, 8, 32, dtype=dtype, device="cuda")
    tables = torch.tensor([[5, 2, 9, 0, 11, 3, 7], [1, 4, 6, 8, 10, 12, 13]], dtype=torch.int32, device="cuda")

    def slots(row, start, count):
        where = np.arange(start, start + count)
        return tables[row].cpu().numpy()[where // 8] * 8 + where % 8

    def run(counts, starts, rows, xs):
        ctx = context(dtype, counts, starts)
        all_slots = np.concatenate([slots(r, s, c) for r, s, c in zip(rows, starts, counts)])
        view = CacheView(need=need, pool=pool, block_tables=tables[rows],
                         slots=torch.tensor(all_slots, dtype=torch.int32, device="cuda"))
        return mixer.forward(torch.cat(xs).cuda(), ctx, view).cpu().double().numpy()

    limit = 1e-5 if dtype == torch.float32 else 3e-2
    first = run([30], [0], [0], [x[:30]])
    assert np.abs(first - ref[:30]).max() < limit
    other = run([7], [0], [1], [x[:7]])          # another request starts in its own pages
    both = run([20, 5], [30, 7], [0, 1], [x[30:], x[7:12]])
    assert np.abs(both[:20] - ref[30:]).max() < limit
    assert np.abs(np.concatenate([other, both[20:]]) - ref[:12]).max() < limit


def test_attention_part_leaves_summands_where_one_kernel_merges_and_projects(model_folders):
    """A decode step of few single tokens in bfloat16: ``forward_summands``
    gives [heads, tokens, hidden] in float32 whose sum is ``forward``'s output
    and the whole-sequence attention; a step with a portion in it, or float32,
    gives the plain output. The block adds the summands up in its norm."""
    from metallix_b200.config import Qwen3Config
    from metallix_b200.parts import CacheView, build_part
    _, config, tensors, _ = model_folders["D"]     # heads of 64 values, three query heads a key/value head
    spec = Qwen3Config.from_dict(config).to_model_spec().layers[1].mixer
    rng = np.random.default_rng(5)
    x = torch.tensor(rng.normal(size=(41, 128))).bfloat16()
    ref = plain.attention_block(x.double().numpy(), np.arange(41), tensors, "model.layers.1.self_attn", config)
    tables = torch.tensor([[5, 2, 9], [1, 4, 6]], dtype=torch.int32, device="cuda")
    for dtype in (torch.bfloat16, torch.float32):
        mixer = build_part("mixer", spec, store(tensors), runtime(dtype))
        need = mixer.cache_need()
        pool = torch.zeros(12, 2, 2, 16, 64, dtype=dtype, device="cuda")

        def run(call, counts, starts, rows, xs):
            where = [np.arange(s, s + c) for s, c in zip(starts, counts)]
            slots = np.concatenate([tables[r].cpu().numpy()[w // 16] * 16 + w % 16 for r, w in zip(rows, where)])
            view = CacheView(need=need, pool=pool, block_tables=tables[rows],
                             slots=torch.tensor(slots, dtype=torch.int32, device="cuda"))
            return call(torch.cat(xs).to(dtype).cuda(), context(dtype, counts, starts), view)

        run(mixer.forward, [40], [0], [0], [x[:40]])
        run(mixer.forward, [20], [0], [1], [x[:20]])
        decode = ([1, 1], [40, 20], [0, 1], [x[40:41], x[20:21]])
        plain_out = run(mixer.forward, *decode)
        summed = run(mixer.forward_summands, *decode)
        if dtype == torch.bfloat16:
            assert summed.shape == (6, 2, 128) and summed.dtype == torch.float32
            total = summed.sum(dim=0)
        else:
            assert summed.shape == (2, 128)
            total = summed
        assert np.abs(total.cpu().double().numpy() - plain_out.cpu().double().numpy()).max() < 2e-2
        assert np.abs(total.cpu().double().numpy() - ref[[40, 20]]).max() < (3e-2 if dtype == torch.bfloat16 else 1e-5)
        mixed = run(mixer.forward_summands, [3, 1], [37, 20], [0, 1], [x[37:40], x[20:21]])
        assert mixed.shape == (4, 128)      # a portion beside the single token: the plain output


def test_layer_order_is_data(model_folders):
    """A layer named twice (with a cache entry of its own for the second run)
    and a layer that reads the cache another layer wrote."""
    from metallix_b200.config import LayerRun, Qwen3Config
    from metallix_b200.engine import Engine, StepEntry
    from metallix_b200.weights import load_tensors
    folder, config, tensors, page = model_folders["B"]
    typed = Qwen3Config.from_dict(config)
    ids = random_ids(8, 45, config["vocab_size"])
    cases = {
        "twice": ([LayerRun(0), LayerRun(1), LayerRun(1, cache=3), LayerRun(2)], [0, 1, 1, 2], None),
        "reads": ([LayerRun(0), LayerRun(1), LayerRun(2, cache=1, write_cache=False)], [0, 1, 2], {2: 1}),
    }
    for label, (order, layers, reads) in cases.items():
        spec = dataclasses.replace(typed.to_model_spec(), order=tuple(order))
        reference = plain.forward_logits(config, tensors, ids, order=layers, reads=reads)
        engine = Engine(typed, load_tensors(folder, typed, device="cuda:0"), dtype="float32",
                        page_tokens=page, num_pages=32, spec=spec)
        whole = engine.step([StepEntry("w", ids, list(range(45)))]).cpu().double().numpy()
        assert np.abs(whole - reference).max() < TOL_F32, label
        parts = [engine.step([StepEntry("p", ids[:20], [19])]), engine.step([StepEntry("p", ids[20:44], [23])]),
                 engine.step([StepEntry("p", ids[44:], [0])])]
        got = np.stack([p.cpu().double().numpy()[0] for p in parts])
        assert np.abs(got - reference[[19, 43, 44]]).max() < TOL_F32, label
        if label == "reads":
            assert len(engine.cache.groups[0].entries) == 2   # layer 2 holds no pages of its own
    with pytest.raises(ValueError, match="before any layer has written"):
        dataclasses.replace(typed.to_model_spec(), order=(LayerRun(0, cache=1, write_cache=False),)).validate()


# ----------------------------------------------------------------- a toy mixer
class RunningMeanMixer:
    """out_t = mean over the request's positions 0..t of (x W^T). The running
    sum is state of fixed size per request; no pages. Torch operations only:
    it stands for a mixer somebody else wrote."""

    def __init__(self, spec, weights, runtime):
        self.weight = weights.take(spec["weight"]).to(runtime.device, torch.float32)
        self.hidden = spec["hidden_size"]
        self.dtype = runtime.dtype

    def cache_need(self):
        from metallix_b200.config import CacheNeed
        return CacheNeed(kind="state", state_shape=(self.hidden,), state_dtype="float32")

    def forward(self, x, ctx, cache):
        projected = x.float() @ self.weight.t()
        out = torch.empty_like(projected)
        for row in range(ctx.num_requests):
            begin, end = ctx.request_offsets[row], ctx.request_offsets[row + 1]
            slot = int(ctx.request_slots[row])
            sums = cache.state[slot] + torch.cumsum(projected[begin:end], dim=0)
            counts = torch.arange(ctx.request_positions[row] + 1, ctx.request_positions[row] + 1 + end - begin,
                                  device=x.device, dtype=torch.float32)
            out[begin:end] = sums / counts[:, None]
            cache.state[slot] = sums[-1]
        return out.to(self.dtype)


def plain_with_running_mean(config, tensors, ids, toy_layer, toy_weight):
    """The plain model with layer ``toy_layer``'s attention replaced by the
    running mean."""
    w = {k: v.astype(np.float64) for k, v in tensors.items()}
    x = plain.embed(w["model.embed_tokens.weight"], ids)
    eps = plain.f32(config["rms_norm_eps"])
    positions = np.arange(len(ids))
    for layer in range(config["num_hidden_layers"]):
        base = f"model.layers.{layer}"
        if layer != toy_layer:
            x = plain.decoder_layer(x, positions, w, layer, config)
            continue
        mixed_in = plain.rms_norm(x, w[f"{base}.input_layernorm.weight"], eps)
        projected = mixed_in @ toy_weight.T
        residual = x + np.cumsum(projected, axis=0) / (positions + 1)[:, None]
        mlp_in = plain.rms_norm(residual, w[f"{base}.post_attention_layernorm.weight"], eps)
        x = residual + plain.swiglu(mlp_in, w[f"{base}.mlp.gate_proj.weight"], w[f"{base}.mlp.up_proj.weight"],
                                    w[f"{base}.mlp.down_proj.weight"])
    normed = plain.rms_norm(x, w["model.norm.weight"], eps)
    return normed @ w["lm_head.weight"].T


def test_a_toy_mixer_with_state_of_its_own(model_folders):
    from metallix_b200.config import PartSpec, Qwen3Config
    from metallix_b200.engine import Engine, StepEntry
    from metallix_b200.parts import register_part, unregister_part
    from metallix_b200.weights import load_tensors
    folder, config, tensors, page = model_folders["B"]
    typed = Qwen3Config.from_dict(config)
    register_part("mixer", "running_mean", RunningMeanMixer)
    try:
        base = typed.to_model_spec()
        layers = list(base.layers)
        layers[1] = dataclasses.replace(layers[1], mixer=PartSpec("running_mean", {
            "hidden_size": 96, "weight": "toy.weight"}))
        spec = dataclasses.replace(base, layers=tuple(layers))
        toy = np.random.default_rng(4).normal(size=(96, 96)) * 0.05
        loaded = load_tensors(folder, typed, device="cuda:0")
        loaded["toy.weight"] = torch.tensor(toy, dtype=torch.float32, device="cuda:0")
        engine = Engine(typed, loaded, dtype="float32", page_tokens=page, num_pages=32, max_requests=3,
                        spec=spec)
        # one group of pages for the two attention layers, one state entry for the toy
        assert len(engine.cache.groups) == 1 and engine.cache.groups[0].entries == [0, 2]
        assert list(engine.cache.states) == [1] and engine.cache.states[1].shape == (3, 96)
        requests = {"a": random_ids(1, 40, 384), "b": random_ids(2, 23, 384), "c": random_ids(3, 31, 384)}
        reference = {k: plain_with_running_mean(config, tensors, ids, 1, toy) for k, ids in requests.items()}
        whole = engine.step([StepEntry("a", requests["a"], list(range(40)))]).cpu().double().numpy()
        assert np.abs(whole - reference["a"]).max() < 5e-5
        engine.release("a")
        # mixed: portions of one request beside another's single tokens; "c"
        # later takes the slot that "b" gives back and must start from zero
        a, b, c = requests["a"], requests["b"], requests["c"]
        engine.step([StepEntry("a", a[:17], [])])
        engine.step([StepEntry("b", b[:22], [])])
        logits = engine.step([StepEntry("a", a[17:39], [21]), StepEntry("b", b[22:], [0])]).cpu().double().numpy()
        assert np.abs(logits[0] - reference["a"][38]).max() < 5e-5
        assert np.abs(logits[1] - reference["b"][22]).max() < 5e-5
        engine.release("b")
        logits = engine.step([StepEntry("a", a[39:], [0]), StepEntry("c", c, [30])]).cpu().double().numpy()
        assert np.abs(logits[0] - reference["a"][39]).max() < 5e-5
        assert np.abs(logits[1] - reference["c"][30]).max() < 5e-5
        # a fork takes the state with it: "e" goes on from "d"'s running sum
        # with other tokens, while "d" goes on with its own
        engine.release("a")
        engine.release("c")
        branch = a[:25] + c[:9]
        expected = plain_with_running_mean(config, tensors, branch, 1, toy)
        engine.step([StepEntry("d", a[:25], [])])
        engine.fork("d", "e")
        logits = engine.step([StepEntry("d", a[25:], list(range(15))),
                              StepEntry("e", c[:9], list(range(9)))]).cpu().double().numpy()
        assert np.abs(logits[:15] - reference["a"][25:]).max() < 5e-5
        assert np.abs(logits[15:] - expected[25:]).max() < 5e-5
        engine.check()
    finally:
        unregister_part("mixer", "running_mean")


# ------------------------------------- a routed feed-forward, another position encoding
class Top1Experts:
    """Every token goes through the one expert its router logit is largest for
    (the first of equal ones): out = gelu(x W_in[e]^T) W_out[e]^T. Router
    logits in float32. Dense torch operations only (every expert runs on every
    token and a one-hot mask picks), so the part can sit inside a captured
    graph; it stands for a feed-forward somebody else wrote."""

    def __init__(self, spec, weights, runtime):
        take = lambda name: weights.take(spec[name]).to(runtime.device, torch.float32)
        self.router, self.w_in, self.w_out = take("router"), take("w_in"), take("w_out")
        self.dtype = runtime.dtype

    def forward(self, x, ctx):
        x32 = x.float()
        chosen = torch.argmax(x32 @ self.router.t(), dim=-1)                    # [tokens]
        mask = torch.nn.functional.one_hot(chosen, self.router.shape[0]).float()  # [tokens, experts]
        hidden = torch.nn.functional.gelu(torch.einsum("th,eih->tei", x32, self.w_in))
        out = torch.einsum("tei,ehi->teh", hidden, self.w_out)
        return (out * mask[:, :, None]).sum(dim=1).to(self.dtype)


class PairwiseRotary:
    """Rotates the pairs (2i, 2i + 1) of every head by position * theta^(-2i/d):
    the interleaved convention, unlike the engine's own rotate-half part. It
    offers no tables for the fused kernel, so the attention mixer calls
    ``apply``; torch operations only."""

    def __init__(self, spec, weights, runtime):
        self.head_dim = spec["head_dim"]
        index = torch.arange(self.head_dim // 2, device=runtime.device, dtype=torch.float64)
        self.frequency = float(spec["theta"]) ** (-2.0 * index / self.head_dim)   # made once: nothing is built while a graph is captured

    def apply(self, q, k, positions):
        def rotate(x):
            tokens = x.shape[0]
            heads = x.shape[1] // self.head_dim
            pairs = x.float().view(tokens, heads, self.head_dim // 2, 2)
            angle = positions.double()[:, None] * self.frequency[None, :]
            cos, sin = torch.cos(angle).float()[:, None, :], torch.sin(angle).float()[:, None, :]
            even, odd = pairs[..., 0], pairs[..., 1]
            out = torch.stack([even * cos - odd * sin, odd * cos + even * sin], dim=-1)
            return out.view(tokens, heads, self.head_dim).to(x.dtype)
        return rotate(q), rotate(k)


def plain_with_toy_parts(config, tensors, ids, toy):
    """The plain model with layer 0's feed-forward replaced by the top-1
    experts and layer 2's rotation by the pairwise one."""
    w = {k: v.astype(np.float64) for k, v in tensors.items()}
    x = plain.embed(w["model.embed_tokens.weight"], ids)
    eps = plain.f32(config["rms_norm_eps"])
    positions = np.arange(len(ids))
    heads, kv_heads, hd = config["num_attention_heads"], config["num_key_value_heads"], config["head_dim"]

    def pairwise(v):
        index = np.arange(hd // 2, dtype=np.float64)
        angle = positions[:, None] * toy["theta"] ** (-2.0 * index / hd)[None, :]
        cos, sin = np.cos(angle)[:, None, :], np.sin(angle)[:, None, :]
        out = np.empty_like(v)
        out[..., 0::2] = v[..., 0::2] * cos - v[..., 1::2] * sin
        out[..., 1::2] = v[..., 1::2] * cos + v[..., 0::2] * sin
        return out

    for layer in range(config["num_hidden_layers"]):
        base = f"model.layers.{layer}"
        attention_in = plain.rms_norm(x, w[f"{base}.input_layernorm.weight"], eps)
        if layer == 2:
            tokens = len(ids)
            q = (attention_in @ w[f"{base}.self_attn.q_proj.weight"].T).reshape(tokens, heads, hd)
            k = (attention_in @ w[f"{base}.self_attn.k_proj.weight"].T).reshape(tokens, kv_heads, hd)
            v = (attention_in @ w[f"{base}.self_attn.v_proj.weight"].T).reshape(tokens, kv_heads, hd)
            q = pairwise(plain.rms_norm(q, w[f"{base}.self_attn.q_norm.weight"], eps))
            k = pairwise(plain.rms_norm(k, w[f"{base}.self_attn.k_norm.weight"], eps))
            mixed = plain.causal_gqa_attention(q, k, v, hd ** -0.5).reshape(tokens, heads * hd)
            residual = x + mixed @ w[f"{base}.self_attn.o_proj.weight"].T
        else:
            residual = x + plain.attention_block(attention_in, positions, w, f"{base}.self_attn", config)
        mlp_in = plain.rms_norm(residual, w[f"{base}.post_attention_layernorm.weight"], eps)
        if layer == 0:
            chosen = np.argmax((mlp_in @ toy["router"].T).astype(np.float32), axis=-1)
            out = np.zeros_like(mlp_in)
            for t, e in enumerate(chosen):
                h = mlp_in[t] @ toy["w_in"][e].T
                h = 0.5 * h * (1.0 + np.vectorize(__import__("math").erf)(h / np.sqrt(2.0)))
                out[t] = h @ toy["w_out"][e].T
            x = residual + out
        else:
            x = residual + plain.swiglu(mlp_in, w[f"{base}.mlp.gate_proj.weight"], w[f"{base}.mlp.up_proj.weight"],
                                        w[f"{base}.mlp.down_proj.weight"])
    normed = plain.rms_norm(x, w["model.norm.weight"], eps)
    return normed @ w["lm_head.weight"].T


def test_a_routed_feed_forward_and_another_position_encoding(model_folders):
    """Parts defined here: a feed-forward with routing in layer 0 (the other
    layers keep SwiGLU) and a position encoding of another convention in layer
    2's attention (which then runs its norm, rotation and cache write as
    separate calls). Registered, built and stepped, whole, in portions and
    token by token through the captured decode graph, without a change to the
    framework's files."""
    from metallix_b200.config import PartSpec, Qwen3Config
    from metallix_b200.engine import Engine, StepEntry
    from metallix_b200.parts import register_part, unregister_part
    from metallix_b200.weights import load_tensors
    folder, config, tensors, page = model_folders["B"]
    typed = Qwen3Config.from_dict(config)
    register_part("feed_forward", "top1_experts", Top1Experts)
    register_part("position", "pairwise_rotary", PairwiseRotary)
    try:
        rng = np.random.default_rng(12)
        toy = {"router": rng.normal(size=(4, 96)), "w_in": rng.normal(size=(4, 40, 96)) * 0.1,
               "w_out": rng.normal(size=(4, 96, 40)) * 0.1, "theta": 500.0}
        base = typed.to_model_spec()
        layers = list(base.layers)
        layers[0] = dataclasses.replace(layers[0], feed_forward=PartSpec("top1_experts", {
            "router": "toy.router", "w_in": "toy.w_in", "w_out": "toy.w_out"}))
        mixer = dict(layers[2].mixer.params)
        mixer["position"] = PartSpec("pairwise_rotary", {"head_dim": config["head_dim"], "theta": toy["theta"]})
        layers[2] = dataclasses.replace(layers[2], mixer=PartSpec("gqa_attention", mixer))
        spec = dataclasses.replace(base, layers=tuple(layers))
        loaded = load_tensors(folder, typed, device="cuda:0")
        for name in ("router", "w_in", "w_out"):
            loaded[f"toy.{name}"] = torch.tensor(toy[name], dtype=torch.float32, device="cuda:0")
        ids = random_ids(5, 70, config["vocab_size"])
        reference = plain_with_toy_parts(config, tensors, ids, toy)
        engine = Engine(typed, loaded, dtype="float32", page_tokens=page, num_pages=32, spec=spec)
        assert not engine.model.blocks[2].mixer.fused and engine.model.blocks[1].mixer.fused
        whole = engine.step([StepEntry("w", ids, list(range(70)))]).cpu().double().numpy()
        # a token whose two best router logits nearly tie may take the other expert: none does here
        assert np.abs(whole - reference).max() < 5e-5
        engine.release("w")
        seen = [engine.step([StepEntry("p", ids[:23], [22])]), engine.step([StepEntry("p", ids[23:50], [0, 26])])]
        got = np.concatenate([s.cpu().double().numpy() for s in seen])
        assert np.abs(got - reference[[22, 23, 49]]).max() < 5e-5
        assert engine.graphs is not None
        for position in range(50, 70):      # token by token: the captured graph holds the toy parts too
            logits = engine.step([StepEntry("p", [ids[position]], [0])]).cpu().double().numpy()
            assert np.abs(logits[0] - reference[position]).max() < 5e-5, position
        engine.check()
    finally:
        unregister_part("feed_forward", "top1_experts")
        unregister_part("position", "pairwise_rotary")


# ------------------------------------------------------- a norm somebody else wrote
class TorchRMSNorm:
    """RMSNorm in torch operations, with the interface a norm part must have
    and nothing more: it says nothing about summands, so the block must hand
    it the mixer's plain output."""

    def __init__(self, spec, weights, runtime):
        self.weight = weights.take(spec["weight"]).to(runtime.device, torch.float32)
        self.eps = float(spec["eps"])

    def forward(self, x, out_dtype, rows_index=None):
        x = x.float() if rows_index is None else x.float()[rows_index.long()]
        return (x * torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + self.eps) * self.weight).to(out_dtype)

    def add_forward(self, residual, delta, out_dtype):
        assert delta is None or delta.dim() == 2, "a norm that does not add summands was handed some"
        if delta is not None:
            residual += delta.float()
        return self.forward(residual, out_dtype)


def test_a_norm_that_adds_no_summands_gets_the_mixers_plain_output(model_folders):
    """Configuration D in bfloat16: decode steps of the engine's own attention
    leave one summand per head for the engine's own norm to add up; with a
    norm of another kind behind the mixer of layer 0 that layer's mixer gives
    its plain output, and the logits still match the plain implementation."""
    from metallix_b200.config import PartSpec, Qwen3Config
    from metallix_b200.engine import Engine, StepEntry
    from metallix_b200.parts import register_part, unregister_part
    from metallix_b200.weights import load_tensors
    folder, config, tensors, page = model_folders["D"]
    typed = Qwen3Config.from_dict(config)
    register_part("norm", "torch_rmsnorm", TorchRMSNorm)
    try:
        base = typed.to_model_spec()
        layers = list(base.layers)
        own = layers[0].feed_forward_norm
        layers[0] = dataclasses.replace(layers[0], feed_forward_norm=PartSpec("torch_rmsnorm", {
            "weight": own["weight"], "eps": own["eps"]}))
        spec = dataclasses.replace(base, layers=tuple(layers))
        engine = Engine(typed, load_tensors(folder, typed, device="cuda:0"), dtype="bfloat16", page_tokens=page,
                        num_pages=64, spec=spec)
        assert engine.model.blocks[0].mix == engine.model.blocks[0].mixer.forward
        assert engine.model.blocks[1].mix == engine.model.blocks[1].mixer.forward_summands
        ids = {"a": random_ids(21, 90, config["vocab_size"]), "b": random_ids(22, 40, config["vocab_size"])}
        reference = {k: plain.forward_logits(config, tensors, v) for k, v in ids.items()}
        engine.step([StepEntry("a", ids["a"][:70], []), StepEntry("b", ids["b"][:20], [])])
        worst = 0.0
        for step in range(20):
            logits = engine.step([StepEntry("a", [ids["a"][70 + step]], [0]),
                                  StepEntry("b", [ids["b"][20 + step]], [0])]).cpu().double().numpy()
            worst = max(worst, np.abs(logits[0] - reference["a"][70 + step]).max(),
                        np.abs(logits[1] - reference["b"][20 + step]).max())
        engine.check()
        assert worst < 3e-2
    finally:
        unregister_part("norm", "torch_rmsnorm")
