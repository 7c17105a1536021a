"""Each CUDA kernel alone against its plain reference, at sizes other than the
engine tests use: head sizes in steps of 16, head counts and groups of any
size, widths and vocabularies that are no power of two."""
import numpy as np
import pytest
import torch

import plain_qwen3 as plain

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def dev(array, dtype=torch.float32):
    return torch.tensor(np.asarray(array), dtype=dtype, device="cuda")


def rounded(array, dtype):
    """The values a tensor of ``dtype`` holds, as float64 numpy."""
    return torch.tensor(np.asarray(array), dtype=dtype).double().numpy()


def tol(dtype, f32=1e-5, bf16=2e-2):
    return f32 if dtype == torch.float32 else bf16


@pytest.fixture(scope="module")
def ops():
    from metallix_b200 import ops
    ops.require_cuda()
    return ops


# ------------------------------------------------------------------ embedding
@pytest.mark.parametrize("dtype", DTYPES)
def test_embed(ops, dtype):
    rng = np.random.default_rng(0)
    table = rng.normal(size=(331, 72))
    ids = rng.integers(0, 331, size=19)
    out = ops.embed(dev(ids, torch.int32), dev(table, dtype))
    assert out.dtype == torch.float32
    assert np.array_equal(out.cpu().double().numpy(), rounded(table, dtype)[ids])


def test_embed_flags_a_bad_id(ops):
    table = torch.zeros(10, 8, device="cuda")
    ops.embed(torch.tensor([3, 10], dtype=torch.int32, device="cuda"), table)
    with pytest.raises(ops.KernelError, match="token id"):
        ops.check_status("cuda")
    ops.check_status("cuda")  # cleared


# ----------------------------------------------------------------------- norms
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("size", [24, 80, 1000, 3000])
def test_rmsnorm(ops, dtype, size):
    rng = np.random.default_rng(size)
    x = rng.normal(size=(7, size)) * 3
    w = 1 + rng.uniform(-0.1, 0.1, size=size)
    eps = 3e-5
    out = ops.rmsnorm(dev(x), dev(w), eps, dtype)
    ref = plain.rms_norm(rounded(x, torch.float32), rounded(w, torch.float32), eps)
    assert np.abs(out.cpu().double().numpy() - ref).max() < tol(dtype, 2e-6, 4e-2)
    picked = ops.rmsnorm(dev(x), dev(w), eps, dtype, rows_index=dev([5, 0, 5], torch.int32))
    assert torch.equal(picked, out[[5, 0, 5]])


@pytest.mark.parametrize("dtype", DTYPES)
def test_add_rmsnorm_sums_in_float32(ops, dtype):
    rng = np.random.default_rng(1)
    x = rng.normal(size=(5, 136))
    delta = rng.normal(size=(5, 136))
    w = 1 + rng.uniform(-0.1, 0.1, size=136)
    residual = dev(x)
    out = ops.add_rmsnorm(residual, dev(delta, dtype), dev(w), 1e-6, dtype)
    total = rounded(x, torch.float32) + rounded(delta, dtype)
    assert np.abs(residual.cpu().double().numpy() - total).max() < 1e-6   # the sum itself stays float32
    ref = plain.rms_norm(total, rounded(w, torch.float32), 1e-6)
    assert np.abs(out.cpu().double().numpy() - ref).max() < tol(dtype, 2e-6, 2e-2)
    again = dev(x)
    ops.add_(again, dev(delta, dtype))
    assert torch.equal(again, residual)


# ------------------------------------------------- q/k norm, rotation, cache
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, kv_heads, head_dim, rotary", [(5, 5, 16, 16), (6, 2, 48, 48),
                                                              (3, 1, 112, 112), (4, 2, 64, 32),
                                                              (6, 2, 64, 64), (4, 2, 128, 128),
                                                              (2, 1, 256, 256)])
def test_qk_norm_rope_cache(ops, dtype, heads, kv_heads, head_dim, rotary):
    rng = np.random.default_rng(heads * head_dim)
    tokens, page_tokens, pages, theta, eps = 11, 4, 9, 1e4, 1e-5
    width = (heads + 2 * kv_heads) * head_dim
    qkv = rng.normal(size=(tokens, width))
    positions = rng.integers(0, 200, size=tokens)
    slots = rng.permutation(pages * page_tokens)[:tokens]
    slots[3] = -1  # this token writes nothing
    qw, kw = 1 + rng.uniform(-0.1, 0.1, size=(2, head_dim))
    half = rotary // 2
    angle = np.arange(256)[:, None] * theta ** (-2.0 * np.arange(half) / rotary)[None, :]
    qkv_d = dev(qkv, dtype)
    q_out = torch.empty(tokens, heads, head_dim, dtype=dtype, device="cuda")
    cache = torch.zeros(pages, 2, kv_heads, page_tokens, head_dim, dtype=dtype, device="cuda")
    q_size, kv_size = heads * head_dim, kv_heads * head_dim
    ops.qk_norm_rope_cache(qkv_d[:, :q_size], qkv_d[:, q_size:q_size + kv_size], qkv_d[:, q_size + kv_size:],
                           q_out, cache, dev(slots, torch.int32), dev(positions, torch.int32), dev(qw), dev(kw),
                           dev(np.cos(angle)), dev(np.sin(angle)), eps)
    ops.check_status("cuda")
    stored = rounded(qkv, dtype)
    q = stored[:, :q_size].reshape(tokens, heads, head_dim)
    k = stored[:, q_size:q_size + kv_size].reshape(tokens, kv_heads, head_dim)
    v = stored[:, q_size + kv_size:].reshape(tokens, kv_heads, head_dim)

    def norm_rotate(x, w):
        x = plain.rms_norm(x, rounded(w, torch.float32), eps)
        turned = plain.rope_half(x[..., :rotary], positions, theta)
        return np.concatenate([turned, x[..., rotary:]], axis=-1)

    q_ref, k_ref = norm_rotate(q, qw), norm_rotate(k, kw)
    limit = tol(dtype, 5e-6, 3e-2)
    assert np.abs(q_out.cpu().double().numpy() - q_ref).max() < limit
    got = cache.cpu().double().numpy()
    expected = np.zeros_like(got)
    for t in range(tokens):
        if slots[t] < 0:
            continue
        page, row = divmod(int(slots[t]), page_tokens)
        expected[page, 0, :, row] = k_ref[t]
        expected[page, 1, :, row] = v[t]
    assert np.abs(got - expected).max() < limit
    assert np.array_equal(got[:, 1], expected[:, 1])  # values are stored as projected


def test_rotation_keeps_accuracy_at_far_positions(ops):
    """cos and sin come from a float64 table: at position 4000 a float32
    product of position and frequency would already be off by 1e-4."""
    head_dim, theta = 64, 1e6
    positions = np.array([0, 1, 4000, 8191])
    x = np.random.default_rng(2).normal(size=(4, 2 * head_dim))
    angle = np.arange(8192)[:, None] * theta ** (-2.0 * np.arange(head_dim // 2) / head_dim)[None, :]
    out = ops.norm_rotate_heads(dev(x), head_dim, dev(positions, torch.int32), cos=dev(np.cos(angle)),
                                sin=dev(np.sin(angle)))
    ref = plain.rope_half(rounded(x, torch.float32).reshape(4, 2, head_dim), positions, theta)
    assert np.abs(out.cpu().double().numpy() - ref).max() < 2e-6


# ------------------------------------------------------------------ attention
def run_attention(ops, dtype, q, k, v, lengths, page_tokens, scale, window=0, shuffle_seed=0):
    """Several requests; request r's last ``lengths[r][1]`` positions are the
    queries, all ``lengths[r][0]`` positions sit in a cache whose pages are
    handed out in shuffled order."""
    heads, head_dim = q[0].shape[1], q[0].shape[2]
    kv_heads = k[0].shape[1]
    rng = np.random.default_rng(shuffle_seed)
    pages_needed = [-(-total // page_tokens) for total, _ in lengths]
    order = rng.permutation(sum(pages_needed) + 3)
    cache = torch.full((len(order), 2, kv_heads, page_tokens, head_dim), float("nan"), dtype=dtype, device="cuda")
    host_cache = np.zeros(cache.shape)
    width = max(pages_needed)
    tables = np.full((len(lengths), width), -1, dtype=np.int32)
    cursor = 0
    q_rows, positions, tile_request, tile_start, tile_length = [], [], [], [], []
    for r, (total, queries) in enumerate(lengths):
        tables[r, :pages_needed[r]] = order[cursor:cursor + pages_needed[r]]
        cursor += pages_needed[r]
        for p in range(total):
            page, row = tables[r, p // page_tokens], p % page_tokens
            host_cache[page, 0, :, row] = k[r][p]
            host_cache[page, 1, :, row] = v[r][p]
        begin = len(positions)
        q_rows.append(q[r][total - queries:total])
        positions += list(range(total - queries, total))
        for first in range(0, queries, 16):
            tile_request.append(r)
            tile_start.append(begin + first)
            tile_length.append(min(16, queries - first))
    cache.copy_(dev(host_cache, dtype))
    q_all = dev(np.concatenate(q_rows), dtype)
    out = torch.empty_like(q_all)
    ops.paged_attention_tile(q_all, cache, out, dev(tables, torch.int32), dev(tile_request, torch.int32),
                             dev(tile_start, torch.int32), dev(tile_length, torch.int32),
                             dev(positions, torch.int32), scale, window)
    ops.check_status("cuda")
    return out.cpu().double().numpy()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, kv_heads, head_dim, page_tokens", [(4, 4, 16, 4), (6, 2, 48, 8),
                                                                   (5, 1, 80, 16), (8, 2, 128, 32),
                                                                   (2, 1, 256, 16)])
def test_paged_attention_mixed_batch(ops, dtype, heads, kv_heads, head_dim, page_tokens):
    rng = np.random.default_rng(head_dim + heads)
    lengths = [(70, 70), (45, 1), (33, 17), (100, 2), (1, 1)]  # (positions, of which queries)
    q = [rounded(rng.normal(size=(n, heads, head_dim)), dtype) for n, _ in lengths]
    k = [rounded(rng.normal(size=(n, kv_heads, head_dim)), dtype) for n, _ in lengths]
    v = [rounded(rng.normal(size=(n, kv_heads, head_dim)), dtype) for n, _ in lengths]
    scale = head_dim ** -0.5
    out = run_attention(ops, dtype, q, k, v, lengths, page_tokens, scale)
    cursor = 0
    for r, (total, queries) in enumerate(lengths):
        ref = plain.causal_gqa_attention(q[r], k[r], v[r], scale)[total - queries:]
        got = out[cursor:cursor + queries]
        cursor += queries
        assert np.abs(got - ref).max() < tol(dtype, 5e-6, 2e-2), (r, total, queries)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [1, 5, 16, 33])
def test_paged_attention_window(ops, dtype, window):
    rng = np.random.default_rng(window)
    heads, kv_heads, head_dim = 4, 2, 32
    lengths = [(90, 90), (77, 1), (50, 9)]
    q = [rounded(rng.normal(size=(n, heads, head_dim)), dtype) for n, _ in lengths]
    k = [rounded(rng.normal(size=(n, kv_heads, head_dim)), dtype) for n, _ in lengths]
    v = [rounded(rng.normal(size=(n, kv_heads, head_dim)), dtype) for n, _ in lengths]
    out = run_attention(ops, dtype, q, k, v, lengths, 8, 0.25, window=window)
    cursor = 0
    for r, (total, queries) in enumerate(lengths):
        ref = plain.causal_gqa_attention(q[r], k[r], v[r], 0.25, window=window)[total - queries:]
        assert np.abs(out[cursor:cursor + queries] - ref).max() < tol(dtype, 5e-6, 2e-2)
        cursor += queries


@pytest.mark.parametrize("dtype", DTYPES)
def test_one_far_key_among_hundreds(ops, dtype):
    """Random keys would average a lost key away. Here one key matches the
    query so strongly that the output must be that key's value: at the first
    position, around page and tile edges, and at the query itself."""
    heads, kv_heads, head_dim, page_tokens, total = 2, 1, 64, 16, 700
    rng = np.random.default_rng(9)
    for target in (0, 15, 16, 31, 32, 511, 512, 683, 698, 699):
        k = rounded(rng.normal(size=(total, kv_heads, head_dim)) * 0.1, dtype)
        v = rounded(rng.normal(size=(total, kv_heads, head_dim)), dtype)
        q = rounded(rng.normal(size=(total, heads, head_dim)) * 0.1, dtype)
        k[target, 0, :] = 0.0
        k[target, 0, 7] = 16.0
        q[-1, :, 7] = 16.0   # score 256 * scale = 32 above everything else
        out = run_attention(ops, dtype, [q], [k], [v], [(total, 1)], page_tokens, head_dim ** -0.5,
                            shuffle_seed=target)
        assert np.abs(out[0] - v[target, 0]).max() < tol(dtype, 1e-5, 1e-2), target


@pytest.mark.parametrize("dtype", DTYPES)
def test_window_edge(ops, dtype):
    """The strong key sits exactly on the window's edge: one position inside
    it is seen, one position outside it is not."""
    heads, kv_heads, head_dim, total, window = 2, 1, 32, 200, 48
    rng = np.random.default_rng(10)
    k = rounded(rng.normal(size=(total, kv_heads, head_dim)) * 0.1, dtype)
    v = rounded(rng.normal(size=(total, kv_heads, head_dim)), dtype)
    q = rounded(rng.normal(size=(total, heads, head_dim)) * 0.1, dtype)
    q[-1, :, 3] = 16.0
    for target, seen in ((total - window, True), (total - window - 1, False)):
        keys = k.copy()
        keys[target, 0, :] = 0.0
        keys[target, 0, 3] = 16.0
        out = run_attention(ops, dtype, [q], [keys], [v], [(total, 1)], 16, head_dim ** -0.5, window=window)
        near = np.abs(out[0] - v[target, 0]).max() < 1e-2
        assert near == seen, (target, seen)


def test_attention_does_not_depend_on_the_cut(ops):
    """float32: the same query gives the same bits alone, in a tile of 16 and
    beside other requests."""
    rng = np.random.default_rng(11)
    heads, kv_heads, head_dim, total = 3, 1, 48, 130
    q = [rng.normal(size=(total, heads, head_dim))]
    k = [rng.normal(size=(total, kv_heads, head_dim))]
    v = [rng.normal(size=(total, kv_heads, head_dim))]
    whole = run_attention(ops, torch.float32, q, k, v, [(total, total)], 8, 0.3)
    last = run_attention(ops, torch.float32, q, k, v, [(total, 1)], 8, 0.3, shuffle_seed=5)
    part = run_attention(ops, torch.float32, q + q, k + k, v + v, [(total, 37), (total - 9, 3)], 8, 0.3,
                         shuffle_seed=6)
    assert np.array_equal(last[0], whole[-1])
    assert np.array_equal(part[:37], whole[-37:])
    assert np.array_equal(part[37:], whole[total - 12:total - 9])


def run_flash(ops, q, k, v, lengths, page_tokens, scale, window=0, seed=0, kernel="mma", tile=128):
    """A tensor-core prompt kernel ("mma": warp-level, "tcgen05": TMA and
    tensor memory) on requests whose last ``queries`` positions are the
    queries (bfloat16), cut into tiles of up to ``tile`` tokens."""
    dtype = torch.bfloat16
    heads, head_dim, kv_heads = q[0].shape[1], q[0].shape[2], k[0].shape[1]
    rng = np.random.default_rng(seed)
    pages_needed = [-(-total // page_tokens) for total, _ in lengths]
    order = rng.permutation(sum(pages_needed) + 3)
    # what no request wrote (free pages, the rest of a last page) is NaN: nothing may be asked of it
    host_cache = np.full((len(order), 2, kv_heads, page_tokens, head_dim), np.nan)
    tables = np.full((len(lengths), max(pages_needed)), -1, dtype=np.int32)
    cursor = 0
    q_rows, positions, tiles = [], [], []
    for r, (total, queries) in enumerate(lengths):
        tables[r, :pages_needed[r]] = order[cursor:cursor + pages_needed[r]]
        cursor += pages_needed[r]
        for p in range(total):
            host_cache[tables[r, p // page_tokens], 0, :, p % page_tokens] = k[r][p]
            host_cache[tables[r, p // page_tokens], 1, :, p % page_tokens] = v[r][p]
        begin = len(positions)
        q_rows.append(q[r][total - queries:total])
        positions += list(range(total - queries, total))
        for first in range(0, queries, tile):
            tiles.append((r, begin + first, min(tile, queries - first)))
    q_all = dev(np.concatenate(q_rows), dtype)
    out = torch.full_like(q_all, float("nan"))
    ops.flash_prefill(q_all, dev(host_cache, dtype), out, dev(tables, torch.int32),
                      dev([t[0] for t in tiles], torch.int32), dev([t[1] for t in tiles], torch.int32),
                      dev([t[2] for t in tiles], torch.int32), dev(positions, torch.int32), scale, window,
                      kernel=kernel)
    ops.check_status("cuda")
    return out.cpu().double().numpy()


FLASH_KERNELS = ("mma", "tcgen05")


@pytest.mark.parametrize("kernel", FLASH_KERNELS)
@pytest.mark.parametrize("heads, kv_heads, head_dim, page_tokens", [(2, 2, 64, 16), (6, 2, 64, 4),
                                                                   (4, 2, 128, 16), (3, 1, 128, 32),
                                                                   (5, 1, 128, 8), (2, 1, 64, 128)])
def test_flash_prefill(ops, heads, kv_heads, head_dim, page_tokens, kernel):
    rng = np.random.default_rng(heads * head_dim + 1)
    dtype = torch.bfloat16
    if kernel == "tcgen05" and page_tokens == 4:
        assert not ops.flash_prefill_tcgen05_supported(head_dim, heads, kv_heads, page_tokens, dtype)
        pytest.skip("a page of 4 tokens does not fill a swizzle group: the warp-level kernel takes it")
    lengths = [(200, 200), (130, 2), (64, 64), (333, 70), (65, 65), (500, 129), (3, 3), (1000, 300)]
    q = [rounded(rng.normal(size=(n, heads, head_dim)), dtype) for n, _ in lengths]
    k = [rounded(rng.normal(size=(n, kv_heads, head_dim)), dtype) for n, _ in lengths]
    v = [rounded(rng.normal(size=(n, kv_heads, head_dim)), dtype) for n, _ in lengths]
    scale = head_dim ** -0.5
    assert ops.flash_prefill_supported(head_dim, heads, kv_heads, dtype)
    for window in (0, 1, 50, 64, 200):
        out = run_flash(ops, q, k, v, lengths, page_tokens, scale, window=window, kernel=kernel,
                        tile=128 if window != 50 else 50)
        cursor = 0
        for r, (total, queries) in enumerate(lengths):
            ref = plain.causal_gqa_attention(q[r], k[r], v[r], scale, window=window or None)[total - queries:]
            assert np.abs(out[cursor:cursor + queries] - ref).max() < 2e-2, (window, r)
            cursor += queries
    assert not ops.flash_prefill_supported(head_dim, heads, kv_heads, torch.float32)
    assert not ops.flash_prefill_supported(48, 3, 1, dtype)


@pytest.mark.parametrize("kernel", FLASH_KERNELS)
def test_flash_prefill_one_far_key_and_cuts(ops, kernel):
    heads, kv_heads, head_dim, total = 4, 2, 128, 700
    dtype = torch.bfloat16
    rng = np.random.default_rng(31)
    for target in (0, 15, 16, 63, 64, 65, 127, 128, 511, 512, 640, 698, 699):
        k = rounded(rng.normal(size=(total, kv_heads, head_dim)) * 0.1, dtype)
        v = rounded(rng.normal(size=(total, kv_heads, head_dim)), dtype)
        q = rounded(rng.normal(size=(total, heads, head_dim)) * 0.1, dtype)
        k[target, :, :] = 0.0
        k[target, :, 5] = 16.0
        q[-1, :, 5] = 16.0
        out = run_flash(ops, [q], [k], [v], [(total, 40)], 16, head_dim ** -0.5, seed=target, kernel=kernel)
        for head in range(heads):
            assert np.abs(out[-1, head] - v[target, head // 2]).max() < 1e-2, (target, head)
    # the same positions whole, as a portion after cached keys, and beside another request
    q = [rounded(rng.normal(size=(300, heads, head_dim)), dtype)]
    k = [rounded(rng.normal(size=(300, kv_heads, head_dim)), dtype)]
    v = [rounded(rng.normal(size=(300, kv_heads, head_dim)), dtype)]
    whole = run_flash(ops, q, k, v, [(300, 300)], 16, 0.09, kernel=kernel)
    part = run_flash(ops, q + q, k + k, v + v, [(300, 77), (250, 5)], 16, 0.09, seed=3, kernel=kernel)
    assert np.array_equal(part[:77], whole[-77:])
    assert np.array_equal(part[77:], whole[245:250])


@pytest.mark.parametrize("shares", [2, 3, 5])
def test_flash_prefill_with_a_tile_s_keys_shared_out(ops, shares):
    """Several blocks take a query tile's key tiles between them and a second
    kernel puts their results together; a tile with fewer key tiles than
    blocks leaves some of them empty-handed."""
    heads, kv_heads, head_dim, page_tokens = 4, 2, 128, 16
    dtype = torch.bfloat16
    rng = np.random.default_rng(shares)
    lengths = [(1500, 200), (130, 130), (700, 3), (40, 40), (1000, 260)]
    q = [rounded(rng.normal(size=(n, heads, head_dim)), dtype) for n, _ in lengths]
    k = [rounded(rng.normal(size=(n, kv_heads, head_dim)), dtype) for n, _ in lengths]
    v = [rounded(rng.normal(size=(n, kv_heads, head_dim)), dtype) for n, _ in lengths]
    scale = head_dim ** -0.5
    assert ops.flash_key_shares(64, 4096) == 2 and ops.flash_key_shares(64, 1000) == 1
    assert ops.flash_key_shares(16, 8192) == 8 and ops.flash_key_shares(256, 8192) == 1
    assert ops.flash_key_shares(16, 8192, window=1024) == 1
    try:
        for window in (0, 300):
            ops.KEY_SHARES = None
            alone = run_flash(ops, q, k, v, lengths, page_tokens, scale, window=window, kernel="tcgen05")
            ops.KEY_SHARES = shares
            shared = run_flash(ops, q, k, v, lengths, page_tokens, scale, window=window, kernel="tcgen05")
            cursor = 0
            for r, (total, queries) in enumerate(lengths):
                ref = plain.causal_gqa_attention(q[r], k[r], v[r], scale, window=window or None)[total - queries:]
                assert np.abs(shared[cursor:cursor + queries] - ref).max() < 2e-2, (window, r)
                cursor += queries
            assert np.abs(shared - alone).max() < 1e-2
    finally:
        ops.KEY_SHARES = None


def run_decode_attention(ops, dtype, q, k, v, totals, page_tokens, scale, window=0, pad_rows=0, seed=0,
                         project=None):
    """One query (the last position) per request through the split-key kernel;
    with ``project`` (a weight on the device) through the kernel that also
    projects: the summands [heads, tokens, hidden] then."""
    heads, head_dim, kv_heads = q[0].shape[1], q[0].shape[2], k[0].shape[1]
    rng = np.random.default_rng(seed)
    pages_needed = [-(-total // page_tokens) for total in totals]
    order = rng.permutation(sum(pages_needed) + 2)
    # what no request wrote (free pages, the rest of a last page) is NaN: nothing may be asked of it
    host_cache = np.full((len(order), 2, kv_heads, page_tokens, head_dim), np.nan)
    tables = np.full((len(totals), max(pages_needed)), -1, dtype=np.int32)
    cursor = 0
    for r, total in enumerate(totals):
        tables[r, :pages_needed[r]] = order[cursor:cursor + pages_needed[r]]
        cursor += pages_needed[r]
        for p in range(total):
            host_cache[tables[r, p // page_tokens], 0, :, p % page_tokens] = k[r][p]
            host_cache[tables[r, p // page_tokens], 1, :, p % page_tokens] = v[r][p]
    q_all = dev(np.stack([q[r][total - 1] for r, total in enumerate(totals)]), dtype)
    out = torch.full_like(q_all, float("nan"))
    rows = list(range(len(totals))) + [-1] * pad_rows
    if project is not None:
        summands = ops.paged_attention_decode_project(
            q_all, dev(host_cache, dtype), dev(tables, torch.int32), dev(rows, torch.int32),
            dev([max(r, 0) for r in rows], torch.int32), dev([t - 1 for t in totals], torch.int32), scale,
            max(totals) + 300, project, window)
        ops.check_status("cuda")
        return summands.cpu().double().numpy()
    ops.paged_attention_decode(q_all, dev(host_cache, dtype), out, dev(tables, torch.int32),
                               dev(rows, torch.int32), dev([max(r, 0) for r in rows], torch.int32),
                               dev([t - 1 for t in totals], torch.int32), scale, max(totals) + 300, window)
    ops.check_status("cuda")
    return out.cpu().double().numpy()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, kv_heads, head_dim, page_tokens", [(2, 2, 64, 16), (6, 2, 64, 8),
                                                                   (4, 2, 128, 16), (8, 1, 128, 32),
                                                                   (5, 1, 128, 4)])
def test_split_key_decode_attention(ops, dtype, heads, kv_heads, head_dim, page_tokens):
    rng = np.random.default_rng(heads + head_dim)
    totals = [1, 255, 256, 257, 700, 33, 512, 1030]
    q = [rounded(rng.normal(size=(n, heads, head_dim)), dtype) for n in totals]
    k = [rounded(rng.normal(size=(n, kv_heads, head_dim)), dtype) for n in totals]
    v = [rounded(rng.normal(size=(n, kv_heads, head_dim)), dtype) for n in totals]
    scale = head_dim ** -0.5
    assert ops.decode_attention_supported(head_dim, heads, kv_heads, dtype)
    out = run_decode_attention(ops, dtype, q, k, v, totals, page_tokens, scale, pad_rows=3)
    for r, total in enumerate(totals):
        ref = plain.causal_gqa_attention(q[r], k[r], v[r], scale)[-1]
        assert np.abs(out[r] - ref).max() < tol(dtype, 5e-6, 2e-2), (r, total)
    for window in (1, 100, 256, 300):
        out = run_decode_attention(ops, dtype, q, k, v, totals, page_tokens, scale, window=window)
        for r, total in enumerate(totals):
            ref = plain.causal_gqa_attention(q[r], k[r], v[r], scale, window=window)[-1]
            assert np.abs(out[r] - ref).max() < tol(dtype, 5e-6, 2e-2), (window, r, total)


@pytest.mark.parametrize("resident", [0, 444, 120, 12])
@pytest.mark.parametrize("heads, kv_heads, head_dim, page_tokens", [(6, 2, 64, 8), (4, 2, 128, 16), (16, 2, 128, 128)])
def test_decode_attention_with_blocks_that_walk_over_tiles(ops, resident, heads, kv_heads, head_dim, page_tokens):
    """The bfloat16 kernel with one block per 128-key tile (0) and with as many
    blocks per (token, key/value head) as keep the grid resident, each walking
    over its tiles (18 blocks of one to two tiles, 5 blocks of up to seven, and
    a step cut into more blocks than are resident):
    the same attention. Lengths around the edges of tiles and of a block's
    rounds; a far key that only one block sees; windows that move the first
    tile."""
    rng = np.random.default_rng(resident + heads)
    totals = [1, 128, 129, 1024, 1025, 2047, 2049, 2176, 3000, 4097]
    dtype = torch.bfloat16
    q = [rounded(rng.normal(size=(1, heads, head_dim)), dtype) for n in totals]
    k = [rounded(rng.normal(size=(n, kv_heads, head_dim)), dtype) for n in totals]
    v = [rounded(rng.normal(size=(n, kv_heads, head_dim)), dtype) for n in totals]
    far = {2176: 3, 3000: 2500, 4097: 1030}     # request length -> position of a key that takes all the weight
    for r, total in enumerate(totals):
        if total in far:
            k[r][far[total], :, :] = 0.0
            k[r][far[total], :, 5] = 24.0
            q[r][0, :, :] = 0.0
            q[r][0, :, 5] = 24.0
    scale = head_dim ** -0.5
    full_q = [np.concatenate([np.zeros((n - 1, heads, head_dim)), q[r]]) for r, n in enumerate(totals)]
    try:
        ops.set_decode_resident_blocks(resident, 48 if resident == 12 else 2048)   # 12: 24 pairs exceed it, 48 / 24 = 2 blocks each
        for window in (0, 200, 1500):
            out = run_decode_attention(ops, dtype, full_q, k, v, totals, page_tokens, scale, window=window, pad_rows=2)
            for r, total in enumerate(totals):
                first = max(0, total - window) if window else 0
                ref = plain_last_row(q[r][0], k[r][first:], v[r][first:], scale)
                assert np.abs(out[r] - ref).max() < 2e-2, (resident, window, total)
                if total in far and (not window or far[total] >= first):
                    assert np.abs(out[r] - v[r][far[total]].repeat(heads // kv_heads, axis=0)).max() < 1e-2
    finally:
        ops.set_decode_resident_blocks(444)


@pytest.mark.parametrize("resident", [0, 444, 12])
@pytest.mark.parametrize("heads, kv_heads, head_dim, page_tokens, hidden, totals", [
    (6, 2, 64, 8, 200, [1, 128, 129, 1025, 3000]),                 # a width that is no multiple of the 128 columns of a block
    (4, 2, 128, 16, 384, [5, 2049, 700, 4097, 130, 2176, 64, 1, 999, 1024, 300, 4500, 77]),   # 13 tokens: two blocks of eight
    (16, 8, 128, 32, 1024, [2048] * 8),
    (2, 1, 128, 16, 136, [300 + 7 * i for i in range(33)]),                   # 33 tokens: five blocks of eight
    (6, 2, 64, 16, 72, [40 + 29 * i for i in range(64)])])                    # 64 tokens
def test_decode_attention_with_the_output_projection(ops, resident, heads, kv_heads, head_dim, page_tokens, hidden,
                                                     totals):
    """The kernel that puts a decode step's splits together and projects them
    head by head: summand h is (the attention output of head h, as the merge
    kernel rounds it to bfloat16) times W_o's columns of that head, summed in
    float32; tokens that no row names give zeros; with one block per tile and
    with blocks that walk over tiles, with and without a window."""
    rng = np.random.default_rng(resident + heads)
    dtype = torch.bfloat16
    q = [rounded(rng.normal(size=(1, heads, head_dim)), dtype) for n in totals]
    k = [rounded(rng.normal(size=(n, kv_heads, head_dim)), dtype) for n in totals]
    v = [rounded(rng.normal(size=(n, kv_heads, head_dim)), dtype) for n in totals]
    full_q = [np.concatenate([np.zeros((n - 1, heads, head_dim)), q[r]]) for r, n in enumerate(totals)]
    weight = rounded(rng.normal(size=(hidden, heads * head_dim)), dtype)
    scale = head_dim ** -0.5
    assert ops.decode_project_supported(head_dim, heads, kv_heads, dtype, len(totals), dev(weight, dtype))
    try:
        ops.set_decode_resident_blocks(resident, 48 if resident == 12 else 2048)
        for window in (0, 1500):
            out = run_decode_attention(ops, dtype, full_q, k, v, totals, page_tokens, scale, window=window, pad_rows=2)
            summands = run_decode_attention(ops, dtype, full_q, k, v, totals, page_tokens, scale, window=window,
                                            pad_rows=2, project=dev(weight, dtype))
            assert summands.shape == (heads, len(totals), hidden)
            for head in range(heads):
                expected = out[:, head, :] @ weight[:, head * head_dim:(head + 1) * head_dim].T
                assert np.abs(summands[head] - expected).max() < 2e-5 * np.abs(expected).max(), (window, head)
    finally:
        ops.set_decode_resident_blocks(444)


def test_decode_projection_refusals_and_tokens_without_a_row(ops):
    dtype = torch.bfloat16
    weight = dev(np.ones((96, 256)), dtype)
    assert not ops.decode_project_supported(128, 2, 1, dtype, 65, weight)          # more than 64 tokens
    assert not ops.decode_project_supported(128, 2, 1, torch.float32, 4, weight)   # bfloat16 only
    assert not ops.decode_project_supported(256, 1, 1, dtype, 4, weight)           # heads of 64 or 128 values
    assert not ops.decode_project_supported(128, 2, 1, dtype, 4, weight[:, 4:])    # rows that no bulk copy can fetch
    # three tokens, the middle one named by no row: its summands are zeros
    q = torch.randn(3, 2, 128, device="cuda").to(dtype)
    cache = torch.randn(4, 2, 1, 16, 128, device="cuda").to(dtype)
    tables = dev([[0, 1], [2, 3], [1, 0]], torch.int32)
    summands = ops.paged_attention_decode_project(q, cache, tables, dev([0, -1, 2], torch.int32),
                                                  dev([0, 0, 2], torch.int32), dev([20, 0, 31], torch.int32), 0.1, 32,
                                                  weight)
    ops.check_status("cuda")
    assert torch.all(summands[:, 1] == 0) and torch.all(summands[:, 0] != 0) and torch.all(summands[:, 2] != 0)


@pytest.mark.parametrize("rows, size, parts", [(8, 1024, 16), (3, 200, 5), (5, 331, 3), (16, 96, 1)])
@pytest.mark.parametrize("out_dtype", DTYPES)
def test_add_rmsnorm_of_summands(ops, rows, size, parts, out_dtype):
    """x += the sum of the parts, then the norm; widths with and without the
    four-values-a-thread kernel."""
    rng = np.random.default_rng(rows + size)
    x = rng.normal(size=(rows, size))
    summands = rng.normal(size=(parts, rows, size))
    weight = 1 + 0.1 * rng.normal(size=size)
    x_dev = dev(x, torch.float32)
    out = ops.add_rmsnorm(x_dev, dev(summands, torch.float32), dev(weight, torch.float32), 1e-5, out_dtype)
    total = x.astype(np.float32).astype(np.float64) + summands.astype(np.float32).astype(np.float64).sum(axis=0)
    assert np.abs(x_dev.cpu().double().numpy() - total).max() < 1e-5
    expected = plain.rms_norm(total, weight.astype(np.float32).astype(np.float64), 1e-5)
    assert np.abs(out.cpu().double().numpy() - expected).max() < tol(out_dtype, 1e-5, 2e-2)


def plain_last_row(q, k, v, scale):
    """Attention of one query [heads, hd] over all of k, v [n, kv_heads, hd]."""
    heads, group = q.shape[0], q.shape[0] // k.shape[1]
    out = np.zeros_like(q)
    for head in range(heads):
        scores = (k[:, head // group, :] @ q[head]) * scale
        weights = np.exp(scores - scores.max())
        out[head] = (weights / weights.sum()) @ v[:, head // group, :]
    return out


def test_split_key_decode_bfloat16_head_dim_256_and_refusals(ops):
    rng = np.random.default_rng(21)
    totals = [300, 17]
    q = [rounded(rng.normal(size=(n, 2, 256)), torch.bfloat16) for n in totals]
    k = [rounded(rng.normal(size=(n, 1, 256)), torch.bfloat16) for n in totals]
    v = [rounded(rng.normal(size=(n, 1, 256)), torch.bfloat16) for n in totals]
    out = run_decode_attention(ops, torch.bfloat16, q, k, v, totals, 16, 1 / 16)
    for r in range(2):
        assert np.abs(out[r] - plain.causal_gqa_attention(q[r], k[r], v[r], 1 / 16)[-1]).max() < 2e-2
    assert not ops.decode_attention_supported(48, 3, 1, torch.bfloat16)    # the caller takes the general kernel
    assert not ops.decode_attention_supported(256, 2, 1, torch.float32)
    assert not ops.decode_attention_supported(128, 16, 1, torch.bfloat16)  # 16 query heads per key/value head
    with pytest.raises(ops.KernelError, match="does not take"):
        ops.paged_attention_decode(torch.zeros(1, 3, 48, device="cuda"), torch.zeros(2, 2, 1, 4, 48, device="cuda"),
                                   torch.zeros(1, 3, 48, device="cuda"),
                                   torch.zeros(1, 1, dtype=torch.int32, device="cuda"),
                                   torch.zeros(1, dtype=torch.int32, device="cuda"),
                                   torch.zeros(1, dtype=torch.int32, device="cuda"),
                                   torch.zeros(1, dtype=torch.int32, device="cuda"), 1.0, 4)


@pytest.mark.parametrize("dtype", DTYPES)
def test_split_key_decode_one_far_key(ops, dtype):
    heads, kv_heads, head_dim, total = 4, 2, 128, 1500
    rng = np.random.default_rng(22)
    for target in (0, 15, 16, 255, 256, 257, 1023, 1024, 1279, 1280, 1498, 1499):
        k = rounded(rng.normal(size=(total, kv_heads, head_dim)) * 0.1, dtype)
        v = rounded(rng.normal(size=(total, kv_heads, head_dim)), dtype)
        q = rounded(rng.normal(size=(total, heads, head_dim)) * 0.1, dtype)
        k[target, :, :] = 0.0
        k[target, :, 9] = 16.0
        q[-1, :, 9] = 16.0
        out = run_decode_attention(ops, dtype, [q], [k], [v], [total], 16, head_dim ** -0.5, seed=target)
        for head in range(heads):
            assert np.abs(out[0, head] - v[target, head // 2]).max() < tol(dtype, 1e-5, 1e-2), (target, head)


def test_split_key_decode_does_not_depend_on_the_batch(ops):
    rng = np.random.default_rng(23)
    totals = [900, 40, 300]
    q = [rng.normal(size=(n, 4, 64)) for n in totals]
    k = [rng.normal(size=(n, 2, 64)) for n in totals]
    v = [rng.normal(size=(n, 2, 64)) for n in totals]
    together = run_decode_attention(ops, torch.float32, q, k, v, totals, 16, 0.125, pad_rows=5)
    for r in range(3):
        alone = run_decode_attention(ops, torch.float32, [q[r]], [k[r]], [v[r]], [totals[r]], 16, 0.125, seed=r + 1)
        assert np.array_equal(alone[0], together[r])


def test_attention_flags_a_bad_page(ops):
    q = torch.zeros(1, 1, 16, device="cuda")
    cache = torch.zeros(2, 2, 1, 4, 16, device="cuda")
    table = torch.tensor([[0, 7]], dtype=torch.int32, device="cuda")
    one = torch.tensor([0], dtype=torch.int32, device="cuda")
    ops.paged_attention_tile(q, cache, torch.empty_like(q), table, one, one, one + 0,
                             torch.tensor([5], dtype=torch.int32, device="cuda"), 1.0)
    with pytest.raises(ops.KernelError, match="block-table"):
        ops.check_status("cuda")


# ------------------------------------------------------------ matrix products
@pytest.mark.parametrize("m, n, k", [(1, 331, 80), (7, 96, 224), (64, 200, 72), (130, 65, 1000)])
def test_gemm_simple_float32_is_true_32_bit(ops, m, n, k):
    rng = np.random.default_rng(m + n)
    a, w = rng.normal(size=(m, k)), rng.normal(size=(n, k))
    out = ops.gemm_simple(dev(a), dev(w))
    ref = rounded(a, torch.float32) @ rounded(w, torch.float32).T
    # float32 products and sums leave a relative error near 1e-7; a
    # reduced-precision matrix mode (10 mantissa bits) would leave about 3e-4
    error = out.cpu().double().numpy() - ref
    assert np.sqrt((error ** 2).mean() / (ref ** 2).mean()) < 1e-6
    one_row = ops.gemm_simple(dev(a[3:4] if m > 3 else a[:1]), dev(w))
    assert torch.equal(one_row[0], out[3 if m > 3 else 0])   # a row does not depend on the batch


@pytest.mark.parametrize("backend", ["simple", "cublas", "auto", "tcgen05"])
@pytest.mark.parametrize("m, n, k", [(1, 384, 96), (5, 200, 136), (64, 331, 80), (300, 448, 192),
                                     (129, 130, 72), (700, 1030, 520)])
def test_gemm_bf16(ops, backend, m, n, k):
    rng = np.random.default_rng(n)
    a, w = rng.normal(size=(m, k)), rng.normal(size=(n, k))
    ref = rounded(a, torch.bfloat16) @ rounded(w, torch.bfloat16).T
    out32 = ops.gemm_bf16(dev(a, torch.bfloat16), dev(w, torch.bfloat16), torch.float32, backend=backend)
    assert out32.dtype == torch.float32
    assert np.abs(out32.cpu().double().numpy() - ref).max() < 1e-3
    out16 = ops.gemm_bf16(dev(a, torch.bfloat16), dev(w, torch.bfloat16), torch.bfloat16, backend=backend)
    assert np.abs(out16.cpu().double().numpy() - ref).max() < 0.02 * np.abs(ref).max()


@pytest.mark.parametrize("kernel", ["load", "stream"])
@pytest.mark.parametrize("m", [1, 3, 8, 9, 16, 31, 64])
@pytest.mark.parametrize("n, k", [(331, 96), (1024, 3072), (40, 32), (4096, 1024), (200, 6144), (136, 48)])
def test_gemm_skinny(ops, m, n, k, kernel):
    """Both weight-streaming kernels: "load" (16-byte loads into registers, up
    to 64 rows, k a multiple of 32) and "stream" (bulk copies into shared
    memory, up to 16 rows, k a multiple of 16)."""
    rng = np.random.default_rng(m + n)
    a, w = rng.normal(size=(m, k)), rng.normal(size=(n, k)) * 0.05
    a_d, w_d = dev(a, torch.bfloat16), dev(w, torch.bfloat16)
    if kernel == "stream":
        # at most 16 rows, and 8 rows of w beside the 8 or 16 rows of a within 200 KiB of shared memory
        takes = m <= 16 and (8 + (8 if m <= 8 else 16)) * (2 * k + 16) <= 200 * 1024
        assert ops.gemm_stream_supported(a_d, w_d) == takes
        if not takes:
            with pytest.raises(ops.KernelError, match="bulk-copy kernel"):
                ops.gemm_skinny(a_d, w_d, kernel="stream")
            return
    else:
        assert ops.gemm_skinny_supported(a_d, w_d) == (k % 32 == 0)
        if k % 32:
            return
    ref = rounded(a, torch.bfloat16) @ rounded(w, torch.bfloat16).T
    out32 = ops.gemm_skinny(a_d, w_d, torch.float32, kernel=kernel)
    ops.check_status("cuda")
    assert np.abs(out32.cpu().double().numpy() - ref).max() < 1e-4 * np.sqrt(k / 32)
    out16 = ops.gemm_skinny(a_d, w_d, torch.bfloat16, kernel=kernel)
    assert (np.abs(out16.cpu().double().numpy() - ref) <= 2.0 ** -8 * np.abs(ref) + 1e-4).all()
    # a row's result does not depend on how many other rows ride along
    alone = ops.gemm_skinny(a_d[m - 1:m].contiguous(), w_d, torch.float32, kernel=kernel)
    assert torch.equal(alone[0], out32[m - 1])
    # what gemm_bf16 picks: the bulk-copy kernel where it takes the call and rows are short, else the other
    picked = "stream" if ops.gemm_stream_supported(a_d, w_d) and (k <= ops.STREAM_K or k % 32) else "load"
    if kernel == picked and ops.gemm_skinny_supported(a_d, w_d):
        assert torch.equal(ops.gemm_bf16(a_d, w_d, torch.float32, backend="skinny"), out32)
        if m <= (ops.SKINNY_ROWS if k <= ops.STREAM_K else ops.SKINNY_ROWS // 2):   # what "auto" picks for so few rows
            assert torch.equal(ops.gemm_bf16(a_d, w_d, torch.float32, backend="auto"), out32)


def test_gemm_stream_refuses_what_does_not_fit(ops):
    wide = dev(np.zeros((16, 6144)), torch.bfloat16)          # 16 rows of x and 8 of W at k = 6144 exceed shared memory
    assert not ops.gemm_stream_supported(wide, dev(np.zeros((64, 6144)), torch.bfloat16))
    assert ops.gemm_stream_supported(wide[:8].contiguous(), dev(np.zeros((64, 6144)), torch.bfloat16))
    assert not ops.gemm_stream_supported(dev(np.zeros((4, 40)), torch.bfloat16), dev(np.zeros((8, 40)), torch.bfloat16))


@pytest.mark.parametrize("kernel", ["load", "stream"])
@pytest.mark.parametrize("m", [1, 8, 13, 24, 64])
def test_gemm_skinny_swiglu(ops, m, kernel):
    rng = np.random.default_rng(m)
    inter, k = 3 * 56, 96
    a, w = rng.normal(size=(m, k)), rng.normal(size=(2 * inter, k)) * 0.3
    if kernel == "stream" and m > 16:
        assert not ops.gemm_stream_supported(dev(a, torch.bfloat16), dev(w, torch.bfloat16), swiglu=True)
        return
    out = ops.gemm_skinny(dev(a, torch.bfloat16), dev(w, torch.bfloat16), swiglu=True, kernel=kernel)
    ops.check_status("cuda")
    gate_up = rounded(rounded(a, torch.bfloat16) @ rounded(w, torch.bfloat16).T, torch.bfloat16)
    g, u = gate_up[:, :inter], gate_up[:, inter:]
    ref = g / (1 + np.exp(-g)) * u
    error = np.abs(out.cpu().double().numpy() - ref)
    # gate and up may each land one bfloat16 step away from the float64 product's rounding
    assert (error <= 3 * 2.0 ** -8 * (np.abs(ref) + np.abs(u) * 0.3 + np.abs(g) * 0.3) + 1e-4).all()
    assert not ops.gemm_skinny_supported(dev(a[:, :80], torch.bfloat16).contiguous(), dev(w[:, :80], torch.bfloat16).contiguous())
    assert not ops.gemm_skinny_supported(dev(np.zeros((65, k)), torch.bfloat16), dev(w, torch.bfloat16))


@pytest.mark.parametrize("m, inter, k", [(1, 56, 96), (130, 200, 136), (513, 3072, 1024)])
def test_tcgen05_swiglu_epilogue(ops, m, inter, k):
    from metallix_b200 import tensor_core
    rng = np.random.default_rng(m)
    a, w = rng.normal(size=(m, k)), rng.normal(size=(2 * inter, k)) * 0.1
    a_d, w_d = dev(a, torch.bfloat16), dev(w, torch.bfloat16)
    out = tensor_core.gemm_swiglu(a_d, w_d)
    ops.check_status("cuda")
    separate = ops.silu_mul(tensor_core.gemm(a_d, w_d))        # the same product, activation as its own kernel
    # the epilogue takes the fast exponential; the two may land one bfloat16 step apart
    gap = (out.double() - separate.double()).abs()
    assert bool((gap <= 2.0 ** -7 * separate.double().abs() + 1e-30).all())
    assert float((gap > 0).double().mean()) < 0.02
    gate_up = rounded(rounded(a, torch.bfloat16) @ rounded(w, torch.bfloat16).T, torch.bfloat16)
    g, u = gate_up[:, :inter], gate_up[:, inter:]
    ref = g / (1 + np.exp(-g)) * u
    assert np.abs(out.cpu().double().numpy() - ref).max() < 3e-2 * np.abs(ref).max()


def test_tcgen05_refuses_what_it_cannot_take(ops):
    from metallix_b200 import tensor_core
    a, w = dev(np.zeros((4, 100)), torch.bfloat16), dev(np.zeros((8, 100)), torch.bfloat16)
    assert not tensor_core.supports(a, w, torch.bfloat16)        # k = 100: rows would not start on 16 bytes
    with pytest.raises(ops.KernelError, match="multiples of 8"):
        tensor_core.gemm(a, w)
    with pytest.raises(ops.KernelError, match="does not take"):
        ops.gemm_bf16(a, w, backend="tcgen05")
    with pytest.raises(ops.KernelError, match="unknown gemm backend"):
        ops.gemm_bf16(a, w, backend="cutlass")
    assert ops.gemm_bf16(a, w, backend="auto").shape == (4, 8)   # auto falls back to the library


@pytest.mark.parametrize("dtype", DTYPES)
def test_silu_mul(ops, dtype):
    rng = np.random.default_rng(4)
    gate_up = rng.normal(size=(9, 2 * 136)) * 3
    out = ops.silu_mul(dev(gate_up, dtype))
    g, u = rounded(gate_up, dtype)[:, :136], rounded(gate_up, dtype)[:, 136:]
    ref = g / (1 + np.exp(-g)) * u
    # float32 inside; a bfloat16 result is the exact value rounded once (half a
    # step is at most 2^-9 of the value)
    error = np.abs(out.cpu().double().numpy() - ref)
    assert (error <= (2.0 ** -21 if dtype == torch.float32 else 2.0 ** -8) * np.abs(ref) + 1e-30).all()


# -------------------------------------------------------------------- picking
def test_argmax_first_maximum_and_finite_flag(ops):
    rng = np.random.default_rng(5)
    logits = rng.normal(size=(6, 151_937)).astype(np.float32)
    logits[0, [100, 90_000]] = 9.0          # a tie: the lower id wins
    logits[1, 151_936] = 11.0               # the last vocabulary row
    logits[2, 0] = 12.0
    ids = ops.argmax(dev(logits)).tolist()
    ops.check_status("cuda")
    assert ids == [plain.greedy_pick(row) for row in logits] and ids[:3] == [100, 151_936, 0]
    logits[4, 77] = np.inf
    ids = ops.argmax(dev(logits)).tolist()
    assert ids[4] == -1 and ids[3] == plain.greedy_pick(logits[3])
    with pytest.raises(ops.KernelError, match="non-finite"):
        ops.check_status("cuda")


@pytest.mark.parametrize("rows, vocab", [(1, 7), (3, 5000), (64, 4096), (300, 2051), (2, 70_001)])
def test_argmax_in_pieces(ops, rows, vocab):
    """A row is cut into pieces; ties within a piece, across pieces and at a
    piece's edge go to the lower id, and rows of any length and alignment work."""
    rng = np.random.default_rng(rows + vocab)
    logits = rng.normal(size=(rows, vocab)).astype(np.float32)
    for r in range(rows):
        where = rng.integers(0, vocab, size=3)
        logits[r, where] = 7.0 + r % 2
    logits[0, [0, vocab - 1]] = 20.0
    ids = ops.argmax(dev(logits)).tolist()
    ops.check_status("cuda")
    assert ids == [plain.greedy_pick(row) for row in logits] and ids[0] == 0
    strided = dev(np.concatenate([logits, logits], axis=1))[:, 1:vocab + 1]   # rows that start off a 16-byte boundary
    assert ops.argmax(strided).tolist() == [plain.greedy_pick(row) for row in strided.cpu().numpy()]


@pytest.mark.parametrize("vocab", [8, 331, 5000])
def test_sample_icdf_matches_the_host_definition(ops, vocab):
    rng = np.random.default_rng(vocab)
    rows = 40
    logits = (rng.normal(size=(rows, vocab)) * 2).astype(np.float32)
    temperature = rng.uniform(0.3, 1.5, size=rows)
    seeds = rng.integers(0, 2 ** 63, size=rows)
    streams = rng.integers(0, 2 ** 40, size=rows)
    positions = rng.integers(0, 5000, size=rows)
    ids = ops.sample_icdf(dev(logits), dev(temperature, torch.float64), dev(seeds, torch.int64),
                          dev(streams, torch.int64), dev(positions, torch.int32)).tolist()
    ops.check_status("cuda")
    for r in range(rows):
        uniform = plain.request_uniform(int(seeds[r]), int(streams[r]), int(positions[r]))
        assert ids[r] == plain.sample_categorical(logits[r], float(temperature[r]), uniform), r


def test_sample_icdf_legal_mask_and_law(ops):
    logits = np.array([[0.3, -0.6, 1.1, 0.0, 0.7, 2.0]], dtype=np.float32).repeat(4000, axis=0)
    legal = np.array([[1, 1, 1, 1, 1, 0]], dtype=np.uint8).repeat(4000, axis=0)
    temperature = np.full(4000, 0.6)
    ids = ops.sample_icdf(dev(logits), dev(temperature, torch.float64),
                          dev(np.full(4000, 11), torch.int64), dev(np.zeros(4000), torch.int64),
                          dev(np.arange(4000), torch.int32), dev(legal, torch.uint8)).cpu().numpy()
    counts = np.bincount(ids, minlength=6)
    assert counts[5] == 0
    weights = np.exp(logits[0, :5].astype(np.float64) / 0.6)
    expected = weights / weights.sum() * 4000
    assert (((counts[:5] - expected) ** 2) / expected).sum() < 40.0   # race.rs:292-330 uses the same bound


def test_sample_race_matches_the_reference_tokens(ops):
    import json, os
    golden = json.load(open(os.path.join(os.path.dirname(__file__), "golden",
                                         "reference_sampler_vectors.json")))["race_v2_tokens"]
    rows = len(golden["tokens"])
    logits = np.array([golden["logits"]], dtype=np.float32).repeat(rows, axis=0)
    legal = np.array([golden["legal"]], dtype=np.uint8).repeat(rows, axis=0)
    ids = ops.sample_race(dev(logits), dev(np.full(rows, golden["temperature"]), torch.float64),
                          dev(np.full(rows, golden["seed"]), torch.int64),
                          dev(np.arange(rows), torch.int32), dev(legal, torch.uint8)).tolist()
    assert ids == golden["tokens"]
    rng = np.random.default_rng(6)
    big = (rng.normal(size=(5, 3001)) * 2).astype(np.float32)
    ids = ops.sample_race(dev(big), dev(np.full(5, 0.8), torch.float64), dev(np.arange(5) + 2 ** 33, torch.int64),
                          dev(np.arange(5) * 7, torch.int32)).tolist()
    assert ids == [plain.sample_race(big[r], 0.8, r + 2 ** 33, r * 7) for r in range(5)]


@pytest.mark.parametrize("top_p, top_k", [(1.0, 5), (0.7, 0), (0.35, 12), (0.9, 1), (1.0, 0), (0.999, 4000)])
def test_nucleus_mask(ops, top_p, top_k):
    rng = np.random.default_rng(int(top_p * 100) + top_k)
    logits = (rng.normal(size=(6, 3000)) * 1.5).astype(np.float32)
    logits[1, :40] = logits[1, 0]        # many equal logits across the cut
    logits[2, :] = 0.25                  # all equal
    logits[3] = np.round(logits[3])      # many ties everywhere
    temperature = np.array([1.0, 0.7, 1.0, 0.5, 2.0, 0.9])
    mask = ops.nucleus_mask(dev(logits), dev(temperature, torch.float64), dev(np.full(6, top_p), torch.float64),
                            dev(np.full(6, top_k), torch.int32)).cpu().numpy().astype(bool)
    ops.check_status("cuda")
    for r in range(6):
        ref = plain.nucleus_mask(logits[r], float(temperature[r]), top_p, top_k or None)
        assert np.array_equal(mask[r], ref), (r, mask[r].sum(), ref.sum())


@pytest.mark.parametrize("vocab", [7, 151_936, 400_003])
def test_nucleus_mask_of_long_and_short_rows(ops, vocab):
    """A row lies in the shared memory of its eight blocks where it fits
    (151,936 does, 400,003 does not); seven tokens leave some blocks empty."""
    rng = np.random.default_rng(vocab)
    logits = (rng.normal(size=(3, vocab)) * 2.0).astype(np.float32)
    logits[1, vocab // 2:] = logits[1, 0]            # a plateau of equal logits that the cut may cross
    temperature = np.array([1.0, 0.6, 1.3])
    for top_p, top_k in ((0.9, 0), (0.5, 40), (1.0, 3), (0.97, vocab - 1)):
        mask = ops.nucleus_mask(dev(logits), dev(temperature, torch.float64), dev(np.full(3, top_p), torch.float64),
                                dev(np.full(3, top_k), torch.int32)).cpu().numpy().astype(bool)
        ops.check_status("cuda")
        for r in range(3):
            ref = plain.nucleus_mask(logits[r], float(temperature[r]), top_p, top_k or None)
            assert np.array_equal(mask[r], ref), (top_p, top_k, r, mask[r].sum(), ref.sum())
    logits[2, 5] = np.nan
    mask = ops.nucleus_mask(dev(logits), dev(temperature, torch.float64), dev(np.full(3, 0.9), torch.float64),
                            dev(np.zeros(3), torch.int32)).cpu().numpy().astype(bool)
    assert mask[2].all() and np.array_equal(mask[0], plain.nucleus_mask(logits[0], 1.0, 0.9, None))
    with pytest.raises(ops.KernelError, match="non-finite"):
        ops.check_status("cuda")


def test_timeline_needs_a_build_of_its_own(ops):
    """The usual library records no timeline and says how to get one."""
    with pytest.raises(ops.KernelError, match="METALLIX_B200_TIMELINE"):
        ops.timeline()


@pytest.mark.parametrize("shape,dtype", [((3, 9, 2, 2, 8, 16), torch.bfloat16),   # pages of three layers
                                         ((1, 5, 7), torch.float32),             # state slots of 28 bytes
                                         ((2, 6, 3), torch.int8)])               # units of no word size
def test_copy_units(shape, dtype):
    """pool[:, target] = pool[:, source] in every entry; other units untouched;
    a unit outside the pool is reported, not copied."""
    from metallix_b200 import ops
    pool = (torch.randn(shape, device="cuda") * 50).to(dtype)
    pairs = [(0, 3), (4, 1), (2, 2)]
    expected = pool.clone()
    for source, target in pairs:
        expected[:, target] = pool[:, source]
    ops.copy_units(pool, torch.tensor(pairs, dtype=torch.int32, device="cuda"))
    assert torch.equal(pool, expected)
    ops.copy_units(pool, torch.tensor([(0, shape[1])], dtype=torch.int32, device="cuda"))
    assert torch.equal(pool, expected)
    with pytest.raises(ops.KernelError, match="outside the page pool"):
        ops.check_status(pool.device)
