"""Python face of the hand-written CUDA kernels.

Every function checks its tensors (device, dtype, layout, sizes) and raises
``KernelError`` for what the kernels do not take; it never falls back to
another implementation. Kernels run on torch's current CUDA stream.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .csrc import build

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}

STATUS_BITS = {1: "a token id outside the vocabulary", 2: "a cache slot or position outside its table",
               4: "a block-table entry outside the page pool", 8: "non-finite logits",
               16: "a bounded wait inside a kernel ran out"}


class KernelError(RuntimeError):
    pass


_P, _I, _L, _F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
_SIGNATURES = {
    "mxb_embed": [_P, _P, _I, _P, _I, _I, _I, _P, _P],
    "mxb_rmsnorm": [_P, _I, _P, _I, _P, _P, _I, _I, _F, _P],
    "mxb_add_rmsnorm": [_P, _P, _I, _P, _I, _P, _I, _I, _F, _P],
    "mxb_add_summands_rmsnorm": [_P, _P, _I, _P, _I, _P, _I, _I, _F, _P],
    "mxb_add": [_P, _P, _I, _L, _P],
    "mxb_copy_units": [_P, _I, _I, _L, _P, _I, _P, _P],
    "mxb_qk_norm_rope_cache": [_P, _P, _P, _L, _L, _L, _P, _P, _P, _P, _P, _P, _P, _P,
                               _I, _I, _I, _I, _I, _I, _I, _I, _F, _I, _P, _P],
    "mxb_paged_attention_tile": [_P, _P, _P, _P, _I, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I,
                                 _F, _I, _P, _P],
    "mxb_paged_attention_decode": [_P, _P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I,
                                   _F, _I, _P, _P],
    "mxb_paged_attention_decode_supported": [_I, _I, _I, _I],
    "mxb_paged_attention_decode_project_supported": [_I, _I, _I, _I, _I, _P, _L],
    "mxb_paged_attention_decode_project": [_P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I,
                                           _F, _P, _L, _I, _P, _P, _P],
    "mxb_paged_attention_split_keys": [],
    "mxb_set_decode_resident_blocks": [_I, _I],
    "mxb_flash_prefill": [_P, _P, _P, _P, _I, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _F, _I, _P, _P],
    "mxb_flash_prefill_supported": [_I, _I, _I, _I],
    "mxb_flash_prefill_tile": [],
    "mxb_flash_prefill_tcgen05": [_P, _P, _P, _P, _I, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _F, _I, _I, _P,
                                  _P, _P],
    "mxb_flash_prefill_tcgen05_supported": [_I, _I, _I, _I, _I],
    "mxb_flash_prefill_tcgen05_tile": [],
    "mxb_gemm_simple": [_P, _I, _P, _P, _I, _I, _I, _I, _L, _L, _L, _P],
    "mxb_gemm_skinny": [_P, _I, _P, _P, _I, _I, _I, _L, _L, _L, _I, _P],
    "mxb_gemm_skinny_supported": [_I, _I, _I, _L, _L],
    "mxb_gemm_stream": [_P, _I, _P, _P, _I, _I, _I, _L, _L, _L, _I, _P, _P],
    "mxb_gemm_stream_supported": [_I, _I, _I, _L, _L, _I],
    "mxb_gemm_tcgen05": [_P, _P, _P, _I, _I, _I, _L, _L, _L, _I, _P, _P],
    "mxb_gemm_tcgen05_supported": [_I, _I, _I, _L, _L],
    "mxb_silu_mul": [_P, _P, _I, _L, _I, _P],
    "mxb_argmax": [_P, _L, _I, _I, _P, _P, _P, _P],
    "mxb_argmax_pieces": [_I, _I],
    "mxb_sample_icdf": [_P, _L, _I, _I, _P, _P, _P, _P, _P, _P, _P, _P, _P],
    "mxb_icdf_pieces": [_I],
    "mxb_sample_race": [_P, _L, _I, _I, _P, _P, _P, _P, _P, _P, _P, _P],
    "mxb_set_chained_launches": [_I],
    "mxb_nucleus_mask": [_P, _L, _I, _I, _P, _P, _P, _P, _P, _P],
}
_functions = {}
_status = {}


def _fn(name: str):
    fn = _functions.get(name)
    if fn is None:
        library = build.kernels()
        try:
            fn = getattr(library, name)
        except AttributeError:
            raise KernelError(f"the kernel library has no entry point {name}") from None
        fn.argtypes = _SIGNATURES[name]
        fn.restype = ctypes.c_int
        _functions[name] = fn
    return fn


_launches = 0


def launch_count() -> int:
    """How many of this library's kernel entry points have been called
    (a replayed CUDA graph counts the calls it captured)."""
    return _launches


def count_launches(count: int) -> None:
    global _launches
    _launches += count


def _call(name: str, *args) -> None:
    global _launches
    _launches += 1
    code = _fn(name)(*args)
    if code != 0:
        raise KernelError(f"{name} failed to launch: CUDA error {code}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current stream's handle; this runs once per launch, so it takes the short way."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _ptr(tensor: Optional[torch.Tensor]) -> Optional[int]:
    return None if tensor is None else tensor.data_ptr()


def _need(condition: bool, message: str) -> None:
    if not condition:
        raise KernelError(message)


def _check(tensor: torch.Tensor, name: str, dtypes, dims: Optional[int] = None) -> None:
    if (isinstance(tensor, torch.Tensor) and tensor.is_cuda and tensor.dtype in dtypes and tensor.is_contiguous()
            and (dims is None or tensor.dim() == dims)):
        return   # the messages below are built only for what fails
    _need(isinstance(tensor, torch.Tensor), f"{name} must be a tensor")
    _need(tensor.is_cuda, f"{name} must be on a CUDA device; there is no CPU path")
    _need(tensor.dtype in dtypes, f"{name} has dtype {tensor.dtype}, expected one of {dtypes}")
    _need(tensor.is_contiguous(), f"{name} must be contiguous")
    if dims is not None:
        _need(tensor.dim() == dims, f"{name} must have {dims} dimensions, has {tensor.dim()}")


def require_cuda() -> None:
    """Fails loudly where the kernels cannot run."""
    if not torch.cuda.is_available():
        raise KernelError("no CUDA device: metallix_b200 runs on a B200 only and has no CPU path")
    build.kernels()


_chained: Optional[bool] = None


def set_chained_launches(enabled: bool) -> None:
    """Lets consecutive kernels of this library overlap (programmatic dependent
    launch): a kernel may start, and fetch weights, while its predecessor is
    still running, and waits for the predecessor before it reads its output.
    The switch belongs to the library; an engine sets it to its own choice
    before it launches."""
    global _chained
    if _chained is not enabled:
        _fn("mxb_set_chained_launches")(1 if enabled else 0)
        _chained = bool(enabled)


TIMELINE_SOURCES = ("norms", "gemm_load", "gemm_stream", "qk_rope", "attention")


def timeline(reset: bool = True):
    """[(nanoseconds, source)] in time order: when each chained kernel
    launched since the last reset got past the wait for the kernel ahead of
    it. Needs the library built with METALLIX_B200_TIMELINE=1 in the
    environment (a build of its own, next to the usual one)."""
    library = build.kernels()
    events = []
    for source in TIMELINE_SOURCES:
        function = getattr(library, f"mxb_timeline_{source}", None)
        if function is None:
            raise KernelError("this build records no timeline: set METALLIX_B200_TIMELINE=1 before the first use")
        function.argtypes = [ctypes.c_void_p, ctypes.c_int]
        function.restype = ctypes.c_int
        buffer = (ctypes.c_ulonglong * 8192)()
        count = function(buffer, 1 if reset else 0)
        events.extend((int(buffer[i]), source) for i in range(count))
    return sorted(events)


def status_word(device) -> torch.Tensor:
    """The int32 word kernels set bits in instead of trapping."""
    word = _status.get(device)
    if word is None:
        key = torch.device(device).index or 0
        if key not in _status:
            _status[key] = torch.zeros(1, dtype=torch.int32, device=device)
        word = _status[device] = _status[key]   # torch.device objects and strings find it directly next time
    return word


_status_host = {}


def fetch_status(device) -> None:
    """Queues a copy of the status word to pinned host memory on the current
    stream; ``raise_status`` reads it once the stream has been synchronised
    (by reading the step's results, say), which saves a synchronisation of
    its own."""
    word = status_word(device)
    host = _status_host.get(device)
    if host is None:
        host = _status_host[device] = torch.zeros(1, dtype=torch.int32, pin_memory=True)
    host.copy_(word, non_blocking=True)


def raise_status(device) -> None:
    """Raises on what the last ``fetch_status`` copy brought (the caller has
    synchronised since); clears the device word then."""
    host = _status_host.get(device)
    value = int(host[0]) if host is not None else 0
    if value:
        status_word(device).zero_()
        reasons = [text for bit, text in STATUS_BITS.items() if value & bit]
        raise KernelError("a kernel refused its input: " + "; ".join(reasons))


def check_status(device) -> None:
    """Reads the status word (synchronises) and raises on any bit; clears it."""
    word = status_word(device)
    value = int(word.item())
    if value:
        word.zero_()
        reasons = [text for bit, text in STATUS_BITS.items() if value & bit]
        raise KernelError("a kernel refused its input: " + "; ".join(reasons))


# ------------------------------------------------------------------ embedding
def embed(ids: torch.Tensor, table: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t] = table[ids[t]] as float32."""
    _check(ids, "ids", (torch.int32,), 1)
    _check(table, "table", tuple(_CODES), 2)
    tokens, (vocab, hidden) = ids.numel(), table.shape
    if out is None:
        out = torch.empty((tokens, hidden), dtype=torch.float32, device=ids.device)
    _check(out, "out", (torch.float32,), 2)
    _need(out.shape == (tokens, hidden), "out has the wrong shape")
    _call("mxb_embed", out.data_ptr(), table.data_ptr(), _CODES[table.dtype], ids.data_ptr(),
          tokens, hidden, vocab, status_word(ids.device).data_ptr(), _stream())
    return out


# ----------------------------------------------------------------------- norms
def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
            rows_index: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * w over the last axis, float32 inside.
    ``rows_index`` picks the rows of ``x`` to normalise."""
    _check(x, "x", tuple(_CODES))
    _check(weight, "weight", (torch.float32,), 1)
    size = x.shape[-1]
    _need(weight.numel() == size, f"weight has {weight.numel()} values for rows of {size}")
    rows = x.numel() // size if rows_index is None else rows_index.numel()
    if rows_index is not None:
        _check(rows_index, "rows_index", (torch.int32,), 1)
        _need(x.dim() == 2, "rows_index needs a 2-d input")
        shape = (rows, size)
    else:
        shape = tuple(x.shape)
    if out is None:
        out = torch.empty(shape, dtype=out_dtype, device=x.device)
    _check(out, "out", (out_dtype,))
    _need(out.numel() == rows * size, "out has the wrong size")
    _call("mxb_rmsnorm", out.data_ptr(), _CODES[out_dtype], x.data_ptr(), _CODES[x.dtype],
          weight.data_ptr(), _ptr(rows_index), rows, size, float(eps), _stream())
    return out


def add_rmsnorm(x: torch.Tensor, delta: torch.Tensor, weight: torch.Tensor, eps: float,
                out_dtype: torch.dtype, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x += delta in float32 (in place), then returns RMSNorm(x) * w. A delta
    of three dimensions, float32 ``[parts, rows, size]``, is a sum its producer
    left in parts: they are added up in their order first."""
    _check(x, "x", (torch.float32,), 2)
    _check(weight, "weight", (torch.float32,), 1)
    rows, size = x.shape
    _need(weight.numel() == size, "weight has the wrong size")
    if out is None:
        out = torch.empty((rows, size), dtype=out_dtype, device=x.device)
    _check(out, "out", (out_dtype,), 2)
    _need(out.shape == x.shape, "out has the wrong shape")
    if delta.dim() == 3:
        _check(delta, "delta", (torch.float32,), 3)
        _need(delta.shape[1:] == x.shape and delta.shape[0] >= 1, "the summands and x differ in shape")
        _call("mxb_add_summands_rmsnorm", x.data_ptr(), delta.data_ptr(), delta.shape[0], out.data_ptr(),
              _CODES[out_dtype], weight.data_ptr(), rows, size, float(eps), _stream())
        return out
    _check(delta, "delta", tuple(_CODES), 2)
    _need(delta.shape == x.shape, "delta and x differ in shape")
    _call("mxb_add_rmsnorm", x.data_ptr(), delta.data_ptr(), _CODES[delta.dtype], out.data_ptr(),
          _CODES[out_dtype], weight.data_ptr(), rows, size, float(eps), _stream())
    return out


def add_(x: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
    """x += delta, the sum in float32."""
    _check(x, "x", (torch.float32,))
    _check(delta, "delta", tuple(_CODES))
    _need(delta.shape == x.shape, "delta and x differ in shape")
    _call("mxb_add", x.data_ptr(), delta.data_ptr(), _CODES[delta.dtype], x.numel(), _stream())
    return x


# ------------------------------------------------------- copies in the cache
def copy_units(pool: torch.Tensor, pairs: torch.Tensor) -> None:
    """pool[:, target] = pool[:, source] for every (source, target) row of
    ``pairs`` (int32 ``[count, 2]`` on the device); ``pool`` is contiguous
    ``[entries, units, ...]``: the pages of a group's layers, or (with a leading
    dimension of one) the slots of a state tensor. No target may be another
    pair's source."""
    _need(pool.is_cuda and pool.is_contiguous() and pool.dim() >= 2, "pool must be a contiguous device tensor")
    _need(pairs.is_cuda and pairs.dtype == torch.int32 and pairs.dim() == 2 and pairs.shape[1] == 2
          and pairs.is_contiguous(), "pairs must be int32 [count, 2] on the device")
    entries, units = pool.shape[0], pool.shape[1]
    unit_bytes = pool[0, 0].numel() * pool.element_size()
    _call("mxb_copy_units", pool.data_ptr(), entries, units, unit_bytes, pairs.data_ptr(), pairs.shape[0],
          status_word(pool.device).data_ptr(), _stream())


# ------------------------------------------------- q/k norm, rotation, cache
def qk_norm_rope_cache(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, q_out: Optional[torch.Tensor],
                       cache: Optional[torch.Tensor], slots: Optional[torch.Tensor],
                       positions: torch.Tensor, q_weight: Optional[torch.Tensor],
                       k_weight: Optional[torch.Tensor], cos: Optional[torch.Tensor],
                       sin: Optional[torch.Tensor], eps: float) -> None:
    """Per-head RMSNorm of q and k (if weights are given), rotate-half rotation
    by ``positions`` (if tables are given), q written to ``q_out``
    [tokens, heads, head_dim], k and v written into ``cache``
    [pages, 2, kv_heads, page_tokens, head_dim] at ``slots`` (a negative slot
    skips the token; ``cache=None`` writes nothing). q, k and v are
    [tokens, heads * head_dim] views whose rows may be strided."""
    dtype = q.dtype
    for name, tensor in (("q", q), ("k", k), ("v", v)):
        _need(tensor.is_cuda and tensor.dtype == dtype and tensor.dtype in _CODES and tensor.dim() == 2
              and tensor.stride(1) == 1, f"{name} must be a CUDA [tokens, width] tensor with unit column stride")
    tokens = q.shape[0]
    _check(positions, "positions", (torch.int32,), 1)
    _need(positions.numel() == tokens and k.shape[0] == tokens and v.shape[0] == tokens, "token counts differ")
    if cache is not None:
        _check(cache, "cache", (dtype,), 5)
        num_pages, two, kv_heads, page_tokens, head_dim = cache.shape
        _need(two == 2, "cache must be [pages, 2, kv_heads, page_tokens, head_dim]")
        _check(slots, "slots", (torch.int32,), 1)
        _need(slots.numel() == tokens, "one slot per token")
    else:
        _need(q_out is not None, "nothing to write")
        head_dim = q_out.shape[-1]
        kv_heads = k.shape[1] // head_dim
        num_pages, page_tokens = 0, 1
    _need(q.shape[1] % head_dim == 0 and k.shape[1] == kv_heads * head_dim and v.shape[1] == kv_heads * head_dim,
          "q, k, v widths do not match the head layout")
    heads = q.shape[1] // head_dim
    if q_out is not None:
        _check(q_out, "q_out", (dtype,), 3)
        _need(q_out.shape == (tokens, heads, head_dim), "q_out must be [tokens, heads, head_dim]")
    for name, weight in (("q_weight", q_weight), ("k_weight", k_weight)):
        if weight is not None:
            _check(weight, name, (torch.float32,), 1)
            _need(weight.numel() == head_dim, f"{name} must have head_dim values")
    rotary_dim, table_positions = 0, 0
    if cos is not None:
        _check(cos, "cos", (torch.float32,), 2)
        _check(sin, "sin", (torch.float32,), 2)
        _need(cos.shape == sin.shape, "cos and sin differ in shape")
        table_positions, rotary_dim = cos.shape[0], cos.shape[1] * 2
        _need(rotary_dim <= head_dim, "rotary_dim exceeds head_dim")
    _call("mxb_qk_norm_rope_cache", q.data_ptr(), k.data_ptr(), v.data_ptr(), q.stride(0), k.stride(0),
          v.stride(0), _ptr(q_out), _ptr(cache), _ptr(slots), positions.data_ptr(), _ptr(q_weight),
          _ptr(k_weight), _ptr(cos), _ptr(sin), table_positions, rotary_dim, tokens, heads, kv_heads,
          head_dim, page_tokens, num_pages, float(eps), _CODES[dtype],
          status_word(q.device).data_ptr(), _stream())


def norm_rotate_heads(x: torch.Tensor, head_dim: int, positions: torch.Tensor,
                      weight: Optional[torch.Tensor] = None, cos: Optional[torch.Tensor] = None,
                      sin: Optional[torch.Tensor] = None, eps: float = 0.0) -> torch.Tensor:
    """Per-head RMSNorm (if ``weight``) and rotation (if tables) of x
    [tokens, n * head_dim]; returns [tokens, n, head_dim]. Writes no cache."""
    _need(x.dim() == 2 and x.shape[1] % head_dim == 0, "x must be [tokens, n * head_dim]")
    out = torch.empty((x.shape[0], x.shape[1] // head_dim, head_dim), dtype=x.dtype, device=x.device)
    empty = x[:, :0]
    qk_norm_rope_cache(x, empty, empty, out, None, None, positions, weight, None, cos, sin, eps)
    return out


def write_cache(k: torch.Tensor, v: torch.Tensor, cache: torch.Tensor, slots: torch.Tensor,
                positions: torch.Tensor) -> None:
    """Stores k and v [tokens, kv_heads * head_dim] as they are at ``slots``."""
    qk_norm_rope_cache(k[:, :0], k, v, None, cache, slots, positions, None, None, None, None, 0.0)


# ------------------------------------------------------------------ attention
def paged_attention_tile(q: torch.Tensor, cache: torch.Tensor, out: torch.Tensor,
                         block_tables: torch.Tensor, tile_request: torch.Tensor,
                         tile_start: torch.Tensor, tile_length: torch.Tensor,
                         positions: torch.Tensor, scale: float, window: int = 0) -> torch.Tensor:
    """Attention of every query token over its request's cached keys (itself
    included) in float32; q and out are [tokens, heads, head_dim]."""
    dtype = q.dtype
    _check(q, "q", tuple(_CODES), 3)
    _check(out, "out", (dtype,), 3)
    _check(cache, "cache", (dtype,), 5)
    _need(out.shape == q.shape, "out and q differ in shape")
    tokens, heads, head_dim = q.shape
    num_pages, two, kv_heads, page_tokens, cache_dim = cache.shape
    _need(two == 2 and cache_dim == head_dim, "cache must be [pages, 2, kv_heads, page_tokens, head_dim]")
    _need(heads % kv_heads == 0, f"{heads} query heads cannot share {kv_heads} key/value heads")
    _need(0 < head_dim <= 256, f"head_dim {head_dim} is outside 1..256")
    _check(block_tables, "block_tables", (torch.int32,), 2)
    for name, tensor in (("tile_request", tile_request), ("tile_start", tile_start),
                         ("tile_length", tile_length), ("positions", positions)):
        _check(tensor, name, (torch.int32,), 1)
    tiles = tile_request.numel()
    _need(tile_start.numel() == tiles and tile_length.numel() == tiles, "tile lists differ in length")
    _need(positions.numel() == tokens, "one position per token")
    _call("mxb_paged_attention_tile", q.data_ptr(), cache.data_ptr(), out.data_ptr(),
          block_tables.data_ptr(), block_tables.shape[1], tile_request.data_ptr(),
          tile_start.data_ptr(), tile_length.data_ptr(), positions.data_ptr(), tiles, heads,
          kv_heads, head_dim, page_tokens, num_pages, int(window or 0), float(scale), _CODES[dtype],
          status_word(q.device).data_ptr(), _stream())
    return out


def flash_prefill_supported(head_dim: int, heads: int, kv_heads: int, dtype: torch.dtype) -> bool:
    """Whether the tensor-core prompt kernel takes this head layout."""
    if dtype not in _CODES:
        return False
    return bool(_fn("mxb_flash_prefill_supported")(head_dim, heads, kv_heads, _CODES[dtype]))


def flash_prefill_tile() -> int:
    """Query tokens per tile of the tensor-core prompt kernel."""
    return _fn("mxb_flash_prefill_tile")()


PROMPT_KERNEL = "auto"   # what flash_prefill's "auto" means: "auto", "tcgen05" or "mma" (for comparisons)


def flash_prefill_tcgen05_supported(head_dim: int, heads: int, kv_heads: int, page_tokens: int,
                                    dtype: torch.dtype) -> bool:
    """Whether the tcgen05 prompt kernel takes this head layout and page size."""
    if dtype not in _CODES:
        return False
    return bool(_fn("mxb_flash_prefill_tcgen05_supported")(head_dim, heads, kv_heads, page_tokens, _CODES[dtype]))


KEY_SHARES = None   # an int forces the number of blocks that share a query tile's keys (tests, comparisons)


def flash_key_shares(blocks: int, longest_context: int, window: int = 0) -> int:
    """How many blocks share the keys of a query tile of the tcgen05 prompt
    kernel: one, unless the step has so few (tile, head) blocks and so many
    keys that most SMs would stand idle (a portion of a prompt behind a long
    context). Each share keeps at least 1,024 keys."""
    if KEY_SHARES is not None:
        return max(1, int(KEY_SHARES))
    keys = min(longest_context, window) if window else longest_context
    if blocks >= 100 or keys < 2048:
        return 1
    return max(1, min(8, 148 // blocks, keys // 1024))


def flash_prefill(q: torch.Tensor, cache: torch.Tensor, out: torch.Tensor, block_tables: torch.Tensor,
                  tile_request: torch.Tensor, tile_start: torch.Tensor, tile_length: torch.Tensor,
                  positions: torch.Tensor, scale: float, window: int = 0, kernel: str = "auto",
                  longest_context: int = 0) -> torch.Tensor:
    """Causal attention of prompt portions on the tensor cores (bfloat16,
    float32 softmax and accumulation); tiles hold up to 128 consecutive tokens
    of one request. ``kernel``: "tcgen05" (TMA, tensor memory), "mma" (the
    warp-level kernel) or "auto" (tcgen05 where it takes the page size).
    ``longest_context`` (the most keys any of the tiles sees, 0: unknown)
    lets the tcgen05 kernel share a tile's keys out among several blocks when
    the tiles alone would leave most of the GPU idle."""
    _check(q, "q", (torch.bfloat16,), 3)
    _check(out, "out", (torch.bfloat16,), 3)
    _check(cache, "cache", (torch.bfloat16,), 5)
    _need(out.shape == q.shape, "out and q differ in shape")
    tokens, heads, head_dim = q.shape
    num_pages, two, kv_heads, page_tokens, cache_dim = cache.shape
    _need(two == 2 and cache_dim == head_dim, "cache must be [pages, 2, kv_heads, page_tokens, head_dim]")
    _need(flash_prefill_supported(head_dim, heads, kv_heads, q.dtype),
          f"the tensor-core prompt kernel does not take head_dim {head_dim} with {heads}/{kv_heads} heads")
    _check(block_tables, "block_tables", (torch.int32,), 2)
    for name, tensor in (("tile_request", tile_request), ("tile_start", tile_start),
                         ("tile_length", tile_length), ("positions", positions)):
        _check(tensor, name, (torch.int32,), 1)
    tiles = tile_request.numel()
    _need(tile_start.numel() == tiles and tile_length.numel() == tiles, "tile lists differ in length")
    _need(positions.numel() == tokens, "one position per token")
    if kernel == "auto":
        kernel = PROMPT_KERNEL
    _need(kernel in ("auto", "tcgen05", "mma"), f"unknown prompt-attention kernel {kernel!r}")
    tcgen05 = flash_prefill_tcgen05_supported(head_dim, heads, kv_heads, page_tokens, q.dtype)
    _need(tcgen05 or kernel != "tcgen05",
          f"the tcgen05 prompt kernel does not take head_dim {head_dim} with pages of {page_tokens} tokens")
    if tcgen05 and kernel != "mma":
        _need(q.is_contiguous() and cache.is_contiguous(), "q and cache must be contiguous")
        shares = flash_key_shares(tiles * heads, int(longest_context), int(window or 0))
        partial = None
        if shares > 1:
            partial = torch.empty(tokens * heads * shares * (head_dim + 2), dtype=torch.float32, device=q.device)
        _call("mxb_flash_prefill_tcgen05", q.data_ptr(), cache.data_ptr(), out.data_ptr(),
              block_tables.data_ptr(), block_tables.shape[1], tile_request.data_ptr(), tile_start.data_ptr(),
              tile_length.data_ptr(), positions.data_ptr(), tokens, tiles, heads, kv_heads, head_dim,
              page_tokens, num_pages, int(window or 0), float(scale), _CODES[q.dtype], shares, _ptr(partial),
              status_word(q.device).data_ptr(), _stream())
        if shares > 1:
            global _launches
            _launches += 1   # the kernel that puts the shares together
        return out
    _call("mxb_flash_prefill", q.data_ptr(), cache.data_ptr(), out.data_ptr(), block_tables.data_ptr(),
          block_tables.shape[1], tile_request.data_ptr(), tile_start.data_ptr(), tile_length.data_ptr(),
          positions.data_ptr(), tiles, heads, kv_heads, head_dim, page_tokens, num_pages,
          int(window or 0), float(scale), _CODES[q.dtype], status_word(q.device).data_ptr(), _stream())
    return out


def decode_attention_supported(head_dim: int, heads: int, kv_heads: int, dtype: torch.dtype) -> bool:
    """Whether the split-key decode kernel takes this head layout."""
    if dtype not in _CODES:
        return False
    return bool(_fn("mxb_paged_attention_decode_supported")(head_dim, heads, kv_heads, _CODES[dtype]))


def decode_split_keys() -> int:
    return _fn("mxb_paged_attention_split_keys")()


def set_decode_resident_blocks(blocks: int, many: int = 2048) -> None:
    """How many blocks of the bfloat16 decode attention the GPU holds at once
    (444: three on each of 148 SMs), and into how many blocks a step with more
    (token, key/value head) pairs than that is cut (2,048). A pair gets that
    many blocks divided by the number of pairs, each walking over its 128-key
    tiles; where a block would be left fewer than two tiles, and with
    ``blocks`` 0, every tile has a block of its own. For comparisons and tests."""
    _need(_fn("mxb_set_decode_resident_blocks")(int(blocks), int(many)) == 0,
          "the number of resident blocks cannot be negative nor exceed that of a step with many pairs")


def paged_attention_decode(q: torch.Tensor, cache: torch.Tensor, out: torch.Tensor,
                           block_tables: torch.Tensor, row_token: torch.Tensor,
                           row_request: torch.Tensor, positions: torch.Tensor, scale: float,
                           longest_context: int, window: int = 0,
                           partial: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Attention of single tokens over their requests' cached keys, split
    along the keys. ``row_token[i]`` is the token (row of q and out) of the
    i-th decoded request, negative for a padding row; ``row_request[i]`` its
    row of ``block_tables``. ``longest_context`` bounds positions + 1 and
    fixes the number of splits. ``partial`` is float32 scratch of
    rows * heads * splits * (head_dim + 2) values, allocated here if absent."""
    dtype = q.dtype
    _check(q, "q", tuple(_CODES), 3)
    _check(out, "out", (dtype,), 3)
    _check(cache, "cache", (dtype,), 5)
    _need(out.shape == q.shape, "out and q differ in shape")
    tokens, heads, head_dim = q.shape
    num_pages, two, kv_heads, page_tokens, cache_dim = cache.shape
    _need(two == 2 and cache_dim == head_dim, "cache must be [pages, 2, kv_heads, page_tokens, head_dim]")
    _need(decode_attention_supported(head_dim, heads, kv_heads, dtype),
          f"the split-key decode kernel does not take head_dim {head_dim} with {heads}/{kv_heads} heads in {dtype}")
    _check(block_tables, "block_tables", (torch.int32,), 2)
    for name, tensor in (("row_token", row_token), ("row_request", row_request), ("positions", positions)):
        _check(tensor, name, (torch.int32,), 1)
    rows = row_token.numel()
    _need(row_request.numel() == rows and positions.numel() == tokens, "row lists do not fit")
    splits = max(1, -(-int(longest_context) // decode_split_keys()))
    need = rows * heads * splits * (head_dim + 2)
    if partial is None:
        partial = torch.empty(need, dtype=torch.float32, device=q.device)
    _check(partial, "partial", (torch.float32,))
    _need(partial.numel() >= need, f"partial holds {partial.numel()} values, {need} are needed")
    _call("mxb_paged_attention_decode", q.data_ptr(), cache.data_ptr(), out.data_ptr(), partial.data_ptr(),
          block_tables.data_ptr(), block_tables.shape[1], row_token.data_ptr(), row_request.data_ptr(),
          positions.data_ptr(), rows, heads, kv_heads, head_dim, page_tokens, num_pages, splits,
          int(window or 0), float(scale), _CODES[dtype], status_word(q.device).data_ptr(), _stream())
    return out


def decode_project_supported(head_dim: int, heads: int, kv_heads: int, dtype: torch.dtype, tokens: int,
                             weight: torch.Tensor) -> bool:
    """Whether ``paged_attention_decode_project`` takes this shape."""
    if dtype not in _CODES or weight.dtype != torch.bfloat16 or weight.dim() != 2 or weight.stride(1) != 1:
        return False
    return bool(_fn("mxb_paged_attention_decode_project_supported")(
        head_dim, heads, kv_heads, _CODES[dtype], tokens, weight.data_ptr(), weight.stride(0)))


def paged_attention_decode_project(q: torch.Tensor, cache: torch.Tensor, block_tables: torch.Tensor,
                                   row_token: torch.Tensor, row_request: torch.Tensor, positions: torch.Tensor,
                                   scale: float, longest_context: int, weight: torch.Tensor,
                                   window: int = 0) -> torch.Tensor:
    """``paged_attention_decode`` followed at once by the output projection
    ``weight`` ``[hidden, heads * head_dim]``, for steps of up to 64 tokens in
    bfloat16. Returns float32 ``[heads, tokens, hidden]``: the projection's sum
    over k left in one summand per head, for ``add_rmsnorm`` to add up."""
    _check(q, "q", (torch.bfloat16,), 3)
    _check(cache, "cache", (torch.bfloat16,), 5)
    tokens, heads, head_dim = q.shape
    num_pages, two, kv_heads, page_tokens, cache_dim = cache.shape
    _need(two == 2 and cache_dim == head_dim, "cache must be [pages, 2, kv_heads, page_tokens, head_dim]")
    _need(weight.is_cuda and weight.dim() == 2 and weight.shape[1] == heads * head_dim, "weight does not fit the heads")
    _need(decode_project_supported(head_dim, heads, kv_heads, q.dtype, tokens, weight),
          f"the decode kernel with the projection does not take {tokens} tokens of {heads}/{kv_heads} heads of {head_dim}")
    _check(block_tables, "block_tables", (torch.int32,), 2)
    for name, tensor in (("row_token", row_token), ("row_request", row_request), ("positions", positions)):
        _check(tensor, name, (torch.int32,), 1)
    rows = row_token.numel()
    _need(row_request.numel() == rows and positions.numel() == tokens, "row lists do not fit")
    splits = max(1, -(-int(longest_context) // decode_split_keys()))
    partial = torch.empty(rows * heads * splits * (head_dim + 2), dtype=torch.float32, device=q.device)
    hidden = weight.shape[0]
    summands = torch.empty((heads, tokens, hidden), dtype=torch.float32, device=q.device)
    _call("mxb_paged_attention_decode_project", q.data_ptr(), cache.data_ptr(), partial.data_ptr(),
          block_tables.data_ptr(), block_tables.shape[1], row_token.data_ptr(), row_request.data_ptr(),
          positions.data_ptr(), rows, tokens, heads, kv_heads, head_dim, page_tokens, num_pages, splits,
          int(window or 0), float(scale), weight.data_ptr(), weight.stride(0), hidden, summands.data_ptr(),
          status_word(q.device).data_ptr(), _stream())
    return summands


# ------------------------------------------------------------ matrix products
def gemm_simple(a: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """a [m, k] times w [n, k] transposed on CUDA cores, float32 accumulation
    in a fixed order."""
    _need(a.is_cuda and w.is_cuda, "operands must be on a CUDA device")
    _need(a.dim() == 2 and w.dim() == 2 and a.shape[1] == w.shape[1], "shapes do not match a @ w.T")
    _need(a.dtype == w.dtype and a.dtype in _CODES, "operands must share float32 or bfloat16")
    _need(a.stride(1) == 1 and w.stride(1) == 1, "rows must be contiguous")
    out_dtype = out_dtype or a.dtype
    m, k = a.shape
    n = w.shape[0]
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype, device=a.device)
    _need(out.shape == (m, n) and out.dtype == out_dtype and out.stride(1) == 1, "out does not fit")
    _call("mxb_gemm_simple", out.data_ptr(), _CODES[out_dtype], a.data_ptr(), w.data_ptr(),
          _CODES[a.dtype], m, n, k, a.stride(0), w.stride(0), out.stride(0), _stream())
    return out


# Up to this many rows "auto" takes the weight-streaming kernel; beyond it every
# block would re-read too much of x and the library product is faster.
SKINNY_ROWS = 16


def gemm_skinny_supported(a: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the weight-streaming kernel takes a [m, k] times w [n, k]
    transposed: bfloat16, at most 64 rows, k a multiple of 32, rows on 16-byte
    boundaries."""
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or a.dim() != 2 or w.dim() != 2:
        return False
    if a.stride(1) != 1 or w.stride(1) != 1 or a.data_ptr() % 16 or w.data_ptr() % 16:
        return False
    return bool(_fn("mxb_gemm_skinny_supported")(a.shape[0], w.shape[0], a.shape[1], a.stride(0), w.stride(0)))


STREAM_COLUMNS = 16384   # wider outputs (the vocabulary) keep the load-based kernel: enough blocks hide its latency


def gemm_stream_supported(a: torch.Tensor, w: torch.Tensor, swiglu: bool = False) -> bool:
    """Whether the bulk-copy weight-streaming kernel takes a [m, k] times w
    [n, k] transposed: bfloat16, at most 16 rows, k a multiple of 16, rows on
    16-byte boundaries, a block's rows of w and a fitting shared memory."""
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or a.dim() != 2 or w.dim() != 2:
        return False
    if a.stride(1) != 1 or w.stride(1) != 1 or a.data_ptr() % 16 or w.data_ptr() % 16:
        return False
    n = w.shape[0]
    if swiglu and n % 2:
        return False
    return bool(_fn("mxb_gemm_stream_supported")(a.shape[0], n, a.shape[1], a.stride(0), w.stride(0),
                                                 n // 2 if swiglu else 0))


# With rows of W longer than STREAM_K the load-based kernel is ahead of the
# library up to this many columns (at 1 / 8 rows 3.2 / 3.1 against 2.5 / 2.7 TB/s
# on 4,096 x 4,096, 4.1 / 3.9 against 3.1 / 3.3 on 4,096 x 12,288) and behind it
# from 5,120 columns on (4.4 / 4.1 against 4.8 / 4.8 TB/s on 5,120 x 8,192, 5.2 /
# 5.0 against 5.7 / 5.8 on 5,120 x 25,600, 4.3 / 4.1 against 4.8 / 5.1 on 10,240 x
# 5,120), until the width of a vocabulary gives it thousands of blocks.
LOAD_COLUMNS = 4096
STREAM_K = 3072   # beyond this k the load-based kernel reads W faster than whole rows by bulk copy


def gemm_skinny_takes(a: torch.Tensor, w: torch.Tensor, swiglu: bool = False) -> bool:
    """Whether one of the two weight-streaming kernels takes the call."""
    return gemm_stream_supported(a, w, swiglu) or gemm_skinny_supported(a, w)


def gemm_skinny(a: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16,
                swiglu: bool = False, out: Optional[torch.Tensor] = None, kernel: str = "auto") -> torch.Tensor:
    """a [m <= 64, k] times w [n, k] transposed, reading w once. With
    ``swiglu`` w holds gate rows then up rows and the result is
    silu(gate) * up, [m, n / 2]. ``kernel``: "stream" (rows of w by bulk copy
    into shared memory, m <= 16), "load" (16-byte loads into registers) or
    "auto": stream where it takes the shape, the output is not wider than
    STREAM_COLUMNS and k is at most STREAM_K (the layers of a small model,
    where fetching W ahead of the wait for x is what counts; with the long
    rows of a large model the loads read faster: 4.8 against 3.2 TB/s on
    [8, 25600] x [5120, 25600])."""
    _need(a.is_cuda and w.is_cuda and a.shape[1] == w.shape[1], "operands do not fit a @ w.T on a CUDA device")
    _need(kernel in ("auto", "stream", "load"), f"unknown weight-streaming kernel {kernel!r}")
    streams = kernel != "load" and gemm_stream_supported(a, w, swiglu)
    _need(streams or kernel != "stream", "the bulk-copy kernel does not take this shape")
    _need(streams or gemm_skinny_supported(a, w), "the weight-streaming kernels take bfloat16, at most 64 rows, "
          "k a multiple of 32 (16 up to 16 rows) and rows on 16-byte boundaries")
    _need(out_dtype in (torch.bfloat16, torch.float32), "out_dtype must be bfloat16 or float32")
    m, k = a.shape
    n = w.shape[0]
    _need(not swiglu or n % 2 == 0, "gate and up rows must pair up")
    columns = n // 2 if swiglu else n
    if out is None:
        out = torch.empty((m, columns), dtype=out_dtype, device=a.device)
    _need(out.shape == (m, columns) and out.dtype == out_dtype and out.stride(1) == 1, "out does not fit")
    loads = gemm_skinny_supported(a, w)
    if streams and (kernel == "stream" or not loads or (columns <= STREAM_COLUMNS and k <= STREAM_K)):
        _call("mxb_gemm_stream", out.data_ptr(), _CODES[out_dtype], a.data_ptr(), w.data_ptr(), m, n, k,
              a.stride(0), w.stride(0), out.stride(0), columns if swiglu else 0,
              status_word(a.device).data_ptr(), _stream())
        return out
    _call("mxb_gemm_skinny", out.data_ptr(), _CODES[out_dtype], a.data_ptr(), w.data_ptr(), m, n, k,
          a.stride(0), w.stride(0), out.stride(0), columns if swiglu else 0, _stream())
    return out


def gemm_bf16(a: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16,
              backend: str = "auto", out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """bfloat16 a [m, k] times w [n, k] transposed with float32 accumulation.

    ``backend``: "skinny" is the weight-streaming kernel for at most 64 rows,
    "tcgen05" the hand-written tensor-core kernel, "cublas" the library product
    (where the reference calls a library matmul too), "simple" the plain
    CUDA-core kernel. "auto": the weight-streaming kernel up to 16 rows, else
    the library for a plain product (fused products pick the tcgen05 kernel
    themselves, see ``parts/feed_forward.py``)."""
    _need(a.is_cuda and w.is_cuda, "operands must be on a CUDA device")
    _need(a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "operands must be bfloat16")
    _need(a.dim() == 2 and w.dim() == 2 and a.shape[1] == w.shape[1], "shapes do not match a @ w.T")
    _need(out_dtype in (torch.bfloat16, torch.float32), "out_dtype must be bfloat16 or float32")
    if backend == "simple":
        return gemm_simple(a, w, out_dtype=out_dtype, out=out)
    # "auto": up to 16 rows; with the long rows of a large model up to 8 (beyond
    # that the library reads them faster: 8B-shaped decode steps of 9 to 16
    # requests took 5.6 ms, of 18 to 24 requests through the library 5.0)
    few = SKINNY_ROWS if a.shape[1] <= STREAM_K else SKINNY_ROWS // 2
    if a.shape[1] > STREAM_K and LOAD_COLUMNS < w.shape[0] <= STREAM_COLUMNS:
        few = 0   # long rows and a middling width: the library reads these faster at any row count
    if (backend == "skinny" or (backend == "auto" and a.shape[0] <= few)) and gemm_skinny_takes(a, w):
        return gemm_skinny(a, w, out_dtype=out_dtype, out=out)
    _need(backend != "skinny", "the weight-streaming kernel does not take this shape")
    if backend == "tcgen05":
        from . import tensor_core
        _need(tensor_core.supports(a, w, out_dtype), "the tcgen05 kernel does not take this call: "
              + tensor_core.why_not(a, w, out_dtype))
        return tensor_core.gemm(a, w, out_dtype=out_dtype, out=out)
    if backend not in ("auto", "cublas"):
        raise KernelError(f"unknown gemm backend {backend!r}")
    # "auto" beyond the few rows of a decode step: a plain product goes to the
    # library, as in the reference (its 2-SM tiles beat the one-SM tcgen05
    # kernel here by 1.2x to 2x on this model's shapes); the tcgen05 kernel runs
    # where the product is fused with what follows it (SwiGLU).
    if out_dtype == torch.float32:
        result = torch.mm(a, w.t(), out_dtype=torch.float32)
    else:
        result = torch.mm(a, w.t())
    if out is not None:
        out.copy_(result)
        return out
    return result


def silu_mul(gate_up: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t, i] = silu(gate_up[t, i]) * gate_up[t, I + i], float32 inside."""
    _check(gate_up, "gate_up", tuple(_CODES), 2)
    tokens, width = gate_up.shape
    _need(width % 2 == 0, "gate_up must hold gate and up side by side")
    inter = width // 2
    if out is None:
        out = torch.empty((tokens, inter), dtype=gate_up.dtype, device=gate_up.device)
    _check(out, "out", (gate_up.dtype,), 2)
    _need(out.shape == (tokens, inter), "out has the wrong shape")
    _call("mxb_silu_mul", out.data_ptr(), gate_up.data_ptr(), _CODES[gate_up.dtype], tokens, inter,
          _stream())
    return out


# -------------------------------------------------------------------- picking
def _logit_rows(logits: torch.Tensor):
    _need(logits.is_cuda and logits.dtype == torch.float32 and logits.dim() == 2 and logits.stride(1) == 1,
          "logits must be CUDA float32 [rows, vocab] with contiguous rows")
    _need(logits.shape[0] <= 65535, f"the pick kernels take up to 65535 rows at a time, not {logits.shape[0]}")
    return logits.shape[0], logits.shape[1], logits.stride(0)


def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Lowest index of each row's maximum; -1 and a status bit for a row with
    a non-finite value."""
    rows, vocab, stride = _logit_rows(logits)
    if out is None:
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    _check(out, "out", (torch.int32,), 1)
    # the first pass leaves one (value, index) pair per piece of a row here
    scratch = torch.empty(rows * _fn("mxb_argmax_pieces")(rows, vocab), dtype=torch.int64, device=logits.device)
    _call("mxb_argmax", logits.data_ptr(), stride, rows, vocab, out.data_ptr(), scratch.data_ptr(),
          status_word(logits.device).data_ptr(), _stream())
    global _launches
    _launches += 1   # two kernels
    return out


def sample_icdf(logits: torch.Tensor, temperature: torch.Tensor, seed: torch.Tensor,
                stream_id: torch.Tensor, position: torch.Tensor, legal: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Inverse-CDF temperature sampling in token-id order, float64 weights;
    the uniform of row r is a function of (seed[r], stream_id[r], position[r])."""
    rows, vocab, stride = _logit_rows(logits)
    _check(temperature, "temperature", (torch.float64,), 1)
    _check(seed, "seed", (torch.int64, torch.uint64), 1)
    _check(stream_id, "stream_id", (torch.int64, torch.uint64), 1)
    _check(position, "position", (torch.int32,), 1)
    _need(temperature.numel() == rows and seed.numel() == rows and stream_id.numel() == rows
          and position.numel() == rows, "one temperature, seed, stream and position per row")
    if legal is not None:
        _check(legal, "legal", (torch.uint8, torch.bool), 2)
        _need(legal.shape == (rows, vocab), "legal must be [rows, vocab]")
    if out is None:
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    # per piece of a row: its maximum, its weight, its last id of positive weight
    scratch = torch.empty(3 * rows * _fn("mxb_icdf_pieces")(vocab), dtype=torch.int64, device=logits.device)
    _call("mxb_sample_icdf", logits.data_ptr(), stride, rows, vocab, temperature.data_ptr(),
          seed.data_ptr(), stream_id.data_ptr(), position.data_ptr(), _ptr(legal), out.data_ptr(),
          scratch.data_ptr(), status_word(logits.device).data_ptr(), _stream())
    global _launches
    _launches += 2   # three kernels
    return out


def sample_race(logits: torch.Tensor, temperature: torch.Tensor, seed: torch.Tensor,
                position: torch.Tensor, legal: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Gumbel-max sampling with Philox noise keyed by (seed, position, id)."""
    rows, vocab, stride = _logit_rows(logits)
    _check(temperature, "temperature", (torch.float64,), 1)
    _check(seed, "seed", (torch.int64, torch.uint64), 1)
    _check(position, "position", (torch.int32,), 1)
    _need(temperature.numel() == rows and seed.numel() == rows and position.numel() == rows,
          "one temperature, seed and position per row")
    if legal is not None:
        _check(legal, "legal", (torch.uint8, torch.bool), 2)
        _need(legal.shape == (rows, vocab), "legal must be [rows, vocab]")
    if out is None:
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    scratch = torch.empty(2 * rows * _fn("mxb_argmax_pieces")(rows, vocab), dtype=torch.int64, device=logits.device)
    _call("mxb_sample_race", logits.data_ptr(), stride, rows, vocab, temperature.data_ptr(),
          seed.data_ptr(), position.data_ptr(), _ptr(legal), out.data_ptr(), scratch.data_ptr(),
          status_word(logits.device).data_ptr(), _stream())
    global _launches
    _launches += 1   # two kernels
    return out


def nucleus_mask(logits: torch.Tensor, temperature: torch.Tensor, top_p: torch.Tensor,
                 top_k: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """uint8 [rows, vocab]: 1 where a token is inside the row's top-k then
    top-p nucleus (descending logit, lower id first on ties)."""
    rows, vocab, stride = _logit_rows(logits)
    _check(temperature, "temperature", (torch.float64,), 1)
    _check(top_p, "top_p", (torch.float64,), 1)
    _check(top_k, "top_k", (torch.int32,), 1)
    _need(temperature.numel() == rows and top_p.numel() == rows and top_k.numel() == rows,
          "one temperature, top_p and top_k per row")
    _need(vocab <= 1 << 22, f"the top-k/top-p kernel takes vocabularies up to {1 << 22} ids, not {vocab}")
    if out is None:
        out = torch.empty((rows, vocab), dtype=torch.uint8, device=logits.device)
    _check(out, "out", (torch.uint8,), 2)
    _call("mxb_nucleus_mask", logits.data_ptr(), stride, rows, vocab, temperature.data_ptr(),
          top_p.data_ptr(), top_k.data_ptr(), out.data_ptr(), status_word(logits.device).data_ptr(),
          _stream())
    return out
