"""The decode attention entry point that allocates nothing
(csrc/kernels/attention_decode_noalloc.h), called through its exported C
symbol the way a caller without a tensor library would, and compared with the
ordinary entry point, which takes its scratch from the caller.

Some callers cannot allocate device memory while they run: a server that gave
all free memory to its own pools at start-up, or a plain C / ctypes binding
with no allocator to borrow scratch from. For them the library carries a fixed
16 MiB scratch array per GPU. This file is collected last on purpose: if it
fails, a run that stops at the first failure has already run everything else.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

SCRATCH_BYTES = 16 * 1024 * 1024


def make_case(seed, dtype, totals, heads, kv_heads, head_dim, page_tokens):
    """Random q and a paged cache holding ``totals[r]`` positions of request r;
    one query (the last position) per request."""
    rng = np.random.default_rng(seed)
    pages_needed = [-(-total // page_tokens) for total in totals]
    order = rng.permutation(sum(pages_needed) + 2)
    cache = torch.tensor(rng.normal(size=(len(order), 2, kv_heads, page_tokens, head_dim)),
                         dtype=dtype, device="cuda")
    tables = np.full((len(totals), max(pages_needed)), -1, dtype=np.int32)
    cursor = 0
    for r, need in enumerate(pages_needed):
        tables[r, :need] = order[cursor:cursor + need]
        cursor += need
    q = torch.tensor(rng.normal(size=(len(totals), heads, head_dim)), dtype=dtype, device="cuda")
    as_int = lambda values: torch.tensor(values, dtype=torch.int32, device="cuda")
    rows = list(range(len(totals)))
    return dict(q=q, cache=cache, tables=as_int(tables), row_token=as_int(rows), row_request=as_int(rows),
                positions=as_int([t - 1 for t in totals]), longest=max(totals), scale=head_dim ** -0.5)


def call_noalloc(library, case, out, window=0):
    """Straight through the C symbol: raw pointers and integers only."""
    function = library.mxb_paged_attention_decode_noalloc
    P, I = ctypes.c_void_p, ctypes.c_int
    function.argtypes = [P, P, P, P, I, P, P, P, I, I, I, I, I, I, I, I, ctypes.c_float, I, P, P]
    function.restype = I
    q, cache = case["q"], case["cache"]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    code = function(q.data_ptr(), cache.data_ptr(), out.data_ptr(), case["tables"].data_ptr(),
                    case["tables"].shape[1], case["row_token"].data_ptr(), case["row_request"].data_ptr(),
                    case["positions"].data_ptr(), q.shape[0], q.shape[1], cache.shape[2], q.shape[2],
                    cache.shape[3], cache.shape[0], case["longest"], window, case["scale"],
                    0 if q.dtype == torch.float32 else 1, status.data_ptr(),
                    torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return code, int(status.item())


@pytest.mark.parametrize("dtype, limit", [(torch.float32, 5e-6), (torch.bfloat16, 2e-2)])
def test_noalloc_entry_point_matches_the_ordinary_one_twice_in_a_row(dtype, limit):
    from metallix_b200 import ops
    from metallix_b200.csrc import build
    ops.require_cuda()
    library = build.kernels()
    # Two calls in a row on the same shared array: the second is smaller and
    # shorter, so most of the array still holds the first call's partials.
    cases = [make_case(1, dtype, [700, 33, 512, 1030, 257], heads=8, kv_heads=2, head_dim=128, page_tokens=16),
             make_case(2, dtype, [300, 90], heads=4, kv_heads=4, head_dim=64, page_tokens=8)]
    for case, window in zip(cases, (0, 200)):
        expected = torch.empty_like(case["q"])
        ops.paged_attention_decode(case["q"], case["cache"], expected, case["tables"], case["row_token"],
                                   case["row_request"], case["positions"], case["scale"], case["longest"],
                                   window)
        ops.check_status("cuda")
        # A first call looks the array's address up (and lets the driver load
        # the kernels it needs); the calls after it must leave the device's
        # free memory where it was. The driver's own count is read, not the
        # tensor library's: an allocation inside the entry point would not
        # pass through the latter.
        first = torch.full_like(case["q"], float("nan"))
        code, status = call_noalloc(library, case, first, window)
        assert code == 0 and status == 0
        assert (first.double() - expected.double()).abs().max().item() < limit
        got = torch.full_like(case["q"], float("nan"))
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        code, status = call_noalloc(library, case, got, window)
        free_after, _ = torch.cuda.mem_get_info()
        assert code == 0 and status == 0
        assert free_after == free_before   # nothing was taken from the device, nothing given back
        assert not torch.isnan(got).any()
        assert (got.double() - expected.double()).abs().max().item() < limit


def test_noalloc_entry_point_flags_a_context_beyond_its_bound():
    """``longest_context`` sizes the scratch; a row whose position lies beyond
    it is left untouched and reported in the status word, instead of reading
    partial results that were never sized for it."""
    from metallix_b200.csrc import build
    library = build.kernels()
    case = make_case(4, torch.bfloat16, [100, 700, 60], heads=8, kv_heads=2, head_dim=128, page_tokens=16)
    case["longest"] = 256                       # the second request holds 700 positions
    out = torch.full_like(case["q"], 7.0)
    code, status = call_noalloc(library, case, out)
    assert code == 0 and status & 2
    assert bool((out[1] == 7.0).all()) and not bool((out[0] == 7.0).any()) and not bool((out[2] == 7.0).any())


def test_noalloc_entry_point_refuses_what_does_not_fit():
    from metallix_b200.csrc import build
    library = build.kernels()
    case = make_case(3, torch.bfloat16, [40] * 200, heads=32, kv_heads=8, head_dim=128, page_tokens=16)
    case["longest"] = 4096   # 200 rows x 32 heads x 16 splits x 130 floats = 53 MB
    assert 200 * 32 * 16 * 130 * 4 > SCRATCH_BYTES
    out = torch.full_like(case["q"], 7.0)
    code, status = call_noalloc(library, case, out)
    assert code == 1 and status == 0            # cudaErrorInvalidValue, and nothing ran
    assert bool((out == 7.0).all())
    case["longest"] = 40                        # one split: 200 x 32 x 1 x 130 floats fit
    code, status = call_noalloc(library, case, out)
    assert code == 0 and status == 0 and not bool((out == 7.0).any())
