"""The decode attention entry point that allocates nothing (tgo_attention_decode_static).

Some callers of the kernels cannot allocate device memory when they call: a program that
gave the whole GPU to another memory manager or lives under a fixed budget, a serving loop
that must not take the device-wide stall of cudaMalloc and cudaFree, or C code with no
tensor allocator. For them the scratch of the split-key decode attention is an array
inside the library. This test calls that entry point through its exported C symbol, with
ctypes and raw pointers, twice in a row, and compares each result with the ordinary entry
point's, which takes its scratch from torch, and with a dense float32 attention written
with torch over the same keys and values (the two entry points share their kernels, so
agreeing with each other alone would not show an error in the arithmetic). The second call
uses other inputs and another split count, so what the first call left in the shared array
must not show.

The file sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

SCRATCH_FLOATS = 2 * 1024 * 1024
E_BAD_ARG, E_TOO_SMALL = 1000, 1001


def static_entry():
    from tgo_b200.kernels.build import load_library
    fn = load_library("attention_flash").tgo_attention_decode_static
    fn.restype = ctypes.c_int
    return fn


def call_static(fn, case, out, H, Hkv, dh, ps, scale, window, n_splits):
    vp, ll, ci = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int
    q = case["q"]
    return fn(vp(q.data_ptr()), ll(q.stride(0)), vp(out.data_ptr()), ll(out.stride(0)),
              vp(case["kc"].data_ptr()), vp(case["vc"].data_ptr()), ci(ps),
              vp(case["bt"].data_ptr()), ci(case["bt"].shape[1]), vp(case["pos"].data_ptr()),
              vp(case["seq"].data_ptr()), ci(q.shape[0]), ci(H), ci(Hkv), ci(dh),
              ctypes.c_float(scale), ci(window), ci(n_splits),
              vp(torch.cuda.current_stream().cuda_stream))


def test_static_scratch_entry_matches_the_allocating_one():
    from test_kernels_gpu import attention_ref, paged_case
    from tgo_b200.kernels import ops
    fn = static_entry()
    H, Hkv, dh, ps = 8, 2, 64, 16
    scale = 1 / math.sqrt(dh)
    for seed, firsts, n_splits, window in ((1, [700, 63, 0, 300], 5, 0), (2, [511, 64, 129, 5], 3, 100)):
        case = paged_case([1, 1, 1, 1], firsts, H, Hkv, dh, ps, torch.bfloat16, seed=seed)
        dense = attention_ref(case, H, Hkv, dh, scale, window)
        want = torch.zeros_like(case["q"])
        ops.attention_flash(case["q"], want, H, Hkv, dh, case["kc"], case["vc"], ps, case["bt"],
                            case["pos"], case["seq"], None, None, scale, window,
                            n_splits=n_splits)
        got = torch.full_like(case["q"], float("nan"))
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        rc = call_static(fn, case, got, H, Hkv, dh, ps, scale, window, n_splits)
        torch.cuda.synchronize()
        assert rc == 0
        assert torch.cuda.memory_allocated() == before          # torch was asked for nothing
        assert torch.allclose(got.float(), want.float(), rtol=2e-2, atol=2e-2)
        assert torch.allclose(got.float().cpu(), dense, rtol=2e-2, atol=2e-2)
    # one split needs no scratch at all and still works
    got = torch.zeros_like(case["q"])
    assert call_static(fn, case, got, H, Hkv, dh, ps, scale, window, 1) == 0
    torch.cuda.synchronize()
    assert torch.allclose(got.float(), want.float(), rtol=2e-2, atol=2e-2)
    assert torch.allclose(got.float().cpu(), dense, rtol=2e-2, atol=2e-2)


def test_static_scratch_entry_takes_the_largest_request_that_fits():
    """209 tokens x 8 heads x 19 splits x (64 + 2) floats = 2 096 688 of the array's 2 097 152:
    the largest request of this shape that fits (one more split would not). Every split's
    partial result lies in the array, the last one ends 464 floats before its end."""
    from test_kernels_gpu import attention_ref, paged_case
    fn = static_entry()
    H, Hkv, dh, ps, T, n_splits = 8, 2, 64, 16, 209, 19
    assert T * H * n_splits * (dh + 2) <= SCRATCH_FLOATS < T * H * (n_splits + 1) * (dh + 2)
    firsts = [(37 * i) % 150 for i in range(T)]
    case = paged_case([1] * T, firsts, H, Hkv, dh, ps, torch.bfloat16, seed=7)
    scale = 1 / math.sqrt(dh)
    dense = attention_ref(case, H, Hkv, dh, scale, 0)
    got = torch.full_like(case["q"], float("nan"))
    assert call_static(fn, case, got, H, Hkv, dh, ps, scale, 0, n_splits) == 0
    torch.cuda.synchronize()
    assert torch.allclose(got.float().cpu(), dense, rtol=2e-2, atol=2e-2)
    assert call_static(fn, case, got, H, Hkv, dh, ps, scale, 0, n_splits + 1) == E_TOO_SMALL


def test_static_scratch_entry_refuses_what_does_not_fit():
    from test_kernels_gpu import paged_case
    fn = static_entry()
    H, Hkv, dh, ps = 8, 2, 64, 16
    case = paged_case([1, 1], [40, 90], H, Hkv, dh, ps, torch.bfloat16, seed=3)
    out = torch.zeros_like(case["q"])
    too_many = SCRATCH_FLOATS // (2 * H * (dh + 2)) + 1           # splits that overflow the array
    assert call_static(fn, case, out, H, Hkv, dh, ps, 0.1, 0, too_many) == E_TOO_SMALL
    assert call_static(fn, case, out, H, Hkv, 80, ps, 0.1, 0, 2) == E_BAD_ARG    # no such head size
    torch.cuda.synchronize()
    assert not out.any()                                          # nothing was launched
