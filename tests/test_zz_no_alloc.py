"""The allocation-free entry point of the decode-step product, called through its exported C symbol.

Embedders that cannot call cudaMalloc (inside a stream capture, with the whole GPU already handed to a cache
pool, or as a plug-in that only receives pointers and a stream) use ``zi_gemm_smallm_noalloc``: its split-K
scratch lives in a static device array inside the library.  The test feeds it the same operands as the
existing entry point (whose scratch comes from torch) and expects the same output, twice in a row on the
shared scratch, with shapes that are cut into K ranges and one that is not, once with the ranges' sums forced
through the array and once the default way.  This file sorts last on purpose.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _rand(*shape, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(torch.bfloat16).to(DEV)


def _call_noalloc(lib, x, w, bias, out):
    fn = lib.zi_gemm_smallm_noalloc
    fn.restype = ctypes.c_int
    p = lambda t: ctypes.c_void_p(0 if t is None else t.data_ptr())      # noqa: E731
    m, k = x.shape
    n = w.shape[0]
    code = 0 if out.dtype == torch.float32 else 1
    rc = fn(p(x), p(w), p(bias), p(out), ctypes.c_int(code), ctypes.c_int(m), ctypes.c_int(n), ctypes.c_int(k),
            ctypes.c_longlong(x.stride(0)), ctypes.c_longlong(w.stride(0)), ctypes.c_longlong(out.stride(0)),
            ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    return rc


def _set_reduction(lib, through_array):
    fn = lib.zi_gemm_smallm_noalloc_reduction
    fn.restype = ctypes.c_int
    return fn(ctypes.c_int(1 if through_array else 0))


@pytest.mark.parametrize("through_array", [True, False])
def test_noalloc_entry_point_matches_the_existing_one_twice_in_a_row(through_array):
    """``through_array``: the sums of the K ranges are written to the built-in array, counted there and added by the
    block that arrives last, so a wrong address, offset or a counter that was not cleared shows in the output.
    Otherwise the ranges meet in distributed shared memory (what a B200 does by default) and the array is only
    cleared.  Either way the output is the existing entry point's, bit for bit, on two calls in a row."""
    from zedinfer_b200 import ops
    from zedinfer_b200.csrc import build
    lib = build.load_library("gemm_smallm")
    # (rows, outputs, K): the feed-forward's down projection is cut into K ranges; the q/k/v projection is not
    cases = [(8, 1536, 8960, True), (5, 2048, 1536, False), (16, 1536, 8960, True), (3, 3584, 18944, False)]
    before_setting = _set_reduction(lib, through_array)
    try:
        for rep in range(2):
            for m, n, k, with_bias in cases:
                x = _rand(m, k, seed=10 * rep + m)
                w = _rand(n, k, seed=100 + n + rep, scale=0.05)
                b = _rand(n, seed=7 + rep) if with_bias else None
                ref = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
                ops.gemm_smallm(x, w, b, ref)
                got = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
                before = torch.cuda.memory_allocated(DEV)
                assert _call_noalloc(lib, x, w, b, got) == 0, build.last_error("gemm_smallm")
                assert torch.cuda.memory_allocated(DEV) == before
                torch.cuda.synchronize()
                assert torch.equal(got, ref)
                exact = (x.double().cpu() @ w.double().cpu().t()) + (b.double().cpu() if b is not None else 0.0)
                assert torch.allclose(got.double().cpu(), exact, atol=6e-2, rtol=2e-2)
    finally:
        _set_reduction(lib, before_setting)


def test_noalloc_entry_point_refuses_what_its_scratch_cannot_hold():
    """N = 4,704 with K = 4,096 is cut in two: 2 * 16 * 4,704 = 150,528 floats of partial sums, more than the
    131,072 the array holds.  The same width with a short K is not cut and needs no scratch."""
    from zedinfer_b200.csrc import build
    lib = build.load_library("gemm_smallm")
    ks = lib.zi_gemm_smallm_ksplit
    ks.restype = ctypes.c_int
    assert ks(ctypes.c_int(4704), ctypes.c_int(4096), ctypes.c_int(0)) == 2
    x = _rand(4, 4096, seed=1)
    w = _rand(4704, 4096, seed=2, scale=0.05)
    out = torch.empty(4, 4704, dtype=torch.bfloat16, device=DEV)
    assert _call_noalloc(lib, x, w, None, out) != 0
    msg = build.last_error("gemm_smallm")
    assert "150528 floats" in msg and "131072" in msg, msg
    assert ks(ctypes.c_int(4704), ctypes.c_int(512), ctypes.c_int(0)) == 1
    assert _call_noalloc(lib, x[:, :512].contiguous(), w[:, :512].contiguous(), None, out) == 0
    big = _rand(17, 64, seed=3)
    assert _call_noalloc(lib, big, _rand(32, 64, seed=4), None, torch.empty(17, 32, dtype=torch.bfloat16, device=DEV)) != 0
    assert "at most 16" in build.last_error("gemm_smallm")
