"""The allocation-free allocator entry point (rdkv_knapsack_batched_static) against the
regular one, called through the C ABI.

Who needs it: code that must run the bit allocator from a place where device memory may
not be allocated any more — an inference engine whose memory plan is frozen after
warm-up, a host callback, a plugin handed nothing but input and output buffers.  The
regular entry point wants a small scratch buffer from the caller; this one keeps it
inside the library.  Both must choose exactly the same bits.

The file name sorts last on purpose: a run that stops at the first failure has then
already been through every other test.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(static: bool, scores, budget, out, eps, max_iters=60, tol=0.01):
    from rdkv_b200 import _lib
    lib = _lib.lib()
    opts = [0.0, 2.0, 4.0, 8.0, 16.0]
    c_bits = (C.c_float * 5)(*opts)
    c_eps = (C.c_float * 5)(*[eps[int(b)] for b in opts])
    B, T = scores.shape
    stream = torch.cuda.current_stream().cuda_stream
    if static:
        st = lib.rdkv_knapsack_batched_static(scores.data_ptr(), scores.stride(0), B, T, budget.data_ptr(), c_bits,
                                              c_eps, 5, max_iters, tol, out.data_ptr(), stream)
    else:
        scratch = torch.empty(3 * B, dtype=torch.int32, device="cuda")
        st = lib.rdkv_knapsack_batched(scores.data_ptr(), scores.stride(0), B, T, budget.data_ptr(), c_bits, c_eps,
                                       5, max_iters, tol, out.data_ptr(), scratch.data_ptr(), stream)
    return st


def test_static_scratch_variant_matches_regular_entry_point_twice():
    from rdkv_b200 import _lib, synth
    eps = synth.ALLOC_EPSILON
    lib = _lib.lib()
    assert lib.rdkv_knapsack_static_max_rows() == 4096
    # two calls in a row with different shapes and budgets: the shared scratch keeps the first
    # call's contents, the second call must not be disturbed by them
    for seed, rows, T, budgets in ((31, 96, 4096, (2.0, 0.5)), (32, 17, 700, (6.0, 1.0))):
        scores = synth.make_scores(rows, T, seed=seed, device="cuda")
        budget = torch.full((rows,), budgets[0], dtype=torch.float32, device="cuda")
        budget[::3] = budgets[1]
        want = torch.empty((rows, T), dtype=torch.int64, device="cuda")
        got = torch.full((rows, T), -1, dtype=torch.int64, device="cuda")
        assert _call(False, scores, budget, want, eps) == 0
        assert _call(True, scores, budget, got, eps) == 0
        torch.cuda.synchronize()
        assert torch.equal(got, want)          # integer choices: bit-exact, like every allocator test
    # more rows than the built-in scratch holds: refused, nothing launched
    big = torch.ones((4097, 8), dtype=torch.float32, device="cuda")
    out = torch.empty((4097, 8), dtype=torch.int64, device="cuda")
    bud = torch.full((4097,), 2.0, dtype=torch.float32, device="cuda")
    assert _call(True, big, bud, out, eps) == 3
