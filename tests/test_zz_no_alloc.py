"""The allocation-free Q4_0 integer-dot entry point against the caller-scratch one.

Some callers may not allocate device memory when they need a matvec (allocator calls are forbidden
where they run, or their memory budget is spent), so the library carries its own fixed activation
scratch.  The result must be identical to mongoose_q4_0_matvec_dp4a, call after call, because both
run the same two kernels and differ only in where the activation blocks are kept.
Collected last on purpose: a failure here cannot hide a failure elsewhere under `pytest -x`.
"""
import numpy as np
import pytest

from mongoose_b200 import kernels as K

pytestmark = pytest.mark.gpu


def dev(t, a):
    return t.from_numpy(np.ascontiguousarray(a)).cuda()


def test_static_scratch_matches_caller_scratch_twice(cuda, oracle, mglib):
    t = cuda
    rng = np.random.default_rng(7)
    # two different shapes in a row: the second call reuses the array the first one filled
    for N, K_ in ((896, 4864), (320, 896)):
        w = (rng.standard_normal((N, K_)) * 0.02).astype(np.float32)
        blocks = dev(t, oracle.quantize(oracle.FMT_Q4_0, w))
        x = dev(t, rng.standard_normal(K_).astype(np.float32))
        want = t.empty(N, device="cuda")
        scratch = t.zeros(K_ // 32 * 40, dtype=t.uint8, device="cuda")
        K.KQ4_0MatvecDP4A(x, blocks, want, N, K_, scratch)
        got = t.full((N + 3,), -5.0, device="cuda")
        assert K.KQ4_0MatvecDP4AStatic(x, blocks, got, N, K_) == 0, K.StaticScratchError()
        t.cuda.synchronize()
        g = got.cpu().numpy()
        assert np.all(g[N:] == -5.0), "wrote past the output"
        assert np.array_equal(g[:N], want.cpu().numpy()), "same kernels, same inputs: results must be identical"
        ref = oracle.matvec(oracle.FMT_Q4_0, oracle.quantize(oracle.FMT_Q4_0, w), x.cpu().numpy(), N, K_)
        assert np.abs(g[:N] - ref).max() <= 3e-2 * np.abs(ref).max()


def test_static_scratch_rejects_oversize_and_bad_arguments(cuda, mglib):
    t = cuda
    x = t.zeros(64, device="cuda")
    out = t.zeros(4, device="cuda")
    w = t.zeros(4 * 2 * 18, dtype=t.uint8, device="cuda")
    assert K.KQ4_0MatvecDP4AStatic(x, w, out, 4, 32768 + 32) == -1
    assert "exceeds" in K.StaticScratchError()
    assert K.KQ4_0MatvecDP4AStatic(x, w, out, 4, 48) == -1          # not a multiple of 32
    assert K.KQ4_0MatvecDP4AStatic(None, w, out, 4, 64) == -1
    assert K.KQ4_0MatvecDP4AStatic(x, w, out, 4, 64) == 0 and K.StaticScratchError() == ""
    t.cuda.synchronize()
