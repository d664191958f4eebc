"""The reference's own CUDA kernels (kernels/mongoose.cu compiled unmodified for sm_100 into
oracle/_ref/libmongoose_ref.so) run on this GPU, against the oracle and against this library, on the
seeded golden cases.  This is what pins the oracle for the per-row formats and the fp32 ops."""
import os

import numpy as np
import pytest

from tests.golden import cases, make_golden
from tests.util import assert_close

pytestmark = pytest.mark.gpu
REF = os.path.join(make_golden.ROOT, "oracle", "_ref", "libmongoose_ref.so")


@pytest.fixture(scope="module")
def triple(cuda, oracle, mglib):
    if not os.path.exists(REF):
        pytest.skip("oracle/_ref/libmongoose_ref.so not built (make -C oracle ref needs the reference tree)")
    c = cases.inputs()
    ref = make_golden.run(make_golden.load_reference(), c)
    ours = make_golden.run(mglib, c)          # same call sequence through this library's symbols
    return c, ref, ours


TOL = {"q8_matvec": 2e-6, "q4_matvec": 2e-6, "rmsnorm_out": 2e-6, "fused_add_rmsnorm": 2e-6, "rope": 1e-6,
       "decode_attention": 2e-6, "silu_gate_mul": 2e-6, "add_inplace": 0.0, "kv_cache_write": 0.0}


def test_library_matches_reference_kernels(triple):
    _, ref, ours = triple
    for name, tol in TOL.items():
        if tol == 0.0:
            assert np.array_equal(ours[name], ref[name]), name
        else:
            assert_close(ours[name], ref[name], tol, name)


def test_oracle_matches_reference_kernels(triple, oracle):
    c, ref, _ = triple
    from tests.test_golden_cpu import oracle_outputs
    want = oracle_outputs(oracle, c)
    for name, tol in TOL.items():
        assert_close(want[name], ref[name], max(tol, 2e-6), name)


def test_committed_golden_vectors_are_current(triple):
    _, ref, _ = triple
    path = os.path.join(make_golden.ROOT, "tests", "golden", "ref_kernels.npz")
    g = np.load(path)
    for name in TOL:
        assert_close(g[name], ref[name], 1e-6, name)     # same kernels, same GPU family: only fp reassociation noise
