"""Block-32 quantized matvecs on raw caller-owned blocks, through the C ABI."""
import numpy as np
import pytest

from mongoose_b200 import kernels as K
from oracle import gen
from tests.util import assert_close

pytestmark = pytest.mark.gpu


def dev(t, a):
    return t.from_numpy(np.ascontiguousarray(a)).cuda()


def test_single_op_config_q8_0(cuda, oracle, mglib):
    """W 4864x896 Q8_0, x ~ N(0,1), seed 0: the single-op configuration."""
    t = cuda
    blocks, x = gen.single_matvec_case(0)
    out = t.empty(4864, device="cuda")
    K.KQ8_0Matvec(dev(t, x), dev(t, blocks), out, 4864, 896)
    t.cuda.synchronize()
    assert_close(out.cpu().numpy(), oracle.matvec(oracle.FMT_Q8_0, blocks, x, 4864, 896), 1e-4, "q8_0 matvec")


@pytest.mark.parametrize("N,K_", [(896, 896), (4864, 896), (896, 4864), (1, 32), (5, 96), (151, 2048)])
@pytest.mark.parametrize("fmt", [0, 1])
def test_raw_block_matvec(cuda, oracle, mglib, N, K_, fmt):
    t = cuda
    rng = np.random.default_rng(N * 13 + K_ + fmt)
    w = (rng.standard_normal((N, K_)) * 0.02).astype(np.float32)
    blocks = oracle.quantize(fmt, w)
    x = rng.standard_normal(K_).astype(np.float32)
    out = t.full((N + 2,), 5.0, device="cuda")
    (K.KQ8_0Matvec if fmt == 0 else K.KQ4_0Matvec)(dev(t, x), dev(t, blocks), out, N, K_)
    t.cuda.synchronize()
    o = out.cpu().numpy()
    assert np.all(o[N:] == 5.0)
    assert_close(o[:N], oracle.matvec(fmt, blocks, x, N, K_), 1e-4, "raw block matvec")


def _act_blocks(raw, nb):
    r = raw.reshape(nb, 40)
    d = r[:, 0:4].copy().view(np.float32)[:, 0]
    s = r[:, 4:8].copy().view(np.float32)[:, 0]
    q = r[:, 8:].copy().view(np.int8)
    return d, s, q


def test_quantize_act_blocks(cuda, mglib):
    t = cuda
    K_ = 896
    x = np.random.default_rng(5).standard_normal(K_).astype(np.float32)
    x[64:96] = 0.0                      # an all-zero block must give d = 0, q = 0
    scratch = t.zeros(K_ // 32 * 40, dtype=t.uint8, device="cuda")
    K.KQ8QuantizeAct(dev(t, x), scratch, K_)
    t.cuda.synchronize()
    d, s, q = _act_blocks(scratch.cpu().numpy(), K_ // 32)
    xb = x.reshape(-1, 32)
    amax = np.abs(xb).max(1)
    assert np.allclose(d, amax / 127.0, rtol=1e-6)
    assert np.all(q[2] == 0) and d[2] == 0
    assert np.abs(q * d[:, None] - xb).max() <= (d.max() * 0.5 + 1e-7)
    assert np.allclose(s, d * q.sum(1), rtol=1e-6, atol=1e-7)


@pytest.mark.parametrize("N,K_", [(896, 896), (896, 4864), (64, 64)])
def test_q4_0_dp4a_family(cuda, oracle, mglib, N, K_):
    """Integer-dot variants: the activation is rounded to int8 per block, so the result carries
    that quantization error (about 1e-2 relative); checked exactly against an integer model of
    the same arithmetic and loosely against the fp32-activation oracle."""
    t = cuda
    rng = np.random.default_rng(N + K_)
    w = (rng.standard_normal((N, K_)) * 0.02).astype(np.float32)
    blocks = oracle.quantize(oracle.FMT_Q4_0, w)
    x = rng.standard_normal(K_).astype(np.float32)
    dx, dw = dev(t, x), dev(t, blocks)
    nb = K_ // 32
    scratch = t.zeros(nb * 40, dtype=t.uint8, device="cuda")
    out = t.empty(N, device="cuda")
    K.KQ4_0MatvecDP4A(dx, dw, out, N, K_, scratch)
    t.cuda.synchronize()
    got = out.cpu().numpy()
    d, s, q = _act_blocks(scratch.cpu().numpy(), nb)
    xq = (q.astype(np.float64) * d[:, None].astype(np.float64)).reshape(-1)
    wd = oracle.dequant(oracle.FMT_Q4_0, blocks, N, K_).astype(np.float64)
    assert_close(got, wd @ xq, 1e-4, "dp4a vs integer model")
    assert_close(got, oracle.matvec(oracle.FMT_Q4_0, blocks, x, N, K_), 3e-2, "dp4a vs fp32 activations")
    out2 = t.empty(N, device="cuda")
    K.KQ4_0MatvecDP4APreq(dw, scratch, out2, N, K_)
    t.cuda.synchronize()
    assert np.array_equal(out2.cpu().numpy(), got)
    # batch of 3 activations
    xs = rng.standard_normal((3, K_)).astype(np.float32)
    sb = t.zeros(3 * nb * 40, dtype=t.uint8, device="cuda")
    K.KQ8QuantizeActBatch(dev(t, xs), sb, K_, 3)
    ob = t.empty(3, N, device="cuda")
    K.KQ4_0MatvecDP4ABatch(dw, sb, ob, N, K_, 3)
    t.cuda.synchronize()
    for i in range(3):
        assert_close(ob[i].cpu().numpy(), oracle.matvec(oracle.FMT_Q4_0, blocks, xs[i], N, K_), 3e-2, "dp4a batch")
