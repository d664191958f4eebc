"""Reference-ABI entry points (mongoose_*) against the CPU oracle, through the C ABI."""
import numpy as np
import pytest

from mongoose_b200 import kernels as K
from tests.util import assert_close

pytestmark = pytest.mark.gpu


def dev(t, a):
    return t.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("seq,dim", [(1, 896), (3, 130), (1, 4864), (2, 32)])
def test_rmsnorm_family(cuda, oracle, mglib, seq, dim):
    t = cuda
    rng = np.random.default_rng(dim)
    x = rng.standard_normal((seq, dim)).astype(np.float32)
    b = rng.standard_normal((seq, dim)).astype(np.float32)
    w = (1 + 0.1 * rng.standard_normal(dim)).astype(np.float32)
    want = np.stack([oracle.rmsnorm(x[i], w) for i in range(seq)])
    dx, dw = dev(t, x), dev(t, w)
    out = t.empty_like(dx)
    K.KRMSNormOut(dx, out, dw, seq, dim)
    t.cuda.synchronize()
    assert_close(out.cpu().numpy(), want, 1e-5, "rmsnorm_out")
    assert np.array_equal(dx.cpu().numpy(), x), "input must not be modified"
    K.KRMSNorm(dx, dw, seq, dim)
    t.cuda.synchronize()
    assert_close(dx.cpu().numpy(), want, 1e-5, "rmsnorm in place")
    want2 = np.stack([oracle.rmsnorm(x[i] + b[i], w) for i in range(seq)])
    da, db = dev(t, x), dev(t, b)
    K.KFusedAddRMSNorm(da, db, out, dw, seq, dim)
    t.cuda.synchronize()
    assert_close(out.cpu().numpy(), want2, 1e-5, "fused_add_rmsnorm")


@pytest.mark.parametrize("n", [1, 255, 4864, 100003])
def test_elementwise(cuda, oracle, mglib, n):
    t = cuda
    rng = np.random.default_rng(n)
    a = rng.standard_normal(n).astype(np.float32) * 3
    b = rng.standard_normal(n).astype(np.float32)
    da, db = dev(t, a), dev(t, b)
    out = t.empty_like(da)
    K.KSiLUGateMul(da, db, out, n)
    t.cuda.synchronize()
    assert_close(out.cpu().numpy(), oracle.silu_gate_mul(a, b), 1e-6, "silu_gate_mul")
    K.KAddInPlace(da, db, n)
    t.cuda.synchronize()
    assert np.array_equal(da.cpu().numpy(), a + b)
    K.KReLU(da, n)
    t.cuda.synchronize()
    assert np.array_equal(da.cpu().numpy(), np.maximum(a + b, 0))
    h = t.empty(n, dtype=t.float16, device="cuda")
    K.KFP32ToFP16(db, h, n)
    back = t.empty(n, dtype=t.float32, device="cuda")
    K.KFP16ToFP32(h, back, n)
    t.cuda.synchronize()
    assert np.array_equal(h.cpu().numpy().view(np.uint16), oracle.f32_to_f16_bits(b))
    assert np.array_equal(back.cpu().numpy(), oracle.f16_bits_to_f32(oracle.f32_to_f16_bits(b)))
    z = t.ones(n, device="cuda")
    K.KZero(z, n * 4)
    K.KCopy(back, da, n * 4)
    K.KSync()
    assert float(z.abs().sum()) == 0.0 and t.equal(back, da)


def test_embedding_gathers(cuda, mglib):
    t = cuda
    rng = np.random.default_rng(0)
    emb = rng.standard_normal((50, 96)).astype(np.float32)
    pe = rng.standard_normal((7, 96)).astype(np.float32)
    ids = rng.integers(0, 50, 7).astype(np.int32)
    out = t.empty(7, 96, device="cuda")
    K.KEmbeddingGather(out, dev(t, emb), dev(t, pe), dev(t, ids), 7, 96)
    t.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), emb[ids] + pe)
    K.KEmbedGather(out, dev(t, emb), dev(t, ids), 7, 96)
    t.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), emb[ids])


@pytest.mark.parametrize("hd,nh,theta", [(64, 14, 1e6), (128, 4, 1e6), (32, 3, 1e4)])
def test_rope_decode_call_pattern(cuda, oracle, mglib, hd, nh, theta):
    """The decode path offsets the table pointers by pos*half and passes seqLen=1
    (cuda_fused_infer.go:423-426)."""
    t = cuda
    c, s = oracle.rope_tables(40, hd, theta)
    x = np.random.default_rng(hd).standard_normal(nh * hd).astype(np.float32)
    dc, ds, dx = dev(t, c), dev(t, s), dev(t, x)
    pos, half = 23, hd // 2
    K.KRoPE(dx, dc.data_ptr() + pos * half * 4, ds.data_ptr() + pos * half * 4, 1, nh * hd, hd, nh)
    t.cuda.synchronize()
    assert_close(dx.cpu().numpy(), oracle.rope(x, c[pos], s[pos], hd, nh), 1e-6, "rope")
    # sequence form: row i uses table row i
    xs = np.random.default_rng(1).standard_normal((5, nh * hd)).astype(np.float32)
    dxs = dev(t, xs)
    K.KRoPE(dxs, dc, ds, 5, nh * hd, hd, nh)
    t.cuda.synchronize()
    want = np.stack([oracle.rope(xs[i], c[i], s[i], hd, nh) for i in range(5)])
    assert_close(dxs.cpu().numpy(), want, 1e-6, "rope seq")


def test_kv_cache_write(cuda, mglib):
    t = cuda
    cache = t.zeros(10, 128, device="cuda")
    src = t.arange(128, device="cuda", dtype=t.float32)
    K.KKVCacheWrite(cache, src, 6, 128)
    t.cuda.synchronize()
    c = cache.cpu().numpy()
    assert np.array_equal(c[6], np.arange(128)) and c[:6].sum() == 0 and c[7:].sum() == 0


@pytest.mark.parametrize("cache_len,hd,nh,nkv", [(1, 64, 14, 2), (33, 64, 14, 2), (232, 64, 14, 2),
                                                 (300, 128, 8, 2), (1024, 64, 32, 4), (5, 32, 4, 4)])
def test_decode_attention_f32(cuda, oracle, mglib, cache_len, hd, nh, nkv):
    t = cuda
    rng = np.random.default_rng(cache_len)
    q = rng.standard_normal(nh * hd).astype(np.float32)
    k = rng.standard_normal((cache_len + 3, nkv * hd)).astype(np.float32)
    v = rng.standard_normal((cache_len + 3, nkv * hd)).astype(np.float32)
    out = t.full((nh * hd + 8,), 7.0, device="cuda")
    K.KDecodeAttention(dev(t, q), dev(t, k), dev(t, v), out, cache_len, nh * hd, nkv * hd, nh, nkv)
    t.cuda.synchronize()
    o = out.cpu().numpy()
    assert np.all(o[nh * hd:] == 7.0), "wrote past the output"
    assert_close(o[:nh * hd], oracle.decode_attention(q, k, v, cache_len, nh, nkv), 1e-5, "decode_attention")


@pytest.mark.parametrize("N,K_", [(896, 896), (128, 896), (4864, 896), (896, 4864), (5, 40), (1, 32), (33, 100)])
def test_rowq8_matvec(cuda, oracle, mglib, N, K_):
    t = cuda
    rng = np.random.default_rng(N * 7 + K_)
    w = (rng.standard_normal((N, K_)) * 0.02).astype(np.float32)
    q, s = oracle.quantize_rowq8(w)
    x = rng.standard_normal(K_).astype(np.float32)
    out = t.full((N + 4,), 9.0, device="cuda")
    K.KQ8Matvec(dev(t, x), dev(t, q), dev(t, s), out, N, K_)
    t.cuda.synchronize()
    o = out.cpu().numpy()
    assert np.all(o[N:] == 9.0)
    assert_close(o[:N], oracle.rowq8_matvec(x, q, s), 1e-5, "q8_matvec")


@pytest.mark.parametrize("N,K_", [(896, 896), (4864, 896), (896, 4864), (3, 64), (7, 36)])
def test_rowq4_matvec(cuda, oracle, mglib, N, K_):
    t = cuda
    rng = np.random.default_rng(N + K_)
    packed = rng.integers(0, 256, (N, K_ // 2), dtype=np.uint8)
    s = np.abs(rng.standard_normal(N)).astype(np.float32) * 0.1
    x = rng.standard_normal(K_).astype(np.float32)
    out = t.empty(N, device="cuda")
    K.KQ4Matvec(dev(t, x), dev(t, packed), dev(t, s), out, N, K_)
    t.cuda.synchronize()
    assert_close(out.cpu().numpy(), oracle.rowq4_matvec(x, packed, s), 1e-5, "q4_matvec")
