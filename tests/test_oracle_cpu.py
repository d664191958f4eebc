"""CPU tests of the oracle itself: codecs, quantizers, known answers."""
import numpy as np

from mongoose_b200 import configs as mc
from oracle import gen


def test_cpu_engine_matmul_known_answer(oracle):
    # The reference's own known-answer test for the CPU engine: cpu_test.go:17-29.
    a = np.array([[1, 2, 3], [4, 5, 6]], np.float32)
    b = np.array([[7, 8], [9, 10], [11, 12]], np.float32)
    out = oracle.cpu_engine_matmul(a, b)
    assert out.tolist() == [[58.0, 64.0], [139.0, 154.0]]


def test_cpu_engine_identity(oracle):
    # cpu_test.go:31-45: multiplying by the identity returns the input.
    rng = np.random.default_rng(1)
    a = rng.standard_normal((4, 4)).astype(np.float32)
    out = oracle.cpu_engine_matmul(a, np.eye(4, dtype=np.float32))
    assert np.array_equal(out, a)


def test_rmsnorm_unit_rms(oracle):
    # cpu_test.go:78-97: with unit weights the output RMS is ~1.
    x = np.random.default_rng(2).standard_normal(896).astype(np.float32) * 3
    y = oracle.rmsnorm(x, np.ones(896, np.float32))
    assert abs(float(np.sqrt(np.mean(y.astype(np.float64) ** 2))) - 1.0) < 1e-3


def test_f16_codec_matches_ieee(oracle):
    rng = np.random.default_rng(0)
    parts = [rng.standard_normal(50000).astype(np.float32) * s for s in (1e-8, 1e-6, 1e-4, 1.0, 100.0, 30000.0)]
    parts.append(np.array([0, -0.0, 65504, 65519.9, 65520, 2 ** -24, 2 ** -25, 2 ** -25 * 1.0001, 6.1e-5],
                          np.float32))
    x = np.concatenate(parts)
    with np.errstate(over="ignore"):
        want = x.astype(np.float16).view(np.uint16)
    assert np.array_equal(oracle.f32_to_f16_bits(x), want)
    allh = np.arange(65536, dtype=np.uint16)
    got = oracle.f16_bits_to_f32(allh)
    ref = allh.view(np.float16).astype(np.float32)
    assert np.all((got == ref) | (np.isnan(got) & np.isnan(ref)))


def test_q8_0_quantizer_layout_and_rounding(oracle):
    w = np.zeros((1, 32), np.float32)
    w[0, :5] = [1.0, -1.0, 0.5, 0.0039, -0.0040]      # amax 1 -> d = 1/127
    blk = oracle.quantize(oracle.FMT_Q8_0, w)[0]
    assert blk.size == 34
    d = blk[:2].view(np.float16)[0]
    assert d == np.float16(1.0 / 127.0)
    q = blk[2:].view(np.int8)
    assert q[:5].tolist() == [127, -127, 64, 0, -1]    # 63.5 rounds away from zero; 0.495 -> 0; -0.508 -> -1
    # dequantized value is float(d) * q exactly
    dq = oracle.dequant(oracle.FMT_Q8_0, blk[None, :], 1, 32)[0]
    assert dq[0] == np.float32(d) * np.float32(127)


def test_q4_0_quantizer_layout(oracle):
    w = np.zeros((1, 32), np.float32)
    w[0, 0], w[0, 16], w[0, 1] = 8.0, -8.0, 1.0       # amax 8 -> d = 1
    blk = oracle.quantize(oracle.FMT_Q4_0, w)[0]
    assert blk.size == 18 and blk[:2].view(np.float16)[0] == np.float16(1.0)
    qs = blk[2:]
    assert qs[0] & 0xF == 15        # +8 -> 16 clamps to 15
    assert qs[0] >> 4 == 0          # -8 -> 0 : element 16 lives in the HIGH nibble of byte 0
    assert qs[1] & 0xF == 9         # element 1 in the low nibble of byte 1
    dq = oracle.dequant(oracle.FMT_Q4_0, blk[None, :], 1, 32)[0]
    assert dq[0] == 7.0 and dq[16] == -8.0 and dq[1] == 1.0


def test_rowq8_quantizer_truncates(oracle):
    # cuda_fused_infer.go:376-381: int(v * inv) truncates toward zero.
    w = np.array([[127.0, 63.9, -63.9, 0.99]], np.float32)
    q, s = oracle.quantize_rowq8(w)
    assert s[0] == np.float32(1.0) and q[0].tolist() == [127, 63, -63, 0]


def test_block_matvec_matches_dequantized_product(oracle):
    rng = np.random.default_rng(3)
    w = rng.standard_normal((96, 256)).astype(np.float32) * 0.02
    x = rng.standard_normal(256).astype(np.float32)
    for fmt in (oracle.FMT_Q8_0, oracle.FMT_Q4_0, oracle.FMT_F16):
        b = oracle.quantize(fmt, w)
        dq = oracle.dequant(fmt, b, 96, 256).astype(np.float64)
        y = oracle.matvec(fmt, b, x, 96, 256)
        assert np.abs(y - dq @ x).max() < 1e-6
        yc = oracle.cpu_engine_matvec(fmt, b, x, 96, 256, 1)
        assert np.abs(yc - dq @ x).max() < 1e-4


def test_single_matvec_case_shapes(oracle):
    blocks, x = gen.single_matvec_case(0)
    assert blocks.shape == (4864, 28 * 34) and x.shape == (896,)
    d = blocks.reshape(4864, 28, 34)[:, :, :2].copy().view(np.float16)
    assert float(d.max()) < 0.02 * 6 / 127 and float(d.min()) >= 0
    y = oracle.matvec(oracle.FMT_Q8_0, blocks, x, 4864, 896)
    assert np.all(np.isfinite(y)) and y.std() > 0


def test_rope_tables_and_rotation(oracle):
    c, s = oracle.rope_tables(16, 64, 1e6)
    assert c.shape == (16, 32) and np.all(c[0] == 1.0) and np.all(s[0] == 0.0)
    assert np.isclose(c[3, 0], np.cos(3.0)) and np.isclose(s[5, 1], np.sin(5.0 / 1e6 ** (2 / 64)))
    x = np.random.default_rng(4).standard_normal(128).astype(np.float32)
    y = oracle.rope(x, c[7], s[7], 64, 2)
    # rotation preserves the norm of every (j, j+32) pair
    xp = x.reshape(2, 2, 32); yp = y.reshape(2, 2, 32)
    assert np.allclose((xp ** 2).sum(1), (yp ** 2).sum(1), rtol=1e-5)


def test_attention_is_a_convex_combination(oracle):
    rng = np.random.default_rng(5)
    q = rng.standard_normal(128).astype(np.float32)
    k = rng.standard_normal((9, 64)).astype(np.float32)
    v = np.ones((9, 64), np.float32) * 2.5
    out = oracle.decode_attention(q, k, v, 9, 4, 2)
    assert np.allclose(out, 2.5, atol=1e-6)
    # a single cached position returns V[0] whatever the scores are
    v1 = rng.standard_normal((1, 64)).astype(np.float32)
    out1 = oracle.decode_attention(q, k[:1], v1, 1, 4, 2)
    assert np.allclose(out1.reshape(4, 32), np.repeat(v1.reshape(2, 32), 2, axis=0), atol=1e-7)


def test_bytes_per_token_match_the_survey():
    assert mc.weight_bytes_per_token(mc.QWEN25_05B) == 524_833_792
    assert mc.kv_bytes_per_position(mc.QWEN25_05B) == 12_288
    assert mc.weight_bytes_per_token(mc.QWEN25_05B_Q4) == 473_546_752   # Q4_0 layers, fp16 lm_head
    assert mc.weight_bytes_per_token(mc.QWEN25_05B.with_(layer_fmt=mc.FMT_Q4_0, head_fmt=mc.FMT_Q4_0)) == 277_853_184
    assert mc.weight_bytes_per_token(mc.TINYLLAMA_11B) == 1_099_071_488
    assert mc.weight_bytes_per_token(mc.QWEN25_7B) == 7_512_178_688
    assert mc.QWEN25_05B.num_weights == 24 * 12 + 2


def test_oracle_model_layer_ranges_compose(oracle):
    """PartialStep over [0,1) then [1,2) equals one call over [0,2)."""
    from tests.util import fill_models
    cfg = mc.TINY
    m = oracle.OracleModel(cfg)
    fill_models(cfg, seed=3, oracle_model=m)
    h0 = m.embed(17)
    a, la = m.step(h0, 0)
    m.reset_kv()
    b, _ = m.step(h0, 0, 0, 1, want_logits=False)
    b, lb = m.step(b, 0, 1, 2)
    assert np.array_equal(a, b) and np.array_equal(la, lb)
    m.close()
