"""fp16-weight decode (SetWeightFP16 / SetWeightRawFP16 / PartialStepFP16) and the replay API
(CaptureGraph / Launch / UpdateAndLaunch / ValidateGraphCapture) against the CPU oracle."""
import numpy as np
import pytest

from mongoose_b200 import configs as mc
from mongoose_b200.fused_infer import CUDAFusedInference, GraphCaptureConfig, MongooseError
from oracle import gen
from oracle import oracle as O
from tests.util import assert_close, fill_models

pytestmark = pytest.mark.gpu

F16_CASES = [mc.TINY.with_(name="tiny-f16", layer_fmt=mc.FMT_F16, head_fmt=mc.FMT_F16),
             mc.QWEN25_05B.with_(name="qwen-width-2L-f16", n_layers=2, vocab=3000, max_seq=48,
                                 layer_fmt=mc.FMT_F16, head_fmt=mc.FMT_F16)]


def fill_fp16(cfg, eng, om, raw: bool, seed=4):
    """Same seeded tensors into the engine (fp16 setters) and the oracle (fp16 blocks)."""
    for idx, kind, rows, cols, fmt in gen.model_slots(cfg):
        if kind == "norm":
            v = gen.norm_vector(seed, idx, cols, 0.1)
            if raw:
                eng.SetWeightRawFP16(idx, b"", 0, v)
            else:
                eng.SetWeightFP16(idx, v)
            om.set_weight(idx, v, 0)
            continue
        w = gen.tensor_f32(seed, idx, rows, cols)
        blocks = O.quantize(mc.FMT_F16, w)             # fp16 bits, round to nearest even
        if raw:
            eng.SetWeightRawFP16(idx, blocks, rows * cols)
        else:
            eng.SetWeightFP16(idx, w)
        om.set_weight(idx, blocks, mc.FMT_F16)


@pytest.mark.parametrize("cfg", F16_CASES, ids=lambda c: c.name)
@pytest.mark.parametrize("raw", [False, True], ids=["from-fp32", "raw-fp16"])
def test_partial_step_fp16_matches_oracle(cuda, oracle, mglib, cfg, raw):
    eng, om = CUDAFusedInference(cfg), oracle.OracleModel(cfg)
    try:
        assert eng.WeightsFP16
        fill_fp16(cfg, eng, om, raw)
        # biases are skipped on the fp16 path: setting one must change nothing
        eng.SetWeightFP16(mc.SLOT_BQ, np.full(cfg.dim, 5.0, np.float32))
        rng = np.random.default_rng(1)
        logits = np.empty(cfg.vocab, np.float32)
        hid = np.empty(cfg.dim, np.float32)
        for pos in range(5):
            h = rng.standard_normal(cfg.dim).astype(np.float32)
            assert eng.PartialStepFP16(h, pos, 0, cfg.n_layers, None, logits) == 0
            _, want = om.step(h, pos, 0, cfg.n_layers)
            assert_close(logits, want, what=f"logits at pos {pos}")
        eng.ResetKV(); om.reset_kv()
        h = rng.standard_normal(cfg.dim).astype(np.float32)
        eng.PartialStepFP16(h, 0, 0, 1, hid, None)
        want_h, _ = om.step(h, 0, 0, 1, want_logits=False)
        assert_close(hid, want_h, what="hidden after layer 0")
    finally:
        eng.close(); om.close()


def test_fp16_setters_refuse_a_quantized_engine(cuda, mglib):
    eng = CUDAFusedInference(mc.TINY)
    try:
        with pytest.raises(MongooseError):
            eng.SetWeightFP16(1, np.zeros((mc.TINY.dim, mc.TINY.dim), np.float32))
        with pytest.raises(MongooseError):
            eng.PartialStepFP16(np.zeros(mc.TINY.dim, np.float32), 0, 0, 1)
    finally:
        eng.close()


REPLAY_CASES = [mc.TINY, mc.TINY_Q4,
                mc.QWEN25_05B.with_(name="qwen-width-2L", n_layers=2, vocab=3000, max_seq=48)]


@pytest.mark.parametrize("cfg", REPLAY_CASES, ids=lambda c: c.name)
@pytest.mark.parametrize("kernels_path", [False, True], ids=["default", "kernels"])
def test_replay_api(cuda, oracle, mglib, monkeypatch, cfg, kernels_path):
    if kernels_path:
        monkeypatch.setenv("MG_NO_MEGA", "1")
    eng, om = CUDAFusedInference(cfg), oracle.OracleModel(cfg)
    try:
        fill_models(cfg, seed=2, jitter=0.1, engine=eng, oracle_model=om)
        rng = np.random.default_rng(9)
        h0 = rng.standard_normal(cfg.dim).astype(np.float32)
        # plain launches and the replay path agree (the reference accepts 1e-3 absolute)
        assert eng.ValidateGraphCapture(h0, 0, cfg.n_layers)
        assert eng.last_validate_diff < 1e-4 * float(np.abs(h0).max()) * 10
        assert eng.CaptureGraph(GraphCaptureConfig(0, cfg.n_layers, StreamCount=3)) is None
        g = eng.CaptureGraph(GraphCaptureConfig(LayerStart=0, LayerEnd=cfg.n_layers), 0)
        assert g is not None and g.captured
        eng.ResetKV(); om.reset_kv()
        for pos in range(4):                       # one handle, every position
            h = rng.standard_normal(cfg.dim).astype(np.float32)
            eng.UploadHidden(h)
            if pos % 2 == 0:
                g.Launch(pos)
            else:
                assert eng.UpdateAndLaunch(g, pos)
            got = eng.ReadHidden()
            want, _ = om.step(h, pos, 0, cfg.n_layers, want_logits=False)
            assert_close(got, want, what=f"hidden at pos {pos}")
        # layer ranges chain on the device-resident hidden state
        first = eng.CaptureGraph(GraphCaptureConfig(0, 1))
        rest = eng.CaptureGraph(GraphCaptureConfig(1, cfg.n_layers))
        eng.ResetKV(); om.reset_kv()
        eng.UploadHidden(h0)
        first.Launch(0)
        rest.Launch(0)
        want, _ = om.step(h0, 0, 0, cfg.n_layers, want_logits=False)
        assert_close(eng.ReadHidden(), want, what="two ranges")
        g.Destroy()
        g.Launch(0)                                # a destroyed handle does nothing
        assert not eng.UpdateAndLaunch(g, 0)
    finally:
        eng.close(); om.close()
