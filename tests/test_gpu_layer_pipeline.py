"""Layer-range pipeline: two engines as stages (SetLayerRange, QueueHiddenTo, WaitMailbox,
PartialStepContinue) and the pinned-host bridge (QueueHiddenToL3 / WaitL3 / GetL3Hidden), against
the CPU oracle.  Both stages sit on cuda:0 unless two GPUs are visible, in which case the second
stage runs on cuda:1 and the hand-over is a peer copy.  Failure cases are made on the host: a
mailbox that nothing was queued to must time out, not wait."""
import time

import numpy as np
import pytest

from mongoose_b200 import configs as mc
from mongoose_b200.fused_infer import CUDAFusedInference, MongooseError
from oracle import gen
from tests.util import assert_close, fill_models

pytestmark = pytest.mark.gpu

CASES = [mc.TINY.with_(name="tiny-4L", n_layers=4),
         mc.QWEN25_05B.with_(name="qwen-width-4L", n_layers=4, vocab=3000, max_seq=48)]


def fill_stage(cfg, eng, first, last, seed=6):
    """The stage's own layers only; the last stage also gets the final norm and lm_head."""
    for idx, kind, rows, cols, fmt in gen.model_slots(cfg):
        layer = idx // 12 if idx < cfg.n_layers * 12 else cfg.n_layers
        if layer < cfg.n_layers and not (first <= layer < last):
            continue
        if layer == cfg.n_layers and last < cfg.n_layers:
            continue
        if kind == "norm":
            eng.SetWeight(idx, gen.norm_vector(seed, idx, cols, 0.1))
        else:
            eng.SetWeight(idx, gen.tensor_f32(seed, idx, rows, cols))


@pytest.mark.parametrize("cfg", CASES, ids=lambda c: c.name)
@pytest.mark.parametrize("kernels_path", [False, True], ids=["default", "kernels"])
def test_two_stage_pipeline_matches_oracle(cuda, oracle, mglib, monkeypatch, cfg, kernels_path):
    import torch
    if kernels_path:
        monkeypatch.setenv("MG_NO_MEGA", "1")
    second_dev = 1 if torch.cuda.device_count() > 1 else 0
    cut = 2
    a, b = CUDAFusedInference(cfg, device=0), CUDAFusedInference(cfg, device=second_dev)
    om = oracle.OracleModel(cfg)
    try:
        a.SetLayerRange(0, cut)
        b.SetLayerRange(cut, cfg.n_layers)
        fill_stage(cfg, a, 0, cut)
        fill_stage(cfg, b, cut, cfg.n_layers)
        fill_models(cfg, seed=6, jitter=0.1, oracle_model=om)
        rng = np.random.default_rng(8)
        logits = np.empty(cfg.vocab, np.float32)
        for pos in range(5):
            h = rng.standard_normal(cfg.dim).astype(np.float32)
            a.PartialStep(h, pos, 0, cut)                  # stage A, hidden state stays on its GPU
            a.QueueHiddenTo(b)
            b.WaitMailbox(2000)
            b.PartialStepContinue(pos, cut, cfg.n_layers, None, logits)
            _, want = om.step(h, pos, 0, cfg.n_layers)
            assert_close(logits, want, what=f"pipeline logits at pos {pos}")
        # a stage refuses layers it does not hold, and the head where it does not live
        with pytest.raises(MongooseError):
            a.PartialStepContinue(0, cut, cfg.n_layers)
        with pytest.raises(MongooseError):
            b.PartialStep(h, 0, 0, cut)
        with pytest.raises(MongooseError):
            a.StepToken(1, 0)
    finally:
        a.close(); b.close(); om.close()


def test_mailbox_times_out_when_nothing_was_queued(cuda, mglib):
    eng = CUDAFusedInference(mc.TINY)
    try:
        t0 = time.perf_counter()
        with pytest.raises(MongooseError, match="nothing was queued"):
            eng.WaitMailbox(50)
        assert 0.04 <= time.perf_counter() - t0 < 1.0
        with pytest.raises(MongooseError):
            eng.WaitL3(10)
    finally:
        eng.close()


def test_mailbox_survives_the_sender(cuda, mglib):
    """The receiving stage waits on its own event: the sender may be gone by the time it asks."""
    cfg = mc.TINY
    a, b = CUDAFusedInference(cfg), CUDAFusedInference(cfg)
    try:
        fill_models(cfg, seed=2, jitter=0.1, engine=a)
        h = np.random.default_rng(5).standard_normal(cfg.dim).astype(np.float32)
        a.PartialStep(h, 0, 0, 1)
        a.QueueHiddenTo(b)
        want = a.ExportHidden()
        a.close()
        b.WaitMailbox(1000)
        assert np.array_equal(b.ExportHidden(), want)
    finally:
        a.close(); b.close()


def test_l3_bridge_returns_the_hidden_state(cuda, oracle, mglib):
    cfg = mc.TINY
    eng, om = CUDAFusedInference(cfg), oracle.OracleModel(cfg)
    try:
        fill_models(cfg, seed=2, jitter=0.1, engine=eng, oracle_model=om)
        h = np.random.default_rng(4).standard_normal(cfg.dim).astype(np.float32)
        eng.PartialStep(h, 0, 0, 1)
        eng.QueueHiddenToL3()                 # copy stream; the compute stream goes on
        eng.PartialStepContinue(0, 1, cfg.n_layers)
        eng.WaitL3(1000)
        want, _ = om.step(h, 0, 0, 1, want_logits=False)
        assert_close(eng.GetL3Hidden(), want, what="hidden after layer 0 through the pinned bridge")
        assert eng.HasL3() and eng.HasMailbox()
    finally:
        eng.close(); om.close()
