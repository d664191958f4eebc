"""Reference entry points that are names over the same engine: StepLayerResident
(cuda_fused_infer_q4.go:451-605), the Q4_0 step calls (:92-444) and the vNode / stream-1 calls
(cuda_fused_infer.go:630-684), each checked against the CPU oracle."""
import numpy as np
import pytest

from mongoose_b200 import configs as mc
from mongoose_b200.fused_infer import CUDAFusedInference, MongooseError
from tests.util import assert_close, fill_models

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("cfg", [mc.TINY, mc.TINY_Q4], ids=lambda c: c.name)
def test_step_layer_resident_snapshots(cuda, oracle, mglib, cfg):
    eng, om = CUDAFusedInference(cfg), oracle.OracleModel(cfg)
    try:
        fill_models(cfg, seed=4, jitter=0.1, engine=eng, oracle_model=om)
        rng = np.random.default_rng(9)
        for pos in range(3):
            h = rng.standard_normal(cfg.dim).astype(np.float32)
            cur = h
            for l in range(cfg.n_layers):
                pre, post = np.empty(cfg.dim, np.float32), np.empty(cfg.dim, np.float32)
                logits = np.empty(cfg.vocab, np.float32)
                last = l == cfg.n_layers - 1
                eng.StepLayerResident(l, pos, h if l == 0 else None, pre, post, logits if (last or l == 0) else None)
                want_h, want_logits = om.step(cur, pos, l, l + 1, want_logits=False)[0], None
                assert_close(pre, cur, 1e-6, f"pos {pos} layer {l}: hidden before the layer")
                assert_close(post, want_h, 1e-4, f"pos {pos} layer {l}: hidden after the layer")
                if last or l == 0:
                    # final norm + lm_head on the layer's output, whichever layer it is
                    _, want_logits = om.step(want_h, pos, cfg.n_layers, cfg.n_layers)
                    assert_close(logits, want_logits, 1e-4, f"pos {pos}: logits on the output of layer {l}")
                cur = want_h if not last else cur
                if not last:
                    # the engine continues on its own hidden state; keep the oracle on the same footing
                    cur = post.copy()
        with pytest.raises(MongooseError):
            eng.StepLayerResident(cfg.n_layers, 0, h)
    finally:
        eng.close(); om.close()


def test_q4_names_and_stream1_calls(cuda, oracle, mglib):
    cfg = mc.TINY_Q4
    eng, om = CUDAFusedInference(cfg), oracle.OracleModel(cfg)
    q8 = CUDAFusedInference(mc.TINY)
    try:
        fill_models(cfg, seed=6, jitter=0.1, engine=eng, oracle_model=om)
        with pytest.raises(MongooseError, match="Q4_0"):
            q8.PartialStepQ4(np.zeros(mc.TINY.dim, np.float32), 0, 0, 1)
        with pytest.raises(MongooseError, match="mg_set_vnode_count"):
            eng.PartialStepQ4ContinueOnStream1(0, 1, cfg.n_layers)
        eng.SetVNodeCount(2)
        assert eng.VNodeCount() == 2
        rng = np.random.default_rng(2)
        logits = np.empty(cfg.vocab, np.float32)
        mid = np.empty(cfg.dim, np.float32)
        for pos in range(3):
            h = rng.standard_normal(cfg.dim).astype(np.float32)
            # stage A on the default stream, stage B "on stream 1" behind the stage-done event
            eng.PartialStepQ4(h, pos, 0, 1, hiddenOut=mid)
            eng.RecordStageDone()
            eng.WaitStageDone()
            eng.PartialStepQ4ContinueOnStream1(pos, 1, cfg.n_layers, logits)
            eng.QueueHiddenToL3OnStream1()
            eng.SyncStream1()
            eng.WaitL3(1000)
            want_mid, _ = om.step(h, pos, 0, 1, want_logits=False)
            want_h, want_logits = om.step(want_mid, pos, 1, cfg.n_layers)
            assert_close(mid, want_mid, 1e-4, f"pos {pos}: stage A")
            assert_close(logits, want_logits, 1e-4, f"pos {pos}: logits from stage B")
            assert_close(eng.GetL3Hidden(), want_h, 1e-4, f"pos {pos}: hidden through the L3 bridge from stream 1")
        eng.SwapHiddenBuffer(); eng.DisableFusedDispatch()
        # PartialStepQ4Continue: the hidden state stays on the device between the two calls
        h = rng.standard_normal(cfg.dim).astype(np.float32)
        om.reset_kv(); eng.ResetKV()
        eng.PartialStepQ4(h, 0, 0, 1)
        eng.PartialStepQ4Continue(0, 1, cfg.n_layers, logitsOut=logits)
        _, want = om.step(h, 0, 0, cfg.n_layers)
        assert_close(logits, want, 1e-4, "PartialStepQ4 + PartialStepQ4Continue")
    finally:
        eng.close(); om.close(); q8.close()
