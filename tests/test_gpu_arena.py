"""One device allocation per engine (the reference's GPUArena, gpu_alloc.go:45-241) and the raw
device-memory calls that draw from it (tw_gpu_alloc / upload / download / zero, cuda_tensor.go:19-44)."""
import numpy as np
import pytest

from mongoose_b200 import configs as mc
from mongoose_b200 import kernels as K
from mongoose_b200.fused_infer import CUDAFusedInference
from tests.util import assert_close, fill_models

pytestmark = pytest.mark.gpu


def test_engine_lives_in_its_arena(cuda, oracle, mglib):
    cfg = mc.TINY
    eng, om = CUDAFusedInference(cfg), oracle.OracleModel(cfg)
    try:
        s0 = eng.ArenaStats()
        assert s0["total"] > 0 and s0["outside"] == 0
        fill_models(cfg, seed=1, jitter=0.1, engine=eng, oracle_model=om)
        eng.BuildFusedDispatch()
        s1 = eng.ArenaStats()
        assert s1["outside"] == 0, "a buffer did not fit the arena sized from the model's shape"
        assert s0["in_use"] < s1["in_use"] <= s1["total"]
        # setting every weight again and rebuilding returns the old planes and tape to the arena
        fill_models(cfg, seed=1, jitter=0.1, engine=eng)
        eng.BuildFusedDispatch()
        s2 = eng.ArenaStats()
        assert s2["in_use"] == s1["in_use"] and s2["outside"] == 0
        logits = np.empty(cfg.vocab, np.float32)
        eng.StepToken(3, 0, logitsOut=logits)
        assert_close(logits, om.step_token(3, 0), 1e-4, "engine on arena memory")
    finally:
        eng.close(); om.close()


def test_raw_device_memory_round_trip(cuda, oracle, mglib):
    t = cuda
    eng = CUDAFusedInference(mc.TINY)
    try:
        before = eng.ArenaStats()
        n = 1000
        a = np.random.default_rng(0).standard_normal(n).astype(np.float32)
        b = np.random.default_rng(1).standard_normal(n).astype(np.float32)
        pa, pb, po = eng.DeviceAlloc(n * 4), eng.DeviceAlloc(n * 4), eng.DeviceAlloc(n * 4)
        assert pa % 256 == 0 and pb % 256 == 0 and len({pa, pb, po}) == 3
        eng.DeviceUpload(pa, a); eng.DeviceUpload(pb, b)
        K.KSiLUGateMul(pa, pb, po, n)                     # a reference-ABI kernel on arena buffers
        t.cuda.synchronize()
        out = np.empty(n, np.float32)
        eng.DeviceDownload(out, po)
        assert_close(out, oracle.silu_gate_mul(a, b), 1e-6, "kernel on arena buffers")
        eng.DeviceZero(po, n * 4)
        eng.DeviceDownload(out, po)
        assert not out.any()
        mid = eng.ArenaStats()
        assert mid["in_use"] == before["in_use"] + 3 * 4096
        # frees coalesce: after releasing all three the largest free block is what it was
        eng.DeviceFree(pb); eng.DeviceFree(pa); eng.DeviceFree(po)
        after = eng.ArenaStats()
        assert after["in_use"] == before["in_use"] and after["largest_free"] == before["largest_free"]
        # a request larger than the arena falls through to the driver and is handed back the same way
        big = eng.DeviceAlloc(before["total"] + (1 << 20))
        assert eng.ArenaStats()["outside"] == 1
        eng.DeviceFree(big)
        assert eng.ArenaStats()["outside"] == 0
    finally:
        eng.close()
