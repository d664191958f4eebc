"""Decode attention beyond the positions the kernels keep in registers.

The persistent kernel's attention holds the first cached K rows (480 positions for head_dim 32 / 64,
240 for head_dim 128) and V rows (240 positions) in registers and takes longer contexts from L2 in
separate loops; the benchmark configurations run to 1024 (TinyLlama) and 384 (7B-class) positions.
Here small models with those head sizes are decoded past 500 positions and the logits are compared
with the CPU oracle, which replays the engine's own tokens.
"""
import numpy as np
import pytest

from mongoose_b200 import configs as mc
from mongoose_b200.fused_infer import CUDAFusedInference
from oracle import gen
from tests.util import assert_close, fill_models

pytestmark = pytest.mark.gpu

CASES = [
    mc.TINY.with_(name="long-hd64", dim=256, n_heads=4, n_kv_heads=1, head_dim=64, ffn_dim=416, vocab=777, max_seq=560),
    mc.TINY.with_(name="long-hd128", dim=256, n_heads=2, n_kv_heads=2, head_dim=128, ffn_dim=160, vocab=130, max_seq=560),
    mc.TINY.with_(name="long-hd32", max_seq=560),
]


@pytest.mark.parametrize("cfg", CASES, ids=lambda c: c.name)
@pytest.mark.parametrize("kernels_path", [False, True], ids=["persistent", "kernels"])
def test_logits_beyond_500_positions(cuda, oracle, mglib, monkeypatch, cfg, kernels_path):
    if kernels_path:
        monkeypatch.setenv("MG_NO_MEGA", "1")
    eng = CUDAFusedInference(cfg)
    om = oracle.OracleModel(cfg)
    fill_models(cfg, seed=3, jitter=0.1, engine=eng, oracle_model=om)
    try:
        n_prompt, n_new = 8, 540
        prompt = gen.prompt_ids(4, n_prompt, cfg.vocab)
        toks = eng.Generate(prompt, n_new)
        # teacher-forced replay on the oracle; logits are checked at positions around and past every
        # boundary of the register-held part (240, 480) and at the end
        check = {100, 239, 240, 241, 300, 479, 480, 481, 500, n_prompt + n_new - 2}
        logits = np.empty(cfg.vocab, np.float32)
        seq = list(prompt) + [int(x) for x in toks]
        om.reset_kv()
        for pos in range(n_prompt + n_new - 1):
            want = om.step_token(seq[pos], pos)
            if pos in check:
                # the KV cache still holds positions < pos from Generate
                eng.StepToken(seq[pos], pos, logitsOut=logits)
                assert_close(logits, want, 1e-4, f"{cfg.name} pos {pos}")
    finally:
        eng.close()
        om.close()
