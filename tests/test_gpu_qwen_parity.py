"""Qwen2.5-0.5B-architecture, random-init Q8_0: 32-token prompt + 200 greedy steps,
engine tokens against the CPU oracle (teacher-forced on the engine's choices)."""
import numpy as np
import pytest

from mongoose_b200 import configs as mc
from mongoose_b200.fused_infer import CUDAFusedInference
from oracle import gen
from tests.util import assert_close, fill_models, greedy_parity

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("cfg", [mc.QWEN25_05B, mc.QWEN25_05B_Q4], ids=lambda c: c.name)
def test_greedy_200_steps(cuda, oracle, mglib, cfg):
    eng = CUDAFusedInference(cfg)
    om = oracle.OracleModel(cfg)
    fill_models(cfg, seed=0, jitter=0.0, engine=eng, oracle_model=om)
    prompt = gen.prompt_ids(0, 32, cfg.vocab)
    toks = eng.Generate(prompt, 200)
    exact, ties, margins = greedy_parity(toks, om, prompt, 200)
    print(f"{cfg.name}: {exact}/200 identical, {len(ties)} ties, min top-2 margin {min(margins):.3e}")
    assert exact + len(ties) == 200 and len(ties) <= 2
    # layer output at the last position, against the oracle's state at that position
    logits = np.empty(cfg.vocab, np.float32)
    eng.StepToken(int(toks[-1]), 231, logitsOut=logits)
    want = om.step_token(int(toks[-1]), 231)
    assert_close(logits, want, 1e-4, "logits at position 231")
    eng.close(); om.close()
