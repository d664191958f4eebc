"""Shared helpers for the parity tests."""
from __future__ import annotations

import numpy as np

from mongoose_b200 import configs as mc
from oracle import gen
from oracle import oracle as O

REL_TOL = 1e-4   # GPU vs fp64-accumulate oracle, relative to max|y| of the vector


def free_port() -> int:
    """A TCP port nothing is listening on right now (for a torchrun rendezvous on 127.0.0.1)."""
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def rel_err(got, want) -> float:
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    denom = np.abs(want).max()
    return float(np.abs(got - want).max() / (denom if denom > 0 else 1.0))


def assert_close(got, want, tol=REL_TOL, what=""):
    e = rel_err(got, want)
    assert np.all(np.isfinite(got)), f"{what}: non-finite output"
    assert e <= tol, f"{what}: relative error {e:.3e} > {tol:.1e}"


def fill_models(cfg: mc.ModelConfig, seed: int = 0, jitter: float = 0.1, engine=None, oracle_model=None,
                raw_slots: bool = False, bias: bool = False):
    """Generate the seeded random-init model and hand it to the engine (SetWeight / SetWeightRaw)
    and/or the oracle.  Returns the dict idx -> (blocks, fmt) of quantized matrices."""
    blocks = {}
    for idx, kind, rows, cols, fmt in gen.model_slots(cfg):
        if kind == "norm":
            v = gen.norm_vector(seed, idx, cols, jitter)
            if engine is not None:
                engine.SetWeight(idx, v)
            if oracle_model is not None:
                oracle_model.set_weight(idx, v, 0)
            continue
        w = gen.tensor_f32(seed, idx, rows, cols)
        need_blocks = oracle_model is not None or raw_slots
        b = O.quantize(fmt, w) if need_blocks else None
        if engine is not None:
            if raw_slots and (idx % 2 == 0):
                engine.SetWeightRaw(idx, b, fmt)
            else:
                engine.SetWeight(idx, w)
        if oracle_model is not None:
            oracle_model.set_weight(idx, b, fmt)
        blocks[idx] = (b, fmt)
        del w
    if bias:
        for l in range(cfg.n_layers):
            for slot, n in ((mc.SLOT_BQ, cfg.dim), (mc.SLOT_BK, cfg.kv_dim), (mc.SLOT_BV, cfg.kv_dim)):
                idx = l * 12 + slot
                rng = np.random.default_rng([seed, idx, 11])
                v = (0.05 * rng.standard_normal(n)).astype(np.float32)
                if engine is not None:
                    engine.SetWeight(idx, v)
                if oracle_model is not None:
                    oracle_model.set_weight(idx, v, 0)
    return blocks


def greedy_parity(engine_tokens, oracle_model, prompt, n_new, tie_tol=1e-5):
    """Replay the engine's greedy tokens through the oracle (teacher-forced with the engine's own
    choices) and compare with the oracle's argmax at every step.  Returns
    (n_exact, ties, margins): a step counts as a tie when the tokens differ but the oracle's logits
    of the two candidates are within tie_tol * max|logit|.  Any other difference raises."""
    cfg = oracle_model.cfg
    oracle_model.reset_kv()
    toks = list(prompt)
    pos = 0
    logits = None
    for t in toks:
        logits = oracle_model.step_token(int(t), pos)
        pos += 1
    exact, ties, margins = 0, [], []
    for i in range(n_new):
        want = int(O.lib().oracle_argmax(logits.ctypes.data, cfg.vocab))
        got = int(engine_tokens[i])
        top2 = np.partition(logits, -2)[-2:]
        margins.append(float(top2[1] - top2[0]))
        if got == want:
            exact += 1
        else:
            gap = float(logits[want] - logits[got])
            scale = float(np.abs(logits).max())
            assert gap <= tie_tol * scale, (
                f"step {i}: engine token {got} vs oracle {want}, logit gap {gap:.3e} "
                f"(scale {scale:.3e}) is not a tie")
            ties.append((i, got, want, gap))
        if i + 1 < n_new:
            logits = oracle_model.step_token(got, pos)
            pos += 1
    return exact, ties, margins
