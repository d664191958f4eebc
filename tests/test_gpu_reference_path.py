"""The reference's PartialStep as a PATH, not op by op.

oracle/ref_chain.py restates the launch sequence of CUDAFusedInference.PartialStep
(cuda_fused_infer.go:414-451) over the kernel entry points.  Here one full-width Qwen2.5-0.5B layer
plus lm_head runs for several positions on per-row INT8 weights (the reference's own quantizer)
 (a) through the reference's kernels (oracle/_ref/libmongoose_ref.so, mongoose.cu unmodified),
 (b) through this library's symbols of the same names,
 (c) on the CPU oracle's ops in the same order,
and the three must agree within 1e-4 on the hidden state, the FFN contribution and the logits.
"""
import os

import numpy as np
import pytest

from mongoose_b200 import configs as mc
from oracle import ref_chain
from tests.util import assert_close

pytestmark = pytest.mark.gpu

CFG = mc.QWEN25_05B.with_(name="qwen-width-1L-rowq8", n_layers=1, vocab=2000, max_seq=8)


def _oracle_step(O, cfg, q, s, norms, cos, sin, kc, vc, h, pos):
    mv = lambda key, x: O.rowq8_matvec(x, q[key], s[key])
    x = O.rmsnorm(h, norms[(0, "norm1")])
    qv = O.rope(mv((0, "wq"), x), cos[pos], sin[pos], cfg.head_dim, cfg.n_heads)
    k = O.rope(mv((0, "wk"), x), cos[pos], sin[pos], cfg.head_dim, cfg.n_kv_heads)
    kc[pos], vc[pos] = k, mv((0, "wv"), x)
    att = O.decode_attention(qv, kc, vc, pos + 1, cfg.n_heads, cfg.n_kv_heads)
    h = h + mv((0, "wo"), att)
    x = O.rmsnorm(h, norms[(0, "norm2")])
    ffn = mv((0, "down"), O.silu_gate_mul(mv((0, "gate"), x), mv((0, "up"), x)))
    h = h + ffn
    logits = mv(("head", None), O.rmsnorm(h, norms[("final", None)]))
    return h, ffn, logits


def test_reference_path_three_ways(cuda, oracle, mglib):
    if not os.path.exists(ref_chain.REF_LIB):
        pytest.skip("oracle/_ref/libmongoose_ref.so not built (make -C oracle ref needs the reference tree)")
    t, O, cfg = cuda, oracle, CFG
    weights, norms = ref_chain.synthetic_model(cfg, seed=2)
    cos, sin = O.rope_tables(cfg.max_seq, cfg.head_dim, cfg.rope_theta)
    ref_lib = ref_chain.load()
    our_lib = ref_chain.load(mglib._name)
    chains = {"reference kernels": (ref_lib, ref_chain.RefChain(t, cfg, weights, norms, cos, sin)),
              "this library": (our_lib, ref_chain.RefChain(t, cfg, weights, norms, cos, sin))}
    q, s = {}, {}
    for key, m in weights.items():
        q[key], s[key] = ref_chain.quantize_q8_rows(m)
    kc = np.zeros((cfg.max_seq, cfg.kv_dim), np.float32)
    vc = np.zeros((cfg.max_seq, cfg.kv_dim), np.float32)
    rng = np.random.default_rng(0)
    for pos in range(5):
        h = rng.standard_normal(cfg.dim).astype(np.float32)
        want_h, want_ffn, want_logits = _oracle_step(O, cfg, q, s, norms, cos, sin, kc, vc, h, pos)
        got = {}
        for name, (lib, ch) in chains.items():
            ch.hidden.copy_(t.from_numpy(h))
            ch.enqueue(lib, pos, 0, 1, head=True)
            t.cuda.synchronize()
            got[name] = (ch.hidden.cpu().numpy(), ch.proj.cpu().numpy(), ch.logits.cpu().numpy())
            assert_close(got[name][0], want_h, 1e-4, f"{name}: hidden at pos {pos}")
            assert_close(got[name][1], want_ffn, 1e-4, f"{name}: FFN contribution at pos {pos}")
            assert_close(got[name][2], want_logits, 1e-4, f"{name}: logits at pos {pos}")
        for i, what in enumerate(("hidden", "FFN contribution", "logits")):
            assert_close(got["this library"][i], got["reference kernels"][i], 1e-4, f"library vs reference kernels: {what} at pos {pos}")
