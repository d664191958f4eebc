"""mongoose_partial_step_q4_fused_graph: the one-call-per-token dispatch on caller-owned buffers.

The reference's fused path (cuda_fused_infer_q4.go:103-131, signature cuda_graph.go:211-222) hands
per-layer pointer arrays, scratch vectors, fp32 KV caches [maxSeq, kvDim] and the RoPE tables to one
C call that enqueues layers [layerStart, layerEnd).  Here it runs on Qwen2.5-0.5B widths with raw
GGUF Q4_0 blocks and is compared, position by position, with the same op order on the CPU oracle
(cuda_fused_infer.go:414-444), fp32 KV included.
"""
import ctypes as C

import numpy as np
import pytest

from mongoose_b200 import _lib
from oracle import gen
from tests.util import assert_close

pytestmark = pytest.mark.gpu

DIM, KV, HD, NH, NKV, FFN, L, MAXSEQ = 896, 128, 64, 14, 2, 4864, 2, 8
SHAPES = {"wq": (DIM, DIM), "wk": (KV, DIM), "wv": (KV, DIM), "wo": (DIM, DIM),
          "wgate": (FFN, DIM), "wup": (FFN, DIM), "wdown": (DIM, FFN)}


def _layer_on_oracle(O, h, w, l, pos, cos, sin, kc, vc):
    """One layer in the reference's op order on the CPU oracle; returns the new hidden state."""
    x = O.rmsnorm(h, w["norm1"][l])
    q = O.matvec(1, w["wq"][l], x, DIM, DIM)
    k = O.matvec(1, w["wk"][l], x, KV, DIM)
    v = O.matvec(1, w["wv"][l], x, KV, DIM)
    q = O.rope(q, cos[pos], sin[pos], HD, NH)
    k = O.rope(k, cos[pos], sin[pos], HD, NKV)
    kc[l][pos] = k
    vc[l][pos] = v
    att = O.decode_attention(q, kc[l], vc[l], pos + 1, NH, NKV)
    h = h + O.matvec(1, w["wo"][l], att, DIM, DIM)
    x = O.rmsnorm(h, w["norm2"][l])
    g = O.matvec(1, w["wgate"][l], x, FFN, DIM)
    u = O.matvec(1, w["wup"][l], x, FFN, DIM)
    return h + O.matvec(1, w["wdown"][l], O.silu_gate_mul(g, u), DIM, FFN)


def test_fused_dispatch_matches_reference_op_order(cuda, oracle, mglib):
    t, O = cuda, oracle
    lib = _lib.load()
    w = {k: [] for k in list(SHAPES) + ["norm1", "norm2"]}
    for l in range(L):
        for i, (name, (r, c)) in enumerate(SHAPES.items()):
            w[name].append(O.quantize(1, gen.tensor_f32(5, l * 16 + i, r, c)))
        w["norm1"].append(gen.norm_vector(5, l * 16 + 9, DIM, 0.1))
        w["norm2"].append(gen.norm_vector(5, l * 16 + 10, DIM, 0.1))
    cos, sin = O.rope_tables(MAXSEQ, HD, 1e6)

    keep = []                      # device tensors stay alive for the whole test

    def dev(a):
        x = t.from_numpy(np.ascontiguousarray(a)).cuda()
        keep.append(x)
        return x

    def ptr_array(tensors):
        return (C.c_void_p * len(tensors))(*[x.data_ptr() for x in tensors])

    d = {k: [dev(a) for a in v] for k, v in w.items()}
    d_kc = [dev(np.zeros((MAXSEQ, KV), np.float32)) for _ in range(L)]
    d_vc = [dev(np.zeros((MAXSEQ, KV), np.float32)) for _ in range(L)]
    arrays = {k: ptr_array(v) for k, v in d.items()}
    a_kc, a_vc = ptr_array(d_kc), ptr_array(d_vc)
    sizes = {"hidden": DIM, "normed": DIM, "Q": DIM, "K": KV, "V": KV, "attnOut": DIM, "proj": DIM, "normed2": DIM,
             "gatePre": FFN, "upOut": FFN, "ffnMid": FFN}
    s = {k: t.zeros(n, device="cuda") for k, n in sizes.items()}
    q8 = t.zeros((FFN // 32) * 40, dtype=t.uint8, device="cuda")
    d_cos, d_sin = dev(cos.astype(np.float32)), dev(sin.astype(np.float32))

    def run(pos, ls, le):
        lib.mongoose_partial_step_q4_fused_graph(
            arrays["norm1"], arrays["wq"], arrays["wk"], arrays["wv"], arrays["wo"], arrays["norm2"],
            arrays["wgate"], arrays["wup"], arrays["wdown"], a_kc, a_vc,
            s["hidden"].data_ptr(), s["normed"].data_ptr(), s["Q"].data_ptr(), s["K"].data_ptr(), s["V"].data_ptr(),
            s["attnOut"].data_ptr(), s["proj"].data_ptr(), s["normed2"].data_ptr(),
            s["gatePre"].data_ptr(), s["upOut"].data_ptr(), s["ffnMid"].data_ptr(),
            q8.data_ptr(), d_cos.data_ptr(), d_sin.data_ptr(),
            DIM, KV, HD, FFN, NH, NKV, HD // 2, pos, ls, le, None)
        t.cuda.synchronize()
        return s["hidden"].cpu().numpy()

    kc = [np.zeros((MAXSEQ, KV), np.float32) for _ in range(L)]
    vc = [np.zeros((MAXSEQ, KV), np.float32) for _ in range(L)]
    rng = np.random.default_rng(1)
    for pos in range(6):
        h = rng.standard_normal(DIM).astype(np.float32)
        s["hidden"].copy_(t.from_numpy(h))
        if pos % 2 == 0:
            got = run(pos, 0, L)                       # all layers in one call
            want = h
            for l in range(L):
                want = _layer_on_oracle(O, want, w, l, pos, cos, sin, kc, vc)
        else:
            mid = run(pos, 0, 1)                       # a layer sub-range, then the rest
            want = _layer_on_oracle(O, h, w, 0, pos, cos, sin, kc, vc)
            assert_close(mid, want, 1e-4, f"pos {pos} after layer 0")
            got = run(pos, 1, L)
            for l in range(1, L):
                want = _layer_on_oracle(O, want, w, l, pos, cos, sin, kc, vc)
        assert_close(got, want, 1e-4, f"pos {pos} hidden")
    for l in range(L):
        assert_close(d_kc[l].cpu().numpy()[:6], kc[l][:6], 1e-4, f"K cache layer {l}")
        assert_close(d_vc[l].cpu().numpy()[:6], vc[l][:6], 1e-4, f"V cache layer {l}")
