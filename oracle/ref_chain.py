"""The reference's PartialStep as a chain of its own kernel entry points (test infrastructure).

`CUDAFusedInference.PartialStep` (cuda_fused_infer.go:392-459) is Go code that cannot be built here,
but all it does per token is call the dlopen'd kernels in a fixed order (cuda_fused_infer.go:414-444,
17 launches per layer) on per-row INT8 weights (quantizeQ8, :363-390: scale = absmax / 127,
q = trunc(v / scale)) with fp32 KV caches.  This module restates that loop over the C symbols, so the
same chain can be driven through oracle/_ref/libmongoose_ref.so (kernels/mongoose.cu compiled
unmodified) and through this repository's libmongoose_kernels.so, and timed as the reference's
device-side work on this GPU.

Note on scales: the reference's kernel multiplies by scales[r] / 127 (mongoose.cu:1561) while its
quantizer already stores absmax / 127; the chain passes what the Go code passes, so the model it
computes is the reference's as written (weights 127 times smaller than intended).  Both libraries
see the same numbers, which is all a parity check needs.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libmongoose_ref.so")

_SIG = {
    "mongoose_q8_matvec": [C.c_void_p] * 4 + [C.c_int, C.c_int, C.c_void_p],
    "mongoose_rmsnorm_out": [C.c_void_p] * 3 + [C.c_int, C.c_int, C.c_void_p],
    "mongoose_rope": [C.c_void_p] * 3 + [C.c_int] * 4 + [C.c_void_p],
    "mongoose_kv_cache_write": [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p],
    "mongoose_decode_attention": [C.c_void_p] * 4 + [C.c_int] * 5 + [C.c_void_p],
    "mongoose_silu_gate_mul": [C.c_void_p] * 3 + [C.c_int, C.c_void_p],
    "mongoose_add_inplace": [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p],
}


def load(path: str = REF_LIB) -> C.CDLL:
    lib = C.CDLL(path)
    for name, args in _SIG.items():
        f = getattr(lib, name)
        f.restype, f.argtypes = None, args
    return lib


def quantize_q8_rows(w: np.ndarray):
    """quantizeQ8 of the reference (cuda_fused_infer.go:363-390): per row absmax / 127, truncation."""
    w = np.asarray(w, np.float32)
    amax = np.abs(w).max(axis=1)
    scale = (amax / np.float32(127.0)).astype(np.float32)
    inv = np.where(scale > 0, np.float32(1.0) / np.where(scale > 0, scale, 1), 0).astype(np.float32)
    q = np.clip(np.trunc(w * inv[:, None]), -128, 127).astype(np.int8)
    return q, scale


class RefChain:
    """Weights of one model on the GPU in the reference's per-row INT8 layout + its scratch set."""

    def __init__(self, torch, cfg, weights_f32, norms, rope_cos, rope_sin):
        """weights_f32: {(layer, name): fp32 matrix} with names wq wk wv wo gate up down, plus
        ("head", None); norms: {(layer, 'norm1'|'norm2')} and ('final', None)."""
        self.t, self.cfg = torch, cfg
        dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
        self.w, self.s, self.n = {}, {}, {}
        for key, m in weights_f32.items():
            q, sc = quantize_q8_rows(m)
            self.w[key], self.s[key] = dev(q), dev(sc)
        for key, v in norms.items():
            self.n[key] = dev(np.asarray(v, np.float32))
        self.cos, self.sin = dev(rope_cos.astype(np.float32)), dev(rope_sin.astype(np.float32))
        z = lambda n: torch.zeros(n, device="cuda")
        c = cfg
        self.kc = [z(c.max_seq * c.kv_dim) for _ in range(c.n_layers)]
        self.vc = [z(c.max_seq * c.kv_dim) for _ in range(c.n_layers)]
        self.hidden, self.normed, self.q, self.k, self.v = z(c.dim), z(c.dim), z(c.dim), z(c.kv_dim), z(c.kv_dim)
        self.attn, self.proj, self.normed2 = z(c.dim), z(c.dim), z(c.dim)
        self.gate, self.up, self.mid = z(c.ffn_dim), z(c.ffn_dim), z(c.ffn_dim)
        self.logits = z(c.vocab)

    def enqueue(self, lib, pos: int, layer_start: int, layer_end: int, head: bool, stream=None):
        """The launches of one PartialStep on `stream` (None = stream 0, as the reference)."""
        c, p = self.cfg, (lambda x: x.data_ptr())
        half = c.head_dim // 2
        cosr, sinr = p(self.cos) + pos * half * 4, p(self.sin) + pos * half * 4
        mv = lambda key, x, out, n, k: lib.mongoose_q8_matvec(p(x), p(self.w[key]), p(self.s[key]), p(out), n, k, stream)
        for l in range(layer_start, layer_end):
            lib.mongoose_rmsnorm_out(p(self.hidden), p(self.normed), p(self.n[(l, "norm1")]), 1, c.dim, stream)
            mv((l, "wq"), self.normed, self.q, c.dim, c.dim)
            mv((l, "wk"), self.normed, self.k, c.kv_dim, c.dim)
            mv((l, "wv"), self.normed, self.v, c.kv_dim, c.dim)
            lib.mongoose_rope(p(self.q), cosr, sinr, 1, c.dim, c.head_dim, c.n_heads, stream)
            lib.mongoose_rope(p(self.k), cosr, sinr, 1, c.kv_dim, c.head_dim, c.n_kv_heads, stream)
            lib.mongoose_kv_cache_write(p(self.kc[l]), p(self.k), pos, c.kv_dim, stream)
            lib.mongoose_kv_cache_write(p(self.vc[l]), p(self.v), pos, c.kv_dim, stream)
            lib.mongoose_decode_attention(p(self.q), p(self.kc[l]), p(self.vc[l]), p(self.attn), pos + 1, c.dim, c.kv_dim,
                                          c.n_heads, c.n_kv_heads, stream)
            mv((l, "wo"), self.attn, self.proj, c.dim, c.dim)
            lib.mongoose_add_inplace(p(self.hidden), p(self.proj), c.dim, stream)
            lib.mongoose_rmsnorm_out(p(self.hidden), p(self.normed2), p(self.n[(l, "norm2")]), 1, c.dim, stream)
            mv((l, "gate"), self.normed2, self.gate, c.ffn_dim, c.dim)
            mv((l, "up"), self.normed2, self.up, c.ffn_dim, c.dim)
            lib.mongoose_silu_gate_mul(p(self.gate), p(self.up), p(self.mid), c.ffn_dim, stream)
            mv((l, "down"), self.mid, self.proj, c.dim, c.ffn_dim)
            lib.mongoose_add_inplace(p(self.hidden), p(self.proj), c.dim, stream)
        if head:
            lib.mongoose_rmsnorm_out(p(self.hidden), p(self.normed), p(self.n[("final", None)]), 1, c.dim, stream)
            mv(("head", None), self.normed, self.logits, c.vocab, c.dim)

    def reset(self):
        for x in self.kc + self.vc:
            x.zero_()


def synthetic_model(cfg, seed: int = 0):
    """fp32 weights of the seeded random-init model in RefChain's naming."""
    from mongoose_b200 import configs as mc
    from mongoose_b200 import synthetic
    names = {mc.SLOT_WQ: "wq", mc.SLOT_WK: "wk", mc.SLOT_WV: "wv", mc.SLOT_WO: "wo", mc.SLOT_GATE: "gate",
             mc.SLOT_UP: "up", mc.SLOT_DOWN: "down"}
    weights, norms = {}, {}
    for idx, kind, rows, cols, _ in synthetic.model_slots(cfg):
        layer, slot = divmod(idx, 12)
        if idx == cfg.n_layers * 12:
            norms[("final", None)] = synthetic.norm_vector(seed, idx, cols, 0.1)
        elif idx == cfg.n_layers * 12 + 1:
            weights[("head", None)] = synthetic.tensor_f32(seed, idx, rows, cols)
        elif kind == "norm":
            norms[(layer, "norm1" if slot == mc.SLOT_NORM1 else "norm2")] = synthetic.norm_vector(seed, idx, cols, 0.1)
        else:
            weights[(layer, names[slot])] = synthetic.tensor_f32(seed, idx, rows, cols)
    return weights, norms
