"""Seeded inputs of the golden cases: shared by the generator (which feeds them to the reference's own
CUDA kernels) and by the tests (which feed them to the oracle and to this library)."""
import numpy as np


def inputs():
    r = np.random.default_rng(20240607)
    c = {}
    w = (r.standard_normal((64, 896)) * 0.02).astype(np.float32)
    amax = np.abs(w).max(1)
    c["q8_w"] = np.clip(np.trunc(w / (amax[:, None] / 127.0)), -128, 127).astype(np.int8)
    c["q8_scales"] = amax.astype(np.float32)                       # the kernel divides by 127 itself
    c["q8_act"] = r.standard_normal(896).astype(np.float32)
    c["q4_w"] = r.integers(0, 256, (48, 64), dtype=np.uint8)       # K = 128
    c["q4_scales"] = (np.abs(r.standard_normal(48)) * 0.1).astype(np.float32)
    c["q4_act"] = r.standard_normal(128).astype(np.float32)
    c["norm_x"] = (r.standard_normal((2, 896)) * 2).astype(np.float32)
    c["norm_w"] = (1 + 0.1 * r.standard_normal(896)).astype(np.float32)
    c["norm_b"] = r.standard_normal((2, 896)).astype(np.float32)
    c["rope_x"] = r.standard_normal(14 * 64).astype(np.float32)
    c["rope_pos"] = np.int64(23)
    c["attn_q"] = r.standard_normal(14 * 64).astype(np.float32)
    c["attn_k"] = r.standard_normal((33, 128)).astype(np.float32)
    c["attn_v"] = r.standard_normal((33, 128)).astype(np.float32)
    c["gate"] = (r.standard_normal(512) * 3).astype(np.float32)
    c["up"] = r.standard_normal(512).astype(np.float32)
    return c
