"""Generates tests/golden/ref_kernels.npz by running the REFERENCE's own CUDA kernels
(kernels/mongoose.cu, built unmodified by `make -C oracle ref` into oracle/_ref/libmongoose_ref.so)
on the seeded inputs of cases.py.  Needs a GPU:

    python tests/golden/make_golden.py [out.npz]
"""
import ctypes as C
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from tests.golden.cases import inputs  # noqa: E402


def load_reference():
    lib = C.CDLL(os.path.join(ROOT, "oracle", "_ref", "libmongoose_ref.so"))
    vp, ci = C.c_void_p, C.c_int
    sig = {
        "mongoose_q8_matvec": [vp, vp, vp, vp, ci, ci, vp],
        "mongoose_q4_matvec": [vp, vp, vp, vp, ci, ci, vp],
        "mongoose_rmsnorm_out": [vp, vp, vp, ci, ci, vp],
        "mongoose_rmsnorm": [vp, vp, ci, ci, vp],
        "mongoose_fused_add_rmsnorm": [vp, vp, vp, vp, ci, ci, vp],
        "mongoose_rope": [vp, vp, vp, ci, ci, ci, ci, vp],
        "mongoose_kv_cache_write": [vp, vp, ci, ci, vp],
        "mongoose_decode_attention": [vp, vp, vp, vp, ci, ci, ci, ci, ci, vp],
        "mongoose_silu_gate_mul": [vp, vp, vp, ci, vp],
        "mongoose_add_inplace": [vp, vp, ci, vp],
    }
    for n, a in sig.items():
        f = getattr(lib, n)
        f.restype, f.argtypes = None, a
    return lib


def run(lib, c):
    """Returns name -> output array for every golden case.  `lib` exposes the reference ABI."""
    from oracle import oracle as O
    keep = []          # device buffers must outlive the (asynchronous) launches that read them

    def d(a):
        t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
        keep.append(t)
        return t

    p = lambda t: t.data_ptr()
    out = {}
    o = torch.empty(64, device="cuda")
    lib.mongoose_q8_matvec(p(d(c["q8_act"])), p(d(c["q8_w"])), p(d(c["q8_scales"])), p(o), 64, 896, None)
    out["q8_matvec"] = o
    o = torch.empty(48, device="cuda")
    lib.mongoose_q4_matvec(p(d(c["q4_act"])), p(d(c["q4_w"])), p(d(c["q4_scales"])), p(o), 48, 128, None)
    out["q4_matvec"] = o
    x, w, b = d(c["norm_x"]), d(c["norm_w"]), d(c["norm_b"])
    o = torch.empty_like(x)
    lib.mongoose_rmsnorm_out(p(x), p(o), p(w), 2, 896, None)
    out["rmsnorm_out"] = o
    o = torch.empty_like(x)
    lib.mongoose_fused_add_rmsnorm(p(x), p(b), p(o), p(w), 2, 896, None)
    out["fused_add_rmsnorm"] = o
    cos, sin = O.rope_tables(40, 64, 1e6)
    pos = int(c["rope_pos"])
    dc, ds, rx = d(cos), d(sin), d(c["rope_x"])
    lib.mongoose_rope(p(rx), p(dc) + pos * 32 * 4, p(ds) + pos * 32 * 4, 1, 14 * 64, 64, 14, None)
    out["rope"] = rx
    o = torch.empty(14 * 64, device="cuda")
    lib.mongoose_decode_attention(p(d(c["attn_q"])), p(d(c["attn_k"])), p(d(c["attn_v"])), p(o), 33, 14 * 64, 128,
                                  14, 2, None)
    out["decode_attention"] = o
    o = torch.empty(512, device="cuda")
    lib.mongoose_silu_gate_mul(p(d(c["gate"])), p(d(c["up"])), p(o), 512, None)
    out["silu_gate_mul"] = o
    a = d(c["gate"])
    lib.mongoose_add_inplace(p(a), p(d(c["up"])), 512, None)
    out["add_inplace"] = a
    cache = torch.zeros(4, 128, device="cuda")
    lib.mongoose_kv_cache_write(p(cache), p(d(c["attn_k"][5])), 2, 128, None)
    out["kv_cache_write"] = cache
    torch.cuda.synchronize()
    return {k: v.cpu().numpy() for k, v in out.items()}


if __name__ == "__main__":
    dst = sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "tests", "golden", "ref_kernels.npz")
    res = run(load_reference(), inputs())
    np.savez_compressed(dst, **res)
    print("wrote", dst, {k: v.shape for k, v in res.items()})
