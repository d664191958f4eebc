"""ctypes binding of oracle/liboracle.so (built by oracle/Makefile).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the
CPU-baseline leg of bench.py, never by the product package.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
FMT_Q8_0, FMT_Q4_0, FMT_F16 = 0, 1, 2


def build(force: bool = False) -> str:
    so = os.path.join(_HERE, "liboracle.so")
    src = os.path.join(_HERE, "oracle.c")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", _HERE, "liboracle.so"])
    return so


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        L = C.CDLL(build())
        vp, cl, ci, cf, cd = C.c_void_p, C.c_long, C.c_int, C.c_float, C.c_double
        sig = {
            "oracle_f32_to_f16_n": (None, [vp, vp, cl]),
            "oracle_f16_to_f32_n": (None, [vp, vp, cl]),
            "oracle_quantize_q8_0": (None, [vp, cl, cl, vp]),
            "oracle_quantize_q4_0": (None, [vp, cl, cl, vp]),
            "oracle_quantize_rowq8": (None, [vp, cl, cl, vp, vp]),
            "oracle_dequant_q8_0": (None, [vp, cl, cl, vp]),
            "oracle_dequant_q4_0": (None, [vp, cl, cl, vp]),
            "oracle_matvec": (None, [ci, vp, vp, vp, cl, cl]),
            "oracle_rowq8_matvec": (None, [vp, vp, vp, vp, cl, cl]),
            "oracle_rowq4_matvec": (None, [vp, vp, vp, vp, cl, cl]),
            "oracle_rmsnorm": (None, [vp, vp, vp, cl, cf]),
            "oracle_rope_tables": (None, [cl, cl, cd, vp, vp]),
            "oracle_rope": (None, [vp, vp, vp, cl, cl]),
            "oracle_decode_attention": (None, [vp, vp, vp, vp, cl, cl, cl, cl, cl]),
            "oracle_decode_attention_f16kv": (None, [vp, vp, vp, vp, cl, cl, cl, cl, cl]),
            "oracle_silu_gate_mul": (None, [vp, vp, vp, cl]),
            "oracle_add_inplace": (None, [vp, vp, cl]),
            "oracle_model_create": (vp, [cl, cl, cl, cl, cl, cl, cl, cl, cl, cd, cf]),
            "oracle_model_destroy": (None, [vp]),
            "oracle_model_set_weight": (None, [vp, cl, vp, ci]),
            "oracle_model_reset_kv": (None, [vp]),
            "oracle_model_embed": (None, [vp, cl, vp]),
            "oracle_model_step": (None, [vp, vp, cl, cl, cl, vp]),
            "oracle_model_step_token": (None, [vp, cl, cl, vp]),
            "oracle_model_kcache": (vp, [vp, cl]),
            "oracle_model_vcache": (vp, [vp, cl]),
            "oracle_argmax": (cl, [vp, cl]),
            "oracle_cpu_engine_matvec": (None, [ci, vp, vp, vp, cl, cl, ci]),
            "oracle_cpu_engine_step_token": (None, [vp, cl, cl, vp, ci]),
            "oracle_cpu_engine_matmul": (None, [vp, vp, vp, cl, cl, cl]),
            "oracle_max_threads": (ci, []),
        }
        for name, (res, args) in sig.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def row_bytes(fmt: int, cols: int) -> int:
    return cols // 32 * 34 if fmt == FMT_Q8_0 else cols // 32 * 18 if fmt == FMT_Q4_0 else cols * 2


def f32_to_f16_bits(x) -> np.ndarray:
    x = _f32(x)
    out = np.empty(x.shape, np.uint16)
    lib().oracle_f32_to_f16_n(_p(x), _p(out), x.size)
    return out


def f16_bits_to_f32(h) -> np.ndarray:
    h = np.ascontiguousarray(h, dtype=np.uint16)
    out = np.empty(h.shape, np.float32)
    lib().oracle_f16_to_f32_n(_p(h), _p(out), h.size)
    return out


def quantize(fmt: int, w) -> np.ndarray:
    """fp32 [rows, cols] -> raw blocks uint8 [rows, row_bytes] (fp16 rows for FMT_F16)."""
    w = _f32(w)
    rows, cols = w.shape
    out = np.empty((rows, row_bytes(fmt, cols)), np.uint8)
    if fmt == FMT_Q8_0:
        lib().oracle_quantize_q8_0(_p(w), rows, cols, _p(out))
    elif fmt == FMT_Q4_0:
        lib().oracle_quantize_q4_0(_p(w), rows, cols, _p(out))
    else:
        out = f32_to_f16_bits(w).view(np.uint8).reshape(rows, cols * 2)
    return out


def dequant(fmt: int, blocks: np.ndarray, rows: int, cols: int) -> np.ndarray:
    blocks = np.ascontiguousarray(blocks)
    out = np.empty((rows, cols), np.float32)
    if fmt == FMT_Q8_0:
        lib().oracle_dequant_q8_0(_p(blocks), rows, cols, _p(out))
    elif fmt == FMT_Q4_0:
        lib().oracle_dequant_q4_0(_p(blocks), rows, cols, _p(out))
    else:
        out = f16_bits_to_f32(blocks.view(np.uint16).reshape(rows, cols))
    return out


def quantize_rowq8(w):
    w = _f32(w)
    rows, cols = w.shape
    q = np.empty((rows, cols), np.int8)
    s = np.empty(rows, np.float32)
    lib().oracle_quantize_rowq8(_p(w), rows, cols, _p(q), _p(s))
    return q, s


def matvec(fmt: int, blocks: np.ndarray, x, N: int, K: int) -> np.ndarray:
    blocks = np.ascontiguousarray(blocks)
    x = _f32(x)
    y = np.empty(N, np.float32)
    lib().oracle_matvec(fmt, _p(blocks), _p(x), _p(y), N, K)
    return y


def rowq8_matvec(act, w_i8, scales) -> np.ndarray:
    w = np.ascontiguousarray(w_i8, dtype=np.int8)
    N, K = w.shape
    act, scales = _f32(act), _f32(scales)
    out = np.empty(N, np.float32)
    lib().oracle_rowq8_matvec(_p(act), _p(w), _p(scales), _p(out), N, K)
    return out


def rowq4_matvec(act, w_packed, scales) -> np.ndarray:
    w = np.ascontiguousarray(w_packed, dtype=np.uint8)
    N, halfK = w.shape
    act, scales = _f32(act), _f32(scales)
    out = np.empty(N, np.float32)
    lib().oracle_rowq4_matvec(_p(act), _p(w), _p(scales), _p(out), N, halfK * 2)
    return out


def rmsnorm(x, w, eps: float = 1e-6) -> np.ndarray:
    x, w = _f32(x), _f32(w)
    out = np.empty_like(x)
    lib().oracle_rmsnorm(_p(x), _p(out), _p(w), x.size, eps)
    return out


def rope_tables(max_seq: int, head_dim: int, theta: float):
    half = head_dim // 2
    c = np.empty((max_seq, half), np.float32)
    s = np.empty((max_seq, half), np.float32)
    lib().oracle_rope_tables(max_seq, head_dim, float(theta), _p(c), _p(s))
    return c, s


def rope(x, cos_row, sin_row, head_dim: int, n_heads: int) -> np.ndarray:
    x = _f32(x).copy()
    cos_row, sin_row = _f32(cos_row), _f32(sin_row)
    lib().oracle_rope(_p(x), _p(cos_row), _p(sin_row), head_dim, n_heads)
    return x


def decode_attention(q, kc, vc, cache_len: int, n_heads: int, n_kv_heads: int) -> np.ndarray:
    """kc / vc: fp32 [>=cache_len, kvDim], or uint16 fp16 bit patterns."""
    q = _f32(q)
    out = np.empty_like(q)
    kv_dim = kc.shape[1]
    if kc.dtype == np.uint16:
        kc, vc = np.ascontiguousarray(kc), np.ascontiguousarray(vc)
        lib().oracle_decode_attention_f16kv(_p(q), _p(kc), _p(vc), _p(out), cache_len, q.size, kv_dim,
                                            n_heads, n_kv_heads)
    else:
        kc, vc = _f32(kc), _f32(vc)
        lib().oracle_decode_attention(_p(q), _p(kc), _p(vc), _p(out), cache_len, q.size, kv_dim, n_heads,
                                      n_kv_heads)
    return out


def silu_gate_mul(g, u) -> np.ndarray:
    g, u = _f32(g), _f32(u)
    out = np.empty_like(g)
    lib().oracle_silu_gate_mul(_p(g), _p(u), _p(out), g.size)
    return out


def cpu_engine_matmul(a, b) -> np.ndarray:
    a, b = _f32(a), _f32(b)
    m, k = a.shape
    n = b.shape[1]
    out = np.empty((m, n), np.float32)
    lib().oracle_cpu_engine_matmul(_p(a), _p(b), _p(out), m, k, n)
    return out


def cpu_engine_matvec(fmt: int, blocks, x, N: int, K: int, nthreads: int = 1) -> np.ndarray:
    blocks = np.ascontiguousarray(blocks)
    x = _f32(x)
    y = np.empty(N, np.float32)
    lib().oracle_cpu_engine_matvec(fmt, _p(blocks), _p(x), _p(y), N, K, nthreads)
    return y


def max_threads() -> int:
    return int(lib().oracle_max_threads())


class OracleModel:
    """Whole-model decode on the CPU; weights are held as the same raw blocks
    the engine consumes.  Index scheme: layer*12 + slot, nL*12 final norm,
    nL*12+1 lm_head (cuda_fused_infer.go:241-272)."""

    def __init__(self, cfg):
        self.cfg = cfg
        self._keep = {}
        self._h = lib().oracle_model_create(cfg.dim, cfg.kv_dim, cfg.head_dim, cfg.n_heads, cfg.n_kv_heads,
                                            cfg.ffn_dim, cfg.vocab, cfg.n_layers, cfg.max_seq,
                                            float(cfg.rope_theta), float(cfg.eps))

    def close(self):
        if self._h:
            lib().oracle_model_destroy(self._h)
            self._h = None

    def __del__(self):
        self.close()

    def set_weight(self, idx: int, data: np.ndarray, fmt: int = FMT_Q8_0):
        data = np.ascontiguousarray(data)
        self._keep[idx] = data
        lib().oracle_model_set_weight(self._h, idx, _p(data), fmt)

    def reset_kv(self):
        lib().oracle_model_reset_kv(self._h)

    def embed(self, token: int) -> np.ndarray:
        out = np.empty(self.cfg.dim, np.float32)
        lib().oracle_model_embed(self._h, int(token), _p(out))
        return out

    def step(self, hidden, pos: int, layer_start: int = 0, layer_end: int | None = None, want_logits=True):
        """Returns (hidden_out, logits or None)."""
        cfg = self.cfg
        layer_end = cfg.n_layers if layer_end is None else layer_end
        h = _f32(hidden).copy()
        logits = np.empty(cfg.vocab, np.float32) if (want_logits and layer_end >= cfg.n_layers) else None
        lib().oracle_model_step(self._h, _p(h), pos, layer_start, layer_end,
                                _p(logits) if logits is not None else None)
        return h, logits

    def step_token(self, token: int, pos: int) -> np.ndarray:
        logits = np.empty(self.cfg.vocab, np.float32)
        lib().oracle_model_step_token(self._h, int(token), pos, _p(logits))
        return logits

    def cpu_engine_step_token(self, token: int, pos: int, nthreads: int = 1) -> np.ndarray:
        logits = np.empty(self.cfg.vocab, np.float32)
        lib().oracle_cpu_engine_step_token(self._h, int(token), pos, _p(logits), nthreads)
        return logits

    def kv_cache(self, layer: int):
        n = self.cfg.max_seq * self.cfg.kv_dim
        kp = lib().oracle_model_kcache(self._h, layer)
        vp = lib().oracle_model_vcache(self._h, layer)
        k = np.ctypeslib.as_array(C.cast(kp, C.POINTER(C.c_uint16)), shape=(n,)).copy()
        v = np.ctypeslib.as_array(C.cast(vp, C.POINTER(C.c_uint16)), shape=(n,)).copy()
        return k.reshape(self.cfg.max_seq, -1), v.reshape(self.cfg.max_seq, -1)
