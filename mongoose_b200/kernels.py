"""K* wrappers: the Python counterpart of the Go dispatch shim in kernels.go
(``KRMSNormOut``, ``KQ8Matvec``, ``KRoPE`` ... kernels.go:598-1136).

Arguments are raw device addresses (ints) or objects with ``data_ptr()``
(torch tensors); everything is enqueued on ``stream`` (default: the legacy
default stream 0, which is what the reference's ``tw_k_*`` trampolines use,
kernels.go:231-294).
"""
from __future__ import annotations

from . import _lib


def _ptr(x):
    if x is None:
        return None
    if isinstance(x, int):
        return x
    return x.data_ptr()


def _stream(stream):
    if stream is None:
        return None
    if isinstance(stream, int):
        return stream
    return stream.cuda_stream   # torch.cuda.Stream


def KernelsLoaded() -> bool:
    try:
        _lib.load()
        return True
    except RuntimeError:
        return False


def KRMSNorm(x, weight, seqLen, dim, stream=None):
    _lib.load().mongoose_rmsnorm(_ptr(x), _ptr(weight), seqLen, dim, _stream(stream))


def KRMSNormOut(inp, out, weight, seqLen, dim, stream=None):
    _lib.load().mongoose_rmsnorm_out(_ptr(inp), _ptr(out), _ptr(weight), seqLen, dim, _stream(stream))


def KFusedAddRMSNorm(a, b, out, weight, seqLen, dim, stream=None):
    _lib.load().mongoose_fused_add_rmsnorm(_ptr(a), _ptr(b), _ptr(out), _ptr(weight), seqLen, dim, _stream(stream))


def KReLU(x, n, stream=None):
    _lib.load().mongoose_relu(_ptr(x), n, _stream(stream))


def KAddInPlace(a, b, n, stream=None):
    _lib.load().mongoose_add_inplace(_ptr(a), _ptr(b), n, _stream(stream))


def KEmbeddingGather(out, tokEmb, posEmb, tokens, seqLen, dim, stream=None):
    _lib.load().mongoose_embedding_gather(_ptr(out), _ptr(tokEmb), _ptr(posEmb), _ptr(tokens), seqLen, dim,
                                          _stream(stream))


def KEmbedGather(out, embed, tokens, seqLen, dim, stream=None):
    _lib.load().mongoose_embed_gather(_ptr(out), _ptr(embed), _ptr(tokens), seqLen, dim, _stream(stream))


def KSiLUGateMul(gate, up, out, n, stream=None):
    _lib.load().mongoose_silu_gate_mul(_ptr(gate), _ptr(up), _ptr(out), n, _stream(stream))


def KRoPE(x, cosTab, sinTab, seqLen, dim, headDim, nHeads, stream=None):
    _lib.load().mongoose_rope(_ptr(x), _ptr(cosTab), _ptr(sinTab), seqLen, dim, headDim, nHeads, _stream(stream))


def KKVCacheWrite(cache, src, pos, kvDim, stream=None):
    _lib.load().mongoose_kv_cache_write(_ptr(cache), _ptr(src), pos, kvDim, _stream(stream))


def KDecodeAttention(Q, Kc, Vc, out, cacheLen, dim, kvDim, nHeads, nKVHeads, stream=None):
    _lib.load().mongoose_decode_attention(_ptr(Q), _ptr(Kc), _ptr(Vc), _ptr(out), cacheLen, dim, kvDim, nHeads,
                                          nKVHeads, _stream(stream))


def KQ8Matvec(act, w_i8, scales, out, N, K, stream=None):
    _lib.load().mongoose_q8_matvec(_ptr(act), _ptr(w_i8), _ptr(scales), _ptr(out), N, K, _stream(stream))


def KQ4Matvec(act, w_packed, scales, out, N, K, stream=None):
    _lib.load().mongoose_q4_matvec(_ptr(act), _ptr(w_packed), _ptr(scales), _ptr(out), N, K, _stream(stream))


def KQ4_0Matvec(act, w_blocks, out, N, K, stream=None):
    _lib.load().mongoose_q4_0_matvec(_ptr(act), _ptr(w_blocks), _ptr(out), N, K, _stream(stream))


def KQ8_0Matvec(act, w_blocks, out, N, K, stream=None):
    _lib.load().mongoose_q8_0_matvec(_ptr(act), _ptr(w_blocks), _ptr(out), N, K, _stream(stream))


def KQ8QuantizeAct(act, q8_out, K, stream=None):
    _lib.load().mongoose_q8_quantize_act(_ptr(act), _ptr(q8_out), K, _stream(stream))


def KQ8QuantizeActBatch(acts, q8_out, K, B, stream=None):
    _lib.load().mongoose_q8_quantize_act_batch(_ptr(acts), _ptr(q8_out), K, B, _stream(stream))


def KQ4_0MatvecDP4A(act, w_blocks, out, N, K, scratch, stream=None):
    _lib.load().mongoose_q4_0_matvec_dp4a(_ptr(act), _ptr(w_blocks), _ptr(out), N, K, _ptr(scratch),
                                          _stream(stream))


def KQ4_0MatvecDP4APreq(w_blocks, q8, out, N, K, stream=None):
    _lib.load().mongoose_q4_0_matvec_dp4a_preq(_ptr(w_blocks), _ptr(q8), _ptr(out), N, K, _stream(stream))


def KQ4_0MatvecDP4ABatch(w_blocks, q8, out, N, K, B, stream=None):
    _lib.load().mongoose_q4_0_matvec_dp4a_batch(_ptr(w_blocks), _ptr(q8), _ptr(out), N, K, B, _stream(stream))


def KQ4_0MatvecDP4AStatic(act, w_blocks, out, N, K, stream=None) -> int:
    """Integer-dot Q4_0 matvec whose activation scratch is a fixed array inside the library: for
    callers that are not allowed to allocate.  Returns the C status (0 = ok)."""
    return _lib.load().mongoose_q4_0_matvec_dp4a_static(_ptr(act), _ptr(w_blocks), _ptr(out), N, K, _stream(stream))


def StaticScratchError() -> str:
    return _lib.load().mongoose_static_scratch_error().decode()


def KCopy(dst, src, nbytes, stream=None):
    _lib.load().mongoose_copy(_ptr(dst), _ptr(src), nbytes, _stream(stream))


def KZero(ptr, nbytes, stream=None):
    _lib.load().mongoose_zero(_ptr(ptr), nbytes, _stream(stream))


def KSync(stream=None):
    _lib.load().mongoose_sync(_stream(stream))


def KFP32ToFP16(inp, out, n, stream=None):
    _lib.load().mongoose_fp32_to_fp16(_ptr(inp), _ptr(out), n, _stream(stream))


def KFP16ToFP32(inp, out, n, stream=None):
    _lib.load().mongoose_fp16_to_fp32(_ptr(inp), _ptr(out), n, _stream(stream))
