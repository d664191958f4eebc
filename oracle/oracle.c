/*
 * CPU oracle for mongoose's fused quantized decode path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file restates, in plain C, the arithmetic
 * of the reference's single-token decode path so that the CUDA library can
 * be checked against it.  Nothing in the shipped library links or calls it.
 *
 * Parity status:
 *   - per-row INT8 / per-row INT4 matvec, RMSNorm, rotate-half RoPE, KV
 *     append, decode attention, SiLU-gate, residual add: pinned against the
 *     reference's own CUDA kernels (kernels/mongoose.cu built unmodified and
 *     run on a B200; golden vectors under tests/golden/).
 *   - block-32 Q8_0 / GGUF Q4_0 matvec: PARITY UNPINNED.  The reference
 *     dlsym's mongoose_q4_0_matvec (kernels.go:206) but ships no source for
 *     it, and has no block-32 int8 kernel at all.  The block layouts follow
 *     cuda_q4_0.go:13-17 (18-byte GGUF block) and kernels/q4_simd.metal:4-19
 *     (nibble order); the quantizers follow metal_impl_darwin.m:5737-5781.
 *
 * Accumulation is in double everywhere ("truth"), outputs are rounded to
 * float once per op.  The *_ref32 variants reproduce the reference kernels'
 * fp32 arithmetic order closely and are used for pinning only.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------ */
/* fp16 codec (IEEE binary16, round-to-nearest-even on encode).        */
/* Decode follows conductor.go:7-24 (HalfToFloat); encode is RNE, not   */
/* the truncating FloatToHalf of conductor.go:27-35, because block     */
/* scales are produced by a C cast (metal_impl_darwin.m:5750).          */
/* ------------------------------------------------------------------ */
ORACLE_API float oracle_f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h >> 15) & 1u;
    uint32_t exp = (uint32_t)(h >> 10) & 0x1fu;
    uint32_t mant = (uint32_t)h & 0x3ffu;
    uint32_t bits;
    if (exp == 0) {
        if (mant == 0) {
            bits = sign << 31;
        } else {
            int e = -1;
            do { mant <<= 1; e++; } while ((mant & 0x400u) == 0);
            mant &= 0x3ffu;
            bits = (sign << 31) | ((uint32_t)(127 - 15 - e) << 23) | (mant << 13);
        }
    } else if (exp == 31) {
        bits = (sign << 31) | 0x7f800000u | (mant << 13);
    } else {
        bits = (sign << 31) | ((exp + 112u) << 23) | (mant << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

ORACLE_API uint16_t oracle_f32_to_f16(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t ax = x & 0x7fffffffu;
    if (ax >= 0x7f800000u) { /* inf / nan */
        return (uint16_t)(sign | 0x7c00u | ((ax > 0x7f800000u) ? 0x200u : 0u));
    }
    if (ax >= 0x477ff000u) { /* rounds to >= 65520 -> inf */
        return (uint16_t)(sign | 0x7c00u);
    }
    if (ax < 0x38800000u) { /* subnormal half or zero */
        if (ax < 0x33000000u) return (uint16_t)sign; /* < 2^-25 -> 0 */
        int e = (int)(ax >> 23);             /* biased exponent */
        uint32_t m = (ax & 0x7fffffu) | 0x800000u;
        int shift = 126 - e;                 /* half-subnormal ulp is 2^-24 */
        uint32_t q = m >> shift;
        uint32_t rem = m & ((1u << shift) - 1u);
        uint32_t half = 1u << (shift - 1);
        if (rem > half || (rem == half && (q & 1u))) q++;
        return (uint16_t)(sign | q);
    }
    uint32_t e = (ax >> 23) - 112u;
    uint32_t m = ax & 0x7fffffu;
    uint32_t q = (e << 10) | (m >> 13);
    uint32_t rem = m & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (q & 1u))) q++;
    return (uint16_t)(sign | q);
}

ORACLE_API void oracle_f32_to_f16_n(const float* in, uint16_t* out, long n) {
    for (long i = 0; i < n; i++) out[i] = oracle_f32_to_f16(in[i]);
}
ORACLE_API void oracle_f16_to_f32_n(const uint16_t* in, float* out, long n) {
    for (long i = 0; i < n; i++) out[i] = oracle_f16_to_f32(in[i]);
}

/* ------------------------------------------------------------------ */
/* Quantizers.                                                         */
/* ------------------------------------------------------------------ */

static inline int round_half_away(float v) {
    /* metal_impl_darwin.m:5755-5756: (int)(v + (v > 0 ? 0.5f : -0.5f)) */
    return (int)(v + (v > 0 ? 0.5f : -0.5f));
}

/* Block-32 Q8_0: 34-byte blocks {fp16 d, int8 q[32]} along the input dim.
 * d = amax/127 (per block), q = round-half-away(v * 127/amax), clamp +-127.
 * Same rounding and clamp as the reference's Metal per-row Q8 quantizer
 * (metal_impl_darwin.m:5765-5781), applied per block of 32. */
ORACLE_API void oracle_quantize_q8_0(const float* w, long rows, long cols, uint8_t* blocks) {
    long nb = cols / 32;
#pragma omp parallel for schedule(static)
    for (long r = 0; r < rows; r++) {
        for (long b = 0; b < nb; b++) {
            const float* src = w + r * cols + b * 32;
            float amax = 0.f;
            for (int j = 0; j < 32; j++) {
                float v = fabsf(src[j]);
                if (v > amax) amax = v;
            }
            uint8_t* blk = blocks + (r * nb + b) * 34;
            uint16_t d = oracle_f32_to_f16(amax / 127.0f);
            memcpy(blk, &d, 2);
            float inv = amax > 0 ? 127.0f / amax : 0.f;
            int8_t* q = (int8_t*)(blk + 2);
            for (int j = 0; j < 32; j++) {
                float v = src[j] * inv;
                if (v > 127.f) v = 127.f;
                if (v < -127.f) v = -127.f;
                q[j] = (int8_t)round_half_away(v);
            }
        }
    }
}

/* GGUF Q4_0: 18-byte blocks {fp16 d, uint8 qs[16]}; byte j holds element j
 * in its low nibble and element j+16 in its high nibble
 * (kernels/q4_simd.metal:4-19); value = d * (nibble - 8).
 * d = amax/8, round-half-away, +8, clamp 0..15 (metal_impl_darwin.m:5744-5761;
 * that quantizer packs sequential pairs, the GGUF order is used here because
 * cuda_q4_0.go:13-14 uploads raw GGUF blocks). */
ORACLE_API void oracle_quantize_q4_0(const float* w, long rows, long cols, uint8_t* blocks) {
    long nb = cols / 32;
#pragma omp parallel for schedule(static)
    for (long r = 0; r < rows; r++) {
        for (long b = 0; b < nb; b++) {
            const float* src = w + r * cols + b * 32;
            float amax = 0.f;
            for (int j = 0; j < 32; j++) {
                float v = fabsf(src[j]);
                if (v > amax) amax = v;
            }
            uint8_t* blk = blocks + (r * nb + b) * 18;
            uint16_t d = oracle_f32_to_f16(amax / 8.0f);
            memcpy(blk, &d, 2);
            float inv = amax > 0 ? 8.0f / amax : 0.f;
            uint8_t* qs = blk + 2;
            for (int j = 0; j < 16; j++) {
                int q0 = round_half_away(src[j] * inv) + 8;
                int q1 = round_half_away(src[j + 16] * inv) + 8;
                if (q0 < 0) q0 = 0;
                if (q0 > 15) q0 = 15;
                if (q1 < 0) q1 = 0;
                if (q1 > 15) q1 = 15;
                qs[j] = (uint8_t)(q0 | (q1 << 4));
            }
        }
    }
}

/* Per-row INT8 exactly as CUDAFusedInference.quantizeQ8
 * (cuda_fused_infer.go:363-383): s = amax/127, q = int(v * (1/s)) which
 * truncates toward zero, clamp [-128,127]; scales[r] = s. */
ORACLE_API void oracle_quantize_rowq8(const float* w, long rows, long cols, int8_t* q, float* scales) {
    for (long r = 0; r < rows; r++) {
        float amax = 0.f;
        for (long c = 0; c < cols; c++) {
            float v = w[r * cols + c];
            if (v < 0) v = -v;
            if (v > amax) amax = v;
        }
        float s = amax / 127.0f;
        scales[r] = s;
        if (s > 0) {
            float inv = 1.0f / s;
            for (long c = 0; c < cols; c++) {
                int v = (int)(w[r * cols + c] * inv);
                if (v > 127) v = 127; else if (v < -128) v = -128;
                q[r * cols + c] = (int8_t)v;
            }
        } else {
            memset(q + r * cols, 0, (size_t)cols);
        }
    }
}

ORACLE_API void oracle_dequant_q8_0(const uint8_t* blocks, long rows, long cols, float* out) {
    long nb = cols / 32;
    for (long r = 0; r < rows; r++)
        for (long b = 0; b < nb; b++) {
            const uint8_t* blk = blocks + (r * nb + b) * 34;
            uint16_t dh;
            memcpy(&dh, blk, 2);
            float d = oracle_f16_to_f32(dh);
            const int8_t* q = (const int8_t*)(blk + 2);
            for (int j = 0; j < 32; j++) out[r * cols + b * 32 + j] = d * (float)q[j];
        }
}

ORACLE_API void oracle_dequant_q4_0(const uint8_t* blocks, long rows, long cols, float* out) {
    long nb = cols / 32;
    for (long r = 0; r < rows; r++)
        for (long b = 0; b < nb; b++) {
            const uint8_t* blk = blocks + (r * nb + b) * 18;
            uint16_t dh;
            memcpy(&dh, blk, 2);
            float d = oracle_f16_to_f32(dh);
            const uint8_t* qs = blk + 2;
            for (int j = 0; j < 16; j++) {
                out[r * cols + b * 32 + j] = d * (float)((int)(qs[j] & 0xF) - 8);
                out[r * cols + b * 32 + j + 16] = d * (float)((int)(qs[j] >> 4) - 8);
            }
        }
}

/* ------------------------------------------------------------------ */
/* Matvecs (double accumulate).  Weight formats:                       */
/*   0 = Q8_0 blocks, 1 = Q4_0 blocks, 2 = fp16 row-major.             */
/* ------------------------------------------------------------------ */
enum { FMT_Q8_0 = 0, FMT_Q4_0 = 1, FMT_F16 = 2 };

static double row_dot(int fmt, const uint8_t* wrow, const float* x, long K) {
    double acc = 0.0;
    long nb = K / 32;
    if (fmt == FMT_Q8_0) {
        for (long b = 0; b < nb; b++) {
            const uint8_t* blk = wrow + b * 34;
            uint16_t dh;
            memcpy(&dh, blk, 2);
            const int8_t* q = (const int8_t*)(blk + 2);
            const float* xb = x + b * 32;
            double s = 0.0;
            for (int j = 0; j < 32; j++) s += (double)xb[j] * (double)q[j];
            acc += (double)oracle_f16_to_f32(dh) * s;
        }
    } else if (fmt == FMT_Q4_0) {
        for (long b = 0; b < nb; b++) {
            const uint8_t* blk = wrow + b * 18;
            uint16_t dh;
            memcpy(&dh, blk, 2);
            const uint8_t* qs = blk + 2;
            const float* xb = x + b * 32;
            double s = 0.0;
            for (int j = 0; j < 16; j++) {
                s += (double)xb[j] * (double)((int)(qs[j] & 0xF) - 8);
                s += (double)xb[j + 16] * (double)((int)(qs[j] >> 4) - 8);
            }
            acc += (double)oracle_f16_to_f32(dh) * s;
        }
    } else {
        const uint16_t* wh = (const uint16_t*)wrow;
        for (long k = 0; k < K; k++) acc += (double)x[k] * (double)oracle_f16_to_f32(wh[k]);
    }
    return acc;
}

static long row_bytes(int fmt, long K) {
    return fmt == FMT_Q8_0 ? (K / 32) * 34 : fmt == FMT_Q4_0 ? (K / 32) * 18 : K * 2;
}

/* y = W x for a block-quantized (or fp16) W of N rows by K columns. */
ORACLE_API void oracle_matvec(int fmt, const void* w, const float* x, float* y, long N, long K) {
    long rb = row_bytes(fmt, K);
#pragma omp parallel for schedule(static)
    for (long r = 0; r < N; r++) y[r] = (float)row_dot(fmt, (const uint8_t*)w + r * rb, x, K);
}

/* Per-row INT8 matvec with the literal kernel semantic
 * out[r] = sum_k act[k] * float(w[r,k]) * (scales[r]/127)
 * (kernels/mongoose.cu:1554-1585). */
ORACLE_API void oracle_rowq8_matvec(const float* act, const int8_t* w, const float* scales, float* out,
                                    long N, long K) {
#pragma omp parallel for schedule(static)
    for (long r = 0; r < N; r++) {
        float scale = scales[r] / 127.0f;
        double acc = 0.0;
        for (long k = 0; k < K; k++) acc += (double)act[k] * (double)w[r * K + k];
        out[r] = (float)(acc * (double)scale);
    }
}

/* Per-row 4-bit matvec: byte k holds element 2k (low) and 2k+1 (high),
 * value = (nibble-8) * scales[r]/7 (kernels/mongoose.cu:1597-1630). */
ORACLE_API void oracle_rowq4_matvec(const float* act, const uint8_t* w, const float* scales, float* out,
                                    long N, long K) {
    long halfK = K / 2;
#pragma omp parallel for schedule(static)
    for (long r = 0; r < N; r++) {
        float scale = scales[r] / 7.0f;
        double acc = 0.0;
        for (long k = 0; k < halfK; k++) {
            uint8_t p = w[r * halfK + k];
            acc += (double)act[2 * k] * (double)((int)(p & 0xF) - 8);
            acc += (double)act[2 * k + 1] * (double)((int)(p >> 4) - 8);
        }
        out[r] = (float)(acc * (double)scale);
    }
}

/* ------------------------------------------------------------------ */
/* Element-wise / normalisation / attention ops.                       */
/* ------------------------------------------------------------------ */

/* out = in * rsqrt(mean(in^2) + eps) * w   (kernels/mongoose.cu:145-175;
 * the reference hard-codes eps = 1e-6 at :170). */
ORACLE_API void oracle_rmsnorm(const float* in, float* out, const float* w, long dim, float eps) {
    double ss = 0.0;
    for (long i = 0; i < dim; i++) ss += (double)in[i] * (double)in[i];
    double scale = 1.0 / sqrt(ss / (double)dim + (double)eps);
    for (long i = 0; i < dim; i++) out[i] = (float)((double)in[i] * scale * (double)w[i]);
}

/* cos/sin tables built in float64 then narrowed, entry [pos*half + j]
 * (cuda_fused_infer.go:181-190). */
ORACLE_API void oracle_rope_tables(long maxSeq, long headDim, double theta, float* cosT, float* sinT) {
    long half = headDim / 2;
    for (long pos = 0; pos < maxSeq; pos++)
        for (long j = 0; j < half; j++) {
            double freq = 1.0 / pow(theta, (double)(2 * j) / (double)headDim);
            double angle = (double)pos * freq;
            cosT[pos * half + j] = (float)cos(angle);
            sinT[pos * half + j] = (float)sin(angle);
        }
}

/* rotate-half RoPE on one position: pairs (x[j], x[j+half]) per head
 * (kernels/mongoose.cu:987-1006).  cosT/sinT point at the row for `pos`. */
ORACLE_API void oracle_rope(float* x, const float* cosT, const float* sinT, long headDim, long nHeads) {
    long half = headDim / 2;
    for (long h = 0; h < nHeads; h++)
        for (long j = 0; j < half; j++) {
            double c = cosT[j], s = sinT[j];
            double x0 = x[h * headDim + j], x1 = x[h * headDim + half + j];
            x[h * headDim + j] = (float)(x0 * c - x1 * s);
            x[h * headDim + half + j] = (float)(x0 * s + x1 * c);
        }
}

/* softmax(Q K^T / sqrt(hd)) V over cacheLen cached positions, one query
 * position, grouped-query heads (kernels/mongoose.cu:853-933).  K and V
 * are fp32 [cacheLen, kvDim]. */
ORACLE_API void oracle_decode_attention(const float* Q, const float* Kc, const float* Vc, float* out,
                                        long cacheLen, long dim, long kvDim, long nHeads, long nKVHeads) {
    long hd = dim / nHeads;
    long group = nHeads / nKVHeads;
    double scale = 1.0 / sqrt((double)hd);
    double* p = (double*)malloc(sizeof(double) * (size_t)cacheLen);
    for (long h = 0; h < nHeads; h++) {
        long kvOff = (h / group) * hd;
        double mx = -1e300;
        for (long t = 0; t < cacheLen; t++) {
            double dot = 0.0;
            for (long d = 0; d < hd; d++) dot += (double)Q[h * hd + d] * (double)Kc[t * kvDim + kvOff + d];
            p[t] = dot * scale;
            if (p[t] > mx) mx = p[t];
        }
        double sum = 0.0;
        for (long t = 0; t < cacheLen; t++) {
            p[t] = exp(p[t] - mx);
            sum += p[t];
        }
        for (long d = 0; d < hd; d++) {
            double acc = 0.0;
            for (long t = 0; t < cacheLen; t++) acc += p[t] * (double)Vc[t * kvDim + kvOff + d];
            out[h * hd + d] = (float)(acc / sum);
        }
    }
    free(p);
}

/* Same with an fp16 KV cache (values decoded to fp32 first). */
ORACLE_API void oracle_decode_attention_f16kv(const float* Q, const uint16_t* Kc, const uint16_t* Vc, float* out,
                                              long cacheLen, long dim, long kvDim, long nHeads, long nKVHeads) {
    size_t n = (size_t)cacheLen * (size_t)kvDim;
    float* kf = (float*)malloc(n * 4);
    float* vf = (float*)malloc(n * 4);
    oracle_f16_to_f32_n(Kc, kf, (long)n);
    oracle_f16_to_f32_n(Vc, vf, (long)n);
    oracle_decode_attention(Q, kf, vf, out, cacheLen, dim, kvDim, nHeads, nKVHeads);
    free(kf);
    free(vf);
}

/* out = g * 1/(1+exp(-g)) * up   (kernels/mongoose.cu:947-956). */
ORACLE_API void oracle_silu_gate_mul(const float* gate, const float* up, float* out, long n) {
    for (long i = 0; i < n; i++) {
        double g = gate[i];
        out[i] = (float)(g / (1.0 + exp(-g)) * (double)up[i]);
    }
}

/* a += b   (kernels/mongoose.cu:211-215). */
ORACLE_API void oracle_add_inplace(float* a, const float* b, long n) {
    for (long i = 0; i < n; i++) a[i] = (float)((double)a[i] + (double)b[i]);
}

/* ------------------------------------------------------------------ */
/* Whole-model decode step: the op order of PartialStep                */
/* (cuda_fused_infer.go:414-451) with block-quantized weights and an   */
/* fp16 KV cache (K after RoPE and V rounded RNE on append).            */
/* Weight slots use the reference's index scheme layer*12 + w          */
/* (cuda_fused_infer.go:241-272): 0 norm1, 1 wq, 2 wk, 3 wv, 4-6 QKV   */
/* bias, 7 wo, 8 norm2, 9 gate, 10 up, 11 down; nL*12 final norm;      */
/* nL*12+1 lm_head.                                                    */
/* ------------------------------------------------------------------ */
typedef struct {
    long dim, kvDim, headDim, nHeads, nKVHeads, ffnDim, vocab, nLayers, maxSeq;
    float eps;
    const void** w;   /* nLayers*12 + 2 borrowed pointers */
    int* fmt;         /* format of each matrix slot */
    float *cosT, *sinT;
    uint16_t **kc, **vc; /* per layer [maxSeq*kvDim] */
    /* scratch */
    float *h, *normed, *q, *k, *v, *attn, *proj, *gate, *up, *mid;
} oracle_model;

ORACLE_API oracle_model* oracle_model_create(long dim, long kvDim, long headDim, long nHeads, long nKVHeads,
                                             long ffnDim, long vocab, long nLayers, long maxSeq, double theta,
                                             float eps) {
    oracle_model* m = (oracle_model*)calloc(1, sizeof(oracle_model));
    m->dim = dim; m->kvDim = kvDim; m->headDim = headDim; m->nHeads = nHeads; m->nKVHeads = nKVHeads;
    m->ffnDim = ffnDim; m->vocab = vocab; m->nLayers = nLayers; m->maxSeq = maxSeq; m->eps = eps;
    long nw = nLayers * 12 + 2;
    m->w = (const void**)calloc((size_t)nw, sizeof(void*));
    m->fmt = (int*)calloc((size_t)nw, sizeof(int));
    long half = headDim / 2;
    m->cosT = (float*)malloc(sizeof(float) * (size_t)(maxSeq * half));
    m->sinT = (float*)malloc(sizeof(float) * (size_t)(maxSeq * half));
    oracle_rope_tables(maxSeq, headDim, theta, m->cosT, m->sinT);
    m->kc = (uint16_t**)calloc((size_t)nLayers, sizeof(void*));
    m->vc = (uint16_t**)calloc((size_t)nLayers, sizeof(void*));
    for (long l = 0; l < nLayers; l++) {
        m->kc[l] = (uint16_t*)calloc((size_t)(maxSeq * kvDim), 2);
        m->vc[l] = (uint16_t*)calloc((size_t)(maxSeq * kvDim), 2);
    }
    long mx = dim > ffnDim ? dim : ffnDim;
    m->h = (float*)calloc((size_t)dim, 4); m->normed = (float*)calloc((size_t)dim, 4);
    m->q = (float*)calloc((size_t)dim, 4); m->k = (float*)calloc((size_t)kvDim, 4);
    m->v = (float*)calloc((size_t)kvDim, 4); m->attn = (float*)calloc((size_t)dim, 4);
    m->proj = (float*)calloc((size_t)mx, 4); m->gate = (float*)calloc((size_t)ffnDim, 4);
    m->up = (float*)calloc((size_t)ffnDim, 4); m->mid = (float*)calloc((size_t)ffnDim, 4);
    return m;
}

ORACLE_API void oracle_model_destroy(oracle_model* m) {
    if (!m) return;
    for (long l = 0; l < m->nLayers; l++) { free(m->kc[l]); free(m->vc[l]); }
    free(m->kc); free(m->vc); free(m->cosT); free(m->sinT); free((void*)m->w); free(m->fmt);
    free(m->h); free(m->normed); free(m->q); free(m->k); free(m->v); free(m->attn);
    free(m->proj); free(m->gate); free(m->up); free(m->mid);
    free(m);
}

/* Borrow a pointer for slot idx.  Norm and bias slots are fp32 vectors
 * (fmt ignored); matrix slots are in `fmt`.  The caller keeps the memory alive. */
ORACLE_API void oracle_model_set_weight(oracle_model* m, long idx, const void* data, int fmt) {
    m->w[idx] = data;
    m->fmt[idx] = fmt;
}

ORACLE_API void oracle_model_reset_kv(oracle_model* m) {
    for (long l = 0; l < m->nLayers; l++) {
        memset(m->kc[l], 0, (size_t)(m->maxSeq * m->kvDim) * 2);
        memset(m->vc[l], 0, (size_t)(m->maxSeq * m->kvDim) * 2);
    }
}

/* Dequantized row `token` of the lm_head matrix: the tied input embedding. */
ORACLE_API void oracle_model_embed(const oracle_model* m, long token, float* out) {
    long idx = m->nLayers * 12 + 1;
    int fmt = m->fmt[idx];
    const uint8_t* row = (const uint8_t*)m->w[idx] + token * row_bytes(fmt, m->dim);
    if (fmt == FMT_Q8_0) oracle_dequant_q8_0(row, 1, m->dim, out);
    else if (fmt == FMT_Q4_0) oracle_dequant_q4_0(row, 1, m->dim, out);
    else oracle_f16_to_f32_n((const uint16_t*)row, out, m->dim);
}

/* One token through layers [layerStart, layerEnd).  hidden is updated in
 * place; logits (vocab floats) are written when layerEnd reaches the last
 * layer and logits != NULL. */
ORACLE_API void oracle_model_step(oracle_model* m, float* hidden, long pos, long layerStart, long layerEnd,
                                  float* logits) {
    long dim = m->dim, kvDim = m->kvDim, hd = m->headDim, half = hd / 2;
    const float* cosT = m->cosT + pos * half;
    const float* sinT = m->sinT + pos * half;
    for (long l = layerStart; l < layerEnd && l < m->nLayers; l++) {
        const void** W = m->w + l * 12;
        const int* F = m->fmt + l * 12;
        oracle_rmsnorm(hidden, m->normed, (const float*)W[0], dim, m->eps);
        oracle_matvec(F[1], W[1], m->normed, m->q, dim, dim);
        oracle_matvec(F[2], W[2], m->normed, m->k, kvDim, dim);
        oracle_matvec(F[3], W[3], m->normed, m->v, kvDim, dim);
        /* optional QKV bias, added before RoPE (cuda_fused_stream.go:319-321);
         * a NULL slot means no bias (cuda_fused_infer.go:255). */
        if (W[4]) oracle_add_inplace(m->q, (const float*)W[4], dim);
        if (W[5]) oracle_add_inplace(m->k, (const float*)W[5], kvDim);
        if (W[6]) oracle_add_inplace(m->v, (const float*)W[6], kvDim);
        oracle_rope(m->q, cosT, sinT, hd, m->nHeads);
        oracle_rope(m->k, cosT, sinT, hd, m->nKVHeads);
        oracle_f32_to_f16_n(m->k, m->kc[l] + pos * kvDim, kvDim);
        oracle_f32_to_f16_n(m->v, m->vc[l] + pos * kvDim, kvDim);
        oracle_decode_attention_f16kv(m->q, m->kc[l], m->vc[l], m->attn, pos + 1, dim, kvDim, m->nHeads,
                                      m->nKVHeads);
        oracle_matvec(F[7], W[7], m->attn, m->proj, dim, dim);
        oracle_add_inplace(hidden, m->proj, dim);
        oracle_rmsnorm(hidden, m->normed, (const float*)W[8], dim, m->eps);
        oracle_matvec(F[9], W[9], m->normed, m->gate, m->ffnDim, dim);
        oracle_matvec(F[10], W[10], m->normed, m->up, m->ffnDim, dim);
        oracle_silu_gate_mul(m->gate, m->up, m->mid, m->ffnDim);
        oracle_matvec(F[11], W[11], m->mid, m->proj, dim, m->ffnDim);
        oracle_add_inplace(hidden, m->proj, dim);
    }
    if (layerEnd >= m->nLayers && logits) {
        long fn = m->nLayers * 12;
        oracle_rmsnorm(hidden, m->normed, (const float*)m->w[fn], dim, m->eps);
        oracle_matvec(m->fmt[fn + 1], m->w[fn + 1], m->normed, logits, m->vocab, dim);
    }
}

/* First index of the maximum (ties resolve to the lowest index). */
ORACLE_API long oracle_argmax(const float* x, long n) {
    long best = 0;
    for (long i = 1; i < n; i++)
        if (x[i] > x[best]) best = i;
    return best;
}

/* Token in, logits out: embed(token) then every layer. */
ORACLE_API void oracle_model_step_token(oracle_model* m, long token, long pos, float* logits) {
    oracle_model_embed(m, token, m->h);
    oracle_model_step(m, m->h, pos, 0, m->nLayers, logits);
}

ORACLE_API const uint16_t* oracle_model_kcache(const oracle_model* m, long layer) { return m->kc[layer]; }
ORACLE_API const uint16_t* oracle_model_vcache(const oracle_model* m, long layer) { return m->vc[layer]; }

/* ------------------------------------------------------------------ */
/* Timed CPU baseline: a port of the reference's pure-Go CPU engine.   */
/* cpu.go:18-32 MatMul is a naive i/j/l triple loop with an fp32        */
/* accumulator; the engine has no quantized op, so a Q8_0 matvec on it  */
/* is "dequantize the row to fp32, then the MatMul inner loop".         */
/* nthreads <= 1 reproduces the single-threaded reference; > 1 splits    */
/* rows across OpenMP threads (labelled as such by the caller).          */
/* ------------------------------------------------------------------ */
ORACLE_API void oracle_cpu_engine_matvec(int fmt, const void* w, const float* x, float* y, long N, long K,
                                         int nthreads) {
    long rb = row_bytes(fmt, K);
#ifdef _OPENMP
    if (nthreads < 1) nthreads = 1;
#pragma omp parallel num_threads(nthreads)
#endif
    {
        float* row = (float*)malloc(sizeof(float) * (size_t)K);
#ifdef _OPENMP
#pragma omp for schedule(static)
#endif
        for (long r = 0; r < N; r++) {
            const uint8_t* wr = (const uint8_t*)w + r * rb;
            if (fmt == FMT_Q8_0) oracle_dequant_q8_0(wr, 1, K, row);
            else if (fmt == FMT_Q4_0) oracle_dequant_q4_0(wr, 1, K, row);
            else oracle_f16_to_f32_n((const uint16_t*)wr, row, K);
            float sum = 0.f;
            for (long l = 0; l < K; l++) sum += row[l] * x[l];
            y[r] = sum;
        }
        free(row);
    }
}

/* One decode step on the CPU-engine port: fp32 everywhere (cpu.go RMSNorm
 * :36-47 with a float accumulator, SoftMax :50-70), same op order as
 * PartialStep.  KV cache fp16 as in the oracle model so both consume the
 * same state.  Returns nothing; writes logits. */
ORACLE_API void oracle_cpu_engine_step_token(oracle_model* m, long token, long pos, float* logits, int nthreads) {
    long dim = m->dim, kvDim = m->kvDim, hd = m->headDim, half = hd / 2;
    oracle_model_embed(m, token, m->h);
    float* hidden = m->h;
    const float* cosT = m->cosT + pos * half;
    const float* sinT = m->sinT + pos * half;
    for (long l = 0; l < m->nLayers; l++) {
        const void** W = m->w + l * 12;
        const int* F = m->fmt + l * 12;
        oracle_rmsnorm(hidden, m->normed, (const float*)W[0], dim, m->eps);
        oracle_cpu_engine_matvec(F[1], W[1], m->normed, m->q, dim, dim, nthreads);
        oracle_cpu_engine_matvec(F[2], W[2], m->normed, m->k, kvDim, dim, nthreads);
        oracle_cpu_engine_matvec(F[3], W[3], m->normed, m->v, kvDim, dim, nthreads);
        oracle_rope(m->q, cosT, sinT, hd, m->nHeads);
        oracle_rope(m->k, cosT, sinT, hd, m->nKVHeads);
        oracle_f32_to_f16_n(m->k, m->kc[l] + pos * kvDim, kvDim);
        oracle_f32_to_f16_n(m->v, m->vc[l] + pos * kvDim, kvDim);
        oracle_decode_attention_f16kv(m->q, m->kc[l], m->vc[l], m->attn, pos + 1, dim, kvDim, m->nHeads,
                                      m->nKVHeads);
        oracle_cpu_engine_matvec(F[7], W[7], m->attn, m->proj, dim, dim, nthreads);
        oracle_add_inplace(hidden, m->proj, dim);
        oracle_rmsnorm(hidden, m->normed, (const float*)W[8], dim, m->eps);
        oracle_cpu_engine_matvec(F[9], W[9], m->normed, m->gate, m->ffnDim, dim, nthreads);
        oracle_cpu_engine_matvec(F[10], W[10], m->normed, m->up, m->ffnDim, dim, nthreads);
        oracle_silu_gate_mul(m->gate, m->up, m->mid, m->ffnDim);
        oracle_cpu_engine_matvec(F[11], W[11], m->mid, m->proj, dim, m->ffnDim, nthreads);
        oracle_add_inplace(hidden, m->proj, dim);
    }
    long fn = m->nLayers * 12;
    oracle_rmsnorm(hidden, m->normed, (const float*)m->w[fn], dim, m->eps);
    oracle_cpu_engine_matvec(m->fmt[fn + 1], m->w[fn + 1], m->normed, logits, m->vocab, dim, nthreads);
}

/* cpu.go:18-32 MatMul verbatim in semantics: C[m,n] = A[m,k] B[k,n]. */
ORACLE_API void oracle_cpu_engine_matmul(const float* a, const float* b, float* out, long m, long k, long n) {
    for (long i = 0; i < m; i++)
        for (long j = 0; j < n; j++) {
            float sum = 0.f;
            for (long l = 0; l < k; l++) sum += a[i * k + l] * b[l * n + j];
            out[i * n + j] = sum;
        }
}

ORACLE_API int oracle_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
