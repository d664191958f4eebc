// Fused single-token decode kernels for the mg_* engine (sm_100a).
//
// One "phase" kernel covers every dequant-matvec of a decode step.  A warp
// owns a tile of R weight rows at a time and streams them with 16-byte
// loads; lanes stride over the row's 16-byte chunks, so a warp instruction
// reads 512 contiguous bytes per row.  The activation vector is staged once
// per CTA in shared memory (after the fused RMSNorm / embedding prologue)
// and shared by the R rows of a tile: as 24-bit fixed point for int8 / 4-bit
// weights (integer dp4a dot products, exact per group of 16), as fp32 for
// fp16 weights.  Block scales are applied once per chunk, accumulation across
// chunks is fp32, and the R sums are reduced with warp shuffles.  The
// epilogue is fused: RoPE + fp16 KV
// append for QKV, residual add for wo/down, SiLU-gate for gate/up, argmax
// for lm_head.
//
// Weight loads do not depend on activations, so each warp issues the loads
// of its first D pipeline stages BEFORE griddepcontrol.wait: under
// programmatic dependent launch the next kernel's weights are already in
// flight while the previous kernel finishes.
#pragma once

#include "mg_common.cuh"

namespace mg {

// Device-resident cursor of the decode loop (one per sequence).
struct StepState {
    int pos;                    // position of the token being processed
    int token;                  // input token id (embedding mode)
    int step;                   // tokens generated since the cursor was set
    int out_cap;                // capacity of out_tokens
    unsigned long long best;    // packed (ordered logit, ~index) running argmax
    unsigned int done;          // CTAs of the lm_head kernel that have finished
    unsigned int pad;
};

enum : int { PRO_PLAIN = 0, PRO_RMS = 1, PRO_RMS_EMBED = 2 };
enum : int { EPI_QKV = 0, EPI_RESID = 1, EPI_SWIGLU = 2, EPI_LOGITS = 3 };

// ---------------------------------------------------------------------
// Tensor-parallel exchange fused into the phase kernels.  A rank's wo / down kernel writes its
// partial sums straight into every rank's receive buffer (peer stores over NVLink), and the
// kernel that consumes the vector (gate/up, the next layer's QKV, lm_head) adds the received
// rows while it stages its input, in rank order, so every rank forms the same bits.  There is no
// separate all-reduce launch and no fence: every element travels as one 8-byte word
// {value, exchange number}, stores of 8 aligned bytes are single accesses, and the receiver
// re-reads a word until it carries the number of the exchange it is waiting for.  Waits are
// bounded and report through XchgStatus instead of spinning for ever.
// ---------------------------------------------------------------------
constexpr int kMaxRanks = 8;

struct XchgStatus {
    int error;      // 0 = ok, 1 = a receive wait ran out
    int slot;       // exchange slot that was waited on
    int sender;     // rank whose row had not arrived
    unsigned int want, seen;
};

struct PushArgs {
    int n;                              // ranks; 0 = no exchange
    unsigned long long* dst[kMaxRanks]; // rank p's receive row for the sending rank, [rows] words
    unsigned int* count;                // sender-local: exchanges of this slot completed so far
    unsigned int* ticket;               // sender-local: CTAs of this launch that have finished
};

struct GatherArgs {
    int n;                              // ranks; 0 = read x_src
    int slot;
    const unsigned long long* rows;     // local receive buffer, [n][K] words
    const unsigned int* count;          // number of the exchange to wait for: this rank's own completed count
    XchgStatus* status;
};

__device__ __forceinline__ unsigned long long ld_relaxed_sys_u64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_relaxed_sys_u64(unsigned long long* p, unsigned long long v) {
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" :: "l"(p), "l"(v) : "memory");
}

// Control words another kernel of the same stream wrote are read from L2: with programmatic
// launch this grid's CTAs share an SM (and its L1) with CTAs of the grid that read the old value
// just before its last CTA replaced it.
__device__ __forceinline__ unsigned int ld_l2_u32(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Deadline of one kernel's receive waits: about a second of SM clock, or none at all once an
// earlier wait has run out (the step's result is void by then; the host reports it).
__device__ __forceinline__ long long xchg_deadline(const XchgStatus* st) {
    return ld_l2_u32(reinterpret_cast<const unsigned int*>(&st->error)) ? 0ll : clock64() + 2000000000ll;
}

__device__ __noinline__ void xchg_timeout(const GatherArgs& g, int sender, unsigned int want, unsigned int seen) {
    if (atomicCAS(&g.status->error, 0, 1) == 0) {
        g.status->slot = g.slot; g.status->sender = sender; g.status->want = want; g.status->seen = seen;
    }
}

// x[i] = sum over senders of their element i, in rank order.  About a second of SM clock at
// most per element; a wait that runs out records where and yields 0 for that term.
__device__ __forceinline__ float xchg_sum(const GatherArgs& g, int K, int i, unsigned int want, long long deadline) {
    float v = 0.f;
    for (int r = 0; r < g.n; r++) {
        const unsigned long long* p = g.rows + (size_t)r * K + i;
        unsigned long long w = ld_relaxed_sys_u64(p);
        while ((unsigned int)(w >> 32) != want) {
            if (clock64() > deadline) { xchg_timeout(g, r, want, (unsigned int)(w >> 32)); w = 0ull; break; }
            w = ld_relaxed_sys_u64(p);
        }
        v += __uint_as_float((unsigned int)w);
    }
    return v;
}

struct PhaseArgs {
    WeightView w[3];      // QKV: wq,wk,wv; SWIGLU: gate,up; else w[0]
    int rows[3];
    int K;
    int nitems;           // tiles of R rows
    // prologue
    int pro;
    const float* x_src;   // PLAIN: input vector; RMS: hidden state
    const float* norm_w;
    float eps;
    WeightView embed;     // RMS_EMBED: lm_head planes, row `token` is the input embedding
    int embed_fmt;
    float* h_store;       // RMS_EMBED: CTA 0 stores the embedded hidden state here
    StepState* st;
    // epilogue
    const float* bias[3];
    const float* resid_in;
    float* out;           // RESID: hidden out; SWIGLU: ffn mid; LOGITS: logits (may be NULL)
    float* q_out;
    __half* k_cache;      // [max_seq, kv_dim] of this layer
    __half* v_cache;
    const float* cos_tab;
    const float* sin_tab;
    int head_dim;
    int kv_dim;
    int* out_tokens;
    int row_base;         // LOGITS: global index of local row 0 (vocab-sharded lm_head)
    int defer_finalize;   // LOGITS: leave the cursor update to finalize_step_kernel (argmax still to be reduced over ranks)
    PushArgs push;        // RESID: send the output rows to every rank instead of (or besides) `out`
    GatherArgs gather;    // RMS prologue: the hidden state is the sum of the received rows; CTA 0 keeps it in h_store
};

__device__ __forceinline__ unsigned long long pack_best(float v, unsigned int idx) {
    unsigned int u = __float_as_uint(v);
    u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    return ((unsigned long long)u << 32) | (unsigned long long)(0xffffffffu - idx);
}

// ---------------------------------------------------------------------
// Prologue: stage the activation vector x[K] in shared memory.
// ---------------------------------------------------------------------
__device__ __forceinline__ float embed_value(const WeightView& e, int fmt, int K, int token, int i) {
    if (fmt == FMT_Q8_0) {
        const int8_t q = reinterpret_cast<const int8_t*>(e.qs)[(size_t)token * K + i];
        const float d = half_bits_to_float(e.ds[(size_t)token * (K / 32) + i / 32]);
        return d * (float)q;
    } else if (fmt == FMT_Q4_0) {
        const int b = i / 32, j = i % 32;
        const uint8_t byte = e.qs[(size_t)token * (K / 2) + b * 16 + (j & 15)];
        const int nib = j < 16 ? (byte & 0xF) : (byte >> 4);
        const float d = half_bits_to_float(e.ds[(size_t)token * (K / 32) + b]);
        return d * (float)(nib - 8);
    } else {
        return half_bits_to_float(reinterpret_cast<const unsigned short*>(e.qs)[(size_t)token * K + i]);
    }
}

__device__ __forceinline__ void stage_x(const PhaseArgs& a, float* xs, float* red) {
    const int K = a.K;
    if (a.pro == PRO_PLAIN) {
        for (int i = threadIdx.x; i < K; i += blockDim.x) xs[i] = a.x_src[i];
        __syncthreads();
        return;
    }
    float ss = 0.f;
    if (a.pro == PRO_RMS_EMBED) {
        const int token = a.st->token;
        for (int i = threadIdx.x; i < K; i += blockDim.x) {
            const float v = embed_value(a.embed, a.embed_fmt, K, token, i);
            xs[i] = v;
            if (blockIdx.x == 0) a.h_store[i] = v;
            ss = fmaf(v, v, ss);
        }
    } else if (a.gather.n > 0) {
        const unsigned int want = ld_l2_u32(a.gather.count);
        const long long deadline = xchg_deadline(a.gather.status);
        for (int i = threadIdx.x; i < K; i += blockDim.x) {
            const float v = xchg_sum(a.gather, K, i, want, deadline);
            xs[i] = v;
            if (blockIdx.x == 0) a.h_store[i] = v;
            ss = fmaf(v, v, ss);
        }
    } else {
        for (int i = threadIdx.x; i < K; i += blockDim.x) {
            const float v = a.x_src[i];
            xs[i] = v;
            ss = fmaf(v, v, ss);
        }
    }
    const float tot = block_sum(ss, red);
    const float scale = rsqrtf(tot / (float)K + a.eps);
    for (int i = threadIdx.x; i < K; i += blockDim.x) xs[i] = xs[i] * scale * a.norm_w[i];
    __syncthreads();
}

// ---------------------------------------------------------------------
// Prologue for int8 / 4-bit weights: the activation vector goes to shared
// memory as 24-bit fixed point, so that the dot products run as dp4a on the
// integer pipe (a third of the instructions of converting every weight to
// fp32) at fp32-class accuracy.  Every group of 16 activations is scaled by
// its own s = max|u| / (2^23 - 1) and rounded to t = a2*65536 + a1*256 + a0
// (a2 signed, a1 and a0 unsigned bytes).  Layout at xq: byte planes
// P0 | P1 | P2 (K bytes each), then one float2 {s, s * sum(t)} per group.
// The RMSNorm weights are folded into the quantized values; the RMS factor
// itself is returned and applied to the finished dot products.
// ---------------------------------------------------------------------
__device__ __forceinline__ float stage_xq(const PhaseArgs& a, uint8_t* xq, float* red, bool want_sum) {
    const int K = a.K;
    uint8_t* P0 = xq;
    uint8_t* P1 = xq + K;
    uint8_t* P2 = xq + 2 * (size_t)K;
    float2* sc = reinterpret_cast<float2*>(xq + 3 * (size_t)K);
    const bool gather = a.pro != PRO_PLAIN && a.pro != PRO_RMS_EMBED && a.gather.n > 0;
    const bool keep = blockIdx.x == 0 && (gather || a.pro == PRO_RMS_EMBED);
    const int token = a.pro == PRO_RMS_EMBED ? a.st->token : 0;
    unsigned int want = 0;
    long long deadline = 0;
    if (gather) {
        want = ld_l2_u32(a.gather.count);
        deadline = xchg_deadline(a.gather.status);
    }
    float ss = 0.f;
    for (int base = 0; base < K; base += 2 * blockDim.x) {
        const int i = base + 2 * threadIdx.x;     // lanes 8j..8j+7 of a warp hold one group of 16
        const bool ok = i < K;
        float v0 = 0.f, v1 = 0.f;
        if (ok) {
            if (a.pro == PRO_RMS_EMBED) {
                v0 = embed_value(a.embed, a.embed_fmt, K, token, i);
                v1 = embed_value(a.embed, a.embed_fmt, K, token, i + 1);
            } else if (gather) {
                v0 = xchg_sum(a.gather, K, i, want, deadline);
                v1 = xchg_sum(a.gather, K, i + 1, want, deadline);
            } else {
                const float2 t = *reinterpret_cast<const float2*>(a.x_src + i);
                v0 = t.x; v1 = t.y;
            }
            if (keep) *reinterpret_cast<float2*>(a.h_store + i) = make_float2(v0, v1);
        }
        ss = fmaf(v0, v0, fmaf(v1, v1, ss));
        float u0 = v0, u1 = v1;
        if (ok && a.pro != PRO_PLAIN) {
            const float2 w = *reinterpret_cast<const float2*>(a.norm_w + i);
            u0 *= w.x; u1 *= w.y;
        }
        float m = fmaxf(fabsf(u0), fabsf(u1));
        m = fmaxf(m, __shfl_xor_sync(MG_FULL_MASK, m, 1));
        m = fmaxf(m, __shfl_xor_sync(MG_FULL_MASK, m, 2));
        m = fmaxf(m, __shfl_xor_sync(MG_FULL_MASK, m, 4));
        // an approximate reciprocal is enough: t is clamped, and the value represented is t * (m / 8388607)
        const float inv = m > 0.f ? 8388607.0f * __frcp_rn(m) : 0.f;
        // the group maximum may round to 2^23, which would not fit the signed top byte: clamp
        const int t0 = max(-8388607, min(8388607, __float2int_rn(u0 * inv)));
        const int t1 = max(-8388607, min(8388607, __float2int_rn(u1 * inv)));
        int ts = 0;
        if (want_sum) {
            ts = t0 + t1;
            ts += __shfl_xor_sync(MG_FULL_MASK, ts, 1);
            ts += __shfl_xor_sync(MG_FULL_MASK, ts, 2);
            ts += __shfl_xor_sync(MG_FULL_MASK, ts, 4);
        }
        if (ok) {
            const unsigned int x = (unsigned)t0, y = (unsigned)t1;
            *reinterpret_cast<unsigned short*>(P0 + i) = (unsigned short)((x & 0xffu) | ((y & 0xffu) << 8));
            *reinterpret_cast<unsigned short*>(P1 + i) = (unsigned short)(((x >> 8) & 0xffu) | (y & 0xff00u));
            *reinterpret_cast<unsigned short*>(P2 + i) = (unsigned short)(((x >> 16) & 0xffu) | ((y >> 8) & 0xff00u));
            if ((threadIdx.x & 7) == 0) {
                const float g = m * (1.0f / 8388607.0f);
                sc[i >> 4] = make_float2(g, g * (float)ts);
            }
        }
    }
    if (a.pro == PRO_PLAIN) {
        __syncthreads();
        return 1.0f;
    }
    const float tot = block_sum(ss, red);
    return rsqrtf(tot / (float)K + a.eps);
}

// ---------------------------------------------------------------------
// Tile addressing: which rows (matrix, row) make up item `it`.
// ---------------------------------------------------------------------
template <int EPI, int R>
struct Tile {
    const uint8_t* q[R];
    const unsigned short* d[R];
    int m;       // matrix index (QKV)
    int r0;      // first row (epilogue bookkeeping)
};

template <int FMT, int EPI, int R>
__device__ __forceinline__ void tile_rows(const PhaseArgs& a, int it, Tile<EPI, R>& t) {
    const int rb = plane_row_bytes(FMT, a.K);
    const int nb = a.K / 32;
    if (EPI == EPI_QKV) {
        static_assert(EPI != EPI_QKV || R == 2, "QKV tiles are row pairs");
        const int half = a.head_dim / 2;
        const int nq = a.rows[0] / 2, nk = a.rows[1] / 2;
        int m = 0, i = it;
        if (i >= nq) { i -= nq; m = 1; }
        if (m == 1 && i >= nk) { i -= nk; m = 2; }
        int r0, r1;
        if (m < 2) {
            const int head = i / half, j = i - head * half;
            r0 = head * a.head_dim + j;
            r1 = r0 + half;
        } else {
            r0 = 2 * i;
            r1 = r0 + 1;
        }
        t.m = m;
        t.r0 = r0;
        t.q[0] = a.w[m].qs + (size_t)r0 * rb;
        t.q[R - 1] = a.w[m].qs + (size_t)r1 * rb;
        t.d[0] = a.w[m].ds + (size_t)r0 * nb;
        t.d[R - 1] = a.w[m].ds + (size_t)r1 * nb;
    } else if (EPI == EPI_SWIGLU) {
        // R/2 gate rows then the matching R/2 up rows
        constexpr int H = R / 2;
        t.m = 0;
        t.r0 = it * H;
#pragma unroll
        for (int r = 0; r < H; r++) {
            int row = it * H + r;
            if (row >= a.rows[0]) row = a.rows[0] - 1;
            t.q[r] = a.w[0].qs + (size_t)row * rb;
            t.d[r] = a.w[0].ds + (size_t)row * nb;
            t.q[H + r] = a.w[1].qs + (size_t)row * rb;
            t.d[H + r] = a.w[1].ds + (size_t)row * nb;
        }
    } else {
        t.m = 0;
        t.r0 = it * R;
#pragma unroll
        for (int r = 0; r < R; r++) {
            int row = it * R + r;
            if (row >= a.rows[0]) row = a.rows[0] - 1;   // clamped rows are computed and discarded
            t.q[r] = a.w[0].qs + (size_t)row * rb;
            t.d[r] = a.w[0].ds + (size_t)row * nb;
        }
    }
}

template <int R>
struct Stage {
    uint4 w[R];
    unsigned short d[R];
};

template <int FMT, int EPI, int R>
__device__ __forceinline__ void load_stage(const Tile<EPI, R>& t, int c, bool valid, Stage<R>& s) {
    using C = Chunk<FMT>;
    if (valid) {
#pragma unroll
        for (int r = 0; r < R; r++) s.w[r] = ld_stream16(t.q[r] + (size_t)c * 16);
        if (C::kScaled) {
#pragma unroll
            for (int r = 0; r < R; r++) s.d[r] = ld_stream_u16(t.d[r] + C::scale_index(c));
        }
    }
}

// ---------------------------------------------------------------------
// The phase kernel.  R rows per tile, D pipeline stages per warp.
// Dynamic shared memory: K floats (x) + 40 floats (reductions).
// ---------------------------------------------------------------------
template <int FMT, int EPI, int R, int D>
__global__ void __launch_bounds__(256) phase_kernel(const PhaseArgs a) {
    using C = Chunk<FMT>;
    extern __shared__ __align__(16) float smem[];
    float* xs = smem;
    float* red = smem + a.K;

    const int lane = threadIdx.x & 31;
    const int wpc = blockDim.x >> 5;
    const int gw = blockIdx.x * wpc + (threadIdx.x >> 5);   // global warp index
    const int nwarps = gridDim.x * wpc;
    const int nchunks = a.K / C::kWeights;
    const int steps = (nchunks + 31) >> 5;
    const int my_items = gw < a.nitems ? (a.nitems - gw + nwarps - 1) / nwarps : 0;
    const int T = my_items * steps;                          // flattened (item, step) iterations

    // ---- weight prefetch: first D stages, independent of the previous kernel ----
    Stage<R> st[D];
    Tile<EPI, R> ld_tile;          // tile of the stage being loaded
    int ld_k = 0, ld_step = 0;     // item ordinal / step of the next stage to load
    if (T > 0) tile_rows<FMT, EPI, R>(a, gw, ld_tile);
#pragma unroll
    for (int j = 0; j < D; j++) {
        if (j < T) {
            const int c = ld_step * 32 + lane;
            load_stage<FMT, EPI, R>(ld_tile, c, c < nchunks, st[j]);
            if (++ld_step == steps) {
                ld_step = 0;
                ++ld_k;
                if (ld_k < my_items) tile_rows<FMT, EPI, R>(a, gw + ld_k * nwarps, ld_tile);
            }
        }
    }

    pdl_launch_dependents();
    pdl_wait();

    constexpr bool kInt = (FMT != FMT_F16);          // int8 / 4-bit weights: integer dot products
    float rms = 1.0f;
    if (kInt) rms = stage_xq(a, reinterpret_cast<uint8_t*>(smem), red, FMT == FMT_Q4_0);
    else stage_x(a, xs, red);
    const uint8_t* P0 = reinterpret_cast<const uint8_t*>(smem);
    const uint8_t* P1 = P0 + a.K;
    const uint8_t* P2 = P0 + 2 * (size_t)a.K;
    const float2* gsc = reinterpret_cast<const float2*>(P0 + 3 * (size_t)a.K);

    const int pos = (EPI == EPI_QKV) ? a.st->pos : 0;
    unsigned long long best = 0ull;

    float acc[R];
#pragma unroll
    for (int r = 0; r < R; r++) acc[r] = 0.f;
    int k = 0, step = 0;           // item ordinal / step being consumed
    Tile<EPI, R> cur;
    if (T > 0) tile_rows<FMT, EPI, R>(a, gw, cur);

    for (int t0 = 0; t0 < T; t0 += D) {
#pragma unroll
        for (int j = 0; j < D; j++) {
            if (t0 + j < T) {
                // ---- consume stage j ----
                const int c = step * 32 + lane;
                if (c < nchunks) {
                    if (FMT == FMT_Q8_0) {
                        // chunk c = activation group c
                        const uint4 p0 = lds16(P0 + (size_t)c * 16), p1 = lds16(P1 + (size_t)c * 16),
                                    p2 = lds16(P2 + (size_t)c * 16);
                        const float gs = gsc[c].x;
#pragma unroll
                        for (int r = 0; r < R; r++) {
                            const float f = group_dot_s8(st[j].w[r], p0, p1, p2);
                            acc[r] = fmaf(half_bits_to_float(st[j].d[r]) * gs, f, acc[r]);
                        }
                    } else if (FMT == FMT_Q4_0) {
                        // chunk c = block c = groups 2c (low nibbles) and 2c+1 (high nibbles)
                        const int ga = 2 * c, gb = 2 * c + 1;
                        const uint4 a0 = lds16(P0 + (size_t)ga * 16), a1 = lds16(P1 + (size_t)ga * 16),
                                    a2 = lds16(P2 + (size_t)ga * 16);
                        const uint4 b0 = lds16(P0 + (size_t)gb * 16), b1 = lds16(P1 + (size_t)gb * 16),
                                    b2 = lds16(P2 + (size_t)gb * 16);
                        const float2 sa = gsc[ga], sb = gsc[gb];
                        const float off = 8.0f * (sa.y + sb.y);      // sum (nib - 8) x = sum nib x - 8 sum x
#pragma unroll
                        for (int r = 0; r < R; r++) {
                            const uint4 w = st[j].w[r];
                            const float fa = group_dot_u4(w.x & 0x0f0f0f0fu, w.y & 0x0f0f0f0fu, w.z & 0x0f0f0f0fu,
                                                          w.w & 0x0f0f0f0fu, a0, a1, a2);
                            const float fb = group_dot_u4((w.x >> 4) & 0x0f0f0f0fu, (w.y >> 4) & 0x0f0f0f0fu,
                                                          (w.z >> 4) & 0x0f0f0f0fu, (w.w >> 4) & 0x0f0f0f0fu, b0, b1, b2);
                            acc[r] = fmaf(half_bits_to_float(st[j].d[r]), fmaf(sa.x, fa, sb.x * fb) - off, acc[r]);
                        }
                    } else {
                        float4 xv[C::kWeights / 4];
                        const float4* xp = reinterpret_cast<const float4*>(xs + (size_t)c * C::kWeights);
#pragma unroll
                        for (int i = 0; i < C::kWeights / 4; i++) xv[i] = xp[i];
#pragma unroll
                        for (int r = 0; r < R; r++) acc[r] += C::dot(st[j].w[r], xv);
                    }
                }
                // ---- refill stage j with iteration t0 + j + D ----
                if (t0 + j + D < T) {
                    const int lc = ld_step * 32 + lane;
                    load_stage<FMT, EPI, R>(ld_tile, lc, lc < nchunks, st[j]);
                    if (++ld_step == steps) {
                        ld_step = 0;
                        ++ld_k;
                        if (ld_k < my_items) tile_rows<FMT, EPI, R>(a, gw + ld_k * nwarps, ld_tile);
                    }
                }
                // ---- end of tile: reduce + epilogue ----
                if (++step == steps) {
#pragma unroll
                    for (int r = 0; r < R; r++) acc[r] = warp_sum(acc[r]) * rms;
                    const int it = gw + k * nwarps;
                    if (EPI == EPI_QKV) {
                        if (lane == 0) {
                            const int half = a.head_dim / 2;
                            float v0 = acc[0], v1 = acc[R - 1];
                            const int r0 = cur.r0;
                            const int r1 = cur.m < 2 ? r0 + half : r0 + 1;
                            const float* b = a.bias[cur.m];
                            if (b) { v0 += b[r0]; v1 += b[r1]; }
                            if (cur.m < 2) {
                                const int j2 = r0 % a.head_dim;
                                const float cs = a.cos_tab[(size_t)pos * half + j2];
                                const float sn = a.sin_tab[(size_t)pos * half + j2];
                                const float o0 = v0 * cs - v1 * sn;
                                const float o1 = v0 * sn + v1 * cs;
                                v0 = o0; v1 = o1;
                            }
                            if (cur.m == 0) {
                                a.q_out[r0] = v0;
                                a.q_out[r1] = v1;
                            } else {
                                __half* dst = (cur.m == 1 ? a.k_cache : a.v_cache) + (size_t)pos * a.kv_dim;
                                dst[r0] = __float2half_rn(v0);
                                dst[r1] = __float2half_rn(v1);
                            }
                        }
                    } else if (EPI == EPI_RESID) {
                        if (lane == 0) {
                            const unsigned long long tag =
                                a.push.n > 0 ? (unsigned long long)(ld_l2_u32(a.push.count) + 1u) << 32 : 0ull;
#pragma unroll
                            for (int r = 0; r < R; r++) {
                                const int row = it * R + r;
                                if (row < a.rows[0]) {
                                    const float v = a.resid_in[row] + acc[r];
                                    if (a.out) a.out[row] = v;
                                    for (int p = 0; p < a.push.n; p++)
                                        st_relaxed_sys_u64(a.push.dst[p] + row, tag | __float_as_uint(v));
                                }
                            }
                        }
                    } else if (EPI == EPI_SWIGLU) {
                        constexpr int H = R / 2;
                        if (lane == 0) {
#pragma unroll
                            for (int r = 0; r < H; r++) {
                                const int row = it * H + r;
                                if (row < a.rows[0]) {
                                    const float g = acc[r], u = acc[H + r];
                                    a.out[row] = g * (1.0f / (1.0f + expf(-g))) * u;
                                }
                            }
                        }
                    } else {  // EPI_LOGITS
                        if (lane == 0) {
#pragma unroll
                            for (int r = 0; r < R; r++) {
                                const int row = it * R + r;
                                if (row < a.rows[0]) {
                                    if (a.out) a.out[row] = acc[r];
                                    const unsigned long long key = pack_best(acc[r], (unsigned)(row + a.row_base));
                                    if (key > best) best = key;
                                }
                            }
                        }
                    }
#pragma unroll
                    for (int r = 0; r < R; r++) acc[r] = 0.f;
                    step = 0;
                    ++k;
                    if (k < my_items) tile_rows<FMT, EPI, R>(a, gw + k * nwarps, cur);
                }
            }
        }
    }

    if (EPI == EPI_RESID) {
        if (a.push.n > 0) {
            // the exchange number advances once every CTA has read it for its own rows
            __syncthreads();
            if (threadIdx.x == 0) {
                const unsigned int ticket = atomicAdd(a.push.ticket, 1u);
                if (ticket == gridDim.x - 1) {
                    *a.push.ticket = 0u;
                    *a.push.count = ld_l2_u32(a.push.count) + 1u;
                }
            }
        }
    }

    if (EPI == EPI_LOGITS) {
        // CTA-level argmax, one atomic per CTA, last CTA advances the cursor.
        unsigned long long* sbest = reinterpret_cast<unsigned long long*>(red);   // 8-byte aligned: K is a multiple of 32
        __syncthreads();
        if (lane == 0) sbest[threadIdx.x >> 5] = best;
        __syncthreads();
        if (threadIdx.x == 0) {
            unsigned long long b = sbest[0];
            for (int w = 1; w < wpc; w++) b = sbest[w] > b ? sbest[w] : b;
            StepState* s = a.st;
            if (b) atomicMax(&s->best, b);
            __threadfence();
            const unsigned int ticket = atomicAdd(&s->done, 1u);
            if (ticket == gridDim.x - 1 && a.defer_finalize) {
                s->done = 0u;
            } else if (ticket == gridDim.x - 1) {
                __threadfence();
                const unsigned long long key = atomicMax(&s->best, 0ull);
                const int tok = (int)(0xffffffffu - (unsigned int)(key & 0xffffffffull));
                if (a.out_tokens && s->step < s->out_cap) a.out_tokens[s->step] = tok;
                s->token = tok;
                s->step += 1;
                s->pos += 1;
                s->best = 0ull;
                s->done = 0u;
            }
        }
    }
}

// Sum of the received rows into a plain vector (the hidden state a layer range hands back to the
// host when no kernel of the same step consumes it).
__global__ void __launch_bounds__(256) xchg_reduce_kernel(const GatherArgs g, float* out, int K) {
    pdl_wait();
    const unsigned int want = ld_l2_u32(g.count);
    const long long deadline = xchg_deadline(g.status);
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < K; i += gridDim.x * blockDim.x)
        out[i] = xchg_sum(g, K, i, want, deadline);
}

// Cursor update after the running argmax has been combined over tensor-parallel ranks.
__global__ void finalize_step_kernel(StepState* s, int* out_tokens) {
    pdl_wait();
    const unsigned long long key = s->best;
    const int tok = (int)(0xffffffffu - (unsigned int)(key & 0xffffffffull));
    if (out_tokens && s->step < s->out_cap) out_tokens[s->step] = tok;
    s->token = tok;
    s->step += 1;
    s->pos += 1;
    s->best = 0ull;
}

// ---------------------------------------------------------------------
// GQA decode attention over the fp16 KV cache of one layer.
// One CTA per query head; scores for every cached position are held in
// shared memory (max_seq floats).  Deterministic reductions.
//   q      : fp32 [dim]          (already rotated)
//   kc, vc : fp16 [max_seq, kv_dim]
//   out    : fp32 [dim]
// ---------------------------------------------------------------------
template <int HD>
__global__ void __launch_bounds__(256) attn_decode_kernel(const float* __restrict__ q,
                                                          const __half* __restrict__ kc,
                                                          const __half* __restrict__ vc,
                                                          float* __restrict__ out, const StepState* st,
                                                          int kv_dim, int n_heads, int n_kv_heads) {
    extern __shared__ __align__(16) float smem[];
    float* qs = smem;                  // HD
    float* red = smem + HD;            // 40
    float* part = red + 40;            // 512: one partial per thread pair component (G groups x HD dims)
    float* sc = part + 512;            // cache_len scores

    pdl_launch_dependents();
    pdl_wait();

    const int head = blockIdx.x;
    const int kvh = head / (n_heads / n_kv_heads);
    const int len = st->pos + 1;
    const float scale = rsqrtf((float)HD);
    const int tid = threadIdx.x;

    if (tid < HD) qs[tid] = q[head * HD + tid];
    __syncthreads();

    // scores
    float mx = -INFINITY;
    for (int t = tid; t < len; t += blockDim.x) {
        const uint4* kp = reinterpret_cast<const uint4*>(kc + (size_t)t * kv_dim + kvh * HD);
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < HD / 8; i++) {
            const uint4 kk = kp[i];
            const __half2* h = reinterpret_cast<const __half2*>(&kk);
            const float4 qa = reinterpret_cast<const float4*>(qs)[2 * i];
            const float4 qb = reinterpret_cast<const float4*>(qs)[2 * i + 1];
            const float2 k0 = __half22float2(h[0]), k1 = __half22float2(h[1]);
            const float2 k2 = __half22float2(h[2]), k3 = __half22float2(h[3]);
            dot = fmaf(qa.x, k0.x, dot);
            dot = fmaf(qa.y, k0.y, dot);
            dot = fmaf(qa.z, k1.x, dot);
            dot = fmaf(qa.w, k1.y, dot);
            dot = fmaf(qb.x, k2.x, dot);
            dot = fmaf(qb.y, k2.y, dot);
            dot = fmaf(qb.z, k3.x, dot);
            dot = fmaf(qb.w, k3.y, dot);
        }
        dot *= scale;
        sc[t] = dot;
        mx = fmaxf(mx, dot);
    }
    // block max
    mx = warp_max(mx);
    {
        const int lane = tid & 31, wid = tid >> 5, nw = blockDim.x >> 5;
        if (lane == 0) red[wid] = mx;
        __syncthreads();
        float m = lane < nw ? red[lane] : -INFINITY;
        m = warp_max(m);
        mx = m;
        __syncthreads();
    }
    float sum = 0.f;
    for (int t = tid; t < len; t += blockDim.x) {
        const float p = expf(sc[t] - mx);
        sc[t] = p;
        sum += p;
    }
    sum = block_sum(sum, red);   // includes the barrier that publishes sc[]
    const float inv = 1.0f / sum;

    // weighted sum of V: thread = (group g, dim pair dp)
    constexpr int DP = HD / 2;                 // dim pairs
    const int G = blockDim.x / DP;             // position groups; G * HD = 2 * blockDim = 512
    const int g = tid / DP, dp = tid % DP;
    float2 o = make_float2(0.f, 0.f);
    if (g < G) {
        for (int t = g; t < len; t += G) {
            const __half2 v = *reinterpret_cast<const __half2*>(vc + (size_t)t * kv_dim + kvh * HD + 2 * dp);
            const float2 vf = __half22float2(v);
            const float p = sc[t];
            o.x = fmaf(p, vf.x, o.x);
            o.y = fmaf(p, vf.y, o.y);
        }
        part[g * HD + 2 * dp] = o.x;
        part[g * HD + 2 * dp + 1] = o.y;
    }
    __syncthreads();
    if (tid < HD) {
        float s = 0.f;
        for (int gg = 0; gg < G; gg++) s += part[gg * HD + tid];
        out[head * HD + tid] = s * inv;
    }
}

}  // namespace mg
