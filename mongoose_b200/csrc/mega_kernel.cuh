// Persistent decode kernel: every layer of a token (and, in the greedy loop,
// many tokens) in ONE cooperative launch, one CTA per SM.
//
// Why: at 0.5 B parameters a layer is ~16 MB of Q8_0 weights, about 2.4 us of
// HBM time, split over five dependent matvec phases.  A kernel boundary costs
// more than a phase.  Here the CTAs stay resident and hand activations to each
// other through L2:
//
//  * Weight tape.  At build time every CTA's share of every matrix is copied
//    into one contiguous per-CTA byte stream in exactly the order the CTA
//    consumes it: tiles of 32 >> s rows in which 1 << s adjacent lanes share a
//    row, stored as [iteration][lane] 16-byte chunks followed by the fp16 block
//    scales in the same order, so a warp reads 512 contiguous, conflict-free
//    bytes per iteration.  A dedicated producer warp walks the tape with bulk
//    asynchronous copies (cp.async.bulk, mbarrier completion) into a ring of
//    shared-memory slots, running up to a ring ahead of the consumers - weights
//    never depend on activations, so HBM streaming is off the dependency chain.
//  * Tagged exchange.  A phase's output vector is written to global memory as
//    8-byte {fp32 value, 32-bit epoch} words.  Consumers poll the words they
//    need until the epoch is the one they expect: data and flag arrive in one
//    atomic 8-byte access, so no fence, no counter and no reset is needed, and
//    a stale buffer can never be mistaken for fresh data.
//  * 15 consumer warps per CTA.  The input vector is staged in shared memory
//    (for int8/4-bit weights as 24-bit fixed point in three byte planes, so
//    the dot products are integer dp4a); every lane accumulates its share of
//    one row, lanes of a row combine with log2(lanes per row) shuffles, and all
//    rows of a tile run their fused epilogue in parallel lanes.  The lanes-per-
//    row split is chosen per phase on the host so that even a phase with eight
//    rows per CTA spreads over several warps.
//
// Every wait (mbarrier, exchange poll) is bounded by a deadline in SM clocks (about 1 s);
// on expiry the kernel records an error code, stops waiting everywhere and
// runs to completion on whatever data it has, so a logic error cannot hang
// the GPU.  The host checks the status word after each launch.
#pragma once

#include "decode_kernels.cuh"

namespace mg {

constexpr int MK_NW = 15;                       // consumer warps
constexpr int MK_CONSUMERS = MK_NW * 32;        // 480
constexpr int MK_THREADS = MK_CONSUMERS + 32;   // + producer warp = 512 threads, 128 registers each
constexpr int MK_SLOT = 16384;                  // default ring slot bytes (MegaArgs::slot_bytes holds the size in use)
constexpr int MK_MAX_SLOTS = 14;
constexpr int MK_PART_FLOATS = 2048;
constexpr int MK_EPOCHS_PER_LAYER = 8;
constexpr long long MK_WAIT_CYCLES = 2000000000ll;         // per wait: about one second of SM clocks

enum : int { PH_QKV = 0, PH_WO = 1, PH_GU = 2, PH_DOWN = 3, PH_HEAD = 4 };
enum : int { MK_OK = 0, MK_ERR_POLL = 1, MK_ERR_FULL = 2, MK_ERR_EMPTY = 3, MK_ERR_RANGE = 4 };

struct MegaStatus {
    int error;          // first error code (0 = none)
    int where;          // phase / tag that timed out
    int cta;
    int pad;
};

struct Tagged {         // one exchanged activation
    float v;
    unsigned int tag;
};

// How a phase's rows are laid over lanes (the same on every CTA).  A warp works on a TILE of
// 32 >> lpr_shift rows; a row is shared by 1 << lpr_shift adjacent lanes, lane `part` of a row taking
// the 16-byte chunks part, part + lpr, part + 2 lpr, ...  The tape stores a tile exactly in the order
// the lanes read it: ni iterations x 32 lanes x 16 bytes, then ni x 32 fp16 block scales.
struct PhaseGeom {
    int lpr_shift;      // log2(lanes per row)
    int ni;             // chunks per lane = ceil(chunks per row / lanes per row)
    int tile_bytes;
    int tpe;            // tiles per ring entry
    int nchunks;        // 16-byte chunks per weight row
};

struct MegaArgs {
    int dim, kv_dim, head_dim, n_heads, n_kv_heads, ffn_dim, vocab, n_layers, max_seq;
    int layer_fmt, head_fmt;
    float eps;
    int ls, le;             // layer range
    int head;               // HEAD_NONE / HEAD_ARGMAX / HEAD_LOGITS (0/1/2)
    int embed;              // 1: hidden state from the embedding row of st->token, 0: from h_in
    int n_steps;            // tokens per launch (greedy feedback between them)
    unsigned int epoch;     // first epoch of this launch
    int hd_shift;           // log2(head_dim)
    int nslot;
    int slot_bytes;       // ring slot size: MK_SLOT, or larger when one tile of the widest matrix needs it
    int prefetch_bytes;   // how far ahead of the ring the producer asks L2 for this CTA's tape (0 = off)
    int xs_floats;          // size of the staged-activation buffer (multiple of 4)
    PhaseGeom geom[5];
    int sc_floats;          // attention score buffer: max_seq rounded up to a multiple of 4
    // weight tape
    const uint8_t* tape;
    const unsigned long long* tape_off;   // [grid][n_layers*4 + 2]
    unsigned long long tape_bytes;
    // small vectors, flat so that no pointer has to be fetched on the dependency chain:
    // norms[layer][2][dim] (attention norm, ffn norm); qkv_bias[layer][dim + 2*kv_dim] or NULL
    const float* norms;
    const float* qkv_bias;
    const float* final_norm;
    WeightView embed_w;
    const float* cos_tab;
    const float* sin_tab;
    __half* kc;             // [layers][max_seq][kv_dim]
    __half* vc;
    // exchange buffers
    Tagged *xh, *xhm, *xq, *xkv, *xattn, *xmid, *xtok;
    // Tensor parallelism (tp_n > 1): dim is the model width, every other size above is this rank's
    // share.  xh / xhm are then receive buffers [tp_n][dim] that every rank writes its partial sums
    // into (peer stores), xbest [tp_n][2] receives the ranks' argmax keys.
    int q_dim;              // rows of Q on this rank (= dim on one GPU)
    int tp_n, tp_rank;
    int vocab_base;         // global index of this rank's first lm_head row
    int vocab_total;        // rows of the embedding table
    Tagged* xh_peer[8];     // rank p's xh / xhm / xbest as mapped here (own entry = the local buffer)
    Tagged* xhm_peer[8];
    Tagged* xbest_peer[8];
    Tagged* xbest;
    // io
    const float* h_in;
    float* h_out;
    float* logits;
    StepState* st;
    int* out_tokens;
    MegaStatus* status;
    long long* trace;       // optional [grid][n_layers*10 + 2] SM-clock stamps of CTA thread 0 (first step)
};

// ---------------------------------------------------------------------
// Row partition shared by the host tape builder and the kernel.
// ---------------------------------------------------------------------
struct PhaseShape {
    int items;      // work items over the whole grid
    int rpi;        // rows per item (2 for RoPE pairs and gate/up pairs)
    int K;          // input dim
    int fmt;
};

__host__ __device__ inline PhaseShape phase_shape_of(int p, int dim, int q_dim, int kv_dim, int ffn, int vocab,
                                                     int layer_fmt, int head_fmt) {
    PhaseShape s{};
    switch (p) {
        case PH_QKV: s.items = (q_dim + 2 * kv_dim) / 2; s.rpi = 2; s.K = dim; s.fmt = layer_fmt; break;
        case PH_WO: s.items = dim; s.rpi = 1; s.K = q_dim; s.fmt = layer_fmt; break;
        case PH_GU: s.items = ffn; s.rpi = 2; s.K = dim; s.fmt = layer_fmt; break;
        case PH_DOWN: s.items = dim; s.rpi = 1; s.K = ffn; s.fmt = layer_fmt; break;
        default: s.items = vocab; s.rpi = 1; s.K = dim; s.fmt = head_fmt; break;
    }
    return s;
}

__host__ __device__ inline int item_begin(int items, int cta, int grid) {
    return (int)(((long long)cta * items) / grid);
}
__host__ __device__ inline int row_q_bytes(int fmt, int K) { return plane_row_bytes(fmt, K); }
__host__ __device__ inline int row_d_bytes(int fmt, int K) { return fmt == FMT_F16 ? 0 : (K / 32) * 2; }
__host__ __device__ inline int chunks_per_row(int fmt, int K) {
    return fmt == FMT_Q8_0 ? K / 16 : fmt == FMT_Q4_0 ? K / 32 : K / 8;
}
__host__ __device__ inline int tile_bytes_of(int fmt, int ni) { return ni * 32 * (fmt == FMT_F16 ? 16 : 18); }
// Lanes per row for a phase whose busiest CTA has max_rows rows: the choice that minimises the
// chunks a warp walks through (tiles per warp x chunks per lane) among those whose tile fits a ring
// slot; row pairs must stay inside a tile, so pair phases use at most 16 lanes per row.
__host__ inline PhaseGeom choose_geom(int fmt, int K, int max_rows, bool pairs, int n_warps, int slot_bytes,
                                      int force_shift = -1) {
    PhaseGeom best{};
    long long best_cost = -1;
    const int nch = chunks_per_row(fmt, K);
    for (int sh = 0; sh <= (pairs ? 4 : 5); sh++) {
        if (force_shift >= 0 && sh != force_shift) continue;
        const int lpr = 1 << sh, rpt = 32 >> sh;
        const int ni = (nch + lpr - 1) / lpr;
        const int tb = tile_bytes_of(fmt, ni);
        if (tb > slot_bytes) continue;
        const int tiles = (max_rows + rpt - 1) / rpt;
        const long long cost = (long long)((tiles + n_warps - 1) / n_warps) * (ni + 6);   // + per-tile overhead
        if (best_cost < 0 || cost < best_cost) {
            best_cost = cost;
            best.lpr_shift = sh; best.ni = ni; best.tile_bytes = tb; best.tpe = slot_bytes / tb; best.nchunks = nch;
        }
    }
    if (best_cost < 0) best.ni = 0;     // no feasible layout
    return best;
}

// QKV pair -> matrix (0 q, 1 k, 2 v) and its two rows.
__host__ __device__ inline void qkv_pair(int item, int dim, int kv_dim, int head_dim, int* m, int* r0, int* r1) {
    const int half = head_dim / 2;
    const int nq = dim / 2, nk = kv_dim / 2;
    int mm = 0, i = item;
    if (i >= nq) { i -= nq; mm = 1; }
    if (mm == 1 && i >= nk) { i -= nk; mm = 2; }
    if (mm < 2) {
        const int head = i / half, j = i - head * half;
        *r0 = head * head_dim + j;
        *r1 = *r0 + half;
    } else {
        *r0 = 2 * i;
        *r1 = 2 * i + 1;
    }
    *m = mm;
}

// ---------------------------------------------------------------------
// Low-level primitives
// ---------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
// Deadlines are counted in SM clocks: reading the clock register costs a few cycles, whereas the
// global nanosecond timer is a slow off-SM read that would sit on every unsuccessful first poll.
__device__ __forceinline__ long long global_ns() { return clock64(); }
__device__ __forceinline__ void mbar_init(unsigned long long* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(unsigned long long* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// global -> this CTA's shared memory, completion counted on an mbarrier
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, unsigned long long* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
// Hint: bring [src, src + bytes) into L2 (16-byte granularity; no completion to wait for).
__device__ __forceinline__ void bulk_prefetch_l2(const void* src, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(MK_CONSUMERS) : "memory"); }

// Exchange words are 64-bit {value (low), tag (high)}: each is read and written as ONE 8-byte
// relaxed gpu-scope access, so value and tag can never be observed torn.
__device__ __forceinline__ uint4 ld_poll16(const void* p) {
    unsigned long long a, b;
    asm volatile("ld.relaxed.gpu.global.v2.u64 {%0,%1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
    return make_uint4((unsigned)a, (unsigned)(a >> 32), (unsigned)b, (unsigned)(b >> 32));
}
__device__ __forceinline__ uint2 ld_poll8(const void* p) {
    unsigned long long a;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(a) : "l"(p) : "memory");
    return make_uint2((unsigned)a, (unsigned)(a >> 32));
}
// System-scope variants for words that another GPU writes or reads (tensor parallelism).
__device__ __forceinline__ uint4 ld_poll16_sys(const void* p) {
    unsigned long long a, b;
    asm volatile("ld.relaxed.sys.global.v2.u64 {%0,%1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
    return make_uint4((unsigned)a, (unsigned)(a >> 32), (unsigned)b, (unsigned)(b >> 32));
}
__device__ __forceinline__ void st_tagged_sys(Tagged* p, float v, unsigned int tag) {
    const unsigned long long w = (unsigned long long)__float_as_uint(v) | ((unsigned long long)tag << 32);
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ void st_tagged(Tagged* p, float v, unsigned int tag) {
    const unsigned long long w = (unsigned long long)__float_as_uint(v) | ((unsigned long long)tag << 32);
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}

// ---------------------------------------------------------------------
// Per-CTA shared memory.  Layout (bytes): ring | xs | hs | part | red | rope | sc | barriers | flag.
// Pointers are recomputed from the shared symbol where they are used, so the compiler keeps
// them as 32-bit shared-space addresses instead of 64-bit generic pointers held in registers.
// ---------------------------------------------------------------------
extern __shared__ __align__(128) uint8_t mk_smem[];
constexpr int MK_ROPE_FLOATS = 256;

struct MkCtx {
    const MegaArgs& a;
    unsigned int entry;           // running ring-entry counter of this thread's role (diagnostics)
    int slot;                     // ring slot of the next entry
    unsigned int par;             // phase parity of that slot
    unsigned long long pf;        // producer: tape offset up to which L2 prefetches have been issued
    __device__ __forceinline__ MkCtx(const MegaArgs& args) : a(args), entry(0), slot(0), par(0), pf(0) {}
    __device__ __forceinline__ void advance() {
        entry++;
        if (++slot == a.nslot) { slot = 0; par ^= 1u; }
    }
    __device__ __forceinline__ uint8_t* ring() const { return mk_smem; }
    __device__ __forceinline__ float* xs() const { return reinterpret_cast<float*>(mk_smem + (size_t)a.nslot * a.slot_bytes); }
    __device__ __forceinline__ float* hs() const { return xs() + a.xs_floats; }
    __device__ __forceinline__ float* part() const { return hs() + a.dim; }
    __device__ __forceinline__ float* red() const { return part() + MK_PART_FLOATS; }
    __device__ __forceinline__ float* rope() const { return red() + 64; }
    __device__ __forceinline__ float* sc() const { return rope() + MK_ROPE_FLOATS; }
    __device__ __forceinline__ unsigned long long* full() const {
        return reinterpret_cast<unsigned long long*>(sc() + a.sc_floats);
    }
    __device__ __forceinline__ unsigned long long* empty() const { return full() + MK_MAX_SLOTS; }
    __device__ __forceinline__ volatile int* abort_flag() const {
        return reinterpret_cast<volatile int*>(empty() + MK_MAX_SLOTS);
    }
    // per phase p: [p] first work item on this CTA, [8+p] item count, [16+p] rows per ring entry,
    // [24+p] consumer warps per K segment
    __device__ __forceinline__ int* phase_tab() const { return const_cast<int*>(reinterpret_cast<volatile int*>(abort_flag())) + 4; }
    __device__ __forceinline__ MegaStatus* status() const { return a.status; }
    __device__ __forceinline__ int nslot() const { return a.nslot; }
};

__device__ __noinline__ void mk_fail_impl(volatile int* abort_flag, MegaStatus* status, int code, int where) {
    *abort_flag = 1;
    if (atomicCAS(&status->error, 0, code) == 0) {
        status->where = where;
        status->cta = blockIdx.x;
    }
}
__device__ __forceinline__ void mk_fail(MkCtx& c, int code, int where) {
    mk_fail_impl(c.abort_flag(), c.status(), code, where);
}

#define MK_TRACE_EVENTS(L) ((L) * 10 + 2)
__device__ __forceinline__ void mk_trace(const MegaArgs& a, int step, int ev) {
    if (a.trace && step == 0 && threadIdx.x == 0)
        a.trace[(size_t)blockIdx.x * MK_TRACE_EVENTS(a.n_layers) + ev] = clock64();
}

// Bounded wait on an mbarrier phase.
__device__ __forceinline__ void mk_wait_bar(MkCtx& c, unsigned long long* bar, uint32_t parity, int code) {
    if (*c.abort_flag()) return;
    if (mbar_try(bar, parity)) return;
    const long long t0 = global_ns();
    for (unsigned int it = 1;; ++it) {
        if (mbar_try(bar, parity)) return;
        if ((it & 63u) == 0u) {
            if (*c.abort_flag()) return;
            if (*(volatile int*)&c.status()->error) { *c.abort_flag() = 1; return; }
            if (global_ns() - t0 > MK_WAIT_CYCLES) { mk_fail(c, code, (int)c.entry); return; }
        }
    }
}

// Poll two adjacent tagged values (16-byte aligned pair).
__device__ __forceinline__ void mk_poll2(MkCtx& c, const Tagged* p, unsigned int tag, float& v0, float& v1) {
    uint4 r = ld_poll16(p);
    if (r.y != tag || r.w != tag) {
        if (!*c.abort_flag()) {
            const long long t0 = global_ns();
            for (unsigned int it = 1;; ++it) {
                r = ld_poll16(p);
                if (r.y == tag && r.w == tag) break;
                if ((it & 63u) == 0u) {
                    if (*c.abort_flag()) break;
                    if (*(volatile int*)&c.status()->error) { *c.abort_flag() = 1; break; }
                    if (global_ns() - t0 > MK_WAIT_CYCLES) { mk_fail(c, MK_ERR_POLL, (int)tag); break; }
                }
            }
        }
    }
    v0 = __uint_as_float(r.x);
    v1 = __uint_as_float(r.z);
}
__device__ __forceinline__ float mk_poll1(MkCtx& c, const Tagged* p, unsigned int tag) {
    uint2 r = ld_poll8(p);
    if (r.y != tag) {
        if (!*c.abort_flag()) {
            const long long t0 = global_ns();
            for (unsigned int it = 1;; ++it) {
                r = ld_poll8(p);
                if (r.y == tag) break;
                if ((it & 63u) == 0u) {
                    if (*c.abort_flag()) break;
                    if (*(volatile int*)&c.status()->error) { *c.abort_flag() = 1; break; }
                    if (global_ns() - t0 > MK_WAIT_CYCLES) { mk_fail(c, MK_ERR_POLL, (int)tag); break; }
                }
            }
        }
    }
    return __uint_as_float(r.x);
}

// Two adjacent exchange words that another GPU may have written, once both carry `tag` (raw
// words: x, z = values, y, w = tags).  Bounded like every wait in this kernel.
__device__ __forceinline__ uint4 mk_poll16_sys(MkCtx& c, const Tagged* q, unsigned int tag) {
    uint4 w = ld_poll16_sys(q);
    if (w.y != tag || w.w != tag) {
        if (!*c.abort_flag()) {
            const long long t0 = global_ns();
            for (unsigned int it = 1;; ++it) {
                w = ld_poll16_sys(q);
                if (w.y == tag && w.w == tag) break;
                if ((it & 63u) == 0u) {
                    if (*c.abort_flag()) break;
                    if (*(volatile int*)&c.status()->error) { *c.abort_flag() = 1; break; }
                    if (global_ns() - t0 > MK_WAIT_CYCLES) { mk_fail(c, MK_ERR_POLL, (int)tag); break; }
                }
            }
        }
    }
    return w;
}

// Two adjacent values of a vector that arrives as one row per rank: the rows are added in rank
// order (every rank forms the same bits).  p points into row 0, rows are `stride` words apart.
__device__ __forceinline__ void mk_poll2_sum(MkCtx& c, const Tagged* p, int stride, int n, unsigned int tag, float& v0,
                                             float& v1) {
    const uint4 first = mk_poll16_sys(c, p, tag);
    v0 = __uint_as_float(first.x);
    v1 = __uint_as_float(first.z);
    for (int r = 1; r < n; r++) {
        const uint4 w = mk_poll16_sys(c, p + (size_t)r * stride, tag);
        v0 += __uint_as_float(w.x);
        v1 += __uint_as_float(w.z);
    }
}

// ---------------------------------------------------------------------
// Fixed-point activations.  For int8 / 4-bit weights the dot products run on
// the integer pipe (dp4a) without giving up fp32-class accuracy: every group
// of 16 consecutive activations is scaled by its own s = max|x| / (2^23 - 1)
// and rounded to a 24-bit integer t = a2*65536 + a1*256 + a0 (a2 signed byte,
// a1 and a0 unsigned bytes).  sum q_i x_i over the group is then
// s * (65536 * dp(q, a2) + 256 * dp(q, a1) + dp(q, a0)) with exact integer
// dot products; the representation error is at most 2^-24 of the group's
// largest element per term.  Shared-memory layout for a vector of K values
// (at xs): byte planes P0 | P1 | P2 (K bytes each, element order), then one
// float2 {s, s * sum(t)} per group of 16.
// ---------------------------------------------------------------------
__device__ __forceinline__ uint8_t* xq_plane(MkCtx& c, int K, int k) {
    return reinterpret_cast<uint8_t*>(c.xs()) + (size_t)k * K;
}
__device__ __forceinline__ float2* xq_scales(MkCtx& c, int K) {
    return reinterpret_cast<float2*>(reinterpret_cast<uint8_t*>(c.xs()) + (size_t)3 * K);
}

// All 32 lanes call; lanes 8j..8j+7 hold the 16 values of one group (u0,u1 each).
// `want_sum`: the group's sum(t) is only needed by 4-bit weights (their -8 offset).
__device__ __forceinline__ void xq_store_pair(MkCtx& c, int K, int i, bool ok, float u0, float u1, bool want_sum) {
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
        const unsigned int a = (unsigned)t0, b = (unsigned)t1;
        *reinterpret_cast<unsigned short*>(xq_plane(c, K, 0) + i) = (unsigned short)((a & 0xffu) | ((b & 0xffu) << 8));
        *reinterpret_cast<unsigned short*>(xq_plane(c, K, 1) + i) = (unsigned short)(((a >> 8) & 0xffu) | (b & 0xff00u));
        *reinterpret_cast<unsigned short*>(xq_plane(c, K, 2) + i) = (unsigned short)(((a >> 16) & 0xffu) | ((b >> 8) & 0xff00u));
        if ((threadIdx.x & 7) == 0) {
            const float sc = m * (1.0f / 8388607.0f);
            xq_scales(c, K)[i >> 4] = make_float2(sc, sc * (float)ts);
        }
    }
}

// Poll n tagged values into shared memory dst[0..n) (n even).  All consumer threads call.
__device__ __forceinline__ void mk_gather(MkCtx& c, const Tagged* src, unsigned int tag, float* dst, int n) {
    for (int i = 2 * threadIdx.x; i < n; i += 2 * MK_CONSUMERS) {
        float a, b;
        mk_poll2(c, src + i, tag, a, b);
        dst[i] = a;
        dst[i + 1] = b;
    }
}
// Re-poll one pair until both tags match (bounded); r holds the first attempt.
__device__ __forceinline__ void mk_poll2_finish(MkCtx& c, const Tagged* p, unsigned int tag, uint4& r) {
    if (r.y == tag && r.w == tag) return;
    if (*c.abort_flag()) return;
    const long long t0 = global_ns();
    for (unsigned int it = 1;; ++it) {
        r = ld_poll16(p);
        if (r.y == tag && r.w == tag) return;
        if ((it & 63u) == 0u) {
            if (*c.abort_flag()) return;
            if (*(volatile int*)&c.status()->error) { *c.abort_flag() = 1; return; }
            if (global_ns() - t0 > MK_WAIT_CYCLES) { mk_fail(c, MK_ERR_POLL, (int)tag); return; }
        }
    }
}

// Same, but the values land in xs as fixed-point planes (n a multiple of 32).  A thread's loads
// for up to four strides are issued together so that their L2 latencies overlap; only then are the
// tags checked (and stale words polled again).
__device__ __forceinline__ void mk_gather_q(MkCtx& c, const Tagged* src, unsigned int tag, int n, bool want_sum) {
    constexpr int STRIDE = 2 * MK_CONSUMERS;
    for (int i0 = 0; i0 < n; i0 += 4 * STRIDE) {
        const int ia = i0 + 2 * (int)threadIdx.x, ib = ia + STRIDE, ic = ib + STRIDE, id = ic + STRIDE;
        const uint4 z = make_uint4(0u, tag, 0u, tag);
        uint4 ra = z, rb = z, rc = z, rd = z;
        if (ia < n) ra = ld_poll16(src + ia);
        if (ib < n) rb = ld_poll16(src + ib);
        if (ic < n) rc = ld_poll16(src + ic);
        if (id < n) rd = ld_poll16(src + id);
        if (ia < n) mk_poll2_finish(c, src + ia, tag, ra);
        if (ib < n) mk_poll2_finish(c, src + ib, tag, rb);
        if (ic < n) mk_poll2_finish(c, src + ic, tag, rc);
        if (id < n) mk_poll2_finish(c, src + id, tag, rd);
        xq_store_pair(c, n, ia, ia < n, __uint_as_float(ra.x), __uint_as_float(ra.z), want_sum);
        if (i0 + STRIDE < n) xq_store_pair(c, n, ib, ib < n, __uint_as_float(rb.x), __uint_as_float(rb.z), want_sum);
        if (i0 + 2 * STRIDE < n) xq_store_pair(c, n, ic, ic < n, __uint_as_float(rc.x), __uint_as_float(rc.z), want_sum);
        if (i0 + 3 * STRIDE < n) xq_store_pair(c, n, id, id < n, __uint_as_float(rd.x), __uint_as_float(rd.z), want_sum);
    }
}

// Sum over the consumer threads (deterministic order); includes one consumer barrier.
__device__ __forceinline__ float mk_block_sum(MkCtx& c, float v) {
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    if (lane == 0) c.red()[w] = v;
    consumer_sync();
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < MK_NW; i++) t += c.red()[i];
    return t;
}

__device__ __forceinline__ float dot8_f16(uint4 w, float4 xa, float4 xb) {
    const __half2* h = reinterpret_cast<const __half2*>(&w);
    const float2 a0 = __half22float2(h[0]), a1 = __half22float2(h[1]);
    const float2 a2 = __half22float2(h[2]), a3 = __half22float2(h[3]);
    float a = a0.x * xa.x;
    a = fmaf(a0.y, xa.y, a); a = fmaf(a1.x, xa.z, a); a = fmaf(a1.y, xa.w, a);
    a = fmaf(a2.x, xb.x, a); a = fmaf(a2.y, xb.y, a); a = fmaf(a3.x, xb.z, a); a = fmaf(a3.y, xb.w, a);
    return a;
}

// ---------------------------------------------------------------------
// Producer warp: stream this CTA's tape through the ring.
// ---------------------------------------------------------------------
__device__ __forceinline__ void mk_produce_phase(MkCtx& c, const MegaArgs& a, const uint8_t* src, int p, int nrows) {
    const PhaseGeom g = a.geom[p];
    const int rpt = 32 >> g.lpr_shift;
    const int ntiles = (nrows + rpt - 1) >> (5 - g.lpr_shift);
    for (int t = 0; t < ntiles; t += g.tpe) {
        const uint32_t bytes = (uint32_t)(min(g.tpe, ntiles - t) * g.tile_bytes);
        const int slot = c.slot;
        const uint32_t par = c.par;
        mk_wait_bar(c, &c.empty()[slot], par ^ 1u, MK_ERR_EMPTY);
        if ((unsigned long long)(src - a.tape) + bytes > a.tape_bytes || bytes == 0 || bytes > (uint32_t)a.slot_bytes || (bytes & 15u) ||
            ((unsigned long long)(src - a.tape) & 15ull)) {
            mk_fail(c, MK_ERR_RANGE, 300000 + p);
            return;
        }
        mbar_expect_tx(&c.full()[slot], bytes);
        bulk_g2s(c.ring() + (size_t)slot * a.slot_bytes, src, bytes, &c.full()[slot]);
        src += bytes;
        c.advance();
        if (a.prefetch_bytes > 0) {
            // The ring alone keeps nslot * slot_bytes in flight per SM, too little to saturate HBM when
            // the activations crowd the ring (wide models).  The tape of a CTA is one contiguous run
            // through all phases and layers, so the producer also asks L2 for the bytes a fixed distance
            // ahead; the ring then fills from L2 and DRAM runs ahead of it.
            const unsigned long long pos = (unsigned long long)(src - a.tape);
            unsigned long long want = pos + (unsigned long long)a.prefetch_bytes;
            if (want > a.tape_bytes) want = a.tape_bytes;
            if (c.pf < pos) c.pf = pos;
            while (c.pf + 16 <= want) {
                unsigned long long n = want - c.pf;
                if (n > 8192ull) n = 8192ull;
                n &= ~15ull;
                bulk_prefetch_l2(a.tape + c.pf, (uint32_t)n);
                c.pf += n;
            }
        }
    }
}

__device__ __forceinline__ void mk_producer(MkCtx& c, const MegaArgs& a) {
    if ((threadIdx.x & 31) != 0) return;
    const unsigned long long* off = a.tape_off + (size_t)blockIdx.x * (a.n_layers * 4 + 2);
    for (int step = 0; step < a.n_steps; step++) {
        for (int l = a.ls; l < a.le; l++)
            for (int p = 0; p < 4; p++) {
                const PhaseShape s = phase_shape_of(p, a.dim, a.q_dim, a.kv_dim, a.ffn_dim, a.vocab, a.layer_fmt, a.head_fmt);
                const int nrows = c.phase_tab()[8 + p] * s.rpi;
                mk_produce_phase(c, a, a.tape + off[l * 4 + p], p, nrows);
            }
        if (a.le >= a.n_layers && a.head) {
            const PhaseShape s = phase_shape_of(PH_HEAD, a.dim, a.q_dim, a.kv_dim, a.ffn_dim, a.vocab, a.layer_fmt, a.head_fmt);
            mk_produce_phase(c, a, a.tape + off[a.n_layers * 4], PH_HEAD, c.phase_tab()[8 + PH_HEAD]);
        }
    }
    // every issued copy has been waited for by the consumers unless the kernel is aborting:
    // then give the copies in flight a bounded time to land before the CTA retires.
    if (*c.abort_flag()) {
        // the last nslot entries: slot s was last filled with parity par (slots before the cursor) or
        // par ^ 1 (slots at and after it)
        for (int sidx = 0; sidx < c.nslot(); sidx++) {
            if (c.entry < (unsigned)c.nslot() && sidx >= (int)c.entry) continue;
            const uint32_t par = sidx < c.slot ? c.par : (c.par ^ 1u);
            const long long t0 = global_ns();
            while (!mbar_try(&c.full()[sidx], par) && global_ns() - t0 < 40000000ll) {}
        }
    }
}

// ---------------------------------------------------------------------
// Consumer side of one matvec phase.
//   EPI_QKV   : pairs -> bias, RoPE -> tagged q / fp16-rounded tagged k,v
//   EPI_RESID : out[r] = hs[r] + dot -> tagged
//   EPI_SWIGLU: pairs (gate, up) -> silu(g) * u -> tagged
//   EPI_LOGITS: logits[r] (plain store if requested) + running argmax
// xs holds the (un-normalised) input vector, `scale` the RMSNorm factor
// (1 for plain inputs; norm weights are already folded into xs).
// ---------------------------------------------------------------------
// ---------------------------------------------------------------------
// One matvec phase on the consumer warps.  ONE code path serves every phase
// (QKV, wo, gate/up, down, lm_head) so that the instructions stay resident in
// the instruction caches across the ~120 phases of a token; only the epilogue
// switches on the phase.  Rows are always processed two at a time:
//   QKV      : the two rows of a RoPE pair  -> bias, rotate -> tagged q / fp16-rounded tagged k,v
//   gate/up  : gate row j and up row j      -> silu(g) * u -> tagged
//   wo, down : two consecutive output rows  -> hs[r] + dot -> tagged
//   lm_head  : two consecutive vocab rows   -> logits (optional) + running argmax
// xs holds the input vector (norm weights already folded in), `scale` is the RMSNorm factor.
// ---------------------------------------------------------------------
template <bool TP>
__device__ __forceinline__ void mk_epilogue(const MegaArgs& a, MkCtx& c, int p, int layer, unsigned int tag,
                                            int row, bool has2, float v0, float v1, unsigned long long& best) {
    const int ib = c.phase_tab()[p];
    {   // self-check: every index an epilogue writes through must lie inside its vector
        const int lim = p == PH_QKV ? (a.q_dim + 2 * a.kv_dim) / 2 : p == PH_GU ? a.ffn_dim : p == PH_HEAD ? a.vocab : a.dim;
        const int idx = (p == PH_QKV || p == PH_GU) ? ib + (row >> 1) : ib + row + (has2 ? 1 : 0);
        if (row < 0 || idx >= lim) { mk_fail(c, MK_ERR_RANGE, 1000 * p + 100000 + row); return; }
    }
    if (p == PH_QKV) {
        // same mapping as qkv_pair(), with the divisions by head_dim/2 done as shifts
        const int item = ib + (row >> 1);
        const int half = a.head_dim >> 1, hs1 = a.hd_shift - 1;
        const int nq = a.q_dim >> 1, nk = a.kv_dim >> 1;
        int m = 0, i = item;
        if (i >= nq) { i -= nq; m = 1; }
        if (m == 1 && i >= nk) { i -= nk; m = 2; }
        int r0, r1;
        if (m < 2) {
            const int head = i >> hs1, j = i - (head << hs1);
            r0 = (head << a.hd_shift) + j;
            r1 = r0 + half;
        } else {
            r0 = 2 * i;
            r1 = r0 + 1;
        }
        if (a.qkv_bias) {
            const float* bias = a.qkv_bias + (size_t)layer * (a.q_dim + 2 * a.kv_dim) +
                                (m == 0 ? 0 : m == 1 ? a.q_dim : a.q_dim + a.kv_dim);
            v0 += bias[r0];
            v1 += bias[r1];
        }
        if (m < 2) {
            const int j = r0 & (a.head_dim - 1);
            const float cs = c.rope()[j], sn = c.rope()[half + j];
            const float t0 = v0 * cs - v1 * sn, t1 = v0 * sn + v1 * cs;
            v0 = t0; v1 = t1;
        }
        if (m == 0) {
            st_tagged(a.xq + r0, v0, tag);
            st_tagged(a.xq + r1, v1, tag);
        } else {
            // K (after RoPE) and V are stored in the cache as fp16: exchange the rounded values
            Tagged* dst = a.xkv + (m == 1 ? 0 : a.kv_dim);
            st_tagged(dst + r0, __half2float(__float2half_rn(v0)), tag);
            st_tagged(dst + r1, __half2float(__float2half_rn(v1)), tag);
        }
    } else if (p == PH_GU) {
        st_tagged(a.xmid + ib + (row >> 1), v0 * (1.0f / (1.0f + expf(-v0))) * v1, tag);
    } else if (p == PH_HEAD) {
        const int r0 = ib + row;
        if (a.head == 2) { a.logits[r0] = v0; if (has2) a.logits[r0 + 1] = v1; }
        unsigned long long key = pack_best(v0, (unsigned)(r0 + a.vocab_base));
        if (key > best) best = key;
        if (has2) { key = pack_best(v1, (unsigned)(r0 + 1 + a.vocab_base)); if (key > best) best = key; }
    } else {
        const int r0 = ib + row;
        if (!TP) {
            Tagged* out = p == PH_WO ? a.xhm : a.xh;
            st_tagged(out + r0, c.hs()[r0] + v0, tag);
            if (has2) st_tagged(out + r0 + 1, c.hs()[r0 + 1] + v1, tag);
        } else {
            // partial sum over this rank's heads / FFN features: into row tp_rank of every rank's receive
            // buffer; rank 0's row carries the residual
            const float w0 = (a.tp_rank == 0 ? c.hs()[r0] : 0.f) + v0;
            const float w1 = has2 ? (a.tp_rank == 0 ? c.hs()[r0 + 1] : 0.f) + v1 : 0.f;
            Tagged* const* peers = p == PH_WO ? a.xhm_peer : a.xh_peer;
            for (int q = 0; q < a.tp_n; q++) {
                Tagged* out = peers[q] + (size_t)a.tp_rank * a.dim + r0;
                st_tagged_sys(out, w0, tag);
                if (has2) st_tagged_sys(out + 1, w1, tag);
            }
        }
    }
}

// Dot product of this lane's share of a tile row with the staged activations.
// tile: [ni][32] x 16-byte weight chunks, then [ni][32] fp16 block scales (lane order).
// Lane `part` of a row takes chunks part, part + lpr, ...; chunks beyond the row are zero in the
// tape (weights and scale), their activation index is clamped so that the loads stay in range.
template <int FMT>
__device__ __forceinline__ float tile_dot(MkCtx& c, const uint8_t* tile, int ni, int lane, int part, int lpr_shift,
                                          int K) {
    float acc = 0.f;
    if (FMT == FMT_F16) {
        const int last = (K >> 3) - 1;
        const float* xs = c.xs();
#pragma unroll 4
        for (int i = 0; i < ni; i++) {
            const uint4 w = lds16(tile + (size_t)(i * 32 + lane) * 16);
            const int ch = min(part + (i << lpr_shift), last);
            const float4 xa = *reinterpret_cast<const float4*>(xs + ch * 8);
            const float4 xb = *reinterpret_cast<const float4*>(xs + ch * 8 + 4);
            acc += dot8_f16(w, xa, xb);
        }
        return acc;
    }
    const unsigned short* ds = reinterpret_cast<const unsigned short*>(tile + (size_t)ni * 512);
    const uint8_t* p0 = xq_plane(c, K, 0);
    const uint8_t* p1 = xq_plane(c, K, 1);
    const uint8_t* p2 = xq_plane(c, K, 2);
    const float2* sc = xq_scales(c, K);
    if (FMT == FMT_Q8_0) {
        const int last = (K >> 4) - 1;
#pragma unroll 4
        for (int i = 0; i < ni; i++) {
            const uint4 w = lds16(tile + (size_t)(i * 32 + lane) * 16);
            const float d = half_bits_to_float(ds[i * 32 + lane]);
            const int g = min(part + (i << lpr_shift), last);          // chunk = activation group
            const float f = group_dot_s8(w, lds16(p0 + g * 16), lds16(p1 + g * 16), lds16(p2 + g * 16));
            acc = fmaf(d * sc[g].x, f, acc);
        }
    } else {
        const int last = (K >> 5) - 1;
#pragma unroll 4
        for (int i = 0; i < ni; i++) {
            const uint4 w = lds16(tile + (size_t)(i * 32 + lane) * 16);
            const float d = half_bits_to_float(ds[i * 32 + lane]);
            const int b = min(part + (i << lpr_shift), last);          // chunk = block = groups 2b, 2b+1
            const int ga = 2 * b, gb = 2 * b + 1;
            // word i holds bytes 4i..4i+3: low nibbles = elements 4i..4i+3 (group A), high = 16+4i.. (group B)
            const float fa = group_dot_u4(w.x & 0x0f0f0f0fu, w.y & 0x0f0f0f0fu, w.z & 0x0f0f0f0fu, w.w & 0x0f0f0f0fu,
                                          lds16(p0 + ga * 16), lds16(p1 + ga * 16), lds16(p2 + ga * 16));
            const float fb = group_dot_u4((w.x >> 4) & 0x0f0f0f0fu, (w.y >> 4) & 0x0f0f0f0fu,
                                          (w.z >> 4) & 0x0f0f0f0fu, (w.w >> 4) & 0x0f0f0f0fu,
                                          lds16(p0 + gb * 16), lds16(p1 + gb * 16), lds16(p2 + gb * 16));
            const float2 sa = sc[ga], sb = sc[gb];
            // sum (nib - 8) x = sum nib x - 8 sum x
            acc = fmaf(d, fmaf(sa.x, fa, sb.x * fb) - 8.0f * (sa.y + sb.y), acc);
        }
    }
    return acc;
}

template <int FMT, bool TP>
__device__ __forceinline__ void mk_phase(const MegaArgs& a, MkCtx& c, int p, int layer, unsigned int tag, float scale,
                                         unsigned long long& best) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const PhaseGeom g = a.geom[p];
    const int K = p == PH_DOWN ? a.ffn_dim : p == PH_WO ? a.q_dim : a.dim;
    const bool pairs = (p == PH_QKV || p == PH_GU);
    const int nrows = c.phase_tab()[8 + p] * (pairs ? 2 : 1);
    const int lpr = 1 << g.lpr_shift;
    const int part = lane & (lpr - 1), rloc = lane >> g.lpr_shift;
    const int ntiles = (nrows + (32 >> g.lpr_shift) - 1) >> (5 - g.lpr_shift);
    int carry = w;                                   // this warp's next tile, relative to the entry's first tile

    for (int t = 0; t < ntiles; t += g.tpe) {
        const int nt = min(g.tpe, ntiles - t);
        const int slot = c.slot;
        int tl = carry;
        carry -= nt;
        // Every warp observes every entry's arrival, also of entries it owns no tile of: a warp that
        // skipped ahead could otherwise meet a slot whose barrier is a whole ring revolution behind,
        // take the stale phase for its own (parity waits cannot tell them apart) and release the slot
        // early.  Waiting on a completed phase costs a few cycles.
        mk_wait_bar(c, &c.full()[slot], c.par, MK_ERR_FULL);
        if (tl < nt) {
            // tiles are dealt to the warps round-robin over the whole phase
            const uint8_t* base = c.ring() + (size_t)slot * a.slot_bytes;
            if (slot < 0 || slot >= a.nslot || nt * g.tile_bytes > a.slot_bytes || g.ni <= 0) {
                mk_fail(c, MK_ERR_RANGE, 200000 + p);
                tl = nt + ((tl - nt) % MK_NW + MK_NW) % MK_NW;      // skip this entry's tiles
            }
            for (; tl < nt; tl += MK_NW) {
                float v = tile_dot<FMT>(c, base + (size_t)tl * g.tile_bytes, g.ni, lane, part, g.lpr_shift, K);
                for (int o = lpr >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(MG_FULL_MASK, v, o);
                v *= scale;
                const int row = ((t + tl) << (5 - g.lpr_shift)) + rloc;       // row within this CTA's phase rows
                if (pairs) {
                    const float v1 = __shfl_down_sync(MG_FULL_MASK, v, lpr);  // the partner row sits lpr lanes up
                    if (part == 0 && (rloc & 1) == 0 && row < nrows) mk_epilogue<TP>(a, c, p, layer, tag, row, true, v, v1, best);
                } else {
                    if (part == 0 && row < nrows) mk_epilogue<TP>(a, c, p, layer, tag, row, false, v, 0.f, best);
                }
            }
            carry = tl - nt;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&c.empty()[slot]);
        c.advance();
    }
}

// Hidden-state staging fused with RMSNorm.  Each thread fetches a pair of elements of the
// hidden state (from an exchange buffer, the embedding row, or a plain vector), keeps the raw
// values in hs (the residual), writes value * norm weight to xs and returns the RMSNorm factor
// 1/sqrt(mean(h^2) + eps), which callers fold into the activation registers.  One barrier.
enum : int { SRC_POLL = 0, SRC_EMBED = 1, SRC_PLAIN = 2 };
template <bool TP>
__device__ __forceinline__ float mk_stage_norm(const MegaArgs& a, MkCtx& c, int src_kind, const Tagged* xsrc,
                                               unsigned int tag, int token, const float* norm_w, bool quant, bool quant_sum) {
    float ss = 0.f;
    for (int i0 = 0; i0 < a.dim; i0 += 2 * MK_CONSUMERS) {
        const int i = i0 + 2 * (int)threadIdx.x;
        const bool ok = i < a.dim;
        float v0 = 0.f, v1 = 0.f;
        float2 nw = make_float2(0.f, 0.f);
        if (ok) {
            nw = *reinterpret_cast<const float2*>(norm_w + i);   // issued before the poll
            if (src_kind == SRC_POLL) {
                if (!TP) mk_poll2(c, xsrc + i, tag, v0, v1);
                else mk_poll2_sum(c, xsrc + i, a.dim, a.tp_n, tag, v0, v1);
            } else if (src_kind == SRC_EMBED) {
                v0 = embed_value(a.embed_w, a.head_fmt, a.dim, token, i);
                v1 = embed_value(a.embed_w, a.head_fmt, a.dim, token, i + 1);
            } else {
                v0 = a.h_in[i];
                v1 = a.h_in[i + 1];
            }
            c.hs()[i] = v0;
            c.hs()[i + 1] = v1;
            ss = fmaf(v0, v0, ss);
            ss = fmaf(v1, v1, ss);
        }
        if (quant) {
            xq_store_pair(c, a.dim, i, ok, v0 * nw.x, v1 * nw.y, quant_sum);
        } else if (ok) {
            c.xs()[i] = v0 * nw.x;
            c.xs()[i + 1] = v1 * nw.y;
        }
    }
    const float tot = mk_block_sum(c, ss);     // barrier: xs and hs are published
    return rsqrtf(tot / (float)a.dim + a.eps);
}

// ---------------------------------------------------------------------
// Attention for one query head on this CTA (fp16 KV cache).
// Cached K/V rows do not depend on this token, so each thread loads the rows it
// will need into registers BEFORE it waits for q: thread t holds the K row of
// position t, thread (group g, dim pair dp) holds V[g + j*Gp][2dp..2dp+1] for
// j < MK_VPF.  Longer contexts take the remainder from L2 in unrolled batches.
// ---------------------------------------------------------------------
constexpr int MK_VPF = 16;

__device__ __forceinline__ float dot8_kq(uint4 kk, const float* q) {
    const __half2* h = reinterpret_cast<const __half2*>(&kk);
    const float4 qa = reinterpret_cast<const float4*>(q)[0];
    const float4 qb = reinterpret_cast<const float4*>(q)[1];
    const float2 k0 = __half22float2(h[0]), k1 = __half22float2(h[1]);
    const float2 k2 = __half22float2(h[2]), k3 = __half22float2(h[3]);
    float d0 = qa.x * k0.x, d1 = qa.y * k0.y;
    d0 = fmaf(qa.z, k1.x, d0); d1 = fmaf(qa.w, k1.y, d1);
    d0 = fmaf(qb.x, k2.x, d0); d1 = fmaf(qb.y, k2.y, d1);
    d0 = fmaf(qb.z, k3.x, d0); d1 = fmaf(qb.w, k3.y, d1);
    return d0 + d1;
}

template <int HD>
__device__ __forceinline__ void mk_attention(const MegaArgs& a, MkCtx& c, int layer, int pos, unsigned int tag_in,
                                             unsigned int tag_out) {
    constexpr int KV = HD / 8;                 // 16-byte pieces of one K row
    constexpr int DP = HD / 2;                 // dim pairs
    constexpr int Gp = MK_CONSUMERS / DP;      // whole position groups: 15 for hd 64, 7 for hd 128, 30 for hd 32
    const int head = blockIdx.x;
    const int kvh = head / (a.n_heads / a.n_kv_heads);
    const int tid = threadIdx.x;
    const size_t lbase = (size_t)layer * a.max_seq * a.kv_dim;
    __half* kc = a.kc + lbase + kvh * HD;
    __half* vc = a.vc + lbase + kvh * HD;
    float* qs = c.xs();                 // HD
    float* kn = c.xs() + HD;            // new K row
    float* vn = c.xs() + 2 * HD;        // new V row
    const int g = tid / DP, dp = tid - g * DP;

    // ---- prefetch cached rows (positions < pos) ----
    uint4 kreg[KV];
#pragma unroll
    for (int i = 0; i < KV; i++) kreg[i] = make_uint4(0u, 0u, 0u, 0u);
    if (tid < pos) {
        const uint4* kp = reinterpret_cast<const uint4*>(kc + (size_t)tid * a.kv_dim);
#pragma unroll
        for (int i = 0; i < KV; i++) kreg[i] = __ldcg(kp + i);
    }
    __half2 vreg[MK_VPF];
#pragma unroll
    for (int j = 0; j < MK_VPF; j++) {
        const int t = g + j * Gp;
        vreg[j] = __floats2half2_rn(0.f, 0.f);
        if (g < Gp && t < pos) vreg[j] = __ldcg(reinterpret_cast<const __half2*>(vc + (size_t)t * a.kv_dim) + dp);
    }

    // ---- gather q, new k, new v (HD values each); append the new row to the cache ----
    for (int i = 2 * tid; i < 3 * HD; i += 2 * MK_CONSUMERS) {
        const int which = i / HD, d = i - which * HD;
        const Tagged* src = which == 0 ? a.xq + head * HD + d
                          : which == 1 ? a.xkv + kvh * HD + d
                                       : a.xkv + a.kv_dim + kvh * HD + d;
        float v0, v1;
        mk_poll2(c, src, tag_in, v0, v1);
        c.xs()[i] = v0;
        c.xs()[i + 1] = v1;
        // every CTA of the KV group appends the (identical) new row; each CTA later reads back
        // only addresses it has written itself
        if (which == 1) *reinterpret_cast<__half2*>(kc + (size_t)pos * a.kv_dim + d) = __floats2half2_rn(v0, v1);
        if (which == 2) *reinterpret_cast<__half2*>(vc + (size_t)pos * a.kv_dim + d) = __floats2half2_rn(v0, v1);
    }
    consumer_sync();

    // ---- scores: thread t owns position t; the new position's K row comes from shared memory ----
    const int len = pos + 1;
    const float scale = rsqrtf((float)HD);
    float mx = -INFINITY;
    if (tid == pos) {
#pragma unroll
        for (int i = 0; i < KV; i++) {
            const float4 ka = reinterpret_cast<const float4*>(kn)[2 * i], kb = reinterpret_cast<const float4*>(kn)[2 * i + 1];
            __half2 h[4] = {__floats2half2_rn(ka.x, ka.y), __floats2half2_rn(ka.z, ka.w), __floats2half2_rn(kb.x, kb.y),
                            __floats2half2_rn(kb.z, kb.w)};      // exact: kn already holds fp16-rounded values
            kreg[i] = *reinterpret_cast<const uint4*>(h);
        }
    }
    if (tid <= pos) {
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < KV; i++) dot += dot8_kq(kreg[i], qs + 8 * i);
        dot *= scale;
        c.sc()[tid] = dot;
        mx = dot;
    }
    for (int t = tid + MK_CONSUMERS; t <= pos; t += MK_CONSUMERS) {     // contexts beyond one row per thread
        float dot = 0.f;
        if (t == pos) {
            for (int d = 0; d < HD; d++) dot = fmaf(qs[d], kn[d], dot);
        } else {
            const uint4* kp = reinterpret_cast<const uint4*>(kc + (size_t)t * a.kv_dim);
            uint4 kk[KV];
#pragma unroll
            for (int i = 0; i < KV; i++) kk[i] = __ldcg(kp + i);
#pragma unroll
            for (int i = 0; i < KV; i++) dot += dot8_kq(kk[i], qs + 8 * i);
        }
        dot *= scale;
        c.sc()[t] = dot;
        mx = fmaxf(mx, dot);
    }
    mx = warp_max(mx);
    const int lane = tid & 31, w = tid >> 5;
    if (lane == 0) c.red()[32 + w] = mx;
    consumer_sync();
    mx = c.red()[32];
#pragma unroll
    for (int i = 1; i < MK_NW; i++) mx = fmaxf(mx, c.red()[32 + i]);
    float sum = 0.f;
    for (int t = tid; t < len; t += MK_CONSUMERS) {
        const float pv = expf(c.sc()[t] - mx);
        c.sc()[t] = pv;
        sum += pv;
    }
    sum = mk_block_sum(c, sum);      // barrier publishes sc[]

    // ---- weighted V ----
    if (g < Gp) {
        float2 acc = make_float2(0.f, 0.f);
#pragma unroll
        for (int j = 0; j < MK_VPF; j++) {
            const int t = g + j * Gp;
            if (t < pos) {
                const float2 vf = __half22float2(vreg[j]);
                const float pv = c.sc()[t];
                acc.x = fmaf(pv, vf.x, acc.x);
                acc.y = fmaf(pv, vf.y, acc.y);
            }
        }
        for (int t0 = g + MK_VPF * Gp; t0 < pos; t0 += 4 * Gp) {        // remainder, four loads in flight
            __half2 vv[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int t = t0 + j * Gp;
                vv[j] = __floats2half2_rn(0.f, 0.f);
                if (t < pos) vv[j] = __ldcg(reinterpret_cast<const __half2*>(vc + (size_t)t * a.kv_dim) + dp);
            }
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int t = t0 + j * Gp;
                if (t < pos) {
                    const float2 vf = __half22float2(vv[j]);
                    const float pv = c.sc()[t];
                    acc.x = fmaf(pv, vf.x, acc.x);
                    acc.y = fmaf(pv, vf.y, acc.y);
                }
            }
        }
        if (g == pos % Gp) {                                             // the new position belongs to one group
            const float pv = c.sc()[pos];
            acc.x = fmaf(pv, vn[2 * dp], acc.x);
            acc.y = fmaf(pv, vn[2 * dp + 1], acc.y);
        }
        c.part()[g * HD + 2 * dp] = acc.x;
        c.part()[g * HD + 2 * dp + 1] = acc.y;
    }
    consumer_sync();
    if (tid < HD) {
        float s = 0.f;
#pragma unroll 1
        for (int gg = 0; gg < Gp; gg++) s += c.part()[gg * HD + tid];
        st_tagged(a.xattn + head * HD + tid, s / sum, tag_out);
    }
    consumer_sync();     // part / xs are reused by the next phase
}

// ---------------------------------------------------------------------
// Consumer warps: the decode loop, one flat loop over phases.
// Phase index ph = layer * 4 + p for the layer phases; ph = L * 4 is lm_head.
// Trace events per layer (mg_trace_step): 2p = input of phase p ready, 2p+1 = phase p done,
// 8 = layer start, 9 = attention done (attention CTAs).
// ---------------------------------------------------------------------
template <bool TP>
__device__ __forceinline__ void mk_consumer(MkCtx& c, const MegaArgs& a) {
    const int tid = threadIdx.x;
    const int L = a.n_layers;
    const int half = a.head_dim / 2;
    const int pos0 = a.st->pos;
    int token = a.st->token;
    const bool do_head = a.le >= L && a.head;
    const int ph_begin = a.ls * 4;
    const int ph_end = a.le * 4 + (do_head ? 1 : 0);

    for (int step = 0; step < a.n_steps; step++) {
        const unsigned int ep = a.epoch + (unsigned)step * (unsigned)(L * MK_EPOCHS_PER_LAYER + 8);
        const int pos = min(pos0 + step, a.max_seq - 1);
        // ---- token of this step (greedy feedback from the previous step) ----
        if (a.embed) {
            if (step > 0) token = (int)__float_as_uint(mk_poll1(c, a.xtok, ep - 8u + 1u));
            token = min(max(token, 0), a.vocab_total - 1);
        }
        // RoPE row of this position: staged once per step, published by the first stage barrier
        if (tid < 2 * half)
            c.rope()[tid] = tid < half ? a.cos_tab[(size_t)pos * half + tid] : a.sin_tab[(size_t)pos * half + tid - half];
        unsigned long long best = 0ull;

        for (int ph = ph_begin; ph < ph_end; ph++) {
            const bool is_head = ph >= L * 4;
            const int l = is_head ? L : (ph >> 2);
            const int p = is_head ? PH_HEAD : (ph & 3);
            // tags of layer l: +1 q/kv, +2 attn, +3 h after wo, +4 ffn mid, +5 h after down
            const unsigned int base = ep + (unsigned)l * MK_EPOCHS_PER_LAYER;
            const unsigned int tag_prev_h = base - MK_EPOCHS_PER_LAYER + 5;
            if (p == PH_QKV) mk_trace(a, step, l * 10 + 8);

            // ---- input staging ----
            float scale = 1.0f;
            if (p == PH_QKV || p == PH_GU || p == PH_HEAD) {
                int kind = SRC_POLL;
                const Tagged* src = a.xh;
                unsigned int tag = tag_prev_h;
                const float* nw = is_head ? a.final_norm : a.norms + (size_t)l * 2 * a.dim;
                if (p == PH_GU) { src = a.xhm; tag = base + 3; nw += a.dim; }
                else if (p == PH_QKV && l == a.ls) kind = a.embed ? SRC_EMBED : SRC_PLAIN;
                scale = mk_stage_norm<TP>(a, c, kind, src, tag, token, nw, (is_head ? a.head_fmt : a.layer_fmt) != FMT_F16,
                                      (is_head ? a.head_fmt : a.layer_fmt) == FMT_Q4_0);
            } else {
                if (p == PH_WO && (int)blockIdx.x < a.n_heads) {
                    if (a.head_dim == 64) mk_attention<64>(a, c, l, pos, base + 1, base + 2);
                    else if (a.head_dim == 128) mk_attention<128>(a, c, l, pos, base + 1, base + 2);
                    else mk_attention<32>(a, c, l, pos, base + 1, base + 2);
                    mk_trace(a, step, l * 10 + 9);
                }
                const bool wo = p == PH_WO;
                if (a.layer_fmt != FMT_F16) mk_gather_q(c, wo ? a.xattn : a.xmid, wo ? base + 2 : base + 4, wo ? a.q_dim : a.ffn_dim, a.layer_fmt == FMT_Q4_0);
                else mk_gather(c, wo ? a.xattn : a.xmid, wo ? base + 2 : base + 4, c.xs(), wo ? a.q_dim : a.ffn_dim);
                consumer_sync();
            }
            if (is_head && blockIdx.x == 0 && a.h_out && step == a.n_steps - 1)
                for (int i = tid; i < a.dim; i += MK_CONSUMERS) a.h_out[i] = c.hs()[i];
            mk_trace(a, step, l * 10 + 2 * (is_head ? 0 : p));

            // ---- matvec + fused epilogue ----
            const unsigned int tag_out = base + (p == PH_QKV ? 1u : p == PH_WO ? 3u : p == PH_GU ? 4u : 5u);
            const int fmt = is_head ? a.head_fmt : a.layer_fmt;
            if (fmt == FMT_Q8_0) mk_phase<FMT_Q8_0, TP>(a, c, p, l, tag_out, scale, best);
            else if (fmt == FMT_Q4_0) mk_phase<FMT_Q4_0, TP>(a, c, p, l, tag_out, scale, best);
            else mk_phase<FMT_F16, TP>(a, c, p, l, tag_out, scale, best);
            consumer_sync();             // xs / hs / part are reused by the next phase
            mk_trace(a, step, l * 10 + 2 * (is_head ? 0 : p) + 1);
        }

        if (!do_head) {
            // partial layer range: CTA 0 hands the hidden state back
            if (blockIdx.x == 0 && a.h_out && step == a.n_steps - 1 && a.le > a.ls) {
                const unsigned int tag_final_h = ep + (unsigned)(a.le - 1) * MK_EPOCHS_PER_LAYER + 5;
                if (!TP) {
                    mk_gather(c, a.xh, tag_final_h, c.hs(), a.dim);
                } else {
                    for (int i = 2 * tid; i < a.dim; i += 2 * MK_CONSUMERS) {
                        float u0, u1;
                        mk_poll2_sum(c, a.xh + i, a.dim, a.tp_n, tag_final_h, u0, u1);
                        c.hs()[i] = u0;
                        c.hs()[i + 1] = u1;
                    }
                }
                consumer_sync();
                for (int i = tid; i < a.dim; i += MK_CONSUMERS) a.h_out[i] = c.hs()[i];
            }
        } else {
            // CTA argmax -> one atomic per CTA -> the last CTA publishes the token
            unsigned long long* sb = reinterpret_cast<unsigned long long*>(c.part());
            unsigned long long wb = best;         // candidates may sit in any lane (cross-segment path)
#pragma unroll
            for (int sh = 16; sh > 0; sh >>= 1) {
                const unsigned long long other = __shfl_xor_sync(MG_FULL_MASK, wb, sh);
                wb = other > wb ? other : wb;
            }
            if ((tid & 31) == 0) sb[tid >> 5] = wb;
            consumer_sync();
            if (tid == 0) {
                unsigned long long b = sb[0];
                for (int i = 1; i < MK_NW; i++) b = sb[i] > b ? sb[i] : b;
                StepState* s = a.st;
                if (b) atomicMax(&s->best, b);
                __threadfence();
                const unsigned int ticket = atomicAdd(&s->done, 1u);
                if (ticket == gridDim.x - 1) {
                    __threadfence();
                    unsigned long long key = atomicMax(&s->best, 0ull);
                    if (TP) {
                        // every rank publishes the key of its vocabulary slice to every rank; the largest
                        // key (highest logit, lowest index) wins on all of them
                        const unsigned int tagx = ep + (unsigned)(L * MK_EPOCHS_PER_LAYER) + 2u;
                        for (int q = 0; q < a.tp_n; q++) {
                            st_tagged_sys(a.xbest_peer[q] + 2 * a.tp_rank, __uint_as_float((unsigned)(key >> 32)), tagx);
                            st_tagged_sys(a.xbest_peer[q] + 2 * a.tp_rank + 1, __uint_as_float((unsigned)key), tagx);
                        }
                        for (int r = 0; r < a.tp_n; r++) {
                            // raw words: the halves of a key are bit patterns, not numbers
                            const uint4 w = mk_poll16_sys(c, a.xbest + 2 * r, tagx);
                            const unsigned long long k = ((unsigned long long)w.x << 32) | (unsigned long long)w.z;
                            key = k > key ? k : key;
                        }
                    }
                    const int tok = (int)(0xffffffffu - (unsigned int)(key & 0xffffffffull));
                    if (a.out_tokens && s->step < s->out_cap) a.out_tokens[s->step] = tok;
                    s->token = tok;
                    s->step += 1;
                    s->pos += 1;
                    s->best = 0ull;
                    s->done = 0u;
                    __threadfence();
                    st_tagged(a.xtok, __uint_as_float((unsigned)tok), ep + (unsigned)(L * MK_EPOCHS_PER_LAYER) + 1u);
                }
            }
            consumer_sync();
        }
    }
}

__host__ __device__ inline size_t mk_smem_bytes(int nslot, int slot_bytes, int xs_floats, int dim, int sc_floats) {
    return (size_t)nslot * slot_bytes + ((size_t)xs_floats + dim + MK_PART_FLOATS + 64 + MK_ROPE_FLOATS + sc_floats) * 4 +
           2 * MK_MAX_SLOTS * 8 + 16 + 144;
}

// TP = false: one GPU (no peer pointers are touched); TP = true: one rank of a tensor-parallel group.
template <bool TP>
__global__ void __launch_bounds__(MK_THREADS, 1) mega_decode_kernel(const MegaArgs a) {
    MkCtx c(a);
    if (threadIdx.x == 0) {
        for (int i = 0; i < a.nslot; i++) {
            mbar_init(&c.full()[i], 1);
            mbar_init(&c.empty()[i], MK_NW);
        }
        *c.abort_flag() = 0;
        for (int p = 0; p <= PH_HEAD; p++) {
            const PhaseShape sh = phase_shape_of(p, a.dim, a.q_dim, a.kv_dim, a.ffn_dim, a.vocab, a.layer_fmt, a.head_fmt);
            const int ib = item_begin(sh.items, blockIdx.x, gridDim.x);
            c.phase_tab()[p] = ib;
            c.phase_tab()[8 + p] = item_begin(sh.items, blockIdx.x + 1, gridDim.x) - ib;
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x >= MK_CONSUMERS) mk_producer(c, a);
    else mk_consumer<TP>(c, a);
}

}  // namespace mg
