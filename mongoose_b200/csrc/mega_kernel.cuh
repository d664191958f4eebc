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
//    consumes it.  The unit is a TILE: 16 row-slots x one block of 32 input
//    columns ("tall"), or 8 rows x two consecutive blocks ("wide", for phases
//    that have only a handful of rows per CTA), stored in the register order of
//    the m16n8k32 integer MMA's A operand (one 16-byte shared-memory load per
//    lane) followed by the tile's 16 fp16 block scales.  A dedicated producer
//    warp walks the tape with bulk asynchronous copies (cp.async.bulk, mbarrier
//    completion) into a ring of shared-memory slots, running up to a ring ahead
//    of the consumers - weights never depend on activations, so HBM streaming
//    is off the dependency chain.
//  * Tagged exchange.  A phase's output vector is written to global memory as
//    8-byte {fp32 value, 32-bit epoch} words.  Consumers poll the words they
//    need until the epoch is the one they expect: data and flag arrive in one
//    atomic 8-byte access, so no fence, no counter and no reset is needed, and
//    a stale buffer can never be mistaken for fresh data.
//  * 15 consumer warps per CTA, all of them busy in every phase.  The input
//    vector is staged in shared memory as 24-bit fixed point in three signed
//    byte planes with one scale per block of 32; the planes are three columns
//    of the MMA's B operand, so ONE mma.sync multiplies a 512-byte weight tile
//    with the whole 24-bit activation block, exactly, in int32.  Per tile a
//    lane then does two int->float conversions and two FMAs with
//    (block scale x activation scale).  A phase's tiles are dealt to the warps
//    as (row-group, K-split) pairs chosen per phase on the host, so that a
//    phase with eight rows per CTA still gives every warp one tile; the K-split
//    partial sums meet in shared memory and one thread per output row runs the
//    fused epilogue (bias + RoPE + fp16 rounding, residual add, SiLU * up,
//    argmax).  fp16 weights use the same tiles with fp32 FMAs.
//
//  * Feed-forward block on one GPU.  A CTA's gate/up rows are a contiguous run
//    of FFN features, so its silu(g) * u values are a window of the down
//    projection's input.  The CTA multiplies that window by ALL rows of the
//    down matrix and adds the row sums, as 64-bit fixed point (associative, so
//    the result does not depend on arrival order), into one of three rotating
//    accumulators; the low byte of every word counts the additions it has
//    received, so the next phase polls data and completion in one load, as
//    with the tagged words.  The FFN-wide middle vector never crosses SMs.
//    Tensor-parallel ranks keep the exchanged middle vector (their partial
//    sums cross GPUs).
//
// Every wait (mbarrier, exchange poll) is bounded by a deadline in SM clocks
// (MegaArgs::wait_cycles, about 1 s by default); on expiry the kernel records
// an error code, stops waiting everywhere and runs to completion on whatever
// data it has, so a logic error cannot hang the GPU.  The host checks the
// status word after each launch.
#pragma once

#include "decode_kernels.cuh"

namespace mg {

constexpr int MK_NW = 15;                       // consumer warps
constexpr int MK_CONSUMERS = MK_NW * 32;        // 480
constexpr int MK_THREADS = MK_CONSUMERS + 32;   // + producer warp = 512 threads, 128 registers each
constexpr int MK_SLOT = 32768;                  // ring slot bytes
constexpr int MK_MAX_SLOTS = 14;
constexpr int MK_PART_FLOATS = 2048;
constexpr int MK_EPOCHS_PER_LAYER = 8;
constexpr long long MK_WAIT_CYCLES = 2000000000ll;         // default per-wait limit: about one second of SM clocks

enum : int { PH_QKV = 0, PH_WO = 1, PH_GU = 2, PH_DOWN = 3, PH_HEAD = 4 };
enum : int { MK_OK = 0, MK_ERR_POLL = 1, MK_ERR_FULL = 2, MK_ERR_EMPTY = 3, MK_ERR_RANGE = 4 };

struct MegaStatus {
    int error;          // first error code (0 = none)
    int where;          // phase / tag that timed out
    int cta;
    int who;            // exchange polls: the rank whose row had not arrived (-1: not an exchange between ranks)
};

struct Tagged {         // one exchanged activation
    float v;
    unsigned int tag;
};

// How a phase's rows are laid over the warps (the same on every CTA).
//   A ROW-GROUP is the set of weight rows one tile column covers: 16 row-slots ("tall") or 8
//   ("wide").  Phases whose work items are row PAIRS (the two rows of a RoPE pair, gate row j and up
//   row j) put the first rows of `ipg` items in the lower half of the slots and the second rows in
//   the upper half.  A tile is one row-group x one k-tile: one block of 32 columns (tall) or two
//   consecutive blocks (wide; MMA rows 8..15 then hold the same 8 rows for the odd block).
//   S warps share a row-group and split its k-tiles (warp kp takes k-tiles kp, kp + S, ...);
//   RS row-groups are in flight at a time, RS * S <= MK_NW.  The tape stores the tiles in the order
//   the warps take them: pass (RS row-groups), round (S k-tiles), row-group, k-split.
struct PhaseGeom {
    int wide;
    int S;
    int RS;
    int nkt;            // k-tiles per row-group
    int ipg_shift;      // log2(work items per row-group)
    int tile_bytes;
    int tpe;            // tiles per ring entry
    int kblocks;        // blocks of 32 (fp16 weights: 16) input columns per row
    int K;              // input width
    int nfull;          // nkt / S: rounds in which every K-split has a tile
};

struct MegaArgs {
    int dim, kv_dim, head_dim, n_heads, n_kv_heads, ffn_dim, vocab, n_layers, max_seq;
    int layer_fmt, head_fmt;
    float eps;
    float inv_dim;          // 1 / dim
    int ls, le;             // layer range
    int head;               // HEAD_NONE / HEAD_ARGMAX / HEAD_LOGITS (0/1/2)
    int embed;              // 1: hidden state from the embedding row of st->token, 0: from h_in
    int n_steps;            // tokens per launch (greedy feedback between them)
    unsigned int epoch;     // first epoch of this launch
    int hd_shift;           // log2(head_dim)
    int nslot;
    int slot_bytes;         // ring slot size
    int prefetch_bytes;     // how far ahead of the ring the producer asks L2 for this CTA's tape (0 = off)
    int xs_floats;          // size of the staged-activation buffer (multiple of 4)
    long long wait_cycles;  // limit of every wait inside the kernel, in SM clocks
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
    long long* trace;       // optional [grid][(n_layers + 1) * MK_EV] SM-clock stamps of CTA thread 0 (first step)
    int trace_step;         // always 0: the step whose stamps are kept
    // Feed-forward block without a grid-wide exchange of its middle vector (one GPU only; see
    // mk_down_fused): three rotating accumulators of dim 64-bit words {fixed-point sum, arrival count}.
    int ffn_fused;
    int acc_buf0;           // accumulator (0..2) of this launch's first layer
    int qkv_cta0;           // the QKV rows are dealt to CTAs qkv_cta0 .. grid-1 (n_heads where that keeps the balance: the
                            // CTAs that run attention then load their cached K/V rows while the others multiply)
    int acc_n;              // additions that complete a word: the CTAs that own gate/up rows + 1 (the residual)
    long long* acc;         // [3][dim]
};

// ---------------------------------------------------------------------
// Work partition shared by the host tape builder and the kernel.
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

// Row-groups are dealt to the CTAs in contiguous, balanced runs (a CTA may get none).
__host__ __device__ inline int unit_begin(int units, int cta, int grid) {
    return (int)(((long long)cta * units) / grid);
}
__host__ __device__ inline int row_q_bytes(int fmt, int K) { return plane_row_bytes(fmt, K); }
__host__ __device__ inline int row_d_bytes(int fmt, int K) { return fmt == FMT_F16 ? 0 : (K / 32) * 2; }
__host__ __device__ inline int tile_bytes_of(int fmt) { return fmt == FMT_Q8_0 ? 544 : fmt == FMT_Q4_0 ? 288 : 512; }
__host__ __device__ inline int kblock_of(int fmt) { return fmt == FMT_F16 ? 16 : 32; }

// Row-slot s (0..15) of a row-group -> which item of the group (j), which of its rows, and, for
// wide tiles, which of the tile's two blocks.
__host__ __device__ inline void slot_item(int wide, int rpi, int s, int* j, int* which, int* kpar) {
    if (!wide) {
        *kpar = 0;
        if (rpi == 2) { *j = s & 7; *which = s >> 3; } else { *j = s; *which = 0; }
    } else {
        *kpar = s >> 3;
        s &= 7;
        if (rpi == 2) { *j = s & 3; *which = s >> 2; } else { *j = s; *which = 0; }
    }
}

// Layout of a phase: tall or wide tiles and the K-split that minimise the tiles the busiest warp
// walks through (plus a charge per pass and for the shared-memory reduction of a K-split).
__host__ inline PhaseGeom choose_geom(int fmt, int K, int items, int rpi, int grid, int n_warps, int slot_bytes,
                                      bool head, int force_wide = -1, int force_s = -1) {
    PhaseGeom best{};
    long long best_cost = -1;
    const int kblk = kblock_of(fmt), nkb = K / kblk;
    for (int wide = 0; wide <= 1; wide++) {
        if (force_wide >= 0 && wide != force_wide) continue;
        const int ipg = (wide ? 8 : 16) / rpi;
        const int units = (items + ipg - 1) / ipg;
        const int max_units = (units + grid - 1) / grid;
        const int nkt = wide ? (nkb + 1) / 2 : nkb;
        for (int S = 1; S <= n_warps; S++) {
            if (force_s >= 0 && S != force_s) continue;
            if (head && S != 1) continue;                  // lm_head: many rows, epilogue inside the warp
            const int RS = n_warps / S;
            if (!head && max_units * 16 > n_warps * 32) continue;       // one epilogue thread per row-slot
            const int passes = (max_units + RS - 1) / RS;
            if (max_units * 16 * (S == 1 ? 1 : ((S + 3) & ~3)) > MK_PART_FLOATS) continue;     // room for the partial sums
            const long long cost = (long long)passes * ((nkt + S - 1) / S) + passes + (S > 1 ? 3 : 0);
            if (best_cost < 0 || cost < best_cost) {
                best_cost = cost;
                best.wide = wide; best.S = S; best.RS = RS; best.nkt = nkt;
                best.ipg_shift = ipg == 16 ? 4 : ipg == 8 ? 3 : 2;
                best.tile_bytes = tile_bytes_of(fmt);
                best.tpe = slot_bytes / best.tile_bytes;
                best.kblocks = nkb;
                best.K = K; best.nfull = nkt / S;
            }
        }
    }
    if (best_cost < 0) best.nkt = 0;     // no feasible layout
    return best;
}

// Fused feed-forward block: first block of columns of the down projection's window on the CTA whose
// gate/up items start at `start` (the window is 2 nkt blocks wide and stays inside the matrix).
__host__ __device__ inline int down_window_block(int start, int kblk, int total_blocks, int nkt) {
    const int b = start / kblk, last = total_blocks - 2 * nkt;
    return b < last ? b : last;
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
    // byte offsets of the regions inside mk_smem, fixed for the launch
    uint32_t xs_off, hs_off, part_off, bar_off;
    int redsel;                   // which half of the RMS partial-sum buffer the current phase uses (0 / 16)
    int probe_base;               // profiling build: trace slot base of the phase being probed (-1: none)
    __device__ __forceinline__ MkCtx(const MegaArgs& args) : a(args), entry(0), slot(0), par(0), pf(0), redsel(0) {
        xs_off = (uint32_t)a.nslot * (uint32_t)a.slot_bytes;
        hs_off = xs_off + 4u * (uint32_t)a.xs_floats;
        part_off = hs_off + 4u * (uint32_t)a.dim;
        bar_off = part_off + 4u * (uint32_t)(MK_PART_FLOATS + 64 + MK_ROPE_FLOATS + a.sc_floats);
    }
    __device__ __forceinline__ void advance() {
        entry++;
        if (++slot == a.nslot) { slot = 0; par ^= 1u; }
    }
    __device__ __forceinline__ uint8_t* ring() const { return mk_smem; }
    __device__ __forceinline__ float* xs() const { return reinterpret_cast<float*>(mk_smem + xs_off); }
    __device__ __forceinline__ float* hs() const { return reinterpret_cast<float*>(mk_smem + hs_off); }
    __device__ __forceinline__ float* part() const { return reinterpret_cast<float*>(mk_smem + part_off); }
    __device__ __forceinline__ float* red() const { return part() + MK_PART_FLOATS; }
    __device__ __forceinline__ float* rope() const { return red() + 64; }
    __device__ __forceinline__ float* sc() const { return rope() + MK_ROPE_FLOATS; }
    __device__ __forceinline__ unsigned long long* full() const {
        return reinterpret_cast<unsigned long long*>(mk_smem + bar_off);
    }
    __device__ __forceinline__ unsigned long long* empty() const { return full() + MK_MAX_SLOTS; }
    __device__ __forceinline__ volatile int* abort_flag() const {
        return reinterpret_cast<volatile int*>(empty() + MK_MAX_SLOTS);
    }
    // per phase p: [p] first row-group of this CTA, [8+p] its number of row-groups;
    // then per phase and consumer warp (MK_WARP_TAB): row-group slot | K-split index << 8
    __device__ __forceinline__ int* phase_tab() const { return const_cast<int*>(reinterpret_cast<volatile int*>(abort_flag())) + 4; }
    __device__ __forceinline__ unsigned short* warp_tab() const { return reinterpret_cast<unsigned short*>(phase_tab() + 16); }
    __device__ __forceinline__ MegaStatus* status() const { return a.status; }
    __device__ __forceinline__ int nslot() const { return a.nslot; }
};

__device__ __noinline__ void mk_fail_impl(volatile int* abort_flag, MegaStatus* status, int code, int where, int who = -1) {
    *abort_flag = 1;
    if (atomicCAS(&status->error, 0, code) == 0) {
        status->where = where;
        status->cta = blockIdx.x;
        status->who = who;
    }
}
__device__ __forceinline__ void mk_fail(MkCtx& c, int code, int where) {
    mk_fail_impl(c.abort_flag(), c.status(), code, where);
}

#ifdef MK_PROBE_P
constexpr int MK_EV = 64;
#else
constexpr int MK_EV = 32;             // trace events per layer
#endif
#define MK_TRACE_EVENTS(L) (((L) + 1) * MK_EV)
__device__ __forceinline__ void mk_trace(const MegaArgs& a, int step, int ev) {
    if (a.trace && step == 0 && threadIdx.x == 0)
        a.trace[(size_t)blockIdx.x * MK_TRACE_EVENTS(a.n_layers) + ev] = clock64();
}

// Waits.  The fast path (the awaited thing is already there) is inlined; everything else lives
// in ONE out-of-line copy per kind of wait, so that the many places that wait add a handful of
// instructions each to the code a phase runs through (the kernel's speed is bounded by the length
// of the instruction stream of a phase as much as by its data).  All waits are bounded.
__device__ __noinline__ void mk_wait_bar_slow(volatile int* abort_flag, MegaStatus* status, long long limit,
                                              uint32_t bar_s, uint32_t parity, int code, int where) {
    if (*abort_flag) return;
    const long long t0 = global_ns();
    for (unsigned int it = 1;; ++it) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(bar_s), "r"(parity) : "memory");
        if (ok) return;
        if ((it & 63u) == 0u) {
            if (*abort_flag) return;
            if (*(volatile int*)&status->error) { *abort_flag = 1; return; }
            if (global_ns() - t0 > limit) { mk_fail_impl(abort_flag, status, code, where); return; }
        }
    }
}
__device__ __forceinline__ void mk_wait_bar(MkCtx& c, unsigned long long* bar, uint32_t parity, int code) {
    if (mbar_try(bar, parity)) return;
    mk_wait_bar_slow(c.abort_flag(), c.status(), c.a.wait_cycles, smem_u32(bar), parity, code, (int)c.entry);
}

// Re-read a pair of exchange words (16-byte aligned) until both carry `tag`; sys = the words may be
// written by another GPU.  Returns the raw words: x, z = values, y, w = tags.
__device__ __noinline__ uint4 mk_poll16_slow(volatile int* abort_flag, MegaStatus* status, long long limit,
                                             const Tagged* p, unsigned int tag, int sys, int who = -1) {
    uint4 r = make_uint4(0u, tag, 0u, tag);
    if (*abort_flag) return r;
    const long long t0 = global_ns();
    for (unsigned int it = 1;; ++it) {
        r = sys ? ld_poll16_sys(p) : ld_poll16(p);
        if (r.y == tag && r.w == tag) return r;
        if ((it & 63u) == 0u) {
            if (*abort_flag) return r;
            if (*(volatile int*)&status->error) { *abort_flag = 1; return r; }
            if (global_ns() - t0 > limit) { mk_fail_impl(abort_flag, status, MK_ERR_POLL, (int)tag, who); return r; }
        }
    }
}
// r holds a first attempt; poll on if it is stale.
__device__ __forceinline__ void mk_poll2_finish(MkCtx& c, const Tagged* p, unsigned int tag, uint4& r) {
    if (r.y != tag || r.w != tag) r = mk_poll16_slow(c.abort_flag(), c.status(), c.a.wait_cycles, p, tag, 0);
}
__device__ __forceinline__ void mk_poll2(MkCtx& c, const Tagged* p, unsigned int tag, float& v0, float& v1) {
    uint4 r = ld_poll16(p);
    mk_poll2_finish(c, p, tag, r);
    v0 = __uint_as_float(r.x);
    v1 = __uint_as_float(r.z);
}
__device__ __forceinline__ uint4 mk_poll16_sys(MkCtx& c, const Tagged* q, unsigned int tag, int who = -1) {
    uint4 w = ld_poll16_sys(q);
    if (w.y != tag || w.w != tag) w = mk_poll16_slow(c.abort_flag(), c.status(), c.a.wait_cycles, q, tag, 1, who);
    return w;
}
// One exchange word (the token of the previous step).
__device__ __forceinline__ float mk_poll1(MkCtx& c, const Tagged* p, unsigned int tag) {
    uint2 r = ld_poll8(p);
    if (r.y != tag && !*c.abort_flag()) {
        const long long t0 = global_ns();
        for (unsigned int it = 1;; ++it) {
            r = ld_poll8(p);
            if (r.y == tag) break;
            if ((it & 63u) == 0u) {
                if (*c.abort_flag()) break;
                if (*(volatile int*)&c.status()->error) { *c.abort_flag() = 1; break; }
                if (global_ns() - t0 > c.a.wait_cycles) { mk_fail(c, MK_ERR_POLL, (int)tag); break; }
            }
        }
    }
    return __uint_as_float(r.x);
}

// Two adjacent values of a vector that arrives as one row per rank: the rows are added in rank
// order (every rank forms the same bits).  p points into row 0, rows are `stride` words apart.
__device__ __forceinline__ void mk_poll2_sum(MkCtx& c, const Tagged* p, int stride, int n, unsigned int tag, float& v0,
                                             float& v1) {
    const uint4 first = mk_poll16_sys(c, p, tag, 0);
    v0 = __uint_as_float(first.x);
    v1 = __uint_as_float(first.z);
    for (int r = 1; r < n; r++) {
        const uint4 w = mk_poll16_sys(c, p + (size_t)r * stride, tag, r);
        v0 += __uint_as_float(w.x);
        v1 += __uint_as_float(w.z);
    }
}

// ---------------------------------------------------------------------
// Fixed-point activations.  For int8 / 4-bit weights the dot products run on
// the integer tensor-core path without giving up fp32-class accuracy: every
// block of 32 consecutive activations is scaled by its own s = max|x| / 8355709
// and rounded to a 24-bit integer T = a2*65536 + a1*256 + a0 with three SIGNED
// byte digits (8355711 = 127*65536 + 127*256 + 127 is the largest such T).
// sum q_i x_i over the block is then s * (65536 dp(q,a2) + 256 dp(q,a1) + dp(q,a0))
// with exact integer dot products; the representation error is at most 2^-23
// of the block's largest element per term.
//
// Shared-memory layout (at xs), chosen so that the B operand of the MMA is one
// 8-byte load per lane: 96 bytes per block, plane 0 | plane 1 | plane 2, and inside a
// 32-byte plane element e = 16h + 4t + b sits at byte 8t + 4h + b (lane t of an MMA quad
// reads its two k-quads, columns 4t.. and 16+4t.., as one 8-byte word).  After the planes
// (one spare block, so that a tile of two blocks may begin at the last block of an odd
// count): one float2 {s, -8 s sum(T)} per block (the second half only for 4-bit weights:
// their stored nibbles carry a +8 offset).
// ---------------------------------------------------------------------
__host__ __device__ inline int xq_plane_bytes(int K) { return ((K >> 5) + 1) * 96; }
// Bytes of the staged-activation buffer a phase with input width K needs.
__host__ __device__ inline int xs_bytes_of(int fmt, int K) {
    return fmt == FMT_F16 ? K * 4 : xq_plane_bytes(K) + ((K >> 5) + 2) * 8;
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
// Sum over the consumer threads (deterministic order); includes one consumer barrier.
__device__ __forceinline__ float mk_block_sum(MkCtx& c, float v) {
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    if (lane == 0) c.red()[48 + w] = v;
    consumer_sync();
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < MK_NW; i++) t += c.red()[48 + i];
    return t;
}

// ---------------------------------------------------------------------
// Producer warp: stream this CTA's tape through the ring.
// ---------------------------------------------------------------------
// Whole rounds of `step` tiles that fit a ring entry of tpe tiles (at least one).  Used by the
// producer and the consumers alike.
__device__ __forceinline__ int rounds_per_entry(int tpe, int step) {
    return max(1, __float2int_rz(__fdividef((float)tpe + 0.5f, (float)step)));
}

__device__ __forceinline__ void mk_produce_entry(MkCtx& c, const MegaArgs& a, const uint8_t*& src, uint32_t bytes, int p) {
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

// The entries of one phase, in the consumers' order (see mk_run_phase).
__device__ __forceinline__ void mk_produce_phase(MkCtx& c, const MegaArgs& a, const uint8_t* src, int p, int nrg) {
    const PhaseGeom g = a.geom[p];
    const int rem = g.nkt - g.nfull * g.S;
    for (int rg0 = 0; rg0 < nrg; rg0 += g.RS) {
        const int nrs = min(g.RS, nrg - rg0);
        const int step = nrs * g.S;
        const int R = rounds_per_entry(g.tpe, step);
        for (int r0 = 0; r0 < g.nfull; r0 += R)
            mk_produce_entry(c, a, src, (uint32_t)(min(R, g.nfull - r0) * step * g.tile_bytes), p);
        if (rem) mk_produce_entry(c, a, src, (uint32_t)(nrs * rem * g.tile_bytes), p);
        if (*c.abort_flag()) return;
    }
}

// Fused down projection: the tiles lie row-group by row-group (nkt tiles each); an entry holds whole
// sets of MK_NW row-groups, one per consumer warp (see mk_down_fused).
__device__ __forceinline__ void mk_produce_down_fused(MkCtx& c, const MegaArgs& a, const uint8_t* src, int nrg) {
    const PhaseGeom g = a.geom[PH_DOWN];
    const int per_entry = (g.tpe / (MK_NW * g.nkt)) * MK_NW;        // row-groups per entry
    for (int rg0 = 0; rg0 < nrg; rg0 += per_entry) {
        mk_produce_entry(c, a, src, (uint32_t)(min(per_entry, nrg - rg0) * g.nkt * g.tile_bytes), PH_DOWN);
        if (*c.abort_flag()) return;
    }
}

__device__ __forceinline__ void mk_producer(MkCtx& c, const MegaArgs& a) {
    if ((threadIdx.x & 31) != 0) return;
    const unsigned long long* off = a.tape_off + (size_t)blockIdx.x * (a.n_layers * 4 + 2);
    for (int step = 0; step < a.n_steps; step++) {
        for (int l = a.ls; l < a.le; l++)
            for (int p = 0; p < 4; p++) {
                if (p == PH_DOWN && a.ffn_fused) mk_produce_down_fused(c, a, a.tape + off[l * 4 + p], c.phase_tab()[8 + p]);
                else mk_produce_phase(c, a, a.tape + off[l * 4 + p], p, c.phase_tab()[8 + p]);
            }
        if (a.le >= a.n_layers && a.head)
            mk_produce_phase(c, a, a.tape + off[a.n_layers * 4], PH_HEAD, c.phase_tab()[8 + PH_HEAD]);
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
// Fused epilogue of one work item.
//   QKV      : the two rows of a RoPE pair  -> bias, rotate -> tagged q / fp16-rounded tagged k,v
//   gate/up  : gate row j and up row j      -> silu(g) * u -> tagged
//   wo, down : one output row               -> hs[r] + dot -> tagged
//   lm_head  : one vocab row                -> logits (optional) + running argmax
// `item` is the index among this rank's items of the phase.
// ---------------------------------------------------------------------
template <bool TP>
__device__ __forceinline__ void mk_epilogue(const MegaArgs& a, MkCtx& c, int p, int layer, unsigned int tag, int item,
                                            float v0, float v1, unsigned long long& best) {
    {   // self-check: every index an epilogue writes through must lie inside its vector
        const int lim = p == PH_QKV ? (a.q_dim + 2 * a.kv_dim) / 2 : p == PH_GU ? a.ffn_dim : p == PH_HEAD ? a.vocab : a.dim;
        if (item < 0 || item >= lim) { mk_fail(c, MK_ERR_RANGE, 1000 * p + 100000); return; }
    }
    if (p == PH_QKV) {
        // same mapping as qkv_pair(), with the divisions by head_dim/2 done as shifts
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
        st_tagged(a.xmid + item, v0 * (1.0f / (1.0f + expf(-v0))) * v1, tag);
    } else if (p == PH_HEAD) {
        if (a.head == 2) a.logits[item] = v0;
        const unsigned long long key = pack_best(v0, (unsigned)(item + a.vocab_base));
        if (key > best) best = key;
    } else {
        // the residual is read before the result is published: the next phase's staging overwrites
        // hs[item] only after it has seen this very word
        const float res = c.hs()[item];
        if (!TP) {
            st_tagged((p == PH_WO ? a.xhm : a.xh) + item, res + v0, tag);
        } else {
            // partial sum over this rank's heads / FFN features: into row tp_rank of every rank's receive
            // buffer; rank 0's row carries the residual
            const float w0 = (a.tp_rank == 0 ? res : 0.f) + v0;
            Tagged* const* peers = p == PH_WO ? a.xhm_peer : a.xh_peer;
            for (int q = 0; q < a.tp_n; q++) st_tagged_sys(peers[q] + (size_t)a.tp_rank * a.dim + item, w0, tag);
        }
    }
}

// ---------------------------------------------------------------------
// Tile arithmetic.  Lane (g = lane >> 2, t = lane & 3) of a warp ends up with the partial sums of
// row-slots g (acc0) and g + 8 (acc1).  Shared memory is addressed with 32-bit shared-space
// addresses throughout, so that the address arithmetic of the inner loop stays in 32 bits.
// ---------------------------------------------------------------------
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ float4 lds128f(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ float2 lds64f(uint32_t addr) {
    float2 v;
    asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr));
    return v;
}

// D (16x8, int32) = A (16x32 signed bytes, row) x B (32x8 signed bytes, col)
__device__ __forceinline__ void mma_s8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint2 b) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b.x), "r"(b.y), "r"(0));
}
// same with unsigned A bytes (4-bit weights unpacked to 0..15)
__device__ __forceinline__ void mma_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint2 b) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b.x), "r"(b.y), "r"(0));
}

// Per-lane constants of a phase (shared-space addresses).
//   B columns: tall tiles put digit plane n/2 in column n (even n < 6); wide tiles put plane n/2 of
//   the even block in even columns and of the odd block in odd columns.  Lane (g, t) supplies column
//   g and receives columns 2t and 2t + 1, i.e. digit plane t.
struct LaneGeom {
    uint32_t a_off;     // this lane's offset inside a tile's A bytes
    uint32_t d_off;     // offset of its pair of block scales inside the tile
    uint32_t b_addr;    // its B word in block 0 (fp16 weights: its float4 of x in block 0)
    uint32_t s_addr;    // float2 {s, -8 s sum T} of block 0
    bool bvalid;        // lane supplies a plane column (others supply zeros)
    int t;
};

template <int FMT>
__device__ __forceinline__ LaneGeom lane_geom(const MkCtx& c, int lane, int wide, int K) {
    LaneGeom L;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t xs = smem_u32(mk_smem) + c.xs_off;
    L.t = t;
    if (FMT == FMT_F16) {
        L.a_off = lane * 16; L.d_off = 0; L.b_addr = xs + t * 16; L.s_addr = 0; L.bvalid = true;
    } else {
        L.a_off = FMT == FMT_Q8_0 ? lane * 16 : lane * 8;
        L.d_off = (FMT == FMT_Q8_0 ? 512 : 256) + g * 4;
        L.bvalid = g < 6 && (wide || (g & 1) == 0);
        L.b_addr = xs + (g >> 1) * 32 + (wide ? (g & 1) * 96 : 0) + t * 8;
        L.s_addr = xs + xq_plane_bytes(K);
    }
    return L;
}

// One tile: `tile` = its ring address, bp = this lane's B word of the tile's (first) block, sp = the
// block's scale pair.  Per tile a lane issues four shared-memory loads, the MMA, two conversions of
// each kind and four multiply-adds; all addresses are kept as running pointers by the caller.
template <int FMT, bool WIDE>
__device__ __forceinline__ void tile_mac(uint32_t tile, uint32_t bp, uint32_t sp, const LaneGeom& L, float& acc0, float& acc1) {
    if (FMT == FMT_F16) {
        // 16 row-slots x 16 columns of halves: lane (g, t) holds columns 4t..4t+3 of slots g and g + 8
        const uint4 A = lds128(tile + L.a_off);
        const float4 xe = lds128f(bp);
        const float4 xo = WIDE ? lds128f(bp + 64) : xe;
        const float2 a0 = __half22float2(*reinterpret_cast<const __half2*>(&A.x));
        const float2 a1 = __half22float2(*reinterpret_cast<const __half2*>(&A.y));
        const float2 b0 = __half22float2(*reinterpret_cast<const __half2*>(&A.z));
        const float2 b1 = __half22float2(*reinterpret_cast<const __half2*>(&A.w));
        acc0 = fmaf(a0.x, xe.x, acc0); acc0 = fmaf(a0.y, xe.y, acc0);
        acc0 = fmaf(a1.x, xe.z, acc0); acc0 = fmaf(a1.y, xe.w, acc0);
        acc1 = fmaf(b0.x, xo.x, acc1); acc1 = fmaf(b0.y, xo.y, acc1);
        acc1 = fmaf(b1.x, xo.z, acc1); acc1 = fmaf(b1.y, xo.w, acc1);
        return;
    }
    uint2 B = make_uint2(0u, 0u);
    if (L.bvalid) B = lds64(bp);
    float4 sc;                                                // {s, off} of the even block, {s, off} of the odd one
    if (WIDE) sc = lds128f(sp);
    else { const float2 s1 = lds64f(sp); sc = make_float4(s1.x, s1.y, s1.x, s1.y); }
    const uint32_t dd = lds32(tile + L.d_off);
    int d[4];
    if (FMT == FMT_Q8_0) {
        const uint4 A = lds128(tile + L.a_off);
        mma_s8s8(d, A.x, A.y, A.z, A.w, B);
    } else {
        // 16 nibble bytes per block: byte 4t+b = element 4t+b (low) and 16+4t+b (high)
        const uint2 A = lds64(tile + L.a_off);
        mma_u8s8(d, A.x & 0x0f0f0f0fu, A.y & 0x0f0f0f0fu, (A.x >> 4) & 0x0f0f0f0fu, (A.y >> 4) & 0x0f0f0f0fu, B);
    }
    const float2 df = __half22float2(*reinterpret_cast<const __half2*>(&dd));    // scales of slots g, g + 8
    // int -> float without the (slow) conversion pipe: |sum| <= 32 * 128 * 127 < 2^22, so adding the integer to
    // the bit pattern of 1.5 * 2^23 and subtracting that constant is exact
    const float c0 = __int_as_float(d[0] + 0x4B400000) - 12582912.0f;
    const float c1 = __int_as_float((WIDE ? d[3] : d[2]) + 0x4B400000) - 12582912.0f;
    if (FMT == FMT_Q8_0) {
        acc0 = fmaf(df.x * sc.x, c0, acc0);
        acc1 = fmaf(df.y * sc.z, c1, acc1);
    } else {
        // sum (nib - 8) x = sum nib x - 8 sum x; the correction rides in the lanes of plane 0
        const float oe = L.t == 0 ? sc.y : 0.f, oo = L.t == 0 ? sc.w : 0.f;
        acc0 = fmaf(df.x, fmaf(sc.x, c0, oe), acc0);
        acc1 = fmaf(df.y, fmaf(sc.z, c1, oo), acc1);
    }
}

// A wide tile whose input side (B words / fp16 weights: x values, and the scale pairs) is already in
// registers: the same columns serve every row-group, so a warp that walks down the rows loads them once.
struct TileIn {
    uint2 B;
    float4 sc;          // {s, off} of the even block, {s, off} of the odd one
    float4 xe, xo;      // fp16 weights: this lane's four x values of the even / odd block
};
template <int FMT>
__device__ __forceinline__ TileIn tile_in(uint32_t bp, uint32_t sp, const LaneGeom& L) {
    TileIn in;
    in.B = make_uint2(0u, 0u);
    in.sc = make_float4(0.f, 0.f, 0.f, 0.f);
    in.xe = in.xo = in.sc;
    if (FMT == FMT_F16) { in.xe = lds128f(bp); in.xo = lds128f(bp + 64); }
    else {
        if (L.bvalid) in.B = lds64(bp);
        in.sc = lds128f(sp);
    }
    return in;
}
template <int FMT>
__device__ __forceinline__ void tile_mac_in(uint32_t tile, const TileIn& in, const LaneGeom& L, float& acc0, float& acc1) {
    if (FMT == FMT_F16) {
        const uint4 A = lds128(tile + L.a_off);
        const float2 a0 = __half22float2(*reinterpret_cast<const __half2*>(&A.x));
        const float2 a1 = __half22float2(*reinterpret_cast<const __half2*>(&A.y));
        const float2 b0 = __half22float2(*reinterpret_cast<const __half2*>(&A.z));
        const float2 b1 = __half22float2(*reinterpret_cast<const __half2*>(&A.w));
        acc0 = fmaf(a0.x, in.xe.x, acc0); acc0 = fmaf(a0.y, in.xe.y, acc0);
        acc0 = fmaf(a1.x, in.xe.z, acc0); acc0 = fmaf(a1.y, in.xe.w, acc0);
        acc1 = fmaf(b0.x, in.xo.x, acc1); acc1 = fmaf(b0.y, in.xo.y, acc1);
        acc1 = fmaf(b1.x, in.xo.z, acc1); acc1 = fmaf(b1.y, in.xo.w, acc1);
        return;
    }
    const uint32_t dd = lds32(tile + L.d_off);
    int d[4];
    if (FMT == FMT_Q8_0) {
        const uint4 A = lds128(tile + L.a_off);
        mma_s8s8(d, A.x, A.y, A.z, A.w, in.B);
    } else {
        const uint2 A = lds64(tile + L.a_off);
        mma_u8s8(d, A.x & 0x0f0f0f0fu, A.y & 0x0f0f0f0fu, (A.x >> 4) & 0x0f0f0f0fu, (A.y >> 4) & 0x0f0f0f0fu, in.B);
    }
    const float2 df = __half22float2(*reinterpret_cast<const __half2*>(&dd));
    const float c0 = __int_as_float(d[0] + 0x4B400000) - 12582912.0f;
    const float c1 = __int_as_float(d[3] + 0x4B400000) - 12582912.0f;
    if (FMT == FMT_Q8_0) {
        acc0 = fmaf(df.x * in.sc.x, c0, acc0);
        acc1 = fmaf(df.y * in.sc.z, c1, acc1);
    } else {
        const float oe = L.t == 0 ? in.sc.y : 0.f, oo = L.t == 0 ? in.sc.w : 0.f;
        acc0 = fmaf(df.x, fmaf(in.sc.x, c0, oe), acc0);
        acc1 = fmaf(df.y, fmaf(in.sc.z, c1, oo), acc1);
    }
}

// The tiles of one pass for this warp: ring entries in order, whole rounds per entry, then the
// incomplete last round.  Every warp observes and releases every entry, also those it has no tile
// in (a warp that skipped ahead could meet a slot whose barrier is a whole ring revolution behind
// and take the stale phase for its own).
#ifdef MK_PROBE_P
#define MK_SET_PROBE(B) c.probe_base = (MK_PROBE_P == 5 ? (B) : -1)
#define MK_ESTAMP(EV) do { if (a.trace && threadIdx.x == 0 && c.probe_base >= 0) a.trace[(size_t)blockIdx.x * MK_TRACE_EVENTS(a.n_layers) + c.probe_base + (EV)] = clock64(); } while (0)
#else
#define MK_SET_PROBE(B) do { } while (0)
#define MK_ESTAMP(EV) do { } while (0)
#endif
template <int FMT, bool WIDE>
__device__ __forceinline__ void mk_pass_tiles(const MegaArgs& a, MkCtx& c, const LaneGeom& L, bool act, int S, int kp, int nfull,
                                              int rem, int R, uint32_t woff, uint32_t wrem, uint32_t rstride, float& acc0,
                                              float& acc1) {
    const int lane = threadIdx.x & 31;
    const uint32_t sm0 = smem_u32(mk_smem);
    // running pointers of this warp's next tile: B word and scale pair advance S k-tiles per round
    constexpr uint32_t kBStep = FMT == FMT_F16 ? (WIDE ? 128u : 64u) : (WIDE ? 192u : 96u);
    constexpr uint32_t kSStep = WIDE ? 16u : 8u;
    uint32_t bp = L.b_addr + (uint32_t)kp * kBStep, sp = L.s_addr + (uint32_t)kp * kSStep;
    const uint32_t bstep = (uint32_t)S * kBStep, sstep = (uint32_t)S * kSStep;
    float acc2 = 0.f, acc3 = 0.f;
    for (int r0 = 0; r0 < nfull; r0 += R) {
        const int rounds = min(R, nfull - r0);
        mk_wait_bar(c, &c.full()[c.slot], c.par, MK_ERR_FULL);
        MK_ESTAMP(32 + 2 * (r0 / R));
        if (act) {
            uint32_t tile = sm0 + (uint32_t)c.slot * (uint32_t)a.slot_bytes + woff;
            int rr = 0;
            for (; rr + 2 <= rounds; rr += 2) {                // two independent tiles in flight
                tile_mac<FMT, WIDE>(tile, bp, sp, L, acc0, acc1);
                tile_mac<FMT, WIDE>(tile + rstride, bp + bstep, sp + sstep, L, acc2, acc3);
                tile += 2 * rstride; bp += 2 * bstep; sp += 2 * sstep;
            }
            if (rr < rounds) { tile_mac<FMT, WIDE>(tile, bp, sp, L, acc0, acc1); bp += bstep; sp += sstep; }
        }
        MK_ESTAMP(33 + 2 * (r0 / R));
        __syncwarp();
        if (lane == 0) mbar_arrive(&c.empty()[c.slot]);
        c.advance();
    }
    if (rem) {                                                 // the incomplete last round: an entry of its own
        mk_wait_bar(c, &c.full()[c.slot], c.par, MK_ERR_FULL);
        if (act && kp < rem) tile_mac<FMT, WIDE>(sm0 + (uint32_t)c.slot * (uint32_t)a.slot_bytes + wrem, bp, sp, L, acc2, acc3);
        __syncwarp();
        if (lane == 0) mbar_arrive(&c.empty()[c.slot]);
        c.advance();
    }
    acc0 += acc2; acc1 += acc3;
}

// ---------------------------------------------------------------------
// Staging of one pair of activations as fixed point (see "Fixed-point activations" above), with
// every address worked out by the caller: dst = plane-0 halfword of the pair, sc_addr = the
// block's float2.  All 32 lanes call; lanes 16j..16j+15 hold one block.  `lead`: first lane of a block.
// ---------------------------------------------------------------------
__device__ __forceinline__ void sts16(uint32_t addr, uint32_t v) {
    asm volatile("st.shared.u16 [%0], %1;" ::"r"(addr), "h"((unsigned short)v));
}
__device__ __forceinline__ void xq_store_fast(uint32_t dst, uint32_t sc_addr, bool ok, bool lead, float u0, float u1,
                                              bool want_sum) {
    float m = fmaxf(fabsf(u0), fabsf(u1));
    m = fmaxf(m, __shfl_xor_sync(MG_FULL_MASK, m, 1));
    m = fmaxf(m, __shfl_xor_sync(MG_FULL_MASK, m, 2));
    m = fmaxf(m, __shfl_xor_sync(MG_FULL_MASK, m, 4));
    m = fmaxf(m, __shfl_xor_sync(MG_FULL_MASK, m, 8));
    // an approximate reciprocal is enough: the value represented is T * (m / 8355709); the factor is two
    // below the largest three-digit T so that neither the reciprocal's nor the product's rounding can
    // carry |T| past 8355711
    float inv;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(inv) : "f"(m));
    inv = m > 1e-30f ? inv * 8355709.0f : 0.f;
    const int t0 = __float2int_rn(u0 * inv), t1 = __float2int_rn(u1 * inv);
    int ts = 0;
    if (want_sum) {
        ts = t0 + t1;
        ts += __shfl_xor_sync(MG_FULL_MASK, ts, 1);
        ts += __shfl_xor_sync(MG_FULL_MASK, ts, 2);
        ts += __shfl_xor_sync(MG_FULL_MASK, ts, 4);
        ts += __shfl_xor_sync(MG_FULL_MASK, ts, 8);
    }
    if (ok) {
        // signed digits a0 = byte 0 of T, a1 = byte 1 of T + 128, a2 = byte 2 of T + 128 + 32768
        sts16(dst, __byte_perm((unsigned)t0, (unsigned)t1, 0x0040));
        sts16(dst + 32, __byte_perm((unsigned)(t0 + 128), (unsigned)(t1 + 128), 0x0051));
        sts16(dst + 64, __byte_perm((unsigned)(t0 + 32896), (unsigned)(t1 + 32896), 0x0062));
        if (lead) {
            const float sc = m > 1e-30f ? m * (1.0f / 8355709.0f) : 0.f;
            asm volatile("st.shared.v2.f32 [%0], {%1,%2};" ::"r"(sc_addr), "f"(sc), "f"(-8.0f * sc * (float)ts));
        }
    }
}

// ---------------------------------------------------------------------
// Input staging.  A thread's share of the phase's input vector is the pairs of elements
// 2 tid + 960 k (k = 0, 1, ...: "strides").  NS strides are handled at a time, all of their loads
// in flight together, with straight-line code (NS is a compile-time constant chosen from the
// vector's length: the shuffles and conversions of the strides then overlap instead of queueing
// behind branches).
// ---------------------------------------------------------------------

// ---------------------------------------------------------------------
// Accumulator words.  Where many CTAs add partial sums into one vector they add 64-bit integers:
// bits 8..63 the value * 2^32, rounded (integer addition is associative, so the sum does not depend
// on the order in which the CTAs arrive and a decode step stays reproducible bit for bit), bits
// 0..7 a 1.  The low byte of a word therefore counts the additions it has received, and a reader
// that knows how many are due (MegaArgs::acc_n <= 255) sees data and completion in ONE 8-byte
// load, exactly as with the tagged exchange words: no counter, no fence, no second round trip.
// Range +-8.4e6, resolution 2.3e-10: far outside / below anything a hidden state holds.
// ---------------------------------------------------------------------
// v * 2^32 without the 64-bit conversion (a long instruction sequence): the integer part of
// v * 2^8 and the remainder * 2^24 are two 32-bit conversions.
__device__ __forceinline__ long long mk_contrib(float v) {
    const float x = v * 256.0f;
    const int hi = __float2int_rn(x);
    const int lo = __float2int_rn((x - (float)hi) * 16777216.0f);
    return ((long long)hi * 16777216ll + (long long)lo) * 256ll + 1ll;
}
__device__ __forceinline__ float mk_acc_value(unsigned int lo, unsigned int hi) {
    const long long w = (long long)(((unsigned long long)hi << 32) | (unsigned long long)lo);
    return __ll2float_rn(w >> 8) * (1.0f / 4294967296.0f);
}
__device__ __forceinline__ void red_add_s64(long long* p, long long v) {
    asm volatile("red.relaxed.gpu.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
// Re-read a pair of accumulator words (16-byte aligned) until both have received n additions.
__device__ __noinline__ uint4 mk_pollacc_slow(volatile int* abort_flag, MegaStatus* status, long long limit,
                                              const Tagged* p, unsigned int n) {
    uint4 r = make_uint4(0u, 0u, 0u, 0u);
    if (*abort_flag) return r;
    const long long t0 = global_ns();
    for (;;) {
        for (int i = 0; i < 64; i++) {
            r = ld_poll16(p);
            if ((r.x & 0xffu) == n && (r.z & 0xffu) == n) return r;
        }
        if (*abort_flag) return r;
        if (global_ns() - t0 > limit) { mk_fail_impl(abort_flag, status, MK_ERR_POLL, 900000 + (int)n); return r; }
    }
}

enum : int { SRC_POLL = 0, SRC_EMBED = 1, SRC_PLAIN = 2, SRC_ACC = 3 };
constexpr int MK_STRIDE = 2 * MK_CONSUMERS;

struct StageSrc {
    int kind;
    const Tagged* src;
    unsigned int tag;
    int n;
    const float* norm_w;
    int token;
};

// Profiling build only (-DMK_PROBE_P=<phase>): extra clock stamps of thread 0 inside that phase.
#ifdef MK_PROBE_P
#define MK_STAMP(EV) do { if (P == MK_PROBE_P && a.trace && threadIdx.x == 0) a.trace[(size_t)blockIdx.x * MK_TRACE_EVENTS(a.n_layers) + trace_base + (EV)] = clock64(); } while (0)
#else
#define MK_STAMP(EV) do { } while (0)
#endif

// The first token's hidden state does not come through an exchange buffer: embedding row or plain vector.
__device__ __noinline__ float2 mk_direct_pair(const MegaArgs& a, int kind, int token, int i) {
    if (kind == SRC_EMBED)
        return make_float2(embed_value(a.embed_w, a.head_fmt, a.dim, token, i), embed_value(a.embed_w, a.head_fmt, a.dim, token, i + 1));
    return make_float2(a.h_in[i], a.h_in[i + 1]);
}

template <int NS, bool NORMED, bool TP>
__device__ __forceinline__ void stage_issue(const MegaArgs& a, const StageSrc& s, int i0, uint4 (&r)[NS], float2 (&nw)[NS]) {
    const int tid = threadIdx.x;
#pragma unroll
    for (int k = 0; k < NS; k++) {
        const int i = i0 + k * MK_STRIDE + 2 * tid;
        r[k] = make_uint4(0u, s.tag, 0u, s.tag);
        nw[k] = make_float2(1.f, 1.f);
        if (i < s.n) {
            if (NORMED) nw[k] = *reinterpret_cast<const float2*>(s.norm_w + i);
            if (s.kind == SRC_POLL) {
                if (!TP || !NORMED) r[k] = ld_poll16(s.src + i);
            } else if (!TP && s.kind == SRC_ACC) {
                // two accumulator words; stage_finish re-reads them until their counts are complete
                r[k] = ld_poll16(s.src + i);
            } else {
                const float2 v = mk_direct_pair(a, s.kind, s.token, i);
                r[k].x = __float_as_uint(v.x); r[k].z = __float_as_uint(v.y);
            }
        }
    }
}

// Completes the loads of NS strides, stages them; ss accumulates the squares of a hidden state.
// st_dst / st_sc: staging addresses of this thread's stride-0 pair; stride number kk0 + k.
// Three straight passes - complete the polls (the only place with calls and branches), residual and
// norm weight, fixed point - so that the shuffle and conversion chains of the NS strides overlap.
template <int NS, int FMT, bool NORMED, bool TP>
__device__ __forceinline__ void stage_finish(const MegaArgs& a, MkCtx& c, const StageSrc& s, int i0, int kk0, uint4 (&r)[NS],
                                             float2 (&nw)[NS], uint32_t st_dst, uint32_t st_sc, float& ss) {
    const int tid = threadIdx.x;
    float v0[NS], v1[NS];
#pragma unroll
    for (int k = 0; k < NS; k++) {
        const int i = i0 + k * MK_STRIDE + 2 * tid;
        v0[k] = 0.f; v1[k] = 0.f;
        if (i < s.n) {
            if (TP && NORMED && s.kind == SRC_POLL) mk_poll2_sum(c, s.src + i, a.dim, a.tp_n, s.tag, v0[k], v1[k]);
            else if (!TP && s.kind == SRC_ACC) {
                if ((r[k].x & 0xffu) != s.tag || (r[k].z & 0xffu) != s.tag)
                    r[k] = mk_pollacc_slow(c.abort_flag(), c.status(), a.wait_cycles, s.src + i, s.tag);
                v0[k] = mk_acc_value(r[k].x, r[k].y); v1[k] = mk_acc_value(r[k].z, r[k].w);
            }
            else { mk_poll2_finish(c, s.src + i, s.tag, r[k]); v0[k] = __uint_as_float(r[k].x); v1[k] = __uint_as_float(r[k].z); }
        }
    }
#pragma unroll
    for (int k = 0; k < NS; k++) {
        const int i = i0 + k * MK_STRIDE + 2 * tid;
        if (NORMED) {
            if (i < s.n) *reinterpret_cast<float2*>(c.hs() + i) = make_float2(v0[k], v1[k]);
            ss = fmaf(v0[k], v0[k], ss);
            ss = fmaf(v1[k], v1[k], ss);
            v0[k] *= nw[k].x; v1[k] *= nw[k].y;
        }
        if (FMT == FMT_F16 && i < s.n) *reinterpret_cast<float2*>(c.xs() + i) = make_float2(v0[k], v1[k]);
    }
    if (FMT != FMT_F16) {
#pragma unroll
        for (int k = 0; k < NS; k++) {
            const int i = i0 + k * MK_STRIDE + 2 * tid;
            xq_store_fast(st_dst + 2880u * (kk0 + k), st_sc + 240u * (kk0 + k), i < s.n, (tid & 15) == 0, v0[k], v1[k], FMT == FMT_Q4_0);
        }
    }
}

// ---------------------------------------------------------------------
// One phase of a layer (or lm_head) on the consumer warps, P and the weight format fixed at
// compile time.  What bounds a phase is the chain of dependent instructions between "the input
// has arrived" and "the output is on its way", so the order of the work is:
//   1. everything that does not depend on the input: the warp's tiles and addresses, the epilogue
//      thread's row indices, residuals, biases and output pointers (this runs while the exchange
//      words of the previous phase are still on their way);
//   2. the input vector is polled and staged in xs; barrier;
//   3. every warp multiplies its tiles and leaves the sums of its 16 row-slots in part[]:
//      [row-group][slot][K-split], the splits of a slot padded with zeros to a multiple of four; barrier;
//   4. one thread per row-slot adds the slot's splits (float4 loads, fixed order), meets the other
//      block's sum (wide tiles) and its partner row (row pairs) by shuffle, and runs the fused epilogue:
//        QKV      : the two rows of a RoPE pair  -> bias, rotate -> tagged q / fp16-rounded tagged k,v
//        gate/up  : gate row j and up row j      -> silu(g) * u -> tagged
//        wo, down : one output row               -> residual + dot -> tagged
//        lm_head  : one vocab row                -> logits (optional) + running argmax
// With a hidden state as input (QKV, gate/up, lm_head) the raw values are kept in hs (the residual),
// the staged values are value * norm weight, and the RMSNorm factor 1/sqrt(mean(h^2) + eps) is
// applied in the epilogue; the warps' sums of squares travel through red[] (alternating halves).
//
// Ring entries of a phase (producer and consumers agree): a PASS is RS row-groups at a time; within
// a pass the tiles come in ROUNDS of (row-groups of the pass) x S tiles, one per working warp;
// an entry holds as many whole rounds as fit a slot, and the last, incomplete round of a pass
// (nkt not a multiple of S) travels in an entry of its own.  So a warp's tiles sit at fixed
// offsets in every entry and the inner loop has no address arithmetic beyond an increment.
// ---------------------------------------------------------------------
template <int P, int FMT, bool TP>
__device__ __forceinline__ void mk_run_phase(const MegaArgs& a, MkCtx& c, const StageSrc& s, int layer, unsigned int tag_out,
                                             int trace_base, unsigned long long& best) {
    constexpr bool kNormed = (P == PH_QKV || P == PH_GU || P == PH_HEAD);
    constexpr bool kPairs = (P == PH_QKV || P == PH_GU);
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    const uint32_t sm0 = smem_u32(mk_smem);

    // ---- 1. set-up that does not depend on the input ----
    const PhaseGeom& g = a.geom[P];
    const int ub = c.phase_tab()[P], nrg = c.phase_tab()[8 + P];
    const int S = g.S, RS = g.RS, nkt = g.nkt, wide = g.wide, tile_bytes = g.tile_bytes;
    const unsigned int rk = c.warp_tab()[P * 16 + w];
    const int rs = rk & 0xff, kp = rk >> 8;                  // rs = 255: this warp has no tiles in the phase
    const LaneGeom L = lane_geom<FMT>(c, lane, wide, g.K);
    const float wt = FMT == FMT_F16 ? 1.0f : L.t == 0 ? 1.0f : L.t == 1 ? 256.0f : L.t == 2 ? 65536.0f : 0.0f;
    const int sp = S == 1 ? 1 : (S + 3) & ~3;                // splits per slot as stored
    const uint32_t part_s = sm0 + c.part_off;
    const int lim = P == PH_QKV ? (a.q_dim + 2 * a.kv_dim) / 2 : P == PH_GU ? a.ffn_dim : P == PH_HEAD ? a.vocab : a.dim;
    // staging addresses of this thread's first pair (element 2 tid); stride k adds 30 blocks
    const uint32_t st_dst = sm0 + c.xs_off + (uint32_t)((tid >> 4) * 96 + ((tid & 7) >> 1) * 8 + ((tid >> 3) & 1) * 4 + (tid & 1) * 2);
    const uint32_t st_sc = sm0 + c.xs_off + (uint32_t)xq_plane_bytes(s.n) + (uint32_t)(tid >> 4) * 8u;
    // epilogue of the (single) row-slot this thread finishes, for the phases that fit one round
    const int nslots = nrg * 16;
    const int e_s = tid & 15;
    const int e_item = ((ub + (tid >> 4)) << g.ipg_shift) + e_s;
    const bool e_act = tid < nslots && e_s < (1 << g.ipg_shift) && e_item < lim;
    const uint32_t e_pr = part_s + (uint32_t)tid * (uint32_t)sp * 4u;
    float e_res = 0.f, e_b0 = 0.f, e_b1 = 0.f;
    int e_m = 0, e_r0 = 0, e_r1 = 0;
    if (P == PH_QKV && e_act) {
        // same mapping as qkv_pair(), with the divisions by head_dim/2 done as shifts
        const int half = a.head_dim >> 1, hs1 = a.hd_shift - 1;
        const int nq = a.q_dim >> 1, nk = a.kv_dim >> 1;
        int i = e_item;
        if (i >= nq) { i -= nq; e_m = 1; }
        if (e_m == 1 && i >= nk) { i -= nk; e_m = 2; }
        if (e_m < 2) {
            const int head = i >> hs1, j = i - (head << hs1);
            e_r0 = (head << a.hd_shift) + j;
            e_r1 = e_r0 + half;
        } else {
            e_r0 = 2 * i;
            e_r1 = e_r0 + 1;
        }
        if (a.qkv_bias) {
            const float* bias = a.qkv_bias + (size_t)layer * (a.q_dim + 2 * a.kv_dim) +
                                (e_m == 0 ? 0 : e_m == 1 ? a.q_dim : a.q_dim + a.kv_dim);
            e_b0 = bias[e_r0];
            e_b1 = bias[e_r1];
        }
    }
    // the residual: hs was staged by this layer's QKV (for wo) / gate-up (for down) phase
    if ((P == PH_WO || P == PH_DOWN) && e_act) e_res = (!TP || a.tp_rank == 0) ? c.hs()[e_item] : 0.f;
    MK_STAMP(23);

    // ---- 2. poll and stage the input, barrier ----
    float ss = 0.f;
    if (FMT != FMT_F16 && ((s.n >> 5) & 1) && tid == 0)    // odd number of blocks: the unused half pair's scale must be finite
        *reinterpret_cast<float2*>(mk_smem + c.xs_off + xq_plane_bytes(s.n) + (s.n >> 5) * 8) = make_float2(0.f, 0.f);
    if (s.n <= MK_STRIDE) {
        uint4 r[1]; float2 nw[1];
        stage_issue<1, kNormed, TP>(a, s, 0, r, nw);
        stage_finish<1, FMT, kNormed, TP>(a, c, s, 0, 0, r, nw, st_dst, st_sc, ss);
    } else if (s.n <= 3 * MK_STRIDE) {
        uint4 r[3]; float2 nw[3];
        stage_issue<3, kNormed, TP>(a, s, 0, r, nw);
        stage_finish<3, FMT, kNormed, TP>(a, c, s, 0, 0, r, nw, st_dst, st_sc, ss);
    } else {
        uint4 r[6]; float2 nw[6];
        for (int i0 = 0, kk = 0; i0 < s.n; i0 += 6 * MK_STRIDE, kk += 6) {
            stage_issue<6, kNormed, TP>(a, s, i0, r, nw);
            stage_finish<6, FMT, kNormed, TP>(a, c, s, i0, kk, r, nw, st_dst, st_sc, ss);
        }
    }
    float e_cs = 1.f, e_sn = 0.f;
    if (kNormed) {
        ss = warp_sum(ss);
        c.redsel ^= 16;
        if (lane == 0) c.red()[c.redsel + w] = ss;
    }
    MK_STAMP(25);
    consumer_sync();                           // xs, hs and the sums of squares are published
    mk_trace(a, 0, trace_base + 2 * (P == PH_HEAD ? 0 : P));
    if (P == PH_HEAD && blockIdx.x == 0 && a.h_out)          // the hidden state that entered lm_head (ExportHidden)
        for (int i = tid; i < a.dim; i += MK_CONSUMERS) a.h_out[i] = c.hs()[i];
    if (P == PH_QKV && e_act && e_m < 2) {                   // (the step's RoPE row is published by this phase's barrier)
        const int j = e_r0 & (a.head_dim - 1);
        e_cs = c.rope()[j]; e_sn = c.rope()[(a.head_dim >> 1) + j];
    }
    // RMSNorm factor of the staged vector, for the epilogue: formed here, where its loads overlap the
    // first tile loads, instead of on the chain behind the phase's last barrier
    float scale = 1.0f;
    if (kNormed && (tid & ~31) < nslots) {
        // (16th entry of a half of red[]: always 0)
        const uint32_t rr = part_s + (uint32_t)(MK_PART_FLOATS + c.redsel) * 4u;
        const float4 r0 = lds128f(rr), r1 = lds128f(rr + 16), r2 = lds128f(rr + 32), r3 = lds128f(rr + 48);
        const float t = ((r0.x + r0.y) + (r0.z + r0.w)) + ((r1.x + r1.y) + (r1.z + r1.w)) +
                        (((r2.x + r2.y) + (r2.z + r2.w)) + ((r3.x + r3.y) + (r3.z + r3.w)));
        scale = rsqrtf(fmaf(t, a.inv_dim, a.eps));
    }
    MK_STAMP(26);

    // ---- 3. tiles ----
#ifdef MK_PROBE_P
    c.probe_base = P == MK_PROBE_P ? trace_base : -1;
#endif
    for (int rg0 = 0; rg0 < nrg; rg0 += RS) {
        const int nrs = min(RS, nrg - rg0);
        const int step = nrs * S;
        const int R = rounds_per_entry(g.tpe, step);
        const bool act = rs < nrs;
        const int rem = nkt - g.nfull * S;
        float acc0 = 0.f, acc1 = 0.f;
        if (wide) mk_pass_tiles<FMT, true>(a, c, L, act, S, kp, g.nfull, rem, R, (uint32_t)((rs * S + kp) * tile_bytes),
                                           (uint32_t)((rs * rem + kp) * tile_bytes), (uint32_t)(step * tile_bytes), acc0, acc1);
        else mk_pass_tiles<FMT, false>(a, c, L, act, S, kp, g.nfull, rem, R, (uint32_t)((rs * S + kp) * tile_bytes),
                                       (uint32_t)((rs * rem + kp) * tile_bytes), (uint32_t)(step * tile_bytes), acc0, acc1);
        MK_STAMP(27);
        if (act) {
            // quad sum: lanes t = 0..2 hold the three digit planes (fp16 weights: four column quarters)
            acc0 *= wt; acc1 *= wt;
            acc0 += __shfl_xor_sync(MG_FULL_MASK, acc0, 1); acc1 += __shfl_xor_sync(MG_FULL_MASK, acc1, 1);
            acc0 += __shfl_xor_sync(MG_FULL_MASK, acc0, 2); acc1 += __shfl_xor_sync(MG_FULL_MASK, acc1, 2);
            // lane t of a quad stores split kp + t: t = 0 the sum, the others the zero padding
            const int col = kp + L.t;
            if (L.t == 0 || (kp == S - 1 && col < sp)) {
                float* part = c.part() + ((rg0 + rs) * 16 + (lane >> 2)) * sp + col;
                part[0] = L.t == 0 ? acc0 : 0.f;
                part[8 * sp] = L.t == 0 ? acc1 : 0.f;        // slot g + 8
            }
        }
    }
    mk_trace(a, 0, trace_base + 11 + 3 * (P == PH_HEAD ? 0 : P));
    consumer_sync();                     // every warp is done with xs; the partial sums are published
    mk_trace(a, 0, trace_base + 12 + 3 * (P == PH_HEAD ? 0 : P));
    const bool to_mid = P == PH_GU && !TP && a.ffn_fused;      // gate/up feeding the down projection of this very CTA
    if (to_mid) {
        // the middle vector of this CTA's down projection: the elements it owns come from the epilogue
        // below, every other position of the window is zero (xs is free: the tiles are done)
        const int e0 = c.phase_tab()[5], lo = ub << g.ipg_shift, hi = min((ub + nrg) << g.ipg_shift, lim);
        float* mid = reinterpret_cast<float*>(mk_smem + c.xs_off + c.phase_tab()[6]);
        for (int j = tid; j < a.geom[PH_DOWN].K; j += MK_CONSUMERS)
            if (e0 + j < lo || e0 + j >= hi) mid[j] = 0.f;
    }

    // ---- 4. epilogue: whole warps (the shuffles need every lane) ----
    if ((tid & ~31) < nslots) {
        MK_STAMP(29);
        const int nq = sp >> 2;
        for (int sl = tid; sl < ((nslots + 31) & ~31); sl += MK_CONSUMERS) {
            float v = 0.f;
            if (sl < nslots) {
                const uint32_t pr = e_pr + (uint32_t)(sl - tid) * (uint32_t)sp * 4u;
                if (S == 1) v = __uint_as_float(lds32(pr));
                else {
                    // up to 16 splits, zero-padded to a multiple of four: all loads at once, the unused quads dropped
                    const float4 f0 = lds128f(pr), f1 = lds128f(pr + 16), f2 = lds128f(pr + 32), f3 = lds128f(pr + 48);
                    const float s0 = (f0.x + f0.y) + (f0.z + f0.w), s1 = (f1.x + f1.y) + (f1.z + f1.w);
                    const float s2 = (f2.x + f2.y) + (f2.z + f2.w), s3 = (f3.x + f3.y) + (f3.z + f3.w);
                    v = (s0 + (nq > 1 ? s1 : 0.f)) + ((nq > 2 ? s2 : 0.f) + (nq > 3 ? s3 : 0.f));
                }
            }
            if (wide) v += __shfl_xor_sync(MG_FULL_MASK, v, 8);               // the odd blocks' sum of the same row
            float v1 = 0.f;
            if (kPairs) v1 = __shfl_xor_sync(MG_FULL_MASK, v, wide ? 4 : 8) * scale;   // second row of a pair
            v *= scale;
            MK_STAMP(30);
            if (P == PH_HEAD) {
                const int item = ((ub + (sl >> 4)) << g.ipg_shift) + e_s;
                if (sl < nslots && e_s < (1 << g.ipg_shift) && item < lim) {
                    if (a.head == 2) a.logits[item] = v;
                    const unsigned long long key = pack_best(v, (unsigned)(item + a.vocab_base));
                    if (key > best) best = key;
                }
            } else if (e_act) {
                if (P == PH_QKV) {
                    float v0 = v + e_b0;
                    v1 += e_b1;
                    const float t0 = v0 * e_cs - v1 * e_sn, t1 = v0 * e_sn + v1 * e_cs;   // K, Q: rotate (V: cs = 1, sn = 0)
                    if (e_m == 0) {
                        st_tagged(a.xq + e_r0, t0, tag_out);
                        st_tagged(a.xq + e_r1, t1, tag_out);
                    } else {
                        // K (after RoPE) and V are stored in the cache as fp16: exchange the rounded values
                        Tagged* dst = a.xkv + (e_m == 1 ? 0 : a.kv_dim);
                        st_tagged(dst + e_r0, __half2float(__float2half_rn(t0)), tag_out);
                        st_tagged(dst + e_r1, __half2float(__float2half_rn(t1)), tag_out);
                    }
                } else if (P == PH_GU) {
                    const float m = v * __fdividef(1.0f, 1.0f + __expf(-v)) * v1;
                    if (to_mid) reinterpret_cast<float*>(mk_smem + c.xs_off + c.phase_tab()[6])[e_item - c.phase_tab()[5]] = m;
                    else st_tagged(a.xmid + e_item, m, tag_out);
                } else if (!TP) {
                    st_tagged((P == PH_WO ? a.xhm : a.xh) + e_item, e_res + v, tag_out);
                } else {
                    // partial sum over this rank's heads / FFN features: into row tp_rank of every rank's receive
                    // buffer; rank 0's row carries the residual
                    Tagged* const* peers = P == PH_WO ? a.xhm_peer : a.xh_peer;
                    for (int q = 0; q < a.tp_n; q++) st_tagged_sys(peers[q] + (size_t)a.tp_rank * a.dim + e_item, e_res + v, tag_out);
                }
            }
        }
    }
    mk_trace(a, 0, trace_base + 2 * (P == PH_HEAD ? 0 : P) + 1);
}

// Rows [lo, hi) of the hidden state this CTA looks after in the fused feed-forward block (residual,
// clearing).  The CTAs that run attention are left out where others exist: they are the critical path.
__device__ __forceinline__ void mk_row_share(const MegaArgs& a, int& lo, int& hi) {
    int b = (int)blockIdx.x - a.n_heads, nb = (int)gridDim.x - a.n_heads;
    if (nb <= 0) { b = blockIdx.x; nb = gridDim.x; }
    lo = hi = 0;
    if (b < 0) return;
    lo = unit_begin(a.dim, b, nb);
    hi = unit_begin(a.dim, b + 1, nb);
}

// ---------------------------------------------------------------------
// Down projection without an exchange of the middle vector (one GPU).
// A CTA's gate/up rows are a contiguous run of FFN features, so the silu(g) * u values it has just
// produced are exactly a window of the down projection's input.  Instead of publishing them and
// waiting for everybody else's, the CTA multiplies ITS window (2 nkt blocks of columns, all rows)
// and adds the partial sums of all rows into the layer's accumulator; the other CTAs do the same
// for their windows.  Every addition also bumps the count in the word's low byte (see "Accumulator
// words"), so the next consumer of the hidden state polls the words themselves until their counts
// are complete: one L2 round trip, and this CTA neither fences nor waits after its additions.
// Three accumulators rotate.  While layer q adds into buffer q % 3, the rows of buffer (q + 1) % 3
// are cleared (mk_clear_next, before the wo phase): it was last read while layer q - 1 was staged,
// and every CTA has passed that point, since this CTA has seen every word of layer q - 1 complete.
// The clearing threads fence after their stores and the CTA's additions of layer q are issued after
// a barrier behind that fence; a CTA that adds into the cleared buffer at layer q + 1 has seen those
// additions, so its own come later than the stores in real time.  The residual enters as one more
// addition per row, made by the CTA that also clears that row (mk_row_share).
//   Weights: wide tiles, row-group = 8 rows, nkt k-tiles = the window; warp w takes row-groups
//   w, w + 15, ..., four of them in flight; their sums leave the warp straight from registers in one
//   reduction instruction (lane t of a quad sends the row of row-group t).
// ---------------------------------------------------------------------
template <int FMT>
__device__ __forceinline__ void mk_down_fused(const MegaArgs& a, MkCtx& c, long long* acc_cur, int trace_base) {
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    const PhaseGeom& g = a.geom[PH_DOWN];
    const int nrg = c.phase_tab()[8 + PH_DOWN];
    const uint32_t sm0 = smem_u32(mk_smem);
#ifdef MK_PROBE_P
    c.probe_base = MK_PROBE_P == PH_DOWN ? trace_base : -1;
#endif
    MK_ESTAMP(23);
    // This CTA's share of the rows: the residual enters there.
    int lo, hi;
    mk_row_share(a, lo, hi);
    for (int i = lo + tid; i < hi; i += MK_CONSUMERS) red_add_s64(acc_cur + i, mk_contrib(c.hs()[i]));
    MK_ESTAMP(25);
    consumer_sync();                                  // the window of the middle vector is complete
    MK_ESTAMP(26);
    if (nrg > 0) {
        if (FMT != FMT_F16) {
            // fixed point: thread tid takes the pair (2 tid, 2 tid + 1) of the window; whole warps (a warp = two blocks)
            if (tid < (g.K >> 1)) {
                const float2 u = *reinterpret_cast<const float2*>(mk_smem + c.xs_off + c.phase_tab()[6] + 8 * tid);
                const uint32_t st_dst = sm0 + c.xs_off + (uint32_t)((tid >> 4) * 96 + ((tid & 7) >> 1) * 8 + ((tid >> 3) & 1) * 4 + (tid & 1) * 2);
                const uint32_t st_sc = sm0 + c.xs_off + (uint32_t)xq_plane_bytes(g.K) + (uint32_t)(tid >> 4) * 8u;
                xq_store_fast(st_dst, st_sc, true, (tid & 15) == 0, u.x, u.y, FMT == FMT_Q4_0);
            }
            consumer_sync();
        }
        mk_trace(a, 0, trace_base + 2 * PH_DOWN);
        const LaneGeom L = lane_geom<FMT>(c, lane, 1, g.K);
        const float wt = FMT == FMT_F16 ? 1.0f : L.t == 0 ? 1.0f : L.t == 1 ? 256.0f : L.t == 2 ? 65536.0f : 0.0f;
        constexpr uint32_t kBStep = FMT == FMT_F16 ? 128u : 192u, kSStep = 16u;
        const int nkt = g.nkt;
        const int per_entry = (g.tpe / (MK_NW * nkt)) * MK_NW;      // row-groups per ring entry
        const uint32_t rg_bytes = (uint32_t)(nkt * g.tile_bytes);
        const TileIn in0 = tile_in<FMT>(L.b_addr, L.s_addr, L);     // the whole window when it is one k-tile wide
        for (int rg0 = 0; rg0 < nrg; rg0 += per_entry) {
            const int n_here = min(per_entry, nrg - rg0);
            mk_wait_bar(c, &c.full()[c.slot], c.par, MK_ERR_FULL);
            MK_ESTAMP(32 + 2 * (rg0 / per_entry));
            const uint32_t base = sm0 + (uint32_t)c.slot * (uint32_t)a.slot_bytes;
            // this warp's row-groups of the entry: w, w + 15, ...; four of them in flight
            for (int j = w; j < n_here; j += 4 * MK_NW) {
                float s0[4], s1[4];
                bool ok[4];
#pragma unroll
                for (int u = 0; u < 4; u++) { s0[u] = 0.f; s1[u] = 0.f; ok[u] = j + u * MK_NW < n_here; }
                const uint32_t t0 = base + (uint32_t)j * rg_bytes;
                if (nkt == 1) {
#pragma unroll
                    for (int u = 0; u < 4; u++)
                        if (ok[u]) tile_mac_in<FMT>(t0 + (uint32_t)(u * MK_NW) * rg_bytes, in0, L, s0[u], s1[u]);
                } else {
                    for (int kt = 0; kt < nkt; kt++) {
                        const TileIn in = tile_in<FMT>(L.b_addr + kt * kBStep, L.s_addr + kt * kSStep, L);
#pragma unroll
                        for (int u = 0; u < 4; u++)
                            if (ok[u]) tile_mac_in<FMT>(t0 + (uint32_t)(u * MK_NW) * rg_bytes + (uint32_t)(kt * g.tile_bytes), in, L, s0[u], s1[u]);
                    }
                }
                // even block + odd block of the same row, then the quad's digit planes
                float v[4];
#pragma unroll
                for (int u = 0; u < 4; u++) v[u] = (s0[u] + s1[u]) * wt;
#pragma unroll
                for (int u = 0; u < 4; u++) v[u] += __shfl_xor_sync(MG_FULL_MASK, v[u], 1);
#pragma unroll
                for (int u = 0; u < 4; u++) v[u] += __shfl_xor_sync(MG_FULL_MASK, v[u], 2);
                // every lane of a quad now holds the four sums: lane t sends the one of row-group u = t, so the
                // four row-groups leave in one conversion and one reduction instruction
                const float mine = L.t == 0 ? v[0] : L.t == 1 ? v[1] : L.t == 2 ? v[2] : v[3];
                const bool okm = L.t == 0 ? ok[0] : L.t == 1 ? ok[1] : L.t == 2 ? ok[2] : ok[3];
                const int r = ((rg0 + j + L.t * MK_NW) << 3) + (lane >> 2);
                if (okm && r < a.dim) red_add_s64(acc_cur + r, mk_contrib(mine));
            }
            MK_ESTAMP(33 + 2 * (rg0 / per_entry));
            __syncwarp();
            if (lane == 0) mbar_arrive(&c.empty()[c.slot]);
            c.advance();
        }
    }
    mk_trace(a, 0, trace_base + 11 + 3 * PH_DOWN);
    consumer_sync();                                  // xs is free again for the next phase's staging
    mk_trace(a, 0, trace_base + 12 + 3 * PH_DOWN);
}

// Clear this CTA's rows of the accumulator the NEXT layer will add into: the same rows whose residual
// it adds in this layer, so that a complete word of this layer proves the clearing of that row done.
// Runs where the CTA would otherwise spin on the attention output; the fence keeps the clearing
// threads until their stores have been performed.
__device__ __forceinline__ void mk_clear_next(const MegaArgs& a, long long* acc_next) {
    int lo, hi;
    mk_row_share(a, lo, hi);
    const int tid = threadIdx.x;
    if (lo + tid < hi) {
        for (int i = lo + tid; i < hi; i += MK_CONSUMERS)
            asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(acc_next + i), "l"(0ll) : "memory");
        __threadfence();
    }
}

// ---------------------------------------------------------------------
// Attention for one query head on this CTA (fp16 KV cache), three barriers.
// Cached K/V rows do not depend on this token, so they are loaded into registers BEFORE q is
// waited for.
//   scores : four adjacent lanes share a position (a quarter of the head's dims each); unit
//            u = tid / 4 takes positions u, u + 120, ...; the first NPRE of them come from registers;
//   softmax: one maximum over the CTA; exp(s - max) is formed where it is used;
//   P . V  : warp w takes positions w, w + 15, ... (the first NV from registers), a lane HD / 32
//            adjacent dims; the warps' partial outputs and partial sums of exp meet in shared memory.
// ---------------------------------------------------------------------
template <int VPL>
__device__ __forceinline__ uint2 ldcg_v(const __half* p) {
    if (VPL == 1) return make_uint2(__ldcg(reinterpret_cast<const unsigned short*>(p)), 0u);
    if (VPL == 2) return make_uint2(__ldcg(reinterpret_cast<const unsigned int*>(p)), 0u);
    return __ldcg(reinterpret_cast<const uint2*>(p));
}
template <int VPL>
__device__ __forceinline__ void fma_v(float (&acc)[VPL], float p, uint2 v) {
    if (VPL == 1) {
        acc[0] = fmaf(p, __half2float(__ushort_as_half((unsigned short)v.x)), acc[0]);
    } else {
        const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&v.x));
        acc[0] = fmaf(p, f0.x, acc[0]); acc[1] = fmaf(p, f0.y, acc[1]);
        if (VPL == 4) {
            const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&v.y));
            acc[2] = fmaf(p, f1.x, acc[2]); acc[3] = fmaf(p, f1.y, acc[3]);
        }
    }
}
// dot of 8 fp16 K values with 8 floats of q in shared memory
__device__ __forceinline__ float dot8_kq(uint4 kk, uint32_t q_s) {
    const __half2* h = reinterpret_cast<const __half2*>(&kk);
    const float4 qa = lds128f(q_s), qb = lds128f(q_s + 16);
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
    constexpr int DPL = HD / 4;                // dims per lane in the score phase
    constexpr int KV4 = DPL / 8;               // 16-byte pieces of K per lane and position
    constexpr int NPRE = HD == 128 ? 2 : 4;    // score passes whose K rows are held in registers
    constexpr int PPP = 8;                     // positions per warp and pass (four lanes each)
    constexpr int VPL = HD / 32;               // dims per lane in P . V
    constexpr int NV = 16;                     // positions per warp whose V rows are held in registers
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    const int head = blockIdx.x;
    const int kvh = head / (a.n_heads / a.n_kv_heads);
    const size_t lbase = (size_t)layer * a.max_seq * a.kv_dim;
    __half* kc = a.kc + lbase + kvh * HD;
    __half* vc = a.vc + lbase + kvh * HD;
    const uint32_t xs_s = smem_u32(mk_smem) + c.xs_off;        // q | new k | new v, HD floats each
    const int uq = lane >> 2, qp = lane & 3;
    // Warp w owns positions w, w + 15, w + 30, ...: it computes their scores AND their share of
    // P . V, so the scores never leave the warp; pass i covers its positions number 8 i .. 8 i + 7.
    const int t_first = w + MK_NW * uq;

    // ---- cached rows (positions < pos) into registers ----
    // Everything below is guarded per warp (a warp's positions of a pass / of a group of four are
    // known from w and pos alone), so a short context skips the passes it does not have instead of
    // walking through their predicated-off loads.
    const int npass = (pos - w + MK_NW * PPP) / (MK_NW * PPP);      // score passes in which this warp has a position <= pos (w <= pos)
    const int nv = w < pos ? (pos - w + MK_NW - 1) / MK_NW : 0;     // cached positions of this warp for P . V
    uint4 kreg[NPRE][KV4];
#pragma unroll
    for (int i = 0; i < NPRE; i++) {
        const int t = t_first + i * (MK_NW * PPP);
#pragma unroll
        for (int j = 0; j < KV4; j++) kreg[i][j] = make_uint4(0u, 0u, 0u, 0u);
        if (w <= pos && i < npass && t < pos) {
            const uint4* kp = reinterpret_cast<const uint4*>(kc + (size_t)t * a.kv_dim + qp * DPL);
#pragma unroll
            for (int j = 0; j < KV4; j++) kreg[i][j] = __ldcg(kp + j);
        }
    }
    uint2 vreg[NV];
#pragma unroll
    for (int j0 = 0; j0 < NV; j0 += 4) {
#pragma unroll
        for (int j = j0; j < j0 + 4; j++) vreg[j] = make_uint2(0u, 0u);
        if (j0 < nv) {
#pragma unroll
            for (int j = j0; j < j0 + 4; j++) {
                const int t = w + j * MK_NW;
                if (t < pos) vreg[j] = ldcg_v<VPL>(vc + (size_t)t * a.kv_dim + lane * VPL);
            }
        }
    }
    MK_ESTAMP(40);

    // ---- gather q, new k, new v (HD values each); append the new row to the cache ----
    for (int i = 2 * tid; i < 3 * HD; i += 2 * MK_CONSUMERS) {
        const int which = i / HD, d = i - which * HD;
        const Tagged* src = which == 0 ? a.xq + head * HD + d
                          : which == 1 ? a.xkv + kvh * HD + d
                                       : a.xkv + a.kv_dim + kvh * HD + d;
        float v0, v1;
        mk_poll2(c, src, tag_in, v0, v1);
        *reinterpret_cast<float2*>(c.xs() + i) = make_float2(v0, v1);
        // every CTA of the KV group appends the (identical) new row; each CTA later reads back
        // only addresses it has written itself
        if (which == 1) *reinterpret_cast<__half2*>(kc + (size_t)pos * a.kv_dim + d) = __floats2half2_rn(v0, v1);
        if (which == 2) *reinterpret_cast<__half2*>(vc + (size_t)pos * a.kv_dim + d) = __floats2half2_rn(v0, v1);
    }
    consumer_sync();
    MK_ESTAMP(41);

    // ---- scores of this warp's positions ----
    const float scale = rsqrtf((float)HD);
    const uint32_t q_s = xs_s + (uint32_t)(qp * DPL) * 4u;
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < NPRE; i++) {
        if (i == 0 || (w <= pos && i < npass)) {                   // uniform over the warp
            const int t = t_first + i * (MK_NW * PPP);
            if (t == pos) {
                // the new position's K row sits in shared memory (fp16-rounded values: the conversion is exact)
                const float* kn = c.xs() + HD + qp * DPL;
#pragma unroll
                for (int j = 0; j < KV4; j++) {
                    __half2 h[4];
#pragma unroll
                    for (int e = 0; e < 4; e++) h[e] = __floats2half2_rn(kn[8 * j + 2 * e], kn[8 * j + 2 * e + 1]);
                    kreg[i][j] = *reinterpret_cast<const uint4*>(h);
                }
            }
            float dot = 0.f;
#pragma unroll
            for (int j = 0; j < KV4; j++) dot += dot8_kq(kreg[i][j], q_s + j * 32);
            dot += __shfl_xor_sync(MG_FULL_MASK, dot, 1);
            dot += __shfl_xor_sync(MG_FULL_MASK, dot, 2);
            dot *= scale;
            if (t <= pos) { if (qp == 0) c.sc()[t] = dot; mx = fmaxf(mx, dot); }
        }
    }
    for (int i = NPRE; w <= pos && i < npass; i++) {              // contexts beyond the registers: rows from L2
        const int t = t_first + i * (MK_NW * PPP);
        uint4 kk[KV4];
#pragma unroll
        for (int j = 0; j < KV4; j++) kk[j] = make_uint4(0u, 0u, 0u, 0u);
        if (t < pos) {
            const uint4* kp = reinterpret_cast<const uint4*>(kc + (size_t)t * a.kv_dim + qp * DPL);
#pragma unroll
            for (int j = 0; j < KV4; j++) kk[j] = __ldcg(kp + j);
        } else if (t == pos) {
            const float* kn = c.xs() + HD + qp * DPL;
#pragma unroll
            for (int j = 0; j < KV4; j++) {
                __half2 h[4];
#pragma unroll
                for (int e = 0; e < 4; e++) h[e] = __floats2half2_rn(kn[8 * j + 2 * e], kn[8 * j + 2 * e + 1]);
                kk[j] = *reinterpret_cast<const uint4*>(h);
            }
        }
        float dot = 0.f;
#pragma unroll
        for (int j = 0; j < KV4; j++) dot += dot8_kq(kk[j], q_s + j * 32);
        dot += __shfl_xor_sync(MG_FULL_MASK, dot, 1);
        dot += __shfl_xor_sync(MG_FULL_MASK, dot, 2);
        dot *= scale;
        if (t <= pos) { if (qp == 0) c.sc()[t] = dot; mx = fmaxf(mx, dot); }
    }
    mx = warp_max(mx);                       // -inf: the warp has no position
    __syncwarp();                            // the scores in sc[] were written by lanes of this warp
    MK_ESTAMP(42);
    MK_ESTAMP(43);

    // ---- this warp's share of P . V, relative to its own maximum ----
    float acc[VPL];
#pragma unroll
    for (int e = 0; e < VPL; e++) acc[e] = 0.f;
    float lsum = 0.f;
    const int last = max(pos - 1, 0);
#pragma unroll
    for (int j0 = 0; j0 < NV; j0 += 4) {
        if (j0 < nv) {
            // a group of four, straight-line: positions beyond the context contribute p = 0 (their V registers hold zeros)
#pragma unroll
            for (int j = j0; j < j0 + 4; j++) {
                const int t = w + j * MK_NW;
                float p = __expf(c.sc()[min(t, last)] - mx);
                p = t < pos ? p : 0.f;
                lsum += p;
                fma_v<VPL>(acc, p, vreg[j]);
            }
        }
    }
    for (int t0 = w + NV * MK_NW; t0 < pos; t0 += 4 * MK_NW) {   // remainder, four loads in flight
        uint2 vv[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int t = t0 + j * MK_NW;
            vv[j] = make_uint2(0u, 0u);
            if (t < pos) vv[j] = ldcg_v<VPL>(vc + (size_t)t * a.kv_dim + lane * VPL);
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int t = t0 + j * MK_NW;
            float p = __expf(c.sc()[min(t, last)] - mx);
            p = t < pos ? p : 0.f;
            lsum += p;
            fma_v<VPL>(acc, p, vv[j]);
        }
    }
    if (w == pos % MK_NW) {                                       // the new position belongs to one warp
        const float p = __expf(c.sc()[pos] - mx);
        lsum += p;
        const float* vn = c.xs() + 2 * HD + lane * VPL;
#pragma unroll
        for (int e = 0; e < VPL; e++) acc[e] = fmaf(p, vn[e], acc[e]);
    }
    MK_ESTAMP(44);
#pragma unroll
    for (int e = 0; e < VPL; e++) c.part()[w * HD + lane * VPL + e] = acc[e];
    if (lane == 0) { c.red()[32 + w] = mx; c.red()[48 + w] = lsum; }
    consumer_sync();
    MK_ESTAMP(45);
    // ---- merge the warps' partial results: weights exp(m_w - M) ----
    if (tid < HD) {
        const uint32_t rr = smem_u32(mk_smem) + c.part_off + (uint32_t)(MK_PART_FLOATS + 32) * 4u;
        float m[16], l[16];
#pragma unroll
        for (int q = 0; q < 4; q++) {
            const float4 mm = lds128f(rr + 16 * q), ll = lds128f(rr + 64 + 16 * q);
            m[4 * q] = mm.x; m[4 * q + 1] = mm.y; m[4 * q + 2] = mm.z; m[4 * q + 3] = mm.w;
            l[4 * q] = ll.x; l[4 * q + 1] = ll.y; l[4 * q + 2] = ll.z; l[4 * q + 3] = ll.w;
        }
        float M = m[0];
#pragma unroll
        for (int g = 1; g < MK_NW; g++) M = fmaxf(M, m[g]);
        float s = 0.f, lt = 0.f;
#pragma unroll
        for (int g = 0; g < MK_NW; g++) {
            const float f = __expf(m[g] - M);                  // 0 for a warp without positions (m = -inf)
            s = fmaf(f, c.part()[g * HD + tid], s);
            lt = fmaf(f, l[g], lt);
        }
        st_tagged(a.xattn + head * HD + tid, __fdividef(s, lt), tag_out);
    }
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
    const bool fused = !TP && a.ffn_fused;
    int qn = 0;                              // layers finished in this launch

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

        // tags of layer l: +1 q/kv, +2 attn, +3 h after wo, +4 ffn mid, +5 h after down
        // (fused feed-forward block: no +4 / +5; the hidden state after the block is accumulator
        //  (acc_buf0 + qn) % 3, each word complete when its count reads acc_n)
#define MK_LAYER(FMT)                                                                                              \
        {                                                                                                          \
            StageSrc s0{SRC_POLL, a.xh, tag_prev_h, a.dim, a.norms + (size_t)l * 2 * a.dim, token};                \
            if (fused) {                                                                                           \
                s0.kind = SRC_ACC;                                                                                 \
                s0.src = reinterpret_cast<const Tagged*>(a.acc + (size_t)((a.acc_buf0 + qn + 2) % 3) * a.dim); \
                s0.tag = (unsigned)a.acc_n;                                                                        \
            }                                                                                                      \
            if (l == a.ls) s0.kind = a.embed ? SRC_EMBED : SRC_PLAIN;                                              \
            mk_run_phase<PH_QKV, FMT, TP>(a, c, s0, l, base + 1, l * MK_EV, best);                                 \
            if ((int)blockIdx.x < a.n_heads) {                                                                     \
                MK_SET_PROBE(l * MK_EV);                                                                           \
                if (a.head_dim == 64) mk_attention<64>(a, c, l, pos, base + 1, base + 2);                          \
                else if (a.head_dim == 128) mk_attention<128>(a, c, l, pos, base + 1, base + 2);                   \
                else mk_attention<32>(a, c, l, pos, base + 1, base + 2);                                           \
                mk_trace(a, step, l * MK_EV + 9);                                                                  \
            }                                                                                                      \
            if (fused) mk_clear_next(a, a.acc + (size_t)((a.acc_buf0 + qn + 1) % 3) * a.dim);                      \
            const StageSrc s1{SRC_POLL, a.xattn, base + 2, a.q_dim, nullptr, token};                               \
            mk_run_phase<PH_WO, FMT, TP>(a, c, s1, l, base + 3, l * MK_EV, best);                                  \
            const StageSrc s2{SRC_POLL, a.xhm, base + 3, a.dim, a.norms + (size_t)l * 2 * a.dim + a.dim, token};   \
            mk_run_phase<PH_GU, FMT, TP>(a, c, s2, l, base + 4, l * MK_EV, best);                                  \
            if (fused) {                                                                                           \
                mk_down_fused<FMT>(a, c, a.acc + (size_t)((a.acc_buf0 + qn) % 3) * a.dim, l * MK_EV);              \
                mk_trace(a, 0, l * MK_EV + 2 * PH_DOWN + 1);                                                       \
            } else {                                                                                               \
                const StageSrc s3{SRC_POLL, a.xmid, base + 4, a.ffn_dim, nullptr, token};                          \
                mk_run_phase<PH_DOWN, FMT, TP>(a, c, s3, l, base + 5, l * MK_EV, best);                            \
            }                                                                                                      \
            qn++;                                                                                                  \
        }
        for (int l = a.ls; l < a.le; l++) {
            const unsigned int base = ep + (unsigned)l * MK_EPOCHS_PER_LAYER;
            const unsigned int tag_prev_h = base - MK_EPOCHS_PER_LAYER + 5;
            mk_trace(a, step, l * MK_EV + 8);
            if (a.layer_fmt == FMT_Q8_0) MK_LAYER(FMT_Q8_0)
            else if (a.layer_fmt == FMT_Q4_0) MK_LAYER(FMT_Q4_0)
            else MK_LAYER(FMT_F16)
        }
#undef MK_LAYER
        if (do_head) {
            const unsigned int base = ep + (unsigned)L * MK_EPOCHS_PER_LAYER;
            StageSrc sh{SRC_POLL, a.xh, base - MK_EPOCHS_PER_LAYER + 5, a.dim, a.final_norm, token};
            if (fused) {
                sh.kind = SRC_ACC;
                sh.src = reinterpret_cast<const Tagged*>(a.acc + (size_t)((a.acc_buf0 + qn + 2) % 3) * a.dim);
                sh.tag = (unsigned)a.acc_n;
            }
            if (a.head_fmt == FMT_Q8_0) mk_run_phase<PH_HEAD, FMT_Q8_0, TP>(a, c, sh, L, base + 5, L * MK_EV, best);
            else if (a.head_fmt == FMT_Q4_0) mk_run_phase<PH_HEAD, FMT_Q4_0, TP>(a, c, sh, L, base + 5, L * MK_EV, best);
            else mk_run_phase<PH_HEAD, FMT_F16, TP>(a, c, sh, L, base + 5, L * MK_EV, best);
        }

        if (!do_head) {
            // partial layer range: CTA 0 hands the hidden state back
            if (blockIdx.x == 0 && a.h_out && step == a.n_steps - 1 && a.le > a.ls) {
                const unsigned int tag_final_h = ep + (unsigned)(a.le - 1) * MK_EPOCHS_PER_LAYER + 5;
                if (fused) {
                    const Tagged* src = reinterpret_cast<const Tagged*>(a.acc + (size_t)((a.acc_buf0 + qn + 2) % 3) * a.dim);
                    for (int i = 2 * tid; i < a.dim; i += 2 * MK_CONSUMERS) {
                        uint4 w = ld_poll16(src + i);
                        if ((w.x & 0xffu) != (unsigned)a.acc_n || (w.z & 0xffu) != (unsigned)a.acc_n)
                            w = mk_pollacc_slow(c.abort_flag(), c.status(), a.wait_cycles, src + i, (unsigned)a.acc_n);
                        c.hs()[i] = mk_acc_value(w.x, w.y);
                        c.hs()[i + 1] = mk_acc_value(w.z, w.w);
                    }
                } else if (!TP) {
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
            // (not in part[]: the threads that run lm_head's epilogue may still be reading it)
            unsigned long long* sb = reinterpret_cast<unsigned long long*>(c.red() + 32);
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
                            const uint4 w = mk_poll16_sys(c, a.xbest + 2 * r, tagx, r);
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
           2 * MK_MAX_SLOTS * 8 + 16 + 64 + 5 * 16 * 2 + 16;
}

// TP = false: one GPU (no peer pointers are touched); TP = true: one rank of a tensor-parallel group.
template <bool TP>
__global__ void __launch_bounds__(MK_THREADS, 1) mega_decode_kernel(const __grid_constant__ MegaArgs a) {
    MkCtx c(a);
    if (threadIdx.x == 0) {
        for (int i = 0; i < a.nslot; i++) {
            mbar_init(&c.full()[i], 1);
            mbar_init(&c.empty()[i], MK_NW);
        }
        *c.abort_flag() = 0;
        c.red()[15] = 0.f; c.red()[31] = 0.f;      // 16th entry of the two halves of the RMS partial sums
        for (int p = 0; p <= PH_HEAD; p++) {
            const PhaseShape sh = phase_shape_of(p, a.dim, a.q_dim, a.kv_dim, a.ffn_dim, a.vocab, a.layer_fmt, a.head_fmt);
            const int ipg = 1 << a.geom[p].ipg_shift;
            const int units = (sh.items + ipg - 1) >> a.geom[p].ipg_shift;
            const int off = p == PH_QKV ? a.qkv_cta0 : 0;
            const int me = (int)blockIdx.x - off, ng = (int)gridDim.x - off;
            const int ub = me < 0 ? 0 : unit_begin(units, me, ng);
            c.phase_tab()[p] = ub;
            c.phase_tab()[8 + p] = me < 0 ? 0 : unit_begin(units, me + 1, ng) - ub;
            for (int w = 0; w < 16; w++) {
                const int S = a.geom[p].S, rs = w / S;
                c.warp_tab()[p * 16 + w] = (unsigned short)(rs < a.geom[p].RS ? (rs | ((w - rs * S) << 8)) : 255);
            }
        }
        if (a.ffn_fused) {
            // down projection on this CTA's own window of the middle vector: all row-groups, or none
            const int kblk = kblock_of(a.layer_fmt);
            const int start = c.phase_tab()[PH_GU] << a.geom[PH_GU].ipg_shift;
            c.phase_tab()[PH_DOWN] = 0;
            c.phase_tab()[8 + PH_DOWN] = c.phase_tab()[8 + PH_GU] > 0 ? (a.dim + 7) >> 3 : 0;
            c.phase_tab()[5] = down_window_block(start, kblk, a.ffn_dim / kblk, a.geom[PH_DOWN].nkt) * kblk;
            c.phase_tab()[6] = a.layer_fmt == FMT_F16 ? 0 : (xs_bytes_of(a.layer_fmt, a.geom[PH_DOWN].K) + 15) & ~15;
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x >= MK_CONSUMERS) mk_producer(c, a);
    else mk_consumer<TP>(c, a);
}

}  // namespace mg

