// Host side of the mg_* decode engine: the counterpart of CUDAFusedInference
// (cuda_fused_infer.go:75-459) written in C++ over the fused sm_100a kernels.
//
// Memory layout in HBM, per weight matrix [rows x K] (K a multiple of 32):
//   qs plane : rows * row_bytes, rows contiguous and 16-byte aligned
//              Q8_0 -> K int8;  Q4_0 -> K/2 bytes, 16 per block in GGUF nibble
//              order;  F16 -> K halves
//   ds plane : rows * K/32 fp16 block scales (Q8_0, Q4_0)
// i.e. the 34/18-byte blocks are split into two streams at upload so that the
// quants can be read with aligned 16-byte loads.  KV caches are fp16
// [layers][max_seq][kv_dim]; activations fp32.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>

#include <algorithm>
#include <chrono>
#include <thread>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <map>
#include <type_traits>
#include <string>
#include <vector>

#include "../../include/mongoose_kernels.h"
#include "decode_kernels.cuh"
#include "mega_kernel.cuh"

using namespace mg;

namespace {

struct DevMatrix {
    uint8_t* qs = nullptr;
    unsigned short* ds = nullptr;
    int rows = 0, cols = 0, fmt = 0;
    bool set = false;
    WeightView view() const { return WeightView{qs, ds}; }
};

struct GraphKey {
    int ls, le, mode, head;
    bool operator<(const GraphKey& o) const {
        if (ls != o.ls) return ls < o.ls;
        if (le != o.le) return le < o.le;
        if (mode != o.mode) return mode < o.mode;
        return head < o.head;
    }
};

struct CachedGraph {
    cudaGraphExec_t exec = nullptr;
    int kernels = 0;
};

// The part of the model one tensor-parallel rank holds.  With size == 1 it is the whole model.
// Q heads [q0, q1) with the KV heads [kv0, kv1) that serve them, FFN features [f0, f1),
// vocabulary rows [v0, v1).
struct Shard {
    int rank = 0, size = 1;
    int q0 = 0, q1 = 0, kv0 = 0, kv1 = 0, f0 = 0, f1 = 0, v0 = 0, v1 = 0;
    int v_stride = 0;                   // rows per rank in the gathered logits (ceil(vocab / size))
};

// NCCL entry points, resolved from the already-loaded libnccl.so.2 when tensor parallelism is
// switched on; a single-GPU user never needs the library.
struct NcclApi {
    void* lib = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
};


// One device allocation per engine, carved at create time and sub-allocated best-fit in 256-byte
// units with coalescing frees: the counterpart of the reference's GPUArena (gpu_alloc.go:45-241).
// Requests the arena cannot serve fall through to cudaMalloc and are remembered as such.
struct Arena {
    uint8_t* base = nullptr;
    size_t size = 0;
    std::map<size_t, size_t> free_blocks;      // offset -> length
    std::map<size_t, size_t> used_blocks;      // offset -> length
    std::map<void*, size_t> outside;           // cudaMalloc'ed because the arena was full
    size_t peak = 0, in_use = 0;

    bool init(size_t bytes) {
        bytes = (bytes + 255) & ~(size_t)255;
        if (cudaMalloc((void**)&base, bytes) != cudaSuccess) { cudaGetLastError(); base = nullptr; return false; }
        size = bytes;
        free_blocks[0] = bytes;
        return true;
    }
    void destroy() {
        for (auto& kv : outside) cudaFree(kv.first);
        outside.clear();
        if (base) cudaFree(base);
        base = nullptr; size = 0; free_blocks.clear(); used_blocks.clear();
    }
    void* alloc(size_t bytes) {
        if (bytes == 0) bytes = 1;
        const size_t need = (bytes + 255) & ~(size_t)255;
        auto best = free_blocks.end();
        for (auto it = free_blocks.begin(); it != free_blocks.end(); ++it)
            if (it->second >= need && (best == free_blocks.end() || it->second < best->second)) best = it;
        if (best == free_blocks.end()) {
            void* p = nullptr;
            if (cudaMalloc(&p, bytes) != cudaSuccess) { cudaGetLastError(); return nullptr; }
            outside[p] = bytes;
            return p;
        }
        const size_t off = best->first, len = best->second;
        free_blocks.erase(best);
        if (len > need) free_blocks[off + need] = len - need;
        used_blocks[off] = need;
        in_use += need;
        peak = std::max(peak, in_use);
        return base + off;
    }
    void release(void* p) {
        if (!p) return;
        auto o = outside.find(p);
        if (o != outside.end()) { cudaFree(p); outside.erase(o); return; }
        const size_t off = (size_t)((uint8_t*)p - base);
        auto u = used_blocks.find(off);
        if (u == used_blocks.end()) return;            // not ours: ignore rather than corrupt the lists
        const size_t len = u->second;
        in_use -= len;
        used_blocks.erase(u);
        size_t start = off, total = len;
        auto next = free_blocks.lower_bound(off);          // first free block behind this one
        if (next != free_blocks.begin()) {
            auto prev = std::prev(next);
            if (prev->first + prev->second == off) { start = prev->first; total += prev->second; free_blocks.erase(prev); }
        }
        auto nx = free_blocks.find(off + len);
        if (nx != free_blocks.end()) { total += nx->second; free_blocks.erase(nx); }
        free_blocks[start] = total;
    }
    size_t largest_free() const {
        size_t m = 0;
        for (auto& kv : free_blocks) m = std::max(m, kv.second);
        return m;
    }
};

}  // namespace

struct mg_engine {
    mg_config cfg{};
    int num_sms = 148;
    cudaStream_t stream = nullptr;
    std::vector<DevMatrix> mats;        // indexed by weight slot
    std::vector<float*> vecs;           // norms / biases by slot
    float *cos_tab = nullptr, *sin_tab = nullptr;
    __half *kc = nullptr, *vc = nullptr;   // [layers][max_seq][kv_dim]
    float *h = nullptr, *h2 = nullptr, *q = nullptr, *attn = nullptr, *mid = nullptr, *logits = nullptr;
    StepState* st = nullptr;
    int* out_tokens = nullptr;
    int out_cap = 0;
    // pinned staging
    int* pin_i = nullptr;               // [0..3] cursor, [4..] prompt ids, then 16 ints for the kernels' status words
    int pin_i_cap = 0;
    float* logits_direct = nullptr;     // this launch writes its logits here (caller's pinned host buffer) instead of e->logits
    bool zero_copy = true;
    std::map<GraphKey, CachedGraph> graphs;
    // persistent-kernel path (mega_kernel.cuh)
    bool use_mega = true;               // allowed by the environment
    bool mega_ok = false;               // built and usable for this model
    uint8_t* tape = nullptr;
    unsigned long long* tape_off = nullptr;
    float* mk_norms = nullptr;          // [layers][2][dim] copy of the norm vectors
    float* mk_bias = nullptr;           // [layers][dim + 2 kv_dim] copy of the QKV biases, NULL if none is set
    Tagged* xbuf = nullptr;             // exchange buffers, one allocation
    MegaStatus* mk_status = nullptr;
    long long* mk_trace = nullptr;      // per-phase clock stamps of the next launch (mg_trace_step)
    bool trace_next = false;
    float* h_in = nullptr;              // hidden-state input of PartialStep on the persistent path
    unsigned int epoch = 16;
    int mk_nslot = 0, mk_slot = MK_SLOT, mk_xs = 0, mk_sc = 0;
    int mk_prefetch = 0;                // L2 prefetch distance of the tape, bytes
    long long mk_wait = MK_WAIT_CYCLES; // limit of every wait inside the persistent kernel, SM clocks
    // feed-forward block without a grid-wide exchange (one GPU): accumulators [3][dim], and the host's
    // mirror of which of them the next launch starts with
    bool ffn_fused = false;
    long long* mk_acc = nullptr;
    int mk_buf = 0;
    int mk_acc_n = 0;                   // additions that complete an accumulator word
    int mk_qkv_cta0 = 0;                // first CTA that owns QKV rows
    PhaseGeom mk_geom[5] = {};
    size_t mk_smem = 0;
    size_t tape_bytes = 0;
    bool built = false;
    bool use_graph = true;
    bool use_pdl = true;
    long long launches = 0;
    int capture_kernels = 0;            // kernels enqueued by the current enqueue_step
    size_t dev_bytes = 0;
    Arena arena;                        // every device buffer of this engine except the peer-mapped exchange buffer
    // layer-range pipeline (mg_set_layer_range, mg_queue_hidden_to, L3 bridge)
    int own_ls = 0, own_le = 0;         // layers this engine holds weights for; [0, n_layers) by default
    cudaEvent_t sent_event = nullptr;   // recorded after this engine's hidden state has been copied to the next stage
    cudaEvent_t mail_event = nullptr;   // this engine's own event: recorded behind the arrival of the hidden state last queued to it
    unsigned int mail_queued = 0, mail_taken = 0;
    float* l3 = nullptr;                // pinned host copy of the hidden state (the reference's "L3 bridge")
    cudaStream_t copy_stream = nullptr;
    cudaEvent_t compute_done = nullptr, l3_done = nullptr;
    bool l3_queued = false;
    // second compute stream of the reference's vNode scheme (SetVNodeCount(2), cuda_fused_infer.go:630-666)
    int vnodes = 1;
    cudaStream_t stream1 = nullptr;
    cudaEvent_t stage_done = nullptr, s1_in = nullptr, s1_out = nullptr;
    // tensor parallelism (mg_tp_init)
    Shard sh;
    ncclComm_t comm = nullptr;
    float* zero_vec = nullptr;          // residual input of the ranks other than 0 (the all-reduce adds rank 0's)
    float* logits_all = nullptr;        // gathered logits, [size][v_stride]
    bool any_weight_set = false;
    // exchange fused into the kernels: receive buffer of this rank, mapped into every peer
    bool tp_fused = false;
    bool absent_peers = false;          // test aid: a tensor-parallel rank whose peers do not exist (mg_tp_init_absent_peers)
    uint8_t* xchg = nullptr;            // [2 slots][size][dim] tagged words, then this rank's counters
    uint8_t* xchg_peer[kMaxRanks] = {}; // rank p's buffer as seen from here (own entry = xchg)
    XchgStatus* xchg_status = nullptr;
    std::string err;
};

namespace {

int fail(mg_engine* e, int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    if (e) e->err = buf;
    return code;
}

// allocation calls of this file in the shape of cudaMalloc / cudaFree, served by the engine's arena
#define ARENA_MALLOC(e, pp, bytes) ((*(pp) = static_cast<std::remove_reference<decltype(*(pp))>::type>((e)->arena.alloc(bytes))) ? cudaSuccess : cudaErrorMemoryAllocation)
#define ARENA_FREE(e, p) (e)->arena.release((void*)(p))

#define MG_CUDA(e, call)                                                                        \
    do {                                                                                        \
        cudaError_t _c = (call);                                                                \
        if (_c != cudaSuccess)                                                                  \
            return fail((e), MG_ERR_CUDA, "%s failed: %s (%s:%d)", #call, cudaGetErrorString(_c), \
                        __FILE__, __LINE__);                                                    \
    } while (0)

template <typename T>
int dev_alloc(mg_engine* e, T** p, size_t count) {
    void* v = e->arena.alloc(count * sizeof(T));
    if (!v) return fail(e, MG_ERR_NOMEM, "device allocation of %zu bytes failed (arena of %zu bytes, %zu in use)",
                        count * sizeof(T), e->arena.size, e->arena.in_use);
    e->dev_bytes += count * sizeof(T);
    *p = static_cast<T*>(v);
    return MG_OK;
}

bool slot_info(const mg_config& c, int idx, bool* is_matrix, int* rows, int* cols, int* fmt) {
    const int nL = c.n_layers;
    if (idx < 0 || idx >= nL * 12 + 2) return false;
    *is_matrix = false;
    *rows = 1;
    *cols = c.dim;
    *fmt = c.layer_fmt;
    if (idx == nL * 12) return true;
    if (idx == nL * 12 + 1) {
        *is_matrix = true; *rows = c.vocab; *cols = c.dim; *fmt = c.head_fmt;
        return true;
    }
    switch (idx % 12) {
        case 0: case 8: break;
        case 1: case 7: *is_matrix = true; *rows = c.dim; *cols = c.dim; break;
        case 2: case 3: *is_matrix = true; *rows = c.kv_dim; *cols = c.dim; break;
        case 4: *cols = c.dim; break;
        case 5: case 6: *cols = c.kv_dim; break;
        case 9: case 10: *is_matrix = true; *rows = c.ffn_dim; *cols = c.dim; break;
        case 11: *is_matrix = true; *rows = c.dim; *cols = c.ffn_dim; break;
    }
    return true;
}

// Tensor-parallel partition of one rank.  Q heads stay whole; when the ranks outnumber the KV
// heads, size / n_kv_heads consecutive ranks share one KV head (each keeps a copy of its K/V rows
// and cache) and split that head's Q group between them, earlier ranks taking the larger part.
// FFN features are split in multiples of 32 so that no quantization block straddles two ranks.
bool make_shard(const mg_config& c, int rank, int size, Shard* out, std::string* why) {
    Shard s;
    s.rank = rank; s.size = size;
    if (size < 1 || rank < 0 || rank >= size) { *why = "rank outside [0, size)"; return false; }
    const int group = c.n_heads / c.n_kv_heads;
    if (c.n_kv_heads % size == 0) {
        const int kvn = c.n_kv_heads / size;
        s.kv0 = rank * kvn; s.kv1 = s.kv0 + kvn;
        s.q0 = s.kv0 * group; s.q1 = s.kv1 * group;
    } else if (size % c.n_kv_heads == 0 && group >= size / c.n_kv_heads) {
        const int m = size / c.n_kv_heads, kv = rank / m, j = rank % m;
        const int base = group / m, extra = group % m;
        s.kv0 = kv; s.kv1 = kv + 1;
        s.q0 = kv * group + j * base + (j < extra ? j : extra);
        s.q1 = s.q0 + base + (j < extra ? 1 : 0);
    } else {
        *why = "the KV heads neither divide among the ranks nor are divided by them";
        return false;
    }
    const int fb = c.ffn_dim / 32;
    if (fb < size) { *why = "fewer FFN blocks than ranks"; return false; }
    const int fbase = fb / size, fextra = fb % size;
    s.f0 = 32 * (rank * fbase + (rank < fextra ? rank : fextra));
    s.f1 = s.f0 + 32 * (fbase + (rank < fextra ? 1 : 0));
    s.v_stride = (c.vocab + size - 1) / size;
    s.v0 = std::min(c.vocab, rank * s.v_stride);
    s.v1 = std::min(c.vocab, s.v0 + s.v_stride);
    *out = s;
    return true;
}

NcclApi g_nccl;

bool load_nccl(std::string* why) {
    if (g_nccl.AllReduce) return true;
    void* lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!lib) lib = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!lib) { *why = std::string("libnccl.so.2 not found: ") + dlerror(); return false; }
    NcclApi a;
    a.lib = lib;
    a.GetUniqueId = (decltype(a.GetUniqueId))dlsym(lib, "ncclGetUniqueId");
    a.CommInitRank = (decltype(a.CommInitRank))dlsym(lib, "ncclCommInitRank");
    a.CommDestroy = (decltype(a.CommDestroy))dlsym(lib, "ncclCommDestroy");
    a.AllReduce = (decltype(a.AllReduce))dlsym(lib, "ncclAllReduce");
    a.AllGather = (decltype(a.AllGather))dlsym(lib, "ncclAllGather");
    a.GetErrorString = (decltype(a.GetErrorString))dlsym(lib, "ncclGetErrorString");
    if (!a.GetUniqueId || !a.CommInitRank || !a.CommDestroy || !a.AllReduce || !a.AllGather || !a.GetErrorString) {
        *why = "libnccl.so.2 lacks an expected symbol";
        return false;
    }
    g_nccl = a;
    return true;
}

#define MG_NCCL(e, call)                                                                          \
    do {                                                                                          \
        ncclResult_t _r = (call);                                                                 \
        if (_r != ncclSuccess)                                                                    \
            return fail((e), MG_ERR_CUDA, "%s failed: %s (%s:%d)", #call, g_nccl.GetErrorString(_r), \
                        __FILE__, __LINE__);                                                      \
    } while (0)

// Sub-rectangle of weight slot idx that this rank keeps: rows [r0, r1) x columns [k0, k1).
void shard_rect(const mg_engine* e, int idx, int rows, int cols, int* r0, int* r1, int* k0, int* k1) {
    const mg_config& c = e->cfg;
    const Shard& s = e->sh;
    *r0 = 0; *r1 = rows; *k0 = 0; *k1 = cols;
    if (s.size == 1 || idx >= c.n_layers * 12) return;   // the head keeps every row: it is also the embedding table
    const int hd = c.head_dim;
    switch (idx % 12) {
        case 1: *r0 = s.q0 * hd; *r1 = s.q1 * hd; break;
        case 2: case 3: *r0 = s.kv0 * hd; *r1 = s.kv1 * hd; break;
        case 4: *k0 = s.q0 * hd; *k1 = s.q1 * hd; break;
        case 5: case 6: *k0 = s.kv0 * hd; *k1 = s.kv1 * hd; break;
        case 7: *k0 = s.q0 * hd; *k1 = s.q1 * hd; break;
        case 9: case 10: *r0 = s.f0; *r1 = s.f1; break;
        case 11: *k0 = s.f0; *k1 = s.f1; break;
        default: break;
    }
}

size_t raw_row_bytes(int fmt, int K) {
    return fmt == FMT_Q8_0 ? (size_t)(K / 32) * 34 : fmt == FMT_Q4_0 ? (size_t)(K / 32) * 18 : (size_t)K * 2;
}

inline int round_half_away(float v) { return (int)(v + (v > 0 ? 0.5f : -0.5f)); }

// Host quantization of one fp32 matrix straight into the two planes.
// Q8_0: d = amax/127 per block of 32, q = round-half-away(v * 127/amax), clamp +-127.
// Q4_0: d = amax/8, nib = round-half-away(v * 8/amax) + 8, clamp 0..15, byte j = elem j | elem j+16 << 4.
// d is stored as fp16 (round to nearest even); the quants use the unrounded fp32 ratio.
// `w` points at the first kept element; consecutive source rows are `ld` floats apart.
void quantize_planes(int fmt, const float* w, size_t ld, int rows, int K, uint8_t* qs, unsigned short* ds) {
    const int nb = K / 32;
    for (int r = 0; r < rows; r++) {
        const float* src = w + (size_t)r * ld;
        if (fmt == FMT_F16) {
            __half* o = reinterpret_cast<__half*>(qs) + (size_t)r * K;
            for (int k = 0; k < K; k++) o[k] = __float2half_rn(src[k]);
            continue;
        }
        for (int b = 0; b < nb; b++) {
            const float* s = src + b * 32;
            float amax = 0.f;
            for (int j = 0; j < 32; j++) {
                const float v = fabsf(s[j]);
                if (v > amax) amax = v;
            }
            if (fmt == FMT_Q8_0) {
                const __half d = __float2half_rn(amax / 127.0f);
                ds[(size_t)r * nb + b] = __half_as_ushort(d);
                const float inv = amax > 0 ? 127.0f / amax : 0.f;
                int8_t* o = reinterpret_cast<int8_t*>(qs) + (size_t)r * K + b * 32;
                for (int j = 0; j < 32; j++) {
                    float v = s[j] * inv;
                    if (v > 127.f) v = 127.f;
                    if (v < -127.f) v = -127.f;
                    o[j] = (int8_t)round_half_away(v);
                }
            } else {
                const __half d = __float2half_rn(amax / 8.0f);
                ds[(size_t)r * nb + b] = __half_as_ushort(d);
                const float inv = amax > 0 ? 8.0f / amax : 0.f;
                uint8_t* o = qs + (size_t)r * (K / 2) + b * 16;
                for (int j = 0; j < 16; j++) {
                    int q0 = round_half_away(s[j] * inv) + 8;
                    int q1 = round_half_away(s[j + 16] * inv) + 8;
                    q0 = q0 < 0 ? 0 : q0 > 15 ? 15 : q0;
                    q1 = q1 < 0 ? 0 : q1 > 15 ? 15 : q1;
                    o[j] = (uint8_t)(q0 | (q1 << 4));
                }
            }
        }
    }
}

// Split raw 34/18-byte blocks into the two planes.  `raw` points at the first kept block (or
// half); consecutive source rows are `ld_bytes` apart; K is the kept width.
void split_raw_blocks(int fmt, const uint8_t* raw, size_t ld_bytes, int rows, int K, uint8_t* qs, unsigned short* ds) {
    const int nb = K / 32;
    if (fmt == FMT_F16) {
        for (int r = 0; r < rows; r++) memcpy(qs + (size_t)r * K * 2, raw + (size_t)r * ld_bytes, (size_t)K * 2);
        return;
    }
    const int bb = fmt == FMT_Q8_0 ? 34 : 18;
    const int qb = bb - 2;
    for (int r = 0; r < rows; r++)
        for (int b = 0; b < nb; b++) {
            const uint8_t* blk = raw + (size_t)r * ld_bytes + (size_t)b * bb;
            const size_t i = (size_t)r * nb + b;
            memcpy(&ds[i], blk, 2);
            memcpy(qs + i * qb, blk + 2, qb);
        }
}

int upload_planes(mg_engine* e, int idx, int fmt, int rows, int K, const std::vector<uint8_t>& qs,
                  const std::vector<unsigned short>& ds) {
    DevMatrix& m = e->mats[idx];
    if (m.qs) { ARENA_FREE(e, m.qs); e->dev_bytes -= (size_t)m.rows * plane_row_bytes(m.fmt, m.cols); m.qs = nullptr; }
    if (m.ds) { ARENA_FREE(e, m.ds); e->dev_bytes -= (size_t)m.rows * (m.cols / 32) * 2; m.ds = nullptr; }
    int rc = dev_alloc(e, &m.qs, qs.size());
    if (rc) return rc;
    MG_CUDA(e, cudaMemcpy(m.qs, qs.data(), qs.size(), cudaMemcpyHostToDevice));
    if (fmt != FMT_F16) {
        rc = dev_alloc(e, &m.ds, ds.size());
        if (rc) return rc;
        MG_CUDA(e, cudaMemcpy(m.ds, ds.data(), ds.size() * 2, cudaMemcpyHostToDevice));
    }
    m.rows = rows; m.cols = K; m.fmt = fmt; m.set = true;
    e->built = false;
    return MG_OK;
}

// ------------------------------------------------------------------
// Kernel selection and launch
// ------------------------------------------------------------------
typedef void (*phase_fn_t)(const PhaseArgs);

template <int FMT>
phase_fn_t phase_fn_fmt(int epi, int R) {
    switch (epi) {
        case EPI_QKV: return phase_kernel<FMT, EPI_QKV, 2, 4>;
        case EPI_SWIGLU: return R == 4 ? phase_kernel<FMT, EPI_SWIGLU, 4, 2> : phase_kernel<FMT, EPI_SWIGLU, 2, 4>;
        case EPI_LOGITS: return phase_kernel<FMT, EPI_LOGITS, 4, 2>;
        default:
            return R == 4 ? phase_kernel<FMT, EPI_RESID, 4, 2>
                 : R == 2 ? phase_kernel<FMT, EPI_RESID, 2, 4>
                          : phase_kernel<FMT, EPI_RESID, 1, 8>;
    }
}

phase_fn_t phase_fn(int fmt, int epi, int R) {
    return fmt == FMT_Q8_0 ? phase_fn_fmt<FMT_Q8_0>(epi, R)
         : fmt == FMT_Q4_0 ? phase_fn_fmt<FMT_Q4_0>(epi, R)
                           : phase_fn_fmt<FMT_F16>(epi, R);
}

const int kMaxDynSmem = 120 * 1024;

int set_kernel_attrs(mg_engine* e) {
    for (int fmt = 0; fmt < 3; fmt++)
        for (int epi = 0; epi < 4; epi++)
            for (int R = 1; R <= 4; R *= 2)
                MG_CUDA(e, cudaFuncSetAttribute((const void*)phase_fn(fmt, epi, R),
                                                cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDynSmem));
    MG_CUDA(e, cudaFuncSetAttribute((const void*)attn_decode_kernel<64>,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDynSmem));
    MG_CUDA(e, cudaFuncSetAttribute((const void*)attn_decode_kernel<128>,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDynSmem));
    MG_CUDA(e, cudaFuncSetAttribute((const void*)attn_decode_kernel<32>,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDynSmem));
    return MG_OK;
}

template <typename... KArgs, typename... Args>
cudaError_t launch(mg_engine* e, cudaStream_t s, void (*kern)(KArgs...), int grid, int threads, size_t smem,
                   Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3((unsigned)threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = e->use_pdl ? 1 : 0;
    e->capture_kernels++;
    return cudaLaunchKernelEx(&cfg, kern, args...);
}

// Warps per CTA and grid for a phase of `nitems` warp tiles: spread over every SM
// first, then up to 8 warps per CTA, then two CTAs per SM; warps loop beyond that.
void phase_shape(const mg_engine* e, int nitems, int* grid, int* threads) {
    const int sms = e->num_sms;
    int wpc = (nitems + sms - 1) / sms;
    if (wpc < 1) wpc = 1;
    if (wpc > 8) wpc = 8;
    int g = (nitems + wpc - 1) / wpc;
    if (g > 2 * sms) g = 2 * sms;
    if (g < 1) g = 1;
    *grid = g;
    *threads = wpc * 32;
}

int launch_phase(mg_engine* e, cudaStream_t s, int fmt, int epi, int R, PhaseArgs& a) {
    int grid, threads;
    phase_shape(e, a.nitems, &grid, &threads);
    const size_t smem = ((size_t)a.K + 40) * sizeof(float);
    if (smem > (size_t)kMaxDynSmem) return fail(e, MG_ERR_UNSUPPORTED, "input dim %d too large", a.K);
    MG_CUDA(e, launch(e, s, phase_fn(fmt, epi, R), grid, threads, smem, a));
    return MG_OK;
}

// Rows per warp tile: the smallest of 1, 2, 4 that gives every warp at most one tile, so that no
// warp runs a second pass while others idle and the rows of a tile share the activation loads.
int pick_rows_per_tile(const mg_engine* e, int rows) {
    const int warps = e->num_sms * 16;
    if (rows > warps * 2) return 4;
    if (rows > warps) return 2;
    return 1;
}

// Layout of the exchange buffer (the same on every rank): [4 slots][size][dim] 8-byte words
// {value, exchange number} (slots 0, 1: per-phase kernels after wo / down; slots 2, 3: persistent
// kernel), then this rank's own counters (count[2], ticket[2]), then [size][2] words for the
// persistent kernel's argmax exchange.
inline size_t xchg_rows_bytes(const mg_engine* e) { return (size_t)4 * e->sh.size * e->cfg.dim * 8; }
inline size_t xchg_bytes(const mg_engine* e) { return xchg_rows_bytes(e) + 256 + (size_t)e->sh.size * 16; }
inline unsigned long long* xchg_best(const mg_engine* e, uint8_t* base) {
    return reinterpret_cast<unsigned long long*>(base + xchg_rows_bytes(e) + 256);
}
inline unsigned long long* xchg_row(const mg_engine* e, uint8_t* base, int slot, int sender) {
    return reinterpret_cast<unsigned long long*>(base) + ((size_t)slot * e->sh.size + sender) * e->cfg.dim;
}
inline unsigned int* xchg_words(const mg_engine* e, uint8_t* base) {
    return reinterpret_cast<unsigned int*>(base + xchg_rows_bytes(e));   // [0..1] count, [2..3] ticket
}

PushArgs make_push(const mg_engine* e, int slot) {
    PushArgs p{};
    if (!e->tp_fused) return p;
    p.n = e->sh.size;
    for (int r = 0; r < p.n; r++) p.dst[r] = xchg_row(e, e->xchg_peer[r], slot, e->sh.rank);
    p.count = xchg_words(e, e->xchg) + slot;
    p.ticket = xchg_words(e, e->xchg) + 2 + slot;
    return p;
}

GatherArgs make_gather(const mg_engine* e, int slot) {
    GatherArgs g{};
    if (!e->tp_fused) return g;
    g.n = e->sh.size;
    g.slot = slot;
    g.rows = xchg_row(e, e->xchg, slot, 0);
    g.count = xchg_words(e, e->xchg) + slot;
    g.status = e->xchg_status;
    return g;
}

enum { MODE_EMBED = 0, MODE_HIDDEN = 1 };
enum { HEAD_NONE = 0, HEAD_ARGMAX = 1, HEAD_LOGITS = 2 };

// One token through layers [ls, le) (+ head).  The op order is PartialStep's
// (cuda_fused_infer.go:414-451) with its 17 launches per layer fused into 5.
int enqueue_step(mg_engine* e, cudaStream_t s, int ls, int le, int mode, int head) {
    const mg_config& c = e->cfg;
    const Shard& sh = e->sh;
    const int L = c.n_layers;
    const bool tp = sh.size > 1;
    // this rank's share of the model (the whole of it without tensor parallelism)
    const int n_heads = sh.q1 - sh.q0, n_kv = sh.kv1 - sh.kv0;
    const int q_dim = n_heads * c.head_dim, kv_dim = n_kv * c.head_dim;
    const int ffn = sh.f1 - sh.f0, vocab = sh.v1 - sh.v0;
    const float* resid_h = (tp && sh.rank != 0) ? e->zero_vec : e->h;     // rank 0 alone adds the residual;
    const float* resid_h2 = (tp && sh.rank != 0) ? e->zero_vec : e->h2;   // the all-reduce sums it in once
    e->capture_kernels = 0;
    for (int l = ls; l < le && l < L; l++) {
        const int b = l * 12;
        const size_t kvoff = (size_t)l * c.max_seq * kv_dim;
        {   // RMSNorm + QKV + bias + RoPE + KV append
            PhaseArgs a{};
            a.w[0] = e->mats[b + 1].view(); a.w[1] = e->mats[b + 2].view(); a.w[2] = e->mats[b + 3].view();
            a.rows[0] = q_dim; a.rows[1] = kv_dim; a.rows[2] = kv_dim;
            a.K = c.dim;
            a.nitems = (q_dim + 2 * kv_dim) / 2;
            const bool embed = (mode == MODE_EMBED && l == 0);
            a.pro = embed ? PRO_RMS_EMBED : PRO_RMS;
            a.x_src = e->h;
            if (l > ls) a.gather = make_gather(e, 1);   // the previous layer's down rows; CTA 0 keeps the sum in h
            a.norm_w = e->vecs[b + 0];
            a.eps = c.rms_eps;
            a.embed = e->mats[L * 12 + 1].view();
            a.embed_fmt = c.head_fmt;
            a.h_store = e->h;
            a.st = e->st;
            a.bias[0] = e->vecs[b + 4]; a.bias[1] = e->vecs[b + 5]; a.bias[2] = e->vecs[b + 6];
            a.q_out = e->q;
            a.k_cache = e->kc + kvoff;
            a.v_cache = e->vc + kvoff;
            a.cos_tab = e->cos_tab; a.sin_tab = e->sin_tab;
            a.head_dim = c.head_dim; a.kv_dim = kv_dim;
            int rc = launch_phase(e, s, c.layer_fmt, EPI_QKV, 2, a);
            if (rc) return rc;
        }
        {   // attention
            const size_t smem = ((size_t)c.head_dim + 40 + 512 + c.max_seq) * sizeof(float);
            if (smem > (size_t)kMaxDynSmem) return fail(e, MG_ERR_UNSUPPORTED, "max_seq %d too large", c.max_seq);
            cudaError_t ce;
            if (c.head_dim == 64)
                ce = launch(e, s, attn_decode_kernel<64>, n_heads, 256, smem, (const float*)e->q,
                            (const __half*)(e->kc + kvoff), (const __half*)(e->vc + kvoff), e->attn,
                            (const StepState*)e->st, kv_dim, n_heads, n_kv);
            else if (c.head_dim == 128)
                ce = launch(e, s, attn_decode_kernel<128>, n_heads, 256, smem, (const float*)e->q,
                            (const __half*)(e->kc + kvoff), (const __half*)(e->vc + kvoff), e->attn,
                            (const StepState*)e->st, kv_dim, n_heads, n_kv);
            else
                ce = launch(e, s, attn_decode_kernel<32>, n_heads, 256, smem, (const float*)e->q,
                            (const __half*)(e->kc + kvoff), (const __half*)(e->vc + kvoff), e->attn,
                            (const StepState*)e->st, kv_dim, n_heads, n_kv);
            MG_CUDA(e, ce);
        }
        {   // wo + residual: h2 = h + Wo attn (a partial sum over this rank's heads under tensor parallelism)
            PhaseArgs a{};
            const int R = pick_rows_per_tile(e, c.dim);
            a.w[0] = e->mats[b + 7].view();
            a.rows[0] = c.dim; a.K = q_dim;
            a.nitems = (c.dim + R - 1) / R;
            a.pro = PRO_PLAIN; a.x_src = e->attn;
            a.resid_in = resid_h; a.out = e->tp_fused ? nullptr : e->h2; a.st = e->st;
            a.push = make_push(e, 0);
            int rc = launch_phase(e, s, c.layer_fmt, EPI_RESID, R, a);
            if (rc) return rc;
            if (tp && !e->tp_fused)
                MG_NCCL(e, g_nccl.AllReduce(e->h2, e->h2, (size_t)c.dim, ncclFloat, ncclSum, e->comm, s));
        }
        {   // RMSNorm + gate/up + SiLU-gate
            PhaseArgs a{};
            const int R = (ffn >= e->num_sms * 16 * 8) ? 4 : 2;
            a.w[0] = e->mats[b + 9].view(); a.w[1] = e->mats[b + 10].view();
            a.rows[0] = ffn; a.rows[1] = ffn; a.K = c.dim;
            a.nitems = (ffn + R / 2 - 1) / (R / 2);
            a.pro = PRO_RMS; a.x_src = e->h2; a.norm_w = e->vecs[b + 8]; a.eps = c.rms_eps;
            a.gather = make_gather(e, 0); a.h_store = e->h2;
            a.out = e->mid; a.st = e->st;
            int rc = launch_phase(e, s, c.layer_fmt, EPI_SWIGLU, R, a);
            if (rc) return rc;
        }
        {   // down + residual: h = h2 + Wd mid (a partial sum over this rank's FFN features)
            PhaseArgs a{};
            const int R = pick_rows_per_tile(e, c.dim);
            a.w[0] = e->mats[b + 11].view();
            a.rows[0] = c.dim; a.K = ffn;
            a.nitems = (c.dim + R - 1) / R;
            a.pro = PRO_PLAIN; a.x_src = e->mid;
            a.resid_in = resid_h2; a.out = e->tp_fused ? nullptr : e->h; a.st = e->st;
            a.push = make_push(e, 1);
            int rc = launch_phase(e, s, c.layer_fmt, EPI_RESID, R, a);
            if (rc) return rc;
            if (tp && !e->tp_fused)
                MG_NCCL(e, g_nccl.AllReduce(e->h, e->h, (size_t)c.dim, ncclFloat, ncclSum, e->comm, s));
        }
    }
    const bool ran_layers = std::min(le, L) > ls;
    const bool head_runs = le >= L && head != HEAD_NONE;
    if (e->tp_fused && ran_layers && !head_runs)   // nothing downstream adds the last down rows: do it here
        MG_CUDA(e, launch(e, s, xchg_reduce_kernel, 4, 256, 0, make_gather(e, 1), e->h, c.dim));
    if (le >= L && head != HEAD_NONE) {
        const DevMatrix& hm = e->mats[L * 12 + 1];
        PhaseArgs a{};
        a.w[0] = WeightView{hm.qs + (size_t)sh.v0 * plane_row_bytes(hm.fmt, hm.cols),
                            hm.ds ? hm.ds + (size_t)sh.v0 * (hm.cols / 32) : nullptr};
        a.rows[0] = vocab; a.K = c.dim;
        a.nitems = (vocab + 3) / 4;
        a.pro = PRO_RMS; a.x_src = e->h; a.norm_w = e->vecs[L * 12]; a.eps = c.rms_eps;
        if (ran_layers) { a.gather = make_gather(e, 1); a.h_store = e->h; }
        a.out = head == HEAD_LOGITS ? e->logits : nullptr;
        a.st = e->st;
        a.out_tokens = e->out_tokens;
        a.row_base = sh.v0;
        a.defer_finalize = tp ? 1 : 0;
        int rc = launch_phase(e, s, c.head_fmt, EPI_LOGITS, 4, a);
        if (rc) return rc;
        if (tp) {
            // greedy token: maximum over ranks of the packed (logit, lowest index) keys, then the cursor update
            MG_NCCL(e, g_nccl.AllReduce(&e->st->best, &e->st->best, 1, ncclUint64, ncclMax, e->comm, s));
            MG_CUDA(e, launch(e, s, finalize_step_kernel, 1, 1, 0, e->st, e->out_tokens));
            if (head == HEAD_LOGITS)
                MG_NCCL(e, g_nccl.AllGather(e->logits, e->logits_all, (size_t)sh.v_stride, ncclFloat, e->comm, s));
        }
    }
    return MG_OK;
}


// ------------------------------------------------------------------
// Persistent-kernel path: tape construction and launch
// ------------------------------------------------------------------
void free_mega(mg_engine* e) {
    auto drop = [&](void* p, size_t bytes) { if (p) { ARENA_FREE(e, p); e->dev_bytes -= bytes; } };
    drop(e->tape, e->tape_bytes); e->tape = nullptr; e->tape_bytes = 0;
    if (e->tape_off) { ARENA_FREE(e, e->tape_off); e->tape_off = nullptr; }
    if (e->mk_norms) { ARENA_FREE(e, e->mk_norms); e->mk_norms = nullptr; }
    if (e->mk_bias) { ARENA_FREE(e, e->mk_bias); e->mk_bias = nullptr; }
    if (e->xbuf) { ARENA_FREE(e, e->xbuf); e->xbuf = nullptr; }
    if (e->mk_status) { ARENA_FREE(e, e->mk_status); e->mk_status = nullptr; }
    if (e->mk_acc) { ARENA_FREE(e, e->mk_acc); e->mk_acc = nullptr; }
    e->ffn_fused = false;
    if (e->mk_trace) { ARENA_FREE(e, e->mk_trace); e->mk_trace = nullptr; }
    if (e->h_in) { ARENA_FREE(e, e->h_in); e->h_in = nullptr; }
    e->mega_ok = false;
}

// The model as the persistent kernel of THIS rank sees it: dim is the model width, every other size
// is the rank's share (the whole model without tensor parallelism); q_dim = rows of Q held here.
mg_config mega_cfg(const mg_engine* e, int* q_dim, int* vocab_base) {
    mg_config c = e->cfg;
    const Shard& sh = e->sh;
    c.n_heads = sh.q1 - sh.q0;
    c.n_kv_heads = sh.kv1 - sh.kv0;
    c.kv_dim = c.n_kv_heads * c.head_dim;
    c.ffn_dim = sh.f1 - sh.f0;
    c.vocab = sh.v1 - sh.v0;
    *q_dim = c.n_heads * c.head_dim;
    *vocab_base = sh.v0;
    return c;
}

// Matrix slots that feed phase p of layer l, in the order the phase's items name them.
void phase_matrices(const mg_config& c, int l, int p, int out[3], int* n) {
    const int b = l * 12;
    switch (p) {
        case PH_QKV: out[0] = b + 1; out[1] = b + 2; out[2] = b + 3; *n = 3; break;
        case PH_WO: out[0] = b + 7; *n = 1; break;
        case PH_GU: out[0] = b + 9; out[1] = b + 10; *n = 2; break;
        case PH_DOWN: out[0] = b + 11; *n = 1; break;
        default: out[0] = c.n_layers * 12 + 1; *n = 1; break;
    }
}

// Rows (matrix ordinal within the phase, row) of work item `item`, in tape order.
inline int item_rows(const mg_config& c, int q_dim, int p, int item, int m_out[2], int r_out[2]) {
    if (p == PH_QKV) {
        int m, r0, r1;
        qkv_pair(item, q_dim, c.kv_dim, c.head_dim, &m, &r0, &r1);
        m_out[0] = m_out[1] = m; r_out[0] = r0; r_out[1] = r1;
        return 2;
    }
    if (p == PH_GU) { m_out[0] = 0; m_out[1] = 1; r_out[0] = r_out[1] = item; return 2; }
    m_out[0] = 0; r_out[0] = item;
    return 1;
}

// Decide whether the persistent kernel can run this model and with how many ring slots.
bool mega_feasible(mg_engine* e, std::string* why) {
    int q_dim, vocab_base;
    const mg_config c = mega_cfg(e, &q_dim, &vocab_base);
    const int G = e->num_sms;
    if (e->sh.size > 1 && !e->tp_fused) { *why = "tensor parallelism through NCCL uses the per-phase kernels"; return false; }
    if (e->sh.size > 1) {
        // MG_TP_MEGA=0 keeps tensor-parallel ranks on the per-phase kernels
        const char* env = getenv("MG_TP_MEGA");
        if (env && env[0] == '0') { *why = "MG_TP_MEGA=0: tensor parallelism on the per-phase kernels"; return false; }
    }
    if (e->sh.size > 1 && e->own_le - e->own_ls != c.n_layers) { *why = "layer ranges are not combined with tensor parallelism"; return false; }
    int coop = 0;
    cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, c.device);
    if (!coop) { *why = "cooperative launch unsupported"; return false; }
    if (c.n_heads > G) { *why = "more query heads than SMs"; return false; }
    if (c.max_seq > 16384) { *why = "max_seq too large for the score buffer"; return false; }
    const int slot = MK_SLOT;
    int xs_bytes = 3 * c.head_dim * 4;          // attention keeps q and the new k, v rows there
    for (int p = 0; p <= PH_HEAD; p++) {
        const PhaseShape s = phase_shape_of(p, c.dim, q_dim, c.kv_dim, c.ffn_dim, c.vocab, c.layer_fmt, c.head_fmt);
        // MG_GEOM="w:s,w:s,w:s,w:s,w:s" pins (wide, K-split) of the five phases (-1 = choose); tuning aid
        int fw = -1, fs = -1;
        if (const char* gs = getenv("MG_GEOM")) {
            int v[10] = {-1, -1, -1, -1, -1, -1, -1, -1, -1, -1};
            sscanf(gs, "%d:%d,%d:%d,%d:%d,%d:%d,%d:%d", &v[0], &v[1], &v[2], &v[3], &v[4], &v[5], &v[6], &v[7], &v[8], &v[9]);
            fw = v[2 * p]; fs = v[2 * p + 1];
        }
        e->mk_geom[p] = choose_geom(s.fmt, s.K, s.items, s.rpi, G, MK_NW, slot, p == PH_HEAD, fw, fs);
        if (e->mk_geom[p].nkt == 0) { *why = "no tile layout for a phase"; return false; }
        if (p == PH_QKV) {
            // Leave the CTAs that run attention without QKV rows where the busiest CTA gets no more rows
            // for it: they then fetch their cached K/V rows while the others multiply.  MG_QKV_ALL=1 keeps them in.
            const int sh = e->mk_geom[p].ipg_shift, units = (s.items + (1 << sh) - 1) >> sh, rest = G - c.n_heads;
            const char* all = getenv("MG_QKV_ALL");
            e->mk_qkv_cta0 = (rest > 0 && !(all && all[0] == '1') && (units + rest - 1) / rest == (units + G - 1) / G) ? c.n_heads : 0;
        }
        xs_bytes = std::max(xs_bytes, xs_bytes_of(s.fmt, s.K));
    }
    // Down projection on each CTA's own window of the middle vector (no exchange between gate/up and
    // down; one GPU).  The window is the blocks of columns the CTA's gate/up items touch, rounded up
    // to whole wide tiles, the same width on every CTA.  MG_FFN_FUSED=0 keeps the exchange.
    e->ffn_fused = false;
    {
        const char* env = getenv("MG_FFN_FUSED");
        const int kblk = kblock_of(c.layer_fmt), total = c.ffn_dim / kblk;
        const PhaseGeom& gu = e->mk_geom[PH_GU];
        const int units = (c.ffn_dim + (1 << gu.ipg_shift) - 1) >> gu.ipg_shift;
        int nkt = 0, owners = 0;
        for (int cta = 0; cta < G; cta++) {
            const int ub = unit_begin(units, cta, G), n = unit_begin(units, cta + 1, G) - ub;
            if (n == 0) continue;
            owners++;
            const int lo = ub << gu.ipg_shift, hi = std::min((ub + n) << gu.ipg_shift, c.ffn_dim);
            nkt = std::max(nkt, ((hi - 1) / kblk - lo / kblk + 2) / 2);
        }
        const int Kl = 2 * nkt * kblk;
        // Worth it?  Against the exchange, the window costs the busiest CTA extra tiles (whole wide tiles
        // times all rows) and one 64-bit reduction per row; it saves every CTA the poll of the whole
        // middle vector.  In CTA cycles, roughly: 20 per tile, 1 per reduction, 1.3 per polled word.
        // Measured on B200 against the exchange: Qwen2.5-0.5B +10 %, TinyLlama-1.1B +3 %, 7B-class
        // widths +8 %; a model as wide as its FFN would lose.  MG_FFN_FUSED=1 / 0 overrides the rule.
        const PhaseGeom& gd = e->mk_geom[PH_DOWN];
        const int d_units = (c.dim + (1 << gd.ipg_shift) - 1) >> gd.ipg_shift;
        const long long exch_tiles = (long long)((d_units + G - 1) / G) * gd.nkt;
        const long long fused_tiles = (long long)((c.dim + 7) >> 3) * nkt;
        const bool pays = 200 * (fused_tiles - exch_tiles) + 10ll * c.dim < 13ll * c.ffn_dim;
        // The rotation of the accumulators is proven for shapes in which every CTA owns gate/up rows (a
        // complete word then shows that EVERY CTA has passed the previous layer); narrower shapes keep
        // the exchange unless the switch forces the fused block (tests do, on tiny models, where a CTA
        // without rows would have to fall a whole layer behind for the difference to matter).
        const bool want = env ? env[0] != '0' : (pays && owners == G);
        if (e->sh.size == 1 && want && owners + 1 <= 255 && c.ffn_dim % kblk == 0 && nkt > 0 && total >= 2 * nkt &&
            Kl <= 2 * MK_CONSUMERS && MK_NW * nkt <= slot / tile_bytes_of(c.layer_fmt)) {
            PhaseGeom g{};
            g.wide = 1; g.S = 1; g.RS = MK_NW; g.nkt = nkt; g.ipg_shift = 3;
            g.tile_bytes = tile_bytes_of(c.layer_fmt); g.tpe = slot / g.tile_bytes;
            g.kblocks = 2 * nkt; g.K = Kl; g.nfull = nkt;
            e->mk_geom[PH_DOWN] = g;
            e->ffn_fused = true;
            e->mk_acc_n = owners + 1;
            const int stage = c.layer_fmt == FMT_F16 ? 0 : (xs_bytes_of(c.layer_fmt, Kl) + 15) & ~15;
            xs_bytes = std::max(xs_bytes, stage + Kl * 4);
        }
    }
    const int xs = ((xs_bytes + 15) / 16) * 4;
    const int sc = (c.max_seq + 3) & ~3;
    int dev_max = 0;
    cudaDeviceGetAttribute(&dev_max, cudaDevAttrMaxSharedMemoryPerBlockOptin, c.device);
    int nslot = MK_MAX_SLOTS;
    while (nslot >= 4 && mk_smem_bytes(nslot, slot, xs, c.dim, sc) > (size_t)dev_max) nslot--;
    if (nslot < 4) { *why = "activations leave no room for the weight ring in shared memory"; return false; }
    e->mk_nslot = nslot; e->mk_slot = slot; e->mk_xs = xs; e->mk_sc = sc;
    e->mk_smem = mk_smem_bytes(nslot, slot, xs, c.dim, sc);
    return true;
}

int build_mega(mg_engine* e) {
    free_mega(e);
    if (!e->use_mega) return MG_OK;
    std::string why;
    bool ok = mega_feasible(e, &why);
    if (ok) {
        int per_sm = 0;
        const void* kern = e->sh.size > 1 ? (const void*)mega_decode_kernel<true> : (const void*)mega_decode_kernel<false>;
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)e->mk_smem) != cudaSuccess ||
            cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, MK_THREADS, e->mk_smem) != cudaSuccess ||
            per_sm < 1) {
            cudaGetLastError();
            ok = false;
            why = "one CTA does not fit an SM";
        }
    }
    if (e->sh.size > 1 && e->comm) {
        // every rank must take the same path: the persistent kernels of the ranks wait for one another
        int* d_ok = nullptr;
        int h_ok = ok ? 1 : 0;
        MG_CUDA(e, cudaMalloc((void**)&d_ok, sizeof(int)));
        MG_CUDA(e, cudaMemcpy(d_ok, &h_ok, sizeof(int), cudaMemcpyHostToDevice));
        MG_NCCL(e, g_nccl.AllReduce(d_ok, d_ok, 1, ncclInt, ncclMin, e->comm, e->stream));
        MG_CUDA(e, cudaStreamSynchronize(e->stream));
        MG_CUDA(e, cudaMemcpy(&h_ok, d_ok, sizeof(int), cudaMemcpyDeviceToHost));
        cudaFree(d_ok);
        if (ok && !h_ok) why = "another rank cannot run it";
        ok = h_ok != 0;
    }
    if (!ok) {
        e->err = "persistent kernel not used: " + why;
        return MG_OK;
    }
    int q_dim, vocab_base;
    const mg_config c = mega_cfg(e, &q_dim, &vocab_base);
    const int G = e->num_sms, L = c.n_layers;
    const int ncol = L * 4 + 2;
    std::vector<unsigned long long> off((size_t)G * ncol);
    unsigned long long total = 0;
    // row-groups of phase p on a CTA: [first, first + count)
    auto phase_units = [&](int p, int cta, int* first) {
        const PhaseShape s = phase_shape_of(p, c.dim, q_dim, c.kv_dim, c.ffn_dim, c.vocab, c.layer_fmt, c.head_fmt);
        const int sh = e->mk_geom[p].ipg_shift;
        const int units = (s.items + (1 << sh) - 1) >> sh;
        const int off = p == PH_QKV ? e->mk_qkv_cta0 : 0;
        if (cta < off) { if (first) *first = 0; return 0; }
        const int ub = unit_begin(units, cta - off, G - off);
        if (first) *first = ub;
        return unit_begin(units, cta - off + 1, G - off) - ub;
    };
    // fused feed-forward block: a CTA with gate/up items multiplies ALL rows of the down projection
    // by its own window of columns (first block: down_window_block)
    auto gu_start = [&](int cta, int* n) {
        int ub = 0;
        *n = phase_units(PH_GU, cta, &ub);
        return ub << e->mk_geom[PH_GU].ipg_shift;
    };
    auto units_of = [&](int p, int cta, int* first) {
        if (p == PH_DOWN && e->ffn_fused) {
            int n = 0;
            gu_start(cta, &n);
            if (first) *first = 0;
            return n > 0 ? (c.dim + 7) >> 3 : 0;
        }
        return phase_units(p, cta, first);
    };
    auto phase_bytes = [&](int p, int cta) {
        return (unsigned long long)units_of(p, cta, nullptr) * e->mk_geom[p].nkt * e->mk_geom[p].tile_bytes;
    };
    // a pipeline stage streams only the layers it owns (and lm_head only with the last layer)
    auto owned = [&](int l) { return l < L ? (l >= e->own_ls && l < e->own_le) : e->own_le >= L; };
    for (int cta = 0; cta < G; cta++) {
        for (int l = 0; l < L; l++)
            for (int p = 0; p < 4; p++) {
                off[(size_t)cta * ncol + l * 4 + p] = total;
                if (owned(l)) total += phase_bytes(p, cta);
            }
        off[(size_t)cta * ncol + L * 4] = total;
        if (owned(L)) total += phase_bytes(PH_HEAD, cta);
        off[(size_t)cta * ncol + L * 4 + 1] = total;
    }
    std::vector<uint8_t> tape((size_t)total + e->mk_slot, 0);

    // fill: one (layer, phase) at a time so that only that phase's matrices are on the host
    std::vector<uint8_t> hq[3];
    std::vector<unsigned short> hd[3];
    MG_CUDA(e, cudaStreamSynchronize(e->stream));
    for (int l = 0; l <= L; l++)
        for (int p = (l < L ? 0 : PH_HEAD); p <= (l < L ? 3 : PH_HEAD); p++) {
            if (!owned(l)) continue;
            int slots[3], nm = 0;
            phase_matrices(c, l, p, slots, &nm);
            const PhaseShape s = phase_shape_of(p, c.dim, q_dim, c.kv_dim, c.ffn_dim, c.vocab, c.layer_fmt, c.head_fmt);
            const int rq = row_q_bytes(s.fmt, s.K), rd = row_d_bytes(s.fmt, s.K);
            for (int m = 0; m < nm; m++) {
                const DevMatrix& M = e->mats[slots[m]];
                // lm_head is stored whole (it is also the embedding table): this rank streams rows [v0, v1)
                const int row0 = p == PH_HEAD ? vocab_base : 0;
                const int nr = p == PH_HEAD ? c.vocab : M.rows;
                hq[m].resize((size_t)nr * rq);
                MG_CUDA(e, cudaMemcpy(hq[m].data(), M.qs + (size_t)row0 * rq, hq[m].size(), cudaMemcpyDeviceToHost));
                hd[m].resize(rd ? (size_t)nr * (s.K / 32) : 0);
                if (rd) MG_CUDA(e, cudaMemcpy(hd[m].data(), M.ds + (size_t)row0 * (s.K / 32), hd[m].size() * 2, cudaMemcpyDeviceToHost));
            }
            const PhaseGeom g = e->mk_geom[p];
            const int ipg = 1 << g.ipg_shift;
            const int col = l < L ? l * 4 + p : L * 4;
            for (int cta = 0; cta < G; cta++) {
                int ub = 0;
                const int nrg = units_of(p, cta, &ub);
                const int kblk = kblock_of(s.fmt), all_blocks = s.K / kblk;
                int kb0 = 0;                         // first block of columns of this CTA's tiles
                if (p == PH_DOWN && e->ffn_fused) {
                    int n = 0;
                    kb0 = down_window_block(gu_start(cta, &n), kblk, all_blocks, g.nkt);
                }
                uint8_t* dst = tape.data() + off[(size_t)cta * ncol + col];
                // tiles in the order the warps take them: pass, round, row-group of the pass, K-split
                // (fused down projection: row-group by row-group, its k-tiles together)
                const bool by_rg = p == PH_DOWN && e->ffn_fused;
                const int oRS = by_rg ? 1 : g.RS, oS = by_rg ? g.nkt : g.S;
                for (int rb = 0; rb * oRS < nrg; rb++) {
                    const int nrs = std::min(oRS, nrg - rb * oRS);
                    for (int k0 = 0; k0 < g.nkt; k0 += oS) {
                        const int nkp = std::min(oS, g.nkt - k0);
                        for (int rs = 0; rs < nrs; rs++)
                            for (int kp = 0; kp < nkp; kp++, dst += g.tile_bytes) {
                                const int rgi = ub + rb * oRS + rs, kt = k0 + kp;
                                // source row and block of every row-slot (nullptr: the slot is empty)
                                const uint8_t* sq[16];
                                const unsigned short* sd[16];
                                for (int sl = 0; sl < 16; sl++) {
                                    int j, which, kpar;
                                    slot_item(g.wide, s.rpi, sl, &j, &which, &kpar);
                                    const int item = rgi * ipg + j;
                                    const int kb = kb0 + (g.wide ? 2 * kt + kpar : kt);
                                    sq[sl] = nullptr; sd[sl] = nullptr;
                                    if (item >= s.items || kb >= all_blocks) continue;
                                    int mm[2], rr[2];
                                    item_rows(c, q_dim, p, item, mm, rr);
                                    const uint8_t* rowq = hq[mm[which]].data() + (size_t)rr[which] * rq;
                                    sq[sl] = rowq + (size_t)kb * (s.fmt == FMT_Q8_0 ? 32 : s.fmt == FMT_Q4_0 ? 16 : 32);
                                    if (rd) sd[sl] = hd[mm[which]].data() + (size_t)rr[which] * (s.K / 32) + kb;
                                }
                                for (int lane = 0; lane < 32; lane++) {
                                    const int gq = lane >> 2, t = lane & 3;
                                    if (s.fmt == FMT_Q8_0) {
                                        // A registers a0..a3 = (slot g, cols 4t..), (slot g+8, cols 4t..), (slot g, cols 16+4t..), (slot g+8, 16+4t..)
                                        for (int i = 0; i < 4; i++) {
                                            const uint8_t* src = sq[gq + 8 * (i & 1)];
                                            if (src) memcpy(dst + lane * 16 + i * 4, src + 16 * (i >> 1) + 4 * t, 4);
                                        }
                                    } else if (s.fmt == FMT_Q4_0) {
                                        // nibble bytes 4t..4t+3 of slots g and g+8
                                        for (int i = 0; i < 2; i++) {
                                            const uint8_t* src = sq[gq + 8 * i];
                                            if (src) memcpy(dst + lane * 8 + i * 4, src + 4 * t, 4);
                                        }
                                    } else {
                                        // halves 4t..4t+3 of slots g and g+8
                                        for (int i = 0; i < 2; i++) {
                                            const uint8_t* src = sq[gq + 8 * i];
                                            if (src) memcpy(dst + lane * 16 + i * 8, src + 8 * t, 8);
                                        }
                                    }
                                }
                                if (rd) {
                                    unsigned short* tds = reinterpret_cast<unsigned short*>(dst + (s.fmt == FMT_Q8_0 ? 512 : 256));
                                    for (int gq = 0; gq < 8; gq++) {
                                        if (sd[gq]) tds[2 * gq] = *sd[gq];
                                        if (sd[gq + 8]) tds[2 * gq + 1] = *sd[gq + 8];
                                    }
                                }
                            }
                    }
                }
            }
        }
    for (int m = 0; m < 3; m++) { hq[m] = {}; hd[m] = {}; }

    int rc;
    e->tape_bytes = tape.size();
    if ((rc = dev_alloc(e, &e->tape, tape.size()))) { e->tape_bytes = 0; return rc; }
    MG_CUDA(e, cudaMemcpy(e->tape, tape.data(), tape.size(), cudaMemcpyHostToDevice));
    tape = {};
    MG_CUDA(e, ARENA_MALLOC(e, &e->tape_off, off.size() * 8));
    MG_CUDA(e, cudaMemcpy(e->tape_off, off.data(), off.size() * 8, cudaMemcpyHostToDevice));
    MG_CUDA(e, ARENA_MALLOC(e, &e->mk_norms, (size_t)L * 2 * c.dim * 4));
    bool any_bias = false;
    for (int l = 0; l < L; l++) {
        if (!owned(l)) continue;
        MG_CUDA(e, cudaMemcpy(e->mk_norms + (size_t)l * 2 * c.dim, e->vecs[l * 12 + 0], (size_t)c.dim * 4, cudaMemcpyDeviceToDevice));
        MG_CUDA(e, cudaMemcpy(e->mk_norms + (size_t)l * 2 * c.dim + c.dim, e->vecs[l * 12 + 8], (size_t)c.dim * 4, cudaMemcpyDeviceToDevice));
        any_bias = any_bias || e->vecs[l * 12 + 4] || e->vecs[l * 12 + 5] || e->vecs[l * 12 + 6];
    }
    if (any_bias) {
        const size_t bw = (size_t)q_dim + 2 * c.kv_dim;
        MG_CUDA(e, ARENA_MALLOC(e, &e->mk_bias, (size_t)L * bw * 4));
        MG_CUDA(e, cudaMemset(e->mk_bias, 0, (size_t)L * bw * 4));     // an unset bias adds zero
        for (int l = 0; l < L; l++) {
            if (!owned(l)) continue;
            const size_t offs[3] = {0, (size_t)q_dim, (size_t)q_dim + c.kv_dim};
            const size_t lens[3] = {(size_t)q_dim, (size_t)c.kv_dim, (size_t)c.kv_dim};
            for (int k = 0; k < 3; k++)
                if (e->vecs[l * 12 + 4 + k])
                    MG_CUDA(e, cudaMemcpy(e->mk_bias + l * bw + offs[k], e->vecs[l * 12 + 4 + k], lens[k] * 4, cudaMemcpyDeviceToDevice));
        }
    }
    const size_t nx = (size_t)2 * c.dim + 2 * q_dim + 2 * c.kv_dim + c.ffn_dim + 2;   // xh xhm | xq | xkv | xattn | xmid | xtok
    MG_CUDA(e, ARENA_MALLOC(e, &e->xbuf, nx * sizeof(Tagged)));
    MG_CUDA(e, cudaMemset(e->xbuf, 0, nx * sizeof(Tagged)));
    MG_CUDA(e, ARENA_MALLOC(e, &e->mk_status, sizeof(MegaStatus)));
    MG_CUDA(e, cudaMemset(e->mk_status, 0, sizeof(MegaStatus)));
    if (e->ffn_fused) {
        MG_CUDA(e, ARENA_MALLOC(e, &e->mk_acc, (size_t)3 * c.dim * 8));
        MG_CUDA(e, cudaMemset(e->mk_acc, 0, (size_t)3 * c.dim * 8));
        e->mk_buf = 0;
    }
    e->mega_ok = true;
    return MG_OK;
}

// One launch of the persistent kernel: n_steps tokens through layers [ls, le).
int launch_mega(mg_engine* e, int ls, int le, int mode, int head, int n_steps) {
    int q_dim, vocab_base;
    const mg_config c = mega_cfg(e, &q_dim, &vocab_base);
    const int L = c.n_layers;
    MegaArgs a{};
    a.dim = c.dim; a.kv_dim = c.kv_dim; a.head_dim = c.head_dim; a.n_heads = c.n_heads; a.n_kv_heads = c.n_kv_heads;
    a.ffn_dim = c.ffn_dim; a.vocab = c.vocab; a.n_layers = L; a.max_seq = c.max_seq;
    a.layer_fmt = c.layer_fmt; a.head_fmt = c.head_fmt; a.eps = c.rms_eps; a.inv_dim = 1.0f / (float)c.dim;
    a.ls = ls; a.le = le; a.head = (le >= L) ? head : 0; a.embed = (mode == MODE_EMBED); a.n_steps = n_steps;
    a.epoch = e->epoch;
    e->epoch += (unsigned)n_steps * (unsigned)(L * MK_EPOCHS_PER_LAYER + 8);
    a.hd_shift = c.head_dim == 32 ? 5 : c.head_dim == 64 ? 6 : 7;
    for (int p = 0; p < 5; p++) a.geom[p] = e->mk_geom[p];
    a.nslot = e->mk_nslot; a.slot_bytes = e->mk_slot; a.prefetch_bytes = e->mk_prefetch; a.xs_floats = e->mk_xs; a.sc_floats = e->mk_sc;
    a.wait_cycles = e->mk_wait;
    a.tape = e->tape; a.tape_off = e->tape_off; a.tape_bytes = e->tape_bytes;
    a.norms = e->mk_norms; a.qkv_bias = e->mk_bias;
    a.final_norm = e->vecs[L * 12];
    a.embed_w = e->mats[L * 12 + 1].view();
    a.cos_tab = e->cos_tab; a.sin_tab = e->sin_tab; a.kc = e->kc; a.vc = e->vc;
    Tagged* x = e->xbuf;
    a.xh = x; x += c.dim; a.xhm = x; x += c.dim; a.xq = x; x += q_dim; a.xkv = x; x += 2 * c.kv_dim;
    a.xattn = x; x += q_dim; a.xmid = x; x += c.ffn_dim; a.xtok = x;
    a.q_dim = q_dim; a.tp_n = e->sh.size; a.tp_rank = e->sh.rank; a.vocab_base = vocab_base; a.vocab_total = e->cfg.vocab;
    if (e->sh.size > 1) {
        // the hidden-state exchanges go through the receive buffers every rank has mapped
        a.xhm = reinterpret_cast<Tagged*>(xchg_row(e, e->xchg, 2, 0));
        a.xh = reinterpret_cast<Tagged*>(xchg_row(e, e->xchg, 3, 0));
        a.xbest = reinterpret_cast<Tagged*>(xchg_best(e, e->xchg));
        for (int p = 0; p < e->sh.size; p++) {
            a.xhm_peer[p] = reinterpret_cast<Tagged*>(xchg_row(e, e->xchg_peer[p], 2, 0));
            a.xh_peer[p] = reinterpret_cast<Tagged*>(xchg_row(e, e->xchg_peer[p], 3, 0));
            a.xbest_peer[p] = reinterpret_cast<Tagged*>(xchg_best(e, e->xchg_peer[p]));
        }
    }
    a.h_in = e->h; a.h_out = e->h; a.logits = e->logits_direct ? e->logits_direct : e->logits; a.st = e->st; a.out_tokens = e->out_tokens;
    a.status = e->mk_status;
    a.ffn_fused = e->ffn_fused ? 1 : 0;
    a.qkv_cta0 = e->mk_qkv_cta0;
    if (e->ffn_fused) {
        // the accumulators rotate on from launch to launch
        const unsigned int n = (unsigned)n_steps * (unsigned)(le - ls);
        a.acc = e->mk_acc; a.acc_n = e->mk_acc_n;
        a.acc_buf0 = e->mk_buf;
        e->mk_buf = (int)((e->mk_buf + n) % 3u);
    }
    a.trace = e->trace_next ? e->mk_trace : nullptr;
    e->trace_next = false;
    void* params[] = {&a};
    const void* kern = e->sh.size > 1 ? (const void*)mega_decode_kernel<true> : (const void*)mega_decode_kernel<false>;
    MG_CUDA(e, cudaLaunchCooperativeKernel(kern, dim3(e->num_sms), dim3(MK_THREADS), params,
                                           e->mk_smem, e->stream));
    e->launches += 1;
    return MG_OK;
}

// Did any wait inside the kernels give up?  The status words are copied to pinned memory behind
// whatever is still queued on the engine's stream, followed by ONE synchronisation (callers need not
// synchronise first).
int check_mega_status(mg_engine* e) {
    MegaStatus* hs = reinterpret_cast<MegaStatus*>(e->pin_i + e->pin_i_cap);
    XchgStatus* hx = reinterpret_cast<XchgStatus*>(e->pin_i + e->pin_i_cap + 8);
    static_assert(sizeof(MegaStatus) <= 32 && sizeof(XchgStatus) <= 32, "status words must fit their pinned slots");
    if (e->tp_fused) MG_CUDA(e, cudaMemcpyAsync(hx, e->xchg_status, sizeof(XchgStatus), cudaMemcpyDeviceToHost, e->stream));
    if (e->mega_ok) MG_CUDA(e, cudaMemcpyAsync(hs, e->mk_status, sizeof(MegaStatus), cudaMemcpyDeviceToHost, e->stream));
    MG_CUDA(e, cudaStreamSynchronize(e->stream));
    if (e->tp_fused) {
        const XchgStatus x = *hx;
        if (x.error) {
            cudaMemset(e->xchg_status, 0, sizeof x);
            return fail(e, MG_ERR_TIMEOUT, "tensor-parallel exchange: rows of rank %d never arrived (slot %d, exchange %u, last seen %u)",
                        x.sender, x.slot, x.want, x.seen);
        }
    }
    if (!e->mega_ok) return MG_OK;
    const MegaStatus s = *hs;
    if (s.error) {
        cudaMemset(e->mk_status, 0, sizeof s);
        if (e->mk_acc) {
            // the aborted launch left the accumulators anywhere: start over
            cudaMemset(e->mk_acc, 0, (size_t)3 * e->cfg.dim * 8);
            e->mk_buf = 0;
        }
        if (s.error == MK_ERR_POLL && s.who >= 0)
            return fail(e, MG_ERR_TIMEOUT, "persistent kernel: the rows of rank %d never arrived (exchange %u, CTA %d)", s.who, (unsigned)s.where, s.cta);
        return fail(e, MG_ERR_TIMEOUT, "persistent kernel: wait %d timed out (where %d, CTA %d)", s.error, s.where, s.cta);
    }
    return MG_OK;
}

// A step may only touch layers this engine holds (the whole model unless mg_set_layer_range narrowed it).
int check_range(mg_engine* e, int ls, int le, bool head, bool embed) {
    const int L = e->cfg.n_layers;
    if (std::min(le, L) > ls && (ls < e->own_ls || std::min(le, L) > e->own_le))
        return fail(e, MG_ERR_STATE, "layers [%d,%d) requested, this engine holds [%d,%d)", ls, le, e->own_ls, e->own_le);
    if ((head || embed) && e->own_le < L && !e->mats[L * 12 + 1].set)
        return fail(e, MG_ERR_STATE, "lm_head (and the tied embedding) live on the stage that holds the last layer");
    return MG_OK;
}

int run_step(mg_engine* e, int ls, int le, int mode, int head) {
    if (int rc = check_range(e, ls, le, head != HEAD_NONE && le >= e->cfg.n_layers, mode == MODE_EMBED)) return rc;
    if (e->mega_ok && le > ls) {
        if (int rc = launch_mega(e, ls, le, mode, head, 1)) return rc;
        if (e->sh.size > 1 && e->comm && head == HEAD_LOGITS && le >= e->cfg.n_layers)   // every rank gets every rank's slice
            MG_NCCL(e, g_nccl.AllGather(e->logits, e->logits_all, (size_t)e->sh.v_stride, ncclFloat, e->comm, e->stream));
        return MG_OK;
    }
    if (!e->use_graph) {
        int rc = enqueue_step(e, e->stream, ls, le, mode, head);
        e->launches += e->capture_kernels;
        return rc;
    }
    GraphKey key{ls, le, mode, head};
    auto it = e->graphs.find(key);
    if (it == e->graphs.end()) {
        cudaGraph_t g = nullptr;
        MG_CUDA(e, cudaStreamBeginCapture(e->stream, cudaStreamCaptureModeThreadLocal));
        int rc = enqueue_step(e, e->stream, ls, le, mode, head);
        cudaError_t ce = cudaStreamEndCapture(e->stream, &g);
        if (rc) { if (g) cudaGraphDestroy(g); return rc; }
        MG_CUDA(e, ce);
        CachedGraph cg;
        cg.kernels = e->capture_kernels;
        ce = cudaGraphInstantiate(&cg.exec, g, 0);
        cudaGraphDestroy(g);
        MG_CUDA(e, ce);
        it = e->graphs.emplace(key, cg).first;
    }
    MG_CUDA(e, cudaGraphLaunch(it->second.exec, e->stream));
    e->launches += it->second.kernels;
    return MG_OK;
}

int ensure_built(mg_engine* e) {
    if (e->built) return MG_OK;
    return mg_build(e);
}

int check_engine(mg_engine* e) {
    if (!e) return MG_ERR_ARG;
    cudaError_t c = cudaSetDevice(e->cfg.device);
    if (c != cudaSuccess) return fail(e, MG_ERR_CUDA, "cudaSetDevice(%d): %s", e->cfg.device, cudaGetErrorString(c));
    return MG_OK;
}

void drop_graphs(mg_engine* e) {
    for (auto& kv : e->graphs)
        if (kv.second.exec) cudaGraphExecDestroy(kv.second.exec);
    e->graphs.clear();
}

}  // namespace

// =====================================================================
// C ABI
// =====================================================================
extern "C" {

const char* mg_version(void) { return "mongoose-b200 decode engine, sm_100a"; }

int mg_create(const mg_config* cfg, mg_engine** out) {
    if (!cfg || !out) return MG_ERR_ARG;
    *out = nullptr;
    const mg_config& c = *cfg;
    if (c.dim <= 0 || c.n_heads <= 0 || c.n_kv_heads <= 0 || c.head_dim <= 0 || c.ffn_dim <= 0 ||
        c.vocab <= 0 || c.n_layers <= 0 || c.max_seq <= 0)
        return MG_ERR_ARG;
    if (c.dim % 32 || c.ffn_dim % 32 || c.kv_dim != c.n_kv_heads * c.head_dim || c.dim != c.n_heads * c.head_dim ||
        c.n_heads % c.n_kv_heads || (c.head_dim != 32 && c.head_dim != 64 && c.head_dim != 128))
        return MG_ERR_ARG;
    if (c.layer_fmt < 0 || c.layer_fmt > 2 || c.head_fmt < 0 || c.head_fmt > 2) return MG_ERR_ARG;
    if (c.max_batch > 1) return MG_ERR_UNSUPPORTED;

    mg_engine* e = new mg_engine();
    e->cfg = c;
    if (e->cfg.rms_eps == 0.f) e->cfg.rms_eps = 1e-6f;
    if (e->cfg.max_batch < 1) e->cfg.max_batch = 1;
    int rc = MG_OK;
    auto bail = [&](int code) { mg_destroy(e); return code; };

    cudaError_t ce = cudaSetDevice(c.device);
    if (ce != cudaSuccess) return bail(MG_ERR_CUDA);
    cudaDeviceProp prop{};
    if (cudaGetDeviceProperties(&prop, c.device) != cudaSuccess) return bail(MG_ERR_CUDA);
    if (prop.major != 10) {
        fprintf(stderr, "[mongoose-b200] device %d is sm_%d%d; this library is built for sm_100a only\n", c.device,
                prop.major, prop.minor);
        return bail(MG_ERR_UNSUPPORTED);
    }
    e->num_sms = prop.multiProcessorCount;
    if (cudaStreamCreateWithFlags(&e->stream, cudaStreamNonBlocking) != cudaSuccess) return bail(MG_ERR_CUDA);

    {
        std::string why;
        if (!make_shard(c, 0, 1, &e->sh, &why)) return bail(MG_ERR_ARG);
    }
    e->own_ls = 0; e->own_le = c.n_layers;
    if (cudaEventCreateWithFlags(&e->sent_event, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&e->mail_event, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&e->compute_done, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&e->l3_done, cudaEventDisableTiming) != cudaSuccess ||
        cudaStreamCreateWithFlags(&e->copy_stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaMallocHost((void**)&e->l3, (size_t)c.dim * sizeof(float)) != cudaSuccess)
        return bail(MG_ERR_CUDA);
    const int nw = c.n_layers * 12 + 2;
    e->mats.resize(nw);
    e->vecs.assign(nw, nullptr);

    e->out_cap = c.max_seq > 4096 ? c.max_seq : 4096;
    const int half = c.head_dim / 2;
    const size_t kv_elems = (size_t)c.n_layers * c.max_seq * c.kv_dim;
    {
        // The arena: every buffer this engine will ever need, from the model's shape - the weight planes,
        // the tape (a second copy of the layer weights and lm_head in consumption order), fp16 KV, tables,
        // activations, exchange words - plus slack for alignment.  (MG_ARENA_MB overrides the size; what
        // does not fit falls through to cudaMalloc.)
        size_t planes = 0;
        for (int idx = 0; idx < nw; idx++) {
            bool is_matrix; int rows, cols, fmt;
            slot_info(c, idx, &is_matrix, &rows, &cols, &fmt);
            planes += is_matrix ? (size_t)rows * plane_row_bytes(fmt, cols) + (fmt == FMT_F16 ? 0 : (size_t)rows * (cols / 32) * 2) + 512
                                : (size_t)cols * 4 + 256;
        }
        size_t want = 2 * planes + planes / 16 + kv_elems * 4 + (size_t)c.max_seq * half * 8 + (size_t)c.vocab * 8 +
                      (size_t)(c.dim * 64 + c.ffn_dim * 16) + (size_t)e->out_cap * 4 + (64u << 20);
        if (const char* mb = getenv("MG_ARENA_MB")) want = (size_t)atoll(mb) << 20;
        if (!e->arena.init(want)) fprintf(stderr, "[mongoose-b200] arena of %zu MB not available: falling back to one allocation per buffer\n", want >> 20);
    }
    if ((rc = dev_alloc(e, &e->cos_tab, (size_t)c.max_seq * half))) return bail(rc);
    if ((rc = dev_alloc(e, &e->sin_tab, (size_t)c.max_seq * half))) return bail(rc);
    if ((rc = dev_alloc(e, &e->kc, kv_elems))) return bail(rc);
    if ((rc = dev_alloc(e, &e->vc, kv_elems))) return bail(rc);
    if ((rc = dev_alloc(e, &e->h, (size_t)c.dim))) return bail(rc);
    if ((rc = dev_alloc(e, &e->h2, (size_t)c.dim))) return bail(rc);
    if ((rc = dev_alloc(e, &e->q, (size_t)c.dim))) return bail(rc);
    if ((rc = dev_alloc(e, &e->attn, (size_t)c.dim))) return bail(rc);
    if ((rc = dev_alloc(e, &e->mid, (size_t)c.ffn_dim))) return bail(rc);
    if ((rc = dev_alloc(e, &e->logits, (size_t)c.vocab))) return bail(rc);
    if ((rc = dev_alloc(e, &e->st, (size_t)1))) return bail(rc);
    if ((rc = dev_alloc(e, &e->out_tokens, (size_t)e->out_cap))) return bail(rc);

    // RoPE tables in float64 on the host, narrowed to fp32 (cuda_fused_infer.go:181-190).
    {
        std::vector<float> cs((size_t)c.max_seq * half), sn((size_t)c.max_seq * half);
        for (int pos = 0; pos < c.max_seq; pos++)
            for (int j = 0; j < half; j++) {
                const double freq = 1.0 / pow(c.rope_theta, (double)(2 * j) / (double)c.head_dim);
                const double ang = (double)pos * freq;
                cs[(size_t)pos * half + j] = (float)cos(ang);
                sn[(size_t)pos * half + j] = (float)sin(ang);
            }
        if (cudaMemcpy(e->cos_tab, cs.data(), cs.size() * 4, cudaMemcpyHostToDevice) != cudaSuccess ||
            cudaMemcpy(e->sin_tab, sn.data(), sn.size() * 4, cudaMemcpyHostToDevice) != cudaSuccess)
            return bail(MG_ERR_CUDA);
    }
    if (cudaMemset(e->kc, 0, kv_elems * 2) != cudaSuccess || cudaMemset(e->vc, 0, kv_elems * 2) != cudaSuccess ||
        cudaMemset(e->h, 0, (size_t)c.dim * 4) != cudaSuccess || cudaMemset(e->out_tokens, 0, (size_t)e->out_cap * 4) != cudaSuccess)
        return bail(MG_ERR_CUDA);
    StepState s0{};
    s0.out_cap = e->out_cap;
    if (cudaMemcpy(e->st, &s0, sizeof s0, cudaMemcpyHostToDevice) != cudaSuccess) return bail(MG_ERR_CUDA);

    e->pin_i_cap = 8 + e->out_cap;
    if (cudaMallocHost((void**)&e->pin_i, (size_t)(e->pin_i_cap + 16) * sizeof(int)) != cudaSuccess) return bail(MG_ERR_NOMEM);
    { const char* zc = getenv("MG_ZERO_COPY"); e->zero_copy = !(zc && zc[0] == '0'); }

    if ((rc = set_kernel_attrs(e))) return bail(rc);
    const char* env = getenv("MG_NO_GRAPH");
    if (env && env[0] == '1') e->use_graph = false;
    env = getenv("MG_NO_MEGA");
    if (env && env[0] == '1') e->use_mega = false;
    env = getenv("MG_NO_PDL");
    if (env && env[0] == '1') e->use_pdl = false;
    // L2 prefetch distance of the persistent kernel's weight stream; 64 KiB measured best on
    // 7B-class widths (layer time 85 -> 75 us), neutral on the 0.5 B model, 384 KiB thrashes L2
    env = getenv("MG_PREFETCH_KB");
    e->mk_prefetch = (env ? atoi(env) : 64) * 1024;
    if (e->mk_prefetch < 0 || e->mk_prefetch > (1 << 20)) e->mk_prefetch = 0;
    *out = e;
    return MG_OK;
}

void mg_destroy(mg_engine* e) {
    if (!e) return;
    cudaSetDevice(e->cfg.device);
    if (e->stream) cudaStreamSynchronize(e->stream);
    drop_graphs(e);
    free_mega(e);
    for (auto& m : e->mats) {
        if (m.qs) ARENA_FREE(e, m.qs);
        if (m.ds) ARENA_FREE(e, m.ds);
    }
    for (float* v : e->vecs)
        if (v) ARENA_FREE(e, v);
    ARENA_FREE(e, e->cos_tab); ARENA_FREE(e, e->sin_tab); ARENA_FREE(e, e->kc); ARENA_FREE(e, e->vc);
    ARENA_FREE(e, e->h); ARENA_FREE(e, e->h2); ARENA_FREE(e, e->q); ARENA_FREE(e, e->attn); ARENA_FREE(e, e->mid); ARENA_FREE(e, e->logits);
    ARENA_FREE(e, e->st); ARENA_FREE(e, e->out_tokens);
    if (e->comm && e->zero_vec) {
        // no rank unmaps or frees its receive buffer while a peer may still be writing to it
        if (g_nccl.AllReduce(e->zero_vec, e->zero_vec, 1, ncclFloat, ncclSum, e->comm, e->stream) == ncclSuccess)
            cudaStreamSynchronize(e->stream);
    }
    for (int p = 0; p < kMaxRanks; p++)
        if (e->xchg_peer[p] && e->xchg_peer[p] != e->xchg) cudaIpcCloseMemHandle(e->xchg_peer[p]);
    if (e->xchg) cudaFree(e->xchg);
    if (e->xchg_status) ARENA_FREE(e, e->xchg_status);
    if (e->zero_vec) ARENA_FREE(e, e->zero_vec);
    if (e->logits_all) ARENA_FREE(e, e->logits_all);
    if (e->comm && g_nccl.CommDestroy) g_nccl.CommDestroy(e->comm);
    if (e->pin_i) cudaFreeHost(e->pin_i);
    if (e->copy_stream) { cudaStreamSynchronize(e->copy_stream); cudaStreamDestroy(e->copy_stream); }
    if (e->l3) cudaFreeHost(e->l3);
    if (e->sent_event) cudaEventDestroy(e->sent_event);
    if (e->mail_event) cudaEventDestroy(e->mail_event);
    if (e->compute_done) cudaEventDestroy(e->compute_done);
    if (e->l3_done) cudaEventDestroy(e->l3_done);
    if (e->stage_done) cudaEventDestroy(e->stage_done);
    if (e->s1_in) cudaEventDestroy(e->s1_in);
    if (e->s1_out) cudaEventDestroy(e->s1_out);
    if (e->stream1) { cudaStreamSynchronize(e->stream1); cudaStreamDestroy(e->stream1); }
    if (e->stream) cudaStreamDestroy(e->stream);
    e->arena.destroy();
    delete e;
}

int mg_num_weights(const mg_engine* e) { return e ? e->cfg.n_layers * 12 + 2 : 0; }

int mg_set_weight(mg_engine* e, int idx, const float* data, size_t count) {
    int rc = check_engine(e);
    if (rc) return rc;
    bool is_matrix; int rows, cols, fmt;
    if (!data || !slot_info(e->cfg, idx, &is_matrix, &rows, &cols, &fmt))
        return fail(e, MG_ERR_ARG, "mg_set_weight: bad slot %d", idx);
    if (count != (size_t)rows * cols)
        return fail(e, MG_ERR_ARG, "mg_set_weight: slot %d wants %d x %d values, got %zu", idx, rows, cols, count);
    int r0, r1, k0, k1;
    shard_rect(e, idx, rows, cols, &r0, &r1, &k0, &k1);
    e->any_weight_set = true;
    if (!is_matrix) {
        if (!e->vecs[idx] && (rc = dev_alloc(e, &e->vecs[idx], (size_t)(k1 - k0)))) return rc;
        MG_CUDA(e, cudaMemcpy(e->vecs[idx], data + k0, (size_t)(k1 - k0) * 4, cudaMemcpyHostToDevice));
        e->built = false;
        return MG_OK;
    }
    const int lr = r1 - r0, lk = k1 - k0;
    std::vector<uint8_t> qs((size_t)lr * plane_row_bytes(fmt, lk));
    std::vector<unsigned short> ds(fmt == FMT_F16 ? 0 : (size_t)lr * (lk / 32));
    quantize_planes(fmt, data + (size_t)r0 * cols + k0, (size_t)cols, lr, lk, qs.data(), ds.data());
    return upload_planes(e, idx, fmt, lr, lk, qs, ds);
}

int mg_set_weight_raw(mg_engine* e, int idx, const void* blocks, size_t bytes, int fmt) {
    int rc = check_engine(e);
    if (rc) return rc;
    bool is_matrix; int rows, cols, slot_fmt;
    if (!blocks || !slot_info(e->cfg, idx, &is_matrix, &rows, &cols, &slot_fmt) || !is_matrix)
        return fail(e, MG_ERR_ARG, "mg_set_weight_raw: slot %d is not a matrix slot", idx);
    if (fmt != slot_fmt)
        return fail(e, MG_ERR_ARG, "mg_set_weight_raw: slot %d is configured for format %d, got %d", idx, slot_fmt, fmt);
    if (bytes != (size_t)rows * raw_row_bytes(fmt, cols))
        return fail(e, MG_ERR_ARG, "mg_set_weight_raw: slot %d wants %zu bytes, got %zu", idx,
                    (size_t)rows * raw_row_bytes(fmt, cols), bytes);
    int r0, r1, k0, k1;
    shard_rect(e, idx, rows, cols, &r0, &r1, &k0, &k1);
    e->any_weight_set = true;
    const int lr = r1 - r0, lk = k1 - k0;
    const size_t ld = raw_row_bytes(fmt, cols);
    std::vector<uint8_t> qs((size_t)lr * plane_row_bytes(fmt, lk));
    std::vector<unsigned short> ds(fmt == FMT_F16 ? 0 : (size_t)lr * (lk / 32));
    split_raw_blocks(fmt, static_cast<const uint8_t*>(blocks) + (size_t)r0 * ld + raw_row_bytes(fmt, k0), ld, lr, lk,
                     qs.data(), ds.data());
    return upload_planes(e, idx, fmt, lr, lk, qs, ds);
}

int mg_build(mg_engine* e) {
    int rc = check_engine(e);
    if (rc) return rc;
    const mg_config& c = e->cfg;
    for (int idx = 0; idx < c.n_layers * 12 + 2; idx++) {
        bool is_matrix; int rows, cols, fmt;
        slot_info(c, idx, &is_matrix, &rows, &cols, &fmt);
        const int w = idx < c.n_layers * 12 ? idx % 12 : -1;
        if (w >= 4 && w <= 6) continue;   // biases are optional (cuda_fused_infer.go:255)
        // a pipeline stage holds its own layers; the final norm and lm_head go with the last layer
        if (w >= 0 && (idx / 12 < e->own_ls || idx / 12 >= e->own_le)) continue;
        if (w < 0 && e->own_le < c.n_layers) continue;
        if (is_matrix ? !e->mats[idx].set : e->vecs[idx] == nullptr)
            return fail(e, MG_ERR_STATE, "mg_build: weight slot %d has not been set", idx);
    }
    drop_graphs(e);
    if ((rc = build_mega(e))) return rc;
    e->built = true;
    return MG_OK;
}

int mg_reset_kv(mg_engine* e) {
    int rc = check_engine(e);
    if (rc) return rc;
    const size_t kv_bytes = (size_t)e->cfg.n_layers * e->cfg.max_seq * e->cfg.kv_dim * 2;
    MG_CUDA(e, cudaMemsetAsync(e->kc, 0, kv_bytes, e->stream));
    MG_CUDA(e, cudaMemsetAsync(e->vc, 0, kv_bytes, e->stream));
    MG_CUDA(e, cudaStreamSynchronize(e->stream));
    return MG_OK;
}

int mg_set_cursor(mg_engine* e, int token, int pos) {
    int rc = check_engine(e);
    if (rc) return rc;
    if (pos < 0 || pos >= e->cfg.max_seq || token < 0 || token >= e->cfg.vocab)
        return fail(e, MG_ERR_ARG, "mg_set_cursor: token %d / pos %d out of range", token, pos);
    MG_CUDA(e, cudaStreamSynchronize(e->stream));
    e->pin_i[0] = pos; e->pin_i[1] = token; e->pin_i[2] = 0;
    MG_CUDA(e, cudaMemcpyAsync(e->st, e->pin_i, 12, cudaMemcpyHostToDevice, e->stream));
    return MG_OK;
}

int mg_get_cursor(mg_engine* e, int* token, int* pos) {
    int rc = check_engine(e);
    if (rc) return rc;
    StepState s{};
    MG_CUDA(e, cudaMemcpyAsync(&s, e->st, sizeof s, cudaMemcpyDeviceToHost, e->stream));
    MG_CUDA(e, cudaStreamSynchronize(e->stream));
    if (token) *token = s.token;
    if (pos) *pos = s.pos;
    return check_mega_status(e);
}

int mg_sync(mg_engine* e) {
    int rc = check_engine(e);
    if (rc) return rc;
    MG_CUDA(e, cudaStreamSynchronize(e->stream));
    return check_mega_status(e);
}

int mg_partial_step(mg_engine* e, const float* hidden_in, int pos, int layer_start, int layer_end,
                    float* hidden_out, float* logits_out) {
    int rc = check_engine(e);
    if (rc) return rc;
    if ((rc = ensure_built(e))) return rc;
    const mg_config& c = e->cfg;
    if (!hidden_in || pos < 0 || pos >= c.max_seq || layer_start < 0 || layer_end < layer_start)
        return fail(e, MG_ERR_ARG, "mg_partial_step: bad arguments (pos %d, layers [%d,%d))", pos, layer_start, layer_end);
    if (layer_end > c.n_layers) layer_end = c.n_layers;
    MG_CUDA(e, cudaStreamSynchronize(e->stream));   // pin_i is reused
    e->pin_i[0] = pos; e->pin_i[1] = 0;
    MG_CUDA(e, cudaMemcpyAsync(e->st, e->pin_i, 8, cudaMemcpyHostToDevice, e->stream));
    MG_CUDA(e, cudaMemcpyAsync(e->h, hidden_in, (size_t)c.dim * 4, cudaMemcpyHostToDevice, e->stream));
    const bool want_logits = layer_end >= c.n_layers && logits_out;
    // A caller's page-locked logits buffer is written by lm_head's epilogue itself (the stores cross
    // PCIe while the phase streams its weights), which saves the 600 KB copy behind the kernel.
    float* direct = nullptr;
    if (want_logits && e->zero_copy && e->sh.size == 1 && e->mega_ok && layer_end > layer_start) {
        cudaPointerAttributes at{};
        if (cudaPointerGetAttributes(&at, logits_out) == cudaSuccess && at.type == cudaMemoryTypeHost && at.devicePointer)
            direct = static_cast<float*>(at.devicePointer);
        else
            cudaGetLastError();
    }
    e->logits_direct = direct;
    rc = run_step(e, layer_start, layer_end, MODE_HIDDEN, want_logits ? HEAD_LOGITS : HEAD_NONE);
    e->logits_direct = nullptr;
    if (rc) return rc;
    if (want_logits && !direct)
        MG_CUDA(e, cudaMemcpyAsync(logits_out, e->sh.size > 1 ? e->logits_all : e->logits, (size_t)c.vocab * 4,
                                   cudaMemcpyDeviceToHost, e->stream));
    else if (!want_logits && hidden_out)
        MG_CUDA(e, cudaMemcpyAsync(hidden_out, e->h, (size_t)c.dim * 4, cudaMemcpyDeviceToHost, e->stream));
    return check_mega_status(e);
}

int mg_set_layer_range(mg_engine* e, int layer_start, int layer_end) {
    int rc = check_engine(e);
    if (rc) return rc;
    if (layer_start < 0 || layer_end <= layer_start || layer_end > e->cfg.n_layers)
        return fail(e, MG_ERR_ARG, "mg_set_layer_range: bad range [%d,%d) of %d layers", layer_start, layer_end, e->cfg.n_layers);
    if (e->sh.size > 1) return fail(e, MG_ERR_UNSUPPORTED, "mg_set_layer_range: not combined with tensor parallelism");
    e->own_ls = layer_start; e->own_le = layer_end;
    e->built = false;
    return MG_OK;
}

int mg_partial_step_continue(mg_engine* e, int pos, int layer_start, int layer_end, float* hidden_out, float* logits_out) {
    int rc = check_engine(e);
    if (rc) return rc;
    if ((rc = ensure_built(e))) return rc;
    const mg_config& c = e->cfg;
    if (pos < 0 || pos >= c.max_seq || layer_start < 0 || layer_end < layer_start)
        return fail(e, MG_ERR_ARG, "mg_partial_step_continue: bad arguments (pos %d, layers [%d,%d))", pos, layer_start, layer_end);
    if (layer_end > c.n_layers) layer_end = c.n_layers;
    MG_CUDA(e, cudaStreamSynchronize(e->stream));   // pin_i is reused; a queued hidden state has landed after this
    e->pin_i[0] = pos; e->pin_i[1] = 0;
    MG_CUDA(e, cudaMemcpyAsync(e->st, e->pin_i, 8, cudaMemcpyHostToDevice, e->stream));
    const bool want_logits = layer_end >= c.n_layers && logits_out;
    if ((rc = run_step(e, layer_start, layer_end, MODE_HIDDEN, want_logits ? HEAD_LOGITS : HEAD_NONE))) return rc;
    if (want_logits)
        MG_CUDA(e, cudaMemcpyAsync(logits_out, e->logits, (size_t)c.vocab * 4, cudaMemcpyDeviceToHost, e->stream));
    else if (hidden_out)
        MG_CUDA(e, cudaMemcpyAsync(hidden_out, e->h, (size_t)c.dim * 4, cudaMemcpyDeviceToHost, e->stream));
    MG_CUDA(e, cudaStreamSynchronize(e->stream));
    return check_mega_status(e);
}

// ---- StepLayerResident (cuda_fused_infer_q4.go:451-605): one layer with snapshots of the hidden state
// before and after it; layer 0 takes the hidden state from the host, later layers continue on the
// device-resident one; logits_out asks for the final norm + lm_head on top of the layer's output.
int mg_step_layer_resident(mg_engine* e, int layer, int pos, const float* hidden_in, float* pre_out, float* post_out,
                           float* logits_out) {
    int rc = check_engine(e);
    if (rc) return rc;
    if ((rc = ensure_built(e))) return rc;
    const mg_config& c = e->cfg;
    if (layer < 0 || layer >= c.n_layers || pos < 0 || pos >= c.max_seq || (layer == 0 && !hidden_in))
        return fail(e, MG_ERR_ARG, "mg_step_layer_resident: bad arguments (layer %d, pos %d)", layer, pos);
    MG_CUDA(e, cudaStreamSynchronize(e->stream));
    e->pin_i[0] = pos; e->pin_i[1] = 0;
    MG_CUDA(e, cudaMemcpyAsync(e->st, e->pin_i, 8, cudaMemcpyHostToDevice, e->stream));
    if (layer == 0) MG_CUDA(e, cudaMemcpyAsync(e->h, hidden_in, (size_t)c.dim * 4, cudaMemcpyHostToDevice, e->stream));
    if (pre_out) MG_CUDA(e, cudaMemcpyAsync(pre_out, e->h, (size_t)c.dim * 4, cudaMemcpyDeviceToHost, e->stream));
    const bool last = layer == c.n_layers - 1;
    const bool fused_head = logits_out && last && !post_out;      // the head in the same launch (post_out needs the layer's output first)
    if ((rc = run_step(e, layer, layer + 1, MODE_HIDDEN, fused_head ? HEAD_LOGITS : HEAD_NONE))) return rc;
    if (post_out && !fused_head) MG_CUDA(e, cudaMemcpyAsync(post_out, e->h, (size_t)c.dim * 4, cudaMemcpyDeviceToHost, e->stream));
    if (logits_out && !fused_head) {
        // final norm + lm_head on the hidden state as it stands (the reference does this for any layer)
        if ((rc = run_step(e, c.n_layers, c.n_layers, MODE_HIDDEN, HEAD_LOGITS))) return rc;
    }
    if (logits_out)
        MG_CUDA(e, cudaMemcpyAsync(logits_out, e->sh.size > 1 ? e->logits_all : e->logits, (size_t)c.vocab * 4,
                                   cudaMemcpyDeviceToHost, e->stream));
    MG_CUDA(e, cudaStreamSynchronize(e->stream));
    return check_mega_status(e);
}

// ---- vNodes (cuda_fused_infer.go:630-684): the reference runs two pipeline stages of one GPU on two
// compute streams with separate scratch sets.  Here a stage is one persistent launch that occupies
// every SM, so two stages of one GPU cannot overlap; "stream 1" is kept as an ordering domain: work
// issued to it runs on the engine's stream behind whatever stream 1 was waiting for, and whatever waits
// on stream 1 afterwards waits for it.
int mg_set_vnode_count(mg_engine* e, int n) {
    int rc = check_engine(e);
    if (rc) return rc;
    if (n < 1 || n > 2) return fail(e, MG_ERR_ARG, "mg_set_vnode_count: 1 or 2 vNodes, not %d", n);
    if (n == 2 && !e->stream1) {
        MG_CUDA(e, cudaStreamCreateWithFlags(&e->stream1, cudaStreamNonBlocking));
        MG_CUDA(e, cudaEventCreateWithFlags(&e->stage_done, cudaEventDisableTiming));
        MG_CUDA(e, cudaEventCreateWithFlags(&e->s1_in, cudaEventDisableTiming));
        MG_CUDA(e, cudaEventCreateWithFlags(&e->s1_out, cudaEventDisableTiming));
    }
    e->vnodes = n;
    return MG_OK;
}
int mg_vnode_count(const mg_engine* e) { return e ? e->vnodes : 0; }

static int need_stream1(mg_engine* e, const char* what) {
    if (int rc = check_engine(e)) return rc;
    if (e->vnodes < 2 || !e->stream1) return fail(e, MG_ERR_STATE, "%s: call mg_set_vnode_count(e, 2) first", what);
    return MG_OK;
}
int mg_record_stage_done(mg_engine* e) {
    if (int rc = need_stream1(e, "mg_record_stage_done")) return rc;
    MG_CUDA(e, cudaEventRecord(e->stage_done, e->stream));
    return MG_OK;
}
int mg_wait_stage_done(mg_engine* e) {
    if (int rc = need_stream1(e, "mg_wait_stage_done")) return rc;
    MG_CUDA(e, cudaStreamWaitEvent(e->stream1, e->stage_done, 0));
    return MG_OK;
}
int mg_sync_stream1(mg_engine* e) {
    if (int rc = need_stream1(e, "mg_sync_stream1")) return rc;
    MG_CUDA(e, cudaStreamSynchronize(e->stream1));
    return check_mega_status(e);
}
// PartialStepQ4ContinueOnStream1 (cuda_fused_infer_q4.go:391-444): asynchronous; results are read after
// mg_sync_stream1 (hidden state: mg_export_hidden; logits: the pointer given here, written by a copy
// that stream 1 also waits for).
int mg_partial_step_continue_on_stream1(mg_engine* e, int pos, int layer_start, int layer_end, float* logits_out) {
    int rc = need_stream1(e, "mg_partial_step_continue_on_stream1");
    if (rc) return rc;
    if ((rc = ensure_built(e))) return rc;
    const mg_config& c = e->cfg;
    if (pos < 0 || pos >= c.max_seq || layer_start < 0 || layer_end < layer_start)
        return fail(e, MG_ERR_ARG, "mg_partial_step_continue_on_stream1: bad arguments (pos %d, layers [%d,%d))", pos, layer_start, layer_end);
    if (layer_end > c.n_layers) layer_end = c.n_layers;
    MG_CUDA(e, cudaStreamSynchronize(e->stream));   // pin_i is reused
    MG_CUDA(e, cudaEventRecord(e->s1_in, e->stream1));
    MG_CUDA(e, cudaStreamWaitEvent(e->stream, e->s1_in, 0));
    e->pin_i[0] = pos; e->pin_i[1] = 0;
    MG_CUDA(e, cudaMemcpyAsync(e->st, e->pin_i, 8, cudaMemcpyHostToDevice, e->stream));
    const bool want_logits = layer_end >= c.n_layers && logits_out;
    if ((rc = run_step(e, layer_start, layer_end, MODE_HIDDEN, want_logits ? HEAD_LOGITS : HEAD_NONE))) return rc;
    if (want_logits)
        MG_CUDA(e, cudaMemcpyAsync(logits_out, e->logits, (size_t)c.vocab * 4, cudaMemcpyDeviceToHost, e->stream));
    MG_CUDA(e, cudaEventRecord(e->s1_out, e->stream));
    MG_CUDA(e, cudaStreamWaitEvent(e->stream1, e->s1_out, 0));
    return MG_OK;
}
int mg_queue_hidden_to_l3_on_stream1(mg_engine* e) {
    if (int rc = need_stream1(e, "mg_queue_hidden_to_l3_on_stream1")) return rc;
    MG_CUDA(e, cudaEventRecord(e->compute_done, e->stream1));
    MG_CUDA(e, cudaStreamWaitEvent(e->copy_stream, e->compute_done, 0));
    MG_CUDA(e, cudaMemcpyAsync(e->l3, e->h, (size_t)e->cfg.dim * sizeof(float), cudaMemcpyDeviceToHost, e->copy_stream));
    MG_CUDA(e, cudaEventRecord(e->l3_done, e->copy_stream));
    MG_CUDA(e, cudaStreamWaitEvent(e->stream, e->l3_done, 0));
    MG_CUDA(e, cudaStreamWaitEvent(e->stream1, e->l3_done, 0));
    e->l3_queued = true;
    return MG_OK;
}

int mg_queue_hidden_to(mg_engine* src, mg_engine* dst) {
    int rc = check_engine(src);
    if (rc) return rc;
    if (!dst || dst == src || dst->cfg.dim != src->cfg.dim)
        return fail(src, MG_ERR_ARG, "mg_queue_hidden_to: the next stage must be another engine of the same width");
    const size_t bytes = (size_t)src->cfg.dim * sizeof(float);
    // the copy must not land while the next stage is still working on its previous hidden state
    if ((rc = check_engine(dst))) return rc;
    MG_CUDA(dst, cudaEventRecord(dst->compute_done, dst->stream));
    if ((rc = check_engine(src))) return rc;
    MG_CUDA(src, cudaStreamWaitEvent(src->stream, dst->compute_done, 0));
    if (src->cfg.device != dst->cfg.device) {
        // over NVLink when the two GPUs can address each other, staged by the driver otherwise
        int can = 0;
        cudaDeviceCanAccessPeer(&can, src->cfg.device, dst->cfg.device);
        if (can && cudaDeviceEnablePeerAccess(dst->cfg.device, 0) != cudaSuccess) cudaGetLastError();   // already on: fine
        MG_CUDA(src, cudaMemcpyPeerAsync(dst->h, dst->cfg.device, src->h, src->cfg.device, bytes, src->stream));
    } else {
        MG_CUDA(src, cudaMemcpyAsync(dst->h, src->h, bytes, cudaMemcpyDeviceToDevice, src->stream));
    }
    MG_CUDA(src, cudaEventRecord(src->sent_event, src->stream));
    // the next stage's stream orders itself after the copy; its host thread may also ask with mg_wait_mailbox
    if ((rc = check_engine(dst))) return rc;
    MG_CUDA(dst, cudaStreamWaitEvent(dst->stream, src->sent_event, 0));
    // the receiver asks its OWN event (recorded on its stream behind the wait for the copy): the sender
    // may be destroyed before mg_wait_mailbox is called
    MG_CUDA(dst, cudaEventRecord(dst->mail_event, dst->stream));
    dst->mail_queued++;
    return MG_OK;
}

int mg_wait_mailbox(mg_engine* e, int timeout_ms) {
    int rc = check_engine(e);
    if (rc) return rc;
    const auto t0 = std::chrono::steady_clock::now();
    auto expired = [&]() {
        return std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count() >= timeout_ms;
    };
    for (;;) {
        if (e->mail_queued != e->mail_taken) {
            const cudaError_t q = cudaEventQuery(e->mail_event);
            if (q == cudaSuccess) { e->mail_taken = e->mail_queued; return MG_OK; }
            if (q != cudaErrorNotReady) return fail(e, MG_ERR_CUDA, "mg_wait_mailbox: %s", cudaGetErrorString(q));
        }
        if (expired())
            return fail(e, MG_ERR_TIMEOUT, "mg_wait_mailbox: no hidden state arrived within %d ms (%s)", timeout_ms,
                        e->mail_queued != e->mail_taken ? "copy still in flight" : "nothing was queued");
        std::this_thread::yield();
    }
}

int mg_queue_hidden_to_l3(mg_engine* e) {
    int rc = check_engine(e);
    if (rc) return rc;
    MG_CUDA(e, cudaEventRecord(e->compute_done, e->stream));
    MG_CUDA(e, cudaStreamWaitEvent(e->copy_stream, e->compute_done, 0));
    MG_CUDA(e, cudaMemcpyAsync(e->l3, e->h, (size_t)e->cfg.dim * sizeof(float), cudaMemcpyDeviceToHost, e->copy_stream));
    MG_CUDA(e, cudaEventRecord(e->l3_done, e->copy_stream));
    // later steps overwrite the hidden state: they start once the copy (dim floats) has read it
    MG_CUDA(e, cudaStreamWaitEvent(e->stream, e->l3_done, 0));
    e->l3_queued = true;
    return MG_OK;
}

int mg_wait_l3(mg_engine* e, int timeout_ms) {
    int rc = check_engine(e);
    if (rc) return rc;
    if (!e->l3_queued) return fail(e, MG_ERR_STATE, "mg_wait_l3: nothing was queued");
    const auto t0 = std::chrono::steady_clock::now();
    for (;;) {
        const cudaError_t q = cudaEventQuery(e->l3_done);
        if (q == cudaSuccess) return MG_OK;
        if (q != cudaErrorNotReady) return fail(e, MG_ERR_CUDA, "mg_wait_l3: %s", cudaGetErrorString(q));
        if (std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count() >= timeout_ms)
            return fail(e, MG_ERR_TIMEOUT, "mg_wait_l3: the copy did not finish within %d ms", timeout_ms);
        std::this_thread::yield();
    }
}

const float* mg_l3_hidden(mg_engine* e) { return e ? e->l3 : nullptr; }

int mg_upload_hidden(mg_engine* e, const float* hidden) {
    int rc = check_engine(e);
    if (rc) return rc;
    if (!hidden) return MG_ERR_ARG;
    MG_CUDA(e, cudaMemcpyAsync(e->h, hidden, (size_t)e->cfg.dim * 4, cudaMemcpyHostToDevice, e->stream));
    MG_CUDA(e, cudaStreamSynchronize(e->stream));
    return MG_OK;
}

int mg_graph_launch(mg_engine* e, int pos, int layer_start, int layer_end) {
    int rc = check_engine(e);
    if (rc) return rc;
    if ((rc = ensure_built(e))) return rc;
    const mg_config& c = e->cfg;
    if (pos < 0 || pos >= c.max_seq || layer_start < 0 || layer_end < layer_start)
        return fail(e, MG_ERR_ARG, "mg_graph_launch: bad arguments (pos %d, layers [%d,%d))", pos, layer_start, layer_end);
    if (layer_end > c.n_layers) layer_end = c.n_layers;
    MG_CUDA(e, cudaStreamSynchronize(e->stream));   // the pinned cursor words are reused
    e->pin_i[0] = pos; e->pin_i[1] = 0;
    MG_CUDA(e, cudaMemcpyAsync(e->st, e->pin_i, 8, cudaMemcpyHostToDevice, e->stream));
    return run_step(e, layer_start, layer_end, MODE_HIDDEN, HEAD_NONE);
}

int mg_validate_replay(mg_engine* e, const float* hidden_in, int layer_start, int layer_end, float* max_diff) {
    int rc = check_engine(e);
    if (rc) return rc;
    if ((rc = ensure_built(e))) return rc;
    if (!hidden_in || !max_diff) return MG_ERR_ARG;
    const int dim = e->cfg.dim;
    std::vector<float> plain(dim), replay(dim);
    // plain launches of the per-phase kernels, one by one, no graph and no persistent kernel
    const bool mega = e->mega_ok, graph = e->use_graph;
    e->mega_ok = false; e->use_graph = false;
    rc = mg_reset_kv(e);
    if (!rc) rc = mg_partial_step(e, hidden_in, 0, layer_start, layer_end, nullptr, nullptr);
    if (!rc) rc = mg_export_hidden(e, plain.data());
    e->mega_ok = mega; e->use_graph = graph;
    if (rc) return rc;
    // the path every other call uses
    if ((rc = mg_reset_kv(e))) return rc;
    if ((rc = mg_upload_hidden(e, hidden_in))) return rc;
    if ((rc = mg_graph_launch(e, 0, layer_start, layer_end))) return rc;
    if ((rc = mg_export_hidden(e, replay.data()))) return rc;
    if ((rc = check_mega_status(e))) return rc;
    float d = 0.f;
    for (int i = 0; i < dim; i++) {
        const float x = fabsf(plain[i] - replay[i]);
        if (!(x <= d)) d = x;      // NaN propagates into the result
    }
    *max_diff = d;
    return MG_OK;
}

int mg_export_hidden(mg_engine* e, float* hidden_out) {
    int rc = check_engine(e);
    if (rc) return rc;
    if (!hidden_out) return MG_ERR_ARG;
    MG_CUDA(e, cudaMemcpyAsync(hidden_out, e->h, (size_t)e->cfg.dim * 4, cudaMemcpyDeviceToHost, e->stream));
    MG_CUDA(e, cudaStreamSynchronize(e->stream));
    return MG_OK;
}

int mg_step_token(mg_engine* e, int token, int pos, int* next_token, float* logits_out) {
    int rc = check_engine(e);
    if (rc) return rc;
    if ((rc = ensure_built(e))) return rc;
    const mg_config& c = e->cfg;
    if (token < 0 || token >= c.vocab || pos < 0 || pos >= c.max_seq)
        return fail(e, MG_ERR_ARG, "mg_step_token: token %d / pos %d out of range", token, pos);
    MG_CUDA(e, cudaStreamSynchronize(e->stream));
    e->pin_i[0] = pos; e->pin_i[1] = token;
    MG_CUDA(e, cudaMemcpyAsync(e->st, e->pin_i, 8, cudaMemcpyHostToDevice, e->stream));
    if ((rc = run_step(e, 0, c.n_layers, MODE_EMBED, logits_out ? HEAD_LOGITS : HEAD_ARGMAX))) return rc;
    if (logits_out)
        MG_CUDA(e, cudaMemcpyAsync(logits_out, e->sh.size > 1 ? e->logits_all : e->logits, (size_t)c.vocab * 4,
                                   cudaMemcpyDeviceToHost, e->stream));
    MG_CUDA(e, cudaMemcpyAsync(e->pin_i + 4, &e->st->token, 4, cudaMemcpyDeviceToHost, e->stream));
    MG_CUDA(e, cudaStreamSynchronize(e->stream));
    if (next_token) *next_token = e->pin_i[4];
    return check_mega_status(e);
}

int mg_enqueue_greedy(mg_engine* e, int n_steps) {
    int rc = check_engine(e);
    if (rc) return rc;
    if ((rc = ensure_built(e))) return rc;
    if (n_steps <= 0) return MG_OK;
    if ((rc = check_range(e, 0, e->cfg.n_layers, true, true))) return rc;
    if (e->mega_ok) return launch_mega(e, 0, e->cfg.n_layers, MODE_EMBED, HEAD_ARGMAX, n_steps);
    for (int i = 0; i < n_steps; i++)
        if ((rc = run_step(e, 0, e->cfg.n_layers, MODE_EMBED, HEAD_ARGMAX))) return rc;
    return MG_OK;
}

int mg_generate(mg_engine* e, const int* prompt, int n_prompt, int n_new, int start_pos, int* out_tokens) {
    int rc = check_engine(e);
    if (rc) return rc;
    if ((rc = ensure_built(e))) return rc;
    const mg_config& c = e->cfg;
    if (!prompt || n_prompt < 1 || n_new < 1 || !out_tokens || start_pos < 0 ||
        start_pos + n_prompt + n_new - 1 > c.max_seq || n_prompt + n_new > e->out_cap)
        return fail(e, MG_ERR_ARG, "mg_generate: %d prompt + %d new tokens from position %d do not fit max_seq %d",
                    n_prompt, n_new, start_pos, c.max_seq);
    for (int i = 0; i < n_prompt; i++)
        if (prompt[i] < 0 || prompt[i] >= c.vocab) return fail(e, MG_ERR_ARG, "mg_generate: prompt id out of range");
    if ((rc = check_range(e, 0, c.n_layers, true, true))) return rc;
    MG_CUDA(e, cudaStreamSynchronize(e->stream));
    e->pin_i[0] = start_pos; e->pin_i[1] = prompt[0]; e->pin_i[2] = 0;
    for (int i = 0; i < n_prompt; i++) e->pin_i[8 + i] = prompt[i];
    MG_CUDA(e, cudaMemcpyAsync(e->st, e->pin_i, 12, cudaMemcpyHostToDevice, e->stream));
    const int total = n_prompt + n_new - 1;
    for (int i = 0; i < n_prompt; i++) {
        if (i > 0)   // prompt tokens override the fed-back argmax
            MG_CUDA(e, cudaMemcpyAsync(&e->st->token, e->pin_i + 8 + i, 4, cudaMemcpyHostToDevice, e->stream));
        if ((rc = run_step(e, 0, c.n_layers, MODE_EMBED, HEAD_ARGMAX))) return rc;
    }
    if (total > n_prompt) {
        if (e->mega_ok) {
            if ((rc = launch_mega(e, 0, c.n_layers, MODE_EMBED, HEAD_ARGMAX, total - n_prompt))) return rc;
        } else {
            for (int i = n_prompt; i < total; i++)
                if ((rc = run_step(e, 0, c.n_layers, MODE_EMBED, HEAD_ARGMAX))) return rc;
        }
    }
    MG_CUDA(e, cudaMemcpyAsync(out_tokens, e->out_tokens + (n_prompt - 1), (size_t)n_new * 4, cudaMemcpyDeviceToHost,
                               e->stream));
    MG_CUDA(e, cudaStreamSynchronize(e->stream));
    return check_mega_status(e);
}

int mg_dequant_rows(mg_engine* e, int idx, int row0, int nrows, float* out) {
    int rc = check_engine(e);
    if (rc) return rc;
    if (!out || idx < 0 || idx >= (int)e->mats.size() || !e->mats[idx].set)
        return fail(e, MG_ERR_ARG, "mg_dequant_rows: slot %d is not a set matrix", idx);
    const DevMatrix& m = e->mats[idx];
    if (row0 < 0 || nrows < 0 || row0 + nrows > m.rows) return fail(e, MG_ERR_ARG, "mg_dequant_rows: rows out of range");
    const int K = m.cols, nb = K / 32, rb = plane_row_bytes(m.fmt, K);
    std::vector<uint8_t> qs((size_t)nrows * rb);
    std::vector<unsigned short> ds(m.fmt == FMT_F16 ? 0 : (size_t)nrows * nb);
    MG_CUDA(e, cudaStreamSynchronize(e->stream));
    MG_CUDA(e, cudaMemcpy(qs.data(), m.qs + (size_t)row0 * rb, qs.size(), cudaMemcpyDeviceToHost));
    if (!ds.empty()) MG_CUDA(e, cudaMemcpy(ds.data(), m.ds + (size_t)row0 * nb, ds.size() * 2, cudaMemcpyDeviceToHost));
    for (int r = 0; r < nrows; r++)
        for (int k = 0; k < K; k++) {
            float v;
            if (m.fmt == FMT_F16) {
                v = __half2float(__ushort_as_half(reinterpret_cast<unsigned short*>(qs.data())[(size_t)r * K + k]));
            } else {
                const float d = __half2float(__ushort_as_half(ds[(size_t)r * nb + k / 32]));
                if (m.fmt == FMT_Q8_0) {
                    v = d * (float)reinterpret_cast<int8_t*>(qs.data())[(size_t)r * K + k];
                } else {
                    const int b = k / 32, j = k % 32;
                    const uint8_t byte = qs[(size_t)r * (K / 2) + b * 16 + (j & 15)];
                    v = d * (float)((j < 16 ? (byte & 0xF) : (byte >> 4)) - 8);
                }
            }
            out[(size_t)r * K + k] = v;
        }
    return MG_OK;
}

int mg_read_kv(mg_engine* e, int layer, int pos0, int npos, uint16_t* k_out, uint16_t* v_out) {
    int rc = check_engine(e);
    if (rc) return rc;
    const mg_config& c = e->cfg;
    if (layer < 0 || layer >= c.n_layers || pos0 < 0 || npos < 0 || pos0 + npos > c.max_seq)
        return fail(e, MG_ERR_ARG, "mg_read_kv: out of range");
    const int kv_dim = (e->sh.kv1 - e->sh.kv0) * c.head_dim;   // this rank's KV heads
    const size_t off = ((size_t)layer * c.max_seq + pos0) * kv_dim;
    const size_t bytes = (size_t)npos * kv_dim * 2;
    MG_CUDA(e, cudaStreamSynchronize(e->stream));
    if (k_out) MG_CUDA(e, cudaMemcpy(k_out, e->kc + off, bytes, cudaMemcpyDeviceToHost));
    if (v_out) MG_CUDA(e, cudaMemcpy(v_out, e->vc + off, bytes, cudaMemcpyDeviceToHost));
    return MG_OK;
}

int mg_trace_step(mg_engine* e, long long* stamps, int capacity, int* n_ctas, int* n_events) {
    int rc = check_engine(e);
    if (rc) return rc;
    if ((rc = ensure_built(e))) return rc;
    if (!e->mega_ok) return fail(e, MG_ERR_UNSUPPORTED, "mg_trace_step: the persistent kernel is not in use (%s)", e->err.c_str());
    const int ev = MK_TRACE_EVENTS(e->cfg.n_layers), G = e->num_sms;
    if (!stamps || capacity < G * ev) return fail(e, MG_ERR_ARG, "mg_trace_step: need room for %d stamps", G * ev);
    if (!e->mk_trace) MG_CUDA(e, ARENA_MALLOC(e, &e->mk_trace, (size_t)G * ev * 8));
    MG_CUDA(e, cudaMemsetAsync(e->mk_trace, 0, (size_t)G * ev * 8, e->stream));
    e->trace_next = true;
    if ((rc = launch_mega(e, 0, e->cfg.n_layers, MODE_EMBED, HEAD_ARGMAX, 1))) return rc;
    MG_CUDA(e, cudaMemcpyAsync(stamps, e->mk_trace, (size_t)G * ev * 8, cudaMemcpyDeviceToHost, e->stream));
    MG_CUDA(e, cudaStreamSynchronize(e->stream));
    if (n_ctas) *n_ctas = G;
    if (n_events) *n_events = ev;
    return check_mega_status(e);
}

// ---- raw device memory from the engine's arena: the counterparts of tw_gpu_alloc / upload / download /
// zero (cuda_tensor.go:19-44) and ArenaStats (gpu_alloc.go:58-66) for callers that keep their own
// device buffers (scratch vectors, caller-owned weights for the mongoose_* entry points).
int mg_device_alloc(mg_engine* e, size_t bytes, void** out) {
    int rc = check_engine(e);
    if (rc) return rc;
    if (!out) return MG_ERR_ARG;
    *out = e->arena.alloc(bytes);
    if (!*out) return fail(e, MG_ERR_NOMEM, "mg_device_alloc: %zu bytes not available", bytes);
    return MG_OK;
}
int mg_device_free(mg_engine* e, void* p) {
    int rc = check_engine(e);
    if (rc) return rc;
    e->arena.release(p);
    return MG_OK;
}
int mg_device_upload(mg_engine* e, void* dst, const void* host, size_t bytes) {
    int rc = check_engine(e);
    if (rc) return rc;
    if (!dst || !host) return MG_ERR_ARG;
    MG_CUDA(e, cudaMemcpy(dst, host, bytes, cudaMemcpyHostToDevice));
    return MG_OK;
}
int mg_device_download(mg_engine* e, void* host, const void* src, size_t bytes) {
    int rc = check_engine(e);
    if (rc) return rc;
    if (!src || !host) return MG_ERR_ARG;
    MG_CUDA(e, cudaMemcpy(host, src, bytes, cudaMemcpyDeviceToHost));
    return MG_OK;
}
int mg_device_zero(mg_engine* e, void* dst, size_t bytes) {
    int rc = check_engine(e);
    if (rc) return rc;
    if (!dst) return MG_ERR_ARG;
    MG_CUDA(e, cudaMemset(dst, 0, bytes));
    return MG_OK;
}
int mg_arena_stats(const mg_engine* e, size_t* total, size_t* in_use, size_t* peak, size_t* largest_free, int* outside) {
    if (!e) return MG_ERR_ARG;
    if (total) *total = e->arena.size;
    if (in_use) *in_use = e->arena.in_use;
    if (peak) *peak = e->arena.peak;
    if (largest_free) *largest_free = e->arena.largest_free();
    if (outside) *outside = (int)e->arena.outside.size();
    return MG_OK;
}

int mg_decode_path(const mg_engine* e) {
    if (!e) return MG_ERR_ARG;
    return (e->mega_ok ? 1 : 0) | (e->mega_ok && e->ffn_fused ? 2 : 0) | (e->tp_fused ? 4 : 0);
}

int mg_set_wait_limit_ms(mg_engine* e, int ms) {
    if (!e || ms <= 0) return MG_ERR_ARG;
    e->mk_wait = (long long)ms * 2000000ll;
    return MG_OK;
}

int mg_tp_partition(const mg_config* cfg, int rank, int size, mg_tp_shard* out) {
    if (!cfg || !out) return MG_ERR_ARG;
    if (cfg->n_heads <= 0 || cfg->n_kv_heads <= 0 || cfg->n_heads % cfg->n_kv_heads || cfg->ffn_dim % 32 || cfg->vocab <= 0)
        return MG_ERR_ARG;
    Shard s;
    std::string why;
    if (!make_shard(*cfg, rank, size, &s, &why)) return MG_ERR_UNSUPPORTED;
    out->q_head0 = s.q0; out->q_head1 = s.q1; out->kv_head0 = s.kv0; out->kv_head1 = s.kv1;
    out->ffn0 = s.f0; out->ffn1 = s.f1; out->vocab0 = s.v0; out->vocab1 = s.v1;
    return MG_OK;
}

int mg_tp_unique_id(void* id_out, size_t bytes) {
    if (!id_out || bytes < sizeof(ncclUniqueId)) return MG_ERR_ARG;
    std::string why;
    if (!load_nccl(&why)) {
        fprintf(stderr, "[mongoose-b200] %s\n", why.c_str());
        return MG_ERR_UNSUPPORTED;
    }
    ncclUniqueId id;
    if (g_nccl.GetUniqueId(&id) != ncclSuccess) return MG_ERR_CUDA;
    memcpy(id_out, &id, sizeof id);
    return MG_OK;
}

int mg_tp_init(mg_engine* e, int rank, int size, const void* id, size_t bytes) {
    int rc = check_engine(e);
    if (rc) return rc;
    if (e->any_weight_set || e->comm) return fail(e, MG_ERR_STATE, "mg_tp_init: call once, before any weight is set");
    if (size == 1 && rank == 0) return MG_OK;
    if (!id || bytes < sizeof(ncclUniqueId)) return fail(e, MG_ERR_ARG, "mg_tp_init: need the %zu-byte id of mg_tp_unique_id", sizeof(ncclUniqueId));
    std::string why;
    Shard s;
    if (!make_shard(e->cfg, rank, size, &s, &why)) return fail(e, MG_ERR_UNSUPPORTED, "mg_tp_init: %s", why.c_str());
    if (s.v1 <= s.v0) return fail(e, MG_ERR_UNSUPPORTED, "mg_tp_init: rank %d would hold no vocabulary rows", rank);
    if (!load_nccl(&why)) return fail(e, MG_ERR_UNSUPPORTED, "mg_tp_init: %s", why.c_str());
    ncclUniqueId uid;
    memcpy(&uid, id, sizeof uid);
    MG_NCCL(e, g_nccl.CommInitRank(&e->comm, size, uid, rank));
    if ((rc = dev_alloc(e, &e->zero_vec, (size_t)e->cfg.dim))) return rc;
    if ((rc = dev_alloc(e, &e->logits_all, (size_t)s.v_stride * size))) return rc;
    MG_CUDA(e, cudaMemset(e->zero_vec, 0, (size_t)e->cfg.dim * 4));
    e->sh = s;
    // Receive buffer of the fused exchange, mapped into every peer through CUDA IPC.  Where a peer
    // cannot be mapped (or MG_TP_NCCL=1 asks for it) the partial sums go through ncclAllReduce.
    const char* env = getenv("MG_TP_NCCL");
    bool want_fused = !(env && env[0] == '1') && size <= kMaxRanks;
    {
        // an allocation of its own, not a piece of the arena: CUDA IPC maps whole allocations into the peers
        MG_CUDA(e, cudaMalloc((void**)&e->xchg, xchg_bytes(e)));
        e->dev_bytes += xchg_bytes(e);
        if ((rc = dev_alloc(e, &e->xchg_status, (size_t)1))) return rc;
        MG_CUDA(e, cudaMemset(e->xchg, 0, xchg_bytes(e)));
        MG_CUDA(e, cudaMemset(e->xchg_status, 0, sizeof(XchgStatus)));
        cudaIpcMemHandle_t mine{};
        int ok = want_fused && cudaIpcGetMemHandle(&mine, e->xchg) == cudaSuccess ? 1 : 0;
        if (!ok) cudaGetLastError();
        // every rank learns every handle (and whether its owner could make one) in one all-gather
        const size_t rec = sizeof(cudaIpcMemHandle_t) + 8;
        uint8_t* d_all = nullptr;
        MG_CUDA(e, cudaMalloc((void**)&d_all, rec * size));
        std::vector<uint8_t> h_all(rec * size, 0);
        memcpy(h_all.data() + rec * rank, &mine, sizeof mine);
        h_all[rec * rank + sizeof mine] = (uint8_t)ok;
        MG_CUDA(e, cudaMemcpy(d_all, h_all.data(), rec * size, cudaMemcpyHostToDevice));
        MG_NCCL(e, g_nccl.AllGather(d_all + rec * rank, d_all, rec, ncclChar, e->comm, e->stream));
        MG_CUDA(e, cudaStreamSynchronize(e->stream));
        MG_CUDA(e, cudaMemcpy(h_all.data(), d_all, rec * size, cudaMemcpyDeviceToHost));
        int all_ok = 1;
        for (int p = 0; p < size; p++) all_ok &= h_all[rec * p + sizeof mine];
        int opened = all_ok;
        if (all_ok) {
            for (int p = 0; p < size && opened; p++) {
                if (p == rank) { e->xchg_peer[p] = e->xchg; continue; }
                cudaIpcMemHandle_t hnd;
                memcpy(&hnd, h_all.data() + rec * p, sizeof hnd);
                void* ptr = nullptr;
                if (cudaIpcOpenMemHandle(&ptr, hnd, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
                    cudaGetLastError();
                    opened = 0;
                } else {
                    e->xchg_peer[p] = static_cast<uint8_t*>(ptr);
                }
            }
        }
        // agree: the fused path is used only if every rank mapped every peer
        int* d_flag = reinterpret_cast<int*>(d_all);
        MG_CUDA(e, cudaMemcpy(d_flag, &opened, sizeof(int), cudaMemcpyHostToDevice));
        MG_NCCL(e, g_nccl.AllReduce(d_flag, d_flag, 1, ncclInt, ncclMin, e->comm, e->stream));
        MG_CUDA(e, cudaStreamSynchronize(e->stream));
        MG_CUDA(e, cudaMemcpy(&opened, d_flag, sizeof(int), cudaMemcpyDeviceToHost));
        cudaFree(d_all);
        e->tp_fused = opened != 0;
        if (!e->tp_fused) e->err = "tensor-parallel exchange through ncclAllReduce (peer mapping unavailable or MG_TP_NCCL=1)";
    }
    // Programmatic dependent launch stays off under tensor parallelism, on both exchange paths: the
    // per-phase kernels alternate with library collectives (NCCL path), and with the in-kernel exchange
    // an early-launched consumer would spin on words that a peer's not-yet-running kernel must write.
    e->use_pdl = false;
    e->built = false;
    return MG_OK;
}

// Test aid for the in-kernel exchange deadline on ONE GPU: rank 0 of a `size`-rank group whose peers do
// not exist.  The receive buffer is this engine's own, every "peer" pointer aliases it, and nothing
// ever writes the other ranks' rows: the first wait for them runs out after the wait limit
// (mg_set_wait_limit_ms), the kernel records which exchange it was and returns, and the step reports
// MG_ERR_TIMEOUT.  No NCCL communicator is made; only the greedy / hidden-state calls are meaningful.
int mg_tp_init_absent_peers(mg_engine* e, int size) {
    int rc = check_engine(e);
    if (rc) return rc;
    if (e->any_weight_set || e->comm || e->xchg) return fail(e, MG_ERR_STATE, "mg_tp_init_absent_peers: call once, before any weight is set");
    if (size < 2 || size > kMaxRanks) return fail(e, MG_ERR_ARG, "mg_tp_init_absent_peers: 2..%d ranks", kMaxRanks);
    std::string why;
    Shard s;
    if (!make_shard(e->cfg, 0, size, &s, &why)) return fail(e, MG_ERR_UNSUPPORTED, "mg_tp_init_absent_peers: %s", why.c_str());
    e->sh = s;
    MG_CUDA(e, cudaMalloc((void**)&e->xchg, xchg_bytes(e)));
    e->dev_bytes += xchg_bytes(e);
    if ((rc = dev_alloc(e, &e->xchg_status, (size_t)1))) return rc;
    MG_CUDA(e, cudaMemset(e->xchg, 0, xchg_bytes(e)));
    MG_CUDA(e, cudaMemset(e->xchg_status, 0, sizeof(XchgStatus)));
    for (int p = 0; p < size; p++) e->xchg_peer[p] = e->xchg;
    e->tp_fused = true;
    e->absent_peers = true;
    e->use_pdl = false;
    e->built = false;
    return MG_OK;
}

cudaStream_t mg_stream(mg_engine* e) { return e ? e->stream : nullptr; }
long long mg_launch_count(const mg_engine* e) { return e ? e->launches : 0; }
size_t mg_device_bytes(const mg_engine* e) { return e ? e->dev_bytes : 0; }
const char* mg_last_error(const mg_engine* e) { return e ? e->err.c_str() : "null engine"; }

}  // extern "C"
