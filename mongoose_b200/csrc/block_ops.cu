// Matvecs on caller-owned RAW quantized blocks (GGUF Q4_0 18-byte blocks,
// Q8_0 34-byte blocks), the int8-activation (dp4a) family, and the fused
// per-token dispatch over caller-owned buffers.
//
// The Go side declares these entry points (kernels.go:62-67, 206-211;
// cuda_graph.go:211-234) but the reference ships no source for them; the
// block layout is the one cuda_q4_0.go:13-17 uploads.  Raw blocks are only
// 2-byte aligned; the engine (mg_*) re-packs blocks at upload and does not
// use this file's kernels.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>

#include <mutex>

#include "../../include/mongoose_kernels.h"
#include "mg_common.cuh"

using namespace mg;

namespace {

struct __align__(8) ActBlock {   // 40 bytes per 32 activations
    float d;                     // amax / 127
    float s;                     // d * sum(q)
    int8_t q[32];
};
static_assert(sizeof(ActBlock) == 40, "activation block is 40 bytes");

// ---------------- fp32-activation matvecs on raw blocks ----------------
// Raw GGUF blocks (34 / 18 bytes) are only 2-byte aligned, so a lane cannot fetch its block with a
// vector load.  Instead a warp takes a CHUNK of 32 consecutive blocks of a row - a contiguous byte
// range - and copies the aligned 4-byte words that cover it from global to shared memory, lane by
// lane (coalesced, every weight byte read once); each lane then pulls the words of ITS block out of
// shared memory, re-aligns them with a funnel shift by 16 or 32 bits, and multiplies them with the
// activation slice staged once per CTA.  One warp walks rows warp, warp + nwarps, ...; the 32 block
// sums meet in a shuffle reduction.
constexpr int kRawWarps = 8;
template <int FMT>
__global__ void __launch_bounds__(kRawWarps * 32) raw_block_matvec_kernel(const float* __restrict__ act,
                                                                         const uint8_t* __restrict__ w, float* out, int N,
                                                                         int K) {
    constexpr int BB = FMT == FMT_Q8_0 ? 34 : 18;           // bytes per block
    constexpr int QW = FMT == FMT_Q8_0 ? 8 : 4;             // 4-byte words of quants per block
    constexpr int CW = (32 * BB + 3) / 4 + 1;               // words that cover a chunk, whatever its alignment
    extern __shared__ __align__(16) float raw_xs[];         // K floats, then kRawWarps * CW words
    uint32_t* stage = reinterpret_cast<uint32_t*>(raw_xs + K) + (threadIdx.x >> 5) * CW;
    const int lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < K; i += blockDim.x) raw_xs[i] = act[i];
    __syncthreads();
    const int nb = K / 32;
    const int nwarps = gridDim.x * kRawWarps;
    for (int row = blockIdx.x * kRawWarps + (threadIdx.x >> 5); row < N; row += nwarps) {
        const size_t row0 = (size_t)row * nb * BB;           // byte offset of the row (always even)
        float acc = 0.f;
        for (int b0 = 0; b0 < nb; b0 += 32) {
            const int nblk = min(32, nb - b0);
            const size_t c0 = row0 + (size_t)b0 * BB, c1 = c0 + (size_t)nblk * BB;
            const size_t a0 = ((size_t)(w + c0)) & ~(size_t)3;                       // first aligned word (address)
            const int nw = (int)((((size_t)(w + c1)) + 3 - a0) >> 2);
            const uint32_t* src = reinterpret_cast<const uint32_t*>(a0);
            for (int i = lane; i < nw; i += 32) stage[i] = __ldcs(src + i);
            __syncwarp();
            if (lane < nblk) {
                const int off = (int)((size_t)(w + c0) - a0) + lane * BB;               // this block inside the staged words
                const uint32_t* q = stage + (off >> 2);
                const int sh = (off & 2) ? 32 : 16;                                     // quants start 2 bytes after the scale
                const uint32_t w0 = q[0];
                const float d = half_bits_to_float((unsigned short)((off & 2) ? (w0 >> 16) : (w0 & 0xffffu)));
                uint32_t qw[QW];
#pragma unroll
                for (int i = 0; i < QW; i++) qw[i] = __funnelshift_rc(q[i], q[i + 1], sh);
                const float4* x = reinterpret_cast<const float4*>(raw_xs + (size_t)(b0 + lane) * 32);
                float s;
                if (FMT == FMT_Q8_0)
                    s = Chunk<FMT_Q8_0>::dot(make_uint4(qw[0], qw[1], qw[2], qw[3]), x) +
                        Chunk<FMT_Q8_0>::dot(make_uint4(qw[4], qw[5], qw[6], qw[7]), x + 4);
                else
                    s = Chunk<FMT_Q4_0>::dot(make_uint4(qw[0], qw[1], qw[2], qw[3]), x);
                acc = fmaf(d, s, acc);
            }
            __syncwarp();
        }
        acc = warp_sum(acc);
        if (lane == 0) out[row] = acc;
    }
}
template <int FMT>
inline size_t raw_matvec_smem(int K) {
    return (size_t)K * 4 + (size_t)kRawWarps * ((32 * (FMT == FMT_Q8_0 ? 34 : 18) + 3) / 4 + 1) * 4;
}

// ---------------- activation quantizer: one warp per block of 32 ----------------
__global__ void __launch_bounds__(256) quantize_act_kernel(const float* __restrict__ act, ActBlock* out,
                                                          int nblocks_total) {
    const int lane = threadIdx.x & 31;
    const int blk = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (blk >= nblocks_total) return;
    const float v = act[(size_t)blk * 32 + lane];
    const float amax = warp_max(fabsf(v));
    const float d = amax / 127.0f;
    const int q = amax > 0.f ? __float2int_rn(v / d) : 0;
    int sum = q;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(MG_FULL_MASK, sum, o);
    out[blk].q[lane] = (int8_t)q;
    if (lane == 0) {
        out[blk].d = d;
        out[blk].s = d * (float)sum;
    }
}

// ---------------- Q4_0 x int8 activations, integer dot products ----------------
// out[b][row] = sum_blocks d_w * (d_a * sum_j nib_j * qa_j - 8 * s_a)
__global__ void __launch_bounds__(256) q4_0_dp4a_kernel(const uint8_t* __restrict__ w,
                                                       const ActBlock* __restrict__ q8, float* out, int N, int K,
                                                       int B) {
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= N) return;
    const int nb = K / 32;
    const uint8_t* wr = w + (size_t)row * nb * 18;
    for (int bi = 0; bi < B; bi++) {
        const ActBlock* qa = q8 + (size_t)bi * nb;
        float acc = 0.f;
        for (int b = lane; b < nb; b += 32) {
            const unsigned short* p = reinterpret_cast<const unsigned short*>(wr + (size_t)b * 18);
            const float dw = half_bits_to_float(p[0]);
            const int* aq = reinterpret_cast<const int*>(qa[b].q);
            int sumi = 0;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const uint32_t word = (uint32_t)p[1 + 2 * i] | ((uint32_t)p[2 + 2 * i] << 16);
                const int lo = (int)(word & 0x0f0f0f0fu), hi = (int)((word >> 4) & 0x0f0f0f0fu);
                sumi = __dp4a(lo, aq[i], sumi);
                sumi = __dp4a(hi, aq[4 + i], sumi);
            }
            acc = fmaf(dw, qa[b].d * (float)sumi - 8.0f * qa[b].s, acc);
        }
        acc = warp_sum(acc);
        if (lane == 0) out[(size_t)bi * N + row] = acc;
    }
}

inline int cdiv(int a, int b) { return (a + b - 1) / b; }

// ---- scratch that lives in the library image, for callers that must not allocate ----
// 40 bytes per 32 activations; 32768 input features at most.
constexpr int kStaticMaxK = 32768;
constexpr size_t kStaticScratchBytes = (size_t)(kStaticMaxK / 32) * sizeof(ActBlock);
static __device__ __align__(256) unsigned char g_static_act_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_static_mu;
void* g_static_ptr[kMaxDevices] = {};      // device address of g_static_act_scratch on each device
thread_local char g_static_err[256] = "";

int static_fail(int code, const char* fmt, int a, int b) {
    snprintf(g_static_err, sizeof g_static_err, fmt, a, b);
    return code;
}

// Grid: every SM gets the same number of CTAs (rows are walked with a stride), enough warps to hide
// the loads.  Wide inputs need more than the default 48 KB of dynamic shared memory: raised once.
template <int FMT>
static void launch_raw_matvec(const float* act, const void* w_blocks, float* out, int N, int K, cudaStream_t stream) {
    if (N <= 0 || K < 32 || K % 32) return;
    static int sms = 0;
    static bool raised = false;
    if (!sms) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (sms <= 0) sms = 148;
    }
    const size_t smem = raw_matvec_smem<FMT>(K);
    if (smem > 48 * 1024 && !raised) {
        cudaFuncSetAttribute((const void*)raw_block_matvec_kernel<FMT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        raised = true;
    }
    const int per_sm = smem > 100 * 1024 ? 1 : smem > 48 * 1024 ? 2 : 4;
    const int grid = std::min(cdiv(N, kRawWarps), sms * per_sm);
    raw_block_matvec_kernel<FMT><<<grid, kRawWarps * 32, smem, stream>>>(act, (const uint8_t*)w_blocks, out, N, K);
}

}  // namespace

extern "C" {

void mongoose_q4_0_matvec(const float* act, const void* w_blocks, float* out, int N, int K, cudaStream_t stream) {
    launch_raw_matvec<FMT_Q4_0>(act, w_blocks, out, N, K, stream);
}

void mongoose_q8_0_matvec(const float* act, const void* w_blocks, float* out, int N, int K, cudaStream_t stream) {
    launch_raw_matvec<FMT_Q8_0>(act, w_blocks, out, N, K, stream);
}

void mongoose_q8_quantize_act(const float* act, void* q8_out, int K, cudaStream_t stream) {
    if (K < 32) return;
    quantize_act_kernel<<<cdiv(K / 32, 8), 256, 0, stream>>>(act, (ActBlock*)q8_out, K / 32);
}

void mongoose_q8_quantize_act_batch(const float* acts, void* q8_out, int K, int B, cudaStream_t stream) {
    if (K < 32 || B <= 0) return;
    const int total = (K / 32) * B;
    quantize_act_kernel<<<cdiv(total, 8), 256, 0, stream>>>(acts, (ActBlock*)q8_out, total);
}

void mongoose_q4_0_matvec_dp4a_preq(const void* w_blocks, const void* q8, float* out, int N, int K,
                                    cudaStream_t stream) {
    if (N <= 0 || K < 32) return;
    q4_0_dp4a_kernel<<<cdiv(N, 8), 256, 0, stream>>>((const uint8_t*)w_blocks, (const ActBlock*)q8, out, N, K, 1);
}

void mongoose_q4_0_matvec_dp4a_batch(const void* w_blocks, const void* q8, float* out, int N, int K, int B,
                                     cudaStream_t stream) {
    if (N <= 0 || K < 32 || B <= 0) return;
    q4_0_dp4a_kernel<<<cdiv(N, 8), 256, 0, stream>>>((const uint8_t*)w_blocks, (const ActBlock*)q8, out, N, K, B);
}

void mongoose_q4_0_matvec_dp4a(const float* act, const void* w_blocks, float* out, int N, int K, void* scratch,
                               cudaStream_t stream) {
    if (N <= 0 || K < 32 || !scratch) return;
    mongoose_q8_quantize_act(act, scratch, K, stream);
    mongoose_q4_0_matvec_dp4a_preq(w_blocks, scratch, out, N, K, stream);
}

// Q4_0 integer-dot matvec that allocates nothing.
//
// Who needs it: code that may not call cudaMalloc at the moment it wants a matvec - a capture-time
// or latency-critical section that forbids allocator calls, a plugin host that owns the memory
// budget and hands out no more, or a caller running after the pool it was given is exhausted.  The
// activation blocks (40 bytes per 32 inputs) that mongoose_q4_0_matvec_dp4a wants in a caller
// buffer live instead in a fixed array inside the library image (40 KiB, room for K <= 32768),
// present on every GPU that loads the library until the process exits.
//
// The array's name is only a host-side handle; the device address is looked up once per device with
// cudaGetSymbolAddress while that device is current.  That lookup happens on the FIRST call on a
// device, so make the first call outside any stream capture.  The address is remembered per device
// for the life of the process: after cudaDeviceReset() the library must not be used on that device
// again (the remembered address belongs to the destroyed context).  Every call overwrites the whole
// region it uses before reading it, so nothing needs clearing between calls, but all calls share
// the one array: two calls that overlap on the GPU (different streams, different threads) race.
// Returns MG_OK, MG_ERR_ARG (NULL pointer, K not a multiple of 32, or K > 32768) or MG_ERR_CUDA;
// mongoose_static_scratch_error() has the text.
int mongoose_q4_0_matvec_dp4a_static(const float* act, const void* w_blocks, float* out, int N, int K,
                                     cudaStream_t stream) {
    g_static_err[0] = 0;
    if (!act || !w_blocks || !out) return static_fail(MG_ERR_ARG, "NULL pointer argument (N=%d K=%d)", N, K);
    if (N <= 0 || K < 32 || K % 32) return static_fail(MG_ERR_ARG, "N=%d must be positive and K=%d a multiple of 32", N, K);
    if (K > kStaticMaxK)
        return static_fail(MG_ERR_ARG, "K=%d exceeds the built-in scratch limit of %d input features", K, kStaticMaxK);
    int dev = -1;
    cudaError_t ce = cudaGetDevice(&dev);
    if (ce != cudaSuccess || dev < 0 || dev >= kMaxDevices)
        return static_fail(MG_ERR_CUDA, "cudaGetDevice failed or device ordinal %d is out of range (%d)", dev, (int)ce);
    void* scratch;
    {
        std::lock_guard<std::mutex> lk(g_static_mu);
        if (!g_static_ptr[dev]) {
            void* p = nullptr;
            ce = cudaGetSymbolAddress(&p, g_static_act_scratch);
            if (ce != cudaSuccess || !p)
                return static_fail(MG_ERR_CUDA, "cudaGetSymbolAddress failed on device %d (error %d)", dev, (int)ce);
            g_static_ptr[dev] = p;
        }
        scratch = g_static_ptr[dev];
    }
    // Each launch's own status is checked: an error that an earlier, unrelated call left behind is
    // cleared first so that it is not taken for one of ours (a sticky error - a faulted context -
    // comes back from the next check all the same, and is reported as what it is).
    (void)cudaGetLastError();
    quantize_act_kernel<<<cdiv(K / 32, 8), 256, 0, stream>>>(act, (ActBlock*)scratch, K / 32);
    if ((ce = cudaGetLastError()) != cudaSuccess)
        return static_fail(MG_ERR_CUDA, "launch of the activation quantizer failed on device %d (CUDA error %d)", dev, (int)ce);
    q4_0_dp4a_kernel<<<cdiv(N, 8), 256, 0, stream>>>((const uint8_t*)w_blocks, (const ActBlock*)scratch, out, N, K, 1);
    if ((ce = cudaGetLastError()) != cudaSuccess)
        return static_fail(MG_ERR_CUDA, "launch of the matvec failed on device %d (CUDA error %d)", dev, (int)ce);
    return MG_OK;
}

const char* mongoose_static_scratch_error(void) { return g_static_err; }

// The reference's per-token op order (cuda_fused_infer.go:414-444 / cuda_fused_infer_q4.go:103-131)
// issued from one C call on caller-owned buffers.
void mongoose_partial_step_q4_fused_graph(
    const float** norm1, const void** wq, const void** wk, const void** wv, const void** wo,
    const float** norm2, const void** wgate, const void** wup, const void** wdown,
    float** kCache, float** vCache,
    float* hidden, float* normed, float* Q, float* K, float* V,
    float* attnOut, float* proj, float* normed2,
    float* gatePre, float* upOut, float* ffnMid,
    void* q8Scratch,
    const float* cosTab, const float* sinTab,
    int dim, int kvDim, int headDim, int ffnDim, int nHeads, int nKVHeads, int halfHead,
    int pos, int layerStart, int layerEnd,
    cudaStream_t stream) {
    (void)q8Scratch;   // fp32 activations throughout: no activation quantization on this path
    const float* cosRow = cosTab + (size_t)pos * halfHead;
    const float* sinRow = sinTab + (size_t)pos * halfHead;
    for (int l = layerStart; l < layerEnd; l++) {
        mongoose_rmsnorm_out(hidden, normed, norm1[l], 1, dim, stream);
        mongoose_q4_0_matvec(normed, wq[l], Q, dim, dim, stream);
        mongoose_q4_0_matvec(normed, wk[l], K, kvDim, dim, stream);
        mongoose_q4_0_matvec(normed, wv[l], V, kvDim, dim, stream);
        mongoose_rope(Q, cosRow, sinRow, 1, dim, headDim, nHeads, stream);
        mongoose_rope(K, cosRow, sinRow, 1, kvDim, headDim, nKVHeads, stream);
        mongoose_kv_cache_write(kCache[l], K, pos, kvDim, stream);
        mongoose_kv_cache_write(vCache[l], V, pos, kvDim, stream);
        mongoose_decode_attention(Q, kCache[l], vCache[l], attnOut, pos + 1, dim, kvDim, nHeads, nKVHeads, stream);
        mongoose_q4_0_matvec(attnOut, wo[l], proj, dim, dim, stream);
        mongoose_add_inplace(hidden, proj, dim, stream);
        mongoose_rmsnorm_out(hidden, normed2, norm2[l], 1, dim, stream);
        mongoose_q4_0_matvec(normed2, wgate[l], gatePre, ffnDim, dim, stream);
        mongoose_q4_0_matvec(normed2, wup[l], upOut, ffnDim, dim, stream);
        mongoose_silu_gate_mul(gatePre, upOut, ffnMid, ffnDim, stream);
        mongoose_q4_0_matvec(ffnMid, wdown[l], proj, dim, ffnDim, stream);
        mongoose_add_inplace(hidden, proj, dim, stream);
    }
}

}  // extern "C"
