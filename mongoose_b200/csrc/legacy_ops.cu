// The mongoose_* entry points that mongoose's Go side binds with dlsym
// (kernels.go:150-226), re-implemented for sm_100a.  Layouts and semantics
// are the reference's: caller-owned fp32 device buffers, per-row INT8/INT4
// weights with fp32 row scales, fp32 KV cache, work enqueued on the given
// stream, no allocation, no status.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "../../include/mongoose_kernels.h"
#include "mg_common.cuh"

using namespace mg;

namespace {

inline int ew_blocks(int n, int per_block) { return (n + per_block - 1) / per_block; }

// ---------------- RMSNorm family (eps 1e-6, kernels/mongoose.cu:170) ----------------
template <bool ADD>
__global__ void __launch_bounds__(256) rmsnorm_rows_kernel(const float* a, const float* b, float* out,
                                                           const float* __restrict__ w, int dim) {
    __shared__ float red[40];
    const size_t base = (size_t)blockIdx.x * dim;
    float ss = 0.f;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        float v = a[base + i];
        if (ADD) v += b[base + i];
        ss = fmaf(v, v, ss);
    }
    const float tot = block_sum(ss, red);
    const float scale = rsqrtf(tot / (float)dim + 1e-6f);
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        float v = a[base + i];
        if (ADD) v += b[base + i];
        out[base + i] = v * scale * w[i];
    }
}

__global__ void relu_kernel(float* x, int n) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
        if (x[i] < 0.f) x[i] = 0.f;
}

__global__ void add_inplace_kernel(float* a, const float* __restrict__ b, int n) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) a[i] += b[i];
}

__global__ void silu_gate_mul_kernel(const float* __restrict__ g, const float* __restrict__ u, float* out, int n) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const float x = g[i];
        out[i] = x * (1.0f / (1.0f + expf(-x))) * u[i];
    }
}

template <bool POS>
__global__ void gather_rows_kernel(float* out, const float* __restrict__ emb, const float* __restrict__ posEmb,
                                   const int* __restrict__ tokens, int dim) {
    const int p = blockIdx.x;
    const size_t src = (size_t)tokens[p] * dim, dst = (size_t)p * dim;
    for (int j = threadIdx.x; j < dim; j += blockDim.x) {
        float v = emb[src + j];
        if (POS) v += posEmb[dst + j];
        out[dst + j] = v;
    }
}

// Rotate-half RoPE; grid = (seqLen, nHeads); table row = sequence index.
__global__ void rope_kernel(float* x, const float* __restrict__ cosT, const float* __restrict__ sinT, int dim,
                            int headDim, int half) {
    const int pos = blockIdx.x, h = blockIdx.y;
    const size_t base = (size_t)pos * dim + (size_t)h * headDim;
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
        const float c = cosT[(size_t)pos * half + j], s = sinT[(size_t)pos * half + j];
        const float x0 = x[base + j], x1 = x[base + half + j];
        x[base + j] = x0 * c - x1 * s;
        x[base + half + j] = x0 * s + x1 * c;
    }
}

__global__ void kv_write_kernel(float* cache, const float* __restrict__ src, int pos, int kvDim) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < kvDim) cache[(size_t)pos * kvDim + i] = src[i];
}

__global__ void f32_to_f16_kernel(const float* __restrict__ in, __half* out, int n) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
        out[i] = __float2half_rn(in[i]);
}
__global__ void f16_to_f32_kernel(const __half* __restrict__ in, float* out, int n) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
        out[i] = __half2float(in[i]);
}

// ---------------- decode attention, fp32 KV (kernels/mongoose.cu:853-933) ----------------
// One CTA per head.  Scores live in dynamic shared memory (cacheLen floats),
// as in the reference.  Lane-per-position dot products, then threads split
// (position group, dim) for the weighted V sum.
__global__ void __launch_bounds__(256) decode_attention_f32_kernel(const float* __restrict__ Q,
                                                                  const float* __restrict__ Kc,
                                                                  const float* __restrict__ Vc, float* out,
                                                                  int cacheLen, int kvDim, int numHeads,
                                                                  int numKVHeads, int hd) {
    extern __shared__ __align__(16) float sm[];
    float* red = sm;                 // 40
    float* qs = sm + 40;             // hd
    float* part = qs + hd;           // 256 partials
    float* sc = part + 256;          // cacheLen
    const int head = blockIdx.x, tid = threadIdx.x;
    const int kvOff = (head / (numHeads / numKVHeads)) * hd;
    const float scale = rsqrtf((float)hd);
    for (int d = tid; d < hd; d += blockDim.x) qs[d] = Q[(size_t)head * hd + d];
    __syncthreads();
    float mx = -INFINITY;
    for (int t = tid; t < cacheLen; t += blockDim.x) {
        const float* kr = Kc + (size_t)t * kvDim + kvOff;
        float dot = 0.f;
        for (int d = 0; d < hd; d++) dot = fmaf(qs[d], kr[d], dot);
        dot *= scale;
        sc[t] = dot;
        mx = fmaxf(mx, dot);
    }
    mx = warp_max(mx);
    {
        const int lane = tid & 31, wid = tid >> 5, nw = blockDim.x >> 5;
        if (lane == 0) red[wid] = mx;
        __syncthreads();
        float m = lane < nw ? red[lane] : -INFINITY;
        mx = warp_max(m);
        __syncthreads();
    }
    float sum = 0.f;
    for (int t = tid; t < cacheLen; t += blockDim.x) {
        const float p = expf(sc[t] - mx);
        sc[t] = p;
        sum += p;
    }
    sum = block_sum(sum, red);
    // threads = G groups x hd dims (hd <= 256)
    const int G = blockDim.x / hd > 0 ? blockDim.x / hd : 1;
    const int g = tid / hd, d = tid % hd;
    if (g < G && tid < G * hd) {
        float acc = 0.f;
        for (int t = g; t < cacheLen; t += G) acc = fmaf(sc[t], Vc[(size_t)t * kvDim + kvOff + d], acc);
        part[tid] = acc;
    }
    __syncthreads();
    if (tid < hd) {
        float s = 0.f;
        for (int gg = 0; gg < G; gg++) s += part[gg * hd + tid];
        out[(size_t)head * hd + tid] = s / sum;
    }
}

// ---------------- per-row INT8 / INT4 matvecs ----------------
// One warp per output row; 16-byte weight loads when the row stride allows,
// fp32 accumulate, scale applied once at the end: out = (scales[r]/127) * sum.
__global__ void __launch_bounds__(256) rowq8_matvec_kernel(const float* __restrict__ act,
                                                          const int8_t* __restrict__ w,
                                                          const float* __restrict__ scales, float* out, int N,
                                                          int K, int vec_ok) {
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= N) return;
    const int8_t* wr = w + (size_t)row * K;
    float acc = 0.f;
    int k0 = 0;
    if (vec_ok) {
        const int nch = K / 16;
        for (int c = lane; c < nch; c += 32) {
            const uint4 ww = ld_stream16(wr + (size_t)c * 16);
            const float4* xp = reinterpret_cast<const float4*>(act + (size_t)c * 16);
            acc = dot4_s8(ww.x, __ldg(xp + 0), acc);
            acc = dot4_s8(ww.y, __ldg(xp + 1), acc);
            acc = dot4_s8(ww.z, __ldg(xp + 2), acc);
            acc = dot4_s8(ww.w, __ldg(xp + 3), acc);
        }
        k0 = nch * 16;
    }
    for (int k = k0 + lane; k < K; k += 32) acc = fmaf(act[k], (float)wr[k], acc);
    acc = warp_sum(acc);
    if (lane == 0) out[row] = acc * (scales[row] / 127.0f);
}

// byte k of a row holds element 2k in the low nibble and 2k+1 in the high nibble.
__global__ void __launch_bounds__(256) rowq4_matvec_kernel(const float* __restrict__ act,
                                                          const uint8_t* __restrict__ w,
                                                          const float* __restrict__ scales, float* out, int N,
                                                          int K, int vec_ok) {
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= N) return;
    const int halfK = K / 2;
    const uint8_t* wr = w + (size_t)row * halfK;
    float acc = 0.f;
    int b0 = 0;
    if (vec_ok) {
        const int nch = halfK / 16;   // 16 bytes = 32 elements
        for (int c = lane; c < nch; c += 32) {
            const uint4 ww = ld_stream16(wr + (size_t)c * 16);
            const uint32_t ws[4] = {ww.x, ww.y, ww.z, ww.w};
            const float4* xp = reinterpret_cast<const float4*>(act + (size_t)c * 32);
#pragma unroll
            for (int i = 0; i < 4; i++) {
                // word i: bytes 4i..4i+3 -> elements 8i..8i+7, interleaved low/high
                const uint32_t lo = ws[i] & 0x0f0f0f0fu, hi = (ws[i] >> 4) & 0x0f0f0f0fu;
                const float4 xa = __ldg(xp + 2 * i), xb = __ldg(xp + 2 * i + 1);
                acc = fmaf(u4_to_f32_magic(lo, 0), xa.x, acc);
                acc = fmaf(u4_to_f32_magic(hi, 0), xa.y, acc);
                acc = fmaf(u4_to_f32_magic(lo, 1), xa.z, acc);
                acc = fmaf(u4_to_f32_magic(hi, 1), xa.w, acc);
                acc = fmaf(u4_to_f32_magic(lo, 2), xb.x, acc);
                acc = fmaf(u4_to_f32_magic(hi, 2), xb.y, acc);
                acc = fmaf(u4_to_f32_magic(lo, 3), xb.z, acc);
                acc = fmaf(u4_to_f32_magic(hi, 3), xb.w, acc);
            }
        }
        b0 = nch * 16;
    }
    for (int k = b0 + lane; k < halfK; k += 32) {
        const uint8_t p = wr[k];
        acc = fmaf(act[2 * k], (float)((int)(p & 0xF) - 8), acc);
        acc = fmaf(act[2 * k + 1], (float)((int)(p >> 4) - 8), acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) out[row] = acc * (scales[row] / 7.0f);
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

extern "C" {

void mongoose_rmsnorm(float* x, const float* weight, int seqLen, int dim, cudaStream_t stream) {
    if (seqLen <= 0 || dim <= 0) return;
    rmsnorm_rows_kernel<false><<<seqLen, 256, 0, stream>>>(x, nullptr, x, weight, dim);
}

void mongoose_rmsnorm_out(const float* in, float* out, const float* weight, int seqLen, int dim,
                          cudaStream_t stream) {
    if (seqLen <= 0 || dim <= 0) return;
    rmsnorm_rows_kernel<false><<<seqLen, 256, 0, stream>>>(in, nullptr, out, weight, dim);
}

void mongoose_fused_add_rmsnorm(const float* a, const float* b, float* out, const float* weight, int seqLen,
                                int dim, cudaStream_t stream) {
    if (seqLen <= 0 || dim <= 0) return;
    rmsnorm_rows_kernel<true><<<seqLen, 256, 0, stream>>>(a, b, out, weight, dim);
}

void mongoose_relu(float* x, int n, cudaStream_t stream) {
    if (n <= 0) return;
    relu_kernel<<<min(ew_blocks(n, 256), 1184), 256, 0, stream>>>(x, n);
}

void mongoose_add_inplace(float* a, const float* b, int n, cudaStream_t stream) {
    if (n <= 0) return;
    add_inplace_kernel<<<min(ew_blocks(n, 256), 1184), 256, 0, stream>>>(a, b, n);
}

void mongoose_silu_gate_mul(const float* gate, const float* up, float* out, int n, cudaStream_t stream) {
    if (n <= 0) return;
    silu_gate_mul_kernel<<<min(ew_blocks(n, 256), 1184), 256, 0, stream>>>(gate, up, out, n);
}

void mongoose_embedding_gather(float* out, const float* tokEmb, const float* posEmb, const int* tokens,
                               int seqLen, int dim, cudaStream_t stream) {
    if (seqLen <= 0 || dim <= 0) return;
    gather_rows_kernel<true><<<seqLen, 256, 0, stream>>>(out, tokEmb, posEmb, tokens, dim);
}

void mongoose_embed_gather(float* out, const float* embed, const int* tokens, int seqLen, int dim,
                           cudaStream_t stream) {
    if (seqLen <= 0 || dim <= 0) return;
    gather_rows_kernel<false><<<seqLen, 256, 0, stream>>>(out, embed, nullptr, tokens, dim);
}

void mongoose_rope(float* x, const float* cosTab, const float* sinTab, int seqLen, int dim, int headDim,
                   int nHeads, cudaStream_t stream) {
    if (seqLen <= 0 || nHeads <= 0 || headDim < 2) return;
    const int half = headDim / 2;
    int threads = half < 32 ? 32 : half > 256 ? 256 : ((half + 31) / 32) * 32;
    rope_kernel<<<dim3(seqLen, nHeads), threads, 0, stream>>>(x, cosTab, sinTab, dim, headDim, half);
}

void mongoose_kv_cache_write(float* cache, const float* src, int pos, int kvDim, cudaStream_t stream) {
    if (kvDim <= 0) return;
    kv_write_kernel<<<ew_blocks(kvDim, 256), 256, 0, stream>>>(cache, src, pos, kvDim);
}

void mongoose_decode_attention(const float* Q, const float* Kcache, const float* Vcache, float* out,
                               int cacheLen, int dim, int kvDim, int nHeads, int nKVHeads,
                               cudaStream_t stream) {
    if (cacheLen <= 0 || nHeads <= 0 || nKVHeads <= 0) return;
    const int hd = dim / nHeads;
    if (hd <= 0 || hd > 256) return;
    const size_t smem = (size_t)(40 + hd + 256 + cacheLen) * sizeof(float);
    if (smem > 200 * 1024) return;   // ~50k cached positions; longer contexts are not supported on this entry point
    if (smem > 48 * 1024)            // per-device attribute, cheap and idempotent
        cudaFuncSetAttribute((const void*)decode_attention_f32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             200 * 1024);
    decode_attention_f32_kernel<<<nHeads, 256, smem, stream>>>(Q, Kcache, Vcache, out, cacheLen, kvDim, nHeads,
                                                               nKVHeads, hd);
}

void mongoose_q8_matvec(const float* act, const void* w_i8, const float* scales, float* out, int N, int K,
                        cudaStream_t stream) {
    if (N <= 0 || K <= 0) return;
    const int vec_ok = (K % 16 == 0) && aligned16(w_i8) && aligned16(act);
    rowq8_matvec_kernel<<<ew_blocks(N, 8), 256, 0, stream>>>(act, (const int8_t*)w_i8, scales, out, N, K, vec_ok);
}

void mongoose_q4_matvec(const float* act, const void* w_packed, const float* scales, float* out, int N, int K,
                        cudaStream_t stream) {
    if (N <= 0 || K <= 0) return;
    const int vec_ok = ((K / 2) % 16 == 0) && aligned16(w_packed) && aligned16(act);
    rowq4_matvec_kernel<<<ew_blocks(N, 8), 256, 0, stream>>>(act, (const uint8_t*)w_packed, scales, out, N, K,
                                                            vec_ok);
}

void mongoose_copy(void* dst, const void* src, size_t bytes, cudaStream_t stream) {
    cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, stream);
}
void mongoose_zero(void* ptr, size_t bytes, cudaStream_t stream) { cudaMemsetAsync(ptr, 0, bytes, stream); }
void mongoose_sync(cudaStream_t stream) { cudaStreamSynchronize(stream); }

void mongoose_fp32_to_fp16(const float* in, void* out, int n, cudaStream_t stream) {
    if (n <= 0) return;
    f32_to_f16_kernel<<<min(ew_blocks(n, 256), 1184), 256, 0, stream>>>(in, (__half*)out, n);
}
void mongoose_fp16_to_fp32(const void* in, float* out, int n, cudaStream_t stream) {
    if (n <= 0) return;
    f16_to_f32_kernel<<<min(ew_blocks(n, 256), 1184), 256, 0, stream>>>((const __half*)in, out, n);
}

}  // extern "C"
