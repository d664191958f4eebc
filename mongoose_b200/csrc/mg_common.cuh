// Shared device helpers for the sm_100a decode kernels.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define MG_WARP 32
#define MG_FULL_MASK 0xffffffffu

// Weight storage formats (values match MG_FMT_* in mongoose_kernels.h).
enum : int { FMT_Q8_0 = 0, FMT_Q4_0 = 1, FMT_F16 = 2 };

namespace mg {

// ---------------------------------------------------------------------
// Programmatic dependent launch.  A kernel launched with the
// programmatic-stream-serialization attribute may start while its
// predecessor is still running; everything before pdl_wait() must touch
// only memory the predecessor never writes (weights).  Without the
// attribute both instructions are no-ops.
// ---------------------------------------------------------------------
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// 16-byte streaming load of read-only weight data (evict-first: each weight
// byte is used once per token).
__device__ __forceinline__ uint4 ld_stream16(const void* p) {
    return __ldcs(reinterpret_cast<const uint4*>(p));
}
__device__ __forceinline__ unsigned short ld_stream_u16(const void* p) {
    return __ldcs(reinterpret_cast<const unsigned short*>(p));
}

__device__ __forceinline__ float half_bits_to_float(unsigned short h) {
    return __half2float(__ushort_as_half(h));
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(MG_FULL_MASK, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(MG_FULL_MASK, v, o));
    return v;
}

// Sum over a whole CTA; every thread gets the result.  `red` is >= 33 floats
// of shared memory.  Deterministic: warp partials are added in warp order.
__device__ __forceinline__ float block_sum(float v, float* red) {
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int nw = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) red[wid] = v;
    __syncthreads();
    if (wid == 0) {
        float t = lane < nw ? red[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

// ---------------------------------------------------------------------
// int8 -> fp32 without the conversion pipe: a byte placed in the low
// mantissa of 2^23 reads as 8388608 + u; with u = q xor 0x80 (= q + 128)
// subtracting 8388736 gives q exactly.
// ---------------------------------------------------------------------
__device__ __forceinline__ float s8_to_f32_magic(uint32_t w_xor80, int byte) {
    // selector: result byte0 = w.byte, bytes 1..3 = 0x00,0x00,0x4B
    uint32_t r;
    const uint32_t sel = 0x7654u & 0xfff0u | (uint32_t)byte;  // b3<-c.b3(7) b2<-c.b2(6) b1<-c.b1(5) b0<-a.byte
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(w_xor80), "r"(0x4B000000u), "r"(sel));
    return __uint_as_float(r) - 8388736.0f;
}

// Dot of 4 packed int8 with 4 floats.
__device__ __forceinline__ float dot4_s8(uint32_t w, float4 x, float acc) {
    const uint32_t u = w ^ 0x80808080u;
    acc = fmaf(s8_to_f32_magic(u, 0), x.x, acc);
    acc = fmaf(s8_to_f32_magic(u, 1), x.y, acc);
    acc = fmaf(s8_to_f32_magic(u, 2), x.z, acc);
    acc = fmaf(s8_to_f32_magic(u, 3), x.w, acc);
    return acc;
}

// Nibble n (0..15) in the low mantissa of 2^23, minus (2^23 + 8) = n - 8 exactly.
__device__ __forceinline__ float u4_to_f32_magic(uint32_t nibbles_as_bytes, int byte) {
    uint32_t r;
    const uint32_t sel = 0x7650u | (uint32_t)byte;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(nibbles_as_bytes), "r"(0x4B000000u), "r"(sel));
    return __uint_as_float(r) - 8388616.0f;
}

// ---------------------------------------------------------------------
// Per-format chunk traits.  A chunk is 16 bytes of the weight plane:
//   Q8_0: 16 int8  = half a block      (x slice: 16 floats)
//   Q4_0: 32 nibbles = one block, byte j = element j (low) / j+16 (high)
//   F16 : 8 halves                      (x slice: 8 floats)
// chunk_dot returns sum_i x[i] * q[i] for the chunk (unscaled for Q8/Q4).
// ---------------------------------------------------------------------
template <int FMT>
struct Chunk;

template <>
struct Chunk<FMT_Q8_0> {
    static constexpr int kWeights = 16;
    static constexpr bool kScaled = true;
    // chunk c of a row belongs to block c/2
    __device__ static __forceinline__ int scale_index(int c) { return c >> 1; }
    __device__ static __forceinline__ float dot(uint4 w, const float4* x) {
        float a = 0.f;
        a = dot4_s8(w.x, x[0], a);
        a = dot4_s8(w.y, x[1], a);
        a = dot4_s8(w.z, x[2], a);
        a = dot4_s8(w.w, x[3], a);
        return a;
    }
};

template <>
struct Chunk<FMT_Q4_0> {
    static constexpr int kWeights = 32;
    static constexpr bool kScaled = true;
    __device__ static __forceinline__ int scale_index(int c) { return c; }
    __device__ static __forceinline__ float dot(uint4 w, const float4* x) {
        // word i holds bytes 4i..4i+3: low nibbles are elements 4i..4i+3, high nibbles 16+4i..16+4i+3
        float a = 0.f;
        const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint32_t lo = ws[i] & 0x0f0f0f0fu;
            const uint32_t hi = (ws[i] >> 4) & 0x0f0f0f0fu;
            const float4 xl = x[i], xh = x[4 + i];
            a = fmaf(u4_to_f32_magic(lo, 0), xl.x, a);
            a = fmaf(u4_to_f32_magic(lo, 1), xl.y, a);
            a = fmaf(u4_to_f32_magic(lo, 2), xl.z, a);
            a = fmaf(u4_to_f32_magic(lo, 3), xl.w, a);
            a = fmaf(u4_to_f32_magic(hi, 0), xh.x, a);
            a = fmaf(u4_to_f32_magic(hi, 1), xh.y, a);
            a = fmaf(u4_to_f32_magic(hi, 2), xh.z, a);
            a = fmaf(u4_to_f32_magic(hi, 3), xh.w, a);
        }
        return a;
    }
};

template <>
struct Chunk<FMT_F16> {
    static constexpr int kWeights = 8;
    static constexpr bool kScaled = false;
    __device__ static __forceinline__ int scale_index(int c) { return c; }
    __device__ static __forceinline__ float dot(uint4 w, const float4* x) {
        const __half2* h = reinterpret_cast<const __half2*>(&w);
        const float2 a0 = __half22float2(h[0]), a1 = __half22float2(h[1]);
        const float2 a2 = __half22float2(h[2]), a3 = __half22float2(h[3]);
        float a = 0.f;
        a = fmaf(a0.x, x[0].x, a);
        a = fmaf(a0.y, x[0].y, a);
        a = fmaf(a1.x, x[0].z, a);
        a = fmaf(a1.y, x[0].w, a);
        a = fmaf(a2.x, x[1].x, a);
        a = fmaf(a2.y, x[1].y, a);
        a = fmaf(a3.x, x[1].z, a);
        a = fmaf(a3.y, x[1].w, a);
        return a;
    }
};

// Device-side view of one weight matrix in the engine's layout:
//   qs : rows * row_bytes bytes, rows contiguous, 16-byte aligned rows
//   ds : rows * K/32 fp16 block scales (NULL for F16)
struct WeightView {
    const uint8_t* qs;
    const unsigned short* ds;
};

__host__ __device__ inline int plane_row_bytes(int fmt, int K) {
    return fmt == FMT_Q8_0 ? K : fmt == FMT_Q4_0 ? K / 2 : K * 2;
}

// ---------------------------------------------------------------------
// Integer dot products against fixed-point activations: a group of 16
// activations is s * t_i with 24-bit integers t = a2*65536 + a1*256 + a0
// (a2 signed byte, a1 and a0 unsigned bytes) held as three byte planes.
// ---------------------------------------------------------------------
__device__ __forceinline__ uint4 lds16(const void* p) { return *reinterpret_cast<const uint4*>(p); }
// signed weights x {unsigned, unsigned, signed} activation bytes
__device__ __forceinline__ int dp4a_su(uint32_t w, uint32_t a, int acc) {
    int r;
    asm("dp4a.s32.u32 %0, %1, %2, %3;" : "=r"(r) : "r"(w), "r"(a), "r"(acc));
    return r;
}
__device__ __forceinline__ int dp4a_ss(uint32_t w, uint32_t a, int acc) {
    int r;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(r) : "r"(w), "r"(a), "r"(acc));
    return r;
}
__device__ __forceinline__ int dp4a_uu(uint32_t w, uint32_t a, int acc) {
    int r;
    asm("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(r) : "r"(w), "r"(a), "r"(acc));
    return r;
}
__device__ __forceinline__ int dp4a_us(uint32_t w, uint32_t a, int acc) {
    int r;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(r) : "r"(w), "r"(a), "r"(acc));
    return r;
}

// 16 signed int8 weights (one uint4) against one activation group: exact integer sum, as float.
__device__ __forceinline__ float group_dot_s8(uint4 w, uint4 p0, uint4 p1, uint4 p2) {
    int i0 = dp4a_su(w.x, p0.x, 0), i1 = dp4a_su(w.x, p1.x, 0), i2 = dp4a_ss(w.x, p2.x, 0);
    i0 = dp4a_su(w.y, p0.y, i0); i1 = dp4a_su(w.y, p1.y, i1); i2 = dp4a_ss(w.y, p2.y, i2);
    i0 = dp4a_su(w.z, p0.z, i0); i1 = dp4a_su(w.z, p1.z, i1); i2 = dp4a_ss(w.z, p2.z, i2);
    i0 = dp4a_su(w.w, p0.w, i0); i1 = dp4a_su(w.w, p1.w, i1); i2 = dp4a_ss(w.w, p2.w, i2);
    return fmaf((float)i2, 65536.0f, fmaf((float)i1, 256.0f, (float)i0));
}
// 16 unsigned nibbles (as bytes in four words) against one activation group.
__device__ __forceinline__ float group_dot_u4(uint32_t n0, uint32_t n1, uint32_t n2, uint32_t n3, uint4 p0, uint4 p1,
                                              uint4 p2) {
    int i0 = dp4a_uu(n0, p0.x, 0), i1 = dp4a_uu(n0, p1.x, 0), i2 = dp4a_us(n0, p2.x, 0);
    i0 = dp4a_uu(n1, p0.y, i0); i1 = dp4a_uu(n1, p1.y, i1); i2 = dp4a_us(n1, p2.y, i2);
    i0 = dp4a_uu(n2, p0.z, i0); i1 = dp4a_uu(n2, p1.z, i1); i2 = dp4a_us(n2, p2.z, i2);
    i0 = dp4a_uu(n3, p0.w, i0); i1 = dp4a_uu(n3, p1.w, i1); i2 = dp4a_us(n3, p2.w, i2);
    return fmaf((float)i2, 65536.0f, fmaf((float)i1, 256.0f, (float)i0));
}


}  // namespace mg
