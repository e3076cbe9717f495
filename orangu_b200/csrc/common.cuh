// Shared device helpers and host-side error plumbing for the sm_100a kernels.
//
// The whole library is compiled with -fmad=false: the arithmetic being reproduced
// (the reference engine's CPU path) never fuses a*b+c, and the per-row fp32 results
// are meant to match it bit for bit.  Where a fused multiply-add is wanted (attention),
// it is spelled __fmaf_rn explicitly.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <string>

namespace ob {

constexpr uint32_t TYPE_F32 = 0, TYPE_Q8_0 = 8, TYPE_Q4_K = 12, TYPE_Q5_K = 13, TYPE_Q6_K = 14;
// Source-only types: per-32 symmetric formats (one f16 scale, 32 signed codes, no min term) whose CPU kernels are the
// Q8_0 loops over the unpacked codes (engine/vecdot.rs:2842-2881, :1277-1340).  They are unpacked to the device's Q8_0
// layout at registration, so every kernel sees TYPE_Q8_0 and gives the CPU's bits; the price is 34 instead of 18 or 22
// bytes per block of HBM traffic.
constexpr uint32_t TYPE_Q4_0 = 2, TYPE_Q5_0 = 6, TYPE_IQ4_NL = 20;
__host__ __device__ inline bool is_sym32_source(uint32_t t) { return t == TYPE_Q4_0 || t == TYPE_Q5_0 || t == TYPE_IQ4_NL; }
constexpr int KV_PAGE = 16;  // tokens per KV page

// ---- one-time kernel set-up, per device ---------------------------------------------
// cudaFuncSetAttribute applies to the device that is current when it is called, and one process may hold
// contexts on several GPUs, so "configured" is a bit per device ordinal, not one flag.  Holds its own lock:
// contexts on the same GPU may launch from different threads.
struct PerDeviceOnce {
    std::mutex mu;
    uint64_t done[4] = {0, 0, 0, 0};  // device ordinals 0..255
    template <class F>
    cudaError_t run(F &&configure) {
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return e;
        std::lock_guard<std::mutex> g(mu);
        uint64_t &word = done[(dev >> 6) & 3];
        const uint64_t bit = 1ull << (dev & 63);
        if (word & bit) return cudaSuccess;
        e = configure();
        if (e == cudaSuccess) word |= bit;
        return e;
    }
};

// ---- device helpers ----------------------------------------------------------------

__device__ __forceinline__ uint4 ldg128(const void *p) { return __ldg(reinterpret_cast<const uint4 *>(p)); }

// Streaming 128-bit load: weights are read once per step, so do not let them displace
// the activations and KV pages other kernels want to find in L1.
__device__ __forceinline__ uint4 ldg128_stream(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// dot of four unsigned bytes of a with four signed bytes of b, accumulated into c
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
// four signed bytes with four signed bytes
__device__ __forceinline__ int dp4a_ss(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// f16 bits -> f32.  Equal to the reference's f16_bits_to_f32 (engine/quant.rs:511-528) for
// every non-NaN input; weights never hold NaN scales that matter.
__device__ __forceinline__ float f16_bits_to_f32(uint32_t bits) { return __half2float(__ushort_as_half((unsigned short)bits)); }

// The reference's activation rounding: f32::round (half away from zero), clamp to +-127,
// NaN -> 0 (engine/vecdot.rs:113-116).
__device__ __forceinline__ int quantize_value(float v, float inv) {
    float r = roundf(__fmul_rn(v, inv));
    if (r != r) return 0;
    r = fminf(fmaxf(r, -127.0f), 127.0f);
    return (int)r;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ int warp_sum_i(int v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// ---- quantized weight as it lives in device memory -----------------------------------
//
// Rows keep the GGUF block contents but are re-laid so that every 16-byte load is aligned:
//   Q4_K  unchanged: nb blocks of 144 B  [d f16 | dmin f16 | scales 12 | qs 128]
//   Q5_K  unchanged: nb blocks of 176 B  [d f16 | dmin f16 | scales 12 | qh 32 | qs 128]
//   Q6_K  nb blocks of 208 B [ql 128 | qh 64 | scales 16], then the nb f16 d values
//   Q8_0  nb runs of 32 int8 codes, then the nb f16 d values
// row_stride is the row size rounded up to 16 bytes.  The byte count per row is the GGUF one.
struct DevWeight {
    const uint8_t *data;
    uint32_t type;
    uint32_t in_dim;
    uint32_t out_dim;
    uint32_t nb;          // blocks per row
    uint32_t d_off;       // byte offset of the f16 d plane inside a row (Q6_K, Q8_0)
    uint64_t row_stride;  // bytes
};

__host__ __device__ inline uint32_t block_elems(uint32_t type) { return type == TYPE_Q8_0 || is_sym32_source(type) ? 32u : 256u; }
__host__ __device__ inline uint32_t block_bytes_gguf(uint32_t type) {
    return type == TYPE_Q8_0 ? 34u : type == TYPE_Q4_K ? 144u : type == TYPE_Q5_K ? 176u : type == TYPE_Q5_0 ? 22u : is_sym32_source(type) ? 18u : 210u;
}

// Quantized activations of one token row, natural element order.
//   q     int8  [in_dim]
//   d     f32   [in_dim/256] (K types) or [in_dim/32] (Q8_0)
//   sums  int16 [in_dim/16]  sum of q per 16
struct ActView {
    const int8_t *q;
    const float *d;
    const int16_t *sums;
};

}  // namespace ob
