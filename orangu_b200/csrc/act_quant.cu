// On-the-fly int8 quantisation of activations, fused with the operator that produces them.
//
// Rule (reference: src/bin/orangu-server/engine/vecdot.rs:95-126 per 32, :3030-3053 per 256):
//   amax = max |x| ignoring NaN;  scale = amax / 127;  inv = scale > 0 ? 1 / scale : 0
//   q = clamp(round_half_away(x * inv), -127, 127), NaN -> 0;  sums = sum of q per 16
// Every step is an IEEE single operation, so the int8 codes and the scales equal the CPU's
// bit for bit whenever the fp32 input does.
//
// One CTA per token row.  A thread owns 8 consecutive elements; a warp owns one 256-block.
#include "common.cuh"
#include "kernels.h"
#include "seqsum.cuh"

namespace ob {

namespace {

constexpr int QT = 512;  // threads per CTA

__device__ __forceinline__ float silu_mul(float g, float u) {
    // silu(x) = x / (1 + exp(-x)), then * up   (engine/tensor.rs:825-827, engine/arch/mod.rs:1099-1105).
    // exp is taken in double and rounded once, the value the CPU oracle uses as well.
    float s = __fdiv_rn(g, __fadd_rn(1.0f, (float)exp((double)(-g))));
    return __fmul_rn(s, u);
}

// Shared-memory index with one pad word per 16, so that lanes reading runs of 16 consecutive
// elements (the sequential-sum scan) fall on different banks.
__device__ __forceinline__ uint32_t padded(uint32_t i) { return i + (i >> 4); }

template <int SOURCE>
__global__ void __launch_bounds__(QT) quantize_kernel(QuantArgs a) {
    const uint32_t row = blockIdx.x;
    const uint32_t dim = a.dim;
    const float *x = a.x + (uint64_t)row * dim;
    const int lane = threadIdx.x & 31;

    float norm_scale = 1.0f;
    extern __shared__ float srow[];  // RMSNORM only: the row, padded()
    if (SOURCE == ACT_RMSNORM) {
        // mean of squares with the squares added left to right, as the CPU adds them (tensor.rs:743)
        __shared__ float bcast;
        for (uint32_t i = threadIdx.x * 4; i < dim; i += QT * 4) {
            const float4 v = *reinterpret_cast<const float4 *>(x + i);
            srow[padded(i)] = v.x;
            srow[padded(i + 1)] = v.y;
            srow[padded(i + 2)] = v.z;
            srow[padded(i + 3)] = v.w;
        }
        __syncthreads();
        __shared__ SeqSumWorkspace<QT> ws;
        const float t = cta_sequential_sum<QT>([&](uint32_t i) { const float v = srow[padded(i)]; return __fmul_rn(v, v); }, dim, ws);
        if (threadIdx.x == 0) {
            const float mean_sq = __fdiv_rn(t, (float)dim);
            bcast = __fdiv_rn(1.0f, sqrtf(__fadd_rn(mean_sq, a.eps)));
        }
        __syncthreads();
        norm_scale = bcast;
    }

    const uint32_t n_chunks = dim / 8;
    for (uint32_t c = threadIdx.x; c < ((n_chunks + 31) & ~31u); c += QT) {
        const bool live = c < n_chunks;
        float v[8];
        if (live) {
            float4 a0 = *reinterpret_cast<const float4 *>(x + c * 8);
            float4 a1 = *reinterpret_cast<const float4 *>(x + c * 8 + 4);
            v[0] = a0.x; v[1] = a0.y; v[2] = a0.z; v[3] = a0.w;
            v[4] = a1.x; v[5] = a1.y; v[6] = a1.z; v[7] = a1.w;
            if (SOURCE == ACT_RMSNORM) {
                float4 w0 = *reinterpret_cast<const float4 *>(a.aux + c * 8);
                float4 w1 = *reinterpret_cast<const float4 *>(a.aux + c * 8 + 4);
                const float w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = __fmul_rn(__fmul_rn(v[i], norm_scale), w[i]);
            } else if (SOURCE == ACT_SWIGLU) {
                const float *up = a.aux + (uint64_t)row * dim;
                float4 u0 = *reinterpret_cast<const float4 *>(up + c * 8);
                float4 u1 = *reinterpret_cast<const float4 *>(up + c * 8 + 4);
                const float u[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = silu_mul(v[i], u[i]);
            }
            if (a.f32_out) {
                float *o = a.f32_out + (uint64_t)row * dim + c * 8;
                *reinterpret_cast<float4 *>(o) = make_float4(v[0], v[1], v[2], v[3]);
                *reinterpret_cast<float4 *>(o + 4) = make_float4(v[4], v[5], v[6], v[7]);
            }
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = 0.0f;
        }
        float m8 = 0.0f;  // fmaxf drops a NaN operand, as f32::max does
#pragma unroll
        for (int i = 0; i < 8; ++i) m8 = fmaxf(m8, fabsf(v[i]));

#pragma unroll
        for (int mode = 0; mode < 2; ++mode) {
            const ActBuf &buf = mode == 0 ? a.k : a.flat;
            if (buf.q == nullptr) continue;
            float amax = m8;
            if (mode == 0) {
                amax = warp_max(amax);  // 32 lanes x 8 = one 256-block
            } else {
                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));  // 4 lanes x 8 = one 32-block
                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
            }
            float scale = __fdiv_rn(amax, 127.0f);
            float inv = scale > 0.0f ? __fdiv_rn(1.0f, scale) : 0.0f;
            int qv[8];
            int s8 = 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                qv[i] = quantize_value(v[i], inv);
                s8 += qv[i];
            }
            int s16 = s8 + __shfl_xor_sync(0xffffffffu, s8, 1);
            if (live) {
                uint32_t lo = (qv[0] & 0xff) | ((qv[1] & 0xff) << 8) | ((qv[2] & 0xff) << 16) | ((uint32_t)(qv[3] & 0xff) << 24);
                uint32_t hi = (qv[4] & 0xff) | ((qv[5] & 0xff) << 8) | ((qv[6] & 0xff) << 16) | ((uint32_t)(qv[7] & 0xff) << 24);
                *reinterpret_cast<uint2 *>(buf.q + (uint64_t)row * buf.dim_cap + c * 8) = make_uint2(lo, hi);
                if ((c & 1) == 0) buf.sums[(uint64_t)row * (buf.dim_cap / 16) + c / 2] = (int16_t)s16;
                if (mode == 0) {
                    if (lane == 0) buf.d[(uint64_t)row * (buf.dim_cap / 256) + c / 32] = scale;
                } else {
                    if ((c & 3) == 0) buf.d[(uint64_t)row * (buf.dim_cap / 32) + c / 4] = scale;
                }
            }
        }
    }
}

}  // namespace

void launch_quantize(int source, const QuantArgs &a, cudaStream_t st) {
    if (a.n_rows == 0) return;
    switch (source) {
    case ACT_PLAIN: quantize_kernel<ACT_PLAIN><<<a.n_rows, QT, 0, st>>>(a); break;
    case ACT_RMSNORM: {
        const size_t smem = ((size_t)a.dim + a.dim / 16 + 16) * 4;
        static PerDeviceOnce once;
        if (once.run([] { return cudaFuncSetAttribute(quantize_kernel<ACT_RMSNORM>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024); }) != cudaSuccess) return;
        quantize_kernel<ACT_RMSNORM><<<a.n_rows, QT, smem, st>>>(a);
        break;
    }
    default: quantize_kernel<ACT_SWIGLU><<<a.n_rows, QT, 0, st>>>(a); break;
    }
}

}  // namespace ob
