// Q5_K products (ggml type 13): the Q4_K arithmetic over five-bit codes.
//
// Reference: dot_k_row_q5_k (engine/vecdot.rs:3181-3210) for one token -- per super-block
//   isum = sum_j sc_j * dot32(code_j, x_j),  imin = sum_j m_j * (bsum_2j + bsum_2j+1),  total += ad * (d * isum - dmin * imin)
// in ascending block order -- and, for several tokens in the prefill order, unpack_k_q5_k + gemm_k_q4_k
// (engine/vecdot.rs:2064-2089, 2213-2303): first every block's  acc -= (ad * dmin) * imin,  then every block's
// acc += ad * (d * isum).  code = nibble + 16 * (bit j of qh[l]) for sub-block j (engine/quant.rs:703-742).
//
// The type only turns up in files quantized with a *_K_M / *_K_S recipe other than Q4_K_M, so this is a plain kernel, not a
// tuned one: a warp owns one output row, streams its 176-byte blocks with 16-byte loads, and serves up to four tokens at a
// time from the quantized activations in global memory (L2-resident: every warp reads the same rows).  The integer sums are
// exact in any order; lane 0 forms the fp32 terms and adds them in the reference's order.  The block layout on the device is
// the GGUF one: [d f16 | dmin f16 | scales 12 | qh 32 | qs 128], every field 16-byte aligned.
#include "common.cuh"
#include "kernels.h"

namespace ob {

namespace {

constexpr int Q5_WARPS = 8, Q5_TT = 4;

// lane l: sub-block pair g = l / 8 (elements 64 g .. 64 g + 63), bytes 4 (l % 8) .. + 3 of that pair's 32 qs bytes;
// low nibbles belong to sub-block 2g, high nibbles to 2g + 1; the fifth bits are bits 2g and 2g + 1 of qh[l_byte].
template <bool GEMM>
__global__ void __launch_bounds__(Q5_WARPS * 32) q5k_kernel(GemvArgs a, uint32_t total_rows) {
    extern __shared__ float q5_terms[];  // GEMM: [warp][2][nb][Q5_TT] (the min terms' integers, then the isums) as int32
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t nb = a.seg[0].w.nb, in_dim = a.seg[0].w.in_dim;
    const uint32_t g = lane >> 3, byte4 = (lane & 7) * 4;
    int32_t *mine = reinterpret_cast<int32_t *>(q5_terms) + (size_t)warp * 2 * nb * Q5_TT;
    for (uint32_t grow = blockIdx.x * Q5_WARPS + warp; grow < total_rows; grow += gridDim.x * Q5_WARPS) {
        int s = 0;
        uint32_t row = grow;
        while (s + 1 < a.n_seg && row >= a.seg[s].w.out_dim) row -= a.seg[s++].w.out_dim;
        const GemvSegment &sg = a.seg[s];
        const uint8_t *wrow = sg.w.data + (uint64_t)row * sg.w.row_stride;
        for (uint32_t tok0 = 0; tok0 < a.n_tokens; tok0 += Q5_TT) {
            const uint32_t nt = min((uint32_t)Q5_TT, a.n_tokens - tok0);
            float acc[Q5_TT] = {0.0f, 0.0f, 0.0f, 0.0f};
            for (uint32_t b = 0; b < nb; ++b) {
                const uint8_t *blk = wrow + (uint64_t)b * 176;
                const uint4 hd = ldg128_stream(blk);
                const uint32_t qs = *reinterpret_cast<const uint32_t *>(blk + 48 + 32 * g + byte4);
                const uint32_t qh = *reinterpret_cast<const uint32_t *>(blk + 16 + byte4);
                // codes of sub-block 2g (low nibbles) and 2g + 1 (high nibbles), four each, as bytes 0..31
                const uint32_t lo = (qs & 0x0f0f0f0fu) | (((qh >> (2 * g)) & 0x01010101u) << 4);
                const uint32_t hi = ((qs >> 4) & 0x0f0f0f0fu) | (((qh >> (2 * g + 1)) & 0x01010101u) << 4);
                // six-bit scale and min of sub-blocks 2g and 2g + 1 (get_scale_min_k4, engine/quant.rs:653-662)
                const uint8_t *sc12 = reinterpret_cast<const uint8_t *>(&hd) + 4;
                auto scale_min = [&](int j, int &sc, int &m) {
                    if (j < 4) {
                        sc = sc12[j] & 63;
                        m = sc12[j + 4] & 63;
                    } else {
                        sc = (sc12[j + 4] & 0xF) | ((sc12[j - 4] >> 6) << 4);
                        m = (sc12[j + 4] >> 4) | ((sc12[j] >> 6) << 4);
                    }
                };
                int sc0, m0, sc1, m1, sc_l = 0, m_l = 0;
                scale_min(2 * (int)g, sc0, m0);
                scale_min(2 * (int)g + 1, sc1, m1);
                if (lane < 8) scale_min(lane, sc_l, m_l);  // lanes 0..7 also carry the min term of sub-block `lane`
                (void)m0;
                (void)m1;
                (void)sc_l;
                const float d = f16_bits_to_f32(hd.x & 0xffffu), dmin = f16_bits_to_f32(hd.x >> 16);
#pragma unroll
                for (uint32_t t = 0; t < Q5_TT; ++t) {
                    if (t >= nt) break;
                    const uint64_t tok = tok0 + t;
                    const int8_t *xq = a.act.q + tok * a.act.dim_cap + (uint64_t)b * 256 + 64 * g + byte4;
                    const int x_lo = *reinterpret_cast<const int *>(xq), x_hi = *reinterpret_cast<const int *>(xq + 32);
                    int isum = sc0 * __dp4a((int)lo, x_lo, 0) + sc1 * __dp4a((int)hi, x_hi, 0);
                    int imin = 0;
                    if (lane < 8) {
                        const int16_t *bs = a.act.sums + tok * (a.act.dim_cap / 16) + (uint64_t)b * 16 + 2 * lane;
                        imin = m_l * ((int)bs[0] + (int)bs[1]);
                    }
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) {
                        isum += __shfl_xor_sync(0xffffffffu, isum, o);
                        imin += __shfl_xor_sync(0xffffffffu, imin, o);
                    }
                    if (a.isum_out && tok == 0 && lane == 0) {
                        a.isum_out[(uint64_t)grow * nb + b] = isum;
                        if (a.imin_out) a.imin_out[(uint64_t)grow * nb + b] = imin;
                    }
                    if (!GEMM) {
                        const float ad = a.act.d[tok * (a.act.dim_cap / 256) + b];
                        acc[t] = __fadd_rn(acc[t], __fmul_rn(ad, __fsub_rn(__fmul_rn(d, (float)isum), __fmul_rn(dmin, (float)imin))));
                    } else if (lane == 0) {
                        mine[(0 * nb + b) * Q5_TT + t] = imin;
                        mine[(1 * nb + b) * Q5_TT + t] = isum;
                    }
                }
            }
            if (GEMM) {  // the two sweeps of gemm_k_q4_k, by lane t for token t
                __syncwarp();
                if (lane < (int)nt) {
                    const uint64_t tok = tok0 + lane;
                    const float *adp = a.act.d + tok * (a.act.dim_cap / 256);
                    float v = 0.0f;
                    for (uint32_t b = 0; b < nb; ++b) {
                        const float dmin = f16_bits_to_f32(*reinterpret_cast<const uint16_t *>(wrow + (uint64_t)b * 176 + 2));
                        v = __fsub_rn(v, __fmul_rn(__fmul_rn(adp[b], dmin), (float)mine[(0 * nb + b) * Q5_TT + lane]));
                    }
                    for (uint32_t b = 0; b < nb; ++b) {
                        const float d = f16_bits_to_f32(*reinterpret_cast<const uint16_t *>(wrow + (uint64_t)b * 176));
                        v = __fadd_rn(v, __fmul_rn(adp[b], __fmul_rn(d, (float)mine[(1 * nb + b) * Q5_TT + lane])));
                    }
                    float *y = sg.y + tok * sg.y_stride + row;
                    *y = sg.epilogue == EPI_ADD_RESIDUAL ? __fadd_rn(sg.residual[tok * sg.y_stride + row], v) : v;
                }
                __syncwarp();
            } else if (lane == 0) {
                for (uint32_t t = 0; t < nt; ++t) {
                    const uint64_t tok = tok0 + t;
                    float *y = sg.y + tok * sg.y_stride + row;
                    *y = sg.epilogue == EPI_ADD_RESIDUAL ? __fadd_rn(sg.residual[tok * sg.y_stride + row], acc[t]) : acc[t];
                }
            }
        }
    }
    (void)in_dim;
}

}  // namespace

void launch_q5k(const GemvArgs &a, int sm_count, cudaStream_t st) {
    uint32_t rows = 0;
    for (int s = 0; s < a.n_seg; ++s) rows += a.seg[s].w.out_dim;
    const int grid = (int)min((uint32_t)sm_count * 4u, max(1u, (rows + Q5_WARPS - 1) / Q5_WARPS));
    const bool gemm = a.gemm_order;
    const size_t smem = gemm ? (size_t)Q5_WARPS * 2 * a.seg[0].w.nb * Q5_TT * 4 : 0;
    if (gemm) {
        static PerDeviceOnce once;
        if (once.run([] { return cudaFuncSetAttribute(q5k_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024); }) != cudaSuccess) return;
        q5k_kernel<true><<<grid, Q5_WARPS * 32, smem, st>>>(a, rows);
    } else {
        q5k_kernel<false><<<grid, Q5_WARPS * 32, 0, st>>>(a, rows);
    }
}

}  // namespace ob
