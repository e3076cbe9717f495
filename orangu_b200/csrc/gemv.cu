// Block-quantized matrix-vector products: Q8_0, Q4_K and Q6_K weights against int8 activations.
//
// What is computed is the reference's single-token kernels, term for term:
//   Q8_0  total += (dw * ad[b]) * (float)dot32_b                    (engine/vecdot.rs:2829-2838)
//   Q4_K  total += ad[s] * (d * (float)isum_s - dmin * (float)imin_s) (engine/vecdot.rs:3152-3178)
//   Q6_K  total += (ad[s] * d) * (float)isum_s                       (engine/vecdot.rs:3215-3241)
// with the blocks of a row added in ascending order by one thread, so a row's fp32 result equals
// the CPU's bit for bit.  Integer parts (dot32/dot16, isum, imin) are exact by construction.
//
// The same kernel serves the prefill product (n_tokens > 1) in the reference's GEMM order, which
// uses the same integers and a different fp32 association (engine/vecdot.rs:2213-2303, 2352-2398):
//   Q4_K  first, over every super-block, acc -= (ad * dmin) * (float)imin; then acc += ad * (d * (float)isum)
//   Q6_K  acc += ad * (d * (float)isum)
//   Q8_0  acc += (ad * dw) * (float)dot32     (identical to the single-token form)
//
// Shape of the kernel.  Decode is HBM-bound: each weight byte is read once.  One CTA of 16
// warps per SM takes a contiguous range of row groups; its warps pull groups off a shared
// counter.  Activations (a few KB, shared by every row) are staged once per CTA in shared
// memory, permuted so that each quarter-warp reads 128 contiguous bytes per 128-bit load.
// K-type super-blocks are split over 4 lanes (two 128-bit loads of codes per lane), Q8_0
// blocks go one per lane; 4-bit codes are consumed straight from the packed words
// (dp4a on w & 0x0f0f0f0f, and on w & 0xf0f0f0f0 followed by one >> 4).
#include <cstdlib>

#include "common.cuh"
#include "kernels.h"

namespace ob {

namespace {

constexpr int GEMV_THREADS = 512;
constexpr int GEMV_WARPS = GEMV_THREADS / 32;
constexpr int R = 2;  // rows per warp pass

struct SmemPlan {
    uint32_t q_bytes;     // per token: permuted int8 activations
    uint32_t nb_pad;      // blocks per row, padded to the permutation period
    uint32_t n_sums;      // per token: per-16 sums
    uint32_t off_q, off_d, off_sums, off_terms, total;
    uint32_t term_sets;   // 2 when the min pass is kept apart (Q4_K, GEMM order)
};

__host__ __device__ inline SmemPlan smem_plan(uint32_t type, uint32_t in_dim, uint32_t T, bool gemm_order) {
    SmemPlan p;
    uint32_t nb = in_dim / block_elems(type);
    p.nb_pad = type == TYPE_Q8_0 ? ((nb + 7) & ~7u) : ((nb + 1) & ~1u);
    p.q_bytes = p.nb_pad * block_elems(type);
    p.n_sums = in_dim / 16;
    p.off_q = 16;
    p.off_d = p.off_q + T * p.q_bytes;
    p.off_sums = p.off_d + T * p.nb_pad * 4;
    p.off_terms = (p.off_sums + T * p.n_sums * 2 + 15) & ~15u;
    p.term_sets = (gemm_order && type == TYPE_Q4_K) ? 2u : 1u;
    p.total = p.off_terms + GEMV_WARPS * p.term_sets * T * R * p.nb_pad * 4;
    return p;
}

// Destination (bytes, within one token's buffer) of natural 16-byte chunk c.
__device__ __forceinline__ uint32_t permuted_chunk(uint32_t type, uint32_t c) {
    if (type == TYPE_Q8_0) {
        uint32_t b = c >> 1, k = c & 1;
        return (b >> 3) * 256 + k * 128 + (b & 7) * 16;
    }
    uint32_t b = c >> 4, c16 = c & 15, j4, k;
    if (type == TYPE_Q4_K) {
        j4 = c16 >> 2;
        k = c16 & 3;
    } else {  // Q6_K: c16 = 8h + 4*khi + 2a + klo
        j4 = ((c16 >> 3) << 1) | ((c16 >> 1) & 1);
        k = (((c16 >> 2) & 1) << 1) | (c16 & 1);
    }
    return ((b >> 1) * 4 + k) * 128 + ((b & 1) * 4 + j4) * 16;
}

template <uint32_t TYPE, int T, bool GEMM>
__global__ void __launch_bounds__(GEMV_THREADS, 1) gemv_kernel(GemvArgs a, uint32_t tok0) {
    extern __shared__ __align__(16) uint8_t smem[];
    constexpr uint32_t type = TYPE;
    const uint32_t in_dim = a.seg[0].w.in_dim;
    const uint32_t nb = a.seg[0].w.nb;
    const SmemPlan sp = smem_plan(type, in_dim, T, GEMM);
    int *next_group = reinterpret_cast<int *>(smem);
    uint8_t *sq = smem + sp.off_q;
    float *sd = reinterpret_cast<float *>(smem + sp.off_d);
    int16_t *ssum = reinterpret_cast<int16_t *>(smem + sp.off_sums);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float *terms = reinterpret_cast<float *>(smem + sp.off_terms) + (size_t)warp * sp.term_sets * T * R * sp.nb_pad;
    float *terms_min = terms + (size_t)T * R * sp.nb_pad;  // Q4_K in GEMM order only
    const uint32_t nt = min((uint32_t)T, a.n_tokens - tok0);

    // groups of R rows, segments concatenated
    uint32_t groups_of[3], total_groups = 0;
    for (int s = 0; s < 3; ++s) {
        groups_of[s] = s < a.n_seg ? (a.seg[s].w.out_dim + R - 1) / R : 0;
        total_groups += groups_of[s];
    }
    const uint32_t g_begin = (uint32_t)(((uint64_t)total_groups * blockIdx.x) / gridDim.x);
    const uint32_t g_end = (uint32_t)(((uint64_t)total_groups * (blockIdx.x + 1)) / gridDim.x);
    if (threadIdx.x == 0) *next_group = (int)g_begin;

    // ---- stage activations -----------------------------------------------------------
    if (TYPE == TYPE_Q8_0 && T == 1 && a.x_f32) {
        // launched with programmatic stream serialisation: this grid may have started while its predecessor was finishing;
        // let the successor do the same, then wait for the predecessor's output (x) to be complete.  Nothing above this point
        // reads or writes memory another kernel touches.
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
        asm volatile("griddepcontrol.wait;" ::: "memory");
        // the row arrives as fp32: quantize it per 32 here (quantize_act, engine/vecdot.rs:95-126) -- four lanes x eight values
        // are one block -- straight into the layout the loop below reads
        const uint32_t n_chunks = in_dim / 8;
        for (uint32_t c = threadIdx.x; c < ((n_chunks + 31) & ~31u); c += GEMV_THREADS) {
            const bool live = c < n_chunks;
            float v[8];
            if (live) {
                const float4 a0 = *reinterpret_cast<const float4 *>(a.x_f32 + c * 8), a1 = *reinterpret_cast<const float4 *>(a.x_f32 + c * 8 + 4);
                v[0] = a0.x; v[1] = a0.y; v[2] = a0.z; v[3] = a0.w;
                v[4] = a1.x; v[5] = a1.y; v[6] = a1.z; v[7] = a1.w;
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = 0.0f;
            }
            float amax = 0.0f;  // fmaxf drops a NaN operand, as f32::max does
#pragma unroll
            for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
            const float scale = __fdiv_rn(amax, 127.0f), inv = scale > 0.0f ? __fdiv_rn(1.0f, scale) : 0.0f;
            int qv[8], s8 = 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                qv[i] = quantize_value(v[i], inv);
                s8 += qv[i];
            }
            const int s16 = s8 + __shfl_xor_sync(0xffffffffu, s8, 1);
            if (live) {
                const uint32_t lo = (qv[0] & 0xff) | ((qv[1] & 0xff) << 8) | ((qv[2] & 0xff) << 16) | ((uint32_t)(qv[3] & 0xff) << 24);
                const uint32_t hi = (qv[4] & 0xff) | ((qv[5] & 0xff) << 8) | ((qv[6] & 0xff) << 16) | ((uint32_t)(qv[7] & 0xff) << 24);
                *reinterpret_cast<uint2 *>(sq + permuted_chunk(type, c >> 1) + (c & 1) * 8) = make_uint2(lo, hi);
                if ((c & 3) == 0) sd[c >> 2] = scale;
                if ((c & 1) == 0 && (c >> 1) < sp.n_sums) ssum[c >> 1] = (int16_t)s16;
            }
        }
    } else {
        const uint32_t chunks = in_dim / 16;
        for (uint32_t i = threadIdx.x; i < nt * chunks; i += GEMV_THREADS) {
            uint32_t t = i / chunks, c = i % chunks;
            uint4 v = *reinterpret_cast<const uint4 *>(a.act.q + (uint64_t)(tok0 + t) * a.act.dim_cap + c * 16);
            *reinterpret_cast<uint4 *>(sq + t * sp.q_bytes + permuted_chunk(type, c)) = v;
        }
        const uint32_t dcap = a.act.dim_cap / block_elems(type);
        for (uint32_t i = threadIdx.x; i < nt * nb; i += GEMV_THREADS) {
            uint32_t t = i / nb, b = i % nb;
            sd[t * sp.nb_pad + b] = a.act.d[(uint64_t)(tok0 + t) * dcap + b];
        }
        for (uint32_t i = threadIdx.x; i < nt * sp.n_sums; i += GEMV_THREADS) {
            uint32_t t = i / sp.n_sums, g = i % sp.n_sums;
            ssum[t * sp.n_sums + g] = a.act.sums[(uint64_t)(tok0 + t) * (a.act.dim_cap / 16) + g];
        }
    }
    __syncthreads();

    while (true) {
        int grp = 0;
        if (lane == 0) grp = atomicAdd(next_group, 1);
        grp = __shfl_sync(0xffffffffu, grp, 0);
        if ((uint32_t)grp >= g_end) break;

        // locate the group
        int s = 0;
        uint32_t gi = (uint32_t)grp;
        while (gi >= groups_of[s]) {
            gi -= groups_of[s];
            ++s;
        }
        const GemvSegment &seg = a.seg[s];
        const uint32_t row0 = gi * R;
        const uint32_t n_rows = min((uint32_t)R, seg.w.out_dim - row0);
        const uint8_t *rowp[R];
#pragma unroll
        for (int r = 0; r < R; ++r) rowp[r] = seg.w.data + (uint64_t)(row0 + (r < (int)n_rows ? r : 0)) * seg.w.row_stride;
        const uint32_t d_off = seg.w.d_off;

        if (type == TYPE_Q8_0) {
            for (uint32_t b0 = 0; b0 < nb; b0 += 32) {
                const uint32_t b = b0 + lane;
                const bool live = b < nb;
                uint4 wa[R], wb[R];
                float dw[R];
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    if (live) {
                        wa[r] = ldg128_stream(rowp[r] + (uint64_t)b * 32);
                        wb[r] = ldg128_stream(rowp[r] + (uint64_t)b * 32 + 16);
                        dw[r] = f16_bits_to_f32(__ldg(reinterpret_cast<const unsigned short *>(rowp[r] + d_off + 2 * b)));
                    } else {
                        wa[r] = wb[r] = make_uint4(0, 0, 0, 0);
                        dw[r] = 0.0f;
                    }
                }
                const uint32_t pos = (b >> 3) * 256 + (b & 7) * 16;
                for (uint32_t t = 0; t < nt; ++t) {
                    if (!live) continue;
                    const uint4 x0 = *reinterpret_cast<const uint4 *>(sq + t * sp.q_bytes + pos);
                    const uint4 x1 = *reinterpret_cast<const uint4 *>(sq + t * sp.q_bytes + pos + 128);
                    const float ad = sd[t * sp.nb_pad + b];
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        int dot = dp4a_ss(wa[r].x, x0.x, 0);
                        dot = dp4a_ss(wa[r].y, x0.y, dot);
                        dot = dp4a_ss(wa[r].z, x0.z, dot);
                        dot = dp4a_ss(wa[r].w, x0.w, dot);
                        dot = dp4a_ss(wb[r].x, x1.x, dot);
                        dot = dp4a_ss(wb[r].y, x1.y, dot);
                        dot = dp4a_ss(wb[r].z, x1.z, dot);
                        dot = dp4a_ss(wb[r].w, x1.w, dot);
                        terms[(t * R + r) * sp.nb_pad + b] = __fmul_rn(__fmul_rn(dw[r], ad), (float)dot);
                        if (a.isum_out && t == 0 && r < (int)n_rows && tok0 == 0) {
                            a.isum_out[(uint64_t)(row0 + r) * nb + b] = dot;
                            if (a.imin_out) a.imin_out[(uint64_t)(row0 + r) * nb + b] = 0;
                        }
                    }
                }
            }
        } else {
            const int j4 = lane & 3;
            const uint32_t chunk_off = (uint32_t)(lane & 7) * 16;
            const uint32_t blk_bytes = type == TYPE_Q4_K ? 144u : 208u;
#pragma unroll 2
            for (uint32_t b0 = 0; b0 < nb; b0 += 8) {
                const uint32_t b = b0 + (lane >> 2);
                const bool live = b < nb;
                uint4 qa[R], qb[R], hd[R], ha[R], hb[R];  // codes; header / Q6_K scales; Q6_K high bits
                float dsup[R];
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    qa[r] = qb[r] = hd[r] = ha[r] = hb[r] = make_uint4(0, 0, 0, 0);
                    dsup[r] = 0.0f;
                    if (live) {
                        const uint8_t *blk = rowp[r] + (uint64_t)b * blk_bytes;
                        if (type == TYPE_Q4_K) {
                            hd[r] = ldg128_stream(blk);
                            qa[r] = ldg128_stream(blk + 16 + 32 * j4);
                            qb[r] = ldg128_stream(blk + 32 + 32 * j4);
                        } else {
                            qa[r] = ldg128_stream(blk + 32 * j4);
                            qb[r] = ldg128_stream(blk + 32 * j4 + 16);
                            ha[r] = ldg128_stream(blk + 128 + 32 * (j4 >> 1));
                            hb[r] = ldg128_stream(blk + 144 + 32 * (j4 >> 1));
                            hd[r] = ldg128_stream(blk + 192);
                            dsup[r] = f16_bits_to_f32(__ldg(reinterpret_cast<const unsigned short *>(rowp[r] + d_off + 2 * b)));
                        }
                    }
                }
                // lanes past the end of the row read block 0's slot (any valid address): their results are never used
                const uint32_t pbase = (live ? (b >> 1) * 512 : 0u) + chunk_off;

                if (type == TYPE_Q4_K) {
                    // 6-bit scale / min of sub-blocks 2*j4 and 2*j4+1 as byte pairs
                    uint32_t scp[R], mp[R];
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        const uint32_t sh = 16u * (j4 & 1);
                        const uint32_t a16 = hd[r].y >> sh, b16 = hd[r].z >> sh, p16 = hd[r].w >> sh;
                        if (j4 < 2) {
                            scp[r] = a16 & 0x3f3fu;
                            mp[r] = b16 & 0x3f3fu;
                        } else {
                            scp[r] = (p16 & 0x0f0fu) | ((a16 >> 2) & 0x3030u);
                            mp[r] = ((p16 >> 4) & 0x0f0fu) | ((b16 >> 2) & 0x3030u);
                        }
                    }
                    for (uint32_t t = 0; t < nt; ++t) {
                        const uint8_t *xq = sq + t * sp.q_bytes + pbase;
                        const uint4 x0 = *reinterpret_cast<const uint4 *>(xq);
                        const uint4 x1 = *reinterpret_cast<const uint4 *>(xq + 128);
                        const uint4 x2 = *reinterpret_cast<const uint4 *>(xq + 256);
                        const uint4 x3 = *reinterpret_cast<const uint4 *>(xq + 384);
                        int bs_a = 0, bs_b = 0;
                        if (live) {
                            const short4 s4 = *reinterpret_cast<const short4 *>(ssum + t * sp.n_sums + b * 16 + 4 * j4);
                            bs_a = s4.x + s4.y;
                            bs_b = s4.z + s4.w;
                        }
                        const float ad = live ? sd[t * sp.nb_pad + b] : 0.0f;
#pragma unroll
                        for (int r = 0; r < R; ++r) {
                            const uint32_t L = 0x0f0f0f0fu, H = 0xf0f0f0f0u;
                            int lo = dp4a_us(qa[r].x & L, x0.x, 0);
                            lo = dp4a_us(qa[r].y & L, x0.y, lo);
                            lo = dp4a_us(qa[r].z & L, x0.z, lo);
                            lo = dp4a_us(qa[r].w & L, x0.w, lo);
                            lo = dp4a_us(qb[r].x & L, x1.x, lo);
                            lo = dp4a_us(qb[r].y & L, x1.y, lo);
                            lo = dp4a_us(qb[r].z & L, x1.z, lo);
                            lo = dp4a_us(qb[r].w & L, x1.w, lo);
                            int hi = dp4a_us(qa[r].x & H, x2.x, 0);
                            hi = dp4a_us(qa[r].y & H, x2.y, hi);
                            hi = dp4a_us(qa[r].z & H, x2.z, hi);
                            hi = dp4a_us(qa[r].w & H, x2.w, hi);
                            hi = dp4a_us(qb[r].x & H, x3.x, hi);
                            hi = dp4a_us(qb[r].y & H, x3.y, hi);
                            hi = dp4a_us(qb[r].z & H, x3.z, hi);
                            hi = dp4a_us(qb[r].w & H, x3.w, hi);
                            hi >>= 4;  // the high nibbles were left in place: every product carried a factor 16
                            int isum = (int)(scp[r] & 0xff) * lo + (int)(scp[r] >> 8) * hi;
                            int imin = (int)(mp[r] & 0xff) * bs_a + (int)(mp[r] >> 8) * bs_b;
                            isum += __shfl_xor_sync(0xffffffffu, isum, 1);
                            imin += __shfl_xor_sync(0xffffffffu, imin, 1);
                            isum += __shfl_xor_sync(0xffffffffu, isum, 2);
                            imin += __shfl_xor_sync(0xffffffffu, imin, 2);
                            if (j4 == 0 && live) {
                                const float d = f16_bits_to_f32(hd[r].x & 0xffffu), dmin = f16_bits_to_f32(hd[r].x >> 16);
                                if (GEMM) {
                                    terms_min[(t * R + r) * sp.nb_pad + b] = __fmul_rn(__fmul_rn(ad, dmin), (float)imin);
                                    terms[(t * R + r) * sp.nb_pad + b] = __fmul_rn(ad, __fmul_rn(d, (float)isum));
                                } else {
                                    const float inner = __fsub_rn(__fmul_rn(d, (float)isum), __fmul_rn(dmin, (float)imin));
                                    terms[(t * R + r) * sp.nb_pad + b] = __fmul_rn(ad, inner);
                                }
                                if (a.isum_out && t == 0 && r < (int)n_rows && tok0 == 0) {
                                    a.isum_out[(uint64_t)(row0 + r) * nb + b] = isum;
                                    if (a.imin_out) a.imin_out[(uint64_t)(row0 + r) * nb + b] = imin;
                                }
                            }
                        }
                    }
                } else {  // Q6_K
                    const int h = j4 >> 1, aa = j4 & 1;
                    for (uint32_t t = 0; t < nt; ++t) {
                        const uint8_t *xq = sq + t * sp.q_bytes + pbase;
                        const uint4 xv[4] = {*reinterpret_cast<const uint4 *>(xq), *reinterpret_cast<const uint4 *>(xq + 128),
                                             *reinterpret_cast<const uint4 *>(xq + 256), *reinterpret_cast<const uint4 *>(xq + 384)};
                        int s16[4] = {0, 0, 0, 0};  // activation sums of the four 16-element groups this lane covers
                        if (live) {
                            const int16_t *sp16 = ssum + t * sp.n_sums + b * 16 + 8 * h + 2 * aa;
                            const short2 p0 = *reinterpret_cast<const short2 *>(sp16);
                            const short2 p1 = *reinterpret_cast<const short2 *>(sp16 + 4);
                            s16[0] = p0.x;
                            s16[1] = p0.y;
                            s16[2] = p1.x;
                            s16[3] = p1.y;
                        }
                        const float ad = live ? sd[t * sp.nb_pad + b] : 0.0f;
#pragma unroll
                        for (int r = 0; r < R; ++r) {
                            const uint32_t qlw[8] = {qa[r].x, qa[r].y, qa[r].z, qa[r].w, qb[r].x, qb[r].y, qb[r].z, qb[r].w};
                            const uint32_t qhw[8] = {ha[r].x, ha[r].y, ha[r].z, ha[r].w, hb[r].x, hb[r].y, hb[r].z, hb[r].w};
                            const uint32_t xw[16] = {xv[0].x, xv[0].y, xv[0].z, xv[0].w, xv[1].x, xv[1].y, xv[1].z, xv[1].w,
                                                     xv[2].x, xv[2].y, xv[2].z, xv[2].w, xv[3].x, xv[3].y, xv[3].z, xv[3].w};
                            int dots[4] = {0, 0, 0, 0};
#pragma unroll
                            for (int w = 0; w < 8; ++w) {
                                const uint32_t tq = qhw[w] >> (2 * aa);
                                const uint32_t vlo = (qlw[w] & 0x0f0f0f0fu) | ((tq << 4) & 0x30303030u);
                                const uint32_t vhi = ((qlw[w] >> 4) & 0x0f0f0f0fu) | (tq & 0x30303030u);
                                dots[w >> 2] = dp4a_us(vlo, xw[w], dots[w >> 2]);
                                dots[2 + (w >> 2)] = dp4a_us(vhi, xw[8 + w], dots[2 + (w >> 2)]);
                            }
                            // signed scales: bytes 2a, 2a+1 of scale word 2h (low half) and 2h+1 (high half)
                            const uint32_t wlo = (h ? hd[r].z : hd[r].x) >> (16 * aa), whi = (h ? hd[r].w : hd[r].y) >> (16 * aa);
                            const int sc0 = (int)(int8_t)(wlo & 0xff), sc1 = (int)(int8_t)((wlo >> 8) & 0xff);
                            const int sc2 = (int)(int8_t)(whi & 0xff), sc3 = (int)(int8_t)((whi >> 8) & 0xff);
                            int isum = sc0 * (dots[0] - 32 * s16[0]) + sc1 * (dots[1] - 32 * s16[1]) + sc2 * (dots[2] - 32 * s16[2]) +
                                       sc3 * (dots[3] - 32 * s16[3]);
                            isum += __shfl_xor_sync(0xffffffffu, isum, 1);
                            isum += __shfl_xor_sync(0xffffffffu, isum, 2);
                            if (j4 == 0 && live) {
                                terms[(t * R + r) * sp.nb_pad + b] =
                                    GEMM ? __fmul_rn(ad, __fmul_rn(dsup[r], (float)isum)) : __fmul_rn(__fmul_rn(ad, dsup[r]), (float)isum);
                                if (a.isum_out && t == 0 && r < (int)n_rows && tok0 == 0) {
                                    a.isum_out[(uint64_t)(row0 + r) * nb + b] = isum;
                                    if (a.imin_out) a.imin_out[(uint64_t)(row0 + r) * nb + b] = 0;
                                }
                            }
                        }
                    }
                }
            }
        }
        __syncwarp();

        // ---- ordered fp32 sum: one lane per (token, row), blocks in ascending order ----
        if (lane < (int)(nt * R)) {
            const uint32_t t = lane / R, r = lane % R;
            if (r < n_rows) {
                const float *tp = terms + (t * R + r) * sp.nb_pad;
                float total = 0.0f;
                if (GEMM && type == TYPE_Q4_K) {
                    const float *tm = terms_min + (t * R + r) * sp.nb_pad;
                    for (uint32_t b = 0; b < nb; ++b) total = __fsub_rn(total, tm[b]);
                }
                for (uint32_t b = 0; b < nb; ++b) total = __fadd_rn(total, tp[b]);
                const uint64_t o = (uint64_t)(tok0 + t) * seg.y_stride + row0 + r;
                if (seg.epilogue == EPI_ADD_RESIDUAL) total = __fadd_rn(seg.residual[o], total);
                seg.y[o] = total;
            }
        }
        __syncwarp();
    }
}

template <uint32_t TYPE, int T, bool GEMM>
void launch_tile(const GemvArgs &a, int grid, size_t smem, cudaStream_t st) {
    static PerDeviceOnce once;  // one per instantiation
    if (once.run([] { return cudaFuncSetAttribute(gemv_kernel<TYPE, T, GEMM>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024); }) != cudaSuccess) return;
    if (TYPE == TYPE_Q8_0 && T == 1 && a.x_f32) {  // the fused single-token form overlaps its launch with its predecessor's tail
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3((unsigned)grid);
        cfg.blockDim = dim3(GEMV_THREADS);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        cudaLaunchKernelEx(&cfg, gemv_kernel<TYPE, T, GEMM>, a, 0u);
        return;
    }
    for (uint32_t tok0 = 0; tok0 < a.n_tokens; tok0 += T) gemv_kernel<TYPE, T, GEMM><<<grid, GEMV_THREADS, smem, st>>>(a, tok0);
}

template <uint32_t TYPE, bool GEMM>
void launch_type(const GemvArgs &a, uint32_t T, int grid, size_t smem, cudaStream_t st) {
    switch (T) {
    case 8: launch_tile<TYPE, 8, GEMM>(a, grid, smem, st); break;
    case 4: launch_tile<TYPE, 4, GEMM>(a, grid, smem, st); break;
    case 2: launch_tile<TYPE, 2, GEMM>(a, grid, smem, st); break;
    default: launch_tile<TYPE, 1, GEMM>(a, grid, smem, st); break;
    }
}

}  // namespace

size_t gemv_smem_bytes(uint32_t type, uint32_t in_dim, uint32_t tile_tokens, bool gemm_order) {
    return smem_plan(type, in_dim, tile_tokens, gemm_order).total;
}

uint32_t gemv_launches(uint32_t type, uint32_t in_dim, uint32_t n_tokens, bool gemm_order) {
    if (type == TYPE_Q5_K) return 1;
    if ((type == TYPE_Q4_K || type == TYPE_Q6_K) && n_tokens >= 9) return 1;  // the tensor-core kernel covers all tokens in one launch
    uint32_t T = 8;
    while (T > 1 && (T / 2 >= n_tokens || gemv_smem_bytes(type, in_dim, T, gemm_order) > 200 * 1024)) T /= 2;
    return (n_tokens + T - 1) / T;
}

void launch_gemv(const GemvArgs &a, int sm_count, cudaStream_t st) {
    if (a.n_tokens == 0 || a.n_seg == 0) return;
    if (a.seg[0].w.type == TYPE_Q5_K) {  // its own kernel, both orders (q5k.cu)
        launch_q5k(a, sm_count, st);
        return;
    }
    static const bool use_mma = [] { const char *e = getenv("OB_MMA"); return !(e && e[0] == '0' && e[1] == 0); }();
    if (gemm_tc5_supported(a) && launch_gemm_tc5(a, sm_count, st)) return;  // many tokens: tcgen05 tiles (gemm_tc5.cu)
    if (use_mma && gemm_mma_supported(a)) {  // many tokens: tensor-core tiles (gemm_mma.cu)
        launch_gemm_mma(a, sm_count, st);
        return;
    }
    const uint32_t type = a.seg[0].w.type, in_dim = a.seg[0].w.in_dim;
    // Q8_0's two orders are the same arithmetic; Q4_K / Q6_K differ only when asked for the GEMM order.
    const bool gemm = a.gemm_order && type != TYPE_Q8_0;
    uint32_t groups = 0;
    for (int s = 0; s < a.n_seg; ++s) groups += (a.seg[s].w.out_dim + R - 1) / R;
    const int grid = (int)min((uint32_t)sm_count, max(1u, (groups + GEMV_WARPS - 1) / GEMV_WARPS));
    const size_t budget = 200 * 1024;
    uint32_t T = 8;
    while (T > 1 && (T / 2 >= a.n_tokens || gemv_smem_bytes(type, in_dim, T, gemm) > budget)) T /= 2;
    const size_t smem = gemv_smem_bytes(type, in_dim, T, gemm);
    if (type == TYPE_Q4_K) {
        if (gemm) launch_type<TYPE_Q4_K, true>(a, T, grid, smem, st);
        else launch_type<TYPE_Q4_K, false>(a, T, grid, smem, st);
    } else if (type == TYPE_Q6_K) {
        if (gemm) launch_type<TYPE_Q6_K, true>(a, T, grid, smem, st);
        else launch_type<TYPE_Q6_K, false>(a, T, grid, smem, st);
    } else {
        launch_type<TYPE_Q8_0, false>(a, T, grid, smem, st);
    }
}

}  // namespace ob
