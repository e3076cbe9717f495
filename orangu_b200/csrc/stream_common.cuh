// Device code shared by the single-token product kernels (stream_gemv.cu: one product per launch; layer_stream.cu: the
// products of a whole decoder layer in one persistent launch): the shared-memory "image" of the quantized activations,
// the activation quantizer, and the integer dot of half a super-block for two rows at once.
//
// Arithmetic is the reference's single-token kernels, unchanged (engine/vecdot.rs:3030-3053 activation quantizer,
// :3152-3178 Q4_K, :3215-3241 Q6_K): exact integer partial sums; the fp32 terms are formed by the callers.
#pragma once

#include <cuda_pipeline.h>

#include "common.cuh"
#include "kernels.h"

namespace ob {

namespace {

// two CTAs of this much (plus the 1 KB the system reserves for each) fit the 228 KB of an SM
constexpr uint32_t SG_MAX_SMEM = 112 * 1024;
constexpr uint32_t ACT_BLOCK_STRIDE = 272;  // bytes per 256 int8 activations: 17 sixteen-byte chunks, so lanes one block apart hit different banks

// bytes of `bpc` blocks of one row inside a slot
__host__ __device__ inline uint32_t part_bytes(uint32_t type, uint32_t bpc) { return type == TYPE_Q4_K ? bpc * 144u : bpc * 208u + ((bpc * 2u + 15u) & ~15u); }

// Two lanes share one super-block of a row pair (each takes half of its 256 elements), so a unit -- 32 lanes -- is 16
// (block, pair) cells = 4.6 KB, half of what one lane per cell would make it: the two-slot ring of a warp is 9 KB and
// sixteen warps fit an SM.  Lanes per pair of rows = 2 x blocks per chunk; a chunk is the smallest power of two that
// covers the row, at most 16 blocks (longer rows are cut into chunks, which also spreads a matrix with few rows over
// more warps).
__host__ __device__ inline uint32_t lanes_per_pair(uint32_t nb) {
    uint32_t bpc = 1;
    while (bpc < nb && bpc < 16) bpc <<= 1;
    return 2 * bpc;
}

__host__ __device__ inline int sg_warps(bool has_q6) { return has_q6 ? 6 : 8; }

// The "image" is what the dot loop reads from shared memory: [nb][272] int8 (256 used), [nb] f32 scales, [nb][8] int16
// sums per 32, [nb][16] int16 sums per 16.  A kernel either builds it in its own shared memory from the fp32 row, or a
// producer builds it once in global memory and every CTA of the consumer copies it.
struct ActImage {
    uint32_t off_d, off_bsum, off_sum16, bytes;
};
__host__ __device__ inline ActImage act_image(uint32_t nb) {
    ActImage im;
    im.off_d = nb * ACT_BLOCK_STRIDE;
    im.off_bsum = (im.off_d + nb * 4 + 15) & ~15u;
    im.off_sum16 = im.off_bsum + nb * 16;
    im.bytes = im.off_sum16 + nb * 32;
    return im;
}

// Per-segment words the loop needs, kept in shared memory so that a run-time segment index costs one load:
// [0,1] w.data  [2,3] w2.data  [4] row stride  [5] type  [6] out_dim  [7] pairs  [8] d_off  [9] epilogue  [10,11] y  [12] first group
constexpr uint32_t SEG_WORDS = 16, SEG_TABLE_BYTES = 3 * SEG_WORDS * 4 + 64;

struct SgSmem {  // byte offsets inside dynamic shared memory
    uint32_t off_act, off_d, off_bsum, off_sum16, off_terms, off_ring, slot_bytes, total;
};

__host__ __device__ inline SgSmem sg_smem(uint32_t in_dim, bool has_q6, uint32_t lp) {
    SgSmem s;
    const uint32_t nb = in_dim / 256, nw = (uint32_t)sg_warps(has_q6);
    s.off_act = SEG_TABLE_BYTES;  // [0, SEG_TABLE_BYTES): the segment table
    const ActImage im = act_image(nb);
    s.off_d = s.off_act + im.off_d;
    s.off_bsum = s.off_act + im.off_bsum;    // int16 [nb][8]  sums per 32
    s.off_sum16 = s.off_act + im.off_sum16;  // int16 [nb][16] sums per 16
    s.off_terms = s.off_act + im.bytes;      // float [warp][pair slot][row][blocks per chunk]  = [warp][32]
    s.off_ring = s.off_terms + nw * 32 * 4;
    s.slot_bytes = (32 / lp) * 2 * part_bytes(has_q6 ? TYPE_Q6_K : TYPE_Q4_K, lp / 2);
    s.total = s.off_ring + nw * 2 * s.slot_bytes;
    return s;
}

// Explicit shared-space accesses with 32-bit addresses (a generic pointer would cost 64-bit address arithmetic per load).
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
__device__ __forceinline__ uint32_t lds16(uint32_t addr) {
    unsigned short v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts32(uint32_t addr, float v) { asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory"); }
__device__ __forceinline__ void cp_async16(uint32_t saddr, const void *g) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(saddr), "l"(g) : "memory");
}

__device__ __forceinline__ float silu_mul_exact(float g, float u) {
    const float s = __fdiv_rn(g, __fadd_rn(1.0f, (float)exp((double)(-g))));
    return __fmul_rn(s, u);
}

// ---- activations of the single token, quantized per 256 ------------------------------------------------------
// One warp, block b of the image: lane l holds elements 8l .. 8l+7 of the block in v.
__device__ __forceinline__ void quantize_block(const float (&v)[8], uint32_t b, uint8_t *img, const ActImage &im) {
    const int lane = threadIdx.x & 31;
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
    amax = warp_max(amax);
    const float scale = __fdiv_rn(amax, 127.0f);
    const float inv = scale > 0.0f ? __fdiv_rn(1.0f, scale) : 0.0f;
    int q[8], s8 = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        q[i] = quantize_value(v[i], inv);
        s8 += q[i];
    }
    const int s16 = s8 + __shfl_xor_sync(0xffffffffu, s8, 1);
    const int s32 = s16 + __shfl_xor_sync(0xffffffffu, s16, 2);
    const uint32_t lo = (q[0] & 0xff) | ((q[1] & 0xff) << 8) | ((q[2] & 0xff) << 16) | ((uint32_t)(q[3] & 0xff) << 24);
    const uint32_t hi = (q[4] & 0xff) | ((q[5] & 0xff) << 8) | ((q[6] & 0xff) << 16) | ((uint32_t)(q[7] & 0xff) << 24);
    *reinterpret_cast<uint2 *>(img + b * ACT_BLOCK_STRIDE + lane * 8) = make_uint2(lo, hi);
    if ((lane & 1) == 0) reinterpret_cast<int16_t *>(img + im.off_sum16)[b * 16 + (lane >> 1)] = (int16_t)s16;
    if ((lane & 3) == 0) reinterpret_cast<int16_t *>(img + im.off_bsum)[b * 8 + (lane >> 2)] = (int16_t)s32;
    if (lane == 0) reinterpret_cast<float *>(img + im.off_d)[b] = scale;
}

// Warps `warp`, `warp + n_warps`, ... of the callers take blocks round-robin; a lane owns 8 consecutive elements of the block.
// x * norm_scale * norm_w is quantized when norm_w != nullptr (tensor.rs:747), x itself otherwise.
__device__ void quantize_image(const float *x, const float *norm_w, float norm_scale, uint32_t nb, uint8_t *img, uint32_t warp, uint32_t n_warps) {
    const int lane = threadIdx.x & 31;
    const ActImage im = act_image(nb);
    // four blocks per pass, all their loads issued before any arithmetic: the pass costs one memory latency, not four
    for (uint32_t bb = warp; bb < nb; bb += 4 * n_warps) {
        float v[4][8];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const uint32_t b = bb + k * n_warps;
            if (b < nb) {
                const uint32_t e0 = b * 256 + lane * 8;
                const float4 x0 = __ldcg(reinterpret_cast<const float4 *>(x + e0)), x1 = __ldcg(reinterpret_cast<const float4 *>(x + e0 + 4));
                v[k][0] = x0.x; v[k][1] = x0.y; v[k][2] = x0.z; v[k][3] = x0.w; v[k][4] = x1.x; v[k][5] = x1.y; v[k][6] = x1.z; v[k][7] = x1.w;
            }
        }
        if (norm_w) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const uint32_t b = bb + k * n_warps;
                if (b < nb) {
                    const uint32_t e0 = b * 256 + lane * 8;
                    const float4 w0 = __ldg(reinterpret_cast<const float4 *>(norm_w + e0)), w1 = __ldg(reinterpret_cast<const float4 *>(norm_w + e0 + 4));
                    const float w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
                    for (int i = 0; i < 8; ++i) v[k][i] = __fmul_rn(__fmul_rn(v[k][i], norm_scale), w[i]);  // (v * scale) * w, tensor.rs:747
                }
            }
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const uint32_t b = bb + k * n_warps;
            if (b >= nb) break;  // warp-uniform
            quantize_block(v[k], b, img, im);
        }
    }
}

// ---- units ---------------------------------------------------------------------------------------------------
// A unit is what one warp processes at a time: PPU = 32 / LP consecutive pairs of rows of one segment x up to LP / 2
// blocks [b0, b0 + nblk).  In the dot, lane l works on pair l / LP, block b0 + (l % LP) / 2, half l % 2 of the block.  In
// the copy, the 2 * PPU row parts of the unit get LP / 2 lanes each: lane l copies chunks l % (LP/2), + LP/2, ... of part
// l / (LP/2).
// A "group" is the PPU pairs of a unit over all blocks of their rows; a warp processes whole groups, chunk by chunk,
// so that the running totals of the rows stay in its registers.

// blk0/blk1: the 144-byte blocks of rows A and B in the slot; xa: the block's 256 int8 activations; bs: its eight per-32 sums.
__device__ __forceinline__ int dp2a_lo(uint32_t a, uint32_t b, int c) {  // c + a.lo16 * b.byte0 + a.hi16 * b.byte1 (a signed, b unsigned)
    int d;
    asm("dp2a.lo.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int dp2a_hi(uint32_t a, uint32_t b, int c) {  // c + a.lo16 * b.byte2 + a.hi16 * b.byte3
    int d;
    asm("dp2a.hi.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// Lane `half` (0 or 1) of the two that share a cell: elements 128 half .. 128 half + 127 of the super-block, i.e. sub-blocks
// 4 half .. 4 half + 3, for rows A and B.  Returns this lane's part of the integer sums; the caller adds the two lanes'.
__device__ __forceinline__ void dot_half_q4k(uint32_t blk0, uint32_t blk1, uint32_t half, uint32_t xa, uint32_t bs, int isum[2], int imin[2], uint32_t dd[2]) {
    const uint32_t blk[2] = {blk0, blk1};
    uint32_t sc[2], mn[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const uint4 hd = lds128(blk[r]);
        dd[r] = hd.x;
        // the 6-bit scales and mins (engine/quant.rs:653-662) of this lane's four sub-blocks as bytes of one word each
        sc[r] = half ? ((hd.w & 0x0f0f0f0fu) | ((hd.y >> 2) & 0x30303030u)) : (hd.y & 0x3f3f3f3fu);
        mn[r] = half ? (((hd.w >> 4) & 0x0f0f0f0fu) | ((hd.z >> 2) & 0x30303030u)) : (hd.z & 0x3f3f3f3fu);
        isum[r] = 0;
    }
#pragma unroll
    for (int gg = 0; gg < 2; ++gg) {  // 64 elements: sub-blocks 4 half + 2 gg (low nibbles) and + 1 (high nibbles)
        const uint32_t xo = xa + 128 * half + 64 * gg, qo = 16 + 64 * half + 32 * gg;
        const uint4 x0 = lds128(xo), x1 = lds128(xo + 16), x2 = lds128(xo + 32), x3 = lds128(xo + 48);
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const uint4 qa = lds128(blk[r] + qo), qb = lds128(blk[r] + qo + 16);
            const uint32_t Lm = 0x0f0f0f0fu, Hm = 0xf0f0f0f0u;
            int lo0 = dp4a_us(qa.x & Lm, x0.x, 0), lo1 = dp4a_us(qa.y & Lm, x0.y, 0);
            lo0 = dp4a_us(qa.z & Lm, x0.z, lo0);
            lo1 = dp4a_us(qa.w & Lm, x0.w, lo1);
            lo0 = dp4a_us(qb.x & Lm, x1.x, lo0);
            lo1 = dp4a_us(qb.y & Lm, x1.y, lo1);
            lo0 = dp4a_us(qb.z & Lm, x1.z, lo0);
            lo1 = dp4a_us(qb.w & Lm, x1.w, lo1);
            int hi0 = dp4a_us(qa.x & Hm, x2.x, 0), hi1 = dp4a_us(qa.y & Hm, x2.y, 0);
            hi0 = dp4a_us(qa.z & Hm, x2.z, hi0);
            hi1 = dp4a_us(qa.w & Hm, x2.w, hi1);
            hi0 = dp4a_us(qb.x & Hm, x3.x, hi0);
            hi1 = dp4a_us(qb.y & Hm, x3.y, hi1);
            hi0 = dp4a_us(qb.z & Hm, x3.z, hi0);
            hi1 = dp4a_us(qb.w & Hm, x3.w, hi1);
            const int lo = lo0 + lo1, hi = (hi0 + hi1) >> 4;  // the high nibbles stayed in place: every product carried a factor 16
            const int sca = (int)((sc[r] >> (16 * gg)) & 0xff), scb = (int)((sc[r] >> (16 * gg + 8)) & 0xff);
            isum[r] += sca * lo + scb * hi;
        }
    }
    const uint2 bsv = lds64(bs + 8 * half);  // this lane's four per-32 sums as two pairs
#pragma unroll
    for (int r = 0; r < 2; ++r) imin[r] = dp2a_hi(bsv.y, mn[r], dp2a_lo(bsv.x, mn[r], 0));
}

// blk0/blk1: the 208-byte blocks [ql 128 | qh 64 | scales 16]; lane `h` takes elements 128 h .. 128 h + 127 (eight groups of 16).
__device__ __forceinline__ void dot_half_q6k(uint32_t blk0, uint32_t blk1, uint32_t h, uint32_t xa, uint32_t s16p, int isum[2]) {
    const uint32_t blk[2] = {blk0, blk1};
    uint32_t xw[32];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const uint4 v = lds128(xa + 128 * h + 16 * k);
        xw[4 * k] = v.x;
        xw[4 * k + 1] = v.y;
        xw[4 * k + 2] = v.z;
        xw[4 * k + 3] = v.w;
    }
    const uint4 sv = lds128(s16p + 16 * h);  // eight int16 sums, groups 8h .. 8h+7
    const int s16[8] = {(int16_t)(sv.x & 0xffff), (int16_t)(sv.x >> 16), (int16_t)(sv.y & 0xffff), (int16_t)(sv.y >> 16),
                        (int16_t)(sv.z & 0xffff), (int16_t)(sv.z >> 16), (int16_t)(sv.w & 0xffff), (int16_t)(sv.w >> 16)};
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const uint2 scw = lds64(blk[r] + 192 + 8 * h);  // signed scales of groups 8h .. 8h+7
        int dots[8] = {0, 0, 0, 0, 0, 0, 0, 0};  // group 2 * run + k
#pragma unroll
        for (int k = 0; k < 2; ++k) {  // k: 16-byte chunk of l (elements l = 16k .. 16k+15 of each run)
            const uint4 qla = lds128(blk[r] + 64 * h + 16 * k);       // runs 0 (low nibble) and 2 (high)
            const uint4 qlb = lds128(blk[r] + 64 * h + 32 + 16 * k);  // runs 1 and 3
            const uint4 qhv = lds128(blk[r] + 128 + 32 * h + 16 * k);
            const uint32_t A[4] = {qla.x, qla.y, qla.z, qla.w}, B[4] = {qlb.x, qlb.y, qlb.z, qlb.w}, Hh[4] = {qhv.x, qhv.y, qhv.z, qhv.w};
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const uint32_t v0 = (A[w] & 0x0f0f0f0fu) | ((Hh[w] << 4) & 0x30303030u);
                const uint32_t v1 = (B[w] & 0x0f0f0f0fu) | ((Hh[w] << 2) & 0x30303030u);
                const uint32_t v2 = ((A[w] >> 4) & 0x0f0f0f0fu) | (Hh[w] & 0x30303030u);
                const uint32_t v3 = ((B[w] >> 4) & 0x0f0f0f0fu) | ((Hh[w] >> 2) & 0x30303030u);
                const int wi = 4 * k + w;  // word index inside a 32-element run
                dots[0 + k] = dp4a_us(v0, xw[wi], dots[0 + k]);
                dots[2 + k] = dp4a_us(v1, xw[8 + wi], dots[2 + k]);
                dots[4 + k] = dp4a_us(v2, xw[16 + wi], dots[4 + k]);
                dots[6 + k] = dp4a_us(v3, xw[24 + wi], dots[6 + k]);
            }
        }
        const uint32_t scb[2] = {scw.x, scw.y};
        int acc = 0;
#pragma unroll
        for (int gi = 0; gi < 8; ++gi) {
            const int sc = (int)(int8_t)((scb[gi >> 2] >> (8 * (gi & 3))) & 0xff);
            acc += sc * (dots[gi] - 32 * s16[gi]);
        }
        isum[r] = acc;
    }
}

}  // namespace

}  // namespace ob
