// Single-token products for decode, built around the weight stream.
//
// One decode step reads every weight byte once and does almost nothing else, so the step time is the
// HBM time plus whatever stops the stream: kernel boundaries, the norm / quantize prologue, the ramp of
// a fresh kernel -- and, on this part, instruction issue: at 6.5 TB/s an SM receives 23 bytes per clock
// and can issue at most four warp instructions in that clock, so the dot loop has to spend well under one
// instruction per 10 bytes.  Hence:
//
//   * one lane owns one whole super-block, for two rows at once: the six-bit scales of the block are unpacked
//     once (10 instructions for all eight scales and mins), the activations are read once per pair of rows,
//     and no cross-lane reduction is needed for the integer sums;
//   * every warp owns two shared-memory slots and fills them with cp.async (16-byte, L1-bypassing) copies of
//     its next "units" (32 lanes' worth of blocks, two rows each), so the bytes in flight do not occupy
//     registers; the first units are requested before anything else happens in the kernel;
//   * the operator that produces the activations is the kernel's prologue (RMSNorm scaling and the int8
//     quantisation, written straight into shared memory in a conflict-free layout), and the operator that
//     consumes the product is its epilogue (residual add, silu(gate) * up, or RoPE and the fp16 KV append);
//   * two small CTAs fit one SM, and the kernel is launched with programmatic stream serialisation: it may
//     start, and request weights, while its predecessor is still running, and waits on the grid dependency
//     only before it reads the predecessor's output.
//
// Arithmetic is the single-token kernels of the reference, unchanged (engine/vecdot.rs:3152-3178 Q4_K,
// :3215-3241 Q6_K): exact integer partial sums, per-super-block fp32 terms with the reference's
// association, terms added in ascending block order by one lane.  The RMSNorm scale comes from
// norm_scale_kernel, which reproduces the CPU's left-to-right sum of squares (seqsum.cuh).
#include <cuda_pipeline.h>

#include "common.cuh"
#include "kernels.h"
#include "seqsum.cuh"

namespace ob {

namespace {

constexpr uint32_t ACT_BLOCK_STRIDE = 272;  // bytes per 256 int8 activations: 17 sixteen-byte chunks, so lanes one block apart hit different banks

// bytes of `lp` blocks of one row inside a slot
__host__ __device__ inline uint32_t part_bytes(uint32_t type, uint32_t lp) { return type == TYPE_Q4_K ? lp * 144u : lp * 208u + ((lp * 2u + 15u) & ~15u); }

// lanes per pair of rows: the smallest power of two that covers min(nb, 32) blocks; at least 2, because each pair also
// needs two lanes for the ordered sums of its two rows
__host__ __device__ inline uint32_t lanes_per_pair(uint32_t nb) {
    uint32_t lp = 2;
    while (lp < nb && lp < 32) lp <<= 1;
    return lp;
}

__host__ __device__ inline int sg_warps(bool has_q6) { return has_q6 ? 3 : 4; }

struct SgSmem {  // byte offsets inside dynamic shared memory
    uint32_t off_act, off_d, off_bsum, off_sum16, off_terms, off_ring, slot_bytes, total;
};

__host__ __device__ inline SgSmem sg_smem(uint32_t in_dim, bool has_q6) {
    SgSmem s;
    const uint32_t nb = in_dim / 256, nw = (uint32_t)sg_warps(has_q6), lp = lanes_per_pair(nb);
    s.off_act = 64;  // [0,64): work counter and broadcast words
    s.off_d = s.off_act + nb * ACT_BLOCK_STRIDE;
    s.off_bsum = (s.off_d + nb * 4 + 15) & ~15u;  // int16 [nb][8]  sums per 32
    s.off_sum16 = s.off_bsum + nb * 16;            // int16 [nb][16] sums per 16
    s.off_terms = s.off_sum16 + nb * 32;           // float [warp][pair slot][row][lp]  = [warp][64]
    s.off_ring = s.off_terms + nw * 64 * 4;
    s.slot_bytes = (32 / lp) * 2 * part_bytes(has_q6 ? TYPE_Q6_K : TYPE_Q4_K, lp);
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

// ---- prologue: activations of the single token, quantized per 256 into shared memory ---------------------
// Every warp takes blocks round-robin; a lane owns 8 consecutive elements of the block.
__device__ void sg_quantize(const StreamArgs &a, uint8_t *smem, const SgSmem &L, float norm_scale, uint32_t n_warps) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t nb = a.in_dim / 256;
    float *sd = reinterpret_cast<float *>(smem + L.off_d);
    int16_t *bsum = reinterpret_cast<int16_t *>(smem + L.off_bsum);
    int16_t *sum16 = reinterpret_cast<int16_t *>(smem + L.off_sum16);
    // four blocks per pass, all their loads issued before any arithmetic: the pass costs one memory latency, not four
    for (uint32_t bb = warp; bb < nb; bb += 4 * n_warps) {
        float v[4][8];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const uint32_t b = bb + k * n_warps;
            if (b < nb) {
                const uint32_t e0 = b * 256 + lane * 8;
                const float4 x0 = *reinterpret_cast<const float4 *>(a.x + e0), x1 = *reinterpret_cast<const float4 *>(a.x + e0 + 4);
                v[k][0] = x0.x; v[k][1] = x0.y; v[k][2] = x0.z; v[k][3] = x0.w; v[k][4] = x1.x; v[k][5] = x1.y; v[k][6] = x1.z; v[k][7] = x1.w;
            }
        }
        if (a.prologue == SG_PRO_RMSNORM) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const uint32_t b = bb + k * n_warps;
                if (b < nb) {
                    const uint32_t e0 = b * 256 + lane * 8;
                    const float4 w0 = __ldg(reinterpret_cast<const float4 *>(a.norm_w + e0)), w1 = __ldg(reinterpret_cast<const float4 *>(a.norm_w + e0 + 4));
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
            float amax = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[k][i]));
            amax = warp_max(amax);
            const float scale = __fdiv_rn(amax, 127.0f);
            const float inv = scale > 0.0f ? __fdiv_rn(1.0f, scale) : 0.0f;
            int q[8], s8 = 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                q[i] = quantize_value(v[k][i], inv);
                s8 += q[i];
            }
            const int s16 = s8 + __shfl_xor_sync(0xffffffffu, s8, 1);
            const int s32 = s16 + __shfl_xor_sync(0xffffffffu, s16, 2);
            const uint32_t lo = (q[0] & 0xff) | ((q[1] & 0xff) << 8) | ((q[2] & 0xff) << 16) | ((uint32_t)(q[3] & 0xff) << 24);
            const uint32_t hi = (q[4] & 0xff) | ((q[5] & 0xff) << 8) | ((q[6] & 0xff) << 16) | ((uint32_t)(q[7] & 0xff) << 24);
            *reinterpret_cast<uint2 *>(smem + L.off_act + b * ACT_BLOCK_STRIDE + lane * 8) = make_uint2(lo, hi);
            if ((lane & 1) == 0) sum16[b * 16 + (lane >> 1)] = (int16_t)s16;
            if ((lane & 3) == 0) bsum[b * 8 + (lane >> 2)] = (int16_t)s32;
            if (lane == 0) sd[b] = scale;
        }
    }
}

// ---- units ---------------------------------------------------------------------------------------------------
// A unit is what one warp processes at a time: `ppu` pairs of rows (32 / lp of them, consecutive in one
// segment) x up to lp blocks [b0, b0 + nblk).  Lane l works on pair l / lp, block b0 + l % lp.
struct Unit {
    uint32_t seg, pair0, n_pairs;  // pairs pair0 .. pair0 + n_pairs - 1 of segment seg
    uint32_t b0, nblk;
    bool valid;
};

__device__ __forceinline__ void pair_rows(const StreamSeg &sg, uint32_t pair, const uint8_t *&rowA, const uint8_t *&rowB) {
    if (sg.w2.data) {
        rowA = sg.w.data + (uint64_t)pair * sg.w.row_stride;
        rowB = sg.w2.data + (uint64_t)pair * sg.w2.row_stride;
    } else {
        rowA = sg.w.data + (uint64_t)(2 * pair) * sg.w.row_stride;
        rowB = 2 * pair + 1 < sg.w.out_dim ? rowA + sg.w.row_stride : nullptr;
    }
}

__device__ __forceinline__ void issue_part(uint32_t dst, const uint8_t *row, uint32_t type, uint32_t d_off, uint32_t lp, uint32_t b0, uint32_t nblk,
                                           int lane) {
    if (type == TYPE_Q4_K) {
        const uint8_t *src = row + (uint64_t)b0 * 144 + lane * 16;
        dst += lane * 16;
        for (uint32_t c = lane; c < nblk * 9; c += 32, src += 512, dst += 512) cp_async16(dst, src);
    } else {
        const uint8_t *src = row + (uint64_t)b0 * 208 + lane * 16;
        uint32_t dm = dst + lane * 16;
        for (uint32_t c = lane; c < nblk * 13; c += 32, src += 512, dm += 512) cp_async16(dm, src);
        const uint8_t *dsrc = row + d_off + 2 * b0;  // f16 d values of these blocks; b0 is a multiple of 32, so 16-byte aligned
        if (lane < (int)((nblk * 2 + 15) / 16)) cp_async16(dst + lp * 208 + lane * 16, dsrc + lane * 16);
    }
}

__device__ __forceinline__ void issue_unit(uint32_t slot, const StreamArgs &a, const Unit &u, uint32_t lp, int lane) {
    const StreamSeg &sg = a.seg[u.seg];
    const uint32_t pb = part_bytes(sg.w.type, lp);
    for (uint32_t j = 0; j < u.n_pairs; ++j) {
        const uint8_t *rowA, *rowB;
        pair_rows(sg, u.pair0 + j, rowA, rowB);
        issue_part(slot + (2 * j) * pb, rowA, sg.w.type, sg.w.d_off, lp, u.b0, u.nblk, lane);
        if (rowB) issue_part(slot + (2 * j + 1) * pb, rowB, sg.w.type, sg.w.d_off, lp, u.b0, u.nblk, lane);
    }
}

// ---- dot of one super-block for two rows, by one lane -------------------------------------------------------------
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

// blk[r]: the 144-byte block of row r in the slot; xa: the block's 256 int8 activations; bs: its eight per-32 sums.
__device__ __forceinline__ void dot_block_q4k(uint32_t blk0, uint32_t blk1, int n_rows, uint32_t xa, uint32_t bs, float ad, float term[2]) {
    const uint32_t blk[2] = {blk0, blk1};
    uint32_t scl[2], sch[2], ml[2], mh[2], dd[2];
    int isum[2] = {0, 0};
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        uint4 hd = make_uint4(0, 0, 0, 0);
        if (r < n_rows) hd = lds128(blk[r]);
        dd[r] = hd.x;
        // the eight 6-bit scales and mins (engine/quant.rs:653-662) as bytes of four words
        scl[r] = hd.y & 0x3f3f3f3fu;
        ml[r] = hd.z & 0x3f3f3f3fu;
        sch[r] = (hd.w & 0x0f0f0f0fu) | ((hd.y >> 2) & 0x30303030u);
        mh[r] = ((hd.w >> 4) & 0x0f0f0f0fu) | ((hd.z >> 2) & 0x30303030u);
    }
#pragma unroll
    for (int g = 0; g < 4; ++g) {  // 64 elements: sub-blocks 2g (low nibbles) and 2g+1 (high nibbles)
        const uint4 x0 = lds128(xa + 64 * g), x1 = lds128(xa + 64 * g + 16), x2 = lds128(xa + 64 * g + 32), x3 = lds128(xa + 64 * g + 48);
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            if (r >= n_rows) continue;
            const uint4 qa = lds128(blk[r] + 16 + 32 * g), qb = lds128(blk[r] + 32 + 32 * g);
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
            const uint32_t scw = g < 2 ? scl[r] : sch[r];
            const int sca = (int)((scw >> (16 * (g & 1))) & 0xff), scb = (int)((scw >> (16 * (g & 1) + 8)) & 0xff);
            isum[r] += sca * lo + scb * hi;
        }
    }
    const uint4 bsv = lds128(bs);  // eight int16 sums as four pairs
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        int imin = dp2a_lo(bsv.x, ml[r], 0);
        imin = dp2a_hi(bsv.y, ml[r], imin);
        imin = dp2a_lo(bsv.z, mh[r], imin);
        imin = dp2a_hi(bsv.w, mh[r], imin);
        const float d = f16_bits_to_f32(dd[r] & 0xffffu), dmin = f16_bits_to_f32(dd[r] >> 16);
        term[r] = __fmul_rn(ad, __fsub_rn(__fmul_rn(d, (float)isum[r]), __fmul_rn(dmin, (float)imin)));
    }
}

// blk[r]: the 208-byte block [ql 128 | qh 64 | scales 16]; dsup[r]: its f16 d; s16: the block's sixteen per-16 sums.
__device__ __forceinline__ void dot_block_q6k(uint32_t blk0, uint32_t blk1, const float dsup[2], int n_rows, uint32_t xa, uint32_t s16p, float ad,
                                              float term[2]) {
    const uint32_t blk[2] = {blk0, blk1};
    int isum[2] = {0, 0};
#pragma unroll
    for (int h = 0; h < 2; ++h) {  // 128 elements: runs 0..3 of 32
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
            if (r >= n_rows) continue;
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
#pragma unroll
            for (int gi = 0; gi < 8; ++gi) {
                const int sc = (int)(int8_t)((scb[gi >> 2] >> (8 * (gi & 3))) & 0xff);
                isum[r] += sc * (dots[gi] - 32 * s16[gi]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) term[r] = __fmul_rn(__fmul_rn(ad, dsup[r]), (float)isum[r]);
}

// ---- the kernel ----------------------------------------------------------------------------------------------
template <int NW>
__global__ void __launch_bounds__(NW * 32, 2) stream_gemv_kernel(StreamArgs a) {
    extern __shared__ __align__(16) uint8_t smem[];
    constexpr bool has_q6 = NW == 3;
    const SgSmem L = sg_smem(a.in_dim, has_q6);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int *next_group = reinterpret_cast<int *>(smem);
    const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(smem);
    const uint32_t terms = sbase + L.off_terms + warp * 256;
    const uint32_t slots = sbase + L.off_ring + warp * 2 * L.slot_bytes;
    const uint32_t nb = a.in_dim / 256, lp = lanes_per_pair(nb), ppu = 32 / lp;

    // groups of ppu pairs, segments concatenated (a group never straddles two segments); this CTA's contiguous share
    uint32_t groups_of[3], pairs_of[3], total_groups = 0;
    for (int s = 0; s < 3; ++s) {
        pairs_of[s] = s >= a.n_seg ? 0u : (a.seg[s].w2.data ? a.seg[s].w.out_dim : (a.seg[s].w.out_dim + 1) / 2);
        groups_of[s] = (pairs_of[s] + ppu - 1) / ppu;
        total_groups += groups_of[s];
    }
    const uint32_t g_begin = (uint32_t)(((uint64_t)total_groups * blockIdx.x) / gridDim.x);
    const uint32_t g_end = (uint32_t)(((uint64_t)total_groups * (blockIdx.x + 1)) / gridDim.x);
    if (threadIdx.x == 0) *next_group = (int)g_begin;
    __syncthreads();

    // the stream of units this warp will process: groups come off the shared counter, a group's units in block order
    Unit cur;
    cur.valid = false;
    cur.b0 = 0;
    cur.nblk = nb;
    auto next_unit = [&]() -> Unit {
        if (!cur.valid || cur.b0 + cur.nblk >= nb) {  // need a new group
            int g = 0;
            if (lane == 0) g = atomicAdd(next_group, 1);
            g = __shfl_sync(0xffffffffu, g, 0);
            if ((uint32_t)g >= g_end) {
                cur.valid = false;
                cur.nblk = nb;
                return cur;
            }
            uint32_t gi = (uint32_t)g;
            int s = 0;
            while (gi >= groups_of[s]) {
                gi -= groups_of[s];
                ++s;
            }
            cur.seg = (uint32_t)s;
            cur.pair0 = gi * ppu;
            cur.n_pairs = min(ppu, pairs_of[s] - cur.pair0);
            cur.b0 = 0;
            cur.valid = true;
        } else {
            cur.b0 += cur.nblk;
        }
        cur.nblk = min(lp, nb - cur.b0);
        return cur;
    };

    // request the first two units before anything else: weights do not depend on the predecessor kernel
    Unit u0 = next_unit();
    if (u0.valid) issue_unit(slots, a, u0, lp, lane);
    __pipeline_commit();
    Unit u1 = next_unit();
    if (u1.valid) issue_unit(slots + L.slot_bytes, a, u1, lp, lane);
    __pipeline_commit();

    // ---- prologue ---------------------------------------------------------------------------------------------
    if (a.wait_dependency) {
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // the successor may start requesting its weights
        asm volatile("griddepcontrol.wait;" ::: "memory");               // the predecessor's output is complete and visible
    }
    const float norm_scale = a.prologue == SG_PRO_RMSNORM ? *a.norm_scale : 1.0f;
    sg_quantize(a, smem, L, norm_scale, NW);
    __syncthreads();

    // ---- main loop: slot 0 / slot 1 alternate ---------------------------------------------------------------------
    const uint32_t pj = lane / lp, bl = lane % lp;
    float tot = 0.0f;  // lanes 2j, 2j+1: rows A, B of the unit's pair j (running over the units of a long row)
    for (int i = 0;; ++i) {
        const Unit u = (i & 1) ? u1 : u0;
        if (!u.valid) break;
        const uint32_t slot = slots + (i & 1) * L.slot_bytes;
        __pipeline_wait_prior(1);
        __syncwarp();
        {
            const StreamSeg &sg = a.seg[u.seg];
            const bool live = pj < u.n_pairs && bl < u.nblk;
            const uint32_t lb = live ? bl : 0, lpj = live ? pj : 0, gb = u.b0 + lb;
            const uint32_t pb = part_bytes(sg.w.type, lp);
            const bool two = sg.w2.data != nullptr || 2 * (u.pair0 + lpj) + 1 < sg.w.out_dim;
            const uint32_t xa = sbase + L.off_act + gb * ACT_BLOCK_STRIDE;
            const float ad = __uint_as_float(lds32(sbase + L.off_d + gb * 4));
            float term[2];
            if (sg.w.type == TYPE_Q4_K) {
                dot_block_q4k(slot + (2 * lpj) * pb + lb * 144, slot + (2 * lpj + 1) * pb + lb * 144, two ? 2 : 1, xa, sbase + L.off_bsum + gb * 16, ad, term);
            } else {
                const uint32_t pA = slot + (2 * lpj) * pb, pB = pA + pb;
                const float dsup[2] = {f16_bits_to_f32(lds16(pA + lp * 208 + 2 * lb)), two ? f16_bits_to_f32(lds16(pB + lp * 208 + 2 * lb)) : 0.0f};
                dot_block_q6k(pA + lb * 208, pB + lb * 208, dsup, two ? 2 : 1, xa, sbase + L.off_sum16 + gb * 32, ad, term);
            }
            if (live) {
                sts32(terms + ((2 * pj) * lp + bl) * 4, term[0]);
                sts32(terms + ((2 * pj + 1) * lp + bl) * 4, term[1]);
            }
        }
        __syncwarp();
        // ordered sum: lane s < 2 * ppu continues the running total of (pair s / 2, row s % 2) over this unit's blocks, in order
        if (u.b0 == 0) tot = 0.0f;
        if (lane < (int)(2 * ppu)) {
            const uint32_t tp = terms + lane * lp * 4;
            for (uint32_t b = 0; b < u.nblk; b += 4) {
                float t4[4];
                if (lp >= 4) {
                    const uint4 v = lds128(tp + b * 4);
                    t4[0] = __uint_as_float(v.x); t4[1] = __uint_as_float(v.y); t4[2] = __uint_as_float(v.z); t4[3] = __uint_as_float(v.w);
                } else {
                    for (int k = 0; k < 4; ++k) t4[k] = b + k < lp ? __uint_as_float(lds32(tp + (b + k) * 4)) : 0.0f;
                }
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    if (b + k < u.nblk) tot = __fadd_rn(tot, t4[k]);
            }
        }
        __syncwarp();
        // refill the slot just consumed
        const Unit nu = next_unit();
        if (nu.valid) issue_unit(slot, a, nu, lp, lane);
        __pipeline_commit();
        if (i & 1) u1 = nu;
        else u0 = nu;

        if (u.b0 + u.nblk < nb) continue;
        // ---- epilogue of the finished pairs: lane 2j holds row A's total, lane 2j+1 row B's --------------------------
        const float tB = __shfl_down_sync(0xffffffffu, tot, 1);
        if ((lane & 1) || lane >= (int)(2 * u.n_pairs)) continue;
        const float tA = tot;
        const StreamSeg &sg = a.seg[u.seg];
        const uint32_t pair = u.pair0 + (lane >> 1);
        const bool hasB = sg.w2.data != nullptr || 2 * pair + 1 < sg.w.out_dim;
        switch (sg.epilogue) {
        case SG_EP_STORE:
            sg.y[2 * pair] = tA;
            if (hasB) sg.y[2 * pair + 1] = tB;
            break;
        case SG_EP_RESIDUAL:
            sg.y[2 * pair] = __fadd_rn(a.residual[2 * pair], tA);
            if (hasB) sg.y[2 * pair + 1] = __fadd_rn(a.residual[2 * pair + 1], tB);
            break;
        case SG_EP_SWIGLU:
            sg.y[pair] = silu_mul_exact(tA, tB);
            break;
        default: {  // q, k, v rows of the token: rotate (q, k) and append (k, v) to the page as f16
            const uint32_t row = 2 * pair, hd = a.head_dim, head = row / hd, idx = (row % hd) / 2;
            const uint32_t pos = *a.position;
            float oa = tA, ob_ = tB;
            if (sg.epilogue != SG_EP_V && 2 * idx < a.rope_dim) {
                const float2 sc = reinterpret_cast<const float2 *>(a.rope_table)[(uint64_t)pos * (a.rope_dim / 2) + idx];  // (sin, cos)
                oa = __fsub_rn(__fmul_rn(tA, sc.y), __fmul_rn(tB, sc.x));
                ob_ = __fadd_rn(__fmul_rn(tA, sc.x), __fmul_rn(tB, sc.y));
            }
            if (sg.epilogue == SG_EP_ROPE_Q) {
                sg.y[row] = oa;
                sg.y[row + 1] = ob_;
            } else {
                const int32_t page = (*a.page_table)[pos / KV_PAGE];
                const uint64_t o = (((uint64_t)page * a.n_head_kv + head) * KV_PAGE + pos % KV_PAGE) * hd + (row % hd);
                __half *pool = sg.epilogue == SG_EP_ROPE_K ? a.k_pool : a.v_pool;
                *reinterpret_cast<__half2 *>(pool + o) = __floats2half2_rn(oa, ob_);
            }
            break;
        }
        }
    }
    __pipeline_wait_prior(0);
}

// 1 / sqrt(mean(x^2) + eps) with the squares added left to right (engine/tensor.rs:743-745), one CTA.
constexpr int NS_THREADS = 1024;
__global__ void __launch_bounds__(NS_THREADS) norm_scale_kernel(const float *__restrict__ x, uint32_t dim, float eps, float *__restrict__ out,
                                                                bool wait_dependency) {
    extern __shared__ float srow[];  // the row, one pad word per 16
    __shared__ SeqSumWorkspace<NS_THREADS> ws;
    if (wait_dependency) {
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
        asm volatile("griddepcontrol.wait;" ::: "memory");
    }
    for (uint32_t i = threadIdx.x; i < dim; i += NS_THREADS) srow[i + (i >> 4)] = x[i];
    __syncthreads();
    const float t = cta_sequential_sum<NS_THREADS>([&](uint32_t i) { const float v = srow[i + (i >> 4)]; return __fmul_rn(v, v); }, dim, ws);
    if (threadIdx.x == 0) *out = __fdiv_rn(1.0f, sqrtf(__fadd_rn(__fdiv_rn(t, (float)dim), eps)));
}

}  // namespace

bool stream_gemv_supported(const StreamArgs &a) {
    if (a.n_seg < 1 || a.n_seg > 3 || a.in_dim % 256) return false;
    bool q6 = false;
    for (int s = 0; s < a.n_seg; ++s) {
        const StreamSeg &g = a.seg[s];
        if (g.w.type != TYPE_Q4_K && g.w.type != TYPE_Q6_K) return false;
        if (g.w.in_dim != a.in_dim) return false;
        if (g.w2.data && (g.w2.type != g.w.type || g.w2.in_dim != a.in_dim || g.w2.out_dim != g.w.out_dim)) return false;
        if (g.epilogue >= SG_EP_ROPE_Q && (g.w.out_dim & 1)) return false;
        q6 = q6 || g.w.type == TYPE_Q6_K;
    }
    return sg_smem(a.in_dim, q6).total <= 108 * 1024;
}

void launch_norm_scale(const float *x, uint32_t dim, float eps, float *out, bool programmatic, cudaStream_t st) {
    static bool configured = false;
    if (!configured) {
        cudaFuncSetAttribute(norm_scale_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
        configured = true;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(1);
    cfg.blockDim = dim3(NS_THREADS);
    cfg.dynamicSmemBytes = ((size_t)dim + dim / 16 + 16) * 4;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = programmatic ? 1 : 0;
    cudaLaunchKernelEx(&cfg, norm_scale_kernel, x, dim, eps, out, programmatic);
}

void launch_stream_gemv(const StreamArgs &a, int sm_count, bool programmatic, cudaStream_t st) {
    bool q6 = false;
    uint32_t pairs = 0;
    for (int s = 0; s < a.n_seg; ++s) {
        q6 = q6 || a.seg[s].w.type == TYPE_Q6_K;
        pairs += a.seg[s].w2.data ? a.seg[s].w.out_dim : (a.seg[s].w.out_dim + 1) / 2;
    }
    const SgSmem L = sg_smem(a.in_dim, q6);
    static bool configured = false;
    if (!configured) {
        cudaFuncSetAttribute(stream_gemv_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 108 * 1024);
        cudaFuncSetAttribute(stream_gemv_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, 108 * 1024);
        configured = true;
    }
    StreamArgs args = a;
    args.wait_dependency = programmatic;
    const uint32_t nw = (uint32_t)sg_warps(q6), ppu = 32 / lanes_per_pair(a.in_dim / 256);
    const uint32_t groups = (pairs + ppu - 1) / ppu;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(std::min<uint32_t>(2u * (uint32_t)sm_count, std::max(1u, (groups + nw - 1) / nw)));  // two CTAs per SM
    cfg.blockDim = dim3(nw * 32);
    cfg.dynamicSmemBytes = L.total;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = programmatic ? 1 : 0;
    if (q6) cudaLaunchKernelEx(&cfg, stream_gemv_kernel<3>, args);
    else cudaLaunchKernelEx(&cfg, stream_gemv_kernel<4>, args);
}

}  // namespace ob
