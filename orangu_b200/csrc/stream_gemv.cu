// Single-token products for decode, built around the weight stream.
//
// One decode step reads every weight byte once and does almost nothing else, so the step time is the
// HBM time plus whatever stops the stream: kernel boundaries, the norm / quantize prologue, the ramp of
// a fresh kernel.  This kernel keeps the stream going through all of them:
//
//   * every warp owns two shared-memory slots and fills them with cp.async (16-byte, L1-bypassing) copies of
//     the next "units" of its rows, so about NW x 4.6-6.7 KB per SM is always in flight without holding
//     registers; the first units are requested before anything else happens;
//   * the operator that produces the activations is the kernel's prologue, computed by every CTA for itself
//     while those first units travel: RMSNorm (with the CPU's left-to-right sum, seqsum.cuh) or SwiGLU-free
//     plain input, then the int8 quantisation, written straight into shared memory in the layout the dot
//     loop reads without bank conflicts;
//   * the operator that consumes the product is its epilogue: residual add, silu(gate) * up, or RoPE and
//     the fp16 KV append for the q/k/v rows;
//   * the kernel is launched with programmatic stream serialisation: it may start, and request weights,
//     while its predecessor is still running (a CTA needs under half an SM's shared memory), and waits on
//     the grid dependency only before it reads the predecessor's output.
//
// Arithmetic is the single-token kernels of the reference, unchanged (engine/vecdot.rs:3152-3178 Q4_K,
// :3215-3241 Q6_K): exact integer partial sums, per-super-block fp32 terms with the reference's
// association, terms added in ascending block order by one lane.  Mapping: a unit is 16 super-blocks of
// two rows; two lanes share a super-block (half each, for both rows, so activations are read once per
// pair of rows); one shuffle completes the integer sums.
#include <cuda_pipeline.h>

#include "common.cuh"
#include "kernels.h"
#include "seqsum.cuh"

namespace ob {

namespace {

constexpr int SG_MAX_WARPS = 8;  // kernels whose segments include Q6_K (larger units) run 6 warps so that two CTAs still fit one SM
constexpr int UNIT_BLOCKS = 16;
constexpr uint32_t ACT_BLOCK_STRIDE = 288;  // bytes per 256 activations: [128][16 pad][128][16 pad]

__host__ __device__ inline uint32_t unit_row_bytes(uint32_t type) { return type == TYPE_Q4_K ? UNIT_BLOCKS * 144u : UNIT_BLOCKS * 208u + 32u; }

struct SgSmem {  // byte offsets inside dynamic shared memory
    uint32_t off_act, off_d, off_bsum, off_sum16, off_terms, off_x, off_ring, slot_bytes, total;
};

__host__ __device__ inline int sg_warps(bool has_q6) { return has_q6 ? 6 : 8; }

__host__ __device__ inline SgSmem sg_smem(uint32_t in_dim, bool has_q6, bool stage_x) {
    const uint32_t SG_WARPS = (uint32_t)sg_warps(has_q6);
    SgSmem s;
    const uint32_t nb = in_dim / 256;
    s.off_act = 64;                                   // [0,64): work counter and flags
    s.off_d = s.off_act + nb * ACT_BLOCK_STRIDE;
    s.off_bsum = (s.off_d + nb * 4 + 15) & ~15u;      // int16 [nb][8]  sums per 32
    s.off_sum16 = s.off_bsum + nb * 16;               // int16 [nb][16] sums per 16
    s.off_terms = s.off_sum16 + nb * 32;
    s.off_x = s.off_terms + SG_WARPS * 2 * UNIT_BLOCKS * 4;  // RMSNORM: the fp32 row, one pad word per 16
    s.off_ring = s.off_x + (stage_x ? ((in_dim + in_dim / 16 + 3) & ~3u) * 4 : 0u);
    s.slot_bytes = 2 * (has_q6 ? UNIT_BLOCKS * 208u + 32u : UNIT_BLOCKS * 144u);
    s.total = s.off_ring + SG_WARPS * 2 * s.slot_bytes;
    return s;
}

// position of activation element e (0..255) of block b inside the padded layout
__device__ __forceinline__ uint32_t act_pos(uint32_t b, uint32_t e) { return b * ACT_BLOCK_STRIDE + (e >> 7) * 144 + (e & 127); }

__device__ __forceinline__ float silu_mul_exact(float g, float u) {
    const float s = __fdiv_rn(g, __fadd_rn(1.0f, (float)exp((double)(-g))));
    return __fmul_rn(s, u);
}

// ---- prologue: activations of the single token, quantized per 256 into shared memory ---------------------
// Every warp takes blocks round-robin; a lane owns 8 consecutive elements of the block.
__device__ __forceinline__ uint32_t padded16(uint32_t i) { return i + (i >> 4); }

__device__ void sg_quantize(const StreamArgs &a, uint8_t *smem, const SgSmem &L, float norm_scale, uint32_t SG_WARPS, const float *sx) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t nb = a.in_dim / 256;
    float *sd = reinterpret_cast<float *>(smem + L.off_d);
    int16_t *bsum = reinterpret_cast<int16_t *>(smem + L.off_bsum);
    int16_t *sum16 = reinterpret_cast<int16_t *>(smem + L.off_sum16);
    for (uint32_t b = warp; b < nb; b += SG_WARPS) {
        const uint32_t e0 = b * 256 + lane * 8;
        float v[8];
        if (sx) {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = sx[padded16(e0 + i)];
        } else {
            const float4 x0 = *reinterpret_cast<const float4 *>(a.x + e0), x1 = *reinterpret_cast<const float4 *>(a.x + e0 + 4);
            v[0] = x0.x; v[1] = x0.y; v[2] = x0.z; v[3] = x0.w; v[4] = x1.x; v[5] = x1.y; v[6] = x1.z; v[7] = x1.w;
        }
        if (a.prologue == SG_PRO_RMSNORM) {
            const float4 w0 = *reinterpret_cast<const float4 *>(a.norm_w + e0), w1 = *reinterpret_cast<const float4 *>(a.norm_w + e0 + 4);
            const float w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = __fmul_rn(__fmul_rn(v[i], norm_scale), w[i]);  // (v * scale) * w, tensor.rs:747
        }
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
        *reinterpret_cast<uint2 *>(smem + L.off_act + act_pos(b, lane * 8)) = make_uint2(lo, hi);
        if ((lane & 1) == 0) sum16[b * 16 + (lane >> 1)] = (int16_t)s16;
        if ((lane & 3) == 0) bsum[b * 8 + (lane >> 2)] = (int16_t)s32;
        if (lane == 0) sd[b] = scale;
    }
}

// ---- units -------------------------------------------------------------------------------------------------
struct Unit {
    const uint8_t *rowA, *rowB;  // rowB == nullptr: the pair has one row
    uint32_t type, d_off;
    uint32_t b0, nblk, nb;       // blocks [b0, b0 + nblk) of nb
    uint32_t seg, pair;
    bool valid;
};

__device__ __forceinline__ void issue_part(uint8_t *dst, const uint8_t *row, const Unit &u, int lane) {
    if (u.type == TYPE_Q4_K) {
        const uint8_t *src = row + (uint64_t)u.b0 * 144;
        for (uint32_t c = lane; c < u.nblk * 9; c += 32) __pipeline_memcpy_async(dst + c * 16, src + c * 16, 16);
    } else {
        const uint8_t *src = row + (uint64_t)u.b0 * 208;
        for (uint32_t c = lane; c < u.nblk * 13; c += 32) __pipeline_memcpy_async(dst + c * 16, src + c * 16, 16);
        const uint8_t *dsrc = row + u.d_off + 2 * u.b0;  // f16 d values of these blocks: 16-byte aligned because b0 % 16 == 0
        if (lane < (int)((u.nblk * 2 + 15) / 16)) __pipeline_memcpy_async(dst + UNIT_BLOCKS * 208 + lane * 16, dsrc + lane * 16, 16);
    }
}

__device__ __forceinline__ void issue_unit(uint8_t *slot, const Unit &u, int lane) {
    issue_part(slot, u.rowA, u, lane);
    if (u.rowB) issue_part(slot + unit_row_bytes(u.type), u.rowB, u, lane);
}

// ---- dot of one unit: lane (bl = lane >> 1, hf = lane & 1) takes half hf of block b0 + bl, for both rows ------
__device__ __forceinline__ void dot_unit_q4k(const uint8_t *slot, const Unit &u, const uint8_t *smem, const SgSmem &L, float *terms, int lane) {
    const uint32_t bl = lane >> 1, hf = lane & 1;
    const bool live = bl < u.nblk;
    const uint32_t gb = u.b0 + (live ? bl : 0);
    const uint8_t *xa = smem + L.off_act + gb * ACT_BLOCK_STRIDE + hf * 144;
    uint4 x[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) x[k] = *reinterpret_cast<const uint4 *>(xa + 16 * k);
    const int16_t *bs = reinterpret_cast<const int16_t *>(smem + L.off_bsum) + gb * 8 + 4 * hf;
    const short4 bsv = *reinterpret_cast<const short4 *>(bs);  // sums of sub-blocks 4hf .. 4hf+3
    const float ad = reinterpret_cast<const float *>(smem + L.off_d)[gb];
    const int n_rows = u.rowB ? 2 : 1;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const uint8_t *blk = slot + r * (UNIT_BLOCKS * 144) + (live ? bl : 0) * 144;
        int isum = 0, imin = 0;
        uint4 hd = make_uint4(0, 0, 0, 0);
        if (r < n_rows) {
            hd = *reinterpret_cast<const uint4 *>(blk);
#pragma unroll
            for (int gi = 0; gi < 2; ++gi) {
                const int g = 2 * hf + gi;
                const uint4 qa = *reinterpret_cast<const uint4 *>(blk + 16 + 32 * g), qb = *reinterpret_cast<const uint4 *>(blk + 32 + 32 * g);
                // 6-bit scale / min of sub-blocks 2g and 2g+1 (engine/quant.rs:653-662) as byte pairs
                const uint32_t sh = 16u * (g & 1);
                const uint32_t a16 = hd.y >> sh, b16 = hd.z >> sh, p16 = hd.w >> sh;
                uint32_t scp, mp;
                if (g < 2) {
                    scp = a16 & 0x3f3fu;
                    mp = b16 & 0x3f3fu;
                } else {
                    scp = (p16 & 0x0f0fu) | ((a16 >> 2) & 0x3030u);
                    mp = ((p16 >> 4) & 0x0f0fu) | ((b16 >> 2) & 0x3030u);
                }
                const uint4 &x0 = x[4 * gi], &x1 = x[4 * gi + 1], &x2 = x[4 * gi + 2], &x3 = x[4 * gi + 3];
                const uint32_t Lm = 0x0f0f0f0fu, Hm = 0xf0f0f0f0u;
                int lo = dp4a_us(qa.x & Lm, x0.x, 0);
                lo = dp4a_us(qa.y & Lm, x0.y, lo);
                lo = dp4a_us(qa.z & Lm, x0.z, lo);
                lo = dp4a_us(qa.w & Lm, x0.w, lo);
                lo = dp4a_us(qb.x & Lm, x1.x, lo);
                lo = dp4a_us(qb.y & Lm, x1.y, lo);
                lo = dp4a_us(qb.z & Lm, x1.z, lo);
                lo = dp4a_us(qb.w & Lm, x1.w, lo);
                int hi = dp4a_us(qa.x & Hm, x2.x, 0);
                hi = dp4a_us(qa.y & Hm, x2.y, hi);
                hi = dp4a_us(qa.z & Hm, x2.z, hi);
                hi = dp4a_us(qa.w & Hm, x2.w, hi);
                hi = dp4a_us(qb.x & Hm, x3.x, hi);
                hi = dp4a_us(qb.y & Hm, x3.y, hi);
                hi = dp4a_us(qb.z & Hm, x3.z, hi);
                hi = dp4a_us(qb.w & Hm, x3.w, hi);
                hi >>= 4;  // the high nibbles stayed in place: every product carried a factor 16
                const int bsa = gi == 0 ? bsv.x : bsv.z, bsb = gi == 0 ? bsv.y : bsv.w;
                isum += (int)(scp & 0xff) * lo + (int)(scp >> 8) * hi;
                imin += (int)(mp & 0xff) * bsa + (int)(mp >> 8) * bsb;
            }
        }
        isum += __shfl_xor_sync(0xffffffffu, isum, 1);
        imin += __shfl_xor_sync(0xffffffffu, imin, 1);
        if (hf == 0 && live && r < n_rows) {
            const float d = f16_bits_to_f32(hd.x & 0xffffu), dmin = f16_bits_to_f32(hd.x >> 16);
            terms[r * UNIT_BLOCKS + bl] = __fmul_rn(ad, __fsub_rn(__fmul_rn(d, (float)isum), __fmul_rn(dmin, (float)imin)));
        }
    }
}

__device__ __forceinline__ void dot_unit_q6k(const uint8_t *slot, const Unit &u, const uint8_t *smem, const SgSmem &L, float *terms, int lane) {
    const uint32_t bl = lane >> 1, h = lane & 1;
    const bool live = bl < u.nblk;
    const uint32_t lb = live ? bl : 0, gb = u.b0 + lb;
    const uint8_t *xa = smem + L.off_act + gb * ACT_BLOCK_STRIDE + h * 144;
    uint32_t xw[32];  // activations 128h .. 128h+127 as 32 words
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const uint4 v = *reinterpret_cast<const uint4 *>(xa + 16 * k);
        xw[4 * k] = v.x;
        xw[4 * k + 1] = v.y;
        xw[4 * k + 2] = v.z;
        xw[4 * k + 3] = v.w;
    }
    const int16_t *s16p = reinterpret_cast<const int16_t *>(smem + L.off_sum16) + gb * 16 + 8 * h;
    const uint4 s16v = *reinterpret_cast<const uint4 *>(s16p);  // eight int16 sums, groups 8h .. 8h+7
    const int s16[8] = {(int16_t)(s16v.x & 0xffff), (int16_t)(s16v.x >> 16), (int16_t)(s16v.y & 0xffff), (int16_t)(s16v.y >> 16),
                        (int16_t)(s16v.z & 0xffff), (int16_t)(s16v.z >> 16), (int16_t)(s16v.w & 0xffff), (int16_t)(s16v.w >> 16)};
    const float ad = reinterpret_cast<const float *>(smem + L.off_d)[gb];
    const int n_rows = u.rowB ? 2 : 1;
    const uint32_t part = UNIT_BLOCKS * 208 + 32;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const uint8_t *blk = slot + r * part + lb * 208;
        int isum = 0;
        float dsup = 0.0f;
        if (r < n_rows) {
            const uint2 scw = *reinterpret_cast<const uint2 *>(blk + 192 + 8 * h);  // signed scales of groups 8h .. 8h+7
            dsup = f16_bits_to_f32(*reinterpret_cast<const unsigned short *>(slot + r * part + UNIT_BLOCKS * 208 + 2 * lb));
            int dots[8] = {0, 0, 0, 0, 0, 0, 0, 0};  // group 2*run + (w >> 2), run = 0..3
#pragma unroll
            for (int k = 0; k < 2; ++k) {  // k: 16-byte chunk of l (elements l = 16k .. 16k+15)
                const uint4 qla = *reinterpret_cast<const uint4 *>(blk + 64 * h + 16 * k);        // runs 0 (low nibble) and 2 (high)
                const uint4 qlb = *reinterpret_cast<const uint4 *>(blk + 64 * h + 32 + 16 * k);   // runs 1 and 3
                const uint4 qhv = *reinterpret_cast<const uint4 *>(blk + 128 + 32 * h + 16 * k);
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
            for (int gidx = 0; gidx < 8; ++gidx) {
                const int sc = (int)(int8_t)((scb[gidx >> 2] >> (8 * (gidx & 3))) & 0xff);
                isum += sc * (dots[gidx] - 32 * s16[gidx]);
            }
        }
        isum += __shfl_xor_sync(0xffffffffu, isum, 1);
        if (h == 0 && live && r < n_rows) terms[r * UNIT_BLOCKS + bl] = __fmul_rn(__fmul_rn(ad, dsup), (float)isum);
    }
}

// ---- the kernel ----------------------------------------------------------------------------------------------
template <int SG_WARPS>
__global__ void __launch_bounds__(SG_WARPS * 32, 2) stream_gemv_kernel(StreamArgs a) {
    constexpr int SG_THREADS = SG_WARPS * 32;
    constexpr bool has_q6 = SG_WARPS == 6;
    extern __shared__ __align__(16) uint8_t smem[];
    const SgSmem L = sg_smem(a.in_dim, has_q6, a.stage_x);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int *next_pair = reinterpret_cast<int *>(smem);
    float *bcast = reinterpret_cast<float *>(smem + 16);
    float *terms = reinterpret_cast<float *>(smem + L.off_terms) + warp * 2 * UNIT_BLOCKS;
    uint8_t *slots = smem + L.off_ring + (size_t)warp * 2 * L.slot_bytes;
    const uint32_t nb = a.in_dim / 256;

    // pairs of rows, segments concatenated; this CTA's contiguous share
    uint32_t pairs_of[3], total_pairs = 0;
    for (int s = 0; s < 3; ++s) {
        pairs_of[s] = s >= a.n_seg ? 0u : (a.seg[s].w2.data ? a.seg[s].w.out_dim : (a.seg[s].w.out_dim + 1) / 2);
        total_pairs += pairs_of[s];
    }
    const uint32_t p_begin = (uint32_t)(((uint64_t)total_pairs * blockIdx.x) / gridDim.x);
    const uint32_t p_end = (uint32_t)(((uint64_t)total_pairs * (blockIdx.x + 1)) / gridDim.x);
    if (threadIdx.x == 0) *next_pair = (int)p_begin;
    __syncthreads();

    // the stream of units this warp will process: pairs come off the shared counter, a pair's units in order
    Unit cur;  // the pair being expanded
    cur.valid = false;
    cur.b0 = 0;
    cur.nb = nb;
    auto next_unit = [&]() -> Unit {
        if (!cur.valid || cur.b0 + cur.nblk >= nb) {  // need a new pair
            int p = 0;
            if (lane == 0) p = atomicAdd(next_pair, 1);
            p = __shfl_sync(0xffffffffu, p, 0);
            if ((uint32_t)p >= p_end) {
                Unit none;
                none.valid = false;
                cur.valid = false;
                cur.nblk = nb;  // keeps asking (and failing) from here on
                return none;
            }
            uint32_t pi = (uint32_t)p;
            int s = 0;
            while (pi >= pairs_of[s]) {
                pi -= pairs_of[s];
                ++s;
            }
            const StreamSeg &sg = a.seg[s];
            cur.seg = (uint32_t)s;
            cur.pair = pi;
            cur.type = sg.w.type;
            cur.d_off = sg.w.d_off;
            if (sg.w2.data) {
                cur.rowA = sg.w.data + (uint64_t)pi * sg.w.row_stride;
                cur.rowB = sg.w2.data + (uint64_t)pi * sg.w2.row_stride;
            } else {
                cur.rowA = sg.w.data + (uint64_t)(2 * pi) * sg.w.row_stride;
                cur.rowB = 2 * pi + 1 < sg.w.out_dim ? cur.rowA + sg.w.row_stride : nullptr;
            }
            cur.b0 = 0;
            cur.valid = true;
        } else {
            cur.b0 += cur.nblk;
        }
        cur.nblk = min((uint32_t)UNIT_BLOCKS, nb - cur.b0);
        return cur;
    };

    // request the first two units before anything else: weights do not depend on the predecessor kernel
    Unit ring[2];
    ring[0] = next_unit();
    if (ring[0].valid) issue_unit(slots, ring[0], lane);
    __pipeline_commit();
    ring[1] = next_unit();
    if (ring[1].valid) issue_unit(slots + L.slot_bytes, ring[1], lane);
    __pipeline_commit();

    // ---- prologue ---------------------------------------------------------------------------------------------
    if (a.wait_dependency) {
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // the successor may start requesting its weights
        asm volatile("griddepcontrol.wait;" ::: "memory");               // the predecessor's output is complete and visible
    }
    float norm_scale = 1.0f;
    const float *sx = nullptr;
    if (a.prologue == SG_PRO_RMSNORM) {
        __shared__ SeqSumWorkspace<SG_THREADS> ws;
        const float *xr = a.x;
        float t;
        if (a.stage_x) {
            float *sxw = reinterpret_cast<float *>(smem + L.off_x);
            for (uint32_t i = threadIdx.x * 4; i < a.in_dim; i += SG_THREADS * 4) {
                const float4 v = *reinterpret_cast<const float4 *>(xr + i);
                sxw[padded16(i)] = v.x;
                sxw[padded16(i + 1)] = v.y;
                sxw[padded16(i + 2)] = v.z;
                sxw[padded16(i + 3)] = v.w;
            }
            __syncthreads();
            sx = sxw;
            t = cta_sequential_sum<SG_THREADS>([&](uint32_t i) { const float v = sx[padded16(i)]; return __fmul_rn(v, v); }, a.in_dim, ws);
        } else {
            t = cta_sequential_sum<SG_THREADS>([&](uint32_t i) { const float v = xr[i]; return __fmul_rn(v, v); }, a.in_dim, ws);
        }
        if (threadIdx.x == 0) *bcast = __fdiv_rn(1.0f, sqrtf(__fadd_rn(__fdiv_rn(t, (float)a.in_dim), a.eps)));
        __syncthreads();
        norm_scale = *bcast;
    }
    sg_quantize(a, smem, L, norm_scale, SG_WARPS, sx);
    __syncthreads();

    // ---- main loop ----------------------------------------------------------------------------------------------
    float tot = 0.0f;  // lane 0: row A, lane 1: row B of the current pair
    for (int i = 0; ring[i & 1].valid; ++i) {
        const Unit u = ring[i & 1];
        uint8_t *slot = slots + (size_t)(i & 1) * L.slot_bytes;
        __pipeline_wait_prior(1);
        __syncwarp();
        if (u.type == TYPE_Q4_K) dot_unit_q4k(slot, u, smem, L, terms, lane);
        else dot_unit_q6k(slot, u, smem, L, terms, lane);
        __syncwarp();
        // ordered sum of this unit's terms: lane r continues row r's running total (ascending blocks)
        if (u.b0 == 0) tot = 0.0f;
        if (lane < 2) {
            const float4 *tp = reinterpret_cast<const float4 *>(terms + lane * UNIT_BLOCKS);
            const float4 t0 = tp[0], t1 = tp[1], t2 = tp[2], t3 = tp[3];
            const float tv[16] = {t0.x, t0.y, t0.z, t0.w, t1.x, t1.y, t1.z, t1.w, t2.x, t2.y, t2.z, t2.w, t3.x, t3.y, t3.z, t3.w};
#pragma unroll
            for (int b = 0; b < UNIT_BLOCKS; ++b)
                if ((uint32_t)b < u.nblk) tot = __fadd_rn(tot, tv[b]);
        }
        __syncwarp();
        // refill the slot just consumed
        ring[i & 1] = next_unit();
        if (ring[i & 1].valid) issue_unit(slot, ring[i & 1], lane);
        __pipeline_commit();

        if (u.b0 + u.nblk < nb) continue;
        // ---- epilogue of the finished pair ----------------------------------------------------------------------
        const float tA = __shfl_sync(0xffffffffu, tot, 0), tB = __shfl_sync(0xffffffffu, tot, 1);
        if (lane != 0) continue;
        const StreamSeg &sg = a.seg[u.seg];
        const bool hasB = u.rowB != nullptr;
        switch (sg.epilogue) {
        case SG_EP_STORE:
            sg.y[2 * u.pair] = tA;
            if (hasB) sg.y[2 * u.pair + 1] = tB;
            break;
        case SG_EP_RESIDUAL:
            sg.y[2 * u.pair] = __fadd_rn(a.residual[2 * u.pair], tA);
            if (hasB) sg.y[2 * u.pair + 1] = __fadd_rn(a.residual[2 * u.pair + 1], tB);
            break;
        case SG_EP_SWIGLU:
            sg.y[u.pair] = silu_mul_exact(tA, tB);
            break;
        default: {  // q, k, v rows of the token: rotate (q, k) and append (k, v) to the page as f16
            const uint32_t row = 2 * u.pair, hd = a.head_dim, head = row / hd, idx = (row % hd) / 2;
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
    return sg_smem(a.in_dim, q6, false).total <= 108 * 1024;
}

void launch_stream_gemv(const StreamArgs &a, int sm_count, bool programmatic, cudaStream_t st) {
    bool q6 = false;
    uint32_t pairs = 0;
    for (int s = 0; s < a.n_seg; ++s) {
        q6 = q6 || a.seg[s].w.type == TYPE_Q6_K;
        pairs += a.seg[s].w2.data ? a.seg[s].w.out_dim : (a.seg[s].w.out_dim + 1) / 2;
    }
    const bool stage_x = a.prologue == SG_PRO_RMSNORM && sg_smem(a.in_dim, q6, true).total <= 108 * 1024;
    const SgSmem L = sg_smem(a.in_dim, q6, stage_x);
    static bool configured = false;
    if (!configured) {
        cudaFuncSetAttribute(stream_gemv_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 108 * 1024);
        cudaFuncSetAttribute(stream_gemv_kernel<6>, cudaFuncAttributeMaxDynamicSharedMemorySize, 108 * 1024);
        configured = true;
    }
    StreamArgs args = a;
    args.wait_dependency = programmatic;
    args.stage_x = stage_x;
    const uint32_t nw = (uint32_t)sg_warps(q6);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(std::min<uint32_t>(2u * (uint32_t)sm_count, std::max(1u, (pairs + nw - 1) / nw)));  // two CTAs per SM
    cfg.blockDim = dim3(nw * 32);
    cfg.dynamicSmemBytes = L.total;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = programmatic ? 1 : 0;
    if (q6) cudaLaunchKernelEx(&cfg, stream_gemv_kernel<6>, args);
    else cudaLaunchKernelEx(&cfg, stream_gemv_kernel<8>, args);
}

}  // namespace ob
