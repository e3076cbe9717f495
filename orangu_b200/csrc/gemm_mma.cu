// Many-token products (batched decode, prefill) of K-quant matrices on the tensor cores.
//
// With T tokens the product is a genuine contraction: every weight byte meets T activations, and the dp4a kernel of
// gemv.cu, which re-reads the weights once per tile of 8 tokens, is bound by instruction issue at a few TMAC/s.  Here a
// warp owns a tile of 16 rows x 64 tokens and walks the row's super-blocks in order.  For every 32-element sub-block
// the 4-bit codes of the 16 rows are one A fragment of mma.sync.m16n8k32 (u8 x s8 -> s32) -- a masked 32-bit word of
// the GGUF block is exactly the four consecutive codes a thread has to supply -- and the int8 activations of 8 tokens
// are the B fragment, so one instruction gives the sub-block's 128 integer dot products.  They are scaled by the 6-bit
// sub-block scale in int32 (exact), the min term comes from the per-32 activation sums with dp2a, and the fp32 term of
// the super-block is formed and accumulated per (row, token) exactly as the CPU kernels do:
//   decode order   total += ad * (d * isum - dmin * imin)                        (engine/vecdot.rs:3152-3178)
//   prefill order  pass 1: total -= (ad * dmin) * imin over all super-blocks;  pass 2: total += ad * (d * isum)
//                                                                                 (engine/vecdot.rs:2119-2143, 2213-2255)
// so the results equal the single-token kernels' and the CPU's bit for bit, whatever the batch size.
//
// A CTA is four warps = 64 rows sharing a 64-token activation tile; the weight blocks (64 x 144 B), the activations
// (64 x 256 B, rows padded to 272 B so the fragment loads are conflict-free), their scales and sums go through a
// two-stage cp.async ring, one super-block per stage.  This is the legacy tensor path (mma.sync): M = 16 rows per warp
// and K = 32 per instruction match the quant format's sub-block; the tcgen05 form (128-row tiles, TMEM accumulators)
// would need the codes unpacked to shared memory first and is not built.
#include <cuda_pipeline.h>

#include "common.cuh"
#include "kernels.h"

namespace ob {

namespace {

constexpr int MM_WARPS = 4, MM_ROWS = 16 * MM_WARPS;
constexpr uint32_t MM_B_ROW = 272;

// shared-memory stage of one super-block: weight blocks of 64 rows | activations of TOK tokens | per-16 sums | token scales |
// per-32 sums | (Q6_K) the rows' d
template <uint32_t TYPE, int NT>
struct MmStage {
    static constexpr uint32_t TOK = 8 * NT;
    static constexpr uint32_t BLK = TYPE == TYPE_Q4_K ? 144 : 208;
    static constexpr uint32_t A = 0, B = MM_ROWS * BLK, S16 = B + TOK * MM_B_ROW, AD = S16 + TOK * 32, BS = AD + TOK * 4, DW = BS + TOK * 16;
    static constexpr uint32_t BYTES = DW + MM_ROWS * 4;
};

__device__ __forceinline__ void mma_u8s8_k32(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_s8s8_k16(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(b0));
}
__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint4 lds_u128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ void cp16(uint32_t saddr, const void *g) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(saddr), "l"(g) : "memory");
}
__device__ __forceinline__ int dp2a_lo_su(uint32_t a, uint32_t b, int c) {  // c + a.lo16 * b.byte0 + a.hi16 * b.byte1 (a signed, b unsigned)
    int d;
    asm("dp2a.lo.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int dp2a_hi_su(uint32_t a, uint32_t b, int c) {  // c + a.lo16 * b.byte2 + a.hi16 * b.byte3
    int d;
    asm("dp2a.hi.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// GEMM: the prefill association (Q4_K: two passes); otherwise every (row, token) is the single-token product.
// NT: n-tiles of 8 tokens per CTA.
// STAGES: depth of the cp.async ring, one super-block per stage: four for the 16-token tile, three for 32 tokens, two for the
// 64-token tile whose stages are 30 KB.  (Measured: the depth does not change the time of any shape -- 4096 x 14336 at 16 tokens
// takes 60 us with two stages and with four; the kernel is bound by its instruction count per super-block, about 600 per warp at
// the 16-token tile, not by the arrival of the stages.)
template <uint32_t TYPE, bool GEMM, int NT, int STAGES>
__global__ void __launch_bounds__(MM_WARPS * 32) gemm_mma_kernel(GemvArgs a) {
    using S = MmStage<TYPE, NT>;
    constexpr uint32_t TOK = S::TOK, BLK = S::BLK;
    extern __shared__ __align__(16) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gid = lane >> 2, tig = lane & 3;
    const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(smem);

    // which segment and which 64-row tile of it
    uint32_t tile = blockIdx.x;
    int si = 0;
    while (si + 1 < a.n_seg && tile >= (a.seg[si].w.out_dim + MM_ROWS - 1) / MM_ROWS) {
        tile -= (a.seg[si].w.out_dim + MM_ROWS - 1) / MM_ROWS;
        ++si;
    }
    const GemvSegment &seg = a.seg[si];
    const uint32_t out_dim = seg.w.out_dim, nb = seg.w.nb;
    const uint32_t row0 = tile * MM_ROWS, tok0 = blockIdx.y * TOK;
    const uint32_t n_tok = min(TOK, a.n_tokens - tok0);

    // activation rows of tokens past the end stay zero in every stage
    for (uint32_t i = tid; i < STAGES * S::BYTES / 16; i += MM_WARPS * 32) *reinterpret_cast<uint4 *>(smem + i * 16) = make_uint4(0, 0, 0, 0);
    // the per-block scales of the tile's tokens (and, Q6_K, of its rows) for the whole row, once: loaded inside the loop they
    // would be a synchronous trip to memory per super-block
    float *ad_all = reinterpret_cast<float *>(smem + STAGES * S::BYTES);  // [TOK][nb]
    float *dw_all = ad_all + TOK * nb;                                    // Q6_K: [MM_ROWS][nb]
    for (uint32_t i = tid; i < TOK * nb; i += MM_WARPS * 32) {
        const uint32_t t = i / nb, b = i % nb;
        ad_all[i] = t < n_tok ? a.act.d[(uint64_t)(tok0 + t) * (a.act.dim_cap / 256) + b] : 0.0f;
    }
    if (TYPE == TYPE_Q6_K)
        for (uint32_t i = tid; i < MM_ROWS * nb; i += MM_WARPS * 32) {
            const uint32_t r = i / nb, b = i % nb, row = min(row0 + r, out_dim - 1);
            dw_all[i] = f16_bits_to_f32(*reinterpret_cast<const uint16_t *>(seg.w.data + (uint64_t)row * seg.w.row_stride + seg.w.d_off + 2 * b));
        }
    __syncthreads();

    auto stage_block = [&](uint32_t b, int st, bool codes) {
        const uint32_t base = sbase + st * S::BYTES;
        if (codes) {
            constexpr uint32_t CPR = BLK / 16;  // 16-byte chunks per row block
            for (uint32_t c = tid; c < MM_ROWS * CPR; c += MM_WARPS * 32) {
                const uint32_t r = c / CPR, j = c % CPR, row = min(row0 + r, out_dim - 1);
                cp16(base + S::A + r * BLK + j * 16, seg.w.data + (uint64_t)row * seg.w.row_stride + (uint64_t)b * BLK + j * 16);
            }
            for (uint32_t c = tid; c < n_tok * 16; c += MM_WARPS * 32) {  // activations: tokens x 256 int8
                const uint32_t t = c >> 4, j = c & 15;
                cp16(base + S::B + t * MM_B_ROW + j * 16, a.act.q + (uint64_t)(tok0 + t) * a.act.dim_cap + (uint64_t)b * 256 + j * 16);
            }
        } else {
            for (uint32_t r = tid; r < MM_ROWS; r += MM_WARPS * 32) {  // only the 16-byte headers: d, dmin, scales and mins
                const uint32_t row = min(row0 + r, out_dim - 1);
                cp16(base + S::A + r * BLK, seg.w.data + (uint64_t)row * seg.w.row_stride + (uint64_t)b * BLK);
            }
        }
        if (TYPE == TYPE_Q4_K) {
            for (uint32_t c = tid; c < n_tok * 2; c += MM_WARPS * 32) {  // per-16 sums: 16 int16 per token
                const uint32_t t = c >> 1, j = c & 1;
                cp16(base + S::S16 + t * 32 + j * 16, a.act.sums + (uint64_t)(tok0 + t) * (a.act.dim_cap / 16) + (uint64_t)b * 16 + j * 8);
            }
        }
    };

    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.0f;

    constexpr int N_PASS = GEMM && TYPE == TYPE_Q4_K ? 2 : 1;
    for (int pass = 0; pass < N_PASS; ++pass) {
        const bool min_pass = N_PASS == 2 && pass == 0;  // pass 1 of the Q4_K prefill order: the min terms of all super-blocks
        for (int p = 0; p < STAGES - 1; ++p) {
            if ((uint32_t)p < nb) stage_block((uint32_t)p, p, !min_pass);
            __pipeline_commit();
        }
        for (uint32_t b = 0; b < nb; ++b) {
            const int st = (int)(b % STAGES);
            if (b + STAGES - 1 < nb) stage_block(b + STAGES - 1, (int)((b + STAGES - 1) % STAGES), !min_pass);  // the stage block b - 1 left
            __pipeline_commit();
            __pipeline_wait_prior(STAGES - 1);
            __syncthreads();  // block b has landed
            const uint32_t base = sbase + st * S::BYTES;
            if (TYPE == TYPE_Q4_K) {  // per-32 sums from the per-16 sums: token t, pair j
                for (uint32_t i = tid; i < TOK * 8; i += MM_WARPS * 32) {
                    const uint32_t w = lds_u32(base + S::S16 + i * 4);
                    reinterpret_cast<int16_t *>(smem + st * S::BYTES + S::BS)[i] = (int16_t)((int)(int16_t)(w & 0xffff) + (int)(int16_t)(w >> 16));
                }
                __syncthreads();
            }

            // this warp's rows gid and gid + 8 of the tile
            const uint32_t arow[2] = {base + S::A + (warp * 16 + gid) * BLK, base + S::A + (warp * 16 + gid + 8) * BLK};
            int isum[NT][4];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) isum[nt][0] = isum[nt][1] = isum[nt][2] = isum[nt][3] = 0;

            if constexpr (TYPE == TYPE_Q4_K) {
                uint32_t scl[2], sch[2], ml[2], mh[2];
                float dd[2], dmin[2];
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    const uint4 hd = lds_u128(arow[r]);
                    dd[r] = f16_bits_to_f32(hd.x & 0xffffu);
                    dmin[r] = f16_bits_to_f32(hd.x >> 16);
                    scl[r] = hd.y & 0x3f3f3f3fu;  // the eight 6-bit scales and mins (engine/quant.rs:653-662) as bytes of four words
                    ml[r] = hd.z & 0x3f3f3f3fu;
                    sch[r] = (hd.w & 0x0f0f0f0fu) | ((hd.y >> 2) & 0x30303030u);
                    mh[r] = ((hd.w >> 4) & 0x0f0f0f0fu) | ((hd.z >> 2) & 0x30303030u);
                }
                if (!min_pass) {
#pragma unroll
                    for (int g = 0; g < 4; ++g) {  // sub-blocks 2g (low nibbles) and 2g + 1 (high nibbles) of bytes 32g .. 32g + 31
                        uint32_t w[2][2];
#pragma unroll
                        for (int r = 0; r < 2; ++r) {
                            w[r][0] = lds_u32(arow[r] + 16 + 32 * g + 4 * tig);
                            w[r][1] = lds_u32(arow[r] + 16 + 32 * g + 16 + 4 * tig);
                        }
                        const uint32_t M = 0x0f0f0f0fu;
                        const uint32_t lo0 = w[0][0] & M, lo1 = w[1][0] & M, lo2 = w[0][1] & M, lo3 = w[1][1] & M;
                        const uint32_t hi0 = (w[0][0] >> 4) & M, hi1 = (w[1][0] >> 4) & M, hi2 = (w[0][1] >> 4) & M, hi3 = (w[1][1] >> 4) & M;
                        const uint32_t scw0 = g < 2 ? scl[0] : sch[0], scw1 = g < 2 ? scl[1] : sch[1];
                        const int sa0 = (int)((scw0 >> (16 * (g & 1))) & 0xff), sb0 = (int)((scw0 >> (16 * (g & 1) + 8)) & 0xff);
                        const int sa1 = (int)((scw1 >> (16 * (g & 1))) & 0xff), sb1 = (int)((scw1 >> (16 * (g & 1) + 8)) & 0xff);
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt) {
                            const uint32_t xb = base + S::B + (8 * nt + gid) * MM_B_ROW + 64 * g + 4 * tig;
                            int c[4] = {0, 0, 0, 0};
                            mma_u8s8_k32(c, lo0, lo1, lo2, lo3, lds_u32(xb), lds_u32(xb + 16));
                            isum[nt][0] += sa0 * c[0];
                            isum[nt][1] += sa0 * c[1];
                            isum[nt][2] += sa1 * c[2];
                            isum[nt][3] += sa1 * c[3];
                            int e[4] = {0, 0, 0, 0};
                            mma_u8s8_k32(e, hi0, hi1, hi2, hi3, lds_u32(xb + 32), lds_u32(xb + 48));
                            isum[nt][0] += sb0 * e[0];
                            isum[nt][1] += sb0 * e[1];
                            isum[nt][2] += sb1 * e[2];
                            isum[nt][3] += sb1 * e[3];
                        }
                    }
                }
                // fp32 terms of this super-block for elements (row gid | gid + 8, token 8 nt + 2 tig | + 1)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
                    for (int k = 0; k < 2; ++k) {
                        const uint32_t t = 8 * nt + 2 * tig + k;
                        const float ad = ad_all[t * nb + b];
                        int imin[2] = {0, 0};
                        if (!GEMM || min_pass) {
                            const uint4 bsv = lds_u128(base + S::BS + t * 16);
#pragma unroll
                            for (int r = 0; r < 2; ++r) {
                                int v = dp2a_lo_su(bsv.x, ml[r], 0);
                                v = dp2a_hi_su(bsv.y, ml[r], v);
                                v = dp2a_lo_su(bsv.z, mh[r], v);
                                imin[r] = dp2a_hi_su(bsv.w, mh[r], v);
                            }
                        }
#pragma unroll
                        for (int r = 0; r < 2; ++r) {
                            float &o = acc[nt][2 * r + k];
                            if (!GEMM) {
                                o = __fadd_rn(o, __fmul_rn(ad, __fsub_rn(__fmul_rn(dd[r], (float)isum[nt][2 * r + k]), __fmul_rn(dmin[r], (float)imin[r]))));
                            } else if (min_pass) {
                                o = __fsub_rn(o, __fmul_rn(__fmul_rn(ad, dmin[r]), (float)imin[r]));
                            } else {
                                o = __fadd_rn(o, __fmul_rn(ad, __fmul_rn(dd[r], (float)isum[nt][2 * r + k])));
                            }
                        }
                    }
                }
            } else {  // Q6_K: block = [ql 128 | qh 64 | signed scales 16]; sixteen sub-blocks of 16 elements
                uint32_t scw[2][4];
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    const uint4 v = lds_u128(arow[r] + 192);
                    scw[r][0] = v.x;
                    scw[r][1] = v.y;
                    scw[r][2] = v.z;
                    scw[r][3] = v.w;
                }
#pragma unroll
                for (int h = 0; h < 2; ++h) {
#pragma unroll
                    for (int is = 0; is < 2; ++is) {
                        // codes l = 16 is + 4 tig .. + 3 of this half: ql bytes l (runs 0, 2) and 32 + l (runs 1, 3), qh bytes l
                        uint32_t v[2][4];
#pragma unroll
                        for (int r = 0; r < 2; ++r) {
                            const uint32_t qa = lds_u32(arow[r] + 64 * h + 16 * is + 4 * tig), qb = lds_u32(arow[r] + 64 * h + 32 + 16 * is + 4 * tig);
                            const uint32_t qh = lds_u32(arow[r] + 128 + 32 * h + 16 * is + 4 * tig);
                            v[r][0] = __vsub4((qa & 0x0f0f0f0fu) | ((qh << 4) & 0x30303030u), 0x20202020u);  // q - 32 as signed bytes
                            v[r][1] = __vsub4((qb & 0x0f0f0f0fu) | ((qh << 2) & 0x30303030u), 0x20202020u);
                            v[r][2] = __vsub4(((qa >> 4) & 0x0f0f0f0fu) | (qh & 0x30303030u), 0x20202020u);
                            v[r][3] = __vsub4(((qb >> 4) & 0x0f0f0f0fu) | ((qh >> 2) & 0x30303030u), 0x20202020u);
                        }
#pragma unroll
                        for (int run = 0; run < 4; ++run) {
                            const int sidx = 8 * h + 2 * run + is;  // scale of elements 128 h + 32 run + 16 is ..
                            const int s0 = (int)(int8_t)((scw[0][sidx >> 2] >> (8 * (sidx & 3))) & 0xff), s1 = (int)(int8_t)((scw[1][sidx >> 2] >> (8 * (sidx & 3))) & 0xff);
#pragma unroll
                            for (int nt = 0; nt < NT; ++nt) {
                                int c[4] = {0, 0, 0, 0};
                                mma_s8s8_k16(c, v[0][run], v[1][run], lds_u32(base + S::B + (8 * nt + gid) * MM_B_ROW + 128 * h + 32 * run + 16 * is + 4 * tig));
                                isum[nt][0] += s0 * c[0];
                                isum[nt][1] += s0 * c[1];
                                isum[nt][2] += s1 * c[2];
                                isum[nt][3] += s1 * c[3];
                            }
                        }
                    }
                }
                const float dw[2] = {dw_all[(warp * 16 + gid) * nb + b], dw_all[(warp * 16 + gid + 8) * nb + b]};
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int k = 0; k < 2; ++k) {
                        const float ad = ad_all[(8 * nt + 2 * tig + k) * nb + b];
#pragma unroll
                        for (int r = 0; r < 2; ++r) {
                            const float fi = (float)isum[nt][2 * r + k];
                            const float term = GEMM ? __fmul_rn(ad, __fmul_rn(dw[r], fi)) : __fmul_rn(__fmul_rn(ad, dw[r]), fi);
                            acc[nt][2 * r + k] = __fadd_rn(acc[nt][2 * r + k], term);
                        }
                    }
            }
            __syncthreads();  // everyone is done with this stage before it is refilled
        }
        __pipeline_wait_prior(0);
    }

    // ---- store
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t row = row0 + warp * 16 + gid + 8 * (i >> 1), t = 8 * nt + 2 * tig + (i & 1);
            if (row < out_dim && t < n_tok) {
                const uint64_t o = (uint64_t)(tok0 + t) * seg.y_stride + row;
                float v = acc[nt][i];
                if (seg.epilogue == EPI_ADD_RESIDUAL) v = __fadd_rn(seg.residual[o], v);
                seg.y[o] = v;
            }
        }
}

template <uint32_t TYPE, bool GEMM, int NT>
void launch_mma_instance(const GemvArgs &a, uint32_t tiles, cudaStream_t st) {
    constexpr int STAGES = NT == 8 ? 2 : NT == 4 ? 3 : 4;
    static PerDeviceOnce once;  // one per instantiation
    if (once.run([] { return cudaFuncSetAttribute(gemm_mma_kernel<TYPE, GEMM, NT, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); }) != cudaSuccess) return;
    const uint32_t nb = a.seg[0].w.nb;
    const size_t smem = (size_t)STAGES * MmStage<TYPE, NT>::BYTES + (size_t)8 * NT * nb * 4 + (TYPE == TYPE_Q6_K ? (size_t)MM_ROWS * nb * 4 : 0);
    const dim3 grid(tiles, (a.n_tokens + 8 * NT - 1) / (8 * NT));
    gemm_mma_kernel<TYPE, GEMM, NT, STAGES><<<grid, MM_WARPS * 32, smem, st>>>(a);
}

template <uint32_t TYPE, bool GEMM>
void launch_mma_nt(const GemvArgs &a, uint32_t tiles, int nt, cudaStream_t st) {
    if (nt == 8) launch_mma_instance<TYPE, GEMM, 8>(a, tiles, st);
    else if (nt == 4) launch_mma_instance<TYPE, GEMM, 4>(a, tiles, st);
    else launch_mma_instance<TYPE, GEMM, 2>(a, tiles, st);
}

}  // namespace

bool gemm_mma_supported(const GemvArgs &a) {
    if (a.n_seg < 1 || a.n_tokens < 9 || a.isum_out) return false;
    const uint32_t type = a.seg[0].w.type;
    if (type != TYPE_Q4_K && type != TYPE_Q6_K) return false;
    for (int s = 0; s < a.n_seg; ++s)
        if (a.seg[s].w.type != type || a.seg[s].w.in_dim != a.seg[0].w.in_dim) return false;
    return true;
}

void launch_gemm_mma(const GemvArgs &a, int sm_count, cudaStream_t st) {
    uint32_t tiles = 0;
    for (int s = 0; s < a.n_seg; ++s) tiles += (a.seg[s].w.out_dim + MM_ROWS - 1) / MM_ROWS;
    // 64 tokens per CTA reuse every weight fragment eight times; fewer when that would leave SMs without a CTA
    int nt = 8;
    while (nt > 2 && (a.n_tokens <= 4u * nt || tiles * ((a.n_tokens + 8 * nt - 1) / (8 * nt)) < 2u * (uint32_t)sm_count)) nt /= 2;
    const bool q4 = a.seg[0].w.type == TYPE_Q4_K;
    if (q4) {
        if (a.gemm_order) launch_mma_nt<TYPE_Q4_K, true>(a, tiles, nt, st);
        else launch_mma_nt<TYPE_Q4_K, false>(a, tiles, nt, st);
    } else {
        if (a.gemm_order) launch_mma_nt<TYPE_Q6_K, true>(a, tiles, nt, st);
        else launch_mma_nt<TYPE_Q6_K, false>(a, tiles, nt, st);
    }
}

}  // namespace ob
