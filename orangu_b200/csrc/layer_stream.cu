// The single-token products of a whole decoder layer in one persistent launch.
//
// Batch-1 decode reads every weight byte once; what keeps it below the HBM rate is not the products themselves but
// what lies between them: a kernel boundary per operator (drain, launch, ramp), and the RMSNorm whose exact
// left-to-right sum (seqsum.cuh) ran as a one-CTA kernel twice per layer while the other SMs idled.  Here one
// CTA per SM stays resident and walks a list of "phases" -- the products between two attention kernels:
//
//     attention-output + residual | norm + gate/up + SwiGLU (+ int8 image) | down + residual | norm + q/k/v + RoPE + KV append
//
// separated by grid barriers (one atomic counter, bounded spin).  Consequences:
//   * the RMSNorm is the prologue of the phase that consumes it: after the barrier every CTA loads the 16 KB row,
//     computes the exact scale itself (same bits everywhere) and quantizes into its own shared memory -- no norm
//     kernel, no image round trip through global memory;
//   * every warp requests the first two units of the NEXT phase's weights before it arrives at the barrier, and the
//     rest of its share is prefetched into L2 while the norm runs, so the weight stream keeps going across operator
//     boundaries;
//   * a layer is two launches (this kernel and the attention kernel) instead of seven.
//
// The dot loop, the unit / group scheme, the fp32 association and the epilogues are those of stream_gemv.cu
// (engine/vecdot.rs:3152-3178 Q4_K, :3215-3241 Q6_K; ascending-block sums by one lane), so results are bit-identical.
//
// Everything a phase reads that an earlier phase of the same launch wrote (the residual row, the image, the SwiGLU
// outputs) is read with L2 loads (ld.global.cg): an SM's L1 may hold the line from before it was rewritten.
#include "seqsum.cuh"
#include "stream_common.cuh"

namespace ob {

namespace {

constexpr int LS_THREADS = 512, LS_WARPS = 16;
constexpr uint32_t LS_TAB_BYTES = 256;  // one segment table (3 x 16 words + pad)

// per-thread view of a phase in flight
struct LsState {
    uint32_t g_first, g_end;  // this warp's groups
    uint32_t ig, ic;          // next unit to request: group, chunk
    uint32_t gb1, gb2;        // first group of segments 1 and 2
};

__device__ __forceinline__ uint32_t ld_acquire_u32(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Segment table of phase `d` into shared memory at `tab`, group offsets into `st`.  Threads 0..2 write; callers synchronise.
template <int LP>
__device__ __forceinline__ void ls_put_table(const LsPhase &d, uint8_t *tab, LsState &st) {
    constexpr uint32_t PPU = 32 / LP;
    uint32_t pairs_of[3], first_of[4];
    first_of[0] = 0;
#pragma unroll
    for (int s = 0; s < 3; ++s) {
        pairs_of[s] = s >= d.a.n_seg ? 0u : (d.a.seg[s].w2.data ? d.a.seg[s].w.out_dim : (d.a.seg[s].w.out_dim + 1) / 2);
        first_of[s + 1] = first_of[s] + (pairs_of[s] + PPU - 1) / PPU;
    }
    st.gb1 = first_of[1];
    st.gb2 = first_of[2];
    const uint32_t G = first_of[3];
    const int t = threadIdx.x;
    if (t < 3 && t < d.a.n_seg) {
        const StreamSeg &g = d.a.seg[t];
        uint32_t *w = reinterpret_cast<uint32_t *>(tab) + t * SEG_WORDS;
        *reinterpret_cast<const uint8_t **>(w) = g.w.data;
        *reinterpret_cast<const uint8_t **>(w + 2) = g.w2.data;
        w[4] = (uint32_t)g.w.row_stride;
        w[5] = g.w.type;
        w[6] = g.w.out_dim;
        w[7] = pairs_of[t];
        w[8] = g.w.d_off;
        w[9] = (uint32_t)g.epilogue;
        *reinterpret_cast<float **>(w + 10) = g.y;
        w[12] = first_of[t];
    }
    const uint32_t warp = threadIdx.x >> 5, nw = d.nw;
    if (warp < nw) {
        const uint32_t n_warps = gridDim.x * nw, gw = blockIdx.x * nw + warp;
        st.g_first = (uint32_t)(((uint64_t)G * gw) / n_warps);
        st.g_end = (uint32_t)(((uint64_t)G * (gw + 1)) / n_warps);
    } else {
        st.g_first = st.g_end = 0;
    }
    st.ig = st.g_first;
    st.ic = 0;
}

// One unit (group g, chunk ch) of the weights into `slot`; tab: shared address of the phase's segment table.
template <int LP, bool Q6>
__device__ __forceinline__ void ls_issue(uint32_t slot, uint32_t g, uint32_t ch, uint32_t tab, const LsState &st, uint32_t nb) {
    constexpr uint32_t PPU = 32 / LP, BPC = LP / 2, HL = BPC;
    constexpr uint32_t PB4 = BPC * 144u, PB6 = BPC * 208u + ((BPC * 2u + 15u) & ~15u);
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t q = lane / HL, sub = lane % HL, cj = q >> 1, cr = q & 1;  // copy role: part q = (pair cj, row cr), chunks sub + HL * k
    const uint32_t e = tab + ((g >= st.gb1) + (g >= st.gb2)) * (SEG_WORDS * 4);
    const uint2 wa = lds64(e), wb = lds64(e + 8);
    const uint4 m = lds128(e + 16);  // row stride, type, out_dim, pairs
    const bool dual = (wb.x | wb.y) != 0;
    const uint32_t pair = min((g - lds32(e + 48)) * PPU + cj, m.w - 1);  // past the segment's last pair: fetch that pair again
    const uint32_t row_index = dual ? pair : min(2 * pair + cr, m.z - 1);
    const uint2 wp = dual && cr ? wb : wa;
    const uint8_t *row = reinterpret_cast<const uint8_t *>(((uint64_t)wp.y << 32) | wp.x) + (uint64_t)row_index * m.x;
    const uint32_t b0 = ch * BPC, nblk = min((uint32_t)BPC, nb - b0);
    if (!Q6 || m.y == TYPE_Q4_K) {
        const uint8_t *src = row + b0 * 144 + sub * 16;
        const uint32_t dst = slot + q * PB4 + sub * 16;
        if (nblk == BPC) {
#pragma unroll
            for (int k = 0; k < 9; ++k) cp_async16(dst + k * HL * 16, src + k * HL * 16);
        } else {
#pragma unroll
            for (int k = 0; k < 9; ++k)
                if (sub + HL * k < nblk * 9) cp_async16(dst + k * HL * 16, src + k * HL * 16);
        }
    } else {
        const uint8_t *src = row + b0 * 208 + sub * 16;
        const uint32_t dst = slot + q * PB6 + sub * 16;
        if (nblk == BPC) {
#pragma unroll
            for (int k = 0; k < 13; ++k) cp_async16(dst + k * HL * 16, src + k * HL * 16);
        } else {
#pragma unroll
            for (int k = 0; k < 13; ++k)
                if (sub + HL * k < nblk * 13) cp_async16(dst + k * HL * 16, src + k * HL * 16);
        }
        // the f16 d values of these blocks; b0 is 0 or a multiple of 8, so the source is 16-byte aligned
        if (sub < (nblk * 2 + 15) / 16) cp_async16(slot + q * PB6 + BPC * 208 + sub * 16, row + lds32(e + 32) + 2 * b0 + sub * 16);
    }
}

// The same unit as an L2 prefetch (no shared memory involved): each of the 2 * PPU row parts is one bulk request.
template <int LP, bool Q6>
__device__ __forceinline__ void ls_prefetch_l2(uint32_t g, uint32_t ch, uint32_t tab, const LsState &st, uint32_t nb) {
    constexpr uint32_t PPU = 32 / LP, BPC = LP / 2;
    const uint32_t lane = threadIdx.x & 31;
    if (lane >= 2 * PPU) return;
    const uint32_t cj = lane >> 1, cr = lane & 1;
    const uint32_t e = tab + ((g >= st.gb1) + (g >= st.gb2)) * (SEG_WORDS * 4);
    const uint2 wa = lds64(e), wb = lds64(e + 8);
    const uint4 m = lds128(e + 16);
    const bool dual = (wb.x | wb.y) != 0;
    const uint32_t pair = min((g - lds32(e + 48)) * PPU + cj, m.w - 1);
    const uint32_t row_index = dual ? pair : min(2 * pair + cr, m.z - 1);
    const uint2 wp = dual && cr ? wb : wa;
    const uint8_t *row = reinterpret_cast<const uint8_t *>(((uint64_t)wp.y << 32) | wp.x) + (uint64_t)row_index * m.x;
    const uint32_t b0 = ch * BPC, nblk = min((uint32_t)BPC, nb - b0);
    const uint32_t bb = (!Q6 || m.y == TYPE_Q4_K) ? 144u : 208u;
    const uint8_t *src = row + b0 * bb;
    const uint32_t bytes = nblk * bb;  // a multiple of 16; rows are 16-byte aligned
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}

__device__ __forceinline__ void ls_advance(uint32_t &g, uint32_t &c, uint32_t nchunk) {
    if (++c == nchunk) {
        c = 0;
        ++g;
    }
}

// Before the barrier: table of the next phase, the first two units of its weights into the (now idle) ring, and as many
// further units as the phase asks for into L2.
template <int LP, bool Q6>
__device__ __noinline__ LsState ls_begin(const LsPhase &d, uint8_t *smem, uint32_t sbase, uint32_t off_tab, uint32_t off_ring) {
    constexpr uint32_t PPU = 32 / LP, BPC = LP / 2;
    constexpr uint32_t PB4 = BPC * 144u, PB6 = BPC * 208u + ((BPC * 2u + 15u) & ~15u);
    constexpr uint32_t SLOT = 2u * PPU * (Q6 ? PB6 : PB4);
    LsState st;
    ls_put_table<LP>(d, smem + off_tab, st);
    __syncthreads();
    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t tab = sbase + off_tab;
    const uint32_t slots = sbase + off_ring + warp * 2 * SLOT;
    const uint32_t nb = d.a.in_dim / 256, nchunk = (nb + BPC - 1) / BPC;
    if (st.ig < st.g_end) ls_issue<LP, Q6>(slots, st.ig, st.ic, tab, st, nb);
    __pipeline_commit();
    ls_advance(st.ig, st.ic, nchunk);
    if (st.ig < st.g_end) ls_issue<LP, Q6>(slots + SLOT, st.ig, st.ic, tab, st, nb);
    __pipeline_commit();
    ls_advance(st.ig, st.ic, nchunk);
    uint32_t pg = st.ig, pc = st.ic;
    for (uint32_t k = 0; k < d.l2_ahead && pg < st.g_end; ++k) {
        ls_prefetch_l2<LP, Q6>(pg, pc, tab, st, nb);
        ls_advance(pg, pc, nchunk);
    }
    return st;
}

// After the barrier: the phase's activation image into shared memory.
__device__ __noinline__ void ls_prologue(const LsPhase &d, uint8_t *smem, uint32_t off_img, uint32_t off_norm) {
    const StreamArgs &a = d.a;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t nb = a.in_dim / 256;
    const ActImage im = act_image(nb);
    uint8_t *img = smem + off_img;
    if (a.prologue == SG_PRO_READY) {  // a producer left the image in global memory
        const uint32_t n16 = im.bytes / 16;
        constexpr uint32_t CB = 3;
        for (uint32_t c0 = threadIdx.x; c0 < n16; c0 += CB * LS_THREADS) {
            uint4 v[CB];
#pragma unroll
            for (uint32_t k = 0; k < CB; ++k)
                if (c0 + k * LS_THREADS < n16) v[k] = __ldcg(reinterpret_cast<const uint4 *>(a.ready) + c0 + k * LS_THREADS);
#pragma unroll
            for (uint32_t k = 0; k < CB; ++k)
                if (c0 + k * LS_THREADS < n16) *reinterpret_cast<uint4 *>(img + (c0 + k * LS_THREADS) * 16) = v[k];
        }
    } else {  // SG_PRO_RMSNORM: exact scale of the row (engine/tensor.rs:743-749), then (x * scale) * w quantized per 256
        float *srow = reinterpret_cast<float *>(smem + off_norm);
        const uint32_t dim = a.in_dim;
        SeqSumWorkspace<LS_THREADS> &ws = *reinterpret_cast<SeqSumWorkspace<LS_THREADS> *>(smem + off_norm + (((dim + dim / 16 + 16) * 4 + 15) & ~15u));
        for (uint32_t i = threadIdx.x * 4; i < dim; i += LS_THREADS * 4) {
            const float4 v = __ldcg(reinterpret_cast<const float4 *>(a.x + i));
            float *p = srow + i + (i >> 4);
            p[0] = v.x;
            p[1] = v.y;
            p[2] = v.z;
            p[3] = v.w;
        }
        __syncthreads();
        const float t = cta_sequential_sum<LS_THREADS>([&](uint32_t i) { const float v = srow[i + (i >> 4)]; return __fmul_rn(v, v); }, dim, ws);
        const float scale = __fdiv_rn(1.0f, sqrtf(__fadd_rn(__fdiv_rn(t, (float)dim), a.eps)));
        for (uint32_t b = warp; b < nb; b += LS_WARPS) {
            const uint32_t e0 = b * 256 + lane * 8;
            const float *sv = srow + e0 + (e0 >> 4);
            const float4 w0 = __ldg(reinterpret_cast<const float4 *>(a.norm_w + e0)), w1 = __ldg(reinterpret_cast<const float4 *>(a.norm_w + e0 + 4));
            const float w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = __fmul_rn(__fmul_rn(sv[i], scale), w[i]);  // tensor.rs:747
            quantize_block(v, b, img, im);
        }
    }
    __syncthreads();
}

struct LsOffsets {  // shared-memory offsets the loop needs
    uint32_t tab, img, terms, ring;
};

// Main loop and epilogues of one phase.
template <int LP, bool Q6>
__device__ __noinline__ void ls_loop(const LsPhase &d, uint32_t sbase, LsOffsets o, LsState st) {
    constexpr int PPU = 32 / LP, BPC = LP / 2;
    constexpr uint32_t PB4 = BPC * 144u, PB6 = BPC * 208u + ((BPC * 2u + 15u) & ~15u);
    constexpr uint32_t SLOT = 2u * PPU * (Q6 ? PB6 : PB4);
    const StreamArgs &a = d.a;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t nb = a.in_dim / 256, nchunk = (nb + BPC - 1) / BPC;
    const uint32_t tab = sbase + o.tab;
    const uint32_t terms = sbase + o.terms + warp * 128;
    const uint32_t slots = sbase + o.ring + warp * 2 * SLOT;
    const ActImage im = act_image(nb);
    const uint32_t s_act = sbase + o.img, s_d = s_act + im.off_d, s_bsum = s_act + im.off_bsum, s_sum16 = s_act + im.off_sum16;

    // ---- main loop ------------------------------------------------------------------------------------------------
    const uint32_t pj = lane / LP, bl = (lane % LP) >> 1, half = lane & 1;  // dot role: pair, block of the chunk, half of the block
    uint32_t cg = st.g_first, cc = 0;
    float tot = 0.0f;  // lanes 2j, 2j+1: rows A, B of the group's pair j, running over the chunks of the row
    uint32_t par = 0;
    while (cg < st.g_end) {
        const uint32_t slot = slots + par * SLOT;
        const uint32_t e = tab + ((cg >= st.gb1) + (cg >= st.gb2)) * (SEG_WORDS * 4);
        const uint32_t b0 = cc * BPC, nblk = min((uint32_t)BPC, nb - b0);
        __pipeline_wait_prior(1);
        __syncwarp();
        {
            const uint32_t gb = min(b0 + bl, nb - 1);  // lanes past the row's end recompute its last block; nobody reads their terms
            const uint32_t xa = s_act + gb * ACT_BLOCK_STRIDE;
            const float ad = __uint_as_float(lds32(s_d + gb * 4));
            int isum[2], imin[2] = {0, 0};
            float term;  // lane `half` ends up with the term of row `half` of the pair
            if (!Q6 || lds32(e + 20) == TYPE_Q4_K) {
                const uint32_t pA = slot + (2 * pj) * PB4 + bl * 144;
                uint32_t dd[2];
                dot_half_q4k(pA, pA + PB4, half, xa, s_bsum + gb * 16, isum, imin, dd);
#pragma unroll
                for (int r = 0; r < 2; ++r) {  // the two lanes of the cell add their halves: exact integers, any order
                    isum[r] += __shfl_xor_sync(0xffffffffu, isum[r], 1);
                    imin[r] += __shfl_xor_sync(0xffffffffu, imin[r], 1);
                }
                const int is = half ? isum[1] : isum[0], imn = half ? imin[1] : imin[0];
                const uint32_t dw = half ? dd[1] : dd[0];
                const float dq = f16_bits_to_f32(dw & 0xffffu), dmin = f16_bits_to_f32(dw >> 16);
                term = __fmul_rn(ad, __fsub_rn(__fmul_rn(dq, (float)is), __fmul_rn(dmin, (float)imn)));
            } else {
                const uint32_t pA = slot + (2 * pj) * PB6, pB = pA + PB6;
                dot_half_q6k(pA + bl * 208, pB + bl * 208, half, xa, s_sum16 + gb * 32, isum);
                isum[0] += __shfl_xor_sync(0xffffffffu, isum[0], 1);
                isum[1] += __shfl_xor_sync(0xffffffffu, isum[1], 1);
                const float dsup = f16_bits_to_f32(lds16((half ? pB : pA) + BPC * 208 + 2 * bl));
                term = __fmul_rn(__fmul_rn(ad, dsup), (float)(half ? isum[1] : isum[0]));
            }
            sts32(terms + ((2 * pj + half) * BPC + bl) * 4, term);
        }
        __syncwarp();
        // ordered sum: lane s < 2 * PPU continues the running total of (pair s / 2, row s % 2) over this chunk's blocks, in order
        if (cc == 0) tot = 0.0f;
        if (lane < 2 * PPU) {
            const uint32_t tp = terms + lane * BPC * 4;
            if constexpr (BPC >= 4) {
                if (nblk == BPC) {
#pragma unroll
                    for (int b = 0; b < BPC; b += 4) {
                        const uint4 v = lds128(tp + b * 4);
                        tot = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(tot, __uint_as_float(v.x)), __uint_as_float(v.y)), __uint_as_float(v.z)), __uint_as_float(v.w));
                    }
                } else {
#pragma unroll
                    for (int b = 0; b < BPC; b += 4) {
                        if (b < (int)nblk) {
                            const uint4 v = lds128(tp + b * 4);
                            tot = __fadd_rn(tot, __uint_as_float(v.x));
                            if (b + 1 < (int)nblk) tot = __fadd_rn(tot, __uint_as_float(v.y));
                            if (b + 2 < (int)nblk) tot = __fadd_rn(tot, __uint_as_float(v.z));
                            if (b + 3 < (int)nblk) tot = __fadd_rn(tot, __uint_as_float(v.w));
                        }
                    }
                }
            } else if constexpr (BPC == 2) {
                const uint2 v = lds64(tp);
                tot = __fadd_rn(tot, __uint_as_float(v.x));
                if (nblk > 1) tot = __fadd_rn(tot, __uint_as_float(v.y));
            } else {
                tot = __fadd_rn(tot, __uint_as_float(lds32(tp)));
            }
        }
        __syncwarp();
        // refill the slot just consumed
        if (st.ig < st.g_end) ls_issue<LP, Q6>(slot, st.ig, st.ic, tab, st, nb);
        __pipeline_commit();
        ls_advance(st.ig, st.ic, nchunk);
        const bool row_done = cc + 1 == nchunk;
        const uint32_t g_done = cg;
        ls_advance(cg, cc, nchunk);
        par ^= 1;
        if (!row_done) continue;

        // ---- epilogue of the finished pairs: lane 2j holds row A's total, lane 2j+1 row B's --------------------------
        const float tB = __shfl_down_sync(0xffffffffu, tot, 1);
        const uint4 m = lds128(e + 16);  // row stride, type, out_dim, pairs
        const uint32_t pair = (g_done - lds32(e + 48)) * PPU + (lane >> 1);
        if ((lane & 1) || lane >= 2 * PPU || pair >= m.w) continue;
        const float tA = tot;
        const uint2 wb = lds64(e + 8), yp = lds64(e + 40);
        float *y = reinterpret_cast<float *>(((uint64_t)yp.y << 32) | yp.x);
        const int epilogue = (int)lds32(e + 36);
        const bool hasB = (wb.x | wb.y) != 0 || 2 * pair + 1 < m.z;
        switch (epilogue) {
        case SG_EP_STORE:
            y[2 * pair] = tA;
            if (hasB) y[2 * pair + 1] = tB;
            break;
        case SG_EP_RESIDUAL:  // the residual row was rewritten earlier in this launch: read it from L2
            y[2 * pair] = __fadd_rn(__ldcg(a.residual + 2 * pair), tA);
            if (hasB) y[2 * pair + 1] = __fadd_rn(__ldcg(a.residual + 2 * pair + 1), tB);
            break;
        case SG_EP_SWIGLU:
            y[pair] = silu_mul_exact(tA, tB);
            break;
        case SG_EP_XCHG:
            break;  // tensor-parallel partials do not take this kernel
        default: {  // q, k, v rows of the token: rotate (q, k) and append (k, v) to the page as f16
            const uint32_t row = 2 * pair, hd = a.head_dim, head = row / hd, idx = (row % hd) / 2;
            const uint32_t pos = *a.position;
            float oa = tA, ob_ = tB;
            if (epilogue != SG_EP_V && 2 * idx < a.rope_dim) {
                const float2 sc = reinterpret_cast<const float2 *>(a.rope_table)[(uint64_t)pos * (a.rope_dim / 2) + idx];  // (sin, cos)
                oa = __fsub_rn(__fmul_rn(tA, sc.y), __fmul_rn(tB, sc.x));
                ob_ = __fadd_rn(__fmul_rn(tA, sc.x), __fmul_rn(tB, sc.y));
            }
            if (epilogue == SG_EP_ROPE_Q) {
                y[row] = oa;
                y[row + 1] = ob_;
            } else {
                const int32_t page = (*a.page_table)[pos / KV_PAGE];
                const uint64_t o = (((uint64_t)page * a.n_head_kv + head) * KV_PAGE + pos % KV_PAGE) * hd + (row % hd);
                __half *pool = epilogue == SG_EP_ROPE_K ? a.k_pool : a.v_pool;
                *reinterpret_cast<__half2 *>(pool + o) = __floats2half2_rn(oa, ob_);
            }
            break;
        }
        }
    }
    __pipeline_wait_prior(0);

    // ---- SwiGLU outputs as the next product's int8 input: the warp that completes a block of 256 quantizes it ---------
    if (a.out_image) {
        constexpr uint32_t UPPU = PPU;
        const uint32_t pairs = a.seg[0].w2.data ? a.seg[0].w.out_dim : (a.seg[0].w.out_dim + 1) / 2;
        const uint32_t p0 = min(st.g_first * UPPU, pairs), p1 = min(st.g_end * UPPU, pairs);
        __syncwarp();
        if (p1 > p0) {
            uint32_t done_blocks = 0;  // bit i: block p0 / 256 + i is complete and ours to quantize
            if (lane == 0) {
                __threadfence();
                for (uint32_t b = p0 / 256; b <= (p1 - 1) / 256; ++b) {
                    const uint32_t cnt = min(p1, (b + 1) * 256) - max(p0, b * 256);
                    if (atomicAdd(&a.out_counters[b], cnt) + cnt == 256) {
                        done_blocks |= 1u << (b - p0 / 256);
                        a.out_counters[b] = 0;
                    }
                }
                if (done_blocks) __threadfence();
            }
            done_blocks = __shfl_sync(0xffffffffu, done_blocks, 0);
            while (done_blocks) {
                const uint32_t b = p0 / 256 + (uint32_t)(__ffs((int)done_blocks) - 1);
                done_blocks &= done_blocks - 1;
                quantize_image(a.seg[0].y, nullptr, 1.0f, pairs / 256, a.out_image, b, pairs / 256);  // stride = block count: block b only
            }
        }
    }
}

#define LS_FOR_SHAPE(d, CALL)                                   \
    do {                                                        \
        if ((d).q6) {                                           \
            switch ((d).lp) {                                   \
            case 2: CALL(2, true); break;                       \
            case 4: CALL(4, true); break;                       \
            case 8: CALL(8, true); break;                       \
            case 16: CALL(16, true); break;                     \
            default: CALL(32, true); break;                     \
            }                                                   \
        } else {                                                \
            switch ((d).lp) {                                   \
            case 2: CALL(2, false); break;                      \
            case 4: CALL(4, false); break;                      \
            case 8: CALL(8, false); break;                      \
            case 16: CALL(16, false); break;                    \
            default: CALL(32, false); break;                    \
            }                                                   \
        }                                                       \
    } while (0)

// phases[0 .. n_phases): run in order by every CTA, a grid barrier between two of them.  barrier: one word, zero at launch.
// status: set to 1 when a barrier wait ran out of time (a CTA missing: the kernel then returns instead of spinning on).
__global__ void __launch_bounds__(LS_THREADS, 1)
layer_stream_kernel(const LsPhase *__restrict__ phases, uint32_t n_phases, LsLayout L, uint32_t *barrier, uint32_t *status, uint32_t timeout_ms, bool wait_dependency) {
    extern __shared__ __align__(16) uint8_t smem[];
    const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(smem);
    LsPhase *desc = reinterpret_cast<LsPhase *>(smem + L.off_desc);
    volatile uint32_t *ctrl = reinterpret_cast<volatile uint32_t *>(smem + L.off_ctrl);
    constexpr uint32_t DESC16 = sizeof(LsPhase) / 16;
    static_assert(sizeof(LsPhase) % 16 == 0, "phase descriptors are copied in 16-byte pieces");

    auto fetch_desc = [&](uint32_t p) {  // descriptors are written at model creation: never stale
        if (threadIdx.x < DESC16) reinterpret_cast<uint4 *>(desc + (p & 1))[threadIdx.x] = __ldg(reinterpret_cast<const uint4 *>(phases + p) + threadIdx.x);
    };
    fetch_desc(0);
    if (threadIdx.x == 0) ctrl[0] = 0;
    __syncthreads();

    LsState st;
#define LS_BEGIN(LP_, Q6_) st = ls_begin<LP_, Q6_>(desc[pb & 1], smem, sbase, L.off_tab + (pb & 1) * LS_TAB_BYTES, L.off_ring)
#define LS_RUN(LP_, Q6_) ls_loop<LP_, Q6_>(desc[p & 1], sbase, LsOffsets{L.off_tab + (p & 1) * LS_TAB_BYTES, L.off_img, L.off_terms, L.off_ring}, st)
    {
        const uint32_t pb = 0;
        LS_FOR_SHAPE(desc[0], LS_BEGIN);  // weights do not depend on the predecessor kernel
    }
    if (wait_dependency) asm volatile("griddepcontrol.wait;" ::: "memory");

    for (uint32_t p = 0; p < n_phases; ++p) {
        if (p + 1 < n_phases) fetch_desc(p + 1);  // visible after the synchronisations inside the phase
        else if (wait_dependency) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
        ls_prologue(desc[p & 1], smem, L.off_img, L.off_norm);
        LS_FOR_SHAPE(desc[p & 1], LS_RUN);
        if (p + 1 == n_phases) break;
        __syncthreads();  // every warp has left the ring and the image
        {
            const uint32_t pb = p + 1;
            LS_FOR_SHAPE(desc[pb & 1], LS_BEGIN);  // the next phase's first units travel while the barrier is crossed
        }
        // ---- grid barrier: everything phase p wrote is visible to everybody before anybody reads it
        __syncthreads();
        if (threadIdx.x == 0) {
            __threadfence();
            atomicAdd(barrier, 1u);
            const uint32_t target = (p + 1) * gridDim.x;
            unsigned long long t0 = 0;
            for (uint32_t spin = 0; ld_acquire_u32(barrier) < target; ++spin) {
                if ((spin & 255u) == 255u) {
                    unsigned long long t1;
                    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
                    if (t0 == 0) t0 = t1;
                    else if (t1 - t0 > (unsigned long long)timeout_ms * 1000000ull) {  // a CTA is missing: report, do not spin on
                        *status = 1u;
                        ctrl[0] = 1u;
                        break;
                    }
                }
            }
            __threadfence();
        }
        __syncthreads();
        if (ctrl[0]) {
            __pipeline_wait_prior(0);  // this thread's copies in flight
            return;
        }
    }
#undef LS_BEGIN
#undef LS_RUN
}

uint32_t align16(uint32_t v) { return (v + 15u) & ~15u; }

}  // namespace

constexpr uint32_t LS_MAX_SMEM = 227 * 1024;

// Shared-memory plan for a list of phases (the largest image, norm workspace and ring any of them needs).
LsLayout layer_stream_layout(const LsPhase *phases, uint32_t n) {
    uint32_t img = 0, norm = 0, ring = 0;
    for (uint32_t i = 0; i < n; ++i) {
        const LsPhase &d = phases[i];
        const uint32_t nb = d.a.in_dim / 256, bpc = d.lp / 2, ppu = 32 / d.lp;
        img = std::max(img, act_image(nb).bytes);
        if (d.a.prologue == SG_PRO_RMSNORM)
            norm = std::max<uint32_t>(norm, align16((d.a.in_dim + d.a.in_dim / 16 + 16) * 4) + align16((uint32_t)sizeof(SeqSumWorkspace<LS_THREADS>)));
        const uint32_t slot = 2u * ppu * part_bytes(d.q6 ? TYPE_Q6_K : TYPE_Q4_K, bpc);
        ring = std::max(ring, d.nw * 2u * slot);
    }
    LsLayout L{};
    L.off_desc = 0;
    L.off_tab = align16(2 * (uint32_t)sizeof(LsPhase));
    L.off_ctrl = L.off_tab + 2 * LS_TAB_BYTES;
    L.off_img = L.off_ctrl + 64;
    L.off_norm = L.off_img + align16(img);
    L.off_terms = L.off_norm + align16(norm);
    L.off_ring = L.off_terms + LS_WARPS * 128;
    L.total = L.off_ring + ring;
    return L;
}

bool layer_stream_phase(const StreamArgs &a, LsPhase *out) {
    if (a.n_seg < 1 || a.n_seg > 3 || a.in_dim % 256) return false;
    if (a.prologue != SG_PRO_READY && a.prologue != SG_PRO_RMSNORM) return false;
    bool q6 = false;
    for (int s = 0; s < a.n_seg; ++s) {
        const StreamSeg &g = a.seg[s];
        if (g.w.type != TYPE_Q4_K && g.w.type != TYPE_Q6_K) return false;
        if (g.w.in_dim != a.in_dim || g.w.row_stride >> 32 || g.w.out_dim == 0) return false;
        if (g.w2.data && (g.w2.type != g.w.type || g.w2.in_dim != a.in_dim || g.w2.out_dim != g.w.out_dim)) return false;
        if (g.epilogue >= SG_EP_ROPE_Q && g.epilogue <= SG_EP_V && (g.w.out_dim & 1)) return false;
        if (g.epilogue == SG_EP_XCHG) return false;
        q6 = q6 || g.w.type == TYPE_Q6_K;
    }
    LsPhase d{};
    d.a = a;
    d.a.wait_dependency = false;
    d.lp = lanes_per_pair(a.in_dim / 256);
    d.q6 = q6 ? 1u : 0u;
    d.nw = q6 ? 12u : 16u;  // a Q6_K unit is 6.7 KB: twelve two-slot rings are what fits beside the image
    d.l2_ahead = 0;
    *out = d;
    return true;
}

bool layer_stream_fits(const LsLayout &L) { return L.total <= LS_MAX_SMEM; }

bool launch_layer_stream(const LsPhase *dev_phases, uint32_t n, const LsLayout &L, int sm_count, uint32_t *barrier, uint32_t *status, uint32_t timeout_ms,
                         bool programmatic, cudaStream_t st) {
    if (n == 0) return true;
    static PerDeviceOnce once;
    if (once.run([] { return cudaFuncSetAttribute(layer_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, LS_MAX_SMEM); }) != cudaSuccess) return false;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)sm_count);  // one CTA per SM, all resident: the barrier counts on it
    cfg.blockDim = dim3(LS_THREADS);
    cfg.dynamicSmemBytes = L.total;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = programmatic ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, layer_stream_kernel, dev_phases, n, L, barrier, status, timeout_ms, programmatic) == cudaSuccess;
}

}  // namespace ob
