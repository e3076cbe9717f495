// Single-token products for decode, built around the weight stream.
//
// One decode step reads every weight byte once and does almost nothing else, so the step time is the
// HBM time plus whatever stops the stream: kernel boundaries, the norm / quantize prologue, the ramp of
// a fresh kernel -- and, on this part, instruction issue: at 6.5 TB/s an SM receives 23 bytes per clock
// and can issue at most four warp instructions in that clock, so the whole loop (copy, dot, sums, bookkeeping)
// has to stay near one instruction per 15-20 bytes.  Hence:
//
//   * two lanes share one super-block, for two rows at once (each takes 128 of its 256 elements and adds its integer
//     sums to the other's with one shuffle): the six-bit scales a lane needs are unpacked into one word, the
//     activations are read once per pair of rows, and the fp32 term is formed once per row;
//   * every warp owns two shared-memory slots and fills them with cp.async (16-byte, L1-bypassing) copies of
//     its next "units" (16 blocks x two rows = 4.6 KB), so the bytes in flight do not occupy registers and sixteen
//     warps fit an SM; the first units are requested before anything else happens in the kernel.  A lane copies
//     from one row only, at a fixed stride, so a unit costs it one pointer computation and 9 copies;
//   * the lanes-per-row-pair count is a template parameter and the work is split statically over all warps of
//     the grid, so the loop has no divisions, no atomics and no per-unit descriptors;
//   * the operator that produces the activations is the kernel's prologue (RMSNorm scaling and the int8
//     quantisation, written straight into shared memory in a conflict-free layout), and the operator that
//     consumes the product is its epilogue (residual add, silu(gate) * up, or RoPE and the fp16 KV append);
//   * two CTAs of eight warps fit one SM, and the kernel is launched with programmatic stream serialisation: it may
//     start, and request weights, while its predecessor is still running, and waits on the grid dependency
//     only before it reads the predecessor's output.
//
// Arithmetic is the single-token kernels of the reference, unchanged (engine/vecdot.rs:3152-3178 Q4_K,
// :3215-3241 Q6_K): exact integer partial sums, per-super-block fp32 terms with the reference's
// association, terms added in ascending block order by one lane.  The RMSNorm scale comes from
// norm_scale_kernel, which reproduces the CPU's left-to-right sum of squares (seqsum.cuh).
#include "seqsum.cuh"
#include "stream_common.cuh"

namespace ob {

namespace {

// ---- the kernel ----------------------------------------------------------------------------------------------
template <int LP, bool Q6>  // LP: lanes (= blocks per unit) of a row pair; Q6: the launch has Q6_K segments (three warps, larger slots)
__global__ void __launch_bounds__(Q6 ? 192 : 256, 2) stream_gemv_kernel(StreamArgs a) {
    extern __shared__ __align__(16) uint8_t smem[];
    constexpr int NW = Q6 ? 6 : 8, PPU = 32 / LP, BPC = LP / 2, HL = BPC;  // BPC: blocks per chunk; HL: lanes copying one row part
    constexpr uint32_t PB4 = BPC * 144u, PB6 = BPC * 208u + ((BPC * 2u + 15u) & ~15u);
    constexpr uint32_t SLOT = 2u * PPU * (Q6 ? PB6 : PB4);
    const SgSmem L = sg_smem(a.in_dim, Q6, LP);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(smem);
    const uint32_t terms = sbase + L.off_terms + warp * 128;
    const uint32_t slots = sbase + L.off_ring + warp * 2 * SLOT;
    const uint32_t nb = a.in_dim / 256, nchunk = (nb + BPC - 1) / BPC;

    // groups of PPU pairs, segments concatenated (a group never straddles two segments)
    uint32_t pairs_of[3], first_of[4];
    first_of[0] = 0;
#pragma unroll
    for (int s = 0; s < 3; ++s) {
        pairs_of[s] = s >= a.n_seg ? 0u : (a.seg[s].w2.data ? a.seg[s].w.out_dim : (a.seg[s].w.out_dim + 1) / 2);
        first_of[s + 1] = first_of[s] + (pairs_of[s] + PPU - 1) / PPU;
    }
    const uint32_t gb1 = first_of[1], gb2 = first_of[2], G = first_of[3];
    {
        auto put = [&](int s, const StreamSeg &g, uint32_t pairs, uint32_t first) {
            uint32_t *t = reinterpret_cast<uint32_t *>(smem) + s * SEG_WORDS;
            *reinterpret_cast<const uint8_t **>(t) = g.w.data;
            *reinterpret_cast<const uint8_t **>(t + 2) = g.w2.data;
            t[4] = (uint32_t)g.w.row_stride;
            t[5] = g.w.type;
            t[6] = g.w.out_dim;
            t[7] = pairs;
            t[8] = g.w.d_off;
            t[9] = (uint32_t)g.epilogue;
            *reinterpret_cast<float **>(t + 10) = g.y;
            t[12] = first;
        };
        if (threadIdx.x == 0) put(0, a.seg[0], pairs_of[0], 0);
        else if (threadIdx.x == 1 && a.n_seg > 1) put(1, a.seg[1], pairs_of[1], gb1);
        else if (threadIdx.x == 2 && a.n_seg > 2) put(2, a.seg[2], pairs_of[2], gb2);
    }
    __syncthreads();

    // this warp's contiguous share of the groups
    const uint32_t n_warps = gridDim.x * NW, gw = blockIdx.x * NW + warp;
    const uint32_t g_end = (uint32_t)(((uint64_t)G * (gw + 1)) / n_warps);
    const uint32_t g_first = (uint32_t)(((uint64_t)G * gw) / n_warps);
    uint32_t ig = g_first, ic = 0;  // next unit to request: group, chunk
    uint32_t cg = ig, cc = 0;                                        // next unit to compute

    const uint32_t q = lane / HL, sub = lane % HL, cj = q >> 1, cr = q & 1;  // copy role: part q = (pair cj, row cr), chunks sub + HL * k
    const uint32_t pj = lane / LP, bl = (lane % LP) >> 1, half = lane & 1;   // dot role: pair, block of the chunk, half of the block

    auto issue = [&](uint32_t slot, uint32_t g, uint32_t ch) {
        const uint32_t e = sbase + ((g >= gb1) + (g >= gb2)) * (SEG_WORDS * 4);
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
    };
    auto advance = [&](uint32_t &g, uint32_t &c) {
        if (++c == nchunk) {
            c = 0;
            ++g;
        }
    };

    // request the first two units before anything else: weights do not depend on the predecessor kernel
    if (ig < g_end) issue(slots, ig, ic);
    __pipeline_commit();
    advance(ig, ic);
    if (ig < g_end) issue(slots + SLOT, ig, ic);
    __pipeline_commit();
    advance(ig, ic);

    // ---- prologue ---------------------------------------------------------------------------------------------
    if (a.wait_dependency) {
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // the successor may start requesting its weights
        asm volatile("griddepcontrol.wait;" ::: "memory");               // the predecessor's output is complete and visible
    }
    const uint32_t xk = a.px.size > 1 ? *reinterpret_cast<const volatile uint32_t *>(a.px.seq) : 0u;  // number of this exchange
    if (a.prologue == SG_PRO_READY) {  // the producer left the image in global memory
        const uint32_t n16 = (L.off_terms - L.off_act) / 16;
        // five chunks per thread at a time, all requested before the first is stored: a store waits for its load, so a
        // plain copy loop would pay one trip to L2 per chunk (an image of 14336 activations is 4.4 chunks per thread)
        constexpr uint32_t CB = 5;
        for (uint32_t c0 = threadIdx.x; c0 < n16; c0 += CB * NW * 32) {
            uint4 v[CB];
#pragma unroll
            for (uint32_t k = 0; k < CB; ++k)
                if (c0 + k * NW * 32 < n16) v[k] = __ldcg(reinterpret_cast<const uint4 *>(a.ready) + c0 + k * NW * 32);
#pragma unroll
            for (uint32_t k = 0; k < CB; ++k)
                if (c0 + k * NW * 32 < n16) *reinterpret_cast<uint4 *>(smem + L.off_act + (c0 + k * NW * 32) * 16) = v[k];
        }
    } else {
        const bool norm = a.prologue == SG_PRO_RMSNORM;
        quantize_image(a.x, norm ? a.norm_w : nullptr, norm ? *a.norm_scale : 1.0f, nb, smem + L.off_act, warp, NW);
    }
    __syncthreads();

    // ---- main loop ------------------------------------------------------------------------------------------------
    float tot = 0.0f;  // lanes 2j, 2j+1: rows A, B of the group's pair j, running over the chunks of the row
    uint32_t par = 0;
    while (cg < g_end) {
        const uint32_t slot = slots + par * SLOT;
        const uint32_t e = sbase + ((cg >= gb1) + (cg >= gb2)) * (SEG_WORDS * 4);
        const uint32_t b0 = cc * BPC, nblk = min((uint32_t)BPC, nb - b0);
        __pipeline_wait_prior(1);
        __syncwarp();
        {
            const uint32_t gb = min(b0 + bl, nb - 1);  // lanes past the row's end recompute its last block; nobody reads their terms
            const uint32_t xa = sbase + L.off_act + gb * ACT_BLOCK_STRIDE;
            const float ad = __uint_as_float(lds32(sbase + L.off_d + gb * 4));
            int isum[2], imin[2] = {0, 0};
            float term;  // lane `half` ends up with the term of row `half` of the pair
            if (!Q6 || lds32(e + 20) == TYPE_Q4_K) {
                const uint32_t pA = slot + (2 * pj) * PB4 + bl * 144;
                uint32_t dd[2];
                dot_half_q4k(pA, pA + PB4, half, xa, sbase + L.off_bsum + gb * 16, isum, imin, dd);
#pragma unroll
                for (int r = 0; r < 2; ++r) {  // the two lanes of the cell add their halves: exact integers, any order
                    isum[r] += __shfl_xor_sync(0xffffffffu, isum[r], 1);
                    imin[r] += __shfl_xor_sync(0xffffffffu, imin[r], 1);
                }
                const int is = half ? isum[1] : isum[0], im = half ? imin[1] : imin[0];
                const uint32_t dw = half ? dd[1] : dd[0];
                const float d = f16_bits_to_f32(dw & 0xffffu), dmin = f16_bits_to_f32(dw >> 16);
                term = __fmul_rn(ad, __fsub_rn(__fmul_rn(d, (float)is), __fmul_rn(dmin, (float)im)));
            } else {
                const uint32_t pA = slot + (2 * pj) * PB6, pB = pA + PB6;
                dot_half_q6k(pA + bl * 208, pB + bl * 208, half, xa, sbase + L.off_sum16 + gb * 32, isum);
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
        if (ig < g_end) issue(slot, ig, ic);
        __pipeline_commit();
        advance(ig, ic);
        const bool row_done = cc + 1 == nchunk;
        const uint32_t g_done = cg;
        advance(cg, cc);
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
        case SG_EP_RESIDUAL:
            y[2 * pair] = __fadd_rn(a.residual[2 * pair], tA);
            if (hasB) y[2 * pair + 1] = __fadd_rn(a.residual[2 * pair + 1], tB);
            break;
        case SG_EP_SWIGLU:
            y[pair] = silu_mul_exact(tA, tB);
            break;
        case SG_EP_XCHG: {  // this rank's partial rows, tagged, into every rank's slot [parity][this rank]
            const uint64_t off = (uint64_t)((xk & 1u) * a.px.size + a.px.rank) * a.px.n + 2 * pair;
            for (uint32_t r = 0; r < a.px.size; ++r) {
                uint2 *dst = a.px.slots[r] + off;
                if (hasB)
                    asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(dst), "r"(__float_as_uint(tA)), "r"(xk + 1u), "r"(__float_as_uint(tB)), "r"(xk + 1u) : "memory");
                else
                    asm volatile("st.volatile.global.v2.u32 [%0], {%1,%2};" ::"l"(dst), "r"(__float_as_uint(tA)), "r"(xk + 1u) : "memory");
            }
            break;
        }
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
    // Every warp adds the number of outputs it stored to the counters of the blocks they belong to; the add that brings a
    // counter to 256 tells its warp that the whole block is in memory.  The counters are left at zero.
    if (a.out_image) {
        const uint32_t pairs = pairs_of[0];
        const uint32_t p0 = min(g_first * PPU, pairs), p1 = min(g_end * PPU, pairs);
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

// 1 / sqrt(mean(x^2) + eps) with the squares added left to right (engine/tensor.rs:743-745), one CTA.  With `image` set the
// CTA goes on to quantize (x * scale) * norm_w per 256, so that the product kernels that follow only copy the result.
constexpr int NS_THREADS = 512;
__global__ void __launch_bounds__(NS_THREADS) norm_scale_kernel(float *__restrict__ x, const float *__restrict__ norm_w, uint32_t dim, float eps,
                                                                float *__restrict__ out, uint8_t *__restrict__ image, obtp::PeerXchg px, bool wait_dependency) {
    extern __shared__ float srow[];  // the row, one pad word per 16
    __shared__ SeqSumWorkspace<NS_THREADS> ws;
    // The weights do not depend on the predecessor: those of this warp's first two blocks are in registers, the others in
    // L2, by the time the scale is known.
    constexpr uint32_t NS_WARPS = NS_THREADS / 32, NS_PRE = 2;
    const uint32_t nb = dim / 256, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // Completing a tensor-parallel exchange means pulling size x dim tagged words; that part is spread over the CTAs of a
    // cluster (each takes a slice of the row from all ranks, sums it, and hands the slice to CTA 0 through distributed shared
    // memory).  Everything else -- the exact sum, the image -- is CTA 0's.
    uint32_t crank, csize;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(crank));
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(csize));
    float wpre[NS_PRE][8];
    if (norm_w && image && crank == 0) {
#pragma unroll
        for (uint32_t k = 0; k < NS_PRE; ++k) {
            const uint32_t b = warp + k * NS_WARPS;
            if (b < nb) {
                const float4 w0 = __ldg(reinterpret_cast<const float4 *>(norm_w + b * 256 + lane * 8)), w1 = __ldg(reinterpret_cast<const float4 *>(norm_w + b * 256 + lane * 8 + 4));
                wpre[k][0] = w0.x; wpre[k][1] = w0.y; wpre[k][2] = w0.z; wpre[k][3] = w0.w; wpre[k][4] = w1.x; wpre[k][5] = w1.y; wpre[k][6] = w1.z; wpre[k][7] = w1.w;
            }
        }
        for (uint32_t i = NS_PRE * NS_WARPS * 256 + threadIdx.x * 32; i < dim; i += NS_THREADS * 32) asm volatile("prefetch.global.L2 [%0];" ::"l"(norm_w + i));
    }
    if (wait_dependency) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
    }
    if (px.size > 1) {
        // complete the pending exchange: every element is read until it carries this exchange's tag (bounded), then
        // x += (p_0 + p_1 + ..) in rank order
        const uint32_t k = *reinterpret_cast<const volatile uint32_t *>(px.seq), tag = k + 1u;
        const uint2 *mine = px.slots[px.rank] + (uint64_t)(k & 1u) * px.size * px.n;
        unsigned long long t0;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
        bool gave_up = false;
        // Four elements x all ranks at a time: every word is requested before any is examined, so a batch costs one
        // trip to memory when the partials are already there (the usual case); words that do not carry the tag yet are
        // read again, one after the other.
        constexpr uint32_t EB = 4, MAX_RANKS = 8;
        const uint32_t lo = (uint32_t)(((uint64_t)dim * crank) / csize), hi = (uint32_t)(((uint64_t)dim * (crank + 1)) / csize);  // this CTA's slice
        uint32_t srow0;  // the row in CTA 0's shared memory
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(srow0) : "r"((uint32_t)__cvta_generic_to_shared(srow)), "r"(0));
        for (uint32_t i0 = lo + threadIdx.x; i0 < hi; i0 += EB * NS_THREADS) {
            uint2 w[EB][MAX_RANKS];
            float xv[EB];
#pragma unroll
            for (uint32_t e = 0; e < EB; ++e) {
                const uint32_t i = i0 + e * NS_THREADS;
#pragma unroll
                for (uint32_t r = 0; r < MAX_RANKS; ++r)
                    if (i < hi && r < px.size)
                        asm volatile("ld.volatile.global.v2.u32 {%0,%1}, [%2];" : "=r"(w[e][r].x), "=r"(w[e][r].y) : "l"(mine + (uint64_t)r * px.n + i) : "memory");
                if (i < hi) xv[e] = __ldcg(x + i);
            }
#pragma unroll
            for (uint32_t e = 0; e < EB; ++e) {
                const uint32_t i = i0 + e * NS_THREADS;
                if (i >= hi) continue;
                float sum = 0.0f;
#pragma unroll
                for (uint32_t r = 0; r < MAX_RANKS; ++r) {
                    if (r >= px.size) continue;
                    const uint2 *src = mine + (uint64_t)r * px.n + i;
                    for (uint32_t spin = 0; w[e][r].y != tag && !gave_up; ++spin) {
                        asm volatile("ld.volatile.global.v2.u32 {%0,%1}, [%2];" : "=r"(w[e][r].x), "=r"(w[e][r].y) : "l"(src) : "memory");
                        if ((spin & 1023u) == 1023u) {
                            unsigned long long t1;
                            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
                            if (t1 - t0 > (unsigned long long)(px.timeout_ms ? px.timeout_ms : 4000u) * 1000000ull) {  // a rank is gone: report and go on with what is there
                                *px.err = 1u;
                                gave_up = true;
                            }
                        }
                    }
                    sum = r == 0 ? __uint_as_float(w[e][r].x) : __fadd_rn(sum, __uint_as_float(w[e][r].x));
                }
                const float v = __fadd_rn(xv[e], sum);
                x[i] = v;
                asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(srow0 + 4u * (i + (i >> 4))), "f"(v) : "memory");
            }
        }
        if (csize > 1) {  // the slices are in CTA 0's shared memory once every CTA of the cluster has arrived
            asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
            asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
            if (crank != 0) return;
        } else {
            __syncthreads();
        }
        if (threadIdx.x == 0) *px.seq = k + 1u;
    } else {
        for (uint32_t i = threadIdx.x; i < dim; i += NS_THREADS) srow[i + (i >> 4)] = __ldcg(x + i);
        __syncthreads();
    }
    // The successor is let in only now: its CTAs start by requesting weights, and that traffic would stand in the way of
    // the loads above, which are on the critical path.
    if (wait_dependency) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const float t = cta_sequential_sum<NS_THREADS>([&](uint32_t i) { const float v = srow[i + (i >> 4)]; return __fmul_rn(v, v); }, dim, ws);
    const float scale = __fdiv_rn(1.0f, sqrtf(__fadd_rn(__fdiv_rn(t, (float)dim), eps)));
    if (threadIdx.x == 0 && out) *out = scale;
    if (!image) return;
    if (!norm_w) {
        quantize_image(x, nullptr, scale, nb, image, warp, NS_WARPS);
        return;
    }
    // (x * scale) * w per 256, the row taken from shared memory (the pad keeps a lane's 8 elements together)
    const ActImage im = act_image(nb);
    for (uint32_t k = 0, b = warp; b < nb; ++k, b += NS_WARPS) {
        const uint32_t e0 = b * 256 + lane * 8;
        const float *sv = srow + e0 + (e0 >> 4);
        float v[8], w[8];
        if (k < NS_PRE) {
#pragma unroll
            for (int i = 0; i < 8; ++i) w[i] = k == 0 ? wpre[0][i] : wpre[1][i];
        } else {
            const float4 w0 = __ldg(reinterpret_cast<const float4 *>(norm_w + e0)), w1 = __ldg(reinterpret_cast<const float4 *>(norm_w + e0 + 4));
            w[0] = w0.x; w[1] = w0.y; w[2] = w0.z; w[3] = w0.w; w[4] = w1.x; w[5] = w1.y; w[6] = w1.z; w[7] = w1.w;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = __fmul_rn(__fmul_rn(sv[i], scale), w[i]);  // tensor.rs:747
        quantize_block(v, b, image, im);
    }
}

// x quantized per 256 into the image, one warp per block.
__global__ void __launch_bounds__(128) quant_image_kernel(const float *__restrict__ x, uint32_t nb, uint8_t *__restrict__ image, bool wait_dependency) {
    if (wait_dependency) {
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
        asm volatile("griddepcontrol.wait;" ::: "memory");
    }
    quantize_image(x, nullptr, 1.0f, nb, image, blockIdx.x * 4 + (threadIdx.x >> 5), gridDim.x * 4);
}

}  // namespace

static uint32_t pick_lp(uint32_t nb) { return lanes_per_pair(nb); }

bool stream_gemv_supported(const StreamArgs &a) {
    if (a.n_seg < 1 || a.n_seg > 3 || a.in_dim % 256) return false;
    bool q6 = false;
    for (int s = 0; s < a.n_seg; ++s) {
        const StreamSeg &g = a.seg[s];
        if (g.w.type != TYPE_Q4_K && g.w.type != TYPE_Q6_K) return false;
        if (g.w.in_dim != a.in_dim || g.w.row_stride >> 32 || g.w.out_dim == 0) return false;
        if (g.w2.data && (g.w2.type != g.w.type || g.w2.in_dim != a.in_dim || g.w2.out_dim != g.w.out_dim)) return false;
        if (g.epilogue >= SG_EP_ROPE_Q && (g.w.out_dim & 1)) return false;
        q6 = q6 || g.w.type == TYPE_Q6_K;
    }
    return sg_smem(a.in_dim, q6, pick_lp(a.in_dim / 256)).total <= SG_MAX_SMEM;
}

size_t act_image_bytes(uint32_t dim) { return act_image(dim / 256).bytes; }

void launch_norm_quant_consume(float *x, const float *norm_w, uint32_t dim, float eps, float *scale_out, uint8_t *image, const obtp::PeerXchg &px,
                               bool programmatic, cudaStream_t st) {
    static PerDeviceOnce once;
    if (once.run([] { return cudaFuncSetAttribute(norm_scale_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024); }) != cudaSuccess) return;
    // with an exchange to complete: a cluster of eight CTAs shares the pull of size x dim tagged words (local memory only).
    // Measured on two GPUs, 8B shape, tokens per second at batch 1: 528 with one CTA, 573 with two, 599 with four, 608 with eight.
    static const unsigned consume_ctas = [] { const char *e = getenv("OB_TP_CONSUME_CTAS"); const int v = e ? atoi(e) : 8; return (unsigned)(v == 1 || v == 2 || v == 4 || v == 8 ? v : 8); }();
    const unsigned ctas = px.size > 1 ? consume_ctas : 1u;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(ctas);
    cfg.blockDim = dim3(NS_THREADS);
    cfg.dynamicSmemBytes = ((size_t)dim + dim / 16 + 16) * 4;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    unsigned n_attr = 0;
    if (programmatic) {
        attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
        ++n_attr;
    }
    if (ctas > 1) {
        attr[n_attr].id = cudaLaunchAttributeClusterDimension;
        attr[n_attr].val.clusterDim.x = ctas;
        attr[n_attr].val.clusterDim.y = 1;
        attr[n_attr].val.clusterDim.z = 1;
        ++n_attr;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    cudaLaunchKernelEx(&cfg, norm_scale_kernel, x, norm_w, dim, eps, scale_out, image, px, programmatic);
}

void launch_norm_quant(const float *x, const float *norm_w, uint32_t dim, float eps, float *scale_out, uint8_t *image, bool programmatic, cudaStream_t st) {
    launch_norm_quant_consume(const_cast<float *>(x), norm_w, dim, eps, scale_out, image, obtp::PeerXchg{}, programmatic, st);  // no exchange: x is only read
}

void launch_norm_scale(const float *x, uint32_t dim, float eps, float *out, bool programmatic, cudaStream_t st) {
    launch_norm_quant(x, nullptr, dim, eps, out, nullptr, programmatic, st);
}

void launch_quant_image(const float *x, uint32_t dim, uint8_t *image, bool programmatic, cudaStream_t st) {
    const uint32_t nb = dim / 256;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((nb + 3) / 4);
    cfg.blockDim = dim3(128);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = programmatic ? 1 : 0;
    cudaLaunchKernelEx(&cfg, quant_image_kernel, x, nb, image, programmatic);
}

template <int LP, bool Q6>
void launch_instance(const cudaLaunchConfig_t &cfg, const StreamArgs &args) {
    static PerDeviceOnce once;  // one per instantiation
    if (once.run([] { return cudaFuncSetAttribute(stream_gemv_kernel<LP, Q6>, cudaFuncAttributeMaxDynamicSharedMemorySize, SG_MAX_SMEM); }) != cudaSuccess) return;
    cudaLaunchKernelEx(&cfg, stream_gemv_kernel<LP, Q6>, args);
}

template <bool Q6>
void launch_lp(uint32_t lp, const cudaLaunchConfig_t &cfg, const StreamArgs &args) {
    switch (lp) {
    case 2: launch_instance<2, Q6>(cfg, args); break;
    case 4: launch_instance<4, Q6>(cfg, args); break;
    case 8: launch_instance<8, Q6>(cfg, args); break;
    case 16: launch_instance<16, Q6>(cfg, args); break;
    default: launch_instance<32, Q6>(cfg, args); break;
    }
}

void launch_stream_gemv(const StreamArgs &a, int sm_count, bool programmatic, cudaStream_t st) {
    bool q6 = false;
    uint32_t groups = 0;
    const uint32_t lp = pick_lp(a.in_dim / 256), ppu = 32 / lp;
    for (int s = 0; s < a.n_seg; ++s) {
        q6 = q6 || a.seg[s].w.type == TYPE_Q6_K;
        const uint32_t pairs = a.seg[s].w2.data ? a.seg[s].w.out_dim : (a.seg[s].w.out_dim + 1) / 2;
        groups += (pairs + ppu - 1) / ppu;
    }
    const SgSmem L = sg_smem(a.in_dim, q6, lp);
    StreamArgs args = a;
    args.wait_dependency = programmatic;
    const uint32_t nw = (uint32_t)sg_warps(q6);
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
    if (q6) launch_lp<true>(lp, cfg, args);
    else launch_lp<false>(lp, cfg, args);
}

}  // namespace ob
