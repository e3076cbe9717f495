// Decode-time attention over the paged fp16 KV cache (flash-decode: split over pages, then merge).
//
// Reference semantics (src/bin/orangu-server/engine/attention.rs:426-549): per query head h with
// kv head h / group, score_p = dot(q_h, k_p) * scale over the causal window 0..=pos, softmax,
// out_h = sum_p w_p * v_p.  K and V are what the fp16 KV mirror holds (kv_cache.rs:26-32); all
// arithmetic here is fp32.  The softmax is evaluated online per tile and the partial results of
// the splits are merged exactly (max-shifted), so the result differs from the reference's
// two-pass form only by fp32 rounding.
//
// Layout: a layer's pool is [page][n_head_kv][16 tokens][head_dim] fp16, so the tile a CTA needs
// for one (page, kv head) is one contiguous 16*head_dim*2-byte run -- read with 16-byte cp.async
// into a two-stage shared-memory ring while the previous tile is consumed.  All `group` query
// heads that share a kv head are handled by the same CTA, so each K/V byte is read once.
#include <cuda_pipeline.h>

#include "common.cuh"
#include "kernels.h"

namespace ob {

namespace {

constexpr int AT_THREADS = 128;
constexpr int TILE_PAGES = 4;
constexpr int TILE_TOK = TILE_PAGES * KV_PAGE;  // 64

template <int HD, int G>
struct AttnSmem {
    __half k[2][TILE_TOK][HD];
    __half v[2][TILE_TOK][HD];
    float q[G][HD];
    float s[G][TILE_TOK];   // scores, head-major (softmax reads along tokens)
    float p[TILE_TOK][G];   // probabilities, token-major (PV reads all heads of a token at once)
    float alpha[G];
    float red[2][G][HD];    // cross-token-group reduction of the output
};

template <int HD, int G>
__global__ void __launch_bounds__(AT_THREADS) attn_decode_kernel(AttnDecodeArgs a) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    AttnSmem<HD, G> &sm = *reinterpret_cast<AttnSmem<HD, G> *>(smem_raw);
    constexpr int CH = HD / 64;  // 16-byte K chunks per lane in the score phase
    const uint32_t split = blockIdx.x, kvh = blockIdx.y, seq = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t n_pos = a.n_pos[seq];
    const uint32_t n_pages = (n_pos + KV_PAGE - 1) / KV_PAGE;
    const uint32_t pages_per_split = ((n_pages + a.n_splits - 1) / a.n_splits + TILE_PAGES - 1) / TILE_PAGES * TILE_PAGES;
    const uint32_t page_begin = min(n_pages, split * pages_per_split);
    const uint32_t page_end = min(n_pages, page_begin + pages_per_split);
    const int32_t *table = a.page_tables[seq];
    const uint32_t head0 = kvh * G;

    // q of the G heads of this kv head
    for (int i = tid; i < G * HD; i += AT_THREADS) sm.q[i / HD][i % HD] = a.q[(uint64_t)seq * a.n_head * HD + (uint64_t)head0 * HD + i];

    auto stage_tile = [&](uint32_t first_page, int st) {
        constexpr int CHUNKS_PER_PAGE = KV_PAGE * HD * 2 / 16;
        for (int j = 0; j < TILE_PAGES; ++j) {
            const uint32_t pg = first_page + j;
            if (pg >= page_end) break;
            const uint64_t base = ((uint64_t)table[pg] * a.n_head_kv + kvh) * KV_PAGE * HD;
            const uint4 *ks = reinterpret_cast<const uint4 *>(a.k_pool + base), *vs = reinterpret_cast<const uint4 *>(a.v_pool + base);
            uint4 *kd = reinterpret_cast<uint4 *>(&sm.k[st][j * KV_PAGE][0]), *vd = reinterpret_cast<uint4 *>(&sm.v[st][j * KV_PAGE][0]);
            for (int c = tid; c < CHUNKS_PER_PAGE; c += AT_THREADS) {
                __pipeline_memcpy_async(kd + c, ks + c, 16);
                __pipeline_memcpy_async(vd + c, vs + c, 16);
            }
        }
        __pipeline_commit();
    };

    float o[G][2];
#pragma unroll
    for (int g = 0; g < G; ++g) o[g][0] = o[g][1] = 0.0f;
    float m_run = -INFINITY, l_run = 0.0f;  // valid in the warp(s) that own a head's softmax
    // second head owned by this warp when G == 8 (two heads per warp)
    float m_run2 = -INFINITY, l_run2 = 0.0f;

    if (page_begin < page_end) stage_tile(page_begin, 0);
    __syncthreads();  // q visible

    // q fragments for the score phase: dims 64*i + 8*dc .. +7
    const int dc = lane & 7, tl = lane >> 3;
    float qr[G][CH * 8];
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int i = 0; i < CH; ++i)
#pragma unroll
            for (int e = 0; e < 8; ++e) qr[g][i * 8 + e] = sm.q[g][i * 64 + dc * 8 + e];

    int st = 0;
    for (uint32_t pg0 = page_begin; pg0 < page_end; pg0 += TILE_PAGES, st ^= 1) {
        __pipeline_wait_prior(0);
        __syncthreads();  // (A) tile pg0 landed; everyone is done with the other stage
        if (pg0 + TILE_PAGES < page_end) stage_tile(pg0 + TILE_PAGES, st ^ 1);
        const uint32_t tile_pos0 = pg0 * KV_PAGE;
        const uint32_t valid = min((uint32_t)TILE_TOK, n_pos - tile_pos0);  // tokens of this tile inside the window

        // ---- scores: warp w takes page w of the tile, 4 tokens x 8 dim-chunks per step
#pragma unroll
        for (int step = 0; step < 4; ++step) {
            const uint32_t tok = warp * KV_PAGE + step * 4 + tl;
            float acc[G];
#pragma unroll
            for (int g = 0; g < G; ++g) acc[g] = 0.0f;
            if (tok < valid) {
#pragma unroll
                for (int i = 0; i < CH; ++i) {
                    const uint4 kv = *reinterpret_cast<const uint4 *>(&sm.k[st][tok][i * 64 + dc * 8]);
                    const __half2 *kh = reinterpret_cast<const __half2 *>(&kv);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float2 kf = __half22float2(kh[e]);
#pragma unroll
                        for (int g = 0; g < G; ++g) {
                            acc[g] = __fmaf_rn(qr[g][i * 8 + 2 * e], kf.x, acc[g]);
                            acc[g] = __fmaf_rn(qr[g][i * 8 + 2 * e + 1], kf.y, acc[g]);
                        }
                    }
                }
            }
#pragma unroll
            for (int g = 0; g < G; ++g) {
                acc[g] += __shfl_xor_sync(0xffffffffu, acc[g], 1);
                acc[g] += __shfl_xor_sync(0xffffffffu, acc[g], 2);
                acc[g] += __shfl_xor_sync(0xffffffffu, acc[g], 4);
            }
            if (dc == 0) {
#pragma unroll
                for (int g = 0; g < G; ++g) sm.s[g][tok] = tok < valid ? __fmul_rn(acc[g], a.scale) : -INFINITY;
            }
        }
        __syncthreads();  // (B)

        // ---- online softmax: head g is owned by warp g % 4 (lanes cover tokens lane, lane + 32)
#pragma unroll
        for (int rep = 0; rep < (G + 3) / 4; ++rep) {
            const int g = warp + 4 * rep;
            if (g < G) {
                float &mr = rep == 0 ? m_run : m_run2;
                float &lr = rep == 0 ? l_run : l_run2;
                const float s0 = sm.s[g][lane], s1 = sm.s[g][lane + 32];
                const float m_new = fmaxf(mr, warp_max(fmaxf(s0, s1)));
                const float p0 = s0 == -INFINITY ? 0.0f : expf(s0 - m_new);
                const float p1 = s1 == -INFINITY ? 0.0f : expf(s1 - m_new);
                const float al = mr == -INFINITY ? 0.0f : expf(mr - m_new);
                lr = __fmaf_rn(lr, al, warp_sum(p0 + p1));
                mr = m_new;
                sm.p[lane][g] = p0;
                sm.p[lane + 32][g] = p1;
                if (lane == 0) sm.alpha[g] = al;
            }
        }
        __syncthreads();  // (C)

        // ---- output: thread owns dims (2*dp, 2*dp+1) for the token half tg of the tile
        {
            constexpr int DP = HD / 2;                 // dim pairs
            constexpr int TG = AT_THREADS / DP;        // token groups (2 for HD 128, 4 for HD 64)
            constexpr int TOK_PER_TG = TILE_TOK / TG;
            const int dp = tid % DP, tg = tid / DP;
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const float al = sm.alpha[g];
                o[g][0] *= al;
                o[g][1] *= al;
            }
            const uint32_t t_end = min((uint32_t)((tg + 1) * TOK_PER_TG), valid);
            for (uint32_t tok = tg * TOK_PER_TG; tok < t_end; ++tok) {
                const float2 vf = __half22float2(*reinterpret_cast<const __half2 *>(&sm.v[st][tok][2 * dp]));
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    const float pw = sm.p[tok][g];
                    o[g][0] = __fmaf_rn(pw, vf.x, o[g][0]);
                    o[g][1] = __fmaf_rn(pw, vf.y, o[g][1]);
                }
            }
        }
    }

    // ---- write this split's partial: o (unnormalised), running max and sum
    {
        constexpr int DP = HD / 2;
        constexpr int TG = AT_THREADS / DP;
        const int dp = tid % DP, tg = tid / DP;
        __syncthreads();
        // reduce the token groups through shared memory, two at a time
        for (int r = TG - 1; r >= 1; --r) {
            if (tg == r) {
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    sm.red[0][g][2 * dp] = o[g][0];
                    sm.red[0][g][2 * dp + 1] = o[g][1];
                }
            }
            __syncthreads();
            if (tg == 0) {
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    o[g][0] += sm.red[0][g][2 * dp];
                    o[g][1] += sm.red[0][g][2 * dp + 1];
                }
            }
            __syncthreads();
        }
        if (tg == 0) {
#pragma unroll
            for (int g = 0; g < G; ++g) {
                float *po = a.part_o + (((uint64_t)seq * a.n_head + head0 + g) * a.n_splits + split) * HD;
                *reinterpret_cast<float2 *>(po + 2 * dp) = make_float2(o[g][0], o[g][1]);
            }
        }
#pragma unroll
        for (int rep = 0; rep < (G + 3) / 4; ++rep) {
            const int g = warp + 4 * rep;
            if (g < G && lane == 0) {
                float *pm = a.part_ml + (((uint64_t)seq * a.n_head + head0 + g) * a.n_splits + split) * 2;
                pm[0] = rep == 0 ? m_run : m_run2;
                pm[1] = rep == 0 ? l_run : l_run2;
            }
        }
    }
}

// grid (n_head, n_seq), HD threads: exact merge of the splits.
__global__ void attn_merge_kernel(AttnDecodeArgs a) {
    const uint32_t head = blockIdx.x, seq = blockIdx.y, d = threadIdx.x;
    const uint32_t hd = a.head_dim;
    const float *pm = a.part_ml + ((uint64_t)seq * a.n_head + head) * a.n_splits * 2;
    const float *po = a.part_o + ((uint64_t)seq * a.n_head + head) * a.n_splits * hd;
    float m = -INFINITY;
    for (uint32_t s = 0; s < a.n_splits; ++s) m = fmaxf(m, pm[2 * s]);
    float acc = 0.0f, l = 0.0f;
    for (uint32_t s = 0; s < a.n_splits; ++s) {
        const float ms = pm[2 * s];
        if (ms == -INFINITY) continue;
        const float w = expf(ms - m);
        l = __fmaf_rn(w, pm[2 * s + 1], l);
        acc = __fmaf_rn(w, po[(uint64_t)s * hd + d], acc);
    }
    a.out[(uint64_t)seq * a.n_head * hd + (uint64_t)head * hd + d] = l > 0.0f ? __fdiv_rn(acc, l) : 0.0f;
}

// Any head_dim (even, <= 256) and any group size: one warp per (row, head), no split.
__global__ void attn_generic_kernel(AttnDecodeArgs a) {
    const uint32_t head = blockIdx.x, seq = blockIdx.y, lane = threadIdx.x;
    const uint32_t hd = a.head_dim, group = (a.n_head + a.n_head_kv - 1) / a.n_head_kv, kvh = head / group;
    const uint32_t n_pos = a.n_pos[seq];
    const int32_t *table = a.page_tables[seq];
    const float *q = a.q + (uint64_t)seq * a.n_head * hd + (uint64_t)head * hd;
    float qv[8], o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint32_t d = lane + 32 * i;
        qv[i] = d < hd ? q[d] : 0.0f;
        o[i] = 0.0f;
    }
    float m = -INFINITY, l = 0.0f;
    for (uint32_t p = 0; p < n_pos; ++p) {
        const uint64_t base = (((uint64_t)table[p / KV_PAGE] * a.n_head_kv + kvh) * KV_PAGE + p % KV_PAGE) * hd;
        float dot = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t d = lane + 32 * i;
            if (d < hd) dot = __fmaf_rn(qv[i], __half2float(a.k_pool[base + d]), dot);
        }
        dot = __fmul_rn(warp_sum(dot), a.scale);
        const float m_new = fmaxf(m, dot);
        const float al = m == -INFINITY ? 0.0f : expf(m - m_new);
        const float pw = expf(dot - m_new);
        l = __fmaf_rn(l, al, pw);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t d = lane + 32 * i;
            if (d < hd) o[i] = __fmaf_rn(pw, __half2float(a.v_pool[base + d]), o[i] * al);
        }
        m = m_new;
    }
    float *out = a.out + (uint64_t)seq * a.n_head * hd + (uint64_t)head * hd;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint32_t d = lane + 32 * i;
        if (d < hd) out[d] = l > 0.0f ? __fdiv_rn(o[i], l) : 0.0f;
    }
}

template <int HD, int G>
void launch_fast(const AttnDecodeArgs &a, cudaStream_t st) {
    static PerDeviceOnce once;  // one per instantiation
    const size_t smem = sizeof(AttnSmem<HD, G>);
    if (once.run([] { return cudaFuncSetAttribute(attn_decode_kernel<HD, G>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(AttnSmem<HD, G>)); }) != cudaSuccess) return;
    dim3 grid(a.n_splits, a.n_head_kv, a.n_seq);
    attn_decode_kernel<HD, G><<<grid, AT_THREADS, smem, st>>>(a);
    attn_merge_kernel<<<dim3(a.n_head, a.n_seq), HD, 0, st>>>(a);
}

template <int HD>
bool launch_hd(const AttnDecodeArgs &a, uint32_t group, cudaStream_t st) {
    switch (group) {
    case 1: launch_fast<HD, 1>(a, st); return true;
    case 2: launch_fast<HD, 2>(a, st); return true;
    case 4: launch_fast<HD, 4>(a, st); return true;
    case 8: launch_fast<HD, 8>(a, st); return true;
    default: return false;
    }
}


// ====================================================================================================
// Fused flash-decode: split, merge and (optionally) int8 quantisation of the output in one kernel.
//
// A CTA has four warps and no barrier inside its loop.  Each warp streams its own 16-token pages of K and V into a
// private two-slot shared-memory ring with cp.async, scores the page for all `G` query heads of the kv head, keeps an
// online softmax per head in registers and accumulates its part of the output.  Scores and outputs are products of
// a [heads x dims] or [heads x tokens] matrix with the fp16 page, so they go through the tensor cores
// (mma.sync m16n8k16, fp32 accumulation).  The fp32 operands (q, and the probabilities) enter as two fp16 rows each, a
// rounded value and the remainder, which keeps their error near 2^-22 instead of 2^-11; with at most 8 heads the
// sixteen rows of the tile have room for both.
//
// The four warps merge through shared memory, the CTA writes one partial per head, and the CTA that finds itself
// last for its (sequence, kv head) -- a counter in global memory tells -- merges the partials of all splits,
// normalises and stores the result.  When the caller passes `image`, that CTA also quantizes its G * HD outputs per
// 256 exactly as the activation quantizer does (engine/vecdot.rs:3030-3053), so the attention-output product can
// start from int8 without another launch.
// ====================================================================================================


template <int HD, int G, int AF_WARPS>
struct AttnFusedSmem {
    static constexpr int ROW = HD * 2 + 16;             // bytes per token row: the pad spreads eight rows over all banks
    uint8_t kv[AF_WARPS][2][2][KV_PAGE * ROW];          // [warp][slot][k|v]
    float q[G][HD];
    float wo[AF_WARPS][G][HD];                          // per-warp partial outputs
    float4 acc_part[AF_WARPS * 32];                     // final merge: partial sums of the threads that share a piece
    float wgt[G][64];                                   // final merge: weight of every split
    float wm[AF_WARPS][G], wl[AF_WARPS][G];
    float red[8];
    int is_last;
};

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
// D (16x8, fp32) += A (16x16, fp16, row) * B (16x8, fp16, col)
__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_half2(float x, float y) {
    const __half2 h = __floats2half2_rn(x, y);
    return *reinterpret_cast<const uint32_t *>(&h);
}
// the fp16 remainders of (x, y) after their fp16 roundings
__device__ __forceinline__ uint32_t pack_half2_rest(float x, float y) {
    const __half2 h = __floats2half2_rn(x, y);
    const float2 f = __half22float2(h);
    return pack_half2(x - f.x, y - f.y);
}

// AF_WARPS: 8 (one CTA per SM; single-token decode, where every SM should be streaming pages) or 4 (two CTAs per SM, whose
// start-up and merge phases overlap each other's streaming; large batches).
template <int HD, int G, int AF_WARPS>
__global__ void __launch_bounds__(AF_WARPS * 32) attn_decode_fused_kernel(AttnDecodeArgs a, bool wait_dependency, bool early_pages) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    using Smem = AttnFusedSmem<HD, G, AF_WARPS>;
    Smem &sm = *reinterpret_cast<Smem *>(smem_raw);
    constexpr int ROW = Smem::ROW;
    constexpr int THREADS = AF_WARPS * 32;
    constexpr bool LO8 = G == 8;          // remainders in rows 8..15 (else in rows 4..7)
    constexpr int KS = HD / 16;           // k-steps of the score product
    constexpr int NT = HD / 8;            // n-tiles of the output product
    const uint32_t split = blockIdx.x, kvh = blockIdx.y, seq = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int gid = lane >> 2, tig = lane & 3;  // the fragment's row (group) and column pair
    const uint32_t head0 = kvh * G;

    // ---- before the grid dependency: everything that the predecessor (which appends this token's K and V and writes q)
    // does not produce -- the window, the page table and all pages but the one the new token lands in
    const uint32_t n_pos = a.n_pos[seq];
    const int32_t *table = a.page_tables[seq];
    const uint32_t n_pages = (n_pos + KV_PAGE - 1) / KV_PAGE;
    const uint32_t pages_per_split = (n_pages + a.n_splits - 1) / a.n_splits;
    const uint32_t page_begin = min(n_pages, split * pages_per_split);
    const uint32_t page_end = min(n_pages, page_begin + pages_per_split);
    const uint32_t kv_base = (uint32_t)__cvta_generic_to_shared(&sm.kv[warp][0][0][0]);
    constexpr uint32_t SLOT_BYTES = 2 * KV_PAGE * ROW, HALF_BYTES = KV_PAGE * ROW;

    auto stage_page = [&](uint32_t pg, int slot) {
        const uint64_t base = ((uint64_t)table[pg] * a.n_head_kv + kvh) * KV_PAGE * HD;
        const uint8_t *ks = reinterpret_cast<const uint8_t *>(a.k_pool + base), *vs = reinterpret_cast<const uint8_t *>(a.v_pool + base);
        constexpr int CPR = HD / 8;  // 16-byte chunks per token row
        constexpr int CHUNKS = KV_PAGE * CPR;
#pragma unroll
        for (int c = 0; c < CHUNKS / 32; ++c) {
            const int ch = lane + 32 * c, tok = ch / CPR, j = ch % CPR;
            const uint32_t dst = kv_base + slot * SLOT_BYTES + tok * ROW + j * 16;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(ks + ch * 16) : "memory");
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + HALF_BYTES), "l"(vs + ch * 16) : "memory");
        }
    };

    // this warp's pages: page_begin + warp, + AF_WARPS, ...
    uint32_t pg = page_begin + warp;
    const uint32_t fresh_page = n_pos ? (n_pos - 1) / KV_PAGE : 0;  // only this page changes under the predecessor
    // (with several rows the predecessor may be writing any page of a shared sequence: then nothing is fetched early)
    const bool defer0 = wait_dependency && (!early_pages || pg == fresh_page), defer1 = wait_dependency && (!early_pages || pg + AF_WARPS == fresh_page);
    if (pg < page_end && !defer0) stage_page(pg, 0);
    if (pg + AF_WARPS < page_end && !defer1) stage_page(pg + AF_WARPS, 1);
    if (wait_dependency) {
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
        asm volatile("griddepcontrol.wait;" ::: "memory");
    }
    if (pg < page_end && defer0) stage_page(pg, 0);
    __pipeline_commit();
    if (pg + AF_WARPS < page_end && defer1) stage_page(pg + AF_WARPS, 1);
    __pipeline_commit();

    for (int i = tid; i < G * HD; i += THREADS) sm.q[i / HD][i % HD] = __ldcg(a.q + (uint64_t)seq * a.n_head * HD + (uint64_t)head0 * HD + i);
    __syncthreads();

    // A fragments of q: row gid holds the rounded q of head gid, row gid + 4 (or + 8) its remainder
    const int my_head = LO8 ? gid : (gid & 3);
    const bool head_ok = my_head < G;
    const bool lo_row = !LO8 && gid >= 4;
    uint32_t qa[KS][LO8 ? 4 : 2];
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
        const float *qh = sm.q[head_ok ? my_head : 0];
        const float x0 = qh[16 * ks + tig * 2], x1 = qh[16 * ks + tig * 2 + 1], x2 = qh[16 * ks + 8 + tig * 2], x3 = qh[16 * ks + 8 + tig * 2 + 1];
        if constexpr (LO8) {
            qa[ks][0] = pack_half2(x0, x1);
            qa[ks][1] = pack_half2_rest(x0, x1);
            qa[ks][2] = pack_half2(x2, x3);
            qa[ks][3] = pack_half2_rest(x2, x3);
        } else {
            qa[ks][0] = !head_ok ? 0u : (lo_row ? pack_half2_rest(x0, x1) : pack_half2(x0, x1));
            qa[ks][1] = !head_ok ? 0u : (lo_row ? pack_half2_rest(x2, x3) : pack_half2(x2, x3));
        }
    }

    float o[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f;
    float m_run = -INFINITY, l_run = 0.0f;  // of head my_head, the same in the lanes that share it

    int slot = 0;
    for (; pg < page_end; pg += AF_WARPS, slot ^= 1) {
        __pipeline_wait_prior(1);
        __syncwarp();
        const uint32_t kb = kv_base + slot * SLOT_BYTES, vb = kb + HALF_BYTES;
        const uint32_t pos0 = pg * KV_PAGE;
        // ---- scores of the 16 tokens: two n-tiles of 8 tokens
        float sv[2][2];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int kk = 0; kk < KS / 2; ++kk) {
                uint32_t b0, b1, b2, b3;  // token rows 8 nt .., dims 32 kk + 8 * (lane / 8) ..
                ldmatrix_x4(kb + (8 * nt + (lane & 7)) * ROW + (32 * kk + 8 * (lane >> 3)) * 2, b0, b1, b2, b3);
                if constexpr (LO8) {
                    mma_16816(c, qa[2 * kk][0], qa[2 * kk][1], qa[2 * kk][2], qa[2 * kk][3], b0, b1);
                    mma_16816(c, qa[2 * kk + 1][0], qa[2 * kk + 1][1], qa[2 * kk + 1][2], qa[2 * kk + 1][3], b2, b3);
                } else {
                    mma_16816(c, qa[2 * kk][0], 0u, qa[2 * kk][1], 0u, b0, b1);
                    mma_16816(c, qa[2 * kk + 1][0], 0u, qa[2 * kk + 1][1], 0u, b2, b3);
                }
            }
            float s0, s1;  // rounded part + remainder part
            if constexpr (LO8) {
                s0 = c[0] + c[2];
                s1 = c[1] + c[3];
            } else {
                s0 = c[0] + __shfl_xor_sync(0xffffffffu, c[0], 16);
                s1 = c[1] + __shfl_xor_sync(0xffffffffu, c[1], 16);
            }
            const uint32_t t0 = pos0 + 8 * nt + tig * 2;
            sv[nt][0] = head_ok && t0 < n_pos ? __fmul_rn(s0, a.scale) : -INFINITY;
            sv[nt][1] = head_ok && t0 + 1 < n_pos ? __fmul_rn(s1, a.scale) : -INFINITY;
        }
        // ---- online softmax: the four lanes of a group hold the head's 16 scores
        float mx = fmaxf(fmaxf(sv[0][0], sv[0][1]), fmaxf(sv[1][0], sv[1][1]));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run, mx);
        float pv[2][2], sum = 0.0f;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                pv[nt][e] = sv[nt][e] == -INFINITY ? 0.0f : expf(sv[nt][e] - m_new);
                sum += pv[nt][e];
            }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        const float al = m_run == -INFINITY ? 0.0f : expf(m_run - m_new);
        l_run = __fmaf_rn(l_run, al, sum);
        m_run = m_new;
        // ---- output: A = probabilities (rounded and remainder rows), B = V through transposing loads
        uint32_t pa[4];
        if constexpr (LO8) {
            pa[0] = pack_half2(pv[0][0], pv[0][1]);
            pa[1] = pack_half2_rest(pv[0][0], pv[0][1]);
            pa[2] = pack_half2(pv[1][0], pv[1][1]);
            pa[3] = pack_half2_rest(pv[1][0], pv[1][1]);
        } else {
            pa[0] = lo_row ? pack_half2_rest(pv[0][0], pv[0][1]) : pack_half2(pv[0][0], pv[0][1]);
            pa[1] = 0u;
            pa[2] = lo_row ? pack_half2_rest(pv[1][0], pv[1][1]) : pack_half2(pv[1][0], pv[1][1]);
            pa[3] = 0u;
        }
        if (__any_sync(0xffffffffu, al != 1.0f)) {
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                o[j][0] *= al;
                o[j][1] *= al;
                o[j][2] *= al;
                o[j][3] *= al;
            }
        }
#pragma unroll
        for (int j = 0; j < NT / 2; ++j) {
            uint32_t b0, b1, b2, b3;  // tokens (lane & 7) + 8 * ((lane >> 3) & 1), dims 16 j + 8 * (lane >> 4) ..
            ldmatrix_x4_trans(vb + ((lane & 7) + 8 * ((lane >> 3) & 1)) * ROW + (16 * j + 8 * (lane >> 4)) * 2, b0, b1, b2, b3);
            mma_16816(o[2 * j], pa[0], pa[1], pa[2], pa[3], b0, b1);
            mma_16816(o[2 * j + 1], pa[0], pa[1], pa[2], pa[3], b2, b3);
        }
        __syncwarp();
        if (pg + 2 * AF_WARPS < page_end) stage_page(pg + 2 * AF_WARPS, slot);
        __pipeline_commit();
    }
    __pipeline_wait_prior(0);

    // ---- the warps' partials meet in shared memory (rounded-row part + remainder-row part)
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        float v0, v1;
        if constexpr (LO8) {
            v0 = o[j][0] + o[j][2];
            v1 = o[j][1] + o[j][3];
        } else {
            v0 = o[j][0] + __shfl_xor_sync(0xffffffffu, o[j][0], 16);
            v1 = o[j][1] + __shfl_xor_sync(0xffffffffu, o[j][1], 16);
        }
        if (head_ok && !lo_row) *reinterpret_cast<float2 *>(&sm.wo[warp][my_head][8 * j + tig * 2]) = make_float2(v0, v1);
    }
    if (head_ok && !lo_row && tig == 0) {
        sm.wm[warp][my_head] = m_run;
        sm.wl[warp][my_head] = l_run;
    }
    __syncthreads();
    for (int i = tid; i < G * HD; i += THREADS) {
        const int g = i / HD, d = i % HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < AF_WARPS; ++w) M = fmaxf(M, sm.wm[w][g]);
        float acc = 0.0f, l = 0.0f;
#pragma unroll
        for (int w = 0; w < AF_WARPS; ++w) {
            const float mw = sm.wm[w][g];
            const float sc = mw == -INFINITY ? 0.0f : expf(mw - M);
            acc = __fmaf_rn(sc, sm.wo[w][g][d], acc);
            l = __fmaf_rn(sc, sm.wl[w][g], l);
        }
        const uint64_t slot_index = ((uint64_t)seq * a.n_head + head0 + g) * a.n_splits + split;
        a.part_o[slot_index * HD + d] = acc;
        if (d == 0) {
            a.part_ml[slot_index * 2] = M;
            a.part_ml[slot_index * 2 + 1] = l;
        }
    }
    // ---- who is last for this (sequence, kv head)?
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const uint32_t done = atomicAdd(&a.counters[seq * a.n_head_kv + kvh], 1u);
        sm.is_last = done == a.n_splits - 1;
        if (sm.is_last) a.counters[seq * a.n_head_kv + kvh] = 0;  // ready for the next launch
    }
    __syncthreads();
    if (!sm.is_last) return;
    __threadfence();

    // ---- merge of all splits.  First every split's weight exp(m_s - M) / (sum of weighted l) per head, in shared memory
    // then the threads sum 16-byte pieces of the partials, each thread its share
    // of the splits with all its loads in flight together.
    float *wgt = &sm.wgt[0][0];   // [G][64], n_splits <= 64
    float4 *acc_area = sm.acc_part;  // [PARTS][NCH]
    for (int g = warp; g < G; g += AF_WARPS) {  // one warp per head
        const float *pm = a.part_ml + ((uint64_t)seq * a.n_head + head0 + g) * a.n_splits * 2;
        float ms[2], ls[2], M = -INFINITY;
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const uint32_t s = lane + 32 * r;
            ms[r] = s < a.n_splits ? __ldcg(pm + 2 * s) : -INFINITY;
            ls[r] = s < a.n_splits ? __ldcg(pm + 2 * s + 1) : 0.0f;
            M = fmaxf(M, ms[r]);
        }
        M = warp_max(M);
        float w[2], l = 0.0f;
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            w[r] = ms[r] == -INFINITY ? 0.0f : expf(ms[r] - M);
            l = __fmaf_rn(w[r], ls[r], l);
        }
        l = warp_sum(l);
        const float inv_l = l > 0.0f ? __fdiv_rn(1.0f, l) : 0.0f;
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const uint32_t s = lane + 32 * r;
            if (s < a.n_splits) wgt[g * 64 + s] = w[r] * inv_l;
        }
    }
    __syncthreads();
    constexpr int NCH = G * HD / 4;                             // 16-byte pieces of the kv head's output
    constexpr int PARTS = THREADS / NCH > 0 ? THREADS / NCH : 1;  // threads per piece, each taking every PARTS-th split
    constexpr int ROUNDS = NCH > THREADS ? NCH / THREADS : 1;
    static_assert(NCH % 32 == 0 && (THREADS % NCH == 0 || NCH % THREADS == 0), "unsupported head shape");
    float4 res[ROUNDS];
#pragma unroll
    for (int rd = 0; rd < ROUNDS; ++rd) {
        const int c = tid % NCH + rd * THREADS, part = tid / NCH;  // part < PARTS
        const int g = c / (HD / 4), d4 = c % (HD / 4);
        const float4 *po = reinterpret_cast<const float4 *>(a.part_o + ((uint64_t)seq * a.n_head + head0 + g) * a.n_splits * HD) + d4;
        float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        for (uint32_t s0 = part; s0 < a.n_splits; s0 += 8 * PARTS) {
            float4 v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const uint32_t s = s0 + u * PARTS;
                v[u] = s < a.n_splits ? __ldcg(po + (uint64_t)s * (HD / 4)) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const uint32_t s = s0 + u * PARTS;
                const float w = s < a.n_splits ? wgt[g * 64 + s] : 0.0f;
                acc.x = __fmaf_rn(w, v[u].x, acc.x);
                acc.y = __fmaf_rn(w, v[u].y, acc.y);
                acc.z = __fmaf_rn(w, v[u].z, acc.z);
                acc.w = __fmaf_rn(w, v[u].w, acc.w);
            }
        }
        if (PARTS > 1) {
            acc_area[part * NCH + c] = acc;
            __syncthreads();
            if (part == 0) {
#pragma unroll
                for (int pp = 1; pp < PARTS; ++pp) {
                    const float4 o2 = acc_area[pp * NCH + c];
                    acc.x += o2.x;
                    acc.y += o2.y;
                    acc.z += o2.z;
                    acc.w += o2.w;
                }
            }
        }
        res[rd] = acc;
        if (part == 0) *reinterpret_cast<float4 *>(a.out + (uint64_t)seq * a.n_head * HD + (uint64_t)(head0 + g) * HD + 4 * d4) = acc;
    }
    if (a.image == nullptr) return;
    if constexpr (G * HD % 256 == 0) {
        // quantize per 256 (engine/vecdot.rs:3030-3053): piece c of this kv head holds elements head0 * HD + 4 c .. + 3 of
        // the row, so a 256-block is 64 consecutive pieces = two warps of the threads with part == 0.
        const uint32_t nb_row = a.n_head * HD / 256;
        uint8_t *img = a.image;
        float *sd = reinterpret_cast<float *>(img + nb_row * 272);
        int16_t *bsum = reinterpret_cast<int16_t *>(img + ((nb_row * 272 + nb_row * 4 + 15) & ~15u));
        int16_t *sum16 = bsum + nb_row * 8;
#pragma unroll
        for (int rd = 0; rd < ROUNDS; ++rd) {
            const int c = tid % NCH + rd * THREADS;
            const bool active = tid / NCH == 0;
            const float4 v = res[rd];
            float amax = active ? fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))) : 0.0f;
            amax = warp_max(amax);
            __syncthreads();
            if (lane == 0) sm.red[warp] = amax;
            __syncthreads();
            amax = fmaxf(sm.red[warp & ~1], sm.red[warp | 1]);
            if (active) {
                const float scale = __fdiv_rn(amax, 127.0f);
                const float inv = scale > 0.0f ? __fdiv_rn(1.0f, scale) : 0.0f;
                const uint32_t blk = head0 * HD / 256 + c / 64, e = (c % 64) * 4;  // block of the row, first element inside it
                const int q0 = quantize_value(v.x, inv), q1 = quantize_value(v.y, inv), q2 = quantize_value(v.z, inv), q3 = quantize_value(v.w, inv);
                *reinterpret_cast<uint32_t *>(img + blk * 272 + e) = (q0 & 0xff) | ((q1 & 0xff) << 8) | ((q2 & 0xff) << 16) | ((uint32_t)(q3 & 0xff) << 24);
                int s = q0 + q1 + q2 + q3;
                s += __shfl_xor_sync(0xffffffffu, s, 1);
                s += __shfl_xor_sync(0xffffffffu, s, 2);
                if ((lane & 3) == 0) sum16[blk * 16 + e / 16] = (int16_t)s;
                s += __shfl_xor_sync(0xffffffffu, s, 4);
                if ((lane & 7) == 0) bsum[blk * 8 + e / 32] = (int16_t)s;
                if ((c % 64) == 0) sd[blk] = scale;
            }
        }
    }
}

template <int HD, int G, int W>
bool launch_fused_warps(const AttnDecodeArgs &a, bool programmatic, cudaStream_t st) {
    static PerDeviceOnce once;  // one per instantiation
    const size_t smem = sizeof(AttnFusedSmem<HD, G, W>);
    if (once.run([] { return cudaFuncSetAttribute(attn_decode_fused_kernel<HD, G, W>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(AttnFusedSmem<HD, G, W>)); }) !=
        cudaSuccess)
        return false;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(a.n_splits, a.n_head_kv, a.n_seq);
    cfg.blockDim = dim3(W * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = programmatic ? 1 : 0;
    cudaLaunchKernelEx(&cfg, attn_decode_fused_kernel<HD, G, W>, a, programmatic, programmatic && a.n_seq == 1);
    return true;
}

template <int HD, int G>
bool launch_fused_instance(const AttnDecodeArgs &a, bool programmatic, cudaStream_t st) {
    // G * HD must be a multiple of the CTA size and the merge maps one 16-byte piece to a thread: 4 warps need G * HD >= 512
    if (a.small_ctas && G * HD >= 512) return launch_fused_warps<HD, G, 4>(a, programmatic, st);
    return launch_fused_warps<HD, G, 8>(a, programmatic, st);
}

}  // namespace

void launch_attn_decode(const AttnDecodeArgs &a, cudaStream_t st) {
    if (a.n_seq == 0) return;
    const uint32_t group = a.n_head / a.n_head_kv;
    bool done = false;
    if (a.n_head % a.n_head_kv == 0 && a.part_o != nullptr) {
        if (a.head_dim == 128) done = launch_hd<128>(a, group, st);
        else if (a.head_dim == 64) done = launch_hd<64>(a, group, st);
    }
    if (!done) attn_generic_kernel<<<dim3(a.n_head, a.n_seq), 32, 0, st>>>(a);
}


bool launch_attn_decode_fused(const AttnDecodeArgs &a, bool programmatic, cudaStream_t st) {
    if (a.n_seq == 0) return true;
    if (!a.counters || !a.part_o || a.n_head % a.n_head_kv) return false;
    const uint32_t group = a.n_head / a.n_head_kv;
    if (a.head_dim == 128) {
        switch (group) {
        case 1: return launch_fused_instance<128, 1>(a, programmatic, st);
        case 2: return launch_fused_instance<128, 2>(a, programmatic, st);
        case 4: return launch_fused_instance<128, 4>(a, programmatic, st);
        case 8: return launch_fused_instance<128, 8>(a, programmatic, st);
        default: return false;
        }
    }
    if (a.head_dim == 64) {
        switch (group) {
        case 2: return launch_fused_instance<64, 2>(a, programmatic, st);
        case 4: return launch_fused_instance<64, 4>(a, programmatic, st);
        case 8: return launch_fused_instance<64, 8>(a, programmatic, st);
        default: return false;
        }
    }
    return false;
}

}  // namespace ob

// ====================================================================================================
// Prefill attention: the rows are consecutive tokens of ONE sequence (a prefill chunk), so all of them attend to the same
// pages.  A CTA takes 16 tokens x the G query heads of one kv head -- warp g holds the 16 x head_dim queries of head g as
// A fragments -- and walks the causal window in tiles of 64 positions (four pages, staged once per CTA in a two-stage
// cp.async ring): S = Q K^T and O += P V through mma.sync.m16n8k16 (f16 x f16 -> f32) with Q and P entered as a rounded
// fp16 part plus its fp16 remainder (two instructions per product), which keeps their error near 2^-22 as in the
// decode kernel; K and V are exactly what the cache holds.  Online softmax in registers; token t sees positions
// 0 .. n_pos[t] - 1.  Every K/V byte of the window is read once per 16 tokens instead of once per token.
// (engine/attention.rs:426-549 is the arithmetic; its CPU loop is also parallel over query tokens, :444.)
// ====================================================================================================
namespace ob {

namespace {

constexpr int PF_TOK = 16, PF_TILE = 64;

template <int HD>
struct PrefillSmem {
    static constexpr int ROW = HD * 2 + 16;  // bytes per position: the pad spreads eight rows over all banks
    uint8_t k[2][PF_TILE * ROW];
    uint8_t v[2][PF_TILE * ROW];
};

template <int HD, int G>
__global__ void __launch_bounds__(G * 32) attn_prefill_kernel(AttnDecodeArgs a) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    using Smem = PrefillSmem<HD>;
    Smem &sm = *reinterpret_cast<Smem *>(smem_raw);
    constexpr int ROW = Smem::ROW, THREADS = G * 32, KS = HD / 16, NT = HD / 8;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gid = lane >> 2, tig = lane & 3;
    const uint32_t tok0 = blockIdx.x * PF_TOK, kvh = blockIdx.y, head = kvh * G + warp;
    const uint32_t n_rows = a.n_seq;
    const uint32_t last_row = min(tok0 + PF_TOK, n_rows) - 1;
    const uint32_t pos_end = a.n_pos[last_row];            // the longest window of this CTA's tokens
    const int32_t *table = a.page_tables[tok0];             // one sequence: every row carries the same table
    const uint32_t n_tiles = (pos_end + PF_TILE - 1) / PF_TILE;
    const uint32_t kb_base = (uint32_t)__cvta_generic_to_shared(&sm.k[0][0]), vb_base = (uint32_t)__cvta_generic_to_shared(&sm.v[0][0]);

    auto stage_tile = [&](uint32_t tile, int st) {
        constexpr int CPR = HD / 8;                       // 16-byte chunks per position
        constexpr int CHUNKS = PF_TILE * CPR;
        for (int ch = tid; ch < CHUNKS; ch += THREADS) {
            const uint32_t p = ch / CPR, j = ch % CPR, pos = tile * PF_TILE + p;
            const uint32_t off = st * PF_TILE * ROW + p * ROW + j * 16;
            if (pos >= pos_end) {  // masked for every token of this CTA: zeros, so that probability 0 times V stays 0
                *reinterpret_cast<uint4 *>(&sm.k[0][0] + off) = make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4 *>(&sm.v[0][0] + off) = make_uint4(0, 0, 0, 0);
                continue;
            }
            const uint64_t base = (((uint64_t)table[pos / KV_PAGE] * a.n_head_kv + kvh) * KV_PAGE + pos % KV_PAGE) * HD;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(kb_base + off), "l"(reinterpret_cast<const uint8_t *>(a.k_pool + base) + j * 16) : "memory");
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(vb_base + off), "l"(reinterpret_cast<const uint8_t *>(a.v_pool + base) + j * 16) : "memory");
        }
    };
    stage_tile(0, 0);
    __pipeline_commit();

    // this thread's query rows: tokens tok0 + gid and tok0 + gid + 8 of head `head`; rounded part and remainder
    const uint32_t r0 = tok0 + gid, r1 = tok0 + gid + 8;
    const uint32_t np0 = r0 < n_rows ? a.n_pos[r0] : 0u, np1 = r1 < n_rows ? a.n_pos[r1] : 0u;
    uint32_t qh[KS][4], ql[KS][4];
    {
        const float *q0 = a.q + (uint64_t)min(r0, n_rows - 1) * a.n_head * HD + (uint64_t)head * HD;
        const float *q1 = a.q + (uint64_t)min(r1, n_rows - 1) * a.n_head * HD + (uint64_t)head * HD;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            const float2 x0 = *reinterpret_cast<const float2 *>(q0 + 16 * ks + 2 * tig), x2 = *reinterpret_cast<const float2 *>(q0 + 16 * ks + 8 + 2 * tig);
            const float2 y0 = *reinterpret_cast<const float2 *>(q1 + 16 * ks + 2 * tig), y2 = *reinterpret_cast<const float2 *>(q1 + 16 * ks + 8 + 2 * tig);
            qh[ks][0] = pack_half2(x0.x, x0.y);
            qh[ks][1] = pack_half2(y0.x, y0.y);
            qh[ks][2] = pack_half2(x2.x, x2.y);
            qh[ks][3] = pack_half2(y2.x, y2.y);
            ql[ks][0] = pack_half2_rest(x0.x, x0.y);
            ql[ks][1] = pack_half2_rest(y0.x, y0.y);
            ql[ks][2] = pack_half2_rest(x2.x, x2.y);
            ql[ks][3] = pack_half2_rest(y2.x, y2.y);
        }
    }
    float o[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;

    for (uint32_t tile = 0; tile < n_tiles; ++tile) {
        const int st = (int)(tile & 1);
        if (tile + 1 < n_tiles) stage_tile(tile + 1, st ^ 1);
        __pipeline_commit();
        __pipeline_wait_prior(1);
        __syncthreads();  // tile `tile` has landed for everybody
        const uint32_t kb = kb_base + st * PF_TILE * ROW, vb = vb_base + st * PF_TILE * ROW;
        const uint32_t pos0 = tile * PF_TILE;
        // ---- scores of the 64 positions: eight n-tiles of 8 positions
        float sc[8][4];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int kk = 0; kk < KS / 2; ++kk) {
                uint32_t b0, b1, b2, b3;  // positions 8 nt .., dims 32 kk + 8 * (lane / 8) ..
                ldmatrix_x4(kb + (8 * nt + (lane & 7)) * ROW + (32 * kk + 8 * (lane >> 3)) * 2, b0, b1, b2, b3);
                mma_16816(c, qh[2 * kk][0], qh[2 * kk][1], qh[2 * kk][2], qh[2 * kk][3], b0, b1);
                mma_16816(c, ql[2 * kk][0], ql[2 * kk][1], ql[2 * kk][2], ql[2 * kk][3], b0, b1);
                mma_16816(c, qh[2 * kk + 1][0], qh[2 * kk + 1][1], qh[2 * kk + 1][2], qh[2 * kk + 1][3], b2, b3);
                mma_16816(c, ql[2 * kk + 1][0], ql[2 * kk + 1][1], ql[2 * kk + 1][2], ql[2 * kk + 1][3], b2, b3);
            }
            const uint32_t p = pos0 + 8 * nt + 2 * tig;  // c[0], c[1]: row gid, positions p, p + 1; c[2], c[3]: row gid + 8
            sc[nt][0] = p < np0 ? __fmul_rn(c[0], a.scale) : -INFINITY;
            sc[nt][1] = p + 1 < np0 ? __fmul_rn(c[1], a.scale) : -INFINITY;
            sc[nt][2] = p < np1 ? __fmul_rn(c[2], a.scale) : -INFINITY;
            sc[nt][3] = p + 1 < np1 ? __fmul_rn(c[3], a.scale) : -INFINITY;
        }
        // ---- online softmax: the four lanes of a quad hold a row's 64 scores
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            mx0 = fmaxf(mx0, fmaxf(sc[nt][0], sc[nt][1]));
            mx1 = fmaxf(mx1, fmaxf(sc[nt][2], sc[nt][3]));
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        const float al0 = m0 == -INFINITY ? 0.0f : expf(m0 - mn0), al1 = m1 == -INFINITY ? 0.0f : expf(m1 - mn1);
        float s0 = 0.0f, s1 = 0.0f;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            sc[nt][0] = sc[nt][0] == -INFINITY ? 0.0f : expf(sc[nt][0] - mn0);
            sc[nt][1] = sc[nt][1] == -INFINITY ? 0.0f : expf(sc[nt][1] - mn0);
            sc[nt][2] = sc[nt][2] == -INFINITY ? 0.0f : expf(sc[nt][2] - mn1);
            sc[nt][3] = sc[nt][3] == -INFINITY ? 0.0f : expf(sc[nt][3] - mn1);
            s0 += sc[nt][0] + sc[nt][1];
            s1 += sc[nt][2] + sc[nt][3];
        }
        s0 += __shfl_xor_sync(0xffffffffu, s0, 1);
        s0 += __shfl_xor_sync(0xffffffffu, s0, 2);
        s1 += __shfl_xor_sync(0xffffffffu, s1, 1);
        s1 += __shfl_xor_sync(0xffffffffu, s1, 2);
        l0 = __fmaf_rn(l0, al0, s0);
        l1 = __fmaf_rn(l1, al1, s1);
        m0 = mn0;
        m1 = mn1;
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            o[j][0] *= al0;
            o[j][1] *= al0;
            o[j][2] *= al1;
            o[j][3] *= al1;
        }
        // ---- output: k-steps of 16 positions; the score fragments of n-tiles 2 j2, 2 j2 + 1 are the A fragment
#pragma unroll
        for (int j2 = 0; j2 < 4; ++j2) {
            const uint32_t ph0 = pack_half2(sc[2 * j2][0], sc[2 * j2][1]), ph1 = pack_half2(sc[2 * j2][2], sc[2 * j2][3]);
            const uint32_t ph2 = pack_half2(sc[2 * j2 + 1][0], sc[2 * j2 + 1][1]), ph3 = pack_half2(sc[2 * j2 + 1][2], sc[2 * j2 + 1][3]);
            const uint32_t pl0 = pack_half2_rest(sc[2 * j2][0], sc[2 * j2][1]), pl1 = pack_half2_rest(sc[2 * j2][2], sc[2 * j2][3]);
            const uint32_t pl2 = pack_half2_rest(sc[2 * j2 + 1][0], sc[2 * j2 + 1][1]), pl3 = pack_half2_rest(sc[2 * j2 + 1][2], sc[2 * j2 + 1][3]);
#pragma unroll
            for (int j = 0; j < NT / 2; ++j) {
                uint32_t b0, b1, b2, b3;  // positions 16 j2 + (lane & 7) + 8 * ((lane >> 3) & 1), dims 16 j + 8 * (lane >> 4) ..
                ldmatrix_x4_trans(vb + (16 * j2 + (lane & 7) + 8 * ((lane >> 3) & 1)) * ROW + (16 * j + 8 * (lane >> 4)) * 2, b0, b1, b2, b3);
                mma_16816(o[2 * j], ph0, ph1, ph2, ph3, b0, b1);
                mma_16816(o[2 * j], pl0, pl1, pl2, pl3, b0, b1);
                mma_16816(o[2 * j + 1], ph0, ph1, ph2, ph3, b2, b3);
                mma_16816(o[2 * j + 1], pl0, pl1, pl2, pl3, b2, b3);
            }
        }
        __syncthreads();  // everybody is done with this stage before it is refilled
    }
    __pipeline_wait_prior(0);

    const float i0 = l0 > 0.0f ? __fdiv_rn(1.0f, l0) : 0.0f, i1 = l1 > 0.0f ? __fdiv_rn(1.0f, l1) : 0.0f;
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        if (r0 < n_rows) *reinterpret_cast<float2 *>(a.out + (uint64_t)r0 * a.n_head * HD + (uint64_t)head * HD + 8 * j + 2 * tig) = make_float2(o[j][0] * i0, o[j][1] * i0);
        if (r1 < n_rows) *reinterpret_cast<float2 *>(a.out + (uint64_t)r1 * a.n_head * HD + (uint64_t)head * HD + 8 * j + 2 * tig) = make_float2(o[j][2] * i1, o[j][3] * i1);
    }
}

template <int HD, int G>
bool launch_prefill_instance(const AttnDecodeArgs &a, cudaStream_t st) {
    static PerDeviceOnce once;  // one per instantiation
    if (once.run([] { return cudaFuncSetAttribute(attn_prefill_kernel<HD, G>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(PrefillSmem<HD>)); }) != cudaSuccess) return false;
    attn_prefill_kernel<HD, G><<<dim3((a.n_seq + PF_TOK - 1) / PF_TOK, a.n_head_kv), G * 32, sizeof(PrefillSmem<HD>), st>>>(a);
    return true;
}

}  // namespace

// n_seq rows = consecutive tokens of one sequence (every row's page table is the same); n_pos non-decreasing.
bool launch_attn_prefill(const AttnDecodeArgs &a, cudaStream_t st) {
    if (a.n_seq == 0) return true;
    if (a.n_head % a.n_head_kv) return false;
    const uint32_t group = a.n_head / a.n_head_kv;
    if (a.head_dim == 128) {
        switch (group) {
        case 1: return launch_prefill_instance<128, 1>(a, st);
        case 2: return launch_prefill_instance<128, 2>(a, st);
        case 4: return launch_prefill_instance<128, 4>(a, st);
        case 8: return launch_prefill_instance<128, 8>(a, st);
        default: return false;
        }
    }
    if (a.head_dim == 64) {
        switch (group) {
        case 1: return launch_prefill_instance<64, 1>(a, st);
        case 2: return launch_prefill_instance<64, 2>(a, st);
        case 4: return launch_prefill_instance<64, 4>(a, st);
        case 8: return launch_prefill_instance<64, 8>(a, st);
        default: return false;
        }
    }
    return false;
}

}  // namespace ob

// ====================================================================================================
// Exact-order attention: the reference's CPU loop reproduced operation for operation, so that the
// output equals the CPU's bit for bit (given the same f16 K/V and the same exp).  Three kernels:
//
//   scores   score[h][p] = fold8(q_h . k_p) * scale.  The dot keeps eight running sums, element i going
//            to sum i % 8, folded ((a0+a4)+(a1+a5))+((a2+a6)+(a3+a7)); multiply and add are separate
//            roundings (engine/tensor.rs:393-430).  Positions are independent: any number of CTAs.
//   softmax  max; e_p = exp(score_p - max); sum left to right; e_p / sum (engine/tensor.rs:809-821).
//            The sum is the warp_sequential_sum of seqsum.cuh.  exp is evaluated in double and rounded
//            once to float, which is what the oracle does too; the reference calls its platform's expf.
//   output   out_h[d] = (..((0 + w_0*v_0[d]) + w_1*v_1[d]) + ..), ascending p, multiply and add rounded
//            separately (engine/attention.rs:515-546, engine/tensor.rs:679-681).  One thread per (h, d)
//            carries the chain; the cost is 4 cycles x positions of latency, which is why windows longer
//            than a configurable bound take the flash-decode kernels above instead.
// ====================================================================================================

#include "seqsum.cuh"

namespace ob {

namespace {

constexpr int SC_THREADS = 128;
constexpr int SC_TILE = 64;  // positions per CTA

template <int G>
__global__ void __launch_bounds__(SC_THREADS) attn_scores_kernel(AttnExactArgs a) {
    extern __shared__ float sq[];  // [G][hd]
    const uint32_t tile = blockIdx.x, kvh = blockIdx.y, row = blockIdx.z;
    const uint32_t n_pos = a.n_pos[row];
    const uint32_t p0 = tile * SC_TILE;
    if (p0 >= n_pos) return;
    const uint32_t hd = a.head_dim, head0 = kvh * G;
    for (uint32_t i = threadIdx.x; i < G * hd; i += SC_THREADS) sq[i] = a.q[(uint64_t)row * a.n_head * hd + (uint64_t)head0 * hd + i];
    __syncthreads();
    const int32_t *table = a.page_tables[row];
    const uint32_t j = threadIdx.x & 7, grp = threadIdx.x >> 3;  // 16 groups of 8 lanes
    const uint32_t chunks = hd / 8;
#pragma unroll
    for (int it = 0; it < SC_TILE / 16; ++it) {
        const uint32_t p = p0 + grp + 16 * it;
        const bool live = p < n_pos;  // uniform within a group of 8
        float acc[G];
#pragma unroll
        for (int g = 0; g < G; ++g) acc[g] = 0.0f;
        if (live) {
            const __half *kp = a.k_pool + (((uint64_t)table[p / KV_PAGE] * a.n_head_kv + kvh) * KV_PAGE + p % KV_PAGE) * hd;
            __half kv[32];  // head_dim <= 256: all loads first, so that they overlap
#pragma unroll
            for (uint32_t c = 0; c < 32; ++c)
                if (c < chunks) kv[c] = kp[8 * c + j];
#pragma unroll
            for (uint32_t c = 0; c < 32; ++c) {
                if (c < chunks) {
                    const float kf = __half2float(kv[c]);
#pragma unroll
                    for (int g = 0; g < G; ++g) acc[g] = __fadd_rn(acc[g], __fmul_rn(sq[g * hd + 8 * c + j], kf));
                }
            }
        }
#pragma unroll
        for (int g = 0; g < G; ++g) {
            acc[g] = __fadd_rn(acc[g], __shfl_xor_sync(0xffffffffu, acc[g], 4));
            acc[g] = __fadd_rn(acc[g], __shfl_xor_sync(0xffffffffu, acc[g], 1));
            acc[g] = __fadd_rn(acc[g], __shfl_xor_sync(0xffffffffu, acc[g], 2));
        }
        if (live && j == 0) {
#pragma unroll
            for (int g = 0; g < G; ++g) a.scores[((uint64_t)row * a.n_head + head0 + g) * a.score_stride + p] = __fmul_rn(acc[g], a.scale);
        }
    }
}

// exp(x) correctly rounded to float through double precision
__device__ __forceinline__ float exp_via_double(float x) { return (float)exp((double)x); }

// grid (n_head, n_rows)
__global__ void __launch_bounds__(128) attn_softmax_kernel(AttnExactArgs a) {
    const uint32_t head = blockIdx.x, row = blockIdx.y;
    const uint32_t n_pos = a.n_pos[row];
    float *s = a.scores + ((uint64_t)row * a.n_head + head) * a.score_stride;
    __shared__ float red[4];
    __shared__ float bcast;
    float mx = -INFINITY;
    for (uint32_t p = threadIdx.x; p < n_pos; p += blockDim.x) mx = fmaxf(mx, s[p]);
    mx = warp_max(mx);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
    __syncthreads();
    mx = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
    for (uint32_t p = threadIdx.x; p < n_pos; p += blockDim.x) s[p] = exp_via_double(__fsub_rn(s[p], mx));
    __syncthreads();
    __shared__ SeqSumWorkspace<128> ws;
    const float total = cta_sequential_sum<128>([&](uint32_t i) { return s[i]; }, n_pos, ws);
    if (threadIdx.x == 0) bcast = total;
    __syncthreads();
    const float sum = bcast;
    if (sum > 0.0f)
        for (uint32_t p = threadIdx.x; p < n_pos; p += blockDim.x) s[p] = __fdiv_rn(s[p], sum);
}

// grid (hd / 16, n_head_kv, n_rows), G * 16 threads: thread (g, d) carries out[h][d] = (..((0 + w_0 v_0[d]) + w_1 v_1[d]) + ..).
// The chain reads its operands from shared memory; the CTA brings them there a tile of 2 * threads positions at a time,
// the next tile's global loads in flight while the current tile is being added.
template <int G>
__global__ void __launch_bounds__(G * 16) attn_output_kernel(AttnExactArgs a) {
    constexpr int NT = G * 16, TILE = 2 * NT;
    __shared__ __align__(16) __half sv[2][TILE][16];
    __shared__ __align__(16) float sw[2][G][TILE];
    const uint32_t slice = blockIdx.x, kvh = blockIdx.y, row = blockIdx.z;
    const uint32_t n_pos = a.n_pos[row], hd = a.head_dim;
    const uint32_t tid = threadIdx.x, g = tid >> 4, d = tid & 15;
    const uint32_t head0 = kvh * G;
    const float *w0 = a.scores + ((uint64_t)row * a.n_head + head0) * a.score_stride;
    const int32_t *table = a.page_tables[row];
    const uint32_t n_tiles = (n_pos + TILE - 1) / TILE;

    uint4 rv[4];      // this thread's share of a tile: positions 2 tid, 2 tid + 1, two 16-byte halves each
    float rw[2 * G];  // and weights tid + NT * i of head i / 2 ... see the index below
    auto load_tile = [&](uint32_t t) {
        const uint32_t p0 = t * TILE;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const uint32_t p = p0 + 2 * tid + i;
            if (p < n_pos) {
                const uint4 *src = reinterpret_cast<const uint4 *>(a.v_pool + (((uint64_t)table[p / KV_PAGE] * a.n_head_kv + kvh) * KV_PAGE + p % KV_PAGE) * hd + slice * 16);
                rv[2 * i] = src[0];
                rv[2 * i + 1] = src[1];
            } else {
                rv[2 * i] = rv[2 * i + 1] = make_uint4(0, 0, 0, 0);
            }
        }
#pragma unroll
        for (int i = 0; i < 2 * G; ++i) {  // element (head i / 2, position tid + NT * (i % 2)) of the tile's weights
            const uint32_t p = p0 + tid + NT * (i & 1);
            rw[i] = p < n_pos ? w0[(uint64_t)(i >> 1) * a.score_stride + p] : 0.0f;
        }
    };
    auto store_tile = [&](int buf) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            *reinterpret_cast<uint4 *>(&sv[buf][2 * tid + i][0]) = rv[2 * i];
            *reinterpret_cast<uint4 *>(&sv[buf][2 * tid + i][8]) = rv[2 * i + 1];
        }
#pragma unroll
        for (int i = 0; i < 2 * G; ++i) sw[buf][i >> 1][tid + NT * (i & 1)] = rw[i];
    };

    float o = 0.0f;
    if (n_tiles) {
        load_tile(0);
        store_tile(0);
    }
    __syncthreads();
    for (uint32_t t = 0; t < n_tiles; ++t) {
        const int buf = (int)(t & 1);
        if (t + 1 < n_tiles) load_tile(t + 1);
        const uint32_t cnt = min((uint32_t)TILE, n_pos - t * TILE);
        for (uint32_t p = 0; p < cnt; ++p) o = __fadd_rn(o, __fmul_rn(sw[buf][g][p], __half2float(sv[buf][p][d])));
        if (t + 1 < n_tiles) store_tile(buf ^ 1);
        __syncthreads();
    }
    a.out[(uint64_t)row * a.n_head * hd + (uint64_t)(head0 + g) * hd + slice * 16 + d] = o;
}

template <int G>
void launch_exact_g(const AttnExactArgs &a, cudaStream_t st) {
    const uint32_t tiles = (a.max_pos + SC_TILE - 1) / SC_TILE;
    attn_scores_kernel<G><<<dim3(tiles, a.n_head_kv, a.n_rows), SC_THREADS, (size_t)G * a.head_dim * 4, st>>>(a);
    attn_softmax_kernel<<<dim3(a.n_head, a.n_rows), 128, 0, st>>>(a);
    attn_output_kernel<G><<<dim3(a.head_dim / 16, a.n_head_kv, a.n_rows), G * 16, 0, st>>>(a);
}

}  // namespace

bool attn_exact_supported(uint32_t n_head, uint32_t n_head_kv, uint32_t head_dim) {
    if (n_head % n_head_kv || head_dim % 16) return false;
    const uint32_t g = n_head / n_head_kv;
    return g == 1 || g == 2 || g == 3 || g == 4 || g == 8;
}

void launch_attn_exact(const AttnExactArgs &a, cudaStream_t st) {
    if (a.n_rows == 0) return;
    switch (a.n_head / a.n_head_kv) {
    case 1: launch_exact_g<1>(a, st); break;
    case 2: launch_exact_g<2>(a, st); break;
    case 3: launch_exact_g<3>(a, st); break;
    case 4: launch_exact_g<4>(a, st); break;
    default: launch_exact_g<8>(a, st); break;
    }
}

}  // namespace ob
