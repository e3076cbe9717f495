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
    static bool configured = false;
    const size_t smem = sizeof(AttnSmem<HD, G>);
    if (!configured) {
        cudaFuncSetAttribute(attn_decode_kernel<HD, G>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        configured = true;
    }
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
            for (uint32_t c = 0; c < chunks; ++c) {
                const float kf = __half2float(kp[8 * c + j]);
#pragma unroll
                for (int g = 0; g < G; ++g) acc[g] = __fadd_rn(acc[g], __fmul_rn(sq[g * hd + 8 * c + j], kf));
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

// grid (hd / 16, n_head_kv, n_rows), G * 16 threads: thread (g, d) carries out[h][d]
template <int G>
__global__ void __launch_bounds__(G * 16) attn_output_kernel(AttnExactArgs a) {
    const uint32_t slice = blockIdx.x, kvh = blockIdx.y, row = blockIdx.z;
    const uint32_t n_pos = a.n_pos[row], hd = a.head_dim;
    const uint32_t g = threadIdx.x >> 4, d = slice * 16 + (threadIdx.x & 15);
    const uint32_t head = kvh * G + g;
    const float *w = a.scores + ((uint64_t)row * a.n_head + head) * a.score_stride;
    const int32_t *table = a.page_tables[row];
    float o = 0.0f;
    for (uint32_t pg = 0; pg * KV_PAGE < n_pos; ++pg) {
        const __half *vp = a.v_pool + ((uint64_t)table[pg] * a.n_head_kv + kvh) * KV_PAGE * hd + d;
        const uint32_t cnt = min((uint32_t)KV_PAGE, n_pos - pg * KV_PAGE);
        float wv[KV_PAGE], vv[KV_PAGE];
#pragma unroll
        for (int t = 0; t < KV_PAGE; ++t) {  // the loads do not depend on the chain: issue them all first
            wv[t] = t < (int)cnt ? w[pg * KV_PAGE + t] : 0.0f;
            vv[t] = t < (int)cnt ? __half2float(vp[(uint32_t)t * hd]) : 0.0f;
        }
#pragma unroll
        for (int t = 0; t < KV_PAGE; ++t)
            if (t < (int)cnt) o = __fadd_rn(o, __fmul_rn(wv[t], vv[t]));
    }
    a.out[(uint64_t)row * a.n_head * hd + (uint64_t)head * hd + d] = o;
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
