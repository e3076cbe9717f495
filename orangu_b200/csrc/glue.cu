// The small fp32 operators around the products: RMSNorm, RoPE + KV append, SwiGLU, residual add,
// repeat penalty and greedy argmax.  Reference arithmetic (paths under src/bin/orangu-server/engine):
//   rmsnorm   tensor.rs:743-749     (v * scale) * w, scale = 1 / sqrt(mean(v^2) + eps)
//   rope      tensor.rs:1162-1176   NORM pairing (2i, 2i+1): (a*cos - b*sin, a*sin + b*cos)
//   kv push   kv_cache.rs:26-32, 756-768   f32 -> f16 round-to-nearest-even
//   swiglu    arch/mod.rs:1099-1105 silu(g) * u, silu(x) = x / (1 + exp(-x))
//   argmax    sampling.rs:336-359   f32::total_cmp order, the last of equal maxima wins
#include "common.cuh"
#include "kernels.h"
#include "seqsum.cuh"

namespace ob {

namespace {

__device__ __forceinline__ uint32_t padded(uint32_t i) { return i + (i >> 4); }

// The squares are added left to right, as the CPU adds them; see seqsum.cuh.
__global__ void __launch_bounds__(512) rmsnorm_kernel(const float *__restrict__ x, const float *__restrict__ w, uint32_t dim, float eps,
                                                      float *__restrict__ out) {
    extern __shared__ float srow[];
    const float *row = x + (uint64_t)blockIdx.x * dim;
    float *orow = out + (uint64_t)blockIdx.x * dim;
    __shared__ float bcast;
    for (uint32_t i = threadIdx.x; i < dim; i += blockDim.x) srow[padded(i)] = row[i];
    __syncthreads();
    __shared__ SeqSumWorkspace<512> ws;
    const float t = cta_sequential_sum<512>([&](uint32_t i) { const float v = srow[padded(i)]; return __fmul_rn(v, v); }, dim, ws);
    if (threadIdx.x == 0) bcast = __fdiv_rn(1.0f, sqrtf(__fadd_rn(__fdiv_rn(t, (float)dim), eps)));
    __syncthreads();
    const float scale = bcast;
    for (uint32_t i = threadIdx.x; i < dim; i += blockDim.x) orow[i] = __fmul_rn(__fmul_rn(srow[padded(i)], scale), w[i]);
}

__global__ void swiglu_kernel(const float *__restrict__ g, const float *__restrict__ u, uint64_t n, float *__restrict__ out) {
    uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float x = g[i];
    float s = __fdiv_rn(x, __fadd_rn(1.0f, (float)exp((double)(-x))));  // exp in double, rounded once (as the oracle)
    out[i] = __fmul_rn(s, u[i]);
}

__global__ void add_kernel(float *__restrict__ a, const float *__restrict__ b, uint64_t n) {
    uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) a[i] = __fadd_rn(a[i], b[i]);
}

// grid (n_tokens); rotates q in place, rotates k and appends k, v to the token's page as f16.
__global__ void __launch_bounds__(256) rope_kv_kernel(RopeKvArgs a) {
    const uint32_t t = blockIdx.x;
    const uint32_t pos = a.positions[t];
    const uint32_t half = a.rope_dim / 2, hd = a.head_dim;
    const float2 *rot = reinterpret_cast<const float2 *>(a.rope_table) + (uint64_t)pos * half;
    float *q = a.q + (uint64_t)t * a.n_head * hd;
    const uint32_t pairs = hd / 2;
    for (uint32_t i = threadIdx.x; i < a.n_head * pairs; i += blockDim.x) {
        const uint32_t h = i / pairs, p = i % pairs;
        if (p < half) {
            const float2 sc = rot[p];  // (sin, cos)
            float2 *e = reinterpret_cast<float2 *>(q + h * hd) + p;
            const float2 v = *e;
            *e = make_float2(__fsub_rn(__fmul_rn(v.x, sc.y), __fmul_rn(v.y, sc.x)), __fadd_rn(__fmul_rn(v.x, sc.x), __fmul_rn(v.y, sc.y)));
        }
    }
    const uint32_t kv_dim = a.n_head_kv * hd;
    const int32_t *table = a.page_tables[t];
    const int32_t page = table[pos / KV_PAGE];
    const uint32_t slot = pos % KV_PAGE;
    const float *k = a.k + (uint64_t)t * kv_dim, *v = a.v + (uint64_t)t * kv_dim;
    for (uint32_t i = threadIdx.x; i < a.n_head_kv * pairs; i += blockDim.x) {
        const uint32_t h = i / pairs, p = i % pairs;
        float2 kk = *(reinterpret_cast<const float2 *>(k + h * hd) + p);
        if (p < half) {
            const float2 sc = rot[p];
            kk = make_float2(__fsub_rn(__fmul_rn(kk.x, sc.y), __fmul_rn(kk.y, sc.x)), __fadd_rn(__fmul_rn(kk.x, sc.x), __fmul_rn(kk.y, sc.y)));
        }
        const float2 vv = *(reinterpret_cast<const float2 *>(v + h * hd) + p);
        const uint64_t o = (((uint64_t)page * a.n_head_kv + h) * KV_PAGE + slot) * hd + 2 * p;
        *reinterpret_cast<__half2 *>(a.k_pool + o) = __floats2half2_rn(kk.x, kk.y);
        *reinterpret_cast<__half2 *>(a.v_pool + o) = __floats2half2_rn(vv.x, vv.y);
    }
}

// The same step for the Qwen-style variants: bias, per-head RMSNorm, either pairing.  One CTA per token; the rows live in
// shared memory between the steps.  The per-head sum of squares is added left to right by one thread per head, as
// rmsnorm_inplace does it (engine/tensor.rs:691-700) -- head_dim is 64..256, so the sequential loop is short.
__global__ void __launch_bounds__(256) qkv_post_kernel(RopeKvArgs a) {
    extern __shared__ float sm[];
    const uint32_t t = blockIdx.x, hd = a.head_dim, half = a.rope_dim / 2;
    const uint32_t q_dim = a.n_head * hd, kv_dim = a.n_head_kv * hd, n_heads = a.n_head + 2 * a.n_head_kv;
    float *sq = sm, *sk = sm + q_dim, *sv = sk + kv_dim, *scale = sv + kv_dim;  // scale[n_head + n_head_kv]
    float *q = a.q + (uint64_t)t * q_dim;
    const float *k = a.k + (uint64_t)t * kv_dim, *v = a.v + (uint64_t)t * kv_dim;
    for (uint32_t i = threadIdx.x; i < q_dim; i += blockDim.x) sq[i] = a.q_bias ? __fadd_rn(q[i], a.q_bias[i]) : q[i];
    for (uint32_t i = threadIdx.x; i < kv_dim; i += blockDim.x) {
        sk[i] = a.k_bias ? __fadd_rn(k[i], a.k_bias[i]) : k[i];
        sv[i] = a.v_bias ? __fadd_rn(v[i], a.v_bias[i]) : v[i];
    }
    __syncthreads();
    if (a.q_norm || a.k_norm) {
        for (uint32_t h = threadIdx.x; h < a.n_head + a.n_head_kv; h += blockDim.x) {
            const bool is_q = h < a.n_head;
            if (is_q ? a.q_norm != nullptr : a.k_norm != nullptr) {
                const float *row = is_q ? sq + h * hd : sk + (h - a.n_head) * hd;
                float sum = 0.0f;
                for (uint32_t i = 0; i < hd; ++i) sum = __fadd_rn(sum, __fmul_rn(row[i], row[i]));
                scale[h] = __fdiv_rn(1.0f, sqrtf(__fadd_rn(__fdiv_rn(sum, (float)hd), a.rms_eps)));
            }
        }
        __syncthreads();
        if (a.q_norm)
            for (uint32_t i = threadIdx.x; i < q_dim; i += blockDim.x) sq[i] = __fmul_rn(__fmul_rn(sq[i], scale[i / hd]), a.q_norm[i % hd]);
        if (a.k_norm)
            for (uint32_t i = threadIdx.x; i < kv_dim; i += blockDim.x) sk[i] = __fmul_rn(__fmul_rn(sk[i], scale[a.n_head + i / hd]), a.k_norm[i % hd]);
        __syncthreads();
    }
    const uint32_t pos = a.positions[t];
    const float2 *rot = reinterpret_cast<const float2 *>(a.rope_table) + (uint64_t)pos * half;
    for (uint32_t i = threadIdx.x; i < (a.n_head + a.n_head_kv) * half; i += blockDim.x) {  // every pair is touched by one thread only
        const uint32_t h = i / half, p = i % half;
        float *head = h < a.n_head ? sq + h * hd : sk + (h - a.n_head) * hd;
        const uint32_t lo = a.neox ? p : 2 * p, hi = a.neox ? p + half : 2 * p + 1;
        const float2 sc = rot[p];  // (sin, cos)
        const float va = head[lo], vb = head[hi];
        head[lo] = __fsub_rn(__fmul_rn(va, sc.y), __fmul_rn(vb, sc.x));
        head[hi] = __fadd_rn(__fmul_rn(va, sc.x), __fmul_rn(vb, sc.y));
    }
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < q_dim; i += blockDim.x) q[i] = sq[i];
    const int32_t page = a.page_tables[t][pos / KV_PAGE];
    const uint32_t slot = pos % KV_PAGE;
    for (uint32_t i = threadIdx.x; i < kv_dim / 2; i += blockDim.x) {
        const uint32_t h = (2 * i) / hd, e = (2 * i) % hd;
        const uint64_t o = (((uint64_t)page * a.n_head_kv + h) * KV_PAGE + slot) * hd + e;
        *reinterpret_cast<__half2 *>(a.k_pool + o) = __floats2half2_rn(sk[2 * i], sk[2 * i + 1]);
        *reinterpret_cast<__half2 *>(a.v_pool + o) = __floats2half2_rn(sv[2 * i], sv[2 * i + 1]);
    }
    (void)n_heads;
}

__global__ void rope_plain_kernel(float *x, uint32_t n_head, uint32_t head_dim, uint32_t rope_dim, const float *__restrict__ sin_cos) {
    const uint32_t half = rope_dim / 2, pairs = head_dim / 2;
    uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_head * pairs) return;
    const uint32_t h = i / pairs, p = i % pairs;
    if (p >= half) return;
    const float sn = sin_cos[2 * p], cs = sin_cos[2 * p + 1];
    float *e = x + h * head_dim + 2 * p;
    const float va = e[0], vb = e[1];
    e[0] = __fsub_rn(__fmul_rn(va, cs), __fmul_rn(vb, sn));
    e[1] = __fadd_rn(__fmul_rn(va, sn), __fmul_rn(vb, cs));
}

// f32::total_cmp as an unsigned key: larger key <=> later in the total order.
__device__ __forceinline__ uint32_t total_order_key(float f) {
    int32_t b = __float_as_int(f);
    b ^= (int32_t)(((uint32_t)(b >> 31)) >> 1);
    return (uint32_t)b ^ 0x80000000u;
}

__global__ void argmax_reset_kernel(unsigned long long *scratch, uint32_t n) {
    uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) scratch[i] = 0ull;
}

// grid (chunks, n_seq).  (key << 32 | index) under max: of equal keys the largest index wins.
__global__ void __launch_bounds__(256) argmax_kernel(ArgmaxArgs a) {
    const uint32_t seq = blockIdx.y;
    const float *l = a.logits + (uint64_t)seq * (a.row_stride ? a.row_stride : a.n_vocab);
    unsigned long long best = 0ull;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < a.n_vocab; i += gridDim.x * blockDim.x) {
        unsigned long long cand = ((unsigned long long)total_order_key(l[i]) << 32) | i;
        best = cand > best ? cand : best;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
        best = other > best ? other : best;
    }
    __shared__ unsigned long long red[8];
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w) best = red[w] > best ? red[w] : best;
        atomicMax(a.scratch + seq, best);
    }
}

__global__ void argmax_finish_kernel(const unsigned long long *scratch, uint32_t *out, uint32_t n) {
    uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = (uint32_t)(scratch[i] & 0xffffffffull);
}

// Tensor parallel: this rank's (key, id) of every row goes, tagged, into every rank's exchange slot; the largest wins.
__global__ void __launch_bounds__(256) argmax_finish_xchg_kernel(const unsigned long long *scratch, uint32_t *out, uint32_t n, uint32_t index_base,
                                                                 obtp::PeerXchg px) {
    const uint32_t k = *reinterpret_cast<const volatile uint32_t *>(px.seq), tag = k + 1u;
    const uint64_t base = (uint64_t)((k & 1u) * px.size) * px.n;
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
        const unsigned long long best = scratch[i];
        const uint32_t key = (uint32_t)(best >> 32), id = (uint32_t)best + index_base;
        for (uint32_t r = 0; r < px.size; ++r)
            asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(px.slots[r] + base + (uint64_t)px.rank * px.n + 2 * i), "r"(key), "r"(tag), "r"(id),
                         "r"(tag)
                         : "memory");
    }
    unsigned long long t0;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    const uint2 *mine = px.slots[px.rank] + base;
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
        unsigned long long best = 0ull;
        bool gave_up = false;
        for (uint32_t r = 0; r < px.size; ++r) {
            const uint2 *src = mine + (uint64_t)r * px.n + 2 * i;
            uint4 w;
            for (uint32_t spin = 0;; ++spin) {
                asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(w.x), "=r"(w.y), "=r"(w.z), "=r"(w.w) : "l"(src) : "memory");
                if ((w.y == tag && w.w == tag) || gave_up) break;
                if ((spin & 1023u) == 1023u) {
                    unsigned long long t1;
                    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
                    if (t1 - t0 > (unsigned long long)(px.timeout_ms ? px.timeout_ms : 4000u) * 1000000ull) {  // a rank is gone: report, go on with what is there
                        *px.err = 1u;
                        gave_up = true;
                    }
                }
            }
            if (w.y == tag && w.w == tag) {
                const unsigned long long cand = ((unsigned long long)w.x << 32) | w.z;
                best = cand > best ? cand : best;
            }
        }
        out[i] = (uint32_t)best;
    }
    __syncthreads();
    if (threadIdx.x == 0) *px.seq = k + 1u;
}

// One CTA per 8 KB chunk: push this rank's chunk to every peer, announce it, wait for the peers' chunks, add in rank order.
// A CTA pushes before it waits and waits only for words that the peers' CTAs of the same chunk write after their own push, so
// no CTA depends on another CTA of its own grid.  Every wait is bounded (the exchange's time limit -> error word).
__global__ void __launch_bounds__(256) bulk_allreduce_add_kernel(float *__restrict__ x, const float *__restrict__ proj, uint32_t count, obtp::PeerXchg px,
                                                                 obtp::PeerBulk bulk) {
    const uint32_t k = *reinterpret_cast<const volatile uint32_t *>(px.seq), tag = k + 1u, par = k & 1u;
    const uint32_t c = blockIdx.x, o = c * obtp::kBulkChunk, n = min(obtp::kBulkChunk, count - o);  // n is a multiple of 4
    const uint64_t area = (uint64_t)(par * px.size + px.rank) * bulk.cap + o;                        // where this rank's chunk lands, in every region
    // push: 16-byte stores into the peers' landing areas
    float4 mine[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        const uint32_t i = (threadIdx.x + u * 256) * 4;
        mine[u] = i < n ? *reinterpret_cast<const float4 *>(proj + o + i) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (i < n)
            for (uint32_t r = 0; r < px.size; ++r)
                if (r != px.rank) *reinterpret_cast<float4 *>(bulk.data[r] + area + i) = mine[u];
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();  // the CTA's stores (ordered before this thread by the barrier) become visible before the arrival words
        for (uint32_t r = 0; r < px.size; ++r)
            if (r != px.rank)
                asm volatile("st.volatile.global.u32 [%0], %1;" ::"l"(bulk.flags[r] + (uint64_t)(par * px.size + px.rank) * bulk.max_chunks + c), "r"(tag) : "memory");
    }
    // wait for the other ranks' arrival words of this chunk
    if (threadIdx.x < px.size && threadIdx.x != px.rank) {
        const uint32_t *f = bulk.flags[px.rank] + (uint64_t)(par * px.size + threadIdx.x) * bulk.max_chunks + c;
        unsigned long long t0;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
        for (uint32_t spin = 0;; ++spin) {
            uint32_t v;
            asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
            if (v == tag) break;
            if ((spin & 1023u) == 1023u) {
                unsigned long long t1;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
                if (t1 - t0 > (unsigned long long)(px.timeout_ms ? px.timeout_ms : 4000u) * 1000000ull) {  // a rank is gone: report, go on with what is there
                    *px.err = 1u;
                    break;
                }
            }
        }
        __threadfence_system();
    }
    __syncthreads();
    // add in rank order; the landing area is read past L1 (the peers wrote it)
    const float *land = bulk.data[px.rank] + (uint64_t)(par * px.size) * bulk.cap + o;
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        const uint32_t i = (threadIdx.x + u * 256) * 4;
        if (i >= n) continue;
        float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        for (uint32_t r = 0; r < px.size; ++r) {
            const float4 v = r == px.rank ? mine[u] : __ldcg(reinterpret_cast<const float4 *>(land + (uint64_t)r * bulk.cap + i));
            if (r == 0) sum = v;
            else sum = make_float4(__fadd_rn(sum.x, v.x), __fadd_rn(sum.y, v.y), __fadd_rn(sum.z, v.z), __fadd_rn(sum.w, v.w));
        }
        float4 xv = *reinterpret_cast<float4 *>(x + o + i);
        xv = make_float4(__fadd_rn(xv.x, sum.x), __fadd_rn(xv.y, sum.y), __fadd_rn(xv.z, sum.z), __fadd_rn(xv.w, sum.w));
        *reinterpret_cast<float4 *>(x + o + i) = xv;
    }
    // the last CTA to finish closes the exchange
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(bulk.done, 1u) == gridDim.x - 1) {
            *bulk.done = 0u;
            *px.seq = k + 1u;
        }
    }
}

// Sequential on purpose: a token that repeats is penalised once per occurrence, compounding.
__global__ void repeat_penalty_kernel(float *logits, uint32_t n_vocab, const uint32_t *recent, uint32_t n_recent, float penalty) {
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    for (uint32_t i = 0; i < n_recent; ++i) {
        const uint32_t tok = recent[i];
        if (tok < n_vocab) {
            const float v = logits[tok];
            logits[tok] = v > 0.0f ? __fdiv_rn(v, penalty) : __fmul_rn(v, penalty);
        }
    }
}

}  // namespace

void launch_rmsnorm(const float *x, const float *w, uint32_t n_tokens, uint32_t dim, float eps, float *out, cudaStream_t st) {
    if (!n_tokens) return;
    static PerDeviceOnce once;
    if (once.run([] { return cudaFuncSetAttribute(rmsnorm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024); }) != cudaSuccess) return;
    rmsnorm_kernel<<<n_tokens, 512, ((size_t)dim + dim / 16 + 16) * 4, st>>>(x, w, dim, eps, out);
}
void launch_swiglu(const float *gate, const float *up, uint64_t n, float *out, cudaStream_t st) {
    if (n) swiglu_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(gate, up, n, out);
}
void launch_add(float *a, const float *b, uint64_t n, cudaStream_t st) {
    if (n) add_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(a, b, n);
}
void launch_rope_kv(const RopeKvArgs &a, cudaStream_t st) {
    if (!a.n_tokens) return;
    if (!a.q_bias && !a.k_bias && !a.v_bias && !a.q_norm && !a.k_norm && !a.neox) {
        rope_kv_kernel<<<a.n_tokens, 256, 0, st>>>(a);
        return;
    }
    const size_t smem = ((size_t)(a.n_head + 2 * a.n_head_kv) * a.head_dim + a.n_head + a.n_head_kv) * 4;
    static PerDeviceOnce once;
    if (once.run([] { return cudaFuncSetAttribute(qkv_post_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); }) != cudaSuccess) return;
    qkv_post_kernel<<<a.n_tokens, 256, smem, st>>>(a);
}
void launch_rope_plain(float *x, uint32_t n_head, uint32_t head_dim, uint32_t rope_dim, const float *sin_cos_row, cudaStream_t st) {
    uint32_t n = n_head * head_dim / 2;
    rope_plain_kernel<<<(n + 255) / 256, 256, 0, st>>>(x, n_head, head_dim, rope_dim, sin_cos_row);
}
void launch_argmax(const ArgmaxArgs &a, cudaStream_t st) {
    if (!a.n_seq) return;
    argmax_reset_kernel<<<(a.n_seq + 255) / 256, 256, 0, st>>>(a.scratch, a.n_seq);
    dim3 grid(min(64u, (a.n_vocab + 255) / 256), a.n_seq);
    argmax_kernel<<<grid, 256, 0, st>>>(a);
    if (a.px.size > 1) argmax_finish_xchg_kernel<<<1, 256, 0, st>>>(a.scratch, a.out, a.n_seq, a.index_base, a.px);
    else argmax_finish_kernel<<<(a.n_seq + 255) / 256, 256, 0, st>>>(a.scratch, a.out, a.n_seq);
}
void launch_bulk_allreduce_add(float *x, const float *proj, uint32_t count, const obtp::PeerXchg &px, const obtp::PeerBulk &bulk, cudaStream_t st) {
    if (!count) return;
    bulk_allreduce_add_kernel<<<(count + obtp::kBulkChunk - 1) / obtp::kBulkChunk, 256, 0, st>>>(x, proj, count, px, bulk);
}
void launch_repeat_penalty(float *logits, uint32_t n_vocab, const uint32_t *recent, uint32_t n_recent, float penalty, cudaStream_t st) {
    if (n_recent && penalty != 1.0f) repeat_penalty_kernel<<<1, 32, 0, st>>>(logits, n_vocab, recent, n_recent, penalty);
}

}  // namespace ob
