// Device-resident Llama-style model: weights, paged fp16 KV pool, forward step and decode graphs.
//
// Reference graph: src/bin/orangu-server/engine/arch/llama.rs:594-932 (run_layers), :1007-1032
// (forward: last-token logits).  Greedy sampling: engine/sampling.rs:336-359.
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <cmath>
#include <map>
#include <vector>

#include "runtime.h"
#include "tp.h"

using namespace obrt;

namespace {

struct LayerDev {
    float *attn_norm = nullptr, *ffn_norm = nullptr;
    float *q_bias = nullptr, *k_bias = nullptr, *v_bias = nullptr, *q_norm = nullptr, *k_norm = nullptr;  // this rank's part; null: absent
    bool variant = false;  // any of the above, or the NEOX pairing: the layer takes the operator-by-operator path
    ob_weight *wq = nullptr, *wk = nullptr, *wv = nullptr, *wo = nullptr, *gate = nullptr, *up = nullptr, *down = nullptr;
};

struct ActPair {  // both granularities for one product input
    ActBuf k, flat;
};

// Per-step metadata, one pinned host block mirrored by one device block.
struct MetaLayout {
    uint32_t T;
    size_t off_tokens, off_positions, off_npos, off_tables, bytes;
    explicit MetaLayout(uint32_t t) : T(t) {
        off_tokens = 0;
        off_positions = off_tokens + (size_t)t * 4;
        off_npos = off_positions + (size_t)t * 4;
        off_tables = (off_npos + (size_t)t * 4 + 15) & ~(size_t)15;
        bytes = off_tables + (size_t)t * 8;
    }
};

__global__ void advance_kernel(uint32_t *tokens, uint32_t *positions, uint32_t *npos, const uint32_t *out_tokens, uint32_t n_seq,
                               uint32_t *history, uint32_t *step_counter) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    const uint32_t step = *step_counter;
    if (i < n_seq) {
        const uint32_t t = out_tokens[i];
        history[(uint64_t)step * n_seq + i] = t;
        tokens[i] = t;
        positions[i] += 1;
        npos[i] += 1;
    }
    __syncthreads();
    if (i == 0) *step_counter = step + 1;
}

// Pages [0, n_pages) of every layer's K and V pools from one sequence's page table to another's: one CTA per (page, layer, K | V).
__global__ void __launch_bounds__(256) copy_pages_kernel(__half *k_pool, __half *v_pool, size_t layer_stride, const int32_t *__restrict__ src_table,
                                                          const int32_t *__restrict__ dst_table, uint32_t page_elems) {
    __half *pool = (blockIdx.z ? v_pool : k_pool) + (size_t)blockIdx.y * layer_stride;
    const uint4 *src = reinterpret_cast<const uint4 *>(pool + (size_t)src_table[blockIdx.x] * page_elems);
    uint4 *dst = reinterpret_cast<uint4 *>(pool + (size_t)dst_table[blockIdx.x] * page_elems);
    for (uint32_t i = threadIdx.x; i < page_elems / 8; i += blockDim.x) dst[i] = src[i];
}

}  // namespace

struct ob_model {
    ob_ctx *ctx = nullptr;
    ob_model_desc cfg{};
    uint32_t tp_rank = 0, tp_size = 1;
    uint32_t n_head_l = 0, n_head_kv_l = 0, n_ff_l = 0, vocab_l = 0, vocab0 = 0;
    std::vector<LayerDev> layers;
    ob_weight *token_embd = nullptr, *output = nullptr;
    float *output_norm = nullptr;
    float *rope_table = nullptr;
    std::vector<void *> owned;  // plain cudaMalloc blocks

    // KV pool: [layer][page][n_head_kv_l][16][head_dim] fp16, K and V
    uint32_t pool_pages = 0;
    __half *k_pool = nullptr, *v_pool = nullptr;
    size_t layer_stride = 0;  // elements
    std::vector<int32_t> free_pages;

    uint32_t T = 0;  // max rows per step
    float *x = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *attn = nullptr, *gate = nullptr, *up = nullptr, *proj = nullptr,
          *logits = nullptr;
    ActPair act_embd, act_attn, act_ff;
    float *part_o = nullptr, *part_ml = nullptr;
    uint32_t *ff_counters = nullptr;    // [n_ff / 256] arrival counters of the SwiGLU outputs, zero between launches
    uint32_t *attn_counters = nullptr;  // [rows][kv heads] arrival counters of the fused attention kernel, zero between launches
    float *norm_scale = nullptr;      // [2] RMSNorm scales for the fused decode kernels (attention norm, FFN / output norm)
    uint8_t *ready_embd = nullptr, *ready_attn = nullptr, *ready_ff = nullptr;  // quantized activations of the single decode token
    float *scores = nullptr;          // exact-order attention scratch [T][n_head_l][score_stride]
    uint32_t score_stride = 0, exact_attn_max_pos = 0;
    uint32_t max_splits = 1;
    size_t row_splits_cap = 0;  // (row, split) pairs part_o / part_ml hold
    uint8_t *d_meta = nullptr, *h_meta = nullptr;
    uint32_t *d_out_tokens = nullptr, *h_out_tokens = nullptr;
    unsigned long long *argmax_scratch = nullptr;
    uint32_t *d_history = nullptr, *d_step_counter = nullptr;
    uint32_t history_cap = 0;
    uint32_t last_T = 0;
    std::map<uint64_t, cudaGraphExec_t> graphs;
    std::map<uint64_t, uint64_t> graph_launches;  // kernels one replay stands for
    obtp::Comm *comm = nullptr;
    obtp::PeerXchg px{};         // size > 1: the single-token step exchanges partials through peer memory instead of NCCL
    obtp::PeerBulk bulk{};       // cap > 0: so do steps of a few rows (decode batches, short prefill chunks)
    bool use_stream = true;  // OB_STREAM_GEMV=0 keeps batch-1 decode on the unfused kernels
    bool stream_ok = false;      // every fused decode kernel of this model's shapes fits (shared memory)
    bool use_fused_attn = true;  // OB_FUSED_ATTN=0 keeps the two-kernel flash-decode
    bool use_prefill_attn = true;  // OB_PREFILL_ATTN=0: prefill chunks take the decode kernel row by row
    bool comm_failed = false;    // a collective could not be enqueued during the last step (reported by check_peer)
    obtp::Rendezvous *rdv = nullptr;  // host-side meeting of the ranks before a step is enqueued (tensor parallel only)
    uint32_t rdv_timeout_ms = 30000;  // OB_TP_RENDEZVOUS_MS; 0 = off
    bool out_of_step = false;         // a rendezvous failed: the ranks no longer run the same sequence of steps
    // Persistent layer kernel (layer_stream.cu): the single-token products between two attention kernels as one launch.
    // Phase list: [q/k/v of layer 0] then per layer [attention-output, gate/up, down, q/k/v of the next layer | output projection].
    bool use_persist = false;    // OB_PERSIST=1; measured slower than one launch per product (barrier waits and the synchronous norm outweigh the launches saved)
    bool persist_ok = false;
    bool launch_failed = false;  // a launch of the persistent kernel was refused (reported after the step)
    std::vector<LsPhase> h_phases;
    LsPhase *d_phases = nullptr;
    LsLayout ls_layout{};
    uint32_t *ls_barriers = nullptr;  // one word per launch of a step, zeroed when the step starts
    uint32_t *ls_status = nullptr;    // set by the kernel when a barrier wait ran out of time
    uint32_t *h_ls_status = nullptr;  // pinned host copy, fetched with every step's results
    uint32_t ls_timeout_ms = 2000;
    bool ls_split = false;            // OB_LS_SPLIT=1: every phase is its own launch
};

struct ob_kv {
    ob_model *m = nullptr;
    uint32_t capacity = 0, len = 0;
    std::vector<int32_t> pages;   // pages held, in position order
    int32_t *d_table = nullptr;   // device copy, room for ceil(capacity / 16) entries
    bool on_demand = false;       // pages are taken from the pool as the sequence grows (ob_kv_create_paged) and go back on truncate
};

namespace {

template <typename Tp>
int dev_alloc(ob_model *m, Tp **out, size_t count) {
    void *p = nullptr;
    OB_CUDA(m->ctx, cudaMalloc(&p, std::max<size_t>(count * sizeof(Tp), 16)));
    m->owned.push_back(p);
    *out = static_cast<Tp *>(p);
    return OB_OK;
}

int upload_f32(ob_model *m, const float *src, size_t n, float **out) {
    int rc = dev_alloc(m, out, n);
    if (rc) return rc;
    OB_CUDA(m->ctx, cudaMemcpyAsync(*out, src, n * 4, cudaMemcpyHostToDevice, m->ctx->stream));
    return OB_OK;
}

int alloc_act(ob_model *m, ActPair *a, uint32_t rows, uint32_t dim) {
    int rc;
    for (ActBuf *b : {&a->k, &a->flat}) {
        const uint32_t grp = b == &a->k ? 256u : 32u;
        if ((rc = dev_alloc(m, &b->q, (size_t)rows * dim))) return rc;
        if ((rc = dev_alloc(m, &b->d, (size_t)rows * (dim / grp + 1)))) return rc;
        if ((rc = dev_alloc(m, &b->sums, (size_t)rows * (dim / 16)))) return rc;
        b->dim_cap = dim;
    }
    return OB_OK;
}

int check_matrix(ob_ctx *ctx, const ob_matrix_desc &d, uint32_t in_dim, uint32_t out_dim, const char *name) {
    if (!d.data) return fail(ctx, OB_ERR_INVALID, std::string("model: ") + name + " has no data");
    if (!type_supported(d.ggml_type)) return fail(ctx, OB_ERR_UNSUPPORTED, std::string("model: ") + name + " has ggml type " + std::to_string(d.ggml_type));
    if (d.in_dim != in_dim || d.out_dim != out_dim)
        return fail(ctx, OB_ERR_INVALID, std::string("model: ") + name + " is [" + std::to_string(d.in_dim) + " -> " + std::to_string(d.out_dim) +
                                             "], expected [" + std::to_string(in_dim) + " -> " + std::to_string(out_dim) + "]");
    if (in_dim % block_elems(d.ggml_type)) return fail(ctx, OB_ERR_UNSUPPORTED, std::string("model: ") + name + ": in_dim is not a whole number of blocks");
    return OB_OK;
}

int slice_weight(ob_model *m, const ob_matrix_desc &d, uint32_t row0, uint32_t n_rows, uint32_t col0, uint32_t n_cols, ob_weight **out) {
    const uint64_t rb = (uint64_t)(d.in_dim / block_elems(d.ggml_type)) * block_bytes_gguf(d.ggml_type);
    return make_weight(m->ctx, d.data, rb, d.ggml_type, d.in_dim, d.out_dim, row0, n_rows, col0, n_cols, out);
}

bool needs_k(std::initializer_list<const ob_weight *> ws) {
    for (auto w : ws)
        if (w->w.type != TYPE_Q8_0) return true;
    return false;
}
bool needs_flat(std::initializer_list<const ob_weight *> ws) {
    for (auto w : ws)
        if (w->w.type == TYPE_Q8_0) return true;
    return false;
}

const ActBuf &act_for(const ActPair &p, const ob_weight *w) { return w->w.type == TYPE_Q8_0 ? p.flat : p.k; }

// Products that share one input: one launch per distinct weight type.
struct ProductOut {
    const ob_weight *w;
    float *y;
    uint32_t y_stride;
    const float *residual;
};

void run_products(ob_model *m, const ActPair &act, std::initializer_list<ProductOut> outs, uint32_t n_tokens, bool gemm_order, cudaStream_t st) {
    std::vector<ProductOut> v(outs);
    std::vector<bool> done(v.size(), false);
    for (size_t i = 0; i < v.size(); ++i) {
        if (done[i]) continue;
        GemvArgs a{};
        a.act = act_for(act, v[i].w);
        a.n_tokens = n_tokens;
        a.gemm_order = gemm_order;
        for (size_t j = i; j < v.size() && a.n_seg < 3; ++j) {
            if (done[j] || v[j].w->w.type != v[i].w->w.type) continue;
            GemvSegment &s = a.seg[a.n_seg++];
            s.w = v[j].w->w;
            s.y = v[j].y;
            s.y_stride = v[j].y_stride;
            s.residual = v[j].residual;
            s.epilogue = v[j].residual ? EPI_ADD_RESIDUAL : EPI_STORE;
            done[j] = true;
        }
        launch_gemv(a, m->ctx->sm_count, st);
        m->ctx->launches += gemv_launches(a.seg[0].w.type, a.seg[0].w.in_dim, n_tokens, gemm_order && a.seg[0].w.type != TYPE_Q8_0);
    }
}

void quantize_into(ob_model *m, int source, const float *x, const float *aux, uint32_t rows, uint32_t dim, const ActPair &dst, bool want_k,
                   bool want_flat, cudaStream_t st) {
    QuantArgs qa{};
    qa.x = x;
    qa.aux = aux;
    qa.eps = m->cfg.rms_eps;
    qa.n_rows = rows;
    qa.dim = dim;
    if (want_k) qa.k = dst.k;
    if (want_flat) qa.flat = dst.flat;
    launch_quantize(source, qa, st);
    m->ctx->launches++;
}

int check_peer(ob_model *m);
int pre_step(ob_model *m);
uint32_t pages_missing(const ob_kv *kv, uint32_t new_len);
int grow_pages(ob_kv *kv, uint32_t new_len);
// Before the synchronisation that ends a step: the persistent kernel's status word comes down with the results.
inline void fetch_status(ob_model *m, cudaStream_t st) {
    if (m->persist_ok) cudaMemcpyAsync(m->h_ls_status, m->ls_status, 4, cudaMemcpyDeviceToHost, st);
}
int build_persistent_phases(ob_model *m);
StreamArgs stream_args(const ob_model *m, uint32_t li, int which);

uint32_t pick_splits(const ob_model *m, uint32_t n_rows) {
    const uint32_t pairs = std::max(1u, n_rows * m->n_head_kv_l);
    uint32_t s = (4u * (uint32_t)m->ctx->sm_count + pairs - 1) / pairs;
    return std::max(1u, std::min(s, m->max_splits));
}

// The fused batch-1 decode kernels of layer li: 1 norm + q/k/v + RoPE + KV append, 2 attention output + residual,
// 3 norm + gate/up + SwiGLU, 4 down + residual, 5 final norm + output projection (li ignored).
StreamArgs stream_args(const ob_model *m, uint32_t li, int which) {
    const ob_model_desc &c = m->cfg;
    const LayerDev &L = m->layers[li];
    const MetaLayout ml(m->T);
    const uint32_t hd = c.head_dim, q_dim = m->n_head_l * hd;
    StreamArgs a{};
    a.eps = c.rms_eps;
    switch (which) {
    case 1:
        a.n_seg = 3;
        a.in_dim = c.n_embd;
        a.prologue = SG_PRO_READY;
        a.ready = m->ready_embd;
        a.seg[0] = StreamSeg{L.wq->w, DevWeight{}, m->q, SG_EP_ROPE_Q};
        a.seg[1] = StreamSeg{L.wk->w, DevWeight{}, nullptr, SG_EP_ROPE_K};
        a.seg[2] = StreamSeg{L.wv->w, DevWeight{}, nullptr, SG_EP_V};
        a.rope_table = m->rope_table;
        a.position = reinterpret_cast<const uint32_t *>(m->d_meta + ml.off_positions);
        a.page_table = reinterpret_cast<const int32_t *const *>(m->d_meta + ml.off_tables);
        a.k_pool = m->k_pool + (size_t)li * m->layer_stride;
        a.v_pool = m->v_pool + (size_t)li * m->layer_stride;
        a.n_head_kv = m->n_head_kv_l;
        a.head_dim = hd;
        a.rope_dim = c.rope_dim;
        break;
    case 2:
        a.n_seg = 1;
        a.in_dim = q_dim;
        a.prologue = SG_PRO_READY;
        a.ready = m->ready_attn;
        a.residual = m->x;
        a.seg[0] = StreamSeg{L.wo->w, DevWeight{}, m->x, SG_EP_RESIDUAL};
        if (m->tp_size > 1) a.seg[0] = StreamSeg{L.wo->w, DevWeight{}, m->proj, SG_EP_STORE};  // this rank's partial; summed over ranks afterwards
        if (m->px.size > 1) {
            a.seg[0].epilogue = SG_EP_XCHG;
            a.px = m->px;
        }
        break;
    case 3:
        a.n_seg = 1;
        a.in_dim = c.n_embd;
        a.prologue = SG_PRO_READY;
        a.ready = m->ready_embd;
        a.seg[0] = StreamSeg{L.gate->w, L.up->w, m->gate, SG_EP_SWIGLU};
        a.out_image = m->ready_ff;
        a.out_counters = m->ff_counters;
        break;
    case 4:
        a.n_seg = 1;
        a.in_dim = m->n_ff_l;
        a.prologue = SG_PRO_READY;
        a.ready = m->ready_ff;
        a.residual = m->x;
        a.seg[0] = StreamSeg{L.down->w, DevWeight{}, m->x, SG_EP_RESIDUAL};
        if (m->tp_size > 1) a.seg[0] = StreamSeg{L.down->w, DevWeight{}, m->proj, SG_EP_STORE};
        if (m->px.size > 1) {
            a.seg[0].epilogue = SG_EP_XCHG;
            a.px = m->px;
        }
        break;
    default:
        a.n_seg = 1;
        a.in_dim = c.n_embd;
        a.prologue = SG_PRO_READY;
        a.ready = m->ready_embd;
        a.seg[0] = StreamSeg{m->output->w, DevWeight{}, m->logits + m->vocab0, SG_EP_STORE};  // this rank's vocabulary rows
        break;
    }
    return a;
}

// The phase list of the persistent layer kernel, when every layer's products take it and the shared memory fits.
int build_persistent_phases(ob_model *m) {
    const ob_model_desc &c = m->cfg;
    auto k_type = [](const ob_weight *w) { return w->w.type == TYPE_Q4_K || w->w.type == TYPE_Q6_K; };
    for (const LayerDev &L : m->layers)
        if (!(k_type(L.wq) && k_type(L.wk) && k_type(L.wv) && k_type(L.wo) && k_type(L.gate) && k_type(L.up) && k_type(L.down) && L.gate->w.type == L.up->w.type))
            return OB_OK;
    if (!k_type(m->output) || (c.head_dim & 1)) return OB_OK;
    uint32_t l2_norm = 8, l2_ready = 2;  // units per warp sent to L2 ahead of the ring (OB_LS_L2_AHEAD overrides both)
    if (const char *e = getenv("OB_LS_L2_AHEAD")) l2_norm = l2_ready = (uint32_t)atoi(e);
    std::vector<LsPhase> ph;
    auto add = [&](uint32_t li, int which) {
        StreamArgs a = stream_args(m, li, which);
        if (which == 1 || which == 3 || which == 5) {  // the norm is the phase's own prologue
            a.prologue = SG_PRO_RMSNORM;
            a.x = m->x;
            a.norm_w = which == 1 ? m->layers[li].attn_norm : which == 3 ? m->layers[li].ffn_norm : m->output_norm;
            a.ready = nullptr;
        }
        LsPhase d;
        if (!layer_stream_phase(a, &d)) return false;
        d.l2_ahead = a.prologue == SG_PRO_RMSNORM ? l2_norm : l2_ready;
        ph.push_back(d);
        return true;
    };
    bool ok = add(0, 1);
    for (uint32_t li = 0; ok && li < c.n_layer; ++li) {
        ok = add(li, 2) && add(li, 3) && add(li, 4);
        if (ok) ok = li + 1 < c.n_layer ? add(li + 1, 1) : add(0, 5);
    }
    if (!ok) return OB_OK;
    const LsLayout L = layer_stream_layout(ph.data(), (uint32_t)ph.size());
    if (!layer_stream_fits(L)) return OB_OK;
    int rc;
    if ((rc = dev_alloc(m, &m->d_phases, ph.size()))) return rc;
    if ((rc = dev_alloc(m, &m->ls_barriers, (size_t)c.n_layer + 2))) return rc;
    if ((rc = dev_alloc(m, &m->ls_status, 4))) return rc;
    OB_CUDA(m->ctx, cudaMemcpy(m->d_phases, ph.data(), ph.size() * sizeof(LsPhase), cudaMemcpyHostToDevice));
    OB_CUDA(m->ctx, cudaMemset(m->ls_barriers, 0, ((size_t)c.n_layer + 2) * 4));
    OB_CUDA(m->ctx, cudaMemset(m->ls_status, 0, 16));
    OB_CUDA(m->ctx, cudaMallocHost(reinterpret_cast<void **>(&m->h_ls_status), 4));
    *m->h_ls_status = 0;
    if (const char *e = getenv("OB_LS_SPLIT")) m->ls_split = e[0] == '1';
    if (const char *e = getenv("OB_LS_TIMEOUT_MS")) m->ls_timeout_ms = (uint32_t)std::max(1, atoi(e));
    m->h_phases = std::move(ph);
    m->ls_layout = L;
    m->persist_ok = true;
    return OB_OK;
}

// Pages an on-demand cache needs before it can hold `new_len` positions (0 for a cache that reserved its pages at creation).
uint32_t pages_missing(const ob_kv *kv, uint32_t new_len) {
    if (!kv->on_demand) return 0;
    const uint32_t need = (new_len + KV_PAGE - 1) / KV_PAGE;
    return need > kv->pages.size() ? need - (uint32_t)kv->pages.size() : 0u;
}

// Takes the missing pages from the pool and appends them to the device table.  The caller has checked that the pool has them.
int grow_pages(ob_kv *kv, uint32_t new_len) {
    const uint32_t n = pages_missing(kv, new_len);
    if (!n) return OB_OK;
    ob_model *m = kv->m;
    const size_t first = kv->pages.size();
    for (uint32_t i = 0; i < n; ++i) {
        kv->pages.push_back(m->free_pages.back());
        m->free_pages.pop_back();
    }
    OB_CUDA(m->ctx, cudaMemcpyAsync(kv->d_table + first, kv->pages.data() + first, (size_t)n * 4, cudaMemcpyHostToDevice, m->ctx->stream));
    OB_CUDA(m->ctx, cudaStreamSynchronize(m->ctx->stream));  // the host vector may reallocate before the copy would otherwise run
    return OB_OK;
}

// Returns true when `image` (the quantized output, for the single-token product kernels) has been written.
// one_sequence: the rows are consecutive tokens of one sequence (a prefill chunk)
bool run_attention(ob_model *m, uint32_t li, uint32_t T, bool exact_attn, uint32_t pos_bound, uint8_t *image, const int32_t *const *d_tables,
                   const uint32_t *d_npos, cudaStream_t st, bool one_sequence = false) {
    const uint32_t hd = m->cfg.head_dim;
    const __half *k_pool = m->k_pool + (size_t)li * m->layer_stride, *v_pool = m->v_pool + (size_t)li * m->layer_stride;
    if (exact_attn) {
        AttnExactArgs at{};
        at.q = m->q;
        at.out = m->attn;
        at.k_pool = k_pool;
        at.v_pool = v_pool;
        at.page_tables = d_tables;
        at.n_pos = d_npos;
        at.scores = m->scores;
        at.score_stride = m->score_stride;
        at.n_rows = T;
        at.n_head = m->n_head_l;
        at.n_head_kv = m->n_head_kv_l;
        at.head_dim = hd;
        at.scale = 1.0f / sqrtf((float)hd);  // llama.rs:823
        at.max_pos = pos_bound;
        launch_attn_exact(at, st);
        m->ctx->launches += 3;
        return false;
    } else {
        AttnDecodeArgs at{};
        at.q = m->q;
        at.out = m->attn;
        at.k_pool = k_pool;
        at.v_pool = v_pool;
        at.page_tables = d_tables;
        at.n_pos = d_npos;
        at.n_seq = T;
        at.n_head = m->n_head_l;
        at.n_head_kv = m->n_head_kv_l;
        at.head_dim = hd;
        at.scale = 1.0f / sqrtf((float)hd);  // llama.rs:823
        at.n_splits = pick_splits(m, T);
        at.part_o = m->part_o;
        at.part_ml = m->part_ml;
        at.max_pos = m->cfg.max_seq_len;
        at.counters = m->attn_counters;
        at.image = image;
        if (one_sequence && T > 1 && m->use_prefill_attn && launch_attn_prefill(at, st)) {  // a prefill chunk: the tiled kernel
            m->ctx->launches += 1;
            return false;
        }
        AttnDecodeArgs fused = at;
        {   // one 8-warp CTA per SM; with at least two (row, kv head) pairs per SM, 4-warp CTAs, two per SM, and the split
            // count that wastes least of the last wave
            const uint32_t pairs = T * m->n_head_kv_l, sms = (uint32_t)m->ctx->sm_count;
            uint32_t best = std::max(1u, sms / pairs);
            fused.small_ctas = pairs >= 2 * sms;
            if (pairs >= sms) {
                const uint32_t slots = fused.small_ctas ? 2 * sms : sms;
                double best_waste = 1e9;
                for (uint32_t s = 1; s <= 4; ++s) {
                    const double waves = (double)pairs * s / slots, waste = (std::ceil(waves) - waves) / std::ceil(waves) + 0.01 * s;
                    if (waste < best_waste) {
                        best_waste = waste;
                        best = s;
                    }
                }
            }
            fused.n_splits = std::max(1u, std::min(m->max_splits, best));
            while (fused.n_splits > 1 && (size_t)T * fused.n_splits > m->row_splits_cap) --fused.n_splits;  // never past the partial buffers
        }
        while (at.n_splits > 1 && (size_t)T * at.n_splits > m->row_splits_cap) --at.n_splits;
        if (m->use_fused_attn && launch_attn_decode_fused(fused, true, st)) {
            m->ctx->launches += 1;
            return image != nullptr && (m->n_head_l / m->n_head_kv_l * hd) % 256 == 0;
        }
        launch_attn_decode(at, st);
        m->ctx->launches += 2;
        return false;
    }
}

// Enqueue one forward step over T rows whose metadata is already in d_meta.
//   gemm_order: the rows are consecutive tokens of one sequence (prefill chunk)
//   logit_row0 / n_logit_rows: which rows get the output projection
//   exact_attn: take the exact-order attention kernels (every row's window <= pos_bound <= exact_attn_max_pos)
void enqueue_step(ob_model *m, uint32_t T, bool gemm_order, uint32_t logit_row0, uint32_t n_logit_rows, bool want_argmax, bool full_logits, bool exact_attn,
                  uint32_t pos_bound, cudaStream_t st) {
    const ob_model_desc &c = m->cfg;
    const MetaLayout ml(m->T);
    const uint32_t *d_tokens = reinterpret_cast<uint32_t *>(m->d_meta + ml.off_tokens);
    const uint32_t *d_positions = reinterpret_cast<uint32_t *>(m->d_meta + ml.off_positions);
    const uint32_t *d_npos = reinterpret_cast<uint32_t *>(m->d_meta + ml.off_npos);
    const int32_t *const *d_tables = reinterpret_cast<const int32_t *const *>(m->d_meta + ml.off_tables);
    const uint32_t n_embd = c.n_embd, hd = c.head_dim;
    const uint32_t q_dim = m->n_head_l * hd, kv_dim = m->n_head_kv_l * hd, n_ff = m->n_ff_l;
    const bool tp = m->tp_size > 1;

    launch_embed(m->token_embd->w, d_tokens, T, m->x, st);
    m->ctx->launches++;

    // Batch-1 decode on one GPU with K-type weights takes the fused streaming kernels (stream_gemv.cu):
    // norm / quantize as prologue, RoPE + KV append, residual and SwiGLU as epilogues, 5 product kernels per layer.
    const bool stream = T == 1 && m->use_stream && m->ready_embd;
    auto k_type = [](const ob_weight *w) { return w->w.type == TYPE_Q4_K || w->w.type == TYPE_Q6_K; };

    // One sequence, one GPU, K-type weights throughout: the products between two attention kernels are one persistent launch
    // (layer_stream.cu) -- a layer is that launch plus the attention kernel.
    if (stream && m->persist_ok && n_logit_rows == 1 && logit_row0 == 0) {
        const uint32_t n_launch = c.n_layer + 1;
        cudaMemsetAsync(m->ls_barriers, 0, (size_t)n_launch * 4, st);
        auto launch = [&](uint32_t first, uint32_t n, uint32_t slot, bool programmatic) {
            if (m->ls_split) {  // one phase per launch (no grid barrier is crossed): isolates the cost of the phases
                for (uint32_t i = 0; i < n; ++i) {
                    if (!launch_layer_stream(m->d_phases + first + i, 1, m->ls_layout, m->ctx->sm_count, m->ls_barriers + slot, m->ls_status, m->ls_timeout_ms, programmatic, st))
                        m->launch_failed = true;
                    m->ctx->launches++;
                }
                return;
            }
            if (!launch_layer_stream(m->d_phases + first, n, m->ls_layout, m->ctx->sm_count, m->ls_barriers + slot, m->ls_status, m->ls_timeout_ms, programmatic, st))
                m->launch_failed = true;
            m->ctx->launches++;
        };
        launch(0, 1, 0, false);
        for (uint32_t li = 0; li < c.n_layer; ++li) {
            if (!run_attention(m, li, T, exact_attn, pos_bound, m->ready_attn, d_tables, d_npos, st)) {
                launch_quant_image(m->attn, q_dim, m->ready_attn, true, st);
                m->ctx->launches++;
            }
            launch(1 + 4 * li, 4, 1 + li, true);
        }
        if (want_argmax) {
            ArgmaxArgs am{};
            am.logits = m->logits;
            am.n_seq = 1;
            am.n_vocab = c.n_vocab;
            am.out = m->d_out_tokens;
            am.scratch = m->argmax_scratch;
            launch_argmax(am, st);
            m->ctx->launches += 3;
        }
        m->last_T = T;
        return;
    }

    // x += sum over ranks of proj for T rows: one kernel through peer memory when the rows fit its landing area, else NCCL + add
    auto reduce_rows = [&](uint32_t rows) {
        const uint64_t count = (uint64_t)rows * n_embd;
        if (m->px.size > 1 && m->bulk.cap && count <= m->bulk.cap && (count & 3) == 0) {
            launch_bulk_allreduce_add(m->x, m->proj, (uint32_t)count, m->px, m->bulk, st);
            m->ctx->launches += 1;
            return;
        }
        if (!obtp::all_reduce_sum(m->comm, m->proj, count, st)) m->comm_failed = true;
        launch_add(m->x, m->proj, count, st);
        m->ctx->launches += 2;
    };
    bool pending_exchange = false;  // a peer exchange has been started and the residual stream does not hold its sum yet
    for (uint32_t li = 0; li < c.n_layer; ++li) {
        const LayerDev &L = m->layers[li];
        const bool stream_layer = stream && m->stream_ok && k_type(L.wq) && k_type(L.wk) && k_type(L.wv) && k_type(L.wo) && k_type(L.gate) && k_type(L.up) &&
                                  k_type(L.down) && L.gate->w.type == L.up->w.type && (hd % 2 == 0) && !L.variant;
        if (stream_layer) {
            const bool peer = tp && m->px.size > 1;
            if (pending_exchange) launch_norm_quant_consume(m->x, L.attn_norm, n_embd, c.rms_eps, nullptr, m->ready_embd, m->px, true, st);
            else launch_norm_quant(m->x, L.attn_norm, n_embd, c.rms_eps, nullptr, m->ready_embd, true, st);
            pending_exchange = false;
            launch_stream_gemv(stream_args(m, li, 1), m->ctx->sm_count, true, st);
            if (!run_attention(m, li, T, exact_attn, pos_bound, m->ready_attn, d_tables, d_npos, st)) {
                launch_quant_image(m->attn, q_dim, m->ready_attn, true, st);
                m->ctx->launches++;
            }
            launch_stream_gemv(stream_args(m, li, 2), m->ctx->sm_count, true, st);
            if (peer) {
                launch_norm_quant_consume(m->x, L.ffn_norm, n_embd, c.rms_eps, nullptr, m->ready_embd, m->px, true, st);
            } else {
                if (tp) {
                    if (!obtp::all_reduce_sum(m->comm, m->proj, n_embd, st)) m->comm_failed = true;
                    launch_add(m->x, m->proj, n_embd, st);
                    m->ctx->launches += 2;
                }
                launch_norm_quant(m->x, L.ffn_norm, n_embd, c.rms_eps, nullptr, m->ready_embd, true, st);
            }
            launch_stream_gemv(stream_args(m, li, 3), m->ctx->sm_count, true, st);
            launch_stream_gemv(stream_args(m, li, 4), m->ctx->sm_count, true, st);
            if (peer) {
                pending_exchange = true;  // completed by the next norm kernel
            } else if (tp) {
                if (!obtp::all_reduce_sum(m->comm, m->proj, n_embd, st)) m->comm_failed = true;
                launch_add(m->x, m->proj, n_embd, st);
                m->ctx->launches += 2;
            }
            m->ctx->launches += 6;
            continue;
        }
        if (pending_exchange) {  // an unfused layer after a fused one: complete the exchange on its own
            launch_norm_quant_consume(m->x, nullptr, n_embd, c.rms_eps, m->norm_scale, nullptr, m->px, true, st);
            m->ctx->launches++;
            pending_exchange = false;
        }
        quantize_into(m, ACT_RMSNORM, m->x, L.attn_norm, T, n_embd, m->act_embd, needs_k({L.wq, L.wk, L.wv}), needs_flat({L.wq, L.wk, L.wv}), st);
        run_products(m, m->act_embd, {{L.wq, m->q, q_dim, nullptr}, {L.wk, m->k, kv_dim, nullptr}, {L.wv, m->v, kv_dim, nullptr}}, T, gemm_order, st);

        RopeKvArgs rk{};
        rk.q = m->q;
        rk.k = m->k;
        rk.v = m->v;
        rk.rope_table = m->rope_table;
        rk.positions = d_positions;
        rk.page_tables = d_tables;
        rk.k_pool = m->k_pool + (size_t)li * m->layer_stride;
        rk.v_pool = m->v_pool + (size_t)li * m->layer_stride;
        rk.n_tokens = T;
        rk.n_head = m->n_head_l;
        rk.n_head_kv = m->n_head_kv_l;
        rk.head_dim = hd;
        rk.rope_dim = c.rope_dim;
        rk.q_bias = L.q_bias;
        rk.k_bias = L.k_bias;
        rk.v_bias = L.v_bias;
        rk.q_norm = L.q_norm;
        rk.k_norm = L.k_norm;
        rk.rms_eps = c.rms_eps;
        rk.neox = c.rope_neox != 0;
        launch_rope_kv(rk, st);
        m->ctx->launches++;

        run_attention(m, li, T, exact_attn, pos_bound, nullptr, d_tables, d_npos, st, gemm_order);

        quantize_into(m, ACT_PLAIN, m->attn, nullptr, T, q_dim, m->act_attn, needs_k({L.wo}), needs_flat({L.wo}), st);
        if (!tp) {
            run_products(m, m->act_attn, {{L.wo, m->x, n_embd, m->x}}, T, gemm_order, st);
        } else {
            run_products(m, m->act_attn, {{L.wo, m->proj, n_embd, nullptr}}, T, gemm_order, st);
            reduce_rows(T);
        }

        quantize_into(m, ACT_RMSNORM, m->x, L.ffn_norm, T, n_embd, m->act_embd, needs_k({L.gate, L.up}), needs_flat({L.gate, L.up}), st);
        run_products(m, m->act_embd, {{L.gate, m->gate, n_ff, nullptr}, {L.up, m->up, n_ff, nullptr}}, T, gemm_order, st);
        quantize_into(m, ACT_SWIGLU, m->gate, m->up, T, n_ff, m->act_ff, needs_k({L.down}), needs_flat({L.down}), st);
        if (!tp) {
            run_products(m, m->act_ff, {{L.down, m->x, n_embd, m->x}}, T, gemm_order, st);
        } else {
            run_products(m, m->act_ff, {{L.down, m->proj, n_embd, nullptr}}, T, gemm_order, st);
            reduce_rows(T);
        }
    }

    // Every rank holds its own columns of the logits.  When only the greedy token is wanted and the ranks share peer memory,
    // each takes the maximum of its columns and the ranks exchange one (key, id) pair per row; otherwise the columns are
    // gathered (the caller wants the logits, or a repeat penalty has to touch them first) and the argmax runs over all of them.
    auto finish_logits = [&](uint32_t rows) {
        const bool pairs_only = tp && want_argmax && !full_logits && m->px.size > 1 && 2 * rows <= m->px.n;
        if (tp && !pairs_only) {
            if (!obtp::all_gather_logits(m->comm, m->logits, rows, c.n_vocab, m->vocab0, m->vocab_l, st)) m->comm_failed = true;
            m->ctx->launches++;
        }
        if (!want_argmax) return;
        ArgmaxArgs am{};
        am.logits = m->logits;
        am.n_seq = rows;
        am.n_vocab = c.n_vocab;
        am.out = m->d_out_tokens;
        am.scratch = m->argmax_scratch;
        if (pairs_only) {
            am.logits = m->logits + m->vocab0;
            am.n_vocab = m->vocab_l;
            am.row_stride = c.n_vocab;
            am.index_base = m->vocab0;
            am.px = m->px;
        }
        launch_argmax(am, st);
        m->ctx->launches += 3;
    };
    if (n_logit_rows == 1 && stream && m->stream_ok && k_type(m->output)) {
        StreamArgs la = stream_args(m, 0, 5);
        if (pending_exchange) launch_norm_quant_consume(m->x, m->output_norm, n_embd, c.rms_eps, nullptr, m->ready_embd, m->px, true, st);
        else launch_norm_quant(m->x + (size_t)logit_row0 * n_embd, m->output_norm, n_embd, c.rms_eps, nullptr, m->ready_embd, true, st);
        pending_exchange = false;
        launch_stream_gemv(la, m->ctx->sm_count, true, st);
        m->ctx->launches += 2;
        finish_logits(1);
    } else if (pending_exchange) {
        launch_norm_quant_consume(m->x, nullptr, n_embd, c.rms_eps, m->norm_scale, nullptr, m->px, true, st);
        m->ctx->launches++;
        pending_exchange = false;
    }
    if (n_logit_rows && !(n_logit_rows == 1 && stream && m->stream_ok && k_type(m->output))) {
        const float *xl = m->x + (size_t)logit_row0 * n_embd;
        quantize_into(m, ACT_RMSNORM, xl, m->output_norm, n_logit_rows, n_embd, m->act_embd, needs_k({m->output}), needs_flat({m->output}), st);
        // Always the single-token kernel: forward() projects one row (llama.rs:1026-1030).
        run_products(m, m->act_embd, {{m->output, m->logits + m->vocab0, c.n_vocab, nullptr}}, n_logit_rows, false, st);
        finish_logits(n_logit_rows);
    }
    m->last_T = T;
}

}  // namespace

extern "C" {

void ob_model_destroy(ob_model *m) {
    if (!m) return;
    ob_ctx *ctx = m->ctx;
    std::lock_guard<std::mutex> g(ctx->mu);
    Bind b(ctx);
    cudaStreamSynchronize(ctx->stream);
    for (auto &kvp : m->graphs) cudaGraphExecDestroy(kvp.second);
    if (m->rdv) obtp::rendezvous_close(m->rdv);
    if (m->comm) obtp::destroy(m->comm);
    auto rel = [&](ob_weight *w) {
        if (w) {
            cudaFree(w->mem);
            delete w;
        }
    };
    for (LayerDev &L : m->layers)
        for (ob_weight *w : {L.wq, L.wk, L.wv, L.wo, L.gate, L.up, L.down}) rel(w);
    if (m->output != m->token_embd) rel(m->output);
    rel(m->token_embd);
    for (void *p : m->owned) cudaFree(p);
    if (m->h_meta) cudaFreeHost(m->h_meta);
    if (m->h_out_tokens) cudaFreeHost(m->h_out_tokens);
    if (m->h_ls_status) cudaFreeHost(m->h_ls_status);
    delete m;
}

int ob_model_create(ob_ctx *ctx, const ob_model_desc *desc, ob_model **out) {
    if (!ctx || !desc || !out) return fail(ctx, OB_ERR_INVALID, "model_create: null argument");
    *out = nullptr;
    const ob_model_desc &c = *desc;
    if (!c.n_layer || !c.n_embd || !c.n_head || !c.n_head_kv || !c.head_dim || !c.n_ff || !c.n_vocab || !c.layers || !c.output_norm)
        return fail(ctx, OB_ERR_INVALID, "model_create: incomplete description");
    if (c.n_head % c.n_head_kv) return fail(ctx, OB_ERR_UNSUPPORTED, "model_create: n_head must be a multiple of n_head_kv");
    if ((c.head_dim & 1) || c.head_dim > 256 || c.rope_dim > c.head_dim || (c.rope_dim & 1))
        return fail(ctx, OB_ERR_UNSUPPORTED, "model_create: head_dim must be even and <= 256, rope_dim even and <= head_dim");
    if (c.n_embd % 32 || c.n_ff % 32) return fail(ctx, OB_ERR_UNSUPPORTED, "model_create: n_embd and n_ff must be multiples of 32");
    const uint32_t tp = std::max(1u, c.tp_size), rank = c.tp_rank;
    if (rank >= tp) return fail(ctx, OB_ERR_INVALID, "model_create: tp_rank >= tp_size");
    if (tp > 1 && (c.n_head_kv % tp || c.n_ff % (tp * 256) || (c.n_head / tp * c.head_dim) % 256 || c.n_vocab % tp))
        return fail(ctx, OB_ERR_UNSUPPORTED, "model_create: tensor-parallel size must divide n_head_kv and n_vocab, and leave n_ff and the head span multiples of 256");
    if (tp > 1 && !c.tp_unique_id) return fail(ctx, OB_ERR_INVALID, "model_create: tp_size > 1 needs tp_unique_id");

    int rc;
    const bool presliced = tp > 1 && c.tp_presliced != 0;
    {  // validate every matrix before touching the device (a presliced description carries the rank's shard shapes)
        const uint32_t ps = presliced ? tp : 1u;
        const uint32_t qd = c.n_head * c.head_dim / ps, kvd = c.n_head_kv * c.head_dim / ps, ffd = c.n_ff / ps;
        if ((rc = check_matrix(ctx, c.token_embd, c.n_embd, c.n_vocab, "token_embd.weight"))) return rc;
        if (c.output.data && (rc = check_matrix(ctx, c.output, c.n_embd, c.n_vocab / ps, "output.weight"))) return rc;
        if (presliced && !c.output.data) return fail(ctx, OB_ERR_INVALID, "model_create: a presliced model needs its output.weight shard (a tied output cannot be cut from the whole token_embd on the device)");
        for (uint32_t i = 0; i < c.n_layer; ++i) {
            const ob_layer_desc &L = c.layers[i];
            if (!L.attn_norm || !L.ffn_norm) return fail(ctx, OB_ERR_INVALID, "model_create: layer norm weights missing");
            if ((rc = check_matrix(ctx, L.wq, c.n_embd, qd, "attn_q.weight"))) return rc;
            if ((rc = check_matrix(ctx, L.wk, c.n_embd, kvd, "attn_k.weight"))) return rc;
            if ((rc = check_matrix(ctx, L.wv, c.n_embd, kvd, "attn_v.weight"))) return rc;
            if ((rc = check_matrix(ctx, L.wo, qd, c.n_embd, "attn_output.weight"))) return rc;
            if ((rc = check_matrix(ctx, L.w_gate, c.n_embd, ffd, "ffn_gate.weight"))) return rc;
            if ((rc = check_matrix(ctx, L.w_up, c.n_embd, ffd, "ffn_up.weight"))) return rc;
            if ((rc = check_matrix(ctx, L.w_down, ffd, c.n_embd, "ffn_down.weight"))) return rc;
        }
    }

    std::unique_lock<std::mutex> g(ctx->mu);
    Bind b(ctx);
    ob_model *m = new ob_model;
    m->ctx = ctx;
    m->cfg = c;
    m->cfg.layers = nullptr;
    m->cfg.output_norm = nullptr;
    m->cfg.tp_unique_id = nullptr;
    m->cfg.rope_freqs = nullptr;
    if (m->cfg.rope_dim == 0) m->cfg.rope_dim = c.head_dim;
    if (m->cfg.max_seq_len == 0) m->cfg.max_seq_len = 4096;
    if (m->cfg.max_batch_tokens == 0) m->cfg.max_batch_tokens = 1;
    if (const char *e = getenv("OB_STREAM_GEMV")) m->use_stream = !(e[0] == '0' && e[1] == 0);
    if (const char *e = getenv("OB_FUSED_ATTN")) m->use_fused_attn = !(e[0] == '0' && e[1] == 0);
    if (const char *e = getenv("OB_PREFILL_ATTN")) m->use_prefill_attn = !(e[0] == '0' && e[1] == 0);
    m->tp_rank = rank;
    m->tp_size = tp;
    m->n_head_l = c.n_head / tp;
    m->n_head_kv_l = c.n_head_kv / tp;
    m->n_ff_l = c.n_ff / tp;
    m->vocab_l = c.n_vocab / tp;
    m->vocab0 = rank * m->vocab_l;
    m->T = m->cfg.max_batch_tokens;
    const uint32_t T = m->T, hd = c.head_dim;
    const uint32_t q_dim = m->n_head_l * hd, kv_dim = m->n_head_kv_l * hd;

    auto bail = [&](int code) {
        g.unlock();
        ob_model_destroy(m);
        return code;
    };

    // ---- weights (sharded: Q/K/V/gate/up/output by rows, Wo/down by input columns)
    m->layers.resize(c.n_layer);
    for (uint32_t i = 0; i < c.n_layer; ++i) {
        const ob_layer_desc &L = c.layers[i];
        LayerDev &D = m->layers[i];
        if ((rc = upload_f32(m, L.attn_norm, c.n_embd, &D.attn_norm))) return bail(rc);
        if ((rc = upload_f32(m, L.ffn_norm, c.n_embd, &D.ffn_norm))) return bail(rc);
        // the optional vectors are always whole; this rank keeps the entries of its own heads
        if (L.q_bias && (rc = upload_f32(m, L.q_bias + (size_t)rank * q_dim, q_dim, &D.q_bias))) return bail(rc);
        if (L.k_bias && (rc = upload_f32(m, L.k_bias + (size_t)rank * kv_dim, kv_dim, &D.k_bias))) return bail(rc);
        if (L.v_bias && (rc = upload_f32(m, L.v_bias + (size_t)rank * kv_dim, kv_dim, &D.v_bias))) return bail(rc);
        if (L.q_norm && (rc = upload_f32(m, L.q_norm, hd, &D.q_norm))) return bail(rc);
        if (L.k_norm && (rc = upload_f32(m, L.k_norm, hd, &D.k_norm))) return bail(rc);
        D.variant = D.q_bias || D.k_bias || D.v_bias || D.q_norm || D.k_norm || c.rope_neox != 0;
        const uint32_t sr = presliced ? 0u : rank;  // a presliced tensor starts at the shard
        if ((rc = slice_weight(m, L.wq, sr * q_dim, q_dim, 0, c.n_embd, &D.wq))) return bail(rc);
        if ((rc = slice_weight(m, L.wk, sr * kv_dim, kv_dim, 0, c.n_embd, &D.wk))) return bail(rc);
        if ((rc = slice_weight(m, L.wv, sr * kv_dim, kv_dim, 0, c.n_embd, &D.wv))) return bail(rc);
        if ((rc = slice_weight(m, L.wo, 0, c.n_embd, sr * q_dim, q_dim, &D.wo))) return bail(rc);
        if ((rc = slice_weight(m, L.w_gate, sr * m->n_ff_l, m->n_ff_l, 0, c.n_embd, &D.gate))) return bail(rc);
        if ((rc = slice_weight(m, L.w_up, sr * m->n_ff_l, m->n_ff_l, 0, c.n_embd, &D.up))) return bail(rc);
        if ((rc = slice_weight(m, L.w_down, 0, c.n_embd, sr * m->n_ff_l, m->n_ff_l, &D.down))) return bail(rc);
    }
    if ((rc = slice_weight(m, c.token_embd, 0, c.n_vocab, 0, c.n_embd, &m->token_embd))) return bail(rc);
    if (c.output.data) {
        if ((rc = slice_weight(m, c.output, presliced ? 0u : m->vocab0, m->vocab_l, 0, c.n_embd, &m->output))) return bail(rc);
    } else if (tp == 1) {
        m->output = m->token_embd;  // tied (llama.rs:133-139)
    } else {
        if ((rc = slice_weight(m, c.token_embd, m->vocab0, m->vocab_l, 0, c.n_embd, &m->output))) return bail(rc);
    }
    if ((rc = upload_f32(m, c.output_norm, c.n_embd, &m->output_norm))) return bail(rc);

    // ---- RoPE table from the host libm, as the reference computes the angles (tensor.rs:1140-1160)
    {
        const uint32_t half = m->cfg.rope_dim / 2, n_pos = m->cfg.max_seq_len;
        std::vector<float> freq(half), tab((size_t)n_pos * half * 2);
        for (uint32_t i = 0; i < half; ++i) {
            freq[i] = powf(c.rope_freq_base, -2.0f * (float)i / (float)m->cfg.rope_dim);
            if (c.rope_freqs) freq[i] /= c.rope_freqs[i];  // tensor.rs:1143-1145
        }
        for (uint32_t p = 0; p < n_pos; ++p)
            for (uint32_t i = 0; i < half; ++i) {
                const float theta = 1.0f * ((float)p * freq[i]);
                tab[((size_t)p * half + i) * 2] = sinf(theta) * 1.0f;
                tab[((size_t)p * half + i) * 2 + 1] = cosf(theta) * 1.0f;
            }
        if ((rc = upload_f32(m, tab.data(), tab.size(), &m->rope_table))) return bail(rc);
        cudaStreamSynchronize(ctx->stream);  // tab goes out of scope
    }

    // ---- KV pool
    {
        const uint64_t tokens = c.kv_pool_tokens ? c.kv_pool_tokens : m->cfg.max_seq_len;
        m->pool_pages = (uint32_t)((tokens + KV_PAGE - 1) / KV_PAGE) + 1;
        m->layer_stride = (size_t)m->pool_pages * m->n_head_kv_l * KV_PAGE * hd;
        if ((rc = dev_alloc(m, &m->k_pool, m->layer_stride * c.n_layer))) return bail(rc);
        if ((rc = dev_alloc(m, &m->v_pool, m->layer_stride * c.n_layer))) return bail(rc);
        cudaMemsetAsync(m->k_pool, 0, m->layer_stride * c.n_layer * 2, ctx->stream);
        cudaMemsetAsync(m->v_pool, 0, m->layer_stride * c.n_layer * 2, ctx->stream);
        m->free_pages.reserve(m->pool_pages);
        for (int32_t p = (int32_t)m->pool_pages - 1; p >= 0; --p) m->free_pages.push_back(p);
    }

    // ---- scratch
    if ((rc = dev_alloc(m, &m->x, (size_t)T * c.n_embd))) return bail(rc);
    if ((rc = dev_alloc(m, &m->q, (size_t)T * q_dim))) return bail(rc);
    if ((rc = dev_alloc(m, &m->k, (size_t)T * kv_dim))) return bail(rc);
    if ((rc = dev_alloc(m, &m->v, (size_t)T * kv_dim))) return bail(rc);
    if ((rc = dev_alloc(m, &m->attn, (size_t)T * q_dim))) return bail(rc);
    if ((rc = dev_alloc(m, &m->gate, (size_t)T * m->n_ff_l))) return bail(rc);
    if ((rc = dev_alloc(m, &m->up, (size_t)T * m->n_ff_l))) return bail(rc);
    if ((rc = dev_alloc(m, &m->proj, (size_t)T * c.n_embd))) return bail(rc);
    if ((rc = dev_alloc(m, &m->logits, (size_t)T * c.n_vocab))) return bail(rc);
    if ((rc = alloc_act(m, &m->act_embd, T, c.n_embd))) return bail(rc);
    if ((rc = alloc_act(m, &m->act_attn, T, q_dim))) return bail(rc);
    if ((rc = alloc_act(m, &m->act_ff, T, m->n_ff_l))) return bail(rc);
    m->max_splits = std::max(1u, std::min(64u, (m->cfg.max_seq_len + 63) / 64));
    {   // rows * pick_splits(rows) never exceeds 4 * SMs + rows; the fused kernel's own rule (run_attention) takes up to
        // four splits per row however many rows there are
        const size_t row_splits = std::max((size_t)4 * ctx->sm_count + T, (size_t)4 * T);
        m->row_splits_cap = row_splits;
        if ((rc = dev_alloc(m, &m->part_o, row_splits * m->n_head_l * hd))) return bail(rc);
        if ((rc = dev_alloc(m, &m->part_ml, row_splits * m->n_head_l * 2))) return bail(rc);
        if ((rc = dev_alloc(m, &m->attn_counters, (size_t)T * m->n_head_kv_l))) return bail(rc);
        OB_CUDA(ctx, cudaMemset(m->attn_counters, 0, (size_t)T * m->n_head_kv_l * 4));
    }
    m->exact_attn_max_pos = attn_exact_supported(m->n_head_l, m->n_head_kv_l, hd) ? std::min(m->cfg.max_seq_len, c.exact_attention_max_pos ? c.exact_attention_max_pos : 1024u) : 0u;
    m->score_stride = (m->exact_attn_max_pos + 63) / 64 * 64;
    if (m->score_stride && (rc = dev_alloc(m, &m->scores, (size_t)T * m->n_head_l * m->score_stride))) return bail(rc);
    if ((rc = dev_alloc(m, &m->norm_scale, 4))) return bail(rc);
    if (c.n_embd % 256 == 0 && (m->n_head_l * c.head_dim) % 256 == 0 && m->n_ff_l % 256 == 0) {
        if ((rc = dev_alloc(m, &m->ready_embd, act_image_bytes(c.n_embd)))) return bail(rc);
        if ((rc = dev_alloc(m, &m->ready_attn, act_image_bytes(m->n_head_l * c.head_dim)))) return bail(rc);
        if ((rc = dev_alloc(m, &m->ready_ff, act_image_bytes(m->n_ff_l)))) return bail(rc);
        if ((rc = dev_alloc(m, &m->ff_counters, m->n_ff_l / 256))) return bail(rc);
        OB_CUDA(ctx, cudaMemset(m->ff_counters, 0, (size_t)m->n_ff_l / 256 * 4));
    }
    const MetaLayout ml(T);
    if ((rc = dev_alloc(m, &m->d_meta, ml.bytes))) return bail(rc);
    if ((rc = dev_alloc(m, &m->d_out_tokens, T))) return bail(rc);
    if ((rc = dev_alloc(m, &m->argmax_scratch, T))) return bail(rc);
    if ((rc = dev_alloc(m, &m->d_step_counter, 4))) return bail(rc);
    if (cudaMallocHost(reinterpret_cast<void **>(&m->h_meta), ml.bytes) != cudaSuccess ||
        cudaMallocHost(reinterpret_cast<void **>(&m->h_out_tokens), (size_t)T * 4) != cudaSuccess)
        return bail(fail(ctx, OB_ERR_OOM, "model_create: pinned host allocation failed"));

    if (tp > 1) {
        std::string err;
        m->comm = obtp::create(c.tp_unique_id, (int)rank, (int)tp, ctx->device, &err);
        if (!m->comm) return bail(fail(ctx, OB_ERR_COMM, "model_create: " + err));
        if (const char *re = getenv("OB_TP_RENDEZVOUS_MS")) m->rdv_timeout_ms = (uint32_t)std::max(0, atoi(re));
        if (m->rdv_timeout_ms) {
            // a node without POSIX shared memory has no meeting point on any rank alike: the guard is then off, not an error
            std::string rerr;
            m->rdv = obtp::rendezvous_open(c.tp_unique_id, (int)rank, (int)tp, &rerr);
        }
        const char *pe = getenv("OB_TP_PEER");
        if (!(pe && pe[0] == '0' && pe[1] == 0) && tp <= 8) {
            std::string perr;
            const uint32_t bulk_rows = std::min<uint32_t>(128u, m->cfg.max_batch_tokens);  // decode batches; longer prefill chunks stay with NCCL
            if (!obtp::peer_init(m->comm, c.n_embd, bulk_rows * c.n_embd, ctx->device, &m->px, &m->bulk, &perr)) {  // no peer access: NCCL all-reduce
                m->px = obtp::PeerXchg{};
                m->bulk = obtp::PeerBulk{};
            }
        }
    }
    cudaError_t e = cudaStreamSynchronize(ctx->stream);
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) return bail(fail(ctx, OB_ERR_CUDA, std::string("model_create: ") + cudaGetErrorString(e)));
    if (m->ready_embd && c.n_layer) {  // do the fused decode kernels cover this model's shapes?
        m->stream_ok = true;
        for (int v = 1; v <= 5; ++v) {
            const StreamArgs sa = stream_args(m, 0, v);
            bool k_types = true;
            for (int sgi = 0; sgi < sa.n_seg; ++sgi) k_types = k_types && (sa.seg[sgi].w.type == TYPE_Q4_K || sa.seg[sgi].w.type == TYPE_Q6_K);
            if (k_types && !stream_gemv_supported(sa)) m->stream_ok = false;
        }
    }
    if (const char *e = getenv("OB_PERSIST")) m->use_persist = e[0] == '1' && e[1] == 0;
    bool any_variant = false;
    for (const LayerDev &D : m->layers) any_variant |= D.variant;
    if (m->stream_ok && m->use_persist && tp == 1 && !any_variant) {
        if ((rc = build_persistent_phases(m))) return bail(rc);
    }
    *out = m;
    return OB_OK;
}

// ------------------------------------------------------------------------------------ KV cache

static int kv_create(ob_model *m, uint32_t capacity_tokens, bool on_demand, ob_kv **out) {
    if (!m || !out || capacity_tokens == 0) return fail(m ? m->ctx : nullptr, OB_ERR_INVALID, "kv_create: bad argument");
    ob_ctx *ctx = m->ctx;
    std::lock_guard<std::mutex> g(ctx->mu);
    *out = nullptr;
    if (capacity_tokens > m->cfg.max_seq_len) return fail(ctx, OB_ERR_CAPACITY, "kv_create: capacity exceeds the model's max_seq_len");
    const uint32_t n_pages = (capacity_tokens + KV_PAGE - 1) / KV_PAGE;
    if (!on_demand && n_pages > m->free_pages.size()) return fail(ctx, OB_ERR_CAPACITY, "kv_create: KV pool exhausted");
    Bind b(ctx);
    ob_kv *kv = new ob_kv;
    kv->m = m;
    kv->capacity = capacity_tokens;
    kv->on_demand = on_demand;
    if (!on_demand)
        for (uint32_t i = 0; i < n_pages; ++i) {
            kv->pages.push_back(m->free_pages.back());
            m->free_pages.pop_back();
        }
    cudaError_t e = cudaMalloc(reinterpret_cast<void **>(&kv->d_table), (size_t)n_pages * 4);
    if (e == cudaSuccess) e = cudaMemsetAsync(kv->d_table, 0, (size_t)n_pages * 4, ctx->stream);
    if (e == cudaSuccess && !kv->pages.empty()) e = cudaMemcpyAsync(kv->d_table, kv->pages.data(), kv->pages.size() * 4, cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) {
        for (int32_t p : kv->pages) m->free_pages.push_back(p);
        if (kv->d_table) cudaFree(kv->d_table);
        delete kv;
        return fail(ctx, OB_ERR_CUDA, std::string("kv_create: ") + cudaGetErrorString(e));
    }
    *out = kv;
    return OB_OK;
}

int ob_kv_create(ob_model *m, uint32_t capacity_tokens, ob_kv **out) { return kv_create(m, capacity_tokens, false, out); }
int ob_kv_create_paged(ob_model *m, uint32_t capacity_tokens, ob_kv **out) { return kv_create(m, capacity_tokens, true, out); }

void ob_kv_destroy(ob_kv *kv) {
    if (!kv) return;
    ob_ctx *ctx = kv->m->ctx;
    std::lock_guard<std::mutex> g(ctx->mu);
    Bind b(ctx);
    cudaStreamSynchronize(ctx->stream);
    for (int32_t p : kv->pages) kv->m->free_pages.push_back(p);
    cudaFree(kv->d_table);
    delete kv;
}

uint32_t ob_kv_len(const ob_kv *kv) { return kv ? kv->len : 0; }

uint32_t ob_kv_pages(const ob_kv *kv) {
    if (!kv) return 0;
    std::lock_guard<std::mutex> g(kv->m->ctx->mu);
    return (uint32_t)kv->pages.size();
}

uint32_t ob_model_free_pages(const ob_model *m) {
    if (!m) return 0;
    std::lock_guard<std::mutex> g(m->ctx->mu);
    return (uint32_t)m->free_pages.size();
}

uint32_t ob_model_pool_pages(const ob_model *m) { return m ? (uint32_t)m->pool_pages : 0u; }
uint32_t ob_model_n_vocab(const ob_model *m) { return m ? m->cfg.n_vocab : 0u; }
uint32_t ob_model_tp_size(const ob_model *m) { return m ? std::max(1u, m->tp_size) : 0u; }
ob_ctx *ob_model_ctx(const ob_model *m) { return m ? m->ctx : nullptr; }

int ob_kv_truncate(ob_kv *kv, uint32_t new_len) {
    if (!kv) return OB_ERR_INVALID;
    std::lock_guard<std::mutex> g(kv->m->ctx->mu);
    if (new_len > kv->len) return fail(kv->m->ctx, OB_ERR_INVALID, "kv_truncate: new_len exceeds the current length");
    kv->len = new_len;
    if (kv->on_demand) {  // whole pages past the new length go back to the pool (the device table keeps stale ids nobody reads)
        const size_t keep = (new_len + KV_PAGE - 1) / KV_PAGE;
        while (kv->pages.size() > keep) {
            kv->m->free_pages.push_back(kv->pages.back());
            kv->pages.pop_back();
        }
    }
    return OB_OK;
}

int ob_kv_read(ob_kv *kv, uint32_t layer, uint32_t pos0, uint32_t n, float *k_out, float *v_out) {
    if (!kv || !k_out || !v_out) return OB_ERR_INVALID;
    ob_model *m = kv->m;
    ob_ctx *ctx = m->ctx;
    std::lock_guard<std::mutex> g(ctx->mu);
    if (layer >= m->cfg.n_layer || (uint64_t)pos0 + n > kv->len) return fail(ctx, OB_ERR_INVALID, "kv_read: out of range");
    Bind b(ctx);
    const uint32_t hd = m->cfg.head_dim, nkv = m->n_head_kv_l, kv_dim = nkv * hd;
    std::vector<__half> page((size_t)nkv * KV_PAGE * hd);
    for (int which = 0; which < 2; ++which) {
        const __half *pool = (which ? m->v_pool : m->k_pool) + (size_t)layer * m->layer_stride;
        float *dst = which ? v_out : k_out;
        int32_t loaded = -1;
        for (uint32_t p = pos0; p < pos0 + n; ++p) {
            const int32_t pg = kv->pages[p / KV_PAGE];
            if (pg != loaded) {
                OB_CUDA(ctx, cudaMemcpyAsync(page.data(), pool + (size_t)pg * page.size(), page.size() * 2, cudaMemcpyDeviceToHost, ctx->stream));
                OB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
                loaded = pg;
            }
            for (uint32_t h = 0; h < nkv; ++h)
                for (uint32_t d = 0; d < hd; ++d)
                    dst[(size_t)(p - pos0) * kv_dim + h * hd + d] = __half2float(page[((size_t)h * KV_PAGE + p % KV_PAGE) * hd + d]);
        }
    }
    return OB_OK;
}

int ob_kv_copy_prefix(ob_kv *dst, const ob_kv *src, uint32_t n) {
    if (!dst || !src || dst->m != src->m) return OB_ERR_INVALID;
    ob_model *m = dst->m;
    ob_ctx *ctx = m->ctx;
    std::lock_guard<std::mutex> g(ctx->mu);
    if (dst->len != 0) return fail(ctx, OB_ERR_INVALID, "kv_copy_prefix: the destination is not empty");
    if (n > src->len || n > dst->capacity) return fail(ctx, OB_ERR_CAPACITY, "kv_copy_prefix: n exceeds the source length or the destination capacity");
    if (pages_missing(dst, n) > m->free_pages.size()) return fail(ctx, OB_ERR_CAPACITY, "kv_copy_prefix: KV pool exhausted");
    Bind b(ctx);
    if (int rc = grow_pages(dst, n)) return rc;
    const size_t page_elems = (size_t)m->n_head_kv_l * KV_PAGE * m->cfg.head_dim;  // a multiple of 8 halves: head_dim is even and a page holds 16 tokens
    const uint32_t n_pages = (n + KV_PAGE - 1) / KV_PAGE;
    if (n_pages) {
        copy_pages_kernel<<<dim3(n_pages, m->cfg.n_layer, 2), 256, 0, ctx->stream>>>(m->k_pool, m->v_pool, m->layer_stride, src->d_table, dst->d_table, (uint32_t)page_elems);
        ctx->launches++;
    }
    OB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    dst->len = n;
    return OB_OK;
}

int ob_profile_gemv(ob_model *m, uint32_t ggml_type, uint32_t variant, uint32_t iters, float *ms_total, uint64_t *bytes_per_pass,
                    uint32_t *launches_per_pass) {
    if (!m || !ms_total || variant > 5) return OB_ERR_INVALID;
    ob_ctx *ctx = m->ctx;
    std::lock_guard<std::mutex> g(ctx->mu);
    Bind b(ctx);
    cudaStream_t st = ctx->stream;
    if (variant) {
        if (m->last_T == 0) return fail(ctx, OB_ERR_INVALID, "profile_gemv: run a decode step first (the fused kernels read its position and page table)");
        uint64_t bytes = 0;
        uint32_t launches = 0;
        auto seg_bytes = [](const StreamSeg &sg) {
            uint64_t n = (uint64_t)sg.w.nb * block_bytes_gguf(sg.w.type) * sg.w.out_dim + 4ull * sg.w.out_dim;
            if (sg.w2.data) n += (uint64_t)sg.w2.nb * block_bytes_gguf(sg.w2.type) * sg.w2.out_dim;
            return n;
        };
        launch_norm_quant(m->x, m->output_norm, m->cfg.n_embd, m->cfg.rms_eps, nullptr, m->ready_embd, false, st);
        launch_quant_image(m->attn, m->n_head_l * m->cfg.head_dim, m->ready_attn, false, st);
        launch_quant_image(m->gate, m->n_ff_l, m->ready_ff, false, st);
        for (uint32_t it = 0; it <= iters; ++it) {  // pass 0 is a warm-up
            if (it == 1) OB_CUDA(ctx, cudaEventRecord(ctx->ev0, st));
            const uint32_t n = variant == 5 ? 1u : m->cfg.n_layer;
            for (uint32_t li = 0; li < n; ++li) {
                StreamArgs a = stream_args(m, li, (int)variant);
                if (a.seg[0].epilogue == SG_EP_XCHG) {  // tensor parallel: time the product on this rank's slice; a store into the
                    a.seg[0].epilogue = SG_EP_STORE;     // peers' exchange slots would carry the tag of the next real exchange
                    a.seg[0].y = m->proj;
                    a.px = obtp::PeerXchg{};
                }
                if (!stream_gemv_supported(a)) return fail(ctx, OB_ERR_UNSUPPORTED, "profile_gemv: this model's tensors do not take the fused kernels");
                launch_stream_gemv(a, ctx->sm_count, true, st);
                if (it == 1) {
                    for (int s = 0; s < a.n_seg; ++s) bytes += seg_bytes(a.seg[s]);
                    bytes += 4ull * a.in_dim;
                    launches++;
                }
            }
        }
        OB_CUDA(ctx, cudaEventRecord(ctx->ev1, st));
        OB_CUDA(ctx, cudaStreamSynchronize(st));
        OB_CUDA(ctx, cudaGetLastError());
        cudaEventElapsedTime(ms_total, ctx->ev0, ctx->ev1);
        ctx->launches += (uint64_t)launches * (iters + 1);
        if (bytes_per_pass) *bytes_per_pass = bytes;
        if (launches_per_pass) *launches_per_pass = launches;
        return OB_OK;
    }
    // any finite activations will do: the kernel's work does not depend on the values
    OB_CUDA(ctx, cudaMemsetAsync(m->x, 0, (size_t)m->cfg.n_embd * 4, st));
    OB_CUDA(ctx, cudaMemsetAsync(m->attn, 0, (size_t)m->n_head_l * m->cfg.head_dim * 4, st));
    OB_CUDA(ctx, cudaMemsetAsync(m->gate, 0, (size_t)m->n_ff_l * 4, st));
    quantize_into(m, ACT_PLAIN, m->x, nullptr, 1, m->cfg.n_embd, m->act_embd, true, true, st);
    quantize_into(m, ACT_PLAIN, m->attn, nullptr, 1, m->n_head_l * m->cfg.head_dim, m->act_attn, true, true, st);
    quantize_into(m, ACT_PLAIN, m->gate, nullptr, 1, m->n_ff_l, m->act_ff, true, true, st);
    uint64_t bytes = 0;
    uint32_t launches = 0;
    for (uint32_t it = 0; it <= iters; ++it) {  // pass 0 is a warm-up
        if (it == 1) OB_CUDA(ctx, cudaEventRecord(ctx->ev0, st));
        for (const LayerDev &L : m->layers) {
            struct Item {
                const ob_weight *w;
                const ActPair *act;
                float *y;
            } items[] = {{L.wq, &m->act_embd, m->q}, {L.wk, &m->act_embd, m->k},  {L.wv, &m->act_embd, m->v},   {L.wo, &m->act_attn, m->proj},
                         {L.gate, &m->act_embd, m->gate}, {L.up, &m->act_embd, m->up}, {L.down, &m->act_ff, m->proj}};
            for (const Item &i : items) {
                if (i.w->w.type != ggml_type) continue;
                GemvArgs a{};
                a.n_seg = 1;
                a.seg[0].w = i.w->w;
                a.seg[0].y = i.y;
                a.seg[0].y_stride = i.w->w.out_dim;
                a.seg[0].epilogue = EPI_STORE;
                a.act = act_for(*i.act, i.w);
                a.n_tokens = 1;
                launch_gemv(a, ctx->sm_count, st);
                if (it == 1) {
                    bytes += (uint64_t)i.w->w.nb * block_bytes_gguf(ggml_type) * i.w->w.out_dim + 4ull * (i.w->w.in_dim + i.w->w.out_dim);
                    launches++;
                }
            }
        }
    }
    OB_CUDA(ctx, cudaEventRecord(ctx->ev1, st));
    OB_CUDA(ctx, cudaStreamSynchronize(st));
    OB_CUDA(ctx, cudaGetLastError());
    if (!launches) return fail(ctx, OB_ERR_INVALID, "profile_gemv: the model has no matrix of that type");
    cudaEventElapsedTime(ms_total, ctx->ev0, ctx->ev1);
    ctx->launches += (uint64_t)launches * (iters + 1);
    if (bytes_per_pass) *bytes_per_pass = bytes;
    if (launches_per_pass) *launches_per_pass = launches;
    return OB_OK;
}

// ------------------------------------------------------------------------------------ forward

}  // extern "C"

namespace {

// One step on the stream: metadata up, kernels, results down; synchronises.
int run_rows(ob_model *m, const std::vector<ob_kv *> &row_kv, const uint32_t *tokens, const uint32_t *positions, bool gemm_order,
             uint32_t logit_row0, uint32_t n_logit_rows, const ob_greedy *greedy, const uint32_t *recent_off, uint32_t seq0,
             uint32_t *out_token, float *out_logits) {
    ob_ctx *ctx = m->ctx;
    const uint32_t T = (uint32_t)row_kv.size();
    const MetaLayout ml(m->T);
    uint32_t *h_tokens = reinterpret_cast<uint32_t *>(m->h_meta + ml.off_tokens);
    uint32_t *h_positions = reinterpret_cast<uint32_t *>(m->h_meta + ml.off_positions);
    uint32_t *h_npos = reinterpret_cast<uint32_t *>(m->h_meta + ml.off_npos);
    const int32_t **h_tables = reinterpret_cast<const int32_t **>(m->h_meta + ml.off_tables);
    uint32_t pos_bound = 0;
    for (uint32_t t = 0; t < T; ++t) {
        h_tokens[t] = tokens[t];
        h_positions[t] = positions[t];
        h_npos[t] = positions[t] + 1;
        h_tables[t] = row_kv[t]->d_table;
        pos_bound = std::max(pos_bound, positions[t] + 1);
    }
    const bool exact_attn = pos_bound <= m->exact_attn_max_pos;
    cudaStream_t st = ctx->stream;
    OB_CUDA(ctx, cudaEventRecord(ctx->ev0, st));
    OB_CUDA(ctx, cudaMemcpyAsync(m->d_meta, m->h_meta, ml.bytes, cudaMemcpyHostToDevice, st));
    const bool penalise = greedy && greedy->repeat_penalty != 1.0f && greedy->recent && greedy->n_recent;
    enqueue_step(m, T, gemm_order, logit_row0, n_logit_rows, out_token != nullptr && !penalise, out_logits != nullptr || penalise, exact_attn, pos_bound, st);
    if (out_token && penalise) {
        // repeat penalty, then argmax (sampling.rs:345-359); the history comes from the caller per call
        for (uint32_t r = 0; r < n_logit_rows; ++r) {
            const uint32_t s = seq0 + r, nr = greedy->n_recent[s];
            const uint32_t start = nr > greedy->repeat_last_n ? nr - greedy->repeat_last_n : 0, cnt = nr - start;
            if (!cnt) continue;
            int rc = ensure(ctx, ctx->saux, (size_t)cnt * 4);
            if (rc) return rc;
            OB_CUDA(ctx, cudaMemcpyAsync(ctx->saux.p, greedy->recent + recent_off[s] + start, (size_t)cnt * 4, cudaMemcpyHostToDevice, st));
            launch_repeat_penalty(m->logits + (size_t)r * m->cfg.n_vocab, m->cfg.n_vocab, static_cast<uint32_t *>(ctx->saux.p), cnt,
                                  greedy->repeat_penalty, st);
            ctx->launches++;
            OB_CUDA(ctx, cudaStreamSynchronize(st));  // saux is reused by the next row
        }
        ArgmaxArgs am{};
        am.logits = m->logits;
        am.n_seq = n_logit_rows;
        am.n_vocab = m->cfg.n_vocab;
        am.out = m->d_out_tokens;
        am.scratch = m->argmax_scratch;
        launch_argmax(am, st);
        ctx->launches += 3;
    }
    if (out_token) OB_CUDA(ctx, cudaMemcpyAsync(m->h_out_tokens, m->d_out_tokens, (size_t)n_logit_rows * 4, cudaMemcpyDeviceToHost, st));
    if (out_logits) OB_CUDA(ctx, cudaMemcpyAsync(out_logits, m->logits, (size_t)n_logit_rows * m->cfg.n_vocab * 4, cudaMemcpyDeviceToHost, st));
    OB_CUDA(ctx, cudaEventRecord(ctx->ev1, st));
    fetch_status(m, st);
    OB_CUDA(ctx, cudaStreamSynchronize(st));
    OB_CUDA(ctx, cudaGetLastError());
    float ms = 0.0f;
    cudaEventElapsedTime(&ms, ctx->ev0, ctx->ev1);
    ctx->last_ms += ms;
    if (out_token) memcpy(out_token, m->h_out_tokens, (size_t)n_logit_rows * 4);
    return check_peer(m);
}

}  // namespace

extern "C" {

int ob_forward(ob_model *m, ob_kv *const *kvs, const uint32_t *tokens, const uint32_t *n_tokens, const uint32_t *start_pos, uint32_t n_seq,
               const ob_greedy *greedy, uint32_t *out_token, float *out_logits) {
    if (!m || !kvs || !tokens || !n_tokens || !start_pos) return fail(m ? m->ctx : nullptr, OB_ERR_INVALID, "forward: null argument");
    ob_ctx *ctx = m->ctx;
    std::lock_guard<std::mutex> g(ctx->mu);
    if (n_seq == 0) return OB_OK;
    Bind b(ctx);
    // ---- validate everything before any state changes
    bool all_single = true;
    uint64_t total = 0;
    std::vector<uint32_t> tok_off(n_seq), recent_off(n_seq, 0);
    for (uint32_t s = 0; s < n_seq; ++s) {
        ob_kv *kv = kvs[s];
        if (!kv || kv->m != m) return fail(ctx, OB_ERR_INVALID, "forward: KV cache missing or from another model");
        if (n_tokens[s] == 0) return fail(ctx, OB_ERR_INVALID, "forward: a sequence carries no tokens");
        if (start_pos[s] != kv->len) return fail(ctx, OB_ERR_INVALID, "forward: start_pos does not continue the KV cache");
        if ((uint64_t)kv->len + n_tokens[s] > kv->capacity) return fail(ctx, OB_ERR_CAPACITY, "forward: KV cache is full");
        for (uint32_t s2 = 0; s2 < s; ++s2)
            if (kvs[s2] == kv) return fail(ctx, OB_ERR_INVALID, "forward: the same KV cache appears twice");
        if (n_tokens[s] != 1) all_single = false;
        tok_off[s] = (uint32_t)total;
        total += n_tokens[s];
        if (s + 1 < n_seq && greedy && greedy->n_recent) recent_off[s + 1] = recent_off[s] + greedy->n_recent[s];
    }
    for (uint64_t i = 0; i < total; ++i)
        if (tokens[i] >= m->cfg.n_vocab) return fail(ctx, OB_ERR_INVALID, "forward: token id out of vocabulary range");
    {   // on-demand caches: all the pages this call needs, or none of them
        uint64_t need = 0;
        for (uint32_t s = 0; s < n_seq; ++s) need += pages_missing(kvs[s], kvs[s]->len + n_tokens[s]);
        if (need > m->free_pages.size()) return fail(ctx, OB_ERR_CAPACITY, "forward: KV pool exhausted");
        for (uint32_t s = 0; s < n_seq; ++s) {
            int rc = grow_pages(kvs[s], kvs[s]->len + n_tokens[s]);
            if (rc) return rc;
        }
    }
    if (int rc = pre_step(m)) return rc;
    ctx->last_ms = 0.0f;

    if (all_single) {
        // decode batch, in slices of at most max_batch_tokens rows
        for (uint32_t s0 = 0; s0 < n_seq; s0 += m->T) {
            const uint32_t n = std::min(m->T, n_seq - s0);
            std::vector<ob_kv *> rows(kvs + s0, kvs + s0 + n);
            int rc = run_rows(m, rows, tokens + s0, start_pos + s0, false, 0, n, greedy, recent_off.data(), s0, out_token ? out_token + s0 : nullptr,
                              out_logits ? out_logits + (size_t)s0 * m->cfg.n_vocab : nullptr);
            if (rc) return rc;
            for (uint32_t i = 0; i < n; ++i) kvs[s0 + i]->len += 1;
        }
        return OB_OK;
    }
    // otherwise sequence by sequence; a multi-token sequence is a prefill in chunks of max_batch_tokens
    for (uint32_t s = 0; s < n_seq; ++s) {
        ob_kv *kv = kvs[s];
        uint32_t done = 0;
        while (done < n_tokens[s]) {
            const uint32_t n = std::min(m->T, n_tokens[s] - done);
            const bool last_chunk = done + n == n_tokens[s];
            std::vector<ob_kv *> rows(n, kv);
            std::vector<uint32_t> pos(n);
            for (uint32_t i = 0; i < n; ++i) pos[i] = kv->len + i;
            // a chunk of one token takes the single-token kernels, exactly as the reference's matmul does
            int rc = run_rows(m, rows, tokens + tok_off[s] + done, pos.data(), n > 1, n - 1, last_chunk ? 1 : 0, greedy, recent_off.data(), s,
                              (last_chunk && out_token) ? out_token + s : nullptr,
                              (last_chunk && out_logits) ? out_logits + (size_t)s * m->cfg.n_vocab : nullptr);
            if (rc) return rc;
            kv->len += n;
            done += n;
        }
    }
    return OB_OK;
}

int ob_last_hidden(ob_model *m, uint32_t n_tokens, float *out) {
    if (!m || !out) return OB_ERR_INVALID;
    ob_ctx *ctx = m->ctx;
    std::lock_guard<std::mutex> g(ctx->mu);
    if (n_tokens > m->last_T) return fail(ctx, OB_ERR_INVALID, "last_hidden: more rows than the last step carried");
    Bind b(ctx);
    OB_CUDA(ctx, cudaMemcpyAsync(out, m->x, (size_t)n_tokens * m->cfg.n_embd * 4, cudaMemcpyDeviceToHost, ctx->stream));
    OB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return OB_OK;
}

// ------------------------------------------------------------------------------------ graphs

}  // extern "C"

namespace {

// After a synchronisation: did a peer exchange of the tensor-parallel step run out of time?
// Tensor parallel: every rank is about to enqueue the same step.  Meet on the host first, so that a rank that is gone (or has
// refused the call on its own arguments) costs the others a time limit here and not a wait inside a collective on the GPU.
int pre_step(ob_model *m) {
    if (!m->rdv) return OB_OK;
    if (m->out_of_step) return fail(m->ctx, OB_ERR_COMM, "tensor parallel: an earlier step lost a rank; the model has to be created again on every rank");
    int missing = -1;
    if (obtp::rendezvous_arrive(m->rdv, m->rdv_timeout_ms, &missing)) return OB_OK;
    m->out_of_step = true;
    return fail(m->ctx, OB_ERR_COMM, "tensor parallel: rank " + std::to_string(missing) + " did not arrive for this step within " + std::to_string(m->rdv_timeout_ms) +
                                         " ms; nothing was launched");
}

int check_peer(ob_model *m) {
    if (gemm_tc5_take_status()) return fail(m->ctx, OB_ERR_CUDA, "a tensor-core product gave up a bounded wait (pipeline barrier); the step's output is not valid");
    if (m->launch_failed) {
        m->launch_failed = false;
        return fail(m->ctx, OB_ERR_CUDA, std::string("launching the persistent layer kernel failed: ") + cudaGetErrorString(cudaGetLastError()));
    }
    if (m->persist_ok) {
        if (*m->h_ls_status) {  // copied down with the step's results (fetch_status)
            *m->h_ls_status = 0;
            cudaMemset(m->ls_status, 0, 4);
            return fail(m->ctx, OB_ERR_CUDA, "the persistent layer kernel gave up at a grid barrier (not every CTA was resident)");
        }
    }
    if (m->comm_failed) {
        m->comm_failed = false;
        return fail(m->ctx, OB_ERR_COMM, std::string("tensor-parallel collective failed: ") + obtp::last_error(m->comm));
    }
    if (m->px.size < 2) return OB_OK;
    uint32_t e = 0;
    if (cudaMemcpy(&e, m->px.err, 4, cudaMemcpyDeviceToHost) != cudaSuccess) return fail(m->ctx, OB_ERR_CUDA, "reading the exchange status failed");
    if (!e) return OB_OK;
    cudaMemset(m->px.err, 0, 4);
    return fail(m->ctx, OB_ERR_COMM, "tensor-parallel exchange: a rank did not deliver its partial within " + std::to_string(m->px.timeout_ms ? m->px.timeout_ms : 4000u) + " ms");
}

// kind 0: H2D metadata + step + D2H token (one host round trip per step)
// kind 1: step + advance (device-resident loop)
// exact: every window stays within exact_attn_max_pos for as long as the graph is replayed
int get_graph(ob_model *m, uint32_t n_seq, int kind, bool exact, cudaGraphExec_t *out, uint64_t *key_out) {
    ob_ctx *ctx = m->ctx;
    const uint64_t key = ((uint64_t)kind << 32) | ((uint64_t)(exact ? 1 : 0) << 33) | n_seq;
    if (key_out) *key_out = key;
    const uint32_t pos_bound = exact ? m->exact_attn_max_pos : m->cfg.max_seq_len;
    auto it = m->graphs.find(key);
    if (it != m->graphs.end()) {
        *out = it->second;
        return OB_OK;
    }
    const MetaLayout ml(m->T);
    cudaStream_t st = ctx->stream;
    // One eager pass first (d_meta must already describe a valid step): it sets the kernels' one-time
    // function attributes outside capture and counts what a step launches.  It rewrites the KV slot of
    // the current position with the values the replay will write again.
    const uint64_t launches_before = ctx->launches;
    enqueue_step(m, n_seq, false, 0, n_seq, true, false, exact, pos_bound, st);
    OB_CUDA(ctx, cudaStreamSynchronize(st));
    OB_CUDA(ctx, cudaGetLastError());
    m->graph_launches[key] = ctx->launches - launches_before + (kind == 1 ? 1 : 0);
    ctx->launches = launches_before;
    cudaGraph_t graph = nullptr;
    OB_CUDA(ctx, cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
    if (kind == 0) cudaMemcpyAsync(m->d_meta, m->h_meta, ml.bytes, cudaMemcpyHostToDevice, st);
    enqueue_step(m, n_seq, false, 0, n_seq, true, false, exact, pos_bound, st);
    if (kind == 0) {
        cudaMemcpyAsync(m->h_out_tokens, m->d_out_tokens, (size_t)n_seq * 4, cudaMemcpyDeviceToHost, st);
        fetch_status(m, st);
    } else {
        advance_kernel<<<(n_seq + 127) / 128, 128, 0, st>>>(reinterpret_cast<uint32_t *>(m->d_meta + ml.off_tokens),
                                                             reinterpret_cast<uint32_t *>(m->d_meta + ml.off_positions),
                                                             reinterpret_cast<uint32_t *>(m->d_meta + ml.off_npos), m->d_out_tokens, n_seq,
                                                             m->d_history, m->d_step_counter);
        ctx->launches++;
    }
    cudaError_t e = cudaStreamEndCapture(st, &graph);
    if (e != cudaSuccess || !graph) return fail(ctx, OB_ERR_CUDA, std::string("graph capture: ") + cudaGetErrorString(e));
    m->ctx->launches = launches_before;  // capture enqueued nothing; replays are counted by their callers
    cudaGraphExec_t exec = nullptr;
    e = cudaGraphInstantiate(&exec, graph, 0);
    cudaGraphDestroy(graph);
    if (e != cudaSuccess) return fail(ctx, OB_ERR_CUDA, std::string("graph instantiate: ") + cudaGetErrorString(e));
    m->graphs[key] = exec;
    *out = exec;
    return OB_OK;
}

}  // namespace

extern "C" {

int ob_decode_greedy(ob_model *m, ob_kv *kv, uint32_t token, uint32_t *out_token) {
    if (!m || !kv || !out_token || kv->m != m) return fail(m ? m->ctx : nullptr, OB_ERR_INVALID, "decode_greedy: bad argument");
    ob_ctx *ctx = m->ctx;
    std::lock_guard<std::mutex> g(ctx->mu);
    if (token >= m->cfg.n_vocab) return fail(ctx, OB_ERR_INVALID, "decode_greedy: token id out of vocabulary range");
    if (kv->len >= kv->capacity) return fail(ctx, OB_ERR_CAPACITY, "decode_greedy: KV cache is full");
    if (pages_missing(kv, kv->len + 1) > m->free_pages.size()) return fail(ctx, OB_ERR_CAPACITY, "decode_greedy: KV pool exhausted");
    Bind b(ctx);
    if (int rc = grow_pages(kv, kv->len + 1)) return rc;
    if (int rc = pre_step(m)) return rc;
    const MetaLayout ml(m->T);
    reinterpret_cast<uint32_t *>(m->h_meta + ml.off_tokens)[0] = token;
    reinterpret_cast<uint32_t *>(m->h_meta + ml.off_positions)[0] = kv->len;
    reinterpret_cast<uint32_t *>(m->h_meta + ml.off_npos)[0] = kv->len + 1;
    reinterpret_cast<const int32_t **>(m->h_meta + ml.off_tables)[0] = kv->d_table;
    cudaGraphExec_t exec;
    uint64_t key = 0;
    const bool exact = kv->len + 1 <= m->exact_attn_max_pos;
    OB_CUDA(ctx, cudaMemcpyAsync(m->d_meta, m->h_meta, ml.bytes, cudaMemcpyHostToDevice, ctx->stream));  // the first build runs a step eagerly
    int rc = get_graph(m, 1, 0, exact, &exec, &key);
    if (rc) return rc;
    OB_CUDA(ctx, cudaEventRecord(ctx->ev0, ctx->stream));
    OB_CUDA(ctx, cudaGraphLaunch(exec, ctx->stream));
    OB_CUDA(ctx, cudaEventRecord(ctx->ev1, ctx->stream));
    OB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    cudaEventElapsedTime(&ctx->last_ms, ctx->ev0, ctx->ev1);
    ctx->launches += m->graph_launches[key];
    kv->len += 1;
    *out_token = m->h_out_tokens[0];
    return check_peer(m);
}

int ob_decode_loop(ob_model *m, ob_kv *const *kvs, const uint32_t *first_tokens, uint32_t n_seq, uint32_t n_steps, uint32_t *out_tokens) {
    if (!m || !kvs || !first_tokens || !out_tokens) return fail(m ? m->ctx : nullptr, OB_ERR_INVALID, "decode_loop: null argument");
    ob_ctx *ctx = m->ctx;
    std::lock_guard<std::mutex> g(ctx->mu);
    if (n_seq == 0 || n_steps == 0) return OB_OK;
    if (n_seq > m->T) return fail(ctx, OB_ERR_CAPACITY, "decode_loop: more sequences than max_batch_tokens");
    for (uint32_t s = 0; s < n_seq; ++s) {
        if (!kvs[s] || kvs[s]->m != m) return fail(ctx, OB_ERR_INVALID, "decode_loop: KV cache missing or from another model");
        if ((uint64_t)kvs[s]->len + n_steps > kvs[s]->capacity) return fail(ctx, OB_ERR_CAPACITY, "decode_loop: KV cache too small for n_steps");
        if (first_tokens[s] >= m->cfg.n_vocab) return fail(ctx, OB_ERR_INVALID, "decode_loop: token id out of vocabulary range");
        for (uint32_t s2 = 0; s2 < s; ++s2)
            if (kvs[s2] == kvs[s]) return fail(ctx, OB_ERR_INVALID, "decode_loop: the same KV cache appears twice");
    }
    Bind b(ctx);
    {
        uint64_t need = 0;
        for (uint32_t s = 0; s < n_seq; ++s) need += pages_missing(kvs[s], kvs[s]->len + n_steps);
        if (need > m->free_pages.size()) return fail(ctx, OB_ERR_CAPACITY, "decode_loop: KV pool exhausted");
        for (uint32_t s = 0; s < n_seq; ++s)
            if (int rc = grow_pages(kvs[s], kvs[s]->len + n_steps)) return rc;
    }
    if (int rc = pre_step(m)) return rc;
    if ((uint64_t)n_steps * n_seq > m->history_cap) {
        int rc = dev_alloc(m, &m->d_history, (size_t)n_steps * n_seq);
        if (rc) return rc;
        m->history_cap = n_steps * n_seq;
        // the graph holds the old pointer: drop loop graphs
        for (auto it = m->graphs.begin(); it != m->graphs.end();) {
            if (((it->first >> 32) & 1) == 1) {
                cudaGraphExecDestroy(it->second);
                it = m->graphs.erase(it);
            } else {
                ++it;
            }
        }
    }
    uint64_t key = 0;
    bool exact = true;
    for (uint32_t s = 0; s < n_seq; ++s) exact = exact && (uint64_t)kvs[s]->len + n_steps <= m->exact_attn_max_pos;
    const MetaLayout ml(m->T);
    for (uint32_t s = 0; s < n_seq; ++s) {
        reinterpret_cast<uint32_t *>(m->h_meta + ml.off_tokens)[s] = first_tokens[s];
        reinterpret_cast<uint32_t *>(m->h_meta + ml.off_positions)[s] = kvs[s]->len;
        reinterpret_cast<uint32_t *>(m->h_meta + ml.off_npos)[s] = kvs[s]->len + 1;
        reinterpret_cast<const int32_t **>(m->h_meta + ml.off_tables)[s] = kvs[s]->d_table;
    }
    OB_CUDA(ctx, cudaMemcpyAsync(m->d_meta, m->h_meta, ml.bytes, cudaMemcpyHostToDevice, ctx->stream));
    cudaGraphExec_t exec;
    int rc = get_graph(m, n_seq, 1, exact, &exec, &key);
    if (rc) return rc;
    cudaStream_t st = ctx->stream;
    OB_CUDA(ctx, cudaMemcpyAsync(m->d_meta, m->h_meta, ml.bytes, cudaMemcpyHostToDevice, st));
    OB_CUDA(ctx, cudaMemsetAsync(m->d_step_counter, 0, 4, st));
    OB_CUDA(ctx, cudaEventRecord(ctx->ev0, st));
    for (uint32_t i = 0; i < n_steps; ++i) OB_CUDA(ctx, cudaGraphLaunch(exec, st));
    OB_CUDA(ctx, cudaEventRecord(ctx->ev1, st));
    OB_CUDA(ctx, cudaMemcpyAsync(out_tokens, m->d_history, (size_t)n_steps * n_seq * 4, cudaMemcpyDeviceToHost, st));
    fetch_status(m, st);
    OB_CUDA(ctx, cudaStreamSynchronize(st));
    OB_CUDA(ctx, cudaGetLastError());
    cudaEventElapsedTime(&ctx->last_ms, ctx->ev0, ctx->ev1);
    ctx->launches += m->graph_launches[key] * n_steps;
    for (uint32_t s = 0; s < n_seq; ++s) kvs[s]->len += n_steps;
    return check_peer(m);
}

namespace {
__global__ void selftest_deliver_kernel(uint2 *slot, uint32_t n, float value, uint32_t tag) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) slot[i] = make_uint2(__float_as_uint(value), tag);
}
}  // namespace

int ob_tp_exchange_selftest(ob_ctx *ctx, uint32_t n, uint32_t timeout_ms, uint32_t n_rounds, const uint8_t *peer_delivers, float *sums_out) {
    if (!ctx || !peer_delivers || n == 0 || n % 256 || n_rounds == 0 || n_rounds > 64) return fail(ctx, OB_ERR_INVALID, "tp_exchange_selftest: bad argument");
    std::lock_guard<std::mutex> g(ctx->mu);
    Bind b(ctx);
    cudaStream_t st = ctx->stream;
    // a two-rank exchange whose slots are all local memory: this "rank 0" delivers every round, "rank 1" only when told to
    uint8_t *region = nullptr;
    float *x = nullptr;
    const size_t slot_bytes = (size_t)2 * 2 * n * sizeof(uint2);
    OB_CUDA(ctx, cudaMalloc(reinterpret_cast<void **>(&region), 512 + slot_bytes));
    if (cudaMalloc(reinterpret_cast<void **>(&x), (size_t)n * 4) != cudaSuccess) {
        cudaFree(region);
        return fail(ctx, OB_ERR_OOM, "tp_exchange_selftest: allocation failed");
    }
    cudaMemsetAsync(region, 0, 512 + slot_bytes, st);
    obtp::PeerXchg px{};
    px.rank = 0;
    px.size = 2;
    px.n = n;
    px.timeout_ms = timeout_ms ? timeout_ms : 50;
    px.seq = reinterpret_cast<uint32_t *>(region);
    px.err = reinterpret_cast<uint32_t *>(region) + 32;
    px.slots[0] = px.slots[1] = reinterpret_cast<uint2 *>(region + 512);
    int rc = OB_OK;
    for (uint32_t k = 0; k < n_rounds; ++k) {  // exchange number k: tag k + 1, slot parity k & 1 (tp.h)
        cudaMemsetAsync(x, 0, (size_t)n * 4, st);
        uint2 *base = px.slots[0] + (size_t)(k & 1u) * 2 * n;
        selftest_deliver_kernel<<<(n + 255) / 256, 256, 0, st>>>(base, n, 1.0f, k + 1);
        if (peer_delivers[k]) selftest_deliver_kernel<<<(n + 255) / 256, 256, 0, st>>>(base + n, n, 2.0f, k + 1);
        launch_norm_quant_consume(x, nullptr, n, 1e-5f, nullptr, nullptr, px, false, st);
        ctx->launches += 2 + (peer_delivers[k] ? 1 : 0);
        uint32_t err = 0;
        float first = 0.0f;
        cudaError_t e = cudaMemcpyAsync(&err, px.err, 4, cudaMemcpyDeviceToHost, st);
        if (e == cudaSuccess) e = cudaMemcpyAsync(&first, x + (n - 1), 4, cudaMemcpyDeviceToHost, st);
        if (e == cudaSuccess) e = cudaStreamSynchronize(st);
        if (e != cudaSuccess) {
            rc = fail(ctx, OB_ERR_CUDA, std::string("tp_exchange_selftest: ") + cudaGetErrorString(e));
            break;
        }
        if (sums_out) sums_out[k] = first;
        if (err) {  // the wait ran out: report as the model's step does, clear, go on with the next round
            cudaMemsetAsync(px.err, 0, 4, st);
            rc = fail(ctx, OB_ERR_COMM, "tensor-parallel exchange: a rank did not deliver its partial within " + std::to_string(px.timeout_ms) + " ms (round " + std::to_string(k) + ")");
            if (sums_out) sums_out[k] = -1.0f;
        }
    }
    cudaStreamSynchronize(st);
    cudaFree(region);
    cudaFree(x);
    return rc;
}

// The few-rows exchange on one GPU: this "rank 0" runs the real kernel; what "rank 1" would have pushed (2 i + 1 at element i,
// and its arrival words) is written beforehand by a copy when peer_delivers is set, and is absent otherwise.  x starts at 0.5,
// rank 0's partial is i, so a delivered exchange leaves 0.5 + 3 i + 1; an undelivered one runs into the time limit.
int ob_tp_bulk_selftest(ob_ctx *ctx, uint32_t count, uint32_t timeout_ms, uint32_t n_rounds, const uint8_t *peer_delivers, float *x_out) {
    if (!ctx || !peer_delivers || !x_out || count == 0 || (count & 3) || count > (1u << 22) || n_rounds == 0 || n_rounds > 16)
        return fail(ctx, OB_ERR_INVALID, "tp_bulk_selftest: bad argument");
    std::lock_guard<std::mutex> g(ctx->mu);
    Bind b(ctx);
    cudaStream_t st = ctx->stream;
    const uint32_t cap = (count + obtp::kBulkChunk - 1) / obtp::kBulkChunk * obtp::kBulkChunk, chunks = cap / obtp::kBulkChunk;
    const size_t flag_bytes = ((size_t)2 * 2 * chunks * 4 + 255) & ~(size_t)255, data_bytes = (size_t)2 * 2 * cap * 4;
    uint8_t *mine = nullptr, *peer = nullptr;  // the two ranks' regions, both local
    float *x = nullptr, *proj = nullptr;
    std::vector<float> h_proj(count), h_peer(count), h_x(count, 0.5f);
    for (uint32_t i = 0; i < count; ++i) {
        h_proj[i] = (float)(i % 1000);
        h_peer[i] = (float)(2 * (i % 1000) + 1);
    }
    cudaError_t e = cudaMalloc(reinterpret_cast<void **>(&mine), 512 + flag_bytes + data_bytes);
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void **>(&peer), 512 + flag_bytes + data_bytes);
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void **>(&x), (size_t)count * 4);
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void **>(&proj), (size_t)count * 4);
    int rc = OB_OK;
    if (e != cudaSuccess) rc = fail(ctx, OB_ERR_OOM, "tp_bulk_selftest: allocation failed");
    if (rc == OB_OK) {
        cudaMemsetAsync(mine, 0, 512 + flag_bytes + data_bytes, st);
        cudaMemsetAsync(peer, 0, 512 + flag_bytes + data_bytes, st);
        cudaMemcpyAsync(proj, h_proj.data(), (size_t)count * 4, cudaMemcpyHostToDevice, st);
        obtp::PeerXchg px{};
        px.rank = 0;
        px.size = 2;
        px.n = 0;
        px.timeout_ms = timeout_ms ? timeout_ms : 50;
        px.seq = reinterpret_cast<uint32_t *>(mine);
        px.err = reinterpret_cast<uint32_t *>(mine) + 32;
        obtp::PeerBulk bk{};
        bk.done = reinterpret_cast<uint32_t *>(mine) + 40;
        bk.cap = cap;
        bk.max_chunks = chunks;
        bk.flags[0] = reinterpret_cast<uint32_t *>(mine + 512);
        bk.flags[1] = reinterpret_cast<uint32_t *>(peer + 512);
        bk.data[0] = reinterpret_cast<float *>(mine + 512 + flag_bytes);
        bk.data[1] = reinterpret_cast<float *>(peer + 512 + flag_bytes);
        std::vector<uint32_t> tags(chunks);
        for (uint32_t k = 0; k < n_rounds && rc == OB_OK; ++k) {
            const uint32_t par = k & 1u;
            cudaMemcpyAsync(x, h_x.data(), (size_t)count * 4, cudaMemcpyHostToDevice, st);
            if (peer_delivers[k]) {  // rank 1's chunks and arrival words of exchange k, in rank 0's region
                std::fill(tags.begin(), tags.end(), k + 1u);
                cudaMemcpyAsync(bk.data[0] + (size_t)(par * 2 + 1) * cap, h_peer.data(), (size_t)count * 4, cudaMemcpyHostToDevice, st);
                cudaMemcpyAsync(bk.flags[0] + (size_t)(par * 2 + 1) * chunks, tags.data(), (size_t)chunks * 4, cudaMemcpyHostToDevice, st);
                cudaStreamSynchronize(st);  // `tags` is reused by the next round
            }
            launch_bulk_allreduce_add(x, proj, count, px, bk, st);
            ctx->launches++;
            uint32_t err = 0, seq = 0;
            e = cudaMemcpyAsync(&err, px.err, 4, cudaMemcpyDeviceToHost, st);
            if (e == cudaSuccess) e = cudaMemcpyAsync(&seq, px.seq, 4, cudaMemcpyDeviceToHost, st);
            if (e == cudaSuccess) e = cudaMemcpyAsync(x_out + (size_t)k * count, x, (size_t)count * 4, cudaMemcpyDeviceToHost, st);
            if (e == cudaSuccess) e = cudaStreamSynchronize(st);
            if (e != cudaSuccess) {
                rc = fail(ctx, OB_ERR_CUDA, std::string("tp_bulk_selftest: ") + cudaGetErrorString(e));
            } else if (seq != k + 1) {
                rc = fail(ctx, OB_ERR_CUDA, "tp_bulk_selftest: the exchange counter did not advance");
            } else if (err) {
                cudaMemsetAsync(px.err, 0, 4, st);
                if (peer_delivers[k]) rc = fail(ctx, OB_ERR_COMM, "tp_bulk_selftest: a delivered exchange ran into the time limit");
            } else if (!peer_delivers[k]) {
                rc = fail(ctx, OB_ERR_CUDA, "tp_bulk_selftest: an undelivered exchange did not report");
            }
        }
        cudaStreamSynchronize(st);
    }
    cudaFree(mine);
    cudaFree(peer);
    cudaFree(x);
    cudaFree(proj);
    return rc;
}

int ob_tp_rendezvous_selftest(const void *id128, uint32_t rank, uint32_t size, uint32_t n_steps, uint32_t timeout_ms, int32_t *missing) {
    std::string err;
    obtp::Rendezvous *r = obtp::rendezvous_open(id128, (int)rank, (int)size, &err);
    if (!r) return fail(nullptr, OB_ERR_COMM, err);
    int who = -1, rc = OB_OK;
    for (uint32_t i = 0; i < n_steps && rc == OB_OK; ++i)
        if (!obtp::rendezvous_arrive(r, timeout_ms ? timeout_ms : 1000u, &who)) rc = fail(nullptr, OB_ERR_COMM, "rendezvous: rank " + std::to_string(who) + " did not arrive");
    if (missing) *missing = who;
    obtp::rendezvous_close(r);
    return rc;
}

int ob_tp_unique_id(void *out128) {
    if (!out128) return OB_ERR_INVALID;
    std::string err;
    if (!obtp::unique_id(out128, &err)) return fail(nullptr, OB_ERR_COMM, err);
    return OB_OK;
}

}  // extern "C"
