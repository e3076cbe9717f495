// Host-callable launchers of the CUDA kernels (internal to the library).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"
#include "tp.h"

namespace ob {

// ---- formats.cu
// src_type: the GGUF type of `src`; w.type is what the device holds (TYPE_Q8_0 for the per-32 symmetric source types).
void launch_repack(const uint8_t *src, uint64_t src_row_bytes, uint32_t src_type, uint32_t row0, uint32_t blk0, const DevWeight &w, cudaStream_t st);
void launch_dequant_rows(const DevWeight &w, uint32_t first_row, uint32_t n_rows, float *out, cudaStream_t st);
void launch_embed(const DevWeight &w, const uint32_t *tokens, uint32_t n_tokens, float *out, cudaStream_t st);

// ---- act_quant.cu
// Writable quantized-activation buffers for up to `rows` token rows of `dim` elements.
struct ActBuf {
    int8_t *q = nullptr;     // [rows][dim]
    float *d = nullptr;      // [rows][dim/group]
    int16_t *sums = nullptr; // [rows][dim/16]
    uint32_t dim_cap = 0;    // row pitch in elements
};
enum ActSource { ACT_PLAIN = 0, ACT_RMSNORM = 1, ACT_SWIGLU = 2 };
struct QuantArgs {
    const float *x;       // [n_rows][dim]   (PLAIN, RMSNORM) or gate (SWIGLU)
    const float *aux;     // RMSNORM: weight [dim]; SWIGLU: up [n_rows][dim]
    float eps;            // RMSNORM
    float *f32_out;       // optional: the fp32 values that were quantized, [n_rows][dim]
    uint32_t n_rows, dim;
    ActBuf k;             // per-256 output (q == nullptr: skip)
    ActBuf flat;          // per-32 output  (q == nullptr: skip)
};
void launch_quantize(int source, const QuantArgs &a, cudaStream_t st);

// ---- gemv.cu
enum GemvEpilogue { EPI_STORE = 0, EPI_ADD_RESIDUAL = 1 };
struct GemvSegment {
    DevWeight w;
    float *y;              // [n_tokens][y_stride]
    const float *residual; // EPI_ADD_RESIDUAL: y = residual + product (may alias y)
    uint32_t y_stride;
    int epilogue;
};
struct GemvArgs {
    GemvSegment seg[3];    // all of one ggml type and one in_dim
    int n_seg;
    ActBuf act;            // activations of the matching granularity
    const float *x_f32 = nullptr;  // Q8_0, one token: the fp32 row instead of `act`; the kernel quantizes it per 32 itself (one launch per product)
    uint32_t n_tokens;
    bool gemm_order;       // false: every (row, token) is the single-token GEMV; true: the prefill GEMM's fp32 order
    int32_t *isum_out;     // optional debug capture (single segment, token 0): [out_dim][nb]
    int32_t *imin_out;
};
void launch_gemv(const GemvArgs &a, int sm_count, cudaStream_t st);
size_t gemv_smem_bytes(uint32_t type, uint32_t in_dim, uint32_t tile_tokens, bool gemm_order);
uint32_t gemv_launches(uint32_t type, uint32_t in_dim, uint32_t n_tokens, bool gemm_order);  // kernels launch_gemv issues

// ---- q5k.cu: Q5_K weights, one kernel for any token count and both fp32 orders
void launch_q5k(const GemvArgs &a, int sm_count, cudaStream_t st);

// ---- gemm_mma.cu: many-token products on the tensor cores (Q4_K and Q6_K; 9 tokens or more)
bool gemm_mma_supported(const GemvArgs &a);
void launch_gemm_mma(const GemvArgs &a, int sm_count, cudaStream_t st);

// ---- gemm_tc5.cu: many-token products on tcgen05 tensor cores with TMEM accumulators, TMA-fed (16 tokens or more)
bool gemm_tc5_supported(const GemvArgs &a);
bool launch_gemm_tc5(const GemvArgs &a, int sm_count, cudaStream_t st);  // false: a tensor map could not be made (nothing was launched)
int gemm_tc5_take_status();  // 1 when a bounded wait inside one of these kernels ran out since the last call

// ---- stream_gemv.cu: fused single-token products for decode (Q4_K / Q6_K weights)
enum StreamPrologue { SG_PRO_PLAIN = 0, SG_PRO_RMSNORM = 1, SG_PRO_READY = 2 };
enum StreamEpilogue { SG_EP_STORE = 0, SG_EP_RESIDUAL = 1, SG_EP_SWIGLU = 2, SG_EP_ROPE_Q = 3, SG_EP_ROPE_K = 4, SG_EP_V = 5, SG_EP_XCHG = 6 };
struct StreamSeg {
    DevWeight w;       // rows 2p, 2p+1 form pair p ...
    DevWeight w2;      // ... unless w2.data != nullptr: then pair p is (w row p, w2 row p)  (gate / up)
    float *y;          // STORE/RESIDUAL/ROPE_Q: [rows]; SWIGLU: [pairs]
    int epilogue;
};
struct StreamArgs {
    StreamSeg seg[3];
    int n_seg;
    uint32_t in_dim;
    int prologue;
    const float *x;          // [in_dim] fp32 input of the token
    const float *norm_w;     // RMSNORM: weight [in_dim]
    const float *norm_scale; // RMSNORM: device word holding 1 / sqrt(mean(x^2) + eps), from launch_norm_scale
    float eps;
    const uint8_t *ready;    // READY: the token's quantized activations as launch_norm_quant / launch_quant_image left them
    const float *residual;   // RESIDUAL: y = residual + product (may alias y)
    // one SWIGLU segment whose row count is a multiple of 256: also leave the outputs quantized per 256 (the next product's READY input)
    uint8_t *out_image;
    uint32_t *out_counters;  // [rows / 256], zero before the launch and after it
    // RoPE + KV append (ROPE_Q / ROPE_K / V)
    const float *rope_table; // [pos][rope_dim/2](sin, cos)
    const uint32_t *position;        // device: position of the token
    const int32_t *const *page_table; // device: pointer to the sequence's page table
    __half *k_pool, *v_pool;
    uint32_t n_head_kv, head_dim, rope_dim;
    // XCHG: the rows are this rank's partial of a contraction-split product; they go into every rank's exchange slot and
    // the last CTA raises this rank's flag everywhere (tp.h).  px.size == 0: unused.
    obtp::PeerXchg px;
    bool wait_dependency;    // launched with programmatic stream serialisation: wait for the predecessor before reading x
};
bool stream_gemv_supported(const StreamArgs &a);
void launch_stream_gemv(const StreamArgs &a, int sm_count, bool programmatic, cudaStream_t st);
void launch_norm_scale(const float *x, uint32_t dim, float eps, float *out, bool programmatic, cudaStream_t st);
// Bytes of the quantized-activation image of one token row of `dim` elements (dim a multiple of 256).
size_t act_image_bytes(uint32_t dim);
// RMSNorm scale as launch_norm_scale (also stored to *scale_out), then (x * scale) * norm_w quantized per 256 into `image`.
void launch_norm_quant(const float *x, const float *norm_w, uint32_t dim, float eps, float *scale_out, uint8_t *image, bool programmatic, cudaStream_t st);
// The same, but first the pending peer exchange is completed: x += the ranks' partials, added in rank order (x is written).
void launch_norm_quant_consume(float *x, const float *norm_w, uint32_t dim, float eps, float *scale_out, uint8_t *image, const obtp::PeerXchg &px,
                               bool programmatic, cudaStream_t st);
// x quantized per 256 into `image`.
void launch_quant_image(const float *x, uint32_t dim, uint8_t *image, bool programmatic, cudaStream_t st);

// ---- layer_stream.cu: the single-token products between two attention kernels as phases of one persistent launch
struct alignas(16) LsPhase {
    StreamArgs a;        // as for launch_stream_gemv; prologue SG_PRO_READY, or SG_PRO_RMSNORM (x: the fp32 row; the exact scale is computed by the phase)
    uint32_t lp;         // lanes per row pair (kernel shape of this phase)
    uint32_t q6;         // the phase has Q6_K segments
    uint32_t nw;         // warps of the CTA that take part in the product
    uint32_t l2_ahead;   // units per warp sent to L2 ahead of the ring while the prologue runs
};
struct LsLayout {  // byte offsets inside the kernel's dynamic shared memory
    uint32_t off_desc;   // two phase descriptors (ping-pong)
    uint32_t off_tab;    // two segment tables (ping-pong)
    uint32_t off_ctrl;   // control words
    uint32_t off_img;    // the activation image of the running phase
    uint32_t off_norm;   // RMSNorm prologue: the fp32 row (one pad word per 16) and the exact-sum workspace
    uint32_t off_terms;  // [warp][32] fp32 terms
    uint32_t off_ring;   // per-warp two-slot weight ring
    uint32_t total;
};
bool layer_stream_phase(const StreamArgs &a, LsPhase *out);              // false: the shape does not take this kernel
LsLayout layer_stream_layout(const LsPhase *phases, uint32_t n);         // host copy of the phases
bool layer_stream_fits(const LsLayout &L);
// barrier: one zeroed word per launch; status: set to 1 when a barrier wait gave up after timeout_ms
bool launch_layer_stream(const LsPhase *dev_phases, uint32_t n, const LsLayout &L, int sm_count, uint32_t *barrier, uint32_t *status, uint32_t timeout_ms,
                         bool programmatic, cudaStream_t st);

// ---- glue.cu
void launch_rmsnorm(const float *x, const float *w, uint32_t n_tokens, uint32_t dim, float eps, float *out, cudaStream_t st);
void launch_swiglu(const float *gate, const float *up, uint64_t n, float *out, cudaStream_t st);
void launch_add(float *a, const float *b, uint64_t n, cudaStream_t st);
struct RopeKvArgs {
    float *q;                 // [n_tokens][n_head*head_dim], rotated in place
    const float *k;           // [n_tokens][kv_dim]
    const float *v;           // [n_tokens][kv_dim]
    const float *rope_table;  // [max_pos][rope_dim/2][2] (sin, cos)
    const uint32_t *positions;   // [n_tokens] absolute position of each token
    const int32_t *const *page_tables; // [n_tokens] device pointers: the page table of each token's sequence
    __half *k_pool;           // this layer's pages [page][n_head_kv][16][head_dim]
    __half *v_pool;
    uint32_t n_tokens, n_head, n_head_kv, head_dim, rope_dim;
    // Qwen2 / Qwen3-style extras (engine/arch/llama.rs:750-780), all optional: biases added to the projected rows, then a
    // per-head RMSNorm of q and k (weights [head_dim]), then the rotation with either pairing.
    const float *q_bias = nullptr, *k_bias = nullptr, *v_bias = nullptr, *q_norm = nullptr, *k_norm = nullptr;
    float rms_eps = 0.0f;
    bool neox = false;  // pairs (i, i + rope_dim/2) instead of (2i, 2i+1)
};
void launch_rope_kv(const RopeKvArgs &a, cudaStream_t st);
void launch_rope_plain(float *x, uint32_t n_head, uint32_t head_dim, uint32_t rope_dim, const float *sin_cos_row, cudaStream_t st);
struct ArgmaxArgs {
    const float *logits;   // [n_seq][n_vocab]
    uint32_t n_seq, n_vocab;
    uint32_t *out;         // [n_seq]
    unsigned long long *scratch; // [n_seq] packed (key, index)
    // Tensor parallel with a peer exchange (px.size > 1): `logits` points at this rank's columns of every row, n_vocab is
    // their count, row_stride the distance between rows (0: n_vocab) and index_base the vocabulary id of the first column.
    // Each rank finds the maximum of its columns; the finish kernel stores (key, id) tagged into every rank's exchange slot,
    // waits for the others' and keeps the largest (key, id): the last of equal maxima wins across ranks as it does within one
    // (engine/sampling.rs:336-343).  2 * n_seq words of the slot are used, so n_seq <= px.n / 2.
    uint32_t row_stride = 0, index_base = 0;
    obtp::PeerXchg px{};
};
void launch_argmax(const ArgmaxArgs &a, cudaStream_t st);
// Tensor parallel, a few rows: x[0..count) += sum over ranks of proj (this rank's partial), through peer memory (tp.h, PeerBulk).
// count <= bulk.cap.  `programmatic` is not used: the kernel is an ordinary stream-ordered launch.
void launch_bulk_allreduce_add(float *x, const float *proj, uint32_t count, const obtp::PeerXchg &px, const obtp::PeerBulk &bulk, cudaStream_t st);
void launch_repeat_penalty(float *logits, uint32_t n_vocab, const uint32_t *recent, uint32_t n_recent, float penalty, cudaStream_t st);

// ---- attention.cu
struct AttnDecodeArgs {
    const float *q;            // [n_seq][n_head*head_dim]
    float *out;                // [n_seq][n_head*head_dim]
    const __half *k_pool;      // layer pages [page][n_head_kv][16][head_dim]
    const __half *v_pool;
    const int32_t *const *page_tables; // [n_seq] device pointers
    const uint32_t *n_pos;     // [n_seq] positions to attend (window 0..n_pos-1), device
    uint32_t n_seq, n_head, n_head_kv, head_dim;
    float scale;
    uint32_t n_splits;         // CTAs per (sequence, kv head)
    float *part_o;             // [n_seq][n_head][n_splits][head_dim]
    float *part_ml;            // [n_seq][n_head][n_splits][2]
    uint32_t max_pos;          // upper bound of n_pos (sizes nothing on the device; bounds the split length)
    // launch_attn_decode_fused only:
    uint32_t *counters;        // [n_seq][n_head_kv], zero before the first launch; the kernel leaves them zero
    uint8_t *image;            // optional, n_seq == 1: the output quantized per 256 for the product that follows (stream_gemv.cu)
    bool small_ctas;           // many (row, kv head) pairs: CTAs of four warps, two per SM
};
void launch_attn_decode(const AttnDecodeArgs &a, cudaStream_t st);
// One kernel: every warp streams its own pages, the CTAs of a (sequence, kv head) leave partials and the last of them to
// finish merges them (and quantizes the result when `image` is set).  False when the shape is not covered.
bool launch_attn_decode_fused(const AttnDecodeArgs &a, bool programmatic, cudaStream_t st);

// The rows (n_seq of them) are consecutive tokens of ONE sequence: tiled tensor-core attention, 16 tokens x the query heads of a kv
// head per CTA, K/V of the window read once per 16 tokens.  Needs no partial buffers.  False when the shape is not covered.
bool launch_attn_prefill(const AttnDecodeArgs &a, cudaStream_t st);

// Exact-order attention (three kernels: scores, softmax, output); see attention.cu.
struct AttnExactArgs {
    const float *q;            // [n_rows][n_head*head_dim]
    float *out;                // [n_rows][n_head*head_dim]
    const __half *k_pool;
    const __half *v_pool;
    const int32_t *const *page_tables; // [n_rows]
    const uint32_t *n_pos;     // [n_rows], device
    float *scores;             // [n_rows][n_head][score_stride] scratch: scores, then probabilities
    uint32_t score_stride;
    uint32_t n_rows, n_head, n_head_kv, head_dim;
    float scale;
    uint32_t max_pos;          // upper bound of n_pos over the rows (sizes the score grid)
};
void launch_attn_exact(const AttnExactArgs &a, cudaStream_t st);
bool attn_exact_supported(uint32_t n_head, uint32_t n_head_kv, uint32_t head_dim);
}  // namespace ob
