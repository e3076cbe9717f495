/*
 * CPU oracle for the quantized decode path: a restatement, in plain C++, of the
 * arithmetic the reference's CPU backend performs.  TEST INFRASTRUCTURE ONLY.
 *
 * Nothing in the product library links, loads or calls this file.  It is used
 * by the test-suite as the checker for the CUDA path, and by the benchmark's
 * CPU-baseline leg as the thing timed on the host cores.
 *
 * The reference is Rust and cannot be compiled in this environment (no cargo /
 * rustc), so this is a restatement rather than the reference itself.  It is
 * pinned to the reference by the known-answer tests the reference carries in
 * its own sources (dequantisation bit checksums, activation-quantiser tie and
 * NaN cases, GEMV/GEMM-versus-dequantise bounds, batch-size independence,
 * attention head-outer form); see tests/test_oracle_golden.py.  Parity for the
 * libm transcendentals is unpinned at the ulp level: the reference calls the
 * platform libm through Rust std.  powf, sinf and cosf (RoPE angles) are the
 * platform's here too; exp (SiLU, softmax) is pinned to the correctly rounded
 * value, (float)exp((double)x), so that a device can reproduce it bit for bit.
 *
 * Every function cites the reference file:line it follows.  Paths are relative
 * to the reference project root; E = src/bin/orangu-server/engine.
 *
 * Build: -O3 -march=native -ffp-contract=off -fopenmp, never -ffast-math.
 * Rust never contracts a*b+c into an FMA, so neither may the compiler here.
 */
#ifndef ORANGU_ORACLE_H
#define ORANGU_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ggml type ids, E/quant.rs:50-112 */
#define OREF_TYPE_F32 0u
#define OREF_TYPE_Q4_0 2u   /* the per-32 symmetric family beside Q8_0: one f16 scale, 32 signed codes, no min term */
#define OREF_TYPE_Q5_0 6u
#define OREF_TYPE_IQ4_NL 20u
#define OREF_TYPE_Q8_0 8u
#define OREF_TYPE_Q4_K 12u
#define OREF_TYPE_Q6_K 14u
#define OREF_TYPE_Q5_K 13u  /* Q4_K with a fifth bit per code; oracle only so far: the device library has no kernel for it */

/* ---- formats ------------------------------------------------------------ */
float oref_f16_to_f32(uint16_t bits);                       /* E/quant.rs:511-528 */
uint16_t oref_f32_to_f16(float v);                          /* IEEE RNE, the rule half::f16::from_f32 implements; E/kv_cache.rs:26-32 */
int oref_block_layout(uint32_t type, uint32_t *block_bytes, uint32_t *block_elems); /* E/quant.rs:132-169 */
int64_t oref_row_bytes(uint32_t type, uint64_t in_dim);
int oref_dequantize(uint32_t type, const uint8_t *bytes, size_t n_elems, float *out); /* E/quant.rs:639-649, 666-697, 746-787 */
void oref_get_scale_min_k4(int j, const uint8_t *scales12, uint8_t *sc, uint8_t *m);  /* E/quant.rs:653-662 */

/* ---- activation quantisers ------------------------------------------------ */
/* per-32 scale; sums per 16.  E/vecdot.rs:95-126 */
void oref_quantize_act(const float *x, size_t n, int8_t *q, float *d, int32_t *sums);
/* per-256 scale; sums per 16.  E/vecdot.rs:3030-3053 */
void oref_quantize_act_k_row(const float *x, size_t n, int8_t *q, float *d, int32_t *sums);

/* ---- GEMV rows ------------------------------------------------------------ */
float oref_dot_q8_0(const uint8_t *row, size_t in_dim, const int8_t *q, const float *d);   /* E/vecdot.rs:2829-2838 */
/* any per-32 type (Q8_0, Q4_0, Q5_0, IQ4_NL) against per-32 quantized activations; E/vecdot.rs:2842-2881 */
float oref_dot_row32(uint32_t type, const uint8_t *row, size_t in_dim, const int8_t *q, const float *d);
float oref_dot_k_row(uint32_t type, const uint8_t *row, size_t in_dim, const int8_t *q,
                     const float *d, const int32_t *sums);                                /* E/vecdot.rs:3152-3178, 3215-3241 */
/* The integer partial sums the GEMV forms before touching fp32: per Q8_0 block the
 * dot32, per Q4_K super-block isum and imin, per Q6_K super-block isum (imin = 0). */
int oref_row_partials(uint32_t type, const uint8_t *row, size_t in_dim, const float *x,
                      int32_t *isum, int32_t *imin);

/* ---- matmul (CpuBackend) -------------------------------------------------- */
/* y[t,o], x is [n_tokens,in_dim]; kernel choice as E/backend/cpu.rs:55-167.
 * n_threads <= 0 means all cores. */
int oref_matmul(const float *x, size_t n_tokens, const uint8_t *raw, uint32_t type,
                size_t in_dim, size_t out_dim, float *y, int n_threads);
/* row-independent decode form, E/backend/cpu.rs:265-317 */
int oref_matmul_decode(const float *x, size_t n_tokens, const uint8_t *raw, uint32_t type,
                       size_t in_dim, size_t out_dim, float *y, int n_threads);
/* full-precision path: dequantise + f32 dot, E/backend/cpu.rs:409-432 */
int oref_matmul_dequant(const float *x, size_t n_tokens, const uint8_t *raw, uint32_t type,
                        size_t in_dim, size_t out_dim, float *y, int n_threads);

/* ---- f32 glue ------------------------------------------------------------- */
float oref_dot(const float *a, const float *b, size_t n);                                  /* E/tensor.rs:393-430 */
void oref_rmsnorm(float *dst, const float *src, const float *weight, size_t n_tokens,
                  size_t dim, float eps);                                                 /* E/tensor.rs:732-757 */
void oref_rope_norm(float *x, size_t n_head, size_t head_dim, size_t pos, size_t rope_dim,
                    float freq_base);                                                     /* E/tensor.rs:1115-1177, NORM layout, no YaRN */
void oref_rope_layout(float *x, size_t n_head, size_t head_dim, size_t pos, size_t rope_dim, float freq_base,
                      const float *freq_factors, int neox);                                /* E/tensor.rs:1115-1177, either pairing */
void oref_rope_table(float *sin_cos, size_t n_pos, size_t rope_dim, float freq_base);     /* the (sin,cos) pairs the loop above applies */
void oref_softmax(float *x, size_t n);                                                    /* E/tensor.rs:809-821 */
float oref_silu(float x);                                                                 /* E/tensor.rs:825-827 */
void oref_swiglu(float *gate, const float *up, size_t n);                                 /* E/arch/mod.rs:1099-1105 */
void oref_add(float *a, const float *b, size_t n);                                        /* E/tensor.rs:1242-1253 */
/* k,v: [n_pos][kv_dim] f32; causal window (0, start_pos+t).  E/attention.rs:725-758 (head-outer form,
 * which the reference pins bit-identical to its production loop :426-549). */
void oref_attention(float *out, const float *q, const float *k, const float *v, size_t kv_dim,
                    size_t n_head, size_t group_size, size_t head_dim, float scale,
                    size_t n_tokens, size_t start_pos, int n_threads);
uint32_t oref_argmax(const float *logits, size_t n);                                      /* E/sampling.rs:336-343 */
void oref_repeat_penalty(float *logits, size_t n_vocab, const uint32_t *recent, size_t n_recent,
                         size_t repeat_last_n, float penalty);                            /* E/sampling.rs:345-359 */

/* ---- Llama graph ---------------------------------------------------------- */
typedef struct {
    const uint8_t *data;
    uint32_t type;
    uint32_t in_dim;
    uint32_t out_dim;
} oref_matrix;

typedef struct {
    const float *attn_norm;
    const float *ffn_norm;
    oref_matrix wq, wk, wv, wo, w_gate, w_up, w_down;
    /* Qwen2/Qwen3-style extras, each NULL when the file has no such tensor (E/arch/llama.rs:45-60, 171-175):
     * attn_{q,k,v}.bias added to every projected row, attn_{q,k}_norm.weight [head_dim] as a per-head RMSNorm before RoPE */
    const float *q_bias, *k_bias, *v_bias, *q_norm, *k_norm;
} oref_layer;

typedef struct {
    uint32_t n_vocab, n_embd, n_layer, n_head, n_head_kv, head_dim, rope_dim, n_ff;
    float rope_freq_base, rms_eps;
    const float *rope_freqs; /* optional rope_freqs.weight, rope_dim / 2 factors dividing the frequencies (E/arch/llama.rs:186-200); NULL: none */
    uint32_t rope_neox;      /* 0: RopeLayout::Norm, pairs (2i, 2i+1) -- llama, mistral; 1: RopeLayout::Neox, pairs (i, i + rope_dim/2) --
                              * qwen2, qwen3, qwen3vl and unknown architectures (rope_layout_for, E/arch/llama.rs:114-119) */
} oref_config;

typedef struct oref_model oref_model;
typedef struct oref_kv oref_kv;

/* The model borrows every pointer; E/arch/llama.rs:125-183 */
oref_model *oref_model_create(const oref_config *cfg, const oref_matrix *token_embd,
                              const float *output_norm, const oref_matrix *output,
                              const oref_layer *layers);
void oref_model_destroy(oref_model *);
/* kv_f16 != 0 rounds K and V through f16 on push (what the reference's GPU mirror holds,
 * E/kv_cache.rs:26-32); 0 keeps f32 (what CpuBackend holds, E/kv_cache.rs:756-768). */
oref_kv *oref_kv_create(const oref_model *, size_t capacity, int kv_f16);
void oref_kv_destroy(oref_kv *);
size_t oref_kv_len(const oref_kv *);
void oref_kv_truncate(oref_kv *, size_t len);
/* logits of the last token, [n_vocab].  E/arch/llama.rs:594-932, 1007-1032.
 * hidden_out (nullable) receives the last layer's residual stream [n_tokens,n_embd]. */
int oref_forward(const oref_model *, oref_kv *, const uint32_t *tokens, size_t n_tokens,
                 size_t start_pos, float *logits, float *hidden_out, int n_threads);

int oref_hardware_threads(void);

#ifdef __cplusplus
}
#endif
#endif
