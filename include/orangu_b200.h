/*
 * orangu_b200 -- C ABI of the B200 (sm_100a) backend for orangu-server's quantized
 * decode path.
 *
 * This is the drop-in boundary: the entry points below are what an FFI crate on the
 * server side binds in place of its CUDA backend.  Each one names the interface of
 * the reference engine it stands in for (paths relative to the reference project
 * root; B = src/bin/orangu-server/engine/backend, E = src/bin/orangu-server/engine).
 *
 * Conventions
 *   - every call returns OB_OK (0) or a negative ob_status; nothing aborts, throws
 *     or longjmps across the boundary.  ob_last_error() gives the text.
 *   - host pointers are borrowed for the duration of the call only.
 *   - a context is bound to one GPU and serialises its calls on an internal mutex,
 *     so it may be shared between threads (the reference's Backend is Send + Sync,
 *     B/mod.rs:309).
 *   - there is no CPU fallback: without a usable sm_100 device ob_init fails.
 */
#ifndef ORANGU_B200_H
#define ORANGU_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
#if defined(__GNUC__)
#pragma GCC visibility push(default) /* the library is built with hidden visibility; these are its exports */
#endif

/* 2: ob_model_desc gained rope_freqs (layout change); the GGUF, static-attention and KV-copy entry points were added.
 * 3: ob_model_desc gained tp_presliced. */
#define OB_ABI_VERSION 4u

typedef enum ob_status {
    OB_OK = 0,
    OB_ERR_INVALID = -1,      /* bad argument (null, shape mismatch, out-of-range token ...) */
    OB_ERR_UNSUPPORTED = -2,  /* ggml type / shape this backend has no kernel for */
    OB_ERR_NO_DEVICE = -3,    /* no CUDA device, or not an sm_100 part */
    OB_ERR_CUDA = -4,         /* a CUDA runtime call failed; text in ob_last_error */
    OB_ERR_OOM = -5,          /* device or pinned-host allocation failed */
    OB_ERR_CAPACITY = -6,     /* KV cache full, batch larger than the model was created for */
    OB_ERR_COMM = -7          /* tensor-parallel communicator failure */
} ob_status;

/* ggml type ids as the GGUF file carries them (E/quant.rs:50-112) */
#define OB_TYPE_F32 0u
#define OB_TYPE_Q8_0 8u
#define OB_TYPE_Q4_K 12u
#define OB_TYPE_Q5_K 13u
#define OB_TYPE_Q6_K 14u
/* Per-32 symmetric types (one f16 scale, 32 signed codes).  The CPU kernels for them are the Q8_0 loops over the unpacked
 * codes (E/vecdot.rs:2842-2881 decode, :1277-1340 + :2598-2629 batched), so the library unpacks them once, at registration,
 * into its Q8_0 layout: results equal the CPU's bit for bit; the device reads 34 bytes per block instead of 18 or 22. */
#define OB_TYPE_Q4_0 2u
#define OB_TYPE_Q5_0 6u
#define OB_TYPE_IQ4_NL 20u

typedef struct ob_ctx ob_ctx;
typedef struct ob_weight ob_weight;
typedef struct ob_model ob_model;
typedef struct ob_kv ob_kv;

/* ------------------------------------------------------------------ context */

/* Replaces CudaBackend::try_init_index (B/cuda.rs:86-124): never panics; any failure
 * is a status and *out stays NULL.  device_ordinal < 0 picks the current device. */
int ob_init(int device_ordinal, ob_ctx **out);
void ob_destroy(ob_ctx *ctx);

/* Text of the last failure on this context (never NULL; "" when none).  ctx == NULL
 * returns the text of the last failed ob_init on the calling thread. */
const char *ob_last_error(const ob_ctx *ctx);

unsigned ob_abi_version(void);

/* Replaces Backend::supports_type (B/mod.rs:479-495): 1 for Q8_0, Q4_K, Q5_K, Q6_K, Q4_0, Q5_0, IQ4_NL (and F32
 * for norm vectors), 0 otherwise, so a missing kernel is a named start-up error. */
int ob_supports_type(uint32_t ggml_type);

/* Replaces Backend::reduced_surface (B/mod.rs:409-434): NULL, because the fused layer
 * chain, device attention and device sampling are all present. */
const char *ob_reduced_surface(void);

/* ------------------------------------------------------------------ weights */

/* Replaces CudaBackend::weight_buffer (B/cuda.rs:216-236): copies a QuantMatrix
 * (E/loader.rs:561-680) to the device.  `raw` is out_dim rows of row_bytes bytes in
 * GGUF block layout, dims[0] = in_dim contiguous.  The bytes are copied; the caller's
 * mapping need not outlive the call. */
int ob_weight_register(ob_ctx *ctx, const uint8_t *raw, uint64_t row_bytes, uint32_t ggml_type,
                       uint32_t in_dim, uint32_t out_dim, ob_weight **out);

/* Tensor-parallel shard of a matrix: rows [row0, row0+n_rows) and input columns
 * [col0, col0+n_cols) of it (col0 and n_cols multiples of the type's block size).
 * Stands in for QuantMatrix::rows (E/loader.rs:627-646), extended to a column range. */
int ob_weight_register_slice(ob_ctx *ctx, const uint8_t *raw, uint64_t row_bytes, uint32_t ggml_type,
                             uint32_t in_dim, uint32_t out_dim, uint32_t row0, uint32_t n_rows,
                             uint32_t col0, uint32_t n_cols, ob_weight **out);
void ob_weight_release(ob_ctx *ctx, ob_weight *w);

/* Replaces QuantMatrix::row (E/loader.rs:585-590): dequantises rows
 * [first_row, first_row+n_rows) to f32 on the device and copies them to out_host. */
int ob_weight_dequantize(ob_ctx *ctx, const ob_weight *w, uint32_t first_row, uint32_t n_rows, float *out_host);

/* ------------------------------------------------------------------- matmul */

/* Replaces Backend::matmul / matmul_into (B/mod.rs:310-342, B/cuda.rs:250-254):
 * y[t,o] = sum_i x[t,i] * w.row(o)[i]; x is [n_tokens, in_dim], y [n_tokens, out_dim],
 * both row-major host f32.  n_tokens == 1 takes the GEMV of the type's family, n_tokens > 1
 * the prefill GEMM, as CpuBackend chooses (B/cpu.rs:55-167). */
int ob_matmul(ob_ctx *ctx, const float *x, uint32_t n_tokens, const ob_weight *w, float *y);

/* Replaces Backend::matmul_decode / matmul_decode_into (B/mod.rs:368-388, B/cpu.rs:265-317):
 * the rows of x are independent sequences; row t of y equals ob_matmul on that row alone,
 * bit for bit. */
int ob_matmul_decode(ob_ctx *ctx, const float *x, uint32_t n_tokens, const ob_weight *w, float *y);

typedef struct ob_matmul_op { /* MatmulOp, B/mod.rs:117-121 */
    const float *x;
    uint32_t n_tokens;
    const ob_weight *w;
    float *y;
} ob_matmul_op;

/* Replaces Backend::matmul_batch / matmul_batch_into / matmul_batch_decode
 * (B/mod.rs:362-407): independent ops, one submission. */
int ob_matmul_batch(ob_ctx *ctx, const ob_matmul_op *ops, uint32_t n_ops, int decode);

/* Same products with x and y already in device memory (no copies, asynchronous on
 * `stream`, a cudaStream_t or NULL for the context's stream).  Has no counterpart in the
 * reference, whose CUDA backend copies per call (B/cuda.rs:325-367); it is what a caller
 * that keeps activations resident uses. */
int ob_matmul_device(ob_ctx *ctx, const float *x_dev, uint32_t n_tokens, const ob_weight *w,
                     float *y_dev, int decode, void *stream);
int ob_synchronize(ob_ctx *ctx);

/* The integer partial sums the GEMV forms before any fp32 arithmetic, for rows
 * [first_row, first_row+n_rows) against one activation row x[in_dim]: per Q8_0 block its
 * dot32; per Q4_K super-block isum and imin; per Q6_K super-block isum (imin 0).
 * isum/imin are [n_rows][in_dim / block] host int32.  This is what dot32/dot16 and the
 * k-row accumulators hold in E/vecdot.rs:471-502, 3152-3241; it exists for parity checks. */
int ob_matmul_partials(ob_ctx *ctx, const float *x, const ob_weight *w, uint32_t first_row,
                       uint32_t n_rows, int32_t *isum, int32_t *imin);

/* --------------------------------------------------------------- glue ops */
/* Host-buffer forms of the small operators around the products.  In the reference they
 * run on the CPU between matmuls when the CUDA backend is active (B/mod.rs:306-307). */

/* tensor::rmsnorm_into (E/tensor.rs:732-757) */
int ob_rmsnorm(ob_ctx *ctx, const float *x, const float *weight, uint32_t n_tokens, uint32_t dim, float eps, float *out);
/* tensor::rope_apply_params_inplace, RopeLayout::Norm, no YaRN (E/tensor.rs:1115-1177); x is [n_head, head_dim] */
int ob_rope(ob_ctx *ctx, float *x, uint32_t n_head, uint32_t head_dim, uint32_t pos, uint32_t rope_dim, float freq_base);
/* arch::swiglu_ffn_into's element-wise part (E/arch/mod.rs:1099-1105): out = silu(gate) * up */
int ob_swiglu(ob_ctx *ctx, const float *gate, const float *up, uint32_t n, float *out);
/* vecdot::quantize_act (per 32) / quantize_act_k_row (per 256) (E/vecdot.rs:79-126, 3030-3053);
 * q [n] int8, d [n/32 or n/256] f32, sums [n/16] int32 */
int ob_quantize_act(ob_ctx *ctx, const float *x, uint32_t n, int per_256, int8_t *q, float *d, int32_t *sums);
/* attention::attention with n_tokens == 1 (E/attention.rs:242-344, 426-549) and the device path it
 * can dispatch to, VulkanBackend::gpu_attention_split (B/vulkan.rs:6330-6342, 10788): one query
 * token q [n_head*head_dim] against n_pos cached positions k,v [n_pos, n_head_kv*head_dim] f32,
 * which are stored as fp16 pages exactly as the KV mirror holds them (E/kv_cache.rs:26-32).
 * exact_order 1 evaluates in the CPU loop's operation order (bit-identical to it); 0 takes the
 * split flash-decode kernels and 2 the one-kernel tensor-core flash-decode that the decode step uses
 * (head_dim 64 or 128; 1, 2, 4 or 8 query heads per kv head; 3 is the same kernel in the four-warp CTA shape it
 * takes for large decode batches); their results differ from the CPU's in the last bits. */
int ob_attention_decode(ob_ctx *ctx, const float *q, const float *k, const float *v, uint32_t n_pos,
                        uint32_t n_head, uint32_t n_head_kv, uint32_t head_dim, float scale, int exact_order, float *out);
/* The split flash-decode attention of ob_attention_decode for callers that must not allocate: a slot's worker
 * thread in the middle of a request, where cudaMalloc / cudaFree would synchronise the whole device and stall
 * the other slots' streams, or a process whose KV pool already holds the rest of the memory.  It has no
 * counterpart in the reference.  All pointers are device pointers supplied by the caller: q_dev
 * [n_head*head_dim] f32; k_pages_dev / v_pages_dev fp16 pages laid out [page][n_head_kv][16][head_dim];
 * page_table_dev int32 page ids of the sequence; out_dev [n_head*head_dim] f32.  The call is asynchronous on
 * `stream` (a cudaStream_t, or NULL for the context's stream).  The partial results of the splits live in a
 * 1 MiB array that is part of the library image on every GPU that loads it: shapes with
 * n_head * min(16, pages/4) * (head_dim + 2) * 4 bytes above 1 MiB are refused with OB_ERR_CAPACITY; head_dim is
 * 64 or 128 and n_head / n_head_kv is 1, 2, 4 or 8.  The first call on a device looks the array's address up
 * (one-time set-up; make that call before starting a stream capture).  Every call on a device shares the
 * array, so calls that may overlap on the GPU must be ordered by the caller. */
int ob_attention_decode_static(ob_ctx *ctx, const float *q_dev, const void *k_pages_dev, const void *v_pages_dev,
                               const int32_t *page_table_dev, uint32_t n_pos, uint32_t n_head, uint32_t n_head_kv,
                               uint32_t head_dim, float scale, float *out_dev, void *stream);
/* sampling::apply_repeat_penalty + argmax (E/sampling.rs:336-359); last index wins ties.
 * recent may be NULL; penalty 1.0 disables it. */
int ob_argmax(ob_ctx *ctx, const float *logits, uint32_t n_vocab, const uint32_t *recent,
              uint32_t n_recent, uint32_t repeat_last_n, float penalty, uint32_t *out_token);

/* ------------------------------------------------- fused surface: the model */

typedef struct ob_matrix_desc {
    const uint8_t *data; /* GGUF block layout, out_dim rows */
    uint32_t ggml_type;
    uint32_t in_dim;
    uint32_t out_dim;
} ob_matrix_desc;

/* One decoder block; the tensors LlamaModel::load_with_backend reads per layer
 * (E/arch/llama.rs:153-183) and FusedLayerInput carries (B/vulkan.rs:6663-6723). */
typedef struct ob_layer_desc {
    const float *attn_norm; /* blk.N.attn_norm.weight  [n_embd] */
    const float *ffn_norm;  /* blk.N.ffn_norm.weight   [n_embd] */
    ob_matrix_desc wq;      /* blk.N.attn_q.weight      [n_embd -> n_head*head_dim] */
    ob_matrix_desc wk;      /* blk.N.attn_k.weight      [n_embd -> n_head_kv*head_dim] */
    ob_matrix_desc wv;      /* blk.N.attn_v.weight */
    ob_matrix_desc wo;      /* blk.N.attn_output.weight [n_head*head_dim -> n_embd] */
    ob_matrix_desc w_gate;  /* blk.N.ffn_gate.weight    [n_embd -> n_ff] */
    ob_matrix_desc w_up;    /* blk.N.ffn_up.weight */
    ob_matrix_desc w_down;  /* blk.N.ffn_down.weight    [n_ff -> n_embd] */
    /* Qwen2 / Qwen3-style extras (E/arch/llama.rs:45-60, 171-175, 750-780); each NULL when the file has no such tensor.
     * Always the FULL vectors, also with tp_presliced (they are small; the model takes its part). */
    const float *q_bias;    /* blk.N.attn_q.bias        [n_head*head_dim]     added to every projected row */
    const float *k_bias;    /* blk.N.attn_k.bias        [n_head_kv*head_dim] */
    const float *v_bias;    /* blk.N.attn_v.bias        [n_head_kv*head_dim] */
    const float *q_norm;    /* blk.N.attn_q_norm.weight [head_dim]            per-head RMSNorm of q after the bias, before RoPE */
    const float *k_norm;    /* blk.N.attn_k_norm.weight [head_dim] */
} ob_layer_desc;

/* ModelConfig (E/loader.rs:34-58) plus run-time sizing. */
typedef struct ob_model_desc {
    uint32_t n_vocab, n_embd, n_layer, n_head, n_head_kv, head_dim, rope_dim, n_ff;
    float rope_freq_base, rms_eps;
    uint32_t max_seq_len;      /* longest context any KV cache of this model will hold */
    uint32_t max_batch_tokens; /* most tokens one ob_forward call will carry (prefill chunk or decode batch) */
    uint64_t kv_pool_tokens;   /* total KV capacity shared by every ob_kv of this model, in tokens; 0 = max_seq_len */
    /* Attention windows up to this many positions are evaluated in the CPU loop's own operation order
     * (bit-identical to CpuBackend given the same f16 cache); longer windows take the split flash-decode
     * kernel, as the reference moves long windows to its split-k device kernel (E/attention.rs:117,
     * 264-300).  0 = 1024. */
    uint32_t exact_attention_max_pos;
    ob_matrix_desc token_embd;   /* token_embd.weight */
    const float *output_norm;    /* output_norm.weight */
    ob_matrix_desc output;       /* output.weight; data == NULL ties it to token_embd (E/arch/llama.rs:133-139) */
    const ob_layer_desc *layers; /* n_layer entries */
    /* tensor parallel: this process is rank tp_rank of tp_size; descriptors above are the FULL
     * tensors and the model keeps its own shard.  tp_size <= 1 means single GPU. */
    uint32_t tp_rank, tp_size;
    const void *tp_unique_id;   /* tp_size > 1: the 128-byte id from ob_tp_unique_id, identical on every rank */
    const float *rope_freqs;    /* optional rope_freqs.weight: rope_dim / 2 factors that divide the rotation frequencies
                                 * (E/arch/llama.rs:186-200, E/tensor.rs:1143-1145); NULL: none */
    uint32_t tp_presliced;      /* tp_size > 1 only.  0: the matrix descriptors are the FULL tensors (the model keeps its shard).
                                 * 1: they already hold this rank's shard and nothing else -- rows [rank * out/tp, +out/tp) of
                                 * attn_q/k/v, ffn_gate/up and output, input columns [rank * in/tp, +in/tp) of attn_output and
                                 * ffn_down (QuantMatrix::rows, E/loader.rs:627-646, and its column counterpart); token_embd
                                 * and the norm vectors are whole.  For hosts that never hold the full tensors (a 70B model
                                 * on eight ranks). */
    uint32_t rope_neox;         /* RopeLayout (E/tensor.rs:873-889): 0 = Norm, pairs (2i, 2i+1) -- llama, mistral; 1 = Neox, pairs
                                 * (i, i + rope_dim/2) -- qwen2, qwen3, qwen3vl (rope_layout_for, E/arch/llama.rs:114-119) */
} ob_model_desc;

/* ------------------------------------------------- GGUF files
 * GgufFile::open (src/gguf.rs:206-275): header, typed metadata, tensor table; the file is mapped read-only and the
 * tensor data pointers below point into the mapping (valid until ob_gguf_close).  Works without a GPU.  A failed call
 * leaves its message in ob_gguf_last_error() (per thread). */
typedef struct ob_gguf ob_gguf;
typedef struct ob_gguf_tensor_info { /* TensorInfo, src/gguf.rs:121-130 */
    const char *name;
    uint32_t ggml_type;
    uint32_t n_dims;
    uint64_t dims[4];   /* GGUF order: dims[0] is the contiguous one (in_dim of a matrix), dims[1] the number of rows */
    const void *data;   /* data section start + offset */
    uint64_t n_bytes;   /* 0 for a type this build does not size */
} ob_gguf_tensor_info;
int ob_gguf_open(const char *path, ob_gguf **out);
void ob_gguf_close(ob_gguf *g);
const char *ob_gguf_last_error(void);
uint32_t ob_gguf_version(const ob_gguf *g);
uint64_t ob_gguf_alignment(const ob_gguf *g);   /* general.alignment, 32 when absent (src/gguf.rs:47) */
uint64_t ob_gguf_data_offset(const ob_gguf *g); /* end of the tensor table rounded up to the alignment (src/gguf.rs:258-266) */
uint64_t ob_gguf_n_tensors(const ob_gguf *g);
int ob_gguf_tensor(const ob_gguf *g, uint64_t index, ob_gguf_tensor_info *out);
int ob_gguf_find_tensor(const ob_gguf *g, const char *name, ob_gguf_tensor_info *out);
int ob_gguf_get_u64(const ob_gguf *g, const char *key, uint64_t *out);   /* any integer or bool value */
int ob_gguf_get_f32(const ob_gguf *g, const char *key, float *out);
int ob_gguf_get_string(const ob_gguf *g, const char *key, const char **out);
/* read_model_config (E/loader.rs:1652-1712) and the tensor lookup of LlamaModel::load_with_backend
 * (E/arch/llama.rs:125-200) for general.architecture == "llama": fills every field of *desc from the file -- required
 * keys embedding_length, block_count, attention.head_count; head_count_kv, key_length, rope.dimension_count,
 * rope.freq_base, layer_norm_rms_epsilon and vocab_size default as the reference's do; output.weight may be absent
 * (tied); rope_freqs.weight is optional.  max_seq_len is set to context_length and max_batch_tokens to 512; the caller
 * adjusts the run-time sizing and the tensor-parallel fields and passes desc to ob_model_create.  desc->layers is
 * owned by g. */
int ob_gguf_model_desc(ob_gguf *g, ob_model_desc *desc);

/* Stands in for LlamaModel::load_with_backend (E/arch/llama.rs:125-230) on the device side:
 * uploads (and shards) every tensor, sizes scratch, builds the RoPE table. */
int ob_model_create(ob_ctx *ctx, const ob_model_desc *desc, ob_model **out);
void ob_model_destroy(ob_model *model);

/* ModelForward::new_kv_cache (E/arch/llama.rs:1002-1005): an empty per-sequence cache of fp16
 * pages (16 tokens per page) with room for capacity_tokens. */
int ob_kv_create(ob_model *model, uint32_t capacity_tokens, ob_kv **out);
/* The same cache with its pages taken on demand: none at creation, one more from the model's pool each time the sequence
 * crosses a 16-token boundary (a call that finds the pool empty returns OB_ERR_CAPACITY and changes nothing), and whole pages
 * past new_len go back on ob_kv_truncate.  The reference sizes each KvCache up front (E/kv_cache.rs:496-511 only moves the
 * length); this is what lets many slots share one pool.  Results are identical to ob_kv_create's. */
int ob_kv_create_paged(ob_model *model, uint32_t capacity_tokens, ob_kv **out);
void ob_kv_destroy(ob_kv *kv);
uint32_t ob_kv_len(const ob_kv *kv);
uint32_t ob_kv_pages(const ob_kv *kv);              /* pages this cache holds now */
uint32_t ob_model_pool_pages(const ob_model *model); /* pages in the model's KV pool */
uint32_t ob_model_free_pages(const ob_model *model); /* of which no cache holds */
uint32_t ob_model_n_vocab(const ob_model *model);
uint32_t ob_model_tp_size(const ob_model *model);    /* 1 for a single-GPU model */
ob_ctx *ob_model_ctx(const ob_model *model);
/* KvCache::truncate (E/kv_cache.rs:496-511): roll back to new_len positions. */
int ob_kv_truncate(ob_kv *kv, uint32_t new_len);
/* Test hook: reads positions [pos0, pos0+n) of one layer back as f32 [n][n_head_kv*head_dim]. */
int ob_kv_read(ob_kv *kv, uint32_t layer, uint32_t pos0, uint32_t n, float *k_out, float *v_out);
/* KvCache::copy_prefix_from (E/kv_cache.rs:1079-1100): makes dst (empty) hold src's first n positions, by a
 * device-side copy of the pages.  Both caches belong to the same model. */
int ob_kv_copy_prefix(ob_kv *dst, const ob_kv *src, uint32_t n);

typedef struct ob_greedy { /* GpuArgmaxSampleInput, B/vulkan.rs:6219-6241 */
    float repeat_penalty;   /* 1.0 = off */
    uint32_t repeat_last_n;
    const uint32_t *recent; /* n_recent ids per sequence, concatenated; may be NULL */
    const uint32_t *n_recent;
} ob_greedy;

/* Replaces ModelForward::forward / forward_maybe_sampling / forward_batch_decode
 * (E/arch/mod.rs:2035-2191, E/arch/llama.rs:949-1032).  n_seq sequences; sequence i carries
 * n_tokens[i] tokens starting at position start_pos[i] (== ob_kv_len(kvs[i])), tokens concatenated.
 * A sequence with several tokens is a prefill chunk (GEMM semantics); sequences with one token
 * each form a decode batch whose rows do not influence one another.
 * out_token  [n_seq]          greedy next token of each sequence (may be NULL)
 * out_logits [n_seq][n_vocab] last-token logits (may be NULL; costs a device-to-host copy) */
int ob_forward(ob_model *model, ob_kv *const *kvs, const uint32_t *tokens, const uint32_t *n_tokens,
               const uint32_t *start_pos, uint32_t n_seq, const ob_greedy *greedy,
               uint32_t *out_token, float *out_logits);

/* One greedy decode step of a single sequence replayed from a captured CUDA graph:
 * the record_decode_chain path (E/arch/llama.rs:302-473), one submission per token and one
 * u32 back.  Equivalent to ob_forward with n_seq = 1, n_tokens = 1, no repeat penalty. */
int ob_decode_greedy(ob_model *model, ob_kv *kv, uint32_t token, uint32_t *out_token);

/* Device-resident decode loop: `n_steps` greedy steps for `n_seq` sequences, feeding each
 * step's token to the next without the host in between; out_tokens [n_steps][n_seq].
 * This is the loop of generate::run (E/generate.rs:859-878) with the sampler on the device. */
int ob_decode_loop(ob_model *model, ob_kv *const *kvs, const uint32_t *first_tokens, uint32_t n_seq,
                   uint32_t n_steps, uint32_t *out_tokens);

/* Hidden state after the last layer for the tokens of the most recent ob_forward call,
 * [n_tokens][n_embd] (what run_layers returns, E/arch/llama.rs:594-932).  Test hook. */
int ob_last_hidden(ob_model *model, uint32_t n_tokens, float *out);

/* Kernel launches issued by this context since creation (for reporting). */
uint64_t ob_launch_count(const ob_ctx *ctx);

/* Milliseconds of device time of the most recent ob_forward / ob_decode_* call, from CUDA
 * events on the context's stream. */
float ob_last_device_ms(const ob_ctx *ctx);

/* Measurement hook (no counterpart in the reference): runs one kind of product kernel for every layer back to
 * back `iters` times, with nothing else in between, and reports the device time between CUDA events on the
 * launching stream.  variant 0: the unfused single-token GEMV of every matrix of `ggml_type`; variants 1-5:
 * the fused batch-1 decode kernels -- 1 norm+q/k/v+RoPE+KV append, 2 attention-output+residual,
 * 3 norm+gate/up+SwiGLU, 4 down+residual, 5 norm+output projection (ggml_type ignored).  bytes_per_pass is the
 * quantized weight bytes one pass reads plus the fp32 in/out vectors; launches_per_pass the kernels it issues. */
int ob_profile_gemv(ob_model *model, uint32_t ggml_type, uint32_t variant, uint32_t iters, float *ms_total,
                    uint64_t *bytes_per_pass, uint32_t *launches_per_pass);

/* --------------------------------------------------------- tensor parallel */
/* No counterpart in the reference: its only multi-GPU mode is a host-bounced layer split
 * (B/multi.rs:16-35).  Rank 0 makes an id, every rank passes the same bytes in ob_model_desc. */
int ob_tp_unique_id(void *out128);
/* Diagnostic, on one GPU (no counterpart in the reference): the single-token step's peer exchange waits for every rank's
 * tagged words with a time limit and, when it runs out, reports OB_ERR_COMM instead of hanging.  This runs n_rounds exchanges
 * of n values (a multiple of 256) through the real consumer kernel with both "ranks" in local memory: rank 0 always delivers
 * (1.0), rank 1 (2.0) only in the rounds whose byte in peer_delivers is non-zero.  sums_out[k] is the summed value of round k
 * (3.0), or -1 when that round's wait ran out after timeout_ms (0 = 50 ms).  Returns OB_ERR_COMM if any round ran out. */
/* The exchange the tensor-parallel steps of a few rows use (one kernel: push the partial to every peer, wait for theirs, add in
 * rank order, add to the residual), run as rank 0 of 2 on one GPU with the peer's part written beforehand by a copy in the
 * rounds whose byte in peer_delivers is non-zero.  x starts at 0.5, the partials are i % 1000 and 2 (i % 1000) + 1:
 * x_out[round][count] receives the result.  Rounds without delivery must end by the time limit (timeout_ms, 0 = 50) and report;
 * OB_OK when every round behaved as it should.  No counterpart in the reference. */
int ob_tp_bulk_selftest(ob_ctx *ctx, uint32_t count, uint32_t timeout_ms, uint32_t n_rounds, const uint8_t *peer_delivers, float *x_out);
/* Host-only check of the ranks' meeting point (no counterpart in the reference, no device): under tensor parallel every
 * ob_forward / ob_decode_* call first meets the other ranks of the node in a small shared-memory segment named after the
 * communicator id, so that a rank that is gone, or that refused the call on its own arguments, costs the others
 * OB_TP_RENDEZVOUS_MS (30000; 0 = off) on the host and an OB_ERR_COMM with nothing launched, not a wait inside a collective.
 * This opens the segment for (id128, rank, size), arrives n_steps times with the given limit and closes; OB_ERR_COMM and
 * *missing = the first absent rank when a step's limit runs out. */
int ob_tp_rendezvous_selftest(const void *id128, uint32_t rank, uint32_t size, uint32_t n_steps, uint32_t timeout_ms, int32_t *missing);
int ob_tp_exchange_selftest(ob_ctx *ctx, uint32_t n, uint32_t timeout_ms, uint32_t n_rounds, const uint8_t *peer_delivers, float *sums_out);

/* ------------------------------------------------- slot pool and decode window */
/* SlotPool (E/scheduler.rs:36-317) + BatchCoordinator (E/batch.rs:184-324) + chunked prefill (E/generate.rs:1299-1338) over
 * ob_forward.  One thread per generating request, as in generate::run: acquire a slot, prefill, call ob_slot_decode per token,
 * release.  Every slot owns an on-demand paged KV cache of the model (ob_kv_create_paged).  Single-GPU models only: the
 * window forms its batches by arrival time, which the ranks of a tensor-parallel model would each see differently, while they
 * must all make the same calls (OB_ERR_UNSUPPORTED for tp_size > 1). */
typedef struct ob_slot_pool ob_slot_pool;
typedef struct ob_slot_pool_desc {
    uint32_t n_slots;              /* concurrent generations (`slots`) */
    uint32_t slot_capacity_tokens; /* longest sequence one slot may hold */
    uint32_t max_queue;            /* SlotPool::with_queue_limit: waiters beyond this are refused; 0 = unbounded */
    uint32_t batch_wait_ms;        /* collection window, ORANGU_BATCH_WAIT_MS; 0 = 4 (E/batch.rs:63) */
    uint32_t prefill_batch;        /* prefill chunk width, ORANGU_PREFILL_BATCH; 0 = 512 (E/generate.rs:1265) */
    uint32_t batch_decode;         /* ORANGU_BATCH_DECODE: 0 = each step runs alone, 1 = steps inside one window run as one batch */
} ob_slot_pool_desc;
typedef struct ob_slot_state { /* SlotState, E/scheduler.rs:29-34 */
    uint32_t id, busy, prompt_tokens, generated_tokens;
} ob_slot_state;
typedef struct ob_slot_pool_stats { /* batch_stats (E/batch.rs:117-122) and the pool's gauges */
    uint64_t batches, batched_seqs, refused;
    uint32_t total, busy, queued, free_pages;
} ob_slot_pool_stats;

/* model == NULL makes a pool that schedules only (no caches, ob_slot_prefill refuses, ob_slot_decode answers
 * token * 31 + slot * 7 + 1 from a host-side stand-in): the form the host-only tests use. */
int ob_slot_pool_create(ob_model *model, const ob_slot_pool_desc *desc, ob_slot_pool **out);
void ob_slot_pool_destroy(ob_slot_pool *pool);
/* SlotPool::try_acquire: whichever slot frees first, waiters served in arrival order.  timeout_ms < 0 waits without limit,
 * 0 does not wait.  OB_ERR_CAPACITY when the queue limit is reached or the time runs out (the caller answers "overloaded"). */
int ob_slot_acquire(ob_slot_pool *pool, int32_t timeout_ms, uint32_t *slot_id);
/* SlotPool::acquire_slot: that slot and no other (a request pinned to the slot that holds its prompt prefix). */
int ob_slot_acquire_id(ob_slot_pool *pool, uint32_t slot_id, int32_t timeout_ms);
/* Drop of SlotGuard: empties the slot's cache (its pages go back to the pool) and wakes the next waiter. */
int ob_slot_release(ob_slot_pool *pool, uint32_t slot_id);
/* prefill: the prompt in chunks of prefill_batch tokens, each continuing the cache; the last chunk's greedy token and/or
 * logits [n_vocab] come back (either may be NULL).  Other slots' decode batches run between the chunks. */
int ob_slot_prefill(ob_slot_pool *pool, uint32_t slot_id, const uint32_t *tokens, uint32_t n_tokens, uint32_t *out_token, float *out_logits);
/* BatchCoordinator::submit: one decode step of this slot's sequence.  Blocks until the batch it joined has run.  greedy may
 * be NULL (plain argmax); its n_recent[0] ids of `recent` are this sequence's penalty window.  A failed batch fails every
 * member with the same status. */
int ob_slot_decode(ob_slot_pool *pool, uint32_t slot_id, uint32_t token, const ob_greedy *greedy, uint32_t *out_token, float *out_logits);
int ob_slot_truncate(ob_slot_pool *pool, uint32_t slot_id, uint32_t new_len);
uint32_t ob_slot_len(const ob_slot_pool *pool, uint32_t slot_id);
ob_kv *ob_slot_kv(ob_slot_pool *pool, uint32_t slot_id);
/* SlotPool::snapshot: fills at most cap entries, returns the slot count. */
uint32_t ob_slot_pool_snapshot(ob_slot_pool *pool, ob_slot_state *out, uint32_t cap);
int ob_slot_pool_get_stats(ob_slot_pool *pool, ob_slot_pool_stats *out);
/* Text of the last failure on slot_id, or (slot_id < 0) of the calling thread's last failed pool call. */
const char *ob_slot_last_error(ob_slot_pool *pool, int64_t slot_id);
/* Host-only check of the pool and the window with a stand-in forward pass (no device, no model): n_threads generating
 * threads contend for n_slots slots and run n_steps decode steps each through the window.  OB_OK when every submitter got
 * its own answer, no slot had two holders and nothing leaked; `out` gets the totals. */
int ob_slot_pool_selftest(uint32_t n_slots, uint32_t n_threads, uint32_t n_steps, uint32_t batch_wait_ms, uint32_t max_queue, ob_slot_pool_stats *out);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
#ifdef __cplusplus
}
#endif
#endif /* ORANGU_B200_H */
