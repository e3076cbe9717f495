// Host runtime and C ABI (include/orangu_b200.h): contexts, device-resident weights, the paged
// KV pool, the Llama-style forward graph and its CUDA-graph decode step.
//
// Graph being reproduced (reference: src/bin/orangu-server/engine/arch/llama.rs:594-932, 1007-1032):
//   x = embed(tokens)
//   per layer:  h = rmsnorm(x, attn_norm); q,k,v = h.Wq, h.Wk, h.Wv; rope(q), rope(k); kv.push(k, v)
//               a = attention(q, kv); x += a.Wo
//               h = rmsnorm(x, ffn_norm); x += (silu(h.Wgate) * h.Wup).Wdown
//   logits = rmsnorm(x[last], output_norm).Woutput;  next = argmax(logits)
// Every product quantizes its input to int8 first (per 256 for Q4_K / Q6_K weights, per 32 for Q8_0);
// that quantisation is fused into the kernel that produces the input.
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <math.h>
#include <stdio.h>
#include <string.h>

#include <algorithm>
#include <mutex>
#include <string>
#include <vector>


#include "runtime.h"

static thread_local std::string g_init_error;

namespace obrt {

int fail(ob_ctx *ctx, int code, const std::string &msg) {
    if (ctx) ctx->err = msg;
    else g_init_error = msg;
    return code;
}

int ensure(ob_ctx *ctx, Scratch &s, size_t bytes) {
    if (bytes <= s.cap) return OB_OK;
    if (s.p) OB_CUDA(ctx, cudaFree(s.p));
    s.p = nullptr;
    s.cap = 0;
    size_t want = std::max(bytes, (size_t)1 << 20);
    OB_CUDA(ctx, cudaMalloc(&s.p, want));
    s.cap = want;
    return OB_OK;
}

bool type_supported(uint32_t t) { return t == TYPE_Q8_0 || t == TYPE_Q4_K || t == TYPE_Q5_K || t == TYPE_Q6_K || is_sym32_source(t); }

}  // namespace obrt

using namespace obrt;

extern "C" {

unsigned ob_abi_version(void) { return OB_ABI_VERSION; }

int ob_supports_type(uint32_t t) { return (t == TYPE_F32 || type_supported(t)) ? 1 : 0; }

const char *ob_reduced_surface(void) { return nullptr; }

const char *ob_last_error(const ob_ctx *ctx) { return ctx ? ctx->err.c_str() : g_init_error.c_str(); }

uint64_t ob_launch_count(const ob_ctx *ctx) { return ctx ? ctx->launches : 0; }
float ob_last_device_ms(const ob_ctx *ctx) { return ctx ? ctx->last_ms : 0.0f; }

int ob_init(int device_ordinal, ob_ctx **out) {
    if (!out) return fail(nullptr, OB_ERR_INVALID, "ob_init: out is null");
    *out = nullptr;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n == 0) return fail(nullptr, OB_ERR_NO_DEVICE, std::string("no CUDA device: ") + cudaGetErrorString(e));
    int dev = device_ordinal;
    if (dev < 0 && cudaGetDevice(&dev) != cudaSuccess) dev = 0;
    if (dev >= n) return fail(nullptr, OB_ERR_NO_DEVICE, "device ordinal out of range");
    cudaDeviceProp prop;
    if ((e = cudaGetDeviceProperties(&prop, dev)) != cudaSuccess) return fail(nullptr, OB_ERR_CUDA, cudaGetErrorString(e));
    if (prop.major != 10) {
        char buf[160];
        snprintf(buf, sizeof buf, "device %d (%s) is sm_%d%d; this library carries sm_100a code only", dev, prop.name, prop.major, prop.minor);
        return fail(nullptr, OB_ERR_NO_DEVICE, buf);
    }
    ob_ctx *ctx = new ob_ctx;
    ctx->device = dev;
    ctx->sm_count = prop.multiProcessorCount;
    int prev = 0;
    cudaGetDevice(&prev);
    cudaSetDevice(dev);
    e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaEventCreate(&ctx->ev0);
    if (e == cudaSuccess) e = cudaEventCreate(&ctx->ev1);
    cudaSetDevice(prev);
    if (e != cudaSuccess) {
        std::string msg = cudaGetErrorString(e);
        delete ctx;
        return fail(nullptr, OB_ERR_CUDA, msg);
    }
    *out = ctx;
    return OB_OK;
}

void ob_destroy(ob_ctx *ctx) {
    if (!ctx) return;
    Bind b(ctx);
    cudaStreamSynchronize(ctx->stream);
    for (Scratch *s : {&ctx->sx, &ctx->sy, &ctx->sq, &ctx->sd, &ctx->ss, &ctx->saux, &ctx->saux2, &ctx->saux3})
        if (s->p) cudaFree(s->p);
    cudaEventDestroy(ctx->ev0);
    cudaEventDestroy(ctx->ev1);
    cudaStreamDestroy(ctx->stream);
    delete ctx;
}

int ob_synchronize(ob_ctx *ctx) {
    if (!ctx) return OB_ERR_INVALID;
    Bind b(ctx);
    OB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (gemm_tc5_take_status()) return fail(ctx, OB_ERR_CUDA, "a tensor-core product gave up a bounded wait (pipeline barrier); its output is not valid");
    return OB_OK;
}

}  // extern "C"

// ------------------------------------------------------------------------------------ weights

namespace obrt {

int make_weight(ob_ctx *ctx, const uint8_t *raw, uint64_t row_bytes, uint32_t type, uint32_t in_dim, uint32_t out_dim, uint32_t row0,
                uint32_t n_rows, uint32_t col0, uint32_t n_cols, ob_weight **out) {
    const bool raw_on_device = false;
    if (!ctx || !raw || !out) return fail(ctx, OB_ERR_INVALID, "weight: null argument");
    *out = nullptr;
    if (!type_supported(type)) return fail(ctx, OB_ERR_UNSUPPORTED, "weight: ggml type " + std::to_string(type) + " has no kernel here");
    const uint32_t be = block_elems(type), bb = block_bytes_gguf(type);
    if (in_dim == 0 || out_dim == 0 || in_dim % be) return fail(ctx, OB_ERR_UNSUPPORTED, "weight: in_dim must be a positive multiple of the block size");
    if (row_bytes != (uint64_t)(in_dim / be) * bb) return fail(ctx, OB_ERR_INVALID, "weight: row_bytes does not match type and in_dim");
    if (n_rows == 0 || n_cols == 0 || (uint64_t)row0 + n_rows > out_dim || (uint64_t)col0 + n_cols > in_dim || col0 % be || n_cols % be)
        return fail(ctx, OB_ERR_INVALID, "weight: slice out of range or not block aligned");
    Bind b(ctx);
    ob_weight *w = new ob_weight;
    w->ctx = ctx;
    DevWeight &d = w->w;
    d.type = is_sym32_source(type) ? TYPE_Q8_0 : type;  // Q4_0, Q5_0, IQ4_NL are held as their unpacked int8 codes + f16 scale
    d.in_dim = n_cols;
    d.out_dim = n_rows;
    d.nb = n_cols / be;
    const uint32_t main_bytes = d.type == TYPE_Q4_K ? 144u : d.type == TYPE_Q5_K ? 176u : (d.type == TYPE_Q6_K ? 208u : 32u);
    d.d_off = d.nb * main_bytes;
    const uint64_t row_size = (uint64_t)d.nb * block_bytes_gguf(d.type);
    d.row_stride = (row_size + 15) & ~(uint64_t)15;
    w->bytes = d.row_stride * n_rows;
    void *mem = nullptr;
    cudaError_t e = cudaMalloc(&mem, w->bytes);
    if (e != cudaSuccess) {
        delete w;
        return fail(ctx, OB_ERR_OOM, std::string("weight: cudaMalloc: ") + cudaGetErrorString(e));
    }
    w->mem = mem;
    d.data = static_cast<const uint8_t *>(mem);
    // stage the needed source rows, then re-lay on the device
    const uint8_t *src_dev = raw + (raw_on_device ? (uint64_t)row0 * row_bytes : 0);
    void *staging = nullptr;
    if (!raw_on_device) {
        const uint64_t src_bytes = row_bytes * n_rows;
        e = cudaMalloc(&staging, src_bytes);
        if (e == cudaSuccess) e = cudaMemcpyAsync(staging, raw + (uint64_t)row0 * row_bytes, src_bytes, cudaMemcpyHostToDevice, ctx->stream);
        if (e != cudaSuccess) {
            if (staging) cudaFree(staging);
            cudaFree(mem);
            delete w;
            return fail(ctx, e == cudaErrorMemoryAllocation ? OB_ERR_OOM : OB_ERR_CUDA, std::string("weight upload: ") + cudaGetErrorString(e));
        }
        src_dev = static_cast<const uint8_t *>(staging);
    }
    if (d.row_stride != row_size) cudaMemsetAsync(mem, 0, w->bytes, ctx->stream);
    launch_repack(src_dev, row_bytes, type, 0, col0 / be, d, ctx->stream);
    ctx->launches++;
    e = cudaStreamSynchronize(ctx->stream);
    if (e == cudaSuccess) e = cudaGetLastError();
    if (staging) cudaFree(staging);
    if (e != cudaSuccess) {
        cudaFree(mem);
        delete w;
        return fail(ctx, OB_ERR_CUDA, std::string("weight re-layout: ") + cudaGetErrorString(e));
    }
    *out = w;
    return OB_OK;
}

}  // namespace obrt

extern "C" {

int ob_weight_register(ob_ctx *ctx, const uint8_t *raw, uint64_t row_bytes, uint32_t type, uint32_t in_dim, uint32_t out_dim, ob_weight **out) {
    if (!ctx) return OB_ERR_INVALID;
    std::lock_guard<std::mutex> g(ctx->mu);
    return make_weight(ctx, raw, row_bytes, type, in_dim, out_dim, 0, out_dim, 0, in_dim, out);
}

int ob_weight_register_slice(ob_ctx *ctx, const uint8_t *raw, uint64_t row_bytes, uint32_t type, uint32_t in_dim, uint32_t out_dim,
                             uint32_t row0, uint32_t n_rows, uint32_t col0, uint32_t n_cols, ob_weight **out) {
    if (!ctx) return OB_ERR_INVALID;
    std::lock_guard<std::mutex> g(ctx->mu);
    return make_weight(ctx, raw, row_bytes, type, in_dim, out_dim, row0, n_rows, col0, n_cols, out);
}

void ob_weight_release(ob_ctx *ctx, ob_weight *w) {
    if (!w) return;
    ob_ctx *c = ctx ? ctx : w->ctx;
    std::lock_guard<std::mutex> g(c->mu);
    Bind b(c);
    cudaStreamSynchronize(c->stream);
    cudaFree(w->mem);
    delete w;
}

int ob_weight_dequantize(ob_ctx *ctx, const ob_weight *w, uint32_t first_row, uint32_t n_rows, float *out_host) {
    if (!ctx || !w || !out_host) return fail(ctx, OB_ERR_INVALID, "dequantize: null argument");
    std::lock_guard<std::mutex> g(ctx->mu);
    if ((uint64_t)first_row + n_rows > w->w.out_dim) return fail(ctx, OB_ERR_INVALID, "dequantize: rows out of range");
    if (n_rows == 0) return OB_OK;
    Bind b(ctx);
    const size_t bytes = (size_t)n_rows * w->w.in_dim * 4;
    int rc = ensure(ctx, ctx->sy, bytes);
    if (rc) return rc;
    launch_dequant_rows(w->w, first_row, n_rows, static_cast<float *>(ctx->sy.p), ctx->stream);
    ctx->launches++;
    OB_CUDA(ctx, cudaMemcpyAsync(out_host, ctx->sy.p, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    OB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return OB_OK;
}

}  // extern "C"

// ------------------------------------------------------------------------------------ matmul

namespace {

// Quantize x_dev [n_tokens][in_dim] with the granularity `type` wants, into ctx scratch.
int quantize_for(ob_ctx *ctx, const float *x_dev, uint32_t n_tokens, uint32_t in_dim, uint32_t type, ActBuf *act, cudaStream_t st) {
    const uint32_t grp = type == TYPE_Q8_0 ? 32u : 256u;
    int rc;
    if ((rc = ensure(ctx, ctx->sq, (size_t)n_tokens * in_dim))) return rc;
    if ((rc = ensure(ctx, ctx->sd, (size_t)n_tokens * (in_dim / grp) * 4))) return rc;
    if ((rc = ensure(ctx, ctx->ss, (size_t)n_tokens * (in_dim / 16) * 2))) return rc;
    act->q = static_cast<int8_t *>(ctx->sq.p);
    act->d = static_cast<float *>(ctx->sd.p);
    act->sums = static_cast<int16_t *>(ctx->ss.p);
    act->dim_cap = in_dim;
    QuantArgs qa{};
    qa.x = x_dev;
    qa.n_rows = n_tokens;
    qa.dim = in_dim;
    if (type == TYPE_Q8_0) qa.flat = *act;
    else qa.k = *act;
    launch_quantize(ACT_PLAIN, qa, st);
    ctx->launches++;
    return OB_OK;
}

int matmul_device(ob_ctx *ctx, const float *x_dev, uint32_t n_tokens, const ob_weight *w, float *y_dev, bool decode, cudaStream_t st,
                  int32_t *isum_out, int32_t *imin_out, uint32_t first_row, uint32_t n_rows) {
    if (n_tokens == 1 && !isum_out && (w->w.type == TYPE_Q4_K || w->w.type == TYPE_Q6_K)) {
        // one token, K-type weights: the streaming kernel of the decode step, quantizing the row in its prologue (one launch)
        StreamArgs sa{};
        sa.n_seg = 1;
        sa.in_dim = w->w.in_dim;
        sa.prologue = SG_PRO_PLAIN;
        sa.x = x_dev;
        sa.seg[0] = StreamSeg{w->w, DevWeight{}, y_dev, SG_EP_STORE};
        if (stream_gemv_supported(sa)) {
            // programmatic serialisation: the kernel requests its first weights while the previous work on the stream is
            // finishing and waits for it before it reads x or writes y, so stream order is kept
            launch_stream_gemv(sa, ctx->sm_count, true, st);
            ctx->launches++;
            return OB_OK;
        }
    }
    // one token, Q8_0: the product kernel quantizes the row in its prologue (one launch instead of two)
    const bool fused_q8 = n_tokens == 1 && w->w.type == TYPE_Q8_0;
    ActBuf act{};
    if (!fused_q8) {
        int rc = quantize_for(ctx, x_dev, n_tokens, w->w.in_dim, w->w.type, &act, st);
        if (rc) return rc;
    }
    GemvArgs a{};
    a.x_f32 = fused_q8 ? x_dev : nullptr;
    a.n_seg = 1;
    a.seg[0].w = w->w;
    if (isum_out) {  // row window for the partial-sum capture
        a.seg[0].w.data += (uint64_t)first_row * w->w.row_stride;
        a.seg[0].w.out_dim = n_rows;
    }
    a.seg[0].y = y_dev;
    a.seg[0].y_stride = a.seg[0].w.out_dim;
    a.seg[0].epilogue = EPI_STORE;
    a.act = act;
    a.n_tokens = n_tokens;
    a.gemm_order = !decode && n_tokens > 1;
    a.isum_out = isum_out;
    a.imin_out = imin_out;
    launch_gemv(a, ctx->sm_count, st);
    ctx->launches += gemv_launches(w->w.type, w->w.in_dim, n_tokens, a.gemm_order && w->w.type != TYPE_Q8_0);
    return OB_OK;
}

int matmul_host(ob_ctx *ctx, const float *x, uint32_t n_tokens, const ob_weight *w, float *y, bool decode) {
    if (!ctx || !x || !w || !y) return fail(ctx, OB_ERR_INVALID, "matmul: null argument");
    if (w->ctx != ctx) return fail(ctx, OB_ERR_INVALID, "matmul: weight belongs to another context");
    if (n_tokens == 0) return OB_OK;
    Bind b(ctx);
    const size_t xb = (size_t)n_tokens * w->w.in_dim * 4, yb = (size_t)n_tokens * w->w.out_dim * 4;
    int rc;
    if ((rc = ensure(ctx, ctx->sx, xb))) return rc;
    if ((rc = ensure(ctx, ctx->sy, yb))) return rc;
    OB_CUDA(ctx, cudaMemcpyAsync(ctx->sx.p, x, xb, cudaMemcpyHostToDevice, ctx->stream));
    rc = matmul_device(ctx, static_cast<const float *>(ctx->sx.p), n_tokens, w, static_cast<float *>(ctx->sy.p), decode, ctx->stream, nullptr,
                       nullptr, 0, 0);
    if (rc) return rc;
    OB_CUDA(ctx, cudaMemcpyAsync(y, ctx->sy.p, yb, cudaMemcpyDeviceToHost, ctx->stream));
    OB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (gemm_tc5_take_status()) return fail(ctx, OB_ERR_CUDA, "a tensor-core product gave up a bounded wait (pipeline barrier); its output is not valid");
    OB_CUDA(ctx, cudaGetLastError());
    return OB_OK;
}

}  // namespace

extern "C" {

int ob_matmul(ob_ctx *ctx, const float *x, uint32_t n_tokens, const ob_weight *w, float *y) {
    if (!ctx) return OB_ERR_INVALID;
    std::lock_guard<std::mutex> g(ctx->mu);
    return matmul_host(ctx, x, n_tokens, w, y, false);
}

int ob_matmul_decode(ob_ctx *ctx, const float *x, uint32_t n_tokens, const ob_weight *w, float *y) {
    if (!ctx) return OB_ERR_INVALID;
    std::lock_guard<std::mutex> g(ctx->mu);
    return matmul_host(ctx, x, n_tokens, w, y, true);
}

int ob_matmul_batch(ob_ctx *ctx, const ob_matmul_op *ops, uint32_t n_ops, int decode) {
    if (!ctx || (!ops && n_ops)) return fail(ctx, OB_ERR_INVALID, "matmul_batch: null argument");
    std::lock_guard<std::mutex> g(ctx->mu);
    // Ops share no data (reference: backend/mod.rs:121-125).  Inputs go up together, the products are
    // queued back to back on the stream, and there is one synchronisation for the whole batch.
    Bind b(ctx);
    size_t xb = 0, yb = 0;
    for (uint32_t i = 0; i < n_ops; ++i) {
        const ob_matmul_op &op = ops[i];
        if (!op.x || !op.w || !op.y) return fail(ctx, OB_ERR_INVALID, "matmul_batch: null pointer in op");
        if (op.w->ctx != ctx) return fail(ctx, OB_ERR_INVALID, "matmul_batch: weight belongs to another context");
        xb += (size_t)op.n_tokens * op.w->w.in_dim * 4;
        yb += (size_t)op.n_tokens * op.w->w.out_dim * 4;
    }
    int rc;
    if ((rc = ensure(ctx, ctx->sx, xb))) return rc;
    if ((rc = ensure(ctx, ctx->sy, yb))) return rc;
    size_t xo = 0, yo = 0;
    for (uint32_t i = 0; i < n_ops; ++i) {
        const ob_matmul_op &op = ops[i];
        if (op.n_tokens == 0) continue;
        const size_t xi = (size_t)op.n_tokens * op.w->w.in_dim * 4, yi = (size_t)op.n_tokens * op.w->w.out_dim * 4;
        float *xd = reinterpret_cast<float *>(static_cast<uint8_t *>(ctx->sx.p) + xo), *yd = reinterpret_cast<float *>(static_cast<uint8_t *>(ctx->sy.p) + yo);
        OB_CUDA(ctx, cudaMemcpyAsync(xd, op.x, xi, cudaMemcpyHostToDevice, ctx->stream));
        if ((rc = matmul_device(ctx, xd, op.n_tokens, op.w, yd, decode != 0, ctx->stream, nullptr, nullptr, 0, 0))) return rc;
        OB_CUDA(ctx, cudaMemcpyAsync(op.y, yd, yi, cudaMemcpyDeviceToHost, ctx->stream));
        xo += xi;
        yo += yi;
    }
    OB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (gemm_tc5_take_status()) return fail(ctx, OB_ERR_CUDA, "a tensor-core product gave up a bounded wait (pipeline barrier); its output is not valid");
    OB_CUDA(ctx, cudaGetLastError());
    return OB_OK;
}

int ob_matmul_device(ob_ctx *ctx, const float *x_dev, uint32_t n_tokens, const ob_weight *w, float *y_dev, int decode, void *stream) {
    if (!ctx || !x_dev || !w || !y_dev) return fail(ctx, OB_ERR_INVALID, "matmul_device: null argument");
    std::lock_guard<std::mutex> g(ctx->mu);
    if (n_tokens == 0) return OB_OK;
    Bind b(ctx);
    cudaStream_t st = stream ? static_cast<cudaStream_t>(stream) : ctx->stream;
    int rc = matmul_device(ctx, x_dev, n_tokens, w, y_dev, decode != 0, st, nullptr, nullptr, 0, 0);
    if (rc) return rc;
    OB_CUDA(ctx, cudaGetLastError());
    return OB_OK;
}

int ob_matmul_partials(ob_ctx *ctx, const float *x, const ob_weight *w, uint32_t first_row, uint32_t n_rows, int32_t *isum, int32_t *imin) {
    if (!ctx || !x || !w || !isum) return fail(ctx, OB_ERR_INVALID, "matmul_partials: null argument");
    std::lock_guard<std::mutex> g(ctx->mu);
    if ((uint64_t)first_row + n_rows > w->w.out_dim) return fail(ctx, OB_ERR_INVALID, "matmul_partials: rows out of range");
    if (n_rows == 0) return OB_OK;
    Bind b(ctx);
    const size_t xb = (size_t)w->w.in_dim * 4, pb = (size_t)n_rows * w->w.nb * 4;
    int rc;
    if ((rc = ensure(ctx, ctx->sx, xb))) return rc;
    if ((rc = ensure(ctx, ctx->sy, (size_t)n_rows * 4))) return rc;
    if ((rc = ensure(ctx, ctx->saux, pb))) return rc;
    if ((rc = ensure(ctx, ctx->saux2, pb))) return rc;
    OB_CUDA(ctx, cudaMemcpyAsync(ctx->sx.p, x, xb, cudaMemcpyHostToDevice, ctx->stream));
    rc = matmul_device(ctx, static_cast<const float *>(ctx->sx.p), 1, w, static_cast<float *>(ctx->sy.p), true, ctx->stream,
                       static_cast<int32_t *>(ctx->saux.p), static_cast<int32_t *>(ctx->saux2.p), first_row, n_rows);
    if (rc) return rc;
    OB_CUDA(ctx, cudaMemcpyAsync(isum, ctx->saux.p, pb, cudaMemcpyDeviceToHost, ctx->stream));
    if (imin) OB_CUDA(ctx, cudaMemcpyAsync(imin, ctx->saux2.p, pb, cudaMemcpyDeviceToHost, ctx->stream));
    OB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    OB_CUDA(ctx, cudaGetLastError());
    return OB_OK;
}

// ------------------------------------------------------------------------------------ glue ops

int ob_rmsnorm(ob_ctx *ctx, const float *x, const float *weight, uint32_t n_tokens, uint32_t dim, float eps, float *out) {
    if (!ctx || !x || !weight || !out || dim == 0) return fail(ctx, OB_ERR_INVALID, "rmsnorm: bad argument");
    std::lock_guard<std::mutex> g(ctx->mu);
    if (n_tokens == 0) return OB_OK;
    Bind b(ctx);
    const size_t xb = (size_t)n_tokens * dim * 4;
    int rc;
    if ((rc = ensure(ctx, ctx->sx, xb))) return rc;
    if ((rc = ensure(ctx, ctx->sy, xb))) return rc;
    if ((rc = ensure(ctx, ctx->saux, (size_t)dim * 4))) return rc;
    OB_CUDA(ctx, cudaMemcpyAsync(ctx->sx.p, x, xb, cudaMemcpyHostToDevice, ctx->stream));
    OB_CUDA(ctx, cudaMemcpyAsync(ctx->saux.p, weight, (size_t)dim * 4, cudaMemcpyHostToDevice, ctx->stream));
    launch_rmsnorm(static_cast<float *>(ctx->sx.p), static_cast<float *>(ctx->saux.p), n_tokens, dim, eps, static_cast<float *>(ctx->sy.p), ctx->stream);
    ctx->launches++;
    OB_CUDA(ctx, cudaMemcpyAsync(out, ctx->sy.p, xb, cudaMemcpyDeviceToHost, ctx->stream));
    OB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return OB_OK;
}

int ob_rope(ob_ctx *ctx, float *x, uint32_t n_head, uint32_t head_dim, uint32_t pos, uint32_t rope_dim, float freq_base) {
    if (!ctx || !x || head_dim == 0 || rope_dim > head_dim || (rope_dim & 1) || (head_dim & 1)) return fail(ctx, OB_ERR_INVALID, "rope: bad argument");
    std::lock_guard<std::mutex> g(ctx->mu);
    Bind b(ctx);
    const uint32_t half = rope_dim / 2;
    // The rotation angles come from the host's libm, exactly as the reference computes them
    // (engine/tensor.rs:1140-1160); the device only applies them.
    std::vector<float> sc(half * 2);
    for (uint32_t i = 0; i < half; ++i) {
        float freq = powf(freq_base, -2.0f * (float)i / (float)rope_dim);
        float theta = 1.0f * ((float)pos * freq);
        sc[2 * i] = sinf(theta) * 1.0f;
        sc[2 * i + 1] = cosf(theta) * 1.0f;
    }
    const size_t xb = (size_t)n_head * head_dim * 4;
    int rc;
    if ((rc = ensure(ctx, ctx->sx, xb))) return rc;
    if ((rc = ensure(ctx, ctx->saux, sc.size() * 4 + 16))) return rc;
    OB_CUDA(ctx, cudaMemcpyAsync(ctx->sx.p, x, xb, cudaMemcpyHostToDevice, ctx->stream));
    OB_CUDA(ctx, cudaMemcpyAsync(ctx->saux.p, sc.data(), sc.size() * 4, cudaMemcpyHostToDevice, ctx->stream));
    launch_rope_plain(static_cast<float *>(ctx->sx.p), n_head, head_dim, rope_dim, static_cast<float *>(ctx->saux.p), ctx->stream);
    ctx->launches++;
    OB_CUDA(ctx, cudaMemcpyAsync(x, ctx->sx.p, xb, cudaMemcpyDeviceToHost, ctx->stream));
    OB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return OB_OK;
}

int ob_swiglu(ob_ctx *ctx, const float *gate, const float *up, uint32_t n, float *out) {
    if (!ctx || !gate || !up || !out) return fail(ctx, OB_ERR_INVALID, "swiglu: null argument");
    std::lock_guard<std::mutex> g(ctx->mu);
    if (n == 0) return OB_OK;
    Bind b(ctx);
    const size_t nb = (size_t)n * 4;
    int rc;
    if ((rc = ensure(ctx, ctx->sx, nb))) return rc;
    if ((rc = ensure(ctx, ctx->sy, nb))) return rc;
    if ((rc = ensure(ctx, ctx->saux, nb))) return rc;
    OB_CUDA(ctx, cudaMemcpyAsync(ctx->sx.p, gate, nb, cudaMemcpyHostToDevice, ctx->stream));
    OB_CUDA(ctx, cudaMemcpyAsync(ctx->saux.p, up, nb, cudaMemcpyHostToDevice, ctx->stream));
    launch_swiglu(static_cast<float *>(ctx->sx.p), static_cast<float *>(ctx->saux.p), n, static_cast<float *>(ctx->sy.p), ctx->stream);
    ctx->launches++;
    OB_CUDA(ctx, cudaMemcpyAsync(out, ctx->sy.p, nb, cudaMemcpyDeviceToHost, ctx->stream));
    OB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return OB_OK;
}

int ob_quantize_act(ob_ctx *ctx, const float *x, uint32_t n, int per_256, int8_t *q, float *d, int32_t *sums) {
    const uint32_t grp = per_256 ? 256u : 32u;
    if (!ctx || !x || !q || !d || n == 0 || n % grp) return fail(ctx, OB_ERR_INVALID, "quantize_act: bad argument");
    std::lock_guard<std::mutex> g(ctx->mu);
    Bind b(ctx);
    int rc;
    if ((rc = ensure(ctx, ctx->sx, (size_t)n * 4))) return rc;
    OB_CUDA(ctx, cudaMemcpyAsync(ctx->sx.p, x, (size_t)n * 4, cudaMemcpyHostToDevice, ctx->stream));
    ActBuf act;
    if ((rc = quantize_for(ctx, static_cast<float *>(ctx->sx.p), 1, n, per_256 ? TYPE_Q4_K : TYPE_Q8_0, &act, ctx->stream))) return rc;
    std::vector<int16_t> s16(n / 16);
    OB_CUDA(ctx, cudaMemcpyAsync(q, act.q, n, cudaMemcpyDeviceToHost, ctx->stream));
    OB_CUDA(ctx, cudaMemcpyAsync(d, act.d, (size_t)(n / grp) * 4, cudaMemcpyDeviceToHost, ctx->stream));
    OB_CUDA(ctx, cudaMemcpyAsync(s16.data(), act.sums, s16.size() * 2, cudaMemcpyDeviceToHost, ctx->stream));
    OB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (sums)
        for (size_t i = 0; i < s16.size(); ++i) sums[i] = s16[i];
    return OB_OK;
}

int ob_argmax(ob_ctx *ctx, const float *logits, uint32_t n_vocab, const uint32_t *recent, uint32_t n_recent, uint32_t repeat_last_n,
              float penalty, uint32_t *out_token) {
    if (!ctx || !logits || !out_token || n_vocab == 0) return fail(ctx, OB_ERR_INVALID, "argmax: bad argument");
    std::lock_guard<std::mutex> g(ctx->mu);
    Bind b(ctx);
    int rc;
    if ((rc = ensure(ctx, ctx->sx, (size_t)n_vocab * 4))) return rc;
    if ((rc = ensure(ctx, ctx->saux, 64))) return rc;
    OB_CUDA(ctx, cudaMemcpyAsync(ctx->sx.p, logits, (size_t)n_vocab * 4, cudaMemcpyHostToDevice, ctx->stream));
    if (recent && n_recent && penalty != 1.0f) {
        const uint32_t start = n_recent > repeat_last_n ? n_recent - repeat_last_n : 0, cnt = n_recent - start;
        if (cnt) {
            if ((rc = ensure(ctx, ctx->saux2, (size_t)cnt * 4))) return rc;
            OB_CUDA(ctx, cudaMemcpyAsync(ctx->saux2.p, recent + start, (size_t)cnt * 4, cudaMemcpyHostToDevice, ctx->stream));
            launch_repeat_penalty(static_cast<float *>(ctx->sx.p), n_vocab, static_cast<uint32_t *>(ctx->saux2.p), cnt, penalty, ctx->stream);
            ctx->launches++;
        }
    }
    ArgmaxArgs a{};
    a.logits = static_cast<float *>(ctx->sx.p);
    a.n_seq = 1;
    a.n_vocab = n_vocab;
    a.scratch = static_cast<unsigned long long *>(ctx->saux.p);
    a.out = reinterpret_cast<uint32_t *>(static_cast<uint8_t *>(ctx->saux.p) + 16);
    launch_argmax(a, ctx->stream);
    ctx->launches += 3;
    OB_CUDA(ctx, cudaMemcpyAsync(out_token, a.out, 4, cudaMemcpyDeviceToHost, ctx->stream));
    OB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return OB_OK;
}

int ob_attention_decode(ob_ctx *ctx, const float *q, const float *k, const float *v, uint32_t n_pos, uint32_t n_head, uint32_t n_head_kv,
                        uint32_t head_dim, float scale, int exact_order, float *out) {
    if (!ctx || !q || !k || !v || !out || n_head == 0 || n_head_kv == 0 || head_dim == 0 || (head_dim & 1) || head_dim > 256)
        return fail(ctx, OB_ERR_INVALID, "attention_decode: bad argument");
    std::lock_guard<std::mutex> g(ctx->mu);
    Bind b(ctx);
    const uint32_t kv_dim = n_head_kv * head_dim, q_dim = n_head * head_dim;
    const uint32_t n_pages = std::max(1u, (n_pos + KV_PAGE - 1) / KV_PAGE);
    // Build a one-layer page pool from the f32 rows: identity page table, K/V rounded to f16.
    std::vector<__half> kp((size_t)n_pages * n_head_kv * KV_PAGE * head_dim, __float2half(0.0f)), vp(kp.size(), __float2half(0.0f));
    for (uint32_t p = 0; p < n_pos; ++p)
        for (uint32_t h = 0; h < n_head_kv; ++h)
            for (uint32_t d = 0; d < head_dim; ++d) {
                size_t o = (((size_t)(p / KV_PAGE) * n_head_kv + h) * KV_PAGE + p % KV_PAGE) * head_dim + d;
                kp[o] = __float2half_rn(k[(size_t)p * kv_dim + h * head_dim + d]);
                vp[o] = __float2half_rn(v[(size_t)p * kv_dim + h * head_dim + d]);
            }
    std::vector<int32_t> table(n_pages);
    for (uint32_t i = 0; i < n_pages; ++i) table[i] = (int32_t)i;
    const uint32_t n_splits = std::max(1u, std::min(16u, n_pages / 4));
    const size_t pool_b = kp.size() * 2, part_o_b = (size_t)n_head * n_splits * head_dim * 4, part_ml_b = (size_t)n_head * n_splits * 8;
    const size_t meta_b = 256 + (size_t)n_pages * 4;
    if (exact_order == 1 && !attn_exact_supported(n_head, n_head_kv, head_dim))
        return fail(ctx, OB_ERR_UNSUPPORTED, "attention_decode: exact order needs head_dim % 16 == 0 and a group of 1, 2, 3, 4 or 8 heads");
    int rc;
    if ((rc = ensure(ctx, ctx->sx, (size_t)q_dim * 4))) return rc;
    if ((rc = ensure(ctx, ctx->sy, (size_t)q_dim * 4))) return rc;
    if ((rc = ensure(ctx, ctx->saux, pool_b * 2))) return rc;
    if ((rc = ensure(ctx, ctx->saux2, part_o_b + part_ml_b))) return rc;
    if ((rc = ensure(ctx, ctx->saux3, meta_b))) return rc;
    uint8_t *meta = static_cast<uint8_t *>(ctx->saux3.p);
    int32_t *d_table = reinterpret_cast<int32_t *>(meta + 256);
    struct {
        const int32_t *table_ptr;
        uint32_t n_pos;
    } hmeta = {d_table, n_pos};
    OB_CUDA(ctx, cudaMemcpyAsync(ctx->sx.p, q, (size_t)q_dim * 4, cudaMemcpyHostToDevice, ctx->stream));
    OB_CUDA(ctx, cudaMemcpyAsync(ctx->saux.p, kp.data(), pool_b, cudaMemcpyHostToDevice, ctx->stream));
    OB_CUDA(ctx, cudaMemcpyAsync(static_cast<uint8_t *>(ctx->saux.p) + pool_b, vp.data(), pool_b, cudaMemcpyHostToDevice, ctx->stream));
    OB_CUDA(ctx, cudaMemcpyAsync(meta, &hmeta.table_ptr, 8, cudaMemcpyHostToDevice, ctx->stream));
    OB_CUDA(ctx, cudaMemcpyAsync(meta + 64, &hmeta.n_pos, 4, cudaMemcpyHostToDevice, ctx->stream));
    OB_CUDA(ctx, cudaMemcpyAsync(d_table, table.data(), (size_t)n_pages * 4, cudaMemcpyHostToDevice, ctx->stream));
    AttnDecodeArgs a{};
    a.q = static_cast<float *>(ctx->sx.p);
    a.out = static_cast<float *>(ctx->sy.p);
    a.k_pool = static_cast<__half *>(ctx->saux.p);
    a.v_pool = reinterpret_cast<__half *>(static_cast<uint8_t *>(ctx->saux.p) + pool_b);
    a.page_tables = reinterpret_cast<const int32_t *const *>(meta);
    a.n_pos = reinterpret_cast<const uint32_t *>(meta + 64);
    a.n_seq = 1;
    a.n_head = n_head;
    a.n_head_kv = n_head_kv;
    a.head_dim = head_dim;
    a.scale = scale;
    a.n_splits = n_splits;
    a.part_o = static_cast<float *>(ctx->saux2.p);
    a.part_ml = reinterpret_cast<float *>(static_cast<uint8_t *>(ctx->saux2.p) + part_o_b);
    a.max_pos = n_pos;
    if (exact_order == 1) {
        const uint32_t stride = (n_pos + 63) / 64 * 64;
        if ((rc = ensure(ctx, ctx->sq, (size_t)n_head * stride * 4))) return rc;
        AttnExactArgs e{};
        e.q = a.q;
        e.out = a.out;
        e.k_pool = a.k_pool;
        e.v_pool = a.v_pool;
        e.page_tables = a.page_tables;
        e.n_pos = a.n_pos;
        e.scores = static_cast<float *>(ctx->sq.p);
        e.score_stride = stride;
        e.n_rows = 1;
        e.n_head = n_head;
        e.n_head_kv = n_head_kv;
        e.head_dim = head_dim;
        e.scale = scale;
        e.max_pos = n_pos;
        launch_attn_exact(e, ctx->stream);
        ctx->launches += 3;
    } else if (exact_order == 2 || exact_order == 3) {  // the one-kernel form the decode step uses (3: its large-batch shape, CTAs of four warps)
        a.small_ctas = exact_order == 3;
        a.counters = reinterpret_cast<uint32_t *>(meta + 128);
        OB_CUDA(ctx, cudaMemsetAsync(a.counters, 0, 128, ctx->stream));
        if (n_head_kv > 32 || !launch_attn_decode_fused(a, false, ctx->stream))
            return fail(ctx, OB_ERR_UNSUPPORTED, "attention_decode: the fused kernel needs head_dim 64 or 128 and 1, 2, 4 or 8 heads per kv head");
        ctx->launches += 1;
    } else {
        launch_attn_decode(a, ctx->stream);
        ctx->launches += 2;
    }
    OB_CUDA(ctx, cudaMemcpyAsync(out, ctx->sy.p, (size_t)q_dim * 4, cudaMemcpyDeviceToHost, ctx->stream));
    OB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    OB_CUDA(ctx, cudaGetLastError());
    return OB_OK;
}

}  // extern "C"
