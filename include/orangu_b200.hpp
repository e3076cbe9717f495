// C++ host-side mirror of the reference engine's `Backend` trait over the C ABI of orangu_b200.h.
//
// The reference's host code is Rust (src/bin/orangu-server/engine/backend/mod.rs:309-496, trait Backend;
// src/bin/orangu-server/engine/loader.rs:561-680, QuantMatrix).  Where no Rust toolchain exists this
// header is the compiled-language form of the same surface: same method names, same argument meaning
// (x is [n_tokens, in_dim] row-major, the result [n_tokens, out_dim]), same construction contract
// (try_init_index returns an empty optional instead of failing loudly) and the same failure behaviour
// after construction (the reference panics; this throws std::runtime_error with the library's text).
#pragma once

#include <cstdint>
#include <memory>
#include <optional>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

#include "orangu_b200.h"

namespace orangu {

// loader.rs:561-680: a 2-D tensor in its GGUF block layout; the bytes are borrowed, as an mmap is.
struct QuantMatrix {
    const uint8_t *bytes = nullptr;
    uint32_t ggml_type = 0;
    uint32_t in_dim = 0;   // dims[0], contiguous
    uint32_t out_dim = 0;  // dims[1]
    // block_layout (engine/quant.rs:132-169): elements and bytes per block of the types this backend takes
    uint64_t row_bytes() const {
        uint32_t be = 256, bb = 210;  // Q6_K
        switch (ggml_type) {
        case OB_TYPE_Q8_0: be = 32; bb = 34; break;
        case OB_TYPE_Q4_0: case OB_TYPE_IQ4_NL: be = 32; bb = 18; break;
        case OB_TYPE_Q5_0: be = 32; bb = 22; break;
        case OB_TYPE_Q4_K: be = 256; bb = 144; break;
        case OB_TYPE_Q5_K: be = 256; bb = 176; break;
        default: break;
        }
        return (uint64_t)(in_dim / be) * bb;
    }
    // loader.rs:627-646
    QuantMatrix rows(uint32_t first, uint32_t count) const { return {bytes + (uint64_t)first * row_bytes(), ggml_type, in_dim, count}; }
    // loader.rs:674-679: identity of the mapping, the key a backend caches its device copy under
    std::pair<const void *, uint64_t> cache_key() const { return {bytes, row_bytes() * out_dim}; }
};

struct MatmulOp {  // backend/mod.rs:117-121
    const float *x;
    uint32_t n_tokens;
    const QuantMatrix *w;
};

class CudaBackend {
  public:
    // backend/cuda.rs:86-124: never throws; empty on any failure.
    static std::optional<CudaBackend> try_init_index(int index) {
        ob_ctx *ctx = nullptr;
        if (ob_init(index, &ctx) != OB_OK) return std::nullopt;
        return CudaBackend(ctx);
    }
    CudaBackend(CudaBackend &&o) noexcept : ctx_(o.ctx_), cache_(std::move(o.cache_)) { o.ctx_ = nullptr; }
    CudaBackend(const CudaBackend &) = delete;
    ~CudaBackend() {
        if (!ctx_) return;
        for (auto &kv : cache_) ob_weight_release(ctx_, kv.second);
        ob_destroy(ctx_);
    }

    // backend/mod.rs:310-313
    std::vector<float> matmul(const float *x, uint32_t n_tokens, const QuantMatrix &w) {
        std::vector<float> y((size_t)n_tokens * w.out_dim);
        check(ob_matmul(ctx_, x, n_tokens, weight(w), y.data()));
        return y;
    }
    // backend/mod.rs:342: the caller's buffer is resized and every element written
    void matmul_into(std::vector<float> &out, const float *x, uint32_t n_tokens, const QuantMatrix &w) {
        out.resize((size_t)n_tokens * w.out_dim);
        check(ob_matmul(ctx_, x, n_tokens, weight(w), out.data()));
    }
    // backend/mod.rs:368-388: rows are independent sequences
    std::vector<float> matmul_decode(const float *x, uint32_t n_tokens, const QuantMatrix &w) {
        std::vector<float> y((size_t)n_tokens * w.out_dim);
        check(ob_matmul_decode(ctx_, x, n_tokens, weight(w), y.data()));
        return y;
    }
    void matmul_decode_into(std::vector<float> &out, const float *x, uint32_t n_tokens, const QuantMatrix &w) {
        out.resize((size_t)n_tokens * w.out_dim);
        check(ob_matmul_decode(ctx_, x, n_tokens, weight(w), out.data()));
    }
    // backend/mod.rs:362-407
    std::vector<std::vector<float>> matmul_batch(const std::vector<MatmulOp> &ops) { return batch(ops, false); }
    void matmul_batch_into(std::vector<std::vector<float>> &outs, const std::vector<MatmulOp> &ops) { outs = batch(ops, false); }
    std::vector<std::vector<float>> matmul_batch_decode(const std::vector<MatmulOp> &ops) { return batch(ops, true); }
    // backend/mod.rs:479-495
    bool supports_type(uint32_t ggml_type) const { return ob_supports_type(ggml_type) != 0; }
    // backend/mod.rs:409-434
    std::optional<std::string> reduced_surface() const {
        const char *s = ob_reduced_surface();
        return s ? std::optional<std::string>(s) : std::nullopt;
    }
    ob_ctx *raw() const { return ctx_; }

  private:
    explicit CudaBackend(ob_ctx *c) : ctx_(c) {}
    void check(int rc) const {
        if (rc != OB_OK) throw std::runtime_error(ob_last_error(ctx_));
    }
    // backend/cuda.rs:216-236: device copy cached by the matrix's identity, never evicted
    ob_weight *weight(const QuantMatrix &w) {
        auto it = cache_.find(w.bytes);
        if (it != cache_.end()) return it->second;
        ob_weight *h = nullptr;
        check(ob_weight_register(ctx_, w.bytes, w.row_bytes(), w.ggml_type, w.in_dim, w.out_dim, &h));
        cache_.emplace(w.bytes, h);
        return h;
    }
    std::vector<std::vector<float>> batch(const std::vector<MatmulOp> &ops, bool decode) {
        std::vector<std::vector<float>> ys(ops.size());
        std::vector<ob_matmul_op> raw(ops.size());
        for (size_t i = 0; i < ops.size(); ++i) {
            ys[i].resize((size_t)ops[i].n_tokens * ops[i].w->out_dim);
            raw[i] = {ops[i].x, ops[i].n_tokens, weight(*ops[i].w), ys[i].data()};
        }
        check(ob_matmul_batch(ctx_, raw.data(), (uint32_t)raw.size(), decode ? 1 : 0));
        return ys;
    }
    ob_ctx *ctx_;
    std::unordered_map<const void *, ob_weight *> cache_;
};

}  // namespace orangu
