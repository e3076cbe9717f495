// C++ host-side mirror of the reference engine's `Backend` trait, of its `ModelForward` / `KvCache` surface for Llama-style
// models and of its `SlotPool`, over the C ABI of orangu_b200.h.
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

class LlamaModel;

// engine/kv_cache.rs: one sequence's cache.  `paged`: pages are taken from the model's pool as the sequence grows and go back
// on truncate (what a slot holds); otherwise they are reserved up front, as ModelForward::new_kv_cache does
// (engine/arch/llama.rs:1002-1005).
class KvCache {
  public:
    KvCache(KvCache &&o) noexcept : kv_(o.kv_), ctx_(o.ctx_) { o.kv_ = nullptr; }
    KvCache(const KvCache &) = delete;
    ~KvCache() {
        if (kv_) ob_kv_destroy(kv_);
    }
    uint32_t len() const { return ob_kv_len(kv_); }
    uint32_t pages() const { return ob_kv_pages(kv_); }
    void truncate(uint32_t new_len) {  // kv_cache.rs:496-511
        if (ob_kv_truncate(kv_, new_len) != OB_OK) throw std::runtime_error(ob_last_error(ctx_));
    }
    void copy_prefix_from(const KvCache &src, uint32_t n) {  // kv_cache.rs:1079-1100
        if (ob_kv_copy_prefix(kv_, src.kv_, n) != OB_OK) throw std::runtime_error(ob_last_error(ctx_));
    }
    ob_kv *raw() const { return kv_; }

  private:
    friend class LlamaModel;
    KvCache(ob_kv *kv, ob_ctx *ctx) : kv_(kv), ctx_(ctx) {}
    ob_kv *kv_;
    ob_ctx *ctx_;
};

// ModelForward for Llama-style models (engine/arch/mod.rs:2035-2191, engine/arch/llama.rs:949-1032) over ob_model.
class LlamaModel {
  public:
    // LlamaModel::load_with_backend (arch/llama.rs:125-230): the descriptor's tensors are copied to the device
    LlamaModel(CudaBackend &be, const ob_model_desc &desc) : ctx_(be.raw()) {
        if (ob_model_create(ctx_, &desc, &m_) != OB_OK) throw std::runtime_error(ob_last_error(ctx_));
    }
    LlamaModel(LlamaModel &&o) noexcept : ctx_(o.ctx_), m_(o.m_) { o.m_ = nullptr; }
    LlamaModel(const LlamaModel &) = delete;
    ~LlamaModel() {
        if (m_) ob_model_destroy(m_);
    }
    KvCache new_kv_cache(uint32_t capacity, bool paged = false) {
        ob_kv *kv = nullptr;
        check((paged ? ob_kv_create_paged : ob_kv_create)(m_, capacity, &kv));
        return KvCache(kv, ctx_);
    }
    // forward: the logits of the last token
    std::vector<float> forward(KvCache &cache, const std::vector<uint32_t> &tokens, uint32_t start_pos) {
        std::vector<float> logits(ob_model_n_vocab(m_));
        const uint32_t n = (uint32_t)tokens.size();
        ob_kv *kv = cache.raw();
        check(ob_forward(m_, &kv, tokens.data(), &n, &start_pos, 1, nullptr, nullptr, logits.data()));
        return logits;
    }
    // forward_maybe_sampling with a greedy sampler: the next token id
    uint32_t forward_maybe_sampling(KvCache &cache, const std::vector<uint32_t> &tokens, uint32_t start_pos, const std::vector<uint32_t> *recent = nullptr,
                                    float repeat_penalty = 1.0f, uint32_t repeat_last_n = 64) {
        const uint32_t n = (uint32_t)tokens.size(), n_recent = recent ? (uint32_t)recent->size() : 0u;
        ob_greedy g{repeat_penalty, repeat_last_n, recent ? recent->data() : nullptr, &n_recent};
        ob_kv *kv = cache.raw();
        uint32_t out = 0;
        check(ob_forward(m_, &kv, tokens.data(), &n, &start_pos, 1, recent && repeat_penalty != 1.0f ? &g : nullptr, &out, nullptr));
        return out;
    }
    // forward_batch_decode (arch/mod.rs:2174-2190): one token per sequence, rows independent
    std::vector<uint32_t> forward_batch_decode(const std::vector<KvCache *> &caches, const std::vector<uint32_t> &tokens) {
        const uint32_t n = (uint32_t)caches.size();
        std::vector<ob_kv *> kvs(n);
        std::vector<uint32_t> ones(n, 1u), start(n), out(n);
        for (uint32_t i = 0; i < n; ++i) {
            kvs[i] = caches[i]->raw();
            start[i] = caches[i]->len();
        }
        check(ob_forward(m_, kvs.data(), tokens.data(), ones.data(), start.data(), n, nullptr, out.data(), nullptr));
        return out;
    }
    // record_decode_chain + argmax (arch/llama.rs:302-473): one captured graph per token
    uint32_t decode_greedy(KvCache &cache, uint32_t token) {
        uint32_t out = 0;
        check(ob_decode_greedy(m_, cache.raw(), token, &out));
        return out;
    }
    uint32_t n_vocab() const { return ob_model_n_vocab(m_); }
    uint32_t free_pages() const { return ob_model_free_pages(m_); }
    ob_model *raw() const { return m_; }

  private:
    void check(int rc) const {
        if (rc != OB_OK) throw std::runtime_error(ob_last_error(ctx_));
    }
    ob_ctx *ctx_;
    ob_model *m_ = nullptr;
};

// SlotPool (engine/scheduler.rs:36-317) with the decode window of BatchCoordinator (engine/batch.rs:184-324).  One thread per
// request: acquire, prefill, decode per token, let the guard go.
class SlotPool {
  public:
    class Guard {  // SlotGuard (scheduler.rs:319-356): releasing empties the slot's cache and wakes the next waiter
      public:
        Guard(Guard &&o) noexcept : pool_(o.pool_), id_(o.id_) { o.pool_ = nullptr; }
        Guard(const Guard &) = delete;
        ~Guard() {
            if (pool_) ob_slot_release(pool_, id_);
        }
        uint32_t id() const { return id_; }
        uint32_t len() const { return ob_slot_len(pool_, id_); }
        uint32_t prefill(const std::vector<uint32_t> &tokens) {
            uint32_t out = 0;
            check(ob_slot_prefill(pool_, id_, tokens.data(), (uint32_t)tokens.size(), &out, nullptr));
            return out;
        }
        uint32_t decode(uint32_t token) {  // BatchCoordinator::submit: blocks until the batch this step joined has run
            uint32_t out = 0;
            check(ob_slot_decode(pool_, id_, token, nullptr, &out, nullptr));
            return out;
        }
        void truncate(uint32_t new_len) { check(ob_slot_truncate(pool_, id_, new_len)); }

      private:
        friend class SlotPool;
        Guard(ob_slot_pool *p, uint32_t id) : pool_(p), id_(id) {}
        void check(int rc) const {
            if (rc != OB_OK) throw std::runtime_error(ob_slot_last_error(pool_, id_));
        }
        ob_slot_pool *pool_;
        uint32_t id_;
    };

    SlotPool(LlamaModel &model, const ob_slot_pool_desc &desc) {
        if (ob_slot_pool_create(model.raw(), &desc, &p_) != OB_OK) throw std::runtime_error(ob_slot_last_error(nullptr, -1));
    }
    SlotPool(const SlotPool &) = delete;
    ~SlotPool() { ob_slot_pool_destroy(p_); }
    // try_acquire: empty when the pool refuses (queue limit reached, or no slot came free within timeout_ms; < 0 waits)
    std::optional<Guard> try_acquire(int32_t timeout_ms = -1) {
        uint32_t id = 0;
        if (ob_slot_acquire(p_, timeout_ms, &id) != OB_OK) return std::nullopt;
        return Guard(p_, id);
    }
    std::optional<Guard> acquire_slot(uint32_t id, int32_t timeout_ms = -1) {
        if (ob_slot_acquire_id(p_, id, timeout_ms) != OB_OK) return std::nullopt;
        return Guard(p_, id);
    }
    std::vector<ob_slot_state> snapshot() {
        std::vector<ob_slot_state> v(ob_slot_pool_snapshot(p_, nullptr, 0));
        ob_slot_pool_snapshot(p_, v.data(), (uint32_t)v.size());
        return v;
    }
    ob_slot_pool_stats stats() {
        ob_slot_pool_stats st{};
        ob_slot_pool_get_stats(p_, &st);
        return st;
    }

  private:
    ob_slot_pool *p_ = nullptr;
};

}  // namespace orangu
