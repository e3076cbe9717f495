// GGUF files: header, metadata, tensor table, memory mapping, and the Llama-family model description.
//
// What the reference does in src/gguf.rs (GgufFile::open, :206-275: magic, version >= 2, u64 counts, typed metadata
// values, tensor infos with offsets relative to the data section, data section aligned to general.alignment or 32) and
// in engine/loader.rs (read_model_config, :1652-1712: which keys are required and how the optional ones default) and
// engine/arch/llama.rs (:125-200: the tensor names, output.weight falling back to token_embd.weight, the optional
// rope_freqs.weight).  Host code only; the device side is ob_model_create, which copies what it needs out of the mapping.
#include <fcntl.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <map>
#include <string>
#include <vector>

#include "../../include/orangu_b200.h"

namespace {

constexpr uint64_t kMaxStringBytes = 100ull << 20, kMaxArrayElements = 200000000ull;  // gguf.rs:41-45: refuse absurd lengths before allocating
constexpr uint64_t kDefaultAlignment = 32;                                           // gguf.rs:47

thread_local std::string g_error;

int gfail(int code, const std::string &msg) {
    g_error = msg;
    return code;
}

struct Value {
    uint32_t type = 0;  // GGUF value type; 9 = array
    uint64_t u = 0;     // integers and bool
    double f = 0.0;     // floats
    std::string s;      // string
    uint32_t elem_type = 0;
    uint64_t count = 0;  // arrays: only type and length are kept
};

struct Tensor {
    std::string name;
    uint32_t n_dims = 0;
    uint64_t dims[4] = {1, 1, 1, 1};
    uint32_t ggml_type = 0;
    uint64_t offset = 0, n_bytes = 0;
};

// elements per block of a type (1 for the unquantized ones, 0 = a type this build does not size)
uint32_t type_block(uint32_t type) {
    switch (type) {
    case 0: case 1: return 1;
    case 8: case 2: case 3: case 6: case 7: case 20: return 32;
    case 12: case 14: case 10: case 11: case 13: case 15: return 256;
    default: return 0;
    }
}

// bytes of a tensor of `n` elements whose rows have dims[0] elements; 0 = a type this build does not size
uint64_t tensor_bytes(uint32_t type, uint64_t n) {
    switch (type) {
    case 0: return n * 4;             // F32
    case 1: return n * 2;             // F16
    case 8: return n / 32 * 34;       // Q8_0
    case 12: return n / 256 * 144;    // Q4_K
    case 14: return n / 256 * 210;    // Q6_K
    case 2: return n / 32 * 18;       // Q4_0
    case 3: return n / 32 * 20;       // Q4_1
    case 6: return n / 32 * 22;       // Q5_0
    case 7: return n / 32 * 24;       // Q5_1
    case 10: return n / 256 * 84;     // Q2_K
    case 11: return n / 256 * 110;    // Q3_K
    case 13: return n / 256 * 176;    // Q5_K
    case 15: return n / 256 * 292;    // Q8_K
    case 20: return n / 32 * 18;      // IQ4_NL
    default: return 0;
    }
}

}  // namespace

struct ob_gguf {
    int fd = -1;
    const uint8_t *map = nullptr;
    uint64_t size = 0;
    uint32_t version = 0;
    uint64_t alignment = kDefaultAlignment, data_offset = 0;
    std::vector<std::pair<std::string, Value>> metadata;
    std::vector<Tensor> tensors;
    std::map<std::string, size_t> by_name;
    std::vector<ob_layer_desc> layers;  // storage behind ob_gguf_model_desc
};

namespace {

struct Reader {
    const uint8_t *p;
    uint64_t size, pos = 0;
    bool ok = true;
    template <typename T>
    T get() {
        T v{};
        if (!ok || pos + sizeof(T) > size) {
            ok = false;
            return v;
        }
        memcpy(&v, p + pos, sizeof(T));
        pos += sizeof(T);
        return v;
    }
    std::string str() {
        const uint64_t n = get<uint64_t>();
        if (!ok || n > kMaxStringBytes || pos + n > size) {
            ok = false;
            return {};
        }
        std::string s(reinterpret_cast<const char *>(p + pos), (size_t)n);
        pos += n;
        return s;
    }
    bool scalar(uint32_t type, Value &v) {
        switch (type) {
        case 0: v.u = get<uint8_t>(); break;
        case 1: v.u = (uint64_t)(int64_t)get<int8_t>(); break;
        case 2: v.u = get<uint16_t>(); break;
        case 3: v.u = (uint64_t)(int64_t)get<int16_t>(); break;
        case 4: v.u = get<uint32_t>(); break;
        case 5: v.u = (uint64_t)(int64_t)get<int32_t>(); break;
        case 6: v.f = get<float>(); break;
        case 7: v.u = get<uint8_t>() != 0; break;
        case 8: v.s = str(); break;
        case 10: v.u = get<uint64_t>(); break;
        case 11: v.u = (uint64_t)get<int64_t>(); break;
        case 12: v.f = get<double>(); break;
        default: ok = false;
        }
        return ok;
    }
    bool value(Value &v) {
        v.type = get<uint32_t>();
        if (v.type != 9) return scalar(v.type, v);
        v.elem_type = get<uint32_t>();
        v.count = get<uint64_t>();
        if (!ok || v.count > kMaxArrayElements || v.elem_type == 9) {
            ok = false;
            return false;
        }
        Value e;
        for (uint64_t i = 0; i < v.count && ok; ++i) scalar(v.elem_type, e);  // skipped, but every element is bounds-checked
        return ok;
    }
};

const Value *find(const ob_gguf *g, const std::string &key) {
    for (const auto &kv : g->metadata)
        if (kv.first == key) return &kv.second;
    return nullptr;
}

bool as_u64(const Value *v, uint64_t *out) {
    if (!v) return false;
    switch (v->type) {
    case 0: case 1: case 2: case 3: case 4: case 5: case 7: case 10: case 11: *out = v->u; return true;
    default: return false;
    }
}

bool as_f32(const Value *v, float *out) {
    if (!v) return false;
    if (v->type == 6 || v->type == 12) {
        *out = (float)v->f;
        return true;
    }
    return false;
}

}  // namespace

extern "C" {

const char *ob_gguf_last_error(void) { return g_error.c_str(); }

void ob_gguf_close(ob_gguf *g) {
    if (!g) return;
    if (g->map) munmap(const_cast<uint8_t *>(g->map), g->size);
    if (g->fd >= 0) close(g->fd);
    delete g;
}

int ob_gguf_open(const char *path, ob_gguf **out) {
    if (!path || !out) return gfail(OB_ERR_INVALID, "gguf_open: null argument");
    *out = nullptr;
    ob_gguf *g = new ob_gguf;
    auto bail = [&](int code, const std::string &msg) {
        ob_gguf_close(g);
        return gfail(code, std::string("gguf_open: ") + path + ": " + msg);
    };
    g->fd = open(path, O_RDONLY);
    if (g->fd < 0) return bail(OB_ERR_INVALID, "cannot open the file");
    struct stat st;
    if (fstat(g->fd, &st) != 0 || st.st_size < 24) return bail(OB_ERR_INVALID, "shorter than a GGUF header");
    g->size = (uint64_t)st.st_size;
    void *m = mmap(nullptr, g->size, PROT_READ, MAP_PRIVATE, g->fd, 0);
    if (m == MAP_FAILED) return bail(OB_ERR_INVALID, "mmap failed");
    g->map = static_cast<const uint8_t *>(m);

    Reader r{g->map, g->size};
    if (memcmp(g->map, "GGUF", 4) != 0) return bail(OB_ERR_INVALID, "not a GGUF file (bad magic)");
    r.pos = 4;
    g->version = r.get<uint32_t>();
    if (g->version < 2) return bail(OB_ERR_UNSUPPORTED, "GGUF version " + std::to_string(g->version) + " is not supported (need 2 or later)");
    const uint64_t n_tensors = r.get<uint64_t>(), n_kv = r.get<uint64_t>();
    if (!r.ok || n_tensors > (1u << 24) || n_kv > (1u << 24)) return bail(OB_ERR_INVALID, "implausible tensor or metadata count");
    for (uint64_t i = 0; i < n_kv; ++i) {
        std::string key = r.str();
        Value v;
        if (!r.ok || !r.value(v)) return bail(OB_ERR_INVALID, "truncated or malformed metadata (entry " + std::to_string(i) + ")");
        g->metadata.emplace_back(std::move(key), std::move(v));
    }
    uint64_t al = 0;
    if (as_u64(find(g, "general.alignment"), &al)) {
        if (al == 0 || (al & (al - 1))) return bail(OB_ERR_INVALID, "general.alignment is not a power of two");
        g->alignment = al;
    }
    for (uint64_t i = 0; i < n_tensors; ++i) {
        Tensor t;
        t.name = r.str();
        t.n_dims = r.get<uint32_t>();
        if (!r.ok || t.n_dims > 4) return bail(OB_ERR_INVALID, "malformed tensor info (entry " + std::to_string(i) + ")");
        uint64_t n = 1;
        for (uint32_t d = 0; d < t.n_dims; ++d) {
            t.dims[d] = r.get<uint64_t>();
            if (t.dims[d] == 0 || n > (1ull << 48) / t.dims[d]) return bail(OB_ERR_INVALID, "tensor " + t.name + " has an implausible shape");
            n *= t.dims[d];
        }
        t.ggml_type = r.get<uint32_t>();
        t.offset = r.get<uint64_t>();
        if (!r.ok) return bail(OB_ERR_INVALID, "truncated tensor table");
        t.n_bytes = tensor_bytes(t.ggml_type, n);
        // a row (dims[0] elements) must be a whole number of blocks, or the byte count above undercounts the tensor
        if (const uint32_t blk = type_block(t.ggml_type); blk > 1 && t.dims[0] % blk)
            return bail(OB_ERR_INVALID, "tensor " + t.name + ": its rows are not a whole number of " + std::to_string(blk) + "-element blocks");
        g->by_name[t.name] = g->tensors.size();
        g->tensors.push_back(std::move(t));
    }
    g->data_offset = (r.pos + g->alignment - 1) / g->alignment * g->alignment;  // gguf.rs:258-266
    for (const Tensor &t : g->tensors) {
        if (t.offset % g->alignment) return bail(OB_ERR_INVALID, "tensor " + t.name + " is not aligned to general.alignment");
        // no sum that could wrap: the offset is compared with what is left after the data section starts
        if (g->data_offset > g->size || t.offset > g->size - g->data_offset || t.n_bytes > g->size - g->data_offset - t.offset)
            return bail(OB_ERR_INVALID, "tensor " + t.name + " reaches past the end of the file");
    }
    *out = g;
    return OB_OK;
}

uint32_t ob_gguf_version(const ob_gguf *g) { return g ? g->version : 0; }
uint64_t ob_gguf_alignment(const ob_gguf *g) { return g ? g->alignment : 0; }
uint64_t ob_gguf_data_offset(const ob_gguf *g) { return g ? g->data_offset : 0; }
uint64_t ob_gguf_n_tensors(const ob_gguf *g) { return g ? g->tensors.size() : 0; }

int ob_gguf_tensor(const ob_gguf *g, uint64_t index, ob_gguf_tensor_info *out) {
    if (!g || !out || index >= g->tensors.size()) return gfail(OB_ERR_INVALID, "gguf_tensor: bad argument");
    const Tensor &t = g->tensors[index];
    out->name = t.name.c_str();
    out->ggml_type = t.ggml_type;
    out->n_dims = t.n_dims;
    for (int d = 0; d < 4; ++d) out->dims[d] = t.dims[d];
    out->data = g->map + g->data_offset + t.offset;
    out->n_bytes = t.n_bytes;
    return OB_OK;
}

int ob_gguf_find_tensor(const ob_gguf *g, const char *name, ob_gguf_tensor_info *out) {
    if (!g || !name || !out) return gfail(OB_ERR_INVALID, "gguf_find_tensor: null argument");
    auto it = g->by_name.find(name);
    if (it == g->by_name.end()) return gfail(OB_ERR_INVALID, std::string("gguf_find_tensor: no tensor named ") + name);
    return ob_gguf_tensor(g, it->second, out);
}

int ob_gguf_get_u64(const ob_gguf *g, const char *key, uint64_t *out) {
    if (!g || !key || !out) return gfail(OB_ERR_INVALID, "gguf_get_u64: null argument");
    return as_u64(find(g, key), out) ? OB_OK : gfail(OB_ERR_INVALID, std::string("gguf_get_u64: no integer metadata named ") + key);
}

int ob_gguf_get_f32(const ob_gguf *g, const char *key, float *out) {
    if (!g || !key || !out) return gfail(OB_ERR_INVALID, "gguf_get_f32: null argument");
    return as_f32(find(g, key), out) ? OB_OK : gfail(OB_ERR_INVALID, std::string("gguf_get_f32: no float metadata named ") + key);
}

int ob_gguf_get_string(const ob_gguf *g, const char *key, const char **out) {
    if (!g || !key || !out) return gfail(OB_ERR_INVALID, "gguf_get_string: null argument");
    const Value *v = find(g, key);
    if (!v || v->type != 8) return gfail(OB_ERR_INVALID, std::string("gguf_get_string: no string metadata named ") + key);
    *out = v->s.c_str();
    return OB_OK;
}

int ob_gguf_model_desc(ob_gguf *g, ob_model_desc *d) {
    if (!g || !d) return gfail(OB_ERR_INVALID, "gguf_model_desc: null argument");
    memset(d, 0, sizeof(*d));
    const Value *av = find(g, "general.architecture");
    if (!av || av->type != 8) return gfail(OB_ERR_INVALID, "gguf_model_desc: general.architecture is missing");
    const std::string arch = av->s;
    // LLAMA_STYLE_ARCHITECTURES, loader.rs:190
    if (arch != "llama" && arch != "qwen2" && arch != "qwen3" && arch != "mistral" && arch != "qwen3vl")
        return gfail(OB_ERR_UNSUPPORTED, "gguf_model_desc: architecture '" + arch + "' is outside this build (llama, mistral, qwen2, qwen3, qwen3vl)");
    auto req = [&](const char *suffix, uint64_t *out) { return as_u64(find(g, arch + "." + suffix), out); };
    uint64_t n_embd = 0, n_layer = 0, n_head = 0, n_head_kv = 0, n_vocab = 0, head_dim = 0, rope_dim = 0, n_ff = 0;
    if (!req("embedding_length", &n_embd) || !req("block_count", &n_layer) || !req("attention.head_count", &n_head))
        return gfail(OB_ERR_INVALID, "gguf_model_desc: " + arch + ".embedding_length, .block_count and .attention.head_count are required");
    if (!req("attention.head_count_kv", &n_head_kv)) n_head_kv = n_head;  // loader.rs:1656-1658
    if (n_head == 0 || n_head_kv == 0) return gfail(OB_ERR_INVALID, "gguf_model_desc: head counts must be nonzero");
    // every layer owns at least nine tensors, and every size is later held in 32 bits
    if (n_layer == 0 || n_layer > g->tensors.size() / 9 || n_layer > 4096)
        return gfail(OB_ERR_INVALID, "gguf_model_desc: " + arch + ".block_count = " + std::to_string(n_layer) + " does not fit the file's " + std::to_string(g->tensors.size()) + " tensors");
    if (n_embd == 0 || n_embd > (1u << 24) || n_head > (1u << 16) || n_head_kv > n_head)
        return gfail(OB_ERR_INVALID, "gguf_model_desc: implausible embedding_length or head counts");
    if (!req("attention.key_length", &head_dim)) head_dim = n_embd / n_head;  // loader.rs:1676-1678
    if (!req("rope.dimension_count", &rope_dim)) rope_dim = head_dim;         // loader.rs:1682-1684
    if (!req("vocab_size", &n_vocab)) {                                       // loader.rs:1660-1671
        const Value *tok = find(g, "tokenizer.ggml.tokens");
        if (tok && tok->type == 9) n_vocab = tok->count;
    }
    float freq_base = 10000.0f, eps = 1e-5f;
    as_f32(find(g, arch + ".rope.freq_base"), &freq_base);
    as_f32(find(g, arch + ".attention.layer_norm_rms_epsilon"), &eps);

    auto matrix = [&](const std::string &name, uint64_t in_dim, uint64_t out_dim, ob_matrix_desc *m, bool optional) -> int {
        auto it = g->by_name.find(name);
        if (it == g->by_name.end()) return optional ? OB_OK : gfail(OB_ERR_INVALID, "gguf_model_desc: tensor " + name + " is missing");
        const Tensor &t = g->tensors[it->second];
        if (t.n_dims != 2 || (in_dim && t.dims[0] != in_dim) || (out_dim && t.dims[1] != out_dim))
            return gfail(OB_ERR_INVALID, "gguf_model_desc: tensor " + name + " has shape " + std::to_string(t.dims[0]) + " x " + std::to_string(t.dims[1]) +
                                             ", expected " + std::to_string(in_dim) + " x " + std::to_string(out_dim));
        if (!ob_supports_type(t.ggml_type))
            return gfail(OB_ERR_UNSUPPORTED, "gguf_model_desc: tensor " + name + " has ggml type " + std::to_string(t.ggml_type) + ", which this build has no kernel for");
        m->data = g->map + g->data_offset + t.offset;
        m->ggml_type = t.ggml_type;
        m->in_dim = (uint32_t)t.dims[0];
        m->out_dim = (uint32_t)t.dims[1];
        return OB_OK;
    };
    auto vector_f32 = [&](const std::string &name, uint64_t min_len, const float **out, bool optional) -> int {
        auto it = g->by_name.find(name);
        if (it == g->by_name.end()) return optional ? OB_OK : gfail(OB_ERR_INVALID, "gguf_model_desc: tensor " + name + " is missing");
        const Tensor &t = g->tensors[it->second];
        uint64_t n = 1;
        for (uint32_t i = 0; i < t.n_dims; ++i) n *= t.dims[i];
        if (t.ggml_type != 0 || n < min_len) return gfail(OB_ERR_INVALID, "gguf_model_desc: tensor " + name + " must be f32 with at least " + std::to_string(min_len) + " entries");
        *out = reinterpret_cast<const float *>(g->map + g->data_offset + t.offset);
        return OB_OK;
    };

    int rc;
    if ((rc = matrix("token_embd.weight", n_embd, n_vocab, &d->token_embd, false))) return rc;
    if (n_vocab == 0) n_vocab = d->token_embd.out_dim;
    if (n_vocab == 0) return gfail(OB_ERR_INVALID, "gguf_model_desc: no vocab_size, no tokenizer.ggml.tokens");
    if ((rc = matrix("output.weight", n_embd, n_vocab, &d->output, true))) return rc;  // absent: tied to token_embd (llama.rs:133-139)
    if ((rc = vector_f32("output_norm.weight", n_embd, &d->output_norm, false))) return rc;
    if ((rc = vector_f32("rope_freqs.weight", rope_dim / 2, &d->rope_freqs, true))) return rc;  // llama.rs:186-200
    g->layers.assign((size_t)n_layer, ob_layer_desc{});
    const uint64_t q_dim = n_head * head_dim, kv_dim = n_head_kv * head_dim;
    for (uint64_t i = 0; i < n_layer; ++i) {
        const std::string p = "blk." + std::to_string(i) + ".";
        ob_layer_desc &L = g->layers[(size_t)i];
        if ((rc = vector_f32(p + "attn_norm.weight", n_embd, &L.attn_norm, false))) return rc;
        if ((rc = vector_f32(p + "ffn_norm.weight", n_embd, &L.ffn_norm, false))) return rc;
        if ((rc = matrix(p + "attn_q.weight", n_embd, q_dim, &L.wq, false))) return rc;
        if ((rc = matrix(p + "attn_k.weight", n_embd, kv_dim, &L.wk, false))) return rc;
        if ((rc = matrix(p + "attn_v.weight", n_embd, kv_dim, &L.wv, false))) return rc;
        if ((rc = matrix(p + "attn_output.weight", q_dim, n_embd, &L.wo, false))) return rc;
        if ((rc = matrix(p + "ffn_gate.weight", n_embd, n_ff, &L.w_gate, false))) return rc;
        if (n_ff == 0) n_ff = L.w_gate.out_dim;  // <arch>.feed_forward_length is optional here: the tensor says it
        if ((rc = matrix(p + "ffn_up.weight", n_embd, n_ff, &L.w_up, false))) return rc;
        if ((rc = matrix(p + "ffn_down.weight", n_ff, n_embd, &L.w_down, false))) return rc;
        // present on Qwen2 / Qwen3-shaped files only (llama.rs:171-175)
        if ((rc = vector_f32(p + "attn_q.bias", q_dim, &L.q_bias, true))) return rc;
        if ((rc = vector_f32(p + "attn_k.bias", kv_dim, &L.k_bias, true))) return rc;
        if ((rc = vector_f32(p + "attn_v.bias", kv_dim, &L.v_bias, true))) return rc;
        if ((rc = vector_f32(p + "attn_q_norm.weight", head_dim, &L.q_norm, true))) return rc;
        if ((rc = vector_f32(p + "attn_k_norm.weight", head_dim, &L.k_norm, true))) return rc;
    }
    uint64_t ff_meta = 0;
    if (req("feed_forward_length", &ff_meta) && n_layer && ff_meta != n_ff)
        return gfail(OB_ERR_INVALID, "gguf_model_desc: " + arch + ".feed_forward_length disagrees with the ffn tensors");
    if (n_vocab > (1ull << 31) || head_dim == 0 || head_dim > (1u << 16) || rope_dim > head_dim || n_ff > (1ull << 31))
        return gfail(OB_ERR_INVALID, "gguf_model_desc: vocabulary, head or feed-forward sizes out of range");
    d->n_vocab = (uint32_t)n_vocab;
    d->n_embd = (uint32_t)n_embd;
    d->n_layer = (uint32_t)n_layer;
    d->n_head = (uint32_t)n_head;
    d->n_head_kv = (uint32_t)n_head_kv;
    d->head_dim = (uint32_t)head_dim;
    d->rope_dim = (uint32_t)rope_dim;
    d->n_ff = (uint32_t)n_ff;
    d->rope_freq_base = freq_base;
    d->rms_eps = eps;
    d->rope_neox = (arch == "llama" || arch == "mistral") ? 0u : 1u;  // rope_layout_for, llama.rs:114-119
    d->layers = g->layers.data();
    uint64_t ctx_train = 0;
    d->max_seq_len = req("context_length", &ctx_train) ? (uint32_t)std::min<uint64_t>(ctx_train, 1u << 20) : 4096u;  // the caller may lower it
    d->max_batch_tokens = 512;
    return OB_OK;
}

}  // extern "C"
