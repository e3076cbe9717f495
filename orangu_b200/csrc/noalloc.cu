// ob_attention_decode_static: split flash-decode attention that never allocates.
//
// Who needs it.  In the server one blocking thread per busy slot drives the device, and several slots have
// kernels in flight at once.  cudaMalloc and cudaFree synchronise the whole device, so a slot that allocates
// attention scratch in the middle of a request stalls every other slot's stream; and once the KV pool has been
// given the rest of the memory, an allocation made per request can simply fail.  Such callers bring their own
// input and output buffers (device pointers) and want the operator to need nothing else.
//
// How.  The partial results of the splits (the only scratch the kernel needs) and the two words of per-call
// metadata live in one file-scope device array of fixed size.  In host code that array's name is only a
// stand-in, not a device address, so the address is fetched once per device with cudaGetSymbolAddress, with that
// device current, and handed to the kernels as an ordinary pointer.
//
// Consequences a caller must know:
//   * the first call on a device performs that one-time set-up (and sets the kernels' shared-memory attribute);
//     make it before any stream capture begins;
//   * every call on a device uses the same array, which keeps the previous call's contents.  Nothing in it has
//     to start at zero -- each (head, split) slot is written before the merge reads it -- but two calls that
//     overlap on the GPU (different streams, no ordering between them) would overwrite each other's partials;
//   * shapes whose partials do not fit the array are refused with OB_ERR_CAPACITY, never truncated;
//   * every GPU that loads the library holds the array (1 MiB + 256 B) until the process exits.
#include <algorithm>

#include "runtime.h"

using namespace obrt;

namespace {

constexpr size_t STATIC_META_BYTES = 256;
constexpr size_t STATIC_PARTIAL_BYTES = 1u << 20;  // 1 MiB of split partials
constexpr uint32_t STATIC_MAX_SPLITS = 16;
constexpr int MAX_DEVICES = 64;

static __device__ __align__(256) unsigned char g_static_scratch[STATIC_META_BYTES + STATIC_PARTIAL_BYTES];

// Device address of g_static_scratch per device ordinal, filled on first use.
unsigned char *g_scratch_addr[MAX_DEVICES] = {nullptr};

// scratch[0..8): the sequence's page-table pointer; scratch[64..68): its window length -- what the attention
// kernels read from device memory.
__global__ void static_meta_kernel(unsigned char *scratch, const int32_t *table, uint32_t n_pos) {
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        *reinterpret_cast<const int32_t **>(scratch) = table;
        *reinterpret_cast<uint32_t *>(scratch + 64) = n_pos;
    }
}

}  // namespace

extern "C" int ob_attention_decode_static(ob_ctx *ctx, const float *q_dev, const void *k_pages_dev, const void *v_pages_dev,
                                          const int32_t *page_table_dev, uint32_t n_pos, uint32_t n_head, uint32_t n_head_kv,
                                          uint32_t head_dim, float scale, float *out_dev, void *stream) {
    if (!ctx || !q_dev || !k_pages_dev || !v_pages_dev || !page_table_dev || !out_dev)
        return fail(ctx, OB_ERR_INVALID, "attention_decode_static: null argument");
    if (n_pos == 0 || n_head == 0 || n_head_kv == 0 || n_head % n_head_kv || (head_dim != 64 && head_dim != 128))
        return fail(ctx, OB_ERR_UNSUPPORTED, "attention_decode_static: needs n_pos > 0, n_head a multiple of n_head_kv, head_dim 64 or 128");
    const uint32_t group = n_head / n_head_kv;
    if (group != 1 && group != 2 && group != 4 && group != 8)
        return fail(ctx, OB_ERR_UNSUPPORTED, "attention_decode_static: heads per KV head must be 1, 2, 4 or 8");
    const uint32_t n_pages = (n_pos + KV_PAGE - 1) / KV_PAGE;
    const uint32_t n_splits = std::max(1u, std::min(STATIC_MAX_SPLITS, n_pages / 4));
    const size_t part_o_bytes = (size_t)n_head * n_splits * head_dim * 4, part_ml_bytes = (size_t)n_head * n_splits * 8;
    if (part_o_bytes + part_ml_bytes > STATIC_PARTIAL_BYTES)
        return fail(ctx, OB_ERR_CAPACITY,
                    "attention_decode_static: n_head * splits * (head_dim + 2) * 4 bytes exceeds the 1 MiB static scratch "
                    "(splits = min(16, pages / 4)); use ob_attention_decode or fewer heads per call");
    std::lock_guard<std::mutex> g(ctx->mu);
    Bind b(ctx);
    if (ctx->device < 0 || ctx->device >= MAX_DEVICES) return fail(ctx, OB_ERR_UNSUPPORTED, "attention_decode_static: device ordinal above 63");
    unsigned char *scratch = g_scratch_addr[ctx->device];
    if (!scratch) {  // one-time set-up for this device, which Bind has made current
        void *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess || !p) return fail(ctx, OB_ERR_CUDA, std::string("attention_decode_static: cudaGetSymbolAddress: ") + cudaGetErrorString(e));
        scratch = static_cast<unsigned char *>(p);
        g_scratch_addr[ctx->device] = scratch;
    }
    cudaStream_t st = stream ? static_cast<cudaStream_t>(stream) : ctx->stream;
    static_meta_kernel<<<1, 32, 0, st>>>(scratch, page_table_dev, n_pos);
    AttnDecodeArgs a{};
    a.q = q_dev;
    a.out = out_dev;
    a.k_pool = static_cast<const __half *>(k_pages_dev);
    a.v_pool = static_cast<const __half *>(v_pages_dev);
    a.page_tables = reinterpret_cast<const int32_t *const *>(scratch);
    a.n_pos = reinterpret_cast<const uint32_t *>(scratch + 64);
    a.n_seq = 1;
    a.n_head = n_head;
    a.n_head_kv = n_head_kv;
    a.head_dim = head_dim;
    a.scale = scale;
    a.n_splits = n_splits;
    a.part_o = reinterpret_cast<float *>(scratch + STATIC_META_BYTES);
    a.part_ml = reinterpret_cast<float *>(scratch + STATIC_META_BYTES + part_o_bytes);
    a.max_pos = n_pos;
    launch_attn_decode(a, st);
    ctx->launches += 3;
    OB_CUDA(ctx, cudaGetLastError());
    return OB_OK;
}
