// Host-side state shared by the runtime translation units (internal).
#pragma once

#include <cuda_runtime.h>

#include <mutex>
#include <string>

#include "../../include/orangu_b200.h"
#include "common.cuh"
#include "kernels.h"

using namespace ob;

struct Scratch {  // grow-only device buffer
    void *p = nullptr;
    size_t cap = 0;
};

struct ob_ctx {
    int device = 0;
    int sm_count = 0;
    cudaStream_t stream = nullptr;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    std::mutex mu;
    std::string err;
    uint64_t launches = 0;
    float last_ms = 0.0f;
    Scratch sx, sy, sq, sd, ss, saux, saux2, saux3;
};

struct ob_weight {
    ob_ctx *ctx;
    DevWeight w;
    void *mem;
    uint64_t bytes;
};

namespace obrt {

int fail(ob_ctx *ctx, int code, const std::string &msg);
int ensure(ob_ctx *ctx, Scratch &s, size_t bytes);
bool type_supported(uint32_t t);

#define OB_CUDA(ctx, expr)                                                                                  \
    do {                                                                                                    \
        cudaError_t e__ = (expr);                                                                           \
        if (e__ != cudaSuccess) {                                                                           \
            return obrt::fail(ctx, e__ == cudaErrorMemoryAllocation ? OB_ERR_OOM : OB_ERR_CUDA,             \
                              std::string(#expr) + ": " + cudaGetErrorString(e__));                         \
        }                                                                                                   \
    } while (0)

struct Bind {  // makes the context's device current for the scope of a call
    int prev = -1;
    explicit Bind(const ob_ctx *c) {
        cudaGetDevice(&prev);
        if (prev != c->device) cudaSetDevice(c->device);
        else prev = -1;
    }
    ~Bind() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

// Uploads (a slice of) a GGUF matrix and re-lays it for the kernels; see DevWeight.
int make_weight(ob_ctx *ctx, const uint8_t *raw, uint64_t row_bytes, uint32_t type, uint32_t in_dim, uint32_t out_dim, uint32_t row0,
                uint32_t n_rows, uint32_t col0, uint32_t n_cols, ob_weight **out);

}  // namespace obrt
