// Tensor-parallel communicator (internal): a thin layer over NCCL, resolved at run time with
// dlopen so that the library has no link-time dependency on it and shares whichever libnccl the
// host process already carries.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include <string>

namespace obtp {

struct Comm;

// Fills 128 bytes; false (with *err) when NCCL cannot be loaded.
bool unique_id(void *out128, std::string *err);
Comm *create(const void *id128, int rank, int size, int device, std::string *err);
void destroy(Comm *);
// In-place fp32 sum over all ranks, enqueued on `st`.
bool all_reduce_sum(Comm *, float *buf, size_t count, cudaStream_t st);
// logits is [rows][n_vocab] with this rank's columns [vocab0, vocab0 + vocab_l) filled; gathers the rest.
bool all_gather_logits(Comm *, float *logits, uint32_t rows, uint32_t n_vocab, uint32_t vocab0, uint32_t vocab_l, cudaStream_t st);
const char *last_error(Comm *);

}  // namespace obtp
