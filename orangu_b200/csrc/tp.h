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

// Host-side rendezvous of the ranks of one node, for use BEFORE a step that contains collectives or exchanges is enqueued:
// a rank that has died, or has failed its own argument checks and returned, is then found on the host after a time limit,
// with nothing launched, instead of the others waiting for it inside a collective on their GPUs.  A small POSIX
// shared-memory segment named after the communicator's id holds one arrival counter per rank.
struct Rendezvous;
Rendezvous *rendezvous_open(const void *id128, int rank, int size, std::string *err);
// Publishes this rank's next step number and waits until every rank has published it.  False when the time runs out;
// *missing is then the first rank that had not arrived.  timeout_ms == 0 returns true at once (the guard is off).
bool rendezvous_arrive(Rendezvous *, uint32_t timeout_ms, int *missing);
void rendezvous_close(Rendezvous *);

// One-shot exchange of the ranks' partial vectors through peer memory (NVLink stores between the GPUs of one node), for
// the single-token decode step where an NCCL all-reduce of 16 KB costs more than the product it follows.
// Every rank owns 2 x size slots of n (value, tag) pairs.  In exchange number k (counted per rank in *seq, the same on
// all ranks) a rank's product kernel stores each element of its partial, together with the tag k + 1 in the same 8-byte
// word, into slot [k & 1][its rank] of EVERY rank; the consumer reads each word until its tag is k + 1 (an 8-byte store
// arrives whole, so no fence or separate flag is needed), adds the values in rank order -- every rank gets the same
// bits -- and increments *seq.  Two parities suffice: nobody can start exchange k + 2 before everybody has finished
// reading exchange k.  A POD: it is passed to kernels by value.
struct PeerXchg {
    uint2 *slots[8];     // slots[r]: rank r's slot array [2][size][n] of (value bits, tag)
    uint32_t *seq;       // this rank: exchanges completed
    uint32_t *err;       // this rank: set to 1 when a wait ran out of time
    uint32_t rank, size, n;
    uint32_t timeout_ms;  // how long the consumer waits for a rank's words before it reports and goes on (0 = 4000)
};
// The same idea for a few rows at a time (decode batches, short prefill chunks): every rank copies its partial [rows][n]
// into a landing area in EVERY rank's memory, chunk by chunk, each chunk followed by a system-scope fence and a tagged
// arrival word; the CTA that owns a chunk waits for the other ranks' arrival words of that chunk only, adds the partials in
// rank order (every rank gets the same bits) and adds the result to the residual stream.  One kernel instead of an NCCL
// all-reduce plus an add; it shares the exchange numbering (*seq), the error word and the time limit of PeerXchg.
struct PeerBulk {
    float *data[8];       // data[r]: rank r's landing area [2][size][cap] as mapped here
    uint32_t *flags[8];   // flags[r]: rank r's arrival words [2][size][max_chunks]
    uint32_t *done;       // this rank: CTAs of the running exchange that have finished
    uint32_t cap;         // floats per (parity, source rank); 0: not set up
    uint32_t max_chunks;
};
constexpr uint32_t kBulkChunk = 2048;  // floats per chunk (8 KB)

// Allocates this rank's region, exchanges CUDA IPC handles over the communicator and maps the peers' regions.
// False (with *err) when peer access is not available; the caller then keeps to NCCL.  bulk_floats: capacity of the
// many-row exchange per source rank (0: none).
bool peer_init(Comm *, uint32_t n, uint32_t bulk_floats, int device, PeerXchg *out, PeerBulk *bulk_out, std::string *err);

}  // namespace obtp
