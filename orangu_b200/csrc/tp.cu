// Tensor-parallel plumbing: the NCCL binding (all-reduce after the contraction-split products, logits gather), resolved with
// dlopen at run time, and the set-up of the peer-memory exchange the single-token step uses instead (a region per rank, CUDA
// IPC handles all-gathered over the communicator, the peers' regions mapped).  The reference engine has no collective of any
// kind; its multi-GPU mode moves activations through host memory between layer ranges (engine/backend/multi.rs:16-35).
#include "tp.h"

#include <dlfcn.h>
#include <fcntl.h>
#include <sched.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/mman.h>
#include <time.h>
#include <unistd.h>

#include <algorithm>

#include <vector>

namespace obtp {

namespace {

typedef struct {
    char internal[128];
} UniqueId;
typedef void *NcclComm;
typedef int NcclResult;
constexpr int kNcclFloat = 7, kNcclSum = 0;

struct Api {
    void *handle = nullptr;
    NcclResult (*GetUniqueId)(UniqueId *) = nullptr;
    NcclResult (*CommInitRank)(NcclComm *, int, UniqueId, int) = nullptr;
    NcclResult (*CommDestroy)(NcclComm) = nullptr;
    NcclResult (*AllReduce)(const void *, void *, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
    NcclResult (*AllGather)(const void *, void *, size_t, int, NcclComm, cudaStream_t) = nullptr;
    NcclResult (*GroupStart)() = nullptr;
    NcclResult (*GroupEnd)() = nullptr;
    const char *(*GetErrorString)(NcclResult) = nullptr;
    std::string err;
};

Api *api() {
    static Api a;
    static bool tried = false;
    if (tried) return a.handle ? &a : nullptr;
    tried = true;
    for (const char *name : {"libnccl.so.2", "libnccl.so"}) {
        a.handle = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
        if (a.handle) break;
    }
    if (!a.handle) {
        a.err = std::string("cannot load libnccl: ") + dlerror();
        return nullptr;
    }
    bool ok = true;
    auto sym = [&](const char *n) {
        void *p = dlsym(a.handle, n);
        if (!p) {
            ok = false;
            a.err = std::string("libnccl lacks ") + n;
        }
        return p;
    };
    a.GetUniqueId = reinterpret_cast<decltype(a.GetUniqueId)>(sym("ncclGetUniqueId"));
    a.CommInitRank = reinterpret_cast<decltype(a.CommInitRank)>(sym("ncclCommInitRank"));
    a.CommDestroy = reinterpret_cast<decltype(a.CommDestroy)>(sym("ncclCommDestroy"));
    a.AllReduce = reinterpret_cast<decltype(a.AllReduce)>(sym("ncclAllReduce"));
    a.AllGather = reinterpret_cast<decltype(a.AllGather)>(sym("ncclAllGather"));
    a.GroupStart = reinterpret_cast<decltype(a.GroupStart)>(sym("ncclGroupStart"));
    a.GroupEnd = reinterpret_cast<decltype(a.GroupEnd)>(sym("ncclGroupEnd"));
    a.GetErrorString = reinterpret_cast<decltype(a.GetErrorString)>(sym("ncclGetErrorString"));
    if (!ok) {
        a.handle = nullptr;
        return nullptr;
    }
    return &a;
}

std::string api_error() { return "NCCL unavailable (libnccl.so.2 could not be loaded or lacks a symbol)"; }

}  // namespace

struct Comm {
    NcclComm comm = nullptr;
    int rank = 0, size = 1;
    std::string err;
    void *peer_region = nullptr;    // this rank's exchange region
    void *peer_mapped[8] = {};      // the peers' regions as mapped here
    unsigned char *scratch = nullptr;  // small device buffer for the set-up collectives, made with the communicator so that
                                       // no rank can fail to have it when the others already wait inside NCCL
};
constexpr size_t kScratchBytes = 8 * sizeof(cudaIpcMemHandle_t) + 64;

bool unique_id(void *out128, std::string *err) {
    Api *a = api();
    if (!a) {
        if (err) *err = api_error();
        return false;
    }
    UniqueId id;
    NcclResult r = a->GetUniqueId(&id);
    if (r != 0) {
        if (err) *err = std::string("ncclGetUniqueId: ") + a->GetErrorString(r);
        return false;
    }
    memcpy(out128, id.internal, 128);
    return true;
}

Comm *create(const void *id128, int rank, int size, int device, std::string *err) {
    Api *a = api();
    if (!a) {
        if (err) *err = api_error();
        return nullptr;
    }
    UniqueId id;
    memcpy(id.internal, id128, 128);
    cudaSetDevice(device);
    Comm *c = new Comm;
    c->rank = rank;
    c->size = size;
    NcclResult r = a->CommInitRank(&c->comm, size, id, rank);
    if (r != 0) {
        if (err) *err = std::string("ncclCommInitRank: ") + a->GetErrorString(r);
        delete c;
        return nullptr;
    }
    if (cudaMalloc(reinterpret_cast<void **>(&c->scratch), kScratchBytes) != cudaSuccess) {  // 576 bytes, right after NCCL took its megabytes
        if (err) *err = "cudaMalloc of the communicator's scratch buffer failed";
        a->CommDestroy(c->comm);
        delete c;
        return nullptr;
    }
    return c;
}

void destroy(Comm *c) {
    if (!c) return;
    for (void *p : c->peer_mapped)
        if (p) cudaIpcCloseMemHandle(p);
    if (c->peer_region) cudaFree(c->peer_region);
    if (c->scratch) cudaFree(c->scratch);
    Api *a = api();
    if (a && c->comm) a->CommDestroy(c->comm);
    delete c;
}

bool all_reduce_sum(Comm *c, float *buf, size_t count, cudaStream_t st) {
    Api *a = api();
    NcclResult r = a->AllReduce(buf, buf, count, kNcclFloat, kNcclSum, c->comm, st);
    if (r != 0) {
        c->err = std::string("ncclAllReduce: ") + a->GetErrorString(r);
        return false;
    }
    return true;
}

bool all_gather_logits(Comm *c, float *logits, uint32_t rows, uint32_t n_vocab, uint32_t vocab0, uint32_t vocab_l, cudaStream_t st) {
    Api *a = api();
    NcclResult r = a->GroupStart();
    for (uint32_t i = 0; i < rows && r == 0; ++i) {
        float *row = logits + (size_t)i * n_vocab;
        r = a->AllGather(row + vocab0, row, vocab_l, kNcclFloat, c->comm, st);
    }
    NcclResult r2 = a->GroupEnd();
    if (r == 0) r = r2;
    if (r != 0) {
        c->err = std::string("ncclAllGather: ") + a->GetErrorString(r);
        return false;
    }
    return true;
}

const char *last_error(Comm *c) { return c ? c->err.c_str() : ""; }

static bool peer_init_local(Comm *c, uint32_t n, uint32_t bulk_floats, int device, PeerXchg *out, PeerBulk *bulk_out, std::string *err) {
    auto bail = [&](const std::string &m) {
        if (err) *err = m;
        return false;
    };
    Api *a = api();
    if (!a || !c || c->size < 2 || c->size > 8) return bail("peer exchange needs 2 to 8 ranks");
    cudaSetDevice(device);
    constexpr size_t kFlagBytes = 256, kLocalBytes = 256;
    const uint32_t bulk_cap = (bulk_floats + kBulkChunk - 1) / kBulkChunk * kBulkChunk, max_chunks = bulk_cap / kBulkChunk;
    const size_t slot_bytes = (size_t)2 * c->size * n * sizeof(uint2);
    const size_t bulk_flag_bytes = ((size_t)2 * c->size * max_chunks * 4 + 255) & ~(size_t)255, bulk_bytes = (size_t)2 * c->size * bulk_cap * 4;
    const size_t total = kFlagBytes + kLocalBytes + slot_bytes + bulk_flag_bytes + bulk_bytes;
    // Every rank reaches the all-gather below, whatever happened before it (a rank that skipped it would leave the others
    // waiting in NCCL); a rank without a region sends a zero handle and fails afterwards.
    cudaIpcMemHandle_t mine;
    memset(&mine, 0, sizeof(mine));
    std::string early;
    if (cudaMalloc(&c->peer_region, total) != cudaSuccess) {
        c->peer_region = nullptr;
        early = "cudaMalloc of the exchange region failed";
    } else {
        cudaMemset(c->peer_region, 0, total);
        if (cudaIpcGetMemHandle(&mine, c->peer_region) != cudaSuccess) early = std::string("cudaIpcGetMemHandle: ") + cudaGetErrorString(cudaGetLastError());
    }
    // all-gather the 64-byte handles through the communicator
    unsigned char *stage = c->scratch;  // preallocated: nothing between here and the collective can fail on one rank only
    cudaMemcpy(stage + (size_t)c->rank * sizeof(mine), &mine, sizeof(mine), cudaMemcpyHostToDevice);
    NcclResult r = a->AllGather(stage + (size_t)c->rank * sizeof(mine), stage, sizeof(mine), /* ncclChar */ 0, c->comm, nullptr);
    cudaError_t e = cudaStreamSynchronize(nullptr);
    std::vector<cudaIpcMemHandle_t> all((size_t)c->size);
    if (r == 0 && e == cudaSuccess) e = cudaMemcpy(all.data(), stage, all.size() * sizeof(mine), cudaMemcpyDeviceToHost);
    if (!early.empty()) return bail(early);
    if (r != 0 || e != cudaSuccess) return bail("exchange of the IPC handles failed");
    PeerXchg px{};
    px.rank = (uint32_t)c->rank;
    px.size = (uint32_t)c->size;
    px.n = n;
    for (int p = 0; p < c->size; ++p) {
        void *base = c->peer_region;
        if (p != c->rank) {
            if (cudaIpcOpenMemHandle(&base, all[(size_t)p], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess)
                return bail(std::string("cudaIpcOpenMemHandle: ") + cudaGetErrorString(cudaGetLastError()));
            c->peer_mapped[p] = base;
        }
        px.slots[p] = reinterpret_cast<uint2 *>(static_cast<unsigned char *>(base) + kFlagBytes + kLocalBytes);
        if (bulk_out) {
            bulk_out->flags[p] = reinterpret_cast<uint32_t *>(static_cast<unsigned char *>(base) + kFlagBytes + kLocalBytes + slot_bytes);
            bulk_out->data[p] = reinterpret_cast<float *>(static_cast<unsigned char *>(base) + kFlagBytes + kLocalBytes + slot_bytes + bulk_flag_bytes);
        }
    }
    uint32_t *local = reinterpret_cast<uint32_t *>(static_cast<unsigned char *>(c->peer_region) + kFlagBytes);
    px.seq = local;
    px.err = local + 32;
    if (bulk_out) {
        bulk_out->done = local + 40;
        bulk_out->cap = bulk_cap;
        bulk_out->max_chunks = max_chunks;
    }
    px.timeout_ms = 4000;
    if (const char *e = getenv("OB_TP_TIMEOUT_MS")) px.timeout_ms = (uint32_t)std::max(1, atoi(e));
    *out = px;
    return true;
}

bool peer_init(Comm *c, uint32_t n, uint32_t bulk_floats, int device, PeerXchg *out, PeerBulk *bulk_out, std::string *err) {
    Api *a = api();
    if (!a || !c) return false;
    // Every rank must take the same path afterwards: the exchange is used only if it could be set up everywhere.
    // Both collectives -- the handle all-gather inside peer_init_local and the agreement below -- run out of the scratch
    // buffer made with the communicator, so a rank whose own allocations fail still reaches them (with a zero handle and
    // a 0 vote) instead of leaving the others waiting inside NCCL.
    const bool mine = peer_init_local(c, n, bulk_floats, device, out, bulk_out, err);
    int *flag = reinterpret_cast<int *>(c->scratch + 8 * sizeof(cudaIpcMemHandle_t));
    const int v = mine ? 1 : 0;
    cudaMemcpy(flag, &v, sizeof(int), cudaMemcpyHostToDevice);
    const NcclResult r = a->AllReduce(flag, flag, 1, /* ncclInt32 */ 2, /* ncclMin */ 2, c->comm, nullptr);
    int all = 0;
    if (r == 0 && cudaStreamSynchronize(nullptr) == cudaSuccess) cudaMemcpy(&all, flag, sizeof(int), cudaMemcpyDeviceToHost);
    if (!all && err && err->empty()) *err = "another rank could not set up the peer exchange";
    return all == 1;
}

// ---- host-side rendezvous ----------------------------------------------------------------------------------------------
struct Rendezvous {
    volatile uint64_t *slots = nullptr;  // one counter per rank, 64 bytes apart
    std::string name;
    int rank = 0, size = 1;
    uint64_t step = 0;
    bool unlinked = false;
};

Rendezvous *rendezvous_open(const void *id128, int rank, int size, std::string *err) {
    if (!id128 || rank < 0 || size < 1 || size > 64 || rank >= size) {
        if (err) *err = "rendezvous: bad rank or size";
        return nullptr;
    }
    uint64_t h = 1469598103934665603ull;  // FNV-1a over the id: the name only has to differ between jobs
    for (int i = 0; i < 128; ++i) h = (h ^ static_cast<const unsigned char *>(id128)[i]) * 1099511628211ull;
    char name[64];
    snprintf(name, sizeof(name), "/ob_tp_%016llx", (unsigned long long)h);
    const int fd = shm_open(name, O_CREAT | O_RDWR, 0600);
    if (fd < 0 || ftruncate(fd, 4096) != 0) {
        if (fd >= 0) close(fd);
        if (err) *err = std::string("rendezvous: shm_open/ftruncate of ") + name + " failed";
        return nullptr;
    }
    void *p = mmap(nullptr, 4096, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);  // a fresh segment reads as zeros
    close(fd);
    if (p == MAP_FAILED) {
        if (err) *err = "rendezvous: mmap failed";
        return nullptr;
    }
    Rendezvous *r = new Rendezvous;
    r->slots = static_cast<volatile uint64_t *>(p);
    r->name = name;
    r->rank = rank;
    r->size = size;
    return r;
}

bool rendezvous_arrive(Rendezvous *r, uint32_t timeout_ms, int *missing) {
    if (!r || timeout_ms == 0) return true;
    const uint64_t step = ++r->step;
    __atomic_store_n(const_cast<uint64_t *>(&r->slots[(size_t)r->rank * 8]), step, __ATOMIC_RELEASE);
    timespec t0;
    clock_gettime(CLOCK_MONOTONIC, &t0);
    for (int p = 0; p < r->size; ++p) {
        for (uint32_t spin = 0; __atomic_load_n(const_cast<uint64_t *>(&r->slots[(size_t)p * 8]), __ATOMIC_ACQUIRE) < step; ++spin) {
            if ((spin & 255u) != 255u) continue;
            timespec t1;
            clock_gettime(CLOCK_MONOTONIC, &t1);
            const int64_t ms = (int64_t)(t1.tv_sec - t0.tv_sec) * 1000 + (t1.tv_nsec - t0.tv_nsec) / 1000000;
            if (ms > (int64_t)timeout_ms) {
                if (missing) *missing = p;
                return false;
            }
            if (spin > 4096u) {  // the others are not about to arrive: stop burning the core
                timespec nap{0, 50000};
                nanosleep(&nap, nullptr);
            } else {
                sched_yield();
            }
        }
    }
    // everybody has the segment mapped by now: its name can go, so that nothing is left behind whichever way the job ends
    if (step == 1 && r->rank == 0 && !r->unlinked) {
        shm_unlink(r->name.c_str());
        r->unlinked = true;
    }
    return true;
}

void rendezvous_close(Rendezvous *r) {
    if (!r) return;
    if (r->rank == 0 && !r->unlinked) shm_unlink(r->name.c_str());
    munmap(const_cast<uint64_t *>(r->slots), 4096);
    delete r;
}

}  // namespace obtp
