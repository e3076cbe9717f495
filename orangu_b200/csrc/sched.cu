// Slot pool and cross-sequence decode coordinator over the C ABI.
//
// The roles of the reference's SlotPool (E/scheduler.rs:36-317: a fixed number of slots, waiters served in arrival order,
// an optional queue limit that refuses instead of growing, pinning to a named slot, a per-slot progress snapshot) and of its
// BatchCoordinator (E/batch.rs:184-324: every generating thread submits its next decode step; steps that arrive inside one
// collection window run as one forward_batch_decode call, led by whichever thread finds the batch full or the window closed),
// with prefill fed in bounded chunks (prefill_in_chunks, E/generate.rs:1299-1338).  Each slot owns an on-demand paged KV cache:
// pages are taken from the model's pool as the sequence grows and go back when the slot is released or rolled back
// (KvCache::truncate, E/kv_cache.rs:496-511), so slots * capacity may exceed the pool and a step that finds it empty fails with
// OB_ERR_CAPACITY without touching any sequence.
//
// All of this is host code: mutex + condition variable, like the reference (its callers are blocking-pool threads).  The only
// device work is what ob_forward / ob_kv_* do.  The coordinator is written against a `forward` callback so that the self-test
// can drive it with a host-side stand-in, the way the reference's own tests use a ModelForward that touches no weights
// (E/batch.rs:326-451).
#include <algorithm>
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstring>
#include <functional>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "../../include/orangu_b200.h"

namespace {

using Clock = std::chrono::steady_clock;

struct Step {  // BatchDecodeRequest + its response (E/batch.rs:151-175)
    uint32_t slot = 0, token = 0;
    float repeat_penalty = 1.0f;
    uint32_t repeat_last_n = 0;
    const uint32_t *recent = nullptr;
    uint32_t n_recent = 0;
    uint32_t *out_token = nullptr;
    float *out_logits = nullptr;
    bool done = false;
    int rc = OB_OK;
    std::string err;
};

// Runs one batch of single-token steps; fills rc/err of every member (all-or-nothing per group, as forward_batch_decode is).
using BatchForward = std::function<void(std::vector<Step *> &)>;

struct Slot {
    ob_kv *kv = nullptr;
    bool busy = false;
    uint32_t prompt_tokens = 0, generated_tokens = 0;
    std::string err;
};

}  // namespace

struct ob_slot_pool {
    ob_model *model = nullptr;
    uint32_t n_vocab = 0;
    ob_slot_pool_desc desc{};
    BatchForward forward;

    // ---- SlotPool
    std::mutex mu;                 // slots, tickets
    std::condition_variable released;
    std::vector<Slot> slots;
    uint64_t next_ticket = 0, serving = 0;  // take_ticket / is_serving (E/scheduler.rs:102-135)
    std::vector<uint64_t> abandoned;        // tickets whose waiter gave up before being served
    uint32_t depth = 0;                     // waiters holding a ticket

    // ---- BatchCoordinator
    std::mutex cmu;
    std::condition_variable cv;
    std::vector<Step *> pending;
    bool window_open = false;
    Clock::time_point deadline;
    uint32_t in_flight = 0;  // batches being executed right now
    uint64_t batches = 0, batched_seqs = 0, refused = 0;

    uint32_t busy_count() {
        std::lock_guard<std::mutex> g(mu);
        uint32_t n = 0;
        for (auto &s : slots) n += s.busy;
        return n;
    }
};

namespace {

thread_local std::string t_err;  // text of the last failure of a pool call on this thread that names no slot

int pool_fail(ob_slot_pool *p, int64_t slot, int code, const std::string &msg) {
    if (p && slot >= 0 && (size_t)slot < p->slots.size()) {
        std::lock_guard<std::mutex> g(p->mu);
        p->slots[(size_t)slot].err = msg;
    }
    t_err = msg;
    return code;
}

// Moves `serving` past tickets whose waiters left, so that an abandoned waiter does not stall the queue.
void skip_abandoned(ob_slot_pool *p) {
    for (bool moved = true; moved;) {
        moved = false;
        for (size_t i = 0; i < p->abandoned.size(); ++i)
            if (p->abandoned[i] == p->serving) {
                p->abandoned.erase(p->abandoned.begin() + (long)i);
                ++p->serving;
                moved = true;
                break;
            }
    }
}

// try_acquire (any slot, slot < 0) and acquire_slot (a named one).  A pinned request holds no ticket: it waits for its slot
// only and therefore cannot delay the queue (E/scheduler.rs:40-52).
int acquire(ob_slot_pool *p, int64_t want, int32_t timeout_ms, uint32_t *out) {
    std::unique_lock<std::mutex> lk(p->mu);
    const bool forever = timeout_ms < 0;
    const auto until = Clock::now() + std::chrono::milliseconds(forever ? 0 : timeout_ms);
    auto take = [&](size_t i) {
        Slot &s = p->slots[i];
        s.busy = true;
        s.prompt_tokens = s.generated_tokens = 0;
        s.err.clear();
        *out = (uint32_t)i;
    };
    if (want >= 0) {
        while (p->slots[(size_t)want].busy) {
            if (forever) p->released.wait(lk);
            else if (p->released.wait_until(lk, until) == std::cv_status::timeout && p->slots[(size_t)want].busy) {
                t_err = "slot_acquire: the named slot stayed busy";
                return OB_ERR_CAPACITY;
            }
        }
        take((size_t)want);
        return OB_OK;
    }
    if (p->desc.max_queue > 0 && p->depth >= p->desc.max_queue) {
        ++p->refused;
        t_err = "slot_acquire: the queue is full";
        return OB_ERR_CAPACITY;  // a_full_queue_refuses_instead_of_growing
    }
    const uint64_t ticket = p->next_ticket++;
    ++p->depth;
    for (;;) {
        if (ticket == p->serving) {
            for (size_t i = 0; i < p->slots.size(); ++i)
                if (!p->slots[i].busy) {
                    take(i);
                    ++p->serving;
                    --p->depth;
                    skip_abandoned(p);
                    p->released.notify_all();  // the next ticket may find another free slot
                    return OB_OK;
                }
        }
        bool timed_out = false;
        if (forever) p->released.wait(lk);
        else timed_out = p->released.wait_until(lk, until) == std::cv_status::timeout;
        if (timed_out) {
            bool free_slot = false;
            for (auto &s : p->slots) free_slot |= !s.busy;
            if (ticket == p->serving && free_slot) continue;  // released in the same instant: take it
            --p->depth;
            ++p->refused;
            if (ticket == p->serving) {
                ++p->serving;
                skip_abandoned(p);
                p->released.notify_all();
            } else {
                p->abandoned.push_back(ticket);
            }
            t_err = "slot_acquire: no slot came free in time";
            return OB_ERR_CAPACITY;
        }
    }
}

// BatchCoordinator::submit (E/batch.rs:207-270).
void submit(ob_slot_pool *p, Step *st) {
    const auto wait = std::chrono::milliseconds(p->desc.batch_wait_ms);
    std::unique_lock<std::mutex> lk(p->cmu);
    if (p->pending.empty()) {
        p->window_open = true;
        p->deadline = Clock::now() + wait;  // fixed by the first arrival of a window, never extended
    }
    p->pending.push_back(st);
    p->cv.notify_all();
    for (;;) {
        if (st->done) return;  // swept into another thread's batch
        lk.unlock();
        const uint32_t target = std::max(1u, p->busy_count());
        lk.lock();
        if (st->done) return;
        // The reference closes a window when it is full or its deadline has passed (E/batch.rs:241-246).  One more condition
        // here: a window whose deadline has passed stays open while another batch is executing -- the model runs one batch at
        // a time, so leading now would only queue behind it, and whoever finishes meanwhile can still join.  Without it, eight
        // streams whose step takes longer than the window never meet: every completion releases one stream into a window of
        // its own (the mean batch of 1.6-2.2 the reference measured, E/batch.rs:66-75).
        if (p->window_open && (p->pending.size() >= target || (Clock::now() >= p->deadline && p->in_flight == 0))) {
            std::vector<Step *> batch;
            batch.swap(p->pending);
            p->window_open = false;
            ++p->batches;
            p->batched_seqs += batch.size();
            ++p->in_flight;
            lk.unlock();
            p->forward(batch);
            lk.lock();
            --p->in_flight;
            for (Step *s : batch) s->done = true;
            p->cv.notify_all();
            return;
        }
        p->cv.wait_for(lk, std::chrono::milliseconds(1));  // POLL_INTERVAL
    }
}

// The product's forward: one ob_forward per group of steps that share their penalty settings (ob_greedy carries one pair
// for the whole call), in slices of the model's batch limit.
void forward_on_model(ob_slot_pool *p, std::vector<Step *> &batch) {
    std::vector<bool> taken(batch.size(), false);
    for (size_t i0 = 0; i0 < batch.size(); ++i0) {
        if (taken[i0]) continue;
        std::vector<Step *> grp;
        for (size_t i = i0; i < batch.size(); ++i)
            if (!taken[i] && batch[i]->repeat_penalty == batch[i0]->repeat_penalty && batch[i]->repeat_last_n == batch[i0]->repeat_last_n) {
                taken[i] = true;
                grp.push_back(batch[i]);
            }
        const uint32_t n = (uint32_t)grp.size();
        std::vector<ob_kv *> kvs(n);
        std::vector<uint32_t> tokens(n), ones(n, 1u), start(n), n_recent(n), recent, out_tok(n);
        bool want_logits = false;
        for (uint32_t i = 0; i < n; ++i) {
            kvs[i] = p->slots[grp[i]->slot].kv;
            tokens[i] = grp[i]->token;
            start[i] = ob_kv_len(kvs[i]);
            n_recent[i] = grp[i]->n_recent;
            recent.insert(recent.end(), grp[i]->recent, grp[i]->recent + grp[i]->n_recent);
            want_logits |= grp[i]->out_logits != nullptr;
        }
        std::vector<float> logits(want_logits ? (size_t)n * p->n_vocab : 0);
        ob_greedy gs{grp[0]->repeat_penalty, grp[0]->repeat_last_n, recent.empty() ? nullptr : recent.data(), n_recent.data()};
        const bool sample = grp[0]->repeat_penalty != 1.0f;
        const int rc = ob_forward(p->model, kvs.data(), tokens.data(), ones.data(), start.data(), n, sample ? &gs : nullptr, out_tok.data(),
                                  want_logits ? logits.data() : nullptr);
        std::string err;
        if (rc != OB_OK) err = ob_last_error(ob_model_ctx(p->model));
        for (uint32_t i = 0; i < n; ++i) {
            grp[i]->rc = rc;
            grp[i]->err = err;
            if (rc != OB_OK) continue;
            if (grp[i]->out_token) *grp[i]->out_token = out_tok[i];
            if (grp[i]->out_logits) std::memcpy(grp[i]->out_logits, logits.data() + (size_t)i * p->n_vocab, (size_t)p->n_vocab * 4);
        }
    }
}

bool slot_held(ob_slot_pool *p, uint32_t slot) {
    std::lock_guard<std::mutex> g(p->mu);
    return slot < p->slots.size() && p->slots[slot].busy;
}

}  // namespace

extern "C" {

// The stand-in for the forward pass of a pool that has no model: the next token of a step is a fixed function of (slot, token),
// so every submitter can tell its own answer from another's (the reference's tests use a ModelForward of that kind,
// E/batch.rs:326-369).
static void forward_stand_in(std::vector<Step *> &b) {
    for (Step *s : b) {
        if (s->out_token) *s->out_token = s->token * 31u + s->slot * 7u + 1u;
        s->rc = OB_OK;
    }
}

int ob_slot_pool_create(ob_model *model, const ob_slot_pool_desc *desc, ob_slot_pool **out) {
    if (!desc || !out || desc->n_slots == 0 || (model && desc->slot_capacity_tokens == 0)) return pool_fail(nullptr, -1, OB_ERR_INVALID, "slot_pool_create: bad argument");
    *out = nullptr;
    if (model && ob_model_tp_size(model) > 1)  // every rank of a tensor-parallel model has to make the same calls; batches formed by arrival time would differ
        return pool_fail(nullptr, -1, OB_ERR_UNSUPPORTED, "slot_pool_create: the decode window serves single-GPU models only");
    ob_slot_pool *p = new ob_slot_pool;
    p->model = model;
    p->desc = *desc;
    if (p->desc.batch_wait_ms == 0) p->desc.batch_wait_ms = 4;    // MAX_BATCH_WAIT_DEFAULT_MS, E/batch.rs:63
    if (p->desc.prefill_batch == 0) p->desc.prefill_batch = 512;  // PREFILL_BATCH_DEFAULT, E/generate.rs:1265
    p->slots.resize(desc->n_slots);
    if (!model) {  // scheduling only (host-side tests, or a host that wants the pool without the library's caches)
        p->forward = forward_stand_in;
        *out = p;
        return OB_OK;
    }
    p->n_vocab = ob_model_n_vocab(model);
    for (auto &s : p->slots) {
        const int rc = ob_kv_create_paged(model, desc->slot_capacity_tokens, &s.kv);
        if (rc != OB_OK) {
            t_err = ob_last_error(ob_model_ctx(model));
            for (auto &s2 : p->slots)
                if (s2.kv) ob_kv_destroy(s2.kv);
            delete p;
            return rc;
        }
    }
    p->forward = [p](std::vector<Step *> &b) { forward_on_model(p, b); };
    *out = p;
    return OB_OK;
}

void ob_slot_pool_destroy(ob_slot_pool *p) {
    if (!p) return;
    for (auto &s : p->slots)
        if (s.kv) ob_kv_destroy(s.kv);
    delete p;
}

int ob_slot_acquire(ob_slot_pool *p, int32_t timeout_ms, uint32_t *slot_id) {
    if (!p || !slot_id) return pool_fail(p, -1, OB_ERR_INVALID, "slot_acquire: null argument");
    return acquire(p, -1, timeout_ms, slot_id);
}

int ob_slot_acquire_id(ob_slot_pool *p, uint32_t slot_id, int32_t timeout_ms) {
    if (!p || slot_id >= p->slots.size()) return pool_fail(p, -1, OB_ERR_INVALID, "slot_acquire_id: no such slot");
    uint32_t got = 0;
    return acquire(p, slot_id, timeout_ms, &got);
}

int ob_slot_release(ob_slot_pool *p, uint32_t slot_id) {
    if (!p || !slot_held(p, slot_id)) return pool_fail(p, -1, OB_ERR_INVALID, "slot_release: the slot is not held");
    if (p->slots[slot_id].kv) {
        const int rc = ob_kv_truncate(p->slots[slot_id].kv, 0);  // every page back to the pool
        if (rc != OB_OK) return pool_fail(p, slot_id, rc, ob_last_error(ob_model_ctx(p->model)));
    }
    {
        std::lock_guard<std::mutex> g(p->mu);
        p->slots[slot_id].busy = false;
    }
    p->released.notify_all();
    p->cv.notify_all();  // the decode target (busy slots) just dropped
    return OB_OK;
}

int ob_slot_prefill(ob_slot_pool *p, uint32_t slot_id, const uint32_t *tokens, uint32_t n_tokens, uint32_t *out_token, float *out_logits) {
    if (!p || !tokens || n_tokens == 0) return pool_fail(p, -1, OB_ERR_INVALID, "slot_prefill: bad argument");
    if (!slot_held(p, slot_id) || !p->model) return pool_fail(p, -1, OB_ERR_INVALID, "slot_prefill: the slot is not held");
    ob_kv *kv = p->slots[slot_id].kv;
    const uint32_t width = p->desc.prefill_batch;
    for (uint32_t done = 0; done < n_tokens;) {
        const uint32_t n = std::min(width, n_tokens - done);
        const uint32_t start = ob_kv_len(kv);
        const bool last = done + n == n_tokens;
        // between chunks the context is free, so decode batches of other slots interleave with a long prompt
        const int rc = ob_forward(p->model, &kv, tokens + done, &n, &start, 1, nullptr, last ? out_token : nullptr, last ? out_logits : nullptr);
        if (rc != OB_OK) return pool_fail(p, slot_id, rc, ob_last_error(ob_model_ctx(p->model)));
        done += n;
        std::lock_guard<std::mutex> g(p->mu);
        p->slots[slot_id].prompt_tokens += n;  // on_chunk -> SlotGuard::set_prompt_tokens
    }
    return OB_OK;
}

int ob_slot_decode(ob_slot_pool *p, uint32_t slot_id, uint32_t token, const ob_greedy *greedy, uint32_t *out_token, float *out_logits) {
    if (!p || (!out_token && !out_logits)) return pool_fail(p, -1, OB_ERR_INVALID, "slot_decode: bad argument");
    if (!slot_held(p, slot_id)) return pool_fail(p, -1, OB_ERR_INVALID, "slot_decode: the slot is not held");
    Step st;
    st.slot = slot_id;
    st.token = token;
    st.out_token = out_token;
    st.out_logits = out_logits;
    if (greedy) {
        st.repeat_penalty = greedy->repeat_penalty;
        st.repeat_last_n = greedy->repeat_last_n;
        st.recent = greedy->recent;
        st.n_recent = greedy->recent && greedy->n_recent ? greedy->n_recent[0] : 0;
    }
    if (p->desc.batch_decode) {
        submit(p, &st);
    } else {  // the reference's default: every sequence steps on its own (ORANGU_BATCH_DECODE unset)
        std::vector<Step *> one{&st};
        {
            std::lock_guard<std::mutex> g(p->cmu);
            ++p->batches;
            ++p->batched_seqs;
        }
        p->forward(one);
    }
    if (st.rc != OB_OK) return pool_fail(p, slot_id, st.rc, st.err);
    std::lock_guard<std::mutex> g(p->mu);
    ++p->slots[slot_id].generated_tokens;
    return OB_OK;
}

int ob_slot_truncate(ob_slot_pool *p, uint32_t slot_id, uint32_t new_len) {
    if (!p || !slot_held(p, slot_id) || !p->slots[slot_id].kv) return pool_fail(p, -1, OB_ERR_INVALID, "slot_truncate: the slot is not held");
    const int rc = ob_kv_truncate(p->slots[slot_id].kv, new_len);
    return rc == OB_OK ? rc : pool_fail(p, slot_id, rc, ob_last_error(ob_model_ctx(p->model)));
}

uint32_t ob_slot_len(const ob_slot_pool *p, uint32_t slot_id) {
    return p && slot_id < p->slots.size() && p->slots[slot_id].kv ? ob_kv_len(p->slots[slot_id].kv) : 0u;
}

ob_kv *ob_slot_kv(ob_slot_pool *p, uint32_t slot_id) { return p && slot_id < p->slots.size() ? p->slots[slot_id].kv : nullptr; }

uint32_t ob_slot_pool_snapshot(ob_slot_pool *p, ob_slot_state *out, uint32_t cap) {
    if (!p) return 0;
    std::lock_guard<std::mutex> g(p->mu);
    const uint32_t n = (uint32_t)p->slots.size();
    for (uint32_t i = 0; out && i < std::min(n, cap); ++i) out[i] = ob_slot_state{i, p->slots[i].busy ? 1u : 0u, p->slots[i].prompt_tokens, p->slots[i].generated_tokens};
    return n;
}

int ob_slot_pool_get_stats(ob_slot_pool *p, ob_slot_pool_stats *out) {
    if (!p || !out) return pool_fail(p, -1, OB_ERR_INVALID, "slot_pool_stats: null argument");
    {
        std::lock_guard<std::mutex> g(p->cmu);
        out->batches = p->batches;
        out->batched_seqs = p->batched_seqs;
    }
    std::lock_guard<std::mutex> g(p->mu);
    out->refused = p->refused;
    out->total = (uint32_t)p->slots.size();
    out->busy = 0;
    for (auto &s : p->slots) out->busy += s.busy;
    out->queued = p->depth;
    out->free_pages = p->model ? ob_model_free_pages(p->model) : 0;
    return OB_OK;
}

const char *ob_slot_last_error(ob_slot_pool *p, int64_t slot_id) {
    if (p && slot_id >= 0 && (size_t)slot_id < p->slots.size()) {
        std::lock_guard<std::mutex> g(p->mu);
        t_err = p->slots[(size_t)slot_id].err;
    }
    return t_err.c_str();
}

// Host-only check of the pool and the coordinator, with a stand-in for the forward pass that touches no device: the next
// token of a step is a fixed function of (slot, token), so every submitter can tell its own answer from another's
// (concurrent_submissions_each_get_their_own_correct_result, E/batch.rs:372-426).  n_threads generating threads contend for
// n_slots slots; each acquires a slot, runs n_steps decode steps through the window and releases.  Returns OB_OK when every
// answer was the submitter's own, no two holders shared a slot and every waiter was served; fills `out` with the totals.
int ob_slot_pool_selftest(uint32_t n_slots, uint32_t n_threads, uint32_t n_steps, uint32_t batch_wait_ms, uint32_t max_queue, ob_slot_pool_stats *out) {
    if (n_slots == 0 || n_threads == 0 || !out) return pool_fail(nullptr, -1, OB_ERR_INVALID, "slot_pool_selftest: bad argument");
    ob_slot_pool pool;
    pool.desc = ob_slot_pool_desc{n_slots, 1, max_queue, batch_wait_ms ? batch_wait_ms : 4, 512, 1};
    pool.slots.resize(n_slots);
    std::vector<int> holders(n_slots, 0);
    std::mutex hmu;
    pool.forward = forward_stand_in;
    std::vector<int> bad(n_threads, 0), refused(n_threads, 0);
    // the first holders of the slots start stepping together, so that the window has company from its first step on
    std::atomic<uint32_t> holders_so_far{0};
    const uint32_t first_wave = std::min(n_threads, n_slots);
    std::vector<std::thread> th;
    for (uint32_t t = 0; t < n_threads; ++t)
        th.emplace_back([&, t] {
            uint32_t slot = 0;
            if (acquire(&pool, -1, -1, &slot) != OB_OK) {
                refused[t] = 1;
                return;
            }
            {
                std::lock_guard<std::mutex> g(hmu);
                if (++holders[slot] != 1) bad[t] = 1;  // every_concurrent_acquire_gets_a_distinct_slot
            }
            if (holders_so_far.fetch_add(1) < first_wave)
                while (holders_so_far.load() < first_wave) std::this_thread::yield();
            uint32_t tok = 1000u * t;
            for (uint32_t i = 0; i < n_steps; ++i) {
                uint32_t next = 0;
                Step st;
                st.slot = slot;
                st.token = tok;
                st.out_token = &next;
                submit(&pool, &st);
                if (st.rc != OB_OK || next != tok * 31u + slot * 7u + 1u) bad[t] = 1;
                tok = next % 50021u;
            }
            {
                std::lock_guard<std::mutex> g(hmu);
                --holders[slot];
            }
            {
                std::lock_guard<std::mutex> g(pool.mu);
                pool.slots[slot].busy = false;
            }
            pool.released.notify_all();
            pool.cv.notify_all();
        });
    for (auto &x : th) x.join();
    out->batches = pool.batches;
    out->batched_seqs = pool.batched_seqs;
    out->refused = pool.refused;
    out->total = n_slots;
    out->busy = pool.busy_count();
    out->queued = pool.depth;
    out->free_pages = 0;
    uint32_t n_bad = 0, n_refused = 0;
    for (uint32_t t = 0; t < n_threads; ++t) {
        n_bad += (uint32_t)bad[t];
        n_refused += (uint32_t)refused[t];
    }
    if (n_bad) return pool_fail(nullptr, -1, OB_ERR_INVALID, "slot_pool_selftest: a submitter received another's answer, or two holders shared a slot");
    if (out->busy != 0 || out->queued != 0) return pool_fail(nullptr, -1, OB_ERR_INVALID, "slot_pool_selftest: slots or tickets leaked");
    if (pool.batched_seqs != (uint64_t)(n_threads - n_refused) * n_steps) return pool_fail(nullptr, -1, OB_ERR_INVALID, "slot_pool_selftest: steps lost");
    if (max_queue == 0 && n_refused) return pool_fail(nullptr, -1, OB_ERR_INVALID, "slot_pool_selftest: an unbounded pool refused");
    return OB_OK;
}

}  // extern "C"
