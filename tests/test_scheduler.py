"""Slot pool, decode collection window and on-demand KV pages.

The host-only cases follow the reference's own tests of SlotPool (src/bin/orangu-server/engine/scheduler.rs:355-639) and
BatchCoordinator (engine/batch.rs:371-451), which use a ModelForward that touches no weights; here the library's self-test
plays that part.  The GPU cases run real sequences through the pool and compare every token with the CPU oracle."""
import threading
import time

import numpy as np
import pytest

import oracle as O
from gpu_common import assert_bit_equal, backend  # noqa: F401
from orangu_b200 import capi, scheduler


def test_concurrent_submissions_each_get_their_own_correct_result():
    rc, st = scheduler.selftest(n_slots=8, n_threads=8, n_steps=200, batch_wait_ms=4)
    assert rc == 0, capi.load().ob_slot_last_error(None, -1)
    assert st["batched_seqs"] == 8 * 200 and st["busy"] == 0 and st["queued"] == 0
    assert st["batches"] < st["batched_seqs"], "eight threads stepping in lockstep must share batches"


def test_solo_submission_completes_via_deadline_fallback():
    rc, st = scheduler.selftest(n_slots=4, n_threads=1, n_steps=5, batch_wait_ms=2)
    assert rc == 0 and st["batches"] == 5 and st["batched_seqs"] == 5


def test_more_requests_than_slots_wait_their_turn_and_all_finish():
    rc, st = scheduler.selftest(n_slots=2, n_threads=9, n_steps=20, batch_wait_ms=1)
    assert rc == 0, capi.load().ob_slot_last_error(None, -1)
    assert st["batched_seqs"] == 9 * 20 and st["refused"] == 0  # an_unbounded_pool_never_refuses


def test_a_full_queue_refuses_instead_of_growing():
    rc, st = scheduler.selftest(n_slots=1, n_threads=12, n_steps=30, batch_wait_ms=1, max_queue=2)
    assert rc == 0, capi.load().ob_slot_last_error(None, -1)
    served = st["batched_seqs"] // 30
    assert served + st["refused"] == 12 and 1 <= served <= 12 and st["busy"] == 0 and st["queued"] == 0


def test_pool_rejects_bad_arguments_without_a_device():
    L = capi.load()
    assert L.ob_slot_pool_create(None, None, None) == -1
    assert L.ob_slot_acquire(None, 0, None) == -1
    assert L.ob_slot_len(None, 0) == 0 and L.ob_kv_pages(None) == 0 and L.ob_model_free_pages(None) == 0
    assert L.ob_slot_pool_selftest(0, 1, 1, 1, 0, None) == -1


# ---- the pool itself, without a model: the cases of the reference's own SlotPool tests (scheduler.rs:355-639) ---------------
def bare_pool(n, **kw):
    return scheduler.SlotPool(None, n_slots=n, slot_capacity_tokens=0, **kw)


def test_acquire_marks_a_slot_busy_and_release_frees_it():
    pool = bare_pool(2)
    assert pool.busy_count() == 0
    g = pool.try_acquire()
    assert pool.busy_count() == 1 and pool.snapshot()[g.id()]["busy"] == 1
    g.release()
    assert pool.busy_count() == 0
    pool.close()


def test_acquire_slot_gives_back_the_slot_that_was_asked_for_and_waits_for_it_even_when_others_are_free():
    pool = bare_pool(3)
    g = pool.acquire_slot(2)
    assert g.id() == 2
    assert pool.acquire_slot(2, timeout_ms=30) is None  # slot 2 is busy; slots 0 and 1 being free does not matter
    got = []
    t = threading.Thread(target=lambda: got.append(pool.acquire_slot(2, timeout_ms=5000)))
    t.start()
    time.sleep(0.05)
    assert not got  # still waiting for that slot
    g.release()
    t.join(5)
    assert got and got[0].id() == 2
    got[0].release()
    pool.close()


def test_every_concurrent_acquire_gets_a_distinct_slot_and_a_third_request_waits_when_both_are_busy():
    pool = bare_pool(2)
    a, b = pool.try_acquire(), pool.try_acquire()
    assert {a.id(), b.id()} == {0, 1}
    got = []
    t = threading.Thread(target=lambda: got.append(pool.try_acquire(5000)))
    t.start()
    time.sleep(0.05)
    assert not got and pool.stats()["queued"] == 1
    freed = b.id()
    b.release()
    t.join(5)
    assert got and got[0].id() == freed and pool.stats()["queued"] == 0
    a.release()
    got[0].release()
    pool.close()


def test_waiters_are_served_in_arrival_order_and_an_abandoned_waiter_does_not_stall_the_queue():
    pool = bare_pool(1)
    held = pool.try_acquire()
    order, lock = [], threading.Lock()

    def waiter(name, timeout_ms):
        g = pool.try_acquire(timeout_ms)
        with lock:
            order.append((name, g is not None))
        if g is not None:
            time.sleep(0.02)
            g.release()

    threads = []
    for name, timeout_ms in (("first", 5000), ("gives up", 60), ("third", 5000), ("fourth", 5000)):
        th = threading.Thread(target=waiter, args=(name, timeout_ms))
        th.start()
        threads.append(th)
        time.sleep(0.03)  # arrival order is the start order
    time.sleep(0.15)      # "gives up" has left the queue by now, from the middle of it
    assert order == [("gives up", False)]
    held.release()
    for th in threads:
        th.join(5)
    assert order == [("gives up", False), ("first", True), ("third", True), ("fourth", True)]
    assert pool.stats()["queued"] == 0 and pool.busy_count() == 0
    pool.close()


def test_a_pinned_waiter_does_not_starve_or_deadlock_unpinned_requests():
    """A request waiting for a named slot holds no place in the queue: the others keep cycling through the free slot."""
    pool = bare_pool(2)
    pinned_holder = pool.acquire_slot(0)
    got = []
    t = threading.Thread(target=lambda: got.append(pool.acquire_slot(0, timeout_ms=5000)))
    t.start()
    time.sleep(0.03)
    for _ in range(5):  # slot 1 keeps serving unpinned requests while the pinned one waits
        g = pool.try_acquire(1000)
        assert g is not None and g.id() == 1
        g.release()
    assert not got
    pinned_holder.release()
    t.join(5)
    assert got and got[0].id() == 0
    got[0].release()
    pool.close()


def test_a_full_queue_refuses_through_the_public_calls_and_counts_it():
    pool = bare_pool(1, max_queue=1)
    held = pool.try_acquire()
    t = threading.Thread(target=lambda: pool.try_acquire(300))  # fills the queue
    t.start()
    time.sleep(0.05)
    assert pool.try_acquire(1000) is None  # refused at once: the queue is full
    assert pool.stats()["refused"] >= 1
    t.join(5)
    held.release()
    pool.close()


def test_decode_steps_through_the_window_of_a_bare_pool_get_their_own_answers():
    pool = bare_pool(4, batch_wait_ms=5)
    results = {}
    all_hold_a_slot = threading.Barrier(4)  # the window's target is the number of busy slots: let every stream hold one first

    def run(i):
        with pool.try_acquire() as slot:
            all_hold_a_slot.wait(10)
            tok, out = 100 * i, []
            for _ in range(50):
                nxt = slot.decode(tok)
                assert nxt == (tok * 31 + slot.id() * 7 + 1) % (1 << 32)
                out.append(nxt)
                tok = nxt % 50021
            results[i] = out

    threads = [threading.Thread(target=run, args=(i,)) for i in range(4)]
    for th in threads:
        th.start()
    for th in threads:
        th.join(30)
    assert len(results) == 4
    st = pool.stats()
    assert st["batched_seqs"] == 200 and st["batches"] < 200
    with pytest.raises(Exception):
        with pool.try_acquire() as slot:
            slot.prefill([1, 2, 3])  # a pool without a model schedules only
    pool.close()


# ------------------------------------------------------------------------------------------ on a GPU

def _build(backend, name="small", seed=11, **kw):
    from orangu_b200 import LlamaModel, synth

    cfg = dict(synth.CONFIGS[name])
    tensors = synth.model_tensors(cfg, seed=seed)
    return cfg, LlamaModel(backend, cfg, tensors, **kw), O.Model(cfg, tensors)


def _oracle_run(ref, toks, n_new, capacity=256):
    rkv = ref.new_kv(capacity, f16=True)
    nxt = O.argmax(ref.forward(rkv, toks, 0))
    out = [nxt]
    for i in range(n_new - 1):
        nxt = O.argmax(ref.forward(rkv, [nxt], len(toks) + i))
        out.append(nxt)
    return out


@pytest.mark.gpu
def test_on_demand_pages_grow_shrink_and_match_the_reserved_cache(backend):
    cfg, model, ref = _build(backend, "tiny", max_seq_len=256, max_batch_tokens=32, kv_pool_tokens=320)
    pool = model.pool_pages
    assert model.free_pages == pool
    toks = np.random.default_rng(1).integers(0, cfg["n_vocab"], 37).astype(np.uint32)
    a, b = model.new_kv_cache(200), model.new_kv_cache(200, paged=True)
    assert a.pages == 13 and b.pages == 0 and model.free_pages == pool - 13
    la, lb = model.forward(a, toks, 0), model.forward(b, toks, 0)
    assert_bit_equal(la, lb, "paged cache logits")
    assert b.pages == 3 and model.free_pages == pool - 16
    for step in range(14):  # crosses the 48-token page boundary
        la, lb = model.forward(a, [5 + step], 37 + step), model.forward(b, [5 + step], 37 + step)
        assert_bit_equal(la, lb, f"paged decode step {step}")
    assert b.pages == 4
    assert model.decode_greedy(a, 3) == model.decode_greedy(b, 3)
    got = model.decode_loop([b], [9], 20)[:, 0]
    want = model.decode_loop([a], [9], 20)[:, 0]
    assert (got == want).all() and b.pages == (len(b) + 15) // 16
    b.truncate(17)
    assert b.pages == 2 and len(b) == 17
    a.truncate(17)
    assert_bit_equal(model.forward(a, [7], 17), model.forward(b, [7], 17), "after rollback")
    # a pool that runs dry refuses the call and changes nothing
    big = [model.new_kv_cache(200, paged=True) for _ in range(3)]
    free = model.free_pages
    long_prompt = np.arange(16 * free + 1, dtype=np.uint32) % cfg["n_vocab"]
    from orangu_b200 import OranguError

    with pytest.raises(OranguError) as e:
        model._forward(big[:1], [list(long_prompt[:200])], [0]) if free * 16 < 200 else model._forward(
            big, [list(long_prompt[:200])] * 3, [0, 0, 0])
    assert e.value.status == -6 and "pool exhausted" in str(e.value)
    assert model.free_pages == free and all(len(c) == 0 and c.pages == 0 for c in big)
    for c in big + [a, b]:
        c.close()
    assert model.free_pages == pool
    model.close()


@pytest.mark.gpu
@pytest.mark.parametrize("batch_decode", [True, False])
def test_concurrent_generations_through_the_pool_match_the_oracle(backend, batch_decode):
    """Six requests over four slots, one thread each (generate::run): chunked prefill, decode through the window,
    release.  Every request's tokens equal the oracle's for its own prompt."""
    cfg, model, ref = _build(backend, "small", max_seq_len=256, max_batch_tokens=16, kv_pool_tokens=1024)
    pool = scheduler.SlotPool(model, n_slots=4, slot_capacity_tokens=128, batch_wait_ms=20, prefill_batch=16, batch_decode=batch_decode)
    rng = np.random.default_rng(5)
    prompts = [rng.integers(0, cfg["n_vocab"], n).astype(np.uint32) for n in (40, 9, 23, 33, 17, 5)]
    n_new = 12
    results, errors = [None] * len(prompts), []

    def run(i):
        try:
            with pool.try_acquire() as slot:
                out = [slot.prefill(prompts[i])]
                while len(out) < n_new:
                    out.append(slot.decode(out[-1]))
                assert len(slot) == len(prompts[i]) + n_new - 1
                results[i] = out
        except Exception as e:  # noqa: BLE001
            errors.append((i, repr(e)))

    threads = [threading.Thread(target=run, args=(i,)) for i in range(len(prompts))]
    for t in threads:
        t.start()
    for t in threads:
        t.join(120)
    assert not errors, errors
    for i, p in enumerate(prompts):
        assert results[i] == _oracle_run(ref, p, n_new), f"request {i}"
    st = pool.stats()
    assert st["busy"] == 0 and st["queued"] == 0 and st["free_pages"] == model.pool_pages
    assert st["batched_seqs"] == len(prompts) * (n_new - 1)
    if batch_decode:
        assert st["batches"] < st["batched_seqs"], "no two steps ever shared a batch"
    else:
        assert st["batches"] == st["batched_seqs"]
    assert [s["busy"] for s in pool.snapshot()] == [0, 0, 0, 0]
    pool.close()
    model.close()


@pytest.mark.gpu
def test_pool_refuses_when_full_pins_slots_and_survives_an_empty_kv_pool(backend):
    cfg, model, ref = _build(backend, "tiny", max_seq_len=256, max_batch_tokens=16, kv_pool_tokens=64)  # 5 pages
    pool = scheduler.SlotPool(model, n_slots=2, slot_capacity_tokens=128, max_queue=1, batch_wait_ms=1)
    a, b = pool.try_acquire(0), pool.try_acquire(0)
    assert {a.id(), b.id()} == {0, 1}
    assert pool.try_acquire(0) is None and pool.try_acquire(30) is None  # both busy: refused, then timed out
    assert pool.stats()["refused"] == 2 and pool.stats()["queued"] == 0
    assert pool.acquire_slot(a.id(), 10) is None  # pinned to a busy slot
    toks = np.arange(48, dtype=np.uint32) % cfg["n_vocab"]
    t_a = a.prefill(toks)  # three pages
    assert pool.snapshot()[a.id()]["prompt_tokens"] == 48
    from orangu_b200 import OranguError

    with pytest.raises(OranguError) as e:
        b.prefill(toks)  # needs three, two are left
    assert e.value.status == -6 and len(b) <= 32
    nxt = a.decode(t_a)
    assert [t_a, nxt] == _oracle_run(ref, toks, 2)
    a.truncate(20)
    assert len(a) == 20 and pool.stats()["free_pages"] >= model.pool_pages - 2 - (len(b) + 15) // 16
    idx = a.id()
    a.release()
    again = pool.acquire_slot(idx, 0)
    assert again is not None and len(again) == 0
    again.release()
    b.release()
    assert pool.stats()["free_pages"] == model.pool_pages
    pool.close()
    model.close()
