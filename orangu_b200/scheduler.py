"""Host-side mirror of the reference's ``SlotPool`` (src/bin/orangu-server/engine/scheduler.rs:36-317) and
``BatchCoordinator`` (engine/batch.rs:184-324) over the C ABI's ob_slot_* entry points.  The logic lives in the library;
this only marshals arguments, so that the tests read like the reference's own."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import capi


class SlotPoolDesc(C.Structure):
    _fields_ = [("n_slots", C.c_uint32), ("slot_capacity_tokens", C.c_uint32), ("max_queue", C.c_uint32),
                ("batch_wait_ms", C.c_uint32), ("prefill_batch", C.c_uint32), ("batch_decode", C.c_uint32)]


class SlotState(C.Structure):
    _fields_ = [("id", C.c_uint32), ("busy", C.c_uint32), ("prompt_tokens", C.c_uint32), ("generated_tokens", C.c_uint32)]


class SlotPoolStats(C.Structure):
    _fields_ = [("batches", C.c_uint64), ("batched_seqs", C.c_uint64), ("refused", C.c_uint64),
                ("total", C.c_uint32), ("busy", C.c_uint32), ("queued", C.c_uint32), ("free_pages", C.c_uint32)]

    def as_dict(self):
        return {k: int(getattr(self, k)) for k, _ in self._fields_}


def selftest(n_slots: int, n_threads: int, n_steps: int, batch_wait_ms: int = 4, max_queue: int = 0):
    """(status, stats) of the library's host-only run of the pool and the window against a stand-in forward pass."""
    st = SlotPoolStats()
    rc = capi.load().ob_slot_pool_selftest(n_slots, n_threads, n_steps, batch_wait_ms, max_queue, C.byref(st))
    return rc, st.as_dict()


class SlotGuard:
    """A held slot (SlotGuard, scheduler.rs:319-356); releasing it empties the slot's cache and wakes the next waiter."""

    def __init__(self, pool: "SlotPool", index: int):
        self.pool, self.index = pool, index

    def id(self) -> int:
        return self.index

    def __len__(self):
        return int(self.pool._lib.ob_slot_len(self.pool._h, self.index))

    def prefill(self, tokens, want_logits: bool = False):
        """generate::prefill (generate.rs:1276-1338): the greedy token after the prompt (and its logits)."""
        t = np.ascontiguousarray(tokens, np.uint32)
        out = C.c_uint32()
        logits = np.empty(self.pool.model.n_vocab, np.float32) if want_logits else None
        self.pool._check(self.index, self.pool._lib.ob_slot_prefill(self.pool._h, self.index, t.ctypes.data, t.size, C.byref(out),
                                                                    logits.ctypes.data if want_logits else None))
        return (int(out.value), logits) if want_logits else int(out.value)

    def decode(self, token: int, recent=None, repeat_penalty: float = 1.0, repeat_last_n: int = 64, want_logits: bool = False):
        """BatchCoordinator::submit (batch.rs:207-270): blocks until the batch this step joined has run."""
        out = C.c_uint32()
        logits = np.empty(self.pool.model.n_vocab, np.float32) if want_logits else None
        gptr = None
        if recent is not None and repeat_penalty != 1.0:
            rec = np.ascontiguousarray(recent, np.uint32)
            nrec = np.asarray([rec.size], np.uint32)
            gs = capi.Greedy(repeat_penalty, repeat_last_n, rec.ctypes.data, nrec.ctypes.data)
            gptr = C.addressof(gs)
        self.pool._check(self.index, self.pool._lib.ob_slot_decode(self.pool._h, self.index, int(token), gptr, C.byref(out),
                                                                   logits.ctypes.data if want_logits else None))
        return (int(out.value), logits) if want_logits else int(out.value)

    def truncate(self, new_len: int):
        self.pool._check(self.index, self.pool._lib.ob_slot_truncate(self.pool._h, self.index, new_len))

    def release(self):
        if self.index is not None:
            self.pool._check(self.index, self.pool._lib.ob_slot_release(self.pool._h, self.index))
            self.index = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.release()


class SlotPool:
    def __init__(self, model, n_slots: int, slot_capacity_tokens: int, max_queue: int = 0, batch_wait_ms: int = 0, prefill_batch: int = 0,
                 batch_decode: bool = True):
        self.model, self._lib = model, (model._lib if model is not None else capi.load())
        d = SlotPoolDesc(n_slots, slot_capacity_tokens, max_queue, batch_wait_ms, prefill_batch, 1 if batch_decode else 0)
        self._h = C.c_void_p()
        # model None: a pool that schedules only, its decode answered by the library's host-side stand-in (tests without a device)
        rc = self._lib.ob_slot_pool_create(model._h if model is not None else None, C.byref(d), C.byref(self._h))
        if rc:
            raise capi.OranguError(rc, (self._lib.ob_slot_last_error(None, -1) or b"").decode())

    def _check(self, slot, rc):
        if rc:
            raise capi.OranguError(rc, (self._lib.ob_slot_last_error(self._h, -1 if slot is None else slot) or b"").decode())

    def try_acquire(self, timeout_ms: int = -1):
        """SlotPool::try_acquire: a SlotGuard, or None when the pool refuses (queue full / time ran out)."""
        out = C.c_uint32()
        rc = self._lib.ob_slot_acquire(self._h, timeout_ms, C.byref(out))
        if rc == -6:
            return None
        self._check(None, rc)
        return SlotGuard(self, int(out.value))

    def acquire_slot(self, index: int, timeout_ms: int = -1):
        rc = self._lib.ob_slot_acquire_id(self._h, index, timeout_ms)
        if rc == -6:
            return None
        self._check(None, rc)
        return SlotGuard(self, index)

    def snapshot(self):
        n = int(self._lib.ob_slot_pool_snapshot(self._h, None, 0))
        arr = (SlotState * n)()
        self._lib.ob_slot_pool_snapshot(self._h, arr, n)
        return [{k: int(getattr(s, k)) for k, _ in SlotState._fields_} for s in arr]

    def stats(self) -> dict:
        st = SlotPoolStats()
        self._check(None, self._lib.ob_slot_pool_get_stats(self._h, C.byref(st)))
        return st.as_dict()

    def busy_count(self) -> int:
        return self.stats()["busy"]

    def close(self):
        if self._h:
            self._lib.ob_slot_pool_destroy(self._h)
            self._h = None
