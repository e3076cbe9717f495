"""Host-side mirror of the reference engine's ``Backend`` trait over the C ABI.

Names, argument meaning and error behaviour follow
src/bin/orangu-server/engine/backend/mod.rs:309-496 (trait Backend) and
src/bin/orangu-server/engine/loader.rs:561-680 (QuantMatrix) of the reference.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import capi

BLOCK = {8: (34, 32), 12: (144, 256), 13: (176, 256), 14: (210, 256), 2: (18, 32), 6: (22, 32), 20: (18, 32)}


def tensor_byte_size(ggml_type: int, n_elems: int) -> int:
    bb, be = BLOCK[ggml_type]
    if n_elems % be:
        raise ValueError(f"{n_elems} elements is not a whole number of {be}-element blocks")
    return n_elems // be * bb


class QuantMatrix:
    """A 2-D tensor kept in its GGUF block layout: ``out_dim`` rows of ``in_dim`` elements
    (loader.rs:561-680).  ``raw`` is the bytes exactly as the file stores them."""

    def __init__(self, raw, ggml_type: int, in_dim: int, out_dim: int):
        self.raw = np.ascontiguousarray(raw, dtype=np.uint8).reshape(-1)
        self.ggml_type_ = int(ggml_type)
        self.in_dim = int(in_dim)
        self.out_dim = int(out_dim)
        if self.ggml_type_ in BLOCK and self.raw.size != self.row_bytes() * self.out_dim:
            raise ValueError("raw size does not match type and shape")
        self._dev = {}  # backend id -> device handle (the reference caches by cache_key, cuda.rs:216-236)

    def ggml_type(self) -> int:
        return self.ggml_type_

    def row_bytes(self) -> int:
        return tensor_byte_size(self.ggml_type_, self.in_dim)

    def raw_bytes(self) -> np.ndarray:
        return self.raw

    def rows(self, first: int, count: int) -> "QuantMatrix":
        """Row-range view (loader.rs:627-646)."""
        rb = self.row_bytes()
        return QuantMatrix(self.raw[first * rb:(first + count) * rb], self.ggml_type_, self.in_dim, count)


@dataclass
class MatmulOp:  # backend/mod.rs:117-121
    x: np.ndarray
    n_tokens: int
    w: QuantMatrix


class CudaBackend:
    """``impl Backend`` over liborangu_b200.  Construct with :meth:`try_init_index`, which returns
    ``None`` on any failure as the reference's does (backend/cuda.rs:86-124); later failures raise
    :class:`OranguError` where the reference panics."""

    def __init__(self, handle):
        self._h = handle
        self._lib = capi.load()
        self._weights = []

    @classmethod
    def try_init_index(cls, index: int = 0):
        try:
            L = capi.load()
        except (OSError, capi.OranguError, AttributeError):
            return None
        h = C.c_void_p()
        if L.ob_init(index, C.byref(h)) != 0:
            return None
        return cls(h)

    @classmethod
    def init(cls, index: int = 0) -> "CudaBackend":
        """Like try_init_index, but says why it failed."""
        L = capi.load()
        h = C.c_void_p()
        capi.check(None, L.ob_init(index, C.byref(h)))
        return cls(h)

    def close(self):
        if self._h:
            for w in self._weights:
                self._lib.ob_weight_release(self._h, w)
            self._weights.clear()
            self._lib.ob_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- Backend -----------------------------------------------------------------------------
    def supports_type(self, ggml_type: int) -> bool:
        return bool(self._lib.ob_supports_type(ggml_type))

    def reduced_surface(self):
        s = self._lib.ob_reduced_surface()
        return s.decode() if s else None

    def _weight(self, w: QuantMatrix):
        h = w._dev.get(id(self))
        if h is None:
            h = C.c_void_p()
            capi.check(self._h, self._lib.ob_weight_register(self._h, w.raw.ctypes.data, w.row_bytes(), w.ggml_type_, w.in_dim, w.out_dim, C.byref(h)))
            w._dev[id(self)] = h
            self._weights.append(h)
        return h

    def _x(self, x, n_tokens, w):
        x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
        if x.size != n_tokens * w.in_dim:
            raise ValueError("x.len() != n_tokens * w.in_dim")
        return x

    def matmul(self, x, n_tokens: int, w: QuantMatrix) -> np.ndarray:
        x = self._x(x, n_tokens, w)
        y = np.empty((n_tokens, w.out_dim), np.float32)
        capi.check(self._h, self._lib.ob_matmul(self._h, x.ctypes.data, n_tokens, self._weight(w), y.ctypes.data))
        return y

    def matmul_into(self, out: np.ndarray, x, n_tokens: int, w: QuantMatrix) -> None:
        out[...] = self.matmul(x, n_tokens, w).reshape(out.shape)

    def matmul_decode(self, x, n_tokens: int, w: QuantMatrix) -> np.ndarray:
        x = self._x(x, n_tokens, w)
        y = np.empty((n_tokens, w.out_dim), np.float32)
        capi.check(self._h, self._lib.ob_matmul_decode(self._h, x.ctypes.data, n_tokens, self._weight(w), y.ctypes.data))
        return y

    def matmul_decode_into(self, out: np.ndarray, x, n_tokens: int, w: QuantMatrix) -> None:
        out[...] = self.matmul_decode(x, n_tokens, w).reshape(out.shape)

    def _batch(self, ops, decode: bool):
        xs = [self._x(op.x, op.n_tokens, op.w) for op in ops]
        ys = [np.empty((op.n_tokens, op.w.out_dim), np.float32) for op in ops]
        arr = (capi.MatmulOpC * len(ops))()
        for i, op in enumerate(ops):
            arr[i].x = xs[i].ctypes.data
            arr[i].n_tokens = op.n_tokens
            arr[i].w = self._weight(op.w)
            arr[i].y = ys[i].ctypes.data
        capi.check(self._h, self._lib.ob_matmul_batch(self._h, arr, len(ops), 1 if decode else 0))
        return ys

    def matmul_batch(self, ops) -> list:
        return self._batch(list(ops), False)

    def matmul_batch_into(self, outs: list, ops) -> None:
        outs[:] = self.matmul_batch(ops)

    def matmul_batch_decode(self, ops) -> list:
        return self._batch(list(ops), True)

    # ---- beyond the trait ----------------------------------------------------------------------
    def row(self, w: QuantMatrix, index: int, count: int = 1) -> np.ndarray:
        """QuantMatrix::row on the device (loader.rs:585-590)."""
        out = np.empty((count, w.in_dim), np.float32)
        capi.check(self._h, self._lib.ob_weight_dequantize(self._h, self._weight(w), index, count, out.ctypes.data))
        return out

    def matmul_partials(self, x, w: QuantMatrix, first_row: int = 0, n_rows: int | None = None):
        n_rows = w.out_dim - first_row if n_rows is None else n_rows
        x = self._x(x, 1, w)
        nb = w.in_dim // BLOCK[w.ggml_type_][1]
        isum = np.empty((n_rows, nb), np.int32)
        imin = np.empty((n_rows, nb), np.int32)
        capi.check(self._h, self._lib.ob_matmul_partials(self._h, x.ctypes.data, self._weight(w), first_row, n_rows, isum.ctypes.data, imin.ctypes.data))
        return isum, imin

    def rmsnorm(self, x, weight, eps: float) -> np.ndarray:
        weight = np.ascontiguousarray(weight, np.float32)
        x = np.ascontiguousarray(x, np.float32)
        out = np.empty_like(x)
        capi.check(self._h, self._lib.ob_rmsnorm(self._h, x.ctypes.data, weight.ctypes.data, x.size // weight.size, weight.size, eps, out.ctypes.data))
        return out

    def rope(self, x, n_head: int, head_dim: int, pos: int, rope_dim: int, freq_base: float) -> np.ndarray:
        x = np.ascontiguousarray(x, np.float32).copy()
        capi.check(self._h, self._lib.ob_rope(self._h, x.ctypes.data, n_head, head_dim, pos, rope_dim, freq_base))
        return x

    def swiglu(self, gate, up) -> np.ndarray:
        gate, up = np.ascontiguousarray(gate, np.float32), np.ascontiguousarray(up, np.float32)
        out = np.empty_like(gate)
        capi.check(self._h, self._lib.ob_swiglu(self._h, gate.ctypes.data, up.ctypes.data, gate.size, out.ctypes.data))
        return out

    def quantize_act(self, x, per_256: bool):
        x = np.ascontiguousarray(x, np.float32).reshape(-1)
        q = np.empty(x.size, np.int8)
        d = np.empty(x.size // (256 if per_256 else 32), np.float32)
        sums = np.empty(x.size // 16, np.int32)
        capi.check(self._h, self._lib.ob_quantize_act(self._h, x.ctypes.data, x.size, 1 if per_256 else 0, q.ctypes.data, d.ctypes.data, sums.ctypes.data))
        return q, d, sums

    def attention_decode(self, q, k, v, n_head: int, n_head_kv: int, head_dim: int, scale: float, exact_order: bool | int = True) -> np.ndarray:
        q = np.ascontiguousarray(q, np.float32).reshape(-1)
        k = np.ascontiguousarray(k, np.float32).reshape(-1, n_head_kv * head_dim)
        v = np.ascontiguousarray(v, np.float32).reshape(-1, n_head_kv * head_dim)
        out = np.empty(n_head * head_dim, np.float32)
        capi.check(self._h, self._lib.ob_attention_decode(self._h, q.ctypes.data, k.ctypes.data, v.ctypes.data, k.shape[0], n_head, n_head_kv, head_dim, scale, int(exact_order), out.ctypes.data))
        return out

    def argmax(self, logits, recent=None, repeat_last_n: int = 64, penalty: float = 1.0) -> int:
        logits = np.ascontiguousarray(logits, np.float32).reshape(-1)
        out = C.c_uint32()
        if recent is not None and len(recent):
            r = np.ascontiguousarray(recent, np.uint32)
            capi.check(self._h, self._lib.ob_argmax(self._h, logits.ctypes.data, logits.size, r.ctypes.data, r.size, repeat_last_n, penalty, C.byref(out)))
        else:
            capi.check(self._h, self._lib.ob_argmax(self._h, logits.ctypes.data, logits.size, None, 0, repeat_last_n, penalty, C.byref(out)))
        return int(out.value)

    def launch_count(self) -> int:
        return int(self._lib.ob_launch_count(self._h))

    def last_device_ms(self) -> float:
        return float(self._lib.ob_last_device_ms(self._h))

    def synchronize(self):
        capi.check(self._h, self._lib.ob_synchronize(self._h))
