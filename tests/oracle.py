"""ctypes binding of the CPU oracle (oracle/orangu_oracle.cpp) -- test infrastructure.

Only tests, the smoke check and the benchmark's CPU-baseline leg import this.
The product package never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB_PATH = os.path.join(ROOT, "oracle", "_build", "liborangu_oracle.so")

F32, Q8_0, Q4_K, Q6_K = 0, 8, 12, 14
Q5_K = 13
Q4_0, Q5_0, IQ4_NL = 2, 6, 20   # per-32 symmetric types: one f16 scale and 32 signed codes per block, like Q8_0
PER_32 = (Q8_0, Q4_0, Q5_0, IQ4_NL)
BLOCK = {Q8_0: (34, 32), Q4_K: (144, 256), Q6_K: (210, 256), F32: (4, 1), Q4_0: (18, 32), Q5_0: (22, 32), IQ4_NL: (18, 32), Q5_K: (176, 256)}


def build(force: bool = False) -> str:
    src = os.path.join(ROOT, "oracle", "orangu_oracle.cpp")
    hdr = os.path.join(ROOT, "oracle", "orangu_oracle.h")
    stale = not os.path.exists(LIB_PATH)
    if not stale and os.path.exists(src):
        stale = os.path.getmtime(LIB_PATH) < max(os.path.getmtime(src), os.path.getmtime(hdr))
    if force or stale:
        subprocess.run(["make", "-C", os.path.join(ROOT, "oracle")], check=True, capture_output=True)
    return LIB_PATH


class Matrix(C.Structure):
    _fields_ = [("data", C.c_void_p), ("type", C.c_uint32), ("in_dim", C.c_uint32), ("out_dim", C.c_uint32)]


class Layer(C.Structure):
    _fields_ = [("attn_norm", C.c_void_p), ("ffn_norm", C.c_void_p)] + [
        (n, Matrix) for n in ("wq", "wk", "wv", "wo", "w_gate", "w_up", "w_down")
    ] + [(n, C.c_void_p) for n in ("q_bias", "k_bias", "v_bias", "q_norm", "k_norm")]


class Config(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("n_vocab", "n_embd", "n_layer", "n_head", "n_head_kv", "head_dim", "rope_dim", "n_ff")] + [
        ("rope_freq_base", C.c_float),
        ("rms_eps", C.c_float),
        ("rope_freqs", C.c_void_p),
        ("rope_neox", C.c_uint32),
    ]


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(LIB_PATH)
        vp, u32, u64, f32, i32 = C.c_void_p, C.c_uint32, C.c_size_t, C.c_float, C.c_int
        L.oref_f16_to_f32.restype = f32
        L.oref_f16_to_f32.argtypes = [C.c_uint16]
        L.oref_f32_to_f16.restype = C.c_uint16
        L.oref_f32_to_f16.argtypes = [f32]
        L.oref_row_bytes.restype = C.c_int64
        L.oref_row_bytes.argtypes = [u32, C.c_uint64]
        L.oref_dequantize.argtypes = [u32, vp, u64, vp]
        L.oref_get_scale_min_k4.argtypes = [i32, vp, vp, vp]
        L.oref_quantize_act.argtypes = [vp, u64, vp, vp, vp]
        L.oref_quantize_act_k_row.argtypes = [vp, u64, vp, vp, vp]
        L.oref_dot_row32.restype = f32
        L.oref_dot_row32.argtypes = [C.c_uint32, vp, u64, vp, vp]
        L.oref_dot_q8_0.restype = f32
        L.oref_dot_q8_0.argtypes = [vp, u64, vp, vp]
        L.oref_dot_k_row.restype = f32
        L.oref_dot_k_row.argtypes = [u32, vp, u64, vp, vp, vp]
        L.oref_row_partials.argtypes = [u32, vp, u64, vp, vp, vp]
        for name in ("oref_matmul", "oref_matmul_decode", "oref_matmul_dequant"):
            getattr(L, name).argtypes = [vp, u64, vp, u32, u64, u64, vp, i32]
        L.oref_dot.restype = f32
        L.oref_dot.argtypes = [vp, vp, u64]
        L.oref_rmsnorm.argtypes = [vp, vp, vp, u64, u64, f32]
        L.oref_rope_norm.argtypes = [vp, u64, u64, u64, u64, f32]
        L.oref_rope_table.argtypes = [vp, u64, u64, f32]
        L.oref_rope_layout.argtypes = [vp, u64, u64, u64, u64, f32, vp, C.c_int]
        L.oref_rope_layout.restype = None
        L.oref_softmax.argtypes = [vp, u64]
        L.oref_silu.restype = f32
        L.oref_silu.argtypes = [f32]
        L.oref_swiglu.argtypes = [vp, vp, u64]
        L.oref_add.argtypes = [vp, vp, u64]
        L.oref_attention.argtypes = [vp, vp, vp, vp, u64, u64, u64, u64, f32, u64, u64, i32]
        L.oref_argmax.restype = u32
        L.oref_argmax.argtypes = [vp, u64]
        L.oref_repeat_penalty.argtypes = [vp, u64, vp, u64, u64, f32]
        L.oref_model_create.restype = vp
        L.oref_model_create.argtypes = [vp, vp, vp, vp, vp]
        L.oref_model_destroy.argtypes = [vp]
        L.oref_kv_create.restype = vp
        L.oref_kv_create.argtypes = [vp, u64, i32]
        L.oref_kv_destroy.argtypes = [vp]
        L.oref_kv_len.restype = u64
        L.oref_kv_len.argtypes = [vp]
        L.oref_kv_truncate.argtypes = [vp, u64]
        L.oref_forward.argtypes = [vp, vp, vp, u64, u64, vp, vp, i32]
        L.oref_hardware_threads.restype = i32
        _lib = L
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _u8(a):
    return np.ascontiguousarray(a, dtype=np.uint8)


def row_bytes(t, in_dim):
    r = lib().oref_row_bytes(t, in_dim)
    if r < 0:
        raise ValueError(f"type {t} in_dim {in_dim}")
    return int(r)


def dequantize(t, raw, n):
    raw = _u8(raw)
    out = np.empty(n, np.float32)
    if lib().oref_dequantize(t, _p(raw), n, _p(out)):
        raise ValueError(f"unsupported type {t}")
    return out


def quantize_act(x, k_row=False):
    x = _f32(x)
    n = x.size
    q = np.empty(n, np.int8)
    d = np.empty(n // (256 if k_row else 32), np.float32)
    sums = np.empty(n // 16, np.int32)
    (lib().oref_quantize_act_k_row if k_row else lib().oref_quantize_act)(_p(x), n, _p(q), _p(d), _p(sums))
    return q, d, sums


def dot_row(t, row, x):
    """The GEMV of the type's family for one row and one fp32 activation vector."""
    row, x = _u8(row), _f32(x)
    if t == Q8_0:
        q, d, _ = quantize_act(x)
        return float(lib().oref_dot_q8_0(_p(row), x.size, _p(q), _p(d)))
    if t in PER_32:
        q, d, _ = quantize_act(x)
        return float(lib().oref_dot_row32(t, _p(row), x.size, _p(q), _p(d)))
    q, d, s = quantize_act(x, True)
    return float(lib().oref_dot_k_row(t, _p(row), x.size, _p(q), _p(d), _p(s)))


def row_partials(t, row, x):
    row, x = _u8(row), _f32(x)
    nb = x.size // BLOCK[t][1]
    isum, imin = np.zeros(nb, np.int32), np.zeros(nb, np.int32)
    if lib().oref_row_partials(t, _p(row), x.size, _p(x), _p(isum), _p(imin)):
        raise ValueError("unsupported")
    return isum, imin


def _mm(fn, x, n_tokens, raw, t, in_dim, out_dim, threads):
    x, raw = _f32(x), _u8(raw)
    assert x.size == n_tokens * in_dim and raw.size == out_dim * row_bytes(t, in_dim)
    y = np.empty((n_tokens, out_dim), np.float32)
    if fn(_p(x), n_tokens, _p(raw), t, in_dim, out_dim, _p(y), threads):
        raise ValueError("unsupported matmul")
    return y


def matmul(x, n_tokens, raw, t, in_dim, out_dim, threads=0):
    return _mm(lib().oref_matmul, x, n_tokens, raw, t, in_dim, out_dim, threads)


def matmul_decode(x, n_tokens, raw, t, in_dim, out_dim, threads=0):
    return _mm(lib().oref_matmul_decode, x, n_tokens, raw, t, in_dim, out_dim, threads)


def matmul_dequant(x, n_tokens, raw, t, in_dim, out_dim, threads=0):
    return _mm(lib().oref_matmul_dequant, x, n_tokens, raw, t, in_dim, out_dim, threads)


def rmsnorm(x, w, eps):
    x, w = _f32(x), _f32(w)
    x2 = x.reshape(-1, w.size)
    out = np.empty_like(x2)
    lib().oref_rmsnorm(_p(out), _p(x2), _p(w), x2.shape[0], w.size, eps)
    return out.reshape(x.shape)


def rope_layout(x, n_head, head_dim, pos, rope_dim, base, neox, freq_factors=None):
    """tensor.rs:1115-1177 with either pairing; returns a rotated copy."""
    x = np.array(x, dtype=np.float32, copy=True)
    ff = np.ascontiguousarray(freq_factors, np.float32) if freq_factors is not None else None
    lib().oref_rope_layout(_p(x), n_head, head_dim, pos, rope_dim, base, _p(ff) if ff is not None else None, 1 if neox else 0)
    return x


def rope_norm(x, n_head, head_dim, pos, rope_dim, base):
    x = _f32(x).copy()
    lib().oref_rope_norm(_p(x), n_head, head_dim, pos, rope_dim, base)
    return x


def rope_table(n_pos, rope_dim, base):
    t = np.empty((n_pos, rope_dim // 2, 2), np.float32)
    lib().oref_rope_table(_p(t), n_pos, rope_dim, base)
    return t


def softmax(x):
    x = _f32(x).copy()
    lib().oref_softmax(_p(x), x.size)
    return x


def swiglu(gate, up):
    g, u = _f32(gate).copy(), _f32(up)
    lib().oref_swiglu(_p(g), _p(u), g.size)
    return g


def attention(q, k, v, n_head, n_head_kv, head_dim, scale, n_tokens, start_pos, threads=0):
    q, k, v = _f32(q), _f32(k), _f32(v)
    out = np.empty(n_tokens * n_head * head_dim, np.float32)
    group = -(-n_head // n_head_kv)
    lib().oref_attention(_p(out), _p(q), _p(k), _p(v), n_head_kv * head_dim, n_head, group, head_dim, scale, n_tokens, start_pos, threads)
    return out.reshape(n_tokens, n_head * head_dim)


def argmax(logits):
    l = _f32(logits)
    return int(lib().oref_argmax(_p(l), l.size))


def repeat_penalty(logits, recent, last_n, penalty):
    l = _f32(logits).copy()
    r = np.ascontiguousarray(recent, dtype=np.uint32)
    lib().oref_repeat_penalty(_p(l), l.size, _p(r), r.size, last_n, penalty)
    return l


def f32_to_f16_bits(v):
    return int(lib().oref_f32_to_f16(float(np.float32(v))))


def hardware_threads():
    return int(lib().oref_hardware_threads())


class Model:
    """Oracle Llama model over a dict of named tensors (see orangu_b200.synth)."""

    def __init__(self, cfg: dict, tensors: dict):
        L = lib()
        self._keep = tensors
        self.cfg = cfg
        c = Config(cfg["n_vocab"], cfg["n_embd"], cfg["n_layer"], cfg["n_head"], cfg["n_head_kv"], cfg["head_dim"],
                   cfg.get("rope_dim", cfg["head_dim"]), cfg["n_ff"], cfg["rope_freq_base"], cfg["rms_eps"],
                   tensors["rope_freqs.weight"]["data"].ctypes.data if "rope_freqs.weight" in tensors else None,
                   1 if cfg.get("rope_neox") else 0)

        def mat(name):
            t = tensors[name]
            return Matrix(t["data"].ctypes.data, t["type"], t["in_dim"], t["out_dim"])

        layers = (Layer * cfg["n_layer"])()
        for i in range(cfg["n_layer"]):
            l = layers[i]
            l.attn_norm = tensors[f"blk.{i}.attn_norm.weight"]["data"].ctypes.data
            l.ffn_norm = tensors[f"blk.{i}.ffn_norm.weight"]["data"].ctypes.data
            for field, suffix in (("wq", "attn_q"), ("wk", "attn_k"), ("wv", "attn_v"), ("wo", "attn_output"),
                                  ("w_gate", "ffn_gate"), ("w_up", "ffn_up"), ("w_down", "ffn_down")):
                setattr(l, field, mat(f"blk.{i}.{suffix}.weight"))
            for field, name in (("q_bias", "attn_q.bias"), ("k_bias", "attn_k.bias"), ("v_bias", "attn_v.bias"),
                                ("q_norm", "attn_q_norm.weight"), ("k_norm", "attn_k_norm.weight")):
                if f"blk.{i}.{name}" in tensors:
                    setattr(l, field, tensors[f"blk.{i}.{name}"]["data"].ctypes.data)
        emb = mat("token_embd.weight")
        out = mat("output.weight") if "output.weight" in tensors else None
        self._h = L.oref_model_create(C.byref(c), C.byref(emb), tensors["output_norm.weight"]["data"].ctypes.data,
                                      C.byref(out) if out is not None else None, layers)

    def new_kv(self, capacity, f16=False):
        return KV(self, capacity, f16)

    def forward(self, kv, tokens, start_pos, want_hidden=False, threads=0):
        toks = np.ascontiguousarray(tokens, dtype=np.uint32)
        logits = np.empty(self.cfg["n_vocab"], np.float32)
        hidden = np.empty((toks.size, self.cfg["n_embd"]), np.float32) if want_hidden else None
        rc = lib().oref_forward(self._h, kv._h, _p(toks), toks.size, start_pos, _p(logits), _p(hidden) if want_hidden else None, threads)
        if rc:
            raise RuntimeError(f"oref_forward failed: {rc}")
        return (logits, hidden) if want_hidden else logits

    def __del__(self):
        if getattr(self, "_h", None):
            lib().oref_model_destroy(self._h)
            self._h = None


class KV:
    def __init__(self, model, capacity, f16):
        self._h = lib().oref_kv_create(model._h, capacity, 1 if f16 else 0)

    def __len__(self):
        return int(lib().oref_kv_len(self._h))

    def truncate(self, n):
        lib().oref_kv_truncate(self._h, n)

    def __del__(self):
        if getattr(self, "_h", None):
            lib().oref_kv_destroy(self._h)
            self._h = None
