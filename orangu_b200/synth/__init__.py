"""Seeded synthetic weights in GGUF block layouts (stand-ins for checkpoints that cannot be fetched here)."""
from __future__ import annotations

import ctypes as C
import os
import zlib

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(os.path.dirname(HERE), "_lib", "libob_synth.so")
F32, Q8_0, Q4_K, Q6_K = 0, 8, 12, 14
Q4_0, Q5_0, IQ4_NL = 2, 6, 20
Q5_K = 13
BLOCK = {Q8_0: (34, 32), Q4_K: (144, 256), Q5_K: (176, 256), Q6_K: (210, 256), Q4_0: (18, 32), Q5_0: (22, 32), IQ4_NL: (18, 32)}
# standard deviation of a uniformly random code of the per-32 symmetric types (sets the block scale for a wanted std)
_CODE_STD = {Q4_0: 4.61, Q5_0: 9.23, IQ4_NL: 70.2}

_lib = None


def _load():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            from .. import build
            build.build_synth()
        L = C.CDLL(_LIB_PATH)
        L.obs_fill_normal.argtypes = [C.c_void_p, C.c_size_t, C.c_uint64, C.c_float]
        L.obs_quantize_rows.argtypes = [C.c_uint32, C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p]
        L.obs_synth_matrix.argtypes = [C.c_uint32, C.c_uint64, C.c_float, C.c_size_t, C.c_size_t, C.c_void_p]
        L.obs_synth_matrix_slice.argtypes = [C.c_uint32, C.c_uint64, C.c_float, C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t, C.c_void_p]
        _lib = L
    return _lib


def seed_of(*parts) -> int:
    return zlib.crc32("/".join(str(p) for p in parts).encode()) | (zlib.adler32(repr(parts).encode()) << 32)


def normal(n: int, seed: int, std: float = 1.0) -> np.ndarray:
    out = np.empty(n, np.float32)
    _load().obs_fill_normal(out.ctypes.data, n, seed, std)
    return out


def quantize(w: np.ndarray, ggml_type: int) -> np.ndarray:
    """Quantize a [rows, in_dim] fp32 matrix into GGUF blocks of `ggml_type`."""
    w = np.ascontiguousarray(w, np.float32)
    rows, in_dim = w.shape
    bb, be = BLOCK[ggml_type]
    out = np.empty(rows * (in_dim // be) * bb, np.uint8)
    if _load().obs_quantize_rows(ggml_type, w.ctypes.data, rows, in_dim, out.ctypes.data):
        raise ValueError("in_dim is not a whole number of blocks")
    return out


def matrix(ggml_type: int, out_dim: int, in_dim: int, seed: int, std: float = 0.02) -> dict:
    """[out_dim, in_dim] ~ N(0, std^2), quantized; the fp32 matrix is never materialised."""
    bb, be = BLOCK[ggml_type]
    if ggml_type == Q5_K:
        # uniformly random scale, min and code bits; d spread over [0.5, 1.5] x the value that gives the wanted std, and
        # dmin = 15.5 d so that the values centre on zero (value = d * sc * code - dmin * m, code 0..31)
        if in_dim % be:
            raise ValueError("in_dim is not a whole number of blocks")
        rng = np.random.default_rng(seed & 0xFFFFFFFFFFFF)
        blocks = rng.integers(0, 256, (out_dim * (in_dim // be), bb), dtype=np.uint8)
        d = (std / (36.0 * 9.23) * rng.uniform(0.5, 1.5, blocks.shape[0])).astype(np.float16)
        blocks[:, 0:2] = d.view(np.uint8).reshape(-1, 2)
        blocks[:, 2:4] = (d.astype(np.float32) * np.float32(15.5)).astype(np.float16).view(np.uint8).reshape(-1, 2)
        return {"data": blocks.reshape(-1), "type": ggml_type, "in_dim": in_dim, "out_dim": out_dim}
    if ggml_type in _CODE_STD:
        # uniformly random codes; block scales spread over [0.5, 1.5] x the value that gives the wanted std
        if in_dim % be:
            raise ValueError("in_dim is not a whole number of blocks")
        rng = np.random.default_rng(seed & 0xFFFFFFFFFFFF)
        blocks = rng.integers(0, 256, (out_dim * (in_dim // be), bb), dtype=np.uint8)
        d = (std / _CODE_STD[ggml_type] * rng.uniform(0.5, 1.5, blocks.shape[0])).astype(np.float16)
        blocks[:, 0:2] = d.view(np.uint8).reshape(-1, 2)
        return {"data": blocks.reshape(-1), "type": ggml_type, "in_dim": in_dim, "out_dim": out_dim}
    out = np.empty(out_dim * (in_dim // be) * bb, np.uint8)
    if _load().obs_synth_matrix(ggml_type, seed, std, out_dim, in_dim, out.ctypes.data):
        raise ValueError("in_dim is not a whole number of blocks")
    return {"data": out, "type": ggml_type, "in_dim": in_dim, "out_dim": out_dim}


def matrix_slice(ggml_type: int, out_dim: int, in_dim: int, seed: int, rows: tuple[int, int], cols: tuple[int, int], std: float = 0.02) -> dict:
    """Rows [rows[0], rows[0] + rows[1]) x columns [cols[0], cols[0] + cols[1]) of matrix(ggml_type, out_dim, in_dim, seed), made
    directly (bit-identical to cutting them out of the whole matrix); column bounds are whole blocks."""
    bb, be = BLOCK[ggml_type]
    if ggml_type in _CODE_STD:
        raise ValueError("slices are made for the generator-backed types only")
    (r0, nr), (c0, nc) = rows, cols
    if r0 + nr > out_dim or c0 % be or nc % be or c0 + nc > in_dim:
        raise ValueError("slice outside the matrix or not on block boundaries")
    out = np.empty(nr * (nc // be) * bb, np.uint8)
    if _load().obs_synth_matrix_slice(ggml_type, seed, std, in_dim, r0, nr, c0, nc, out.ctypes.data):
        raise ValueError("bad slice")
    return {"data": out, "type": ggml_type, "in_dim": nc, "out_dim": nr}


CONFIGS = {
    # Llama-style shapes; weights N(0, 0.02^2), norm weights all ones
    "tiny": dict(n_vocab=512, n_embd=256, n_layer=2, n_head=4, n_head_kv=2, head_dim=64, n_ff=512, rope_freq_base=10000.0, rms_eps=1e-5),
    "small": dict(n_vocab=2048, n_embd=512, n_layer=3, n_head=8, n_head_kv=2, head_dim=64, n_ff=1536, rope_freq_base=500000.0, rms_eps=1e-5),
    "1b": dict(n_vocab=128256, n_embd=2048, n_layer=16, n_head=32, n_head_kv=8, head_dim=64, n_ff=8192, rope_freq_base=500000.0, rms_eps=1e-5),
    "8b": dict(n_vocab=128256, n_embd=4096, n_layer=32, n_head=32, n_head_kv=8, head_dim=128, n_ff=14336, rope_freq_base=500000.0, rms_eps=1e-5),
    "70b": dict(n_vocab=128256, n_embd=8192, n_layer=80, n_head=64, n_head_kv=8, head_dim=128, n_ff=28672, rope_freq_base=500000.0, rms_eps=1e-5),
}


def _model_tensor_shards(cfg, seed, n_layer, types, rank, size):
    e, hd = cfg["n_embd"], cfg["head_dim"]
    qd, kvd, ff, V = cfg["n_head"] * hd, cfg["n_head_kv"] * hd, cfg["n_ff"], cfg["n_vocab"]
    t = {}

    def rows(name, key, default, out_dim, in_dim):  # split by output rows
        n = out_dim // size
        t[name] = matrix_slice(types.get(key, default), out_dim, in_dim, seed_of(seed, name), (rank * n, n), (0, in_dim))

    def cols(name, key, default, out_dim, in_dim):  # split by the contraction dimension
        n = in_dim // size
        t[name] = matrix_slice(types.get(key, default), out_dim, in_dim, seed_of(seed, name), (0, out_dim), (rank * n, n))

    t["token_embd.weight"] = matrix(types.get("token_embd", Q4_K), V, e, seed_of(seed, "token_embd.weight"))
    rows("output.weight", "output", Q6_K, V, e)
    t["output_norm.weight"] = {"data": np.ones(e, np.float32), "type": F32}
    for i in range(n_layer):
        p = f"blk.{i}."
        t[p + "attn_norm.weight"] = {"data": np.ones(e, np.float32), "type": F32}
        t[p + "ffn_norm.weight"] = {"data": np.ones(e, np.float32), "type": F32}
        rows(p + "attn_q.weight", "attn_q", Q4_K, qd, e)
        rows(p + "attn_k.weight", "attn_k", Q4_K, kvd, e)
        rows(p + "attn_v.weight", "attn_v", Q6_K, kvd, e)
        cols(p + "attn_output.weight", "attn_output", Q4_K, e, qd)
        rows(p + "ffn_gate.weight", "ffn_gate", Q4_K, ff, e)
        rows(p + "ffn_up.weight", "ffn_up", Q4_K, ff, e)
        cols(p + "ffn_down.weight", "ffn_down", Q4_K, e, ff)
    return t


def model_tensors(cfg: dict, seed: int = 0, n_layer: int | None = None, types: dict | None = None, tp: tuple[int, int] | None = None) -> dict:
    """Q4_K_M-style model: Q4_K everywhere except attn_v and output in Q6_K; token_embd Q4_K; norms f32 ones.
    `types` overrides per tensor suffix, e.g. {"attn_q": Q8_0}.  tp = (rank, size): only that rank's tensor-parallel shards
    are made (rows of Q/K/V/gate/up/output, input columns of attn_output/ffn_down; token_embd whole) -- the same bytes the
    whole tensors hold there -- for LlamaModel(..., tp_presliced=True)."""
    types = types or {}
    if tp is not None and tp[1] > 1:
        return _model_tensor_shards(cfg, seed, cfg["n_layer"] if n_layer is None else n_layer, types, tp[0], tp[1])
    n_layer = cfg["n_layer"] if n_layer is None else n_layer
    e, hd = cfg["n_embd"], cfg["head_dim"]
    qd, kvd, ff, V = cfg["n_head"] * hd, cfg["n_head_kv"] * hd, cfg["n_ff"], cfg["n_vocab"]
    t = {}

    def mat(name, key, default, out_dim, in_dim):
        t[name] = matrix(types.get(key, default), out_dim, in_dim, seed_of(seed, name))

    mat("token_embd.weight", "token_embd", Q4_K, V, e)
    mat("output.weight", "output", Q6_K, V, e)
    t["output_norm.weight"] = {"data": np.ones(e, np.float32), "type": F32}
    for i in range(n_layer):
        p = f"blk.{i}."
        t[p + "attn_norm.weight"] = {"data": np.ones(e, np.float32), "type": F32}
        t[p + "ffn_norm.weight"] = {"data": np.ones(e, np.float32), "type": F32}
        mat(p + "attn_q.weight", "attn_q", Q4_K, qd, e)
        mat(p + "attn_k.weight", "attn_k", Q4_K, kvd, e)
        mat(p + "attn_v.weight", "attn_v", Q6_K, kvd, e)
        mat(p + "attn_output.weight", "attn_output", Q4_K, e, qd)
        mat(p + "ffn_gate.weight", "ffn_gate", Q4_K, ff, e)
        mat(p + "ffn_up.weight", "ffn_up", Q4_K, ff, e)
        mat(p + "ffn_down.weight", "ffn_down", Q4_K, e, ff)
    return t


def add_qwen_extras(cfg: dict, tensors: dict, seed: int = 0, bias: bool = True, qk_norm: bool = True) -> dict:
    """Adds the per-layer tensors Qwen2 (q/k/v bias) and Qwen3 (per-head q/k RMSNorm weights) files carry
    (engine/arch/llama.rs:45-60).  Biases N(0, 0.1^2); norm weights 1 + N(0, 0.1^2).  Always the whole vectors."""
    hd = cfg["head_dim"]
    qd, kvd = cfg["n_head"] * hd, cfg["n_head_kv"] * hd
    n_layer = 1 + max(int(k.split(".")[1]) for k in tensors if k.startswith("blk."))
    for i in range(n_layer):
        p = f"blk.{i}."
        if bias:
            for name, n in (("attn_q.bias", qd), ("attn_k.bias", kvd), ("attn_v.bias", kvd)):
                tensors[p + name] = {"data": (normal(n, seed_of(seed, p + name)) * np.float32(0.1)).astype(np.float32), "type": F32}
        if qk_norm:
            for name in ("attn_q_norm.weight", "attn_k_norm.weight"):
                tensors[p + name] = {"data": (np.float32(1.0) + normal(hd, seed_of(seed, p + name)) * np.float32(0.1)).astype(np.float32), "type": F32}
    return tensors
