"""GGUF files: a writer for synthetic models and a thin wrapper over the library's reader (ob_gguf_*).

The reader is the C++ one (csrc/gguf.cu), which follows src/gguf.rs:206-275 and engine/loader.rs:1652-1712; the writer
exists so that tests and the examples can produce files of the layout the reference loads: magic, version 3, u64
counts, typed metadata, tensor infos with data-section-relative offsets, data aligned to general.alignment."""
from __future__ import annotations

import ctypes as C
import struct

import numpy as np

from . import capi

_TYPES = {"u8": 0, "i8": 1, "u16": 2, "i16": 3, "u32": 4, "i32": 5, "f32": 6, "bool": 7, "str": 8, "arr": 9, "u64": 10, "i64": 11, "f64": 12}
_FMT = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<B", 10: "<Q", 11: "<q", 12: "<d"}


def _string(s: str) -> bytes:
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def _value(kind: str, v) -> bytes:
    t = _TYPES[kind]
    if kind == "str":
        return struct.pack("<I", t) + _string(v)
    if kind == "arr":  # (element kind, values)
        ek, vals = v
        et = _TYPES[ek]
        body = b"".join(_string(x) if ek == "str" else struct.pack(_FMT[et], x) for x in vals)
        return struct.pack("<IIQ", t, et, len(vals)) + body
    return struct.pack("<I", t) + struct.pack(_FMT[t], v)


def write_gguf(path: str, cfg: dict, tensors: dict, alignment: int = 32, extra_metadata: list | None = None, version: int = 3) -> None:
    """cfg: a synth.CONFIGS-style dict; tensors: name -> {"data", "type", ["in_dim", "out_dim"]} (orangu_b200.synth)."""
    a = cfg.get("architecture", "llama")  # metadata keys carry the architecture's name (loader.rs:1652-1712)
    meta = [("general.architecture", "str", a), ("general.alignment", "u32", alignment),
            (f"{a}.embedding_length", "u32", cfg["n_embd"]), (f"{a}.block_count", "u32", cfg["n_layer"]),
            (f"{a}.attention.head_count", "u32", cfg["n_head"]), (f"{a}.attention.head_count_kv", "u32", cfg["n_head_kv"]),
            (f"{a}.attention.key_length", "u32", cfg["head_dim"]), (f"{a}.rope.dimension_count", "u32", cfg.get("rope_dim", cfg["head_dim"])),
            (f"{a}.feed_forward_length", "u32", cfg["n_ff"]), (f"{a}.context_length", "u32", cfg.get("n_ctx_train", 4096)),
            (f"{a}.vocab_size", "u32", cfg["n_vocab"]), (f"{a}.rope.freq_base", "f32", cfg["rope_freq_base"]),
            (f"{a}.attention.layer_norm_rms_epsilon", "f32", cfg["rms_eps"])] + list(extra_metadata or [])
    head = b"GGUF" + struct.pack("<IQQ", version, len(tensors), len(meta))
    for k, kind, v in meta:
        head += _string(k) + _value(kind, v)
    infos, blobs, off = b"", [], 0
    for name, t in tensors.items():
        raw = np.ascontiguousarray(t["data"]).view(np.uint8).reshape(-1)
        dims = [t["in_dim"], t["out_dim"]] if "in_dim" in t else [int(np.asarray(t["data"]).size)]
        infos += _string(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", t["type"], off)
        blobs.append((off, raw))
        off = (off + raw.size + alignment - 1) // alignment * alignment
    start = (len(head) + len(infos) + alignment - 1) // alignment * alignment
    with open(path, "wb") as f:
        f.write(head + infos)
        f.write(b"\0" * (start - len(head) - len(infos)))
        pos = 0
        for o, raw in blobs:
            f.write(b"\0" * (o - pos))
            f.write(raw.tobytes())
            pos = o + raw.size


class GgufFile:
    """An open, memory-mapped GGUF file (ob_gguf)."""

    def __init__(self, path: str):
        self._lib = capi.load()
        h = C.c_void_p()
        rc = self._lib.ob_gguf_open(path.encode(), C.byref(h))
        if rc:
            raise capi.OranguError(rc, self._lib.ob_gguf_last_error().decode())
        self._h = h

    def close(self):
        if self._h:
            self._lib.ob_gguf_close(self._h)
            self._h = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    version = property(lambda self: self._lib.ob_gguf_version(self._h))
    alignment = property(lambda self: self._lib.ob_gguf_alignment(self._h))
    data_offset = property(lambda self: self._lib.ob_gguf_data_offset(self._h))

    def _check(self, rc):
        if rc:
            raise capi.OranguError(rc, self._lib.ob_gguf_last_error().decode())

    def tensors(self) -> list[dict]:
        out = []
        info = capi.GgufTensorInfo()
        for i in range(self._lib.ob_gguf_n_tensors(self._h)):
            self._check(self._lib.ob_gguf_tensor(self._h, i, C.byref(info)))
            out.append({"name": info.name.decode(), "type": info.ggml_type, "dims": list(info.dims[:info.n_dims]), "n_bytes": info.n_bytes, "address": info.data})
        return out

    def tensor_bytes(self, name: str) -> np.ndarray:
        info = capi.GgufTensorInfo()
        self._check(self._lib.ob_gguf_find_tensor(self._h, name.encode(), C.byref(info)))
        return np.ctypeslib.as_array((C.c_uint8 * info.n_bytes).from_address(info.data)).copy()

    def get_u64(self, key: str) -> int:
        v = C.c_uint64()
        self._check(self._lib.ob_gguf_get_u64(self._h, key.encode(), C.byref(v)))
        return v.value

    def get_f32(self, key: str) -> float:
        v = C.c_float()
        self._check(self._lib.ob_gguf_get_f32(self._h, key.encode(), C.byref(v)))
        return v.value

    def get_string(self, key: str) -> str:
        v = C.c_char_p()
        self._check(self._lib.ob_gguf_get_string(self._h, key.encode(), C.byref(v)))
        return v.value.decode()

    def model_desc(self) -> capi.ModelDesc:
        d = capi.ModelDesc()
        self._check(self._lib.ob_gguf_model_desc(self._h, C.byref(d)))
        return d
