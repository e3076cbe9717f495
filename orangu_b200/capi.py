"""ctypes binding of include/orangu_b200.h.  Loads the in-tree library and fails loudly otherwise."""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(HERE, "_lib", "liborangu_b200.so")

STATUS = {0: "OB_OK", -1: "OB_ERR_INVALID", -2: "OB_ERR_UNSUPPORTED", -3: "OB_ERR_NO_DEVICE", -4: "OB_ERR_CUDA",
          -5: "OB_ERR_OOM", -6: "OB_ERR_CAPACITY", -7: "OB_ERR_COMM"}


class OranguError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"{STATUS.get(status, status)}: {message}")
        self.status = status
        self.message = message


class MatrixDesc(C.Structure):
    _fields_ = [("data", C.c_void_p), ("ggml_type", C.c_uint32), ("in_dim", C.c_uint32), ("out_dim", C.c_uint32)]


class LayerDesc(C.Structure):
    _fields_ = [("attn_norm", C.c_void_p), ("ffn_norm", C.c_void_p)] + [
        (n, MatrixDesc) for n in ("wq", "wk", "wv", "wo", "w_gate", "w_up", "w_down")] + [
        (n, C.c_void_p) for n in ("q_bias", "k_bias", "v_bias", "q_norm", "k_norm")]


class ModelDesc(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("n_vocab", "n_embd", "n_layer", "n_head", "n_head_kv", "head_dim", "rope_dim", "n_ff")] + [
        ("rope_freq_base", C.c_float), ("rms_eps", C.c_float),
        ("max_seq_len", C.c_uint32), ("max_batch_tokens", C.c_uint32), ("kv_pool_tokens", C.c_uint64), ("exact_attention_max_pos", C.c_uint32),
        ("token_embd", MatrixDesc), ("output_norm", C.c_void_p), ("output", MatrixDesc),
        ("layers", C.POINTER(LayerDesc)), ("tp_rank", C.c_uint32), ("tp_size", C.c_uint32), ("tp_unique_id", C.c_void_p),
        ("rope_freqs", C.c_void_p), ("tp_presliced", C.c_uint32), ("rope_neox", C.c_uint32)]


class MatmulOpC(C.Structure):
    _fields_ = [("x", C.c_void_p), ("n_tokens", C.c_uint32), ("w", C.c_void_p), ("y", C.c_void_p)]


class Greedy(C.Structure):
    _fields_ = [("repeat_penalty", C.c_float), ("repeat_last_n", C.c_uint32), ("recent", C.c_void_p), ("n_recent", C.c_void_p)]


# name -> (restype, argtypes); every symbol the header declares
_vp, _u32, _u64, _i32, _f32 = C.c_void_p, C.c_uint32, C.c_uint64, C.c_int, C.c_float
_PP = C.POINTER(C.c_void_p)
class GgufTensorInfo(C.Structure):
    _fields_ = [("name", C.c_char_p), ("ggml_type", C.c_uint32), ("n_dims", C.c_uint32), ("dims", C.c_uint64 * 4), ("data", C.c_void_p), ("n_bytes", C.c_uint64)]


SIGNATURES = {
    "ob_gguf_open": (_i32, [C.c_char_p, _PP]),
    "ob_gguf_close": (None, [_vp]),
    "ob_gguf_last_error": (C.c_char_p, []),
    "ob_gguf_version": (C.c_uint32, [_vp]),
    "ob_gguf_alignment": (_u64, [_vp]),
    "ob_gguf_data_offset": (_u64, [_vp]),
    "ob_gguf_n_tensors": (_u64, [_vp]),
    "ob_gguf_tensor": (_i32, [_vp, _u64, C.POINTER(GgufTensorInfo)]),
    "ob_gguf_find_tensor": (_i32, [_vp, C.c_char_p, C.POINTER(GgufTensorInfo)]),
    "ob_gguf_get_u64": (_i32, [_vp, C.c_char_p, C.POINTER(C.c_uint64)]),
    "ob_gguf_get_f32": (_i32, [_vp, C.c_char_p, C.POINTER(C.c_float)]),
    "ob_gguf_get_string": (_i32, [_vp, C.c_char_p, C.POINTER(C.c_char_p)]),
    "ob_gguf_model_desc": (_i32, [_vp, C.POINTER(ModelDesc)]),
    "ob_init": (_i32, [_i32, _PP]),
    "ob_destroy": (None, [_vp]),
    "ob_last_error": (C.c_char_p, [_vp]),
    "ob_abi_version": (C.c_uint, []),
    "ob_supports_type": (_i32, [_u32]),
    "ob_reduced_surface": (C.c_char_p, []),
    "ob_weight_register": (_i32, [_vp, _vp, _u64, _u32, _u32, _u32, _PP]),
    "ob_weight_register_slice": (_i32, [_vp, _vp, _u64, _u32, _u32, _u32, _u32, _u32, _u32, _u32, _PP]),
    "ob_weight_release": (None, [_vp, _vp]),
    "ob_weight_dequantize": (_i32, [_vp, _vp, _u32, _u32, _vp]),
    "ob_matmul": (_i32, [_vp, _vp, _u32, _vp, _vp]),
    "ob_matmul_decode": (_i32, [_vp, _vp, _u32, _vp, _vp]),
    "ob_matmul_batch": (_i32, [_vp, _vp, _u32, _i32]),
    "ob_matmul_device": (_i32, [_vp, _vp, _u32, _vp, _vp, _i32, _vp]),
    "ob_synchronize": (_i32, [_vp]),
    "ob_matmul_partials": (_i32, [_vp, _vp, _vp, _u32, _u32, _vp, _vp]),
    "ob_rmsnorm": (_i32, [_vp, _vp, _vp, _u32, _u32, _f32, _vp]),
    "ob_rope": (_i32, [_vp, _vp, _u32, _u32, _u32, _u32, _f32]),
    "ob_swiglu": (_i32, [_vp, _vp, _vp, _u32, _vp]),
    "ob_quantize_act": (_i32, [_vp, _vp, _u32, _i32, _vp, _vp, _vp]),
    "ob_attention_decode": (_i32, [_vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _f32, _i32, _vp]),
    "ob_attention_decode_static": (_i32, [_vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _f32, _vp, _vp]),
    "ob_argmax": (_i32, [_vp, _vp, _u32, _vp, _u32, _u32, _f32, _vp]),
    "ob_model_create": (_i32, [_vp, C.POINTER(ModelDesc), _PP]),
    "ob_model_destroy": (None, [_vp]),
    "ob_kv_create": (_i32, [_vp, _u32, _PP]),
    "ob_kv_create_paged": (_i32, [_vp, _u32, _PP]),
    "ob_kv_destroy": (None, [_vp]),
    "ob_kv_pages": (_u32, [_vp]),
    "ob_model_pool_pages": (_u32, [_vp]),
    "ob_model_free_pages": (_u32, [_vp]),
    "ob_model_n_vocab": (_u32, [_vp]),
    "ob_model_tp_size": (_u32, [_vp]),
    "ob_model_ctx": (_vp, [_vp]),
    "ob_kv_len": (_u32, [_vp]),
    "ob_kv_truncate": (_i32, [_vp, _u32]),
    "ob_kv_read": (_i32, [_vp, _u32, _u32, _u32, _vp, _vp]),
    "ob_kv_copy_prefix": (_i32, [_vp, _vp, _u32]),
    "ob_profile_gemv": (_i32, [_vp, _u32, _u32, _u32, _vp, _vp, _vp]),
    "ob_forward": (_i32, [_vp, _vp, _vp, _vp, _vp, _u32, _vp, _vp, _vp]),
    "ob_decode_greedy": (_i32, [_vp, _vp, _u32, _vp]),
    "ob_decode_loop": (_i32, [_vp, _vp, _vp, _u32, _u32, _vp]),
    "ob_last_hidden": (_i32, [_vp, _u32, _vp]),
    "ob_launch_count": (_u64, [_vp]),
    "ob_last_device_ms": (_f32, [_vp]),
    "ob_tp_unique_id": (_i32, [_vp]),
    "ob_tp_exchange_selftest": (_i32, [_vp, _u32, _u32, _u32, _vp, _vp]),
    "ob_tp_rendezvous_selftest": (_i32, [_vp, _u32, _u32, _u32, _u32, _vp]),
    "ob_tp_bulk_selftest": (_i32, [_vp, _u32, _u32, _u32, _vp, _vp]),
    "ob_slot_pool_create": (_i32, [_vp, _vp, _PP]),
    "ob_slot_pool_destroy": (None, [_vp]),
    "ob_slot_acquire": (_i32, [_vp, _i32, _vp]),
    "ob_slot_acquire_id": (_i32, [_vp, _u32, _i32]),
    "ob_slot_release": (_i32, [_vp, _u32]),
    "ob_slot_prefill": (_i32, [_vp, _u32, _vp, _u32, _vp, _vp]),
    "ob_slot_decode": (_i32, [_vp, _u32, _u32, _vp, _vp, _vp]),
    "ob_slot_truncate": (_i32, [_vp, _u32, _u32]),
    "ob_slot_len": (_u32, [_vp, _u32]),
    "ob_slot_kv": (_vp, [_vp, _u32]),
    "ob_slot_pool_snapshot": (_u32, [_vp, _vp, _u32]),
    "ob_slot_pool_get_stats": (_i32, [_vp, _vp]),
    "ob_slot_last_error": (C.c_char_p, [_vp, C.c_int64]),
    "ob_slot_pool_selftest": (_i32, [_u32, _u32, _u32, _u32, _u32, _vp]),
}

_lib = None


def lib_path() -> str:
    return _LIB_PATH


def load():
    """The loaded library.  Raises if it has not been built: there is no fallback path."""
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            raise OranguError(-3, f"{_LIB_PATH} is missing; build it with `python -m orangu_b200.build`")
        L = C.CDLL(_LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)  # AttributeError if the library lacks a declared symbol
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def check(ctx, status: int):
    if status != 0:
        msg = load().ob_last_error(ctx)
        raise OranguError(status, msg.decode() if msg else "")
