"""Host-side mirror of the reference's ``ModelForward`` for Llama-style models
(src/bin/orangu-server/engine/arch/mod.rs:2035-2191, arch/llama.rs) over the C ABI."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import capi
from .backend import CudaBackend

LAYER_VECTORS = (("q_bias", "attn_q.bias"), ("k_bias", "attn_k.bias"), ("v_bias", "attn_v.bias"),
                 ("q_norm", "attn_q_norm.weight"), ("k_norm", "attn_k_norm.weight"))  # Qwen2 / Qwen3 extras, arch/llama.rs:45-60
LAYER_FIELDS = (("wq", "attn_q"), ("wk", "attn_k"), ("wv", "attn_v"), ("wo", "attn_output"),
                ("w_gate", "ffn_gate"), ("w_up", "ffn_up"), ("w_down", "ffn_down"))


def _matrix(t) -> capi.MatrixDesc:
    return capi.MatrixDesc(t["data"].ctypes.data, t["type"], t["in_dim"], t["out_dim"])


class KvCache:
    """Per-sequence paged fp16 KV cache (ModelForward::new_kv_cache, arch/llama.rs:1002-1005)."""

    def __init__(self, model: "LlamaModel", capacity: int, paged: bool = False):
        self.model = model
        self._lib = model._lib
        self._h = C.c_void_p()
        create = self._lib.ob_kv_create_paged if paged else self._lib.ob_kv_create  # paged: pages on demand, back on truncate
        capi.check(model.backend._h, create(model._h, capacity, C.byref(self._h)))
        self.capacity = capacity

    @property
    def pages(self) -> int:
        return int(self._lib.ob_kv_pages(self._h))

    def __len__(self):
        return int(self._lib.ob_kv_len(self._h))

    def truncate(self, new_len: int):
        capi.check(self.model.backend._h, self._lib.ob_kv_truncate(self._h, new_len))

    def read(self, layer: int, pos0: int, n: int):
        kvd = self.model.kv_dim_local
        k = np.empty((n, kvd), np.float32)
        v = np.empty((n, kvd), np.float32)
        capi.check(self.model.backend._h, self._lib.ob_kv_read(self._h, layer, pos0, n, k.ctypes.data, v.ctypes.data))
        return k, v

    def copy_prefix_from(self, src: "KvCache", n: int):
        """KvCache::copy_prefix_from (kv_cache.rs:1079-1100)."""
        capi.check(self.model.backend._h, self._lib.ob_kv_copy_prefix(self._h, src._h, n))

    def close(self):
        if self._h:
            if self.model._h and self.model.backend._h:  # after the backend is gone the handle is no longer valid: leave it
                self._lib.ob_kv_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            if self.model._h:
                self.close()
        except Exception:
            pass


class LlamaModel:
    """Built from a dict of named tensors (GGUF names, arch/llama.rs:125-183): each value is
    ``{"data": np.ndarray, "type": ggml_type, "in_dim": .., "out_dim": ..}``; norm vectors are f32."""

    def __init__(self, backend: CudaBackend, cfg: dict, tensors: dict, max_seq_len: int = 4096, max_batch_tokens: int = 512,
                 kv_pool_tokens: int = 0, exact_attention_max_pos: int = 0, tp_rank: int = 0, tp_size: int = 1, tp_unique_id: bytes | None = None,
                 tp_presliced: bool = False):
        self.backend = backend
        self._lib = backend._lib
        self.cfg = dict(cfg)
        n_layer = cfg["n_layer"]
        layers = (capi.LayerDesc * n_layer)()
        for i in range(n_layer):
            layers[i].attn_norm = tensors[f"blk.{i}.attn_norm.weight"]["data"].ctypes.data
            layers[i].ffn_norm = tensors[f"blk.{i}.ffn_norm.weight"]["data"].ctypes.data
            for field, name in LAYER_FIELDS:
                setattr(layers[i], field, _matrix(tensors[f"blk.{i}.{name}.weight"]))
            for field, name in LAYER_VECTORS:
                if f"blk.{i}.{name}" in tensors:
                    setattr(layers[i], field, tensors[f"blk.{i}.{name}"]["data"].ctypes.data)  # f32, contiguous, kept alive by the caller's dict
        d = capi.ModelDesc()
        for k in ("n_vocab", "n_embd", "n_layer", "n_head", "n_head_kv", "head_dim", "n_ff"):
            setattr(d, k, cfg[k])
        d.rope_dim = cfg.get("rope_dim", cfg["head_dim"])
        d.rope_freq_base = cfg["rope_freq_base"]
        d.rms_eps = cfg["rms_eps"]
        d.rope_neox = 1 if cfg.get("rope_neox") else 0  # rope_layout_for, arch/llama.rs:114-119
        d.max_seq_len = max_seq_len
        d.max_batch_tokens = max_batch_tokens
        d.kv_pool_tokens = kv_pool_tokens
        d.exact_attention_max_pos = exact_attention_max_pos
        d.token_embd = _matrix(tensors["token_embd.weight"])
        d.output_norm = tensors["output_norm.weight"]["data"].ctypes.data
        if "output.weight" in tensors:
            d.output = _matrix(tensors["output.weight"])
        d.layers = layers
        d.tp_rank, d.tp_size = tp_rank, tp_size
        d.tp_presliced = 1 if (tp_presliced and tp_size > 1) else 0  # the tensors are this rank's shards already (synth.model_tensors(..., tp=(rank, size)))
        self._id = C.create_string_buffer(tp_unique_id, 128) if tp_unique_id else None
        d.tp_unique_id = C.addressof(self._id) if self._id else None
        if "rope_freqs.weight" in tensors:  # llama.rs:186-200
            self._rope_freqs = np.ascontiguousarray(tensors["rope_freqs.weight"]["data"], np.float32)
            if self._rope_freqs.size < d.rope_dim // 2:
                raise ValueError("rope_freqs.weight is shorter than rope_dim / 2")
            d.rope_freqs = self._rope_freqs.ctypes.data
        self._h = C.c_void_p()
        capi.check(backend._h, self._lib.ob_model_create(backend._h, C.byref(d), C.byref(self._h)))
        self.n_vocab = cfg["n_vocab"]
        self.kv_dim_local = cfg["n_head_kv"] // max(1, tp_size) * cfg["head_dim"]
        self.max_batch_tokens = max_batch_tokens

    @classmethod
    def from_gguf(cls, backend: CudaBackend, path: str, max_seq_len: int = 0, max_batch_tokens: int = 512, kv_pool_tokens: int = 0,
                  exact_attention_max_pos: int = 0, tp_rank: int = 0, tp_size: int = 1, tp_unique_id: bytes | None = None) -> "LlamaModel":
        """LlamaModel::load_with_backend (arch/llama.rs:125-230) from a .gguf file: the library maps the file, reads the
        configuration and the tensor table (ob_gguf_open, ob_gguf_model_desc) and uploads its share of every tensor."""
        from .gguf import GgufFile

        self = cls.__new__(cls)
        self.backend, self._lib = backend, backend._lib
        with GgufFile(path) as g:
            d = g.model_desc()
            if max_seq_len:
                d.max_seq_len = max_seq_len
            d.max_batch_tokens, d.kv_pool_tokens, d.exact_attention_max_pos = max_batch_tokens, kv_pool_tokens, exact_attention_max_pos
            d.tp_rank, d.tp_size = tp_rank, tp_size
            self._id = C.create_string_buffer(tp_unique_id, 128) if tp_unique_id else None
            d.tp_unique_id = C.addressof(self._id) if self._id else None
            self.cfg = {k: getattr(d, k) for k in ("n_vocab", "n_embd", "n_layer", "n_head", "n_head_kv", "head_dim", "rope_dim", "n_ff", "rope_freq_base", "rms_eps")}
            self._h = C.c_void_p()
            capi.check(backend._h, self._lib.ob_model_create(backend._h, C.byref(d), C.byref(self._h)))  # copies what it needs out of the mapping
        self.n_vocab = self.cfg["n_vocab"]
        self.kv_dim_local = self.cfg["n_head_kv"] // max(1, tp_size) * self.cfg["head_dim"]
        self.max_batch_tokens = max_batch_tokens
        return self

    def new_kv_cache(self, capacity: int, paged: bool = False) -> KvCache:
        return KvCache(self, capacity, paged)

    @property
    def free_pages(self) -> int:
        return int(self._lib.ob_model_free_pages(self._h))

    @property
    def pool_pages(self) -> int:
        return int(self._lib.ob_model_pool_pages(self._h))

    # ModelForward::forward (arch/llama.rs:1007-1032): logits of the last token
    def forward(self, cache: KvCache, tokens, start_pos: int) -> np.ndarray:
        return self._forward([cache], [list(tokens)], [start_pos], want_logits=True)[1][0]

    # ModelForward::forward_maybe_sampling with a greedy sampler (arch/llama.rs:949-1000): next token id
    def forward_maybe_sampling(self, cache: KvCache, tokens, start_pos: int, recent=None, repeat_penalty: float = 1.0, repeat_last_n: int = 64) -> int:
        g = None
        if recent is not None and repeat_penalty != 1.0:
            g = ([np.ascontiguousarray(recent, np.uint32)], repeat_penalty, repeat_last_n)
        return int(self._forward([cache], [list(tokens)], [start_pos], want_tokens=True, greedy=g)[0][0])

    # ModelForward::forward_batch_decode (arch/mod.rs:2174-2190): one token per sequence
    def forward_batch_decode(self, caches, tokens, want_logits: bool = False):
        toks, logits = self._forward(list(caches), [[int(t)] for t in tokens], [len(c) for c in caches], want_tokens=True, want_logits=want_logits)
        return (toks, logits) if want_logits else toks

    def _forward(self, caches, token_lists, start_pos, want_tokens=False, want_logits=False, greedy=None):
        n_seq = len(caches)
        kvs = (C.c_void_p * n_seq)(*[c._h for c in caches])
        flat = np.ascontiguousarray([t for l in token_lists for t in l], dtype=np.uint32)
        n_tok = np.ascontiguousarray([len(l) for l in token_lists], dtype=np.uint32)
        sp = np.ascontiguousarray(start_pos, dtype=np.uint32)
        out_tok = np.zeros(n_seq, np.uint32) if want_tokens else None
        out_log = np.empty((n_seq, self.n_vocab), np.float32) if want_logits else None
        gptr = None
        if greedy is not None:
            recents, penalty, last_n = greedy
            rec = np.ascontiguousarray(np.concatenate(recents), np.uint32)
            nrec = np.ascontiguousarray([len(r) for r in recents], np.uint32)
            gs = capi.Greedy(penalty, last_n, rec.ctypes.data, nrec.ctypes.data)
            gptr = C.addressof(gs)
        capi.check(self.backend._h, self._lib.ob_forward(
            self._h, kvs, flat.ctypes.data, n_tok.ctypes.data, sp.ctypes.data, n_seq, gptr,
            out_tok.ctypes.data if want_tokens else None, out_log.ctypes.data if want_logits else None))
        return out_tok, out_log

    def decode_greedy(self, cache: KvCache, token: int) -> int:
        """One greedy step replayed from the captured CUDA graph (record_decode_chain, arch/llama.rs:302-473)."""
        out = C.c_uint32()
        capi.check(self.backend._h, self._lib.ob_decode_greedy(self._h, cache._h, int(token), C.byref(out)))
        return int(out.value)

    def decode_loop(self, caches, first_tokens, n_steps: int) -> np.ndarray:
        """n_steps greedy steps for every sequence without the host in between; [n_steps, n_seq] token ids."""
        n_seq = len(caches)
        kvs = (C.c_void_p * n_seq)(*[c._h for c in caches])
        ft = np.ascontiguousarray(first_tokens, dtype=np.uint32)
        out = np.empty((n_steps, n_seq), np.uint32)
        capi.check(self.backend._h, self._lib.ob_decode_loop(self._h, kvs, ft.ctypes.data, n_seq, n_steps, out.ctypes.data))
        return out

    def profile_gemv(self, ggml_type: int, iters: int, variant: int = 0):
        """(ms_total, bytes_per_pass, launches_per_pass) of the single-token GEMVs of one weight type, run alone."""
        ms, nbytes, nl = C.c_float(), C.c_uint64(), C.c_uint32()
        capi.check(self.backend._h, self._lib.ob_profile_gemv(self._h, ggml_type, variant, iters, C.byref(ms), C.byref(nbytes), C.byref(nl)))
        return ms.value, nbytes.value, nl.value

    def last_hidden(self, n_tokens: int) -> np.ndarray:
        out = np.empty((n_tokens, self.cfg["n_embd"]), np.float32)
        capi.check(self.backend._h, self._lib.ob_last_hidden(self._h, n_tokens, out.ctypes.data))
        return out

    def close(self):
        if self._h:
            self._lib.ob_model_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            if self.backend._h:
                self.close()
        except Exception:
            pass
