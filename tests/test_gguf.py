"""GGUF files: the library's reader against files written here (layout of src/gguf.rs:206-275), the model description
it derives (engine/loader.rs:1652-1712, engine/arch/llama.rs:125-200), and -- on a GPU -- a model loaded from a file
against the same model built from the tensors and against the oracle."""
import os
import struct

import numpy as np
import pytest

from gpu_common import backend  # noqa: F401
from orangu_b200 import capi, synth
from orangu_b200.gguf import GgufFile, write_gguf


PER_32_MIX = {"token_embd": 2, "output": 6, "attn_q": 2, "attn_k": 20, "attn_v": 6, "attn_output": 2, "ffn_gate": 20, "ffn_up": 2, "ffn_down": 6}


def tiny(seed=5, with_output=True, rope_freqs=False, types=None):
    cfg = dict(synth.CONFIGS["tiny"])
    tensors = synth.model_tensors(cfg, seed=seed, types=types)
    if not with_output:
        del tensors["output.weight"]
    if rope_freqs:
        tensors["rope_freqs.weight"] = {"data": np.linspace(1.0, 8.0, cfg["head_dim"] // 2).astype(np.float32), "type": 0}
    return cfg, tensors


@pytest.mark.parametrize("alignment", [32, 64, 4096])
def test_reader_sees_what_the_writer_wrote(tmp_path, alignment):
    cfg, tensors = tiny(rope_freqs=True)
    path = str(tmp_path / "tiny.gguf")
    write_gguf(path, cfg, tensors, alignment=alignment, extra_metadata=[("tokenizer.ggml.tokens", "arr", ("str", ["a", "bc", "def"])), ("general.name", "str", "tiny")])
    with GgufFile(path) as g:
        assert g.version == 3 and g.alignment == alignment and g.data_offset % alignment == 0
        assert g.get_string("general.architecture") == "llama" and g.get_string("general.name") == "tiny"
        assert g.get_u64("llama.block_count") == cfg["n_layer"] and abs(g.get_f32("llama.rope.freq_base") - cfg["rope_freq_base"]) < 1e-3
        infos = {t["name"]: t for t in g.tensors()}
        assert set(infos) == set(tensors)
        for name, t in tensors.items():
            raw = np.ascontiguousarray(t["data"]).view(np.uint8).reshape(-1)
            assert infos[name]["type"] == t["type"] and infos[name]["n_bytes"] == raw.size
            assert infos[name]["address"] % alignment == (g.data_offset % alignment)  # mapping is page aligned; offsets keep the alignment
            assert (g.tensor_bytes(name) == raw).all(), name
            if "in_dim" in t:
                assert infos[name]["dims"] == [t["in_dim"], t["out_dim"]]  # dims[0] is the contiguous one
        d = g.model_desc()
        for k in ("n_vocab", "n_embd", "n_layer", "n_head", "n_head_kv", "head_dim", "n_ff"):
            assert getattr(d, k) == cfg[k], k
        assert d.rope_dim == cfg["head_dim"] and abs(d.rms_eps - cfg["rms_eps"]) < 1e-12 and d.rope_freqs
        assert d.layers[1].w_down.in_dim == cfg["n_ff"] and d.layers[1].w_down.out_dim == cfg["n_embd"] and d.layers[0].wv.ggml_type == 14


def test_per_32_symmetric_tensors_are_sized_and_described(tmp_path):
    cfg, tensors = tiny(types=PER_32_MIX)
    path = str(tmp_path / "mix.gguf")
    write_gguf(path, cfg, tensors)
    with GgufFile(path) as g:
        infos = {t["name"]: t for t in g.tensors()}
        for name, t in tensors.items():
            assert infos[name]["type"] == t["type"] and infos[name]["n_bytes"] == np.ascontiguousarray(t["data"]).view(np.uint8).size, name
        desc = g.model_desc()  # every tensor type has a kernel
        assert desc is not None


def test_defaults_and_tied_output(tmp_path):
    """head_count_kv, key_length, rope.dimension_count, freq_base, eps and vocab_size default as the reference's loader does."""
    cfg, tensors = tiny(with_output=False)
    cfg["n_head_kv"] = cfg["n_head"]  # so that the default (== n_head) matches the k/v tensors
    tensors = synth.model_tensors(cfg, seed=5)
    del tensors["output.weight"]
    path = str(tmp_path / "min.gguf")
    write_gguf(path, cfg, tensors)
    # rewrite with only the required keys
    from orangu_b200 import gguf as G

    meta = [("general.architecture", "str", "llama"), ("llama.embedding_length", "u32", cfg["n_embd"]), ("llama.block_count", "u64", cfg["n_layer"]),
            ("llama.attention.head_count", "i32", cfg["n_head"]), ("tokenizer.ggml.tokens", "arr", ("str", ["t%d" % i for i in range(cfg["n_vocab"])]))]
    head = b"GGUF" + struct.pack("<IQQ", 3, len(tensors), len(meta))
    for k, kind, v in meta:
        head += G._string(k) + G._value(kind, v)
    infos, blobs, off = b"", [], 0
    for name, t in tensors.items():
        raw = np.ascontiguousarray(t["data"]).view(np.uint8).reshape(-1)
        dims = [t["in_dim"], t["out_dim"]] if "in_dim" in t else [int(np.asarray(t["data"]).size)]
        infos += G._string(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", x) for x in dims) + struct.pack("<IQ", t["type"], off)
        blobs.append((off, raw))
        off = (off + raw.size + 31) // 32 * 32
    start = (len(head) + len(infos) + 31) // 32 * 32
    with open(path, "wb") as f:
        f.write(head + infos + b"\0" * (start - len(head) - len(infos)))
        pos = 0
        for o, raw in blobs:
            f.write(b"\0" * (o - pos) + raw.tobytes())
            pos = o + raw.size
    with GgufFile(path) as g:
        assert g.alignment == 32
        d = g.model_desc()
        assert d.n_head_kv == cfg["n_head"] and d.head_dim == cfg["n_embd"] // cfg["n_head"] and d.rope_dim == d.head_dim
        assert d.n_vocab == cfg["n_vocab"] and abs(d.rope_freq_base - 10000.0) < 1e-3 and abs(d.rms_eps - 1e-5) < 1e-12
        assert d.n_ff == cfg["n_ff"] and not d.output.data and not d.rope_freqs  # tied output, no frequency factors


def test_malformed_files_are_refused_with_a_message(tmp_path):
    cfg, tensors = tiny()
    good = str(tmp_path / "good.gguf")
    write_gguf(good, cfg, tensors)
    blob = open(good, "rb").read()

    def refused(data, needle):
        p = str(tmp_path / "bad.gguf")
        open(p, "wb").write(data)
        with pytest.raises(capi.OranguError) as e:
            GgufFile(p)
        assert needle in str(e.value), str(e.value)

    refused(b"GGML" + blob[4:], "bad magic")
    refused(blob[:4] + struct.pack("<I", 1) + blob[8:], "version 1")
    refused(blob[:16], "shorter than")
    refused(blob[:len(blob) // 2], "past the end")                                     # tensor data cut off
    refused(blob[:24] + struct.pack("<Q", 1 << 40) + blob[32:], "malformed metadata")  # a key length of a terabyte
    refused(blob[:8] + struct.pack("<Q", 1 << 40) + blob[16:], "implausible")
    with pytest.raises(capi.OranguError):
        GgufFile(str(tmp_path / "missing.gguf"))
    # a tensor offset chosen so that data_offset + offset wraps around 2^64 must not pass the bounds check
    with GgufFile(good) as g:
        data_offset = g.data_offset
    first_off = blob.index(struct.pack("<IQ", tensors["token_embd.weight"]["type"], 0), 24) + 4  # the first tensor's offset field
    wrap = (1 << 64) - data_offset + 64
    wrap -= wrap % 32
    refused(blob[:first_off] + struct.pack("<Q", wrap) + blob[first_off + 8:], "past the end")
    # rows that are not a whole number of blocks (a Q4_K tensor 100 elements wide)
    odd = dict(tensors)
    odd["blk.0.attn_q.weight"] = dict(tensors["blk.0.attn_q.weight"], in_dim=100)
    p_odd = str(tmp_path / "odd.gguf")
    write_gguf(p_odd, cfg, odd)
    with pytest.raises(capi.OranguError) as e:
        GgufFile(p_odd)
    assert "whole number of 256-element blocks" in str(e.value)
    # a block count far beyond what the file's tensors could make up is an error, not an allocation
    p_big = str(tmp_path / "big.gguf")
    huge = dict(cfg, n_layer=(1 << 32) - 1)
    write_gguf(p_big, huge, tensors)
    with GgufFile(p_big) as g, pytest.raises(capi.OranguError) as e:
        g.model_desc()
    assert "block_count" in str(e.value)
    # a model whose architecture or tensor types are outside the build is named, not crashed on
    p = str(tmp_path / "arch.gguf")
    write_gguf(p, cfg, tensors)
    data = open(p, "rb").read().replace(b"\x05\x00\x00\x00\x00\x00\x00\x00llama", b"\x05\x00\x00\x00\x00\x00\x00\x00gemma", 1)
    open(p, "wb").write(data)
    with GgufFile(p) as g, pytest.raises(capi.OranguError) as e:
        g.model_desc()
    assert "gemma" in str(e.value)
    bad = dict(tensors)
    bad["blk.0.attn_q.weight"] = dict(tensors["blk.0.attn_q.weight"], type=10)  # Q2_K: sized, but no kernel
    bad["blk.0.attn_q.weight"]["data"] = np.zeros(cfg["n_head"] * cfg["head_dim"] * cfg["n_embd"] // 256 * 84, np.uint8)
    write_gguf(p, cfg, bad)
    with GgufFile(p) as g, pytest.raises(capi.OranguError) as e:
        g.model_desc()
    assert "blk.0.attn_q.weight" in str(e.value) and "10" in str(e.value)


@pytest.mark.parametrize("arch,bias,qk_norm,neox", [("qwen2", True, False, 1), ("qwen3", False, True, 1), ("mistral", False, False, 0), ("qwen3vl", True, True, 1)])
def test_llama_style_architectures_and_their_extra_tensors(tmp_path, arch, bias, qk_norm, neox):
    """LLAMA_STYLE_ARCHITECTURES (loader.rs:190); attn_{q,k,v}.bias and attn_{q,k}_norm.weight are optional per file
    (arch/llama.rs:171-175); the pairing follows the architecture (rope_layout_for, arch/llama.rs:114-119)."""
    cfg, tensors = tiny()
    cfg["architecture"] = arch
    synth.add_qwen_extras(cfg, tensors, seed=3, bias=bias, qk_norm=qk_norm)
    path = str(tmp_path / "q.gguf")
    write_gguf(path, cfg, tensors)
    with GgufFile(path) as g:
        assert g.get_string("general.architecture") == arch
        d = g.model_desc()
        assert d.rope_neox == neox and d.n_head == cfg["n_head"]
        for i in range(cfg["n_layer"]):
            L = d.layers[i]
            assert bool(L.q_bias) == bool(L.k_bias) == bool(L.v_bias) == bias and bool(L.q_norm) == bool(L.k_norm) == qk_norm
            if bias:
                got = np.ctypeslib.as_array((capi.C.c_float * (cfg["n_head_kv"] * cfg["head_dim"])).from_address(L.k_bias))
                assert (got == tensors[f"blk.{i}.attn_k.bias"]["data"]).all()


@pytest.mark.gpu
def test_qwen3_style_file_runs_and_equals_the_oracle(backend, tmp_path):
    import oracle as O
    import orangu_b200
    from gpu_common import assert_bit_equal

    cfg, tensors = tiny(seed=13)
    cfg.update(architecture="qwen3", rope_neox=True)
    synth.add_qwen_extras(cfg, tensors, seed=4)
    path = str(tmp_path / "q3.gguf")
    write_gguf(path, cfg, tensors)
    model, ref = orangu_b200.LlamaModel.from_gguf(backend, path, max_seq_len=64, max_batch_tokens=16), O.Model(cfg, tensors)
    toks = np.random.default_rng(2).integers(0, cfg["n_vocab"], 19).astype(np.uint32)
    kv, rkv = model.new_kv_cache(40), ref.new_kv(40, f16=True)
    assert_bit_equal(model.forward(kv, toks, 0), ref.forward(rkv, toks, 0), "prefill logits")
    assert_bit_equal(model.forward(kv, [5], 19), ref.forward(rkv, [5], 19), "decode step")


@pytest.mark.gpu
@pytest.mark.parametrize("with_output,rope_freqs,types", [(True, False, None), (False, True, None), (True, False, PER_32_MIX)])
def test_model_from_a_file_equals_the_model_from_tensors_and_the_oracle(backend, tmp_path, with_output, rope_freqs, types):
    import oracle as O
    import orangu_b200
    from gpu_common import assert_bit_equal

    be = backend
    cfg, tensors = tiny(seed=9, with_output=with_output, rope_freqs=rope_freqs, types=types)
    path = str(tmp_path / "m.gguf")
    write_gguf(path, cfg, tensors, alignment=64)
    from_file = orangu_b200.LlamaModel.from_gguf(be, path, max_seq_len=64, max_batch_tokens=16)
    from_mem = orangu_b200.LlamaModel(be, cfg, tensors, max_seq_len=64, max_batch_tokens=16)
    ref = O.Model(cfg, tensors)
    toks = np.random.default_rng(1).integers(0, cfg["n_vocab"], 11).astype(np.uint32)
    ka, kb, kr = from_file.new_kv_cache(32), from_mem.new_kv_cache(32), ref.new_kv(32, f16=True)
    a, b, want = from_file.forward(ka, toks, 0), from_mem.forward(kb, toks, 0), ref.forward(kr, toks, 0)
    assert_bit_equal(a, want, "prefill logits, model from the file")
    assert_bit_equal(b, want, "prefill logits, model from tensors")
    tok = O.argmax(want)
    for step in range(4):
        a, want = from_file.forward(ka, [tok], 11 + step), ref.forward(kr, [tok], 11 + step)
        assert_bit_equal(a, want, f"decode step {step}")
        tok = O.argmax(want)
