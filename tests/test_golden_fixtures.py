"""The committed vectors of tests/golden/hotpath.npz (made by tests/golden/make_golden.py): the CPU oracle must still
produce them bit for bit, and -- on a GPU -- so must the CUDA path through the C ABI."""
import os

import numpy as np
import pytest

import oracle as O

G = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "hotpath.npz"))


def same_bits(a, b):
    a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
    assert a.shape == b.shape and a.dtype == b.dtype, (a.shape, b.shape, a.dtype, b.dtype)
    return bool((a.view(np.uint8) == b.view(np.uint8)).all())


@pytest.mark.parametrize("t", [8, 12, 13, 14])
def test_oracle_products(t):
    w, x = G[f"mm{t}_w"], G[f"mm{t}_x"]
    assert same_bits(O.matmul_decode(x, 3, w, t, 512, 6), G[f"mm{t}_decode"])
    assert same_bits(O.matmul(x, 3, w, t, 512, 6), G[f"mm{t}_prefill"])
    assert same_bits(O.dequantize(t, w, 6 * 512), G[f"mm{t}_dequant"])


def test_oracle_glue():
    for k in (0, 1):
        q, d, s = O.quantize_act(G["q_x"], bool(k))
        assert same_bits(q, G[f"q{k}_q"]) and same_bits(d, G[f"q{k}_d"]) and same_bits(s, G[f"q{k}_s"])
    assert same_bits(O.rmsnorm(G["norm_x"], G["norm_w"], 1e-5), G["norm_y"])
    assert same_bits(O.rope_norm(G["rope_x"], 4, 64, 37, 64, 500000.0), G["rope_y"])
    assert same_bits(O.swiglu(G["swiglu_g"], G["swiglu_u"]), G["swiglu_y"])
    assert same_bits(O.rope_layout(G["rope2_x"], 4, 64, 23, 32, 10000.0, True, G["rope2_ff"]), G["rope2_y"])
    assert same_bits(O.attention(G["att_q"], G["att_k"], G["att_v"], 4, 2, 64, 0.125, 1, 40), G["att_y"])


def test_oracle_model():
    from orangu_b200 import synth

    cfg = dict(synth.CONFIGS["tiny"])
    ref = O.Model(cfg, synth.model_tensors(cfg, seed=77))
    kv = ref.new_kv(32, f16=True)
    assert same_bits(ref.forward(kv, G["model_tokens"], 0), G["model_logits"][0])
    for i in range(3):
        assert same_bits(ref.forward(kv, [int(G["model_greedy"][i])], 9 + i), G["model_logits"][i + 1])


def qwen_style_tiny():
    from orangu_b200 import synth

    cfg = dict(synth.CONFIGS["tiny"], rope_neox=True)
    return cfg, synth.add_qwen_extras(cfg, synth.model_tensors(cfg, seed=78), seed=79)


def test_oracle_qwen_style_model():
    cfg, tensors = qwen_style_tiny()
    ref = O.Model(cfg, tensors)
    kv = ref.new_kv(32, f16=True)
    assert same_bits(ref.forward(kv, G["qmodel_tokens"], 0), G["qmodel_logits"][0])
    for i in range(3):
        assert same_bits(ref.forward(kv, [int(G["qmodel_greedy"][i])], 11 + i), G["qmodel_logits"][i + 1])


@pytest.fixture(scope="module")
def backend():
    import orangu_b200

    be = orangu_b200.CudaBackend.init(0)
    yield be
    be.close()


@pytest.mark.gpu
@pytest.mark.parametrize("t", [8, 12, 13, 14])
def test_cuda_products(backend, t):
    from orangu_b200 import QuantMatrix

    w = QuantMatrix(G[f"mm{t}_w"], t, 512, 6)
    x = G[f"mm{t}_x"]
    assert same_bits(backend.matmul_decode(x, 3, w), G[f"mm{t}_decode"])
    assert same_bits(backend.matmul(x, 3, w), G[f"mm{t}_prefill"])
    assert same_bits(backend.row(w, 0, 6).reshape(-1), G[f"mm{t}_dequant"])


@pytest.mark.gpu
def test_cuda_glue(backend):
    for k in (0, 1):
        q, d, s = backend.quantize_act(G["q_x"], bool(k))
        assert same_bits(q, G[f"q{k}_q"]) and same_bits(d, G[f"q{k}_d"]) and same_bits(s, G[f"q{k}_s"])
    assert same_bits(backend.rmsnorm(G["norm_x"], G["norm_w"], 1e-5), G["norm_y"])
    assert same_bits(backend.rope(G["rope_x"], 4, 64, 37, 64, 500000.0), G["rope_y"])
    assert same_bits(backend.swiglu(G["swiglu_g"], G["swiglu_u"]), G["swiglu_y"])
    assert same_bits(backend.attention_decode(G["att_q"], G["att_k"], G["att_v"], 4, 2, 64, 0.125, exact_order=True), G["att_y"].reshape(-1))


@pytest.mark.gpu
def test_cuda_model(backend):
    from orangu_b200 import LlamaModel, synth

    cfg = dict(synth.CONFIGS["tiny"])
    model = LlamaModel(backend, cfg, synth.model_tensors(cfg, seed=77), max_seq_len=64, max_batch_tokens=16)
    kv = model.new_kv_cache(32)
    assert same_bits(model.forward(kv, G["model_tokens"], 0).reshape(-1), G["model_logits"][0].reshape(-1))
    tok = backend.argmax(G["model_logits"][0])
    for i in range(3):
        assert tok == int(G["model_greedy"][i])
        logits = model.forward(kv, [tok], 9 + i)
        assert same_bits(logits.reshape(-1), G["model_logits"][i + 1].reshape(-1))
        tok = backend.argmax(logits)


@pytest.mark.gpu
def test_cuda_qwen_style_model(backend):
    from orangu_b200 import LlamaModel

    cfg, tensors = qwen_style_tiny()
    model = LlamaModel(backend, cfg, tensors, max_seq_len=64, max_batch_tokens=16)
    kv = model.new_kv_cache(32)
    assert same_bits(model.forward(kv, G["qmodel_tokens"], 0).reshape(-1), G["qmodel_logits"][0].reshape(-1))
    tok = backend.argmax(G["qmodel_logits"][0])
    for i in range(3):
        assert tok == int(G["qmodel_greedy"][i])
        logits = model.forward(kv, [tok], 11 + i)
        assert same_bits(logits.reshape(-1), G["qmodel_logits"][i + 1].reshape(-1))
        tok = backend.argmax(logits)
