"""The synthetic weight builder: deterministic, and its blocks decode (through the oracle) to values close to the source."""
import numpy as np
import pytest

import oracle as O
from orangu_b200 import synth


def test_normal_is_seeded_and_standard():
    a = synth.normal(200000, 7)
    assert (a == synth.normal(200000, 7)).all()
    assert not (a == synth.normal(200000, 8)).all()
    assert abs(a.mean()) < 0.01 and abs(a.std() - 1.0) < 0.01
    # any sub-range reproduces: element e depends on (seed, e) only
    m = synth.matrix(synth.Q8_0, 4, 64, 3)
    assert (m["data"] == synth.matrix(synth.Q8_0, 4, 64, 3)["data"]).all()


@pytest.mark.parametrize("t,tol", [(synth.Q8_0, 0.008), (synth.Q4_K, 0.10), (synth.Q6_K, 0.03)])
def test_quantizers_round_trip_through_the_reference_decode_rules(t, tol):
    w = synth.normal(16 * 1024, 11, 0.02).reshape(16, 1024)
    raw = synth.quantize(w, t)
    assert raw.size == 16 * O.row_bytes(t, 1024)
    back = O.dequantize(t, raw, w.size).reshape(w.shape)
    assert np.isfinite(back).all()
    rms = np.sqrt(np.mean((back - w) ** 2)) / np.sqrt(np.mean(w ** 2))
    assert rms < tol, rms


@pytest.mark.parametrize("t", [synth.Q4_0, synth.Q5_0, synth.IQ4_NL])
def test_per_32_symmetric_matrices_are_seeded_finite_and_of_the_wanted_scale(t):
    m = synth.matrix(t, 64, 1024, 21, std=0.02)
    assert m["data"].size == 64 * O.row_bytes(t, 1024)
    assert (m["data"] == synth.matrix(t, 64, 1024, 21, std=0.02)["data"]).all()
    assert not (m["data"] == synth.matrix(t, 64, 1024, 22, std=0.02)["data"]).all()
    w = O.dequantize(t, m["data"], 64 * 1024)
    assert np.isfinite(w).all()
    assert 0.5 * 0.02 < w.std() < 2.0 * 0.02, w.std()


def test_q6_k_scales_take_both_signs_and_q4_k_uses_all_six_bits():
    w = synth.normal(64 * 256, 5, 0.02).reshape(64, 256)
    q6 = synth.quantize(w, synth.Q6_K).reshape(64, 210)
    sc = q6[:, 192:208].view(np.int8)
    assert (sc < 0).any() and (sc > 0).any()
    q4 = synth.quantize(w, synth.Q4_K).reshape(64, 144)
    assert (q4[:, 4:8] & 63).max() == 63


def test_model_tensors_have_the_gguf_names_and_q4_k_m_types():
    cfg = synth.CONFIGS["tiny"]
    t = synth.model_tensors(cfg, seed=1)
    assert t["blk.0.attn_v.weight"]["type"] == synth.Q6_K and t["output.weight"]["type"] == synth.Q6_K
    assert t["blk.1.ffn_down.weight"]["type"] == synth.Q4_K and t["token_embd.weight"]["type"] == synth.Q4_K
    assert t["blk.0.ffn_down.weight"]["in_dim"] == cfg["n_ff"] and t["blk.0.attn_k.weight"]["out_dim"] == cfg["n_head_kv"] * cfg["head_dim"]
    assert (t["blk.0.attn_norm.weight"]["data"] == 1).all()
