"""Writes tests/golden/hotpath.npz: seeded inputs of every operator on the hot path with the CPU oracle's outputs.

Run from the repository root:  python tests/golden/make_golden.py
The oracle (oracle/orangu_oracle.cpp) is the CPU restatement of the reference's arithmetic and is itself pinned to the
reference's own known-answer tests by tests/test_oracle_golden.py; these vectors freeze its outputs so that the CUDA
path can be compared on a machine that has neither the oracle's build nor the reference tree, and so that a change of
the oracle that alters a bit shows up as a failing CPU test.  Small on purpose (a few hundred KB)."""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import oracle as O  # noqa: E402
from orangu_b200 import synth  # noqa: E402


def main():
    rng = np.random.default_rng(20240607)
    out = {}
    # products: 6 rows x 512 (Q8_0: 16 blocks of 32; K types: 2 super-blocks), 3 tokens
    for t in (8, 12, 14):
        m = synth.matrix(t, 6, 512, seed=1000 + t)
        x = rng.standard_normal((3, 512)).astype(np.float32)
        out[f"mm{t}_w"], out[f"mm{t}_x"] = m["data"], x
        out[f"mm{t}_decode"] = O.matmul_decode(x, 3, m["data"], t, 512, 6)
        out[f"mm{t}_prefill"] = O.matmul(x, 3, m["data"], t, 512, 6)
        out[f"mm{t}_dequant"] = O.dequantize(t, m["data"], 6 * 512)
    # activation quantizers
    xq = (rng.standard_normal(512) * np.repeat(rng.uniform(0.01, 30.0, 16), 32)).astype(np.float32)
    out["q_x"] = xq
    for k in (False, True):
        q, d, s = O.quantize_act(xq, k)
        out[f"q{int(k)}_q"], out[f"q{int(k)}_d"], out[f"q{int(k)}_s"] = q, d, s
    # glue
    xn, wn = rng.standard_normal((2, 256)).astype(np.float32), rng.uniform(0.5, 1.5, 256).astype(np.float32)
    out["norm_x"], out["norm_w"], out["norm_y"] = xn, wn, O.rmsnorm(xn, wn, 1e-5)
    xr = rng.standard_normal(4 * 64).astype(np.float32)
    out["rope_x"], out["rope_y"] = xr, O.rope_norm(xr, 4, 64, 37, 64, 500000.0)
    g, u = rng.standard_normal(300).astype(np.float32) * 4, rng.standard_normal(300).astype(np.float32)
    out["swiglu_g"], out["swiglu_u"], out["swiglu_y"] = g, u, O.swiglu(g, u)
    # attention: 4 heads over 2 kv heads, head_dim 64, one query at position 40 (41 keys), f16-exact K/V
    q = rng.standard_normal(4 * 64).astype(np.float32)
    k = rng.standard_normal((41, 2 * 64)).astype(np.float16).astype(np.float32)
    v = rng.standard_normal((41, 2 * 64)).astype(np.float16).astype(np.float32)
    out["att_q"], out["att_k"], out["att_v"] = q, k, v
    out["att_y"] = O.attention(q, k, v, 4, 2, 64, 0.125, 1, 40)
    # the tiny model: 9-token prefill, then 3 greedy steps
    cfg = dict(synth.CONFIGS["tiny"])
    tensors = synth.model_tensors(cfg, seed=77)
    ref = O.Model(cfg, tensors)
    kv = ref.new_kv(32, f16=True)
    toks = rng.integers(0, cfg["n_vocab"], 9).astype(np.uint32)
    logits = [ref.forward(kv, toks, 0)]
    steps = [O.argmax(logits[0])]
    for i in range(3):
        logits.append(ref.forward(kv, [steps[-1]], 9 + i))
        steps.append(O.argmax(logits[-1]))
    out["model_tokens"], out["model_logits"], out["model_greedy"] = toks, np.stack(logits), np.array(steps, np.uint32)
    # (new vectors are appended below so that the random stream of the ones above never changes)
    # Q5_K products, as the K types above
    m = synth.matrix(13, 6, 512, seed=1013)
    x = rng.standard_normal((3, 512)).astype(np.float32)
    out["mm13_w"], out["mm13_x"] = m["data"], x
    out["mm13_decode"] = O.matmul_decode(x, 3, m["data"], 13, 512, 6)
    out["mm13_prefill"] = O.matmul(x, 3, m["data"], 13, 512, 6)
    out["mm13_dequant"] = O.dequantize(13, m["data"], 6 * 512)
    # rotation with the NEOX pairing and frequency factors
    xr2 = rng.standard_normal(4 * 64).astype(np.float32)
    ff = np.linspace(1.0, 8.0, 16).astype(np.float32)
    out["rope2_x"], out["rope2_ff"], out["rope2_y"] = xr2, ff, O.rope_layout(xr2, 4, 64, 23, 32, 10000.0, True, ff)
    # the tiny model as a Qwen3-style file would have it: q/k/v bias, per-head q/k norm, NEOX pairing
    qcfg = dict(synth.CONFIGS["tiny"], rope_neox=True)
    qt = synth.add_qwen_extras(qcfg, synth.model_tensors(qcfg, seed=78), seed=79)
    qref = O.Model(qcfg, qt)
    qkv = qref.new_kv(32, f16=True)
    qtoks = rng.integers(0, qcfg["n_vocab"], 11).astype(np.uint32)
    qlogits = [qref.forward(qkv, qtoks, 0)]
    qsteps = [O.argmax(qlogits[0])]
    for i in range(3):
        qlogits.append(qref.forward(qkv, [qsteps[-1]], 11 + i))
        qsteps.append(O.argmax(qlogits[-1]))
    out["qmodel_tokens"], out["qmodel_logits"], out["qmodel_greedy"] = qtoks, np.stack(qlogits), np.array(qsteps, np.uint32)
    np.savez_compressed(os.path.join(HERE, "hotpath.npz"), **out)
    print("wrote", os.path.join(HERE, "hotpath.npz"), os.path.getsize(os.path.join(HERE, "hotpath.npz")), "bytes")


if __name__ == "__main__":
    main()
