"""Parity of the fp32 glue operators (RMSNorm, RoPE, SwiGLU, attention, argmax) with the CPU oracle."""
import numpy as np
import pytest

import oracle as O
from gpu_common import assert_bit_equal, backend, bits  # noqa: F401
from orangu_b200 import synth
from refdata import xorshift32_kv

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n_tokens,dim", [(1, 256), (3, 2048), (5, 4096), (2, 8192)])
def test_rmsnorm(backend, n_tokens, dim):
    x = synth.normal(n_tokens * dim, 1, 2.0).reshape(n_tokens, dim)
    w = 1.0 + 0.1 * synth.normal(dim, 2)
    got = backend.rmsnorm(x, w, 1e-5)
    want = O.rmsnorm(x, w, 1e-5)
    # the sum of squares is a tree on the device and left-to-right on the CPU: a few ulp
    assert np.max(np.abs(got - want) / np.maximum(np.abs(want), 1e-6)) < 1e-5


@pytest.mark.parametrize("pos", [0, 1, 17, 1000, 8191])
@pytest.mark.parametrize("n_head,head_dim,rope_dim", [(4, 64, 64), (32, 128, 128), (2, 128, 64)])
def test_rope_is_bit_exact(backend, pos, n_head, head_dim, rope_dim):
    x = synth.normal(n_head * head_dim, pos + 1)
    got = backend.rope(x, n_head, head_dim, pos, rope_dim, 500000.0)
    want = O.rope_norm(x, n_head, head_dim, pos, rope_dim, 500000.0)
    assert_bit_equal(got, want, f"rope pos {pos}")


def test_swiglu(backend):
    g = synth.normal(14336, 3, 3.0)
    u = synth.normal(14336, 4, 3.0)
    g[:4] = [0.0, -0.0, 80.0, -80.0]
    got = backend.swiglu(g, u)
    want = O.swiglu(g, u)
    assert np.max(np.abs(got - want) / np.maximum(np.abs(want), 1e-6)) < 1e-5
    assert got[0] == 0.0 and np.isfinite(got).all()


def f16_round(a):
    return a.astype(np.float16).astype(np.float32)


@pytest.mark.parametrize("n_head,n_head_kv", [(8, 1), (8, 2), (4, 4), (6, 3), (1, 1), (32, 8)])
@pytest.mark.parametrize("head_dim", [16, 64, 128])
@pytest.mark.parametrize("n_pos", [1, 8, 40, 331])
def test_decode_attention_reference_shapes(backend, n_head, n_head_kv, head_dim, n_pos):
    seed = 0x12345678 ^ (n_head * 31 + head_dim)
    k, v = xorshift32_kv(n_pos, n_head_kv * head_dim, seed) if n_pos * n_head_kv * head_dim <= 40000 else (
        synth.normal(n_pos * n_head_kv * head_dim, 1).reshape(n_pos, -1), synth.normal(n_pos * n_head_kv * head_dim, 2).reshape(n_pos, -1))
    q = (((np.arange(n_head * head_dim) % 17).astype(np.float32) - 8.0) / 8.0).astype(np.float32)
    got = backend.attention_decode(q, k, v, n_head, n_head_kv, head_dim, 0.125)
    # the cache holds f16 (kv_cache.rs:26-32): the oracle attends over the rounded values
    want = O.attention(q, f16_round(k), f16_round(v), n_head, n_head_kv, head_dim, 0.125, 1, n_pos - 1)[0]
    assert np.abs(got - want).max() < 2e-5


def test_decode_attention_long_context_8b_shape(backend):
    n_pos, n_head, n_kv, hd = 4096 + 37, 32, 8, 128
    k = synth.normal(n_pos * n_kv * hd, 5).reshape(n_pos, -1)
    v = synth.normal(n_pos * n_kv * hd, 6).reshape(n_pos, -1)
    q = synth.normal(n_head * hd, 7)
    got = backend.attention_decode(q, k, v, n_head, n_kv, hd, 1.0 / np.sqrt(hd))
    want = O.attention(q, f16_round(k), f16_round(v), n_head, n_kv, hd, 1.0 / np.sqrt(hd), 1, n_pos - 1)[0]
    assert np.abs(got - want).max() < 2e-5


def test_argmax_tie_rule_and_penalty(backend):
    assert backend.argmax([1.0, 3.0, 3.0, 2.0]) == 2
    assert backend.argmax([0.0, -0.0]) == 0 and backend.argmax([-0.0, 0.0]) == 1
    assert backend.argmax([-np.inf, -np.inf]) == 1
    l = synth.normal(128256, 8)
    l[[5, 70000, 128255]] = l.max() + 1.0
    assert backend.argmax(l) == 128255 == O.argmax(l)
    recent = [128255, 70000, 70000, 3]
    assert backend.argmax(l, recent, 64, 1.3) == O.argmax(O.repeat_penalty(l, recent, 64, 1.3)) == 5
    assert backend.argmax(l, recent, 1, 1.3) == O.argmax(O.repeat_penalty(l, recent, 1, 1.3)) == 128255
    assert backend.argmax(l, recent, 64, 1.0) == 128255
