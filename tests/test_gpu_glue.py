"""Parity of the fp32 glue operators (RMSNorm, RoPE, SwiGLU, attention, argmax) with the CPU oracle."""
import numpy as np
import pytest

import oracle as O
from gpu_common import assert_bit_equal, backend, bits  # noqa: F401
from orangu_b200 import synth
from refdata import xorshift32_kv

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n_tokens,dim", [(1, 256), (3, 2048), (5, 4096), (2, 8192), (1, 32), (2, 2080)])
def test_rmsnorm_is_bit_exact(backend, n_tokens, dim):
    """The squares are summed left to right on the CPU; the device reproduces that sum exactly."""
    x = synth.normal(n_tokens * dim, 1, 2.0).reshape(n_tokens, dim)
    w = 1.0 + 0.1 * synth.normal(dim, 2)
    assert_bit_equal(backend.rmsnorm(x, w, 1e-5), O.rmsnorm(x, w, 1e-5), f"rmsnorm [{n_tokens}x{dim}]")


def adversarial_rows(dim):
    rng = np.random.default_rng(dim)
    rows = []
    rows.append(np.zeros(dim, np.float32))
    r = np.zeros(dim, np.float32); r[dim // 2] = 3.0; rows.append(r)                       # one term, late
    rows.append(np.full(dim, 1.0, np.float32))                                              # exact integers, many binade crossings
    rows.append(np.full(dim, np.float32(2.0 ** -12), np.float32))                           # squares of 2^-24: ties against a sum near 1
    r = np.full(dim, np.float32(2.0 ** -12), np.float32); r[0] = 1.0; rows.append(r)        # every later term is exactly half an ulp... then less
    r = np.full(dim, np.float32(2.0 ** -11.5), np.float32); r[0] = 1.0; rows.append(r)
    rows.append((rng.standard_normal(dim) * np.exp(rng.standard_normal(dim) * 6)).astype(np.float32))  # 30 binades of range
    r = rng.standard_normal(dim).astype(np.float32); r[::7] = 0; r[5] = 1e18; rows.append(r)  # a huge early term
    r = rng.standard_normal(dim).astype(np.float32) * 1e-22; rows.append(r)                 # subnormal squares
    r = rng.standard_normal(dim).astype(np.float32); r[dim - 3] = 1e19; rows.append(r)       # overflow of the square to inf
    r = rng.standard_normal(dim).astype(np.float32); r[3] = np.nan; rows.append(r)
    r = np.sqrt(np.arange(dim, dtype=np.float32)); rows.append(r)                            # 0,1,2,3,.. as squares (rounded)
    for k in range(6):                                                                       # half-integers relative to the running ulp
        base = np.float32(2.0 ** (k - 3))
        r = np.full(dim, base, np.float32); r[1::2] *= np.float32(1.5); rows.append(r)
    return np.stack(rows)


@pytest.mark.parametrize("dim", [64, 512, 4096, 8192])
def test_rmsnorm_sequential_sum_adversarial(backend, dim):
    x = adversarial_rows(dim)
    w = np.ones(dim, np.float32)
    with np.errstate(all="ignore"):
        want = O.rmsnorm(x, w, 1e-5)
    got = backend.rmsnorm(x, w, 1e-5)
    nan = np.isnan(want)
    assert (np.isnan(got) == nan).all()
    assert (bits(got)[~nan] == bits(want)[~nan]).all()


@pytest.mark.parametrize("pos", [0, 1, 17, 1000, 8191])
@pytest.mark.parametrize("n_head,head_dim,rope_dim", [(4, 64, 64), (32, 128, 128), (2, 128, 64)])
def test_rope_is_bit_exact(backend, pos, n_head, head_dim, rope_dim):
    x = synth.normal(n_head * head_dim, pos + 1)
    got = backend.rope(x, n_head, head_dim, pos, rope_dim, 500000.0)
    want = O.rope_norm(x, n_head, head_dim, pos, rope_dim, 500000.0)
    assert_bit_equal(got, want, f"rope pos {pos}")


def test_swiglu_is_bit_exact(backend):
    g = synth.normal(14336, 3, 3.0)
    u = synth.normal(14336, 4, 3.0)
    g[:6] = [0.0, -0.0, 80.0, -80.0, 104.0, -104.0]
    got = backend.swiglu(g, u)
    assert_bit_equal(got, O.swiglu(g, u), "silu(g) * u")
    assert got[0] == 0.0 and np.isfinite(got).all()


def f16_round(a):
    return a.astype(np.float16).astype(np.float32)


def attention_case(n_head, n_head_kv, head_dim, n_pos):
    seed = 0x12345678 ^ (n_head * 31 + head_dim)
    n = n_pos * n_head_kv * head_dim
    if n <= 40000:
        k, v = xorshift32_kv(n_pos, n_head_kv * head_dim, seed)
    else:
        k, v = synth.normal(n, seed).reshape(n_pos, -1), synth.normal(n, seed + 1).reshape(n_pos, -1)
    q = (((np.arange(n_head * head_dim) % 17).astype(np.float32) - 8.0) / 8.0).astype(np.float32)
    # the cache holds f16 (kv_cache.rs:26-32): the oracle attends over the rounded values
    want = O.attention(q, f16_round(k), f16_round(v), n_head, n_head_kv, head_dim, 0.125, 1, n_pos - 1)[0]
    return q, k, v, want


@pytest.mark.parametrize("n_head,n_head_kv", [(8, 1), (8, 2), (4, 4), (6, 3), (1, 1), (32, 8)])
@pytest.mark.parametrize("head_dim", [16, 64, 128])
@pytest.mark.parametrize("n_pos", [1, 8, 40, 331])
def test_exact_order_attention_is_bit_exact(backend, n_head, n_head_kv, head_dim, n_pos):
    q, k, v, want = attention_case(n_head, n_head_kv, head_dim, n_pos)
    got = backend.attention_decode(q, k, v, n_head, n_head_kv, head_dim, 0.125, exact_order=True)
    assert_bit_equal(got, want, "exact-order attention")


@pytest.mark.parametrize("n_head,n_head_kv", [(8, 1), (8, 2), (4, 4), (6, 3), (1, 1), (32, 8)])
@pytest.mark.parametrize("head_dim", [16, 64, 128])
@pytest.mark.parametrize("n_pos", [1, 8, 40, 331])
def test_flash_decode_attention_within_rounding(backend, n_head, n_head_kv, head_dim, n_pos):
    q, k, v, want = attention_case(n_head, n_head_kv, head_dim, n_pos)
    got = backend.attention_decode(q, k, v, n_head, n_head_kv, head_dim, 0.125, exact_order=False)
    assert np.abs(got - want).max() < 2e-5


@pytest.mark.parametrize("n_head,n_head_kv", [(4, 4), (8, 4), (8, 2), (32, 8), (8, 1), (64, 8)])
@pytest.mark.parametrize("head_dim", [64, 128])
@pytest.mark.parametrize("n_pos", [1, 17, 40, 331, 1500])
@pytest.mark.parametrize("mode", [2, 3])
def test_fused_tensor_core_flash_decode_within_rounding(backend, n_head, n_head_kv, head_dim, n_pos, mode):
    """The one-kernel flash-decode: scores and outputs on the tensor cores with q and the probabilities split into two
    fp16 parts -- the result has to stay at fp32 rounding level, not fp16."""
    if n_head // n_head_kv == 1 and head_dim == 64:
        pytest.skip("one head of 64 dims per kv head is not a shape of the fused kernel")
    q, k, v, want = attention_case(n_head, n_head_kv, head_dim, n_pos)
    got = backend.attention_decode(q, k, v, n_head, n_head_kv, head_dim, 0.125, exact_order=mode)  # 3: CTAs of four warps
    assert np.abs(got - want).max() < 2e-5


def test_attention_long_context_8b_shape(backend):
    n_pos, n_head, n_kv, hd = 4096 + 37, 32, 8, 128
    k = synth.normal(n_pos * n_kv * hd, 5).reshape(n_pos, -1)
    v = synth.normal(n_pos * n_kv * hd, 6).reshape(n_pos, -1)
    q = synth.normal(n_head * hd, 7)
    scale = float(np.float32(1.0) / np.sqrt(np.float32(hd)))
    want = O.attention(q, f16_round(k), f16_round(v), n_head, n_kv, hd, scale, 1, n_pos - 1)[0]
    assert_bit_equal(backend.attention_decode(q, k, v, n_head, n_kv, hd, scale, exact_order=True), want, "exact order, 4133 positions")
    got = backend.attention_decode(q, k, v, n_head, n_kv, hd, scale, exact_order=False)
    assert np.abs(got - want).max() < 2e-5
    got = backend.attention_decode(q, k, v, n_head, n_kv, hd, scale, exact_order=2)
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
