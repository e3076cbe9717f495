"""Parity of the quantized products with the CPU oracle, through the C ABI, on a B200.

Bars: block unpacking and integer partial sums bit-exact; per-row fp32 within 1e-3 of the term
magnitude (the kernels are built to match bit for bit, which is asserted where it holds by
construction: same quantized activations, same term order)."""
import numpy as np
import pytest

import oracle as O
from gpu_common import assert_bit_equal, backend, bits, rel_err  # noqa: F401
from orangu_b200 import QuantMatrix, MatmulOp, synth
from refdata import activations, fixture_bytes, fixture_row, k_fixture
from test_oracle_golden import adversarial_blocks

pytestmark = pytest.mark.gpu
Q8_0, Q4_K, Q5_K, Q6_K = 8, 12, 13, 14
TYPES = [Q8_0, Q4_K, Q5_K, Q6_K]


def gauss_matrix(t, out_dim, in_dim, seed):
    m = synth.matrix(t, out_dim, in_dim, seed)
    return QuantMatrix(m["data"], t, in_dim, out_dim)


def lcg_matrix(t, out_dim, in_dim, seed):
    raw, _ = k_fixture(t, in_dim, out_dim, 1, seed)
    return QuantMatrix(raw, t, in_dim, out_dim)


# ---- block unpacking ----------------------------------------------------------------------------
@pytest.mark.parametrize("t,count", [(Q8_0, 256), (Q4_K, 512), (Q6_K, 512)])
def test_device_dequantize_reproduces_the_reference_golden_checksums(backend, t, count):
    from refdata import bit_checksum

    golden = {Q8_0: 0xC5D58782F54E52E5, Q4_K: 0x9A7268A432A5C5FA, Q6_K: 0x61001D333CB0CFD1}
    bb, be = O.BLOCK[t]
    raw = fixture_bytes(count // be * bb)
    w = QuantMatrix(raw, t, count, 1)
    got = backend.row(w, 0)
    # NaN payloads may differ between f16 decoders (the reference pins that too); compare as the oracle does
    want = O.dequantize(t, raw, count)
    nan = np.isnan(want)
    assert (np.isnan(got[0]) == nan).all()
    assert (bits(got[0])[~nan] == bits(want)[~nan]).all()
    if not nan.any():
        assert bit_checksum(got[0]) == golden[t]


@pytest.mark.parametrize("t", TYPES)
@pytest.mark.parametrize("in_dim,out_dim", [(256, 5), (768, 7), (2048, 33), (4096, 16)])
def test_device_rows_equal_quantmatrix_row(backend, t, in_dim, out_dim):
    for w in (gauss_matrix(t, out_dim, in_dim, 3), lcg_matrix(t, out_dim, in_dim, 17)):
        got = backend.row(w, 0, out_dim)
        want = O.dequantize(t, w.raw, in_dim * out_dim).reshape(out_dim, in_dim)
        assert_bit_equal(got, want, f"type {t} [{out_dim}x{in_dim}]")
        assert_bit_equal(backend.row(w, out_dim - 1), want[-1:], "last row alone")


# ---- activation quantizer -------------------------------------------------------------------------
def test_activation_quantizer_bit_exact_including_adversarial_blocks(backend):
    rng = np.random.default_rng(0)
    x32 = np.concatenate(adversarial_blocks() + [rng.standard_normal(32 * 5).astype(np.float32)])
    q, d, s = backend.quantize_act(x32, per_256=False)
    wq, wd, ws = O.quantize_act(x32)
    assert (q == wq).all() and (bits(d) == bits(wd)).all() and (s == ws).all()
    x256 = np.concatenate(adversarial_blocks() + [rng.standard_normal(256 * 7 - 32 * 7).astype(np.float32) * 3])
    q, d, s = backend.quantize_act(x256, per_256=True)
    wq, wd, ws = O.quantize_act(x256, k_row=True)
    assert (q == wq).all() and (bits(d) == bits(wd)).all() and (s == ws).all()


# ---- integer partial sums -------------------------------------------------------------------------
@pytest.mark.parametrize("t", TYPES)
@pytest.mark.parametrize("in_dim", [256, 1792, 4096])
def test_integer_partial_sums_bit_exact(backend, t, in_dim):
    out_dim = 9
    for w, x in ((lcg_matrix(t, out_dim, in_dim, 5), activations(in_dim)),
                 (gauss_matrix(t, out_dim, in_dim, 6), synth.normal(in_dim, 99))):
        isum, imin = backend.matmul_partials(x, w)
        rb = w.row_bytes()
        for o in range(out_dim):
            wi, wm = O.row_partials(t, w.raw[o * rb:(o + 1) * rb], x)
            assert (isum[o] == wi).all(), f"isum row {o}"
            assert (imin[o] == wm).all(), f"imin row {o}"


# ---- GEMV ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("t", TYPES)
@pytest.mark.parametrize("in_dim,out_dim", [(256, 5), (256, 11), (512, 8), (2048, 64), (5632, 37)])
def test_gemv_equals_the_cpu_kernels_bit_for_bit(backend, t, in_dim, out_dim):
    for w, x in ((lcg_matrix(t, out_dim, in_dim, 1), activations(in_dim)),
                 (gauss_matrix(t, out_dim, in_dim, 2), synth.normal(in_dim, 7))):
        got = backend.matmul(x, 1, w)
        want = O.matmul(x, 1, w.raw, t, in_dim, out_dim)
        assert_bit_equal(got, want, f"gemv type {t} [{out_dim}x{in_dim}]")
        ref = O.matmul_dequant(x, 1, w.raw, t, in_dim, out_dim)
        mag = O.matmul_dequant(np.abs(x), 1, np.ascontiguousarray(w.raw), t, in_dim, out_dim)  # loose yardstick
        assert rel_err(got, ref, np.abs(mag).max()) < 0.02


def test_config_q8_0_gemv_4096(backend):
    """The single-GEMV case: 4096x4096 N(0, 0.02^2) weights in Q8_0, N(0,1) activations."""
    w = gauss_matrix(Q8_0, 4096, 4096, 1234)
    x = synth.normal(4096, 4321)
    got = backend.matmul(x, 1, w)
    want = O.matmul(x, 1, w.raw, Q8_0, 4096, 4096)
    assert_bit_equal(got, want, "Q8_0 4096x4096")
    deq = O.matmul_dequant(x, 1, w.raw, Q8_0, 4096, 4096)
    assert np.abs(got - deq).max() / np.abs(deq).max() < 0.01


@pytest.mark.parametrize("t", [Q4_K, Q6_K])
@pytest.mark.parametrize("out_dim,in_dim", [(4096, 4096), (14336, 4096), (4096, 14336)])
def test_sweep_shapes_batch_1_and_8(backend, t, out_dim, in_dim):
    w = gauss_matrix(t, out_dim, in_dim, 42)
    x = synth.normal(8 * in_dim, 43)
    assert_bit_equal(backend.matmul(x[:in_dim], 1, w), O.matmul(x[:in_dim], 1, w.raw, t, in_dim, out_dim), "batch 1")
    assert_bit_equal(backend.matmul_decode(x, 8, w), O.matmul_decode(x, 8, w.raw, t, in_dim, out_dim), "decode batch 8")
    assert_bit_equal(backend.matmul(x, 8, w), O.matmul(x, 8, w.raw, t, in_dim, out_dim), "prefill batch 8")


@pytest.mark.parametrize("t", [Q4_K, Q6_K])
def test_sweep_shape_batch_64(backend, t):
    out_dim, in_dim, n = 4096, 4096, 64
    w = gauss_matrix(t, out_dim, in_dim, 44)
    x = synth.normal(n * in_dim, 45)
    assert_bit_equal(backend.matmul(x, n, w), O.matmul(x, n, w.raw, t, in_dim, out_dim), "prefill batch 64")
    assert_bit_equal(backend.matmul_decode(x, n, w), O.matmul_decode(x, n, w.raw, t, in_dim, out_dim), "decode batch 64")


@pytest.mark.parametrize("t", [Q4_K, Q6_K])
@pytest.mark.parametrize("out_dim,in_dim", [(4096, 4096), (14336, 4096), (4096, 14336)])
def test_sweep_shapes_batch_512(backend, t, out_dim, in_dim):
    """The sweep's largest batch on all three shapes: the prefill GEMM (two-pass order for Q4_K) and, on a slice of the
    rows, the decode contract (every row equals the single-token kernel)."""
    n = 512
    w = gauss_matrix(t, out_dim, in_dim, 46)
    x = synth.normal(n * in_dim, 47)
    assert_bit_equal(backend.matmul(x, n, w), O.matmul(x, n, w.raw, t, in_dim, out_dim), f"prefill batch 512, type {t} [{out_dim}x{in_dim}]")
    got = np.asarray(backend.matmul_decode(x, n, w)).reshape(n, out_dim)
    for tok in (0, 255, 511):
        alone = O.matmul(x[tok * in_dim:(tok + 1) * in_dim], 1, w.raw, t, in_dim, out_dim)
        assert_bit_equal(got[tok], np.asarray(alone).reshape(-1), f"decode batch 512 row {tok}")


@pytest.mark.parametrize("n", [64, 512])
def test_q8_0_4096_batches_64_and_512(backend, n):
    """Q8_0 at many tokens: the flat GEMM (engine/vecdot.rs:2598-2629) and the decode batch, kernels backend/cpu.rs:76-90 picks."""
    out_dim = in_dim = 4096
    w = gauss_matrix(Q8_0, out_dim, in_dim, 48)
    x = synth.normal(n * in_dim, 49)
    assert_bit_equal(backend.matmul(x, n, w), O.matmul(x, n, w.raw, Q8_0, in_dim, out_dim), f"Q8_0 prefill batch {n}")
    assert_bit_equal(backend.matmul_decode(x, n, w), O.matmul_decode(x, n, w.raw, Q8_0, in_dim, out_dim), f"Q8_0 decode batch {n}")


# ---- decode batches and prefill ---------------------------------------------------------------------
@pytest.mark.parametrize("t", TYPES)
@pytest.mark.parametrize("out_dim", [5, 8, 11])
def test_decode_batch_row_equals_decoding_alone(backend, t, out_dim):
    in_dim, n = 256, 6
    raw, x = k_fixture(t, in_dim, out_dim, n, 31)
    w = QuantMatrix(raw, t, in_dim, out_dim)
    batch = backend.matmul_decode(x, n, w)
    for tok in range(n):
        alone = backend.matmul(x[tok * in_dim:(tok + 1) * in_dim], 1, w)
        assert_bit_equal(batch[tok:tok + 1], alone, f"token {tok}")
    assert_bit_equal(batch, O.matmul_decode(x, n, raw, t, in_dim, out_dim), "against the oracle")


@pytest.mark.parametrize("t", TYPES)
@pytest.mark.parametrize("in_dim", [256, 2048, 8192])
def test_prefill_gemm_reference_fixture_5_rows_7_tokens(backend, t, in_dim):
    out_dim, n = 5, 7
    raw, x = k_fixture(t, in_dim, out_dim, n, 4242)
    w = QuantMatrix(raw, t, in_dim, out_dim)
    got = backend.matmul(x, n, w)
    assert_bit_equal(got, O.matmul(x, n, raw, t, in_dim, out_dim), f"gemm type {t} in_dim {in_dim}")


@pytest.mark.parametrize("t", TYPES)
def test_prefill_result_is_independent_of_the_batch_size(backend, t):
    in_dim, out_dim = 512, 4
    raw, x = k_fixture(t, in_dim, out_dim, 19, 77)
    w = QuantMatrix(raw, t, in_dim, out_dim)
    full = backend.matmul(x, 19, w)
    for n in (2, 3, 5, 7, 9, 17):
        assert_bit_equal(backend.matmul(x[:n * in_dim], n, w), full[:n], f"{n} of 19 tokens")


def test_matmul_batch_is_the_same_as_separate_calls(backend):
    in_dim = 1024
    ws = [gauss_matrix(t, od, in_dim, 9 + i) for i, (t, od) in enumerate([(Q4_K, 40), (Q4_K, 16), (Q6_K, 16), (Q8_0, 12)])]
    x = synth.normal(3 * in_dim, 5)
    ops = [MatmulOp(x, 3, w) for w in ws]
    for got, w in zip(backend.matmul_batch(ops), ws):
        assert_bit_equal(got, backend.matmul(x, 3, w), "prefill op")
    for got, w in zip(backend.matmul_batch_decode(ops), ws):
        assert_bit_equal(got, backend.matmul_decode(x, 3, w), "decode op")
    out = np.zeros((3, 40), np.float32)
    backend.matmul_into(out, x, 3, ws[0])
    assert_bit_equal(out, backend.matmul(x, 3, ws[0]), "matmul_into")


def test_weight_slices_for_tensor_parallel(backend):
    """A row range and an input-column range of a matrix behave as the corresponding sub-matrix."""
    import ctypes as C
    from orangu_b200 import capi

    L = capi.load()
    for t in TYPES + SYM32:
        in_dim, out_dim = 2048, 24
        w = gauss_matrix(t, out_dim, in_dim, 77)
        x = synth.normal(in_dim, 3)
        h = C.c_void_p()
        capi.check(backend._h, L.ob_weight_register_slice(backend._h, w.raw.ctypes.data, w.row_bytes(), t, in_dim, out_dim, 8, 8, 512, 1024, C.byref(h)))
        y = np.empty((1, 8), np.float32)
        xs = np.ascontiguousarray(x[512:1536])
        capi.check(backend._h, L.ob_matmul(backend._h, xs.ctypes.data, 1, h, y.ctypes.data))
        L.ob_weight_release(backend._h, h)
        be = O.BLOCK[t][1]
        bb = O.BLOCK[t][0]
        rows = w.raw.reshape(out_dim, -1)[8:16]
        sub = np.ascontiguousarray(rows[:, (512 // be) * bb:(1536 // be) * bb])
        assert_bit_equal(y, O.matmul(xs, 1, sub, t, 1024, 8), f"slice type {t}")


# ---- Q4_0, Q5_0, IQ4_NL: per-32 symmetric types, unpacked at registration into the Q8_0 layout ------------
SYM32 = [2, 6, 20]
SYM32_GOLDEN = {2: 0x162325C968C10725, 6: 0x813F8949E12B3725, 20: 0x7956C82FEBA12125}  # E/quant.rs:1389-1420, 256 elements


@pytest.mark.parametrize("t", SYM32)
def test_per_32_symmetric_types_dequantize_to_the_reference_checksums(backend, t):
    from refdata import bit_checksum

    bb, be = O.BLOCK[t]
    raw = fixture_bytes(256 // be * bb)
    got = backend.row(QuantMatrix(raw, t, 256, 1), 0)
    want = O.dequantize(t, raw, 256)
    nan = np.isnan(want)
    assert (np.isnan(got[0]) == nan).all()
    assert (bits(got[0])[~nan] == bits(want)[~nan]).all()
    if not nan.any():
        assert bit_checksum(got[0]) == SYM32_GOLDEN[t]


@pytest.mark.parametrize("t", SYM32)
@pytest.mark.parametrize("in_dim,out_dim", [(32, 3), (896, 7), (4864, 33)])
def test_per_32_symmetric_rows_partials_and_gemv_are_bit_exact(backend, t, in_dim, out_dim):
    for w, x in ((lcg_matrix(t, out_dim, in_dim, 17), activations(in_dim)),
                 (gauss_matrix(t, out_dim, in_dim, 3), synth.normal(in_dim, 7))):
        want_rows = O.dequantize(t, w.raw, in_dim * out_dim).reshape(out_dim, in_dim)
        assert_bit_equal(backend.row(w, 0, out_dim), want_rows, f"rows, type {t}")
        isum, _ = backend.matmul_partials(x, w)
        rb = w.row_bytes()
        for o in range(out_dim):
            wi, _ = O.row_partials(t, w.raw[o * rb:(o + 1) * rb], x)
            assert (isum[o] == wi).all(), f"isum row {o}"
        assert_bit_equal(backend.matmul(x, 1, w), O.matmul(x, 1, w.raw, t, in_dim, out_dim), f"gemv type {t} [{out_dim}x{in_dim}]")


@pytest.mark.parametrize("t", SYM32)
def test_per_32_symmetric_batches_are_bit_exact(backend, t):
    in_dim, out_dim = 896, 37
    w = gauss_matrix(t, out_dim, in_dim, 21)
    for n in (2, 7, 64):
        x = synth.normal(n * in_dim, 40 + n)
        assert_bit_equal(backend.matmul(x, n, w), O.matmul(x, n, w.raw, t, in_dim, out_dim), f"prefill, {n} tokens")
        assert_bit_equal(backend.matmul_decode(x, n, w), O.matmul_decode(x, n, w.raw, t, in_dim, out_dim), f"decode batch, {n} rows")
    raw, x = k_fixture(t, 2048, 5, 7, 4242)  # the reference's 5-row, 7-token fixture shape
    assert_bit_equal(backend.matmul(x, 7, QuantMatrix(raw, t, 2048, 5)), O.matmul(x, 7, raw, t, 2048, 5), "fixture")


# ---- error behaviour ---------------------------------------------------------------------------------
def test_unsupported_and_invalid_inputs_are_statuses(backend):
    import ctypes as C
    from orangu_b200 import capi, OranguError

    L = capi.load()
    h = C.c_void_p()
    raw = np.zeros(144, np.uint8)
    assert L.ob_weight_register(backend._h, raw.ctypes.data, 84, 10, 256, 1, C.byref(h)) == -2  # Q2_K: no kernel
    assert b"ggml type 10" in L.ob_last_error(backend._h)
    assert L.ob_weight_register(backend._h, raw.ctypes.data, 100, 12, 256, 1, C.byref(h)) == -1  # wrong row_bytes
    assert L.ob_weight_register(backend._h, raw.ctypes.data, 144, 12, 200, 1, C.byref(h)) == -2  # not a block multiple
    w = gauss_matrix(Q4_K, 4, 256, 1)
    with pytest.raises(ValueError):
        backend.matmul(np.zeros(255, np.float32), 1, w)
    assert backend.matmul(np.zeros(0, np.float32), 0, w).shape == (0, 4)
    assert backend.supports_type(12) and backend.supports_type(13) and not backend.supports_type(10)
    assert backend.reduced_surface() is None
