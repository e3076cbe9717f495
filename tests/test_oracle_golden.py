"""Pins the CPU oracle to the reference's own known-answer tests.

Each test restates the *inputs and expected answers* of a test the reference
carries in its sources (cited per test; E = src/bin/orangu-server/engine in
the reference tree) and checks the oracle against them.  None of this needs a
GPU or the reference tree at run time.
"""
import numpy as np
import pytest

import oracle as O
from refdata import activations, fixture_bytes, bit_checksum, fixture_row, k_fixture, pseudo_bytes, xorshift32_kv

Q8_0, Q4_K, Q6_K = O.Q8_0, O.Q4_K, O.Q6_K
Q4_0, Q5_0, IQ4_NL = O.Q4_0, O.Q5_0, O.IQ4_NL
Q5_K = O.Q5_K


# ---- E/quant.rs:1389-1463 -------------------------------------------------
GOLDEN = [
    (O.F32, 64, 0x1EB2_B799_2AE6_E834),
    (Q8_0, 256, 0xC5D5_8782_F54E_52E5),
    (Q4_0, 256, 0x1623_25C9_68C1_0725),
    (Q5_0, 256, 0x813F_8949_E12B_3725),
    (IQ4_NL, 256, 0x7956_C82F_EBA1_2125),
    (Q4_K, 512, 0x9A72_68A4_32A5_C5FA),
    (Q5_K, 512, 0x41C7_0B9B_E169_6E6D),
    (Q6_K, 512, 0x6100_1D33_3CB0_CFD1),
]


@pytest.mark.parametrize("t,count,expected", GOLDEN)
def test_dequantize_golden_checksums(t, count, expected):
    bb, be = O.BLOCK[t]
    raw = fixture_bytes(count // be * bb)
    values = O.dequantize(t, raw, count)
    assert values.size == count
    assert bit_checksum(values) == expected


# ---- E/quant.rs:1671-1690 -------------------------------------------------
def test_f16_decode_matches_ieee_for_every_non_nan_input():
    bits = np.arange(65536, dtype=np.uint16)
    want = bits.view(np.float16).astype(np.float32)
    got = np.array([O.lib().oref_f16_to_f32(int(b)) for b in bits], dtype=np.float32)
    nan = np.isnan(want)
    assert nan.sum() == 2046  # every NaN payload of binary16
    assert np.isnan(got[nan]).all()
    assert (got[~nan].view(np.uint32) == want[~nan].view(np.uint32)).all()


def test_f32_to_f16_is_round_to_nearest_even():
    rng = np.random.default_rng(5)
    vals = np.concatenate([
        rng.standard_normal(4000).astype(np.float32) * 3,
        rng.standard_normal(2000).astype(np.float32) * 1e-6,
        np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e9, -1e9, 2.0**-24, 2.0**-25, 2.0**-25 * 1.0001, 6.1e-5, np.inf, -np.inf], np.float32),
        (np.arange(2048, dtype=np.float32) + 0.5) * np.float32(2.0**-10),  # exact ties
    ])
    want = vals.astype(np.float16).view(np.uint16)
    got = np.array([O.f32_to_f16_bits(v) for v in vals], dtype=np.uint16)
    assert (got == want).all()


# ---- E/quant.rs:1845-1929 -------------------------------------------------
def test_q4_k_scale_unpacking_known_block():
    one = np.array([1.0], np.float16).view(np.uint8)
    zero = np.array([0.0], np.float16).view(np.uint8)
    block = np.concatenate([one, zero, np.array([1, 1, 1, 1, 0, 0, 0, 0, 1, 1, 1, 1], np.uint8), np.full(128, 0x55, np.uint8)])
    assert (O.dequantize(Q4_K, block, 256) == 5.0).all()


@pytest.mark.parametrize("scale_byte,want", [(2, -64.0), (0xFE, 64.0)])
def test_q6_k_zero_quant_and_signed_scales(scale_byte, want):
    block = np.concatenate([np.zeros(128 + 64, np.uint8), np.full(16, scale_byte, np.uint8), np.array([1.0], np.float16).view(np.uint8)])
    assert (O.dequantize(Q6_K, block, 256) == want).all()


def test_get_scale_min_k4_all_twelve_byte_patterns():
    rng = np.random.default_rng(0)
    for _ in range(200):
        s = rng.integers(0, 256, 12, dtype=np.uint8)
        for j in range(8):
            sc = np.zeros(1, np.uint8)
            m = np.zeros(1, np.uint8)
            O.lib().oref_get_scale_min_k4(j, s.ctypes.data, sc.ctypes.data, m.ctypes.data)
            if j < 4:
                want = (s[j] & 63, s[j + 4] & 63)
            else:
                want = ((s[j + 4] & 0xF) | ((s[j - 4] >> 6) << 4), (s[j + 4] >> 4) | ((s[j] >> 6) << 4))
            assert (int(sc[0]), int(m[0])) == (int(want[0]), int(want[1]))


# ---- E/vecdot.rs:4259-4264, 4395-4410, 4274-4344 --------------------------
def test_activation_quantizer_all_zero_block():
    q, d, s = O.quantize_act(np.zeros(64, np.float32))
    assert not d.any() and not q.any() and not s.any()


def test_activation_quantizer_rounds_ties_away_from_zero():
    x = np.full(32, 254.0, np.float32)
    x[1:5] = [1.0, 3.0, -1.0, -3.0]
    q, d, _ = O.quantize_act(x)
    assert list(q[1:5]) == [1, 2, -1, -2]
    assert d[0] == np.float32(2.0)


def adversarial_blocks():
    blocks = [np.zeros(32, np.float32)]
    ties = np.full(32, 254.0, np.float32)
    below_half = np.nextafter(np.float32(0.5), np.float32(0.0))
    for i in range(1, 32):
        ties[i] = {1: 1.0, 2: -1.0, 3: 3.0, 4: -3.0, 5: 2.0 * below_half, 6: -2.0 * below_half}.get(i % 8, 5.0)
    blocks.append(ties)
    tiny = np.full(32, np.finfo(np.float32).tiny, np.float32)
    tiny[0] = 1.0e30
    tiny[7] = -np.float32(1e-45)
    tiny[9] = np.float32(1e-45)
    blocks.append(tiny)
    nans = np.full(32, 4.0, np.float32)
    nans[[0, 3, 31]] = [np.nan, -np.nan, np.nan]
    blocks.append(nans)
    infs = np.ones(32, np.float32)
    infs[5], infs[6] = np.inf, -np.inf
    blocks.append(infs)
    neg = np.full(32, 0.25, np.float32)
    neg[13], neg[20] = -100.0, -60.0
    blocks.append(neg)
    lcg = 0x12345678
    spread = np.zeros(32, np.float32)
    for i in range(32):
        lcg = (lcg * 1664525 + 1013904223) & 0xFFFFFFFF
        spread[i] = np.float32(np.float32(lcg >> 8) / np.float32(8388608.0)) - np.float32(0.5)
    spread[0], spread[1] = 1.0, -1.0
    blocks.append(spread)
    return blocks


def quantize_block_written_out(x):
    """f32::max / round / clamp / `as i8`, one value at a time, in numpy float32."""
    amax = np.float32(0.0)
    for v in x:
        a = np.abs(v)
        if not np.isnan(a) and a > amax:
            amax = a
    with np.errstate(all="ignore"):
        scale = np.float32(amax / np.float32(127.0))
        inv = np.float32(1.0) / scale if scale > 0 else np.float32(0.0)
        q = []
        for v in x:
            y = np.float32(v * inv)
            if np.isnan(y):
                q.append(0)
                continue
            r = np.float32(np.trunc(y + np.copysign(np.float32(0.5), y))) if abs(y) < 8388608.0 else y
            # |y| + 0.5 can round up across an integer for the value just below 0.5
            if abs(y) < 0.5:
                r = np.float32(0.0)
            q.append(int(max(-127.0, min(127.0, float(r)))))
    return scale, np.array(q, np.int8)


def test_activation_quantizer_adversarial_blocks():
    blocks = adversarial_blocks()
    x = np.concatenate(blocks)
    q, d, sums = O.quantize_act(x)
    for b, blk in enumerate(blocks):
        scale, want = quantize_block_written_out(blk)
        assert d[b].view(np.uint32) == scale.view(np.uint32), f"block {b} scale"
        assert (q[b * 32:(b + 1) * 32] == want).all(), f"block {b}"
        assert sums[2 * b] == int(want[:16].astype(np.int32).sum()) and sums[2 * b + 1] == int(want[16:].astype(np.int32).sum())
    # spelled-out expectations from the reference's comments
    assert list(q[32 + 1:32 + 8]) == [1, -1, 2, -2, 0, 0, 3]
    assert q[3 * 32] == 0 and q[3 * 32 + 3] == 0 and d[3] == np.float32(4.0 / 127.0)
    assert not q[4 * 32:5 * 32].any() and np.isinf(d[4])
    assert q[5 * 32 + 13] == -127


def test_k_row_quantizer_matches_per_256_rule():
    rng = np.random.default_rng(3)
    x = rng.standard_normal(1024).astype(np.float32)
    q, d, sums = O.quantize_act(x, k_row=True)
    for s in range(4):
        blk = x[s * 256:(s + 1) * 256]
        scale = np.float32(np.abs(blk).max() / np.float32(127.0))
        inv = np.float32(1.0) / scale
        y = blk * inv
        want = np.clip(np.trunc(y + np.copysign(np.float32(0.5), y)), -127, 127).astype(np.int8)
        assert d[s] == scale
        assert (q[s * 256:(s + 1) * 256] == want).all()
        assert (sums[s * 16:(s + 1) * 16] == want.reshape(16, 16).astype(np.int32).sum(1)).all()


# ---- E/vecdot.rs:3436-3526 (check) and 4011-4040 (k-row) ------------------
def dequant_reference(t, row, x):
    w = O.dequantize(t, row, x.size).astype(np.float64)
    terms = w * x.astype(np.float64)
    return terms.sum(), np.abs(terms).sum()


@pytest.mark.parametrize("in_dim", [32, 256, 896, 4096])
@pytest.mark.parametrize("seed", [1, 7, 99])
def test_q8_0_gemv_within_int8_budget(in_dim, seed):
    row = fixture_row(Q8_0, in_dim, seed)
    x = activations(in_dim)
    ref, mag = dequant_reference(Q8_0, row, x)
    got = O.dot_row(Q8_0, row, x)
    assert abs(got - ref) <= 0.01 * max(mag, 1e-6)


# E/vecdot.rs:4176-4180 (Q4_0), :3854 (Q5_0), :3891 (IQ4_NL) run the same check on the per-32 symmetric types
@pytest.mark.parametrize("t", [Q4_0, Q5_0, IQ4_NL])
@pytest.mark.parametrize("in_dim", [32, 896, 4864])
@pytest.mark.parametrize("seed", [1, 7, 99])
def test_per_32_symmetric_gemv_within_int8_budget(t, in_dim, seed):
    row = fixture_row(t, in_dim, seed)
    x = activations(in_dim)
    ref, mag = dequant_reference(t, row, x)
    got = O.dot_row(t, row, x)
    assert abs(got - ref) <= 0.01 * max(mag, 1e-6)


# E/vecdot.rs:4226-4235: an all-zero Q4_0 payload unpacks to -8 everywhere (its own zero point, not Q5_0's -16)
def test_q4_0_zero_payload_is_minus_eight():
    block = np.zeros(18, np.uint8)
    block[0:2] = np.frombuffer(np.float16(1.0).tobytes(), np.uint8)
    assert (O.dequantize(Q4_0, block, 32) == -8.0).all()
    q5 = np.zeros(22, np.uint8)
    q5[0:2] = block[0:2]
    assert (O.dequantize(Q5_0, q5, 32) == -16.0).all()


def test_per_32_symmetric_types_equal_q8_0_on_the_unpacked_codes():
    """Their dot is the Q8_0 loop over the unpacked codes (E/vecdot.rs:2842-2881), so a Q8_0 row holding those codes
    must give the same bits, single token and batched."""
    x1 = activations(896)
    xb = activations(896 * 5).reshape(5, 896)
    for t in (Q4_0, Q5_0, IQ4_NL):
        raw = fixture_row(t, 896 * 6, 3)  # six rows
        codes = O.dequantize(t, raw, 896 * 6) / np.float32(0.125)
        assert (codes == np.round(codes)).all() and np.abs(codes).max() <= 127
        as_q8 = np.zeros((896 * 6 // 32, 34), np.uint8)
        as_q8[:, 0:2] = [0x00, 0x30]
        as_q8[:, 2:] = codes.astype(np.int8).view(np.uint8).reshape(-1, 32)
        for x in (x1, xb):
            n_tok = 1 if x.ndim == 1 else x.shape[0]
            a = O.matmul(x, n_tok, raw, t, 896, 6)
            b = O.matmul(x, n_tok, as_q8.reshape(-1), Q8_0, 896, 6)
            assert a.tobytes() == b.tobytes()


@pytest.mark.parametrize("t", [Q4_K, Q6_K])
@pytest.mark.parametrize("in_dim", [256, 2048, 5632])
@pytest.mark.parametrize("seed", [1, 7, 99])
def test_k_row_gemv_within_int8_budget(t, in_dim, seed):
    row = fixture_row(t, in_dim, seed)
    x = activations(in_dim)
    ref, mag = dequant_reference(t, row, x)
    got = O.dot_row(t, row, x)
    assert abs(got - ref) <= 0.02 * max(mag, 1e-6)


def test_row_partials_reassemble_to_the_row_total():
    """isum/imin are what the fp32 epilogue consumes: rebuilding the total from them must
    reproduce the GEMV bit for bit (E/vecdot.rs:3176, 3238, 2835)."""
    x = activations(2048)
    for t in (Q4_K, Q6_K, Q8_0):
        row = fixture_row(t, 2048, 5)
        isum, imin = O.row_partials(t, row, x)
        bb = O.BLOCK[t][0]
        blocks = row.reshape(-1, bb)
        total = np.float32(0)
        if t == Q8_0:
            _, d, _ = O.quantize_act(x)
            for b in range(len(blocks)):
                dw = blocks[b, :2].view(np.float16).astype(np.float32)[0]
                total = np.float32(total + np.float32(np.float32(dw * d[b]) * np.float32(isum[b])))
        else:
            _, d, _ = O.quantize_act(x, True)
            for s in range(len(blocks)):
                if t == Q4_K:
                    dd = blocks[s, 0:2].view(np.float16).astype(np.float32)[0]
                    dm = blocks[s, 2:4].view(np.float16).astype(np.float32)[0]
                    inner = np.float32(np.float32(dd * np.float32(isum[s])) - np.float32(dm * np.float32(imin[s])))
                    total = np.float32(total + np.float32(d[s] * inner))
                else:
                    dd = blocks[s, 208:210].view(np.float16).astype(np.float32)[0]
                    total = np.float32(total + np.float32(np.float32(d[s] * dd) * np.float32(isum[s])))
        assert np.float32(O.dot_row(t, row, x)).view(np.uint32) == total.view(np.uint32)


# ---- Q5_K (oracle only so far): E/quant.rs:1872-1888, E/vecdot.rs:4127-4133, 4141-4166 ----------------------
def q5_k_high_bit_block():
    block = np.zeros(176, np.uint8)
    block[0:2] = np.frombuffer(np.float16(1.0).tobytes(), np.uint8)  # d = 1, dmin = 0
    block[4:16] = [1, 1, 1, 1, 0, 0, 0, 0, 1, 1, 1, 1]                # every scale 1, every min 0
    block[16:48] = 0xFF                                               # qh: every high bit set; qs: every nibble 0
    return block


def test_q5_k_high_bit_reaches_every_sub_block():
    block = q5_k_high_bit_block()
    assert (O.dequantize(Q5_K, block, 256) == 16.0).all()
    # decode and batched forms see the same codes: with x = 1 everywhere a row sums 256 * 16 * (quantized 1.0)
    x = np.ones(256, np.float32)
    one = O.matmul(x, 1, block, Q5_K, 256, 1)[0, 0]
    many = O.matmul(np.tile(x, 5), 5, block, Q5_K, 256, 1)[:, 0]
    assert abs(one - 4096.0) < 1e-2 and (np.abs(many - 4096.0) < 1e-2).all()


@pytest.mark.parametrize("in_dim", [256, 3072, 4864])
@pytest.mark.parametrize("seed", [1, 7, 99])
def test_q5_k_gemv_within_int8_budget(in_dim, seed):
    row = fixture_row(Q5_K, in_dim, seed)
    x = activations(in_dim)
    ref, mag = dequant_reference(Q5_K, row, x)
    got = O.dot_row(Q5_K, row, x)
    assert abs(got - ref) <= 0.02 * max(mag, 1e-6)
    isum, imin = O.row_partials(Q5_K, row, x)
    assert isum.size == in_dim // 256 and imin.size == in_dim // 256


# ---- E/vecdot.rs:4416-4549 -------------------------------------------------
@pytest.mark.parametrize("t", [Q4_K, Q6_K, Q5_K])
@pytest.mark.parametrize("in_dim", [256, 2048, 8192])
def test_k_gemm_matches_dequantize_reference(t, in_dim):
    out_dim, n_tokens = 5, 7
    raw, x = k_fixture(t, in_dim, out_dim, n_tokens, 4242)
    got = O.matmul(x, n_tokens, raw, t, in_dim, out_dim)
    rb = O.row_bytes(t, in_dim)
    for o in range(out_dim):
        for tok in range(n_tokens):
            ref, mag = dequant_reference(t, raw[o * rb:(o + 1) * rb], x[tok * in_dim:(tok + 1) * in_dim])
            assert abs(got[tok, o] - ref) <= 0.01 * max(mag, 1e-6)


@pytest.mark.parametrize("t", [Q4_K, Q6_K, Q8_0])
def test_gemm_result_is_independent_of_the_batch_size(t):
    in_dim, out_dim = 512, 4
    raw, x = k_fixture(t, in_dim, out_dim, 8, 77)
    full = O.matmul(x, 8, raw, t, in_dim, out_dim)
    for n in (2, 3, 5, 7):
        part = O.matmul(x[:n * in_dim], n, raw, t, in_dim, out_dim)
        assert (part.view(np.uint32) == full[:n].view(np.uint32)).all()


# ---- E/backend/cpu.rs:543-650 ----------------------------------------------
@pytest.mark.parametrize("t", [Q4_K, Q6_K, Q8_0])
@pytest.mark.parametrize("out_dim", [5, 8, 11])
def test_decode_batch_row_equals_decoding_alone(t, out_dim):
    in_dim, n = 256, 6
    raw, x = k_fixture(t, in_dim, out_dim, n, 31)
    batch = O.matmul_decode(x, n, raw, t, in_dim, out_dim)
    for tok in range(n):
        alone = O.matmul(x[tok * in_dim:(tok + 1) * in_dim], 1, raw, t, in_dim, out_dim)
        assert (alone.view(np.uint32) == batch[tok:tok + 1].view(np.uint32)).all()


def test_prefill_and_decode_forms_agree_to_rounding():
    """Same integers, different fp32 order (E/vecdot.rs:3500-3507 holds them to 1e-3 of the terms)."""
    for t in (Q4_K, Q6_K, Q8_0):
        in_dim, out_dim, n = 2048, 6, 5
        raw, x = k_fixture(t, in_dim, out_dim, n, 9)
        a = O.matmul(x, n, raw, t, in_dim, out_dim)
        b = O.matmul_decode(x, n, raw, t, in_dim, out_dim)
        mag = np.abs(O.matmul_dequant(np.abs(x), n, raw, t, in_dim, out_dim)).max()
        assert np.abs(a - b).max() <= 1e-3 * mag
        if t == Q8_0:  # per-32 on both sides and the same order: identical
            assert (a.view(np.uint32) == b.view(np.uint32)).all()


# ---- E/tensor.rs:1596-1609, 1667-1782 ---------------------------------------
def test_softmax_structure_max_subtract_left_to_right_sum_one_divide():
    """expf may differ from a correctly rounded exp by an ulp, so the exponentials are taken
    from the oracle's own output scale and the structure around them is checked exactly."""
    rng = np.random.default_rng(1)
    for n in (1, 2, 7, 64, 257):
        row = (rng.standard_normal(n) * 4).astype(np.float32)
        got = O.softmax(row)
        e = np.exp((row - row.max()).astype(np.float64))
        want = e / e.sum()
        assert np.abs(got - want).max() < 1e-6
        assert abs(float(got.astype(np.float64).sum()) - 1.0) < 1e-5
        assert got[np.argmax(row)] == got.max()
    # all -inf but one: the finite one takes everything
    assert list(O.softmax(np.array([-np.inf, 2.0, -np.inf], np.float32))) == [0.0, 1.0, 0.0]


def test_rope_identity_at_position_zero_and_norm_preservation():
    rng = np.random.default_rng(2)
    x = rng.standard_normal(4 * 64).astype(np.float32)
    assert (O.rope_norm(x, 4, 64, 0, 64, 10000.0) == x).all()
    y = O.rope_norm(x, 4, 64, 17, 64, 500000.0)
    assert np.allclose((y.reshape(-1, 2) ** 2).sum(1), (x.reshape(-1, 2) ** 2).sum(1), rtol=1e-5)
    # NORM pairing rotates (2i, 2i+1): rotating a vector with only element 0 set touches 0 and 1 only
    e = np.zeros(64, np.float32)
    e[0] = 1
    z = O.rope_norm(e, 1, 64, 3, 64, 10000.0)
    assert z[0] != 1 and z[1] != 0 and not z[2:].any()
    tab = O.rope_table(20, 64, 500000.0)
    a, b = x.reshape(4, 32, 2)[..., 0], x.reshape(4, 32, 2)[..., 1]
    sn, cs = tab[17, :, 0], tab[17, :, 1]
    want = np.stack([a * cs - b * sn, a * sn + b * cs], -1).reshape(-1)
    assert (want.view(np.uint32) == y.view(np.uint32)).all()


def test_rope_layouts_as_the_reference_tests_state_them():
    """tensor.rs:1731-1783 (rope_neox_layout_rotates_pairs_offset_by_half, rope_norm_layout_rotates_consecutive_pairs),
    :1785-1823 (rope_freq_factors_divide_the_rotation_frequency), :1825-1842 (rope_layouts_preserve_total_energy)."""
    x = np.arange(1, 9, dtype=np.float32)
    theta = [np.float32(3.0) * np.float32(np.float32(10000.0) ** np.float32(-2.0 * p / 8.0)) for p in range(4)]
    neox, norm = O.rope_layout(x, 1, 8, 3, 8, 10000.0, True), O.rope_layout(x, 1, 8, 3, 8, 10000.0, False)
    want_neox, want_norm = x.copy(), x.copy()
    for p in range(4):
        sn, cs = np.float32(np.sin(theta[p])), np.float32(np.cos(theta[p]))
        a, b = want_neox[p], want_neox[p + 4]
        want_neox[p], want_neox[p + 4] = a * cs - b * sn, a * sn + b * cs
        a, b = want_norm[2 * p], want_norm[2 * p + 1]
        want_norm[2 * p], want_norm[2 * p + 1] = a * cs - b * sn, a * sn + b * cs
    assert np.abs(neox - want_neox).max() < 1e-6 and np.abs(norm - want_norm).max() < 1e-6
    assert (neox != norm).any(), "NORM and NEOX must not coincide"
    assert (norm.view(np.uint32) == O.rope_norm(x, 1, 8, 3, 8, 10000.0).view(np.uint32)).all()
    # a factor of 32 on pair 0 rotates it 32 times slower: the angle of (1, 0) after rotation is theta / 32
    e = np.zeros(8, np.float32)
    e[0] = 1
    ff = np.array([32.0, 1.0, 1.0, 1.0], np.float32)
    for is_neox, hi in ((True, 4), (False, 1)):
        plain, slowed = O.rope_layout(e, 1, 8, 5, 8, 10000.0, is_neox), O.rope_layout(e, 1, 8, 5, 8, 10000.0, is_neox, ff)
        ang_plain, ang_slow = np.arctan2(plain[hi], plain[0]), np.arctan2(slowed[hi], slowed[0])
        assert abs(ang_slow * 32 - (ang_plain % (2 * np.pi))) < 1e-4 or abs(ang_slow * 32 - 5.0) < 1e-4
    rng = np.random.default_rng(6)
    y = rng.standard_normal(3 * 16).astype(np.float32)
    for is_neox in (True, False):
        r = O.rope_layout(y, 3, 16, 11, 8, 10000.0, is_neox)  # rope_dim < head_dim: the tail of every head is left alone
        assert abs(float((r.astype(np.float64) ** 2).sum()) - float((y.astype(np.float64) ** 2).sum())) < 1e-4
        assert (r.reshape(3, 16)[:, 8:] == y.reshape(3, 16)[:, 8:]).all()


def test_rmsnorm_written_out():
    rng = np.random.default_rng(4)
    x = rng.standard_normal((3, 96)).astype(np.float32)
    w = rng.standard_normal(96).astype(np.float32)
    got = O.rmsnorm(x, w, 1e-5)
    for t in range(3):
        s = np.float32(0)
        for v in x[t]:
            s = np.float32(s + np.float32(v * v))
        scale = np.float32(1.0) / np.sqrt(np.float32(np.float32(s / np.float32(96)) + np.float32(1e-5)))
        want = (x[t] * scale) * w
        assert (want.view(np.uint32) == got[t].view(np.uint32)).all()


# ---- E/attention.rs:725-851 --------------------------------------------------
@pytest.mark.parametrize("n_head,n_head_kv", [(8, 1), (8, 2), (4, 4), (6, 3), (1, 1)])
@pytest.mark.parametrize("head_dim", [16, 64, 128])
@pytest.mark.parametrize("n_tokens", [1, 5, 33])
def test_attention_against_an_independent_float64_form(n_head, n_head_kv, head_dim, n_tokens):
    seed = 0x12345678 ^ (n_head * 31 + head_dim)
    n_pos = n_tokens + 7
    k, v = xorshift32_kv(n_pos, n_head_kv * head_dim, seed)
    row = n_head * head_dim
    q = (((np.arange(n_tokens * row) % 17).astype(np.float32) - 8.0) / 8.0).astype(np.float32)
    start_pos = 3
    got = O.attention(q, k, v, n_head, n_head_kv, head_dim, 0.125, n_tokens, start_pos)
    g = n_head // n_head_kv
    k3 = k.reshape(n_pos, n_head_kv, head_dim).astype(np.float64)
    v3 = v.reshape(n_pos, n_head_kv, head_dim).astype(np.float64)
    q3 = q.reshape(n_tokens, n_head, head_dim).astype(np.float64)
    for t in range(n_tokens):
        L = start_pos + t + 1
        for h in range(n_head):
            s = (k3[:L, h // g] @ q3[t, h]) * 0.125
            p = np.exp(s - s.max())
            p /= p.sum()
            want = p @ v3[:L, h // g]
            assert np.abs(got[t, h * head_dim:(h + 1) * head_dim] - want).max() < 2e-5


# ---- E/sampling.rs:336-359 ---------------------------------------------------
def test_argmax_last_index_wins_ties_and_total_order():
    assert O.argmax([1.0, 3.0, 3.0, 2.0]) == 2
    assert O.argmax([0.0, -0.0]) == 0          # total_cmp: -0 < +0
    assert O.argmax([-0.0, 0.0]) == 1
    assert O.argmax([1.0, np.nan, 5.0]) == 1   # positive NaN sorts above everything
    assert O.argmax([-np.inf, -np.inf]) == 1
    assert O.argmax([7.0]) == 0


def test_repeat_penalty_compounds_and_respects_last_n():
    l = np.array([2.0, -2.0, 4.0, 1.0], np.float32)
    got = O.repeat_penalty(l, [0, 1, 0, 9], 64, 2.0)
    assert list(got) == [0.5, -4.0, 4.0, 1.0]      # token 0 twice, out-of-range id ignored
    got = O.repeat_penalty(l, [0, 1, 2], 1, 2.0)
    assert list(got) == [2.0, -2.0, 2.0, 1.0]      # only the last one
    assert list(O.repeat_penalty(l, [0, 1], 64, 1.0)) == list(l)


def test_oracle_graph_applies_bias_then_head_norm_then_rope_in_the_reference_order():
    """arch/llama.rs:750-809: q = Wq x; q += bias; per-head RMSNorm; RoPE (pairing by architecture).  One layer, one token,
    checked against the same steps written out with the oracle's own operators."""
    from orangu_b200 import synth

    cfg = dict(synth.CONFIGS["tiny"], n_layer=1, rope_neox=True)
    t = synth.add_qwen_extras(cfg, synth.model_tensors(cfg, seed=9), seed=10)
    m = O.Model(cfg, t)
    toks = np.array([7, 300, 12], np.uint32)
    logits, hidden = m.forward(m.new_kv(8), toks, 0, want_hidden=True)
    e, hd, nh, nkv, ff = cfg["n_embd"], cfg["head_dim"], cfg["n_head"], cfg["n_head_kv"], cfg["n_ff"]

    def mm(x, n, name):
        w = t[name]
        return O.matmul(x, n, w["data"], w["type"], w["in_dim"], w["out_dim"]).reshape(n, -1)

    emb = t["token_embd.weight"]
    rb = O.row_bytes(emb["type"], e)
    rows = np.ascontiguousarray(emb["data"]).view(np.uint8).reshape(-1, rb)
    x = np.stack([O.dequantize(emb["type"], rows[int(tok)], e) for tok in toks])
    normed = O.rmsnorm(x, t["blk.0.attn_norm.weight"]["data"], cfg["rms_eps"])
    q, k, v = mm(normed, 3, "blk.0.attn_q.weight"), mm(normed, 3, "blk.0.attn_k.weight"), mm(normed, 3, "blk.0.attn_v.weight")
    q, k, v = q + t["blk.0.attn_q.bias"]["data"], k + t["blk.0.attn_k.bias"]["data"], v + t["blk.0.attn_v.bias"]["data"]
    q = O.rmsnorm(q.reshape(3 * nh, hd), t["blk.0.attn_q_norm.weight"]["data"], cfg["rms_eps"]).reshape(3, -1)
    k = O.rmsnorm(k.reshape(3 * nkv, hd), t["blk.0.attn_k_norm.weight"]["data"], cfg["rms_eps"]).reshape(3, -1)
    for pos in range(3):
        q[pos] = O.rope_layout(q[pos], nh, hd, pos, hd, cfg["rope_freq_base"], True)
        k[pos] = O.rope_layout(k[pos], nkv, hd, pos, hd, cfg["rope_freq_base"], True)
    att = O.attention(q, k, v, nh, nkv, hd, np.float32(1.0) / np.sqrt(np.float32(hd)), 3, 0)
    proj = mm(att.reshape(3, -1), 3, "blk.0.attn_output.weight")
    x = x + proj
    n2 = O.rmsnorm(x, t["blk.0.ffn_norm.weight"]["data"], cfg["rms_eps"])
    g, u = mm(n2, 3, "blk.0.ffn_gate.weight"), mm(n2, 3, "blk.0.ffn_up.weight")
    x = x + mm(O.swiglu(g, u), 3, "blk.0.ffn_down.weight")
    assert (x.view(np.uint32) == hidden.view(np.uint32)).all()
