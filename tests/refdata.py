"""Deterministic inputs the reference's own tests use, restated as generators.

E = src/bin/orangu-server/engine in the reference tree.
"""
import numpy as np

BLOCK = {8: (34, 32), 12: (144, 256), 14: (210, 256), 0: (4, 1), 2: (18, 32), 6: (22, 32), 20: (18, 32), 13: (176, 256)}


def fixture_bytes(n):
    """xorshift64 byte stream, E/quant.rs:1427-1437."""
    state = 0x2545F4914F6CDD1D
    out = np.empty(n, np.uint8)
    M = (1 << 64) - 1
    for i in range(n):
        state ^= (state << 13) & M
        state ^= state >> 7
        state ^= (state << 17) & M
        out[i] = (state >> 33) & 0xFF
    return out


def bit_checksum(values):
    """FNV-1a-style fold over the f32 bit patterns, E/quant.rs:1442-1446."""
    acc = 0xCBF29CE484222325
    M = (1 << 64) - 1
    for b in np.ascontiguousarray(values, np.float32).view(np.uint32):
        acc = ((acc ^ int(b)) * 0x00000100000001B3) & M
    return acc


def pseudo_bytes(n, seed):
    """LCG byte stream, E/vecdot.rs:3415-3423."""
    s = (seed | 1) & 0xFFFFFFFF
    # vectorised LCG: s_k = a^k s_0 + c (a^k - 1)/(a - 1), done iteratively in chunks for speed
    out = np.empty(n, np.uint8)
    a, c = 1664525, 1013904223
    for i in range(n):
        s = (s * a + c) & 0xFFFFFFFF
        out[i] = (s >> 16) & 0xFF
    return out


def pseudo_bytes_fast(n, seed):
    """Same stream as pseudo_bytes, computed with numpy uint32 wrap-around in O(log n) passes."""
    s0 = np.uint32((seed | 1) & 0xFFFFFFFF)
    a = np.ones(n, np.uint32)
    c = np.zeros(n, np.uint32)
    # affine maps f_k(s) = A_k s + C_k by doubling
    A = np.empty(n, np.uint32)
    Cc = np.empty(n, np.uint32)
    with np.errstate(over="ignore"):
        ak, ck = np.uint32(1664525), np.uint32(1013904223)
        A[0], Cc[0] = ak, ck
        filled = 1
        while filled < n:
            take = min(filled, n - filled)
            # f_{filled + j} = f_filled-th power composed: f_{i+filled}(s) = f_i(f_filled_total(s))
            Af, Cf = A[filled - 1], Cc[filled - 1]
            A[filled:filled + take] = A[:take] * Af
            Cc[filled:filled + take] = A[:take] * Cf + Cc[:take]
            filled += take
        s = A * s0 + Cc
    return ((s >> np.uint32(16)) & np.uint32(0xFF)).astype(np.uint8)


def activations(n):
    """E/vecdot.rs:3425-3429."""
    i = np.arange(n, dtype=np.int64)
    return (((i * 37 % 23).astype(np.float32) - np.float32(11.0)) * np.float32(0.031)).astype(np.float32)


def _pin_scales(raw, t):
    bb = BLOCK[t][0]
    blocks = raw.reshape(-1, bb)
    if t in (8, 2, 6, 20):  # one leading f16 scale (E/vecdot.rs:3459-3461)
        blocks[:, 0:2] = [0x00, 0x30]
    elif t in (12, 13):  # Q5_K shares Q4_K's leading d / dmin pair (E/vecdot.rs:3467-3471)
        blocks[:, 0:2] = [0x00, 0x30]
        blocks[:, 2:4] = [0x00, 0x2C]
    elif t == 14:
        blocks[:, 208:210] = [0x00, 0x30]
    else:
        raise ValueError(t)
    return raw


def fixture_row(t, in_dim, seed):
    """E/vecdot.rs:3647-3681: LCG payload, f16 scales pinned to 0.125 (and dmin 0.0625)."""
    bb, be = BLOCK[t]
    return _pin_scales(pseudo_bytes_fast(in_dim // be * bb, seed), t)


def k_fixture(t, in_dim, out_dim, n_tokens, seed):
    """E/vecdot.rs:4425-4455; also used here for Q8_0 with the same pinning rule as fixture_row."""
    bb, be = BLOCK[t]
    raw = _pin_scales(pseudo_bytes_fast(in_dim // be * bb * out_dim, seed), t)
    return raw, activations(in_dim * n_tokens)


def xorshift32_kv(n_pos, kv_dim, seed):
    """E/attention.rs:760-780: K and V rows interleaved from one xorshift32 stream."""
    s = seed & 0xFFFFFFFF
    k = np.empty((n_pos, kv_dim), np.float32)
    v = np.empty((n_pos, kv_dim), np.float32)
    M = 0xFFFFFFFF
    umax = np.float32(M)

    def nxt():
        nonlocal s
        s ^= (s << 13) & M
        s ^= s >> 17
        s ^= (s << 5) & M
        return np.float32(np.float32(np.float32(s) / umax) * np.float32(2.0)) - np.float32(1.0)

    for p in range(n_pos):
        for i in range(kv_dim):
            k[p, i] = nxt()
        for i in range(kv_dim):
            v[p, i] = nxt()
    return k, v
