/*
 * CPU oracle: restatement of the reference's CPU arithmetic for the quantized
 * decode path.  TEST INFRASTRUCTURE ONLY -- see orangu_oracle.h.
 *
 * E = src/bin/orangu-server/engine in the reference tree.
 */
#include "orangu_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <vector>

#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

constexpr size_t ACT_BLOCK = 32;    /* E/vecdot.rs ACT_BLOCK */
constexpr size_t GROUP = 16;        /* E/vecdot.rs:63 */
constexpr size_t SUPER_BLOCK = 256; /* E/vecdot.rs:1800 */
constexpr size_t SUBS = 8;
constexpr size_t TOKEN_TILE = 4;    /* E/vecdot.rs:1682 */

/* exp for f32: the reference calls f32::exp, i.e. the platform libm's expf, whose last bit is not
 * specified (glibc documents 0.502 ULP).  The oracle pins it to the correctly rounded value, taken
 * in double and rounded once, which a device can reproduce; glibc's expf returns that same value
 * for all but about one argument in several hundred. */
inline float exp_f32(float x) { return (float)exp((double)x); }

inline float bits_f32(uint32_t b) {
    float f;
    memcpy(&f, &b, 4);
    return f;
}
inline uint32_t f32_bits(float f) {
    uint32_t b;
    memcpy(&b, &f, 4);
    return b;
}

/* E/quant.rs:511-528 */
inline float f16_to_f32(uint16_t bits) {
    const uint32_t SHIFTED_EXP = 0x7c00u << 13;
    uint32_t out = ((uint32_t)bits & 0x7fffu) << 13;
    uint32_t exp = SHIFTED_EXP & out;
    out += (127u - 15u) << 23;
    if (exp == SHIFTED_EXP) {
        out += (128u - 16u) << 23;
    } else if (exp == 0) {
        out += 1u << 23;
        out = f32_bits(bits_f32(out) - bits_f32(113u << 23));
    }
    return bits_f32(out | (((uint32_t)bits & 0x8000u) << 16));
}

inline float read_f16(const uint8_t *p) { return f16_to_f32((uint16_t)(p[0] | (p[1] << 8))); }

/* IEEE-754 binary32 -> binary16, round to nearest even. */
inline uint16_t f32_to_f16(float v) {
    uint32_t x = f32_bits(v);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t mag = x & 0x7fffffffu;
    if (mag >= 0x7f800000u) { /* inf / nan */
        if (mag == 0x7f800000u) return (uint16_t)(sign | 0x7c00u);
        return (uint16_t)(sign | 0x7e00u | ((mag >> 13) & 0x3ffu));
    }
    if (mag >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u); /* >= 65520 rounds to inf */
    if (mag < 0x33000001u) return (uint16_t)sign;              /* <= 2^-25 rounds to 0 */
    int32_t e = (int32_t)(mag >> 23) - 127;
    uint32_t m = (mag & 0x7fffffu) | 0x800000u;
    uint32_t shift;
    uint32_t base;
    if (e < -14) { /* subnormal half */
        shift = (uint32_t)(13 + (-14 - e));
        base = 0;
    } else {
        shift = 13;
        base = (uint32_t)(e + 15) << 10;
        m &= 0x7fffffu;
    }
    uint32_t q = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1u);
    uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u))) q += 1;
    return (uint16_t)(sign | (base + q)); /* a carry out of the mantissa bumps the exponent */
}

/* E/quant.rs:653-662 */
inline void scale_min_k4(int j, const uint8_t *q, uint8_t *sc, uint8_t *m) {
    if (j < 4) {
        *sc = q[j] & 63;
        *m = q[j + 4] & 63;
    } else {
        *sc = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4));
        *m = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
    }
}

/* ---- dequantisers ----------------------------------------------------- */

/* E/quant.rs:639-649 */
void dequantize_q8_0(const uint8_t *bytes, size_t n, float *out) {
    size_t nb = (n + 31) / 32, w = 0;
    for (size_t b = 0; b < nb; ++b) {
        const uint8_t *blk = bytes + b * 34;
        float d = read_f16(blk);
        for (size_t i = 0; i < 32 && w < n; ++i, ++w) out[w] = (float)(int8_t)blk[2 + i] * d;
    }
}

/* The per-32 symmetric family (Q4_0, Q5_0, IQ4_NL): block = f16 d, [Q5_0: 4 bytes of fifth bits,] 16 bytes of nibbles;
 * the low nibbles are elements 0..15, the high nibbles 16..31.  E/vecdot.rs:1001-1016 (the shared bit extraction),
 * :1019-1025 (Q4_0: bias 8), :1036-1038 (Q5_0: bias 16), E/quant.rs:1320-1336 + E/iq_grids.rs:5941 (IQ4_NL: the
 * nibble indexes the format's 16 non-uniform levels). */
const int8_t IQ4NL_LEVELS[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};

inline bool is_sym32(uint32_t type) { return type == OREF_TYPE_Q4_0 || type == OREF_TYPE_Q5_0 || type == OREF_TYPE_IQ4_NL; }
inline size_t sym32_block_bytes(uint32_t type) { return type == OREF_TYPE_Q5_0 ? 22 : 18; }

/* writes the block's 32 signed codes, returns its scale */
float unpack_sym32(uint32_t type, const uint8_t *blk, int8_t *w) {
    const float d = read_f16(blk);
    if (type == OREF_TYPE_IQ4_NL) {
        for (int j = 0; j < 16; ++j) {
            w[j] = IQ4NL_LEVELS[blk[2 + j] & 0x0F];
            w[16 + j] = IQ4NL_LEVELS[blk[2 + j] >> 4];
        }
        return d;
    }
    const bool five = type == OREF_TYPE_Q5_0;
    const uint32_t qh = five ? ((uint32_t)blk[2] | ((uint32_t)blk[3] << 8) | ((uint32_t)blk[4] << 16) | ((uint32_t)blk[5] << 24)) : 0u;
    const uint8_t *qs = blk + (five ? 6 : 2);
    const int bias = five ? 16 : 8;
    for (int j = 0; j < 16; ++j) {
        const uint32_t hi_lo = ((qh >> j) << 4) & 0x10, hi_hi = (qh >> (j + 12)) & 0x10;
        w[j] = (int8_t)((int)((qs[j] & 0x0Fu) | hi_lo) - bias);
        w[16 + j] = (int8_t)((int)((uint32_t)(qs[j] >> 4) | hi_hi) - bias);
    }
    return d;
}

/* E/quant.rs:537-555 (Q4_0), :560-580 (Q5_0), :1320-1336 (IQ4_NL): code times scale, one rounding */
void dequantize_sym32(uint32_t type, const uint8_t *bytes, size_t n, float *out) {
    size_t nb = (n + 31) / 32, o = 0;
    int8_t w[32];
    for (size_t b = 0; b < nb; ++b) {
        const float d = unpack_sym32(type, bytes + b * sym32_block_bytes(type), w);
        for (size_t i = 0; i < 32 && o < n; ++i, ++o) out[o] = (float)w[i] * d;
    }
}

/* E/quant.rs:666-697 */
void dequantize_q4_k(const uint8_t *bytes, size_t n, float *out) {
    size_t nb = (n + 255) / 256;
    float tmp[256];
    for (size_t b = 0; b < nb; ++b) {
        const uint8_t *blk = bytes + b * 144;
        float d = read_f16(blk), dmin = read_f16(blk + 2);
        const uint8_t *scales = blk + 4, *qs = blk + 16;
        size_t w = 0;
        int is = 0;
        for (size_t q_offset = 0; q_offset < 256; q_offset += 64) {
            uint8_t sc1, m1, sc2, m2;
            scale_min_k4(is, scales, &sc1, &m1);
            scale_min_k4(is + 1, scales, &sc2, &m2);
            float d1 = d * (float)sc1, mm1 = dmin * (float)m1;
            float d2 = d * (float)sc2, mm2 = dmin * (float)m2;
            const uint8_t *q = qs + q_offset / 2;
            for (int i = 0; i < 32; ++i) tmp[w++] = d1 * (float)(q[i] & 0x0F) - mm1;
            for (int i = 0; i < 32; ++i) tmp[w++] = d2 * (float)(q[i] >> 4) - mm2;
            is += 2;
        }
        size_t take = std::min<size_t>(256, n - b * 256);
        memcpy(out + b * 256, tmp, take * sizeof(float));
    }
}

/* E/quant.rs:703-742: block = d, dmin, scales[12], qh[32], qs[128]; code = nibble + 16 * (bit of qh[l] for the sub-block) */
void dequantize_q5_k(const uint8_t *bytes, size_t n, float *out) {
    size_t nb = (n + 255) / 256;
    float tmp[256];
    for (size_t b = 0; b < nb; ++b) {
        const uint8_t *blk = bytes + b * 176;
        float d = read_f16(blk), dmin = read_f16(blk + 2);
        const uint8_t *scales = blk + 4, *qh = blk + 16, *qs = blk + 48;
        size_t w = 0;
        int is = 0;
        uint8_t u1 = 1, u2 = 2;
        for (size_t q_offset = 0; q_offset < 256; q_offset += 64) {
            uint8_t sc1, m1, sc2, m2;
            scale_min_k4(is, scales, &sc1, &m1);
            scale_min_k4(is + 1, scales, &sc2, &m2);
            float d1 = d * (float)sc1, mm1 = dmin * (float)m1;
            float d2 = d * (float)sc2, mm2 = dmin * (float)m2;
            const uint8_t *q = qs + q_offset / 2;
            for (int l = 0; l < 32; ++l) tmp[w++] = d1 * (float)((int)(q[l] & 0x0F) + ((qh[l] & u1) ? 16 : 0)) - mm1;
            for (int l = 0; l < 32; ++l) tmp[w++] = d2 * (float)((int)(q[l] >> 4) + ((qh[l] & u2) ? 16 : 0)) - mm2;
            is += 2;
            u1 = (uint8_t)(u1 << 2);
            u2 = (uint8_t)(u2 << 2);
        }
        size_t take = std::min<size_t>(256, n - b * 256);
        memcpy(out + b * 256, tmp, take * sizeof(float));
    }
}

/* E/quant.rs:746-787 */
void dequantize_q6_k(const uint8_t *bytes, size_t n, float *out) {
    size_t nb = (n + 255) / 256;
    float values[256];
    for (size_t b = 0; b < nb; ++b) {
        const uint8_t *blk = bytes + b * 210;
        const uint8_t *ql = blk, *qh = blk + 128, *sc = blk + 192;
        float d = read_f16(blk + 208);
        size_t ql_off = 0, qh_off = 0, sc_off = 0;
        for (size_t y_off = 0; y_off < 256; y_off += 128) {
            for (size_t l = 0; l < 32; ++l) {
                size_t is = l / 16;
                int q1 = (int)((ql[ql_off + l] & 0xF) | ((qh[qh_off + l] & 3) << 4)) - 32;
                int q2 = (int)((ql[ql_off + l + 32] & 0xF) | (((qh[qh_off + l] >> 2) & 3) << 4)) - 32;
                int q3 = (int)((ql[ql_off + l] >> 4) | (((qh[qh_off + l] >> 4) & 3) << 4)) - 32;
                int q4 = (int)((ql[ql_off + l + 32] >> 4) | (((qh[qh_off + l] >> 6) & 3) << 4)) - 32;
                values[y_off + l] = d * (float)(int8_t)sc[sc_off + is] * (float)q1;
                values[y_off + l + 32] = d * (float)(int8_t)sc[sc_off + is + 2] * (float)q2;
                values[y_off + l + 64] = d * (float)(int8_t)sc[sc_off + is + 4] * (float)q3;
                values[y_off + l + 96] = d * (float)(int8_t)sc[sc_off + is + 6] * (float)q4;
            }
            ql_off += 64;
            qh_off += 32;
            sc_off += 8;
        }
        size_t take = std::min<size_t>(256, n - b * 256);
        memcpy(out + b * 256, values, take * sizeof(float));
    }
}

/* ---- activation quantiser --------------------------------------------- */

/* One block of `len` values sharing a scale; E/vecdot.rs:101-123 (len 32) and
 * :3036-3050 (len 256).  f32::max ignores a NaN operand, f32::round is half away
 * from zero, f32::clamp propagates NaN and the `as i8` cast turns NaN into 0. */
inline float quantize_span(const float *x, size_t len, int8_t *q, int32_t *sums) {
    float amax = 0.0f;
    for (size_t i = 0; i < len; ++i) amax = fmaxf(amax, fabsf(x[i]));
    float scale = amax / 127.0f;
    float inv = scale > 0.0f ? 1.0f / scale : 0.0f;
    for (size_t g = 0; g < len / GROUP; ++g) {
        int32_t sum = 0;
        for (size_t i = 0; i < GROUP; ++i) {
            float r = roundf(x[g * GROUP + i] * inv);
            int8_t qi;
            if (r != r) {
                qi = 0;
            } else {
                r = r < -127.0f ? -127.0f : (r > 127.0f ? 127.0f : r);
                qi = (int8_t)r;
            }
            q[g * GROUP + i] = qi;
            sum += qi;
        }
        if (sums) sums[g] = sum;
    }
    return scale;
}

/* ---- integer dots, E/vecdot.rs:471-502, 676-707 ------------------------- */
inline int32_t dot32(const int8_t *w, const int8_t *x) {
    int32_t s = 0;
    for (int i = 0; i < 32; ++i) s += (int32_t)w[i] * (int32_t)x[i];
    return s;
}
inline int32_t dot16(const int8_t *w, const int8_t *x) {
    int32_t s = 0;
    for (int i = 0; i < 16; ++i) s += (int32_t)w[i] * (int32_t)x[i];
    return s;
}

/* E/vecdot.rs:1074-1075 Q6K_RUNS: (ql_add, hshift, high) */
struct Q6Run {
    int ql_add, hshift, high;
};
const Q6Run Q6K_RUNS[4] = {{0, 0, 0}, {32, 2, 0}, {0, 4, 1}, {32, 6, 1}};

/* E/vecdot.rs:1193-1207, scalar arm */
inline void unpack_q6k_run(const uint8_t *ql_run, const uint8_t *qh_run, int hshift, int high, int8_t *w) {
    for (int j = 0; j < 32; ++j) {
        int lo = high ? (ql_run[j] >> 4) : (ql_run[j] & 0x0F);
        int hi = (qh_run[j] >> hshift) & 3;
        w[j] = (int8_t)((lo | (hi << 4)) - 32);
    }
}

struct ActRow {
    const int8_t *q;
    const float *d;
    const int32_t *sums;
};

/* E/vecdot.rs:2829-2838 */
float dot_q8_0(const uint8_t *row, size_t in_dim, const ActRow &a) {
    float total = 0.0f;
    size_t nb = in_dim / 32;
    for (size_t b = 0; b < nb; ++b) {
        const uint8_t *blk = row + b * 34;
        float dw = read_f16(blk);
        total += dw * a.d[b] * (float)dot32((const int8_t *)(blk + 2), a.q + b * 32);
    }
    return total;
}

/* E/vecdot.rs:2842-2852 (IQ4_NL), :2856-2867 (Q5_0), :2871-2881 (Q4_0): the Q8_0 loop over the unpacked codes */
float dot_sym32(uint32_t type, const uint8_t *row, size_t in_dim, const ActRow &a) {
    float total = 0.0f;
    int8_t w[32];
    const size_t nb = in_dim / 32, bb = sym32_block_bytes(type);
    for (size_t b = 0; b < nb; ++b) {
        const float dw = unpack_sym32(type, row + b * bb, w);
        total += dw * a.d[b] * (float)dot32(w, a.q + b * 32);
    }
    return total;
}

/* E/vecdot.rs:3152-3178; `out` (nullable) receives isum, imin per super-block */
float dot_k_row_q4_k(const uint8_t *row, size_t in_dim, const ActRow &a, int32_t *isum_out, int32_t *imin_out) {
    float total = 0.0f;
    int8_t w[32];
    size_t ns = in_dim / 256;
    for (size_t s = 0; s < ns; ++s) {
        const uint8_t *blk = row + s * 144;
        float d = read_f16(blk), dmin = read_f16(blk + 2);
        const uint8_t *scales = blk + 4, *qs = blk + 16;
        size_t sb = s * SUBS;
        int32_t isum = 0, imin = 0;
        for (int g = 0; g < 4; ++g) {
            const uint8_t *bytes = qs + g * 32;
            for (int half = 0; half < 2; ++half) {
                int shift = half * 4;
                uint8_t sc, m;
                scale_min_k4(g * 2 + half, scales, &sc, &m);
                size_t b = sb + g * 2 + half;
                for (int j = 0; j < 32; ++j) w[j] = (int8_t)((bytes[j] >> shift) & 0x0F);
                isum += (int32_t)sc * dot32(w, a.q + b * 32);
                imin += (int32_t)m * (a.sums[b * 2] + a.sums[b * 2 + 1]);
            }
        }
        if (isum_out) isum_out[s] = isum;
        if (imin_out) imin_out[s] = imin;
        total += a.d[s] * (d * (float)isum - dmin * (float)imin);
    }
    return total;
}

/* E/vecdot.rs:3181-3210: the Q4_K loop over five-bit codes */
float dot_k_row_q5_k(const uint8_t *row, size_t in_dim, const ActRow &a, int32_t *isum_out, int32_t *imin_out) {
    float total = 0.0f;
    int8_t w[32];
    size_t ns = in_dim / 256;
    for (size_t s = 0; s < ns; ++s) {
        const uint8_t *blk = row + s * 176;
        float d = read_f16(blk), dmin = read_f16(blk + 2);
        const uint8_t *scales = blk + 4, *qh = blk + 16, *qs = blk + 48;
        size_t sb = s * SUBS;
        int32_t isum = 0, imin = 0;
        for (int g = 0; g < 4; ++g) {
            const uint8_t *bytes = qs + g * 32;
            for (int half = 0; half < 2; ++half) {
                int shift = half * 4;
                uint8_t sc, m;
                scale_min_k4(g * 2 + half, scales, &sc, &m);
                const uint8_t hi_mask = (uint8_t)(1u << (g * 2 + half));
                size_t b = sb + g * 2 + half;
                for (int j = 0; j < 32; ++j) w[j] = (int8_t)(((bytes[j] >> shift) & 0x0F) + ((qh[j] & hi_mask) ? 16 : 0));
                isum += (int32_t)sc * dot32(w, a.q + b * 32);
                imin += (int32_t)m * (a.sums[b * 2] + a.sums[b * 2 + 1]);
            }
        }
        if (isum_out) isum_out[s] = isum;
        if (imin_out) imin_out[s] = imin;
        total += a.d[s] * (d * (float)isum - dmin * (float)imin);
    }
    return total;
}

/* E/vecdot.rs:3215-3241 */
float dot_k_row_q6_k(const uint8_t *row, size_t in_dim, const ActRow &a, int32_t *isum_out) {
    float total = 0.0f;
    int8_t w[32];
    size_t ns = in_dim / 256;
    for (size_t s = 0; s < ns; ++s) {
        const uint8_t *blk = row + s * 210;
        const uint8_t *ql = blk, *qh = blk + 128, *sc = blk + 192;
        float d = read_f16(blk + 208);
        size_t base = s * SUPER_BLOCK;
        int32_t isum = 0;
        size_t r = 0;
        for (int h = 0; h < 2; ++h) {
            const uint8_t *qh_run = qh + h * 32;
            for (int k = 0; k < 4; ++k) {
                const Q6Run &run = Q6K_RUNS[k];
                unpack_q6k_run(ql + h * 64 + run.ql_add, qh_run, run.hshift, run.high, w);
                const int8_t *x = a.q + base + r * 32;
                isum += (int32_t)(int8_t)sc[2 * r] * dot16(w, x) + (int32_t)(int8_t)sc[2 * r + 1] * dot16(w + 16, x + 16);
                ++r;
            }
        }
        if (isum_out) isum_out[s] = isum;
        total += a.d[s] * d * (float)isum;
    }
    return total;
}

/* ---- prefill GEMM: activations ------------------------------------------ */

/* E/vecdot.rs:1836-1911 */
struct ActQ8K {
    size_t n_tokens, n_block, n_super, n_tile;
    std::vector<int8_t> q;    /* [tile][block][token][32] */
    std::vector<float> d;     /* [tile][super][token] */
    std::vector<int16_t> bsum; /* [tile][super][token][8] */
    void quantize(const float *x, size_t in_dim, size_t nt) {
        n_tokens = nt;
        n_block = in_dim / 32;
        n_super = in_dim / SUPER_BLOCK;
        n_tile = (nt + TOKEN_TILE - 1) / TOKEN_TILE;
        q.assign(n_tile * n_block * TOKEN_TILE * 32, 0);
        d.assign(n_tile * n_super * TOKEN_TILE, 0.0f);
        bsum.assign(n_tile * n_super * TOKEN_TILE * SUBS, 0);
#pragma omp parallel for schedule(static)
        for (size_t t = 0; t < nt; ++t) {
            size_t tl = t / TOKEN_TILE, k = t % TOKEN_TILE;
            const float *row = x + t * in_dim;
            int8_t tmp[256];
            int32_t sums[16];
            for (size_t s = 0; s < n_super; ++s) {
                float scale = quantize_span(row + s * SUPER_BLOCK, SUPER_BLOCK, tmp, sums);
                d[(tl * n_super + s) * TOKEN_TILE + k] = scale;
                for (size_t j = 0; j < SUBS; ++j) {
                    size_t b = s * SUBS + j;
                    memcpy(&q[((tl * n_block + b) * TOKEN_TILE + k) * 32], tmp + j * 32, 32);
                    bsum[((tl * n_super + s) * TOKEN_TILE + k) * SUBS + j] = (int16_t)(sums[2 * j] + sums[2 * j + 1]);
                }
            }
        }
    }
};

/* E/vecdot.rs:2469-2526 */
struct ActQ8Flat {
    size_t n_tokens, n_block, n_tile;
    std::vector<int8_t> q; /* [tile][block][token][32] */
    std::vector<float> d;  /* [tile][block][token] */
    void quantize(const float *x, size_t in_dim, size_t nt) {
        n_tokens = nt;
        n_block = in_dim / ACT_BLOCK;
        n_tile = (nt + TOKEN_TILE - 1) / TOKEN_TILE;
        q.assign(n_tile * n_block * TOKEN_TILE * ACT_BLOCK, 0);
        d.assign(n_tile * n_block * TOKEN_TILE, 0.0f);
#pragma omp parallel for schedule(static)
        for (size_t t = 0; t < nt; ++t) {
            size_t tl = t / TOKEN_TILE, k = t % TOKEN_TILE;
            const float *row = x + t * in_dim;
            for (size_t b = 0; b < n_block; ++b) {
                d[(tl * n_block + b) * TOKEN_TILE + k] =
                    quantize_span(row + b * ACT_BLOCK, ACT_BLOCK, &q[((tl * n_block + b) * TOKEN_TILE + k) * ACT_BLOCK], nullptr);
            }
        }
    }
};

/* ---- prefill GEMM: unpacked weight rows ---------------------------------- */

/* E/vecdot.rs:1920-1975 KRow */
struct KRow {
    std::vector<int8_t> q;
    std::vector<int16_t> sc, mins;
    std::vector<float> d, dmin;
    bool q6 = false;
};

/* E/vecdot.rs:2064-2089: as unpack_k_q4_k, codes carry their fifth bit; the row then takes the Q4_K GEMM (:2119-2143) */
void unpack_k_q5_k(const uint8_t *row, size_t in_dim, KRow &out) {
    size_t ns = in_dim / 256;
    out.q6 = false;
    out.q.resize(in_dim);
    out.sc.resize(in_dim / 32);
    out.mins.resize(in_dim / 32);
    out.d.resize(ns);
    out.dmin.resize(ns);
    size_t sb = 0;
    for (size_t s = 0; s < ns; ++s) {
        const uint8_t *blk = row + s * 176;
        out.d[s] = read_f16(blk);
        out.dmin[s] = read_f16(blk + 2);
        const uint8_t *scales = blk + 4, *qh = blk + 16, *qs = blk + 48;
        for (int g = 0; g < 4; ++g) {
            const uint8_t *bytes = qs + g * 32;
            for (int half = 0; half < 2; ++half) {
                uint8_t sc, m;
                scale_min_k4(g * 2 + half, scales, &sc, &m);
                const uint8_t hi_mask = (uint8_t)(1u << (g * 2 + half));
                int8_t *w = &out.q[(sb + half) * 32];
                for (int j = 0; j < 32; ++j) w[j] = (int8_t)(((bytes[j] >> (half * 4)) & 0x0F) + ((qh[j] & hi_mask) ? 16 : 0));
                out.sc[sb + half] = sc;
                out.mins[sb + half] = m;
            }
            sb += 2;
        }
    }
}

/* E/vecdot.rs:2036-2058 */
void unpack_k_q4_k(const uint8_t *row, size_t in_dim, KRow &out) {
    size_t ns = in_dim / 256;
    out.q6 = false;
    out.q.resize(in_dim);
    out.sc.resize(in_dim / 32);
    out.mins.resize(in_dim / 32);
    out.d.resize(ns);
    out.dmin.resize(ns);
    size_t sb = 0;
    for (size_t s = 0; s < ns; ++s) {
        const uint8_t *blk = row + s * 144;
        out.d[s] = read_f16(blk);
        out.dmin[s] = read_f16(blk + 2);
        const uint8_t *scales = blk + 4, *qs = blk + 16;
        for (int g = 0; g < 4; ++g) {
            const uint8_t *bytes = qs + g * 32;
            for (int half = 0; half < 2; ++half) {
                uint8_t sc, m;
                scale_min_k4(g * 2 + half, scales, &sc, &m);
                int8_t *w = &out.q[(sb + half) * 32];
                for (int j = 0; j < 32; ++j) w[j] = (int8_t)((bytes[j] >> (half * 4)) & 0x0F);
                out.sc[sb + half] = sc;
                out.mins[sb + half] = m;
            }
            sb += 2;
        }
    }
}

/* E/vecdot.rs:2119-2143 */
void unpack_k_q6_k(const uint8_t *row, size_t in_dim, KRow &out) {
    size_t ns = in_dim / 256;
    out.q6 = true;
    out.q.resize(in_dim);
    out.sc.resize(in_dim / GROUP);
    out.mins.clear();
    out.d.resize(ns);
    out.dmin.clear();
    for (size_t s = 0; s < ns; ++s) {
        const uint8_t *blk = row + s * 210;
        const uint8_t *ql = blk, *qh = blk + 128, *sc = blk + 192;
        out.d[s] = read_f16(blk + 208);
        size_t base = s * SUPER_BLOCK;
        for (int h = 0; h < 2; ++h) {
            const uint8_t *qh_run = qh + h * 32;
            for (int k = 0; k < 4; ++k) {
                const Q6Run &run = Q6K_RUNS[k];
                size_t e0 = base + h * 128 + k * 32;
                unpack_q6k_run(ql + h * 64 + run.ql_add, qh_run, run.hshift, run.high, &out.q[e0]);
                size_t gi = e0 / GROUP;
                out.sc[gi] = (int16_t)(int8_t)sc[gi % 16];
                out.sc[gi + 1] = (int16_t)(int8_t)sc[(gi + 1) % 16];
            }
        }
    }
}

inline void store_tile(size_t tl, const float *acc, float *out, size_t n_out) { /* E/vecdot.rs:2402-2406 */
    size_t base = tl * TOKEN_TILE;
    size_t n = base < n_out ? std::min(TOKEN_TILE, n_out - base) : 0;
    for (size_t i = 0; i < n; ++i) out[base + i] = acc[i];
}

/* E/vecdot.rs:2213-2303: pass 1 mins over every super-block, then the symmetric pass */
void gemm_k_q4_k(const KRow &w, const ActQ8K &a, float *out) {
    for (size_t tl = 0; tl < a.n_tile; ++tl) {
        float acc[TOKEN_TILE] = {0, 0, 0, 0};
        const int8_t *qtile = &a.q[tl * a.n_block * TOKEN_TILE * 32];
        const float *dtile = &a.d[tl * a.n_super * TOKEN_TILE];
        const int16_t *btile = &a.bsum[tl * a.n_super * TOKEN_TILE * SUBS];
        for (size_t s = 0; s < a.n_super; ++s) {
            const float *ad = dtile + s * TOKEN_TILE;
            const int16_t *m = &w.mins[s * SUBS];
            float dm = w.dmin[s];
            for (size_t k = 0; k < TOKEN_TILE; ++k) {
                const int16_t *bs = btile + (s * TOKEN_TILE + k) * SUBS;
                int32_t i0 = 0;
                for (size_t j = 0; j < SUBS; ++j) i0 += (int32_t)m[j] * (int32_t)bs[j];
                acc[k] -= ad[k] * dm * (float)i0;
            }
        }
        for (size_t s = 0; s < a.n_super; ++s) {
            int32_t isum[TOKEN_TILE] = {0, 0, 0, 0};
            for (size_t j = 0; j < SUBS; ++j) {
                size_t b = s * SUBS + j;
                int32_t sc = w.sc[b];
                const int8_t *q0 = &w.q[b * 32];
                const int8_t *xq = qtile + b * TOKEN_TILE * 32;
                for (size_t k = 0; k < TOKEN_TILE; ++k) isum[k] += sc * dot32(q0, xq + k * 32);
            }
            float d0 = w.d[s];
            const float *ad = dtile + s * TOKEN_TILE;
            for (size_t k = 0; k < TOKEN_TILE; ++k) acc[k] += ad[k] * (d0 * (float)isum[k]);
        }
        store_tile(tl, acc, out, a.n_tokens);
    }
}

/* E/vecdot.rs:2352-2398 */
void gemm_k_q6_k(const KRow &w, const ActQ8K &a, float *out) {
    const size_t Q6K_GROUPS = SUPER_BLOCK / GROUP;
    for (size_t tl = 0; tl < a.n_tile; ++tl) {
        float acc[TOKEN_TILE] = {0, 0, 0, 0};
        const int8_t *qtile = &a.q[tl * a.n_block * TOKEN_TILE * 32];
        const float *dtile = &a.d[tl * a.n_super * TOKEN_TILE];
        for (size_t s = 0; s < a.n_super; ++s) {
            int32_t isum[TOKEN_TILE] = {0, 0, 0, 0};
            for (size_t g = 0; g < Q6K_GROUPS; ++g) {
                size_t e = s * SUPER_BLOCK + g * GROUP;
                int32_t sc = w.sc[s * Q6K_GROUPS + g];
                const int8_t *q0 = &w.q[e];
                const int8_t *xq = qtile + (e / 32) * TOKEN_TILE * 32;
                size_t off = e % 32;
                for (size_t k = 0; k < TOKEN_TILE; ++k) isum[k] += sc * dot16(q0, xq + k * 32 + off);
            }
            float d0 = w.d[s];
            const float *ad = dtile + s * TOKEN_TILE;
            for (size_t k = 0; k < TOKEN_TILE; ++k) acc[k] += ad[k] * (d0 * (float)isum[k]);
        }
        store_tile(tl, acc, out, a.n_tokens);
    }
}

/* E/vecdot.rs:2598-2629 with the Q8_0 unpack of :1246-1255 (scale = f16 d, q = the int8 codes) */
void gemm_flat_q8_0(const uint8_t *row, const ActQ8Flat &a, float *out) {
    for (size_t tl = 0; tl < a.n_tile; ++tl) {
        float acc[TOKEN_TILE] = {0, 0, 0, 0};
        const int8_t *qtile = &a.q[tl * a.n_block * TOKEN_TILE * ACT_BLOCK];
        const float *dtile = &a.d[tl * a.n_block * TOKEN_TILE];
        for (size_t b = 0; b < a.n_block; ++b) {
            const uint8_t *blk = row + b * 34;
            float s0 = read_f16(blk);
            const int8_t *q0 = (const int8_t *)(blk + 2);
            const int8_t *xq = qtile + b * TOKEN_TILE * ACT_BLOCK;
            const float *ad = dtile + b * TOKEN_TILE;
            for (size_t k = 0; k < TOKEN_TILE; ++k) acc[k] += ad[k] * s0 * (float)dot32(q0, xq + k * ACT_BLOCK);
        }
        store_tile(tl, acc, out, a.n_tokens);
    }
}

/* The same accumulation over a row unpacked to (codes, per-32 scale): E/vecdot.rs:1277-1292 (Q4_0), :1246-1275 (Q5_0 and
 * Q8_0), :1318-1340 (IQ4_NL) feed E/vecdot.rs:2598-2629 */
void gemm_flat_sym32(uint32_t type, const uint8_t *row, const ActQ8Flat &a, float *out) {
    const size_t bb = sym32_block_bytes(type);
    std::vector<int8_t> codes(a.n_block * 32);
    std::vector<float> scale(a.n_block);
    for (size_t b = 0; b < a.n_block; ++b) scale[b] = unpack_sym32(type, row + b * bb, &codes[b * 32]);
    for (size_t tl = 0; tl < a.n_tile; ++tl) {
        float acc[TOKEN_TILE] = {0, 0, 0, 0};
        const int8_t *qtile = &a.q[tl * a.n_block * TOKEN_TILE * ACT_BLOCK];
        const float *dtile = &a.d[tl * a.n_block * TOKEN_TILE];
        for (size_t b = 0; b < a.n_block; ++b) {
            const float s0 = scale[b];
            const int8_t *q0 = &codes[b * 32];
            const int8_t *xq = qtile + b * TOKEN_TILE * ACT_BLOCK;
            const float *ad = dtile + b * TOKEN_TILE;
            for (size_t k = 0; k < TOKEN_TILE; ++k) acc[k] += ad[k] * s0 * (float)dot32(q0, xq + k * ACT_BLOCK);
        }
        store_tile(tl, acc, out, a.n_tokens);
    }
}

int set_threads(int n_threads) {
#ifdef _OPENMP
    int n = n_threads > 0 ? n_threads : omp_get_num_procs();
    omp_set_num_threads(n);
    return n;
#else
    (void)n_threads;
    return 1;
#endif
}

bool supported(uint32_t type, size_t in_dim) {
    if (type == OREF_TYPE_Q8_0 || is_sym32(type)) return in_dim % 32 == 0;
    if (type == OREF_TYPE_Q4_K || type == OREF_TYPE_Q6_K || type == OREF_TYPE_Q5_K) return in_dim % 256 == 0;
    return false;
}

/* one token against every row, GEMV of the type's family; E/backend/cpu.rs:100-143 */
void gemv_token(const float *x, const uint8_t *raw, uint32_t type, size_t in_dim, size_t out_dim, float *y, size_t y_stride) {
    size_t rb = (size_t)oref_row_bytes(type, in_dim);
    std::vector<int8_t> q(in_dim);
    std::vector<int32_t> sums(in_dim / GROUP);
    if (type == OREF_TYPE_Q8_0 || is_sym32(type)) {
        std::vector<float> d(in_dim / 32);
        oref_quantize_act(x, in_dim, q.data(), d.data(), sums.data());
        ActRow a{q.data(), d.data(), sums.data()};
        if (type == OREF_TYPE_Q8_0) {
#pragma omp parallel for schedule(static)
            for (size_t o = 0; o < out_dim; ++o) y[o * y_stride] = dot_q8_0(raw + o * rb, in_dim, a);
        } else {
#pragma omp parallel for schedule(static)
            for (size_t o = 0; o < out_dim; ++o) y[o * y_stride] = dot_sym32(type, raw + o * rb, in_dim, a);
        }
    } else {
        std::vector<float> d(in_dim / 256);
        oref_quantize_act_k_row(x, in_dim, q.data(), d.data(), sums.data());
        ActRow a{q.data(), d.data(), sums.data()};
        if (type == OREF_TYPE_Q4_K) {
#pragma omp parallel for schedule(static)
            for (size_t o = 0; o < out_dim; ++o) y[o * y_stride] = dot_k_row_q4_k(raw + o * rb, in_dim, a, nullptr, nullptr);
        } else if (type == OREF_TYPE_Q5_K) {
#pragma omp parallel for schedule(static)
            for (size_t o = 0; o < out_dim; ++o) y[o * y_stride] = dot_k_row_q5_k(raw + o * rb, in_dim, a, nullptr, nullptr);
        } else {
#pragma omp parallel for schedule(static)
            for (size_t o = 0; o < out_dim; ++o) y[o * y_stride] = dot_k_row_q6_k(raw + o * rb, in_dim, a, nullptr);
        }
    }
}

} // namespace

extern "C" {

float oref_f16_to_f32(uint16_t bits) { return f16_to_f32(bits); }
uint16_t oref_f32_to_f16(float v) { return f32_to_f16(v); }

int oref_block_layout(uint32_t type, uint32_t *bb, uint32_t *be) {
    switch (type) {
    case OREF_TYPE_F32: *bb = 4; *be = 1; return 0;
    case OREF_TYPE_Q8_0: *bb = 34; *be = 32; return 0;
    case OREF_TYPE_Q4_0: case OREF_TYPE_IQ4_NL: *bb = 18; *be = 32; return 0;
    case OREF_TYPE_Q5_0: *bb = 22; *be = 32; return 0;
    case OREF_TYPE_Q4_K: *bb = 144; *be = 256; return 0;
    case OREF_TYPE_Q5_K: *bb = 176; *be = 256; return 0;
    case OREF_TYPE_Q6_K: *bb = 210; *be = 256; return 0;
    default: return -1;
    }
}

int64_t oref_row_bytes(uint32_t type, uint64_t in_dim) {
    uint32_t bb, be;
    if (oref_block_layout(type, &bb, &be)) return -1;
    if (in_dim % be) return -1;
    return (int64_t)(in_dim / be * bb);
}

int oref_dequantize(uint32_t type, const uint8_t *bytes, size_t n, float *out) {
    switch (type) {
    case OREF_TYPE_F32: memcpy(out, bytes, n * 4); return 0;
    case OREF_TYPE_Q8_0: dequantize_q8_0(bytes, n, out); return 0;
    case OREF_TYPE_Q4_0: case OREF_TYPE_Q5_0: case OREF_TYPE_IQ4_NL: dequantize_sym32(type, bytes, n, out); return 0;
    case OREF_TYPE_Q4_K: dequantize_q4_k(bytes, n, out); return 0;
    case OREF_TYPE_Q5_K: dequantize_q5_k(bytes, n, out); return 0;
    case OREF_TYPE_Q6_K: dequantize_q6_k(bytes, n, out); return 0;
    default: return -1;
    }
}

void oref_get_scale_min_k4(int j, const uint8_t *s, uint8_t *sc, uint8_t *m) { scale_min_k4(j, s, sc, m); }

void oref_quantize_act(const float *x, size_t n, int8_t *q, float *d, int32_t *sums) {
    for (size_t b = 0; b < n / ACT_BLOCK; ++b)
        d[b] = quantize_span(x + b * ACT_BLOCK, ACT_BLOCK, q + b * ACT_BLOCK, sums ? sums + b * 2 : nullptr);
}

void oref_quantize_act_k_row(const float *x, size_t n, int8_t *q, float *d, int32_t *sums) {
    for (size_t s = 0; s < n / SUPER_BLOCK; ++s)
        d[s] = quantize_span(x + s * SUPER_BLOCK, SUPER_BLOCK, q + s * SUPER_BLOCK, sums ? sums + s * 16 : nullptr);
}

float oref_dot_q8_0(const uint8_t *row, size_t in_dim, const int8_t *q, const float *d) {
    ActRow a{q, d, nullptr};
    return dot_q8_0(row, in_dim, a);
}

float oref_dot_row32(uint32_t type, const uint8_t *row, size_t in_dim, const int8_t *q, const float *d) {
    ActRow a{q, d, nullptr};
    if (type == OREF_TYPE_Q8_0) return dot_q8_0(row, in_dim, a);
    if (is_sym32(type)) return dot_sym32(type, row, in_dim, a);
    return NAN;
}

float oref_dot_k_row(uint32_t type, const uint8_t *row, size_t in_dim, const int8_t *q, const float *d, const int32_t *sums) {
    ActRow a{q, d, sums};
    if (type == OREF_TYPE_Q4_K) return dot_k_row_q4_k(row, in_dim, a, nullptr, nullptr);
    if (type == OREF_TYPE_Q5_K) return dot_k_row_q5_k(row, in_dim, a, nullptr, nullptr);
    if (type == OREF_TYPE_Q6_K) return dot_k_row_q6_k(row, in_dim, a, nullptr);
    return NAN;
}

int oref_row_partials(uint32_t type, const uint8_t *row, size_t in_dim, const float *x, int32_t *isum, int32_t *imin) {
    if (!supported(type, in_dim)) return -1;
    std::vector<int8_t> q(in_dim);
    std::vector<int32_t> sums(in_dim / GROUP);
    if (type == OREF_TYPE_Q8_0 || is_sym32(type)) {
        std::vector<float> d(in_dim / 32);
        oref_quantize_act(x, in_dim, q.data(), d.data(), sums.data());
        int8_t w[32];
        for (size_t b = 0; b < in_dim / 32; ++b) {
            if (type == OREF_TYPE_Q8_0) memcpy(w, row + b * 34 + 2, 32);
            else unpack_sym32(type, row + b * sym32_block_bytes(type), w);
            isum[b] = dot32(w, q.data() + b * 32);
            if (imin) imin[b] = 0;
        }
        return 0;
    }
    std::vector<float> d(in_dim / 256);
    oref_quantize_act_k_row(x, in_dim, q.data(), d.data(), sums.data());
    ActRow a{q.data(), d.data(), sums.data()};
    if (type == OREF_TYPE_Q4_K) {
        dot_k_row_q4_k(row, in_dim, a, isum, imin);
    } else if (type == OREF_TYPE_Q5_K) {
        dot_k_row_q5_k(row, in_dim, a, isum, imin);
    } else {
        dot_k_row_q6_k(row, in_dim, a, isum);
        if (imin) memset(imin, 0, (in_dim / 256) * sizeof(int32_t));
    }
    return 0;
}

int oref_matmul(const float *x, size_t n_tokens, const uint8_t *raw, uint32_t type, size_t in_dim, size_t out_dim, float *y, int n_threads) {
    if (!supported(type, in_dim)) return -1;
    set_threads(n_threads);
    size_t rb = (size_t)oref_row_bytes(type, in_dim);
    if (n_tokens == 1) {
        gemv_token(x, raw, type, in_dim, out_dim, y, 1);
        return 0;
    }
    /* accumulate transposed [out_dim][n_tokens], then transpose; E/backend/cpu.rs:385-396 */
    std::vector<float> yt(out_dim * n_tokens);
    if (type == OREF_TYPE_Q8_0) {
        ActQ8Flat a;
        a.quantize(x, in_dim, n_tokens);
#pragma omp parallel for schedule(static)
        for (size_t o = 0; o < out_dim; ++o) gemm_flat_q8_0(raw + o * rb, a, &yt[o * n_tokens]);
    } else if (is_sym32(type)) {
        ActQ8Flat a;
        a.quantize(x, in_dim, n_tokens);
#pragma omp parallel for schedule(static)
        for (size_t o = 0; o < out_dim; ++o) gemm_flat_sym32(type, raw + o * rb, a, &yt[o * n_tokens]);
    } else {
        ActQ8K a;
        a.quantize(x, in_dim, n_tokens);
#pragma omp parallel
        {
            KRow w;
#pragma omp for schedule(static)
            for (size_t o = 0; o < out_dim; ++o) {
                if (type == OREF_TYPE_Q4_K || type == OREF_TYPE_Q5_K) {
                    if (type == OREF_TYPE_Q4_K) unpack_k_q4_k(raw + o * rb, in_dim, w);
                    else unpack_k_q5_k(raw + o * rb, in_dim, w);
                    gemm_k_q4_k(w, a, &yt[o * n_tokens]);
                } else {
                    unpack_k_q6_k(raw + o * rb, in_dim, w);
                    gemm_k_q6_k(w, a, &yt[o * n_tokens]);
                }
            }
        }
    }
#pragma omp parallel for schedule(static)
    for (size_t t = 0; t < n_tokens; ++t)
        for (size_t o = 0; o < out_dim; ++o) y[t * out_dim + o] = yt[o * n_tokens + t];
    return 0;
}

int oref_matmul_decode(const float *x, size_t n_tokens, const uint8_t *raw, uint32_t type, size_t in_dim, size_t out_dim, float *y, int n_threads) {
    if (!supported(type, in_dim)) return -1;
    set_threads(n_threads);
    for (size_t t = 0; t < n_tokens; ++t) gemv_token(x + t * in_dim, raw, type, in_dim, out_dim, y + t * out_dim, 1);
    return 0;
}

int oref_matmul_dequant(const float *x, size_t n_tokens, const uint8_t *raw, uint32_t type, size_t in_dim, size_t out_dim, float *y, int n_threads) {
    int64_t rb = oref_row_bytes(type, in_dim);
    if (rb < 0) return -1;
    set_threads(n_threads);
#pragma omp parallel
    {
        std::vector<float> w(in_dim);
#pragma omp for schedule(static)
        for (size_t o = 0; o < out_dim; ++o) {
            oref_dequantize(type, raw + o * (size_t)rb, in_dim, w.data());
            for (size_t t = 0; t < n_tokens; ++t) y[t * out_dim + o] = oref_dot(x + t * in_dim, w.data(), in_dim);
        }
    }
    return 0;
}

/* E/tensor.rs:393-430 (the portable form: eight chains, pairwise fold, scalar tail) */
float oref_dot(const float *a, const float *b, size_t n) {
    float acc0[4] = {0, 0, 0, 0}, acc1[4] = {0, 0, 0, 0};
    size_t chunks = n / 8;
    for (size_t c = 0; c < chunks; ++c) {
        const float *x = a + c * 8, *y = b + c * 8;
        for (int lane = 0; lane < 4; ++lane) {
            acc0[lane] += x[lane] * y[lane];
            acc1[lane] += x[4 + lane] * y[4 + lane];
        }
    }
    float total = ((acc0[0] + acc1[0]) + (acc0[1] + acc1[1])) + ((acc0[2] + acc1[2]) + (acc0[3] + acc1[3]));
    for (size_t i = chunks * 8; i < n; ++i) total += a[i] * b[i];
    return total;
}

/* E/tensor.rs:743-749 */
void oref_rmsnorm(float *dst, const float *src, const float *weight, size_t n_tokens, size_t dim, float eps) {
    for (size_t t = 0; t < n_tokens; ++t) {
        const float *row = src + t * dim;
        float *out = dst + t * dim;
        float sum = 0.0f;
        for (size_t i = 0; i < dim; ++i) sum += row[i] * row[i];
        float mean_sq = sum / (float)dim;
        float scale = 1.0f / sqrtf(mean_sq + eps);
        for (size_t i = 0; i < dim; ++i) out[i] = row[i] * scale * weight[i];
    }
}

/* E/tensor.rs:1140-1160 with ext_factor 0, freq_scale 1, mscale 1, no freq factors */
void oref_rope_table(float *sin_cos, size_t n_pos, size_t rope_dim, float freq_base) {
    size_t half = rope_dim / 2;
    for (size_t pos = 0; pos < n_pos; ++pos) {
        for (size_t i = 0; i < half; ++i) {
            float freq = powf(freq_base, -2.0f * (float)i / (float)rope_dim);
            float theta_extrap = (float)pos * freq;
            float theta = 1.0f * theta_extrap;
            sin_cos[(pos * half + i) * 2] = sinf(theta) * 1.0f;
            sin_cos[(pos * half + i) * 2 + 1] = cosf(theta) * 1.0f;
        }
    }
}

/* E/tensor.rs:1162-1176, RopeLayout::Norm */
static void rope_norm_ff(float *x, size_t n_head, size_t head_dim, size_t pos, size_t rope_dim, float freq_base, const float *freq_factors,
                         int neox = 0);

void oref_rope_layout(float *x, size_t n_head, size_t head_dim, size_t pos, size_t rope_dim, float freq_base, const float *freq_factors, int neox) {
    rope_norm_ff(x, n_head, head_dim, pos, rope_dim, freq_base, freq_factors, neox);
}

void oref_rope_norm(float *x, size_t n_head, size_t head_dim, size_t pos, size_t rope_dim, float freq_base) {
    rope_norm_ff(x, n_head, head_dim, pos, rope_dim, freq_base, nullptr);
}

/* E/tensor.rs:1140-1176 with optional frequency factors (freq /= ff[i], :1143-1145); the pairing is :1167-1170 */
static void rope_norm_ff(float *x, size_t n_head, size_t head_dim, size_t pos, size_t rope_dim, float freq_base, const float *freq_factors, int neox) {
    size_t half = rope_dim / 2;
    std::vector<float> rot(half * 2);
    for (size_t i = 0; i < half; ++i) {
        float freq = powf(freq_base, -2.0f * (float)i / (float)rope_dim);
        if (freq_factors) freq /= freq_factors[i];
        float theta = 1.0f * ((float)pos * freq);
        rot[2 * i] = sinf(theta) * 1.0f;
        rot[2 * i + 1] = cosf(theta) * 1.0f;
    }
    for (size_t h = 0; h < n_head; ++h) {
        float *head = x + h * head_dim;
        for (size_t i = 0; i < half; ++i) {
            float sn = rot[2 * i], cs = rot[2 * i + 1];
            size_t lo = neox ? i : 2 * i, hi = neox ? i + half : 2 * i + 1;
            float a = head[lo], b = head[hi];
            head[lo] = a * cs - b * sn;
            head[hi] = a * sn + b * cs;
        }
    }
}

/* E/tensor.rs:809-821 */
void oref_softmax(float *x, size_t n) {
    float mx = -INFINITY;
    for (size_t i = 0; i < n; ++i) mx = fmaxf(mx, x[i]);
    float sum = 0.0f;
    for (size_t i = 0; i < n; ++i) {
        x[i] = exp_f32(x[i] - mx);
        sum += x[i];
    }
    if (sum > 0.0f)
        for (size_t i = 0; i < n; ++i) x[i] /= sum;
}

float oref_silu(float x) { return x / (1.0f + exp_f32(-x)); }

void oref_swiglu(float *gate, const float *up, size_t n) {
    for (size_t i = 0; i < n; ++i) gate[i] = oref_silu(gate[i]);
    for (size_t i = 0; i < n; ++i) gate[i] *= up[i];
}

void oref_add(float *a, const float *b, size_t n) {
    for (size_t i = 0; i < n; ++i) a[i] += b[i];
}

void oref_attention(float *out, const float *q, const float *k, const float *v, size_t kv_dim, size_t n_head, size_t group_size,
                    size_t head_dim, float scale, size_t n_tokens, size_t start_pos, int n_threads) {
    set_threads(n_threads);
    size_t row = n_head * head_dim;
#pragma omp parallel
    {
        std::vector<float> scores;
#pragma omp for schedule(dynamic, 1) collapse(2)
        for (size_t t = 0; t < n_tokens; ++t) {
            for (size_t h = 0; h < n_head; ++h) {
                size_t window_end = start_pos + t;
                size_t n_pos = window_end + 1;
                size_t kv_head = h / group_size;
                const float *qh = q + t * row + h * head_dim;
                float *o = out + t * row + h * head_dim;
                for (size_t i = 0; i < head_dim; ++i) o[i] = 0.0f;
                scores.resize(n_pos);
                for (size_t p = 0; p < n_pos; ++p)
                    scores[p] = oref_dot(qh, k + p * kv_dim + kv_head * head_dim, head_dim) * scale;
                oref_softmax(scores.data(), n_pos);
                for (size_t p = 0; p < n_pos; ++p) {
                    const float *vh = v + p * kv_dim + kv_head * head_dim;
                    float w = scores[p];
                    for (size_t i = 0; i < head_dim; ++i) o[i] += w * vh[i]; /* E/tensor.rs:679-681: multiply, then add */
                }
            }
        }
    }
}

/* E/sampling.rs:336-343: max_by(total_cmp) keeps the LAST of equal maxima */
uint32_t oref_argmax(const float *logits, size_t n) {
    if (n == 0) return 0;
    auto key = [](float f) -> int32_t {
        int32_t b = (int32_t)f32_bits(f);
        return b ^ (int32_t)(((uint32_t)(b >> 31)) >> 1); /* f32::total_cmp ordering key */
    };
    size_t best = 0;
    int32_t bk = key(logits[0]);
    for (size_t i = 1; i < n; ++i) {
        int32_t kk = key(logits[i]);
        if (kk >= bk) {
            bk = kk;
            best = i;
        }
    }
    return (uint32_t)best;
}

void oref_repeat_penalty(float *logits, size_t n_vocab, const uint32_t *recent, size_t n_recent, size_t repeat_last_n, float penalty) {
    if (penalty == 1.0f || n_recent == 0) return;
    size_t start = n_recent > repeat_last_n ? n_recent - repeat_last_n : 0;
    for (size_t i = start; i < n_recent; ++i) {
        uint32_t tok = recent[i];
        if (tok < n_vocab) {
            float v = logits[tok];
            logits[tok] = v > 0.0f ? v / penalty : v * penalty;
        }
    }
}

/* ---- Llama graph --------------------------------------------------------- */

struct oref_model {
    oref_config cfg;
    oref_matrix token_embd, output;
    const float *output_norm;
    std::vector<oref_layer> layers;
};

struct oref_kv {
    size_t capacity, kv_dim, len;
    int f16;
    std::vector<std::vector<float>> k, v; /* per layer [pos][kv_dim] */
};

oref_model *oref_model_create(const oref_config *cfg, const oref_matrix *token_embd, const float *output_norm, const oref_matrix *output,
                              const oref_layer *layers) {
    oref_model *m = new oref_model;
    m->cfg = *cfg;
    m->token_embd = *token_embd;
    m->output = output ? *output : *token_embd; /* tied output, E/arch/llama.rs:133-139 */
    m->output_norm = output_norm;
    m->layers.assign(layers, layers + cfg->n_layer);
    return m;
}
void oref_model_destroy(oref_model *m) { delete m; }

oref_kv *oref_kv_create(const oref_model *m, size_t capacity, int kv_f16) {
    oref_kv *kv = new oref_kv;
    kv->capacity = capacity;
    kv->kv_dim = (size_t)m->cfg.n_head_kv * m->cfg.head_dim;
    kv->len = 0;
    kv->f16 = kv_f16;
    kv->k.resize(m->cfg.n_layer);
    kv->v.resize(m->cfg.n_layer);
    for (auto &x : kv->k) x.reserve(capacity * kv->kv_dim);
    for (auto &x : kv->v) x.reserve(capacity * kv->kv_dim);
    return kv;
}
void oref_kv_destroy(oref_kv *kv) { delete kv; }
size_t oref_kv_len(const oref_kv *kv) { return kv->len; }
void oref_kv_truncate(oref_kv *kv, size_t len) {
    if (len >= kv->len) return;
    kv->len = len;
    for (auto &x : kv->k) x.resize(len * kv->kv_dim);
    for (auto &x : kv->v) x.resize(len * kv->kv_dim);
}

static int mm(const float *x, size_t n_tokens, const oref_matrix &w, float *y, int n_threads) {
    return oref_matmul(x, n_tokens, w.data, w.type, w.in_dim, w.out_dim, y, n_threads);
}

int oref_forward(const oref_model *m, oref_kv *kv, const uint32_t *tokens, size_t n_tokens, size_t start_pos, float *logits,
                 float *hidden_out, int n_threads) {
    const oref_config &c = m->cfg;
    size_t n_embd = c.n_embd, head_dim = c.head_dim, n_head = c.n_head, n_head_kv = c.n_head_kv;
    size_t kv_dim = n_head_kv * head_dim, q_dim = n_head * head_dim, n_ff = c.n_ff;
    if (n_tokens == 0 || start_pos != kv->len || start_pos + n_tokens > kv->capacity) return -1;
    set_threads(n_threads);

    std::vector<float> x(n_tokens * n_embd), normed(n_tokens * n_embd), q(n_tokens * q_dim), k(n_tokens * kv_dim), v(n_tokens * kv_dim),
        attn_out(n_tokens * q_dim), proj(n_tokens * n_embd), gate(n_tokens * n_ff), up(n_tokens * n_ff);
    int64_t erb = oref_row_bytes(m->token_embd.type, n_embd);
    for (size_t t = 0; t < n_tokens; ++t) { /* E/arch/llama.rs:608-614 */
        if (tokens[t] >= c.n_vocab) return -2;
        oref_dequantize(m->token_embd.type, m->token_embd.data + (size_t)tokens[t] * (size_t)erb, n_embd, &x[t * n_embd]);
    }
    float scale = 1.0f / sqrtf((float)head_dim); /* E/arch/llama.rs:823 */

    for (size_t li = 0; li < c.n_layer; ++li) {
        const oref_layer &L = m->layers[li];
        oref_rmsnorm(normed.data(), x.data(), L.attn_norm, n_tokens, n_embd, c.rms_eps);
        if (mm(normed.data(), n_tokens, L.wq, q.data(), n_threads)) return -3;
        if (mm(normed.data(), n_tokens, L.wk, k.data(), n_threads)) return -3;
        if (mm(normed.data(), n_tokens, L.wv, v.data(), n_threads)) return -3;
        /* E/arch/llama.rs:750-780: biases (add_bias_per_row, E/tensor.rs:1233-1239), then the per-head RMSNorm of q and k */
        for (size_t t = 0; t < n_tokens; ++t) {
            if (L.q_bias) oref_add(&q[t * q_dim], L.q_bias, q_dim);
            if (L.k_bias) oref_add(&k[t * kv_dim], L.k_bias, kv_dim);
            if (L.v_bias) oref_add(&v[t * kv_dim], L.v_bias, kv_dim);
        }
        if (L.q_norm) oref_rmsnorm(q.data(), q.data(), L.q_norm, n_tokens * n_head, head_dim, c.rms_eps);
        if (L.k_norm) oref_rmsnorm(k.data(), k.data(), L.k_norm, n_tokens * n_head_kv, head_dim, c.rms_eps);
        std::vector<float> &ck = kv->k[li], &cv = kv->v[li];
        for (size_t t = 0; t < n_tokens; ++t) { /* E/arch/llama.rs:787-809 */
            size_t pos = start_pos + t;
            rope_norm_ff(&q[t * q_dim], n_head, head_dim, pos, c.rope_dim, c.rope_freq_base, c.rope_freqs, (int)c.rope_neox);
            rope_norm_ff(&k[t * kv_dim], n_head_kv, head_dim, pos, c.rope_dim, c.rope_freq_base, c.rope_freqs, (int)c.rope_neox);
            for (size_t i = 0; i < kv_dim; ++i) {
                float kk = k[t * kv_dim + i], vv = v[t * kv_dim + i];
                if (kv->f16) {
                    kk = f16_to_f32(f32_to_f16(kk));
                    vv = f16_to_f32(f32_to_f16(vv));
                }
                ck.push_back(kk);
                cv.push_back(vv);
            }
        }
        oref_attention(attn_out.data(), q.data(), ck.data(), cv.data(), kv_dim, n_head, (n_head + n_head_kv - 1) / n_head_kv, head_dim, scale,
                       n_tokens, start_pos, n_threads);
        if (mm(attn_out.data(), n_tokens, L.wo, proj.data(), n_threads)) return -3;
        oref_add(x.data(), proj.data(), n_tokens * n_embd);
        oref_rmsnorm(normed.data(), x.data(), L.ffn_norm, n_tokens, n_embd, c.rms_eps);
        if (mm(normed.data(), n_tokens, L.w_gate, gate.data(), n_threads)) return -3;
        if (mm(normed.data(), n_tokens, L.w_up, up.data(), n_threads)) return -3;
        oref_swiglu(gate.data(), up.data(), n_tokens * n_ff);
        if (mm(gate.data(), n_tokens, L.w_down, proj.data(), n_threads)) return -3;
        oref_add(x.data(), proj.data(), n_tokens * n_embd);
    }
    kv->len = start_pos + n_tokens;
    if (hidden_out) memcpy(hidden_out, x.data(), n_tokens * n_embd * sizeof(float));
    if (logits) { /* E/arch/llama.rs:1026-1030 */
        std::vector<float> last(x.begin() + (n_tokens - 1) * n_embd, x.end());
        oref_rmsnorm(last.data(), last.data(), m->output_norm, 1, n_embd, c.rms_eps);
        if (mm(last.data(), 1, m->output, logits, n_threads)) return -3;
    }
    return 0;
}

int oref_hardware_threads(void) {
#ifdef _OPENMP
    return omp_get_num_procs();
#else
    return 1;
#endif
}

} /* extern "C" */
