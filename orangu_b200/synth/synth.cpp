/*
 * Synthetic weight builder: seeded N(0, std^2) matrices quantized into GGUF block
 * layouts (Q8_0, Q4_K, Q6_K).  Host-side helper for tests and benchmarks; real
 * checkpoints cannot be downloaded where this runs, and the reference engine only
 * reads GGUF files -- it has no weight quantizer -- so the quantizers here are
 * written from the format definitions (the decode rules in the reference's
 * src/bin/orangu-server/engine/quant.rs:639-649, 666-697, 746-787).  Any byte
 * pattern those rules decode is valid input; parity never depends on how the bytes
 * were chosen, only on both sides reading the same ones.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <vector>

#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

inline uint64_t mix64(uint64_t z) {
    z += 0x9e3779b97f4a7c15ull;
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
}

/* Two standard normals from one 64-bit counter hash (Box-Muller). */
inline void normal_pair(uint64_t seed, uint64_t counter, float *a, float *b) {
    uint64_t h = mix64(seed ^ mix64(counter));
    float u1 = ((float)(uint32_t)(h >> 40) + 0.5f) * (1.0f / 16777216.0f); /* (0,1) */
    float u2 = ((float)(uint32_t)((h >> 8) & 0xffffffu)) * (1.0f / 16777216.0f);
    float r = sqrtf(-2.0f * logf(u1));
    float phi = 6.28318530717958647692f * u2;
    *a = r * cosf(phi);
    *b = r * sinf(phi);
}

void fill_normal(float *out, size_t first, size_t n, uint64_t seed, float std) {
    /* element e comes from pair e/2, so any sub-range reproduces the same values */
    size_t e = first, end = first + n;
    while (e < end) {
        float a, b;
        normal_pair(seed, e / 2, &a, &b);
        if (e & 1) {
            out[e - first] = b * std;
            e += 1;
        } else {
            out[e - first] = a * std;
            if (e + 1 < end) out[e + 1 - first] = b * std;
            e += 2;
        }
    }
}

inline uint16_t f32_to_f16(float v) {
    uint32_t x;
    memcpy(&x, &v, 4);
    uint32_t sign = (x >> 16) & 0x8000u, mag = x & 0x7fffffffu;
    if (mag >= 0x7f800000u) return (uint16_t)(sign | (mag == 0x7f800000u ? 0x7c00u : 0x7e00u));
    if (mag >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);
    if (mag < 0x33000001u) return (uint16_t)sign;
    int32_t e = (int32_t)(mag >> 23) - 127;
    uint32_t m = (mag & 0x7fffffu) | 0x800000u, shift, base;
    if (e < -14) {
        shift = (uint32_t)(13 + (-14 - e));
        base = 0;
    } else {
        shift = 13;
        base = (uint32_t)(e + 15) << 10;
        m &= 0x7fffffu;
    }
    uint32_t q = m >> shift, rem = m & ((1u << shift) - 1u), half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u))) q += 1;
    return (uint16_t)(sign | (base + q));
}

inline float f16_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16, exp = (h >> 10) & 0x1f, man = h & 0x3ffu, out;
    if (exp == 0) {
        if (man == 0) {
            out = sign;
        } else {
            int e = -1;
            do {
                man <<= 1;
                ++e;
            } while (!(man & 0x400u));
            out = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
        }
    } else if (exp == 31) {
        out = sign | 0x7f800000u | (man << 13);
    } else {
        out = sign | ((exp + 112) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &out, 4);
    return f;
}

inline void put_f16(uint8_t *p, uint16_t h) {
    p[0] = (uint8_t)(h & 0xff);
    p[1] = (uint8_t)(h >> 8);
}

inline int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

/* Q8_0: d = amax/127 stored as f16; codes = round_half_away(x / d). 34 bytes per 32. */
void quantize_q8_0(const float *x, size_t n, uint8_t *out) {
    for (size_t b = 0; b < n / 32; ++b) {
        const float *v = x + b * 32;
        uint8_t *blk = out + b * 34;
        float amax = 0;
        for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(v[i]));
        float d = amax / 127.0f;
        float inv = d > 0 ? 1.0f / d : 0.0f;
        put_f16(blk, f32_to_f16(d));
        for (int i = 0; i < 32; ++i) blk[2 + i] = (uint8_t)(int8_t)clampi((int)roundf(v[i] * inv), -127, 127);
    }
}

/* Q4_K: eight affine sub-blocks of 32 (x ~ scale*q - min, q in 0..15), the eight scales and mins
 * themselves stored as 6-bit multiples of two f16 super-block factors d and dmin. 144 bytes per 256. */
void quantize_q4_k(const float *x, size_t n, uint8_t *out) {
    for (size_t s = 0; s < n / 256; ++s) {
        const float *v = x + s * 256;
        uint8_t *blk = out + s * 144;
        float scale[8], mn[8];
        float max_scale = 0, max_min = 0;
        for (int j = 0; j < 8; ++j) {
            float lo = 0.0f, hi = 0.0f; /* the grid always contains zero, so min <= 0 <= max */
            for (int i = 0; i < 32; ++i) {
                lo = fminf(lo, v[j * 32 + i]);
                hi = fmaxf(hi, v[j * 32 + i]);
            }
            scale[j] = (hi - lo) / 15.0f;
            mn[j] = -lo;
            max_scale = fmaxf(max_scale, scale[j]);
            max_min = fmaxf(max_min, mn[j]);
        }
        uint16_t dh = f32_to_f16(max_scale / 63.0f), dmh = f32_to_f16(max_min / 63.0f);
        float d = f16_to_f32(dh), dmin = f16_to_f32(dmh);
        put_f16(blk, dh);
        put_f16(blk + 2, dmh);
        uint8_t sc[8], m[8];
        for (int j = 0; j < 8; ++j) {
            sc[j] = (uint8_t)clampi(d > 0 ? (int)roundf(scale[j] / d) : 0, 0, 63);
            m[j] = (uint8_t)clampi(dmin > 0 ? (int)roundf(mn[j] / dmin) : 0, 0, 63);
        }
        uint8_t *ps = blk + 4;
        for (int j = 0; j < 4; ++j) {
            ps[j] = (uint8_t)((sc[j] & 63) | ((sc[j + 4] >> 4) << 6));
            ps[j + 4] = (uint8_t)((m[j] & 63) | ((m[j + 4] >> 4) << 6));
            ps[j + 8] = (uint8_t)((sc[j + 4] & 0xF) | ((m[j + 4] & 0xF) << 4));
        }
        uint8_t *qs = blk + 16;
        for (int g = 0; g < 4; ++g) {
            float dl0 = d * sc[2 * g], ml0 = dmin * m[2 * g];
            float dl1 = d * sc[2 * g + 1], ml1 = dmin * m[2 * g + 1];
            float il0 = dl0 > 0 ? 1.0f / dl0 : 0.0f, il1 = dl1 > 0 ? 1.0f / dl1 : 0.0f;
            for (int i = 0; i < 32; ++i) {
                int q0 = clampi((int)roundf((v[64 * g + i] + ml0) * il0), 0, 15);
                int q1 = clampi((int)roundf((v[64 * g + 32 + i] + ml1) * il1), 0, 15);
                qs[32 * g + i] = (uint8_t)(q0 | (q1 << 4));
            }
        }
    }
}

/* Q6_K: sixteen symmetric groups of 16 (x ~ d*sc*q, q in -32..31), sc a signed 8-bit multiple of one
 * f16 factor d.  Each group's largest-magnitude value is mapped to the code -32, the one extreme the
 * 6-bit range has a full step for, so the group scale takes the opposite sign of that value. 210 bytes per 256. */
void quantize_q6_k(const float *x, size_t n, uint8_t *out) {
    for (size_t s = 0; s < n / 256; ++s) {
        const float *v = x + s * 256;
        uint8_t *blk = out + s * 210;
        float gs[16];
        float max_abs_scale = 0;
        for (int g = 0; g < 16; ++g) {
            float ext = 0;
            for (int i = 0; i < 16; ++i)
                if (fabsf(v[g * 16 + i]) > fabsf(ext)) ext = v[g * 16 + i];
            gs[g] = ext / -32.0f;
            max_abs_scale = fmaxf(max_abs_scale, fabsf(gs[g]));
        }
        uint16_t dh = f32_to_f16(max_abs_scale / 127.0f);
        float d = f16_to_f32(dh);
        int8_t sc[16];
        int8_t q[256];
        for (int g = 0; g < 16; ++g) {
            sc[g] = (int8_t)clampi(d > 0 ? (int)roundf(gs[g] / d) : 0, -127, 127);
            float step = d * (float)sc[g];
            float inv = step != 0 ? 1.0f / step : 0.0f;
            for (int i = 0; i < 16; ++i) q[g * 16 + i] = (int8_t)clampi((int)roundf(v[g * 16 + i] * inv), -32, 31);
        }
        uint8_t *ql = blk, *qh = blk + 128;
        memset(blk, 0, 192);
        for (int h = 0; h < 2; ++h) {
            for (int l = 0; l < 32; ++l) {
                int c1 = q[128 * h + l] + 32, c2 = q[128 * h + 32 + l] + 32, c3 = q[128 * h + 64 + l] + 32, c4 = q[128 * h + 96 + l] + 32;
                ql[64 * h + l] = (uint8_t)((c1 & 0xF) | ((c3 & 0xF) << 4));
                ql[64 * h + 32 + l] = (uint8_t)((c2 & 0xF) | ((c4 & 0xF) << 4));
                qh[32 * h + l] = (uint8_t)((c1 >> 4) | ((c2 >> 4) << 2) | ((c3 >> 4) << 4) | ((c4 >> 4) << 6));
            }
        }
        memcpy(blk + 192, sc, 16);
        put_f16(blk + 208, dh);
    }
}

size_t row_bytes(uint32_t type, size_t in_dim) {
    switch (type) {
    case 8: return in_dim % 32 ? 0 : in_dim / 32 * 34;
    case 12: return in_dim % 256 ? 0 : in_dim / 256 * 144;
    case 14: return in_dim % 256 ? 0 : in_dim / 256 * 210;
    default: return 0;
    }
}

void quantize_row(uint32_t type, const float *x, size_t n, uint8_t *out) {
    if (type == 8) quantize_q8_0(x, n, out);
    else if (type == 12) quantize_q4_k(x, n, out);
    else quantize_q6_k(x, n, out);
}

} // namespace

extern "C" {

void obs_fill_normal(float *out, size_t n, uint64_t seed, float std) {
    const size_t chunk = 1 << 16;
    size_t n_chunks = (n + chunk - 1) / chunk;
#pragma omp parallel for schedule(static)
    for (size_t c = 0; c < n_chunks; ++c) {
        size_t first = c * chunk;
        fill_normal(out + first, first, std::min(chunk, n - first), seed, std);
    }
}

int obs_quantize_rows(uint32_t type, const float *w, size_t n_rows, size_t in_dim, uint8_t *out) {
    size_t rb = row_bytes(type, in_dim);
    if (!rb) return -1;
#pragma omp parallel for schedule(static)
    for (size_t r = 0; r < n_rows; ++r) quantize_row(type, w + r * in_dim, in_dim, out + r * rb);
    return 0;
}

/* [out_dim][in_dim] ~ N(0, std^2) from `seed`, quantized row by row; the fp32 matrix is never held whole. */
int obs_synth_matrix(uint32_t type, uint64_t seed, float std, size_t out_dim, size_t in_dim, uint8_t *out) {
    size_t rb = row_bytes(type, in_dim);
    if (!rb) return -1;
#pragma omp parallel
    {
        std::vector<float> row(in_dim);
#pragma omp for schedule(static)
        for (size_t r = 0; r < out_dim; ++r) {
            fill_normal(row.data(), r * in_dim, in_dim, seed, std);
            quantize_row(type, row.data(), in_dim, out + r * rb);
        }
    }
    return 0;
}

/* Rows [row0, row0 + n_rows) x columns [col0, col0 + n_cols) of the matrix obs_synth_matrix(type, seed, std, *, in_dim)
 * makes, quantized: the values come from a counter-based generator and the block quantizers work block by block, so a
 * shard is produced directly, bit-identical to the same region cut out of the whole matrix (col0 and n_cols are whole
 * blocks).  This is what lets every rank of a tensor-parallel run build only its own slices of a large model. */
int obs_synth_matrix_slice(uint32_t type, uint64_t seed, float std, size_t in_dim, size_t row0, size_t n_rows, size_t col0, size_t n_cols, uint8_t *out) {
    size_t rb = row_bytes(type, n_cols);
    if (!rb || !row_bytes(type, in_dim) || col0 + n_cols > in_dim || !row_bytes(type, col0 ? col0 : n_cols)) return -1;
#pragma omp parallel
    {
        std::vector<float> row(n_cols);
#pragma omp for schedule(static)
        for (size_t r = 0; r < n_rows; ++r) {
            fill_normal(row.data(), (row0 + r) * in_dim + col0, n_cols, seed, std);
            quantize_row(type, row.data(), n_cols, out + r * rb);
        }
    }
    return 0;
}

} /* extern "C" */
