// GGUF block formats on the device: re-layout at registration and exact dequantisation.
//
// Dequantisation follows the reference's decode rules operation for operation
// (src/bin/orangu-server/engine/quant.rs:639-649 Q8_0, :666-697 Q4_K, :703-742 Q5_K, :746-787 Q6_K),
// so a row read back from the device equals QuantMatrix::row bit for bit.
#include "common.cuh"
#include "kernels.h"

namespace ob {

// One thread per destination block.  src rows are GGUF rows of `src_row_bytes`; the
// destination takes blocks [blk0, blk0+nb) of rows [row0, row0+n_rows).
// The 16 levels an IQ4_NL nibble indexes (engine/iq_grids.rs:5941; a constant of the format).
__constant__ int8_t IQ4NL_LEVELS[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};

__global__ void repack_kernel(const uint8_t *__restrict__ src, uint64_t src_row_bytes, uint32_t src_type, uint32_t row0, uint32_t blk0, DevWeight w) {
    uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    uint64_t total = (uint64_t)w.out_dim * w.nb;
    if (idx >= total) return;
    uint32_t r = (uint32_t)(idx / w.nb), b = (uint32_t)(idx % w.nb);
    const uint8_t *s = src + (uint64_t)(row0 + r) * src_row_bytes + (uint64_t)(blk0 + b) * block_bytes_gguf(src_type);
    uint8_t *drow = const_cast<uint8_t *>(w.data) + (uint64_t)r * w.row_stride;
    if (is_sym32_source(src_type)) {
        // low nibbles are elements 0..15, high nibbles 16..31; Q5_0 adds a fifth bit per element from the 32-bit qh and
        // subtracts 16, Q4_0 subtracts 8, IQ4_NL looks the nibble up (engine/vecdot.rs:1001-1016, :1019-1038)
        int8_t *d = reinterpret_cast<int8_t *>(drow + (uint64_t)b * 32);
        const bool five = src_type == TYPE_Q5_0;
        const uint32_t qh = five ? ((uint32_t)s[2] | ((uint32_t)s[3] << 8) | ((uint32_t)s[4] << 16) | ((uint32_t)s[5] << 24)) : 0u;
        const uint8_t *qs = s + (five ? 6 : 2);
        const int bias = five ? 16 : 8;
        for (int j = 0; j < 16; ++j) {
            if (src_type == TYPE_IQ4_NL) {
                d[j] = IQ4NL_LEVELS[qs[j] & 0x0F];
                d[16 + j] = IQ4NL_LEVELS[qs[j] >> 4];
            } else {
                const uint32_t hi_lo = ((qh >> j) << 4) & 0x10, hi_hi = (qh >> (j + 12)) & 0x10;
                d[j] = (int8_t)((int)((qs[j] & 0x0Fu) | hi_lo) - bias);
                d[16 + j] = (int8_t)((int)((uint32_t)(qs[j] >> 4) | hi_hi) - bias);
            }
        }
        drow[w.d_off + 2 * b] = s[0];
        drow[w.d_off + 2 * b + 1] = s[1];
    } else if (w.type == TYPE_Q4_K) {
        uint8_t *d = drow + (uint64_t)b * 144;
        for (int i = 0; i < 144; ++i) d[i] = s[i];
    } else if (w.type == TYPE_Q5_K) {
        uint8_t *d = drow + (uint64_t)b * 176;
        for (int i = 0; i < 176; ++i) d[i] = s[i];
    } else if (w.type == TYPE_Q6_K) {
        uint8_t *d = drow + (uint64_t)b * 208;
        for (int i = 0; i < 208; ++i) d[i] = s[i];
        drow[w.d_off + 2 * b] = s[208];
        drow[w.d_off + 2 * b + 1] = s[209];
    } else {  // Q8_0
        uint8_t *d = drow + (uint64_t)b * 32;
        for (int i = 0; i < 32; ++i) d[i] = s[2 + i];
        drow[w.d_off + 2 * b] = s[0];
        drow[w.d_off + 2 * b + 1] = s[1];
    }
}

__device__ __forceinline__ void scale_min_k4(int j, const uint8_t *q, int &sc, int &m) {
    if (j < 4) {
        sc = q[j] & 63;
        m = q[j + 4] & 63;
    } else {
        sc = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4);
        m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
    }
}

// Element e of row r, decoded exactly as the reference decodes it.
__device__ float dequant_element(const DevWeight &w, uint32_t r, uint32_t e) {
    const uint8_t *row = w.data + (uint64_t)r * w.row_stride;
    if (w.type == TYPE_Q8_0) {
        uint32_t b = e >> 5;
        float d = f16_bits_to_f32(row[w.d_off + 2 * b] | (row[w.d_off + 2 * b + 1] << 8));
        return __fmul_rn((float)(int8_t)row[b * 32 + (e & 31)], d);
    }
    uint32_t b = e >> 8, i = e & 255;
    if (w.type == TYPE_Q4_K) {
        const uint8_t *blk = row + (uint64_t)b * 144;
        float d = f16_bits_to_f32(blk[0] | (blk[1] << 8)), dmin = f16_bits_to_f32(blk[2] | (blk[3] << 8));
        int j = i >> 5, sc, m;
        scale_min_k4(j, blk + 4, sc, m);
        uint8_t byte = blk[16 + (j >> 1) * 32 + (i & 31)];
        int q = (j & 1) ? (byte >> 4) : (byte & 0x0F);
        float dl = __fmul_rn(d, (float)sc), ml = __fmul_rn(dmin, (float)m);
        return __fsub_rn(__fmul_rn(dl, (float)q), ml);
    }
    if (w.type == TYPE_Q5_K) {  // quant.rs:703-742
        const uint8_t *blk = row + (uint64_t)b * 176;
        float d = f16_bits_to_f32(blk[0] | (blk[1] << 8)), dmin = f16_bits_to_f32(blk[2] | (blk[3] << 8));
        int j = i >> 5, sc, m;
        scale_min_k4(j, blk + 4, sc, m);
        uint8_t byte = blk[48 + (j >> 1) * 32 + (i & 31)];
        int q = ((j & 1) ? (byte >> 4) : (byte & 0x0F)) + (((blk[16 + (i & 31)] >> j) & 1) ? 16 : 0);
        float dl = __fmul_rn(d, (float)sc), ml = __fmul_rn(dmin, (float)m);
        return __fsub_rn(__fmul_rn(dl, (float)q), ml);
    }
    // Q6_K
    const uint8_t *blk = row + (uint64_t)b * 208;
    float d = f16_bits_to_f32(row[w.d_off + 2 * b] | (row[w.d_off + 2 * b + 1] << 8));
    uint32_t h = i >> 7, rr = (i >> 5) & 3, l = i & 31;
    uint8_t qlb = blk[64 * h + 32 * (rr & 1) + l];
    uint8_t qhb = blk[128 + 32 * h + l];
    int lo = (rr & 2) ? (qlb >> 4) : (qlb & 0x0F);
    int q = (lo | (((qhb >> (2 * rr)) & 3) << 4)) - 32;
    int sc = (int8_t)blk[192 + (i >> 4)];
    return __fmul_rn(__fmul_rn(d, (float)sc), (float)q);
}

__global__ void dequant_rows_kernel(DevWeight w, uint32_t first_row, uint32_t n_rows, float *__restrict__ out) {
    uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    uint64_t total = (uint64_t)n_rows * w.in_dim;
    if (idx >= total) return;
    uint32_t r = (uint32_t)(idx / w.in_dim), e = (uint32_t)(idx % w.in_dim);
    out[idx] = dequant_element(w, first_row + r, e);
}

// Embedding lookup: out[t] = dequantised row tokens[t]  (llama.rs:608-614)
__global__ void embed_kernel(DevWeight w, const uint32_t *__restrict__ tokens, uint32_t n_tokens, float *__restrict__ out) {
    uint32_t t = blockIdx.y;
    uint32_t e = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= n_tokens || e >= w.in_dim) return;
    out[(uint64_t)t * w.in_dim + e] = dequant_element(w, tokens[t], e);
}

void launch_repack(const uint8_t *src, uint64_t src_row_bytes, uint32_t src_type, uint32_t row0, uint32_t blk0, const DevWeight &w, cudaStream_t st) {
    uint64_t total = (uint64_t)w.out_dim * w.nb;
    repack_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(src, src_row_bytes, src_type, row0, blk0, w);
}

void launch_dequant_rows(const DevWeight &w, uint32_t first_row, uint32_t n_rows, float *out, cudaStream_t st) {
    uint64_t total = (uint64_t)n_rows * w.in_dim;
    dequant_rows_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(w, first_row, n_rows, out);
}

void launch_embed(const DevWeight &w, const uint32_t *tokens, uint32_t n_tokens, float *out, cudaStream_t st) {
    dim3 grid((w.in_dim + 255) / 256, n_tokens);
    embed_kernel<<<grid, 256, 0, st>>>(w, tokens, n_tokens, out);
}

}  // namespace ob
