// Many-token products on the fifth-generation tensor cores: tcgen05.mma (kind::i8) with accumulators in tensor memory,
// operands brought into shared memory by TMA (cp.async.bulk.tensor, no multicast: every tensor map covers this GPU's own
// memory and every CTA fetches its own tiles).
//
// The arithmetic is the reference's, so the results equal the CPU's bit for bit at any batch size:
//   Q8_0 (engine/vecdot.rs:2598-2629 flat GEMM, :2829-2838 decode): acc += (ad_b * s_b) * (f32)dot32_b per block of 32, in
//   block order.  The int8 codes of a row are already a K-major int8 matrix, so TMA loads them straight into the
//   128-byte-swizzled operand layout.  One fp32 rounding per 32 elements means every K = 32 step needs its own integer
//   result: each tcgen05.mma (M = 128 rows, N = 64 tokens, K = 32) writes a fresh accumulator, four per pipeline step in
//   one half of tensor memory while the epilogue warps drain the other half (tcgen05.ld), scale and accumulate in fp32.
//
// Roles in a CTA of ten warps: warps 0-7 epilogue (warp w reads the 32 tensor-memory lanes of quadrant w % 4, token columns
// 32 * (w / 4) ..), warp 8 lane 0 issues the TMA loads, warp 9 allocates tensor memory and its lane 0 issues the MMAs.
// Stages and accumulator halves are handed over through mbarriers; every wait is bounded -- a wait that runs out sets a
// status word, makes all roles leave their loops, and the CTA frees its tensor memory and returns.
#include <atomic>

#include <cuda.h>  // CUtensorMap and its enums; cuTensorMapEncodeTiled is looked up through the runtime, libcuda is not linked

#include "common.cuh"
#include "kernels.h"

namespace ob {

namespace {

constexpr int TC_M = 128, TC_N = 64;
constexpr int TC_EPI_WARPS = 8;
constexpr int TC_TMA_WARP = 8, TC_MMA_WARP = 9;
constexpr int TC_THREADS = 10 * 32;
constexpr uint32_t TC_POLL_LIMIT = 1u << 22;  // polls of one wait before it gives up (tens of milliseconds)

__device__ uint32_t g_tc5_status;  // set to 1 when a wait ran out
std::atomic<bool> g_tc5_launched{false};  // host: a kernel of this file has been launched since the status was last read

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ---- mbarrier ------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory"); }
__device__ __forceinline__ void mbar_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// False when the wait was abandoned: this one ran out of polls, or another role's did (*abort is then set).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t *abort) {
    for (uint32_t i = 0; i < TC_POLL_LIMIT; ++i) {
        if (mbar_try(bar, parity)) return true;
        if ((i & 63u) == 63u && *abort) return false;
    }
    *abort = 1u;
    g_tc5_status = 1u;
    return false;
}

// ---- TMA -----------------------------------------------------------------------------------------------------------
// Tile at (x, y) of the tensor `tm` describes -> shared memory; completion counts on `bar`.  x * element size must be a
// multiple of 16 bytes (all callers pass multiples of 128 bytes or of four floats).
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *tm, int32_t x, int32_t y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
                 "l"(reinterpret_cast<uint64_t>(tm)), "r"(x), "r"(y), "r"(bar)
                 : "memory");
}

// ---- tensor memory and tcgen05 -----------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t slot, uint32_t cols) {  // one whole warp
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {  // the same warp
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D (tensor memory, int32, 128 lanes x N columns) [+]= A (128 x 32 int8, K-major) * B (N x 32 int8, K-major)^T
__device__ __forceinline__ void umma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// All MMAs this thread has issued so far arrive on `bar` when they have completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// This warp's 32 lanes x 32 consecutive columns: thread i gets lane i's words.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, "
        "%23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]),
          "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]),
          "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]),
                   "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile in the 128-byte swizzle: rows of 128 bytes, groups of eight rows 1024
// bytes apart, tile base 1024-byte aligned.  A K = 32 step inside the 128-byte row advances the start address by 32 bytes.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t saddr) {
    return (uint64_t)((saddr >> 4) & 0x3fffu) | (1ull << 16) /* leading byte offset: unused with a swizzle */ | (64ull << 32) /* 1024 B between row groups */ |
           (1ull << 46) /* descriptor version of this architecture */ | (2ull << 61) /* 128-byte swizzle */;
}
// Instruction descriptor: int32 accumulator, A and B signed (1) or unsigned (0) 8-bit, both K-major, N columns, M = 128.
__host__ __device__ constexpr uint32_t umma_idesc_i8(uint32_t a_signed, uint32_t b_signed, uint32_t n) {
    return (2u << 4) | (a_signed << 7) | (b_signed << 10) | ((n >> 3) << 17) | ((128u >> 4) << 24);
}

// ---- Q8_0 ------------------------------------------------------------------------------------------------------------
constexpr int Q8_STAGES = 4;
constexpr uint32_t Q8_A_BYTES = TC_M * 128, Q8_B_BYTES = TC_N * 128, Q8_XD_BYTES = TC_N * 16;
struct Q8Smem {  // offsets from the 1024-byte aligned base
    static constexpr uint32_t A = 0, B = A + Q8_STAGES * Q8_A_BYTES, XD = B + Q8_STAGES * Q8_B_BYTES, BAR = XD + Q8_STAGES * Q8_XD_BYTES;
    static constexpr uint32_t FULL = BAR, EMPTY = FULL + 8 * Q8_STAGES, ACC_FULL = EMPTY + 8 * Q8_STAGES, ACC_EMPTY = ACC_FULL + 16, SLOT = ACC_EMPTY + 16, ABORT = SLOT + 8;
    static constexpr uint32_t BYTES = ABORT + 8, ALLOC = BYTES + 1024;
};

struct TcQ8Args {
    GemvSegment seg;
    uint32_t n_tokens, n_steps;  // steps of four blocks (128 elements)
};

__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc5_q8_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_xd, TcQ8Args a) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem = smem_raw + (sbase - smem_u32(smem_raw));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t row0 = blockIdx.x * TC_M, tok0 = blockIdx.y * TC_N;
    volatile uint32_t *abort = reinterpret_cast<volatile uint32_t *>(smem + Q8Smem::ABORT);
    const uint32_t n_steps = a.n_steps;

    if (threadIdx.x == 0) {
        for (int s = 0; s < Q8_STAGES; ++s) {
            mbar_init(sbase + Q8Smem::FULL + 8 * s, 1);                  // the producer's expect_tx arrival
            mbar_init(sbase + Q8Smem::EMPTY + 8 * s, 1 + TC_EPI_WARPS);  // MMA completion + the epilogue warps (they read the token scales)
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(sbase + Q8Smem::ACC_FULL + 8 * b, 1);
            mbar_init(sbase + Q8Smem::ACC_EMPTY + 8 * b, TC_EPI_WARPS);
        }
        *abort = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == TC_MMA_WARP) tmem_alloc(sbase + Q8Smem::SLOT, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *reinterpret_cast<volatile uint32_t *>(smem + Q8Smem::SLOT);

    if (warp == TC_TMA_WARP) {
        if (lane == 0) {
            for (uint32_t it = 0; it < n_steps; ++it) {
                const uint32_t s = it % Q8_STAGES;
                if (it >= Q8_STAGES && !mbar_wait(sbase + Q8Smem::EMPTY + 8 * s, ((it / Q8_STAGES) & 1u) ^ 1u, abort)) break;
                const uint32_t full = sbase + Q8Smem::FULL + 8 * s;
                mbar_expect_tx(full, Q8_A_BYTES + Q8_B_BYTES + Q8_XD_BYTES);
                tma_load_2d(sbase + Q8Smem::A + s * Q8_A_BYTES, &tm_w, (int32_t)(it * 128), (int32_t)row0, full);
                tma_load_2d(sbase + Q8Smem::B + s * Q8_B_BYTES, &tm_x, (int32_t)(it * 128), (int32_t)tok0, full);
                tma_load_2d(sbase + Q8Smem::XD + s * Q8_XD_BYTES, &tm_xd, (int32_t)(it * 4), (int32_t)tok0, full);
            }
        }
    } else if (warp == TC_MMA_WARP) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_i8(1, 1, TC_N);
            for (uint32_t it = 0; it < n_steps; ++it) {
                const uint32_t s = it % Q8_STAGES, buf = it & 1u;
                if (!mbar_wait(sbase + Q8Smem::FULL + 8 * s, (it / Q8_STAGES) & 1u, abort)) break;
                if (it >= 2 && !mbar_wait(sbase + Q8Smem::ACC_EMPTY + 8 * buf, ((it / 2) & 1u) ^ 1u, abort)) break;
                tc_fence_after();
                const uint64_t da = umma_desc_sw128(sbase + Q8Smem::A + s * Q8_A_BYTES), db = umma_desc_sw128(sbase + Q8Smem::B + s * Q8_B_BYTES);
#pragma unroll
                for (uint32_t j = 0; j < 4; ++j)  // block j of the step: its own accumulator, nothing is added up on the tensor core
                    umma_i8(tmem + buf * 256 + j * TC_N, da + 2 * j, db + 2 * j, idesc, 0u);
                umma_commit(sbase + Q8Smem::EMPTY + 8 * s);
                umma_commit(sbase + Q8Smem::ACC_FULL + 8 * buf);
            }
        }
    } else {
        // ---- epilogue: thread = one row x 32 tokens
        const uint32_t quad = warp & 3u, half = warp >> 2;
        const uint32_t row = row0 + quad * 32 + lane;
        const bool row_ok = row < a.seg.w.out_dim;
        const uint8_t *wrow = a.seg.w.data + (uint64_t)min(row, a.seg.w.out_dim - 1) * a.seg.w.row_stride + a.seg.w.d_off;
        float acc[32];
#pragma unroll
        for (int t = 0; t < 32; ++t) acc[t] = 0.0f;
        uint2 sw_next = __ldg(reinterpret_cast<const uint2 *>(wrow));  // the row's four f16 block scales of step 0
        for (uint32_t it = 0; it < n_steps; ++it) {
            const uint32_t s = it % Q8_STAGES, buf = it & 1u;
            const uint2 swb = sw_next;
            if (it + 1 < n_steps) sw_next = __ldg(reinterpret_cast<const uint2 *>(wrow + 8 * (it + 1)));
            if (!mbar_wait(sbase + Q8Smem::ACC_FULL + 8 * buf, (it / 2) & 1u, abort)) break;
            tc_fence_after();
            const float sw[4] = {f16_bits_to_f32(swb.x & 0xffffu), f16_bits_to_f32(swb.x >> 16), f16_bits_to_f32(swb.y & 0xffffu), f16_bits_to_f32(swb.y >> 16)};
            const float4 *xd = reinterpret_cast<const float4 *>(smem + Q8Smem::XD + s * Q8_XD_BYTES) + half * 32;  // [token] the four block scales
#pragma unroll
            for (uint32_t j = 0; j < 4; ++j) {
                uint32_t r[32];
                tmem_ld32(tmem + ((quad * 32) << 16) + buf * 256 + j * TC_N + half * 32, r);
                tmem_ld_wait();
#pragma unroll
                for (int t = 0; t < 32; ++t) {
                    const float4 d4 = xd[t];
                    const float ad = j == 0 ? d4.x : j == 1 ? d4.y : j == 2 ? d4.z : d4.w;
                    acc[t] = __fadd_rn(acc[t], __fmul_rn(__fmul_rn(ad, sw[j]), (float)(int)r[t]));  // (ad_b * s_b) * dot32_b, vecdot.rs:2620
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(sbase + Q8Smem::ACC_EMPTY + 8 * buf);
                mbar_arrive(sbase + Q8Smem::EMPTY + 8 * s);
            }
        }
        if (!*abort && row_ok) {
#pragma unroll
            for (int t = 0; t < 32; ++t) {
                const uint32_t tok = tok0 + half * 32 + t;
                if (tok < a.n_tokens) {
                    const uint64_t o = (uint64_t)tok * a.seg.y_stride + row;
                    float v = acc[t];
                    if (a.seg.epilogue == EPI_ADD_RESIDUAL) v = __fadd_rn(a.seg.residual[o], v);
                    a.seg.y[o] = v;
                }
            }
        }
    }
    if (*abort) {  // let copies that are still in flight land before the shared memory goes away
        for (int i = 0; i < 200; ++i) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == TC_MMA_WARP) tmem_dealloc(tmem, 512);
}

// ---- Q4_K -----------------------------------------------------------------------------------------------------------
// The 4-bit codes cannot go to the tensor core as they are: every 32-element sub-block has its own 6-bit scale, and
// isum = sum_j sc_j * dot32_j has to be exact.  So the scale is folded into the operand, in two digits that keep every
// product inside a byte: sc = 8 * sc_hi + sc_lo (both 0..7), code * digit <= 105, and
//     isum = 8 * dot(code * sc_hi, x) + dot(code * sc_lo, x),      imin = dot(m_j(i), x)
// (the min term sum_j m_j * bsum_j is itself a dot product with the sub-block's min as the "weight" of each of its
// elements).  Eight expander warps turn each half super-block of 128 rows (TMA-loaded GGUF blocks) into those three
// unsigned-byte planes in the swizzled operand layout -- a packed 32-bit multiply scales four codes at once -- the MMA
// thread accumulates each plane over the super-block's eight K = 32 steps in its own tensor-memory accumulator, and the
// epilogue warps form the super-block's fp32 term per (row, token) in the CPU's association and order:
//   decode order   acc += ad * (d * isum - dmin * imin)                          (engine/vecdot.rs:3152-3178)
//   prefill order  first for every super-block acc -= (ad * dmin) * imin, then acc += ad * (d * isum)
//                  (engine/vecdot.rs:2119-2143, 2213-2255): two sweeps over K in one launch, the first over the block
//                  headers only (min plane), the accumulators staying in registers.
constexpr int K4_RING = 8;
constexpr int K4_EXP_WARPS = 4;
constexpr int K4_TMA_WARP = 12, K4_MMA_WARP = 13;
constexpr int K4_THREADS = 14 * 32;
constexpr uint32_t K4_RAW_BYTES = TC_M * 144, K4_PLANE_BYTES = TC_M * 128;
// N: tokens per CTA tile.  The tensor core fetches its operands from shared memory at a fixed rate, so an MMA's time goes
// with (128 + N) * 32 bytes rather than with its 128 * N * 32 multiply-adds: 128 tokens per tile amortise the three planes
// of the weights over twice the work of 64.  Tensor memory (512 columns) holds planes * N columns per accumulator buffer:
// two buffers for the prefill order (two planes at most), one for the decode order at N = 128 (three planes).
template <int N>
struct K4Smem {
    static constexpr uint32_t IN_STAGES = N == 64 ? 3 : 2;
    static constexpr uint32_t B_BYTES = 2 * N * 128;
    static constexpr uint32_t RAW = 0, B = RAW + IN_STAGES * K4_RAW_BYTES;          // a raw stage is 18 KB: B stays 1024-byte aligned
    static constexpr uint32_t PLANES = B + IN_STAGES * B_BYTES;                     // [2 stages][3 planes][128 x 128]
    static constexpr uint32_t XD = PLANES + 2 * 3 * K4_PLANE_BYTES;                  // [ring][N] token scales
    static constexpr uint32_t DD = XD + K4_RING * N * 4;                             // [ring][128] d | dmin << 16
    static constexpr uint32_t BAR = DD + K4_RING * TC_M * 4;
    static constexpr uint32_t IN_FULL = BAR, IN_EMPTY = IN_FULL + 32, PL_FULL = IN_EMPTY + 32, PL_EMPTY = PL_FULL + 16, ACC_FULL = PL_EMPTY + 16,
                              ACC_EMPTY = ACC_FULL + 16, SLOT = ACC_EMPTY + 16, ABORT = SLOT + 8;
    static constexpr uint32_t BYTES = ABORT + 8, ALLOC = BYTES + 1024;
};
static_assert(K4_RAW_BYTES % 1024 == 0, "operand tiles must stay 1024-byte aligned");
static_assert(K4Smem<128>::ALLOC <= 227 * 1024 && K4Smem<64>::ALLOC <= 227 * 1024, "shared memory plan does not fit");

struct TcK4Args {
    GemvSegment seg;
    GemvSegment seg2;      // a second matrix of the same type and width served by the same launch (tiles0 < gridDim.x), e.g. ffn_up next to ffn_gate
    uint32_t tiles0;       // row tiles of `seg`; CTAs with blockIdx.x >= tiles0 work on seg2
    const float *act_d;    // [token][pitch] per-256 activation scales
    uint32_t act_d_pitch;
    uint32_t n_tokens, nb;
};

template <bool GEMM, int N>
__global__ void __launch_bounds__(K4_THREADS, 1)
gemm_tc5_q4k_kernel(const __grid_constant__ CUtensorMap tm_raw0, const __grid_constant__ CUtensorMap tm_hdr0, const __grid_constant__ CUtensorMap tm_raw1,
                    const __grid_constant__ CUtensorMap tm_hdr1, const __grid_constant__ CUtensorMap tm_x, TcK4Args a) {
    using S = K4Smem<N>;
    constexpr uint32_t IN_STAGES = S::IN_STAGES;
    constexpr uint32_t MAX_PLANES = GEMM ? 2 : 3, ACC_STRIDE = MAX_PLANES * N, NBUF = 2 * ACC_STRIDE <= 512 ? 2 : 1;
    constexpr int TPT = N / 2;  // tokens per epilogue thread
    extern __shared__ uint8_t smem_raw[];
    const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem = smem_raw + (sbase - smem_u32(smem_raw));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // two matrices in one launch fill the last wave better than two launches: 2 x 448 CTAs are 6.05 waves of 148, not 2 x 4
    const bool second = blockIdx.x >= a.tiles0;
    const CUtensorMap &tm_raw = second ? tm_raw1 : tm_raw0, &tm_hdr = second ? tm_hdr1 : tm_hdr0;
    const GemvSegment &seg = second ? a.seg2 : a.seg;
    const uint32_t row0 = (blockIdx.x - (second ? a.tiles0 : 0u)) * TC_M, tok0 = blockIdx.y * N;
    volatile uint32_t *abort = reinterpret_cast<volatile uint32_t *>(smem + S::ABORT);
    const uint32_t nb = a.nb;
    const uint32_t n_visits = GEMM ? 2 * nb : nb;  // super-block visits; in the prefill order the first nb are the min sweep
    // planes of a visit: decode order lo, hi, min; prefill order min alone, then lo, hi
    auto n_planes = [&](uint32_t u) -> uint32_t { return GEMM ? (u < nb ? 1u : 2u) : 3u; };

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < IN_STAGES; ++s) {
            mbar_init(sbase + S::IN_FULL + 8 * s, 1);
            mbar_init(sbase + S::IN_EMPTY + 8 * s, 1 + K4_EXP_WARPS);  // MMA completion (activations) + the expanders (blocks)
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(sbase + S::PL_FULL + 8 * b, K4_EXP_WARPS);
            mbar_init(sbase + S::PL_EMPTY + 8 * b, 1);
            mbar_init(sbase + S::ACC_FULL + 8 * b, 1);
            mbar_init(sbase + S::ACC_EMPTY + 8 * b, TC_EPI_WARPS);
        }
        *abort = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == K4_MMA_WARP) tmem_alloc(sbase + S::SLOT, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *reinterpret_cast<volatile uint32_t *>(smem + S::SLOT);

    if (warp == K4_TMA_WARP) {
        if (lane == 0) {
            for (uint32_t u = 0; u < n_visits; ++u) {
                const uint32_t slot = u % IN_STAGES, s = u % nb;
                const bool min_sweep = GEMM && u < nb;
                if (u >= IN_STAGES && !mbar_wait(sbase + S::IN_EMPTY + 8 * slot, ((u / IN_STAGES) & 1u) ^ 1u, abort)) break;
                const uint32_t full = sbase + S::IN_FULL + 8 * slot;
                mbar_expect_tx(full, (min_sweep ? TC_M * 16u : K4_RAW_BYTES) + S::B_BYTES);
                if (min_sweep) tma_load_2d(sbase + S::RAW + slot * K4_RAW_BYTES, &tm_hdr, (int32_t)(s * 144), (int32_t)row0, full);  // the 16-byte headers
                else tma_load_2d(sbase + S::RAW + slot * K4_RAW_BYTES, &tm_raw, (int32_t)(s * 144), (int32_t)row0, full);
                tma_load_2d(sbase + S::B + slot * S::B_BYTES, &tm_x, (int32_t)(s * 256), (int32_t)tok0, full);
                tma_load_2d(sbase + S::B + slot * S::B_BYTES + N * 128, &tm_x, (int32_t)(s * 256 + 128), (int32_t)tok0, full);
            }
        }
    } else if (warp == K4_MMA_WARP) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_i8(0, 1, N);  // unsigned planes x signed activations
            bool ok = true;
            for (uint32_t u = 0; u < n_visits && ok; ++u) {
                const uint32_t slot = u % IN_STAGES, buf = u % NBUF, np = n_planes(u);
                for (uint32_t h = 0; h < 2; ++h) {
                    const uint32_t v = 2 * u + h, ps = v & 1u;
                    if (!(ok = mbar_wait(sbase + S::PL_FULL + 8 * ps, (v / 2) & 1u, abort))) break;
                    if (h == 0) {
                        if (!(ok = mbar_wait(sbase + S::IN_FULL + 8 * slot, (u / IN_STAGES) & 1u, abort))) break;
                        if (u >= NBUF && !(ok = mbar_wait(sbase + S::ACC_EMPTY + 8 * buf, ((u / NBUF) & 1u) ^ 1u, abort))) break;
                    }
                    tc_fence_after();
                    const uint64_t db = umma_desc_sw128(sbase + S::B + slot * S::B_BYTES + h * N * 128);
                    for (uint32_t p = 0; p < np; ++p) {
                        const uint64_t da = umma_desc_sw128(sbase + S::PLANES + (ps * 3 + p) * K4_PLANE_BYTES);
#pragma unroll
                        for (uint32_t k = 0; k < 4; ++k) umma_i8(tmem + buf * ACC_STRIDE + p * N, da + 2 * k, db + 2 * k, idesc, (h | k) ? 1u : 0u);
                    }
                    umma_commit(sbase + S::PL_EMPTY + 8 * ps);
                    if (h == 1) {
                        umma_commit(sbase + S::IN_EMPTY + 8 * slot);
                        umma_commit(sbase + S::ACC_FULL + 8 * buf);
                    }
                }
            }
        }
    } else if (warp >= TC_EPI_WARPS) {
        // ---- expanders: thread = one row of the half super-block in flight (two runs of 64 elements)
        const uint32_t r = threadIdx.x - TC_EPI_WARPS * 32;
        const uint32_t swz = r & 7u, row_off = (r >> 3) * 1024 + swz * 128;
        bool ok = true;
        for (uint32_t u = 0; u < n_visits && ok; ++u) {
            const uint32_t slot = u % IN_STAGES, s = u % nb;
            const bool min_sweep = GEMM && u < nb, main_sweep = GEMM && u >= nb;
            if (!(ok = mbar_wait(sbase + S::IN_FULL + 8 * slot, (u / IN_STAGES) & 1u, abort))) break;
            const uint8_t *raw = smem + S::RAW + slot * K4_RAW_BYTES + r * (min_sweep ? 16u : 144u);
            const uint4 hd = *reinterpret_cast<const uint4 *>(raw);
            reinterpret_cast<uint32_t *>(smem + S::DD)[(u % K4_RING) * TC_M + r] = hd.x;
            if (r < (uint32_t)N) {
                const uint32_t tok = tok0 + r;
                reinterpret_cast<float *>(smem + S::XD)[(u % K4_RING) * N + r] = tok < a.n_tokens ? __ldg(a.act_d + (uint64_t)tok * a.act_d_pitch + s) : 0.0f;
            }
            // the eight 6-bit scales and mins (engine/quant.rs:653-662) as bytes of two words each
            const uint32_t scl = hd.y & 0x3f3f3f3fu, ml = hd.z & 0x3f3f3f3fu;
            const uint32_t sch = (hd.w & 0x0f0f0f0fu) | ((hd.y >> 2) & 0x30303030u), mh = ((hd.w >> 4) & 0x0f0f0f0fu) | ((hd.z >> 2) & 0x30303030u);
            for (uint32_t h = 0; h < 2; ++h) {
                const uint32_t v = 2 * u + h, ps = v & 1u;
                if (v >= 2 && !(ok = mbar_wait(sbase + S::PL_EMPTY + 8 * ps, ((v / 2) & 1u) ^ 1u, abort))) break;
                uint8_t *pl = smem + S::PLANES + ps * 3 * K4_PLANE_BYTES + row_off;
#pragma unroll
                for (uint32_t gl = 0; gl < 2; ++gl) {
                    const uint32_t g = 2 * h + gl;  // 64 elements 64 g .. of the super-block: sub-blocks 2g (low nibbles), 2g + 1 (high)
                    const uint32_t scw = h == 0 ? scl : sch, mw = h == 0 ? ml : mh, sh = 16 * gl;
                    const uint32_t sa = (scw >> sh) & 0xffu, sb = (scw >> (sh + 8)) & 0xffu, ma = (mw >> sh) & 0xffu, mb = (mw >> (sh + 8)) & 0xffu;
                    // 16-byte chunks 4 gl .. 4 gl + 3 of the row's 128 bytes, swizzled: low-nibble sub-block in the first two, high in the last two
                    const uint32_t c0 = ((4 * gl + 0) ^ swz) * 16, c1 = ((4 * gl + 1) ^ swz) * 16, c2 = ((4 * gl + 2) ^ swz) * 16, c3 = ((4 * gl + 3) ^ swz) * 16;
                    if (!min_sweep) {
                        const uint4 qa = *reinterpret_cast<const uint4 *>(raw + 16 + 32 * g), qb = *reinterpret_cast<const uint4 *>(raw + 32 + 32 * g);
                        const uint32_t M = 0x0f0f0f0fu;
                        const uint32_t la[8] = {qa.x & M, qa.y & M, qa.z & M, qa.w & M, qb.x & M, qb.y & M, qb.z & M, qb.w & M};
                        const uint32_t ha[8] = {(qa.x >> 4) & M, (qa.y >> 4) & M, (qa.z >> 4) & M, (qa.w >> 4) & M, (qb.x >> 4) & M, (qb.y >> 4) & M, (qb.z >> 4) & M, (qb.w >> 4) & M};
                        const uint32_t sal = sa & 7u, sah = sa >> 3, sbl = sb & 7u, sbh = sb >> 3;
                        uint8_t *plo = pl, *phi = pl + K4_PLANE_BYTES;
                        // four codes (each <= 15) times a digit (<= 7) in one multiply: no byte reaches 256
                        *reinterpret_cast<uint4 *>(plo + c0) = make_uint4(la[0] * sal, la[1] * sal, la[2] * sal, la[3] * sal);
                        *reinterpret_cast<uint4 *>(plo + c1) = make_uint4(la[4] * sal, la[5] * sal, la[6] * sal, la[7] * sal);
                        *reinterpret_cast<uint4 *>(plo + c2) = make_uint4(ha[0] * sbl, ha[1] * sbl, ha[2] * sbl, ha[3] * sbl);
                        *reinterpret_cast<uint4 *>(plo + c3) = make_uint4(ha[4] * sbl, ha[5] * sbl, ha[6] * sbl, ha[7] * sbl);
                        *reinterpret_cast<uint4 *>(phi + c0) = make_uint4(la[0] * sah, la[1] * sah, la[2] * sah, la[3] * sah);
                        *reinterpret_cast<uint4 *>(phi + c1) = make_uint4(la[4] * sah, la[5] * sah, la[6] * sah, la[7] * sah);
                        *reinterpret_cast<uint4 *>(phi + c2) = make_uint4(ha[0] * sbh, ha[1] * sbh, ha[2] * sbh, ha[3] * sbh);
                        *reinterpret_cast<uint4 *>(phi + c3) = make_uint4(ha[4] * sbh, ha[5] * sbh, ha[6] * sbh, ha[7] * sbh);
                    }
                    if (!main_sweep) {
                        uint8_t *pm = pl + (GEMM ? 0u : 2u * K4_PLANE_BYTES);
                        const uint32_t wa = ma * 0x01010101u, wb = mb * 0x01010101u;
                        *reinterpret_cast<uint4 *>(pm + c0) = make_uint4(wa, wa, wa, wa);
                        *reinterpret_cast<uint4 *>(pm + c1) = make_uint4(wa, wa, wa, wa);
                        *reinterpret_cast<uint4 *>(pm + c2) = make_uint4(wb, wb, wb, wb);
                        *reinterpret_cast<uint4 *>(pm + c3) = make_uint4(wb, wb, wb, wb);
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the tensor core reads these planes through the async proxy
                __syncwarp();
                if (lane == 0) mbar_arrive(sbase + S::PL_FULL + 8 * ps);
            }
            if (!ok) break;
            __syncwarp();
            if (lane == 0) mbar_arrive(sbase + S::IN_EMPTY + 8 * slot);  // this warp is done with the blocks of the visit
        }
    } else {
        // ---- epilogue: thread = one row x N / 2 tokens
        const uint32_t quad = warp & 3u, half = warp >> 2, rl = quad * 32 + lane;
        const uint32_t row = row0 + rl;
        const bool row_ok = row < seg.w.out_dim;
        float acc[TPT];
#pragma unroll
        for (int t = 0; t < TPT; ++t) acc[t] = 0.0f;
        for (uint32_t u = 0; u < n_visits; ++u) {
            const uint32_t buf = u % NBUF, ring = u % K4_RING;
            const bool min_sweep = GEMM && u < nb;
            if (!mbar_wait(sbase + S::ACC_FULL + 8 * buf, (u / NBUF) & 1u, abort)) break;
            tc_fence_after();
            const uint32_t dw = reinterpret_cast<const uint32_t *>(smem + S::DD)[ring * TC_M + rl];
            const float d = f16_bits_to_f32(dw & 0xffffu), dmin = f16_bits_to_f32(dw >> 16);
            const float *xd = reinterpret_cast<const float *>(smem + S::XD) + ring * N + half * TPT;
            const uint32_t tbase = tmem + ((quad * 32) << 16) + buf * ACC_STRIDE + half * TPT;
#pragma unroll
            for (int c = 0; c < TPT / 16; ++c) {  // 16 tokens at a time
                uint32_t p0[16], p1[16], p2[16];
                tmem_ld16(tbase + c * 16, p0);
                if (!GEMM || !min_sweep) tmem_ld16(tbase + N + c * 16, p1);
                if (!GEMM) tmem_ld16(tbase + 2 * N + c * 16, p2);
                tmem_ld_wait();
#pragma unroll
                for (int t = 0; t < 16; ++t) {
                    const float ad = xd[c * 16 + t];
                    float &o = acc[c * 16 + t];
                    if (!GEMM) {
                        const int isum = (int)(p1[t] << 3) + (int)p0[t], imin = (int)p2[t];
                        o = __fadd_rn(o, __fmul_rn(ad, __fsub_rn(__fmul_rn(d, (float)isum), __fmul_rn(dmin, (float)imin))));
                    } else if (min_sweep) {
                        o = __fsub_rn(o, __fmul_rn(__fmul_rn(ad, dmin), (float)(int)p0[t]));
                    } else {
                        const int isum = (int)(p1[t] << 3) + (int)p0[t];
                        o = __fadd_rn(o, __fmul_rn(ad, __fmul_rn(d, (float)isum)));
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(sbase + S::ACC_EMPTY + 8 * buf);
        }
        if (!*abort && row_ok) {
#pragma unroll
            for (int t = 0; t < TPT; ++t) {
                const uint32_t tok = tok0 + half * TPT + t;
                if (tok < a.n_tokens) {
                    const uint64_t o = (uint64_t)tok * seg.y_stride + row;
                    float v = acc[t];
                    if (seg.epilogue == EPI_ADD_RESIDUAL) v = __fadd_rn(seg.residual[o], v);
                    seg.y[o] = v;
                }
            }
        }
    }
    if (*abort) {
        for (int i = 0; i < 200; ++i) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == K4_MMA_WARP) tmem_dealloc(tmem, 512);
}

// ---- host ------------------------------------------------------------------------------------------------------------
using EncodeTiled = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                 CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_fn() {
    static EncodeTiled fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) p = nullptr;
        return reinterpret_cast<EncodeTiled>(p);
    }();
    return fn;
}

// 2-D tensor of `rows` rows of `cols` elements, rows `pitch` bytes apart, read in boxes of box_cols x box_rows.
bool make_map_2d(CUtensorMap *tm, CUtensorMapDataType type, uint32_t elem_bytes, const void *base, uint64_t cols, uint64_t rows, uint64_t pitch, uint32_t box_cols,
                 uint32_t box_rows, CUtensorMapSwizzle swz) {
    EncodeTiled fn = encode_fn();
    if (!fn || (reinterpret_cast<uintptr_t>(base) & 15) || (pitch & 15) || ((uint64_t)box_cols * elem_bytes & 15)) return false;
    const cuuint64_t dims[2] = {cols, rows}, strides[1] = {pitch};
    const cuuint32_t box[2] = {box_cols, box_rows}, estr[2] = {1, 1};
    return fn(tm, type, 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

bool gemm_tc5_supported(const GemvArgs &a) {
    static const bool enabled = [] { const char *e = getenv("OB_TC5"); return !(e && e[0] == '0' && e[1] == 0); }();
    if (!enabled || a.n_seg < 1 || a.n_tokens < 16 || a.isum_out || !encode_fn()) return false;
    const uint32_t type = a.seg[0].w.type, in_dim = a.seg[0].w.in_dim;
    if (type == TYPE_Q8_0) {
        if (in_dim % 128 || a.act.dim_cap % 128) return false;
    } else if (type == TYPE_Q4_K) {
        if (in_dim % 256 || a.act.dim_cap % 16) return false;
        // A CTA owns 128 rows x 64 or 128 tokens and walks the whole row (the fp32 order forbids splitting K), so a small
        // matrix at a small batch gives too few CTAs: the 64-row mma.sync tiles (gemm_mma.cu) fill the GPU better there.
        uint32_t ctas = 0;
        const uint32_t tok_tile = a.n_tokens > 64 ? 128 : 64;
        for (int s = 0; s < a.n_seg; ++s) ctas += ((a.seg[s].w.out_dim + TC_M - 1) / TC_M) * ((a.n_tokens + tok_tile - 1) / tok_tile);
        if (ctas < 96) return false;
    } else {
        return false;  // Q6_K stays on the mma.sync tiles (gemm_mma.cu)
    }
    for (int s = 0; s < a.n_seg; ++s)
        if (a.seg[s].w.type != type || a.seg[s].w.in_dim != in_dim || (a.seg[s].w.row_stride & 15) || (type == TYPE_Q8_0 && (a.seg[s].w.d_off & 7))) return false;
    return true;
}

template <bool GEMM, int N>
static bool launch_q4k_instance(const GemvArgs &a, int sm_count, cudaStream_t st) {
    static PerDeviceOnce once;
    if (once.run([] { return cudaFuncSetAttribute(gemm_tc5_q4k_kernel<GEMM, N>, cudaFuncAttributeMaxDynamicSharedMemorySize, K4Smem<N>::ALLOC); }) != cudaSuccess) return false;
    const uint32_t in_dim = a.seg[0].w.in_dim, nb = in_dim / 256;
    CUtensorMap tm_x;
    if (!make_map_2d(&tm_x, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.act.q, in_dim, a.n_tokens, a.act.dim_cap, 128, N, CU_TENSOR_MAP_SWIZZLE_128B)) return false;
    auto maps = [&](const GemvSegment &g, CUtensorMap *raw, CUtensorMap *hdr) {
        return make_map_2d(raw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, g.w.data, (uint64_t)nb * 144, g.w.out_dim, g.w.row_stride, 144, TC_M, CU_TENSOR_MAP_SWIZZLE_NONE) &&
               make_map_2d(hdr, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, g.w.data, (uint64_t)nb * 144, g.w.out_dim, g.w.row_stride, 16, TC_M, CU_TENSOR_MAP_SWIZZLE_NONE);
    };
    const uint32_t tok_tiles = (a.n_tokens + N - 1) / N, sms = (uint32_t)std::max(1, sm_count);
    auto tiles = [&](int s) { return (a.seg[s].w.out_dim + TC_M - 1) / TC_M; };
    auto waves = [&](uint32_t ctas) { return (ctas + sms - 1) / sms; };
    for (int s = 0; s < a.n_seg; ++s) {
        // pair this matrix with the next one when one launch takes fewer waves than two
        const bool pair = s + 1 < a.n_seg && waves((tiles(s) + tiles(s + 1)) * tok_tiles) < waves(tiles(s) * tok_tiles) + waves(tiles(s + 1) * tok_tiles);
        CUtensorMap raw0, hdr0, raw1, hdr1;
        if (!maps(a.seg[s], &raw0, &hdr0) || !maps(a.seg[pair ? s + 1 : s], &raw1, &hdr1)) return false;
        TcK4Args k{};
        k.seg = a.seg[s];
        k.seg2 = a.seg[pair ? s + 1 : s];
        k.tiles0 = tiles(s);
        k.act_d = a.act.d;
        k.act_d_pitch = a.act.dim_cap / 256;
        k.n_tokens = a.n_tokens;
        k.nb = nb;
        const dim3 grid(tiles(s) + (pair ? tiles(s + 1) : 0u), tok_tiles);
        gemm_tc5_q4k_kernel<GEMM, N><<<grid, K4_THREADS, K4Smem<N>::ALLOC, st>>>(raw0, hdr0, raw1, hdr1, tm_x, k);
        g_tc5_launched.store(true, std::memory_order_relaxed);
        if (pair) ++s;
    }
    return true;
}

static bool launch_q4k(const GemvArgs &a, int sm_count, cudaStream_t st) {
    const bool wide = a.n_tokens > 64;  // 128-token tiles once there are tokens for them
    if (a.gemm_order) return wide ? launch_q4k_instance<true, 128>(a, sm_count, st) : launch_q4k_instance<true, 64>(a, sm_count, st);
    return wide ? launch_q4k_instance<false, 128>(a, sm_count, st) : launch_q4k_instance<false, 64>(a, sm_count, st);
}

bool launch_gemm_tc5(const GemvArgs &a, int sm_count, cudaStream_t st) {
    if (a.seg[0].w.type == TYPE_Q4_K) return launch_q4k(a, sm_count, st);
    static PerDeviceOnce once;
    if (once.run([] { return cudaFuncSetAttribute(gemm_tc5_q8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Q8Smem::ALLOC); }) != cudaSuccess) return false;
    const uint32_t in_dim = a.seg[0].w.in_dim;
    CUtensorMap tm_x, tm_xd;
    if (!make_map_2d(&tm_x, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.act.q, in_dim, a.n_tokens, a.act.dim_cap, 128, TC_N, CU_TENSOR_MAP_SWIZZLE_128B)) return false;
    if (!make_map_2d(&tm_xd, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, a.act.d, in_dim / 32, a.n_tokens, (uint64_t)(a.act.dim_cap / 32) * 4, 4, TC_N, CU_TENSOR_MAP_SWIZZLE_NONE))
        return false;
    for (int s = 0; s < a.n_seg; ++s) {
        const GemvSegment &g = a.seg[s];
        CUtensorMap tm_w;
        if (!make_map_2d(&tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, g.w.data, in_dim, g.w.out_dim, g.w.row_stride, 128, TC_M, CU_TENSOR_MAP_SWIZZLE_128B)) return false;
        TcQ8Args k{};
        k.seg = g;
        k.n_tokens = a.n_tokens;
        k.n_steps = in_dim / 128;
        const dim3 grid((g.w.out_dim + TC_M - 1) / TC_M, (a.n_tokens + TC_N - 1) / TC_N);
        gemm_tc5_q8_kernel<<<grid, TC_THREADS, Q8Smem::ALLOC, st>>>(tm_w, tm_x, tm_xd, k);
        g_tc5_launched.store(true, std::memory_order_relaxed);
    }
    return true;
}

// 1 when a bounded wait of one of these kernels ran out since the last call (and clears it).  Synchronises with the device.
int gemm_tc5_take_status() {
    if (!g_tc5_launched.exchange(false)) return 0;
    uint32_t v = 0;
    if (cudaMemcpyFromSymbol(&v, g_tc5_status, 4) != cudaSuccess) return 0;
    if (v) {
        const uint32_t z = 0;
        cudaMemcpyToSymbol(g_tc5_status, &z, 4);
    }
    return (int)v;
}

}  // namespace ob
