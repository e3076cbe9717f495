// Exact reproduction, by one warp, of a left-to-right fp32 sum of non-negative terms:
//     s = 0;  for i in 0..n:  s = fl32(s + t_i)
//
// The reference sums that way in RMSNorm (engine/tensor.rs:743, `iter().map(|v| v * v).sum()`) and in
// softmax (engine/tensor.rs:811-815).  A tree reduction gives a value that differs in the last bits, and
// because the next operator quantizes to int8, a last-bit difference now and then flips a code and the
// two computations drift apart.  A single thread doing n dependent additions is exact but costs
// 4 cycles x n.  This does the same arithmetic in parallel:
//
// While s stays inside one binade [2^e, 2^(e+1)) its ulp u is fixed, s = S*u with S an integer, and
// adding t >= 0 is the integer update  S += round(t / u)  with the tie (t/u exactly half way) broken
// towards an even S -- which depends on S only through its parity.  So every term is a function
// f(S) = S + a[S & 1] described by two integers, such functions compose associatively
// ((g o f)(S) = S + f_a[p] + g_a[(p + f_a[p]) & 1]), and a warp scan composes 32 x K of them at once.
// The sum is monotone, so if the composed result is still inside the binade the guess "u was fixed"
// held for every step.  Where it leaves the binade, the chunk of K terms containing the crossing is
// redone with real float additions and the scan resumes with the new ulp.  A sum of n similar terms
// crosses about log2(n) binades.
#pragma once

#include <stdint.h>

namespace ob {

namespace seqsum_detail {

constexpr uint32_t SAT = 1u << 26;  // any increment this large leaves the binade

__device__ __forceinline__ uint32_t sat_add(uint32_t a, uint32_t b) {
    uint32_t c = a + b;
    return c > SAT ? SAT : c;
}

// The increment of term t (bits tb) under ulp exponent "es" (biased exponent field of s): a[parity].
__device__ __forceinline__ void term_function(uint32_t tb, int es, uint32_t &a0, uint32_t &a1) {
    const int et_field = (int)((tb >> 23) & 0xff);
    if (et_field == 255) {  // inf / NaN: force the serial path
        a0 = a1 = SAT;
        return;
    }
    const uint32_t m = et_field ? ((tb & 0x7fffffu) | 0x800000u) : (tb & 0x7fffffu);
    const int sh = es - (et_field ? et_field : 1);  // t = m * 2^(et-150), u = 2^(es-150)
    if (m == 0 || sh >= 25) {
        a0 = a1 = 0;  // below half an ulp
    } else if (sh <= 0) {
        const uint32_t T = sh < -2 ? SAT : (m << (-sh));  // a multiple of u; m << 3 already exceeds 2^24
        a0 = a1 = T > SAT ? SAT : T;
    } else {
        const uint32_t T = sh == 24 ? 0u : (m >> sh);
        const uint32_t rem = m & ((1u << sh) - 1u), half = 1u << (sh - 1);
        if (rem > half) {
            a0 = a1 = T + 1;
        } else if (rem < half) {
            a0 = a1 = T;
        } else {  // tie: the even neighbour of S + T + 1/2
            a0 = T + (T & 1u);
            a1 = T + ((T + 1u) & 1u);
        }
    }
}

}  // namespace seqsum_detail

// term(i) must return the i-th term (>= 0, or NaN/inf) and be callable by any lane for any i < n.
// Every lane of the warp must call this; every lane returns the sum.
template <int K, class F>
__device__ float warp_sequential_sum(F term, uint32_t n) {
    using namespace seqsum_detail;
    const int lane = threadIdx.x & 31;
    float s = 0.0f;
    uint32_t i = 0;
    while (i < n) {
        const uint32_t sb = __float_as_uint(s);
        const int es = (int)((sb >> 23) & 0xff);
        if (es == 0 || es == 255 || (sb >> 31)) {  // zero, subnormal, inf, NaN (or a negative term got in): one real addition
            s = __fadd_rn(s, term(i));
            ++i;
            continue;
        }
        const uint32_t S = (sb & 0x7fffffu) | 0x800000u;
        const uint32_t cnt = min((uint32_t)(32 * K), n - i);
        // this lane's K consecutive terms, composed in order
        uint32_t c0 = 0, c1 = 0;
        const uint32_t first = i + (uint32_t)lane * K;
#pragma unroll
        for (int j = 0; j < K; ++j) {
            const uint32_t idx = first + j;
            if (idx < i + cnt) {
                uint32_t a0, a1;
                term_function(__float_as_uint(term(idx)), es, a0, a1);
                const uint32_t n0 = sat_add(c0, (c0 & 1u) ? a1 : a0);
                const uint32_t n1 = sat_add(c1, ((1u + c1) & 1u) ? a1 : a0);
                c0 = n0;
                c1 = n1;
            }
        }
        // inclusive scan of function composition over the lanes (earlier lanes act first)
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const uint32_t l0 = __shfl_up_sync(0xffffffffu, c0, d), l1 = __shfl_up_sync(0xffffffffu, c1, d);
            if (lane >= d) {
                const uint32_t n0 = sat_add(l0, (l0 & 1u) ? c1 : c0);
                const uint32_t n1 = sat_add(l1, ((1u + l1) & 1u) ? c1 : c0);
                c0 = n0;
                c1 = n1;
            }
        }
        const uint32_t S_end = S + ((S & 1u) ? c1 : c0);  // after this lane's last term, if the ulp never changed
        const uint32_t bad = __ballot_sync(0xffffffffu, S_end >= (1u << 24));
        const int first_bad = bad ? (__ffs(bad) - 1) : 32;
        if (first_bad > 0) {
            const uint32_t S_ok = __shfl_sync(0xffffffffu, S_end, first_bad - 1);
            s = __uint_as_float((sb & 0xff800000u) | (S_ok & 0x7fffffu));
        }
        if (first_bad == 32) {
            i += cnt;
        } else {
            i += (uint32_t)first_bad * K;
            const uint32_t stop = min(i + (uint32_t)K, n);
            for (; i < stop; ++i) s = __fadd_rn(s, term(i));  // the chunk where the binade changes
        }
    }
    return s;
}

}  // namespace ob
