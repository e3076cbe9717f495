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


// ----------------------------------------------------------------------------------------------------
// The same sum by a whole CTA, with the sequential part reduced to a few dozen steps.
//
// The binade of every partial sum is known in advance, up to a rigorous margin: with E_i the exact prefix
// sum (taken in double), the sequentially rounded s_i satisfies |s_i - E_i| <= i * 2^-24 * s_i.  A term whose
// two neighbouring partial sums are, with that margin, inside one binade is "safe": its increment function
// can be formed without knowing S.  All safe functions are formed in parallel; a thread whose terms are all
// safe composes them; runs of such threads are composed by a segmented warp scan; and only the threads that
// hold an unsafe term (the start of the sum and the ~log2(n) binade crossings) are added with real float
// additions, one after the other.  Every application checks that s really is in the assumed binade; if that
// ever failed the warp-level routine above recomputes the sum from scratch.
// ----------------------------------------------------------------------------------------------------
struct SeqSumRecord {
    uint32_t c0, c1;   // composed function: of the thread's terms, then (after the warp's scan) of its segment so far
    uint32_t es;       // biased exponent of the binade the function assumes (0: the thread has no terms)
    uint32_t dirty;    // the thread holds a term that must be added for real
};

template <int THREADS>
struct SeqSumWorkspace {
    SeqSumRecord rec[THREADS];
    double warp_tot[THREADS / 32];
    uint32_t seg_end[THREADS / 32];  // per warp: lanes that end a segment
    float result;
};

// Every thread of the CTA must call this (it contains __syncthreads); every thread returns the sum.
template <int THREADS, class F>
__device__ float cta_sequential_sum(F term, uint32_t n, SeqSumWorkspace<THREADS> &ws) {
    using namespace seqsum_detail;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t ept = (n + THREADS - 1) / THREADS;
    const uint32_t first = min(n, (uint32_t)tid * ept), last = min(n, first + ept);

    // ---- exact prefix sums in double ------------------------------------------------------------
    double local = 0.0;
    for (uint32_t i = first; i < last; ++i) local += (double)term(i);
    double incl = local;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const double up = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += up;
    }
    if (lane == 31) ws.warp_tot[warp] = incl;
    __syncthreads();
    double base = incl - local;
    for (int w = 0; w < warp; ++w) base += ws.warp_tot[w];

    // ---- classify and compose this thread's terms -------------------------------------------------
    uint32_t c0 = 0, c1 = 0, es_run = 0, dirty = 0;
    double prev = base;
    for (uint32_t i = first; i < last; ++i) {
        const float t = term(i);
        const double cur = prev + (double)t;
        const double margin = (double)(i + 2) * 6.1e-8;  // > (i + 1) * 2^-24, with room for the double sum's own error
        const double lo = prev * (1.0 - margin), hi = cur * (1.0 + margin);
        // both bounds as floats' binades: safe iff identical, normal and finite
        const float flo = __double2float_rd(lo), fhi = __double2float_ru(hi);
        const uint32_t elo = (__float_as_uint(flo) >> 23) & 0xff, ehi = (__float_as_uint(fhi) >> 23) & 0xff;
        const bool safe = elo == ehi && elo != 0 && elo != 255 && !(margin >= 0.25) && t >= 0.0f;
        if (!safe || (es_run != 0 && es_run != elo)) {
            dirty = 1;
        } else {
            es_run = elo;
            uint32_t a0, a1;
            term_function(__float_as_uint(t), (int)elo, a0, a1);
            const uint32_t n0 = sat_add(c0, (c0 & 1u) ? a1 : a0);
            const uint32_t n1 = sat_add(c1, ((1u + c1) & 1u) ? a1 : a0);
            c0 = n0;
            c1 = n1;
        }
        prev = cur;
    }

    // ---- every warp composes the runs of its own 32 threads: segmented inclusive scan ------------------
    {
        const uint32_t prev_es = __shfl_up_sync(0xffffffffu, es_run, 1);
        const uint32_t prev_dirty = __shfl_up_sync(0xffffffffu, dirty, 1);
        // a dirty lane, an empty lane or a change of binade starts a new segment
        const bool head = lane == 0 || dirty != 0 || prev_dirty != 0 || es_run == 0 || prev_es != es_run;
        const uint32_t seg_start = __ballot_sync(0xffffffffu, head);
        const uint32_t below = seg_start & (0xffffffffu >> (31 - lane));
        const int my_head = 31 - __clz(below);
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const uint32_t l0 = __shfl_up_sync(0xffffffffu, c0, d), l1 = __shfl_up_sync(0xffffffffu, c1, d);
            if (lane - d >= my_head) {
                const uint32_t n0 = sat_add(l0, (l0 & 1u) ? c1 : c0);
                const uint32_t n1 = sat_add(l1, ((1u + l1) & 1u) ? c1 : c0);
                c0 = n0;
                c1 = n1;
            }
        }
        ws.rec[tid] = SeqSumRecord{c0, c1, es_run, dirty};
        if (lane == 0) ws.seg_end[warp] = (seg_start >> 1) | 0x80000000u;  // lane l ends a segment iff lane l+1 starts one
    }
    __syncthreads();

    // ---- warp 0 walks the segments in order ----------------------------------------------------------------
    if (warp == 0) {
        float s = 0.0f;
        bool ok = true;
        for (int chunk = 0; chunk < THREADS / 32 && ok; ++chunk) {
            uint32_t todo = ws.seg_end[chunk];
            while (todo && ok) {
                const int e = __ffs(todo) - 1;
                todo &= todo - 1;
                const SeqSumRecord r = ws.rec[chunk * 32 + e];
                if (r.dirty) {
                    const uint32_t o = (uint32_t)(chunk * 32 + e);
                    const uint32_t b = min(n, o * ept), en = min(n, b + ept);
                    for (uint32_t i = b; i < en; i += 4) {  // fetch four terms, then add them: the loads overlap
                        const float t0 = term(i), t1 = i + 1 < en ? term(i + 1) : 0.0f, t2 = i + 2 < en ? term(i + 2) : 0.0f,
                                    t3 = i + 3 < en ? term(i + 3) : 0.0f;
                        s = __fadd_rn(s, t0);
                        if (i + 1 < en) s = __fadd_rn(s, t1);
                        if (i + 2 < en) s = __fadd_rn(s, t2);
                        if (i + 3 < en) s = __fadd_rn(s, t3);
                    }
                } else if (r.es != 0) {
                    const uint32_t sb = __float_as_uint(s);
                    const uint32_t S = (sb & 0x7fffffu) | 0x800000u;
                    const uint32_t S2 = S + ((S & 1u) ? r.c1 : r.c0);
                    if (((sb >> 23) & 0x1ff) != r.es || S2 >= (1u << 24)) {
                        ok = false;  // the assumed binade did not hold: recompute below
                    } else {
                        s = __uint_as_float((sb & 0xff800000u) | (S2 & 0x7fffffu));
                    }
                }
            }
        }
        if (!ok) s = warp_sequential_sum<16>(term, n);
        if (lane == 0) ws.result = s;
    }
    __syncthreads();
    return ws.result;
}

}  // namespace ob
