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

#ifndef SEQSUM_MARK
#define SEQSUM_MARK(i)      // a timing harness may define these to record the clock at phase boundaries
#define SEQSUM_VALUE(i, v)  // ... and a value
#endif

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
// The binade of every partial sum is known in advance, up to a rigorous margin: with E_i the exact prefix sum, the
// sequentially rounded s_i satisfies |s_i - E_i| <= i * 2^-24 * s_i; E_i itself is taken from an fp32 scan (a few dozen
// additions of non-negative values: relative error below 4e-6, which the margin includes).  A thread whose partial
// sums are, with that margin, inside one binade is "safe": its terms' increment functions can be formed without
// knowing S.  All safe functions are formed in parallel; a thread whose terms are all safe composes them; runs of such
// threads are composed by a segmented warp scan; and only the threads that hold an unsafe term (the start of the sum
// and the ~log2(n) binade crossings) are added with real float additions, one after the other.  Every application
// checks that s really is in the assumed binade -- the margins only decide how often that holds, never the result:
// if it ever failed the warp-level routine above recomputes the sum from scratch.
//
// The increment function of a term comes from the adder itself: inside a binade the bit pattern of s is its
// significand, so with s_even = 2^e (significand 2^23) and s_odd = 2^e + ulp,
//     a[0] = bits(fl(s_even + t)) - bits(s_even),   a[1] = bits(fl(s_odd + t)) - bits(s_odd)
// are exactly the integers by which a sum of even / odd significand grows (round to nearest, ties to even), and a
// difference of 2^23 - 1 or more says that the term alone leaves the binade.
// ----------------------------------------------------------------------------------------------------
constexpr int SEQSUM_MAX_EVENTS = 256;

template <int THREADS, int MAX_EVENTS = SEQSUM_MAX_EVENTS>
struct SeqSumWorkspace {
    // The serial part of the sum as a list of events in term order.  An event is either a composed increment function of
    // a run of safe terms (a0, a1 by parity; es = the binade it assumes) or up to four terms to be added for real.
    uint4 ev_fn[MAX_EVENTS];      // a0, a1, es, dirty
    float4 ev_terms[MAX_EVENTS];  // four terms, +0 where there is none (s + 0 == s)
    float ev_s[MAX_EVENTS];       // the sum after each event
    float warp_tot[THREADS / 32];
    uint32_t warp_events[THREADS / 32];
    float result;
};

namespace seqsum_detail {

// a[parity] of term t in the binade whose biased exponent is es (1..254); t >= 0 or NaN
__device__ __forceinline__ void term_function_add(float t, uint32_t es, uint32_t &a0, uint32_t &a1) {
    const uint32_t be = es << 23, bo = be | 1u;
    const uint32_t d0 = __float_as_uint(__fadd_rn(__uint_as_float(be), t)) - be;
    const uint32_t d1 = __float_as_uint(__fadd_rn(__uint_as_float(bo), t)) - bo;
    a0 = d0 >= (1u << 23) - 1u ? SAT : d0;  // leaves the binade (inf and NaN land here too)
    a1 = d1 >= (1u << 23) - 1u ? SAT : d1;
}

}  // namespace seqsum_detail

// E > 0: every thread has at most E terms and keeps them in registers (one evaluation of term() each, and loops of known
// length); E == 0: any number of terms, re-evaluated where needed.
template <int THREADS, int MAX_EVENTS, int E, class F>
__device__ __forceinline__ float cta_sequential_sum_impl(F term, uint32_t n, SeqSumWorkspace<THREADS, MAX_EVENTS> &ws) {
    using namespace seqsum_detail;
    constexpr int NWARP = THREADS / 32;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t ept = (n + THREADS - 1) / THREADS;
    const uint32_t first = min(n, (uint32_t)tid * ept), last = min(n, first + ept);

    SEQSUM_MARK(0);
    // ---- prefix sums (fp32, additions only: every partial is a sum of non-negative values) -----------------------
    float tv[E > 0 ? E : 1];
    float local = 0.0f;
    if constexpr (E > 0) {
#pragma unroll
        for (int j = 0; j < E; ++j) tv[j] = first + j < last ? term(first + j) : 0.0f;  // + 0 changes no sum and composes as the identity
#pragma unroll
        for (int j = 0; j < E; ++j) local += tv[j];
    } else {
        for (uint32_t i = first; i < last; ++i) local += term(i);
    }
    float incl = local;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const float up = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += up;
    }
    if (lane == 31) ws.warp_tot[warp] = incl;
    float base = __shfl_up_sync(0xffffffffu, incl, 1);  // the lanes before this one
    if (lane == 0) base = 0.0f;
    __syncthreads();
    {   // plus the totals of the warps before this one: a shuffle scan over the (at most 32) warp totals
        float wt = lane < NWARP ? ws.warp_tot[lane] : 0.0f;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const float up = __shfl_up_sync(0xffffffffu, wt, d);
            if (lane >= d) wt += up;
        }
        const float before = __shfl_sync(0xffffffffu, wt, warp > 0 ? warp - 1 : 0);
        if (warp > 0) base += before;
    }

    SEQSUM_MARK(1);
    // ---- classify and compose this thread's terms -------------------------------------------------
    // With the margin of the thread's last term, [base * (1 - m), (base + local) * (1 + m)] contains every partial sum the
    // thread can see; if both ends are in one binade, every term of the thread is safe in that binade.
    uint32_t c0 = 0, c1 = 0, es_run = 0, dirty = 0;
    if (first < last) {
        const float m_last = (float)(last + 1 + ept) * 6.1e-8f + 2.0e-6f;  // > last * 2^-24, plus the scan's own error (ept + ~11 additions)
        const float flo = __fmul_rd(base, __fsub_rd(1.0f, m_last)), fhi = __fmul_ru(__fadd_ru(base, local), __fadd_ru(1.0f, m_last));
        const uint32_t elo = (__float_as_uint(flo) >> 23) & 0xff, ehi = (__float_as_uint(fhi) >> 23) & 0xff;
        if (elo == ehi && elo != 0 && elo != 255 && !(m_last >= 0.25f)) {
            es_run = elo;
            auto compose = [&](float t) {
                if (!(t >= 0.0f)) dirty = 1;  // negative or NaN: not this routine's case, add for real
                uint32_t a0, a1;
                term_function_add(t, elo, a0, a1);
                const uint32_t n0 = sat_add(c0, (c0 & 1u) ? a1 : a0);
                const uint32_t n1 = sat_add(c1, ((1u + c1) & 1u) ? a1 : a0);
                c0 = n0;
                c1 = n1;
            };
            if constexpr (E > 0) {
#pragma unroll
                for (int j = 0; j < E; ++j) compose(tv[j]);
            } else {
                for (uint32_t i = first; i < last; ++i) compose(term(i));
            }
        } else {
            dirty = 1;
        }
    }

    SEQSUM_MARK(2);
    // ---- every warp composes the runs of its own 32 threads: segmented inclusive scan ------------------
    const uint32_t prev_es = __shfl_up_sync(0xffffffffu, es_run, 1);
    const uint32_t prev_dirty = __shfl_up_sync(0xffffffffu, dirty, 1);
    // a dirty lane, an empty lane or a change of binade starts a new segment
    const bool head = lane == 0 || dirty != 0 || prev_dirty != 0 || es_run == 0 || prev_es != es_run;
    const uint32_t seg_start = __ballot_sync(0xffffffffu, head);
    {
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
    }
    // events of this lane: a dirty thread's terms four at a time; the end of a clean segment; nothing for a thread without terms
    const bool seg_end = lane == 31 || ((seg_start >> (lane + 1)) & 1u);
    const uint32_t my_events = first >= last ? 0u : (dirty ? (last - first + 3) / 4 : (seg_end ? 1u : 0u));
    uint32_t ev_incl = my_events;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const uint32_t up = __shfl_up_sync(0xffffffffu, ev_incl, d);
        if (lane >= d) ev_incl += up;
    }
    if (lane == 31) ws.warp_events[warp] = ev_incl;
    __syncthreads();
    uint32_t total;
    {
        uint32_t we = lane < NWARP ? ws.warp_events[lane] : 0u;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const uint32_t up = __shfl_up_sync(0xffffffffu, we, d);
            if (lane >= d) we += up;
        }
        total = __shfl_sync(0xffffffffu, we, 31);
        const uint32_t before = __shfl_sync(0xffffffffu, we, warp > 0 ? warp - 1 : 0);
        uint32_t pos = (warp > 0 ? before : 0u) + ev_incl - my_events;
        if (total <= (uint32_t)MAX_EVENTS && my_events) {
            if (dirty) {
                if constexpr (E > 0) {
#pragma unroll
                    for (int j = 0; j < E; j += 4) {
                        if (first + j < last) {
                            ws.ev_fn[pos] = make_uint4(0u, 0u, 0u, 1u);
                            ws.ev_terms[pos] = make_float4(tv[j], j + 1 < E ? tv[j + 1] : 0.0f, j + 2 < E ? tv[j + 2] : 0.0f, j + 3 < E ? tv[j + 3] : 0.0f);
                            ++pos;
                        }
                    }
                } else {
                    for (uint32_t i = first; i < last; i += 4, ++pos) {
                        ws.ev_fn[pos] = make_uint4(0u, 0u, 0u, 1u);
                        ws.ev_terms[pos] = make_float4(term(i), i + 1 < last ? term(i + 1) : 0.0f, i + 2 < last ? term(i + 2) : 0.0f, i + 3 < last ? term(i + 3) : 0.0f);
                    }
                }
            } else {
                ws.ev_fn[pos] = make_uint4(c0, c1, es_run, 0u);
                ws.ev_terms[pos] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            }
        }
    }
    __syncthreads();

    SEQSUM_MARK(3);
    SEQSUM_VALUE(10, total);
    // ---- warp 0 applies the events in order -----------------------------------------------------------------------
    // The dependent chain per event is four additions (dirty) or the increment added to the bit pattern (clean: inside a
    // binade, adding a * ulp is adding a to the bits).  The next event's load runs ahead; the value after every event is
    // stored, and whether every clean event really found and left s in its binade is checked afterwards, by all lanes at
    // once.  (One warp issues an instruction every five cycles or so, so the walk costs about 70 cycles per event;
    // unrolled and shuffle-fed variants that compute both kinds of event were measured two to three times slower.)
    if (warp == 0) {
        float s = 0.0f;
        bool ok = total <= (uint32_t)MAX_EVENTS;
        if (ok) {
            uint4 fn = ws.ev_fn[0];
            float4 tm = ws.ev_terms[0];
            for (uint32_t k = 0; k < total; ++k) {
                const uint4 f = fn;
                const float4 t = tm;
                if (k + 1 < total) {
                    fn = ws.ev_fn[k + 1];
                    tm = ws.ev_terms[k + 1];
                }
                if (f.w) {
                    s = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(s, t.x), t.y), t.z), t.w);
                } else {
                    const uint32_t sb = __float_as_uint(s);
                    s = __uint_as_float(sb + ((sb & 1u) ? f.y : f.x));
                }
                ws.ev_s[k] = s;
            }
            __syncwarp();
            bool bad = false;
            for (uint32_t k = lane; k < total; k += 32) {
                const uint4 f = ws.ev_fn[k];
                if (!f.w) {  // the assumed binade must hold before and after
                    const uint32_t before = k ? __float_as_uint(ws.ev_s[k - 1]) : 0u, after = __float_as_uint(ws.ev_s[k]);
                    bad = bad || (before >> 23) != f.z || (after >> 23) != f.z;
                }
            }
            ok = !__any_sync(0xffffffffu, bad);
        }
        SEQSUM_MARK(4);
        SEQSUM_VALUE(11, ok ? 1 : 0);
        if (!ok) s = warp_sequential_sum<16>(term, n);
        if (lane == 0) ws.result = s;
    }
    __syncthreads();
    return ws.result;
}

// Every thread of the CTA must call this (it contains __syncthreads); every thread returns the sum.
template <int THREADS, int MAX_EVENTS, class F>
__device__ float cta_sequential_sum(F term, uint32_t n, SeqSumWorkspace<THREADS, MAX_EVENTS> &ws) {
    const uint32_t ept = (n + THREADS - 1) / THREADS;  // the same in every thread
    if (ept <= 8) return cta_sequential_sum_impl<THREADS, MAX_EVENTS, 8>(term, n, ws);
    if (ept <= 16) return cta_sequential_sum_impl<THREADS, MAX_EVENTS, 16>(term, n, ws);
    return cta_sequential_sum_impl<THREADS, MAX_EVENTS, 0>(term, n, ws);
}

}  // namespace ob
