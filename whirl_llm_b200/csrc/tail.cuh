// The per-row tail of the sampling path: sort the selected candidates, probabilities in f64, top-k / top-p / min-p on
// the sorted prefix, then the draw.  It restates, for a group of GPU threads, what the reference does on the host in
// sampling::filterCands (src/sampling/sampler.cpp:15-78), sampleRow (:118-131, the candidate part) and sampleRace
// (:82-106, the race part).
// Running sums: the host adds the probabilities one after the other in candidate order.  Here the group's first warp
// adds them in blocks - every lane a contiguous block of candidates in order, then a scan of the lanes' block sums in
// lane order - so the cumulative sum at a candidate is made of the same terms in the same order up to how they are
// grouped; results agree with the host's to the last bits of a double, and a cut or a draw can differ only when a
// cumulative sum meets its bound that closely (the parity tests count draws within 1e-6 of a boundary).  The draw compares
// against u * z instead of dividing every kept probability by z first (unless the caller reads the probabilities).
#pragma once

#include "common.cuh"

namespace wb {

enum RowStatus : int32_t {
    ROW_DONE = 0,       // token drawn from a closed (or reached) candidate set
    ROW_ESCALATE = 1,   // the kept set may reach past the candidates: needs a larger candidate set
    ROW_OPEN_TAIL = 2,  // open set and the draw fell past the candidates: needs the id-order walk of the row
    ROW_RETRY = 3,      // internal: the single-pass kernel could not finish the row (its candidate log overflowed, a guessed
                        // threshold left too few candidates, a NaN met a sum); the multi-pass kernel redoes the row
    ROW_LARGE_K = 4,    // internal: top_k above the single-pass kernel's limit (or too large for the row's length); the
                        // multi-pass kernel takes the row
    ROW_PENDING = 5,    // internal: listed by the single-pass kernel and not answered yet (what a row keeps when a role gave up)
};

struct TailIn {
    float inv_t;
    uint32_t top_k;
    double top_p, min_p, u;
    float m, sum;
    uint32_t cnt;       // valid candidates in cand[]
    uint32_t cap;       // power of two >= cnt; cand[cnt..cap) must be 0
    uint32_t V;         // row width (cnt == V means the candidates are the whole row)
    uint64_t race_key;  // spec::raceBase(seed, pos) when race != 0
    int32_t race;
    int32_t presorted;  // cand[0..cnt) is already in descending order
    int32_t want_p;     // the caller reads p[] afterwards: leave the kept probabilities renormalised there
    int32_t have_e;     // q[0..cnt) already holds exp((l - m) * inv_t) of the candidates in cand[]'s order (which is sorted)
    int32_t sum_of_e;   // sample_tail_quick: the normaliser is the sum of those exponentials, rounded to f32 (sum is not read)
};
struct TailOut {
    int32_t status;
    uint32_t token, n;
    int32_t closed;
    double cum;  // cumulative mass of the walked candidates (ROW_OPEN_TAIL: where the id-order walk continues)
    float sum;          // sample_tail_quick with sum_of_e: the normaliser it used
    int32_t undecided;  // sample_tail_quick: a sum met a bound too closely to call
};

// f64 exp / log / division are long instruction sequences: one copy each, called (the tail runs once per row, and a
// kernel whose code does not fit the instruction cache pays for every line it has to fetch again).
static __device__ __noinline__ double f64_exp(double x) { return exp(x); }
static __device__ __noinline__ double f64_log(double x) { return log(x); }
static __device__ __noinline__ double f64_div(double a, double b) { return a / b; }

__device__ __forceinline__ uint64_t mix64(uint64_t z) {  // include/whirl/spec_sample.h:53-57
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
// E(v) = -ln(1 - U(base, v)), src/common/spec_sample.cpp:83-87
static __device__ __noinline__ double race_e(uint64_t base, uint32_t token) {
    const uint64_t z = mix64(base + (uint64_t(token) + 1ull) * 0xE7037ED1A0B428DBull);
    const double u = double(z >> 11) * (1.0 / 9007199254740992.0);
    return -f64_log(1.0 - u);
}

// Bitonic sort of cand[0..cap) in descending composite order (= logit desc, id asc).
template <int NT>
__device__ __noinline__ void sort_desc(const Group<NT>& g, uint64_t* cand, uint32_t cap) {
#pragma unroll 1
    for (uint32_t k = 2; k <= cap; k <<= 1) {
#pragma unroll 1
        for (uint32_t j = k >> 1; j > 0; j >>= 1) {
#pragma unroll 1
            for (uint32_t t = g.tid; t < (cap >> 1); t += NT) {
                // t enumerates the pairs (i, i ^ j) with i's bit j clear
                const uint32_t i = ((t & ~(j - 1)) << 1) | (t & (j - 1));
                const uint32_t q = i | j;
                const uint64_t a = cand[i], b = cand[q];
                const bool desc = (i & k) == 0;
                if (desc ? (a < b) : (a > b)) {
                    cand[i] = b;
                    cand[q] = a;
                }
            }
            g.sync();
        }
    }
}

// Descending order for exactly 4 * NT candidates, four of them in every thread's registers: exchanges at distances below 4
// run inside a thread, below 128 over warp shuffles, and only the few at 128 and above go through shared memory (with a
// barrier pair each).  cand[] holds the result.
template <int NT>
__device__ __noinline__ void sort_desc_x4(const Group<NT>& g, uint64_t* cand) {
    constexpr uint32_t CAP = 4 * NT;
    unsigned long long v0, v1, v2, v3;
    const uint32_t base = uint32_t(g.tid) * 4;
    v0 = cand[base], v1 = cand[base + 1], v2 = cand[base + 2], v3 = cand[base + 3];
    auto cx = [](unsigned long long& a, unsigned long long& b, bool desc) {  // a before b
        const unsigned long long lo = a < b ? a : b, hi = a < b ? b : a;
        a = desc ? hi : lo, b = desc ? lo : hi;
    };
    auto keep = [](unsigned long long mine, unsigned long long other, bool keep_max) {
        return keep_max ? (mine > other ? mine : other) : (mine < other ? mine : other);
    };
#pragma unroll 1
    for (uint32_t k = 2; k <= CAP; k <<= 1) {
#pragma unroll 1
        for (uint32_t j = k >> 1; j > 0; j >>= 1) {
            if (j >= 128) {
                g.sync();  // (the reads of the exchange before this one are over)
                cand[base] = v0, cand[base + 1] = v1, cand[base + 2] = v2, cand[base + 3] = v3;
                g.sync();
                const bool km = ((base & j) == 0) == ((base & k) == 0);  // (the same for the thread's four: j, k >= 4)
                v0 = keep(v0, cand[base ^ j], km), v1 = keep(v1, cand[(base + 1) ^ j], km);
                v2 = keep(v2, cand[(base + 2) ^ j], km), v3 = keep(v3, cand[(base + 3) ^ j], km);
            } else if (j >= 4) {
                const int lx = int(j >> 2);
                const bool km = ((base & j) == 0) == ((base & k) == 0);
                v0 = keep(v0, __shfl_xor_sync(0xffffffffu, v0, lx), km), v1 = keep(v1, __shfl_xor_sync(0xffffffffu, v1, lx), km);
                v2 = keep(v2, __shfl_xor_sync(0xffffffffu, v2, lx), km), v3 = keep(v3, __shfl_xor_sync(0xffffffffu, v3, lx), km);
            } else if (j == 2) {
                // pairs (0, 2) and (1, 3); k >= 4, so the direction is the same for the thread's four
                const bool desc = (base & k) == 0;
                cx(v0, v2, desc), cx(v1, v3, desc);
            } else {
                // j == 1: pairs (0, 1) and (2, 3); for k == 2 the second pair runs the other way
                const bool d01 = (base & k) == 0, d23 = ((base + 2) & k) == 0;
                cx(v0, v1, d01), cx(v2, v3, d23);
            }
        }
    }
    g.sync();
    cand[base] = v0, cand[base + 1] = v1, cand[base + 2] = v2, cand[base + 3] = v3;
    g.sync();
}

// ---- sums over the sorted candidates, by one warp.  Lane l owns the l-th block of ceil(n / 32) consecutive terms: terms are
// added in candidate order inside a block and the block sums are combined in block order.  (The host adds all terms in one
// sequence; the two orders differ by rounding in the last place only, the same size as the difference between the
// device's and the host's exp.)
__device__ __forceinline__ double warp_excl_scan(double v, double* total) {
    double incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const double t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane_id() >= o) incl += t;
    }
    *total = __shfl_sync(0xffffffffu, incl, 31);
    return incl - v;
}
// sum of v[0..n)
static __device__ __noinline__ double warp_total(const double* v, uint32_t n) {
    const uint32_t S = (n + 31) / 32, b = lane_id() * S, e = min(n, b + S);
    double s = 0;
#pragma unroll 1
    for (uint32_t i = b; i < e; ++i) s += v[i];
    double tot;
    warp_excl_scan(s, &tot);
    return tot;
}
// smallest j with cum(v[0..j]) >= t (STRICT: > t), n when there is none; *cum_end = the sum of everything walked
template <bool STRICT>
__device__ __noinline__ uint32_t warp_first_reach(const double* v, uint32_t n, double t, double* cum_end) {
    const uint32_t S = (n + 31) / 32, b = min(n, lane_id() * S), e = min(n, b + S);
    double s = 0;
#pragma unroll 1
    for (uint32_t i = b; i < e; ++i) s += v[i];
    double tot;
    double cum = warp_excl_scan(s, &tot);
    uint32_t first = n;
#pragma unroll 1
    for (uint32_t i = b; i < e; ++i) {
        cum += v[i];
        if (first == n && (STRICT ? cum > t : cum >= t)) first = i;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) first = min(first, __shfl_xor_sync(0xffffffffu, first, o));
    *cum_end = tot;
    return first;
}

// The first i in [0, n) for which pred(i) holds, n when there is none; pred is false up to some place and true from
// there on.  One warp, 32 probes per step.
template <class Pred>
__device__ __forceinline__ uint32_t warp_first_true(uint32_t n, Pred pred) {
    const uint32_t lane = uint32_t(lane_id());
    uint32_t lo = 0, len = n;
#pragma unroll 1
    while (len > 32u) {
        const uint32_t stride = (len + 31u) / 32u;
        const uint32_t off = min(len, (lane + 1u) * stride);  // the last place of the lane's stretch
        const uint32_t bal = __ballot_sync(0xffffffffu, pred(lo + off - 1u));
        if (!bal) return n;
        const uint32_t f = uint32_t(__ffs(int(bal))) - 1u;
        lo += f * stride, len = min(stride, len - f * stride);
    }
    const uint32_t bal = __ballot_sync(0xffffffffu, lane < len && pred(lo + lane));
    return bal ? lo + uint32_t(__ffs(int(bal))) - 1u : n;
}

// The same outcome as sample_tail, decided on the exponentials themselves: with e[i] = exp((l_i - m) * inv_t) and c[i]
// their running sums, "the probabilities up to i, each divided by z, reach top_p" is c[i] >= top_p * z in the same
// units, and likewise for the min-p bound and the draw, so no candidate is divided at all, one scan over the whole group
// gives every partial sum any of the steps asks for, and each cut is a search in a monotone array.  The two ways of
// computing agree unless a sum meets its bound within rounding; such a row is left undecided (the function returns false
// and the caller runs sample_tail), so that every decision made here is the one sample_tail makes: a comparison is
// trusted only when its two sides differ by more than 1e-11 of the normaliser, against at most 2e-12 of accumulated
// rounding in either form for up to 16384 candidates.
// cand: sorted; e[0..cnt): the exponentials (kept intact); c: cnt + NT / 32 doubles of scratch.  Not for rows drawn by
// the race, nor for callers that read the kept probabilities.
template <int NT>
__device__ __noinline__ bool sample_tail_quick(const Group<NT>& g, const TailIn& in, const uint64_t* cand, double* c, const double* e, TailOut* res) {
    const uint32_t cnt = in.cnt;
    // ---- running sums: thread t adds its stretch in order; the stretches' sums are combined in order
    {
        const uint32_t S = (cnt + NT - 1) / NT, b = min(cnt, uint32_t(g.tid) * S), en = min(cnt, b + S);
        double s = 0;
#pragma unroll 1
        for (uint32_t i = b; i < en; ++i) s += e[i];
        double wtot;
        double run = warp_excl_scan(s, &wtot);
        if (NT > 32) {
            double* wsum = c + cnt;
            if ((g.tid & 31) == 31) wsum[g.tid >> 5] = wtot;
            g.sync();
            double before = 0;
#pragma unroll 1
            for (int w = 0; w < (g.tid >> 5); ++w) before += wsum[w];
            run += before;
        }
#pragma unroll 1
        for (uint32_t i = b; i < en; ++i) run += e[i], c[i] = run;
    }
    g.sync();
    if (g.tid < 32) {
        const double inf = __longlong_as_double(0x7FF0000000000000ll);
        const double sum = in.sum_of_e ? double(float(c[cnt - 1])) : double(in.sum);
        uint32_t n = cnt, token = 0;
        bool closed = cnt == in.V, esc = false, tight = !(sum > 0.0 && sum < inf);
        int32_t status = ROW_DONE;
        double walked = 0.0;
        auto close_to = [&](const double* v, uint32_t j, uint32_t lim, double t, double tol) {
            bool r = false;
            if (j < lim) r = fabs(v[j] - t) <= tol;
            if (j > 0) r = r || fabs(v[j - 1] - t) <= tol;
            return r;
        };
        if (in.top_k > 0) {
            if (in.top_k <= cnt) n = in.top_k, closed = true;
            else if (!closed) esc = true;
        }
        if (!esc && !tight && in.top_p < 1.0) {
            const double z = closed ? c[n - 1] : sum;
            const double bound = in.top_p * z;
            const uint32_t j = warp_first_true(n, [&](uint32_t i) { return c[i] >= bound; });
            tight = close_to(c, j, n, bound, 1e-11 * z);
            if (j < n) n = j + 1, closed = true;
            else if (!closed) esc = true;
        }
        if (!esc && !tight && in.min_p > 0) {
            const double thr = in.min_p * e[0];
            const uint32_t j = warp_first_true(n, [&](uint32_t i) { return !(e[i] >= thr); });
            tight = close_to(e, j, n, thr, 1e-11 * thr);
            if (j == n && !closed) esc = true;
            else n = j > 1 ? j : 1, closed = true;
        }
        if (esc) status = ROW_ESCALATE;
        if (!esc && !tight) {
            const double z = closed ? c[n - 1] : sum;
            const double t = in.u * z;
            const uint32_t i = warp_first_true(n, [&](uint32_t k) { return c[k] > t; });
            tight = close_to(c, i, n, t, 1e-11 * z);
            const bool hit = i < n;
            token = cand_id(cand[hit ? i : n - 1]);  // closed and not hit: the last candidate is the fallback
            status = (hit || closed) ? ROW_DONE : ROW_OPEN_TAIL;
            if (status == ROW_OPEN_TAIL) walked = f64_div(c[n - 1], sum);
        }
        if (g.tid == 0) {
            res->status = status, res->token = token, res->n = n, res->closed = closed, res->cum = walked;
            res->sum = float(sum), res->undecided = tight;
        }
    }
    g.sync();
    return res->undecided == 0;
}

// cand: the exact candidate set (any order unless in.presorted, padded with zeros up to cap); p, q: scratch of
// cap + 2 * NT / 32 doubles each; res: one shared TailOut.  On return (after the group's barrier) cand is sorted,
// p[0..n) holds the kept probabilities (renormalised when closed) and *res the outcome.
// The steps are those of the host filter (sampler.cpp:15-78); exponentials, divisions and comparisons run on all
// threads, the running sums on the group's first warp (see above for their order).
template <int NT>
__device__ __noinline__ void sample_tail(const Group<NT>& g, const TailIn& in, uint64_t* cand, double* p, double* q, TailOut* res) {
    if (!in.presorted) sort_desc<NT>(g, cand, in.cap);
    const double inv_t = double(in.inv_t), sum = double(in.sum);
#pragma unroll 1
    for (uint32_t i = g.tid; i < in.cnt; i += NT) {
        const float l = float_of_key(cand_key(cand[i]));
        const double e = in.have_e ? q[i] : f64_exp(double(__fsub_rn(l, in.m)) * inv_t);
        p[i] = f64_div(e, sum);
    }
    g.sync();
    // ---- top-k, and the normaliser of the top-p walk (sampler.cpp:35-49)
    if (g.tid < 32) {
        uint32_t n = in.cnt;
        bool closed = in.cnt == in.V, esc = false;
        if (in.top_k > 0) {
            if (in.top_k <= in.cnt) n = in.top_k, closed = true;
            else if (!closed) esc = true;
        }
        double z = 1.0;
        if (!esc && in.top_p < 1.0 && closed) z = warp_total(p, n);
        if (g.tid == 0) {
            res->status = esc ? ROW_ESCALATE : ROW_DONE;
            res->n = n, res->closed = closed, res->cum = z, res->token = 0;
        }
    }
    g.sync();
    if (res->status == ROW_ESCALATE) return;
    if (in.top_p < 1.0) {
        // (as the host filter: every probability divided by z, then the walk until the running sum reaches top_p)
        const double z = res->cum;
        const uint32_t n0 = res->n;
#pragma unroll 1
        for (uint32_t i = g.tid; i < n0; i += NT) q[i] = f64_div(p[i], z);
        g.sync();
    }
    // ---- top-p cut, min-p cut, the renormaliser (sampler.cpp:50-74)
    if (g.tid < 32) {
        uint32_t n = res->n;
        bool closed = res->closed != 0, esc = false;
        if (in.top_p < 1.0) {
            double walked;
            const uint32_t j = warp_first_reach<false>(q, n, in.top_p, &walked);
            if (j < n) n = j + 1, closed = true;
            else if (!closed) esc = true;
        }
        if (!esc && in.min_p > 0) {
            const double thr = in.min_p * p[0];
            uint32_t j = n;  // first candidate below the threshold
#pragma unroll 1
            for (uint32_t i = lane_id(); i < n; i += 32)
                if (!(p[i] >= thr)) {
                    j = i;
                    break;
                }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) j = min(j, __shfl_xor_sync(0xffffffffu, j, o));
            if (j == n && !closed) esc = true;
            else n = j > 1 ? j : 1, closed = true;
        }
        double z = 1.0;
        if (!esc && closed) z = warp_total(p, n);
        if (g.tid == 0) {
            res->status = esc ? ROW_ESCALATE : ROW_DONE;
            res->n = n, res->closed = closed, res->cum = z;
        }
    }
    g.sync();
    if (res->status == ROW_ESCALATE) return;
    const uint32_t n = res->n;
    const bool closed = res->closed != 0;
    // A closed set is renormalised by z.  Only a caller that reads the probabilities needs them divided; the draw itself
    // compares against u * z (and the race's argmin of E / p does not change when every p is scaled alike).
    const double z_draw = (closed && !in.want_p) ? res->cum : 1.0;
    if (closed && in.want_p) {
        const double z = res->cum;
#pragma unroll 1
        for (uint32_t i = g.tid; i < n; i += NT) p[i] = f64_div(p[i], z);
    }
    g.sync();
    bool do_race = in.race != 0;
    if (do_race && !closed) {
        // open target: candidates vs tail by the stream-0 uniform (u < their mass S), src/sampling/sampler.cpp:84-93
        if (g.tid < 32) {
            const double S = warp_total(p, n);
            if (g.tid == 0) res->cum = S;
        }
        g.sync();
        do_race = in.u < res->cum;
        g.sync();
    }
    if (do_race) {
        // argmin over the kept candidates of E(id) / p, the first on ties
        double bk = __longlong_as_double(0x7FF0000000000000ll);
        uint32_t bi = 0xffffffffu;
#pragma unroll 1
        for (uint32_t i = g.tid; i < n; i += NT) {
            if (!(p[i] > 0)) continue;
            const double k = f64_div(race_e(in.race_key, cand_id(cand[i])), p[i]);
            if (k < bk) bk = k, bi = i;  // i ascends per thread: strict < keeps the first
        }
        // group argmin through shared scratch above the kept set is not available here; reduce with warp shuffles and
        // let thread 0 combine the warps through p[] beyond cap (callers give p at least cap + NT/32*2 doubles)
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const double ok = __shfl_xor_sync(0xffffffffu, bk, o);
            const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ok < bk || (ok == bk && oi < bi)) bk = ok, bi = oi;
        }
        double* wk = p + in.cap;
        if ((g.tid & 31) == 0) {
            wk[(g.tid >> 5) * 2] = bk;
            wk[(g.tid >> 5) * 2 + 1] = __longlong_as_double((long long)bi);
        }
        g.sync();
        if (g.tid == 0) {
#pragma unroll 1
            for (int w = 1; w < NT / 32; ++w) {
                const double ok = wk[w * 2];
                const uint32_t oi = (uint32_t)__double_as_longlong(wk[w * 2 + 1]);
                if (ok < bk || (ok == bk && oi < bi)) bk = ok, bi = oi;
            }
            res->token = cand_id(cand[bi == 0xffffffffu ? 0 : bi]);
            res->status = ROW_DONE;
        }
        g.sync();
        return;
    }
    if (g.tid < 32) {
        // inverse CDF over the kept candidates (sampleRow with no excluded token): the first i with cum > u
        double walked;
        const uint32_t i = warp_first_reach<true>(p, n, in.u * z_draw, &walked);
        if (g.tid == 0) {
            const bool hit = i < n;
            res->token = cand_id(cand[hit ? i : (n ? n - 1 : 0)]);  // closed and not hit: the last candidate is the fallback
            res->cum = walked;
            res->status = (hit || closed) ? ROW_DONE : ROW_OPEN_TAIL;
        }
    }
    g.sync();
}

}  // namespace wb
