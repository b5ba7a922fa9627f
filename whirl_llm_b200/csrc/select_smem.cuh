// Exact selection inside shared memory by a group of NT threads: the K-th largest of a set of distinct 64-bit
// candidates by adaptive-range histogram passes (2048 bins over [lo, hi] of what is left), finishing by direct
// ranking once the bin that holds the answer has few entries.
#pragma once

#include "common.cuh"

namespace wb {

constexpr int SEL_BINS = 2048;
constexpr int SEL_LIST = 256;  // rank directly when the target bin holds at most this many entries

struct SelScratch {
    unsigned long long lo, hi, kth;
    uint32_t bin, need, eq, lcnt, wcnt;
    uint32_t klo, khi, maxc;
    uint32_t wsum[32];
};


// Scanning the SEL_BINS counters of hist from the top bin down, find the bin where the running count reaches `need`
// (1 <= need <= total).  Every thread owns SEL_BINS / NT consecutive bins in registers; one barrier pair.  Results in
// sc->bin (the bin), sc->need (rank wanted inside that bin), sc->eq (entries in that bin).  nb <= SEL_BINS bins are used.
template <int NT>
__device__ __noinline__ void find_bin_desc(const Group<NT>& g, const uint32_t* hist, uint32_t need, SelScratch* sc, uint32_t* wsum) {
    constexpr int PER = SEL_BINS / NT;
    static_assert(PER >= 4 && PER % 4 == 0, "bins per thread");
    uint32_t c[PER];
    // thread t owns bins [SEL_BINS - (t + 1) * PER, SEL_BINS - t * PER), scanned from its top down
    const uint4* src = reinterpret_cast<const uint4*>(hist + SEL_BINS - (g.tid + 1) * PER);
#pragma unroll
    for (int q = 0; q < PER / 4; ++q) {
        const uint4 v = src[q];
        c[q * 4] = v.x, c[q * 4 + 1] = v.y, c[q * 4 + 2] = v.z, c[q * 4 + 3] = v.w;
    }
    uint32_t s = 0;
#pragma unroll
    for (int j = 0; j < PER; ++j) s += c[j];
    const uint32_t incl_w = warp_scan_incl(s);
    if ((g.tid & 31) == 31) wsum[g.tid >> 5] = incl_w;
    g.sync();
    uint32_t before = 0;
#pragma unroll 1
    for (int w = 0; w < (g.tid >> 5); ++w) before += wsum[w];
    const uint32_t incl = before + incl_w, excl = incl - s;
    if (excl < need && incl >= need) {
        uint32_t r = need - excl;
        bool found = false;
#pragma unroll
        for (int j = PER - 1; j >= 0; --j) {  // c[PER - 1] is the thread's top bin
            if (!found) {
                if (c[j] >= r) {
                    sc->bin = SEL_BINS - (g.tid + 1) * PER + j, sc->need = r, sc->eq = c[j];
                    found = true;
                } else {
                    r -= c[j];
                }
            }
        }
    }
    g.sync();
}

// The K-th largest of buf[0..cnt) (1 <= K <= cnt; entries distinct; zeros allowed as "empty", they rank last).
// hist: SEL_BINS words of shared scratch (also used as a list of up to SEL_LIST candidates).  Every thread of the
// group calls it and gets the same answer.
// MASKED: entries whose bit 31 is clear (log entries that still carry a raw logit) count as empty.
template <int NT, bool MASKED = false>
__device__ __noinline__ unsigned long long select_kth(const Group<NT>& g, const unsigned long long* buf, uint32_t cnt, uint32_t K,
                                         uint32_t* hist, SelScratch* sc) {
    auto entry = [&](uint32_t i) -> unsigned long long {
        const unsigned long long c = buf[i];
        return (MASKED && !(c & 0x80000000ull)) ? 0ull : c;
    };
    if (g.tid == 0) sc->lo = ~0ull, sc->hi = 0ull;
    g.sync();
    {
        unsigned long long lo = ~0ull, hi = 0ull;
#pragma unroll 1
        for (uint32_t i = g.tid; i < cnt; i += NT) {
            const unsigned long long c = entry(i);
            lo = c < lo ? c : lo, hi = c > hi ? c : hi;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const unsigned long long l2 = __shfl_xor_sync(0xffffffffu, lo, o), h2 = __shfl_xor_sync(0xffffffffu, hi, o);
            lo = l2 < lo ? l2 : lo, hi = h2 > hi ? h2 : hi;
        }
        if ((g.tid & 31) == 0) atomicMin(&sc->lo, lo), atomicMax(&sc->hi, hi);
    }
    g.sync();
    unsigned long long lo = sc->lo, hi = sc->hi;
    uint32_t need = K;
#pragma unroll 1
    for (int pass = 0; pass < 8; ++pass) {
        const unsigned long long range = hi - lo;
        if (range == 0) return lo;
        const int bits = 64 - __clzll((long long)range);
        const int sa = bits > 11 ? bits - 11 : 0;  // (range >> sa) < SEL_BINS
#pragma unroll 1
        for (int i = g.tid; i < SEL_BINS / 4; i += NT) reinterpret_cast<uint4*>(hist)[i] = make_uint4(0, 0, 0, 0);
        g.sync();
#pragma unroll 1
        for (uint32_t i = g.tid; i < cnt; i += NT) {
            const unsigned long long c = entry(i);
            if (c >= lo && c <= hi) atomicAdd(&hist[uint32_t((c - lo) >> sa)], 1u);
        }
        g.sync();
        find_bin_desc<NT>(g, hist, need, sc, sc->wsum);
        if (g.tid == 0) sc->lcnt = 0;
        g.sync();
        const uint32_t b = sc->bin, cb = sc->eq;
        need = sc->need;
        const unsigned long long nlo = lo + ((unsigned long long)b << sa);
        if (sa == 0) return nlo;
        unsigned long long nhi = nlo + ((1ull << sa) - 1);
        nhi = nhi > hi ? hi : nhi;
        if (cb <= SEL_LIST) {
            unsigned long long* list = reinterpret_cast<unsigned long long*>(hist);
#pragma unroll 1
            for (uint32_t i = g.tid; i < cnt; i += NT) {
                const unsigned long long c = entry(i);
                if (c >= nlo && c <= nhi) list[atomicAdd(&sc->lcnt, 1u)] = c;
            }
            g.sync();
#pragma unroll 1
            for (uint32_t t = g.tid; t < cb; t += NT) {
                const unsigned long long mine = list[t];
                uint32_t rank = 0;
#pragma unroll 1
                for (uint32_t j = 0; j < cb; ++j) rank += list[j] > mine;
                if (rank == need - 1) sc->kth = mine;
            }
            g.sync();
            return sc->kth;
        }
        lo = nlo, hi = nhi;
        g.sync();
    }
    return lo;
}

// Entries >= kth of buf[0..cnt) -> dst[0..), any order; after the call sc->wcnt holds how many.
template <int NT>
__device__ __noinline__ void write_survivors(const Group<NT>& g, const unsigned long long* buf, uint32_t cnt, unsigned long long kth,
                                unsigned long long* dst, uint32_t dst_cap, SelScratch* sc) {
    if (g.tid == 0) sc->wcnt = 0;
    g.sync();
    const uint32_t rounds = (cnt + NT - 1) / NT;
#pragma unroll 1
    for (uint32_t r = 0; r < rounds; ++r) {
        const uint32_t i = r * NT + g.tid;
        const unsigned long long c = i < cnt ? buf[i] : 0ull;
        const bool take = i < cnt && c >= kth && c != 0ull;
        const uint32_t bal = __ballot_sync(0xffffffffu, take);
        if (bal) {
            uint32_t base = 0;
            if (lane_id() == 0) base = atomicAdd(&sc->wcnt, uint32_t(__popc(bal)));
            base = __shfl_sync(0xffffffffu, base, 0);
            const uint32_t pos = base + __popc(bal & ((1u << lane_id()) - 1));
            if (take && pos < dst_cap) dst[pos] = c;
        }
    }
    g.sync();
}

// The K largest of buf[0..cnt) in descending order, by one histogram instead of a selection followed by a sorting
// network: the entries' ordering keys are spread over SB_BINS bins between the smallest and the largest key (the bin is
// monotone in the key, equal keys share a bin), a scan of the bin counts gives every bin its first place in the output,
// the entries are scattered to their bins' places, and each one then finds its exact place by counting the larger
// entries of its own bin.  The bin that straddles place K goes through a side list (xlist), where its entries rank
// themselves and the first of them take the places that are left.  Work per entry is a few instructions plus the size of
// its bin, against the several hundred compare-exchanges per entry of a network.
// buf: entries distinct; zero = empty; entries below `floor` count as empty too (the caller knows that at least
// min(K, what is there) entries are at or above it).  K <= 4 * NT (sc->wsum holds one word per warp: NT <= 1024).  bins: SB_BINS words; out: K entries; xlist: SB_X
// entries.  Returns false, with nothing usable in out, when one bin holds more than SB_X entries (many equal logits): the
// caller then takes the selection-and-network path.  On success sc->wcnt = entries written, out[0..wcnt) descending.
constexpr int SB_BINS = 1024;
constexpr int SB_X = 256;
template <int NT>
__device__ __noinline__ bool bucket_sort_top(const Group<NT>& g, const unsigned long long* buf, uint32_t cnt, uint32_t K,
                                             unsigned long long floor, uint32_t* bins, unsigned long long* out,
                                             unsigned long long* xlist, SelScratch* sc) {
    constexpr int PER = SB_BINS / NT;  // bins per thread
    static_assert(PER >= 1 && PER * NT == SB_BINS && SB_X <= NT, "whole bins per thread, one side-list entry per thread");
    // ---- the keys' range
    if (g.tid == 0) sc->klo = 0xffffffffu, sc->khi = 0u, sc->maxc = 0u, sc->bin = 0xffffffffu, sc->need = 0u, sc->eq = 0u, sc->wcnt = 0u;
#pragma unroll
    for (int j = 0; j < PER; ++j) bins[PER * g.tid + j] = 0u;
    g.sync();
    {
        uint32_t lo = 0xffffffffu, hi = 0u;
#pragma unroll 4
        for (uint32_t i = g.tid; i < cnt; i += NT) {
            const unsigned long long c = buf[i];
            if (c != 0ull && c >= floor) {
                const uint32_t k = cand_key(c);
                lo = min(lo, k), hi = max(hi, k);
            }
        }
        lo = __reduce_min_sync(0xffffffffu, lo), hi = __reduce_max_sync(0xffffffffu, hi);
        if ((g.tid & 31) == 0) atomicMin(&sc->klo, lo), atomicMax(&sc->khi, hi);
    }
    g.sync();
    const uint32_t klo = sc->klo, khi = sc->khi;
    if (klo > khi) {  // (nothing there)
        g.sync();
        return true;
    }
    // bin 0 holds the largest keys
    const float inv = float(SB_BINS) / (float(khi - klo) + 1.0f) * 0.99999f;
    auto bin_of = [&](unsigned long long c) -> uint32_t {
        const uint32_t b = uint32_t(float(cand_key(c) - klo) * inv);
        return uint32_t(SB_BINS - 1) - min(b, uint32_t(SB_BINS - 1));
    };
#pragma unroll 4
    for (uint32_t i = g.tid; i < cnt; i += NT) {
        const unsigned long long c = buf[i];
        if (c != 0ull && c >= floor) atomicAdd(&bins[bin_of(c)], 1u);
    }
    g.sync();
    // ---- every bin's first place: an exclusive scan of the counts (every thread owns PER consecutive bins)
    {
        uint32_t c[PER], st[PER], s = 0;
#pragma unroll
        for (int j = 0; j < PER; ++j) c[j] = bins[PER * g.tid + j], s += c[j];
        const uint32_t incl_w = warp_scan_incl(s);
        if ((g.tid & 31) == 31) sc->wsum[g.tid >> 5] = incl_w;
        g.sync();
        uint32_t before = 0;
#pragma unroll 1
        for (int w = 0; w < (g.tid >> 5); ++w) before += sc->wsum[w];
        uint32_t run = before + incl_w - s;
        uint32_t mc = 0;
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            st[j] = run, run += c[j];
            bins[PER * g.tid + j] = st[j];
            if (st[j] < K) mc = max(mc, c[j]);
            if (st[j] < K && st[j] + c[j] > K) sc->bin = uint32_t(PER * g.tid + j), sc->need = K - st[j], sc->eq = c[j];  // (at most one bin)
        }
        mc = __reduce_max_sync(0xffffffffu, mc);
        if ((g.tid & 31) == 0 && mc) atomicMax(&sc->maxc, mc);
        if (g.tid == NT - 1) sc->lcnt = run;  // entries in all
    }
    g.sync();
    if (sc->maxc > uint32_t(SB_X)) {
        g.sync();
        return false;
    }
    const uint32_t xbin = sc->bin, x_need = sc->need, x_cnt = sc->eq, total = sc->lcnt;
    const uint32_t kept = total < K ? total : K;
    const uint32_t x_start = xbin != 0xffffffffu ? K - x_need : kept;  // places filled by whole bins
    // ---- scatter: a bin's counter now hands out its places (and ends as the bin's end); bins past place K drop out
#pragma unroll 2
    for (uint32_t i = g.tid; i < cnt; i += NT) {
        const unsigned long long c = buf[i];
        if (c != 0ull && c >= floor) {
            const uint32_t b = bin_of(c);
            if (b == xbin) {
                xlist[atomicAdd(&sc->wcnt, 1u)] = c;
            } else {
                const uint32_t pos = atomicAdd(&bins[b], 1u);
                if (pos < K) out[pos] = c;
            }
        }
    }
    g.sync();
    // ---- the exact place of every kept entry: its bin's first place plus the larger entries of the bin
    unsigned long long item[4];
    uint32_t np[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const uint32_t i = uint32_t(r) * NT + uint32_t(g.tid);
        np[r] = 0xffffffffu;
        if (i < x_start) {
            const unsigned long long mine = out[i];
            const uint32_t b = bin_of(mine);
            const uint32_t e = bins[b], s0 = b ? bins[b - 1] : 0u;  // (the bins before a kept one are whole bins: their counters hold their ends)
            uint32_t rank = 0;
#pragma unroll 4
            for (uint32_t j = s0; j < e; ++j) rank += out[j] > mine;
            item[r] = mine, np[r] = s0 + rank;
        }
    }
    unsigned long long xi = 0ull;
    uint32_t xp = 0xffffffffu;
    if (uint32_t(g.tid) < x_cnt) {
        xi = xlist[g.tid];
        uint32_t rank = 0;
#pragma unroll 4
        for (uint32_t j = 0; j < x_cnt; ++j) rank += xlist[j] > xi;
        if (rank < x_need) xp = x_start + rank;
    }
    g.sync();
#pragma unroll
    for (int r = 0; r < 4; ++r)
        if (np[r] != 0xffffffffu) out[np[r]] = item[r];
    if (xp != 0xffffffffu) out[xp] = xi;
    if (g.tid == 0) sc->wcnt = kept;
    g.sync();
    return true;
}

// A lower bound of the K-th largest ordering key among n floats in shared memory (1 <= K <= n): the key's top 22 bits
// by two digit passes (11 + 11), low bits zero, so at least K elements have a key at or above the result.  NaN ranks
// lowest.  hist: SEL_BINS words.
template <int NT, typename T>
__device__ __noinline__ uint32_t select_key_bound(const Group<NT>& g, const T* x, uint32_t n, uint32_t K, uint32_t* hist, SelScratch* sc) {
    uint32_t prefix = 0, mask = 0, need = K;
    const int shifts[2] = {21, 10};
#pragma unroll 1
    for (int ps = 0; ps < 2; ++ps) {
#pragma unroll 1
        for (int i = g.tid; i < SEL_BINS / 4; i += NT) reinterpret_cast<uint4*>(hist)[i] = make_uint4(0, 0, 0, 0);
        g.sync();
#pragma unroll 1
        for (uint32_t i = g.tid; i < n; i += NT) {
            const float v = sizeof(T) == 4 ? reinterpret_cast<const float*>(x)[i] : bf16_to_f32(reinterpret_cast<const uint16_t*>(x)[i]);
            const uint32_t k = key_of(v);
            if ((k & mask) == prefix) atomicAdd(&hist[(k >> shifts[ps]) & 2047u], 1u);
        }
        g.sync();
        find_bin_desc<NT>(g, hist, need, sc, sc->wsum);
        prefix |= sc->bin << shifts[ps];
        need = sc->need;
        mask |= 2047u << shifts[ps];
        g.sync();
    }
    return prefix;
}

}  // namespace wb
