// Logit penalties over a row's token history, looked up while the row is scanned.
//
// No counterpart in the reference: it parses presence / frequency penalties and ignores them
// (src/server/engine_start.cpp:70-73) and has no repetition penalty.  The rule here, for every distinct history token t
// (0 <= t < V) with count c, on the raw logit and in f32 without fusing:
//     l = x[t];  l = (l > 0) ? l / rep : l * rep;  l = l - (pres + freq * float(c))
// History ids outside [0, V) are skipped.
//
// Layout in shared memory: a V-bit map (bit t set = t is in the history), tested once per 128-bit load, and an open
// addressing table of (t + 1) | count << 19 words for the counts.  V < 2^19, history length <= kMaxHist.
#pragma once

#include "common.cuh"
#include "kernels.h"

namespace wb {

constexpr int kMaxHist = 4096;
constexpr int kPenSlots = 8192;  // table slots (power of two, at least 2 * kMaxHist)
constexpr uint32_t kPenIdBits = 19;
constexpr uint32_t kPenMaxV = (1u << kPenIdBits) - 1;

// The number of history ids a row's penalties read: hist_len clamped to the row of the history array and to kMaxHist
// (the one clamp every kernel uses).
__device__ __forceinline__ int hist_len_of(const RowParams& P, int row) {
    if (!P.hist || !P.hist_len) return 0;
    int hl = P.hist_len[row];
    hl = hl < 0 ? 0 : hl;
    hl = int64_t(hl) > P.hist_stride ? int(P.hist_stride) : hl;
    return hl > kMaxHist ? kMaxHist : hl;
}

struct PenaltyTable {
    uint32_t* bitmap;  // ceil(V / 32) words
    uint32_t* slots;   // kPenSlots words
    float rep, pres, freq;
    bool on;

    __device__ __forceinline__ static uint32_t hash(uint32_t t) { return (t * 2654435761u) >> (32 - 13); }

    // all threads of the group: clear, then insert the history (call sync between and after)
    // (bitmap and slots are 16-byte aligned and padded to multiples of four words)
    __device__ __forceinline__ void clear(int tid, int nt, uint32_t V) {
        const uint32_t quads = (((V + 31) >> 5) + 3) >> 2;
        const uint4 z = make_uint4(0, 0, 0, 0);
        for (uint32_t i = tid; i < quads; i += nt) reinterpret_cast<uint4*>(bitmap)[i] = z;
        for (uint32_t i = tid; i < kPenSlots / 4; i += nt) reinterpret_cast<uint4*>(slots)[i] = z;
    }
    __device__ __forceinline__ void insert(int32_t t, uint32_t V) {
        if (t < 0 || uint32_t(t) >= V) return;
        atomicOr(&bitmap[uint32_t(t) >> 5], 1u << (t & 31));
        const uint32_t tag = uint32_t(t) + 1;
        uint32_t h = hash(uint32_t(t));
        for (int probe = 0; probe < kPenSlots; ++probe) {
            const uint32_t old = atomicCAS(&slots[h], 0u, tag | (1u << kPenIdBits));
            if (old == 0) return;
            if ((old & kPenMaxV) == tag) {
                atomicAdd(&slots[h], 1u << kPenIdBits);
                return;
            }
            h = (h + 1) & (kPenSlots - 1);
        }
    }
    // the same for c occurrences at once
    __device__ __forceinline__ void insert_n(int32_t t, uint32_t V, uint32_t c) {
        if (t < 0 || uint32_t(t) >= V) return;
        atomicOr(&bitmap[uint32_t(t) >> 5], 1u << (t & 31));
        const uint32_t tag = uint32_t(t) + 1;
        uint32_t h = hash(uint32_t(t));
        for (int probe = 0; probe < kPenSlots; ++probe) {
            const uint32_t old = atomicCAS(&slots[h], 0u, tag | (c << kPenIdBits));
            if (old == 0) return;
            if ((old & kPenMaxV) == tag) {
                atomicAdd(&slots[h], c << kPenIdBits);
                return;
            }
            h = (h + 1) & (kPenSlots - 1);
        }
    }
    __device__ __forceinline__ uint32_t count(uint32_t t) const {
        const uint32_t tag = t + 1;
        uint32_t h = hash(t);
        for (int probe = 0; probe < kPenSlots; ++probe) {
            const uint32_t s = slots[h];
            if (s == 0) return 0;
            if ((s & kPenMaxV) == tag) return s >> kPenIdBits;
            h = (h + 1) & (kPenSlots - 1);
        }
        return 0;
    }
    __device__ __forceinline__ bool hit(uint32_t t) const { return (bitmap[t >> 5] >> (t & 31)) & 1u; }
    // bits of ids [i, i + w), i a multiple of w, w <= 32 dividing 32
    __device__ __forceinline__ uint32_t bits(uint32_t i, uint32_t w) const {
        return (bitmap[i >> 5] >> (i & 31)) & (w == 32 ? 0xffffffffu : ((1u << w) - 1));
    }
    __device__ __forceinline__ float apply(float l, uint32_t t) const {
        const uint32_t c = count(t);
        l = (l > 0.f) ? __fdiv_rn(l, rep) : __fmul_rn(l, rep);
        return __fsub_rn(l, __fadd_rn(pres, __fmul_rn(freq, float(c))));
    }
};

}  // namespace wb
