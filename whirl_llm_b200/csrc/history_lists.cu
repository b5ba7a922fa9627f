// Per-row hit lists for the single-pass sampler: every row's token history, reduced to its distinct tokens with their
// counts and put in the order in which that kernel meets them, stage by stage (see penalty.cuh).  The sampler then
// applies the penalties by walking a list, with no table in its shared memory and nothing built while logits stream.
//
// No counterpart in the reference (it has no logit penalties; see penalty.cuh for the rule).
//
// One CTA per row at a time: a count table in shared memory removes duplicates, the distinct tokens are counted per
// stage, a scan turns the counts into places, and every used table word goes to its stage's next place.
// Traffic: the history is read once (4 bytes per entry) and at most as much is written.
#include <cuda_runtime.h>

#include <cstdint>

#include "common.cuh"
#include "kernels.h"
#include "penalty.cuh"

namespace wb {

constexpr int HL_THREADS = 512;  // (a row takes half as long as with 256, and the rows spread over the SMs more evenly)

__global__ void __launch_bounds__(HL_THREADS) history_lists_kernel(const int32_t* hist, const int32_t* hist_len, int64_t hist_stride, int rows,
                                                                    uint32_t n, uint32_t* lists, uint32_t* starts) {
    __shared__ __align__(16) uint32_t table[kPenSlots];  // (token + 1) | count << 19
    __shared__ __align__(16) uint32_t bounds[132];       // [0] = 0, [1 + g]: stage g (n < 2^19: at most 128 stages)
    const int tid = threadIdx.x, lane = tid & 31;
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        uint32_t* st = starts + size_t(row) * kHitStartStride;
        uint32_t* list = lists + size_t(row) * kHitListStride;
        int hl = hist_len[row];
        hl = hl < 0 ? 0 : hl;
        hl = int64_t(hl) > hist_stride ? int(hist_stride) : hl;
        hl = hl > kMaxHist ? kMaxHist : hl;
        if (hl == 0) {
            if (tid < kHitStartStride) st[tid] = 0u;
            continue;
        }
        const uint4 z = make_uint4(0, 0, 0, 0);
        for (uint32_t i = tid; i < kPenSlots / 4; i += HL_THREADS) reinterpret_cast<uint4*>(table)[i] = z;
        if (tid < 132) bounds[tid] = 0u;
        __syncthreads();
        // pass 1: count every token in the table; the first sight of a token also counts it in its stage
        const int32_t* hrow = hist + size_t(row) * hist_stride;
        int32_t hv[kMaxHist / HL_THREADS];  // (all loads first: one trip to memory instead of one per token)
#pragma unroll
        for (int u = 0; u < kMaxHist / HL_THREADS; ++u) hv[u] = (tid + u * HL_THREADS) < hl ? hrow[tid + u * HL_THREADS] : -1;
#pragma unroll
        for (int u = 0; u < kMaxHist / HL_THREADS; ++u) {
            const uint32_t t = uint32_t(hv[u]);
            if (t >= n) continue;  // (negative ids too)
            const uint32_t tag = t + 1;
            uint32_t h = PenaltyTable::hash(t);
            // (a few tokens make up much of a skewed history: a repeat of a token already in the table is one add whose
            // result nobody waits for, found with a plain load; only a first sight pays for a compare-and-swap)
            for (int probe = 0; probe < kPenSlots; ++probe) {
                uint32_t old = *reinterpret_cast<volatile uint32_t*>(&table[h]);
                if (old == 0) old = atomicCAS(&table[h], 0u, tag | (1u << kPenIdBits));
                if (old == 0) {
                    atomicAdd(&bounds[1 + t / kHitStage], 1u);
                    break;
                }
                if ((old & kPenMaxV) == tag) {
                    atomicAdd(&table[h], 1u << kPenIdBits);
                    break;
                }
                h = (h + 1) & (kPenSlots - 1);
            }
        }
        __syncthreads();
        // stage sizes -> stage starts (exclusive scan over bounds[1 ..], four stages per lane of the first warp)
        if (tid < 32) {
            uint32_t c[4], sum = 0;
#pragma unroll
            for (int u = 0; u < 4; ++u) c[u] = bounds[1 + 4 * lane + u], sum += c[u];
            uint32_t inc = sum;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t y = __shfl_up_sync(0xffffffffu, inc, o);
                if (lane >= o) inc += y;
            }
            uint32_t base = inc - sum;
#pragma unroll
            for (int u = 0; u < 4; ++u) bounds[1 + 4 * lane + u] = base, base += c[u];
        }
        __syncthreads();
        // pass 2: every used table word is one distinct token with its count; it goes to its stage's next place
        for (uint32_t i = tid; i < kPenSlots / 4; i += HL_THREADS) {
            const uint4 q = reinterpret_cast<const uint4*>(table)[i];
            const uint32_t e4[4] = {q.x, q.y, q.z, q.w};
            uint32_t pos[4];  // (the four places first, then the four stores: the atomics' round trips overlap)
#pragma unroll
            for (int u = 0; u < 4; ++u) pos[u] = e4[u] ? atomicAdd(&bounds[1 + ((e4[u] & kPenMaxV) - 1) / kHitStage], 1u) : 0u;
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (e4[u]) list[pos[u]] = ((e4[u] & kPenMaxV) - 1) | (e4[u] & ~kPenMaxV);
        }
        __syncthreads();
        // (the scatter moved every stage's start to its end: bounds[c] is now the start of stage c, and of the list's end)
        if (tid < kHitStartStride) st[tid] = bounds[tid < 129 ? tid : 128];
        __syncthreads();  // the table and the bounds are cleared for the next row after this
    }
    }

size_t history_lists_ws_bytes(int rows) { return size_t(rows) * (2 * size_t(kHitListStride) + kHitStartStride) * 4; }

cudaError_t history_lists_launch(RowParams& prm, int rows, int n, int dtype, void* ws, int sm_count, cudaStream_t st) {
    (void)dtype;
    uint32_t* lists = static_cast<uint32_t*>(ws);
    uint32_t* starts = lists + size_t(rows) * kHitListStride;
    prm.hit_list = lists, prm.hit_start = starts;
    prm.hit_val = reinterpret_cast<float*>(starts + size_t(rows) * kHitStartStride);
    (void)sm_count;
    const int grid = rows;  // one CTA per row: four of them fit an SM, and a free SM takes the next row
    history_lists_kernel<<<grid, HL_THREADS, 0, st>>>(prm.hist, prm.hist_len, prm.hist_stride, rows, uint32_t(n), lists, starts);
    return cudaGetLastError();
}

}  // namespace wb
