// Vocab-sharded logits (a tensor-parallel lm_head): every GPU selects the K_s best of its own slice of each row with
// GLOBAL token ids (whirl_topk_rows with id_offset) plus the slice's {max, sum exp}; the slices' candidates are exchanged
// (NCCL all-gather over NVLink, done by the host layer); this kernel merges them and samples.
//
// No counterpart in the reference (single GPU).  Exactness: the global K best are inside the union of the per-slice K_s
// best whenever K <= K_s, so candidate sets and tokens equal those of the unsharded row; the merged normaliser
// sum_s sum_s * exp((m_s - m) * inv_t) differs from the unsharded f32 sum by rounding only.
#include "kernels.h"
#include "select_smem.cuh"
#include "tail.cuh"

namespace wb {

constexpr int MT = 512;  // threads per CTA

struct MShared {
    SelScratch sel;
    TailOut res;
    float m, sum;
};

// ids / vals: [shards][rows][Ks] with cand_stride words from one shard's block to the next; stats: [shards][rows][2] with
// stat_stride words between blocks (rows * Ks and rows * 2 for three dense arrays; rows * (2 Ks + 2) for both when every
// shard's ids, vals and stats lie in one packed block, as an all-gather of such blocks leaves them).  One CTA per row
// (grid-strided).
__global__ void __launch_bounds__(MT) merge_sample_kernel(const int32_t* ids, const float* vals, const float* stats, int shards,
                                                           size_t cand_stride, size_t stat_stride, int rows, int Ks, int n_total,
                                                           RowParams P, RowOutputs out, int cap_all) {
    extern __shared__ __align__(16) uint8_t smem[];
    unsigned long long* all = reinterpret_cast<unsigned long long*>(smem);            // cap_all
    uint32_t* hist = reinterpret_cast<uint32_t*>(all + cap_all);                      // SEL_BINS
    unsigned long long* hand = reinterpret_cast<unsigned long long*>(hist + SEL_BINS);  // pow2(Ks)
    int cap_hand = 1;
    while (cap_hand < Ks) cap_hand <<= 1;
    double* tp = reinterpret_cast<double*>(hand + cap_hand);                          // cap_hand + 2 * MT / 32
    double* tq = tp + cap_hand + 2 * MT / 32;
    MShared* sh = reinterpret_cast<MShared*>(tq + cap_hand + 2 * MT / 32);
    const Group<MT> g{int(threadIdx.x), 0};
    const uint32_t total = uint32_t(shards) * uint32_t(Ks);
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        __syncthreads();
        const float inv_t = P.inv_t ? P.inv_t[row] : P.inv_t_scalar;
        const bool greedy = P.greedy && P.greedy[row];
        // ---- candidates of all slices (entries a slice left empty carry id < 0)
        for (uint32_t i = g.tid; i < total; i += MT) {
            const uint32_t s = i / uint32_t(Ks), j = i % uint32_t(Ks);
            const size_t at = size_t(s) * cand_stride + size_t(row) * Ks + j;
            const int32_t id = ids[at];
            all[i] = id >= 0 ? make_cand(key_of(fmaxf(vals[at], -INFINITY)), uint32_t(id)) : 0ull;
        }
        // ---- merged row statistics
        if (g.tid < 32) {
            float m = -INFINITY;
            for (int s = g.tid; s < shards; s += 32) m = fmaxf(m, stats[size_t(s) * stat_stride + size_t(row) * 2]);
            m = warp_max(m);
            double z = 0;
            for (int s = g.tid; s < shards; s += 32) {
                const float ms = stats[size_t(s) * stat_stride + size_t(row) * 2];
                if (ms != -INFINITY) z += double(stats[size_t(s) * stat_stride + size_t(row) * 2 + 1]) * exp(double(__fsub_rn(ms, m)) * double(inv_t));
            }
            z = warp_sum(z);
            if (g.tid == 0) sh->m = m, sh->sum = float(z);
        }
        __syncthreads();
        // ---- the global K best: K = top_k when it fits in what one slice contributes, else everything one slice could give
        uint32_t top_k = P.top_k ? uint32_t(max(P.top_k[row], 0)) : 0u;
        uint32_t K = greedy ? 1u : ((top_k > 0 && top_k <= uint32_t(Ks)) ? top_k : uint32_t(Ks));
        if (K > uint32_t(n_total)) K = uint32_t(n_total);
        // (ranked by one histogram where that applies - see bucket_sort_top -, else selected here and sorted by the tail)
        static_assert(SEL_BINS >= SB_BINS + 2 * SB_X, "bins and side list fit the select scratch");
        uint32_t kept;
        bool sorted = false;
        if (K <= 4u * MT && K <= uint32_t(cap_hand) &&
            bucket_sort_top<MT>(g, all, total, K, 0ull, hist, hand, reinterpret_cast<unsigned long long*>(hist + SB_BINS), &sh->sel)) {
            kept = sh->sel.wcnt;
            sorted = true;
        } else {
            const unsigned long long kth = select_kth<MT>(g, all, total, K, hist, &sh->sel);
            write_survivors<MT>(g, all, total, kth, hand, uint32_t(cap_hand), &sh->sel);
            kept = min(sh->sel.wcnt, K);
        }
        uint32_t cap = 1;
        while (cap < kept) cap <<= 1;
        __syncthreads();
        for (uint32_t i = kept + g.tid; i < cap; i += MT) hand[i] = 0ull;
        __syncthreads();
        if (greedy) {
            if (g.tid == 0) {
                const uint32_t tok = kept ? cand_id(hand[0]) : 0;
                out.token[row] = int32_t(tok);
                if (out.status) out.status[row] = ROW_DONE;
                if (out.n_kept) out.n_kept[row] = 1;
                if (out.closed) out.closed[row] = 1;
                if (out.stats) out.stats[2 * row] = sh->m, out.stats[2 * row + 1] = 0.f;
                if (out.kept_ids && out.kept_cap > 0) out.kept_ids[size_t(row) * out.kept_cap] = int32_t(tok);
                if (out.kept_p && out.kept_cap > 0) out.kept_p[size_t(row) * out.kept_cap] = 1.0;
            }
            continue;
        }
        TailIn in;
        in.inv_t = inv_t, in.top_k = top_k, in.top_p = P.top_p ? P.top_p[row] : 1.0, in.min_p = P.min_p ? P.min_p[row] : 0.0;
        in.u = P.u ? P.u[row] : 0.0, in.m = sh->m, in.sum = sh->sum, in.cnt = kept, in.cap = cap, in.V = uint32_t(n_total);
        in.race = P.race_key != nullptr, in.race_key = P.race_key ? P.race_key[row] : 0, in.presorted = sorted;
        in.want_p = out.kept_p != nullptr && out.kept_cap > 0;
        in.have_e = 0, in.sum_of_e = 0;
        bool decided = false;
        if (!in.race && !in.want_p && kept > 0) {
            // the division-free form first (sample_tail_quick); it leaves a row undecided when a sum meets a bound too closely
            if (!sorted) sort_desc<MT>(g, reinterpret_cast<uint64_t*>(hand), cap), in.presorted = 1;
            for (uint32_t i = g.tid; i < kept; i += MT) tq[i] = f64_exp(double(__fsub_rn(float_of_key(cand_key(hand[i])), in.m)) * double(inv_t));
            __syncthreads();
            in.have_e = 1;
            decided = sample_tail_quick<MT>(g, in, reinterpret_cast<const uint64_t*>(hand), tp, tq, &sh->res);
        }
        if (!decided) sample_tail<MT>(g, in, reinterpret_cast<uint64_t*>(hand), tp, tq, &sh->res);
        const TailOut r = sh->res;
        if (g.tid == 0) {
            out.token[row] = int32_t(r.token);
            if (out.status) out.status[row] = r.status;
            if (out.n_kept) out.n_kept[row] = int32_t(r.n);
            if (out.closed) out.closed[row] = r.closed;
            if (out.stats) out.stats[2 * row] = sh->m, out.stats[2 * row + 1] = sh->sum;
            if (out.counters && r.status == ROW_ESCALATE) atomicAdd(&out.counters[0], 1u);
            if (out.counters && r.status == ROW_OPEN_TAIL) atomicAdd(&out.counters[1], 1u);
        }
        if (r.status != ROW_ESCALATE) {
            const uint32_t nk = min(r.n, uint32_t(max(out.kept_cap, 0)));
            for (uint32_t j = g.tid; j < nk; j += MT) {
                if (out.kept_ids) out.kept_ids[size_t(row) * out.kept_cap + j] = int32_t(cand_id(hand[j]));
                if (out.kept_p) out.kept_p[size_t(row) * out.kept_cap + j] = tp[j];
            }
        }
    }
}

cudaError_t merge_sample_launch(const int32_t* ids, const float* vals, const float* stats, int shards, size_t cand_stride,
                                size_t stat_stride, int rows, int Ks, int n_total, const RowParams& P, const RowOutputs& out, int sm_count, cudaStream_t st) {
    const int cap_all = shards * Ks;
    int cap_hand = 1;
    while (cap_hand < Ks) cap_hand <<= 1;
    const size_t smem = size_t(cap_all) * 8 + SEL_BINS * 4 + size_t(cap_hand) * 8 + 2 * (size_t(cap_hand) + 2 * MT / 32) * 8 + sizeof(MShared) + 64;
    if (smem > 232448) return cudaErrorInvalidConfiguration;
    cudaError_t e = cudaFuncSetAttribute(merge_sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) return e;
    const int per_sm = smem > 110000 ? 1 : 2;
    const int grid = rows < per_sm * sm_count ? rows : per_sm * sm_count;
    merge_sample_kernel<<<grid, MT, smem, st>>>(ids, vals, stats, shards, cand_stride, stat_stride, rows, Ks, n_total, P, out, cap_all);
    return cudaGetLastError();
}

}  // namespace wb
