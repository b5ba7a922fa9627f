// The single-pass fused sampler: every logits row is read from HBM once, by plain 128-bit loads.
//
// One persistent CTA per SM, two roles that never meet at a CTA-wide barrier while rows stream:
//   stream warps (16)   Each thread keeps P_PF tiles of 64 bytes on their way from global memory in registers (a software
//                       pipeline that runs on across row boundaries), folds every tile into a per-lane running maximum
//                       (and, where the row needs its softmax normaliser, a running sum of exponentials), and tests the
//                       tile's maximum against the row's threshold.  The few logits at or above the threshold are
//                       appended to the row's candidate log in shared memory.
//   tail group (8 warps) Before a row streams: its first threshold, from a strided sample of the row (the "scout": the K-th
//                       largest of a sample is reached by at least K logits of the row), and, with penalties, a bit map of
//                       the row's history tokens.  While it streams: the exact K-th largest of the log so far is a valid
//                       and ever tighter threshold.  When it is through: the penalised history tokens join the log, the
//                       exact K best are ranked, then top-k / top-p / min-p in f64, the draw and the row's outputs.
// The two roles work on alternating row slots (two logs, two bit maps), so the tail of one row overlaps the streaming of
// the next.
//
// Why a threshold from partial data is exact: an element is dropped only when it is below a value that at least K
// elements of the same row reach, so the K best are always in the log; the final select over the log is exact.
//
// Penalties.  The tokens of a row's history are kept out of the stream (their raw logits must not count) and join the
// row with their penalised values at its end.  A row that needs no normaliser looks the bit map up only for the rare
// logit that passes the threshold; a row that needs one masks every quad of logits with four bits of the map.
//
// It replaces the reference's topk_rows kernel (seven passes over the row, kernels/shared/sample_cand_topk_rows.h:11-98),
// the candidate download, and the host filter and draw (src/sampling/sampler.cpp:15-147).
#include <type_traits>

#include "kernels.h"
#include "penalty.cuh"
#include "select_smem.cuh"
#include "tail.cuh"

namespace wb {

constexpr int P_SW = 16;                 // stream warps
constexpr int P_ST = P_SW * 32;
#ifndef WB_TW
#define WB_TW 8
#endif
constexpr int P_TW = WB_TW;              // tail warps
constexpr int P_TT = P_TW * 32;
constexpr int P_THREADS = P_ST + P_TT;
#ifndef WB_PF
#define WB_PF 2
#endif
constexpr int P_PF = WB_PF;              // tiles on their way per stream thread (64 bytes each)
constexpr int P_L = 4096;                // candidate log entries per row slot
constexpr int P_RED = P_SW + P_TW;       // partial (max, exponent, sum) triples per row: stream warps, then tail warps

struct PSlot {
    unsigned long long tau;  // current threshold candidate; elements must beat it to be logged
    uint32_t cnt;            // log entries reserved so far (may exceed P_L: overflow); bit 31: a NaN poisoned a sum
    int32_t row;
    float red_m[P_RED];
    float red_e[P_RED];
    double red_s[P_RED];
    uint32_t wbound[P_SW];   // per stream warp: its own lower bound (an ordering key)
};

struct PShared {
    PSlot slot[2];
    SelScratch sel;
    TailOut res;
    uint32_t flag[4];
    uint32_t sbound[P_TW];   // the scout's per-warp bounds
};

__device__ __forceinline__ unsigned long long ldv_u64(const unsigned long long* p) {
    return *reinterpret_cast<const volatile unsigned long long*>(p);
}
__device__ __forceinline__ uint32_t ldv_u32(const uint32_t* p) { return *reinterpret_cast<const volatile uint32_t*>(p); }
__device__ __forceinline__ uint4 ld_stream(const uint4* p) { return __ldcs(p); }

// Called by one warp of every CTA once all the CTA's rows have their status.  The CTA that gets here last lists the rows
// the multi-pass kernel has to take (a.fin_list, a.fin_counts[1]; bit 30: redo at the first level), so that no helper
// launch is needed between the two kernels.  a.fin_counts[2] is the ticket (zero before the launch, zero again after).
__device__ void list_leftovers(const SelectArgs& a) {
    const int lane = lane_id();
    __threadfence();
    uint32_t last = 0;
    if (lane == 0) last = atomicAdd(reinterpret_cast<unsigned int*>(a.fin_counts + 2), 1u) == gridDim.x - 1 ? 1u : 0u;
    last = __shfl_sync(0xffffffffu, last, 0);
    if (!last) return;
    __threadfence();
    const int32_t* status = a.out.status;
    int cnt = 0;
    for (int base = 0; base < a.rows; base += 256) {
        int st8[8];  // (eight loads on their way at once: this is the last thing the kernel does)
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int r = base + 32 * j + lane;
            st8[j] = r < a.rows ? __ldcg(status + r) : int(ROW_DONE);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int r = base + 32 * j + lane;
            const int st = st8[j];
            const bool redo = st == ROW_RETRY || st == ROW_OPEN_TAIL;
            const bool take = redo || st == ROW_LARGE_K || st == ROW_ESCALATE;
            const uint32_t bal = __ballot_sync(0xffffffffu, take);
            if (take) a.fin_list[cnt + __popc(bal & ((1u << lane) - 1))] = r | (redo ? (1 << 30) : 0);
            cnt += __popc(bal);
        }
    }
    if (lane == 0) a.fin_counts[1] = cnt, a.fin_counts[2] = 0;
}

// The r-th largest of the warp's 32 * G keys (kv[0..G) per lane; 0 = none), by taking the largest away r - 1 times.
// Equal keys of distinct elements count separately.  0 when the warp holds fewer than r keys.
template <int G>
__device__ __forceinline__ uint32_t warp_rth_largest(uint32_t (&kv)[G], uint32_t r) {
    const int lane = lane_id();
    uint32_t kr = 0;
    for (uint32_t i = 0; i < r; ++i) {
        uint32_t mx = kv[0];
#pragma unroll
        for (int j = 1; j < G; ++j) mx = kv[j] > mx ? kv[j] : mx;
        kr = __reduce_max_sync(0xffffffffu, mx);
        if (kr == 0) break;
        const uint32_t holders = __ballot_sync(0xffffffffu, mx == kr);
        if (lane == __ffs(holders) - 1) {
            bool gone = false;
#pragma unroll
            for (int j = 0; j < G; ++j)
                if (!gone && kv[j] == kr) kv[j] = 0, gone = true;
        }
    }
    return kr;
}

template <typename T>
__global__ void __launch_bounds__(P_THREADS, 1) single_pass_kernel(SelectArgs a, int bm_words, int max_k) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int VE = 16 / int(sizeof(T));      // logits per 128-bit load
    constexpr uint32_t TILE_Q = P_ST * 4;        // 128-bit words per tile
    unsigned long long* logs = reinterpret_cast<unsigned long long*>(smem);              // 2 * P_L
    uint32_t* hist = reinterpret_cast<uint32_t*>(logs + 2 * P_L);                        // SEL_BINS
    unsigned long long* hand = reinterpret_cast<unsigned long long*>(hist + SEL_BINS);   // max_k: a row's candidates
    double* tail_p = reinterpret_cast<double*>(hand + max_k);                            // max_k + 2 * P_TW
    double* tail_q = tail_p + max_k + 2 * P_TW;
    uint64_t* bars = reinterpret_cast<uint64_t*>(tail_q + max_k + 2 * P_TW);             // 4
    PShared* sh = reinterpret_cast<PShared*>(bars + 4);
    uint32_t* bitmaps = reinterpret_cast<uint32_t*>((reinterpret_cast<uintptr_t>(sh + 1) + 15) & ~uintptr_t(15));  // 2 * bm_words
    uint32_t* pslots = bitmaps + 2 * size_t(bm_words);                                   // kPenSlots (only with penalties)
    uint64_t *boot_done = bars, *closed = bars + 2;  // per slot: the slot is the row's / every stream warp is through the row

    const int tid = threadIdx.x;
    const uint32_t n = uint32_t(a.n);
    const int n_rows = a.row_count ? min(*a.row_count, a.rows) : a.rows;
    const int my_rows = n_rows > int(blockIdx.x) ? (n_rows - int(blockIdx.x) + int(gridDim.x) - 1) / int(gridDim.x) : 0;
    const uint32_t row_q = n / VE;  // 128-bit words per row (rows are 16-byte multiples)
    const uint32_t n_tiles = (row_q + TILE_Q - 1) / TILE_Q;
    const bool sample = a.mode == MODE_SAMPLE;
    const RowParams& P = a.prm;
    auto row_of = [&](int k) -> int {
        const int li = int(blockIdx.x) + k * int(gridDim.x);
        return a.row_list ? a.row_list[li] : li;
    };
    // rows whose top_k is above this launch's limit are left to the multi-pass kernel (both roles skip them alike)
    auto is_large = [&](int row) -> bool {
        if (!sample || !P.top_k) return false;
        if (P.greedy && P.greedy[row]) return false;
        return P.top_k[row] > max_k;
    };
    auto next_row = [&](int k) -> int {
        for (++k; k < my_rows && is_large(row_of(k)); ++k) {}
        return k;
    };
    // candidates wanted for a row (both roles must agree)
    auto k_of = [&](int row) -> uint32_t {
        uint32_t K;
        if (sample) {
            const bool greedy = P.greedy && P.greedy[row];
            const uint32_t tk = P.top_k ? uint32_t(max(P.top_k[row], 0)) : 0u;
            K = greedy ? 1u : ((tk > 0 && tk <= uint32_t(max_k)) ? tk : uint32_t(min(a.level_k, max_k)));
        } else {
            K = uint32_t(a.K);
        }
        return K > n ? n : K;
    };
    // Rows whose kept set is closed by their own top_k need no softmax normaliser: every probability the filter compares
    // is a ratio inside the candidate set, so the row sum cancels.  When the caller does not ask for the row statistics
    // either, the stream warps skip the exponentials and the tail normalises over the candidates.
    auto no_sum_row = [&](int row) -> bool {
        if (!sample) return false;
        if (P.greedy && P.greedy[row]) return true;
        if (a.out.stats || !P.top_k) return false;
        const int tk = P.top_k[row];
        return tk >= 1 && tk <= max_k && uint32_t(tk) <= n;
    };
    // does the row have penalties to apply (both roles must agree)
    auto pen_row = [&](int row) -> bool {
        if (!sample || !P.hist || bm_words == 0 || P.hist_len[row] <= 0) return false;
        const float r = P.rep ? P.rep[row] : 1.f, pr = P.pres ? P.pres[row] : 0.f, fr = P.freq ? P.freq[row] : 0.f;
        return r != 1.f || pr != 0.f || fr != 0.f;
    };

    if (tid == 0) {
        for (int p = 0; p < 2; ++p) mbar_init(&boot_done[p], 1), mbar_init(&closed[p], P_SW);
        mbar_fence_init();
    }
    for (int i = tid; i < 2 * P_L; i += P_THREADS) logs[i] = 0ull;
    __syncthreads();
    if (my_rows == 0 || next_row(-1) >= my_rows) {
        if (a.out.status && sample)
            for (int k = tid; k < my_rows; k += P_THREADS) a.out.status[row_of(k)] = ROW_LARGE_K;
        if (a.fin_list) {
            __threadfence();
            __syncthreads();
            if (tid < 32) list_leftovers(a);
        }
        return;
    }

    // =========================================================== tail group
    if (tid >= P_ST) {
        const Group<P_TT> g{tid - P_ST, 1};
        const int lane = lane_id(), tw = g.tid >> 5;

        // ---- a slot becomes a row's: the history bit map, the first threshold (the scout), an empty log
        auto boot = [&](int k, int o) {
            const int p = o & 1;
            PSlot* sl = &sh->slot[p];
            const int row = row_of(k);
            const uint32_t K = k_of(row);
            const bool pen_on = pen_row(row);
            uint32_t* bm = bitmaps + size_t(p) * bm_words;
            if (pen_on) {
                const uint4 z = make_uint4(0, 0, 0, 0);
                for (int i = g.tid; i < bm_words / 4; i += P_TT) reinterpret_cast<uint4*>(bm)[i] = z;
                g.sync();
                const int32_t* h = P.hist + size_t(row) * P.hist_stride;
                int hl = P.hist_len[row];
                hl = int64_t(hl) > P.hist_stride ? int(P.hist_stride) : hl;
                hl = hl > kMaxHist ? kMaxHist : hl;
                for (int i = g.tid; i < hl; i += P_TT) {
                    const uint32_t t = uint32_t(h[i]);
                    if (t < n) atomicOr(&bm[t >> 5], 1u << (t & 31));
                }
                g.sync();
            }
            // The scout: 32 logits per thread, 8192 per row, in chunks of one warp-wide load spread evenly over the row
            // (the whole row when it is no longer than that).  Every thread keeps the maxima of its four groups of eight;
            // each warp names the r-th largest of what it holds, r = ceil(K / warps): the smallest of those bounds is
            // reached by at least K distinct logits of the row.  History tokens do not count (bit map).
            constexpr int SC_LD = 32 / VE;                 // loads per thread
            constexpr uint32_t NC = SC_LD * P_TW;           // chunks
            constexpr uint32_t CE = 32 * VE;                // logits per chunk
            const uint4* xr = reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(a.x) + size_t(row) * n);
            uint4 sv[SC_LD];
            uint32_t sid[SC_LD];
#pragma unroll
            for (int l = 0; l < SC_LD; ++l) {
                const uint32_t c = uint32_t(l) * P_TW + uint32_t(tw);
                const uint32_t start = n <= NC * CE ? c * CE : uint32_t((uint64_t(c) * n) / NC) & ~uint32_t(VE - 1);
                sid[l] = start + uint32_t(lane) * VE;
                const uint32_t nw = sizeof(T) == 4 ? 0xff800000u : 0xff80ff80u;  // -inf
                sv[l] = sid[l] + VE <= n ? __ldg(xr + sid[l] / VE) : make_uint4(nw, nw, nw, nw);
            }
            float gm[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int l = 0; l < SC_LD; ++l) {
                float v[VE];
                const uint32_t w4[4] = {sv[l].x, sv[l].y, sv[l].z, sv[l].w};
                if (sizeof(T) == 4) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) v[j] = __uint_as_float(w4[j]);
                } else {
#pragma unroll
                    for (int j = 0; j < 4; ++j) v[2 * j] = __uint_as_float(w4[j] << 16), v[2 * j + 1] = __uint_as_float(w4[j] & 0xffff0000u);
                }
                if (pen_on && sid[l] < n) {
                    const uint32_t bits = (bm[sid[l] >> 5] >> (sid[l] & 31)) & ((1u << VE) - 1);
#pragma unroll
                    for (int j = 0; j < VE; ++j)
                        if ((bits >> j) & 1u) v[j] = -INFINITY;
                }
                float mx = v[0];
#pragma unroll
                for (int j = 1; j < VE; ++j) mx = fmaxf(mx, v[j]);
                const int grp = l * 4 / SC_LD;  // f32: two loads per group of eight; bf16: one
                gm[grp] = fmaxf(gm[grp], mx);
            }
            // (a group that is all -inf, e.g. past the end of a short row, must not count as an element: key 0)
            const uint32_t r = (K + P_TW - 1) / P_TW;
            uint32_t kb = 0;
            if (r <= 8) {
                uint32_t kv[1];
                const float mx = fmaxf(fmaxf(gm[0], gm[1]), fmaxf(gm[2], gm[3]));
                kv[0] = mx == -INFINITY ? 0u : key_of(mx);
                kb = warp_rth_largest<1>(kv, r);
            } else if (r <= 64) {
                uint32_t kv[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) kv[j] = gm[j] == -INFINITY ? 0u : key_of(gm[j]);
                kb = warp_rth_largest<4>(kv, r);
            }
            if (lane == 0) sh->sbound[tw] = kb;
            g.sync();
            if (g.tid == 0) {
                uint32_t kmin = 0xffffffffu;
                for (int w = 0; w < P_TW; ++w) kmin = min(kmin, sh->sbound[w]);
                sl->tau = (unsigned long long)kmin << 32;
                sl->cnt = 0;
                sl->row = row;
                for (int w = 0; w < P_SW; ++w) sl->wbound[w] = 0u;
                mbar_arrive(&boot_done[p]);
            }
            g.sync();
        };

        // ---- raise a streaming row's threshold to the exact K-th largest of its log so far, when the log has grown
        uint32_t rf_last[2] = {0, 0}, rf_step[2] = {0, 0};
        auto maybe_refine = [&](int p, uint32_t K) {
            PSlot* sl = &sh->slot[p];
            if (g.tid == 0) {
                const uint32_t c = ldv_u32(&sl->cnt) & 0x7fffffffu;
                sh->flag[2] = c < uint32_t(P_L) ? c : uint32_t(P_L);
            }
            g.sync();
            const uint32_t nlog = sh->flag[2];
            g.sync();
            if (!(nlog >= K && nlog >= 64 && nlog >= rf_last[p] + rf_step[p])) return false;
            // (entries reserved but not written yet read as zero and rank last: the bound stays valid)
            const unsigned long long kth = select_kth<P_TT>(g, logs + size_t(p) * P_L, nlog, K, hist, &sh->sel);
            if (g.tid == 0 && kth > ldv_u64(&sl->tau)) *reinterpret_cast<volatile unsigned long long*>(&sl->tau) = kth;
            rf_last[p] = nlog;
            rf_step[p] = 2 * K > 128 ? 2 * K : 128;
            g.sync();
            return true;
        };

        if (sample && a.out.status)
            for (int k = g.tid; k < my_rows; k += P_TT)
                if (is_large(row_of(k))) a.out.status[row_of(k)] = ROW_LARGE_K;
        {
            const int k0 = next_row(-1);
            boot(k0, 0);
            const int k1 = next_row(k0);
            if (k1 < my_rows) boot(k1, 1);
        }
        int ord = 0;
        for (int k = next_row(-1); k < my_rows; ++ord) {
            const int kn = next_row(k);
            const int kn2 = kn < my_rows ? next_row(kn) : my_rows;
            const int p = ord & 1;
            PSlot* sl = &sh->slot[p];
            unsigned long long* log = logs + size_t(p) * P_L;
            const int row = row_of(k);
            const uint32_t K = k_of(row);
            const uint32_t K_next = kn < my_rows ? k_of(row_of(kn)) : 1u;
            // ---- while the row streams: raise its threshold
            for (uint32_t spin = 0;; ++spin) {
                if (g.tid == 0) sh->flag[1] = mbar_try_wait(&closed[p], (ord >> 1) & 1) ? 1u : 0u;
                g.sync();
                const bool done = sh->flag[1] != 0;
                g.sync();
                if (done) break;
                if (spin > (1u << 21)) {
                    if (g.tid == 0) atomicExch(a.err, 3u);
                    return;
                }
                if (!maybe_refine(p, K)) __nanosleep(500);
            }
            mbar_wait(&closed[p], (ord >> 1) & 1);  // acquire the stream warps' writes
            rf_last[p] = rf_step[p] = 0;
            // ---- the row is through
            const bool greedy = sample && P.greedy && P.greedy[row];
            const float inv_t = P.inv_t ? P.inv_t[row] : P.inv_t_scalar;
            const bool no_sum = no_sum_row(row);
            const bool pen_on = pen_row(row);
            if (pen_on) {
                // The row's distinct history tokens with their counts (an open-addressing table in shared memory), their raw
                // logits from global memory, the penalty, and their place in the row: one more contributor per tail warp to the
                // row's maximum and sum, and the tokens that can be among the K best go to the log.
                const uint4 z = make_uint4(0, 0, 0, 0);
                for (int i = g.tid; i < kPenSlots / 4; i += P_TT) reinterpret_cast<uint4*>(pslots)[i] = z;
                g.sync();
                {
                    const int32_t* h = P.hist + size_t(row) * P.hist_stride;
                    int hl = P.hist_len[row];
                    hl = int64_t(hl) > P.hist_stride ? int(P.hist_stride) : hl;
                    hl = hl > kMaxHist ? kMaxHist : hl;
                    int32_t hv[kMaxHist / P_TT];
#pragma unroll
                    for (int u = 0; u < kMaxHist / P_TT; ++u) hv[u] = (g.tid + u * P_TT) < hl ? h[g.tid + u * P_TT] : -1;
#pragma unroll
                    for (int u = 0; u < kMaxHist / P_TT; ++u) {
                        const uint32_t t = uint32_t(hv[u]);
                        if (t >= n) continue;  // (negative ids too)
                        const uint32_t tag = t + 1;
                        uint32_t hsh = PenaltyTable::hash(t);
                        for (int probe = 0; probe < kPenSlots; ++probe) {
                            uint32_t old = ldv_u32(&pslots[hsh]);
                            if (old == 0) old = atomicCAS(&pslots[hsh], 0u, tag | (1u << kPenIdBits));
                            if (old == 0) break;
                            if ((old & kPenMaxV) == tag) {
                                atomicAdd(&pslots[hsh], 1u << kPenIdBits);
                                break;
                            }
                            hsh = (hsh + 1) & (kPenSlots - 1);
                        }
                    }
                }
                g.sync();
                if (kn < my_rows) maybe_refine(p ^ 1, K_next);
                const float pen_rep = P.rep ? P.rep[row] : 1.f, pen_pres = P.pres ? P.pres[row] : 0.f, pen_freq = P.freq ? P.freq[row] : 0.f;
                const T* xr = reinterpret_cast<const T*>(a.x) + size_t(row) * n;
                const float cexp = inv_t * kLog2e;
                float m_t = -INFINITY, e_t = 0.f, s_t = 0.f;
                const unsigned long long tau = ldv_u64(&sl->tau);
                const float tau_f = cand_key(tau) ? float_of_key(cand_key(tau)) : -INFINITY;
                for (int base = 0; base < kPenSlots; base += 4 * P_TT) {
                    const uint4 q = reinterpret_cast<const uint4*>(pslots + base)[g.tid];
                    const uint32_t e4[4] = {q.x, q.y, q.z, q.w};
                    float r4[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {  // (the loads first, then the arithmetic)
                        const uint32_t id = (e4[j] & kPenMaxV) - 1;
                        r4[j] = 0.f;
                        if (e4[j]) r4[j] = sizeof(T) == 4 ? __ldg(reinterpret_cast<const float*>(xr) + id) : bf16_to_f32(__ldg(reinterpret_cast<const uint16_t*>(xr) + id));
                    }
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        if (!e4[j]) continue;
                        const uint32_t id = (e4[j] & kPenMaxV) - 1;
                        float l = r4[j];
                        l = (l > 0.f) ? __fdiv_rn(l, pen_rep) : __fmul_rn(l, pen_rep);
                        const float x = __fsub_rn(l, __fadd_rn(pen_pres, __fmul_rn(pen_freq, float(e4[j] >> kPenIdBits))));
                        if (!no_sum) {
                            if (x > m_t) {
                                const float ne = ceilf(x * cexp);
                                s_t = (m_t == -INFINITY) ? 0.f : s_t * ex2_approx(e_t - ne);
                                e_t = ne, m_t = x;
                            }
                            if (m_t != -INFINITY) s_t += ex2_approx(fmaf(x, cexp, -e_t));
                        }
                        if (x >= tau_f) {
                            const unsigned long long cnd = make_cand(key_of(x), id);
                            if (cnd > tau) {
                                const uint32_t pos = atomicAdd(&sl->cnt, 1u) & 0x7fffffffu;
                                if (pos < uint32_t(P_L)) log[pos] = cnd;
                            }
                        }
                    }
                }
                const bool saw_nan = !no_sum && (s_t != s_t);
                if (__any_sync(0xffffffffu, saw_nan) && lane == 0) atomicOr(&sl->cnt, 0x80000000u);
                const float wm = warp_max(m_t);
                float we = e_t;
                if (m_t == -INFINITY) we = -INFINITY;
                we = warp_max(we);
                double ds = (m_t == -INFINITY) ? 0.0 : double(s_t) * double(ex2_approx(e_t - we));
                ds = warp_sum(ds);
                if (lane == 0) sl->red_m[P_SW + tw] = wm, sl->red_e[P_SW + tw] = we, sl->red_s[P_SW + tw] = ds;
                g.sync();
            }
            const uint32_t total_raw = sl->cnt;  // bit 31: a NaN logit met a sum
            const bool nan_row = (total_raw & 0x80000000u) != 0;
            const uint32_t total = total_raw & 0x7fffffffu;
            const bool overflow = total > uint32_t(P_L) || nan_row;
            const uint32_t nlog = total > uint32_t(P_L) ? uint32_t(P_L) : total;
            // row max and normaliser: combine the warps' partials, one per lane (not needed when the row is normalised
            // over its candidates)
            float M = -INFINITY, sum = 0.f;
            if (!no_sum) {
                const int n_red = P_SW + (pen_on ? P_TW : 0);
                static_assert(P_RED <= 32, "one partial per lane");
                const float mw = lane < n_red ? sl->red_m[lane] : -INFINITY;
                M = warp_max(mw);
                const double cexp = double(inv_t * kLog2e);
                const double term = (lane < n_red && mw != -INFINITY) ? sl->red_s[lane] * exp2(double(sl->red_e[lane]) - double(M) * cexp) : 0.0;
                sum = float(warp_sum(term));
            }
            uint32_t kept = 0;
            bool presorted = false;
            if (!overflow) {
                // Most of the log was appended under an earlier, looser threshold: only entries at or above the current one
                // can be among the K best (at least K of them are).  Few survive, so rank them against each other: the
                // rank is the position in the sorted order.
                unsigned long long* list = reinterpret_cast<unsigned long long*>(hist);  // up to SEL_BINS / 2 entries
                write_survivors<P_TT>(g, log, nlog, sl->tau, list, SEL_BINS / 2, &sh->sel);
                const uint32_t m = sh->sel.wcnt;
                if (m <= 2u * P_TT) {
                    for (uint32_t t = g.tid; t < m; t += P_TT) {
                        const unsigned long long mine = list[t];
                        uint32_t rank = 0;
                        for (uint32_t j = 0; j < m; ++j) rank += list[j] > mine;
                        if (rank < K) hand[rank] = mine;
                    }
                    kept = m < K ? m : K;
                    presorted = true;
                } else if (nlog > K) {
                    const unsigned long long kth = select_kth<P_TT>(g, log, nlog, K, hist, &sh->sel);
                    write_survivors<P_TT>(g, log, nlog, kth, hand, uint32_t(max_k), &sh->sel);
                    kept = sh->sel.wcnt < uint32_t(max_k) ? sh->sel.wcnt : uint32_t(max_k);
                } else {
                    for (uint32_t i = g.tid; i < nlog; i += P_TT) hand[i] = log[i];
                    kept = nlog;
                }
            }
            uint32_t cap = 1;
            while (cap < kept) cap <<= 1;
            g.sync();
            for (uint32_t i = kept + g.tid; i < cap; i += P_TT) hand[i] = 0ull;
            // the log is free for row k + 2 once it is zero again
            for (uint32_t i = g.tid; i < nlog; i += P_TT) log[i] = 0ull;
            g.sync();
            if (kn < my_rows) maybe_refine(p ^ 1, K_next);
            if (overflow) {
                // more candidates than the log holds (rows in adversarial order), or a NaN in a sum: the multi-pass kernel
                // takes the row
                if (g.tid == 0) a.out.status[row] = ROW_RETRY;
            } else if (!sample) {
                if (g.tid == 0) a.out.status[row] = ROW_DONE;
                if (!presorted) sort_desc<P_TT>(g, reinterpret_cast<uint64_t*>(hand), cap);
                const T* xr = reinterpret_cast<const T*>(a.x) + size_t(row) * n;
                for (uint32_t j = g.tid; j < kept; j += P_TT) {
                    const uint32_t id = cand_id(hand[j]);
                    a.ids[size_t(row) * a.K + j] = int32_t(id) + a.id_offset;
                    a.vals[size_t(row) * a.K + j] = sizeof(T) == 4 ? reinterpret_cast<const float*>(xr)[id] : bf16_to_f32(reinterpret_cast<const uint16_t*>(xr)[id]);
                }
                if (g.tid == 0) a.stats[2 * row] = M, a.stats[2 * row + 1] = sum;
            } else if (greedy) {
                if (g.tid == 0) {
                    const uint32_t tok = kept ? cand_id(hand[0]) : 0;
                    a.out.token[row] = int32_t(tok);
                    a.out.status[row] = ROW_DONE;
                    if (a.out.n_kept) a.out.n_kept[row] = 1;
                    if (a.out.closed) a.out.closed[row] = 1;
                    if (a.out.stats) a.out.stats[2 * row] = kept ? float_of_key(cand_key(hand[0])) : -INFINITY, a.out.stats[2 * row + 1] = 0.f;
                    if (a.out.kept_ids && a.out.kept_cap > 0) a.out.kept_ids[size_t(row) * a.out.kept_cap] = int32_t(tok);
                    if (a.out.kept_p && a.out.kept_cap > 0) a.out.kept_p[size_t(row) * a.out.kept_cap] = 1.0;
                }
            } else {
                // probabilities, the top-k / top-p / min-p cuts, the draw and the row's outputs
                TailIn in;
                in.inv_t = inv_t;
                in.top_k = P.top_k ? uint32_t(max(P.top_k[row], 0)) : 0u;
                in.top_p = P.top_p ? P.top_p[row] : 1.0, in.min_p = P.min_p ? P.min_p[row] : 0.0, in.u = P.u ? P.u[row] : 0.0;
                if (no_sum) {
                    // normalise over the candidates themselves (sorted or not, hand[] holds exactly the kept ones)
                    if (g.tid < 32) {
                        unsigned long long top = 0ull;
                        for (uint32_t i = lane; i < kept; i += 32) top = hand[i] > top ? hand[i] : top;
                        top = warp_max(uint64_t(top));
                        const float Mc = float_of_key(cand_key(top));
                        for (uint32_t i = lane; i < kept; i += 32) tail_q[i] = exp(double(__fsub_rn(float_of_key(cand_key(hand[i])), Mc)) * double(inv_t));
                        __syncwarp();
                        const float sc = float(warp_total(tail_q, kept));
                        if (lane == 0) sh->res.cum = double(sc), sh->res.token = __float_as_uint(Mc);
                    }
                    g.sync();
                    M = __uint_as_float(sh->res.token), sum = float(sh->res.cum);
                    g.sync();
                }
                in.m = M, in.sum = sum, in.cnt = kept, in.cap = cap, in.V = n;
                in.race = P.race_key != nullptr, in.race_key = P.race_key ? P.race_key[row] : 0;
                in.presorted = presorted;
                sample_tail<P_TT>(g, in, reinterpret_cast<uint64_t*>(hand), tail_p, tail_q, &sh->res);
                const TailOut r = sh->res;
                if (g.tid == 0) {
                    a.out.token[row] = int32_t(r.token);
                    a.out.status[row] = r.status;
                    if (a.out.n_kept) a.out.n_kept[row] = int32_t(r.n);
                    if (a.out.closed) a.out.closed[row] = r.closed;
                    if (a.out.stats) a.out.stats[2 * row] = M, a.out.stats[2 * row + 1] = sum;
                    if (a.out.counters && r.status == ROW_ESCALATE) atomicAdd(&a.out.counters[0], 1u);
                    if (a.out.counters && r.status == ROW_OPEN_TAIL) atomicAdd(&a.out.counters[1], 1u);
                }
                if (r.status != ROW_ESCALATE) {
                    const uint32_t nk = min(r.n, uint32_t(max(a.out.kept_cap, 0)));
                    for (uint32_t j = g.tid; j < nk; j += P_TT) {
                        if (a.out.kept_ids) a.out.kept_ids[size_t(row) * a.out.kept_cap + j] = int32_t(cand_id(hand[j]));
                        if (a.out.kept_p) a.out.kept_p[size_t(row) * a.out.kept_cap + j] = tail_p[j];
                    }
                }
                g.sync();
            }
            if (kn < my_rows) maybe_refine(p ^ 1, K_next);
            // ---- the slot goes to the row after the next
            if (kn2 < my_rows) boot(kn2, ord + 2);
            k = kn;
        }
        // Every row of this CTA has its status.
        if (a.fin_list) {
            __threadfence();
            g.sync();
            if (g.tid < 32) list_leftovers(a);
        }
        return;
    }

    // =========================================================== stream warps
    const int lane = lane_id(), sw = tid >> 5;
    const uint4 ninf4 = sizeof(T) == 4 ? make_uint4(0xff800000u, 0xff800000u, 0xff800000u, 0xff800000u)
                                       : make_uint4(0xff80ff80u, 0xff80ff80u, 0xff80ff80u, 0xff80ff80u);
    // ---- the load cursor runs P_PF tiles ahead of the tile being worked on, across row boundaries
    int k_ld = next_row(-1);
    uint32_t t_ld = 0;
    const uint4* row_ld = reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(a.x) + size_t(row_of(k_ld)) * n);
    auto load_tile = [&](uint4(&b)[4]) {
        if (k_ld >= my_rows) return;
        const uint32_t q0 = t_ld * TILE_Q + uint32_t(tid);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t qi = q0 + uint32_t(j) * P_ST;
            b[j] = qi < row_q ? ld_stream(row_ld + qi) : ninf4;
        }
        if (++t_ld == n_tiles) {
            t_ld = 0;
            k_ld = next_row(k_ld);
            if (k_ld < my_rows) row_ld = reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(a.x) + size_t(row_of(k_ld)) * n);
        }
    };
    uint4 buf[P_PF][4];
#pragma unroll
    for (int j = 0; j < P_PF; ++j) load_tile(buf[j]);

    // ---- row state
    int k = next_row(-1), ord = 0;
    uint32_t t = 0;
    bool fail = false;
    PSlot* sl = nullptr;
    unsigned long long* log = nullptr;
    const uint32_t* bm = nullptr;
    bool no_sum = false, pen_on = false, renew_ok = false;
    float cexp = 0.f, m_t = -INFINITY, e_t = 0.f, s_t = 0.f, tau_f = -INFINITY;
    unsigned long long tau_seen = 0ull;
    uint32_t rth = 1, next_renew = 1;

    auto row_begin = [&]() {
        const int p = ord & 1;
        const int row = row_of(k);
        sl = &sh->slot[p];
        log = logs + size_t(p) * P_L;
        bm = bitmaps + size_t(p) * bm_words;
        // the slot (log, threshold, bit map) is this row's once the tail group says so
        if (!mbar_wait(&boot_done[p], (ord >> 1) & 1)) {
            if (lane == 0) atomicExch(a.err, 4u);
            fail = true;
            return;
        }
        no_sum = no_sum_row(row);
        pen_on = pen_row(row);
        const float inv_t = P.inv_t ? P.inv_t[row] : P.inv_t_scalar;
        cexp = inv_t * kLog2e;
        m_t = -INFINITY, e_t = 0.f, s_t = 0.f;
        tau_seen = 0ull, tau_f = -INFINITY;
        rth = (k_of(row) + P_SW - 1) / P_SW;
        // a warp's own bound from its lane maxima is valid only when those hold no raw logit of a history token
        renew_ok = rth <= 32 && (!pen_on || !no_sum);
        next_renew = 1;
    };

    auto process = [&](const uint4(&cur)[4]) {
        {
            const unsigned long long tq = ldv_u64(&sl->tau);
            if (tq > tau_seen) tau_seen = tq, tau_f = float_of_key(cand_key(tq));
        }
        const unsigned long long tau = tau_seen;
        float xv[4 * VE];
        uint32_t qid[4];  // first token id of each 128-bit word
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            qid[j] = (t * TILE_Q + uint32_t(tid) + uint32_t(j) * P_ST) * VE;
            const uint32_t w4[4] = {cur[j].x, cur[j].y, cur[j].z, cur[j].w};
            float* x = xv + j * VE;
            if (sizeof(T) == 4) {
#pragma unroll
                for (int e = 0; e < 4; ++e) x[e] = __uint_as_float(w4[e]);
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e) x[2 * e] = __uint_as_float(w4[e] << 16), x[2 * e + 1] = __uint_as_float(w4[e] & 0xffff0000u);
            }
        }
        if (pen_on && !no_sum) {
            // the normaliser must not see the raw logits of history tokens: take them out of every word
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (qid[j] < n) {
                    const uint32_t bits = (bm[qid[j] >> 5] >> (qid[j] & 31)) & ((1u << VE) - 1);
                    if (bits) {
#pragma unroll
                        for (int e = 0; e < VE; ++e)
                            if ((bits >> e) & 1u) xv[j * VE + e] = -INFINITY;
                    }
                }
            }
        }
        // maxima of the words; fmaxf skips NaN, so a NaN logit never raises a maximum
        float qm[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float mx = xv[j * VE];
#pragma unroll
            for (int e = 1; e < VE; ++e) mx = fmaxf(mx, xv[j * VE + e]);
            qm[j] = mx;
        }
        const float vm = fmaxf(fmaxf(qm[0], qm[1]), fmaxf(qm[2], qm[3]));
        if (!no_sum) {
            if (vm > m_t) {
                // new reference exponent: an integer at or above m * cexp, so every term is at most 1 and
                // x * cexp - e is one fused operation with a single rounding
                const float ne = ceilf(vm * cexp);
                s_t = (m_t == -INFINITY) ? 0.f : s_t * ex2_approx(e_t - ne);
                e_t = ne, m_t = vm;
            }
            if (m_t != -INFINITY) {
                float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int j = 0; j < 4 * VE; ++j) acc[j & 3] += ex2_approx(fmaf(xv[j], cexp, -e_t));
                s_t += (acc[0] + acc[1]) + (acc[2] + acc[3]);
            }
        } else {
            m_t = fmaxf(m_t, vm);
        }
        if (vm >= tau_f) {
            // rare: this lane holds an element that may beat the threshold
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (qm[j] >= tau_f) {
#pragma unroll
                    for (int e = 0; e < VE; ++e) {
                        const float x = xv[j * VE + e];
                        const uint32_t id = qid[j] + e;
                        if (x >= tau_f && id < n) {
                            const unsigned long long cnd = make_cand(key_of(x), id);
                            // (a row that masks its words above has no history token left here)
                            const bool hist_tok = pen_on && no_sum && ((bm[id >> 5] >> (id & 31)) & 1u);
                            if (cnd > tau && !hist_tok) {
                                const uint32_t pos = atomicAdd(&sl->cnt, 1u);
                                if (pos < uint32_t(P_L)) log[pos] = cnd;
                            }
                        }
                    }
                }
            }
        }
        // this warp's own bound, renewed each time the part of the row seen has doubled: the rth largest of its lane maxima
        // (16 * rth >= K distinct logits of the row reach the smallest of the 16 warps' bounds; the other warps' entries
        // may be older: any of their bounds for this row is valid)
        if (renew_ok && t + 1 == next_renew && t + 1 < n_tiles) {
            next_renew *= 2;
            uint32_t kv[1] = {m_t == -INFINITY ? 0u : key_of(m_t)};
            const uint32_t kr = warp_rth_largest<1>(kv, rth);
            if (lane == 0) sl->wbound[sw] = kr;
            __syncwarp();
            const uint32_t kmin = __reduce_min_sync(0xffffffffu, lane < P_SW ? ldv_u32(&sl->wbound[lane]) : 0xffffffffu);
            // (a plain compare and store: a lost update only leaves the threshold at another valid, lower bound)
            if (lane == 0) {
                const unsigned long long c = (unsigned long long)kmin << 32;
                if (c > ldv_u64(&sl->tau)) *reinterpret_cast<volatile unsigned long long*>(&sl->tau) = c;
            }
        }
    };

    auto row_end = [&]() {
        const int p = ord & 1;
        if (!no_sum) {
            // a NaN logit poisons the f32 sum: such rows are redone by the multi-pass kernel, which counts NaN as -inf
            const bool saw_nan = s_t != s_t;
            if (__any_sync(0xffffffffu, saw_nan) && lane == 0) atomicOr(&sl->cnt, 0x80000000u);
            const float wm = warp_max(m_t);
            float we = e_t;
            if (m_t == -INFINITY) we = -INFINITY;
            we = warp_max(we);
            double ds = (m_t == -INFINITY) ? 0.0 : double(s_t) * double(ex2_approx(e_t - we));
            ds = warp_sum(ds);
            if (lane == 0) sl->red_m[sw] = wm, sl->red_e[sw] = we, sl->red_s[sw] = ds;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&closed[p]);
    };

    while (k < my_rows && !fail) {
#pragma unroll
        for (int j = 0; j < P_PF; ++j) {
            if (k < my_rows && !fail) {
                uint4 cur[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) cur[q] = buf[j][q];
                load_tile(buf[j]);
                if (t == 0) row_begin();
                if (!fail) {
                    process(cur);
                    if (++t == n_tiles) {
                        row_end();
                        t = 0;
                        k = next_row(k);
                        ++ord;
                    }
                }
            }
        }
    }
}

static size_t single_pass_smem(int bm_words, int max_k, bool pen) {
    return size_t(2) * P_L * 8 + SEL_BINS * 4 + size_t(max_k) * 8 + 2 * (size_t(max_k) + 2 * P_TW) * 8 + 4 * 8 + sizeof(PShared) + 16 +
           size_t(2) * bm_words * 4 + (pen ? size_t(kPenSlots) * 4 : 0) + 128;
}

static int single_pass_bm_words(const SelectArgs& a) {
    const bool pen = a.mode == MODE_SAMPLE && a.prm.hist != nullptr;
    return pen ? ((a.n + 31) / 32 + 3) & ~3 : 0;
}

bool single_pass_supported(const SelectArgs& a, int dtype) {
    const size_t es = dtype == 0 ? 4 : 2;
    if (reinterpret_cast<uintptr_t>(a.x) % 16 != 0 || (size_t(a.n) * es) % 16 != 0) return false;  // 128-bit loads need 16-byte rows
    if (a.mode == MODE_TOPK && a.K > kSinglePassMaxK) return false;
    if (a.mode == MODE_DRAFT) return false;
    const bool pen = a.mode == MODE_SAMPLE && a.prm.hist != nullptr;
    return single_pass_smem(single_pass_bm_words(a), kSinglePassMaxK, pen) <= 232448;
}

cudaError_t single_pass_launch(const SelectArgs& a, int dtype, int sm_count, cudaStream_t st) {
    const bool pen = a.mode == MODE_SAMPLE && a.prm.hist != nullptr;
    const int bm_words = single_pass_bm_words(a);
    const int max_k = kSinglePassMaxK;
    const size_t smem = single_pass_smem(bm_words, max_k, pen);
    const int grid = a.rows < sm_count ? a.rows : sm_count;
    const cudaError_t em = cudaMemsetAsync(a.err, 0, 64, st);  // the error words, the list count and tickets, the scratch locks
    if (em != cudaSuccess) return em;
    if (dtype == 0) {
        const cudaError_t e = cudaFuncSetAttribute(single_pass_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
        if (e != cudaSuccess) return e;
        single_pass_kernel<float><<<grid, P_THREADS, smem, st>>>(a, bm_words, max_k);
    } else {
        const cudaError_t e = cudaFuncSetAttribute(single_pass_kernel<uint16_t>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
        if (e != cudaSuccess) return e;
        single_pass_kernel<uint16_t><<<grid, P_THREADS, smem, st>>>(a, bm_words, max_k);
    }
    return cudaGetLastError();
}

}  // namespace wb
