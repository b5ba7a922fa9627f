// General candidate selection: the K best of each row for any K up to 16384 and any row width / alignment, one CTA
// per row, several passes over the row (which stays in L2); and, past that, the whole row sorted.  This is the path
// for what the single-pass kernel (single_pass.cu) does not take: K above its limit (the reference's 16384-candidate
// escalation launch, src/server/engine_sampling.cpp:65-78, and its whole-row step, :79-83), rows that are not 16-byte
// aligned, rows to redo, and the id-order walk of open rows.
//
// Replaces topk_rows (kernels/shared/sample_cand_topk_rows.h:11-98) with two differences in results: ties at the K-th
// logit are broken by the lower token id (the rule of every host comparator of the path,
// src/sampling/sampler.cpp:18-21) instead of by atomic arrival order, and the candidates come out sorted
// (logit desc, id asc) instead of unordered.  The softmax normaliser is accumulated in f32 per thread against a
// running maximum and combined in f64.
#include "kernels.h"
#include "penalty.cuh"
#include "tail.cuh"

namespace wb {

constexpr int GT = 1024;      // threads per CTA
constexpr int GBINS = 2048;   // histogram bins (11-bit digits)

template <typename T>
__device__ __forceinline__ float raw_elem(const T* row, uint32_t i) {
    if (sizeof(T) == 4) return reinterpret_cast<const float*>(row)[i];
    return bf16_to_f32(reinterpret_cast<const uint16_t*>(row)[i]);
}
template <typename T>
__device__ __forceinline__ float elem(const T* row, uint32_t i, const PenaltyTable& pt) {
    float x = raw_elem(row, i);
    if (pt.on && pt.hit(i)) x = pt.apply(x, i);
    return x;
}

// BODY (a statement that reads the float V_ and the index I_) for every logit of the row that this thread owns, each
// thread's indices in ascending order.  The loads go out in batches before the first of them is used (with one load in
// flight per thread a CTA reads a row at a few GB/s): four 128-bit words per batch when the row is 16-byte aligned and a
// whole number of words long (the thread then owns words tid, tid + GT, ...), else eight single logits (tid, tid + GT, ...).
template <typename T>
__device__ __forceinline__ float word_elem(const uint4& w, int e) {
    const uint32_t u[4] = {w.x, w.y, w.z, w.w};
    if (sizeof(T) == 4) return __uint_as_float(u[e]);
    return __uint_as_float((e & 1) ? (u[e >> 1] & 0xffff0000u) : (u[e >> 1] << 16));
}
#define WB_ELEM_STEP_(PT, V_, I_, RAW, BODY)                      \
    {                                                             \
        float V_ = (RAW);                                         \
        if ((PT).on && (PT).hit(I_)) V_ = (PT).apply(V_, I_);     \
        BODY                                                      \
    }
#define WB_FOR_EACH_ELEM(TY, ROW, N, TID, PT, V_, I_, BODY)                                                        \
    do {                                                                                                           \
        constexpr uint32_t ve_ = 16 / sizeof(TY);                                                                  \
        if ((reinterpret_cast<uintptr_t>(ROW) & 15) == 0 && (N) % ve_ == 0) {                                      \
            const uint4* rq_ = reinterpret_cast<const uint4*>(ROW);                                                \
            const uint32_t nq_ = (N) / ve_;                                                                        \
            uint32_t q0_ = uint32_t(TID);                                                                          \
            _Pragma("unroll 1") for (; q0_ + 3u * GT < nq_; q0_ += 4u * GT) {                                      \
                uint4 w_[4];                                                                                       \
                _Pragma("unroll") for (int j_ = 0; j_ < 4; ++j_) w_[j_] = rq_[q0_ + uint32_t(j_) * GT];            \
                _Pragma("unroll") for (int j_ = 0; j_ < 4; ++j_) {                                                 \
                    _Pragma("unroll") for (int e_ = 0; e_ < int(ve_); ++e_) {                                      \
                        const uint32_t I_ = (q0_ + uint32_t(j_) * GT) * ve_ + uint32_t(e_);                        \
                        WB_ELEM_STEP_(PT, V_, I_, word_elem<TY>(w_[j_], e_), BODY)                                 \
                    }                                                                                              \
                }                                                                                                  \
            }                                                                                                      \
            _Pragma("unroll 1") for (; q0_ < nq_; q0_ += GT) {                                                     \
                const uint4 w1_ = rq_[q0_];                                                                        \
                _Pragma("unroll") for (int e_ = 0; e_ < int(ve_); ++e_) {                                          \
                    const uint32_t I_ = q0_ * ve_ + uint32_t(e_);                                                  \
                    WB_ELEM_STEP_(PT, V_, I_, word_elem<TY>(w1_, e_), BODY)                                        \
                }                                                                                                  \
            }                                                                                                      \
        } else {                                                                                                   \
            uint32_t i0_ = uint32_t(TID);                                                                          \
            _Pragma("unroll 1") for (; i0_ + 7u * GT < (N); i0_ += 8u * GT) {                                      \
                float raw_[8];                                                                                     \
                _Pragma("unroll") for (int j_ = 0; j_ < 8; ++j_) raw_[j_] = raw_elem((ROW), i0_ + uint32_t(j_) * GT); \
                _Pragma("unroll") for (int j_ = 0; j_ < 8; ++j_) {                                                 \
                    const uint32_t I_ = i0_ + uint32_t(j_) * GT;                                                   \
                    WB_ELEM_STEP_(PT, V_, I_, raw_[j_], BODY)                                                      \
                }                                                                                                  \
            }                                                                                                      \
            _Pragma("unroll 1") for (; i0_ < (N); i0_ += GT) {                                                     \
                const uint32_t I_ = i0_;                                                                           \
                WB_ELEM_STEP_(PT, V_, I_, raw_elem((ROW), I_), BODY)                                               \
            }                                                                                                      \
        }                                                                                                          \
    } while (0)

struct GShared {
    uint32_t prefix, remain, cnt, eq;
    float m;
    float sum;
    TailOut res;
    float red_m[32];
    double red_s[32];
    uint64_t red_c[32];
};

// One digit pass of a radix select over values v(i) of the elements that pass `keep(i)`: finds, going from the top bin
// down (DESC) or from the bottom bin up, the bin where the running count reaches sh->remain; updates prefix / remain.
// hist must be zero on entry and is zero again on exit.
template <bool DESC>
__device__ void pick_bin(uint32_t* hist, GShared* sh, int shift, int bits) {
    __syncthreads();
    if (threadIdx.x < 32) {
        const int nb = 1 << bits, per = nb / 32;
        const int l = lane_id();
        // lane l owns `per` consecutive bins, in scan order
        uint32_t s = 0;
        for (int j = 0; j < per; ++j) {
            const int b = DESC ? nb - 1 - (l * per + j) : l * per + j;
            s += hist[b];
        }
        const uint32_t incl = warp_scan_incl(s), excl = incl - s;
        const uint32_t rem = sh->remain;
        const bool mine = excl < rem && incl >= rem;
        if (mine) {
            uint32_t r = rem - excl;
            for (int j = 0; j < per; ++j) {
                const int b = DESC ? nb - 1 - (l * per + j) : l * per + j;
                const uint32_t c = hist[b];
                if (c >= r) {
                    sh->prefix |= uint32_t(b) << shift;
                    sh->remain = r;
                    sh->eq = c;
                    break;
                }
                r -= c;
            }
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < GBINS; i += GT) hist[i] = 0;
    __syncthreads();
}

template <typename T>
__device__ void full_row(const SelectArgs& a, int row, int cap_max, int pen_words, uint64_t* tile, GShared* sh, uint32_t* pen_mem,
                         uint64_t* fc, double* fp);
template <typename T>
__device__ int select_row(const SelectArgs& a, int row, int level_k, int cap_max, int pen_words, uint64_t* cand,
                          uint32_t* hist, GShared* sh, uint32_t* pen_mem);
template <typename T>
__device__ void full_row(const SelectArgs& a, int row, int cap_max, int pen_words, uint64_t* tile, GShared* sh,
                         uint32_t* pen_mem, uint64_t* fc, double* fp);

// The tail of draft_sample_rows (kernels/spec_sample.hip:132-205) on at most 32 candidates, by one warp with one
// candidate per lane: map the ids, order by (logit desc, id asc) by counting ranks, q = softmax at the request
// temperature in f32 (the operations and their order as in spec::draftDist, src/common/spec_sample.cpp:33-81: the
// sums run over the lanes in rank order, every lane adding the same broadcast terms), top-k / top-p / min-p,
// renormalise, then the race draw argmin E(id) / q in f64; writes the token to the control area and q to qbuf.
// Call with all 32 lanes of one warp.
__device__ void draft_tail(const SelectArgs& a, int row, const unsigned long long* cand, uint32_t K, float m, float sum, float inv_t) {
    constexpr uint32_t FULL = 0xffffffffu;
    const DraftArgs& d = a.draft;
    const int lane = lane_id();
    // ---- this lane's candidate
    const bool have = uint32_t(lane) < K;
    int my_id = 0x7fffffff;
    float my_lg = -INFINITY;  // (a NaN logit only fills a slot past the numbers, with p = 0)
    if (have) {
        const unsigned long long c = cand[lane];
        const uint32_t raw = cand_id(c), k = cand_key(c);
        my_id = d.map ? d.map[raw] : int(raw);
        my_lg = k ? float_of_key(k) : -INFINITY;
    }
    // ---- rank = the candidates ahead of this one; then lane r takes the candidate of rank r
    int rank = 0;
#pragma unroll 1
    for (int j = 0; j < 32; ++j) {
        const float lj = __shfl_sync(FULL, my_lg, j);
        const int ij = __shfl_sync(FULL, my_id, j);
        const bool hj = uint32_t(j) < K;
        const bool ahead = have ? (hj && (lj > my_lg || (lj == my_lg && (ij < my_id || (ij == my_id && j < lane))))) : (hj || j < lane);
        rank += ahead ? 1 : 0;
    }
    int src = 0;
#pragma unroll 1
    for (int j = 0; j < 32; ++j) src = __shfl_sync(FULL, rank, j) == lane ? j : src;
    const int id = __shfl_sync(FULL, my_id, src);
    const float lg = __shfl_sync(FULL, my_lg, src);
    float p = uint32_t(lane) < K ? __fdiv_rn(expf(__fmul_rn(__fsub_rn(lg, m), inv_t)), sum) : 0.f;
    // the sum of the first `cnt` probabilities, added in rank order
    auto serial_sum = [&](uint32_t cnt) {
        float z = 0.f;
#pragma unroll 1
        for (uint32_t i = 0; i < cnt; ++i) z = __fadd_rn(z, __shfl_sync(FULL, p, int(i)));
        return z;
    };
    // ---- the cuts
    const int tk = d.top_k[row];
    uint32_t nk = K;
    const bool closed = tk > 0 && uint32_t(tk) <= K;
    if (closed) nk = uint32_t(tk);
    const float top_p = d.top_p[row];
    if (top_p < 1.f) {
        const float z = closed ? serial_sum(nk) : 1.f;
        float cum = 0.f;
        uint32_t cut = nk;
#pragma unroll 1
        for (uint32_t j = 0; j < nk; ++j) {
            cum = __fadd_rn(cum, __fdiv_rn(__shfl_sync(FULL, p, int(j)), z));
            if (cum >= top_p) {
                cut = j + 1;
                break;
            }
        }
        nk = cut;
    }
    const float min_p = d.min_p[row];
    if (min_p > 0.f && nk > 0) {
        const float th = __fmul_rn(min_p, __shfl_sync(FULL, p, 0));
        const uint32_t ok = __ballot_sync(FULL, uint32_t(lane) < nk && p >= th);
        const uint32_t j = ok == FULL ? 32u : uint32_t(__ffs(int(~ok))) - 1u;  // the leading run of lanes at or above th
        nk = j > 1 ? j : 1;
    }
    const float z = serial_sum(nk);
    p = __fdiv_rn(p, z);
    // ---- the race: the smallest E(id) / q, the lower rank on a tie
    const unsigned long long rkey = ((unsigned long long)d.key_hi[row] << 32) | d.key_lo[row];
    double key = __longlong_as_double(0x7FF0000000000000ll);
    if (uint32_t(lane) < nk && p > 0.f) key = race_e(rkey, uint32_t(id)) / double(p);
    int pick = key < __longlong_as_double(0x7FF0000000000000ll) ? lane : 32;  // (32: this lane does not take part)
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const double ok = __shfl_xor_sync(FULL, key, o);
        const int op = __shfl_xor_sync(FULL, pick, o);
        if (op < 32 && (pick == 32 || ok < key || (ok == key && op < pick))) key = ok, pick = op;
    }
    pick = pick == 32 ? 0 : pick;
    const int tok = __shfl_sync(FULL, id, pick);
    int32_t* q = d.qbuf + d.qoff[row];
    if (lane == 0) {
        d.ctl_all[d.area[row] + 16 + d.r] = tok;
        q[0] = int32_t(nk);
    }
    if (uint32_t(lane) < nk) {
        q[1 + lane] = id;
        q[1 + 32 + lane] = __float_as_int(p);
    }
}

// grid-strided over the rows (or over the entries of row_list); one row at a time per CTA
template <typename T>
__global__ void __launch_bounds__(GT, 1) select_generic_kernel(SelectArgs a, int cap_max, int pen_words) {
    // A launch over the single-pass kernel's leftovers is made a programmatic dependent of it: its CTAs come up as that
    // kernel's CTAs leave their SMs and wait here until all of it has completed and its writes are visible (with no such
    // dependency the wait returns at once).
    asm volatile("griddepcontrol.wait;" ::: "memory");
    extern __shared__ __align__(16) uint8_t smem[];
    uint64_t* cand = reinterpret_cast<uint64_t*>(smem);
    uint32_t* hist = reinterpret_cast<uint32_t*>(smem + size_t(cap_max) * 8);
    GShared* sh = reinterpret_cast<GShared*>(hist + GBINS);
    uint32_t* pen_mem = reinterpret_cast<uint32_t*>((reinterpret_cast<uintptr_t>(sh + 1) + 15) & ~uintptr_t(15));

    const int n_rows = a.row_count ? min(*a.row_count, a.rows) : a.rows;
    if (a.row_list && n_rows == 0 && a.batch_counters && a.fin_counts) {
        // An empty list of leftover rows (the usual case after the single-pass kernel: every row has its answer, so there
        // is nothing to count either).  Only a wait that ran out without costing a row its answer is still to report.
        if (blockIdx.x == 0 && threadIdx.x == 0 && a.err && __ldcg(a.err) != 0u) atomicAdd(&a.batch_counters[WHIRL_CNT_TIMEOUT], 1u);
        return;
    }
    for (int li = blockIdx.x; li < n_rows; li += gridDim.x) {
        __syncthreads();  // the previous row's shared state is dead
        const int entry = a.row_list ? a.row_list[li] : li;
        // bit 30 of a list entry: redo the row at the first candidate level (the single-pass kernel gave it up)
        const int row = entry & 0x3fffffff;
        int level = a.level_k;
        if ((entry >> 30) & 1) {
            // (the first level as the single-pass kernel takes it: the row's own top_k when it is at most kSinglePassMaxK,
            // else kFirstLevelK candidates)
            level = min(a.level_k, kFirstLevelK);
            if (a.mode == MODE_SAMPLE && a.prm.top_k) {
                const int tk = a.prm.top_k[row];
                if (tk > kFirstLevelK && tk <= kSinglePassMaxK) level = min(a.level_k, kSinglePassMaxK);
            }
        }
        int st = select_row<T>(a, row, level, cap_max, pen_words, cand, hist, sh, pen_mem);
        if (st == ROW_ESCALATE && level < a.level_k) {
            // a row redone at the first level whose kept set may reach past it: on to this launch's level, as a row that the
            // single-pass kernel had escalated itself
            if (threadIdx.x == 0 && a.batch_counters) atomicAdd(&a.batch_counters[WHIRL_CNT_ESCALATED], 1u);
            __syncthreads();
            level = a.level_k;
            st = select_row<T>(a, row, level, cap_max, pen_words, cand, hist, sh, pen_mem);
        }
        // Third level: the kept set may reach past 16384 candidates, so the whole row is sorted (the reference's last
        // escalation step, src/server/engine_sampling.cpp:79-83, filterCands with complete = true).  That needs 16 bytes
        // per logit of global scratch: a few areas are shared by the CTAs through locks, and the wait for one is bounded
        // (a row that gets none stays reported as not answered).
        if (st == ROW_ESCALATE && level == kGenericMaxK && a.full_ws && a.mode == MODE_SAMPLE) {
            __shared__ int s_slot;
            __syncthreads();
            if (threadIdx.x == 0) {
                s_slot = -1;
                for (uint32_t spin = 0; spin < (1u << 20) && s_slot < 0; ++spin) {
                    for (int q = 0; q < a.full_slots; ++q)
                        if (atomicCAS(&a.full_locks[q], 0u, 1u) == 0u) {
                            s_slot = q;
                            break;
                        }
                    if (s_slot < 0) __nanosleep(2000);
                }
                __threadfence();
            }
            __syncthreads();
            const int slot = s_slot;
            if (slot >= 0) {
                uint64_t* fc = reinterpret_cast<uint64_t*>(static_cast<uint8_t*>(a.full_ws) + size_t(slot) * 16 * a.full_npad);
                double* fp = reinterpret_cast<double*>(fc + a.full_npad);
                full_row<T>(a, row, cap_max, pen_words, cand, sh, pen_mem, fc, fp);
                __syncthreads();
                if (threadIdx.x == 0) {
                    __threadfence();
                    atomicExch(&a.full_locks[slot], 0u);
                }
            }
        }
    }
    // the CTA that finishes last counts the rows of the whole batch that are still without an answer
    if (a.batch_counters && a.fin_counts) {
        __shared__ uint32_t s_last;
        __syncthreads();
        if (threadIdx.x == 0) {
            __threadfence();
            s_last = atomicAdd(reinterpret_cast<unsigned int*>(a.fin_counts + 3), 1u) == gridDim.x - 1 ? 1u : 0u;
        }
        __syncthreads();
        if (s_last) {
            __threadfence();
            uint32_t c = 0;
            for (int r = threadIdx.x; r < a.rows; r += blockDim.x) c += __ldcg(a.out.status + r) != ROW_DONE;
            c = warp_sum(c);
            if ((threadIdx.x & 31) == 0 && c) atomicAdd(&a.batch_counters[WHIRL_CNT_UNRESOLVED], c);
            if (threadIdx.x == 0) {
                a.fin_counts[3] = 0;
                // a bounded wait of the kernel before this one ran out (the error word says which)
                if (a.err && __ldcg(a.err) != 0u) atomicAdd(&a.batch_counters[WHIRL_CNT_TIMEOUT], 1u);
            }
        }
    }
}

// returns the row's status (ROW_DONE for the modes that have none)
template <typename T>
__device__ int select_row(const SelectArgs& a, int row, int level_k, int cap_max, int pen_words, uint64_t* cand,
                          uint32_t* hist, GShared* sh, uint32_t* pen_mem) {
    const uint32_t n = uint32_t(a.n);
    const T* x = reinterpret_cast<const T*>(a.x) + size_t(row) * n;
    const int tid = threadIdx.x;
    const bool sample = a.mode == MODE_SAMPLE;
    const bool draft = a.mode == MODE_DRAFT;
    if (draft) {
        // kernels/spec_sample.hip:42-45: rows that do not sample keep their greedy draft; a chain stopped by the p-min
        // cut-off at or before r is skipped
        if (a.draft.on[row] == 0) return ROW_DONE;
        const int32_t* c = a.draft.ctl_all + a.draft.area[row];
        if (c[49] != 0 && c[48] <= a.draft.r) return ROW_DONE;
    }
    const RowParams& P = a.prm;
    const float inv_t = draft ? a.draft.inv_t[row] : (P.inv_t ? P.inv_t[row] : P.inv_t_scalar);

    // ---- penalties table
    PenaltyTable pt;
    pt.on = false;
    if (sample && P.hist && hist_len_of(P, row) > 0) {
        pt.rep = P.rep ? P.rep[row] : 1.f, pt.pres = P.pres ? P.pres[row] : 0.f, pt.freq = P.freq ? P.freq[row] : 0.f;
        pt.on = pt.rep != 1.f || pt.pres != 0.f || pt.freq != 0.f;
    }
    if (pt.on) {
        pt.bitmap = pen_mem;
        pt.slots = pen_mem + pen_words;
        pt.clear(tid, GT, n);
        __syncthreads();
        const int32_t* h = P.hist + size_t(row) * P.hist_stride;
        const int hl = hist_len_of(P, row);
        for (int i = tid; i < hl; i += GT) pt.insert(h[i], n);
    }
    for (int i = tid; i < GBINS; i += GT) hist[i] = 0;
    if (tid == 0) sh->prefix = 0, sh->cnt = 0, sh->eq = 0;
    __syncthreads();

    // ---- greedy rows: the first maximum
    if (sample && P.greedy && P.greedy[row]) {
        uint64_t best = 0;  // composite of the best element; 0 = none
        WB_FOR_EACH_ELEM(T, x, n, tid, pt, v, i, {
            if (v == v) {
                const uint64_t c = make_cand(key_of(v), i);
                best = c > best ? c : best;
            }
        });
        best = warp_max(best);
        if (lane_id() == 0) sh->red_c[tid >> 5] = best;
        __syncthreads();
        if (tid < 32) {
            best = warp_max(sh->red_c[tid]);
            if (tid == 0) {
                const uint32_t tok = best ? cand_id(best) : 0;
                a.out.token[row] = int32_t(tok);
                a.out.status[row] = ROW_DONE;
                if (a.out.n_kept) a.out.n_kept[row] = 1;
                if (a.out.closed) a.out.closed[row] = 1;
                if (a.out.stats) a.out.stats[2 * row] = best ? float_of_key(cand_key(best)) : -INFINITY, a.out.stats[2 * row + 1] = 0.f;
                if (a.out.kept_ids && a.out.kept_cap > 0) a.out.kept_ids[size_t(row) * a.out.kept_cap] = int32_t(tok);
                if (a.out.kept_p && a.out.kept_cap > 0) a.out.kept_p[size_t(row) * a.out.kept_cap] = 1.0;
            }
        }
        return ROW_DONE;
    }

    // ---- candidates wanted for this row
    uint32_t top_k = 0, K;
    if (sample) {
        top_k = P.top_k ? uint32_t(max(P.top_k[row], 0)) : 0u;
        K = (top_k > 0 && top_k <= uint32_t(level_k)) ? top_k : uint32_t(level_k);
    } else if (draft) {
        // draftCands (include/whirl/spec_sample.h:94): min(top_k, 32), 32 when top_k is off
        const int tk = a.draft.top_k[row];
        K = (tk > 0 && tk < 32) ? uint32_t(tk) : 32u;
    } else {
        K = uint32_t(a.K);
    }
    if (K > n) K = n;

    // ---- pass 0: max and sum exp((x - max) * inv_t)
    {
        const float c = inv_t * kLog2e;
        float m = -INFINITY, s = 0.f;
        WB_FOR_EACH_ELEM(T, x, n, tid, pt, v, i, {
            if (v > m) {
                s = (m == -INFINITY) ? 0.f : s * ex2_approx((m - v) * c);
                m = v;
            }
            if (v == v && m != -INFINITY) s += ex2_approx((v - m) * c);
        });
        const float wm = warp_max(m);
        double ds = (m == -INFINITY) ? 0.0 : double(s) * double(ex2_approx((m - wm) * c));
        ds = warp_sum(ds);
        if (lane_id() == 0) sh->red_m[tid >> 5] = wm, sh->red_s[tid >> 5] = ds;
        __syncthreads();
        if (tid < 32) {
            const float pm = sh->red_m[tid];
            const float M = warp_max(pm);
            double t = (pm == -INFINITY) ? 0.0 : sh->red_s[tid] * double(ex2_approx((pm - M) * c));
            t = warp_sum(t);
            if (tid == 0) sh->m = M, sh->sum = float(t);
        }
        __syncthreads();
    }

    // ---- the K-th largest key by three digit passes (11 + 11 + 10 bits)
    if (tid == 0) sh->remain = K;
    uint32_t mask = 0;
    const int shifts[3] = {21, 10, 0}, widths[3] = {11, 11, 10};
    for (int ps = 0; ps < 3 && K > 0; ++ps) {
        const uint32_t prefix = sh->prefix;
        const uint32_t bm = (1u << widths[ps]) - 1;
        const int sh_ps = shifts[ps];
        WB_FOR_EACH_ELEM(T, x, n, tid, pt, v, i, {
            const uint32_t k = key_of(v);
            if ((k & mask) == prefix) atomicAdd(&hist[(k >> sh_ps) & bm], 1u);
        });
        pick_bin<true>(hist, sh, shifts[ps], widths[ps]);
        mask |= bm << shifts[ps];
    }
    const uint32_t thr = sh->prefix, need = sh->remain, n_eq = sh->eq;
    // ---- more ties at the K-th key than wanted: the `need` lowest ids among them, by three digit passes on the id
    uint32_t id_thr = 0xffffffffu;
    if (K > 0 && n_eq > need) {
        __syncthreads();
        if (tid == 0) sh->prefix = 0;
        __syncthreads();
        uint32_t imask = 0;
        for (int ps = 0; ps < 3; ++ps) {
            const uint32_t prefix = sh->prefix;
            const uint32_t bm = (1u << widths[ps]) - 1;
            for (uint32_t i = tid; i < n; i += GT) {
                if ((i & imask) != prefix) continue;
                if (key_of(elem(x, i, pt)) == thr) atomicAdd(&hist[(i >> shifts[ps]) & bm], 1u);
            }
            pick_bin<false>(hist, sh, shifts[ps], widths[ps]);
            imask |= bm << shifts[ps];
        }
        id_thr = sh->prefix;
    }
    // ---- collect
    uint32_t cap = 1;
    while (cap < K) cap <<= 1;
    if (K > 0) {
        WB_FOR_EACH_ELEM(T, x, n, tid, pt, v, i, {
            const uint32_t k = key_of(v);
            if (k > thr || (k == thr && i <= id_thr)) {
                const uint32_t pos = atomicAdd(&sh->cnt, 1u);
                if (pos < cap) cand[pos] = make_cand(k, i);
            }
        });
    }
    for (uint32_t i = K + tid; i < cap; i += GT) cand[i] = 0;
    __syncthreads();
    const Group<GT> g{tid, 0};
    if (draft) {
        if (tid < 32) draft_tail(a, row, reinterpret_cast<const unsigned long long*>(cand), K, sh->m, sh->sum, inv_t);
        return ROW_DONE;
    }
    if (!sample) {
        sort_desc<GT>(g, cand, cap);
        for (uint32_t j = tid; j < K; j += GT) {
            const uint32_t id = cand_id(cand[j]);
            a.ids[size_t(row) * a.K + j] = int32_t(id) + a.id_offset;
            a.vals[size_t(row) * a.K + j] = raw_elem(x, id);
        }
        if (tid == 0) {
            a.stats[2 * row] = sh->m, a.stats[2 * row + 1] = sh->sum;
            if (a.out.status) a.out.status[row] = ROW_DONE;
        }
        return ROW_DONE;
    }
    // ---- filter and draw
    TailIn in;
    in.inv_t = inv_t, in.top_k = top_k, in.top_p = P.top_p ? P.top_p[row] : 1.0, in.min_p = P.min_p ? P.min_p[row] : 0.0;
    in.u = P.u ? P.u[row] : 0.0, in.m = sh->m, in.sum = sh->sum, in.cnt = K, in.cap = cap, in.V = n;
    in.race = P.race_key != nullptr, in.race_key = P.race_key ? P.race_key[row] : 0;
    double* p = reinterpret_cast<double*>(a.ws) + size_t(blockIdx.x) * 2 * (size_t(cap_max) + 2 * GT / 32);
    double* q = p + size_t(cap_max) + 2 * GT / 32;
    // the tail's race scratch sits at p + in.cap; keep it inside this row's slice
    in.presorted = 0;
    in.want_p = a.out.kept_p != nullptr && a.out.kept_cap > 0;
    in.have_e = 0;
    sample_tail<GT>(g, in, cand, p, q, &sh->res);
    TailOut r = sh->res;
    if (r.status == ROW_OPEN_TAIL) {
        // An open set (no top-k / top-p / min-p at all) whose draw fell past its candidates: the reference walks the rest of
        // the vocabulary in id order, adding exp((x - m) * inv_t) / sum until the running sum passes u
        // (src/sampling/sampler.cpp:132-146).  Here: every thread sums a contiguous block of ids, a scan places the blocks,
        // and the thread whose block the draw falls into walks it again.
        __syncthreads();
        // GBINS slots: the candidates' ids, open addressing (0 = empty, id + 1 stored).  An open set has at most
        // kFirstLevelK candidates, so the table stays at most an eighth full; every probe sequence is bounded by the
        // table size all the same (a full table would end the insert without a slot and the lookup without a match).
        static_assert(GBINS >= 4 * kFirstLevelK && (GBINS & (GBINS - 1)) == 0, "candidate id set of the open-set walk");
        uint32_t* set = hist;
        for (uint32_t i = tid; i < r.n && i < uint32_t(GBINS / 2); i += GT) {
            const uint32_t id = cand_id(cand[i]);
            uint32_t h = (id * 2654435761u) >> 21;
            for (int probe = 0; probe < GBINS; ++probe) {
                if (atomicCAS(&set[h], 0u, id + 1) == 0u) break;
                h = (h + 1) & (GBINS - 1);
            }
        }
        __syncthreads();
        auto member = [&](uint32_t id) -> bool {
            uint32_t h = (id * 2654435761u) >> 21;
            for (int probe = 0; probe < GBINS; ++probe) {
                const uint32_t v = set[h];
                if (v == 0) return false;
                if (v == id + 1) return true;
                h = (h + 1) & (GBINS - 1);
            }
            return false;
        };
        const double it = double(inv_t), zs = double(sh->sum);
        const uint32_t S = (n + GT - 1) / GT, b0 = min(n, uint32_t(tid) * S), b1 = min(n, b0 + S);
        double loc = 0;
        int my_last = -1;
        for (uint32_t v = b0; v < b1; ++v) {
            if (member(v)) continue;
            loc += exp(double(__fsub_rn(elem(x, v, pt), sh->m)) * it) / zs;
            my_last = int(v);
        }
        double incl = loc;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const double up = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane_id() >= o) incl += up;
        }
        if (lane_id() == 31) sh->red_s[tid >> 5] = incl;
        if (tid == 0) sh->cnt = 0xffffffffu, sh->eq = 0;
        __syncthreads();
        double before = r.cum;  // the candidates' mass, already walked
        for (int w = 0; w < (tid >> 5); ++w) before += sh->red_s[w];
        const double excl = before + incl - loc;
        if (my_last >= 0) atomicMax(&sh->eq, uint32_t(my_last) + 1);
        if (excl <= in.u && excl + loc > in.u) {
            double cum = excl;
            for (uint32_t v = b0; v < b1; ++v) {
                if (member(v)) continue;
                cum += exp(double(__fsub_rn(elem(x, v, pt), sh->m)) * it) / zs;
                if (cum > in.u) {
                    atomicMin(&sh->cnt, v);
                    break;
                }
            }
        }
        __syncthreads();
        // not reached (rounding): the last id walked, or the top candidate when nothing was walked
        r.token = sh->cnt != 0xffffffffu ? sh->cnt : (sh->eq ? sh->eq - 1 : cand_id(cand[0]));
        r.status = ROW_DONE;
        __syncthreads();
        for (int i = tid; i < GBINS; i += GT) hist[i] = 0;
    }
    if (tid == 0) {
        a.out.token[row] = int32_t(r.token);
        a.out.status[row] = r.status;
        if (a.out.n_kept) a.out.n_kept[row] = int32_t(r.n);
        if (a.out.closed) a.out.closed[row] = r.closed;
        if (a.out.stats) a.out.stats[2 * row] = sh->m, a.out.stats[2 * row + 1] = sh->sum;
        if (a.out.counters && r.status == ROW_ESCALATE) atomicAdd(&a.out.counters[0], 1u);
        if (a.out.counters && sh->res.status == ROW_OPEN_TAIL) atomicAdd(&a.out.counters[1], 1u);
    }
    if (r.status != ROW_ESCALATE) {
        const uint32_t nk = min(r.n, uint32_t(max(a.out.kept_cap, 0)));
        for (uint32_t j = tid; j < nk; j += GT) {
            if (a.out.kept_ids) a.out.kept_ids[size_t(row) * a.out.kept_cap + j] = int32_t(cand_id(cand[j]));
            if (a.out.kept_p) a.out.kept_p[size_t(row) * a.out.kept_cap + j] = p[j];
        }
    }
    return int(r.status);
}

// ---- third level: the whole row ---------------------------------------------------------------------------------
// fc[0 .. npad): every logit of the row as a candidate (penalties applied; NaN ranks below everything and gets p = 0),
// padded with zeros to a power of two and sorted (logit desc, id asc) by a bitonic network: exchanges at a distance of a
// tile or more run on global memory (L2), the rest on one tile at a time in shared memory.  fp[i]: the probability of
// fc[i].  Then the steps of filterCands with complete = true (src/sampling/sampler.cpp:15-78: exact maximum, fp64
// normaliser cast to fp32, top-k, top-p against the kept mass, min-p, renormalise; the set is closed) and the draw
// (sampleRow :118-131 / sampleRace :94-106).  Sums that the host accumulates one by one are accumulated here per thread
// over a contiguous run and combined in order, so they differ from the host's in the last bits only.
__device__ __forceinline__ void cmp_swap_desc(uint64_t& lo, uint64_t& hi, bool up) {
    // `up` half of the network keeps the larger element first (the final order is descending)
    if (up ? lo < hi : lo > hi) {
        const uint64_t t = lo;
        lo = hi, hi = t;
    }
}

// sum of v[i] / z over i < count (combined in index order); every thread returns the total
__device__ double block_sum_over(const double* v, uint32_t count, double z, GShared* sh) {
    const int tid = threadIdx.x;
    const uint32_t S = (count + GT - 1) / GT, b0 = min(count, uint32_t(tid) * S), b1 = min(count, b0 + S);
    double loc = 0;
    for (uint32_t i = b0; i < b1; ++i) loc += v[i] / z;
    double incl = loc;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const double up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane_id() >= o) incl += up;
    }
    __syncthreads();
    if (lane_id() == 31) sh->red_s[tid >> 5] = incl;
    __syncthreads();
    double tot = 0;
    for (int w = 0; w < GT / 32; ++w) tot += sh->red_s[w];
    return tot;
}

// smallest j < count with cum_j >= t (STRICT: > t), cum_j = sum of v[i] / z over i <= j; count when there is none
template <bool STRICT>
__device__ uint32_t block_first_reach(const double* v, uint32_t count, double z, double t, GShared* sh) {
    const int tid = threadIdx.x;
    const uint32_t S = (count + GT - 1) / GT, b0 = min(count, uint32_t(tid) * S), b1 = min(count, b0 + S);
    double loc = 0;
    for (uint32_t i = b0; i < b1; ++i) loc += v[i] / z;
    double incl = loc;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const double up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane_id() >= o) incl += up;
    }
    __syncthreads();
    if (lane_id() == 31) sh->red_s[tid >> 5] = incl;
    if (tid == 0) sh->cnt = count;
    __syncthreads();
    double cum = incl - loc;
    for (int w = 0; w < (tid >> 5); ++w) cum += sh->red_s[w];
    for (uint32_t i = b0; i < b1; ++i) {
        cum += v[i] / z;
        if (STRICT ? cum > t : cum >= t) {
            atomicMin(&sh->cnt, i);
            break;
        }
    }
    __syncthreads();
    const uint32_t r = sh->cnt;
    __syncthreads();
    return r;
}

template <typename T>
__device__ void full_row(const SelectArgs& a, int row, int cap_max, int pen_words, uint64_t* tile, GShared* sh, uint32_t* pen_mem,
                         uint64_t* fc, double* fp) {
    const uint32_t n = uint32_t(a.n), npad = a.full_npad;
    const T* x = reinterpret_cast<const T*>(a.x) + size_t(row) * n;
    const int tid = threadIdx.x;
    const RowParams& P = a.prm;
    const float inv_t = P.inv_t ? P.inv_t[row] : P.inv_t_scalar;
    // the penalty table built for the row by select_row is still in shared memory
    PenaltyTable pt;
    pt.on = false;
    if (P.hist && hist_len_of(P, row) > 0) {
        pt.rep = P.rep ? P.rep[row] : 1.f, pt.pres = P.pres ? P.pres[row] : 0.f, pt.freq = P.freq ? P.freq[row] : 0.f;
        pt.on = pt.rep != 1.f || pt.pres != 0.f || pt.freq != 0.f;
    }
    pt.bitmap = pen_mem, pt.slots = pen_mem + pen_words;

    for (uint32_t i = tid; i < npad; i += GT) fc[i] = i < n ? make_cand(key_of(elem(x, i, pt)), i) : 0ull;
    __syncthreads();
    // ---- sort
    const uint32_t TS = uint32_t(cap_max) < npad ? uint32_t(cap_max) : npad;  // tile (a power of two, as npad is)
    // all exchanges of the stages k_lo .. k_hi at distances below the tile size, tile by tile
    auto tiles = [&](uint32_t k_lo, uint32_t k_hi) {
        for (uint32_t base = 0; base < npad; base += TS) {
            for (uint32_t i = tid; i < TS; i += GT) tile[i] = fc[base + i];
            __syncthreads();
            for (uint32_t k = k_lo; k <= k_hi; k <<= 1) {
                for (uint32_t j = min(k >> 1, TS >> 1); j > 0; j >>= 1) {
                    for (uint32_t q = tid; q < TS / 2; q += GT) {
                        const uint32_t t = ((q & ~(j - 1)) << 1) | (q & (j - 1));
                        cmp_swap_desc(tile[t], tile[t | j], ((base + t) & k) == 0);
                    }
                    __syncthreads();
                }
            }
            for (uint32_t i = tid; i < TS; i += GT) fc[base + i] = tile[i];
            __syncthreads();
        }
    };
    tiles(2, TS);
    for (uint32_t k = TS << 1; k <= npad && k != 0; k <<= 1) {
        for (uint32_t j = k >> 1; j >= TS; j >>= 1) {
            for (uint32_t q = tid; q < npad / 2; q += GT) {
                const uint32_t t = ((q & ~(j - 1)) << 1) | (q & (j - 1));
                uint64_t lo = fc[t], hi = fc[t | j];
                const uint64_t lo0 = lo;
                cmp_swap_desc(lo, hi, (t & k) == 0);
                if (lo != lo0) fc[t] = lo, fc[t | j] = hi;
            }
            __syncthreads();
        }
        tiles(k, k);
    }
    // ---- probabilities (sampler.cpp:23-34 with complete = true)
    const float m = float_of_key(cand_key(fc[0]));
    const double it = double(inv_t);
    for (uint32_t i = tid; i < n; i += GT) {
        const uint32_t key = cand_key(fc[i]);
        fp[i] = key ? exp(double(__fsub_rn(float_of_key(key), m)) * it) : 0.0;
    }
    __syncthreads();
    const float sum = float(block_sum_over(fp, n, 1.0, sh));
    for (uint32_t i = tid; i < n; i += GT) fp[i] = fp[i] / double(sum);
    __syncthreads();
    // ---- top-k, top-p, min-p, renormalise (the set is closed from the start: every logit is a candidate)
    const uint32_t top_k = P.top_k ? uint32_t(max(P.top_k[row], 0)) : 0u;
    const double top_p = P.top_p ? P.top_p[row] : 1.0, min_p = P.min_p ? P.min_p[row] : 0.0, u = P.u ? P.u[row] : 0.0;
    uint32_t nk = n;
    if (top_k > 0 && top_k <= n) nk = top_k;
    if (top_p < 1.0) {
        const double z = block_sum_over(fp, nk, 1.0, sh);
        const uint32_t j = block_first_reach<false>(fp, nk, z, top_p, sh);
        if (j < nk) nk = j + 1;
    }
    if (min_p > 0) {
        const double thr = min_p * fp[0];
        if (tid == 0) sh->cnt = nk;
        __syncthreads();
        for (uint32_t i = tid; i < nk; i += GT)
            if (!(fp[i] >= thr)) {
                atomicMin(&sh->cnt, i);
                break;  // (later ones of this thread are larger indices)
            }
        __syncthreads();
        const uint32_t j = sh->cnt;
        __syncthreads();
        nk = j > 1 ? j : 1;
    }
    {
        const double z = block_sum_over(fp, nk, 1.0, sh);
        for (uint32_t i = tid; i < nk; i += GT) fp[i] = fp[i] / z;
        __syncthreads();
    }
    // ---- the draw
    uint32_t token;
    if (P.race_key != nullptr) {
        // argmin over the kept candidates of E(id) / p, the first on ties
        const uint64_t rk = P.race_key[row];
        double bk = __longlong_as_double(0x7FF0000000000000ll);
        uint32_t bi = 0xffffffffu;
        for (uint32_t i = tid; i < nk; i += GT) {
            if (!(fp[i] > 0)) continue;
            const double kk = race_e(rk, cand_id(fc[i])) / fp[i];
            if (kk < bk) bk = kk, bi = i;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const double ok = __shfl_xor_sync(0xffffffffu, bk, o);
            const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ok < bk || (ok == bk && oi < bi)) bk = ok, bi = oi;
        }
        __syncthreads();
        if (lane_id() == 0) sh->red_s[tid >> 5] = bk, sh->red_c[tid >> 5] = bi;
        __syncthreads();
        for (int w = 0; w < GT / 32; ++w) {
            const double ok = sh->red_s[w];
            const uint32_t oi = uint32_t(sh->red_c[w]);
            if (w == 0 || ok < bk || (ok == bk && oi < bi)) bk = ok, bi = oi;
        }
        token = cand_id(fc[bi == 0xffffffffu ? 0 : bi]);
        __syncthreads();
    } else {
        const uint32_t j = block_first_reach<true>(fp, nk, 1.0, u, sh);
        token = cand_id(fc[j < nk ? j : nk - 1]);  // not reached (rounding): the last kept candidate
    }
    if (tid == 0) {
        a.out.token[row] = int32_t(token);
        a.out.status[row] = ROW_DONE;
        if (a.out.n_kept) a.out.n_kept[row] = int32_t(nk);
        if (a.out.closed) a.out.closed[row] = 1;
        if (a.out.stats) a.out.stats[2 * row] = m, a.out.stats[2 * row + 1] = sum;
    }
    const uint32_t ncap = min(nk, uint32_t(max(a.out.kept_cap, 0)));
    for (uint32_t j = tid; j < ncap; j += GT) {
        if (a.out.kept_ids) a.out.kept_ids[size_t(row) * a.out.kept_cap + j] = int32_t(cand_id(fc[j]));
        if (a.out.kept_p) a.out.kept_p[size_t(row) * a.out.kept_cap + j] = fp[j];
    }
    __syncthreads();
}

uint32_t select_full_npad(int n) {
    uint32_t p = 1;
    while (p < uint32_t(n)) p <<= 1;
    return p;
}
size_t select_full_ws_bytes(int n) {
    if (n <= 0 || n > (1 << 20)) return 0;
    return size_t(kFullSlots) * 16 * select_full_npad(n);
}

static int pow2_at_least(int k) {
    int c = 1;
    while (c < k) c <<= 1;
    return c;
}

size_t select_generic_ws_bytes(int ctas, int K) {
    return size_t(ctas) * 2 * (size_t(pow2_at_least(K < 1 ? 1 : K)) + 2 * GT / 32) * sizeof(double);
}

cudaError_t select_generic_launch(const SelectArgs& a, int dtype, int sm_count, cudaStream_t st) {
    // (a launch over a list of leftover rows, usually empty or short, gets one CTA per SM: its CTAs loop over the list)
    const int per_sm = a.row_list ? 1 : 2;
    const int grid = a.rows < per_sm * sm_count ? a.rows : per_sm * sm_count;
    const int kmax = a.mode == MODE_TOPK ? a.K : (a.mode == MODE_DRAFT ? 32 : a.level_k);
    const int cap = pow2_at_least(kmax < 1 ? 1 : (kmax > a.n ? a.n : kmax));
    const bool pen = a.mode == MODE_SAMPLE && a.prm.hist != nullptr;
    const int pen_words = pen ? ((a.n + 31) / 32 + 3) & ~3 : 0;
    const size_t smem = size_t(cap) * 8 + GBINS * 4 + sizeof(GShared) + (pen ? size_t(pen_words) * 4 + kPenSlots * 4 : 0) + 48;
    // (over a list of leftovers the launch may overlap the end of the kernel before it in the stream: see the kernel's top)
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(unsigned(grid)), cfg.blockDim = dim3(GT), cfg.dynamicSmemBytes = smem, cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr, cfg.numAttrs = a.row_list ? 1 : 0;
    cudaError_t e;
    if (dtype == 0) {
        e = cudaFuncSetAttribute(select_generic_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
        if (e != cudaSuccess) return e;
        e = cudaLaunchKernelEx(&cfg, select_generic_kernel<float>, a, cap, pen_words);
    } else {
        e = cudaFuncSetAttribute(select_generic_kernel<uint16_t>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
        if (e != cudaSuccess) return e;
        e = cudaLaunchKernelEx(&cfg, select_generic_kernel<uint16_t>, a, cap, pen_words);
    }
    if (e != cudaSuccess) return e;
    return cudaGetLastError();
}

}  // namespace wb
