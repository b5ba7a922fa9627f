// The single-pass fused sampler for rows that keep at most 256 candidates: every logits row is read from HBM once.
//
// One persistent CTA per SM, 25 warps in five roles that never meet at a CTA-wide barrier while rows stream:
//   producer (1 thread)     bulk async copies (TMA, cp.async.bulk + mbarrier) of the CTA's rows into a ring of shared
//                           memory stages, running ahead across row boundaries.  The first few stages of a row go
//                           through the ring twice (the second time they come from L2).
//   stream (16 warps)       consume the stages: running max / sum exp for the softmax normaliser and a threshold test;
//                           the few logits above the threshold are appended to the row's candidate log.  The first
//                           pass over a row's head only accumulates; then the warps agree on a first threshold (their
//                           one meeting per row); the second pass over the head only logs.
//   penalty warps (3)       only when histories are given: take the raw logits of a stage's history tokens out before
//                           the stream warps read it (lists prepared by history_lists_kernel) and put them aside.
//   tail group (4 warps)    concurrently: raise the row's threshold (the K-th largest of the log so far is a valid
//                           lower bound of the row's K-th largest); when a row is through: apply the penalties to the
//                           tokens put aside and add them to the row, then its exact K best, in order.
//   draw warp (1)           with the row's candidates from the tail group: top-k / top-p / min-p in f64, the draw, the
//                           outputs, while the tail group is already on the next row.
//
// Why a threshold from partial data is exact: an element is dropped only when it is below a value that at least K
// elements of the same row reach, so the K best are always in the log; the final select over the log is exact.
//
// It replaces the reference's topk_rows kernel (seven passes over the row, kernels/shared/sample_cand_topk_rows.h:11-98),
// the candidate download, and the host filter and draw (src/sampling/sampler.cpp:15-147).
#include <type_traits>

#include "kernels.h"
#include "penalty.cuh"
#include "select_smem.cuh"
#include "tail.cuh"

namespace wb {

constexpr int A_SW = 16;                      // stream warps
constexpr int A_ST = A_SW * 32;
constexpr int A_TW = 4;                       // tail warps
constexpr int A_TT = A_TW * 32;
constexpr int A_PW = 3;                       // penalty warps (with them 25 warps: at most seven per scheduler, 72 registers
                                              // each, which the kernel fits without spilling; two were 7 % slower with penalties)
constexpr int A_THREADS = 32 + A_ST + A_TT + 32 + A_PW * 32;  // copies, stream warps, tail warps, draw warp, penalty warps
constexpr int A_CH = 4096;                    // logits per ring stage
constexpr int A_L = 3040;                     // candidate log entries per row slot (sized so that a 10th ring stage fits)
constexpr int A_MAXSTAGES = 16;
constexpr int A_S0 = 8;                       // stages at the head of a row that are read twice (see the stream warps)

struct ASlot {
    unsigned long long tau;  // current threshold candidate; elements must beat it to be logged
    uint32_t cnt;            // log entries reserved so far (may exceed A_L: overflow)
    int32_t row;
    float red_m[A_SW + A_TW];  // per stream warp, then per tail warp (the row's history tokens): max, reference exponent, scaled sum
    float red_e[A_SW + A_TW];
    double red_s[A_SW + A_TW];
};

// what the tail group hands to the draw warp with a row's candidates
struct DrawIn {
    int32_t row;
    uint32_t kept, cap;  // candidates, and the power of two they are padded to
    float M, sum;        // row maximum and normaliser (unused when the row is normalised over its candidates)
    uint32_t presorted;
    uint32_t skip;       // nothing to draw (the tail group finished the row itself)
};

struct AShared {
    ASlot slot[2];
    DrawIn draw[2];
    SelScratch sel;
    TailOut res;
    uint32_t flag[4];
    uint32_t pbnd[A_PW][136];  // per penalty warp: the places of the current row's stages in its hit list
};

__device__ __forceinline__ unsigned long long ld_volatile_u64(const unsigned long long* p) {
    return *reinterpret_cast<const volatile unsigned long long*>(p);
}
__device__ __forceinline__ uint32_t ld_volatile_u32(const uint32_t* p) { return *reinterpret_cast<const volatile uint32_t*>(p); }

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

template <typename T>
__global__ void __launch_bounds__(A_THREADS, 1) sample_async_kernel(SelectArgs a, int stages, int pen, int ch_bytes) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* ring = smem;                                                          // stages * ch_bytes
    unsigned long long* logs = reinterpret_cast<unsigned long long*>(ring + size_t(stages) * ch_bytes);  // 2 * A_L
    uint32_t* hist = reinterpret_cast<uint32_t*>(logs + 2 * A_L);                 // SEL_BINS
    unsigned long long* hand = reinterpret_cast<unsigned long long*>(hist + SEL_BINS);   // 2 * kAsyncMaxK: a row's candidates, per slot
    double* tail_p = reinterpret_cast<double*>(hand + 2 * kAsyncMaxK);                 // 2 * (kAsyncMaxK + 2 * A_TW)
    double* tail_q = tail_p + kAsyncMaxK + 2 * A_TW;
    uint64_t* bars = reinterpret_cast<uint64_t*>(tail_q + kAsyncMaxK + 2 * A_TW);  // 3 * A_MAXSTAGES + 14
    AShared* sh = reinterpret_cast<AShared*>(bars + 3 * A_MAXSTAGES + 14);
    uint32_t* wbound = reinterpret_cast<uint32_t*>((reinterpret_cast<uintptr_t>(sh + 1) + 15) & ~uintptr_t(15));  // 2 * A_SW: per slot, each stream warp's bound key
    uint64_t *full = bars, *empty = bars + A_MAXSTAGES, *patched = bars + 2 * A_MAXSTAGES;
    uint64_t *closed = bars + 3 * A_MAXSTAGES, *boot_done = closed + 2, *head_done = closed + 4;  // per slot: the slot is the row's / every stream warp has named its bound
    uint64_t *draw_full = closed + 6, *draw_empty = closed + 8, *hv_ready = closed + 10;  // per slot: the candidates are there / the draw warp is done with them

    const int tid = threadIdx.x, warp = tid >> 5;
    const uint32_t n = uint32_t(a.n);
    const int n_rows = a.row_count ? min(*a.row_count, a.rows) : a.rows;
    const int my_rows = n_rows > int(blockIdx.x) ? (n_rows - int(blockIdx.x) + int(gridDim.x) - 1) / int(gridDim.x) : 0;
    const uint32_t n_chunks = (n + A_CH - 1) / A_CH;
    // A row goes through the ring as: its first s0 stages, those s0 stages once more, then the rest (see the stream warps).
    const uint32_t s0 = n_chunks < uint32_t(A_S0) ? n_chunks : uint32_t(A_S0), n_seq = n_chunks + s0;
    auto seq_stage = [&](uint32_t i) -> uint32_t { return i < s0 ? i : i - s0; };
    const size_t row_bytes = size_t(n) * sizeof(T);
    auto row_of = [&](int k) -> int {
        const int li = int(blockIdx.x) + k * int(gridDim.x);
        return a.row_list ? a.row_list[li] : li;
    };
    // rows whose top_k is above this kernel's limit are left to the large-K kernel (every role skips them alike)
    auto is_large = [&](int row) -> bool {
        if (a.mode != MODE_SAMPLE || !a.prm.top_k) return false;
        if (a.prm.greedy && a.prm.greedy[row]) return false;
        const int tk = a.prm.top_k[row];
        return tk > kAsyncMaxK && tk <= kStreamMaxK;
    };
    auto next_row = [&](int k) -> int {
        for (++k; k < my_rows && is_large(row_of(k)); ++k) {}
        return k;
    };

    if (tid == 0) {
        for (int s = 0; s < stages; ++s) mbar_init(&full[s], 1), mbar_init(&empty[s], A_SW), mbar_init(&patched[s], 1);
        for (int p = 0; p < 2; ++p) mbar_init(&closed[p], A_SW), mbar_init(&boot_done[p], 1);
        for (int p = 0; p < 2; ++p) mbar_init(&head_done[p], A_SW);
        for (int p = 0; p < 2; ++p) mbar_init(&draw_full[p], 1), mbar_init(&draw_empty[p], 1), mbar_init(&hv_ready[p], A_PW);
        mbar_fence_init();
    }
    for (int i = tid; i < 2 * A_L; i += A_THREADS) logs[i] = 0ull;
    __syncthreads();
    if (my_rows == 0 || next_row(-1) >= my_rows) {
        if (tid < my_rows && a.out.status && a.mode == MODE_SAMPLE)
            for (int k = tid; k < my_rows; k += A_THREADS) a.out.status[row_of(k)] = ROW_LARGE_K;
        if (a.fin_list) {
            __threadfence();
            __syncthreads();
            if (warp == 0) list_leftovers(a);
        }
        return;
    }

    // =========================================================== producer
    if (warp == 0) {
        if (lane_id() != 0) return;
        uint32_t it = 0;
#ifdef WB_PHASE_TIMERS
        long long tp_wait = 0;
#endif
#ifdef WB_STAGGER
        for (uint32_t d = 0; d < (blockIdx.x & 7u) * WB_STAGGER; ++d) __nanosleep(1000);
#endif
        for (int k = next_row(-1); k < my_rows; k = next_row(k)) {
            const uint8_t* src = reinterpret_cast<const uint8_t*>(a.x) + size_t(row_of(k)) * row_bytes;
            for (uint32_t i = 0; i < n_seq; ++i, ++it) {
                const uint32_t c = seq_stage(i);
                const uint32_t s = it % stages, use = it / stages;
#ifdef WB_PHASE_TIMERS
                const long long tw0 = clock64();
#endif
                if (!mbar_wait(&empty[s], (use & 1) ^ 1)) {
                    atomicExch(a.err, 1u);
                    return;
                }
#ifdef WB_PHASE_TIMERS
                tp_wait += clock64() - tw0;
#endif
                const size_t off = size_t(c) * ch_bytes;
                const uint32_t bytes = uint32_t(row_bytes - off < size_t(ch_bytes) ? row_bytes - off : size_t(ch_bytes));
                // (with penalties the stage was also written to: those writes, seen through the barriers, stay before the copy)
                if (pen) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                mbar_expect_tx(&full[s], bytes);
                bulk_g2s(ring + size_t(s) * ch_bytes, src + off, bytes, &full[s]);
            }
        }
#ifdef WB_PHASE_TIMERS
        atomicAdd(reinterpret_cast<unsigned long long*>(a.err + 16) + 7, (unsigned long long)tp_wait);
#endif
        return;
    }

    const bool sample = a.mode == MODE_SAMPLE;
    const RowParams& P = a.prm;
    // candidates wanted for a row (the stream and the tail group must agree)
    auto k_of = [&](int row) -> uint32_t {
        uint32_t K;
        if (sample) {
            const bool greedy = P.greedy && P.greedy[row];
            const uint32_t tk = P.top_k ? uint32_t(max(P.top_k[row], 0)) : 0u;
            K = greedy ? 1u : ((tk > 0 && tk <= uint32_t(kAsyncMaxK)) ? tk : uint32_t(min(a.level_k, kAsyncMaxK)));
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
        return tk >= 1 && tk <= kAsyncMaxK && uint32_t(tk) <= n;
    };

    // does the row have penalties to apply (every role must agree)
    auto pen_row = [&](int row) -> bool {
        if (!sample || !P.hit_list || P.hist_len[row] <= 0) return false;
        const float r = P.rep ? P.rep[row] : 1.f, pr = P.pres ? P.pres[row] : 0.f, fr = P.freq ? P.freq[row] : 0.f;
        return r != 1.f || pr != 0.f || fr != 0.f;
    };

    // =========================================================== penalty warps
    // They walk the row's hit list (its distinct history tokens with their counts, stage by stage; history_lists_kernel)
    // while the row streams, taking the stages in turn: as soon as a stage has landed its warp takes the raw logits of the
    // stage's history tokens out (replaced by -inf, so the stream warps see them as absent), puts them aside in global
    // memory, and hands the stage on to the stream warps.  Nothing else: the tail group applies the penalties and adds the
    // tokens to the row once the row has streamed.  They depend on no threshold and no row slot, so they run as far ahead
    // of the stream warps as the ring allows.  The first s0 stages come twice (see the stream warps); the second time their
    // tokens are only taken out again.  Entries are read in blocks of 128 (four per lane, loaded together), the first
    // block of a warp's next stage while it works on the current one.
    if (warp >= 2 + A_SW + A_TW) {
        if (!pen) return;
        const int lane = lane_id(), pw = warp - (2 + A_SW + A_TW);
        constexpr uint32_t none = 0xffffffffu;
        constexpr uint32_t PB = 128;  // entries per block: four per lane
        uint32_t it0 = 0;             // ring position of this row's first stage
        int ord = 0;
#ifdef WB_PHASE_TIMERS
        long long tq_wait = 0, tq_take = 0, tq_pref = 0, tq_row = 0;
        const long long tq_begin = clock64();
#endif
        for (int k = next_row(-1); k < my_rows; k = next_row(k), ++ord, it0 += n_seq) {
            const int p = ord & 1;
            const int row = row_of(k);
            const bool pen_on = pen_row(row);
            const uint32_t* hl_row = P.hit_list + size_t(row) * kHitListStride;
            float* hv_row = P.hit_val + size_t(row) * kHitListStride;
            // The places of the row's stages in its list, [c] = first entry of stage c (c = 0 .. n_chunks), in shared memory:
            // this warp runs one instruction after the other next to five busy warps on its scheduler, so what it does
            // per stage is kept short (two broadcast loads here; one 32-entry block in the common case below).
            uint32_t* bnd = sh->pbnd[pw];
            if (pen_on) {
                const uint32_t* hs = P.hit_start + size_t(row) * kHitStartStride;
                for (uint32_t c = lane; c <= n_chunks; c += 32) bnd[c] = min(hs[c], uint32_t(kMaxHist));
            }
            __syncwarp();
            uint32_t s_nx = 0, e_nx = 0, w_nx[4] = {none, none, none, none};
            auto prefetch = [&](uint32_t i) {
                s_nx = e_nx = 0;
                w_nx[0] = w_nx[1] = w_nx[2] = w_nx[3] = none;
                if (pen_on && i < n_seq) {
                    const uint32_t cc = seq_stage(i);
                    s_nx = bnd[cc], e_nx = bnd[cc + 1];
                    if (s_nx + lane < e_nx) w_nx[0] = hl_row[s_nx + lane];
                    if (e_nx - s_nx > 32) {  // (seldom: the same for the whole warp)
#pragma unroll
                        for (int j = 1; j < 4; ++j)
                            if (s_nx + 32 * j + lane < e_nx) w_nx[j] = hl_row[s_nx + 32 * j + lane];
                    }
                }
            };
            // this warp's places in the row's sequence of stages: i0, i0 + A_PW, ...
            uint32_t i = (uint32_t(pw) + A_PW - it0 % A_PW) % A_PW;
            prefetch(i);
            for (; i < n_seq; i += A_PW) {
                const uint32_t c = seq_stage(i);
                const bool keep = i < s0 || i >= 2 * s0;  // (not on the second visit of the first stages)
                const uint32_t it = it0 + i, st_slot = it % uint32_t(stages), st_phase = (it / uint32_t(stages)) & 1u;
                uint32_t cur = s_nx;
                const uint32_t end = e_nx;
                uint32_t w[4] = {w_nx[0], w_nx[1], w_nx[2], w_nx[3]};
#ifdef WB_PHASE_TIMERS
                const long long tq0 = clock64();
#endif
                if (!mbar_wait(&full[st_slot], st_phase)) {
                    if (lane == 0) atomicExch(a.err, 7u);
                    return;
                }
#ifdef WB_PHASE_TIMERS
                const long long tq1 = clock64();
                tq_wait += tq1 - tq0;
#endif
                T* stage_mem = reinterpret_cast<T*>(ring + size_t(st_slot) * ch_bytes);
                // entry e, at place idx of the list, leaves the stage
                auto take_out = [&](uint32_t e, uint32_t idx) {
                    if (e == none) return;
                    const uint32_t off = (e & kPenMaxV) - c * A_CH;
                    if (off >= uint32_t(A_CH)) {
                        // (cannot happen with a list from history_lists_kernel: never write outside the stage)
                        atomicExch(a.err, 20u);
                        return;
                    }
                    T* at = stage_mem + off;
                    if (sizeof(T) == 4) {
                        if (keep) hv_row[idx] = *reinterpret_cast<float*>(at);
                        *reinterpret_cast<uint32_t*>(at) = 0xff800000u;
                    } else {
                        if (keep) hv_row[idx] = __uint_as_float(uint32_t(*reinterpret_cast<uint16_t*>(at)) << 16);
                        *reinterpret_cast<uint16_t*>(at) = 0xff80u;
                    }
                };
                if (cur < end) {
                    take_out(w[0], cur + lane);
                    if (end - cur > 32) {
#pragma unroll
                        for (int j = 1; j < 4; ++j) take_out(w[j], cur + 32 * j + lane);
                    }
                    cur += PB;
                }
                // (a stage with more than 128 tokens, the low ids as a rule: 512 entries per trip to memory)
                while (cur < end) {
                    uint32_t big[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) big[j] = cur + 32 * j + lane < end ? hl_row[cur + 32 * j + lane] : none;
#pragma unroll
                    for (int j = 0; j < 16; ++j) take_out(big[j], cur + 32 * j + lane);
                    cur += 4 * PB;
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&patched[st_slot]);  // the stream warps may read the stage
#ifdef WB_PHASE_TIMERS
                const long long tq2 = clock64();
                tq_take += tq2 - tq1;
#endif
                prefetch(i + A_PW);
#ifdef WB_PHASE_TIMERS
                tq_pref += clock64() - tq2;
#endif
            }
#ifdef WB_PHASE_TIMERS
            const long long tq3 = clock64();
#endif
            // every raw logit of the row's history tokens is put aside: the tail group may read them
            __threadfence_block();
            __syncwarp();
            if (lane == 0) mbar_arrive(&hv_ready[p]);
#ifdef WB_PHASE_TIMERS
            tq_row += clock64() - tq3;
#endif
        }
#ifdef WB_PHASE_TIMERS
        if (pw == 0 && lane == 0) {
            unsigned long long* dbg = reinterpret_cast<unsigned long long*>(a.err + 16);
            atomicAdd(&dbg[24], (unsigned long long)tq_wait), atomicAdd(&dbg[25], (unsigned long long)tq_take), atomicAdd(&dbg[26], (unsigned long long)tq_pref);
            atomicAdd(&dbg[27], (unsigned long long)tq_row), atomicAdd(&dbg[28], (unsigned long long)(clock64() - tq_begin));
        }
#endif
        return;
    }

    // =========================================================== draw warp
    // Takes a row's candidates from the tail group and does the rest of the row on its own: probabilities, the top-k /
    // top-p / min-p cuts, the draw and the row's outputs, while the tail group is already busy with the next row.
    if (warp == 1 + A_SW + A_TW) {
        if (!sample) return;
        const int lane = lane_id();
        const Group<32> gw{lane, 0};
        int ord = 0;
        for (int k = next_row(-1); k < my_rows; k = next_row(k), ++ord) {
            const int p = ord & 1;
            if (!mbar_wait(&draw_full[p], (ord >> 1) & 1)) {
                if (lane == 0) atomicExch(a.err, 8u);
                return;
            }
            const DrawIn d = sh->draw[p];
            if (!d.skip) {
                const int row = d.row;
                unsigned long long* hd = hand + size_t(p) * kAsyncMaxK;
                const float inv_t = P.inv_t ? P.inv_t[row] : P.inv_t_scalar;
                const uint32_t kept = d.kept;
                float M = d.M, sum = d.sum;
                TailIn in;
                in.inv_t = inv_t;
                in.top_k = P.top_k ? uint32_t(max(P.top_k[row], 0)) : 0u;
                in.top_p = P.top_p ? P.top_p[row] : 1.0, in.min_p = P.min_p ? P.min_p[row] : 0.0, in.u = P.u ? P.u[row] : 0.0;
                if (no_sum_row(row)) {
                    // normalise over the candidates themselves (sorted or not, hd[] holds exactly the kept ones)
                    unsigned long long top = 0ull;
                    for (uint32_t i = lane; i < kept; i += 32) top = hd[i] > top ? hd[i] : top;
                    top = warp_max(uint64_t(top));
                    M = float_of_key(cand_key(top));
                    for (uint32_t i = lane; i < kept; i += 32) tail_q[i] = exp(double(__fsub_rn(float_of_key(cand_key(hd[i])), M)) * double(inv_t));
                    __syncwarp();
                    sum = float(warp_total(tail_q, kept));
                    __syncwarp();
                }
                in.m = M, in.sum = sum, in.cnt = kept, in.cap = d.cap, in.V = n;
                in.race = P.race_key != nullptr, in.race_key = P.race_key ? P.race_key[row] : 0;
                in.presorted = d.presorted != 0;
                sample_tail<32>(gw, in, reinterpret_cast<uint64_t*>(hd), tail_p, tail_q, &sh->res);
                const TailOut r = sh->res;
                if (lane == 0) {
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
                    for (uint32_t j = lane; j < nk; j += 32) {
                        if (a.out.kept_ids) a.out.kept_ids[size_t(row) * a.out.kept_cap + j] = int32_t(cand_id(hd[j]));
                        if (a.out.kept_p) a.out.kept_p[size_t(row) * a.out.kept_cap + j] = tail_p[j];
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&draw_empty[p]);
        }
        // Every row of this CTA has its status (the tail group's writes came before its last hand-over).
        if (a.fin_list) list_leftovers(a);
        return;
    }

    // =========================================================== tail
    if (warp > A_SW) {  // (the draw warp and the penalty warps have returned above)
        const Group<A_TT> g{tid - 32 - A_ST, 2};

        // slot o & 1 becomes the row's (the CTA's k-th): no threshold yet, an empty log (zeroed when its last row finished)
        auto bootstrap = [&](int k, int o) -> bool {
            const int p = o & 1;
            g.sync();
            if (g.tid < A_SW) wbound[p * A_SW + g.tid] = 0u;
            g.sync();
            if (g.tid == 0) {
                sh->slot[p].tau = 0ull;
                sh->slot[p].cnt = 0;
                sh->slot[p].row = row_of(k);
                mbar_arrive(&boot_done[p]);
            }
            return true;
        };

#ifdef WB_PHASE_TIMERS
        long long tt[8] = {0, 0, 0, 0, 0, 0, 0, 0};  // bootstrap, refine, final, total; final split: combine, rank, clear, draw
        const long long tt0 = clock64();
#define TT_ADD(i, t0) do { if (g.tid == 0) tt[i] += clock64() - (t0); } while (0)
#else
#define TT_ADD(i, t0)
#endif
        if (sample && a.out.status)
            for (int k = g.tid; k < my_rows; k += A_TT)
                if (is_large(row_of(k))) a.out.status[row_of(k)] = ROW_LARGE_K;
        if (!bootstrap(next_row(-1), 0)) {
            if (g.tid == 0) atomicExch(a.err, 2u);
            return;
        }
        int ord = 0;
        uint32_t carry_last = 0, carry_step = 0;  // refinement state of the next row, when its first one ran early
        for (int k = next_row(-1); k < my_rows; ++ord) {
            const int kn = next_row(k);
            const int p = ord & 1;
            ASlot* sl = &sh->slot[p];
            unsigned long long* log = logs + size_t(p) * A_L;
            const int row = row_of(k);
            const uint32_t K = k_of(row);
            bool booted = kn >= my_rows;
            uint32_t n_last = carry_last;
#ifdef WB_PHASE_TIMERS
            uint32_t n_refine = 0;
#endif
            // the first refinement as soon as the log holds K entries, later ones when it has grown by a few K
            uint32_t step = carry_step;
            carry_last = carry_step = 0;
            // ---- while the row streams: raise its threshold, prepare the next row
            for (uint32_t spin = 0;; ++spin) {
                if (g.tid == 0) {
                    sh->flag[1] = mbar_try_wait(&closed[p], (ord >> 1) & 1) ? 1u : 0u;
                    const uint32_t c = ld_volatile_u32(&sl->cnt);
                    sh->flag[2] = c < uint32_t(A_L) ? c : uint32_t(A_L);
                }
                g.sync();
                const bool done = sh->flag[1] != 0;
                const uint32_t nlog = sh->flag[2];
                g.sync();
                if (done) break;
                if (spin > (1u << 22)) {
                    if (g.tid == 0) atomicExch(a.err, 3u);
                    return;
                }
                if (nlog >= K && nlog >= 64 && nlog >= n_last + step) {
#ifdef WB_PHASE_TIMERS
                    const long long tr0 = clock64();
#endif
                    // the exact K-th largest of the log so far: tighter than the stream warps' own bound from their maxima
                    // (entries reserved but not written yet read as zero and rank last: the bound stays valid)
                    const unsigned long long kth = select_kth<A_TT>(g, log, nlog, K, hist, &sh->sel);
                    if (g.tid == 0 && kth > ld_volatile_u64(&sl->tau)) *reinterpret_cast<volatile unsigned long long*>(&sl->tau) = kth;
                    n_last = nlog;
                    step = 2 * K > 128 ? 2 * K : 128;
#ifdef WB_PHASE_TIMERS
                    ++n_refine;
                    TT_ADD(1, tr0);
#endif
                    g.sync();
                } else if (!booted) {
#ifdef WB_PHASE_TIMERS
                    const long long tb0 = clock64();
#endif
                    if (!bootstrap(kn, ord + 1)) {
                        if (g.tid == 0) atomicExch(a.err, 2u);
                        return;
                    }
                    TT_ADD(0, tb0);
                    booted = true;
                } else {
                    __nanosleep(1000);
                }
            }
            if (!booted && !bootstrap(kn, ord + 1)) {
                if (g.tid == 0) atomicExch(a.err, 2u);
                return;
            }
            // acquire the stream warps' writes
            mbar_wait(&closed[p], (ord >> 1) & 1);
#ifdef WB_PHASE_TIMERS
            const long long tf0 = clock64();
#endif
            // ---- the row is through
            if (pen) {
                // The row's history tokens, taken out of the stages by the penalty warps, get their penalty and join the row
                // here (all the group's threads: one warp took a third of a row's time for it): each tail warp is one more
                // contributor to the row's maximum and sum, and the tokens that can be among the K best go to the log.
                if (!mbar_wait(&hv_ready[p], (ord >> 1) & 1)) {
                    if (g.tid == 0) atomicExch(a.err, 6u);
                    return;
                }
                const bool skip_sum = no_sum_row(row);
                const float inv_t_j = P.inv_t ? P.inv_t[row] : P.inv_t_scalar;
                const float cexp = inv_t_j * kLog2e;
                float m_t = -INFINITY, e_t = 0.f, s_t = 0.f;
                if (pen_row(row)) {
                    const float pen_rep = P.rep ? P.rep[row] : 1.f, pen_pres = P.pres ? P.pres[row] : 0.f, pen_freq = P.freq ? P.freq[row] : 0.f;
                    const uint32_t* hl_row = P.hit_list + size_t(row) * kHitListStride;
                    const float* hv_row = P.hit_val + size_t(row) * kHitListStride;
                    const uint32_t n_hit = min(P.hit_start[size_t(row) * kHitStartStride + n_chunks], uint32_t(kMaxHist));
                    const unsigned long long tau = ld_volatile_u64(&sl->tau);
                    const float tau_f = float_of_key(cand_key(tau));
                    for (uint32_t base = 0; base < n_hit; base += 4 * A_TT) {
                        uint32_t e4[4];
                        float r4[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j) {  // (the loads first, then the arithmetic)
                            const uint32_t idx = base + j * A_TT + g.tid;
                            e4[j] = idx < n_hit ? hl_row[idx] : 0xffffffffu;
                            r4[j] = idx < n_hit ? __ldcg(hv_row + idx) : 0.f;
                        }
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            if (e4[j] == 0xffffffffu) continue;
                            float l = r4[j];
                            l = (l > 0.f) ? __fdiv_rn(l, pen_rep) : __fmul_rn(l, pen_rep);
                            const float x = __fsub_rn(l, __fadd_rn(pen_pres, __fmul_rn(pen_freq, float(e4[j] >> kPenIdBits))));
                            if (!skip_sum) {
                                if (x > m_t) {
                                    const float ne = ceilf(x * cexp);
                                    s_t = (m_t == -INFINITY) ? 0.f : s_t * ex2_approx(e_t - ne);
                                    e_t = ne, m_t = x;
                                }
                                if (m_t != -INFINITY) s_t += ex2_approx(fmaf(x, cexp, -e_t));
                            } else {
                                m_t = fmaxf(m_t, x);
                            }
                            if (x >= tau_f) {
                                const unsigned long long cnd = make_cand(key_of(x), e4[j] & kPenMaxV);
                                if (cnd > tau) {
                                    const uint32_t pos = atomicAdd(&sl->cnt, 1u);
                                    if (pos < uint32_t(A_L)) log[pos] = cnd;
                                }
                            }
                        }
                    }
                }
                const bool saw_nan = !skip_sum && (s_t != s_t);
                if (__any_sync(0xffffffffu, saw_nan) && (g.tid & 31) == 0) atomicOr(&sl->cnt, 0x80000000u);
                const float wm = warp_max(m_t);
                float we = e_t;
                if (m_t == -INFINITY) we = -INFINITY;
                we = warp_max(we);
                double ds = (m_t == -INFINITY) ? 0.0 : double(s_t) * double(ex2_approx(e_t - we));
                ds = warp_sum(ds);
                if ((g.tid & 31) == 0) sl->red_m[A_SW + (g.tid >> 5)] = wm, sl->red_e[A_SW + (g.tid >> 5)] = we, sl->red_s[A_SW + (g.tid >> 5)] = ds;
                g.sync();
            }
            const uint32_t total = sl->cnt;  // bit 31: a warp met a NaN logit
            const bool overflow = total > uint32_t(A_L);
#ifdef WB_PHASE_TIMERS
            if (g.tid == 0) {
                if (overflow) atomicAdd(&a.err[1], 1u);
                atomicMax(&a.err[2], total);
                atomicAdd(&a.err[3], n_refine);
            }
#endif
            const uint32_t nlog = overflow ? uint32_t(A_L) : total;
            // row max and normaliser: combine the warps' partials, one per lane (not needed when the row is normalised
            // over its candidates)
            const bool greedy = sample && P.greedy && P.greedy[row];
            const float inv_t = P.inv_t ? P.inv_t[row] : P.inv_t_scalar;
            const bool no_sum = no_sum_row(row);
            float M = -INFINITY, sum = 0.f;
            if (!no_sum) {
                const int n_red = A_SW + (pen ? A_TW : 0), ln = g.tid & 31;
                static_assert(A_SW + A_TW <= 32, "one partial per lane");
                const float mw = ln < n_red ? sl->red_m[ln] : -INFINITY;
                M = warp_max(mw);
                const double cexp = double(inv_t * kLog2e);
                const double term = (ln < n_red && mw != -INFINITY) ? sl->red_s[ln] * exp2(double(sl->red_e[ln]) - double(M) * cexp) : 0.0;
                sum = float(warp_sum(term));
            }
            unsigned long long* hand_p = hand + size_t(p) * kAsyncMaxK;
            // the draw warp is done with this slot's candidates (its row two rows ago)
            if (sample && !mbar_wait(&draw_empty[p], ((ord >> 1) & 1) ^ 1)) {
                if (g.tid == 0) atomicExch(a.err, 9u);
                return;
            }
#ifdef WB_PHASE_TIMERS
            const long long tf1 = clock64();
            TT_ADD(4, tf0);
#endif
            uint32_t kept = 0;
            bool presorted = false;
            if (!overflow) {
                // Most of the log was appended under an earlier, looser threshold: only entries at or above the current one
                // can be among the K best (at least K of them are).  Few survive, so rank them against each other: the
                // rank is the position in the sorted order.
                unsigned long long* list = reinterpret_cast<unsigned long long*>(hist);  // up to SEL_BINS / 2 entries
                write_survivors<A_TT>(g, log, nlog, sl->tau, list, SEL_BINS / 2, &sh->sel);
                const uint32_t m = sh->sel.wcnt;
                if (m <= uint32_t(kAsyncMaxK)) {
                    for (uint32_t t = g.tid; t < m; t += A_TT) {
                        const unsigned long long mine = list[t];
                        uint32_t rank = 0;
                        for (uint32_t j = 0; j < m; ++j) rank += list[j] > mine;
                        if (rank < K) hand_p[rank] = mine;
                    }
                    kept = m < K ? m : K;
                    presorted = true;
                } else if (nlog > K) {
                    const unsigned long long kth = select_kth<A_TT>(g, log, nlog, K, hist, &sh->sel);
                    write_survivors<A_TT>(g, log, nlog, kth, hand_p, kAsyncMaxK, &sh->sel);
                    kept = sh->sel.wcnt < uint32_t(kAsyncMaxK) ? sh->sel.wcnt : uint32_t(kAsyncMaxK);
                } else {
                    for (uint32_t i = g.tid; i < nlog; i += A_TT) hand_p[i] = log[i];
                    kept = nlog;
                }
            }
#ifdef WB_PHASE_TIMERS
            const long long tf2 = clock64();
            TT_ADD(5, tf1);
#endif
            uint32_t cap = 1;
            while (cap < kept) cap <<= 1;
            g.sync();
            for (uint32_t i = kept + g.tid; i < cap; i += A_TT) hand_p[i] = 0ull;
            // the log is free for row k + 2 once it is zero again
            for (uint32_t i = g.tid; i < nlog; i += A_TT) log[i] = 0ull;
            g.sync();
#ifdef WB_PHASE_TIMERS
            const long long tf3 = clock64();
            TT_ADD(6, tf2);
#endif
            if (overflow) {
                // more candidates than the log holds (rows in adversarial order): the multi-pass kernel takes the row
                if (g.tid == 0) a.out.status[row] = ROW_RETRY;
            } else if (!sample) {
                if (g.tid == 0) a.out.status[row] = ROW_DONE;
                if (!presorted) sort_desc<A_TT>(g, reinterpret_cast<uint64_t*>(hand_p), cap);
                const T* xr = reinterpret_cast<const T*>(a.x) + size_t(row) * n;
                for (uint32_t j = g.tid; j < kept; j += A_TT) {
                    const uint32_t id = cand_id(hand_p[j]);
                    a.ids[size_t(row) * a.K + j] = int32_t(id) + a.id_offset;
                    a.vals[size_t(row) * a.K + j] = sizeof(T) == 4 ? reinterpret_cast<const float*>(xr)[id] : bf16_to_f32(reinterpret_cast<const uint16_t*>(xr)[id]);
                }
                if (g.tid == 0) a.stats[2 * row] = M, a.stats[2 * row + 1] = sum;
            } else if (greedy) {
                if (g.tid == 0) {
                    const uint32_t tok = kept ? cand_id(hand_p[0]) : 0;
                    a.out.token[row] = int32_t(tok);
                    a.out.status[row] = ROW_DONE;
                    if (a.out.n_kept) a.out.n_kept[row] = 1;
                    if (a.out.closed) a.out.closed[row] = 1;
                    if (a.out.stats) a.out.stats[2 * row] = kept ? float_of_key(cand_key(hand_p[0])) : -INFINITY, a.out.stats[2 * row + 1] = 0.f;
                    if (a.out.kept_ids && a.out.kept_cap > 0) a.out.kept_ids[size_t(row) * a.out.kept_cap] = int32_t(tok);
                    if (a.out.kept_p && a.out.kept_cap > 0) a.out.kept_p[size_t(row) * a.out.kept_cap] = 1.0;
                }
            }
            if (sample) {
                // hand the candidates to the draw warp (or tell it that this row needs none of its work)
                if (g.tid == 0) {
                    DrawIn d;
                    d.row = row, d.kept = kept, d.cap = cap, d.M = M, d.sum = sum, d.presorted = presorted ? 1u : 0u;
                    d.skip = (overflow || greedy) ? 1u : 0u;
                    sh->draw[p] = d;
                    __threadfence();  // (a status written above is read by another CTA at the end of the kernel)
                    mbar_arrive(&draw_full[p]);  // (after the barrier above: every thread's candidates are written)
                }
            }
            g.sync();
            TT_ADD(2, tf0);
#ifdef WB_PHASE_TIMERS
            TT_ADD(7, tf3);
#endif
            k = kn;
        }
#ifdef WB_PHASE_TIMERS
        if (g.tid == 0) {
            tt[3] = clock64() - tt0;
            unsigned long long* dbg = reinterpret_cast<unsigned long long*>(a.err + 16);
            for (int i = 0; i < 4; ++i) atomicAdd(&dbg[i], (unsigned long long)tt[i]), atomicAdd(&dbg[8 + i], (unsigned long long)tt[4 + i]);
        }
#endif
        return;
    }

    // =========================================================== stream
    // Each warp reads its share of every stage (f32: logits [128 w, 128 w + 128) of each half stage; bf16: logits [256 w,
    // 256 w + 256)), keeps per-lane running maxima and sums, and appends the logits that can still be among the K best to
    // the row's log.  What "can still be" means needs a threshold, and a row has none when it starts.  So the first s0
    // stages of a row come through the ring twice: the first time the warps only accumulate; then every warp names the
    // r-th largest of its 32 lane maxima, r = ceil(K / 16) (16 r >= K distinct logits of the row are at or above the
    // smallest of those 16 values, so it is a valid threshold); the second time (a re-read a few microseconds later, from
    // L2) the warps only log, against that threshold.  The rest of the row does both at once, and the threshold keeps
    // rising: from the warps' maxima again after more of the row, and from the tail group's exact K-th best of the log.
    const int lane = lane_id(), sw = (tid - 32) >> 5;
    static_assert(A_CH / 8 == A_ST, "eight elements per thread per stage");
    static_assert(A_CH == kHitStage, "the hit lists are grouped by this kernel's stages");
    uint32_t st_slot = 0, st_phase = 0;  // ring position of this warp and the parity it waits for
    uint32_t st_ring[2] = {0, 0};
    uint64_t* ready = pen ? patched : full;  // with penalties a stage is read only after a penalty warp has been over it
    constexpr int M_BOTH = 0, M_ACC = 1, M_LOG = 2;
#ifdef WB_PHASE_TIMERS
    long long ts_wait = 0, ts_proc = 0, ts_setup = 0, ts_slow = 0, ts_bound = 0;
#endif
    int ord = 0;
    for (int k = next_row(-1); k < my_rows; k = next_row(k), ++ord) {
#ifdef WB_PHASE_TIMERS
        const long long tsu0 = clock64();
#endif
        const int p = ord & 1;
        const int row = row_of(k);
        ASlot* sl = &sh->slot[p];
        unsigned long long* log = logs + size_t(p) * A_L;
        const bool greedy = no_sum_row(row);  // no exponentials for this row (greedy, or closed by its top_k)
        const float inv_t = P.inv_t ? P.inv_t[row] : P.inv_t_scalar;
        const float cexp = inv_t * kLog2e;
        float m_t = -INFINITY, e_t = 0.f, s_t = 0.f;  // running max, reference exponent ceil(m_t * cexp), sum 2^(x * cexp - e_t)
#ifdef WB_PHASE_TIMERS
        ts_setup += clock64() - tsu0;
#endif
        bool st_fail = false;
        unsigned long long tau_seen = 0ull;
        float tau_f = -INFINITY;
        uint32_t* wb_row = wbound + p * A_SW;
        const uint32_t rth = (k_of(row) + A_SW - 1) / A_SW;  // each warp's share of the K candidates

        // NS consecutive stages at once (more independent work per warp, fixed costs paid once)
        auto stage = [&](uint32_t c, auto ns_tag, auto mode_tag) {
            constexpr int NS = decltype(ns_tag)::value;
            constexpr int MODE = decltype(mode_tag)::value;
            constexpr int NE = 8 * NS;   // elements per thread
            constexpr int NQ = 2 * NS;   // quads of 4 consecutive elements
#ifdef WB_PHASE_TIMERS
            const long long tw0 = clock64();
#endif
            float xv[NE];
            uint32_t qid[NQ];
            bool qv[NQ];
            if (MODE != M_ACC) {
                const unsigned long long t = ld_volatile_u64(&sl->tau);
                if (t > tau_seen) tau_seen = t, tau_f = float_of_key(cand_key(t));
            }
            const unsigned long long tau = tau_seen;
#pragma unroll
            for (int h = 0; h < NS; ++h) {
                if (!mbar_wait(&ready[st_slot], st_phase)) {
                    if (lane == 0) atomicExch(a.err, 5u);
                    st_fail = true;
                    return;
                }
                const uint4* vec = reinterpret_cast<const uint4*>(ring + size_t(st_slot) * ch_bytes);
                float* x = xv + 8 * h;
                const int st_tid = tid - 32;
                if (sizeof(T) == 4) {
                    qid[2 * h] = (c + h) * A_CH + 4 * st_tid, qid[2 * h + 1] = qid[2 * h] + 4 * A_ST;
                    qv[2 * h] = qid[2 * h] < n, qv[2 * h + 1] = qid[2 * h + 1] < n;  // (only the row's last stage can be short)
                    const uint4 ninf = make_uint4(0xff800000u, 0xff800000u, 0xff800000u, 0xff800000u);
                    const uint4 q0 = qv[2 * h] ? vec[st_tid] : ninf;
                    const uint4 q1 = qv[2 * h + 1] ? vec[st_tid + A_ST] : ninf;
                    x[0] = __uint_as_float(q0.x), x[1] = __uint_as_float(q0.y), x[2] = __uint_as_float(q0.z), x[3] = __uint_as_float(q0.w);
                    x[4] = __uint_as_float(q1.x), x[5] = __uint_as_float(q1.y), x[6] = __uint_as_float(q1.z), x[7] = __uint_as_float(q1.w);
                } else {
                    qid[2 * h] = (c + h) * A_CH + 8 * st_tid, qid[2 * h + 1] = qid[2 * h] + 4;
                    qv[2 * h] = qv[2 * h + 1] = qid[2 * h] < n;
                    const uint4 q = qv[2 * h] ? vec[st_tid] : make_uint4(0xff80ff80u, 0xff80ff80u, 0xff80ff80u, 0xff80ff80u);
                    x[0] = __uint_as_float(q.x << 16), x[1] = __uint_as_float(q.x & 0xffff0000u);
                    x[2] = __uint_as_float(q.y << 16), x[3] = __uint_as_float(q.y & 0xffff0000u);
                    x[4] = __uint_as_float(q.z << 16), x[5] = __uint_as_float(q.z & 0xffff0000u);
                    x[6] = __uint_as_float(q.w << 16), x[7] = __uint_as_float(q.w & 0xffff0000u);
                }
                st_ring[h] = st_slot;
                if (++st_slot == uint32_t(stages)) st_slot = 0, st_phase ^= 1u;
            }
#ifdef WB_PHASE_TIMERS
            const long long tw1 = clock64();
            ts_wait += tw1 - tw0;
#endif
            // maxima of the quads; fmaxf skips NaN, so a NaN logit never raises a maximum
            float qm[NQ];
#pragma unroll
            for (int q = 0; q < NQ; ++q) qm[q] = fmaxf(fmaxf(xv[4 * q], xv[4 * q + 1]), fmaxf(xv[4 * q + 2], xv[4 * q + 3]));
            // Every loaded register has been consumed, so the shared-memory reads have completed (instructions issue in
            // order and the fmaxf had to wait for the data): only now may the producer overwrite the stages.
            __syncwarp();
            if (lane == 0) {
#pragma unroll
                for (int h = 0; h < NS; ++h) mbar_arrive(&empty[st_ring[h]]);
            }
            float vm = qm[0];
#pragma unroll
            for (int q = 1; q < NQ; ++q) vm = fmaxf(vm, qm[q]);
            if (MODE != M_LOG) {
                if (!greedy) {
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
                        for (int j = 0; j < NE; ++j) acc[j & 3] += ex2_approx(fmaf(xv[j], cexp, -e_t));
                        s_t += (acc[0] + acc[1]) + (acc[2] + acc[3]);
                    }
                } else {
                    m_t = fmaxf(m_t, vm);
                }
            }
#ifdef WB_PHASE_TIMERS
            const long long tsl0 = clock64();
#endif
            if (MODE != M_ACC && vm >= tau_f) {
                // rare: this lane holds an element that may beat the threshold
#pragma unroll
                for (int q = 0; q < NQ; ++q) {
                    if (qm[q] >= tau_f && qv[q]) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float x = xv[4 * q + j];
                            if (x >= tau_f) {
                                const unsigned long long cnd = make_cand(key_of(x), qid[q] + j);
                                if (cnd > tau) {
                                    const uint32_t pos = atomicAdd(&sl->cnt, 1u);
                                    if (pos < uint32_t(A_L)) log[pos] = cnd;
                                }
                            }
                        }
                    }
                }
            }
#ifdef WB_PHASE_TIMERS
            const long long tsl1 = clock64();
            ts_slow += tsl1 - tsl0;
            ts_proc += tsl1 - tw1;
#endif
        };
        // this warp's bound: the rth largest of its lane maxima (the largest is taken away rth - 1 times; keys are
        // order-preserving, 0 is below every logit)
        auto own_bound = [&]() -> uint32_t {
            uint32_t kv = key_of(m_t), kr = 0;
            for (uint32_t i = 0; i < rth; ++i) {
                kr = __reduce_max_sync(0xffffffffu, kv);
                if (kr == 0) break;
                const uint32_t holders = __ballot_sync(0xffffffffu, kv == kr);
                if (lane == __ffs(holders) - 1) kv = 0;
            }
            return kr;
        };
        auto run = [&](uint32_t c0, uint32_t c1, auto mode_tag) {
            using one = std::integral_constant<int, 1>;
            using two = std::integral_constant<int, 2>;
            uint32_t c = c0;
            for (; c + 2 <= c1 && !st_fail; c += 2) stage(c, two{}, mode_tag);
            if (c < c1 && !st_fail) stage(c, one{}, mode_tag);
        };
        // ---- the head of the row: accumulate, agree on the first threshold, then log
        run(0, s0, std::integral_constant<int, M_ACC>{});
        if (st_fail) return;
        // the slot (log, threshold, bounds, partials) is this row's once the tail group says so: not needed before here
        if (!mbar_wait(&boot_done[p], (ord >> 1) & 1)) {
            if (lane == 0) atomicExch(a.err, 4u);
            return;
        }
        {
#ifdef WB_PHASE_TIMERS
            const long long tb0 = clock64();
#endif
            const uint32_t kr = own_bound();
            if (lane == 0) {
                wb_row[sw] = kr;
                mbar_arrive(&head_done[p]);
            }
            if (!mbar_wait(&head_done[p], (ord >> 1) & 1)) {
                if (lane == 0) atomicExch(a.err, 11u);
                return;
            }
            const uint32_t kmin = __reduce_min_sync(0xffffffffu, lane < A_SW ? ld_volatile_u32(&wb_row[lane]) : 0xffffffffu);
            tau_seen = (unsigned long long)kmin << 32, tau_f = float_of_key(kmin);
            if (sw == 0 && lane == 0 && tau_seen > ld_volatile_u64(&sl->tau)) *reinterpret_cast<volatile unsigned long long*>(&sl->tau) = tau_seen;
#ifdef WB_PHASE_TIMERS
            ts_bound += clock64() - tb0;
#endif
        }
        run(0, s0, std::integral_constant<int, M_LOG>{});
        // ---- the rest of the row, with a fresh bound from the maxima each time the row seen so far has grown by half
        for (uint32_t c0 = s0, nb = s0 + (s0 + 1) / 2; c0 < n_chunks && !st_fail;) {
            const uint32_t c1 = nb < n_chunks ? ((nb + 1) & ~1u) < n_chunks ? ((nb + 1) & ~1u) : n_chunks : n_chunks;
            run(c0, c1, std::integral_constant<int, M_BOTH>{});
            c0 = c1;
            if (c0 < n_chunks && !st_fail) {
#ifdef WB_PHASE_TIMERS
                const long long tb0 = clock64();
#endif
                // (the other warps' entries may be older: any of their bounds for this row is valid)
                const uint32_t kr = own_bound();
                if (lane == 0) wb_row[sw] = kr;
                __syncwarp();
                const uint32_t kmin = __reduce_min_sync(0xffffffffu, lane < A_SW ? ld_volatile_u32(&wb_row[lane]) : 0xffffffffu);
                // (a plain compare and store: a lost update only leaves the threshold at another valid, lower bound)
                if (lane == 0) {
                    const unsigned long long cand = (unsigned long long)kmin << 32;
                    if (cand > ld_volatile_u64(&sl->tau)) *reinterpret_cast<volatile unsigned long long*>(&sl->tau) = cand;
                }
#ifdef WB_PHASE_TIMERS
                ts_bound += clock64() - tb0;
#endif
            }
            nb = c0 + (c0 + 1) / 2;
        }
        if (st_fail) return;
        // a NaN logit poisons the f32 sum: such rows are redone by the multi-pass kernel, which counts NaN as -inf
        const bool saw_nan = !greedy && (s_t != s_t);
        if (__any_sync(0xffffffffu, saw_nan) && lane == 0) atomicOr(&sl->cnt, 0x80000000u);
        // ---- the row is through for this warp: partials, then close
        {
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
    }
#ifdef WB_PHASE_TIMERS
    if (tid == 32) {
        unsigned long long* dbg = reinterpret_cast<unsigned long long*>(a.err + 16);
        atomicAdd(&dbg[4], (unsigned long long)ts_wait), atomicAdd(&dbg[5], (unsigned long long)ts_proc), atomicAdd(&dbg[6], (unsigned long long)ts_setup);
        atomicAdd(&dbg[12], (unsigned long long)ts_slow), atomicAdd(&dbg[13], (unsigned long long)ts_bound);
    }
#endif
}

static size_t async_fixed_smem() {
    return size_t(2) * A_SW * 4 + size_t(2) * A_L * 8 + SEL_BINS * 4 + size_t(2) * kAsyncMaxK * 8 + 2 * (kAsyncMaxK + 2 * A_TW) * 8 +
           (3 * A_MAXSTAGES + 14) * 8 + sizeof(AShared) + 128;
}

bool sample_async_supported(const SelectArgs& a, int dtype) {
    const size_t es = dtype == 0 ? 4 : 2;
    if (reinterpret_cast<uintptr_t>(a.x) % 16 != 0 || (size_t(a.n) * es) % 16 != 0) return false;  // bulk copies need 16-byte rows
    if (a.mode == MODE_TOPK && a.K > kAsyncMaxK) return false;
    const int ch_bytes = int(A_CH * es);
    return async_fixed_smem() + 3 * size_t(ch_bytes) <= 232448;
}

// (with penalties: a.prm.hit_list / hit_start must have been filled by history_lists_launch on the same stream)
cudaError_t sample_async_launch(const SelectArgs& a, int dtype, int sm_count, cudaStream_t st) {
    const size_t es = dtype == 0 ? 4 : 2;
    const bool pen = a.mode == MODE_SAMPLE && a.prm.hist != nullptr;
    if (pen && (!a.prm.hit_list || !a.prm.hit_start)) return cudaErrorInvalidValue;
    const int ch_bytes = int(A_CH * es);
    const size_t fixed = async_fixed_smem();
    int stages = int((232448 - fixed) / ch_bytes);
    if (stages > A_MAXSTAGES) stages = A_MAXSTAGES;
    if (stages < 3) return cudaErrorInvalidConfiguration;
    const size_t smem = fixed + size_t(stages) * ch_bytes;
    const int grid = a.rows < sm_count ? a.rows : sm_count;
    const cudaError_t em = cudaMemsetAsync(a.err, 0, 64, st);  // the error words, the list count and tickets, the scratch locks
    if (em != cudaSuccess) return em;
    if (dtype == 0) {
        const cudaError_t e = cudaFuncSetAttribute(sample_async_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
        if (e != cudaSuccess) return e;
        sample_async_kernel<float><<<grid, A_THREADS, smem, st>>>(a, stages, pen ? 1 : 0, ch_bytes);
    } else {
        const cudaError_t e = cudaFuncSetAttribute(sample_async_kernel<uint16_t>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
        if (e != cudaSuccess) return e;
        sample_async_kernel<uint16_t><<<grid, A_THREADS, smem, st>>>(a, stages, pen ? 1 : 0, ch_bytes);
    }
    return cudaGetLastError();
}

}  // namespace wb
