// The single-pass fused sampler for B200: every logits row is read from HBM exactly once.
//
// One persistent CTA per SM, three roles (warp specialised):
//   producer  (1 warp)   streams the CTA's rows through a ring of shared-memory stages with bulk async copies (TMA,
//                        cp.async.bulk + mbarrier), running ahead of the consumers across row boundaries;
//   stream    (16 warps) consume the stages: penalties from a shared bit map, running max / sum exp for the softmax
//                        normaliser, and a threshold filter that appends the few elements that can still be among the
//                        row's K best to a candidate buffer; when the buffer fills, an exact select raises the threshold;
//   epilogue  (4 warps)  take each finished row's exact K candidates, sort them, apply top-k / top-p / min-p in f64 and
//                        draw the token, while the stream warps are already on the next row.
//
// It replaces, in one launch and with no host round trip, the reference's topk_rows kernel (seven passes over the row,
// kernels/shared/sample_cand_topk_rows.h:11-98), the candidate download, and the host filter and draw
// (src/sampling/sampler.cpp:15-147).  Selection is exact: a candidate is (key, ~id) with key an order-preserving
// image of the logit, so "larger candidate" is "logit desc, id asc", the order of the host comparators.
#include "kernels.h"
#include "penalty.cuh"
#include "select_smem.cuh"
#include "tail.cuh"

namespace wb {

constexpr int SW = 16;                 // stream warps
constexpr int ST = SW * 32;            // stream threads
constexpr int EW = 4;                  // epilogue warps
constexpr int ET = EW * 32;
constexpr int NTHREADS = 32 + ST + ET;  // + the producer warp
constexpr int CH_ELEMS = 4096;         // logits per ring stage
constexpr int BUF_CAP = 8192;          // candidate buffer entries
constexpr int BUF_TRIG = 4096;         // select when the buffer holds more than this after a stage
constexpr int NBINS = SEL_BINS;
constexpr int HAND = 2;                // hand-over buffers between stream and epilogue

struct Hand {
    int32_t row;
    uint32_t cnt;
    float m, sum;
};

struct StreamShared {
    SelScratch sel;
    unsigned long long tau;
    uint32_t cnt, abort_flag;
    float tau_f;
    float red_m[SW];
    double red_s[SW];
    Hand hand[HAND];
    TailOut res;
};

#ifdef WB_PHASE_TIMERS
#define WB_T(var) const long long var = clock64()
#define WB_ACC(i, t0, t1) do { if (g.tid == 0) tacc[i] += (t1) - (t0); } while (0)
#else
#define WB_T(var)
#define WB_ACC(i, t0, t1)
#endif

__device__ __forceinline__ uint32_t ld_volatile(const uint32_t* p) { return *reinterpret_cast<const volatile uint32_t*>(p); }

template <typename T>
__global__ void __launch_bounds__(NTHREADS, 1)
sample_stream_kernel(SelectArgs a, int stages, int pen_words, int ch_bytes) {
    extern __shared__ __align__(128) uint8_t smem[];
    // ---- carve shared memory
    uint8_t* ring = smem;                                                          // stages * ch_bytes
    unsigned long long* buf = reinterpret_cast<unsigned long long*>(ring + size_t(stages) * ch_bytes);  // BUF_CAP
    uint32_t* hist = reinterpret_cast<uint32_t*>(buf + BUF_CAP);                  // NBINS (8 KiB: also 1024 staged candidates)
    unsigned long long* hand_c = reinterpret_cast<unsigned long long*>(hist + NBINS);  // HAND * kStreamMaxK
    double* tail_p = reinterpret_cast<double*>(hand_c + HAND * kStreamMaxK);       // 2 * (kStreamMaxK + 2 * EW)
    double* tail_q = tail_p + kStreamMaxK + 2 * EW;
    uint64_t* bars = reinterpret_cast<uint64_t*>(tail_q + kStreamMaxK + 2 * EW);   // 2 * stages + 2 * HAND
    StreamShared* sh = reinterpret_cast<StreamShared*>(bars + 2 * 32 + 2 * HAND);
    uint32_t* pen_mem = reinterpret_cast<uint32_t*>((reinterpret_cast<uintptr_t>(sh + 1) + 15) & ~uintptr_t(15));
    uint64_t *full = bars, *empty = bars + 32, *hfull = bars + 64, *hempty = bars + 64 + HAND;

    const int tid = threadIdx.x, warp = tid >> 5;
    const uint32_t n = uint32_t(a.n);
    const int rows = a.row_count ? min(*a.row_count, a.rows) : a.rows;
    const int my_rows = rows > int(blockIdx.x) ? (rows - int(blockIdx.x) + int(gridDim.x) - 1) / int(gridDim.x) : 0;
    auto row_of = [&](int k) -> int {
        const int li = int(blockIdx.x) + k * int(gridDim.x);
        return a.row_list ? (a.row_list[li] & 0x3fffffff) : li;
    };
    const uint32_t n_chunks = (n + CH_ELEMS - 1) / CH_ELEMS;
    const size_t row_bytes = size_t(n) * sizeof(T);

    if (tid == 0) {
        for (int s = 0; s < stages; ++s) mbar_init(&full[s], 1), mbar_init(&empty[s], SW);
        for (int h = 0; h < HAND; ++h) mbar_init(&hfull[h], 1), mbar_init(&hempty[h], 1);
        sh->abort_flag = 0;
        mbar_fence_init();
    }
    __syncthreads();
    if (my_rows == 0) return;

    // =========================================================== producer
    if (warp == 0) {
        if (lane_id() != 0) return;
        uint32_t it = 0;
        for (int k = 0; k < my_rows; ++k) {
            const int row = row_of(k);
            const uint8_t* src = reinterpret_cast<const uint8_t*>(a.x) + size_t(row) * row_bytes;
            for (uint32_t c = 0; c < n_chunks; ++c, ++it) {
                const uint32_t s = it % stages, use = it / stages;
                if (!mbar_wait(&empty[s], (use & 1) ^ 1)) {
                    atomicExch(a.err, 1u);
                    return;
                }
                const size_t off = size_t(c) * ch_bytes;
                const uint32_t bytes = uint32_t(row_bytes - off < size_t(ch_bytes) ? row_bytes - off : size_t(ch_bytes));
                mbar_expect_tx(&full[s], bytes);
                bulk_g2s(ring + size_t(s) * ch_bytes, src + off, bytes, &full[s]);
            }
        }
        return;
    }

    const bool sample = a.mode == MODE_SAMPLE;
    const RowParams& P = a.prm;

    // =========================================================== epilogue
    if (warp > SW) {
        const Group<ET> g{tid - 32 - ST, 2};
        for (int k = 0; k < my_rows; ++k) {
            const int h = k % HAND;
            bool ok = true;
            if (g.tid == 0) ok = mbar_wait(&hfull[h], (k / HAND) & 1);
            if (g.sync_or(!ok)) {
                if (g.tid == 0) atomicExch(a.err, 2u);
                return;
            }
            if (g.tid != 0) mbar_wait(&hfull[h], (k / HAND) & 1);  // acquire for every thread (already complete)
            const Hand hd = sh->hand[h];
            const int row = hd.row;
            unsigned long long* cand = hand_c + size_t(h) * kStreamMaxK;
            uint32_t cap = 1;
            while (cap < hd.cnt) cap <<= 1;
            for (uint32_t i = hd.cnt + g.tid; i < cap; i += ET) cand[i] = 0;
            g.sync();
            if (!sample) {
                sort_desc<ET>(g, reinterpret_cast<uint64_t*>(cand), cap);
                const T* xr = reinterpret_cast<const T*>(a.x) + size_t(row) * n;
                for (uint32_t j = g.tid; j < hd.cnt; j += ET) {
                    const uint32_t id = cand_id(cand[j]);
                    a.ids[size_t(row) * a.K + j] = int32_t(id) + a.id_offset;
                    a.vals[size_t(row) * a.K + j] = sizeof(T) == 4 ? reinterpret_cast<const float*>(xr)[id] : bf16_to_f32(reinterpret_cast<const uint16_t*>(xr)[id]);
                }
                if (g.tid == 0) a.stats[2 * row] = hd.m, a.stats[2 * row + 1] = hd.sum;
            } else if (P.greedy && P.greedy[row]) {
                if (g.tid == 0) {
                    const uint32_t tok = hd.cnt ? cand_id(cand[0]) : 0;
                    a.out.token[row] = int32_t(tok);
                    a.out.status[row] = ROW_DONE;
                    if (a.out.n_kept) a.out.n_kept[row] = 1;
                    if (a.out.closed) a.out.closed[row] = 1;
                    if (a.out.stats) a.out.stats[2 * row] = hd.cnt ? float_of_key(cand_key(cand[0])) : -INFINITY, a.out.stats[2 * row + 1] = 0.f;
                    if (a.out.kept_ids && a.out.kept_cap > 0) a.out.kept_ids[size_t(row) * a.out.kept_cap] = int32_t(tok);
                    if (a.out.kept_p && a.out.kept_cap > 0) a.out.kept_p[size_t(row) * a.out.kept_cap] = 1.0;
                }
            } else {
                TailIn in;
                in.inv_t = P.inv_t ? P.inv_t[row] : P.inv_t_scalar;
                in.top_k = P.top_k ? uint32_t(max(P.top_k[row], 0)) : 0u;
                in.top_p = P.top_p ? P.top_p[row] : 1.0, in.min_p = P.min_p ? P.min_p[row] : 0.0, in.u = P.u ? P.u[row] : 0.0;
                in.m = hd.m, in.sum = hd.sum, in.cnt = hd.cnt, in.cap = cap, in.V = n;
                in.race = P.race_key != nullptr, in.race_key = P.race_key ? P.race_key[row] : 0;
                in.presorted = 0;
                sample_tail<ET>(g, in, reinterpret_cast<uint64_t*>(cand), tail_p, tail_q, &sh->res);
                const TailOut r = sh->res;
                if (g.tid == 0) {
                    a.out.token[row] = int32_t(r.token);
                    a.out.status[row] = r.status;
                    if (a.out.n_kept) a.out.n_kept[row] = int32_t(r.n);
                    if (a.out.closed) a.out.closed[row] = r.closed;
                    if (a.out.stats) a.out.stats[2 * row] = hd.m, a.out.stats[2 * row + 1] = hd.sum;
                    if (a.out.counters && r.status == ROW_ESCALATE) atomicAdd(&a.out.counters[0], 1u);
                    if (a.out.counters && r.status == ROW_OPEN_TAIL) atomicAdd(&a.out.counters[1], 1u);
                }
                if (r.status != ROW_ESCALATE) {
                    const uint32_t nk = min(r.n, uint32_t(max(a.out.kept_cap, 0)));
                    for (uint32_t j = g.tid; j < nk; j += ET) {
                        if (a.out.kept_ids) a.out.kept_ids[size_t(row) * a.out.kept_cap + j] = int32_t(cand_id(cand[j]));
                        if (a.out.kept_p) a.out.kept_p[size_t(row) * a.out.kept_cap + j] = tail_p[j];
                    }
                }
            }
            g.sync();
            if (g.tid == 0) mbar_arrive(&hempty[h]);
        }
        return;
    }

    // =========================================================== stream
    const Group<ST> g{tid - 32, 1};
    const int lane = lane_id();
    constexpr int EPV = 16 / sizeof(T);           // elements per 128-bit vector
    constexpr int VPT = CH_ELEMS / EPV / ST;      // vectors per thread per stage (2 for f32, 1 for bf16)
    constexpr int QPT = VPT * EPV / 4;            // quads of 4 consecutive elements per thread per stage (2)
    static_assert(QPT == 2, "stage geometry");
    uint32_t it = 0;
    PenaltyTable pt;
    pt.bitmap = pen_mem, pt.slots = pen_mem + pen_words;
#ifdef WB_PHASE_TIMERS
    long long tacc[8] = {0, 0, 0, 0, 0, 0, 0, 0};  // setup, wait full, process, barrier, select, final, hand wait, total
    const long long t_begin = clock64();
#endif

    for (int k = 0; k < my_rows; ++k) {
        const int row = row_of(k);
        WB_T(t_s0);
        // ---- the row's settings
        bool greedy = false;
        uint32_t K;
        float inv_t = P.inv_t ? P.inv_t[row] : P.inv_t_scalar;
        if (sample) {
            greedy = P.greedy && P.greedy[row];
            const uint32_t tk = P.top_k ? uint32_t(max(P.top_k[row], 0)) : 0u;
            K = greedy ? 1u : ((tk > 0 && tk <= uint32_t(kStreamMaxK)) ? tk : uint32_t(a.level_k));
        } else {
            K = uint32_t(a.K);
        }
        if (K > n) K = n;
        const bool need_sum = !greedy;
        const float cexp = inv_t * kLog2e;
        pt.on = false;
        if (sample && P.hist && P.hist_len[row] > 0) {
            pt.rep = P.rep ? P.rep[row] : 1.f, pt.pres = P.pres ? P.pres[row] : 0.f, pt.freq = P.freq ? P.freq[row] : 0.f;
            pt.on = pt.rep != 1.f || pt.pres != 0.f || pt.freq != 0.f;
        }
        if (pt.on) {
            const int32_t* hrow = P.hist + size_t(row) * P.hist_stride;
            const int hl = min(P.hist_len[row], kMaxHist);
            int32_t hv[kMaxHist / ST];
#pragma unroll
            for (int j = 0; j < kMaxHist / ST; ++j) hv[j] = (g.tid + j * ST) < hl ? hrow[g.tid + j * ST] : -1;
            pt.clear(g.tid, ST, n);
            g.sync();
#pragma unroll
            for (int j = 0; j < kMaxHist / ST; ++j) pt.insert(hv[j], n);
        }
        if (g.tid == 0) sh->cnt = 0, sh->tau = 0ull, sh->tau_f = -INFINITY;
        g.sync();
        unsigned long long tau = 0ull;
        float tau_f = -INFINITY;
        float m_t = -INFINITY, s_t = 0.f;
        WB_T(t_s1);
        WB_ACC(0, t_s0, t_s1);

        for (uint32_t c = 0; c < n_chunks; ++c, ++it) {
            const uint32_t s = it % stages, use = it / stages;
            WB_T(t_w0);
            const bool ok = mbar_wait(&full[s], use & 1);
            WB_T(t_w1);
            WB_ACC(1, t_w0, t_w1);
            if (!ok) sh->abort_flag = 1;
            const uint4* vec = reinterpret_cast<const uint4*>(ring + size_t(s) * ch_bytes);
            float xv[8];
            uint32_t qid[QPT];
            bool qvalid[QPT];
            if (sizeof(T) == 4) {
                qid[0] = c * CH_ELEMS + 4 * g.tid, qid[1] = qid[0] + 4 * ST;
                qvalid[0] = qid[0] < n, qvalid[1] = qid[1] < n;
                const uint4 q0 = qvalid[0] && ok ? vec[g.tid] : make_uint4(0xff800000u, 0xff800000u, 0xff800000u, 0xff800000u);
                const uint4 q1 = qvalid[1] && ok ? vec[g.tid + ST] : make_uint4(0xff800000u, 0xff800000u, 0xff800000u, 0xff800000u);
                xv[0] = __uint_as_float(q0.x), xv[1] = __uint_as_float(q0.y), xv[2] = __uint_as_float(q0.z), xv[3] = __uint_as_float(q0.w);
                xv[4] = __uint_as_float(q1.x), xv[5] = __uint_as_float(q1.y), xv[6] = __uint_as_float(q1.z), xv[7] = __uint_as_float(q1.w);
            } else {
                qid[0] = c * CH_ELEMS + 8 * g.tid, qid[1] = qid[0] + 4;
                qvalid[0] = qvalid[1] = qid[0] < n;
                const uint4 q = qvalid[0] && ok ? vec[g.tid] : make_uint4(0xff80ff80u, 0xff80ff80u, 0xff80ff80u, 0xff80ff80u);
                xv[0] = __uint_as_float(q.x << 16), xv[1] = __uint_as_float(q.x & 0xffff0000u);
                xv[2] = __uint_as_float(q.y << 16), xv[3] = __uint_as_float(q.y & 0xffff0000u);
                xv[4] = __uint_as_float(q.z << 16), xv[5] = __uint_as_float(q.z & 0xffff0000u);
                xv[6] = __uint_as_float(q.w << 16), xv[7] = __uint_as_float(q.w & 0xffff0000u);
            }
            // NaN counts as -inf (as the reference's draft kernel does, kernels/spec_sample.hip:61,118)
#pragma unroll
            for (int j = 0; j < 8; ++j) xv[j] = fmaxf(xv[j], -INFINITY);
            // Every loaded register has been consumed above, so the shared-memory reads have completed (instructions issue
            // in order and the fmaxf had to wait for the data): only now may the producer overwrite the stage.
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);
            if (pt.on) {
                // history tokens among this thread's 8 elements: one bit each.  A lane loops over its own hits only, so
                // the warp pays for the most hits any lane has (one or two), not for all eight positions.
                uint32_t bits = (qvalid[0] ? pt.bits(qid[0], 4) : 0u) | ((qvalid[1] ? pt.bits(qid[1], 4) : 0u) << 4);
                while (bits) {
                    const int j = __ffs(bits) - 1;
                    bits &= bits - 1;
                    float x = xv[0];
#pragma unroll
                    for (int e = 1; e < 8; ++e) x = j == e ? xv[e] : x;
                    x = fmaxf(pt.apply(x, qid[j >> 2] + (j & 3)), -INFINITY);
#pragma unroll
                    for (int e = 0; e < 8; ++e) xv[e] = j == e ? x : xv[e];
                }
            }
            float vmax[QPT];
#pragma unroll
            for (int q = 0; q < QPT; ++q) vmax[q] = fmaxf(fmaxf(xv[q * 4], xv[q * 4 + 1]), fmaxf(xv[q * 4 + 2], xv[q * 4 + 3]));
            if (need_sum) {
                const float vm = fmaxf(vmax[0], vmax[1]);
                if (vm > m_t) {
                    s_t = (m_t == -INFINITY) ? 0.f : s_t * ex2_approx((m_t - vm) * cexp);
                    m_t = vm;
                }
                if (m_t != -INFINITY) {
                    float e[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) e[j] = ex2_approx((xv[j] - m_t) * cexp);
                    s_t += ((e[0] + e[1]) + (e[2] + e[3])) + ((e[4] + e[5]) + (e[6] + e[7]));
                }
            }
            const bool pass = (qvalid[0] && vmax[0] >= tau_f) || (qvalid[1] && vmax[1] >= tau_f);
            if (__ballot_sync(0xffffffffu, pass)) {
                uint32_t take = 0;
                unsigned long long comp[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    comp[j] = make_cand(key_of(xv[j]), qid[j >> 2] + (j & 3));
                    if (pass && qvalid[j >> 2] && comp[j] > tau) take |= 1u << j;
                }
                const uint32_t nl = __popc(take);
                const uint32_t incl = warp_scan_incl(nl);
                const uint32_t tot = __shfl_sync(0xffffffffu, incl, 31);
                if (tot) {
                    uint32_t base = 0;
                    if (lane == 31) base = atomicAdd(&sh->cnt, tot);
                    base = __shfl_sync(0xffffffffu, base, 31);
                    uint32_t pos = base + incl - nl;
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        if ((take >> j) & 1u) {
                            if (pos < BUF_CAP) buf[pos] = comp[j];
                            ++pos;
                        }
                }
            }
            // every stream thread is past the stage: does the buffer need a select?
            const bool last = c + 1 == n_chunks;
            WB_T(t_p1);
            WB_ACC(2, t_w1, t_p1);
            const bool flag = g.sync_or(ld_volatile(&sh->cnt) > BUF_TRIG || ld_volatile(&sh->abort_flag) != 0);
            WB_T(t_b1);
            WB_ACC(3, t_p1, t_b1);
            if (flag) {
                if (ld_volatile(&sh->abort_flag)) {
                    if (g.tid == 0) atomicExch(a.err, 3u);
                    return;
                }
                if (!last) {
                    const uint32_t cnt = sh->cnt;
                    const unsigned long long kth = select_kth<ST>(g, buf, cnt, K, hist, &sh->sel);
                    unsigned long long* stage = reinterpret_cast<unsigned long long*>(hist);
                    write_survivors<ST>(g, buf, cnt, kth, stage, kStreamMaxK, &sh->sel);
                    const uint32_t kept = sh->sel.wcnt;
                    for (uint32_t i = g.tid; i < kept; i += ST) buf[i] = stage[i];
                    if (g.tid == 0) sh->cnt = kept, sh->tau = kth, sh->tau_f = float_of_key(cand_key(kth));
                    g.sync();
                    tau = kth;
                    tau_f = float_of_key(cand_key(kth));
                }
                WB_T(t_c1);
                WB_ACC(4, t_b1, t_c1);
            }
        }
        WB_T(t_f0);
        // ---- the row is through: exact K candidates to the epilogue, with the row's max and normaliser
        {
            float wm = warp_max(m_t);
            double ds = (m_t == -INFINITY) ? 0.0 : double(s_t) * double(ex2_approx((m_t - wm) * cexp));
            ds = warp_sum(ds);
            if (lane == 0) sh->red_m[g.tid >> 5] = wm, sh->red_s[g.tid >> 5] = ds;
        }
        const int h = k % HAND;
        bool ok = true;
        WB_T(t_h0);
        if (g.tid == 0) ok = mbar_wait(&hempty[h], ((k / HAND) & 1) ^ 1);
        if (g.sync_or(!ok)) {
            if (g.tid == 0) atomicExch(a.err, 4u);
            return;
        }
        WB_T(t_h1);
        WB_ACC(6, t_h0, t_h1);
        const uint32_t cnt = sh->cnt;
        unsigned long long* dst = hand_c + size_t(h) * kStreamMaxK;
        uint32_t kept;
        if (cnt > K) {
            const unsigned long long kth = select_kth<ST>(g, buf, cnt, K, hist, &sh->sel);
            write_survivors<ST>(g, buf, cnt, kth, dst, kStreamMaxK, &sh->sel);
            kept = sh->sel.wcnt;
        } else {
            for (uint32_t i = g.tid; i < cnt; i += ST) dst[i] = buf[i];
            kept = cnt;
        }
        if (g.tid == 0) {
            float M = -INFINITY;
            for (int w = 0; w < SW; ++w) M = fmaxf(M, sh->red_m[w]);
            double S = 0;
            for (int w = 0; w < SW; ++w)
                if (sh->red_m[w] != -INFINITY) S += sh->red_s[w] * double(ex2_approx((sh->red_m[w] - M) * cexp));
            Hand hd;
            hd.row = row, hd.cnt = kept;
            if (need_sum) hd.m = M, hd.sum = float(S);
            else hd.m = 0.f, hd.sum = 0.f;
            sh->hand[h] = hd;
        }
        g.sync();
        if (g.tid == 0) mbar_arrive(&hfull[h]);
        WB_T(t_f1);
        WB_ACC(5, t_f0, t_f1);
    }
#ifdef WB_PHASE_TIMERS
    if (g.tid == 0) {
        tacc[7] = clock64() - t_begin;
        unsigned long long* dbg = reinterpret_cast<unsigned long long*>(a.err + 4);
        for (int i = 0; i < 8; ++i) atomicAdd(&dbg[i], (unsigned long long)tacc[i]);
    }
#endif
}

static size_t stream_fixed_smem(bool pen, int pen_words) {
    return size_t(BUF_CAP) * 8 + NBINS * 4 + size_t(HAND) * kStreamMaxK * 8 + 2 * (kStreamMaxK + 2 * EW) * 8 + (2 * 32 + 2 * HAND) * 8 +
           sizeof(StreamShared) + (pen ? size_t(pen_words) * 4 + kPenSlots * 4 : 0) + 128;
}

bool sample_stream_supported(const SelectArgs& a, int dtype) {
    const size_t es = dtype == 0 ? 4 : 2;
    if (reinterpret_cast<uintptr_t>(a.x) % 16 != 0 || (size_t(a.n) * es) % 16 != 0) return false;  // bulk copies need 16-byte rows
    if (a.mode == MODE_TOPK && a.K > kStreamMaxK) return false;
    const bool pen = a.mode == MODE_SAMPLE && a.prm.hist != nullptr;
    const int pen_words = pen ? ((a.n + 31) / 32 + 3) & ~3 : 0;
    const size_t ch_bytes = CH_ELEMS * es;
    return stream_fixed_smem(pen, pen_words) + 3 * ch_bytes <= 232448;
}

cudaError_t sample_stream_launch(const SelectArgs& a, int dtype, int sm_count, cudaStream_t st) {
    const size_t es = dtype == 0 ? 4 : 2;
    const bool pen = a.mode == MODE_SAMPLE && a.prm.hist != nullptr;
    const int pen_words = pen ? ((a.n + 31) / 32 + 3) & ~3 : 0;
    const int ch_bytes = int(CH_ELEMS * es);
    const size_t fixed = stream_fixed_smem(pen, pen_words);
    int stages = int((232448 - fixed) / ch_bytes);
    if (stages > 16) stages = 16;
    if (stages < 3) return cudaErrorInvalidConfiguration;
    const size_t smem = fixed + size_t(stages) * ch_bytes;
    const int grid = a.rows < sm_count ? a.rows : sm_count;
    cudaError_t e = cudaMemsetAsync(a.err, 0, 4, st);
    if (e != cudaSuccess) return e;
    if (dtype == 0) {
        e = cudaFuncSetAttribute(sample_stream_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
        if (e != cudaSuccess) return e;
        sample_stream_kernel<float><<<grid, NTHREADS, smem, st>>>(a, stages, pen_words, ch_bytes);
    } else {
        e = cudaFuncSetAttribute(sample_stream_kernel<uint16_t>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
        if (e != cudaSuccess) return e;
        sample_stream_kernel<uint16_t><<<grid, NTHREADS, smem, st>>>(a, stages, pen_words, ch_bytes);
    }
    return cudaGetLastError();
}

}  // namespace wb
