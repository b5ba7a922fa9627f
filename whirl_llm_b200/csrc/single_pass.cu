// The single-pass fused sampler: every logits row is read from HBM once, through a ring of shared-memory stages
// filled by bulk async copies (TMA, cp.async.bulk + mbarrier).
//
// One persistent CTA per SM, four roles that never meet at a CTA-wide barrier while rows stream:
//   producer (1 thread)   bulk copies of 16 KiB stages of the CTA's rows into the ring, running ahead across row
//                         boundaries.
//   stream warps (16)     consume the stages, two per iteration: the largest logit of what the lane just read (and, where
//                         the row needs its softmax normaliser, a running sum of exponentials), and a threshold test on
//                         it.  The few logits at or above the threshold are appended to the row's candidate log.
//   threshold keeper      (1 warp) for rows that keep at most 64 candidates: follows the log while it fills, holds the 64
//                         largest keys seen in sorted order (bitonic merges of 32-key batches) and raises the threshold to
//                         the K-th of them.
//   tail group (8 warps)  when a row is through: its exact K best, ranked (by counting for K <= 64, by one histogram over
//                         the keys' range for larger K: bucket_sort_top); top-k / top-p / min-p in f64, the draw and the
//                         row's outputs (one warp for rows of up to 256 candidates, while the others fetch the parameters
//                         of the row after the next and prepare its penalties; the whole group for larger rows).
// The roles work on alternating row slots (two logs, two word maps), so the tail of one row overlaps the streaming of the
// next.
//
// Thresholds.  An element is dropped only when it is below a value that at least K elements of the same row reach, so
// the K best are always in the log and the final select over the log is exact.
//   * First threshold (the stream warps' one meeting per row, after their first iteration, whose logits are still in
//     registers and are tested afterwards): every warp publishes its largest lane maxima in descending order, and every
//     warp finds the largest 20-bit key prefix that rank0 of the published keys reach.  For K <= 64, rank0 = K: a valid
//     bound, close to the K-th largest logit read so far.  For larger K, rank0 is a guess (first_rank): the rank that,
//     scaled from the first iteration to the whole row, leaves K candidates 3.5 standard deviations below the expected
//     count.  A row whose guess leaves fewer than K logged candidates is done again by the multi-pass kernel; a row
//     whose K on its length would need a rank beyond what the warps publish goes there from the start.
//   * Later thresholds: the keeper warp (K <= 64); for larger K the tail group, which selects the exact K-th largest of
//     the log when the log has grown enough (marked entries, which carry raw logits, count as absent there).
//
// Penalties.  A raw logit of a history token must count nowhere.  The tail group builds, a row ahead, a bit map of the
// 16-byte words (4 f32 / 8 bf16 logits) that hold a history token.  Nothing of a row is ever fetched a second time from
// global memory: random 16-byte reads at that rate are more than the memory can serve while it streams.
//   * A row that needs no normaliser and whose penalties can only lower a logit (the usual case): a word with a history
//     token counts for no bound, and one of its logits is looked at only when it passes the threshold raw; it is then
//     logged with a mark, and the tail group applies the penalty to the few marked entries before it ranks the log
//     (their counts: an f32 row's from the table of its history, built while it streams; a bf16 row's, which streams in
//     half the time, from a scan of the history).
//   * Any other penalised row: the stream warps put the marked words aside (from their registers into a side buffer in
//     global memory that stays in L2) and see -inf instead; the tail group, which has built the table of the row's
//     distinct history tokens with their counts meanwhile, brings them in at the end of the row, history tokens with
//     their penalty, the others as they are.
//
// Every wait has a budget (SelectArgs::wait_limit).  A role whose wait runs out records which in the error word and
// returns; the rows it leaves without an answer keep the status "pending" and are done by the multi-pass kernel.
//
// It replaces the reference's topk_rows kernel (seven passes over the row, kernels/shared/sample_cand_topk_rows.h:11-98),
// the candidate download, and the host filter and draw (src/sampling/sampler.cpp:15-147).
#include <type_traits>

#include "kernels.h"
#include "penalty.cuh"
#include "select_smem.cuh"
#include "tail.cuh"

namespace wb {

constexpr int Q_SW = 16;                 // stream warps
constexpr int Q_ST = Q_SW * 32;
constexpr int Q_TW = 8;                  // tail warps
constexpr int Q_TT = Q_TW * 32;
constexpr int Q_THREADS = 32 + Q_ST + Q_TT + 32;  // producer warp, stream warps, tail group, threshold keeper
constexpr int Q_SB = 16384;              // bytes per ring stage
constexpr int Q_SQ = Q_SB / 16;          // 128-bit words per stage
constexpr int Q_MAXSTAGES = 8;
constexpr int Q_NS = 2;                  // ring stages per iteration of a stream warp
constexpr int Q_L = 2944;                // candidate log entries per row slot (sized so that penalised f32 rows of 262,144
                                         // logits leave room for seven ring stages)
constexpr int Q_RED = Q_SW + Q_TW;       // partial (max, exponent, sum) triples per row: stream warps, then tail warps
constexpr int Q_PT = Q_TT - 32;          // tail threads that prepare penalties (all tail warps but the first)
static_assert(Q_SQ == 2 * Q_ST, "two 128-bit words per stream thread and stage");

// What the roles need to know about a row, fetched once (by one tail warp, a row ahead) into shared memory: while the rows
// stream a load from global memory takes microseconds, so nobody on the path of a row reads parameters from there.
struct QRow {
    uint32_t rank0;          // first_rank of the row
    int32_t row;             // index in the batch
    uint32_t K;              // candidates wanted
    uint32_t top_k;
    uint32_t flags;          // QF_*
    float inv_t;
    float rep, pres, freq;
    int32_t hist_len;        // clamped; 0 without penalties
    double top_p, min_p, u;
    unsigned long long race_key;
};
// QF_LAZY: penalised, no normaliser wanted, and the penalties can only lower a logit (repetition >= 1, presence and
// frequency >= 0): a history token then matters only if its RAW logit passes the threshold, which the stream sees.
enum : uint32_t { QF_NO_SUM = 1u, QF_PEN = 2u, QF_GREEDY = 4u, QF_LAZY = 8u };

constexpr int Q_TOP = 16;       // lane maxima a stream warp publishes for a row's first threshold (the first 8 for a small-K row)
constexpr int Q_SMALL_K = 64;   // rows keeping at most this many candidates: exact first threshold, threshold kept by the keeper warp
constexpr float Q_GUESS_Z = 3.5f;  // standard deviations between a guessed first threshold's expected count and K
constexpr int Q_RANK_MAX = 192; // largest rank among the published maxima a first threshold may be taken at
static_assert(Q_SW * Q_TOP == 256, "eight published keys per lane");

// The rank, among the logits of a row's first iteration, that the row's first threshold is taken at.  Small K: K itself
// (the K-th largest of a part of the row is a valid bound).  Larger K: a guess - the rank that, scaled from the first
// iteration (it0 logits) to the whole row (n logits), leaves K candidates 3.5 standard deviations below the expected
// count (for K = 1024 on 262,144 f32 logits: rank 59, about 2000 candidates expected, between the K wanted and the log's
// 2944 places with 3.5 deviations to spare on either side; the stream warps publish one maximum per lane, so a lane
// holding two of the first-ranked logits makes the count a few per cent larger).  A row that ends with fewer than K logged candidates is redone by the multi-pass kernel.
__device__ __forceinline__ uint32_t first_rank(uint32_t K, uint32_t n, uint32_t it0) {
    if (K <= uint32_t(Q_SMALL_K)) return K;
    const float x = float(K) * float(it0 < n ? it0 : n) / float(n);
    const float r = 0.5f * (Q_GUESS_Z + sqrtf(Q_GUESS_Z * Q_GUESS_Z + 4.f * x));
    return uint32_t(ceilf(r * r));
}

// How far the log has to grow past its size at the last refinement (0: none yet) before the tail group refines the
// threshold again.  The first refinement waits for twice the candidates wanted (a quarter of the log at least): until then
// the log is no burden.  Once the log has needed one, the next ones follow closely, so that a row whose first threshold
// was guessed low is cut back several times before its log is full.
__device__ __forceinline__ uint32_t refine_step(uint32_t K, uint32_t last) {
    if (last == 0) return 2 * K > uint32_t(Q_L) / 4 ? 2 * K : uint32_t(Q_L) / 4;
    return K / 4 > 128u ? K / 4 : 128u;
}

struct QSlot {
    unsigned long long tau;  // current threshold candidate; elements must beat it to be logged
    uint32_t cnt;            // log entries reserved so far (may exceed Q_L: overflow); bit 31: a NaN poisoned a sum
    uint32_t side_cnt;       // words put aside in the side buffer (penalised rows that need their normaliser)
    uint32_t done_warps;     // stream warps that are through the row (the threshold keeper watches this, then closes the row too)
    QRow cfg;
    float red_m[Q_RED];
    float red_e[Q_RED];
    double red_s[Q_RED];
    alignas(16) uint32_t wtop[Q_SW * Q_TOP];  // per stream warp: its Q_TOP largest lane maxima of the row's first iteration, descending
};

constexpr int Q_MAXR = 512;  // rows per CTA and launch

// The word map's layout: bit `lane` of map word ((it * Q_SW + warp) * 4 + j) is the 128-bit word the stream thread
// (warp, lane) reads as its j-th of iteration it, so one 128-bit shared-memory load per warp and iteration gives the
// thread its four bits.  (Needs two stages per iteration.)
static_assert(Q_NS == 2, "the word map is laid out for two stages per iteration");
__device__ __forceinline__ uint32_t gbm_word_of(uint32_t wq) {
    const uint32_t it = wq / (2 * Q_SQ), in = wq % (2 * Q_SQ);
    return ((it * Q_SW + (in % Q_ST) / 32) << 2) | (in / Q_ST);
}

struct QShared {
    QSlot slot[2];
    SelScratch sel;
    TailOut res;
    uint32_t flag[4];
    uint32_t lcount[32];      // building the row list: rows kept per warp
    int32_t n_list;
    int32_t rlist[Q_MAXR];    // the CTA's rows, in order (rows left to the multi-pass kernel are not in it)
};

__device__ __forceinline__ unsigned long long ldv_u64(const unsigned long long* p) {
    return *reinterpret_cast<const volatile unsigned long long*>(p);
}
__device__ __forceinline__ uint32_t ldv_u32(const uint32_t* p) { return *reinterpret_cast<const volatile uint32_t*>(p); }

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
    int cnt = 0, n_redo = 0;
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
            const bool redo = st == ROW_RETRY || st == ROW_OPEN_TAIL || st == ROW_PENDING;
            const bool take = redo || st == ROW_LARGE_K || st == ROW_ESCALATE;
            const uint32_t bal = __ballot_sync(0xffffffffu, take);
            if (take) a.fin_list[cnt + __popc(bal & ((1u << lane) - 1))] = r | (redo ? (1 << 30) : 0);
            cnt += __popc(bal);
            n_redo += __popc(__ballot_sync(0xffffffffu, redo));
        }
    }
    if (lane == 0) {
        a.fin_counts[1] = cnt, a.fin_counts[2] = 0;
        if (a.out.counters && n_redo) atomicAdd(&a.out.counters[WHIRL_CNT_REDO], uint32_t(n_redo));
    }
}

// ---- the table of a row's distinct history tokens: (token + 1) | count << 19, open addressing, kPenSlots words
__device__ __forceinline__ void pen_table_insert(uint32_t* pslots, uint32_t t, uint32_t c) {
    const uint32_t tag = t + 1;
    uint32_t hsh = PenaltyTable::hash(t);
#pragma unroll 1
    for (int probe = 0; probe < kPenSlots; ++probe) {
        uint32_t old = ldv_u32(&pslots[hsh]);
        if (old == 0) old = atomicCAS(&pslots[hsh], 0u, tag | (c << kPenIdBits));
        if (old == 0) return;
        if ((old & kPenMaxV) == tag) {
            atomicAdd(&pslots[hsh], c << kPenIdBits);
            return;
        }
        hsh = (hsh + 1) & (kPenSlots - 1);
    }
}
// occurrences of token id in the history (0: not a history token)
__device__ __forceinline__ uint32_t pen_table_count(const uint32_t* pslots, uint32_t id) {
    const uint32_t tag = id + 1;
    uint32_t hsh = PenaltyTable::hash(id);
#pragma unroll 1
    for (int probe = 0; probe < kPenSlots; ++probe) {
        const uint32_t sv = pslots[hsh];
        if (sv == 0) return 0u;
        if ((sv & kPenMaxV) == tag) return sv >> kPenIdBits;
        hsh = (hsh + 1) & (kPenSlots - 1);
    }
    return 0u;
}

// One candidate into a row's log, if it beats the threshold (x is a number: the caller has compared it).
// unsure: the logit comes from a word that holds a history token and is logged raw; bit 31 of the entry's low half (always
// set otherwise: it is ~id) is cleared to say so, and the tail group looks the token up before it ranks the log.
__device__ __forceinline__ void log_append(QSlot* sl, unsigned long long* log, float x, uint32_t id, unsigned long long tau,
                                           bool unsure = false) {
    const uint32_t u = __float_as_uint(x + 0.0f);  // -0 + +0 = +0: the two zeros share a key
    const uint32_t key = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    unsigned long long cnd = make_cand(key, id);
    if (cnd > tau) {
        if (unsure) cnd &= ~0x80000000ull;
        const uint32_t pos = atomicAdd(&sl->cnt, 1u) & 0x7fffffffu;
        if (pos < uint32_t(Q_L)) log[pos] = cnd;
    }
}
__device__ __forceinline__ float penalised(float l, uint32_t cnt, float rep, float pres, float freq) {
    l = (l > 0.f) ? __fdiv_rn(l, rep) : __fmul_rn(l, rep);
    return __fsub_rn(l, __fadd_rn(pres, __fmul_rn(freq, float(cnt))));
}

// A 128-bit word w (place wq in the row) that was kept out of the stream comes into its row: history tokens with their
// penalty, the others as they are: into the caller's running maximum / sum, and into the log when they can be among the
// K best.
struct JoinCtx {
    const uint32_t* pslots;
    QSlot* sl;
    unsigned long long* log;
    float rep, pres, freq, cexp;
    bool no_sum;
    float m_t, e_t, s_t;
    unsigned long long tau;
    float tau_f;
};
template <int VE>
__device__ __forceinline__ void join_word(JoinCtx& c, uint32_t wq, uint4 w) {
    const uint32_t w4[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int j = 0; j < VE; ++j) {
        const uint32_t cnt = pen_table_count(c.pslots, wq * VE + j);
        float l;
        if (VE == 4) l = __uint_as_float(w4[j]);
        else l = __uint_as_float((j & 1) ? (w4[j >> 1] & 0xffff0000u) : (w4[j >> 1] << 16));
        const float x = cnt ? penalised(l, cnt, c.rep, c.pres, c.freq) : l;
        if (!c.no_sum) {
            if (x > c.m_t) {
                const float ne = ceilf(x * c.cexp);
                c.s_t = (c.m_t == -INFINITY) ? 0.f : c.s_t * ex2_approx(c.e_t - ne);
                c.e_t = ne, c.m_t = x;
            }
            if (c.m_t != -INFINITY) c.s_t += ex2_approx(fmaf(x, c.cexp, -c.e_t));
        }
        if (x >= c.tau_f) log_append(c.sl, c.log, x, wq * VE + j, c.tau);
    }
}

// The largest of N floats by three-input maxima (max.f32 with three operands, sm_100: comparisons and maxima share the
// half-rate ALU pipe, which is what the stream loop runs out of first).  Like fmaxf, it skips NaN.
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
template <int N>
__device__ __forceinline__ float max_of(const float* v) {
    float t[N];
#pragma unroll
    for (int i = 0; i < N; ++i) t[i] = v[i];
    int n = N;
#pragma unroll
    for (int lvl = 0; lvl < 4; ++lvl) {  // (3^4 >= 32)
        const int m = (n + 2) / 3;
#pragma unroll
        for (int i = 0; i < (N + 2) / 3; ++i) {
            if (i < m) {
                const int b = 3 * i;
                t[i] = b + 2 < n ? fmax3(t[b], t[b + 1], t[b + 2]) : (b + 1 < n ? fmaxf(t[b], t[b + 1]) : t[b]);
            }
        }
        n = m;
    }
    return t[0];
}

// Two bf16 maxima in one instruction (max.bf16x2 skips NaN like fmaxf): a bf16 row has twice the logits per byte, and
// widening each of them to f32 before comparing would cost the stream warps three times the ALU work of an f32 row.
__device__ __forceinline__ uint32_t bmax2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("max.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ float bmax2_wide(uint32_t m) { return fmaxf(__uint_as_float(m << 16), __uint_as_float(m & 0xffff0000u)); }
// The largest logit of NWORDS 128-bit words of a row of T.
template <typename T, int NWORDS>
__device__ __forceinline__ float words_max(const uint4* w) {
    if (sizeof(T) == 4) {
        float x[NWORDS * 4];
#pragma unroll
        for (int i = 0; i < NWORDS; ++i)
            x[4 * i] = __uint_as_float(w[i].x), x[4 * i + 1] = __uint_as_float(w[i].y), x[4 * i + 2] = __uint_as_float(w[i].z),
                  x[4 * i + 3] = __uint_as_float(w[i].w);
        return max_of<NWORDS * 4>(x);
    } else {
        uint32_t m[NWORDS];
#pragma unroll
        for (int i = 0; i < NWORDS; ++i) m[i] = bmax2(bmax2(w[i].x, w[i].y), bmax2(w[i].z, w[i].w));
#pragma unroll
        for (int s = 1; s < NWORDS; s <<= 1)
#pragma unroll
            for (int i = 0; i + s < NWORDS; i += 2 * s) m[i] = bmax2(m[i], m[i + s]);
        return bmax2_wide(m[0]);
    }
}

// ---- the small-K threshold keeper (a warp of its own, while a row streams)
// 32 ordering keys, one per lane, into descending order over the lanes (a bitonic network of shuffles).
__device__ __forceinline__ uint32_t warp_sort_desc(uint32_t x, int lane) {
#pragma unroll
    for (int k = 2; k <= 32; k <<= 1) {
#pragma unroll
        for (int j = k >> 1; j > 0; j >>= 1) {
            const uint32_t o = __shfl_xor_sync(0xffffffffu, x, j);
            const bool take_max = ((lane & j) == 0) == ((lane & k) == 0);
            x = take_max ? max(x, o) : min(x, o);
        }
    }
    return x;
}
// a bitonic sequence over the lanes into descending order
__device__ __forceinline__ uint32_t warp_merge_desc(uint32_t x, int lane) {
#pragma unroll
    for (int j = 16; j > 0; j >>= 1) {
        const uint32_t o = __shfl_xor_sync(0xffffffffu, x, j);
        x = (lane & j) == 0 ? max(x, o) : min(x, o);
    }
    return x;
}

// Rows that want at most 64 candidates: one warp follows the row's log while the stream warps fill it, keeps the 64
// largest keys it has seen in sorted order (two per lane) and raises the row's threshold to the K-th of them.  That is
// the K-th largest logit of the part of the row streamed so far, short of entries it skips - not written yet when it
// came by, or logged raw from a word that holds a history token - and the K-th largest of any subset of a row is a valid
// lower bound.  Returns 0 when every stream warp is through the row, 2 when the wait ran out.
static __device__ __noinline__ uint32_t keep_threshold_small_k(QSlot* sl, const unsigned long long* log, uint32_t K, uint32_t limit) {
    const int lane = lane_id();
    uint32_t top_a = 0u, top_b = 0u;  // ranks lane and 32 + lane
    uint32_t done = 0, tau_key = 0;
#pragma unroll 1
    for (uint32_t spin = 0; spin < 4 * limit; ++spin) {
        uint32_t through = 0, c = 0;
        if (lane == 0) {
            through = ldv_u32(&sl->done_warps) == uint32_t(Q_SW) ? 1u : 0u;
            c = ldv_u32(&sl->cnt) & 0x7fffffffu;
        }
        through = __shfl_sync(0xffffffffu, through, 0);
        c = __shfl_sync(0xffffffffu, c, 0);
        if (through) return 0u;  // (a threshold is of no use any more)
        c = c < uint32_t(Q_L) ? c : uint32_t(Q_L);
        const uint32_t pending = c - done;
        if (pending >= 8u) {
            const uint32_t nb = pending < 32u ? pending : 32u;
            const unsigned long long e = uint32_t(lane) < nb ? ldv_u64(&log[done + lane]) : 0ull;
            uint32_t v = (e & 0x80000000ull) ? cand_key(e) : 0u;  // (0: not written yet, or logged raw)
            done += nb;
            if (!__any_sync(0xffffffffu, v > __shfl_sync(0xffffffffu, top_b, 31))) continue;  // nothing enters the 64
            v = warp_sort_desc(v, lane);
            // the 32 largest of (ranks 32..63, the batch), then the two halves of (ranks 0..31, those)
            const uint32_t d = warp_merge_desc(max(top_b, __shfl_sync(0xffffffffu, v, 31 - lane)), lane);
            const uint32_t dr = __shfl_sync(0xffffffffu, d, 31 - lane);
            const uint32_t hi = max(top_a, dr), lo = min(top_a, dr);
            top_a = warp_merge_desc(hi, lane);
            top_b = warp_merge_desc(lo, lane);
            const uint32_t kk = K <= 32u ? __shfl_sync(0xffffffffu, top_a, int(K) - 1) : __shfl_sync(0xffffffffu, top_b, int(K) - 33);
            if (kk > tau_key) {
                tau_key = kk;
                // (a plain compare and store, as the stream warps do: a lost update leaves another valid bound)
                if (lane == 0 && ((unsigned long long)kk << 32) > ldv_u64(&sl->tau))
                    *reinterpret_cast<volatile unsigned long long*>(&sl->tau) = (unsigned long long)kk << 32;
            }
            continue;
        }
        __nanosleep(100);
    }
    return 2u;
}


template <typename T>
__global__ void __launch_bounds__(Q_THREADS, 1) single_pass_kernel(SelectArgs a, int stages, int gbm_words, int max_k, int hand_k) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int VE = 16 / int(sizeof(T));      // logits per 128-bit word
    constexpr bool LAZY_TABLE = sizeof(T) == 4;  // rows that only mark log entries: the history's table is built while they stream
    uint8_t* ring = smem;                                                                // stages * Q_SB
    unsigned long long* logs = reinterpret_cast<unsigned long long*>(ring + size_t(stages) * Q_SB);  // 2 * Q_L
    uint32_t* hist = reinterpret_cast<uint32_t*>(logs + 2 * Q_L);                        // SEL_BINS
    // (hand, tail_p, tail_q serve rows of up to hand_k candidates; a row of more finds the room in its own log, see below)
    unsigned long long* hand = reinterpret_cast<unsigned long long*>(hist + SEL_BINS);   // hand_k: a row's candidates
    double* tail_p = reinterpret_cast<double*>(hand + hand_k);                           // hand_k + 2 * Q_TW
    double* tail_q = tail_p + hand_k + 2 * Q_TW;
    uint64_t* bars = reinterpret_cast<uint64_t*>(tail_q + hand_k + 2 * Q_TW);            // 2 * Q_MAXSTAGES + 6
    QShared* sh = reinterpret_cast<QShared*>(bars + 2 * Q_MAXSTAGES + 6);
    uint32_t* gbms = reinterpret_cast<uint32_t*>((reinterpret_cast<uintptr_t>(sh + 1) + 15) & ~uintptr_t(15));  // 2 * gbm_words
    uint32_t* pslots = gbms + 2 * size_t(gbm_words);                                     // kPenSlots (only with penalties)
    uint64_t *full = bars, *empty = bars + Q_MAXSTAGES;
    // per slot: the slot is the row's / every stream warp is through the row / every stream warp has named its first bound
    uint64_t *boot_done = bars + 2 * Q_MAXSTAGES, *closed = boot_done + 2, *head_done = boot_done + 4;

    const int tid = threadIdx.x, warp = tid >> 5;
    // (the kernel after this one in the stream, if it was launched as a programmatic dependent, may bring its CTAs up as
    // this kernel's CTAs leave; it waits for this whole grid before it reads anything)
    asm volatile("griddepcontrol.launch_dependents;");
    const uint32_t n = uint32_t(a.n);
    const int n_rows = a.row_count ? min(*a.row_count, a.rows) : a.rows;
    const int my_rows = n_rows > int(blockIdx.x) ? (n_rows - int(blockIdx.x) + int(gridDim.x) - 1) / int(gridDim.x) : 0;
    const uint32_t row_q = n / VE;  // 128-bit words per row (rows are 16-byte multiples)
    const uint32_t n_chunks = (row_q + Q_SQ - 1) / Q_SQ;
    const size_t row_bytes = size_t(n) * sizeof(T);
    const bool sample = a.mode == MODE_SAMPLE;
    const RowParams& P = a.prm;
    // the CTA's side buffers (one per slot): kMaxHist words and their places in the row
    uint8_t* const side_base = static_cast<uint8_t*>(a.side_ws) + size_t(blockIdx.x) * 2 * kMaxHist * 20;
    auto side_w = [&](int p) { return reinterpret_cast<uint4*>(side_base + size_t(p) * kMaxHist * 20); };
    auto side_q = [&](int p) { return reinterpret_cast<uint32_t*>(side_base + size_t(p) * kMaxHist * 20 + size_t(kMaxHist) * 16); };

    if (tid == 0) {
        for (int s = 0; s < stages; ++s) mbar_init(&full[s], 1), mbar_init(&empty[s], Q_SW);
        for (int p = 0; p < 2; ++p) mbar_init(&boot_done[p], 1), mbar_init(&closed[p], Q_SW + 1), mbar_init(&head_done[p], Q_SW);
        mbar_fence_init();
    }
    // The first two rows' parameters and histories are asked for now (into L2): the tail group reads them as soon as the
    // rows are listed, and the stream warps cannot start before it has.
    if (sample && !a.row_list && tid < 2 * 160) {
        const int which = tid / 160, t = tid % 160;
        const int r = int(blockIdx.x) + which * int(gridDim.x);
        if (which < my_rows) {
            const void* ptr = nullptr;
            if (t < 128) {
                if (P.hist && gbm_words && int64_t(t) * 32 < P.hist_stride) ptr = P.hist + size_t(r) * P.hist_stride + size_t(t) * 32;
            } else {
                switch (t - 128) {
                    case 0: ptr = P.inv_t ? P.inv_t + r : nullptr; break;
                    case 1: ptr = P.top_p ? P.top_p + r : nullptr; break;
                    case 2: ptr = P.min_p ? P.min_p + r : nullptr; break;
                    case 3: ptr = P.u ? P.u + r : nullptr; break;
                    case 4: ptr = P.race_key ? P.race_key + r : nullptr; break;
                    case 5: ptr = P.hist_len ? P.hist_len + r : nullptr; break;
                    case 6: ptr = P.rep ? P.rep + r : nullptr; break;
                    case 7: ptr = P.pres ? P.pres + r : nullptr; break;
                    case 8: ptr = P.freq ? P.freq + r : nullptr; break;
                    default: break;
                }
            }
            if (ptr) asm volatile("prefetch.global.L2 [%0];" ::"l"(ptr));
        }
    }
    // (the tail group's own indices, for the lambdas below; they mean nothing in the other warps)
    const Group<Q_TT> t_g{tid - 32 - Q_ST, 1};
    const Group<Q_PT> t_gp{t_g.tid - 32, 2};  // the tail warps but the first
    const int t_lane = lane_id(), t_tw = t_g.tid >> 5;
    const bool boot_warp = warp > Q_SW + 1 && warp <= Q_SW + Q_TW;  // tail warps 1 ..

    // ---- a row's parameters come into the slot it will stream through (one warp, every t_lane fetching one of them)
    auto fetch_params = [&](int p, int row) {
        QSlot* sl = &sh->slot[p];
        // t_lane: 0 inv_t, 1 top_k, 2 greedy, 3 top_p, 4 min_p, 5 u, 6 race_key, 7 hist_len, 8 rep, 9 pres, 10 freq
        unsigned long long v = 0ull;
        if (t_lane == 0) v = __float_as_uint(P.inv_t ? P.inv_t[row] : P.inv_t_scalar);
        if (sample) {
            if (t_lane == 1) v = P.top_k ? uint32_t(max(P.top_k[row], 0)) : 0u;
            if (t_lane == 2) v = (P.greedy && P.greedy[row]) ? 1u : 0u;
            if (t_lane == 3) v = (unsigned long long)__double_as_longlong(P.top_p ? P.top_p[row] : 1.0);
            if (t_lane == 4) v = (unsigned long long)__double_as_longlong(P.min_p ? P.min_p[row] : 0.0);
            if (t_lane == 5) v = (unsigned long long)__double_as_longlong(P.u ? P.u[row] : 0.0);
            if (t_lane == 6) v = P.race_key ? P.race_key[row] : 0ull;
            if (t_lane == 7 && gbm_words) v = uint32_t(hist_len_of(P, row));
            if (t_lane == 8) v = __float_as_uint(P.rep ? P.rep[row] : 1.f);
            if (t_lane == 9) v = __float_as_uint(P.pres ? P.pres[row] : 0.f);
            if (t_lane == 10) v = __float_as_uint(P.freq ? P.freq[row] : 0.f);
        }
        const float inv_t = __uint_as_float(uint32_t(__shfl_sync(0xffffffffu, v, 0)));
        const uint32_t top_k = uint32_t(__shfl_sync(0xffffffffu, v, 1));
        const bool greedy = __shfl_sync(0xffffffffu, v, 2) != 0;
        const unsigned long long top_p = __shfl_sync(0xffffffffu, v, 3), min_p = __shfl_sync(0xffffffffu, v, 4);
        const unsigned long long u = __shfl_sync(0xffffffffu, v, 5), race_key = __shfl_sync(0xffffffffu, v, 6);
        const int hist_len = int(uint32_t(__shfl_sync(0xffffffffu, v, 7)));
        const float rep = sample ? __uint_as_float(uint32_t(__shfl_sync(0xffffffffu, v, 8))) : 1.f;
        const float pres = __uint_as_float(uint32_t(__shfl_sync(0xffffffffu, v, 9)));
        const float freq = __uint_as_float(uint32_t(__shfl_sync(0xffffffffu, v, 10)));
        if (t_lane == 0) {
            QRow c;
            c.row = row, c.top_k = top_k, c.inv_t = inv_t;
            // candidates wanted: the row's own top_k when it fits, else the first level's
            uint32_t K = sample ? (greedy ? 1u : ((top_k > 0 && top_k <= uint32_t(max_k)) ? top_k : uint32_t(min(a.level_k, max_k)))) : uint32_t(a.K);
            c.K = K > n ? n : K;
            c.rank0 = first_rank(c.K, n, uint32_t(Q_NS * Q_SQ * VE));
            // Rows whose kept set is closed by their own top_k need no softmax normaliser: every probability the filter
            // compares is a ratio inside the candidate set, so the row sum cancels.  When the caller does not ask for the
            // row statistics either, the stream warps skip the exponentials and the tail normalises over the candidates.
            const bool no_sum = sample && (greedy || (!a.out.stats && P.top_k && top_k >= 1 && top_k <= uint32_t(max_k) && top_k <= n));
            const bool pen = sample && hist_len > 0 && (rep != 1.f || pres != 0.f || freq != 0.f);
            const bool lazy = pen && no_sum && rep >= 1.f && pres >= 0.f && freq >= 0.f;
            c.flags = (no_sum ? QF_NO_SUM : 0u) | (pen ? QF_PEN : 0u) | (greedy ? QF_GREEDY : 0u) | (lazy ? QF_LAZY : 0u);
            c.rep = rep, c.pres = pres, c.freq = freq, c.hist_len = pen ? hist_len : 0;
            c.top_p = __longlong_as_double((long long)top_p), c.min_p = __longlong_as_double((long long)min_p);
            c.u = __longlong_as_double((long long)u), c.race_key = race_key;
            sl->cfg = c;
        }
        __syncwarp();
    };

    // ---- a slot becomes a row's (the tail warps but the first; the slot's log and word map are zero): parameters and the
    // map of the words that hold a history token (slot_prepare), then the stream warps are told (slot_release)
    auto slot_prepare = [&](int p, int row) {
        QSlot* sl = &sh->slot[p];
        if (t_tw == 1) fetch_params(p, row);
        t_gp.sync();
        const int hl = sl->cfg.hist_len;  // (0 without penalties)
        if (hl > 0) {
            uint32_t* gbm = gbms + size_t(p) * gbm_words;
            const int32_t* h = P.hist + size_t(row) * P.hist_stride;
            constexpr int HB = (kMaxHist + Q_PT - 1) / Q_PT;
            int32_t hv[HB];  // (all loads first: one trip to memory)
#pragma unroll
            for (int u = 0; u < HB; ++u) hv[u] = (u * Q_PT + t_gp.tid) < hl ? h[u * Q_PT + t_gp.tid] : -1;
#pragma unroll
            for (int u = 0; u < HB; ++u) {
                const uint32_t t = uint32_t(hv[u]);
                if (t < n) {
                    const uint32_t wd = gbm_word_of(t / VE), bit = 1u << ((t / VE) & 31);
                    if (!(ldv_u32(&gbm[wd]) & bit)) atomicOr(&gbm[wd], bit);
                }
            }
            t_gp.sync();
        }
    };
    auto slot_release = [&](int p) {
        QSlot* sl = &sh->slot[p];
        if (t_gp.tid == 0) {
            sl->tau = 0ull;
            sl->cnt = 0;
            sl->side_cnt = 0;
            sl->done_warps = 0;
            for (int w = Q_SW; w < Q_RED; ++w) sl->red_m[w] = -INFINITY, sl->red_e[w] = -INFINITY, sl->red_s[w] = 0.0;
            mbar_arrive(&boot_done[p]);
        }
    };
    auto slot_boot = [&](int p, int row) {
        slot_prepare(p, row);
        slot_release(p);
    };

    for (int i = tid; i < 2 * Q_L; i += Q_THREADS) logs[i] = 0ull;
    for (int i = tid; i < 2 * gbm_words; i += Q_THREADS) gbms[i] = 0u;
    __syncthreads();  // (barriers, logs and word maps are ready)
    // The first slot is prepared while the rows are listed, for the row the list will most likely start with (the CTA's
    // first): the stream warps cannot start before it is.
    bool early_boot = false;
    if (sample && !a.row_list && my_rows > 0 && boot_warp) {
        slot_prepare(0, int(blockIdx.x));
        early_boot = true;
    }
    // ---- the CTA's rows: rows blockIdx.x, + gridDim.x, ...; rows whose top_k is above this launch's limit are left to the
    // multi-pass kernel (marked here, not listed).  my_rows <= Q_MAXR <= Q_THREADS: one row per thread.
    {
        const int k = tid;
        int row = -1;
        bool keep = false;
        if (k < my_rows) {
            const int li = int(blockIdx.x) + k * int(gridDim.x);
            row = a.row_list ? a.row_list[li] : li;
            keep = true;
            // rows whose top_k is above this launch's limit, and rows whose first threshold would have to be taken deeper
            // among the first iteration's maxima than the stream warps publish (a large K on a short row)
            uint32_t K = uint32_t(a.K);
            if (sample) {
                const int tk = P.top_k ? P.top_k[row] : 0;
                const bool greedy = P.greedy && P.greedy[row];
                if (!greedy && tk > max_k) keep = false;
                K = greedy ? 1u : ((tk > 0 && tk <= max_k) ? uint32_t(tk) : uint32_t(min(a.level_k, max_k)));
            }
            K = K > n ? n : K;
            if (first_rank(K, n, uint32_t(Q_NS * Q_SQ * VE)) > uint32_t(Q_RANK_MAX)) keep = false;
            // (a listed row stays "pending" until it has its answer: a role that gives up leaves it so, and the multi-pass
            // kernel takes it)
            if (a.out.status) a.out.status[row] = keep ? ROW_PENDING : ROW_LARGE_K;
        }
        const uint32_t bal = __ballot_sync(0xffffffffu, keep);
        if ((tid & 31) == 0 && warp < 32) sh->lcount[warp] = uint32_t(__popc(bal));
        __syncthreads();
        uint32_t before = 0;
        for (int w = 0; w < warp && w < 32; ++w) before += sh->lcount[w];
        if (keep) sh->rlist[before + __popc(bal & ((1u << (tid & 31)) - 1))] = row;
        if (tid == 0) {
            uint32_t tot = 0;
            for (int w = 0; w < (Q_THREADS + 31) / 32 && w < 32; ++w) tot += sh->lcount[w];
            sh->n_list = int32_t(tot);
        }
    }
    __syncthreads();
    const int n_list = sh->n_list;
    const int32_t* rlist = sh->rlist;
    if (n_list == 0) {
        if (a.fin_list) {
            __threadfence();
            __syncthreads();
            if (tid < 32) list_leftovers(a);
        }
        return;
    }

    // =========================================================== producer
    if (warp == 0) {
        if (lane_id() != 0) return;
        uint32_t s = 0, par = 1;  // ring stage and the parity of its "empty" barrier to wait for
        uint32_t issued = 0;      // copies issued so far
        const uint64_t once = l2_evict_first_policy();
        bool gave_up = false;
#pragma unroll 1
        for (int i = 0; i < n_list && !gave_up; ++i) {
            const uint8_t* src = reinterpret_cast<const uint8_t*>(a.x) + size_t(rlist[i]) * row_bytes;
            uint32_t left = uint32_t(row_bytes);  // (a row is below 4 GiB: n < 2^30 elements of at most 4 bytes)
#pragma unroll 1
            for (uint32_t c = 0; c < n_chunks; ++c) {
                if (!mbar_wait(&empty[s], par, a.wait_limit)) {
                    atomicExch(a.err, 1u);
                    gave_up = true;
                    break;
                }
                const uint32_t bytes = left < uint32_t(Q_SB) ? left : uint32_t(Q_SB);
                // (tests only: one copy of CTA 0 is left out, so that the waits for it run out)
                const bool lose = a.lose_copy && blockIdx.x == 0 && i == 0 && c == 3;
                if (!lose) {
                    mbar_expect_tx(&full[s], bytes);
                    bulk_g2s_once(ring + size_t(s) * Q_SB, src, bytes, &full[s], once);
                    ++issued;
                }
                src += Q_SB, left -= bytes;
                if (++s == uint32_t(stages)) s = 0, par ^= 1u;
            }
        }
        // This thread's last copies may still be on their way into the ring when the other roles have given up: the CTA's
        // shared memory must outlive them, so each one's "full" phase is awaited (bounded; at once in a run without
        // faults, where the stream warps have consumed them).  A stage armed in ring round r completes phase r of its
        // barrier, and this thread waited for parity (r & 1) ^ 1 of the stage's "empty" barrier before it.
        {
            uint32_t bs = s, bpar = par;
#pragma unroll 1
            for (uint32_t k = 0; k < uint32_t(stages) && k < issued; ++k) {
                if (bs == 0) bs = uint32_t(stages), bpar ^= 1u;
                --bs;
                mbar_wait(&full[bs], bpar ^ 1u, a.wait_limit);
            }
        }
        return;
    }

    // =========================================================== threshold keeper
    // One warp follows every row from the moment its slot is handed out until the last stream warp is through it: for
    // rows that want at most 64 candidates it keeps the threshold at the K-th largest of the log (see
    // keep_threshold_small_k); then it adds its arrival to the row's "closed" barrier, so that the slot is not given to
    // another row while this warp could still write a threshold into it.
    if (warp == 1 + Q_SW + Q_TW) {
        const int lane = lane_id();
#pragma unroll 1
        for (int ord = 0; ord < n_list; ++ord) {
            const int p = ord & 1;
            QSlot* sl = &sh->slot[p];
            if (!mbar_wait(&boot_done[p], (ord >> 1) & 1, a.wait_limit)) {
                if (lane == 0) atomicExch(a.err, 6u);
                return;
            }
            const uint32_t K = sl->cfg.K;
            uint32_t what = 2u;
            if (K <= uint32_t(Q_SMALL_K)) {
                what = keep_threshold_small_k(sl, logs + size_t(p) * Q_L, K, a.wait_limit);
            } else {
#pragma unroll 1
                for (uint32_t spin = 0; spin < 4 * a.wait_limit && what != 0u; ++spin) {
                    if (ldv_u32(&sl->done_warps) == uint32_t(Q_SW)) what = 0u;
                    else __nanosleep(500);
                }
            }
            if (what != 0u) {
                if (lane == 0) atomicExch(a.err, 6u);
                return;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&closed[p]);
        }
        return;
    }

    // =========================================================== tail group
    if (warp > Q_SW) {
        const Group<Q_TT> g{tid - 32 - Q_ST, 1};
        const Group<Q_PT> gp{g.tid - 32, 2};  // the tail warps but the first
        const int lane = lane_id(), tw = g.tid >> 5;

        // ---- the table of the distinct history tokens of the row in slot p, with their counts, for when the row is through
        // (the tail warps but the first, while the row streams).  Equal tokens of one warp-wide step go in as one insert;
        // the history comes through the select scratch (which nobody uses now), half of it at a time, so that the loads of a
        // half are all on their way at once and the inserts are one rolled loop.
        auto build_table = [&](int p) {
            const QRow cfg = sh->slot[p].cfg;
            if (!(cfg.flags & QF_PEN) || ((cfg.flags & QF_LAZY) && !LAZY_TABLE)) return;  // (only rows that will look tokens up)
            constexpr int HALF = kMaxHist / 2;
            constexpr int HP = (HALF + Q_PT - 1) / Q_PT;
            static_assert(HALF <= SEL_BINS, "half a history fits the scratch");
            const int32_t* h = P.hist + size_t(cfg.row) * P.hist_stride;
            const int hl = cfg.hist_len;
            int32_t* stage_h = reinterpret_cast<int32_t*>(hist);
            for (int i = gp.tid; i < kPenSlots / 4; i += Q_PT) reinterpret_cast<uint4*>(pslots)[i] = make_uint4(0, 0, 0, 0);
#pragma unroll 1
            for (int half = 0; half * HALF < hl; ++half) {
                int32_t hv[HP];
#pragma unroll
                for (int u = 0; u < HP; ++u) {
                    const int i = half * HALF + u * Q_PT + gp.tid;
                    hv[u] = (u * Q_PT + gp.tid < HALF && i < hl) ? h[i] : -1;
                }
#pragma unroll
                for (int u = 0; u < HP; ++u)
                    if (u * Q_PT + gp.tid < HALF) stage_h[u * Q_PT + gp.tid] = hv[u];
                gp.sync();
                const int cnt_h = min(HALF, hl - half * HALF);
#pragma unroll 1
                for (int base = 0; base < cnt_h; base += Q_PT) {
                    const int i = base + gp.tid;
                    const uint32_t t = i < cnt_h ? uint32_t(stage_h[i]) : 0xffffffffu;
                    const bool valid = t < n;  // (negative ids too)
                    const uint32_t peers = __match_any_sync(0xffffffffu, valid ? t : 0xfffffff0u - uint32_t(lane));
                    if (valid && lane == __ffs(peers) - 1) pen_table_insert(pslots, t, uint32_t(__popc(peers)));
                }
                gp.sync();
            }
        };

        // ---- raise a streaming row's threshold to the exact K-th largest of its log so far (rows of more than 64
        // candidates: the keeper warp does it for the others).  This is what keeps the log of a row whose first threshold
        // was a guess from filling up.  Marked entries carry raw logits and count as absent.
        uint32_t rf_last[2] = {0, 0};
        auto maybe_refine = [&](int p, uint32_t K, bool allowed, bool masked) {
            QSlot* sl = &sh->slot[p];
            if (g.tid == 0) {
                const uint32_t c = ldv_u32(&sl->cnt) & 0x7fffffffu;
                sh->flag[2] = c < uint32_t(Q_L) ? c : uint32_t(Q_L);
            }
            g.sync();
            const uint32_t nlog = sh->flag[2];
            g.sync();
            const uint32_t step = refine_step(K, rf_last[p]);
            if (!allowed || !(nlog >= K && nlog >= rf_last[p] + step)) return false;
            // The select makes several passes over the log's first nlog places and needs them to read the same every time.
            // A place is reserved before it is written, so a place that still reads zero is waited for (every entry is
            // non-zero; the writer is a few instructions away); what the stream warps append meanwhile lies behind nlog.
            {
                const unsigned long long* lg = logs + size_t(p) * Q_L;
#pragma unroll 1
                for (uint32_t i = g.tid; i < nlog; i += Q_TT) {
#pragma unroll 1
                    for (uint32_t spin = 0; spin < 100000u && ldv_u64(&lg[i]) == 0ull; ++spin) {
                    }
                }
                g.sync();
            }
            // (a row with marked entries: they carry raw logits and count as absent; the K-th largest of the others is a
            // valid bound all the same)
            const unsigned long long kth = masked ? select_kth<Q_TT, true>(g, logs + size_t(p) * Q_L, nlog, K, hist, &sh->sel)
                                                  : select_kth<Q_TT, false>(g, logs + size_t(p) * Q_L, nlog, K, hist, &sh->sel);
            if (g.tid == 0 && kth > ldv_u64(&sl->tau)) *reinterpret_cast<volatile unsigned long long*>(&sl->tau) = kth;
            rf_last[p] = nlog;
            g.sync();
            return true;
        };

        // ---- a row's outputs from its candidates (cand[0..kept), padded with zeros up to cap, a power of two; bp, bq:
        // cap + 2 * NT / 32 doubles each), by a group of NT threads: the first tail warp for rows of up to hand_k
        // candidates, the whole tail group for larger ones.
        auto finish_row = [&](auto grp, const QRow& cfg, uint64_t* cand, double* bp, double* bq, uint32_t kept, uint32_t cap, bool presorted,
                              bool overflow, bool nan_seen, float M, float sum) {
            constexpr int NT = decltype(grp)::size;
            const bool greedy = (cfg.flags & QF_GREEDY) != 0;
            const float inv_t = cfg.inv_t;
            const bool no_sum = (cfg.flags & QF_NO_SUM) != 0;
            const int row = cfg.row;
            const bool first = grp.tid == 0;
            if (overflow) {
                // more candidates than the log holds (rows in adversarial order), fewer than K (a guessed first threshold that
                // was too high), or a NaN in a sum: the multi-pass kernel takes the row
                if (first) {
                    a.out.status[row] = ROW_RETRY;
                    if (nan_seen && a.out.counters) atomicAdd(&a.out.counters[WHIRL_CNT_NAN_ROWS], 1u);
                }
            } else if (!sample) {
                if (first) a.out.status[row] = ROW_DONE;
                if (!presorted) sort_desc<NT>(grp, cand, cap);
                const T* xr = reinterpret_cast<const T*>(a.x) + size_t(row) * n;
#pragma unroll 1
                for (uint32_t j = grp.tid; j < kept; j += NT) {
                    const uint32_t id = cand_id(cand[j]);
                    a.ids[size_t(row) * a.K + j] = int32_t(id) + a.id_offset;
                    a.vals[size_t(row) * a.K + j] = sizeof(T) == 4 ? reinterpret_cast<const float*>(xr)[id] : bf16_to_f32(reinterpret_cast<const uint16_t*>(xr)[id]);
                }
                if (first) a.stats[2 * row] = M, a.stats[2 * row + 1] = sum;
            } else if (greedy) {
                if (first) {
                    const uint32_t tok = kept ? cand_id(cand[0]) : 0;
                    a.out.token[row] = int32_t(tok);
                    a.out.status[row] = ROW_DONE;
                    if (a.out.n_kept) a.out.n_kept[row] = 1;
                    if (a.out.closed) a.out.closed[row] = 1;
                    if (a.out.stats) a.out.stats[2 * row] = kept ? float_of_key(cand_key(cand[0])) : -INFINITY, a.out.stats[2 * row + 1] = 0.f;
                    if (a.out.kept_ids && a.out.kept_cap > 0) a.out.kept_ids[size_t(row) * a.out.kept_cap] = int32_t(tok);
                    if (a.out.kept_p && a.out.kept_cap > 0) a.out.kept_p[size_t(row) * a.out.kept_cap] = 1.0;
                }
            } else {
                // probabilities, the top-k / top-p / min-p cuts, the draw
                TailIn in;
                in.inv_t = inv_t;
                in.top_k = cfg.top_k;
                in.top_p = cfg.top_p, in.min_p = cfg.min_p, in.u = cfg.u;
                in.m = M, in.sum = sum, in.cnt = kept, in.cap = cap, in.V = n;
                in.race = P.race_key != nullptr, in.race_key = cfg.race_key;
                in.want_p = a.out.kept_p != nullptr && a.out.kept_cap > 0;
                in.have_e = 0, in.sum_of_e = no_sum;
                if (!presorted) sort_desc<NT>(grp, cand, cap), presorted = true;
                in.presorted = 1;
                bool decided = false;
                if (kept > 0 && (no_sum || (!in.race && !in.want_p))) {
                    // the candidates' exponentials (a row normalised over its candidates: cand[] holds exactly the kept ones,
                    // the largest first)
                    if (no_sum) M = float_of_key(cand_key(cand[0])), in.m = M;
#pragma unroll 1
                    for (uint32_t i = grp.tid; i < kept; i += NT) bq[i] = f64_exp(double(__fsub_rn(float_of_key(cand_key(cand[i])), M)) * double(inv_t));
                    grp.sync();
                    in.have_e = 1;
                    if (!in.race && !in.want_p && kept <= 16384u) {
                        decided = sample_tail_quick<NT>(grp, in, cand, bp, bq, &sh->res);
                        if (decided && no_sum) sum = sh->res.sum;
                        grp.sync();
                    }
                }
                if (!decided) {
                    if (no_sum) {
                        if (grp.tid < 32) {
                            const double tot = warp_total(bq, kept);
                            if (first) sh->res.cum = tot;
                        }
                        grp.sync();
                        sum = float(sh->res.cum);
                        grp.sync();
                        in.sum = sum;
                    }
                    sample_tail<NT>(grp, in, cand, bp, bq, &sh->res);
                }
                const TailOut r = sh->res;
                if (first) {
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
#pragma unroll 1
                    for (uint32_t j = grp.tid; j < nk; j += NT) {
                        if (a.out.kept_ids) a.out.kept_ids[size_t(row) * a.out.kept_cap + j] = int32_t(cand_id(cand[j]));
                        if (a.out.kept_p) a.out.kept_p[size_t(row) * a.out.kept_cap + j] = bp[j];
                    }
                }
            }
        };

        // order -1 is the start: nothing to finish, the first two rows' slots to hand out, the first row's table
#pragma unroll 1
        for (int ord = -1; ord < n_list; ++ord) {
            const int p = ord & 1;
            QSlot* sl = &sh->slot[p];
            unsigned long long* log = logs + size_t(p) * Q_L;
            QRow cfg;
            uint32_t kept = 0, cap = 1;
            bool presorted = false, overflow = false, nan_seen = false, big_done = false;
            float M = -INFINITY, sum = 0.f;
            if (ord >= 0) {
                cfg = sl->cfg;
                const uint32_t K = cfg.K;
                const bool no_sum = (cfg.flags & QF_NO_SUM) != 0, pen_on = (cfg.flags & QF_PEN) != 0, lazy = (cfg.flags & QF_LAZY) != 0;
                // (a row with marked log entries that has no table will want its history when it is through: the loads go out now)
                constexpr int HB = kMaxHist / Q_TT;
                int32_t hv[HB];
                if (lazy && !LAZY_TABLE) {
                    const int32_t* h = P.hist + size_t(cfg.row) * P.hist_stride;
#pragma unroll
                    for (int u = 0; u < HB; ++u) hv[u] = (u * Q_TT + g.tid) < cfg.hist_len ? h[u * Q_TT + g.tid] : -1;
                }
                // ---- while the row streams
                // (one thread watches the row; the others wait at the group's barrier, where they take no issue slot from the
                // stream warps)
#pragma unroll 1
                for (;;) {
                    if (g.tid == 0) {
                        uint32_t what = 2u;  // 0: the row is through, 1: the log wants a refinement, 2: gave up
                        const uint32_t step = refine_step(K, rf_last[p]);
#pragma unroll 1
                        for (uint32_t spin = 0; spin < 4 * a.wait_limit; ++spin) {
                            if (mbar_try_wait(&closed[p], (ord >> 1) & 1)) {
                                what = 0u;
                                break;
                            }
                            const uint32_t c = ldv_u32(&sl->cnt) & 0x7fffffffu;
                            if (K > uint32_t(Q_SMALL_K) && c >= K && c >= rf_last[p] + step && c <= uint32_t(Q_L)) {
                                what = 1u;
                                break;
                            }
                            __nanosleep(300);
                        }
                        sh->flag[1] = what;
                    }
                    g.sync();
                    const uint32_t what = sh->flag[1];
                    g.sync();
                    if (what == 0u) break;
                    if (what == 2u) {
                        // (the rows not answered keep their "pending" status; the CTA still hands in its ticket)
                        if (g.tid == 0) atomicExch(a.err, 3u);
                        goto tail_done;
                    }
                    maybe_refine(p, K, true, lazy);
                }
                mbar_wait(&closed[p], (ord >> 1) & 1, a.wait_limit);  // acquire the stream warps' writes
                rf_last[p] = 0;
                // ---- the row is through
                if (pen_on) {
                    const unsigned long long tau = sl->tau;
                    const float tau_f = cand_key(tau) ? float_of_key(cand_key(tau)) : -INFINITY;
                    if (lazy) {
                        // (An f32 row streams long enough for the tail warps to build the table of its history meanwhile; a
                        // bf16 row is through in half the time, so its few marked tokens are counted against the history
                        // itself.)
                        if (LAZY_TABLE) {
                            // The marked entries of the log: logged raw from a word that holds a history token.  A history token
                            // among them gets its penalty now (another logit of such a word stays as it is); its count comes from
                            // the table of the row's history, which the other tail warps built while the row streamed.
                            const uint32_t nl = min(sl->cnt & 0x7fffffffu, uint32_t(Q_L));
#pragma unroll 1
                            for (uint32_t i = g.tid; i < nl; i += Q_TT) {
                                const unsigned long long c = log[i];
                                if (c != 0ull && !(c & 0x80000000ull)) {
                                    const uint32_t id = ~uint32_t(c) & 0x7fffffffu;
                                    float x = float_of_key(cand_key(c));
                                    const uint32_t times = pen_table_count(pslots, id);
                                    if (times) x = penalised(x, times, cfg.rep, cfg.pres, cfg.freq);
                                    log[i] = make_cand(key_of(x), id);
                                }
                            }
                        } else {
                            // The marked entries of the log: logged raw from a word that holds a history token.  A history token
                            // among them gets its penalty now (another logit of such a word stays as it is).  They are few, so
                            // their counts come from a scan of the history, not from a table: every thread holds its share of the
                            // history in registers and all of them count one marked token after the other.
                            uint32_t* mlist = hist;                 // places in the log of the marked entries
                            uint32_t* mcnt = hist + SEL_BINS / 2;   // their counts
                            const uint32_t nl = min(sl->cnt & 0x7fffffffu, uint32_t(Q_L));
                            if (g.tid == 0) sh->flag[3] = 0u;
                            g.sync();
#pragma unroll 1
                            for (uint32_t i = g.tid; i < nl; i += Q_TT) {
                                const unsigned long long c = log[i];
                                if (c != 0ull && !(c & 0x80000000ull)) {
                                    const uint32_t at = atomicAdd(&sh->flag[3], 1u);
                                    if (at < uint32_t(SEL_BINS / 2)) mlist[at] = i, mcnt[at] = 0u;
                                }
                            }
                            g.sync();
                            const uint32_t nm = sh->flag[3];
                            if (nm > uint32_t(SEL_BINS / 2)) {
                                if (g.tid == 0) atomicOr(&sl->cnt, 0x80000000u);  // (more than the scratch holds: the multi-pass kernel takes the row)
                            } else if (nm > 0) {
#pragma unroll 1
                                for (uint32_t m = 0; m < nm; ++m) {
                                    const int32_t id = int32_t(~uint32_t(log[mlist[m]]) & 0x7fffffffu);
                                    uint32_t c = 0;
#pragma unroll
                                    for (int u = 0; u < HB; ++u) c += hv[u] == id;
                                    c = __reduce_add_sync(0xffffffffu, c);
                                    if (lane == 0 && c) atomicAdd(&mcnt[m], c);
                                }
                                g.sync();
#pragma unroll 1
                                for (uint32_t m = g.tid; m < nm; m += Q_TT) {
                                    const unsigned long long c = log[mlist[m]];
                                    const uint32_t id = ~uint32_t(c) & 0x7fffffffu;
                                    float x = float_of_key(cand_key(c));
                                    if (mcnt[m]) x = penalised(x, mcnt[m], cfg.rep, cfg.pres, cfg.freq);
                                    log[mlist[m]] = make_cand(key_of(x), id);
                                }
                            }
                        }
                    } else {
                        // the words put aside by the stream warps come in: history tokens with their penalty, the others as
                        // they are; every tail warp is one more contributor to the row's maximum and sum
                        const uint32_t ns = min(sl->side_cnt, uint32_t(kMaxHist));
                        JoinCtx jc;
                        jc.pslots = pslots, jc.sl = sl, jc.log = log;
                        jc.rep = cfg.rep, jc.pres = cfg.pres, jc.freq = cfg.freq, jc.cexp = cfg.inv_t * kLog2e;
                        jc.no_sum = no_sum;
                        jc.m_t = -INFINITY, jc.e_t = 0.f, jc.s_t = 0.f;
                        jc.tau = tau, jc.tau_f = tau_f;
                        constexpr int PB = 2;  // words per thread and trip to memory
#pragma unroll 1
                        for (uint32_t base = 0; base < ns; base += PB * Q_TT) {
                            uint32_t wq[PB];
                            uint4 wv[PB];
#pragma unroll
                            for (int j = 0; j < PB; ++j) {  // (the loads first, then the arithmetic)
                                const uint32_t i = base + uint32_t(j) * Q_TT + uint32_t(g.tid);
                                wq[j] = i < ns ? __ldcg(side_q(p) + i) : 0xffffffffu;
                                wv[j] = i < ns ? __ldcg(side_w(p) + i) : make_uint4(0, 0, 0, 0);
                            }
#pragma unroll
                            for (int j = 0; j < PB; ++j)
                                if (wq[j] < row_q) join_word<VE>(jc, wq[j], wv[j]);
                        }
                        if (!no_sum) {
                            const float m_t = jc.m_t, e_t = jc.e_t, s_t = jc.s_t;
                            const bool saw_nan = s_t != s_t;
                            if (__any_sync(0xffffffffu, saw_nan) && lane == 0) atomicOr(&sl->cnt, 0x80000000u);
                            const float wm = warp_max(m_t);
                            float we = e_t;
                            if (m_t == -INFINITY) we = -INFINITY;
                            we = warp_max(we);
                            double ds = (m_t == -INFINITY) ? 0.0 : double(s_t) * double(ex2_approx(e_t - we));
                            ds = warp_sum(ds);
                            if (lane == 0) sl->red_m[Q_SW + tw] = wm, sl->red_e[Q_SW + tw] = we, sl->red_s[Q_SW + tw] = ds;
                        }
                    }
                    g.sync();
                }
                const float inv_t = cfg.inv_t;
                const uint32_t total_raw = sl->cnt;  // bit 31: a NaN logit met a sum
                const bool nan_row = (total_raw & 0x80000000u) != 0;
                const uint32_t total = total_raw & 0x7fffffffu;
                nan_seen = nan_row;
                overflow = total > uint32_t(Q_L) || nan_row || (pen_on && !lazy && sl->side_cnt > uint32_t(kMaxHist));
                const uint32_t nlog = total > uint32_t(Q_L) ? uint32_t(Q_L) : total;
                // row max and normaliser: combine the warps' partials, one per lane (not needed when the row is normalised
                // over its candidates)
                if (!no_sum) {
                    const int n_red = Q_SW + ((pen_on && !lazy) ? Q_TW : 0);
                    static_assert(Q_RED <= 32, "one partial per lane");
                    const float mw = lane < n_red ? sl->red_m[lane] : -INFINITY;
                    M = warp_max(mw);
                    const double cexp = double(inv_t * kLog2e);
                    const double term = (lane < n_red && mw != -INFINITY) ? sl->red_s[lane] * exp2(double(sl->red_e[lane]) - double(M) * cexp) : 0.0;
                    sum = float(warp_sum(term));
                }
                // (a guessed first threshold that left fewer than K candidates: the row is done again)
                if (K > uint32_t(Q_SMALL_K) && total < K && total < n) overflow = true;
                big_done = K > uint32_t(hand_k) && !overflow;
                if (big_done) {
                    // More candidates than the hand holds: the K best of the log go to the select scratch, the whole group
                    // sorts them and draws, with the probabilities in the row's log (which nobody reads any more).
                    unsigned long long* list = reinterpret_cast<unsigned long long*>(hist);  // SEL_BINS / 2 entries
                    static_assert(SEL_BINS / 2 >= kSinglePassMaxK && size_t(Q_L) * 8 >= 2 * size_t(kSinglePassMaxK + 2 * Q_TW) * 8, "room for a large-K row");
                    // (the hand and the first tail warp's scratch lie idle for such a row: they hold the bins)
                    uint32_t* bins = reinterpret_cast<uint32_t*>(hand);
                    constexpr uint32_t bcap = 4 * Q_TT;
                    static_assert(bcap == SEL_BINS / 2 && bcap >= kSinglePassMaxK, "the select scratch holds the candidates");
                    static_assert(size_t(kSinglePassHandK) * 8 + 2 * (size_t(kSinglePassHandK) + 2 * Q_TW) * 8 >= size_t(SB_BINS) * 4 + size_t(SB_X) * 8,
                                  "bins and side list fit the hand and its scratch");
                    uint32_t bk;
                    bool short_of_k = false;
                    if (bucket_sort_top<Q_TT>(g, log, nlog, K, sl->tau, bins, list, reinterpret_cast<unsigned long long*>(bins + SB_BINS), &sh->sel)) {
                        bk = sh->sel.wcnt;
                        // (A guessed threshold is checked against the number of logged entries, marked ones included; when
                        // penalties then take so many of them below the threshold that fewer than K stay at or above it, the
                        // K-th best may be a logit that was never logged: the row is done again.)
                        short_of_k = bk < K && sl->tau != 0ull;
                    } else {
                        // (many equal logits: the K-th largest of the log, the entries at or above it, a sorting network)
                        const unsigned long long kth = nlog > K ? select_kth<Q_TT>(g, log, nlog, K, hist, &sh->sel) : 0ull;
                        g.sync();
                        write_survivors<Q_TT>(g, log, nlog, kth, list, uint32_t(SEL_BINS / 2), &sh->sel);
                        bk = sh->sel.wcnt < uint32_t(SEL_BINS / 2) ? sh->sel.wcnt : uint32_t(SEL_BINS / 2);
                        g.sync();
                        for (uint32_t i = bk + g.tid; i < bcap; i += Q_TT) list[i] = 0ull;  // (the network takes four per thread)
                        g.sync();
                        sort_desc_x4<Q_TT>(g, reinterpret_cast<uint64_t*>(list));
                    }
                    double* bp = reinterpret_cast<double*>(log);
                    finish_row(g, cfg, reinterpret_cast<uint64_t*>(list), bp, bp + bcap + 2 * Q_TW, bk, bcap, true, short_of_k, false, M, sum);
                    g.sync();
                    for (uint32_t i = g.tid; i < uint32_t(Q_L); i += Q_TT) log[i] = 0ull;
                } else if (!overflow) {
                    // Most of the log was appended under an earlier, looser threshold: only entries at or above the current one
                    // can be among the K best (at least K of them are).  Few survive, so rank them against each other: the
                    // rank is the position in the sorted order.
                    unsigned long long* list = reinterpret_cast<unsigned long long*>(hist);  // up to SEL_BINS / 2 entries
                    // (more than 64 candidates: the histogram ranks them; it gives up on rows of many equal logits)
                    static_assert(SEL_BINS >= SB_BINS + 2 * SB_X, "bins and side list fit the select scratch");
                    const bool ranked = K > uint32_t(Q_SMALL_K) && bucket_sort_top<Q_TT>(g, log, nlog, K, sl->tau, hist, hand,
                                                                                         reinterpret_cast<unsigned long long*>(hist + SB_BINS), &sh->sel);
                    if (ranked) {
                        kept = sh->sel.wcnt;
                        presorted = true;
                        if (kept < K && sl->tau != 0ull) overflow = true;  // (penalties left fewer than K at or above a guessed threshold)
                    } else {
                        write_survivors<Q_TT>(g, log, nlog, sl->tau, list, SEL_BINS / 2, &sh->sel);
                        const uint32_t m = sh->sel.wcnt;
                        if (m <= 2u * Q_TT) {
#pragma unroll 1
                            for (uint32_t t = g.tid; t < m; t += Q_TT) {
                                const unsigned long long mine = list[t];
                                uint32_t rank = 0;
#pragma unroll 4
                                for (uint32_t j = 0; j < m; ++j) rank += list[j] > mine;
                                if (rank < K) hand[rank] = mine;
                            }
                            kept = m < K ? m : K;
                            presorted = true;
                        } else if (nlog > K) {
                            const unsigned long long kth = select_kth<Q_TT>(g, log, nlog, K, hist, &sh->sel);
                            write_survivors<Q_TT>(g, log, nlog, kth, hand, uint32_t(hand_k), &sh->sel);
                            kept = sh->sel.wcnt < uint32_t(hand_k) ? sh->sel.wcnt : uint32_t(hand_k);
                        } else {
                            for (uint32_t i = g.tid; i < nlog; i += Q_TT) hand[i] = log[i];
                            kept = nlog;
                        }
                    }
                }
                while (cap < kept) cap <<= 1;
                g.sync();
                for (uint32_t i = kept + g.tid; i < cap; i += Q_TT) hand[i] = 0ull;
                // the slot is free for the row after the next once its log and its word map are zero again
                for (uint32_t i = g.tid; i < nlog; i += Q_TT) log[i] = 0ull;
                if (pen_on) {
                    uint32_t* gbm = gbms + size_t(p) * gbm_words;
                    for (int i = g.tid; i < gbm_words / 4; i += Q_TT) reinterpret_cast<uint4*>(gbm)[i] = make_uint4(0, 0, 0, 0);
                }
                g.sync();
            }
            if (tw > 0) {
                // ---- the freed slot goes to the row after the next (at the start: both slots go out), then the table of the
                // row that streams now
                if (ord < 0) {
                    if (!(early_boot && rlist[0] == int(blockIdx.x))) {
                        if (early_boot) {  // (prepared for a row that is not listed: its marks go)
                            for (int i = gp.tid; i < gbm_words; i += Q_PT) gbms[i] = 0u;
                            gp.sync();
                        }
                        slot_prepare(0, rlist[0]);
                    }
                    slot_release(0);
                    if (n_list > 1) slot_boot(1, rlist[1]);
                } else if (ord + 2 < n_list) {
                    slot_boot(p, rlist[ord + 2]);
                }
                if (ord + 1 < n_list) build_table(p ^ 1);
            } else if (ord >= 0 && !big_done) {
                // ---- the first tail warp: the row's outputs
                finish_row(Group<32>{lane, 0}, cfg, reinterpret_cast<uint64_t*>(hand), tail_p, tail_q, kept, cap, presorted, overflow, nan_seen, M, sum);
            }
            g.sync();
        }
    tail_done:
        // Every row of this CTA has its status.
        if (a.fin_list) {
            __threadfence();
            g.sync();
            if (g.tid < 32) list_leftovers(a);
        }
        return;
    }

    // =========================================================== stream warps
    const int lane = lane_id(), sw = warp - 1, st_tid = tid - 32;
    const uint32_t nw = sizeof(T) == 4 ? 0xff800000u : 0xff80ff80u;  // -inf
    const uint4 ninf4 = make_uint4(nw, nw, nw, nw);
    uint32_t st_slot = 0, st_phase = 0;  // ring position of this warp and the parity it waits for
    const uint32_t n_iter = (n_chunks + Q_NS - 1) / Q_NS;
    const uint32_t full_iters = row_q / (Q_NS * Q_SQ);  // iterations whose words all lie inside the row
#pragma unroll 1
    for (int ord = 0; ord < n_list; ++ord) {
        const int p = ord & 1;
        QSlot* sl = &sh->slot[p];
        unsigned long long* log = logs + size_t(p) * Q_L;
        const uint32_t* gbm = gbms + size_t(p) * gbm_words;
        // the slot (parameters, log, threshold, word map) is this row's once the tail group says so
        if (!mbar_wait(&boot_done[p], (ord >> 1) & 1, a.wait_limit)) {
            if (lane == 0) atomicExch(a.err, 4u);
            return;
        }
        const uint32_t row_flags = sl->cfg.flags;
        const float cexp = sl->cfg.inv_t * kLog2e;
        // the lane's running maximum, reference exponent ceil(m1 * cexp), sum 2^(x * cexp - e_t)
        float m1 = -INFINITY, e_t = 0.f, s_t = 0.f;
        uint32_t tau_key = 0u;  // the threshold's ordering key as this warp last saw it (0: none)
        float tau_f = -INFINITY;
        bool st_fail = false;
        const volatile uint32_t* tau_hi = reinterpret_cast<const volatile uint32_t*>(&sl->tau) + 1;

        // The row's iterations, in one of three forms so that the common rows run a short loop: PLAIN (no normaliser, no
        // penalties), LAZY (no normaliser, penalties that only lower a logit), GENERAL (the rest).
        constexpr int SM_PLAIN = 0, SM_LAZY = 1, SM_GENERAL = 2;
        auto run_row = [&](auto mode_tag) {
            constexpr int MODE = decltype(mode_tag)::value;
            constexpr int NW = 2 * Q_NS;  // 128-bit words per thread and iteration
#pragma unroll 1
            for (uint32_t iter = 0; iter < n_iter; ++iter) {
                const uint32_t c = Q_NS * iter;
                // (In the GENERAL form the row's flags go through an empty asm so that the compiler sees values it cannot hoist:
                // it would make one copy of this whole body per combination of them, and the kernel's code has to fit the
                // instruction cache.)
                uint32_t fl = row_flags;
                if (MODE == SM_GENERAL) asm volatile("" : "+r"(fl));
                const bool no_sum = MODE != SM_GENERAL || (fl & QF_NO_SUM) != 0;
                const bool pen_on = MODE == SM_LAZY || (MODE == SM_GENERAL && (fl & QF_PEN) != 0);
                const bool lazy = MODE == SM_LAZY;
                const bool whole = iter < full_iters;  // (only the row's last iteration can be short)
                uint4 w[NW];
                uint32_t st_ring[Q_NS];
#pragma unroll
                for (int h = 0; h < Q_NS; ++h) {
                    st_ring[h] = st_slot;
                    if (whole || c + uint32_t(h) < n_chunks) {
                        if (!mbar_wait(&full[st_slot], st_phase, a.wait_limit)) {
                            if (lane == 0) atomicExch(a.err, 5u);
                            st_fail = true;
                            return;
                        }
                    }
                    const uint4* vec = reinterpret_cast<const uint4*>(ring + size_t(st_slot) * Q_SB);
#pragma unroll
                    for (int j = 0; j < 2; ++j) w[2 * h + j] = vec[j * Q_ST + st_tid];  // (a stage that is not the row's reads as
                                                                                        // whatever the ring holds: masked below)
                    if (whole || c + uint32_t(h) < n_chunks) {
                        if (++st_slot == uint32_t(stages)) st_slot = 0, st_phase ^= 1u;
                    }
                }
                const uint32_t wq0 = c * Q_SQ + uint32_t(st_tid);  // word i of this thread is at wq0 + i * Q_ST in the row
                if (!whole) {
#pragma unroll
                    for (int i = 0; i < NW; ++i)
                        if (wq0 + uint32_t(i) * Q_ST >= row_q) w[i] = ninf4;
                }
                // words that hold a history token (one 128-bit load gives the thread its four bits)
                uint32_t marked = 0;  // bit i: word i
                // (a row that only marks log entries needs the bits for its bounds in iteration 0; later it looks them up when
                // it has something to log)
                if (pen_on && (!lazy || iter == 0)) {
                    const uint4 mw = *reinterpret_cast<const uint4*>(gbm + ((iter * Q_SW + uint32_t(sw)) << 2));
                    marked = ((mw.x >> lane) & 1u) | (((mw.y >> lane) & 1u) << 1) | (((mw.z >> lane) & 1u) << 2) | (((mw.w >> lane) & 1u) << 3);
                    if (!lazy) {
                        // they are put aside for the tail group, as they are, and count as -inf here
#pragma unroll
                        for (int i = 0; i < NW; ++i) {
                            const bool mk = (marked >> i) & 1u;
                            const uint32_t bal = __ballot_sync(0xffffffffu, mk);
                            if (bal) {
                                uint32_t at = 0;
                                if (lane == 0) at = atomicAdd(&sl->side_cnt, uint32_t(__popc(bal)));
                                at = __shfl_sync(0xffffffffu, at, 0) + uint32_t(__popc(bal & ((1u << lane) - 1)));
                                if (mk && at < uint32_t(kMaxHist)) {
                                    __stcg(side_w(p) + at, w[i]);
                                    __stcg(side_q(p) + at, wq0 + uint32_t(i) * Q_ST);
                                }
                                if (mk) w[i] = ninf4;
                            }
                        }
                        marked = 0;
                    }
                }
                // The logits as f32: free for an f32 row; a bf16 row widens them only where it needs them one by one (the sum of
                // the GENERAL form, an iteration with something to log).
                float xv[NW * VE];
                auto widen = [&]() {
#pragma unroll
                    for (int i = 0; i < NW; ++i) {
                        const uint32_t w4[4] = {w[i].x, w[i].y, w[i].z, w[i].w};
                        float* x = xv + i * VE;
                        if (sizeof(T) == 4) {
#pragma unroll
                            for (int e = 0; e < 4; ++e) x[e] = __uint_as_float(w4[e]);
                        } else {
#pragma unroll
                            for (int e = 0; e < 4; ++e) x[2 * e] = __uint_as_float(w4[e] << 16), x[2 * e + 1] = __uint_as_float(w4[e] & 0xffff0000u);
                        }
                    }
                };
                constexpr bool WIDEN_FIRST = sizeof(T) == 4 || MODE == SM_GENERAL;
                if (WIDEN_FIRST) widen();
                // the iteration's largest logit (a NaN logit never raises a maximum)
                const float vm = words_max<T, NW>(w);
                // Every loaded register has been consumed, so the shared-memory reads have completed (instructions issue in
                // order and the maximum had to wait for the data): only now may the producer overwrite the stages.
                __syncwarp();
                if (lane == 0) {
#pragma unroll
                    for (int h = 0; h < Q_NS; ++h)
                        if (whole || c + uint32_t(h) < n_chunks) mbar_arrive(&empty[st_ring[h]]);
                }
                if (!no_sum) {
                    if (vm > m1) {
                        // new reference exponent: an integer at or above m * cexp, so every term is at most 1 and
                        // x * cexp - e is one fused operation with a single rounding
                        const float ne = ceilf(vm * cexp);
                        s_t = (m1 == -INFINITY) ? 0.f : s_t * ex2_approx(e_t - ne);
                        e_t = ne;
                    }
                    if (fmaxf(vm, m1) != -INFINITY) {
                        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                        for (int j = 0; j < NW * VE; ++j) acc[j & 3] += ex2_approx(fmaf(xv[j], cexp, -e_t));
                        s_t += (acc[0] + acc[1]) + (acc[2] + acc[3]);
                    }
                }
                // The lane's maximum: what the first threshold is made of (iteration 0: the largest of the logits the lane has
                // just read), and the running maximum of the sum (the GENERAL form).  For the threshold the marked words do not
                // count: their raw logits are not the row's.
                if (MODE == SM_GENERAL || iter == 0) {
                    float vb = vm;
                    if (lazy) {
                        vb = -INFINITY;
#pragma unroll
                        for (int i = 0; i < NW; ++i)
                            if (!((marked >> i) & 1u)) vb = fmaxf(vb, words_max<T, 1>(w + i));
                    }
                    m1 = fmaxf(m1, vb);
                }
                if (iter == 0) {
                    // The row's first threshold: the warps meet (their one meeting per row); what this lane read is tested against
                    // the agreed threshold below, from its registers.
                    // The warp publishes its largest lane maxima, in descending order: 8 for a small-K row, Q_TOP otherwise.
                    const uint32_t rank0 = sl->cfg.rank0;
                    {
                        const bool small_k = sl->cfg.K <= uint32_t(Q_SMALL_K);
                        const int ntop = small_k ? 8 : Q_TOP;
                        // (0: none; the lane maxima in descending order over the lanes: 15 shuffle steps)
                        const uint32_t mine = warp_sort_desc(m1 == -INFINITY ? 0u : key_of(m1), lane);
                        // (a small-K row's 128 keys lie packed at the front: four per lane to read back instead of eight)
                        if (lane < ntop) sl->wtop[sw * ntop + lane] = mine;
                        __syncwarp();
                    }
                    if (lane == 0) mbar_arrive(&head_done[p]);
                    if (!mbar_wait(&head_done[p], (ord >> 1) & 1, a.wait_limit)) {
                        if (lane == 0) atomicExch(a.err, 11u);
                        st_fail = true;
                        return;
                    }
                    // The row's first threshold: the largest key prefix (20 bits) that at least rank0 of the published keys
                    // reach.  That many logits of the row lie at or above it.  For a small-K row rank0 is K and this is a bound
                    // on the K-th largest logit of the row, close to the K-th largest read so far; for a larger K rank0 is
                    // first_rank's guess.
                    uint32_t kmin = 0u;
                    {
                        const bool small_k = sl->cfg.K <= uint32_t(Q_SMALL_K);
                        // (written before the meeting's barrier)
                        const uint4 qa = *reinterpret_cast<const uint4*>(&sl->wtop[small_k ? 4 * lane : 8 * lane]);
                        const uint4 qb = small_k ? make_uint4(0u, 0u, 0u, 0u) : *reinterpret_cast<const uint4*>(&sl->wtop[8 * lane + 4]);
                        // (All published keys share their leading bits - sign, exponent, often some of the mantissa - and the
                        // answer shares them too: the search starts below the common prefix of the largest and the smallest.)
                        uint32_t hi = max(max(qa.x, qa.y), max(qa.z, qa.w)), lo = 0xffffffffu, nz = 0;
                        if (!small_k) hi = max(hi, max(max(qb.x, qb.y), max(qb.z, qb.w)));
                        {
                            const uint32_t v8[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
#pragma unroll
                            for (int i = 0; i < 8; ++i)
                                if (v8[i] != 0u) lo = min(lo, v8[i]), ++nz;
                        }
                        hi = __reduce_max_sync(0xffffffffu, hi);
                        lo = __reduce_min_sync(0xffffffffu, lo);
                        nz = __reduce_add_sync(0xffffffffu, nz);
                        int b_start = -1;
                        if (nz >= rank0 && hi != 0u) {  // (else: fewer keys than rank0, no threshold)
                            const uint32_t diff = hi ^ lo;
                            if (diff == 0u) {
                                kmin = hi & 0xfffff000u;  // (all keys equal)
                            } else {
                                b_start = 31 - __clz(int(diff));
                                kmin = b_start >= 31 ? 0u : (hi & ~((2u << b_start) - 1u));
                                if (b_start < 12) kmin &= 0xfffff000u;
                            }
                        }
#pragma unroll 1
                        for (int b = b_start; b >= 12; --b) {
                            const uint32_t cand = kmin | (1u << b);
                            uint32_t c = (qa.x >= cand ? 1u : 0u) + (qa.y >= cand ? 1u : 0u) + (qa.z >= cand ? 1u : 0u) + (qa.w >= cand ? 1u : 0u);
                            if (!small_k) c += (qb.x >= cand ? 1u : 0u) + (qb.y >= cand ? 1u : 0u) + (qb.z >= cand ? 1u : 0u) + (qb.w >= cand ? 1u : 0u);
                            if (__reduce_add_sync(0xffffffffu, c) >= rank0) kmin = cand;
                        }
                    }
                    if (kmin) tau_key = kmin, tau_f = float_of_key(kmin);
                    if (sw == 0 && lane == 0) {
                        const unsigned long long t0 = (unsigned long long)kmin << 32;
                        if (t0 > ldv_u64(&sl->tau)) *reinterpret_cast<volatile unsigned long long*>(&sl->tau) = t0;
                    }
                } else {
                    const uint32_t tk = *tau_hi;
                    if (tk > tau_key) tau_key = tk, tau_f = float_of_key(tk);
                }
                if (__any_sync(0xffffffffu, vm >= tau_f)) {
                    // Some lane holds logits that may beat the threshold.
                    if (lazy && iter != 0) {
                        const uint4 mw = *reinterpret_cast<const uint4*>(gbm + ((iter * Q_SW + uint32_t(sw)) << 2));
                        marked = ((mw.x >> lane) & 1u) | (((mw.y >> lane) & 1u) << 1) | (((mw.z >> lane) & 1u) << 2) | (((mw.w >> lane) & 1u) << 3);
                    }
                    if (!WIDEN_FIRST) widen();
                    uint32_t hm = 0;  // bit j: this lane's logit j is at or above the threshold
#pragma unroll
                    for (int j = 0; j < NW * VE; ++j) hm |= (xv[j] >= tau_f ? 1u : 0u) << j;
                    // (each lane with logits to log reserves its places itself: few lanes have any, and a scan over the warp
                    // would put its latency in front of every one of them)
                    uint32_t pos = 0;
                    if (hm) pos = atomicAdd(&sl->cnt, uint32_t(__popc(hm))) & 0x7fffffffu;
#pragma unroll 1
                    while (hm) {
                        const int j = __ffs(int(hm)) - 1;
                        hm &= hm - 1;
                        // logit j out of the registers: a tree of selects on the bits of j
                        float t[NW * VE];
#pragma unroll
                        for (int q = 0; q < NW * VE; ++q) t[q] = xv[q];
#pragma unroll
                        for (int lvl = 0; (1 << lvl) < NW * VE; ++lvl) {
                            const bool odd = (j >> lvl) & 1;
#pragma unroll
                            for (int q = 0; q < (NW * VE) >> (lvl + 1); ++q) t[q] = odd ? t[2 * q + 1] : t[2 * q];
                        }
                        const int wi = j / VE;  // (VE is a power of two)
                        const uint32_t id = (wq0 + uint32_t(wi) * Q_ST) * VE + uint32_t(j % VE);
                        const uint32_t u = __float_as_uint(t[0] + 0.0f);  // -0 + +0 = +0: the two zeros share a key
                        const uint32_t key = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
                        unsigned long long cnd = make_cand(key, id);
                        if ((marked >> wi) & 1u) cnd &= ~0x80000000ull;  // logged raw from a word that holds a history token
                        if (pos < uint32_t(Q_L)) log[pos] = cnd;
                        ++pos;
                    }
                }
            }
        };
        if ((row_flags & (QF_NO_SUM | QF_PEN)) == QF_NO_SUM) run_row(std::integral_constant<int, SM_PLAIN>{});
        else if (row_flags & QF_LAZY) run_row(std::integral_constant<int, SM_LAZY>{});
        else run_row(std::integral_constant<int, SM_GENERAL>{});
        if (st_fail) return;
        // ---- the row is through for this warp: partials, then close
        if (!(row_flags & QF_NO_SUM)) {
            // a NaN logit poisons the f32 sum: such rows are redone by the multi-pass kernel, which counts NaN as -inf
            const bool saw_nan = s_t != s_t;
            if (__any_sync(0xffffffffu, saw_nan) && lane == 0) atomicOr(&sl->cnt, 0x80000000u);
            const float wm = warp_max(m1);
            float we = e_t;
            if (m1 == -INFINITY) we = -INFINITY;
            we = warp_max(we);
            double ds = (m1 == -INFINITY) ? 0.0 : double(s_t) * double(ex2_approx(e_t - we));
            ds = warp_sum(ds);
            if (lane == 0) sl->red_m[sw] = wm, sl->red_e[sw] = we, sl->red_s[sw] = ds;
        }
        if ((row_flags & (QF_PEN | QF_LAZY)) == QF_PEN) __threadfence();  // (words put aside in global memory are read by the tail group)
        __syncwarp();
        if (lane == 0) {
            atomicAdd(&sl->done_warps, 1u);
            mbar_arrive(&closed[p]);
        }
    }
}

static int single_pass_gbm_words(const SelectArgs& a, int dtype) {
    const bool pen = a.mode == MODE_SAMPLE && a.prm.hist != nullptr;
    const int ve = dtype == 0 ? 4 : 8;
    // one map word per stream warp, word of the thread and iteration (see gbm_word_of)
    return pen ? ((a.n / ve + 2 * Q_SQ - 1) / (2 * Q_SQ)) * Q_SW * 4 : 0;
}

static size_t single_pass_fixed_smem(int gbm_words, int hand_k, bool pen) {
    return size_t(2) * Q_L * 8 + SEL_BINS * 4 + size_t(hand_k) * 8 + 2 * (size_t(hand_k) + 2 * Q_TW) * 8 + (2 * Q_MAXSTAGES + 6) * 8 +
           sizeof(QShared) + 16 + size_t(2) * gbm_words * 4 + (pen ? size_t(kPenSlots) * 4 : 0) + 128;
}

bool single_pass_supported(const SelectArgs& a, int dtype) {
    const size_t es = dtype == 0 ? 4 : 2;
    if (reinterpret_cast<uintptr_t>(a.x) % 16 != 0 || (size_t(a.n) * es) % 16 != 0) return false;  // bulk copies need 16-byte rows
    // Rows shorter than one iteration of the stream warps (two ring stages) leave most warps without logits, so no bound
    // on the K-th largest comes out of the first meeting and the candidate log would take the whole row: the multi-pass
    // kernel serves such rows (vocabularies below 8192 / 16384 tokens).
    if (size_t(a.n) * es < size_t(Q_NS) * Q_SB) return false;
    if (a.mode == MODE_TOPK) {
        // (the rule of first_rank: a large K on a short row would need a first threshold deeper than the stream warps publish)
        if (a.K > kSinglePassMaxK) return false;
        const uint32_t K = uint32_t(a.K) > uint32_t(a.n) ? uint32_t(a.n) : uint32_t(a.K);
        if (K > uint32_t(Q_SMALL_K)) {
            const uint32_t it0 = uint32_t(Q_NS) * Q_SB / uint32_t(es);
            const float x = float(K) * float(it0 < uint32_t(a.n) ? it0 : uint32_t(a.n)) / float(a.n);
            const float r = 0.5f * (Q_GUESS_Z + sqrtf(Q_GUESS_Z * Q_GUESS_Z + 4.f * x));
            if (uint32_t(ceilf(r * r)) > uint32_t(Q_RANK_MAX)) return false;
        }
    }
    if (a.mode == MODE_DRAFT) return false;
    if (a.rows > Q_MAXR * 100) return false;  // (more rows per CTA than its row list holds: far beyond any batch of logits)
    const bool pen = a.mode == MODE_SAMPLE && a.prm.hist != nullptr;
    return single_pass_fixed_smem(single_pass_gbm_words(a, dtype), kSinglePassHandK, pen) + 3 * size_t(Q_SB) <= 232448;
}

cudaError_t single_pass_launch(const SelectArgs& args, int dtype, int sm_count, cudaStream_t st) {
    SelectArgs a = args;
    if (a.wait_limit == 0) a.wait_limit = kWaitLimit;  // the budget of every wait inside the kernel
    const bool pen = a.mode == MODE_SAMPLE && a.prm.hist != nullptr;
    const int gbm_words = single_pass_gbm_words(a, dtype);
    const int max_k = kSinglePassMaxK, hand_k = kSinglePassHandK;
    const size_t fixed = single_pass_fixed_smem(gbm_words, hand_k, pen);
    int stages = int((232448 - fixed) / Q_SB);
    if (stages > Q_MAXSTAGES) stages = Q_MAXSTAGES;
    if (stages < 3) return cudaErrorInvalidConfiguration;
    const size_t smem = fixed + size_t(stages) * Q_SB;
    const int grid = a.rows < sm_count ? a.rows : sm_count;
    if ((a.rows + grid - 1) / grid > Q_MAXR) return cudaErrorInvalidConfiguration;
    const cudaError_t em = cudaMemsetAsync(a.err, 0, 64, st);  // the error words, the list count and tickets, the scratch locks
    if (em != cudaSuccess) return em;
    if (dtype == 0) {
        const cudaError_t e = cudaFuncSetAttribute(single_pass_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
        if (e != cudaSuccess) return e;
        single_pass_kernel<float><<<grid, Q_THREADS, smem, st>>>(a, stages, gbm_words, max_k, hand_k);
    } else {
        const cudaError_t e = cudaFuncSetAttribute(single_pass_kernel<uint16_t>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
        if (e != cudaSuccess) return e;
        single_pass_kernel<uint16_t><<<grid, Q_THREADS, smem, st>>>(a, stages, gbm_words, max_k, hand_k);
    }
    return cudaGetLastError();
}

size_t single_pass_side_bytes(int sm_bound) { return size_t(sm_bound < 1 ? 1 : sm_bound) * 2 * kMaxHist * 20; }

}  // namespace wb
