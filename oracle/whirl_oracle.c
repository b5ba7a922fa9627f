/*
 * CPU oracle of the WHIRL token-sampling path.  TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C restatement of the reference's host sampling algorithm, used as the checker for the CUDA
 * kernels and as the "port" CPU baseline of bench.py.  Nothing in the shipped library links, loads or
 * calls this file; only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / reference legs do.
 *
 * Every function names the reference source it follows (paths relative to the reference project root).
 * Parity status:
 *   PINNED   against the reference's own code (oracle/_ref, built from the reference sources in place) and
 *            against the fixtures under tests/golden/ that were generated from it:
 *            uniforms and race keys, first-max, top-k rows with stats, the candidate filter, the row
 *            prepare escalation, inverse-CDF and race draws, probOf, draftDist, the spec race draw,
 *            greedy / sampling draft acceptance and the relaxed-acceptance rules.
 *   UNPINNED (no counterpart in the reference; the semantics are this build's own and are written
 *            beside each function): logit penalties, Philox4x32-10 uniforms (pinned only to the published
 *            Random123 known-answer vectors), bf16 widening, accept/residual speculative sampling, the
 *            vocab-shard candidate merge.
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------------------------------
 * counter-hash uniforms and race keys
 * ---------------------------------------------------------------------------------------------- */

/* splitmix64 finaliser: include/whirl/spec_sample.h:53-57 */
static uint64_t mix64(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

static double top53(uint64_t z) { return (double)(z >> 11) * (1.0 / 9007199254740992.0); }

/* src/common/spec_sample.cpp:13-21; stream 0 is Sampler::uniform (src/sampling/sampler.h:46-52) */
ORC_API double orc_uniform(uint64_t seed, uint64_t pos_idx, uint32_t stream) {
    if (stream != 0) seed ^= (uint64_t)stream * 0xD1B54A32D192ED03ull;
    return top53(mix64(seed + (pos_idx + 1) * 0x9E3779B97F4A7C15ull));
}

/* include/whirl/spec_sample.h:58-60 */
ORC_API uint64_t orc_race_base(uint64_t seed, uint64_t pos_idx) {
    return mix64((seed ^ 0xA0761D6478BD642Full) + (pos_idx + 1) * 0x9E3779B97F4A7C15ull);
}

/* src/common/spec_sample.cpp:83-87 */
ORC_API double orc_race_e(uint64_t base, uint32_t token) {
    const double u = top53(mix64(base + ((uint64_t)token + 1) * 0xE7037ED1A0B428DBull));
    return -log(1.0 - u);
}

/* Philox4x32-10 (Salmon et al., SC'11; the Random123 reference constants).  UNPINNED by the reference, which has
 * no Philox; checked against the published known-answer vectors in tests.  out[4] for a 128-bit counter and a
 * 64-bit key. */
ORC_API void orc_philox4x32_10(const uint32_t ctr[4], const uint32_t key[2], uint32_t out[4]) {
    uint32_t c0 = ctr[0], c1 = ctr[1], c2 = ctr[2], c3 = ctr[3], k0 = key[0], k1 = key[1];
    for (int r = 0; r < 10; ++r) {
        const uint64_t p0 = (uint64_t)0xD2511F53u * c0, p1 = (uint64_t)0xCD9E8D57u * c2;
        const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0, n1 = (uint32_t)p1;
        const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1, n3 = (uint32_t)p0;
        c0 = n0, c1 = n1, c2 = n2, c3 = n3;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    out[0] = c0, out[1] = c1, out[2] = c2, out[3] = c3;
}

/* The build's Philox uniform stream: key = seed (lo, hi), counter = (pos lo, pos hi, row, stream); the uniform
 * is the top 53 bits of (out0 : out1).  UNPINNED (the convention is this build's). */
ORC_API double orc_philox_uniform(uint64_t seed, uint64_t pos_idx, uint32_t row, uint32_t stream) {
    const uint32_t ctr[4] = {(uint32_t)pos_idx, (uint32_t)(pos_idx >> 32), row, stream};
    const uint32_t key[2] = {(uint32_t)seed, (uint32_t)(seed >> 32)};
    uint32_t o[4];
    orc_philox4x32_10(ctr, key, o);
    return top53(((uint64_t)o[0] << 32) | o[1]);
}

/* ------------------------------------------------------------------------------------------------
 * input formats
 * ---------------------------------------------------------------------------------------------- */

/* bf16 -> f32 is exact (a 16-bit left shift).  UNPINNED: the reference reads f32 logits only
 * (kernels/shared/sample_cand_topk_rows.h:11). */
ORC_API void orc_bf16_to_f32(const uint16_t* src, float* dst, size_t n) {
    for (size_t i = 0; i < n; ++i) {
        const uint32_t b = (uint32_t)src[i] << 16;
        memcpy(&dst[i], &b, 4);
    }
}

/* Logit penalties over a row's token history.  UNPINNED: the reference parses presence / frequency penalties
 * and ignores them (src/server/engine_start.cpp:70-73) and has no repetition penalty.  This build's rule, applied
 * to the raw logits before any selection, for every distinct history token t with 0 <= t < V and count c:
 *     l = x[t];  l = (l > 0) ? l / rep : l * rep;  l = l - (pres + freq * (float)c);      (all f32, no fusing)
 * History ids outside [0, V) are skipped.  Returns how many ids were skipped. */
ORC_API int orc_apply_penalties(float* x, uint32_t V, const int32_t* hist, uint32_t hist_len, float rep, float pres,
                                float freq) {
    int skipped = 0;
    uint32_t* cnt = (uint32_t*)calloc(V ? V : 1, sizeof(uint32_t));
    for (uint32_t i = 0; i < hist_len; ++i) {
        if (hist[i] < 0 || (uint32_t)hist[i] >= V) {
            ++skipped;
            continue;
        }
        cnt[hist[i]] += 1;
    }
    for (uint32_t i = 0; i < hist_len; ++i) {
        if (hist[i] < 0 || (uint32_t)hist[i] >= V) continue;
        const uint32_t t = (uint32_t)hist[i];
        const uint32_t c = cnt[t];
        if (c == 0) continue; /* already done for an earlier occurrence */
        cnt[t] = 0;
        volatile float l = x[t];
        l = (l > 0.0f) ? l / rep : l * rep;
        volatile float fc = freq * (float)c;
        volatile float sub = pres + fc;
        l = l - sub;
        x[t] = l;
    }
    free(cnt);
    return skipped;
}

/* ------------------------------------------------------------------------------------------------
 * greedy picks
 * ---------------------------------------------------------------------------------------------- */

/* kernels/shared/block_argmax.h:1-22: every thread starts from best = -inf, idx = 0 and takes x[i] only when x[i] > best
 * (strict), the tree reduction prefers the lower index on ties.  So the result is the first index of the maximum, a NaN
 * logit is never taken (x > best is false for it), and a row with nothing above -inf answers 0.  The host helper of the
 * kernel test (tests/kernels/test_misc.cpp:30-35, firstMax) agrees except when x[0] is NaN, where it stays at 0; the kernel
 * is the behaviour followed here. */
ORC_API int32_t orc_first_max(const float* x, uint32_t n) {
    uint32_t b = 0;
    float best = -INFINITY;
    for (uint32_t i = 0; i < n; ++i)
        if (x[i] > best) best = x[i], b = i;
    return (int32_t)b;
}

/* tests/kernels/test_misc.cpp:37-42 (softmaxTop): probability of the first max at temperature 1 */
ORC_API double orc_softmax_top(const float* x, uint32_t n) {
    const int32_t b = orc_first_max(x, n);
    double s = 0;
    for (uint32_t i = 0; i < n; ++i) s += exp((double)x[i] - x[b]);
    return 1.0 / s;
}

/* kernels/shared/sample_pick_set_tokens.h:60-81 (draft_pick_body): greedy draft r, its probability and the
 * device-side p-min chain cut-off in ctl[0] (drafts kept) / ctl[1] (chain stopped).  prob is the f32 the kernel
 * writes; the oracle computes it as (float)(1 / sum) with the sum in f64. */
ORC_API void orc_draft_pick(const float* x, uint32_t n, int32_t* tok, float* prob, int32_t* ctl, int32_t r,
                            int32_t n_min, float p_min, const int32_t* map) {
    if (r > 0 && ctl[1] != 0) return;
    const int32_t top = orc_first_max(x, n);
    const float p = (float)orc_softmax_top(x, n);
    tok[r] = map ? map[top] : top;
    prob[r] = p;
    if (p_min > 0.f && r >= n_min && p < p_min) {
        ctl[0] = r;
        ctl[1] = 1;
    } else {
        ctl[0] = r + 1;
        if (r == 0) ctl[1] = 0;
    }
}

/* ------------------------------------------------------------------------------------------------
 * candidates
 * ---------------------------------------------------------------------------------------------- */

typedef struct {
    uint32_t id;
    float logit;
    double p;
} orc_cand;

/* The order every host comparator of the path uses: logit descending, id ascending
 * (src/sampling/sampler.cpp:18-21, tests/server/mock_backend.cpp:537-540).  -0.0 == +0.0. */
static int cand_before(const orc_cand* a, const orc_cand* b) {
    if (a->logit != b->logit) return a->logit > b->logit;
    return a->id < b->id;
}
static int cand_cmp(const void* pa, const void* pb) {
    const orc_cand *a = (const orc_cand*)pa, *b = (const orc_cand*)pb;
    if (cand_before(a, b)) return -1;
    if (cand_before(b, a)) return 1;
    return 0;
}

/* keep the k best of x[0..n) in a binary heap whose root is the worst kept candidate */
static void heap_sift(orc_cand* h, uint32_t k, uint32_t i) {
    for (;;) {
        uint32_t w = i;
        const uint32_t l = 2 * i + 1, r = l + 1;
        if (l < k && cand_before(&h[w], &h[l])) w = l;
        if (r < k && cand_before(&h[w], &h[r])) w = r;
        if (w == i) return;
        const orc_cand t = h[i];
        h[i] = h[w];
        h[w] = t;
        i = w;
    }
}

/* The device top-k as the reference's host double states it (tests/server/mock_backend.cpp:523-548,
 * MockModel::topkRows): exact max, sum over the whole row of exp((x - max) * inv_t) accumulated in f64 in index
 * order and cast to f32, and the k best by (logit desc, id asc), written in that order.  out arrays hold
 * min(k, n) entries.  scratch: k candidates. */
static void topk_row(const float* x, uint32_t n, uint32_t k, float inv_t, orc_cand* out, float* m_out, float* sum_out) {
    float m = -INFINITY;
    for (uint32_t i = 0; i < n; ++i) m = x[i] > m ? x[i] : m;
    double sum = 0;
    for (uint32_t i = 0; i < n; ++i) sum += exp((double)(x[i] - m) * inv_t);
    *m_out = m;
    *sum_out = (float)sum;
    const uint32_t kk = k < n ? k : n;
    if (kk == 0) return;
    for (uint32_t i = 0; i < kk; ++i) out[i] = (orc_cand){i, x[i], 0};
    for (uint32_t i = kk / 2; i-- > 0;) heap_sift(out, kk, i);
    for (uint32_t i = kk; i < n; ++i) {
        const orc_cand c = {i, x[i], 0};
        if (cand_before(&c, &out[0])) {
            out[0] = c;
            heap_sift(out, kk, 0);
        }
    }
    qsort(out, kk, sizeof(orc_cand), cand_cmp);
}

ORC_API void orc_topk_rows(const float* x, uint32_t rows, uint32_t n, uint32_t k, float inv_t, int32_t* ids, float* vals,
                           float* stats) {
    orc_cand* c = (orc_cand*)malloc(sizeof(orc_cand) * (k ? k : 1));
    for (uint32_t r = 0; r < rows; ++r) {
        topk_row(x + (size_t)r * n, n, k, inv_t, c, &stats[2 * r], &stats[2 * r + 1]);
        const uint32_t kk = k < n ? k : n;
        for (uint32_t j = 0; j < kk; ++j) {
            ids[(size_t)r * k + j] = (int32_t)c[j].id;
            vals[(size_t)r * k + j] = c[j].logit;
        }
    }
    free(c);
}

/* ------------------------------------------------------------------------------------------------
 * the sampler
 * ---------------------------------------------------------------------------------------------- */

/* The fields of struct Sampler (src/sampling/sampler.h:26-53) the arithmetic reads or writes. */
typedef struct {
    float inv_t;
    uint32_t top_k;
    double top_p, min_p;
    uint64_t seed, pos_idx;
    int32_t race;
    /* row state */
    uint32_t n;
    int32_t closed;
    float m, sum;
    uint32_t full_used, big_used;
    /* where the uniform of an inverse-CDF draw comes from: 0 = the (seed, pos_idx) hash, 1 = u_given */
    int32_t use_u;
    double u_given;
} orc_sampler;

static double sampler_u(const orc_sampler* s) { return s->use_u ? s->u_given : orc_uniform(s->seed, s->pos_idx, 0); }

/* filterCands (src/sampling/sampler.cpp:15-78): sort, probabilities against (m, sum), then top-k, top-p, min-p on the
 * sorted prefix; 0 when the kept set may reach past the candidates. */
static int filter_cands(orc_sampler* s, orc_cand* c, size_t count, int complete) {
    qsort(c, count, sizeof(orc_cand), cand_cmp);
    if (complete) {
        float mx = -INFINITY;
        for (size_t i = 0; i < count; ++i) mx = c[i].logit > mx ? c[i].logit : mx;
        double z = 0;
        for (size_t i = 0; i < count; ++i) z += exp((double)(c[i].logit - mx) * s->inv_t);
        s->m = mx;
        s->sum = (float)z;
    }
    for (size_t i = 0; i < count; ++i) c[i].p = exp((double)(c[i].logit - s->m) * s->inv_t) / (double)s->sum;
    size_t n = count;
    int closed = complete;
    if (s->top_k > 0) {
        if (s->top_k <= count) {
            n = s->top_k;
            closed = 1;
        } else if (!complete) {
            return 0;
        }
    }
    if (s->top_p < 1.0) {
        double z = 1.0;
        if (closed) {
            z = 0;
            for (size_t i = 0; i < n; ++i) z += c[i].p;
        }
        double cum = 0;
        int found = 0;
        for (size_t j = 0; j < n; ++j) {
            cum += c[j].p / z;
            if (cum >= s->top_p) {
                n = j + 1;
                found = 1;
                break;
            }
        }
        if (found) closed = 1;
        else if (!closed) return 0;
    }
    if (s->min_p > 0) {
        const double thr = s->min_p * c[0].p;
        size_t j = 0;
        while (j < n && c[j].p >= thr) ++j;
        if (j == n && !closed) return 0;
        n = j > 1 ? j : 1;
        closed = 1;
    }
    if (closed) {
        double z = 0;
        for (size_t i = 0; i < n; ++i) z += c[i].p;
        for (size_t i = 0; i < n; ++i) c[i].p /= z;
    }
    s->n = (uint32_t)n;
    s->closed = closed;
    return 1;
}

ORC_API int orc_filter_cands(orc_sampler* s, uint32_t* ids, float* logits, double* p, uint32_t count, int complete) {
    orc_cand* c = (orc_cand*)malloc(sizeof(orc_cand) * (count ? count : 1));
    for (uint32_t i = 0; i < count; ++i) c[i] = (orc_cand){ids[i], logits[i], 0};
    const int ok = filter_cands(s, c, count, complete);
    for (uint32_t i = 0; i < count; ++i) ids[i] = c[i].id, logits[i] = c[i].logit, p[i] = c[i].p;
    free(c);
    return ok;
}

/* SampleBuffers::prepareRow (src/server/engine_sampling.cpp:51-84) over a host row: top-ks candidates with the
 * row's (max, sum), then top-kb, then the whole row.  The reference engine uses ks = 256, kb = 16384; its tests use
 * ks = 4, kb = 16 (tests/server/sampling_cases.h:32,69-90).  c holds max(V, kb) candidates. */
static void prepare_row(orc_sampler* s, const float* x, uint32_t V, uint32_t ks, uint32_t kb, orc_cand* c) {
    float m, sum;
    if (ks > V) ks = V;
    topk_row(x, V, ks, s->inv_t, c, &m, &sum);
    s->m = m, s->sum = sum;
    if (filter_cands(s, c, ks, 0)) return;
    s->big_used += 1;
    if (kb > V) kb = V;
    topk_row(x, V, kb, s->inv_t, c, &m, &sum);
    s->m = m, s->sum = sum;
    if (filter_cands(s, c, kb, 0)) return;
    s->full_used += 1;
    for (uint32_t j = 0; j < V; ++j) c[j] = (orc_cand){j, x[j], 0};
    filter_cands(s, c, V, 1);
}

static uint32_t sample_row(orc_sampler* s, const orc_cand* c, const float* x, uint32_t V, int has_ex, uint32_t ex,
                           double p_ex, uint8_t* marks);

/* sampleRace (src/sampling/sampler.cpp:82-106) */
static uint32_t sample_race(orc_sampler* s, const orc_cand* c, const float* x, uint32_t V, uint8_t* marks) {
    if (!s->closed) {
        double S = 0;
        for (uint32_t i = 0; i < s->n; ++i) S += c[i].p;
        if (!(sampler_u(s) < S)) {
            s->race = 0;
            const uint32_t t = sample_row(s, c, x, V, 0, 0, 0, marks);
            s->race = 1;
            return t;
        }
    }
    const uint64_t base = orc_race_base(s->seed, s->pos_idx);
    uint32_t best = c[0].id;
    double bk = INFINITY;
    for (uint32_t i = 0; i < s->n; ++i) {
        if (!(c[i].p > 0)) continue;
        const double k = orc_race_e(base, c[i].id) / c[i].p;
        if (k < bk) bk = k, best = c[i].id;
    }
    return best;
}

/* sampleRow (src/sampling/sampler.cpp:118-147): inverse CDF over the kept candidates, skipping ex; a closed set
 * falls back to its last candidate, an open one walks the rest of the vocabulary in id order. */
static uint32_t sample_row(orc_sampler* s, const orc_cand* c, const float* x, uint32_t V, int has_ex, uint32_t ex,
                           double p_ex, uint8_t* marks) {
    if (s->race && !has_ex) return sample_race(s, c, x, V, marks);
    const double target = sampler_u(s) * (1.0 - p_ex);
    double cum = 0;
    int has_last = 0;
    uint32_t last = 0;
    for (uint32_t i = 0; i < s->n; ++i) {
        if (has_ex && c[i].id == ex) continue;
        cum += c[i].p;
        last = c[i].id, has_last = 1;
        if (cum > target) return c[i].id;
    }
    if (s->closed) return has_last ? last : c[0].id;
    s->full_used += 1;
    memset(marks, 0, V);
    for (uint32_t i = 0; i < s->n; ++i) marks[c[i].id] = 1;
    for (uint32_t j = 0; j < V; ++j) {
        if (marks[j]) continue;
        if (has_ex && j == ex) continue;
        cum += exp((double)(x[j] - s->m) * s->inv_t) / (double)s->sum;
        last = j, has_last = 1;
        if (cum > target) return j;
    }
    return has_last ? last : c[0].id;
}

/* probOf (src/sampling/sampler.cpp:108-116) */
static double prob_of(const orc_sampler* s, const orc_cand* c, const float* x, uint32_t t) {
    for (uint32_t i = 0; i < s->n; ++i)
        if (c[i].id == t) return c[i].p;
    if (s->closed) return 0;
    return exp((double)(x[t] - s->m) * s->inv_t) / (double)s->sum;
}

/* One row through prepareRow + sampleRow.  kept_ids / kept_p (may be null) receive the first min(n, kept_cap)
 * kept candidates in order.  greedy rows (greedy != 0) return the first max and n = 1. */
typedef struct {
    uint32_t token, n;
    int32_t closed;
    float m, sum;
    uint32_t big_used, full_used;
} orc_row_out;

static void sample_one(const float* x, uint32_t V, orc_sampler* s, int greedy, uint32_t ks, uint32_t kb, orc_cand* c,
                       uint8_t* marks, orc_row_out* o, uint32_t* kept_ids, double* kept_p, uint32_t kept_cap) {
    if (greedy) {
        o->token = (uint32_t)orc_first_max(x, V);
        o->n = 1, o->closed = 1, o->m = x[o->token], o->sum = 0, o->big_used = o->full_used = 0;
        if (kept_ids && kept_cap) kept_ids[0] = o->token;
        if (kept_p && kept_cap) kept_p[0] = 1.0;
        return;
    }
    s->big_used = s->full_used = 0;
    prepare_row(s, x, V, ks, kb, c);
    const uint32_t nk = s->n < kept_cap ? s->n : kept_cap;
    for (uint32_t i = 0; i < nk; ++i) {
        if (kept_ids) kept_ids[i] = c[i].id;
        if (kept_p) kept_p[i] = c[i].p;
    }
    o->n = s->n, o->closed = s->closed, o->m = s->m, o->sum = s->sum;
    o->token = sample_row(s, c, x, V, 0, 0, 0, marks);
    o->big_used = s->big_used, o->full_used = s->full_used;
}

/* Batch parameters, one entry per row (null pointer = the default in brackets). */
typedef struct {
    const float* inv_t;      /* [1] */
    const uint32_t* top_k;   /* [0 = off] */
    const double* top_p;     /* [1] */
    const double* min_p;     /* [0] */
    const uint8_t* greedy;   /* [0] */
    const uint8_t* race;     /* [0] */
    const uint64_t* seed;    /* [0] */
    const uint64_t* pos_idx; /* [0] */
    const double* u;         /* inverse-CDF uniform per row; null = the (seed, pos_idx) hash */
    /* penalties (UNPINNED); hist rows of hist_stride ids, hist_len[r] valid */
    const int32_t* hist;
    const uint32_t* hist_len;
    uint64_t hist_stride;
    const float* rep;  /* [1] */
    const float* pres; /* [0] */
    const float* freq; /* [0] */
    uint32_t ks, kb;   /* escalation sizes, the engine's 256 / 16384 */
} orc_batch;

typedef struct {
    const float* x;
    const uint16_t* xb; /* bf16 rows when x is null */
    uint32_t rows, V;
    const orc_batch* b;
    orc_row_out* out;
    uint32_t* kept_ids;
    double* kept_p;
    uint32_t kept_cap;
    uint32_t r0, r1;
} job_t;

static void* job_run(void* arg) {
    job_t* j = (job_t*)arg;
    const orc_batch* b = j->b;
    const uint32_t V = j->V;
    const uint32_t kb = b->kb ? b->kb : 16384, ks = b->ks ? b->ks : 256;
    orc_cand* c = (orc_cand*)malloc(sizeof(orc_cand) * (V > kb ? V : kb));
    uint8_t* marks = (uint8_t*)malloc(V ? V : 1);
    float* tmp = (float*)malloc(sizeof(float) * (V ? V : 1));
    for (uint32_t r = j->r0; r < j->r1; ++r) {
        const float* x;
        int own = 0;
        if (j->x) x = j->x + (size_t)r * V;
        else {
            orc_bf16_to_f32(j->xb + (size_t)r * V, tmp, V);
            x = tmp, own = 1;
        }
        const float rep = b->rep ? b->rep[r] : 1.f, pres = b->pres ? b->pres[r] : 0.f, freq = b->freq ? b->freq[r] : 0.f;
        if (b->hist && b->hist_len && b->hist_len[r] > 0 && (rep != 1.f || pres != 0.f || freq != 0.f)) {
            if (!own) {
                memcpy(tmp, x, sizeof(float) * V);
                x = tmp;
            }
            orc_apply_penalties(tmp, V, b->hist + (size_t)r * b->hist_stride, b->hist_len[r], rep, pres, freq);
        }
        orc_sampler s;
        memset(&s, 0, sizeof s);
        s.inv_t = b->inv_t ? b->inv_t[r] : 1.f;
        s.top_k = b->top_k ? b->top_k[r] : 0;
        s.top_p = b->top_p ? b->top_p[r] : 1.0;
        s.min_p = b->min_p ? b->min_p[r] : 0.0;
        s.seed = b->seed ? b->seed[r] : 0;
        s.pos_idx = b->pos_idx ? b->pos_idx[r] : 0;
        s.race = b->race ? b->race[r] : 0;
        if (b->u) s.use_u = 1, s.u_given = b->u[r];
        sample_one(x, V, &s, b->greedy ? b->greedy[r] : 0, ks, kb, c, marks, &j->out[r],
                   j->kept_ids ? j->kept_ids + (size_t)r * j->kept_cap : 0, j->kept_p ? j->kept_p + (size_t)r * j->kept_cap : 0,
                   j->kept_cap);
    }
    free(tmp);
    free(marks);
    free(c);
    return 0;
}

/* rows x V logits (f32 in x, or bf16 in xb when x is null) -> one orc_row_out per row, on `threads` host threads
 * (rows split evenly; rows are independent). */
ORC_API void orc_sample_rows(const float* x, const uint16_t* xb, uint32_t rows, uint32_t V, const orc_batch* b,
                             orc_row_out* out, uint32_t* kept_ids, double* kept_p, uint32_t kept_cap, int threads) {
    if (threads < 1) threads = 1;
    if ((uint32_t)threads > rows) threads = rows ? (int)rows : 1;
    pthread_t* th = (pthread_t*)malloc(sizeof(pthread_t) * threads);
    job_t* jobs = (job_t*)malloc(sizeof(job_t) * threads);
    for (int t = 0; t < threads; ++t) {
        jobs[t] = (job_t){x, xb, rows, V, b, out, kept_ids, kept_p, kept_cap, (uint32_t)((uint64_t)rows * t / threads),
                          (uint32_t)((uint64_t)rows * (t + 1) / threads)};
        if (t > 0) pthread_create(&th[t], 0, job_run, &jobs[t]);
    }
    job_run(&jobs[0]);
    for (int t = 1; t < threads; ++t) pthread_join(th[t], 0);
    free(jobs);
    free(th);
}

/* ------------------------------------------------------------------------------------------------
 * draft distribution and the coupled race (speculative sampling, current reference rule)
 * ---------------------------------------------------------------------------------------------- */

#define ORC_QMAX 32   /* include/whirl/spec_sample.h:40 */
#define ORC_QWORDS 72 /* include/whirl/spec_sample.h:43 */

typedef struct {
    uint32_t n;
    uint32_t id[ORC_QMAX];
    float p[ORC_QMAX];
} orc_qdist;

/* draftDist (src/common/spec_sample.cpp:33-81): the device q filter in f32, same operation order. */
ORC_API void orc_draft_dist(const uint32_t* ids, const float* logits, uint32_t count, float m, float sum, float inv_t,
                            uint32_t top_k, float top_p, float min_p, orc_qdist* q) {
    memset(q, 0, sizeof *q);
    const uint32_t K = count < ORC_QMAX ? count : ORC_QMAX;
    float lg[ORC_QMAX];
    for (uint32_t i = 0; i < K; ++i) q->id[i] = ids[i], lg[i] = logits[i];
    for (uint32_t i = 1; i < K; ++i) {
        uint32_t j = i;
        while (j > 0 && (lg[j - 1] < lg[j] || (lg[j - 1] == lg[j] && q->id[j - 1] > q->id[j]))) {
            const float tl = lg[j - 1];
            lg[j - 1] = lg[j], lg[j] = tl;
            const uint32_t ti = q->id[j - 1];
            q->id[j - 1] = q->id[j], q->id[j] = ti;
            --j;
        }
    }
    for (uint32_t i = 0; i < K; ++i) {
        volatile float a = (lg[i] - m);
        a = a * inv_t;
        q->p[i] = expf(a) / sum;
    }
    uint32_t n = K;
    const int closed = top_k > 0 && top_k <= K;
    if (closed) n = top_k;
    if (top_p < 1.f) {
        volatile float z = 1.f;
        if (closed) {
            z = 0.f;
            for (uint32_t i = 0; i < n; ++i) z = z + q->p[i];
        }
        volatile float cum = 0.f;
        for (uint32_t j = 0; j < n; ++j) {
            cum = cum + q->p[j] / z;
            if (cum >= top_p) {
                n = j + 1;
                break;
            }
        }
    }
    if (min_p > 0.f && n > 0) {
        const float thr = min_p * q->p[0];
        uint32_t j = 0;
        while (j < n && q->p[j] >= thr) ++j;
        n = j > 1 ? j : 1;
    }
    volatile float z = 0.f;
    for (uint32_t i = 0; i < n; ++i) z = z + q->p[i];
    for (uint32_t i = 0; i < n; ++i) q->p[i] = q->p[i] / z;
    q->n = n;
}

/* spec::sampleRace (src/common/spec_sample.cpp:89-101) */
ORC_API uint32_t orc_spec_sample_race(const orc_qdist* q, uint64_t base) {
    uint32_t best = q->n > 0 ? q->id[0] : 0;
    double bk = INFINITY;
    for (uint32_t i = 0; i < q->n; ++i) {
        if (!(q->p[i] > 0.f)) continue;
        const double k = orc_race_e(base, q->id[i]) / (double)q->p[i];
        if (k < bk) bk = k, best = q->id[i];
    }
    return best;
}

/* draft_sample_rows for one row (kernels/spec_sample.hip:34-205) as its kernel test states it
 * (tests/kernels/test_misc.cpp:357-417): K = draftCands(top_k) best logits (NaN as -inf), m / sum over the row in
 * f64 cast to f32, q = draftDist, token = race draw; words receives the 72-word q entry.  map may be null. */
ORC_API uint32_t orc_draft_sample_row(const float* x, uint32_t n, const int32_t* map, uint32_t top_k, float inv_t,
                                      float top_p, float min_p, uint64_t race_key, int32_t* words) {
    float* xc = (float*)malloc(sizeof(float) * n);
    for (uint32_t i = 0; i < n; ++i) xc[i] = x[i] == x[i] ? x[i] : -INFINITY;
    uint32_t K = (top_k > 0 && top_k < ORC_QMAX) ? top_k : ORC_QMAX; /* draftCands, include/whirl/spec_sample.h:94 */
    if (K > n) K = n;
    orc_cand c[ORC_QMAX];
    float m, sum;
    topk_row(xc, n, K, inv_t, c, &m, &sum);
    uint32_t ids[ORC_QMAX];
    float lg[ORC_QMAX];
    for (uint32_t i = 0; i < K; ++i) ids[i] = map ? (uint32_t)map[c[i].id] : c[i].id, lg[i] = c[i].logit;
    orc_qdist q;
    orc_draft_dist(ids, lg, K, m, sum, inv_t, top_k, top_p, min_p, &q);
    if (words) {
        memset(words, 0, 4 * ORC_QWORDS);
        words[0] = (int32_t)q.n;
        for (uint32_t i = 0; i < q.n; ++i) {
            words[1 + i] = (int32_t)q.id[i];
            memcpy(&words[1 + ORC_QMAX + i], &q.p[i], 4);
        }
    }
    free(xc);
    return orc_spec_sample_race(&q, race_key);
}

/* ------------------------------------------------------------------------------------------------
 * relaxed acceptance rules (include/whirl/relax_accept.h)
 * ---------------------------------------------------------------------------------------------- */

typedef struct {
    int32_t on;
    uint32_t k;
    float alpha, eps, delta;
} orc_relax;

static uint32_t relax_topk(const orc_relax* p) { return p->k < 1 ? 1 : (p->k > 16 ? 16 : p->k); } /* :49 */

/* acceptGreedy (include/whirl/relax_accept.h:55-73) */
ORC_API int orc_relax_accept_greedy(const orc_relax* p, const int32_t* ids, const float* logits, uint32_t n, float m,
                                    uint32_t draft) {
    uint32_t at = n;
    for (uint32_t i = 0; i < n; ++i)
        if ((uint32_t)ids[i] == draft) {
            at = i;
            break;
        }
    if (at == n) return 0;
    const float ld = logits[at];
    uint32_t rank = 0;
    for (uint32_t i = 0; i < n; ++i) {
        if (i == at) continue;
        if (logits[i] > ld || (logits[i] == ld && (uint32_t)ids[i] < draft)) ++rank;
    }
    if (rank >= relax_topk(p)) return 0;
    return exp((double)ld - (double)m) >= (double)p->alpha;
}

/* extendsRepeat (include/whirl/relax_accept.h:78-90), n-gram 6 over the last 4096 tokens */
ORC_API int orc_relax_extends_repeat(const uint32_t* hist, size_t hist_n, const uint32_t* tail, size_t tail_n, size_t ng,
                                     size_t window) {
    const size_t hn = hist_n < window ? hist_n : window;
    const size_t s = hn + tail_n;
    if (s < ng + 1) return 0;
#define AT(i) ((i) < hn ? hist[hist_n - hn + (i)] : tail[(i)-hn])
    for (size_t i = 0; i + ng < s; ++i) {
        size_t j = 0;
        while (j < ng && AT(i + j) == AT(s - ng + j)) ++j;
        if (j == ng) return 1;
    }
#undef AT
    return 0;
}

/* acceptTypical (include/whirl/relax_accept.h:93-96) */
ORC_API int orc_relax_accept_typical(const orc_relax* p, double p_draft, double h) {
    return p_draft >= fmin((double)p->eps, (double)p->delta * exp(-h));
}

/* ------------------------------------------------------------------------------------------------
 * draft acceptance (src/sampling/acceptor.cpp)
 * ---------------------------------------------------------------------------------------------- */

typedef struct {
    uint32_t acc, chosen, relaxed;
    double relax_gap;
    uint64_t pos_idx;
    uint32_t full_used, big_used;
} orc_accepted;

/* Acceptor::greedy (src/sampling/acceptor.cpp:30-61).  relax_host: [max_rows*k] i32 ids | [max_rows*k] f32 logits |
 * [max_rows*2] f32 (max, sum).  hist / next: the repeat guard's inputs (Engine::relaxRepeats as the tests state it,
 * tests/sampling/sampling_unit.inc:113-118). */
ORC_API void orc_accept_greedy(const int32_t* argmax, const uint32_t* dr, uint32_t nd, uint32_t row0, int relax,
                               const orc_relax* rp, const uint8_t* relax_host, uint32_t max_rows, const uint32_t* hist,
                               size_t hist_n, uint32_t next, orc_accepted* out) {
    const uint32_t rk = relax_topk(rp);
    uint32_t acc = 0;
    out->relaxed = 0, out->relax_gap = 0;
    while (acc < nd) {
        if ((uint32_t)argmax[acc] == dr[acc]) {
            ++acc;
            continue;
        }
        if (!relax) break;
        const size_t gr = row0 + acc;
        const int32_t* rids = (const int32_t*)relax_host + gr * rk;
        const float* rvals = (const float*)(relax_host + (size_t)max_rows * rk * 4) + gr * rk;
        const float* rst = (const float*)(relax_host + (size_t)max_rows * rk * 8);
        uint32_t tail[32];
        tail[0] = next;
        for (uint32_t r = 0; r <= acc; ++r) tail[r + 1] = dr[r];
        if (!orc_relax_accept_greedy(rp, rids, rvals, rk, rst[2 * gr], dr[acc]) ||
            orc_relax_extends_repeat(hist, hist_n, tail, acc + 2, 6, 4096))
            break;
        for (uint32_t j = 0; j < rk; ++j)
            if ((uint32_t)rids[j] == dr[acc]) out->relax_gap += (double)(rst[2 * gr] - rvals[j]);
        ++acc;
        out->relaxed += 1;
    }
    out->acc = acc;
    out->chosen = (uint32_t)argmax[acc];
    out->pos_idx = 0, out->full_used = out->big_used = 0;
}

/* Acceptor::sample (src/sampling/acceptor.cpp:63-100) over host verify rows (rows[row0 + r] is verify row r):
 * prepareRow -> pos_idx = n_gen + acc -> typical check -> draw; accept iff the draw equals the draft. */
ORC_API void orc_accept_sample(const float* rows, uint32_t V, orc_sampler* sm, const uint32_t* dr, uint32_t nd,
                               uint32_t row0, int typ, uint32_t n_gen, const orc_relax* rp, const uint32_t* hist,
                               size_t hist_n, uint32_t next, uint32_t ks, uint32_t kb, orc_accepted* out) {
    orc_cand* c = (orc_cand*)malloc(sizeof(orc_cand) * (V > kb ? V : kb));
    uint8_t* marks = (uint8_t*)malloc(V ? V : 1);
    uint32_t acc = 0;
    out->relaxed = 0, out->relax_gap = 0;
    sm->big_used = sm->full_used = 0;
    for (;;) {
        const float* x = rows + (size_t)(row0 + acc) * V;
        prepare_row(sm, x, V, ks, kb, c);
        sm->pos_idx = (uint64_t)n_gen + acc;
        if (typ && acc < nd) {
            const double pd = prob_of(sm, c, x, dr[acc]);
            double h = 0;
            for (uint32_t i = 0; i < sm->n; ++i)
                if (c[i].p > 0) h -= c[i].p * log(c[i].p);
            uint32_t tail[32];
            tail[0] = next;
            for (uint32_t r = 0; r <= acc; ++r) tail[r + 1] = dr[r];
            if (orc_relax_accept_typical(rp, pd, h) && !orc_relax_extends_repeat(hist, hist_n, tail, acc + 2, 6, 4096)) {
                ++acc;
                out->relaxed += 1;
                continue;
            }
        }
        const uint32_t t = sample_row(sm, c, x, V, 0, 0, 0, marks);
        if (acc < nd && t == dr[acc]) {
            ++acc;
            continue;
        }
        out->chosen = t;
        break;
    }
    out->acc = acc;
    out->pos_idx = sm->pos_idx, out->full_used = sm->full_used, out->big_used = sm->big_used;
    free(marks);
    free(c);
}

/* ------------------------------------------------------------------------------------------------
 * accept / residual speculative sampling (UNPINNED)
 * ---------------------------------------------------------------------------------------------- */

/* The rule BASELINE config 3 names (Leviathan et al. / Chen et al. 2023), which the reference removed
 * (include/whirl/spec_sample.h:21-24).  This build's statement, per sequence with L drafts, full-vocabulary
 * p = softmax(target * inv_t), q = softmax(draft * inv_t), both in f64 as exp((double)(x - max) * inv_t) / sum with the
 * f64 sum accumulated in index order:
 *   for j = 0..L-1:  accept draft d_j iff u_acc[j] * q(d_j) < p(d_j)  (q(d_j) == 0 accepts);
 *                    on the first rejection draw from r(v) = max(0, p(v) - q(v)) by inverse CDF in id order:
 *                    the first v with cum_r(v) > u_res[j] * sum_r (last v with r(v) > 0 as the fallback; d_j's own
 *                    argmax-of-p fallback when sum_r == 0) and stop;
 *   all accepted:    the bonus token from target row L by inverse CDF in id order: first v with cum_p(v) > u_res[L].
 * target: (L+1) rows, draft: L rows, each V wide.  The deterministic-draft case (q a point mass) reduces to the
 * reference's residual helper sampleRow(src, s, ex, p_ex) (src/sampling/sampler.cpp:118-131) on a closed full row. */
static void softmax_stats(const float* x, uint32_t V, float inv_t, float* m_out, double* z_out) {
    float m = -INFINITY;
    for (uint32_t i = 0; i < V; ++i) m = x[i] > m ? x[i] : m;
    double z = 0;
    for (uint32_t i = 0; i < V; ++i) z += exp((double)(x[i] - m) * inv_t);
    *m_out = m, *z_out = z;
}

ORC_API void orc_spec_accept_residual(const float* target, const float* draft, uint32_t V, uint32_t L,
                                      const int32_t* draft_tok, float inv_t, const double* u_acc, const double* u_res,
                                      uint32_t* n_acc, uint32_t* next_tok) {
    uint32_t acc = 0;
    for (; acc < L; ++acc) {
        const float *t = target + (size_t)acc * V, *d = draft + (size_t)acc * V;
        float mp, mq;
        double zp, zq;
        softmax_stats(t, V, inv_t, &mp, &zp);
        softmax_stats(d, V, inv_t, &mq, &zq);
        const uint32_t tok = (uint32_t)draft_tok[acc];
        const double p = exp((double)(t[tok] - mp) * inv_t) / zp, q = exp((double)(d[tok] - mq) * inv_t) / zq;
        if (u_acc[acc] * q < p || q == 0) continue;
        double sr = 0;
        for (uint32_t v = 0; v < V; ++v) {
            const double r = exp((double)(t[v] - mp) * inv_t) / zp - exp((double)(d[v] - mq) * inv_t) / zq;
            if (r > 0) sr += r;
        }
        uint32_t pick = (uint32_t)orc_first_max(t, V);
        if (sr > 0) {
            const double targ = u_res[acc] * sr;
            double cum = 0;
            for (uint32_t v = 0; v < V; ++v) {
                const double r = exp((double)(t[v] - mp) * inv_t) / zp - exp((double)(d[v] - mq) * inv_t) / zq;
                if (!(r > 0)) continue;
                cum += r;
                pick = v;
                if (cum > targ) break;
            }
        }
        *n_acc = acc, *next_tok = pick;
        return;
    }
    const float* t = target + (size_t)L * V;
    float mp;
    double zp;
    softmax_stats(t, V, inv_t, &mp, &zp);
    double cum = 0;
    uint32_t pick = 0;
    for (uint32_t v = 0; v < V; ++v) {
        cum += exp((double)(t[v] - mp) * inv_t) / zp;
        pick = v;
        if (cum > u_res[L]) break;
    }
    *n_acc = L, *next_tok = pick;
}

/* ------------------------------------------------------------------------------------------------
 * vocab-sharded candidates (UNPINNED)
 * ---------------------------------------------------------------------------------------------- */

/* Merge of per-shard top-ks candidates for one row: shard s holds ks ids (already global), logits and its local
 * (max m_s, sum_s = sum exp((x - m_s) * inv_t)).  The merged row statistics are m = max m_s and
 * sum = (float) sum_s sum_s * exp((double)(m_s - m) * inv_t); the merged candidates are the k best of the union by
 * (logit desc, id asc).  Exact whenever ks >= min(k, shard width). */
ORC_API void orc_merge_shards(const int32_t* ids, const float* vals, const float* stats, uint32_t shards, uint32_t ks,
                              uint32_t k, float inv_t, int32_t* out_ids, float* out_vals, float* out_stats) {
    const uint32_t tot = shards * ks;
    orc_cand* c = (orc_cand*)malloc(sizeof(orc_cand) * (tot ? tot : 1));
    float m = -INFINITY;
    for (uint32_t s = 0; s < shards; ++s) m = stats[2 * s] > m ? stats[2 * s] : m;
    double z = 0;
    for (uint32_t s = 0; s < shards; ++s) z += (double)stats[2 * s + 1] * exp((double)(stats[2 * s] - m) * inv_t);
    for (uint32_t i = 0; i < tot; ++i) c[i] = (orc_cand){(uint32_t)ids[i], vals[i], 0};
    qsort(c, tot, sizeof(orc_cand), cand_cmp);
    const uint32_t kk = k < tot ? k : tot;
    for (uint32_t i = 0; i < kk; ++i) out_ids[i] = (int32_t)c[i].id, out_vals[i] = c[i].logit;
    out_stats[0] = m, out_stats[1] = (float)z;
    free(c);
}

/* sizes of the structs above, for the ctypes mirror */
ORC_API void orc_sizes(uint32_t out[8]) {
    out[0] = sizeof(orc_sampler);
    out[1] = sizeof(orc_row_out);
    out[2] = sizeof(orc_batch);
    out[3] = sizeof(orc_qdist);
    out[4] = sizeof(orc_accepted);
    out[5] = sizeof(orc_relax);
    out[6] = sizeof(orc_cand);
    out[7] = 0;
}
