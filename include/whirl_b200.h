/*
 * whirl_b200: the token-sampling hot path of WHIRL for NVIDIA B200 (sm_100a), behind a C ABI.
 *
 * Every entry point is stream-ordered and asynchronous unless it says otherwise, never allocates, never throws and
 * never aborts: it returns a WHIRL_* status, and whirl_last_error() gives a message for the calling thread.  The
 * caller owns all buffers (device pointers unless a name says host) and passes a workspace sized by
 * whirl_workspace_bytes().  One CUDA context per GPU; calls on different streams may overlap when their workspaces
 * differ.  `stream` is a cudaStream_t.  Logits rows are dense: row r starts at x + r * n elements.
 *
 * Each declaration names the reference interface it stands in for (paths relative to the reference project).
 */
#ifndef WHIRL_B200_H
#define WHIRL_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* status codes (the reference throws hip::Error / std::invalid_argument instead, include/whirl/hip.h:31-40) */
enum {
    WHIRL_OK = 0,
    WHIRL_ERR_INVALID = 1,     /* a bad argument: null pointer, negative size, K out of range ... */
    WHIRL_ERR_CUDA = 2,        /* a CUDA call failed; whirl_last_error() has its text */
    WHIRL_ERR_WORKSPACE = 3,   /* workspace missing or too small */
    WHIRL_ERR_UNSUPPORTED = 4, /* a documented limit was exceeded */
    WHIRL_ERR_TIMEOUT = 5      /* a bounded device-side wait ran out (reported through the error word) */
};

/* element type of the logits */
enum { WHIRL_F32 = 0, WHIRL_BF16 = 1 };

/* per-row outcome written by whirl_sample_rows */
enum {
    WHIRL_ROW_DONE = 0,      /* token drawn */
    WHIRL_ROW_ESCALATE = 1,  /* the kept set may reach past 16384 candidates and the whole-row level could not run (a row of
                                more than 2^20 logits, or no scratch area came free in time): not answered */
    WHIRL_ROW_OPEN_TAIL = 2  /* open set whose draw fell past the candidates; whirl_sample_rows walks the row itself, so this
                                is only seen from whirl_merge_sample_rows (no row to walk there) */
};

/* indices into the counters array of whirl_sample_rows */
enum {
    WHIRL_CNT_ESCALATED = 0, /* rows that needed the second candidate level (the reference's Sampler::big_used) */
    WHIRL_CNT_OPEN_TAIL = 1, /* rows whose draw walked the row in id order (Sampler::full_used) */
    WHIRL_CNT_UNRESOLVED = 2,/* rows left with a status other than WHIRL_ROW_DONE */
    WHIRL_CNT_TIMEOUT = 3,   /* calls in which a bounded device-side wait ran out (whirl_check names the wait) */
    WHIRL_CNT_REDO = 4,      /* rows the single-pass kernel handed to the multi-pass kernel to do again: more candidates
                                than its log holds, a NaN in a sum, an open-set walk, or a row a wait that ran out left
                                unanswered */
    WHIRL_CNT_NAN_ROWS = 5,  /* rows of those in which a NaN logit met the normaliser */
    WHIRL_CNT_WORDS = 8
};

/* limits */
#define WHIRL_MAX_K 16384        /* candidates per row of whirl_topk_rows (the reference's k_big) */
#define WHIRL_STREAM_MAX_K 1024  /* top_k served by the single-pass kernel; larger values take the multi-pass one */
#define WHIRL_MAX_HIST 4096      /* history ids per row for the penalties */
#define WHIRL_Q_WORDS 72         /* i32 words of one draft-distribution entry (include/whirl/spec_sample.h:43) */
#define WHIRL_Q_MAX 32           /* support of a draft distribution (include/whirl/spec_sample.h:40) */
#define WHIRL_CTL_WORDS 64       /* i32 words of one sequence's control area (include/whirl/model_types.h:55-61) */

typedef struct whirl_sample_params whirl_sample_params;
typedef struct whirl_sample_out whirl_sample_out;

const char* whirl_status_string(int status);
const char* whirl_last_error(void);
int whirl_version(void);

/* Kernel launches this process has made through the library so far, per family: [0] greedy picks, [1] multi-pass
 * selection, [2] single-pass sampler, [3] small helper kernels.  Fills min(n, 4) entries.  (The reference logs launches
 * with WHIRL_LAUNCH_LOG, src/hip/launch_log.h.) */
void whirl_launch_counts(uint64_t* out, int n);

/* Bytes of workspace that cover every entry point below for batches of up to `rows` rows of `n` logits. */
size_t whirl_workspace_bytes(int rows, int n);

/* ------------------------------------------------------------------------------------------------------------------
 * Greedy picks.  Same results as the reference kernels: the first index of the maximum.
 * ---------------------------------------------------------------------------------------------------------------- */

/* argmax(x, n, out, ids, pos, advance): kernels/shared/misc_kv_argmax_kv_store.h:32-42 (launch: src/model/qwen35/
 * forward/run.cpp:59,66).  out[0] = ids[0] = first max of x[0..n); pos[0] += advance.  ids / pos may be null. */
int whirl_argmax(const void* x, int dtype, int n, int* out, int* ids, int* pos, int advance, void* ws, size_t ws_bytes,
                 void* stream);

/* argmax_rows(x, n, out), grid = rows: kernels/shared/sample_pick_set_tokens.h:15-21. */
int whirl_argmax_rows(const void* x, int dtype, int rows, int n, int* out, void* ws, size_t ws_bytes, void* stream);

/* argmax_rows_to(x, n, out, RowIdx dst): kernels/shared/sample_pick_set_tokens.h:47-53.  out[dst[row]] = first max.
 * dst is a device array of `rows` ints (the reference passes 32 of them by value). */
int whirl_argmax_rows_to(const void* x, int dtype, int rows, int n, int* out, const int* dst, void* ws, size_t ws_bytes,
                         void* stream);

/* argmax_prob(x, n, out_tok, out_prob): kernels/shared/sample_pick_set_tokens.h:96-105; here for `rows` rows:
 * out_tok[row] = first max, out_prob[row] = 1 / sum exp(x - max). */
int whirl_argmax_prob(const void* x, int dtype, int rows, int n, int* out_tok, float* out_prob, void* ws, size_t ws_bytes,
                      void* stream);

/* draft_pick(x, n, tok, prob, ctl, r, n_min, p_min, map): kernels/shared/sample_pick_set_tokens.h:60-86.  Greedy draft r
 * (through map when given), its probability, and the p-min chain cut-off in ctl[0] (drafts kept) / ctl[1] (stopped). */
int whirl_draft_pick(const void* x, int dtype, int n, int* tok, float* prob, int* ctl, int r, int n_min, float p_min,
                     const int* map, void* ws, size_t ws_bytes, void* stream);

/* draft_pick_rows(x, n, ctl_all, RowIdx area, r, n_min, p_min, map): kernels/shared/sample_pick_set_tokens.h:88-92.  Row b
 * writes into the control area at ctl_all + area[b]: words [16,32) tokens, [32,48) probabilities, 48 / 49 the cut-off.
 * area is a device array of `rows` ints. */
int whirl_draft_pick_rows(const void* x, int dtype, int rows, int n, int* ctl_all, const int* area, int r, int n_min,
                          float p_min, const int* map, void* ws, size_t ws_bytes, void* stream);

/* The greedy pick of whirl_argmax_rows without a workspace and without any allocation.  No counterpart in the reference.
 * It is for hosts that cannot give the library device memory at call time: an engine that fixes its whole memory plan at
 * start-up and bans cudaMalloc afterwards, or a call site with no workspace pointer to pass.  The scratch that splits a row
 * over several thread blocks sits in a fixed array inside the library (about 257 KiB on every GPU that loads it, held
 * until the process exits), sized for at most WHIRL_STATIC_MAX_ROWS rows; more rows are refused with
 * WHIRL_ERR_UNSUPPORTED.  The first call on each device looks the array's device address up (make that call before any
 * stream capture begins).  All calls share the one array, which keeps the previous call's contents (the call clears the
 * part that must start at zero): two calls that overlap on the GPU, on different streams, race on it. */
#define WHIRL_STATIC_MAX_ROWS 256
int whirl_argmax_rows_static(const void* x, int dtype, int rows, int n, int* out, void* stream);

/* draft_sample_rows(x, n, ctl_all, RowIdx area, r, map, DSampArgs a, qbuf): kernels/spec_sample.hip:34-205 (launch:
 * src/model/qwen35/forward/mtp_verify.cpp:344).  Rows with on != 0 replace their greedy draft r by a token drawn from the
 * draft distribution q by the race coupled to the target sampler: q = softmax at the request temperature over the
 * min(top_k, 32) largest logits (32 when top_k is 0; NaN logits never ahead of numbers), then top-k / top-p / min-p in
 * f32, renormalised; token = argmin E(id) / q.  Writes the token to word 16 + r of the row's control area and q
 * ([n | ids[32] | p bits[32]], WHIRL_Q_WORDS words) to qbuf + qoff[row].  A row whose chain was stopped by the p-min
 * cut-off at or before r (words 48 / 49) is skipped.  The reference's by-value DSampArgs of eight 32-entry arrays
 * (kernels/kernel_args.h:55-66) becomes eight device arrays of `rows` entries. */
typedef struct whirl_dsamp_args {
    const int32_t* on;
    const int32_t* top_k;
    const int32_t* qoff;
    const float* inv_t;
    const float* top_p;
    const float* min_p;
    const uint32_t* key_lo; /* spec::raceBase(seed, output index of draft r), include/whirl/spec_sample.h:58-60 */
    const uint32_t* key_hi;
} whirl_dsamp_args;
int whirl_draft_sample_rows(const void* x, int dtype, int rows, int n, int* ctl_all, const int* area, int r, const int* map,
                            const whirl_dsamp_args* args, int* qbuf, void* stream);

/* ------------------------------------------------------------------------------------------------------------------
 * Candidates.
 * ---------------------------------------------------------------------------------------------------------------- */

/* topk_rows(x, n, K, inv_t, ids, vals, stats), grid = rows: kernels/shared/sample_cand_topk_rows.h:11-98; the device
 * seam ServerModel::topkRows (src/server/backend.h:96-99).  ids / vals [rows][K], stats [rows][2] = {max,
 * sum exp((x - max) * inv_t)}.  The K candidates are exactly the K best by (logit desc, id asc), the order of the
 * host comparators, and come out in that order (the reference leaves them unordered and fills ties at the K-th logit
 * in arrival order).  K <= min(n, WHIRL_MAX_K) entries per row are written when K > n.  inv_t_rows (device, may be
 * null) overrides inv_t per row. */
int whirl_topk_rows(const void* x, int dtype, int rows, int n, int K, float inv_t, const float* inv_t_rows, int* ids,
                    float* vals, float* stats, void* ws, size_t ws_bytes, void* stream);

/* ------------------------------------------------------------------------------------------------------------------
 * Vocab-sharded logits (the output of a tensor-parallel lm_head).  No counterpart in the reference, which runs on one GPU
 * (include/whirl/gpu_select.h:23-25 leaves multi-GPU for later).
 * ---------------------------------------------------------------------------------------------------------------- */

/* whirl_topk_rows on one vocabulary slice: x is [rows][n] with n the slice width; every id written is id_offset + the
 * index inside the slice, i.e. a global token id.  Entries beyond min(K, n) are left untouched: pre-fill ids with -1. */
int whirl_topk_rows_shard(const void* x, int dtype, int rows, int n, int K, int id_offset, float inv_t, const float* inv_t_rows,
                          int* ids, float* vals, float* stats, void* ws, size_t ws_bytes, void* stream);

/* Merge the slices' candidates and sample: ids / vals are [shards][rows][K_s] and stats [shards][rows][2], the layout an
 * all-gather of each rank's whirl_topk_rows_shard outputs produces.  Row statistics merge as m = max m_s,
 * sum = sum_s sum_s * exp((m_s - m) * inv_t); the candidates are the global min(top_k, K_s) best (exact, because the
 * global K best lie inside the union of the slices' K_s best when K <= K_s), then top-k / top-p / min-p and the draw as
 * in whirl_sample_rows.  A row whose kept set may reach past K_s candidates comes back WHIRL_ROW_ESCALATE.
 * Limits: K_s <= 1024, shards * K_s <= 16384; penalties (params->hist) are not accepted here. */
int whirl_merge_sample_rows(const int* ids, const float* vals, const float* stats, int shards, int rows, int K_s, int n_total,
                            const whirl_sample_params* params, const whirl_sample_out* out, void* stream);

/* The same merge on PACKED blocks.  One rank's block is whirl_shard_block_words(rows, K_s) 4-byte words:
 *     ids [rows][K_s] i32 | vals [rows][K_s] f32 | stats [rows][2] f32
 * A rank points whirl_topk_rows_shard's three outputs into its own block and all-gathers the blocks with one collective
 * (ncclAllGather / all_gather_into_tensor) into `blocks` = [shards] blocks, which this call reads in place: no
 * repacking copy on either side of the exchange. */
size_t whirl_shard_block_words(int rows, int K_s);
int whirl_merge_sample_rows_packed(const void* blocks, int shards, int rows, int K_s, int n_total, const whirl_sample_params* params,
                                   const whirl_sample_out* out, void* stream);

/* ------------------------------------------------------------------------------------------------------------------
 * The fused sampler: penalties -> candidates -> top-k / top-p / min-p -> draw, one token per row, all on the device.
 * It replaces the round trip topk_rows -> download -> sampling::filterCands -> sampling::sampleRow
 * (src/server/engine_decode.cpp:383-406, src/server/engine_sampling.cpp:51-84, src/sampling/sampler.cpp:15-147).
 * ---------------------------------------------------------------------------------------------------------------- */

/* Per-row parameters, device arrays of `rows` entries; a null pointer means the default in brackets.  These are the
 * fields of sampling::Sampler (src/sampling/sampler.h:26-53) that the arithmetic reads. */
struct whirl_sample_params {
    const float* inv_t;         /* [1] 1 / temperature */
    const int32_t* top_k;       /* [0 = off] */
    const double* top_p;        /* [1] */
    const double* min_p;        /* [0] */
    const uint8_t* greedy;      /* [0] non-zero: the token is the row's first maximum (Sampler.greedy requests) */
    const double* u;            /* [0] uniform in [0,1) of the inverse-CDF draw: Sampler::uniform() of the row's
                                   (seed, output index), or any host stream such as Philox */
    const uint64_t* race_key;   /* [null: inverse CDF] spec::raceBase(seed, index): draw by the exponential race */
    /* penalties (no counterpart in the reference, which ignores them: src/server/engine_start.cpp:70-73) */
    const int32_t* hist;        /* [null] [rows][hist_stride] token ids, hist_len[row] valid; hist_stride <= WHIRL_MAX_HIST */
    const int32_t* hist_len;
    int64_t hist_stride;
    const float* rep;           /* [1] repetition: l > 0 ? l / rep : l * rep */
    const float* pres;          /* [0] presence: l -= pres */
    const float* freq;          /* [0] frequency: l -= freq * count */
};

/* Outputs, device arrays; only token is required. */
struct whirl_sample_out {
    int32_t* token;     /* [rows] */
    int32_t* status;    /* [rows] WHIRL_ROW_* (may be null) */
    int32_t* n_kept;    /* [rows] size of the kept set, Sampler.n */
    int32_t* closed;    /* [rows] Sampler.closed */
    float* stats;       /* [rows][2] max, sum exp((x - max) * inv_t) of the penalised row */
    int32_t* kept_ids;  /* [rows][kept_cap] the kept candidates in order, first min(n, kept_cap) */
    double* kept_p;     /* [rows][kept_cap] their probabilities (renormalised when closed) */
    int32_t kept_cap;
    uint32_t* counters; /* [WHIRL_CNT_WORDS] added to, never cleared */
};

/* ws: whirl_workspace_bytes(rows, n) bytes of device memory, contents arbitrary; a workspace serves one call at a time
 * (calls on different streams need their own).  Rows of 16-byte aligned logits, at least 32 KiB long, that keep at most
 * WHIRL_STREAM_MAX_K candidates at the first level (their top_k, or 256 without one) are read from memory once; other
 * rows, and rows that need the second (16384 candidates) or third (whole row) level, take several passes.  When stats is
 * null, rows whose top_k closes their kept set skip the softmax normaliser altogether.  Every row comes back
 * WHIRL_ROW_DONE but for the corner cases named at WHIRL_ROW_ESCALATE; counters and whirl_check report what the device
 * met on the way. */
int whirl_sample_rows(const void* x, int dtype, int rows, int n, const whirl_sample_params* params,
                      const whirl_sample_out* out, void* ws, size_t ws_bytes, void* stream);

/* ------------------------------------------------------------------------------------------------------------------
 * Speculative acceptance.
 * ---------------------------------------------------------------------------------------------------------------- */

/* The accept loop of sampling::Acceptor::sample (src/sampling/acceptor.cpp:63-100, exact rules: `sample` and `specsample`)
 * on the device: tokens[row] is the sampler's token of every verify row (whirl_sample_rows; with race_key it is the race
 * draw that drafts from whirl_draft_sample_rows are coupled to).  Sequence s checks drafts[s * draft_stride + 0 .. nd[s])
 * against rows row0[s] + 0 ..: acc[s] = drafts kept, chosen[s] = tokens[row0[s] + acc[s]].  This removes the per-cycle
 * readCtl synchronisation and candidate download (src/server/engine_decode.cpp:399-405). */
int whirl_accept_tokens(const int* tokens, const int* drafts, int draft_stride, const int* nd, const int* row0, int seqs, int* acc,
                        int* chosen, void* stream);

/* The whole accept step of sampling::Acceptor (src/sampling/acceptor.cpp:30-100) on the device, relaxed rules
 * included, so that an engine running relaxed acceptance needs no per-cycle readCtl synchronisation and candidate
 * download either (src/server/engine_decode.cpp:399-405).  One call decides `seqs` sequences; sequence s checks
 * drafts[s * draft_stride + 0 .. nd[s]) against the verify rows row0[s] + 0 .. row0[s] + nd[s] of the batch.
 *
 *   greedy[s] != 0   Acceptor::greedy: draft j is kept iff it is tokens[row0 + j] (the row's argmax,
 *                    whirl_argmax_rows / a greedy row of whirl_sample_rows); with relax_on[s], a draft that is not is
 *                    still kept when relax::acceptGreedy passes on the row's rk best logits (rk_ids / rk_vals /
 *                    rk_stats = the outputs of whirl_topk_rows with K = rk >= the rule's k: rank below k and
 *                    exp(l_draft - l_max) >= alpha, include/whirl/relax_accept.h:55-73) and the kept tokens would not
 *                    extend a repeated 6-gram of the sequence's last 4096 tokens (relax::extendsRepeat, :78-90, over
 *                    hist[s] followed by next[s] and the drafts up to j, as Engine::relaxRepeats builds it);
 *                    relax_gap[s] += l_max - l_draft for every draft kept that way.
 *   greedy[s] == 0   Acceptor::sample: draft j is kept iff it is tokens[row0 + j] (the sampler's draw at output index
 *                    n_gen + j, whirl_sample_rows with u / race_key made for those indices: that is the reference's
 *                    RNG contract, src/sampling/acceptor.h:10-12); with relax_on[s], before that comparison, a draft is
 *                    kept when p(draft) >= min(eps, delta * exp(-H)) on the row's filtered distribution
 *                    (relax::acceptTypical, :93-96) and it would not extend a repeat.  p(draft) is the reference's
 *                    probOf (src/sampling/sampler.cpp:108-116): the draft's entry of the kept set, else 0 on a closed
 *                    row and exp((x[draft] - max) * inv_t) / sum on an open one (x, dtype, n, inv_t: the verify logits,
 *                    read for that one element; raw logits, so rows with penalties need closed sets); H is the entropy
 *                    of the kept set (kept_ids / kept_p / n_kept / closed / stats = the outputs of whirl_sample_rows
 *                    with that kept_cap).  A row that kept more than kept_cap candidates cannot be judged: the draft
 *                    then takes the exact comparison and flags[s] gets WHIRL_ACCEPT_TRUNCATED.
 *
 * acc[s] = drafts kept, chosen[s] = tokens[row0[s] + acc[s]] (the target's own pick after them), relaxed[s] += drafts
 * kept by a relaxed rule, relax_gap[s] as above, flags[s] written.  relaxed / relax_gap / flags may be null.  Arrays
 * that a rule in use needs and that are null make the call fail with WHIRL_ERR_INVALID.
 * Sums that the reference forms in index order (H) are formed in another order here: a decision can differ only when
 * p(draft) meets its threshold to the last bits. */
enum { WHIRL_ACCEPT_TRUNCATED = 1 };
typedef struct whirl_relax_params { /* relax::Params, include/whirl/relax_accept.h:44-50 */
    uint32_t k;
    float alpha, eps, delta;
} whirl_relax_params;
typedef struct whirl_accept_in {
    const int32_t* tokens;   /* [rows] */
    const int32_t* drafts;   /* [seqs][draft_stride] */
    int64_t draft_stride;
    const int32_t* nd;       /* [seqs] */
    const int32_t* row0;     /* [seqs] */
    const uint8_t* greedy;   /* [seqs] (null = all sampling) */
    const uint8_t* relax_on; /* [seqs] (null = exact rules everywhere) */
    /* repeat guard */
    const int32_t* next;     /* [seqs] the sequence's token before the drafts */
    const int32_t* hist;     /* [seqs][hist_stride] the sequence's tokens so far, oldest first */
    int64_t hist_stride;
    const int32_t* hist_len; /* [seqs] */
    /* relaxed greedy rule */
    const int32_t* rk_ids;   /* [rows][rk] */
    const float* rk_vals;    /* [rows][rk] */
    const float* rk_stats;   /* [rows][2] (max, sum) */
    int32_t rk;
    /* typical rule */
    int32_t kept_cap;
    const int32_t* kept_ids; /* [rows][kept_cap] */
    const double* kept_p;    /* [rows][kept_cap] */
    const int32_t* n_kept;   /* [rows] */
    const int32_t* closed;   /* [rows] */
    const float* stats;      /* [rows][2] (max, sum) */
    const void* x;           /* [rows][n] verify logits (open rows only; may be null when every row is closed) */
    int32_t dtype, n;
    const float* inv_t;      /* [rows] (null = 1) */
} whirl_accept_in;
int whirl_accept_rows(const whirl_accept_in* in, const whirl_relax_params* relax, int seqs, int* acc, int* chosen, int* relaxed,
                      double* relax_gap, int* flags, void* stream);

/* The accept / residual rule (Leviathan et al., Chen et al. 2023) that the reference replaced by the race coupling
 * (include/whirl/spec_sample.h:21-24); its residual helper sampleRow(src, s, ex, p_ex) is still in the reference
 * (src/sampling/sampler.cpp:118-131).  Per sequence: target is [L + 1][n] logits, draft [L][n], full-vocabulary
 * p = softmax(target * inv_t), q = softmax(draft * inv_t).  For j = 0 .. L-1 draft_tok[j] is accepted iff
 * u_acc[j] * q(d) < p(d) (or q(d) == 0); at the first rejection next_tok is drawn from max(0, p - q) by inverse CDF in
 * id order with u_res[j]; after L acceptances next_tok is drawn from p of row L with u_res[L].  n_acc = drafts kept.
 * Arrays: draft_tok [seqs][L], inv_t [seqs] (null = 1), u_acc [seqs][L], u_res [seqs][L + 1]. */
size_t whirl_spec_workspace_bytes(int seqs, int L);
int whirl_spec_accept_residual(const void* target, const void* draft, int dtype, int seqs, int L, int n, const int* draft_tok,
                               const float* inv_t, const double* u_acc, const double* u_res, int* n_acc, int* next_tok, void* ws,
                               size_t ws_bytes, void* stream);

/* ---- draw generators ------------------------------------------------------------------------------------------------
 * The reference draws one uniform per sampled row on the host, Sampler::uniform(seed, pos) (src/sampling/sampler.h:46-52,
 * the stream-0 case of spec::uniform, src/common/spec_sample.cpp:13-21), and keys the race draw with
 * spec::raceBase(seed, pos) (include/whirl/spec_sample.h:58-60).  The three host functions below return exactly those
 * values (no device needed); whirl_fill_draws computes them on the device for `rows` (seed, pos) pairs held there, into
 * the u / race_key arrays whirl_sample_rows takes.  Philox4x32-10 is offered beside them for callers that want a
 * counter-based generator per (seed, pos, row, stream): key = seed (lo, hi), counter = (pos lo, pos hi, row, stream),
 * uniform = top 53 bits of out0:out1.  The reference has no Philox; this convention is the library's own. */
enum { WHIRL_GEN_SPLITMIX = 0, WHIRL_GEN_PHILOX = 1 };
double whirl_uniform_splitmix(uint64_t seed, uint64_t pos_idx, uint32_t stream_id);
uint64_t whirl_race_base(uint64_t seed, uint64_t pos_idx);
void whirl_philox4x32_10(const uint32_t ctr[4], const uint32_t key[2], uint32_t out[4]);
double whirl_uniform_philox4x32(uint64_t seed, uint64_t pos_idx, uint32_t row, uint32_t stream_id);
/* seed, pos_idx [rows] u64 on the device -> u [rows] f64 (may be null), race_key [rows] u64 (may be null).  With
 * WHIRL_GEN_PHILOX the row index is the counter's third word. */
int whirl_fill_draws(const uint64_t* seed, const uint64_t* pos_idx, int rows, int generator, uint32_t stream_id, double* u,
                     uint64_t* race_key, void* stream);

/* Reads the device error word that the last whirl_sample_rows / whirl_topk_rows call on this workspace left (the call
 * synchronises `stream`).  WHIRL_OK, or WHIRL_ERR_TIMEOUT when a bounded wait inside the single-pass kernel ran out;
 * *where (may be null) then gets which wait: 1 producer / ring stage free, 3 tail group / row streamed, 4 stream warps /
 * slot ready, 5 stream warps / ring stage full, 11 stream warps / threshold meeting.  The rows such a wait left
 * unanswered were handed to the multi-pass kernel, so the outputs stand unless counters[WHIRL_CNT_UNRESOLVED] is
 * non-zero; the code still tells the caller that the device did not behave. */
int whirl_check(const void* ws, size_t ws_bytes, int rows, void* stream, uint32_t* where);

/* Testing aid, per calling thread: the following whirl_sample_rows / whirl_topk_rows calls give every wait of the
 * single-pass kernel a budget of about wait_us microseconds (0 = the default, about a second), and with lose_copy != 0
 * the first CTA leaves one bulk copy of its first row out, so that the waits on it run out and the error path above
 * can be exercised without a fault.  whirl_test_waits(0, 0) restores the defaults. */
void whirl_test_waits(uint32_t wait_us, int lose_copy);

/* The same call on HOST buffers: logits, parameters and outputs are host pointers; the call copies them to the device
 * (workspace + staging it allocates on first use and keeps), runs whirl_sample_rows in row chunks that overlap the
 * copies, copies the outputs back and synchronises.  For callers that hold logits in host memory and for end-to-end
 * measurement; a serving engine whose logits are already on the device calls whirl_sample_rows.  Returns
 * WHIRL_ERR_TIMEOUT (outputs written all the same) when a device-side wait ran out in one of the chunks. */
int whirl_sample_rows_host(const void* x_host, int dtype, int rows, int n, const whirl_sample_params* params_host,
                           const whirl_sample_out* out_host, int device);
/* Releases what whirl_sample_rows_host keeps. */
void whirl_host_release(void);
/* Message of the last failing whirl_sample_rows_host call on this thread. */
const char* whirl_host_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* WHIRL_B200_H */
