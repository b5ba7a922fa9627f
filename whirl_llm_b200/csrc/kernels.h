// Host-visible declarations of the kernel launchers (internal to the library; the public surface is
// include/whirl_b200.h).
#pragma once

#include <cuda_runtime.h>

#include "../../include/whirl_b200.h"
#include <stddef.h>
#include <stdint.h>

namespace wb {

// set by api.cu: the calling thread's error message and the launch counters
void set_last_error(const char* msg);
void count_launch(int family);

// ---- greedy picks (rowscan.cu)
enum { RS_ARGMAX = 0, RS_ARGMAX_PROB = 1, RS_DRAFT_PICK = 2 };

struct RowScanArgs {
    const void* x;  // [rows][n] f32 or bf16
    int n;
    // RS_ARGMAX: out[dst ? dst[row] : row] = first max; ids / pos / advance as the reference's argmax()
    int* out;
    const int* dst;
    int* ids;
    int* pos;
    int advance;
    // RS_ARGMAX_PROB: out[row], prob[row].  RS_DRAFT_PICK with ctl_all == null: tok / prob / ctl of one sequence
    float* prob;
    // RS_DRAFT_PICK
    int* tok;
    int* ctl;
    int* ctl_all;     // per-sequence control areas; row b's area starts at ctl_all + area[b]
    const int* area;  // device [rows]
    int r, n_min;
    float p_min;
    const int* map;
    void* ws;
};

size_t rowscan_ws_bytes(int rows, int splits);
int rowscan_splits(int rows, int n, int sm_count);
cudaError_t rowscan_launch(const RowScanArgs& a, int dtype, int mode, int rows, int splits, cudaStream_t st);

// ---- selection + sampling (select_generic.cu, single_pass.cu)

// Per-row parameters as device arrays (null = the default in brackets); the fields of the reference's
// sampling::Sampler (src/sampling/sampler.h:26-53) plus this build's penalties.
struct RowParams {
    const float* inv_t;        // [inv_t_scalar]
    float inv_t_scalar;
    const int32_t* top_k;      // [0 = off]
    const double* top_p;       // [1]
    const double* min_p;       // [0]
    const uint8_t* greedy;     // [0] non-zero: the row's token is its first maximum
    const double* u;           // [0] uniform of the inverse-CDF draw (and of the race's open-target choice)
    const uint64_t* race_key;  // [null = inverse CDF] spec::raceBase(seed, pos) per row; the race draw
    // penalties over each row's token history
    const int32_t* hist;       // [rows][hist_stride]
    const int32_t* hist_len;   // [rows]
    int64_t hist_stride;
    const float* rep;          // [1]
    const float* pres;         // [0]
    const float* freq;         // [0]
};

struct RowOutputs {
    int32_t* token;     // [rows]
    int32_t* status;    // [rows] RowStatus
    int32_t* n_kept;    // [rows] (may be null)
    int32_t* closed;    // [rows] (may be null)
    float* stats;       // [rows][2] max, sum (may be null)
    int32_t* kept_ids;  // [rows][kept_cap] (may be null)
    double* kept_p;     // [rows][kept_cap] (may be null)
    int32_t kept_cap;
    uint32_t* counters;  // [8] batch counters (may be null), see WHIRL_CNT_*
};

enum { MODE_TOPK = 0, MODE_SAMPLE = 1, MODE_DRAFT = 2 };

// draft_sample_rows per-row parameters (the reference passes them by value: kernels/kernel_args.h:55-66), device arrays
struct DraftArgs {
    const int32_t* on;
    const int32_t* top_k;
    const int32_t* qoff;  // i32 word offset of the row's q entry in qbuf
    const float* inv_t;
    const float* top_p;
    const float* min_p;
    const uint32_t* key_lo;  // race key base, spec::raceBase(seed, output index of draft r)
    const uint32_t* key_hi;
    int32_t* ctl_all;
    const int32_t* area;  // word offset of each row's 64-word control area
    int32_t r;
    const int32_t* map;   // token id of each logits row entry (draft-head vocabulary subset), may be null
    int32_t* qbuf;
};

struct SelectArgs {
    const void* x;  // [rows][n]
    int rows, n;
    int mode;
    // MODE_TOPK: K candidates per row into ids / vals ([rows][K], sorted logit desc, id asc), stats [rows][2]
    int K;
    int32_t* ids;
    float* vals;
    float* stats;
    // MODE_SAMPLE
    RowParams prm;
    RowOutputs out;
    const int32_t* row_list;  // optional: process rows row_list[0..rows) of the batch (the escalated ones); bit 30 of an
                              // entry marks a row to redo at the first candidate level
    const int32_t* row_count; // optional device count overriding `rows` (with row_list)
    int level_k;              // candidates for rows without a usable top_k (256 first level, 16384 second)
    void* ws;                 // generic: [rows][level cap] doubles of probability scratch
    DraftArgs draft;          // MODE_DRAFT
    int32_t id_offset;        // MODE_TOPK: added to every id written (a vocabulary slice's first token id)
    uint32_t* err;            // device error word (bounded waits that ran out)
    uint32_t wait_limit;      // single-pass sampler: budget of every wait, in suspensions of about a microsecond (0 = the default)
    uint32_t lose_copy;       // single-pass sampler, tests only: the producer of CTA 0 leaves out one bulk copy, so that waits run out
    // single-pass sampler, MODE_SAMPLE: its last CTA lists the rows it left to the multi-pass kernel in fin_list (rows with
    // top_k above its limit, and rows whose kept set may reach past 256 candidates; with bit 30: rows to redo at the first
    // level) and their number in fin_counts[1].  fin_counts[2] and [3] are the two kernels' tickets (zero before a launch).
    int32_t* fin_list;
    int32_t* fin_counts;
    void* side_ws;            // single-pass sampler: side buffers for the words kept out of the stream (single_pass_side_bytes)
    uint32_t* batch_counters; // multi-pass kernel: its last CTA adds the batch's rows still without an answer, and a wait of
                              // the kernel before it that ran out, to these WHIRL_CNT_* words (or null)
    // multi-pass kernel, third level (the whole row: the reference's last escalation step, src/server/engine_sampling.cpp:79-83):
    // full_slots scratch areas of 16 * full_npad bytes each in global memory, handed out through full_locks (zero = free)
    void* full_ws;
    uint32_t* full_locks;
    int full_slots;
    uint32_t full_npad;       // row length rounded up to a power of two
};

constexpr int kGenericMaxK = 16384;
size_t select_generic_ws_bytes(int ctas, int K);  // ctas = min(rows, 2 * SMs)
constexpr int kFullSlots = 4;
size_t select_full_ws_bytes(int n);               // 0 when the row is too long for the third level (n > 2^20)
uint32_t select_full_npad(int n);
cudaError_t select_generic_launch(const SelectArgs& a, int dtype, int sm_count, cudaStream_t st);

// single-pass kernel (single_pass.cu): rows keeping at most kSinglePassMaxK candidates, 16-byte aligned rows
constexpr int kFirstLevelK = 256;     // candidates of a row without a usable top_k at the first level (the reference's k_small,
                                      // src/server/engine_sampling.h:20)
constexpr int kSinglePassMaxK = 1024;  // candidates a row may keep in the single-pass kernel
constexpr int kSinglePassHandK = 256;  // ... of which rows up to this many are finished by one warp from dedicated shared memory
cudaError_t single_pass_launch(const SelectArgs& a, int dtype, int sm_count, cudaStream_t st);
size_t single_pass_side_bytes(int sm_bound);  // bytes of SelectArgs::side_ws for a GPU of up to sm_bound SMs
bool single_pass_supported(const SelectArgs& a, int dtype);

// ---- speculative acceptance (spec_accept.cu)
size_t spec_stats_bytes(int seqs, int L);
cudaError_t accept_tokens_launch(const int32_t* tokens, const int32_t* dr, int dr_stride, const int32_t* nd, const int32_t* row0,
                                 int seqs, int32_t* acc, int32_t* chosen, cudaStream_t st);
cudaError_t accept_rows_launch(const whirl_accept_in& in, const whirl_relax_params& rp, int seqs, int32_t* acc, int32_t* chosen,
                               int32_t* relaxed, double* gap, int32_t* flags, cudaStream_t st);
cudaError_t accept_residual_launch(const void* target, const void* draft, int dtype, int seqs, int L, int n, const int32_t* draft_tok,
                                   const float* inv_t, const double* u_acc, const double* u_res, void* stats_ws, int32_t* n_acc,
                                   int32_t* next_tok, cudaStream_t st);

// ---- vocab-sharded candidates (merge.cu)
cudaError_t merge_sample_launch(const int32_t* ids, const float* vals, const float* stats, int shards, size_t cand_stride,
                                size_t stat_stride, int rows, int Ks,
                                int n_total, const RowParams& P, const RowOutputs& out, int sm_count, cudaStream_t st);

}  // namespace wb
