// The C ABI of the library (include/whirl_b200.h): argument checks, workspace carving, launches.  No allocation and no
// synchronisation here, except in whirl_sample_rows_host, which owns its staging.
#include "../../include/whirl_b200.h"

#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>

#include "kernels.h"
#include "tail.cuh"

namespace {

thread_local std::string g_err;
// testing aid (whirl_test_waits): wait budget and lost copy of this thread's single-pass launches
thread_local uint32_t g_wait_limit = 0;
thread_local uint32_t g_lose_copy = 0;

// host-side launch counters per kernel family (whirl_launch_counts)
std::atomic<uint64_t> g_launch[4];
enum { LC_ROWSCAN = 0, LC_GENERIC = 1, LC_SINGLE = 2, LC_AUX = 3 };
void bump(int which, uint64_t n = 1) { g_launch[which].fetch_add(n, std::memory_order_relaxed); }

int fail(int code, const char* msg) {
    g_err = msg;
    return code;
}
int fail_cuda(cudaError_t e, const char* where) {
    g_err = std::string(where) + ": " + cudaGetErrorString(e);
    return WHIRL_ERR_CUDA;
}

int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
        cached[dev] = v;
    }
    return cached[dev];
}

constexpr int kMaxSplits = 64;
constexpr int kSmBound = 256;  // upper bound on SMs used when sizing the workspace

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// workspace layout (all offsets 256-byte aligned)
struct Ws {
    size_t off_scan, off_status, off_list, off_list2, off_count, off_err, off_locks, off_p, off_side, off_full, total;
};
Ws ws_layout(int rows, int n = 0) {
    Ws w;
    size_t o = 0;
    w.off_scan = o;
    o = align_up(o + wb::rowscan_ws_bytes(rows, kMaxSplits), 256);
    w.off_status = o;
    o = align_up(o + size_t(rows) * 4, 256);
    w.off_list = o;
    o = align_up(o + size_t(rows) * 4, 256);
    w.off_list2 = o;
    o = align_up(o + size_t(rows) * 4, 256);
    w.off_err = o;  // four error words, four count / ticket words, eight scratch-area locks (cleared together: 64 bytes)
    w.off_count = o + 16;
    w.off_locks = o + 32;
    o = align_up(o + 512, 256);
    w.off_p = o;
    o = align_up(o + wb::select_generic_ws_bytes(std::min(rows, 2 * kSmBound), wb::kGenericMaxK), 256);
    w.off_side = o;  // the single-pass sampler's side buffers (penalised rows that need their normaliser)
    o = align_up(o + wb::single_pass_side_bytes(std::min(rows, kSmBound)), 256);
    w.off_full = o;  // the third escalation level's scratch areas (the only part that depends on the row length)
    o = align_up(o + wb::select_full_ws_bytes(n), 256);
    w.total = o;
    return w;
}

bool bad_dtype(int d) { return d != WHIRL_F32 && d != WHIRL_BF16; }

// rows flagged with `want` -> list, count (one CTA; rows is at most a few thousand)
__global__ void gather_rows_kernel(const int32_t* status, int rows, int want, int32_t* list, int32_t* count) {
    __shared__ int s_n;
    if (threadIdx.x == 0) s_n = 0;
    __syncthreads();
    for (int base = 0; base < rows; base += blockDim.x) {
        const int r = base + threadIdx.x;
        const bool f = r < rows && (status[r] == want || status[r] == wb::ROW_PENDING);
        // order inside the list does not matter: rows are independent
        if (f) list[atomicAdd(&s_n, 1)] = r;
    }
    __syncthreads();
    if (threadIdx.x == 0) *count = s_n;
}

// After the small-K single-pass kernel: rows left to the large-K kernel -> list_a; rows for the multi-pass kernel ->
// list_b (a row whose candidate log overflowed, or an open set whose draw fell past its candidates and needs the
// id-order walk of the row, is redone at the first level: bit 30; a row whose kept set may reach past its candidates goes
// to the second level).  counts[0], counts[1].
__global__ void gather_two_kernel(const int32_t* status, int rows, int32_t* list_a, int32_t* list_b, int32_t* counts) {
    __shared__ int s_a, s_b;
    if (threadIdx.x == 0) s_a = 0, s_b = 0;
    __syncthreads();
    for (int base = 0; base < rows; base += blockDim.x) {
        const int r = base + threadIdx.x;
        if (r >= rows) continue;
        const int st = status[r];
        if (st == wb::ROW_LARGE_K) list_a[atomicAdd(&s_a, 1)] = r;
        else if (st == wb::ROW_ESCALATE) list_b[atomicAdd(&s_b, 1)] = r;
        else if (st == wb::ROW_RETRY || st == wb::ROW_OPEN_TAIL) list_b[atomicAdd(&s_b, 1)] = r | (1 << 30);
    }
    __syncthreads();
    if (threadIdx.x == 0) counts[0] = s_a, counts[1] = s_b;
}

__global__ void count_unresolved_kernel(const int32_t* status, int rows, uint32_t* counters) {
    int c = 0;
    for (int r = threadIdx.x; r < rows; r += blockDim.x) c += status[r] != wb::ROW_DONE;
    c = int(wb::warp_sum(uint32_t(c)));
    if ((threadIdx.x & 31) == 0 && c) atomicAdd(&counters[WHIRL_CNT_UNRESOLVED], uint32_t(c));
}

int scan_call(int mode, const void* x, int dtype, int rows, int n, wb::RowScanArgs a, void* ws, size_t ws_bytes, void* stream) {
    if (!x || rows < 0 || n <= 0 || bad_dtype(dtype)) return fail(WHIRL_ERR_INVALID, "rowscan: bad x / rows / n / dtype");
    if (rows == 0) return WHIRL_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int splits = wb::rowscan_splits(rows, n, sm_count());
    if (splits > kMaxSplits) splits = kMaxSplits;
    if (splits > 1) {
        const size_t need = wb::rowscan_ws_bytes(rows, splits);
        if (!ws || ws_bytes < need) return fail(WHIRL_ERR_WORKSPACE, "rowscan: workspace missing or too small");
        // the tickets start at zero; the last CTA of each row puts them back, this covers a first use
        const cudaError_t e = cudaMemsetAsync(ws, 0, size_t((rows + 3) & ~3) * sizeof(int), st);
        if (e != cudaSuccess) return fail_cuda(e, "cudaMemsetAsync");
    }
    a.x = x, a.n = n, a.ws = ws;
    const cudaError_t e = wb::rowscan_launch(a, dtype, mode, rows, splits, st);
    bump(LC_ROWSCAN);
    return e == cudaSuccess ? WHIRL_OK : fail_cuda(e, "rowscan launch");
}

}  // namespace

namespace wb {
void set_last_error(const char* msg) { g_err = msg; }
void count_launch(int family) { bump(family); }
}  // namespace wb

#pragma GCC visibility push(default)
extern "C" {

const char* whirl_status_string(int s) {
    switch (s) {
    case WHIRL_OK: return "ok";
    case WHIRL_ERR_INVALID: return "invalid argument";
    case WHIRL_ERR_CUDA: return "CUDA error";
    case WHIRL_ERR_WORKSPACE: return "workspace missing or too small";
    case WHIRL_ERR_UNSUPPORTED: return "outside a documented limit";
    case WHIRL_ERR_TIMEOUT: return "device-side wait ran out";
    }
    return "?";
}
const char* whirl_last_error(void) { return g_err.c_str(); }
int whirl_version(void) { return 100; }

size_t whirl_workspace_bytes(int rows, int n) {
    return ws_layout(rows < 1 ? 1 : rows, n).total;
}

int whirl_argmax(const void* x, int dtype, int n, int* out, int* ids, int* pos, int advance, void* ws, size_t ws_bytes,
                 void* stream) {
    if (!out) return fail(WHIRL_ERR_INVALID, "argmax: out is null");
    wb::RowScanArgs a{};
    a.out = out, a.ids = ids, a.pos = pos, a.advance = advance;
    return scan_call(wb::RS_ARGMAX, x, dtype, 1, n, a, ws, ws_bytes, stream);
}
int whirl_argmax_rows(const void* x, int dtype, int rows, int n, int* out, void* ws, size_t ws_bytes, void* stream) {
    if (!out) return fail(WHIRL_ERR_INVALID, "argmax_rows: out is null");
    wb::RowScanArgs a{};
    a.out = out;
    return scan_call(wb::RS_ARGMAX, x, dtype, rows, n, a, ws, ws_bytes, stream);
}
int whirl_argmax_rows_to(const void* x, int dtype, int rows, int n, int* out, const int* dst, void* ws, size_t ws_bytes,
                         void* stream) {
    if (!out || !dst) return fail(WHIRL_ERR_INVALID, "argmax_rows_to: out / dst is null");
    wb::RowScanArgs a{};
    a.out = out, a.dst = dst;
    return scan_call(wb::RS_ARGMAX, x, dtype, rows, n, a, ws, ws_bytes, stream);
}
int whirl_argmax_prob(const void* x, int dtype, int rows, int n, int* out_tok, float* out_prob, void* ws, size_t ws_bytes,
                      void* stream) {
    if (!out_tok || !out_prob) return fail(WHIRL_ERR_INVALID, "argmax_prob: out is null");
    wb::RowScanArgs a{};
    a.out = out_tok, a.prob = out_prob;
    return scan_call(wb::RS_ARGMAX_PROB, x, dtype, rows, n, a, ws, ws_bytes, stream);
}
int whirl_draft_pick(const void* x, int dtype, int n, int* tok, float* prob, int* ctl, int r, int n_min, float p_min,
                     const int* map, void* ws, size_t ws_bytes, void* stream) {
    if (!tok || !prob || !ctl || r < 0) return fail(WHIRL_ERR_INVALID, "draft_pick: tok / prob / ctl is null or r < 0");
    wb::RowScanArgs a{};
    a.tok = tok, a.prob = prob, a.ctl = ctl, a.r = r, a.n_min = n_min, a.p_min = p_min, a.map = map;
    return scan_call(wb::RS_DRAFT_PICK, x, dtype, 1, n, a, ws, ws_bytes, stream);
}
int whirl_draft_pick_rows(const void* x, int dtype, int rows, int n, int* ctl_all, const int* area, int r, int n_min,
                          float p_min, const int* map, void* ws, size_t ws_bytes, void* stream) {
    if (!ctl_all || !area || r < 0 || r >= 16) return fail(WHIRL_ERR_INVALID, "draft_pick_rows: ctl_all / area is null or r outside [0,16)");
    wb::RowScanArgs a{};
    a.ctl_all = ctl_all, a.area = area, a.r = r, a.n_min = n_min, a.p_min = p_min, a.map = map;
    return scan_call(wb::RS_DRAFT_PICK, x, dtype, rows, n, a, ws, ws_bytes, stream);
}

int whirl_topk_rows(const void* x, int dtype, int rows, int n, int K, float inv_t, const float* inv_t_rows, int* ids,
                    float* vals, float* stats, void* ws, size_t ws_bytes, void* stream) {
    return whirl_topk_rows_shard(x, dtype, rows, n, K, 0, inv_t, inv_t_rows, ids, vals, stats, ws, ws_bytes, stream);
}

int whirl_topk_rows_shard(const void* x, int dtype, int rows, int n, int K, int id_offset, float inv_t, const float* inv_t_rows,
                          int* ids, float* vals, float* stats, void* ws, size_t ws_bytes, void* stream) {
    if (!x || !ids || !vals || !stats || rows < 0 || n <= 0 || bad_dtype(dtype)) return fail(WHIRL_ERR_INVALID, "topk_rows: bad pointer / rows / n / dtype");
    if (K < 1) return fail(WHIRL_ERR_INVALID, "topk_rows: K < 1");
    if (K > WHIRL_MAX_K) return fail(WHIRL_ERR_UNSUPPORTED, "topk_rows: K above WHIRL_MAX_K");
    if (rows == 0) return WHIRL_OK;
    wb::SelectArgs a{};
    a.x = x, a.rows = rows, a.n = n, a.mode = wb::MODE_TOPK, a.K = K, a.ids = ids, a.vals = vals, a.stats = stats;
    a.id_offset = id_offset;
    a.wait_limit = g_wait_limit, a.lose_copy = g_lose_copy;
    a.prm.inv_t = inv_t_rows, a.prm.inv_t_scalar = inv_t;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t e;
    // the single-pass kernels report through an error word and a per-row status in the workspace
    const Ws w = ws_layout(rows);
    const bool have_ws = ws && ws_bytes >= w.total;
    uint8_t* base = static_cast<uint8_t*>(ws);
    if (have_ws) {
        a.err = reinterpret_cast<uint32_t*>(base + w.off_err);
        a.out.status = reinterpret_cast<int32_t*>(base + w.off_status);
    }
    if (have_ws && wb::single_pass_supported(a, dtype)) {
        e = wb::single_pass_launch(a, dtype, sm_count(), st);
        bump(LC_SINGLE);
        if (e == cudaSuccess) {
            // rows whose candidate log overflowed (adversarial element order) are redone by the multi-pass kernel
            int32_t* list = reinterpret_cast<int32_t*>(base + w.off_list);
            int32_t* count = reinterpret_cast<int32_t*>(base + w.off_count);
            gather_rows_kernel<<<1, 1024, 0, st>>>(a.out.status, rows, wb::ROW_RETRY, list, count);
            wb::SelectArgs b = a;
            b.row_list = list, b.row_count = count;
            e = wb::select_generic_launch(b, dtype, sm_count(), st);
            bump(LC_AUX);
            bump(LC_GENERIC);
        }
    } else {
        a.out.status = nullptr;
        e = wb::select_generic_launch(a, dtype, sm_count(), st);
        bump(LC_GENERIC);
    }
    return e == cudaSuccess ? WHIRL_OK : fail_cuda(e, "topk_rows launch");
}

int whirl_sample_rows(const void* x, int dtype, int rows, int n, const whirl_sample_params* prm, const whirl_sample_out* out,
                      void* ws, size_t ws_bytes, void* stream) {
    if (!x || !prm || !out || !out->token || rows < 0 || n <= 0 || bad_dtype(dtype)) return fail(WHIRL_ERR_INVALID, "sample_rows: bad pointer / rows / n / dtype");
    if (rows == 0) return WHIRL_OK;
    const Ws w = ws_layout(rows, n);
    if (!ws || ws_bytes < w.total) return fail(WHIRL_ERR_WORKSPACE, "sample_rows: workspace missing or too small (whirl_workspace_bytes)");
    if (prm->hist) {
        if (!prm->hist_len) return fail(WHIRL_ERR_INVALID, "sample_rows: hist without hist_len");
        if (prm->hist_stride < 0 || prm->hist_stride > WHIRL_MAX_HIST) return fail(WHIRL_ERR_UNSUPPORTED, "sample_rows: hist_stride above WHIRL_MAX_HIST");
        if (uint32_t(n) > (1u << 19) - 1) return fail(WHIRL_ERR_UNSUPPORTED, "sample_rows: penalties need n < 2^19");
    }
    if (out->kept_cap < 0) return fail(WHIRL_ERR_INVALID, "sample_rows: kept_cap < 0");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    uint8_t* base = static_cast<uint8_t*>(ws);
    wb::SelectArgs a{};
    a.x = x, a.rows = rows, a.n = n, a.mode = wb::MODE_SAMPLE;
    a.prm.inv_t = prm->inv_t, a.prm.inv_t_scalar = 1.f, a.prm.top_k = prm->top_k, a.prm.top_p = prm->top_p, a.prm.min_p = prm->min_p;
    a.prm.greedy = prm->greedy, a.prm.u = prm->u, a.prm.race_key = prm->race_key;
    a.prm.hist = prm->hist, a.prm.hist_len = prm->hist_len, a.prm.hist_stride = prm->hist_stride;
    a.prm.rep = prm->rep, a.prm.pres = prm->pres, a.prm.freq = prm->freq;
    a.out.token = out->token, a.out.n_kept = out->n_kept, a.out.closed = out->closed, a.out.stats = out->stats;
    a.out.kept_ids = out->kept_ids, a.out.kept_p = out->kept_p, a.out.kept_cap = out->kept_cap, a.out.counters = out->counters;
    a.out.status = out->status ? out->status : reinterpret_cast<int32_t*>(base + w.off_status);
    a.ws = base + w.off_p;
    a.err = reinterpret_cast<uint32_t*>(base + w.off_err);
    a.side_ws = base + w.off_side;
    a.wait_limit = g_wait_limit, a.lose_copy = g_lose_copy;
    // level 1: top_k candidates (the set closes there), or 256 of them as the reference's first launch does
    // (k_small, src/server/engine_sampling.h:20)
    a.level_k = wb::kFirstLevelK;
    int32_t* list_a = reinterpret_cast<int32_t*>(base + w.off_list);
    int32_t* list_b = reinterpret_cast<int32_t*>(base + w.off_list2);
    int32_t* counts = reinterpret_cast<int32_t*>(base + w.off_count);
    cudaError_t e;
    if (wb::single_pass_supported(a, dtype)) {
        // Rows keeping at most 256 candidates in one pass.  The kernel's last CTA lists what is left for the multi-pass
        // kernel below: rows with top_k above 256, rows whose kept set may reach past 256 candidates (second level, up to
        // 16384: k_big, src/server/engine_sampling.h:21), and rows to redo (candidate log overflow, NaN, open-set walk).
        a.fin_list = list_b, a.fin_counts = counts;
        e = wb::single_pass_launch(a, dtype, sm_count(), st);
        bump(LC_SINGLE);
        if (e != cudaSuccess) return fail_cuda(e, "sample_rows single-pass kernel");
        wb::SelectArgs b = a;
        b.level_k = wb::kGenericMaxK, b.row_list = list_b, b.row_count = counts + 1;
        b.out.counters = nullptr;  // (counters[0] and [1] were counted by the first kernel)
        b.batch_counters = out->counters;
        if (wb::select_full_ws_bytes(n) != 0) {
            b.full_ws = base + w.off_full, b.full_locks = reinterpret_cast<uint32_t*>(base + w.off_locks);
            b.full_slots = wb::kFullSlots, b.full_npad = wb::select_full_npad(n);
        }
        e = wb::select_generic_launch(b, dtype, sm_count(), st);
        bump(LC_GENERIC);
        if (e != cudaSuccess) return fail_cuda(e, "sample_rows multi-pass kernel");
        e = cudaGetLastError();
        return e == cudaSuccess ? WHIRL_OK : fail_cuda(e, "sample_rows");
    } else {
        e = wb::select_generic_launch(a, dtype, sm_count(), st);
        bump(LC_GENERIC);
        if (e != cudaSuccess) return fail_cuda(e, "sample_rows level 1");
        gather_two_kernel<<<1, 1024, 0, st>>>(a.out.status, rows, list_a, list_b, counts);
        bump(LC_AUX);
    }
    // level 2: the rows whose kept set may reach past those candidates, with up to 16384 (k_big, :21); and the rows the
    // single-pass kernel gave up, at level 1
    wb::SelectArgs b = a;
    b.level_k = wb::kGenericMaxK, b.row_list = list_b, b.row_count = counts + 1;
    b.out.counters = nullptr;  // counters[0] counted the level-1 escalations already
    if (wb::select_full_ws_bytes(n) != 0) {
        e = cudaMemsetAsync(base + w.off_locks, 0, 32, st);
        if (e != cudaSuccess) return fail_cuda(e, "cudaMemsetAsync");
        b.full_ws = base + w.off_full, b.full_locks = reinterpret_cast<uint32_t*>(base + w.off_locks);
        b.full_slots = wb::kFullSlots, b.full_npad = wb::select_full_npad(n);
    }
    e = wb::select_generic_launch(b, dtype, sm_count(), st);
    bump(LC_GENERIC);
    if (e != cudaSuccess) return fail_cuda(e, "sample_rows level 2");
    if (out->counters) { count_unresolved_kernel<<<1, 256, 0, st>>>(a.out.status, rows, out->counters); bump(LC_AUX); }
    e = cudaGetLastError();
    return e == cudaSuccess ? WHIRL_OK : fail_cuda(e, "sample_rows");
}

int whirl_check(const void* ws, size_t ws_bytes, int rows, void* stream, uint32_t* where) {
    if (!ws || rows < 0) return fail(WHIRL_ERR_INVALID, "check: ws is null or rows < 0");
    const Ws w = ws_layout(rows < 1 ? 1 : rows);
    if (ws_bytes < w.off_err + 64) return fail(WHIRL_ERR_WORKSPACE, "check: workspace too small for this row count");
    uint32_t word = 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaMemcpyAsync(&word, static_cast<const uint8_t*>(ws) + w.off_err, 4, cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return fail_cuda(e, "check");
    if (where) *where = word;
    if (word == 0) return WHIRL_OK;
    g_err = "a bounded wait of the single-pass kernel ran out (wait " + std::to_string(word) + ")";
    return WHIRL_ERR_TIMEOUT;
}

void whirl_test_waits(uint32_t wait_us, int lose_copy) { g_wait_limit = wait_us, g_lose_copy = lose_copy ? 1u : 0u; }


int whirl_draft_sample_rows(const void* x, int dtype, int rows, int n, int* ctl_all, const int* area, int r, const int* map,
                            const whirl_dsamp_args* da, int* qbuf, void* stream) {
    if (!x || !ctl_all || !area || !da || !qbuf || rows < 0 || n <= 0 || bad_dtype(dtype) || r < 0 || r >= 16)
        return fail(WHIRL_ERR_INVALID, "draft_sample_rows: bad pointer / rows / n / dtype / r");
    if (!da->on || !da->top_k || !da->qoff || !da->inv_t || !da->top_p || !da->min_p || !da->key_lo || !da->key_hi)
        return fail(WHIRL_ERR_INVALID, "draft_sample_rows: every array of whirl_dsamp_args is required");
    if (rows == 0) return WHIRL_OK;
    wb::SelectArgs a{};
    a.x = x, a.rows = rows, a.n = n, a.mode = wb::MODE_DRAFT;
    a.prm.inv_t_scalar = 1.f;
    a.draft.on = da->on, a.draft.top_k = da->top_k, a.draft.qoff = da->qoff, a.draft.inv_t = da->inv_t, a.draft.top_p = da->top_p;
    a.draft.min_p = da->min_p, a.draft.key_lo = da->key_lo, a.draft.key_hi = da->key_hi;
    a.draft.ctl_all = ctl_all, a.draft.area = area, a.draft.r = r, a.draft.map = map, a.draft.qbuf = qbuf;
    const cudaError_t e = wb::select_generic_launch(a, dtype, sm_count(), static_cast<cudaStream_t>(stream));
    bump(LC_GENERIC);
    return e == cudaSuccess ? WHIRL_OK : fail_cuda(e, "draft_sample_rows launch");
}

int whirl_accept_tokens(const int* tokens, const int* drafts, int draft_stride, const int* nd, const int* row0, int seqs, int* acc,
                        int* chosen, void* stream) {
    if (!tokens || !drafts || !nd || !row0 || !acc || !chosen || seqs < 0 || draft_stride < 0)
        return fail(WHIRL_ERR_INVALID, "accept_tokens: bad pointer / seqs / draft_stride");
    if (seqs == 0) return WHIRL_OK;
    const cudaError_t e = wb::accept_tokens_launch(tokens, drafts, draft_stride, nd, row0, seqs, acc, chosen, static_cast<cudaStream_t>(stream));
    bump(LC_AUX);
    return e == cudaSuccess ? WHIRL_OK : fail_cuda(e, "accept_tokens launch");
}

int whirl_accept_rows(const whirl_accept_in* in, const whirl_relax_params* relax, int seqs, int* acc, int* chosen, int* relaxed,
                      double* relax_gap, int* flags, void* stream) {
    if (!in || !relax || !acc || !chosen || seqs < 0 || !in->tokens || !in->drafts || !in->nd || !in->row0 || in->draft_stride < 0)
        return fail(WHIRL_ERR_INVALID, "accept_rows: bad pointer / seqs / draft_stride");
    if (in->relax_on) {
        // (which rule a sequence takes is known on the device only: every array a relaxed rule may read has to be there)
        if (!in->next || (in->hist && (!in->hist_len || in->hist_stride < 0)))
            return fail(WHIRL_ERR_INVALID, "accept_rows: relaxed rules need next (and hist_len with hist)");
        const bool have_greedy = in->rk_ids && in->rk_vals && in->rk_stats && in->rk >= 1 && in->rk <= 32;
        const bool have_typical = in->kept_ids && in->kept_p && in->n_kept && in->closed && in->stats && in->kept_cap >= 1;
        if (in->greedy && !have_greedy) return fail(WHIRL_ERR_INVALID, "accept_rows: the relaxed greedy rule needs rk_ids / rk_vals / rk_stats, 1 <= rk <= 32");
        if (!have_typical && !(in->greedy && have_greedy)) return fail(WHIRL_ERR_INVALID, "accept_rows: the typical rule needs kept_ids / kept_p / n_kept / closed / stats");
        if (have_greedy && uint32_t(in->rk) < (relax->k < 1 ? 1u : (relax->k > 16 ? 16u : relax->k)))
            return fail(WHIRL_ERR_INVALID, "accept_rows: rk below the rule's k");
        if (in->x && (bad_dtype(in->dtype) || in->n <= 0)) return fail(WHIRL_ERR_INVALID, "accept_rows: x with a bad dtype / n");
    }
    if (seqs == 0) return WHIRL_OK;
    const cudaError_t e = wb::accept_rows_launch(*in, *relax, seqs, acc, chosen, relaxed, relax_gap, flags, static_cast<cudaStream_t>(stream));
    bump(LC_AUX);
    return e == cudaSuccess ? WHIRL_OK : fail_cuda(e, "accept_rows launch");
}

size_t whirl_spec_workspace_bytes(int seqs, int L) { return wb::spec_stats_bytes(seqs < 0 ? 0 : seqs, L < 0 ? 0 : L) + 256; }

int whirl_spec_accept_residual(const void* target, const void* draft, int dtype, int seqs, int L, int n, const int* draft_tok,
                               const float* inv_t, const double* u_acc, const double* u_res, int* n_acc, int* next_tok, void* ws,
                               size_t ws_bytes, void* stream) {
    if (!target || (!draft && L > 0) || (!draft_tok && L > 0) || (!u_acc && L > 0) || !u_res || !n_acc || !next_tok || seqs < 0 ||
        L < 0 || n <= 0 || bad_dtype(dtype))
        return fail(WHIRL_ERR_INVALID, "spec_accept_residual: bad pointer / seqs / L / n / dtype");
    if (seqs == 0) return WHIRL_OK;
    if (!ws || ws_bytes < whirl_spec_workspace_bytes(seqs, L)) return fail(WHIRL_ERR_WORKSPACE, "spec_accept_residual: workspace (whirl_spec_workspace_bytes)");
    void* aligned = reinterpret_cast<void*>((reinterpret_cast<uintptr_t>(ws) + 255) & ~uintptr_t(255));
    const cudaError_t e = wb::accept_residual_launch(target, draft, dtype, seqs, L, n, draft_tok, inv_t, u_acc, u_res, aligned, n_acc,
                                                     next_tok, static_cast<cudaStream_t>(stream));
    bump(LC_AUX, 3);
    return e == cudaSuccess ? WHIRL_OK : fail_cuda(e, "spec_accept_residual launch");
}

namespace {
int merge_call(const int* ids, const float* vals, const float* stats, int shards, size_t cand_stride, size_t stat_stride, int rows, int K_s,
               int n_total, const whirl_sample_params* prm, const whirl_sample_out* out, void* stream) {
    if (!ids || !vals || !stats || !prm || !out || !out->token || shards < 1 || rows < 0 || K_s < 1 || n_total < 1)
        return fail(WHIRL_ERR_INVALID, "merge_sample_rows: bad pointer / shards / rows / K_s / n_total");
    if (K_s > WHIRL_STREAM_MAX_K || size_t(shards) * K_s > 16384) return fail(WHIRL_ERR_UNSUPPORTED, "merge_sample_rows: K_s above 1024 or shards * K_s above 16384");
    if (prm->hist) return fail(WHIRL_ERR_UNSUPPORTED, "merge_sample_rows: penalties belong to the per-slice selection");
    if (rows == 0) return WHIRL_OK;
    wb::RowParams P{};
    P.inv_t = prm->inv_t, P.inv_t_scalar = 1.f, P.top_k = prm->top_k, P.top_p = prm->top_p, P.min_p = prm->min_p;
    P.greedy = prm->greedy, P.u = prm->u, P.race_key = prm->race_key;
    wb::RowOutputs O{};
    O.token = out->token, O.status = out->status, O.n_kept = out->n_kept, O.closed = out->closed, O.stats = out->stats;
    O.kept_ids = out->kept_ids, O.kept_p = out->kept_p, O.kept_cap = out->kept_cap, O.counters = out->counters;
    const cudaError_t e = wb::merge_sample_launch(ids, vals, stats, shards, cand_stride, stat_stride, rows, K_s, n_total, P, O, sm_count(),
                                                  static_cast<cudaStream_t>(stream));
    bump(LC_AUX);
    return e == cudaSuccess ? WHIRL_OK : fail_cuda(e, "merge_sample_rows launch");
}
}  // namespace

int whirl_merge_sample_rows(const int* ids, const float* vals, const float* stats, int shards, int rows, int K_s, int n_total,
                            const whirl_sample_params* prm, const whirl_sample_out* out, void* stream) {
    return merge_call(ids, vals, stats, shards, size_t(rows < 0 ? 0 : rows) * size_t(K_s < 0 ? 0 : K_s), size_t(rows < 0 ? 0 : rows) * 2, rows, K_s,
                      n_total, prm, out, stream);
}

size_t whirl_shard_block_words(int rows, int K_s) { return rows < 0 || K_s < 0 ? 0 : size_t(rows) * (2 * size_t(K_s) + 2); }

int whirl_merge_sample_rows_packed(const void* blocks, int shards, int rows, int K_s, int n_total, const whirl_sample_params* prm,
                                   const whirl_sample_out* out, void* stream) {
    if (!blocks || rows < 0 || K_s < 1) return fail(WHIRL_ERR_INVALID, "merge_sample_rows_packed: bad pointer / rows / K_s");
    const size_t words = whirl_shard_block_words(rows, K_s);
    const int32_t* base = static_cast<const int32_t*>(blocks);
    return merge_call(base, reinterpret_cast<const float*>(base + size_t(rows) * K_s), reinterpret_cast<const float*>(base + 2 * size_t(rows) * K_s),
                      shards, words, words, rows, K_s, n_total, prm, out, stream);
}

void whirl_launch_counts(uint64_t* out, int n) {
    for (int i = 0; i < n && i < 4; ++i) out[i] = g_launch[i].load(std::memory_order_relaxed);
}

}  // extern "C"
#pragma GCC visibility pop
