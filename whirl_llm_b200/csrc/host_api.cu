// whirl_sample_rows_host: the fused sampler for callers whose logits live in HOST memory.  It owns device staging
// (allocated on first use, grown when a larger batch comes, released by whirl_host_release) and overlaps the
// host-to-device copy of one block of rows with the sampling of the previous one on two streams.
#include "../../include/whirl_b200.h"

#include <cuda_runtime.h>

#include <algorithm>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

namespace {

struct Staging {
    int device = -1;
    cudaStream_t st[2] = {nullptr, nullptr};
    void* logits[2] = {nullptr, nullptr};
    size_t logits_bytes = 0;
    void* ws[2] = {nullptr, nullptr};
    size_t ws_bytes = 0;
    void* prm = nullptr;  // parameter and output arrays of the whole batch
    size_t prm_bytes = 0;
    cudaEvent_t prm_ready = nullptr;
};
Staging g_s;
std::mutex g_mu;
thread_local std::string g_herr;

void release_locked() {
    if (g_s.device < 0) return;
    cudaSetDevice(g_s.device);
    for (int i = 0; i < 2; ++i) {
        if (g_s.logits[i]) cudaFree(g_s.logits[i]);
        if (g_s.ws[i]) cudaFree(g_s.ws[i]);
        if (g_s.st[i]) cudaStreamDestroy(g_s.st[i]);
    }
    if (g_s.prm) cudaFree(g_s.prm);
    if (g_s.prm_ready) cudaEventDestroy(g_s.prm_ready);
    g_s = Staging{};
}

size_t up(size_t v) { return (v + 255) / 256 * 256; }

#define CK(call)                                                              \
    do {                                                                      \
        const cudaError_t e_ = (call);                                        \
        if (e_ != cudaSuccess) {                                              \
            g_herr = std::string(#call) + ": " + cudaGetErrorString(e_);      \
            return WHIRL_ERR_CUDA;                                            \
        }                                                                     \
    } while (0)

}  // namespace

#pragma GCC visibility push(default)
extern "C" {

const char* whirl_host_last_error(void) { return g_herr.c_str(); }

void whirl_host_release(void) {
    std::lock_guard<std::mutex> lk(g_mu);
    release_locked();
}

int whirl_sample_rows_host(const void* x, int dtype, int rows, int n, const whirl_sample_params* p, const whirl_sample_out* o,
                           int device) {
    if (!x || !p || !o || !o->token || rows < 0 || n <= 0 || (dtype != WHIRL_F32 && dtype != WHIRL_BF16)) {
        g_herr = "sample_rows_host: bad pointer / rows / n / dtype";
        return WHIRL_ERR_INVALID;
    }
    if (rows == 0) return WHIRL_OK;
    std::lock_guard<std::mutex> lk(g_mu);
    CK(cudaSetDevice(device));
    if (g_s.device >= 0 && g_s.device != device) release_locked();
    const size_t es = dtype == WHIRL_F32 ? 4 : 2;
    const size_t row_bytes = size_t(n) * es;
    // rows per block: about 64 MiB of logits, so that copies run at full PCIe rate and sampling hides behind them
    int blk = int(std::max<size_t>(1, (size_t(64) << 20) / row_bytes));
    blk = std::min(blk, rows);
    if (g_s.device < 0) {
        g_s.device = device;
        for (int i = 0; i < 2; ++i) CK(cudaStreamCreateWithFlags(&g_s.st[i], cudaStreamNonBlocking));
        CK(cudaEventCreateWithFlags(&g_s.prm_ready, cudaEventDisableTiming));
    }
    const size_t need_l = size_t(blk) * row_bytes;
    if (g_s.logits_bytes < need_l) {
        for (int i = 0; i < 2; ++i) {
            if (g_s.logits[i]) CK(cudaFree(g_s.logits[i]));
            g_s.logits[i] = nullptr;
            CK(cudaMalloc(&g_s.logits[i], need_l));
        }
        g_s.logits_bytes = need_l;
    }
    const size_t need_w = whirl_workspace_bytes(blk, n);
    if (g_s.ws_bytes < need_w) {
        for (int i = 0; i < 2; ++i) {
            if (g_s.ws[i]) CK(cudaFree(g_s.ws[i]));
            g_s.ws[i] = nullptr;
            CK(cudaMalloc(&g_s.ws[i], need_w));
        }
        g_s.ws_bytes = need_w;
    }
    // ---- device copies of the per-row arrays
    struct Arr {
        const void* host;
        size_t elem;   // bytes per row
        size_t off;
    };
    const size_t H = p->hist ? size_t(p->hist_stride) : 0;
    Arr in[12] = {{p->inv_t, 4, 0}, {p->top_k, 4, 0}, {p->top_p, 8, 0}, {p->min_p, 8, 0}, {p->greedy, 1, 0}, {p->u, 8, 0},
                  {p->race_key, 8, 0}, {p->hist, 4 * H, 0}, {p->hist_len, 4, 0}, {p->rep, 4, 0}, {p->pres, 4, 0}, {p->freq, 4, 0}};
    const size_t cap = size_t(std::max(o->kept_cap, 0));
    Arr out[7] = {{o->token, 4, 0}, {o->status, 4, 0}, {o->n_kept, 4, 0}, {o->closed, 4, 0}, {o->stats, 8, 0},
                  {o->kept_ids, 4 * cap, 0}, {o->kept_p, 8 * cap, 0}};
    size_t tot = 0;
    for (Arr& a : in) a.off = tot, tot += a.host ? up(a.elem * rows) : 0;
    for (Arr& a : out) a.off = tot, tot += a.host ? up(a.elem * rows) : 0;
    const size_t cnt_off = tot;
    tot += 256;
    if (g_s.prm_bytes < tot) {
        if (g_s.prm) CK(cudaFree(g_s.prm));
        g_s.prm = nullptr;
        CK(cudaMalloc(&g_s.prm, tot));
        g_s.prm_bytes = tot;
    }
    uint8_t* base = static_cast<uint8_t*>(g_s.prm);
    for (const Arr& a : in)
        if (a.host && a.elem) CK(cudaMemcpyAsync(base + a.off, a.host, a.elem * rows, cudaMemcpyHostToDevice, g_s.st[0]));
    CK(cudaMemsetAsync(base + cnt_off, 0, 256, g_s.st[0]));
    CK(cudaEventRecord(g_s.prm_ready, g_s.st[0]));
    CK(cudaStreamWaitEvent(g_s.st[1], g_s.prm_ready, 0));
    // ---- blocks of rows, alternating streams
    int b = 0;
    for (int r0 = 0; r0 < rows; r0 += blk, ++b) {
        const int nr = std::min(blk, rows - r0);
        const int s = b & 1;
        CK(cudaMemcpyAsync(g_s.logits[s], static_cast<const uint8_t*>(x) + size_t(r0) * row_bytes, size_t(nr) * row_bytes,
                           cudaMemcpyHostToDevice, g_s.st[s]));
        auto at = [&](const Arr& a) -> void* { return a.host ? base + a.off + a.elem * size_t(r0) : nullptr; };
        whirl_sample_params dp{};
        dp.inv_t = static_cast<const float*>(at(in[0])), dp.top_k = static_cast<const int32_t*>(at(in[1]));
        dp.top_p = static_cast<const double*>(at(in[2])), dp.min_p = static_cast<const double*>(at(in[3]));
        dp.greedy = static_cast<const uint8_t*>(at(in[4])), dp.u = static_cast<const double*>(at(in[5]));
        dp.race_key = static_cast<const uint64_t*>(at(in[6])), dp.hist = static_cast<const int32_t*>(at(in[7]));
        dp.hist_len = static_cast<const int32_t*>(at(in[8])), dp.hist_stride = p->hist_stride;
        dp.rep = static_cast<const float*>(at(in[9])), dp.pres = static_cast<const float*>(at(in[10])), dp.freq = static_cast<const float*>(at(in[11]));
        whirl_sample_out dout{};
        dout.token = static_cast<int32_t*>(at(out[0])), dout.status = static_cast<int32_t*>(at(out[1]));
        dout.n_kept = static_cast<int32_t*>(at(out[2])), dout.closed = static_cast<int32_t*>(at(out[3]));
        dout.stats = static_cast<float*>(at(out[4])), dout.kept_ids = static_cast<int32_t*>(at(out[5]));
        dout.kept_p = static_cast<double*>(at(out[6])), dout.kept_cap = o->kept_cap;
        dout.counters = reinterpret_cast<uint32_t*>(base + cnt_off);  // (always: the error report comes through them)
        const int rc = whirl_sample_rows(g_s.logits[s], dtype, nr, n, &dp, &dout, g_s.ws[s], g_s.ws_bytes, g_s.st[s]);
        if (rc != WHIRL_OK) {
            g_herr = whirl_last_error();
            return rc;
        }
        void* host_out[7] = {o->token, o->status, o->n_kept, o->closed, o->stats, o->kept_ids, o->kept_p};
        for (int i = 0; i < 7; ++i)
            if (out[i].host && out[i].elem)
                CK(cudaMemcpyAsync(static_cast<uint8_t*>(host_out[i]) + out[i].elem * size_t(r0), base + out[i].off + out[i].elem * size_t(r0),
                                   out[i].elem * nr, cudaMemcpyDeviceToHost, g_s.st[s]));
    }
    CK(cudaStreamSynchronize(g_s.st[0]));
    CK(cudaStreamSynchronize(g_s.st[1]));
    uint32_t c[WHIRL_CNT_WORDS];
    CK(cudaMemcpy(c, base + cnt_off, sizeof c, cudaMemcpyDeviceToHost));
    if (o->counters)
        for (int i = 0; i < WHIRL_CNT_WORDS; ++i) o->counters[i] += c[i];
    if (c[WHIRL_CNT_TIMEOUT]) {
        g_herr = "sample_rows_host: a bounded device-side wait ran out in " + std::to_string(c[WHIRL_CNT_TIMEOUT]) + " chunk(s); " +
                 std::to_string(c[WHIRL_CNT_UNRESOLVED]) + " row(s) without an answer";
        return WHIRL_ERR_TIMEOUT;
    }
    return WHIRL_OK;
}

}  // extern "C"
#pragma GCC visibility pop
