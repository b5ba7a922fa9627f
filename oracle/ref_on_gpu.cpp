// The reference's OWN host sampling code (SampleBuffers, filterCands, sampleRow, Acceptor: compiled in place from the
// reference checkout, see oracle/Makefile) running UNCHANGED on top of this library's GPU kernels, through the two seams
// the reference engine itself uses:
//   server::ServerModel::topkRows  ->  whirl_topk_rows           (src/server/backend.h:96-99)
//   device::Backend::download      ->  cudaMemcpy device-to-host (src/device/backend.h:38-40)
// TEST INFRASTRUCTURE ONLY (built into oracle/_ref/, run by tests/test_gpu_ref_seam.py).  For every seeded case the same
// reference code also runs over the reference's host double (tests/iso/fake_server_model.h, host memory); the accept
// counts, chosen tokens, kept-set sizes and escalation counters of the two runs must be identical.
#include <cuda_runtime.h>

#include "iso/fake_server_model.h"
#include "sampling/acceptor.h"
#include "sampling/sampler.h"
#include "server/engine_sampling.h"
#include "whirl/relax_accept.h"
#include "whirl_b200.h"

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <optional>
#include <span>
#include <vector>

using namespace whirl;

namespace {

#define CUDA_OK(x)                                                                  \
    do {                                                                            \
        const cudaError_t e_ = (x);                                                 \
        if (e_ != cudaSuccess) {                                                    \
            std::fprintf(stderr, "%s: %s\n", #x, cudaGetErrorString(e_));          \
            std::exit(2);                                                           \
        }                                                                           \
    } while (0)

// device::Backend over the CUDA runtime; host::Backend over malloc (the reference's NullBackend is Windows-only)
class Backend final : public device::Backend {
public:
    explicit Backend(bool gpu) : gpu_(gpu) {}
    void copyAsync(device::DevPtr dst, device::DevPtr src, std::uint64_t bytes, device::Stream) override {
        if (gpu_) CUDA_OK(cudaMemcpy(reinterpret_cast<void*>(dst), reinterpret_cast<const void*>(src), bytes, cudaMemcpyDefault));
        else std::memcpy(reinterpret_cast<void*>(dst), reinterpret_cast<const void*>(src), bytes);
    }
    void download(void* dst, device::DevPtr src, std::uint64_t bytes) override {
        if (gpu_) CUDA_OK(cudaMemcpy(dst, reinterpret_cast<const void*>(src), bytes, cudaMemcpyDeviceToHost));
        else std::memcpy(dst, reinterpret_cast<const void*>(src), bytes);
    }
    device::Stream streamCreateNonBlocking() override { return nullptr; }
    void streamDestroy(device::Stream) override {}
    void streamSync(device::Stream) override {}
    void streamWaitEvent(device::Stream, device::Event) override {}
    device::Event eventCreate() override { return nullptr; }
    void eventDestroy(device::Event) override {}
    void eventRecord(device::Event, device::Stream) override {}
    bool eventDone(device::Event) override { return true; }
    void eventSync(device::Event) override {}
    void* hostMalloc(std::uint64_t bytes) override { return std::malloc(bytes); }
    void hostFree(void* p) override { std::free(p); }
    device::DevPtr malloc(std::uint64_t bytes) override {
        void* p = nullptr;
        if (gpu_) {
            CUDA_OK(cudaMalloc(&p, bytes ? bytes : 1));
            CUDA_OK(cudaMemset(p, 0, bytes ? bytes : 1));
        } else {
            p = std::calloc(bytes ? bytes : 1, 1);
        }
        return reinterpret_cast<device::DevPtr>(p);
    }
    void free(device::DevPtr p) override {
        if (gpu_) cudaFree(reinterpret_cast<void*>(p));
        else std::free(reinterpret_cast<void*>(p));
    }
    void setDevice(int) override {}
    const char* lastErrorString() const override { return ""; }
    hip::MemInfo memInfo() override { return {}; }
    hip::WddmMemInfo wddmMemInfo() override { return {}; }
    hip::LocalMemSnap localMemSnap() override { return {}; }
    hip::UmaMem umaMemory(int) override { return {}; }

private:
    bool gpu_;
};

// server::ServerModel whose logits live on the GPU and whose topkRows is this library's kernel; everything the sampling
// path does not call is a no-op, as in the reference's own test double
class GpuModel final : public server::ServerModel {
public:
    GpuModel(device::Backend& ops, std::uint32_t n_vocab, std::uint32_t rows) : ops_(ops) {
        cfg_.n_vocab = n_vocab;
        cfg_.n_embd = 8;
        logits_ = ops_.malloc(static_cast<std::uint64_t>(n_vocab) * 4 * rows);
        ws_bytes_ = whirl_workspace_bytes(static_cast<int>(rows), static_cast<int>(n_vocab));
        ws_ = ops_.malloc(ws_bytes_);
    }
    ~GpuModel() override {
        ops_.free(logits_);
        ops_.free(ws_);
    }
    const qwen35::Config& cfg() const override { return cfg_; }
    device::Stream stream() const override { return {}; }
    server::DevPtr logits() const override { return logits_; }
    server::DevPtr hn() const override { return logits_; }
    server::DevPtr mtpH() const override { return logits_; }
    server::DevPtr seqHid(std::uint32_t) const override { return logits_; }
    std::span<const server::DevPtr> convState() const override { return {}; }
    std::span<const server::DevPtr> ssmState() const override { return {}; }
    std::uint64_t convBytes() const override { return 0; }
    std::uint64_t ssmBytes() const override { return 0; }
    std::uint32_t curSeq() const override { return 0; }
    std::uint32_t poolPages() const override { return 0; }
    std::uint32_t seqPages() const override { return 0; }
    std::uint32_t maxBatch() const override { return qwen35::max_small_batch; }
    std::uint32_t snapSets() const override { return 0; }
    void ensureSnapshots(std::uint32_t) override {}
    bool gdnReplay() const override { return false; }
    bool fusedDecode() const override { return false; }
    bool canSegment() const override { return false; }
    std::vector<server::KvArr> kvArrays() const override { return {}; }
    void selectSeq(std::uint32_t) override {}
    void commitSeq(std::uint32_t) override {}
    void dropPending(std::uint32_t) override {}
    void setPending(std::uint32_t, std::uint32_t) override {}
    void restoreSeqSnapshot(std::uint32_t, std::uint32_t) override {}
    void mapPages(std::uint32_t, std::uint32_t, std::span<const std::int32_t>) override {}
    void reset() override {}
    void forward(std::span<const std::uint32_t>, std::uint32_t) override {}
    void prefillMtpChunk(std::span<const std::uint32_t>, std::uint32_t, std::size_t, std::size_t, std::optional<server::DevPtr>) override {}
    void prefillSegs(std::span<const server::PSeg>, bool) override {}
    void segLogitsToFront(std::uint32_t) override {}
    std::uint32_t argmax() override {
        int* d = nullptr;
        CUDA_OK(cudaMalloc(&d, 4));
        if (whirl_argmax(reinterpret_cast<const void*>(logits_), WHIRL_F32, static_cast<int>(cfg_.n_vocab), d, nullptr, nullptr, 0,
                         reinterpret_cast<void*>(ws_), ws_bytes_, nullptr) != WHIRL_OK)
            std::exit(3);
        int h = 0;
        CUDA_OK(cudaMemcpy(&h, d, 4, cudaMemcpyDeviceToHost));
        cudaFree(d);
        return static_cast<std::uint32_t>(h);
    }
    void setDraftCutoff(float, std::uint32_t) override {}
    void mtpBatchStepEx(std::span<const server::MSeg>, std::uint32_t, bool) override {}
    std::uint32_t verifyBatchEnqueue(std::span<const server::VSeg>) override { return 0; }
    void readCtl(std::span<std::int32_t>) override {}
    void mtpEnqueue(server::DevPtr, std::span<const std::uint32_t>, std::uint32_t) override {}
    // the seam: ServerModel::topkRows -> whirl_topk_rows, asynchronous on the (default) model stream
    void topkRows(std::uint32_t row0, std::uint32_t rows, std::uint32_t k, float inv_t, server::DevPtr ids, server::DevPtr vals,
                  server::DevPtr stats) override {
        const auto* x = reinterpret_cast<const float*>(logits_) + static_cast<std::uint64_t>(row0) * cfg_.n_vocab;
        const int rc = whirl_topk_rows(x, WHIRL_F32, static_cast<int>(rows), static_cast<int>(cfg_.n_vocab), static_cast<int>(k), inv_t,
                                       nullptr, reinterpret_cast<int*>(ids), reinterpret_cast<float*>(vals),
                                       reinterpret_cast<float*>(stats), reinterpret_cast<void*>(ws_), ws_bytes_, nullptr);
        if (rc != WHIRL_OK) {
            std::fprintf(stderr, "whirl_topk_rows: %s\n", whirl_last_error());
            std::exit(3);
        }
        ++launches;
    }
    int launches = 0;

private:
    device::Backend& ops_;
    qwen35::Config cfg_{};
    server::DevPtr logits_ = 0, ws_ = 0;
    std::size_t ws_bytes_ = 0;
};

std::uint32_t lcg(std::uint32_t& s) {
    s = s * 1664525u + 1013904223u;
    return s >> 8;
}

struct Outcome {
    std::uint32_t acc, chosen, big, full, relaxed;
    std::size_t n;
    bool closed;
    bool operator==(const Outcome& o) const {
        return acc == o.acc && chosen == o.chosen && big == o.big && full == o.full && relaxed == o.relaxed && n == o.n && closed == o.closed;
    }
};

template <class Model>
Outcome runCase(Model& model, device::Backend& ops, const std::vector<float>& rows_host, std::uint32_t n_rows, std::uint32_t V,
                sampling::Sampler proto, const std::vector<std::uint32_t>& dr, std::uint32_t nd, bool typ, std::uint32_t n_gen,
                const relax::Params& rp) {
    ops.copyAsync(model.logits(), reinterpret_cast<device::DevPtr>(rows_host.data()), static_cast<std::uint64_t>(n_rows) * V * 4, nullptr);
    server::SampleBuffers sb(model, ops);
    sb.alloc(1, false, 0);
    sampling::Sampler sm = proto;
    sm.cands = sb.cands();
    sb.fetchCands(sm, n_rows);  // the engine's first launch: top-256 of every verify row, one download
    const sampling::Acceptor acceptor(rp);
    const sampling::Drafts d{std::span<const std::uint32_t>(dr.data(), dr.size()), nd, 0};
    std::uint32_t relaxed = 0;
    const sampling::RepeatGuard repeats = [](std::uint32_t) { return false; };
    const sampling::Accepted a = acceptor.sample(sb, sm, d, typ, n_gen, repeats, relaxed);
    return Outcome{a.acc, a.chosen, sm.big_used, sm.full_used, relaxed, sm.n, sm.closed};
}

}  // namespace

int main(int argc, char** argv) {
    const int n_cases = argc > 1 ? std::atoi(argv[1]) : 60;
    const std::uint32_t V = 20000;  // > k_big, so every escalation level is reachable (as the reference's own iso test)
    Backend gpu_ops(true), host_ops(false);
    GpuModel gpu(gpu_ops, V, qwen35::max_small_batch);
    test::FakeServerModel host(host_ops, V);
    std::uint32_t g = 0xB200u;
    int same = 0, accepted = 0, escal = 0, walks = 0;
    for (int it = 0; it < n_cases; ++it) {
        const std::uint32_t nd = lcg(g) % 5, n_rows = nd + 1;
        const float spreads[6] = {0.3f, 1.0f, 2.0f, 3.0f, 4.0f, 6.0f};
        const float spread = spreads[lcg(g) % 6];
        std::vector<float> rows(static_cast<std::size_t>(n_rows) * V);
        std::uint32_t ls = lcg(g);
        for (auto& l : rows) l = static_cast<float>(static_cast<int>(lcg(ls) % 20001) - 10000) / 10000.0f * spread;
        sampling::Sampler sm;
        const double temps[4] = {0.5, 0.8, 1.0, 1.6};
        sm.temp = temps[lcg(g) % 4];
        sm.inv_t = static_cast<float>(1.0 / sm.temp);
        const std::uint32_t tks[5] = {0, 0, 5, 40, 600};
        sm.top_k = tks[lcg(g) % 5];
        const double tps[4] = {1, 1, 0.9, 0.97};
        sm.top_p = tps[lcg(g) % 4];
        const double mps[3] = {0, 0, 0.05};
        sm.min_p = mps[lcg(g) % 3];
        sm.seed = lcg(g);
        sm.race = lcg(g) % 2 == 0;
        const std::uint32_t n_gen = lcg(g) % 1000;
        const bool typ = lcg(g) % 3 == 0;
        relax::Params rp;
        rp.on = typ;
        // drafts: the row's best tokens, so that some are accepted
        std::vector<std::uint32_t> dr(15, 0);
        for (std::uint32_t r = 0; r < nd; ++r) {
            const float* x = rows.data() + static_cast<std::size_t>(r) * V;
            std::uint32_t b = 0;
            for (std::uint32_t i = 1; i < V; ++i)
                if (x[i] > x[b]) b = i;
            dr[r] = lcg(g) % 4 == 0 ? (b + 1) % V : b;
        }
        const Outcome a = runCase(gpu, gpu_ops, rows, n_rows, V, sm, dr, nd, typ, n_gen, rp);
        const Outcome b = runCase(host, host_ops, rows, n_rows, V, sm, dr, nd, typ, n_gen, rp);
        if (a == b) ++same;
        else
            std::fprintf(stderr, "case %d differs: gpu acc %u chosen %u n %zu big %u full %u | host acc %u chosen %u n %zu big %u full %u\n", it,
                         a.acc, a.chosen, a.n, a.big, a.full, b.acc, b.chosen, b.n, b.big, b.full);
        accepted += static_cast<int>(b.acc);
        escal += static_cast<int>(b.big);
        walks += static_cast<int>(b.full);
    }
    // greedy seam: ServerModel::argmax
    std::vector<float> one(V);
    std::uint32_t ls = 77;
    for (auto& l : one) l = static_cast<float>(lcg(ls) % 1000);
    one[123] = one[9000] = 5000.f;
    gpu_ops.copyAsync(gpu.logits(), reinterpret_cast<device::DevPtr>(one.data()), static_cast<std::uint64_t>(V) * 4, nullptr);
    const bool greedy_ok = gpu.argmax() == 123u;
    std::printf("ref_on_gpu: %d / %d cases identical, accepted drafts %d, escalations %d, full-row reads %d, kernel launches %d, argmax %s\n",
                same, n_cases, accepted, escal, walks, gpu.launches, greedy_ok ? "ok" : "WRONG");
    return (same == n_cases && greedy_ok && gpu.launches > 0) ? 0 : 1;
}
