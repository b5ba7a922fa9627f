// C entry points over the UNMODIFIED reference sampling sources.  TEST INFRASTRUCTURE ONLY.
//
// This file is compiled together with the reference's own src/sampling/sampler.cpp, src/sampling/acceptor.cpp,
// src/common/spec_sample.cpp and src/server/engine_sampling.cpp, taken in place from the reference checkout (see
// oracle/Makefile; nothing of the reference is copied into this repository), into oracle/_ref/libwhirl_ref.so.
// It exists to (1) pin oracle/whirl_oracle.c against the real reference code, (2) generate the fixtures under
// tests/golden/, and (3) serve as the "reference" CPU arm of bench.py.  The shipped library never loads it.
//
// The struct layouts mirror oracle/whirl_oracle.c so that one ctypes binding drives both.
// The reference's test doubles are used as they are: tests/iso/fake_server_model.h (host topkRows) under the real
// SampleBuffers, and tests/server/sampling_cases.h (hostPrepare with its 4 / 16 escalation sizes) for small
// vocabularies.  The only new piece is HostBackend, a device::Backend whose "device" is host memory, because the
// reference's NullBackend builds on Windows only (src/device/null_backend.cpp).

#include "iso/fake_server_model.h"
#include "sampling/acceptor.h"
#include "sampling/sampler.h"
#include "server/engine_sampling.h"
#include "whirl/model_types.h"
#include "whirl/relax_accept.h"
#include "whirl/spec_sample.h"

#include <algorithm>
#include <array>
#include <atomic>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <limits>
#include <optional>
#include <set>
#include <span>
#include <string>
#include <thread>
#include <vector>

// the reference's fixed acceptance cases and its host row-prepare, included the way its own test program does
// (tests/sampling/sampling_tests.cpp:36-41)
namespace whirl::server {
using sampling::Cand;
using sampling::Sampler;
#include "server/sampling_oldref.inc"
#include "server/sampling_cases.h"
}  // namespace whirl::server

using namespace whirl;

namespace {

class HostBackend final : public device::Backend {
public:
    void copyAsync(device::DevPtr dst, device::DevPtr src, std::uint64_t bytes, device::Stream) override {
        std::memcpy(reinterpret_cast<void*>(dst), reinterpret_cast<const void*>(src), bytes);
    }
    void download(void* dst, device::DevPtr src, std::uint64_t bytes) override {
        std::memcpy(dst, reinterpret_cast<const void*>(src), bytes);
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
        return reinterpret_cast<device::DevPtr>(std::calloc(bytes ? bytes : 1, 1));
    }
    void free(device::DevPtr p) override { std::free(reinterpret_cast<void*>(p)); }
    void setDevice(int) override {}
    const char* lastErrorString() const override { return ""; }
    hip::MemInfo memInfo() override { return {}; }
    hip::WddmMemInfo wddmMemInfo() override { return {}; }
    hip::LocalMemSnap localMemSnap() override { return {}; }
    hip::UmaMem umaMemory(int) override { return {}; }
};

struct Sm {  // == orc_sampler
    float inv_t;
    std::uint32_t top_k;
    double top_p, min_p;
    std::uint64_t seed, pos_idx;
    std::int32_t race;
    std::uint32_t n;
    std::int32_t closed;
    float m, sum;
    std::uint32_t full_used, big_used;
    std::int32_t use_u;
    double u_given;
};
struct RowOut {  // == orc_row_out
    std::uint32_t token, n;
    std::int32_t closed;
    float m, sum;
    std::uint32_t big_used, full_used;
};
struct Batch {  // == orc_batch
    const float* inv_t;
    const std::uint32_t* top_k;
    const double* top_p;
    const double* min_p;
    const std::uint8_t* greedy;
    const std::uint8_t* race;
    const std::uint64_t* seed;
    const std::uint64_t* pos_idx;
    const double* u;
    const std::int32_t* hist;
    const std::uint32_t* hist_len;
    std::uint64_t hist_stride;
    const float* rep;
    const float* pres;
    const float* freq;
    std::uint32_t ks, kb;
};
struct Accepted {  // == orc_accepted
    std::uint32_t acc, chosen, relaxed;
    double relax_gap;
    std::uint64_t pos_idx;
    std::uint32_t full_used, big_used;
};
struct Relax {  // == orc_relax
    std::int32_t on;
    std::uint32_t k;
    float alpha, eps, delta;
};
struct QD {  // == orc_qdist
    std::uint32_t n;
    std::uint32_t id[32];
    float p[32];
};

sampling::Sampler toSampler(const Sm& s, std::vector<sampling::Cand>* cands) {
    sampling::Sampler o;
    o.temp = s.inv_t > 0 ? 1.0 / s.inv_t : 0;
    o.inv_t = s.inv_t;
    o.top_k = s.top_k;
    o.top_p = s.top_p;
    o.min_p = s.min_p;
    o.seed = s.seed;
    o.pos_idx = s.pos_idx;
    o.race = s.race != 0;
    o.cands = cands;
    o.m = s.m;
    o.sum = s.sum;
    return o;
}
void fromSampler(const sampling::Sampler& o, Sm& s) {
    s.n = static_cast<std::uint32_t>(o.n);
    s.closed = o.closed;
    s.m = o.m;
    s.sum = o.sum;
    s.pos_idx = o.pos_idx;
    s.full_used = o.full_used;
    s.big_used = o.big_used;
}
relax::Params toRelax(const Relax& r) {
    relax::Params p;
    p.on = r.on != 0;
    p.k = r.k;
    p.alpha = r.alpha;
    p.eps = r.eps;
    p.delta = r.delta;
    return p;
}

// sampling::RowSource over host rows with the reference test's hostPrepare (escalation sizes acase::ks / acase::kb)
struct SmallRows final : sampling::RowSource {
    const std::vector<std::vector<float>>* rows = nullptr;
    std::vector<std::uint8_t> marks;
    server::acase::Trace tr;
    std::uint32_t V = 0;
    void prepareRow(sampling::Sampler& s, std::uint32_t r) override {
        server::acase::hostPrepare(
            s, r, *rows, [](sampling::Sampler& x, std::size_t n, bool c) { return sampling::filterCands(x, n, c); }, tr);
    }
    const float* loadFullRow(std::uint32_t gr) override { return (*rows)[gr].data(); }
    float logitAt(std::uint32_t gr, std::uint32_t t) override { return (*rows)[gr][t]; }
    std::uint32_t nVocab() const override { return V; }
    std::uint8_t* inCands() override { return marks.data(); }
};

int firstMax(const float* x, std::uint32_t n) {  // tests/kernels/test_misc.cpp:30-35
    std::uint32_t b = 0;
    for (std::uint32_t i = 1; i < n; ++i)
        if (x[i] > x[b]) b = i;
    return static_cast<int>(b);
}

void engineRows(const float* x, std::uint32_t V, const Batch* b, RowOut* out, std::uint32_t* kept_ids, double* kept_p,
                std::uint32_t kept_cap, std::uint32_t r0, std::uint32_t r1) {
    HostBackend hb;
    test::FakeServerModel model(hb, V);
    server::SampleBuffers sb(model, hb);
    sb.alloc(1, false, 0);
    auto* lg = reinterpret_cast<float*>(model.logits());
    const std::uint32_t group = qwen35::max_small_batch;
    for (std::uint32_t g0 = r0; g0 < r1; g0 += group) {
        const std::uint32_t g1 = std::min(r1, g0 + group);
        std::memcpy(lg, x + static_cast<std::size_t>(g0) * V, static_cast<std::size_t>(g1 - g0) * V * 4);
        for (std::uint32_t r = g0; r < g1; ++r) {
            RowOut& o = out[r];
            if (b->greedy && b->greedy[r]) {
                const float* xr = lg + static_cast<std::size_t>(r - g0) * V;
                o = RowOut{static_cast<std::uint32_t>(firstMax(xr, V)), 1, 1, 0, 0, 0, 0};
                o.m = xr[o.token];
                if (kept_ids && kept_cap) kept_ids[static_cast<std::size_t>(r) * kept_cap] = o.token;
                if (kept_p && kept_cap) kept_p[static_cast<std::size_t>(r) * kept_cap] = 1.0;
                continue;
            }
            sampling::Sampler s;
            s.cands = sb.cands();
            s.inv_t = b->inv_t ? b->inv_t[r] : 1.f;
            s.temp = 1.0 / s.inv_t;
            s.top_k = b->top_k ? b->top_k[r] : 0;
            s.top_p = b->top_p ? b->top_p[r] : 1.0;
            s.min_p = b->min_p ? b->min_p[r] : 0.0;
            s.seed = b->seed ? b->seed[r] : 0;
            s.pos_idx = b->pos_idx ? b->pos_idx[r] : 0;
            s.race = b->race && b->race[r];
            // the engine's order for one slot: the small top-k of its rows, then prepareRow, then the draw
            // (src/server/engine_prefill.cpp:204-211); inv_t differs per row here, so one fetch per row
            s.row_base = 0;
            sb.launchTopk(r - g0, 1, server::k_small, s.inv_t, sb.sampDev(), server::max_rows, r - g0);
            hb.download(sb.sampHost().data(), sb.sampDev(), server::SampleBuffers::sampBytes());
            sb.prepareRow(s, r - g0);
            const std::uint32_t nk = std::min<std::uint32_t>(static_cast<std::uint32_t>(s.n), kept_cap);
            for (std::uint32_t i = 0; i < nk; ++i) {
                if (kept_ids) kept_ids[static_cast<std::size_t>(r) * kept_cap + i] = (*s.cands)[i].id;
                if (kept_p) kept_p[static_cast<std::size_t>(r) * kept_cap + i] = (*s.cands)[i].p;
            }
            o.n = static_cast<std::uint32_t>(s.n);
            o.closed = s.closed;
            o.m = s.m;
            o.sum = s.sum;
            o.token = sampling::sampleRow(sb, s, std::nullopt, 0);
            o.big_used = s.big_used;
            o.full_used = s.full_used;
        }
    }
}

}  // namespace

extern "C" {

double ref_uniform(std::uint64_t seed, std::uint64_t pos, std::uint32_t stream) { return spec::uniform(seed, pos, stream); }
double ref_sampler_uniform(std::uint64_t seed, std::uint64_t pos) {
    sampling::Sampler s;
    s.seed = seed;
    s.pos_idx = pos;
    return s.uniform();
}
std::uint64_t ref_race_base(std::uint64_t seed, std::uint64_t pos) { return spec::raceBase(seed, pos); }
double ref_race_e(std::uint64_t base, std::uint32_t token) { return spec::raceE(base, token); }

// sampling::filterCands on explicit candidates
int ref_filter_cands(Sm* s, std::uint32_t* ids, float* logits, double* p, std::uint32_t count, int complete) {
    std::vector<sampling::Cand> c(count);
    for (std::uint32_t i = 0; i < count; ++i) c[i] = {ids[i], logits[i], 0};
    sampling::Sampler o = toSampler(*s, &c);
    const bool ok = sampling::filterCands(o, count, complete != 0);
    fromSampler(o, *s);
    for (std::uint32_t i = 0; i < count; ++i) ids[i] = c[i].id, logits[i] = c[i].logit, p[i] = c[i].p;
    return ok;
}

// rows through the real engine buffers: SampleBuffers over FakeServerModel::topkRows (k_small 256, k_big 16384),
// filterCands, sampleRow.  V >= 16384 (the engine's k_big launch reads that many candidates).  The reference has no
// penalties, no bf16 rows and draws its uniform from (seed, pos_idx): a batch that asks for those is refused (-1).
int ref_sample_rows(const float* x, const std::uint16_t* xb, std::uint32_t rows, std::uint32_t V, const Batch* b,
                    RowOut* out, std::uint32_t* kept_ids, double* kept_p, std::uint32_t kept_cap, int threads) {
    if (!x || xb || b->u || b->hist || V < server::k_big) return -1;
    if (threads < 1) threads = 1;
    if (static_cast<std::uint32_t>(threads) > rows) threads = rows ? static_cast<int>(rows) : 1;
    std::vector<std::thread> th;
    for (int t = 1; t < threads; ++t)
        th.emplace_back(engineRows, x, V, b, out, kept_ids, kept_p, kept_cap,
                        static_cast<std::uint32_t>(static_cast<std::uint64_t>(rows) * t / threads),
                        static_cast<std::uint32_t>(static_cast<std::uint64_t>(rows) * (t + 1) / threads));
    engineRows(x, V, b, out, kept_ids, kept_p, kept_cap, 0, static_cast<std::uint32_t>(static_cast<std::uint64_t>(rows) / threads));
    for (auto& t : th) t.join();
    return 0;
}

// The timed CPU arm of the benchmark: `threads` persistent workers, each with ONE FakeServerModel + SampleBuffers kept for
// the whole call, each sampling its own block of rows `reps` times (output index pos_idx + rep * rows, so every pass
// draws with fresh uniforms).  Per row and pass: the raw row is copied into the model's logits buffer (the stand-in for
// the forward pass that leaves logits there), this repository's penalty rule is applied to it (the reference has no
// penalties, src/server/engine_start.cpp:70-73; rule: oracle/whirl_oracle.c, orc_apply_penalties), then the reference's
// own launchTopk -> download -> SampleBuffers::prepareRow -> sampleRow runs unchanged
// (src/server/engine_prefill.cpp:204-211).  Set-up (allocations, thread start) is outside the time: *seconds is the
// span from the moment every worker is ready to the moment the last one is done.  tokens[rows]: the first pass.
int ref_bench_rows(const float* x, std::uint32_t rows, std::uint32_t V, const Batch* b, int threads, int reps, double* seconds,
                   std::uint32_t* tokens) {
    if (!x || !seconds || b->u || V < server::k_big || rows == 0 || reps < 1) return -1;
    if (threads < 1) threads = 1;
    if (static_cast<std::uint32_t>(threads) > rows) threads = static_cast<int>(rows);
    std::atomic<int> ready{0};
    std::atomic<bool> go{false};
    using clk = std::chrono::steady_clock;
    std::vector<clk::time_point> t_end(threads);
    clk::time_point t_start;
    auto worker = [&](int t) {
        const std::uint32_t r0 = static_cast<std::uint32_t>(static_cast<std::uint64_t>(rows) * t / threads);
        const std::uint32_t r1 = static_cast<std::uint32_t>(static_cast<std::uint64_t>(rows) * (t + 1) / threads);
        HostBackend hb;
        test::FakeServerModel model(hb, V);
        server::SampleBuffers sb(model, hb);
        sb.alloc(1, false, 0);
        auto* lg = reinterpret_cast<float*>(model.logits());
        std::vector<std::uint16_t> cnt(V, 0);
        std::vector<std::uint32_t> seen;
        seen.reserve(4096);
        ready.fetch_add(1);
        while (!go.load(std::memory_order_acquire)) std::this_thread::yield();
        for (int rep = 0; rep < reps; ++rep) {
            for (std::uint32_t r = r0; r < r1; ++r) {
                std::memcpy(lg, x + static_cast<std::size_t>(r) * V, static_cast<std::size_t>(V) * 4);
                if (b->hist && b->hist_len && b->hist_len[r] > 0) {
                    const float rp = b->rep ? b->rep[r] : 1.f, pr = b->pres ? b->pres[r] : 0.f, fr = b->freq ? b->freq[r] : 0.f;
                    const std::int32_t* h = b->hist + static_cast<std::size_t>(r) * b->hist_stride;
                    seen.clear();
                    for (std::uint32_t i = 0; i < b->hist_len[r]; ++i) {
                        const std::uint32_t tk = static_cast<std::uint32_t>(h[i]);
                        if (tk >= V) continue;
                        if (cnt[tk]++ == 0) seen.push_back(tk);
                    }
                    for (const std::uint32_t tk : seen) {
                        float l = lg[tk];
                        l = (l > 0.f) ? l / rp : l * rp;
                        volatile float fc = fr * static_cast<float>(cnt[tk]);
                        volatile float sub = pr + fc;
                        lg[tk] = l - sub;
                        cnt[tk] = 0;
                    }
                }
                sampling::Sampler s;
                s.cands = sb.cands();
                s.inv_t = b->inv_t ? b->inv_t[r] : 1.f;
                s.temp = 1.0 / s.inv_t;
                s.top_k = b->top_k ? b->top_k[r] : 0;
                s.top_p = b->top_p ? b->top_p[r] : 1.0;
                s.min_p = b->min_p ? b->min_p[r] : 0.0;
                s.seed = b->seed ? b->seed[r] : 0;
                s.pos_idx = (b->pos_idx ? b->pos_idx[r] : 0) + static_cast<std::uint64_t>(rep) * rows;
                s.race = b->race && b->race[r];
                s.row_base = 0;
                sb.launchTopk(0, 1, server::k_small, s.inv_t, sb.sampDev(), server::max_rows, 0);
                hb.download(sb.sampHost().data(), sb.sampDev(), server::SampleBuffers::sampBytes());
                sb.prepareRow(s, 0);
                const std::uint32_t tok = sampling::sampleRow(sb, s, std::nullopt, 0);
                if (rep == 0 && tokens) tokens[r] = tok;
            }
        }
        t_end[t] = clk::now();
    };
    std::vector<std::thread> th;
    for (int t = 0; t < threads; ++t) th.emplace_back(worker, t);
    while (ready.load() < threads) std::this_thread::yield();
    t_start = clk::now();
    go.store(true, std::memory_order_release);
    for (auto& t : th) t.join();
    clk::time_point last = t_end[0];
    for (int t = 1; t < threads; ++t) last = std::max(last, t_end[t]);
    *seconds = std::chrono::duration<double>(last - t_start).count();
    return 0;
}

// small vocabularies: the reference test's hostPrepare (escalation 4 -> 16 -> V) + sampleRow
int ref_sample_rows_small(const float* x, std::uint32_t rows, std::uint32_t V, const Batch* b, RowOut* out,
                          std::uint32_t* kept_ids, double* kept_p, std::uint32_t kept_cap) {
    if (b->u || b->hist || V < server::acase::kb) return -1;
    std::vector<std::vector<float>> hr(rows, std::vector<float>(V));
    for (std::uint32_t r = 0; r < rows; ++r) std::memcpy(hr[r].data(), x + static_cast<std::size_t>(r) * V, V * 4);
    SmallRows src;
    src.rows = &hr;
    src.marks.assign(V, 0);
    src.V = V;
    std::vector<sampling::Cand> cands(std::max(V, server::acase::kb));
    for (std::uint32_t r = 0; r < rows; ++r) {
        RowOut& o = out[r];
        if (b->greedy && b->greedy[r]) {
            o = RowOut{static_cast<std::uint32_t>(firstMax(hr[r].data(), V)), 1, 1, 0, 0, 0, 0};
            o.m = hr[r][o.token];
            if (kept_ids && kept_cap) kept_ids[static_cast<std::size_t>(r) * kept_cap] = o.token;
            if (kept_p && kept_cap) kept_p[static_cast<std::size_t>(r) * kept_cap] = 1.0;
            continue;
        }
        sampling::Sampler s;
        s.cands = &cands;
        s.inv_t = b->inv_t ? b->inv_t[r] : 1.f;
        s.top_k = b->top_k ? b->top_k[r] : 0;
        s.top_p = b->top_p ? b->top_p[r] : 1.0;
        s.min_p = b->min_p ? b->min_p[r] : 0.0;
        s.seed = b->seed ? b->seed[r] : 0;
        s.pos_idx = b->pos_idx ? b->pos_idx[r] : 0;
        s.race = b->race && b->race[r];
        s.row_base = 0;
        const std::uint64_t pos = s.pos_idx;
        src.prepareRow(s, r);
        s.pos_idx = pos;
        const std::uint32_t nk = std::min<std::uint32_t>(static_cast<std::uint32_t>(s.n), kept_cap);
        for (std::uint32_t i = 0; i < nk; ++i) {
            if (kept_ids) kept_ids[static_cast<std::size_t>(r) * kept_cap + i] = cands[i].id;
            if (kept_p) kept_p[static_cast<std::size_t>(r) * kept_cap + i] = cands[i].p;
        }
        o.n = static_cast<std::uint32_t>(s.n);
        o.closed = s.closed;
        o.m = s.m;
        o.sum = s.sum;
        o.token = sampling::sampleRow(src, s, std::nullopt, 0);
        o.big_used = s.big_used;
        o.full_used = s.full_used;
    }
    return 0;
}

// the residual helper sampleRow(src, s, ex, p_ex) on a row prepared as above (small vocabularies)
std::uint32_t ref_sample_row_excluding(const float* x, std::uint32_t V, Sm* sm, std::uint32_t ex, double p_ex) {
    std::vector<std::vector<float>> hr(1, std::vector<float>(x, x + V));
    SmallRows src;
    src.rows = &hr;
    src.marks.assign(V, 0);
    src.V = V;
    std::vector<sampling::Cand> cands(std::max(V, server::acase::kb));
    sampling::Sampler s = toSampler(*sm, &cands);
    const std::uint64_t pos = s.pos_idx;
    s.row_base = 0;
    src.prepareRow(s, 0);
    s.pos_idx = pos;
    const std::uint32_t t = sampling::sampleRow(src, s, ex, p_ex);
    fromSampler(s, *sm);
    return t;
}

double ref_prob_of(const float* x, std::uint32_t V, Sm* sm, std::uint32_t t) {
    std::vector<std::vector<float>> hr(1, std::vector<float>(x, x + V));
    SmallRows src;
    src.rows = &hr;
    src.marks.assign(V, 0);
    src.V = V;
    std::vector<sampling::Cand> cands(std::max(V, server::acase::kb));
    sampling::Sampler s = toSampler(*sm, &cands);
    s.row_base = 0;
    src.prepareRow(s, 0);
    fromSampler(s, *sm);
    return sampling::probOf(src, s, t);
}

void ref_draft_dist(const std::uint32_t* ids, const float* logits, std::uint32_t count, float m, float sum, float inv_t,
                    std::uint32_t top_k, float top_p, float min_p, QD* q) {
    const spec::QDist d = spec::draftDist(std::span<const std::uint32_t>(ids, count), std::span<const float>(logits, count), m,
                                          sum, inv_t, top_k, top_p, min_p);
    q->n = d.n;
    std::memcpy(q->id, d.id, sizeof d.id);
    std::memcpy(q->p, d.p, sizeof d.p);
}
std::uint32_t ref_spec_sample_race(const QD* q, std::uint64_t base) {
    spec::QDist d;
    d.n = q->n;
    std::memcpy(d.id, q->id, sizeof d.id);
    std::memcpy(d.p, q->p, sizeof d.p);
    return spec::sampleRace(d, base);
}
std::uint32_t ref_draft_cands(std::uint32_t top_k) { return spec::draftCands(top_k); }

int ref_relax_accept_greedy(const Relax* p, const std::int32_t* ids, const float* logits, std::uint32_t n, float m,
                            std::uint32_t draft) {
    return relax::acceptGreedy(toRelax(*p), std::span<const std::int32_t>(ids, n), std::span<const float>(logits, n), m, draft);
}
int ref_relax_extends_repeat(const std::uint32_t* hist, std::size_t hn, const std::uint32_t* tail, std::size_t tn, std::size_t ng,
                             std::size_t window) {
    return relax::extendsRepeat(std::span<const std::uint32_t>(hist, hn), std::span<const std::uint32_t>(tail, tn), ng, window);
}
int ref_relax_accept_typical(const Relax* p, double pd, double h) { return relax::acceptTypical(toRelax(*p), pd, h); }

void ref_accept_greedy(const std::int32_t* argmax, const std::uint32_t* dr, std::uint32_t nd, std::uint32_t row0, int rlx,
                       const Relax* rp, const std::uint8_t* relax_host, std::uint32_t max_rows, const std::uint32_t* hist,
                       std::size_t hist_n, std::uint32_t next, Accepted* out) {
    const relax::Params prm = toRelax(*rp);
    const sampling::Acceptor acceptor(prm);
    const sampling::Drafts d{std::span<const std::uint32_t>(dr, nd ? nd : 1), nd, row0};
    const sampling::RepeatGuard repeats = [&](std::uint32_t a) {
        std::array<std::uint32_t, qwen35::max_ng_drafts + 2> tail{};
        tail[0] = next;
        for (std::uint32_t r = 0; r <= a; ++r) tail[r + 1] = dr[r];
        return relax::extendsRepeat(std::span<const std::uint32_t>(hist, hist_n), std::span<const std::uint32_t>(tail.data(), a + 2));
    };
    std::uint32_t relaxed = 0;
    double gap = 0;
    const sampling::Accepted a =
        acceptor.greedy(argmax, d, rlx != 0, sampling::RelaxRows{relax_host, max_rows, prm.topk()}, repeats, relaxed, gap);
    *out = Accepted{a.acc, a.chosen, relaxed, gap, 0, 0, 0};
}

// Acceptor::sample over host verify rows with the reference test's hostPrepare (4 / 16 escalation)
void ref_accept_sample(const float* rows, std::uint32_t V, Sm* sm, const std::uint32_t* dr, std::uint32_t nd, std::uint32_t row0,
                       int typ, std::uint32_t n_gen, const Relax* rp, const std::uint32_t* hist, std::size_t hist_n,
                       std::uint32_t next, std::uint32_t n_rows, Accepted* out) {
    std::vector<std::vector<float>> hr(n_rows, std::vector<float>(V));
    for (std::uint32_t r = 0; r < n_rows; ++r) std::memcpy(hr[r].data(), rows + static_cast<std::size_t>(r) * V, V * 4);
    SmallRows src;
    src.rows = &hr;
    src.marks.assign(V, 0);
    src.V = V;
    std::vector<sampling::Cand> cands(std::max(V, server::acase::kb));
    sampling::Sampler s = toSampler(*sm, &cands);
    const relax::Params prm = toRelax(*rp);
    const sampling::Acceptor acceptor(prm);
    const sampling::Drafts d{std::span<const std::uint32_t>(dr, nd ? nd : 1), nd, row0};
    const sampling::RepeatGuard repeats = [&](std::uint32_t a) {
        std::array<std::uint32_t, qwen35::max_ng_drafts + 2> tail{};
        tail[0] = next;
        for (std::uint32_t r = 0; r <= a; ++r) tail[r + 1] = dr[r];
        return relax::extendsRepeat(std::span<const std::uint32_t>(hist, hist_n), std::span<const std::uint32_t>(tail.data(), a + 2));
    };
    std::uint32_t relaxed = 0;
    const sampling::Accepted a = acceptor.sample(src, s, d, typ != 0, n_gen, repeats, relaxed);
    fromSampler(s, *sm);
    *out = Accepted{a.acc, a.chosen, relaxed, 0, s.pos_idx, s.full_used, s.big_used};
}

// The reference's 33 fixed acceptance cases (tests/server/sampling_cases.h:234-272) run on the reference code:
// per case acc, chosen, relaxed, gap bits, pos_idx, full_used, big_used; and the case inputs for the oracle.
std::uint32_t ref_case_count() { return static_cast<std::uint32_t>(server::acase::cases().size()); }
const char* ref_case_name(std::uint32_t i) { return server::acase::cases()[i].name; }

struct CaseInfo {
    std::int32_t greedy, relax, race;
    double temp;
    std::uint32_t top_k;
    double top_p, min_p;
    std::uint64_t seed;
    std::uint32_t n_gen, nd, row0, V, n_rows, next, hist_n;
};
// fills info, the verify rows [n_rows][V], the resolved drafts [15], the argmax words [16], the relax host block, hist [16]
void ref_case_inputs(std::uint32_t i, CaseInfo* info, float* rows, std::uint32_t* dr, std::int32_t* argmax,
                     std::uint8_t* relax_host, std::uint32_t relax_cap, std::uint32_t* hist) {
    using namespace server;
    const acase::Case& c = acase::cases()[i];
    // resolve 't' drafts the way acase::runResolved does, on the current reference code
    acase::Inputs in = acase::makeInputs(c);
    auto core = [&](const acase::Case& cc, acase::Inputs& ii) {
        SmallRows src;
        src.rows = &ii.rows;
        src.marks.assign(cc.V, 0);
        src.V = cc.V;
        std::vector<sampling::Cand> cands(std::max(cc.V, acase::kb));
        sampling::Sampler sm;
        sm.temp = cc.temp;
        sm.inv_t = cc.temp > 0 ? static_cast<float>(1.0 / cc.temp) : 1.0f;
        sm.top_k = cc.top_k;
        sm.top_p = cc.top_p;
        sm.min_p = cc.min_p;
        sm.seed = cc.seed;
        sm.race = cc.race;
        sm.cands = &cands;
        std::uint32_t relaxed = 0;
        double gap = 0;
        const sampling::Acceptor acceptor(ii.rp);
        const sampling::Drafts d{std::span<const std::uint32_t>(ii.dr.data(), ii.dr.size()), cc.nd, cc.row0};
        const sampling::RepeatGuard repeats = [&](std::uint32_t a) {
            std::array<std::uint32_t, qwen35::max_ng_drafts + 2> tail{};
            tail[0] = ii.next;
            for (std::uint32_t r = 0; r <= a; ++r) tail[r + 1] = ii.dr[r];
            return relax::extendsRepeat(std::span<const std::uint32_t>(ii.hist), std::span<const std::uint32_t>(tail.data(), a + 2));
        };
        return cc.greedy ? acceptor.greedy(ii.ctl.data() + qwen35::ctl_rows, d, cc.relax,
                                           sampling::RelaxRows{ii.relax_host.data(), acase::max_rows_t, ii.rp.topk()}, repeats,
                                           relaxed, gap)
                         : acceptor.sample(src, sm, d, cc.relax, cc.n_gen, repeats, relaxed);
    };
    for (std::uint32_t r = 0; r < c.nd; ++r) {
        if (c.drafts[r] != 't') continue;
        acase::Case t = c;
        t.nd = r;
        in.dr[r] = core(t, in).chosen;
    }
    *info = CaseInfo{c.greedy, c.relax, c.race, c.temp, c.top_k, c.top_p, c.min_p, c.seed, c.n_gen, c.nd, c.row0, c.V,
                     static_cast<std::uint32_t>(in.rows.size()), in.next, static_cast<std::uint32_t>(in.hist.size())};
    for (std::size_t r = 0; r < in.rows.size(); ++r) std::memcpy(rows + r * c.V, in.rows[r].data(), c.V * 4);
    for (std::uint32_t r = 0; r < 15; ++r) dr[r] = in.dr[r];
    for (std::uint32_t r = 0; r < 16; ++r) argmax[r] = in.ctl[r];
    std::memcpy(relax_host, in.relax_host.data(), std::min<std::size_t>(relax_cap, in.relax_host.size()));
    for (std::size_t r = 0; r < in.hist.size() && r < 16; ++r) hist[r] = in.hist[r];
}
std::uint32_t ref_case_relax_bytes(std::uint32_t i) {
    return static_cast<std::uint32_t>(server::acase::makeInputs(server::acase::cases()[i]).relax_host.size());
}
std::uint32_t ref_case_max_rows() { return server::acase::max_rows_t; }

}  // extern "C"
