// Speculative acceptance on the device.
//
// (1) accept_tokens: the reference's current rule (include/whirl/spec_sample.h:8-24, src/sampling/acceptor.cpp:63-100 without
//     the relaxed branch): the target token of every verify row is a function of (target logits, seed, index) alone - drawn by
//     whirl_sample_rows, inverse CDF or race - and a draft is kept iff it equals that token.  This kernel is the accept loop.
// (2) spec_accept_residual: the Leviathan / Chen rule the reference removed (include/whirl/spec_sample.h:21-24) and BASELINE
//     config 3 names: accept draft d with probability min(1, p(d) / q(d)), on the first rejection draw from
//     max(0, p - q) / sum, after L acceptances the bonus token from p.  No counterpart in the reference today; the
//     exact statement of the rule is in include/whirl_b200.h (whirl_spec_accept_residual).
#include "kernels.h"
#include "common.cuh"

namespace wb {

// ---------------------------------------------------------------- (1)
// tokens[rows]: the sampler's token of every verify row.  Sequence s has nd[s] drafts dr[s][0..nd) checked against rows
// row0[s] + 0 .. row0[s] + nd[s]; acc[s] = drafts kept, chosen[s] = the token after them.
__global__ void accept_tokens_kernel(const int32_t* tokens, const int32_t* dr, int dr_stride, const int32_t* nd, const int32_t* row0,
                                     int seqs, int32_t* acc, int32_t* chosen) {
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= seqs) return;
    const int n = nd[s], r0 = row0[s];
    int a = 0;
    while (a < n && tokens[r0 + a] == dr[size_t(s) * dr_stride + a]) ++a;
    acc[s] = a;
    chosen[s] = tokens[r0 + a];
}

// ---------------------------------------------------------------- (1b)
// The accept loops of sampling::Acceptor with the relaxed rules (src/sampling/acceptor.cpp:30-100,
// include/whirl/relax_accept.h:44-96): one warp per sequence walks the drafts in order; the rules' inner loops (the
// search and rank over a row's best logits, the kept set's entropy, the 6-gram search over the last 4096 tokens) run
// across the lanes.

// relax::extendsRepeat over hist[0..hist_n) followed by tail = (next, drafts[0..n_dr)): true when the last 6 tokens of
// that sequence occur earlier in its last (min(hist_n, 4096) + tail) tokens.
__device__ bool extends_repeat(const int32_t* hist, uint32_t hist_n, int32_t next, const int32_t* drafts, uint32_t n_dr) {
    constexpr uint32_t NG = 6, WINDOW = 4096;
    const int lane = lane_id();
    const uint32_t hn = hist_n < WINDOW ? hist_n : WINDOW;
    const uint32_t tail_n = n_dr + 1, s = hn + tail_n;
    if (s < NG + 1) return false;
    const int32_t* h = hist + (hist_n - hn);
    auto at = [&](uint32_t i) -> int32_t { return i < hn ? h[i] : (i == hn ? next : drafts[i - hn - 1]); };
    int32_t last[NG];
#pragma unroll
    for (uint32_t j = 0; j < NG; ++j) last[j] = at(s - NG + j);
    bool hit = false;
#pragma unroll 1
    for (uint32_t base = 0; base + NG < s && !hit; base += 32) {
        const uint32_t i = base + uint32_t(lane);
        bool m = i + NG < s;
#pragma unroll
        for (uint32_t j = 0; j < NG; ++j) m = m && at(i + j) == last[j];
        hit = __any_sync(0xffffffffu, m);
    }
    return hit;
}

__global__ void __launch_bounds__(128) accept_rows_kernel(whirl_accept_in in, whirl_relax_params rp, int seqs, int32_t* acc_out,
                                                          int32_t* chosen, int32_t* relaxed_out, double* gap_out, int32_t* flags_out) {
    constexpr uint32_t FULL = 0xffffffffu;
    const int s = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (s >= seqs) return;
    const int lane = lane_id();
    const uint32_t nd = uint32_t(in.nd[s]);
    const int r0 = in.row0[s];
    const int32_t* dr = in.drafts + size_t(s) * in.draft_stride;
    const bool greedy = in.greedy && in.greedy[s];
    const bool relax = in.relax_on && in.relax_on[s];
    const uint32_t topk = rp.k < 1 ? 1u : (rp.k > 16 ? 16u : rp.k);  // relax::Params::topk
    const int32_t* hist = in.hist ? in.hist + size_t(s) * in.hist_stride : nullptr;
    const uint32_t hist_n = in.hist && in.hist_len ? uint32_t(max(in.hist_len[s], 0)) : 0u;
    const int32_t next = in.next ? in.next[s] : 0;
    uint32_t acc = 0, n_relaxed = 0;
    int flags = 0;
    double gap = 0.0;
#pragma unroll 1
    while (acc < nd) {
        const int row = r0 + int(acc);
        const int32_t d = dr[acc];
        const bool exact = in.tokens[row] == d;
        if (greedy) {
            if (exact) {
                ++acc;
                continue;
            }
            if (!relax || !in.rk_ids) break;
            // relax::acceptGreedy on the row's rk best logits, one per lane
            const bool have = lane < in.rk;
            const int32_t id = have ? in.rk_ids[size_t(row) * in.rk + lane] : -1;
            const float lg = have ? in.rk_vals[size_t(row) * in.rk + lane] : 0.f;
            const uint32_t found = __ballot_sync(FULL, have && id == d);
            if (!found) break;
            const int at = __ffs(int(found)) - 1;
            const float ld = __shfl_sync(FULL, lg, at);
            const uint32_t ahead = __ballot_sync(FULL, have && lane != at && (lg > ld || (lg == ld && uint32_t(id) < uint32_t(d))));
            const float m = in.rk_stats[2 * size_t(row)];
            if (uint32_t(__popc(ahead)) >= topk || !(exp(double(ld) - double(m)) >= double(rp.alpha))) break;
            if (extends_repeat(hist, hist_n, next, dr, acc + 1)) break;
            // (every entry equal to the draft counts, as in the reference's loop: ids of a top-k are distinct)
            gap += double(__popc(found)) * double(__fsub_rn(m, ld));
            ++acc, ++n_relaxed;
            continue;
        }
        if (relax && in.kept_ids) {
            // typical acceptance on the row's kept set: p(draft) (the reference's probOf) and the entropy
            const uint32_t nk = uint32_t(in.n_kept[row]);
            if (nk > uint32_t(in.kept_cap)) {
                flags |= WHIRL_ACCEPT_TRUNCATED;
            } else {
                const int32_t* kid = in.kept_ids + size_t(row) * in.kept_cap;
                const double* kp = in.kept_p + size_t(row) * in.kept_cap;
                double h = 0.0, pd = -1.0;
                uint32_t first = 0xffffffffu;  // the first entry that is the draft
#pragma unroll 1
                for (uint32_t i = lane; i < nk; i += 32) {
                    const double p = kp[i];
                    if (p > 0) h -= p * log(p);
                    if (kid[i] == d && i < first) first = i, pd = p;
                }
                h = warp_sum(h);
                const uint32_t fmin_i = __reduce_min_sync(FULL, first);
                const uint32_t owner = __ballot_sync(FULL, first == fmin_i);  // (all lanes when no entry is the draft)
                pd = __shfl_sync(FULL, pd, __ffs(int(owner)) - 1);
                if (fmin_i == 0xffffffffu) {
                    pd = 0.0;
                    if (!in.closed[row] && in.x && d >= 0 && d < in.n) {
                        const float xv = in.dtype == WHIRL_F32 ? reinterpret_cast<const float*>(in.x)[size_t(row) * in.n + d]
                                                               : bf16_to_f32(reinterpret_cast<const uint16_t*>(in.x)[size_t(row) * in.n + d]);
                        const float it = in.inv_t ? in.inv_t[row] : 1.f;
                        pd = exp(double(__fsub_rn(xv, in.stats[2 * size_t(row)])) * double(it)) / double(in.stats[2 * size_t(row) + 1]);
                    }
                }
                const double thr = fmin(double(rp.eps), double(rp.delta) * exp(-h));
                if (pd >= thr && !extends_repeat(hist, hist_n, next, dr, acc + 1)) {
                    ++acc, ++n_relaxed;
                    continue;
                }
            }
        }
        if (!exact) break;
        ++acc;
    }
    if (lane == 0) {
        acc_out[s] = int32_t(acc);
        chosen[s] = in.tokens[r0 + int(acc)];
        if (relaxed_out) relaxed_out[s] += int32_t(n_relaxed);
        if (gap_out) gap_out[s] += gap;
        if (flags_out) flags_out[s] = flags;
    }
}

// ---------------------------------------------------------------- (2)
constexpr int RT = 1024;

template <typename T>
__device__ __forceinline__ float ld(const T* row, uint32_t i) {
    if (sizeof(T) == 4) return reinterpret_cast<const float*>(row)[i];
    return bf16_to_f32(reinterpret_cast<const uint16_t*>(row)[i]);
}

struct RowStat {
    float m;
    float pad;
    double z;  // sum exp((double)(x - m) * inv_t), blocked order
};

// one CTA per row of `x` ([rows][n]); inv_t per sequence, rows_per_seq rows per sequence
template <typename T>
__global__ void __launch_bounds__(RT) row_stats_kernel(const T* x, int n, int rows_per_seq, const float* inv_t, RowStat* out) {
    __shared__ float sm[32];
    __shared__ double sz[32];
    const int row = blockIdx.x;
    const T* xr = x + size_t(row) * n;
    const double it = double(inv_t ? inv_t[row / rows_per_seq] : 1.f);
    float m = -INFINITY;
    for (uint32_t i = threadIdx.x; i < uint32_t(n); i += RT) m = fmaxf(m, ld(xr, i));
    m = warp_max(m);
    if (lane_id() == 0) sm[threadIdx.x >> 5] = m;
    __syncthreads();
    m = sm[0];
    for (int w = 1; w < RT / 32; ++w) m = fmaxf(m, sm[w]);
    double z = 0;
    for (uint32_t i = threadIdx.x; i < uint32_t(n); i += RT) {
        const float v = ld(xr, i);
        if (v == v) z += exp(double(__fsub_rn(v, m)) * it);
    }
    z = warp_sum(z);
    if (lane_id() == 0) sz[threadIdx.x >> 5] = z;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0;
        for (int w = 0; w < RT / 32; ++w) t += sz[w];
        out[row].m = m, out[row].z = t;
    }
}

struct RShared {
    double wsum[32];
    double total, targ;
    int j_rej, pick, last;
    unsigned long long best;
};

// one CTA per sequence
template <typename T>
__global__ void __launch_bounds__(RT) accept_residual_kernel(const T* target, const T* draft, int n, int L, const int32_t* draft_tok,
                                                             const float* inv_t, const double* u_acc, const double* u_res,
                                                             const RowStat* st_t, const RowStat* st_d, int32_t* n_acc, int32_t* next_tok) {
    __shared__ RShared sh;
    const int s = blockIdx.x, tid = threadIdx.x;
    const double it = double(inv_t ? inv_t[s] : 1.f);
    const T* trow = target + size_t(s) * (L + 1) * n;
    const T* drow = draft + size_t(s) * L * n;
    if (tid == 0) {
        int j = 0;
        for (; j < L; ++j) {
            const uint32_t tok = uint32_t(draft_tok[size_t(s) * L + j]);
            const RowStat a = st_t[size_t(s) * (L + 1) + j], b = st_d[size_t(s) * L + j];
            const double p = exp(double(__fsub_rn(ld(trow + size_t(j) * n, tok), a.m)) * it) / a.z;
            const double q = exp(double(__fsub_rn(ld(drow + size_t(j) * n, tok), b.m)) * it) / b.z;
            if (!(u_acc[size_t(s) * L + j] * q < p || q == 0)) break;
        }
        sh.j_rej = j;
        sh.pick = -1, sh.last = -1, sh.best = 0ull;
    }
    __syncthreads();
    const int j = sh.j_rej;
    const bool bonus = j == L;
    const T* t = trow + size_t(j) * n;
    const T* d = bonus ? nullptr : drow + size_t(j) * n;
    const RowStat a = st_t[size_t(s) * (L + 1) + j];
    const RowStat b = bonus ? RowStat{0.f, 0.f, 1.0} : st_d[size_t(s) * L + j];
    auto weight = [&](uint32_t v) -> double {
        const float tv = ld(t, v);
        const double p = tv == tv ? exp(double(__fsub_rn(tv, a.m)) * it) / a.z : 0.0;
        if (bonus) return p;
        const float dv = ld(d, v);
        const double q = dv == dv ? exp(double(__fsub_rn(dv, b.m)) * it) / b.z : 0.0;
        const double r = p - q;
        return r > 0 ? r : 0.0;
    };
    // thread-contiguous blocks of ids, so that the running sum walks the vocabulary in id order
    const uint32_t S = (uint32_t(n) + RT - 1) / RT, b0 = min(uint32_t(n), tid * S), b1 = min(uint32_t(n), b0 + S);
    double loc = 0;
    int my_last = -1;
    for (uint32_t v = b0; v < b1; ++v) {
        const double w = weight(v);
        if (w > 0) loc += w, my_last = int(v);
    }
    // block exclusive scan of loc in thread order
    double incl = loc;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const double up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane_id() >= o) incl += up;
    }
    if (lane_id() == 31) sh.wsum[tid >> 5] = incl;
    atomicMax(&sh.last, my_last);
    __syncthreads();
    double before = 0;
    for (int w = 0; w < (tid >> 5); ++w) before += sh.wsum[w];
    const double excl = before + incl - loc;
    if (tid == RT - 1) {
        sh.total = excl + loc;
        // the residual draw targets u * sum(r); the bonus draw walks p until it passes u
        sh.targ = bonus ? u_res[size_t(s) * (L + 1) + L] : u_res[size_t(s) * (L + 1) + j] * (excl + loc);
    }
    __syncthreads();
    const double targ = sh.targ;
    if (excl <= targ && excl + loc > targ) {
        // the draw falls inside this thread's block: walk it again
        double cum = excl;
        for (uint32_t v = b0; v < b1; ++v) {
            const double w = weight(v);
            if (!(w > 0)) continue;
            cum += w;
            if (cum > targ) {
                sh.pick = int(v);  // at most one thread's block holds the target
                break;
            }
        }
    }
    // the first maximum of the target row, for a residual of zero mass
    if (!bonus) {
        unsigned long long best = 0;
        for (uint32_t v = tid; v < uint32_t(n); v += RT) {
            const float tv = ld(t, v);
            if (tv == tv) {
                const unsigned long long c = make_cand(key_of(tv), v);
                best = c > best ? c : best;
            }
        }
        best = warp_max(uint64_t(best));
        if (lane_id() == 0) atomicMax(&sh.best, best);
    }
    __syncthreads();
    if (tid == 0) {
        int pick = sh.pick;
        if (pick < 0) pick = (!bonus && !(sh.total > 0)) ? int(cand_id(sh.best)) : (sh.last >= 0 ? sh.last : 0);
        n_acc[s] = j;
        next_tok[s] = pick;
    }
}

size_t spec_stats_bytes(int seqs, int L) { return size_t(seqs) * (2 * L + 1) * sizeof(RowStat); }

cudaError_t accept_rows_launch(const whirl_accept_in& in, const whirl_relax_params& rp, int seqs, int32_t* acc, int32_t* chosen,
                               int32_t* relaxed, double* gap, int32_t* flags, cudaStream_t st) {
    accept_rows_kernel<<<(seqs + 3) / 4, 128, 0, st>>>(in, rp, seqs, acc, chosen, relaxed, gap, flags);
    return cudaGetLastError();
}

cudaError_t accept_tokens_launch(const int32_t* tokens, const int32_t* dr, int dr_stride, const int32_t* nd, const int32_t* row0,
                                 int seqs, int32_t* acc, int32_t* chosen, cudaStream_t st) {
    accept_tokens_kernel<<<(seqs + 127) / 128, 128, 0, st>>>(tokens, dr, dr_stride, nd, row0, seqs, acc, chosen);
    return cudaGetLastError();
}

cudaError_t accept_residual_launch(const void* target, const void* draft, int dtype, int seqs, int L, int n, const int32_t* draft_tok,
                                   const float* inv_t, const double* u_acc, const double* u_res, void* stats_ws, int32_t* n_acc,
                                   int32_t* next_tok, cudaStream_t st) {
    RowStat* st_t = static_cast<RowStat*>(stats_ws);
    RowStat* st_d = st_t + size_t(seqs) * (L + 1);
    if (dtype == 0) {
        row_stats_kernel<float><<<seqs * (L + 1), RT, 0, st>>>(static_cast<const float*>(target), n, L + 1, inv_t, st_t);
        if (L > 0) row_stats_kernel<float><<<seqs * L, RT, 0, st>>>(static_cast<const float*>(draft), n, L, inv_t, st_d);
        accept_residual_kernel<float><<<seqs, RT, 0, st>>>(static_cast<const float*>(target), static_cast<const float*>(draft), n, L, draft_tok,
                                                          inv_t, u_acc, u_res, st_t, st_d, n_acc, next_tok);
    } else {
        row_stats_kernel<uint16_t><<<seqs * (L + 1), RT, 0, st>>>(static_cast<const uint16_t*>(target), n, L + 1, inv_t, st_t);
        if (L > 0) row_stats_kernel<uint16_t><<<seqs * L, RT, 0, st>>>(static_cast<const uint16_t*>(draft), n, L, inv_t, st_d);
        accept_residual_kernel<uint16_t><<<seqs, RT, 0, st>>>(static_cast<const uint16_t*>(target), static_cast<const uint16_t*>(draft), n, L,
                                                             draft_tok, inv_t, u_acc, u_res, st_t, st_d, n_acc, next_tok);
    }
    return cudaGetLastError();
}

}  // namespace wb
