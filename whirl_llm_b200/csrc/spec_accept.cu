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
