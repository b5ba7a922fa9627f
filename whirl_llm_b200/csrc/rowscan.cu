// Greedy picks: one pass over each logits row with 128-bit loads.
//
// Replaces, for sm_100a, the reference's argmax / argmax_rows / argmax_rows_to / argmax_prob / draft_pick /
// draft_pick_rows (kernels/shared/misc_kv_argmax_kv_store.h:30-42, kernels/shared/sample_pick_set_tokens.h:15-105,
// kernels/shared/block_argmax.h, block_argmax_psum.h).  Same results: the FIRST index of the maximum (strict >, ties
// to the lower index), and for the probability variants 1 / sum exp(x - max) at temperature 1.  Differences in how:
// one pass instead of two (online max / sum), a row may be split over several CTAs when there are fewer rows than
// SMs (partials meet in a small workspace; the last CTA to arrive combines them), and per-row tables are device
// arrays instead of 32-entry by-value structs.
#include "../../include/whirl_b200.h"

#include <mutex>

#include "common.cuh"
#include "kernels.h"

namespace wb {

struct Part {  // one CTA's result for its slice of a row
    float v;   // max
    int idx;   // its first index
    float m;   // == v when the slice has a number, the softmax reference point
    float s;   // sum exp(x - m) over the slice
};

__device__ __forceinline__ void take(float x, int i, float& best, int& idx) {
    if (x > best) best = x, idx = i;
}

// Per-thread state over a slice [begin, end) of one row.  SUM also accumulates sum exp(x - m_t) against the thread's
// running max m_t (rescaled when m_t grows), so no second pass is needed.
template <typename T, bool SUM>
struct Scan {
    float best = -INFINITY;
    int idx = 0;
    float s = 0.f;
    __device__ __forceinline__ void one(float x, int i) {
        if (SUM) {
            if (x > best) {
                s = (best == -INFINITY) ? 0.f : s * ex2_approx((best - x) * kLog2e);
                best = x, idx = i;
            }
            if (x == x && best != -INFINITY) s += ex2_approx((x - best) * kLog2e);
        } else {
            take(x, i, best, idx);
        }
    }
    __device__ __forceinline__ void four(float a, float b, float c, float d, int i) {
        if (SUM) {
            const float vm = fmaxf(fmaxf(a, b), fmaxf(c, d));
            if (vm > best) {
                // the first of the four that reaches vm
                const int k = a == vm ? 0 : (b == vm ? 1 : (c == vm ? 2 : 3));
                s = (best == -INFINITY) ? 0.f : s * ex2_approx((best - vm) * kLog2e);
                best = vm, idx = i + k;
            }
            if (best != -INFINITY) {
                const float e0 = a == a ? ex2_approx((a - best) * kLog2e) : 0.f, e1 = b == b ? ex2_approx((b - best) * kLog2e) : 0.f;
                const float e2 = c == c ? ex2_approx((c - best) * kLog2e) : 0.f, e3 = d == d ? ex2_approx((d - best) * kLog2e) : 0.f;
                s += (e0 + e1) + (e2 + e3);
            }
        } else {
            take(a, i, best, idx), take(b, i + 1, best, idx), take(c, i + 2, best, idx), take(d, i + 3, best, idx);
        }
    }
};

template <typename T, bool SUM>
__device__ void scan_slice(const T* __restrict__ row, int begin, int end, Scan<T, SUM>& st) {
    constexpr int EPV = 16 / sizeof(T);  // elements per 128-bit load
    const int tid = threadIdx.x, nt = blockDim.x;
    // scalar head up to the first 16-byte boundary of the row's memory
    const uintptr_t a0 = reinterpret_cast<uintptr_t>(row + begin);
    int head = int(((16 - (a0 & 15)) & 15) / sizeof(T));
    if (head > end - begin) head = end - begin;
    for (int i = begin + tid; i < begin + head; i += nt) st.one(sizeof(T) == 4 ? ((const float*)row)[i] : bf16_to_f32(((const uint16_t*)row)[i]), i);
    const int vb = begin + head;
    const int nvec = (end - vb) / EPV;
    const uint4* v = reinterpret_cast<const uint4*>(row + vb);
    // each thread walks its vectors in increasing index order, so its own first maximum is kept by the strict compare
#pragma unroll 4
    for (int j = tid; j < nvec; j += nt) {
        const uint4 q = __ldg(v + j);
        const int i = vb + j * EPV;
        if (sizeof(T) == 4) {
            st.four(__uint_as_float(q.x), __uint_as_float(q.y), __uint_as_float(q.z), __uint_as_float(q.w), i);
        } else {
            st.four(__uint_as_float(q.x << 16), __uint_as_float(q.x & 0xffff0000u), __uint_as_float(q.y << 16), __uint_as_float(q.y & 0xffff0000u), i);
            st.four(__uint_as_float(q.z << 16), __uint_as_float(q.z & 0xffff0000u), __uint_as_float(q.w << 16), __uint_as_float(q.w & 0xffff0000u), i + 4);
        }
    }
    for (int i = vb + nvec * EPV + tid; i < end; i += nt) st.one(sizeof(T) == 4 ? ((const float*)row)[i] : bf16_to_f32(((const uint16_t*)row)[i]), i);
}

__device__ __forceinline__ void merge(Part& a, const Part& b, bool with_sum) {
    // (value desc, index asc); sums are brought to the larger reference point
    if (with_sum) {
        const float M = fmaxf(a.m, b.m);
        if (M == -INFINITY) a.s = 0.f;
        else a.s = (a.m == -INFINITY ? 0.f : a.s * ex2_approx((a.m - M) * kLog2e)) + (b.m == -INFINITY ? 0.f : b.s * ex2_approx((b.m - M) * kLog2e));
        a.m = M;
    }
    if (b.v > a.v || (b.v == a.v && b.idx < a.idx)) a.v = b.v, a.idx = b.idx;
}

template <bool SUM>
__device__ Part block_reduce(Part p, Part* sh) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Part q;
        q.v = __shfl_xor_sync(0xffffffffu, p.v, o);
        q.idx = __shfl_xor_sync(0xffffffffu, p.idx, o);
        q.m = __shfl_xor_sync(0xffffffffu, p.m, o);
        q.s = __shfl_xor_sync(0xffffffffu, p.s, o);
        merge(p, q, SUM);
    }
    const int w = threadIdx.x >> 5, nw = blockDim.x >> 5;
    if (lane_id() == 0) sh[w] = p;
    __syncthreads();
    if (w == 0) {
        p = lane_id() < nw ? sh[lane_id()] : Part{-INFINITY, 0x7fffffff, -INFINITY, 0.f};
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            Part q;
            q.v = __shfl_xor_sync(0xffffffffu, p.v, o);
            q.idx = __shfl_xor_sync(0xffffffffu, p.idx, o);
            q.m = __shfl_xor_sync(0xffffffffu, p.m, o);
            q.s = __shfl_xor_sync(0xffffffffu, p.s, o);
            merge(p, q, SUM);
        }
    }
    return p;  // valid in warp 0
}

// grid = (splits, rows).  ws: [rows] tickets (zero on entry, zero again on exit) then [rows][splits] Parts.
template <typename T, int MODE>
__global__ void __launch_bounds__(1024) rowscan_kernel(RowScanArgs a) {
    constexpr bool SUM = MODE != RS_ARGMAX;
    __shared__ Part sh[32];
    __shared__ int s_last;
    const int row = blockIdx.y, splits = gridDim.x, sp = blockIdx.x;
    int *tok = a.tok, *ctl = a.ctl;
    float* prob = a.prob;
    if (MODE == RS_DRAFT_PICK) {
        if (a.ctl_all) {
            // the 64-word control area of the row's sequence (include/whirl/model_types.h:55-61):
            // [16, 32) draft tokens, [32, 48) draft probabilities, 48 drafts kept, 49 chain stopped
            int* base = a.ctl_all + a.area[row];
            tok = base + 16, prob = reinterpret_cast<float*>(base + 32), ctl = base + 48;
        }
        // kernels/shared/sample_pick_set_tokens.h:62: a stopped chain skips the later drafts
        if (a.r > 0 && ctl[1] != 0) return;
    }
    const T* x = reinterpret_cast<const T*>(a.x) + size_t(row) * a.n;
    const int per = ((a.n + splits - 1) / splits + 7) & ~7;
    const int begin = min(a.n, sp * per), end = min(a.n, begin + per);
    Scan<T, SUM> st;
    scan_slice<T, SUM>(x, begin, end, st);
    Part p{st.best, st.best == -INFINITY ? 0x7fffffff : st.idx, st.best, st.s};
    p = block_reduce<SUM>(p, sh);
    if (splits > 1) {
        int* tickets = reinterpret_cast<int*>(a.ws);
        Part* parts = reinterpret_cast<Part*>(tickets + ((gridDim.y + 3) & ~3)) + size_t(row) * splits;
        if (threadIdx.x == 0) {
            parts[sp] = p;
            __threadfence();
            const int t = atomicAdd(&tickets[row], 1);
            s_last = t == splits - 1;
        }
        __syncthreads();
        if (!s_last) return;
        __threadfence();
        if (threadIdx.x < 32) {
            p = Part{-INFINITY, 0x7fffffff, -INFINITY, 0.f};
            for (int i = lane_id(); i < splits; i += 32) merge(p, parts[i], SUM);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                Part q;
                q.v = __shfl_xor_sync(0xffffffffu, p.v, o);
                q.idx = __shfl_xor_sync(0xffffffffu, p.idx, o);
                q.m = __shfl_xor_sync(0xffffffffu, p.m, o);
                q.s = __shfl_xor_sync(0xffffffffu, p.s, o);
                merge(p, q, SUM);
            }
            if (threadIdx.x == 0) tickets[row] = 0;  // ready for the next launch
        }
    }
    if (threadIdx.x != 0) return;
    const int top = p.idx == 0x7fffffff ? 0 : p.idx;  // no number in the row: index 0, as the reference's scan
    if (MODE == RS_ARGMAX) {
        a.out[a.dst ? a.dst[row] : row] = top;
        if (a.ids) a.ids[0] = top;           // argmax(): feeds the next decode step,
        if (a.pos) a.pos[0] += a.advance;    // misc_kv_argmax_kv_store.h:37-41
    } else if (MODE == RS_ARGMAX_PROB) {
        a.out[row] = top;
        a.prob[row] = 1.f / p.s;
    } else {
        const float pr = 1.f / p.s;
        int* c = ctl;
        tok[a.r] = a.map ? a.map[top] : top;
        prob[a.r] = pr;
        if (a.p_min > 0.f && a.r >= a.n_min && pr < a.p_min) {
            c[0] = a.r;
            c[1] = 1;
        } else {
            c[0] = a.r + 1;
            if (a.r == 0) c[1] = 0;
        }
    }
}

size_t rowscan_ws_bytes(int rows, int splits) {
    return size_t((rows + 3) & ~3) * sizeof(int) + size_t(rows) * splits * sizeof(Part);
}

int rowscan_splits(int rows, int n, int sm_count) {
    if (rows >= 2 * sm_count) return 1;
    int s = (2 * sm_count + rows - 1) / rows;
    const int max_s = n / 8192 > 1 ? n / 8192 : 1;  // at least 8192 elements per CTA
    if (s > max_s) s = max_s;
    if (s > 64) s = 64;
    return s < 1 ? 1 : s;
}

cudaError_t rowscan_launch(const RowScanArgs& a, int dtype, int mode, int rows, int splits, cudaStream_t st) {
    const dim3 grid(splits, rows), block(a.n >= 65536 ? 1024 : 256);
#define WB_RS(T, M) rowscan_kernel<T, M><<<grid, block, 0, st>>>(a)
    if (dtype == 0) {
        if (mode == RS_ARGMAX) WB_RS(float, RS_ARGMAX);
        else if (mode == RS_ARGMAX_PROB) WB_RS(float, RS_ARGMAX_PROB);
        else WB_RS(float, RS_DRAFT_PICK);
    } else {
        if (mode == RS_ARGMAX) WB_RS(uint16_t, RS_ARGMAX);
        else if (mode == RS_ARGMAX_PROB) WB_RS(uint16_t, RS_ARGMAX_PROB);
        else WB_RS(uint16_t, RS_DRAFT_PICK);
    }
#undef WB_RS
    return cudaGetLastError();
}

}  // namespace wb

// ---------------------------------------------------------------------------------------------------------------------
// whirl_argmax_rows_static: the greedy pick for callers that may not allocate device memory.
//
// Some hosts hand a sampler no allocator at all: an engine that sizes every device buffer once at start-up and forbids
// cudaMalloc afterwards (an allocation synchronises the device and can fail late), or a plugin that is called where no
// workspace pointer can be threaded through.  For them the split-row scratch of the greedy pick (one ticket per row and
// one partial result per row and split) lives in the file-scope device array below instead of a caller workspace.
// Every GPU that loads this library holds the array (about 257 KiB) until the process exits.
// ---------------------------------------------------------------------------------------------------------------------
namespace {

constexpr int kStaticSplits = 64;
constexpr size_t kStaticBytes = size_t((WHIRL_STATIC_MAX_ROWS + 3) & ~3) * sizeof(int) +
                                size_t(WHIRL_STATIC_MAX_ROWS) * kStaticSplits * sizeof(wb::Part);
static __device__ __align__(256) unsigned char g_static_scratch[kStaticBytes];

// In host code the array's name is only a handle: the address a kernel can use comes from cudaGetSymbolAddress, asked once
// per device with that device current.
std::mutex g_static_mu;
void* g_static_ptr[64] = {nullptr};

cudaError_t static_scratch(void** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lk(g_static_mu);
    if (!g_static_ptr[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess) return e;
        g_static_ptr[dev] = p;
    }
    *out = g_static_ptr[dev];
    return cudaSuccess;
}

}  // namespace

#pragma GCC visibility push(default)
extern "C" int whirl_argmax_rows_static(const void* x, int dtype, int rows, int n, int* out, void* stream) {
    if (!x || !out || rows < 0 || n <= 0 || (dtype != WHIRL_F32 && dtype != WHIRL_BF16)) {
        wb::set_last_error("argmax_rows_static: bad pointer / rows / n / dtype");
        return WHIRL_ERR_INVALID;
    }
    if (rows > WHIRL_STATIC_MAX_ROWS) {
        wb::set_last_error("argmax_rows_static: more than WHIRL_STATIC_MAX_ROWS rows; use whirl_argmax_rows with a workspace");
        return WHIRL_ERR_UNSUPPORTED;
    }
    if (rows == 0) return WHIRL_OK;
    void* scratch = nullptr;
    cudaError_t e = static_scratch(&scratch);  // the first call on a device looks the address up
    if (e != cudaSuccess) {
        wb::set_last_error(cudaGetErrorString(e));
        return WHIRL_ERR_CUDA;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int sms = 148;
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    int splits = wb::rowscan_splits(rows, n, sms);
    if (splits > kStaticSplits) splits = kStaticSplits;
    if (splits > 1) {
        // the tickets must start at zero; the array keeps whatever the last call left
        e = cudaMemsetAsync(scratch, 0, size_t((rows + 3) & ~3) * sizeof(int), st);
        if (e != cudaSuccess) {
            wb::set_last_error(cudaGetErrorString(e));
            return WHIRL_ERR_CUDA;
        }
    }
    wb::RowScanArgs a{};
    a.x = x, a.n = n, a.out = out, a.ws = scratch;
    e = wb::rowscan_launch(a, dtype, wb::RS_ARGMAX, rows, splits, st);
    wb::count_launch(0);
    if (e != cudaSuccess) {
        wb::set_last_error(cudaGetErrorString(e));
        return WHIRL_ERR_CUDA;
    }
    return WHIRL_OK;
}
#pragma GCC visibility pop
