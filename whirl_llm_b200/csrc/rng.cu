// The draw generators of the sampling path, as host functions and as one device fill kernel, so that a caller can make
// the per-row uniforms and race keys where its seeds and positions live.
//
//   splitmix uniform   Sampler::uniform (src/sampling/sampler.h:46-52) = spec::uniform stream 0
//                      (src/common/spec_sample.cpp:13-21): the top 53 bits of the splitmix64 finaliser
//                      (include/whirl/spec_sample.h:53-57) of seed + (pos + 1) * golden-ratio constant.
//   race base          spec::raceBase (include/whirl/spec_sample.h:58-60).
//   Philox4x32-10      Salmon et al., SC'11.  The reference has no Philox: the (key, counter) convention is this
//                      library's own — key = seed (lo, hi), counter = (pos lo, pos hi, row, stream), uniform = top 53
//                      bits of out0:out1 — and it is checked against the published known-answer vectors.
#include "../../include/whirl_b200.h"

#include <cuda_runtime.h>

#include "kernels.h"

namespace {

__host__ __device__ inline uint64_t mix64(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
__host__ __device__ inline double top53(uint64_t z) { return double(z >> 11) * (1.0 / 9007199254740992.0); }

__host__ __device__ inline double uniform_splitmix(uint64_t seed, uint64_t pos, uint32_t stream) {
    if (stream != 0) seed ^= uint64_t(stream) * 0xD1B54A32D192ED03ull;
    return top53(mix64(seed + (pos + 1) * 0x9E3779B97F4A7C15ull));
}
__host__ __device__ inline uint64_t race_base(uint64_t seed, uint64_t pos) {
    return mix64((seed ^ 0xA0761D6478BD642Full) + (pos + 1) * 0x9E3779B97F4A7C15ull);
}

__host__ __device__ inline void philox4x32_10(const uint32_t c[4], const uint32_t k[2], uint32_t out[4]) {
    uint32_t c0 = c[0], c1 = c[1], c2 = c[2], c3 = c[3], k0 = k[0], k1 = k[1];
    for (int r = 0; r < 10; ++r) {
        const uint64_t p0 = uint64_t(0xD2511F53u) * c0, p1 = uint64_t(0xCD9E8D57u) * c2;
        const uint32_t n0 = uint32_t(p1 >> 32) ^ c1 ^ k0, n1 = uint32_t(p1);
        const uint32_t n2 = uint32_t(p0 >> 32) ^ c3 ^ k1, n3 = uint32_t(p0);
        c0 = n0, c1 = n1, c2 = n2, c3 = n3;
        k0 += 0x9E3779B9u, k1 += 0xBB67AE85u;
    }
    out[0] = c0, out[1] = c1, out[2] = c2, out[3] = c3;
}
__host__ __device__ inline double uniform_philox(uint64_t seed, uint64_t pos, uint32_t row, uint32_t stream) {
    const uint32_t ctr[4] = {uint32_t(pos), uint32_t(pos >> 32), row, stream};
    const uint32_t key[2] = {uint32_t(seed), uint32_t(seed >> 32)};
    uint32_t o[4];
    philox4x32_10(ctr, key, o);
    return top53((uint64_t(o[0]) << 32) | o[1]);
}

// one thread per row
__global__ void fill_draws_kernel(const uint64_t* seed, const uint64_t* pos, int rows, int generator, uint32_t stream_id,
                                  double* u, uint64_t* race_key) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= rows) return;
    const uint64_t s = seed[r], p = pos[r];
    if (u) u[r] = generator == WHIRL_GEN_PHILOX ? uniform_philox(s, p, uint32_t(r), stream_id) : uniform_splitmix(s, p, stream_id);
    if (race_key) race_key[r] = race_base(s, p);
}

}  // namespace

#pragma GCC visibility push(default)
extern "C" {

double whirl_uniform_splitmix(uint64_t seed, uint64_t pos_idx, uint32_t stream_id) { return uniform_splitmix(seed, pos_idx, stream_id); }
uint64_t whirl_race_base(uint64_t seed, uint64_t pos_idx) { return race_base(seed, pos_idx); }
void whirl_philox4x32_10(const uint32_t ctr[4], const uint32_t key[2], uint32_t out[4]) { philox4x32_10(ctr, key, out); }
double whirl_uniform_philox4x32(uint64_t seed, uint64_t pos_idx, uint32_t row, uint32_t stream_id) {
    return uniform_philox(seed, pos_idx, row, stream_id);
}

int whirl_fill_draws(const uint64_t* seed, const uint64_t* pos_idx, int rows, int generator, uint32_t stream_id, double* u,
                     uint64_t* race_key, void* stream) {
    if (!seed || !pos_idx || rows < 0 || (generator != WHIRL_GEN_SPLITMIX && generator != WHIRL_GEN_PHILOX) || (!u && !race_key)) {
        wb::set_last_error("fill_draws: bad pointer / rows / generator");
        return WHIRL_ERR_INVALID;
    }
    if (rows == 0) return WHIRL_OK;
    fill_draws_kernel<<<(rows + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(seed, pos_idx, rows, generator, stream_id, u, race_key);
    wb::count_launch(3);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        wb::set_last_error(cudaGetErrorString(e));
        return WHIRL_ERR_CUDA;
    }
    return WHIRL_OK;
}

}  // extern "C"
#pragma GCC visibility pop
