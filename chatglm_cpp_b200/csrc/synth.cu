// Counter-based synthetic data for benchmarks and tests: element i of tensor t under seed s is
//     table[splitmix64(s * 0x9E3779B97F4A7C15 + t * 0xBF58476D1CE4E5B9 + i) >> 48]
// where table is a 65536-entry value table supplied by the caller (the N(0,1) quantiles in f32 or f16).  Integer
// arithmetic only, so a host implementation of the same three lines (oracle/attn_oracle.c: oracle_synth_fill_*)
// produces the same bits: a CPU arm and a GPU arm can work on identical caches without moving them across the bus.
// Not part of the attention path; exported for bench.py and the tests.
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/cglm_attn.h"

namespace {

__host__ __device__ inline uint64_t splitmix64(uint64_t z) {
    z ^= z >> 30; z *= 0xBF58476D1CE4E5B9ull;
    z ^= z >> 27; z *= 0x94D049BB133111EBull;
    z ^= z >> 31;
    return z;
}

template <typename T>
__global__ void synth_fill_kernel(T *__restrict__ dst, long long n, uint64_t base, long long first, const T *__restrict__ table) {
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n; i += stride) {
        dst[i] = __ldg(table + (splitmix64(base + static_cast<uint64_t>(first + i)) >> 48));
    }
}

template <typename T>
int synth_fill(T *dst, long long n, unsigned long long seed, unsigned long long tensor_id, long long first, const T *table,
               void *cuda_stream) {
    if (!dst || !table || n < 0 || first < 0) return CGLM_ERR_INVALID_ARG;
    if (n == 0) return CGLM_OK;
    const uint64_t base = seed * 0x9E3779B97F4A7C15ull + tensor_id * 0xBF58476D1CE4E5B9ull;
    const long long want = (n + 255) / 256;
    const int blocks = static_cast<int>(want < 148 * 16 ? want : 148 * 16);
    synth_fill_kernel<T><<<blocks, 256, 0, static_cast<cudaStream_t>(cuda_stream)>>>(dst, n, base, first, table);
    return cudaGetLastError() == cudaSuccess ? CGLM_OK : CGLM_ERR_CUDA;
}

}  // namespace

extern "C" {

int cglm_synth_fill_f16(void *dst, long long n, unsigned long long seed, unsigned long long tensor_id, long long first,
                        const void *table_f16, void *cuda_stream) {
    return synth_fill(static_cast<uint16_t *>(dst), n, seed, tensor_id, first, static_cast<const uint16_t *>(table_f16), cuda_stream);
}

int cglm_synth_fill_f32(float *dst, long long n, unsigned long long seed, unsigned long long tensor_id, long long first,
                        const float *table_f32, void *cuda_stream) {
    return synth_fill(dst, n, seed, tensor_id, first, table_f32, cuda_stream);
}

}  // extern "C"
