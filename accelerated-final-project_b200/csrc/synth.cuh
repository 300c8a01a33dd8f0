// Device-side synthetic input generator: the same counter-based arithmetic as the CPU oracle's
// oracle_fill_uniform / oracle_fill_normal, so tests and the benchmark can create inputs in HBM.
#pragma once

#include "common.cuh"

namespace b200attn {

__device__ __forceinline__ uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

template <typename T>
__global__ void synth_fill_kernel(T *dst, long long n, uint64_t key, long long index0, int dist) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const uint64_t u = splitmix64(key + (uint64_t)(index0 + i));
        float v;
        if (dist == 0) {
            v = -1.0f + 2.0f * ((float)(u >> 40) * (1.0f / 16777216.0f));
        } else {
            const float u1 = ((float)(u >> 40) + 1.0f) * (1.0f / 16777216.0f);
            const float u2 = (float)((u >> 16) & 0xffffffu) * (1.0f / 16777216.0f);
            v = sqrtf(-2.0f * logf(u1)) * cosf(6.28318530717958647692f * u2);
        }
        dst[i] = OutCvt<T>::one(v);
    }
}

inline void launch_synth_fill(void *dst, long long n, unsigned long long seed, unsigned long long tensor_id,
                              long long index0, int dist, int dtype, int sm_count, cudaStream_t st) {
    const uint64_t key = ((uint64_t)seed << 40) + ((uint64_t)tensor_id << 36);
    long long blocks = (n + 255) / 256;
    const long long cap = (long long)sm_count * 16;
    if (blocks > cap) blocks = cap;
    if (dtype == 0) synth_fill_kernel<float><<<(unsigned)blocks, 256, 0, st>>>((float *)dst, n, key, index0, dist);
    else synth_fill_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, st>>>((__nv_bfloat16 *)dst, n, key, index0, dist);
}

}  // namespace b200attn
