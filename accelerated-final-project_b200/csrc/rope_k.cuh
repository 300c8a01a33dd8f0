// "Rotate once and keep it": writes RoPE(X) for a [B,H,L,D] tensor, the producer a KV-cache caller runs
// when keys are appended, so that attention can then take K as already rotated (the *_Q_ONLY encodings).
// Replaces rope_kernel, final/rope.cu:1240-1280, as used by attention_forward_separate_rope
// (final/rope.cu:1379-1416) - without that kernel's position taken modulo 64 (:1257): the position
// of row l of every (b,h) slice is pos0 + l.
//
// Memory-bound element-wise work: a thread owns one 16-byte vector position of one row (two vectors for
// the rotate-half pairing: columns d and d + rotary_dim/2) and walks over the (b,h) slices with it, so the
// angle arithmetic - theta = (float)pos * (1 / powf(base, 2i / rotary_dim)), sincosf, exactly the fp32
// arithmetic of the reference tables (final/rope.cu:20-40) - is done once per (row, pair) and not once per
// element.  The products are fp32; a bf16 result is rounded once.
#pragma once

#include "common.cuh"

namespace b200attn {

struct RopeKParams {
    const void *X;
    void *Y;
    long long BH;
    int L, D, rd;
    int half;                 // 0: pairs (2i, 2i+1); 1: pairs (i, i + rd/2)
    int pos0;
    float base;
    const float *cos_cache, *sin_cache;   // optional [>= pos0 + L][rd], value of pair i at columns 2i and 2i+1
    int sinus;                // 1: additive sinusoidal encoding instead of a rotation - x[2i] += sin, x[2i+1] += cos of
                              // pos / 10000^(2i/D) (final/sinusoidal.cu:143-161); then rd = D, half = 0, base = 10000
};

template <typename T> struct RopeVec;
template <> struct RopeVec<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void load(const float *p, float (&x)[4]) {
        const float4 v = *reinterpret_cast<const float4 *>(p);
        x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
    }
    static __device__ __forceinline__ void store(float *p, const float (&x)[4]) {
        *reinterpret_cast<float4 *>(p) = make_float4(x[0], x[1], x[2], x[3]);
    }
};
template <> struct RopeVec<__half> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void load(const __half *p, float (&x)[8]) {
        const uint4 v = *reinterpret_cast<const uint4 *>(p);
        const __half *h = reinterpret_cast<const __half *>(&v);
#pragma unroll
        for (int e = 0; e < 8; ++e) x[e] = __half2float(h[e]);
    }
    static __device__ __forceinline__ void store(__half *p, const float (&x)[8]) {
        uint4 v;
        __half2 *h = reinterpret_cast<__half2 *>(&v);
#pragma unroll
        for (int e = 0; e < 4; ++e) h[e] = __floats2half2_rn(x[2 * e], x[2 * e + 1]);
        *reinterpret_cast<uint4 *>(p) = v;
    }
};
template <> struct RopeVec<__nv_bfloat16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void load(const __nv_bfloat16 *p, float (&x)[8]) {
        const uint4 v = *reinterpret_cast<const uint4 *>(p);
        const __nv_bfloat16 *h = reinterpret_cast<const __nv_bfloat16 *>(&v);
#pragma unroll
        for (int e = 0; e < 8; ++e) x[e] = __bfloat162float(h[e]);
    }
    static __device__ __forceinline__ void store(__nv_bfloat16 *p, const float (&x)[8]) {
        uint4 v;
        __nv_bfloat162 *h = reinterpret_cast<__nv_bfloat162 *>(&v);
#pragma unroll
        for (int e = 0; e < 4; ++e) h[e] = __floats2bfloat162_rn(x[2 * e], x[2 * e + 1]);
        *reinterpret_cast<uint4 *>(p) = v;
    }
};

__device__ __forceinline__ void rope_angle(const RopeKParams &p, int pos, int pair, float &c, float &s) {
    if (p.cos_cache != nullptr) {
        c = p.cos_cache[(long long)pos * p.rd + 2 * pair];
        s = p.sin_cache[(long long)pos * p.rd + 2 * pair];
    } else {
        const float freq = 1.0f / powf(p.base, (2.0f * (float)pair) / (float)p.rd);
        sincosf((float)pos * freq, &s, &c);
    }
}

// Vector path: D, rd (interleaved) or rd/2 (half) are multiples of the vector width and the pointers are
// 16-byte aligned.  Work items of a row: interleaved - D/N vectors; half - rd/(2N) vector pairs plus
// (D - rd)/N copy vectors.
template <typename T>
__global__ void __launch_bounds__(256) rope_k_vec_kernel(const RopeKParams p) {
    constexpr int N = RopeVec<T>::N;
    const T *X = reinterpret_cast<const T *>(p.X);
    T *Y = reinterpret_cast<T *>(p.Y);
    const int nrot = p.half ? p.rd / (2 * N) : p.rd / N;   // items that rotate
    const int nitem = nrot + (p.D - p.rd) / N;
    const long long total = (long long)p.L * nitem;
    const long long slab = (long long)p.L * p.D;
    for (long long w = (long long)blockIdx.x * blockDim.x + threadIdx.x; w < total; w += (long long)gridDim.x * blockDim.x) {
        const int l = (int)(w / nitem), it = (int)(w - (long long)l * nitem);
        const int pos = p.pos0 + l;
        const long long row = (long long)l * p.D;
        if (it >= nrot) {   // beyond rotary_dim: copy
            const long long off = row + p.rd + (long long)(it - nrot) * N;
            for (long long bh = 0; bh < p.BH; ++bh)
                *reinterpret_cast<uint4 *>(Y + bh * slab + off) = *reinterpret_cast<const uint4 *>(X + bh * slab + off);
        } else if (p.half) {
            const int d = it * N;   // columns d..d+N-1 pair with d + rd/2 ..
            float c[N], s[N];
#pragma unroll
            for (int e = 0; e < N; ++e) rope_angle(p, pos, d + e, c[e], s[e]);
            for (long long bh = 0; bh < p.BH; ++bh) {
                float lo[N], hi[N], ylo[N], yhi[N];
                RopeVec<T>::load(X + bh * slab + row + d, lo);
                RopeVec<T>::load(X + bh * slab + row + d + p.rd / 2, hi);
#pragma unroll
                for (int e = 0; e < N; ++e) { ylo[e] = lo[e] * c[e] - hi[e] * s[e]; yhi[e] = lo[e] * s[e] + hi[e] * c[e]; }
                RopeVec<T>::store(Y + bh * slab + row + d, ylo);
                RopeVec<T>::store(Y + bh * slab + row + d + p.rd / 2, yhi);
            }
        } else {
            const int d = it * N;   // pairs (d, d+1), (d+2, d+3), ...
            float c[N / 2], s[N / 2];
#pragma unroll
            for (int e = 0; e < N / 2; ++e) rope_angle(p, pos, d / 2 + e, c[e], s[e]);
            for (long long bh = 0; bh < p.BH; ++bh) {
                float x[N], y[N];
                RopeVec<T>::load(X + bh * slab + row + d, x);
#pragma unroll
                for (int e = 0; e < N / 2; ++e) {
                    if (p.sinus) { y[2 * e] = x[2 * e] + s[e]; y[2 * e + 1] = x[2 * e + 1] + c[e]; }
                    else { y[2 * e] = x[2 * e] * c[e] - x[2 * e + 1] * s[e]; y[2 * e + 1] = x[2 * e] * s[e] + x[2 * e + 1] * c[e]; }
                }
                RopeVec<T>::store(Y + bh * slab + row + d, y);
            }
        }
    }
}

// Any shape and alignment: a thread owns one pair (or one copied column) of one row.
template <typename T>
__global__ void __launch_bounds__(256) rope_k_scalar_kernel(const RopeKParams p) {
    const T *X = reinterpret_cast<const T *>(p.X);
    T *Y = reinterpret_cast<T *>(p.Y);
    const int npair = p.rd / 2, nitem = npair + (p.D - p.rd);
    const long long total = (long long)p.L * nitem;
    const long long slab = (long long)p.L * p.D;
    for (long long w = (long long)blockIdx.x * blockDim.x + threadIdx.x; w < total; w += (long long)gridDim.x * blockDim.x) {
        const int l = (int)(w / nitem), it = (int)(w - (long long)l * nitem);
        const long long row = (long long)l * p.D;
        if (it >= npair) {
            const long long off = row + p.rd + (it - npair);
            for (long long bh = 0; bh < p.BH; ++bh) Y[bh * slab + off] = X[bh * slab + off];
        } else {
            float c, s;
            rope_angle(p, p.pos0 + l, it, c, s);
            const int d0 = p.half ? it : 2 * it, d1 = p.half ? it + npair : 2 * it + 1;
            for (long long bh = 0; bh < p.BH; ++bh) {
                const float a = to_f32(X[bh * slab + row + d0]), b = to_f32(X[bh * slab + row + d1]);
                Y[bh * slab + row + d0] = OutCvt<T>::one(p.sinus ? a + s : a * c - b * s);
                Y[bh * slab + row + d1] = OutCvt<T>::one(p.sinus ? b + c : a * s + b * c);
            }
        }
    }
}

template <typename T>
inline cudaError_t launch_rope_k(const RopeKParams &p, int sm_count, cudaStream_t st) {
    constexpr int N = RopeVec<T>::N;
    const bool aligned = (((uintptr_t)p.X | (uintptr_t)p.Y) & 15) == 0;
    const bool vec = aligned && p.D % N == 0 && (p.half ? (p.rd % (2 * N) == 0) : (p.rd % N == 0));
    const long long items = (long long)p.L * (vec ? (p.half ? p.rd / (2 * N) : p.rd / N) + (p.D - p.rd) / N : p.rd / 2 + (p.D - p.rd));
    long long blocks = (items + 255) / 256;
    const long long cap = (long long)sm_count * 8;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    if (vec) rope_k_vec_kernel<T><<<(unsigned)blocks, 256, 0, st>>>(p);
    else rope_k_scalar_kernel<T><<<(unsigned)blocks, 256, 0, st>>>(p);
    return cudaGetLastError();
}

}  // namespace b200attn
