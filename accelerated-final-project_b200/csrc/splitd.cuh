// Split-head_d attention forward on CUDA cores: the path for the memory-bound regime
// (sequence 16-64, head_d 512-8192) and the general path for every shape the tensor-core kernel
// does not take.
//
// One query row of the reference kernel (final/attention.cu:84-191) is one CTA that re-streams all
// of K and V.  Here a head is cut along head_d instead: a CTA owns the column slice [v0, v0+w) of
// Q, K and V of one head, so every input byte is read from HBM exactly once.
//
//   phase 1  S_part[i][j] = sum_{d in slice} Q~[i][d] * K~[j][d]      (Q~,K~: Q,K with the
//            positional encoding applied while the slice is loaded into shared memory)
//            partial scores of the slices of a head are summed into an fp32 scratch matrix in
//            L2 with red.global.add;
//   barrier  per-head arrival counter (all slices of the head are co-resident: cooperative launch);
//   phase 2  every slice CTA reads the complete Lq x Lk scores, redoes the (cheap) softmax with
//            warp-shuffle max / sum, and computes O[:, slice] = P * V[:, slice] from the V slice
//            it staged in shared memory during phase 1.
//
// The fused kernel holds Lq, Lk <= 64.  Larger sequences run the same device functions as two
// launches (scores, then softmax+PV) tiled 64 x 64 over queries and keys.
#pragma once

#include "tc_common.cuh"

namespace b200attn {

constexpr int SD_THREADS = 256;   // 16 x 16 thread grid over a 64 x 64 score tile
constexpr int SD_TILE = 64;       // query / key tile edge
constexpr int SD_PT_PITCH = 68;   // floats per row of the transposed probability tile

struct SplitDParams {
    const void *Q, *K, *V;
    void *O;
    long long BH;            // number of (batch, head) slices in this launch
    int Lq, Lk, D;
    int ds;                  // slice width in columns (multiple of 8)
    int nsplit;              // number of slices = ceil(D / ds)
    int pe, rotary_dim;
    float rope_base, scale;
    const float *cos_cache, *sin_cache;   // optional [max(Lq,Lk), rotary_dim]
    float *S;                // scratch scores [BH][Lq][Lk], all zero on entry when nsplit > 1
    unsigned *counters;      // fused kernel: [2*BH] arrive / done counters, zero on entry and on exit
    unsigned *err;           // error word (KernelErr bits)
    unsigned *err_sys;       // optional mirror flag in mapped host memory (may be null)
    unsigned spin_limit;     // polls before a wait gives up
    unsigned wait_extra;     // 0; a test sets it to make the head barrier wait for arrivals that never come
    int use_tma;             // fp32, no PE, D % 4 == 0: stage slices with three tiled TMA loads (tensor maps)
    int dv;                  // two-pass PV kernel: width of an output column slice
};

// Virtual -> physical column.  In "virtual" column order RoPE partners are always adjacent
// (2t, 2t+1): identity for every kind except rotate-half, where virtual 2t is physical t and
// virtual 2t+1 is physical t + rotary_dim/2.  Q and K use the same order, so scores are unchanged.
__device__ __forceinline__ int phys_col(int v, int pe, int rd) {
    return (pe_pairs_halves(pe) && v < rd) ? ((v >> 1) + (v & 1) * (rd >> 1)) : v;
}

// Loads rows [0, rows) x virtual columns [v0, v0+w) of a [*, D] matrix into shared memory as fp32
// (row pitch `pitch` floats), applying the positional encoding on the way.  Rows [rows, rows_pad)
// and columns [w, 8*ceil(w/8)) are zero-filled.  apply_pe = 0 loads plain values (V, pre-rotated K).
template <typename T>
__device__ void load_slice(float *dst, int pitch, const T *src, int rows, int rows_pad, int pos0,
                           int D, int v0, int w, int pe, int rd, bool apply_pe,
                           const float *freq_s, const float *cos_cache, const float *sin_cache) {
    const int ngroups = (w + 7) >> 3;
    const bool half = pe_pairs_halves(pe);
    const bool rope = apply_pe && pe_is_rope(pe);
    const bool sinus = apply_pe && (pe == PE_SINUSOIDAL);
    constexpr int VEC = 16 / (int)sizeof(T);  // elements per 16-byte vector: 4 (fp32) or 8 (bf16)
    const bool base_aligned = ((reinterpret_cast<uintptr_t>(src) & 15) == 0);
    for (int idx = threadIdx.x; idx < rows_pad * ngroups; idx += blockDim.x) {
        const int row = idx / ngroups, g = idx - row * ngroups;
        const int v = v0 + 8 * g;
        const int n = min(8, v0 + w - v);
        float x[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) x[e] = 0.0f;
        if (row < rows) {
            const T *rp = src + (long long)row * D;
            if (half && v + 8 <= rd && n == 8 && base_aligned && (D % 4 == 0) && (rd % 8 == 0)) {
                // rotate-half: 4 consecutive columns at v/2 and their 4 partners at v/2 + rd/2
                const T *lo = rp + (v >> 1), *hi = lo + (rd >> 1);
                if constexpr (sizeof(T) == 4) {
                    float4 a = *reinterpret_cast<const float4 *>(lo), b = *reinterpret_cast<const float4 *>(hi);
                    x[0] = a.x; x[2] = a.y; x[4] = a.z; x[6] = a.w;
                    x[1] = b.x; x[3] = b.y; x[5] = b.z; x[7] = b.w;
                } else {
                    uint2 a = *reinterpret_cast<const uint2 *>(lo), b = *reinterpret_cast<const uint2 *>(hi);
                    const T *pa = reinterpret_cast<const T *>(&a);
                    const T *pb = reinterpret_cast<const T *>(&b);
#pragma unroll
                    for (int t = 0; t < 4; ++t) { x[2 * t] = to_f32(pa[t]); x[2 * t + 1] = to_f32(pb[t]); }
                }
            } else if ((!half || v >= rd) && n == 8 && base_aligned && (D % VEC == 0)) {
                if constexpr (sizeof(T) == 4) {
                    float4 a = *reinterpret_cast<const float4 *>(rp + v), b = *reinterpret_cast<const float4 *>(rp + v + 4);
                    x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
                    x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
                } else {
                    uint4 a = *reinterpret_cast<const uint4 *>(rp + v);
                    const T *pa = reinterpret_cast<const T *>(&a);
#pragma unroll
                    for (int t = 0; t < 8; ++t) x[t] = to_f32(pa[t]);
                }
            } else {
                for (int e = 0; e < n; ++e) x[e] = to_f32(rp[phys_col(v + e, pe, rd)]);
            }
            if (rope || sinus) {
                const int pos = pos0 + row;
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    const int vc = v + 2 * t;  // virtual column of the pair's first element
                    const bool in_rot = rope ? (vc + 1 < rd) : (vc < D);
                    if (in_rot && 2 * t < n) {
                        const int p = vc >> 1;
                        float c, s;
                        if (cos_cache != nullptr && rope) {
                            c = cos_cache[(long long)pos * rd + 2 * p];
                            s = sin_cache[(long long)pos * rd + 2 * p];
                        } else {
                            // same arithmetic as the reference CPU tables: theta = pos * freq in fp32
                            const float theta = (float)pos * freq_s[p - (v0 >> 1)];
                            sincosf(theta, &s, &c);
                        }
                        if (rope) {
                            const float xe = x[2 * t], xo = x[2 * t + 1];
                            x[2 * t] = xe * c - xo * s;
                            x[2 * t + 1] = xe * s + xo * c;
                        } else {
                            x[2 * t] += s;
                            if (2 * t + 1 < n) x[2 * t + 1] += c;
                        }
                    }
                }
            }
        }
        float4 *d4 = reinterpret_cast<float4 *>(dst + (long long)row * pitch + 8 * g);
        d4[0] = make_float4(x[0], x[1], x[2], x[3]);
        d4[1] = make_float4(x[4], x[5], x[6], x[7]);
    }
}

// freq_s[p - v0/2] = 1 / powf(base, 2p / rd) for the pairs of this slice (final/rope.cu:29,
// final/sinusoidal.cu:848; sinusoidal uses rd = D, base = 10000).
__device__ __forceinline__ void fill_freqs(float *freq_s, int v0, int w, float base, int rd) {
    const int p0 = v0 >> 1, np = (w + 1) >> 1;
    for (int i = threadIdx.x; i < np; i += blockDim.x)
        freq_s[i] = 1.0f / powf(base, (2.0f * (float)(p0 + i)) / (float)rd);
}

__device__ __forceinline__ void zero_rows(float *dst, int pitch, int row_begin, int row_end, int ncols) {
    const int n = (row_end - row_begin) * ncols;
    for (int i = threadIdx.x; i < n; i += blockDim.x) dst[(long long)(row_begin + i / ncols) * pitch + (i % ncols)] = 0.0f;
}

// Packed fp32 FMA (two lanes per instruction, sm_100): acc.xy += a.xy * b.xy
__device__ __forceinline__ void ffma2(float2 &acc, const float2 a, const float2 b) {
    unsigned long long &c = reinterpret_cast<unsigned long long &>(acc);
    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(c) : "l"(reinterpret_cast<const unsigned long long &>(a)), "l"(reinterpret_cast<const unsigned long long &>(b)));
}

// 64 x 64 score tile on a 16 x 16 thread grid: thread (ty,tx) owns rows ty+16r, keys tx+16c.  The
// (x,y) and (z,w) halves of the float4 operands feed packed FMAs; each score is kept as two partial
// sums that are added at the end.
template <int RQ, int RK>
__device__ __forceinline__ void qk_tile(const float *Qs, const float *Ks, int pitch, int wq, float (&acc)[4][4]) {
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
    const float *qp = Qs + (long long)ty * pitch, *kp = Ks + (long long)tx * pitch;
    float2 a2[RQ][RK];
#pragma unroll
    for (int r = 0; r < RQ; ++r)
#pragma unroll
        for (int c = 0; c < RK; ++c) a2[r][c] = make_float2(0.0f, 0.0f);
    // software pipeline: the operands of step d+4 are loaded while the FMAs of step d issue
    float4 q[RQ], k[RK], qn[RQ], kn[RK];
#pragma unroll
    for (int r = 0; r < RQ; ++r) q[r] = *reinterpret_cast<const float4 *>(qp + (long long)(16 * r) * pitch);
#pragma unroll
    for (int c = 0; c < RK; ++c) k[c] = *reinterpret_cast<const float4 *>(kp + (long long)(16 * c) * pitch);
#pragma unroll 2
    for (int d = 0; d < wq; d += 4) {
        const int dn = (d + 4 < wq) ? d + 4 : d;
#pragma unroll
        for (int r = 0; r < RQ; ++r) qn[r] = *reinterpret_cast<const float4 *>(qp + (long long)(16 * r) * pitch + dn);
#pragma unroll
        for (int c = 0; c < RK; ++c) kn[c] = *reinterpret_cast<const float4 *>(kp + (long long)(16 * c) * pitch + dn);
#pragma unroll
        for (int r = 0; r < RQ; ++r)
#pragma unroll
            for (int c = 0; c < RK; ++c) {
                ffma2(a2[r][c], make_float2(q[r].x, q[r].y), make_float2(k[c].x, k[c].y));
                ffma2(a2[r][c], make_float2(q[r].z, q[r].w), make_float2(k[c].z, k[c].w));
            }
#pragma unroll
        for (int r = 0; r < RQ; ++r) q[r] = qn[r];
#pragma unroll
        for (int c = 0; c < RK; ++c) k[c] = kn[c];
    }
#pragma unroll
    for (int r = 0; r < RQ; ++r)
#pragma unroll
        for (int c = 0; c < RK; ++c) acc[r][c] += a2[r][c].x + a2[r][c].y;
}

__device__ __forceinline__ void qk_dispatch(const float *Qs, const float *Ks, int pitch, int wq, int nq, int nk,
                                            float (&acc)[4][4]) {
    const int rq = nq <= 16 ? 1 : (nq <= 32 ? 2 : 4), rk = nk <= 16 ? 1 : (nk <= 32 ? 2 : 4);
#define B200ATTN_QK(A, B) if (rq == A && rk == B) { qk_tile<A, B>(Qs, Ks, pitch, wq, acc); return; }
    B200ATTN_QK(4, 4) B200ATTN_QK(2, 4) B200ATTN_QK(1, 4) B200ATTN_QK(4, 2) B200ATTN_QK(2, 2)
    B200ATTN_QK(1, 2) B200ATTN_QK(4, 1) B200ATTN_QK(2, 1) B200ATTN_QK(1, 1)
#undef B200ATTN_QK
}

// Adds (or, with a single slice, stores) a thread's part of the score tile to S[i0.., j0..].
__device__ __forceinline__ void emit_scores(float *S, int Lk, int i0, int j0, int nq, int nk, const float (&acc)[4][4],
                                            bool accumulate) {
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int i = ty + 16 * r, j = tx + 16 * c;
            if (i < nq && j < nk) {
                float *p = S + (long long)(i0 + i) * Lk + (j0 + j);
                if (accumulate) atomicAdd(p, acc[r][c]); else *p = acc[r][c];
            }
        }
}

// One PV unit: rows r0..r0+3, columns 4*c4..4*c4+3 of the V slice, keys [0, nj).
__device__ __forceinline__ void pv_unit(const float *Pt, const float *Vs, int vpitch, int nj, int r0, int c4,
                                        float (&o)[4][4]) {
    const float *pp = Pt + r0, *vp = Vs + 4 * c4;
#pragma unroll 8
    for (int j = 0; j < nj; ++j) {
        const float4 p = *reinterpret_cast<const float4 *>(pp + j * SD_PT_PITCH);
        const float4 v = *reinterpret_cast<const float4 *>(vp + (long long)j * vpitch);
        o[0][0] = fmaf(p.x, v.x, o[0][0]); o[0][1] = fmaf(p.x, v.y, o[0][1]); o[0][2] = fmaf(p.x, v.z, o[0][2]); o[0][3] = fmaf(p.x, v.w, o[0][3]);
        o[1][0] = fmaf(p.y, v.x, o[1][0]); o[1][1] = fmaf(p.y, v.y, o[1][1]); o[1][2] = fmaf(p.y, v.z, o[1][2]); o[1][3] = fmaf(p.y, v.w, o[1][3]);
        o[2][0] = fmaf(p.z, v.x, o[2][0]); o[2][1] = fmaf(p.z, v.y, o[2][1]); o[2][2] = fmaf(p.z, v.z, o[2][2]); o[2][3] = fmaf(p.z, v.w, o[2][3]);
        o[3][0] = fmaf(p.w, v.x, o[3][0]); o[3][1] = fmaf(p.w, v.y, o[3][1]); o[3][2] = fmaf(p.w, v.z, o[3][2]); o[3][3] = fmaf(p.w, v.w, o[3][3]);
    }
}

template <typename T>
__device__ __forceinline__ void store_unit(T *O, int D, int nq, int w, int v0, int r0, int c4, const float (&o)[4][4]) {
    const int c = 4 * c4;
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        if (r0 + r >= nq) break;
        T *op = O + (long long)(r0 + r) * D + v0 + c;
        if (c + 4 <= w && (D % 4 == 0) && ((reinterpret_cast<uintptr_t>(O) & 15) == 0)) {
            if constexpr (sizeof(T) == 4) {
                *reinterpret_cast<float4 *>(op) = make_float4(o[r][0], o[r][1], o[r][2], o[r][3]);
            } else {
                T h[4] = {OutCvt<T>::one(o[r][0]), OutCvt<T>::one(o[r][1]), OutCvt<T>::one(o[r][2]), OutCvt<T>::one(o[r][3])};
                *reinterpret_cast<uint2 *>(op) = *reinterpret_cast<const uint2 *>(h);
            }
        } else {
            for (int e = 0; e < 4 && c + e < w; ++e) op[e] = OutCvt<T>::one(o[r][e]);
        }
    }
}

// ------------------------------------------------------------------------------------------------
// Fused kernel: grid (nsplit, BH), cooperative launch, Lq <= 64 and Lk <= 64.
// Dynamic shared memory: Qs[64][ds+4] | Ks[64][ds+4] | Vs[64][ds+4] | Pt[64][68] | freq[ds/2].
// ------------------------------------------------------------------------------------------------
// Optional phase timestamps (build with -DB200ATTN_SD_PROFILE): CTA b writes globaltimer at stage k to sd_stamps[b*8+k].
#ifdef B200ATTN_SD_PROFILE
__device__ unsigned long long sd_stamps[8 * 1024];
#define SD_STAMP(k) do { if (threadIdx.x == 0) { unsigned long long t_; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_)); \
    sd_stamps[(blockIdx.y * gridDim.x + blockIdx.x) * 8 + (k)] = t_; } } while (0)
#else
#define SD_STAMP(k)
#endif

template <typename T>
__global__ void __launch_bounds__(SD_THREADS, 1)
splitd_fused_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const SplitDParams p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bar_qk, bar_v;
    __shared__ unsigned s_flag;

    SD_STAMP(0);
    const int slice = blockIdx.x;
    const long long bh = blockIdx.y;
    const int v0 = slice * p.ds;
    const int w = min(p.ds, p.D - v0);
    bool tma = false;
    if constexpr (sizeof(T) == 4) tma = (p.use_tma != 0);
    // TMA tiles are packed (row pitch = ds, chosen with ds/4 odd so that 16 rows spread over all
    // banks); the register-staged path pads the pitch instead
    const int pitch = tma ? p.ds : p.ds + 4;
    const int Lq = p.Lq, Lk = p.Lk, D = p.D;
    const int rq_pad = Lq <= 16 ? 16 : (Lq <= 32 ? 32 : 64), rk_pad = Lk <= 16 ? 16 : (Lk <= 32 ? 32 : 64);

    float *Qs = reinterpret_cast<float *>(smem_raw);
    float *Ks = Qs + SD_TILE * pitch;
    float *Vs = Ks + SD_TILE * pitch;
    float *Pt = Vs + SD_TILE * pitch;
    float *freq_s = Pt + SD_TILE * SD_PT_PITCH;

    const T *Qg = reinterpret_cast<const T *>(p.Q) + bh * Lq * D;
    const T *Kg = reinterpret_cast<const T *>(p.K) + bh * Lk * D;
    const T *Vg = reinterpret_cast<const T *>(p.V) + bh * Lk * D;
    T *Og = reinterpret_cast<T *>(p.O) + bh * Lq * D;
    float *Sg = p.S + bh * Lq * Lk;

    const int wq = (w + 3) & ~3;

    // ---- stage the slice ----
    if (tma) {
        if (threadIdx.x == 0) {
            mbar_init(&bar_qk, 1);
            mbar_init(&bar_v, 1);
            mbar_fence_init();
            // one tiled load per tensor: box = [L rows x ds columns] at (column v0, row bh*L); columns
            // beyond head_d read as zero and still count as transferred bytes
            mbar_expect_tx(&bar_qk, (uint32_t)(Lq + Lk) * (uint32_t)p.ds * 4u);
            tma_load_2d(Qs, &tmQ, v0, (int)(bh * Lq), &bar_qk);
            tma_load_2d(Ks, &tmK, v0, (int)(bh * Lk), &bar_qk);
            mbar_expect_tx(&bar_v, (uint32_t)Lk * (uint32_t)p.ds * 4u);
            tma_load_2d(Vs, &tmV, v0, (int)(bh * Lk), &bar_v);
        }
        __syncthreads();
        zero_rows(Qs, pitch, Lq, rq_pad, wq);
        zero_rows(Ks, pitch, Lk, rk_pad, wq);
    } else {
        const bool need_freq = (p.pe != PE_NONE) && !(p.cos_cache != nullptr && p.pe != PE_SINUSOIDAL);
        if (need_freq) {
            fill_freqs(freq_s, v0, w, p.pe == PE_SINUSOIDAL ? 10000.0f : p.rope_base, p.pe == PE_SINUSOIDAL ? D : p.rotary_dim);
            __syncthreads();
        }
        load_slice<T>(Qs, pitch, Qg, Lq, rq_pad, 0, D, v0, w, p.pe, p.rotary_dim, true, freq_s, p.cos_cache, p.sin_cache);
        load_slice<T>(Ks, pitch, Kg, Lk, rk_pad, 0, D, v0, w, p.pe, p.rotary_dim, pe_encodes_k(p.pe), freq_s,
                      p.cos_cache, p.sin_cache);
        load_slice<T>(Vs, pitch, Vg, Lk, Lk, 0, D, v0, w, PE_NONE, 0, false, nullptr, nullptr, nullptr);
    }

    bool ok = true;
    if (tma) ok = mbar_wait(&bar_qk, 0, p.spin_limit);
    __syncthreads();
    SD_STAMP(1);

    // ---- phase 1: partial scores of this slice ----
    float acc[4][4];
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[r][c] = 0.0f;
    if (ok) qk_dispatch(Qs, Ks, pitch, wq, Lq, Lk, acc);
    const bool single = (p.nsplit == 1);
    emit_scores(Sg, Lk, 0, 0, Lq, Lk, acc, !single);

    // ---- per-head barrier: all slices of this head have added their partial scores ----
    SD_STAMP(2);
    __threadfence();
    __syncthreads();
    SD_STAMP(3);
    if (threadIdx.x == 0) {
        unsigned flag = ok ? 0u : KERR_MBAR_TIMEOUT;
        if (!single) {
            atomicAdd(&p.counters[2 * bh], 1u);
            unsigned seen = 0;
            for (unsigned it = 0; it < p.spin_limit; ++it) {
                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(&p.counters[2 * bh]) : "memory");
                if (seen >= (unsigned)p.nsplit + p.wait_extra) break;
                __nanosleep(40);
            }
            if (seen < (unsigned)p.nsplit + p.wait_extra) flag |= KERR_HEAD_BARRIER_TIMEOUT;
        }
        if (flag) report_kernel_error(p.err, p.err_sys, flag);
        s_flag = flag;
    }
    __syncthreads();
    SD_STAMP(4);
    const bool failed = (s_flag != 0);

    // ---- phase 2a: softmax of the full score matrix into the transposed tile Pt[j][i] ----
    if (!failed) {
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        const int lq4 = (Lq + 3) & ~3;
        // all score loads of the warp's (up to 8) rows are issued before any of them is used: the
        // matrix lives in L2 and one dependent round trip per row would cost more than the softmax
        constexpr int RPW = SD_TILE / (SD_THREADS / 32);
        float s0[RPW], s1[RPW];
#pragma unroll
        for (int k = 0; k < RPW; ++k) {
            const int i = warp + k * (SD_THREADS / 32);
            s0[k] = -INFINITY; s1[k] = -INFINITY;
            if (i < Lq) {
                if (lane < Lk) s0[k] = __ldcg(Sg + (long long)i * Lk + lane);
                if (lane + 32 < Lk) s1[k] = __ldcg(Sg + (long long)i * Lk + lane + 32);
            }
        }
#ifdef B200ATTN_SD_PROFILE
        { float acc_ = 0.f; for (int k = 0; k < RPW; ++k) acc_ += s0[k] + s1[k]; if (acc_ == 123.456f) Pt[0] = acc_; }
        SD_STAMP(7);
#endif
        // the warp's rows go through max / exp / sum in lock step, so that the shuffle and
        // special-function latencies of the eight rows overlap instead of adding up
        float mx[RPW], e0[RPW], e1[RPW], tot[RPW];
#pragma unroll
        for (int k = 0; k < RPW; ++k) {
            s0[k] *= p.scale; s1[k] *= p.scale;
            mx[k] = fmaxf(s0[k], s1[k]);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int k = 0; k < RPW; ++k) mx[k] = fmaxf(mx[k], __shfl_xor_sync(0xffffffffu, mx[k], o));
#pragma unroll
        for (int k = 0; k < RPW; ++k) {
            const int i = warp + k * (SD_THREADS / 32);
            e0[k] = (i < Lq && lane < Lk) ? __expf(s0[k] - mx[k]) : 0.0f;   // arguments are <= 0: 2 ulp
            e1[k] = (i < Lq && lane + 32 < Lk) ? __expf(s1[k] - mx[k]) : 0.0f;
            tot[k] = e0[k] + e1[k];
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int k = 0; k < RPW; ++k) tot[k] += __shfl_xor_sync(0xffffffffu, tot[k], o);
#pragma unroll
        for (int k = 0; k < RPW; ++k) {
            const int i = warp + k * (SD_THREADS / 32);
            if (i < lq4) {
                const float inv = (i < Lq) ? __frcp_rn(tot[k]) : 0.0f;
                if (lane < Lk) Pt[lane * SD_PT_PITCH + i] = e0[k] * inv;
                if (lane + 32 < Lk) Pt[(lane + 32) * SD_PT_PITCH + i] = e1[k] * inv;
            }
        }
    }
    // every thread has read its scores (they are in Pt now); the count of readers is taken here,
    // without waiting for the answer: the clean-up itself is at the very end of the kernel
    __syncthreads();
    // ---- phase 2b: O[:, slice] = P * V[:, slice] ----
    SD_STAMP(5);
    bool okv = true;
    if (tma) okv = mbar_wait(&bar_v, 0, p.spin_limit);
    if (!okv && threadIdx.x == 0) report_kernel_error(p.err, p.err_sys, (unsigned)KERR_MBAR_TIMEOUT);
    if (failed || !okv) {
        // never leave the CTA while its own bulk copies may still be landing in shared memory
        if (tma) { mbar_wait(&bar_qk, 0, p.spin_limit); mbar_wait(&bar_v, 0, p.spin_limit); }
        return;
    }
    const int ncol4 = (w + 3) >> 2;
    const int nunits = ((Lq + 3) >> 2) * ncol4;
    for (int u = threadIdx.x; u < nunits; u += SD_THREADS) {
        const int r0 = (u / ncol4) * 4, c4 = u % ncol4;
        float o[4][4];
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int c = 0; c < 4; ++c) o[r][c] = 0.0f;
        pv_unit(Pt, Vs, pitch, Lk, r0, c4, o);
        store_unit<T>(Og, D, Lq, w, v0, r0, c4, o);
    }
    SD_STAMP(6);
    // ---- scratch hygiene, off the critical path: the last slice of the head to get here (all of them
    // read S before their PV phase) zeroes the head's scores and counters for the next call ----
    if (threadIdx.x == 0)
        s_flag = (single || atomicAdd(&p.counters[2 * bh + 1], 1u) == (unsigned)p.nsplit - 1u) ? 1u : 0u;
    __syncthreads();
    if (s_flag) {
        for (int i = threadIdx.x; i < Lq * Lk; i += SD_THREADS) Sg[i] = 0.0f;
        if (threadIdx.x == 0 && !single) { p.counters[2 * bh] = 0u; p.counters[2 * bh + 1] = 0u; }
    }
}

// ------------------------------------------------------------------------------------------------
// Two-pass path, pass 1: S[bh][i][j] (+)= sum over this CTA's column chunks.  grid (nsplit, nqt*nkt, BH);
// a CTA loops over ceil(nchunks/nsplit) chunks of ds columns, so nsplit = 1 needs no atomics.
// Dynamic shared memory: Qs[64][ds+4] | Ks[64][ds+4] | freq[ds/2].
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(SD_THREADS) splitd_scores_kernel(const SplitDParams p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int nkt = (p.Lk + SD_TILE - 1) / SD_TILE;
    const int qt = blockIdx.y / nkt, kt = blockIdx.y % nkt;
    const long long bh = blockIdx.z;
    const int pitch = p.ds + 4;
    const int i0 = qt * SD_TILE, j0 = kt * SD_TILE;
    const int nq = min(SD_TILE, p.Lq - i0), nk = min(SD_TILE, p.Lk - j0);
    const int rq_pad = nq <= 16 ? 16 : (nq <= 32 ? 32 : 64), rk_pad = nk <= 16 ? 16 : (nk <= 32 ? 32 : 64);
    float *Qs = reinterpret_cast<float *>(smem_raw);
    float *Ks = Qs + SD_TILE * pitch;
    float *freq_s = Ks + SD_TILE * pitch;
    const T *Qg = reinterpret_cast<const T *>(p.Q) + (bh * p.Lq + i0) * p.D;
    const T *Kg = reinterpret_cast<const T *>(p.K) + (bh * p.Lk + j0) * p.D;
    const bool need_freq = (p.pe != PE_NONE) && !(p.cos_cache != nullptr && p.pe != PE_SINUSOIDAL);

    float acc[4][4];
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[r][c] = 0.0f;

    // this CTA sums the column chunks [c0, c1) of width ds; the nsplit CTAs of a tile add up in S
    const int nchunks = (p.D + p.ds - 1) / p.ds;
    const int per = (nchunks + p.nsplit - 1) / p.nsplit;
    const int c0 = blockIdx.x * per, c1 = min(nchunks, c0 + per);
    for (int ch = c0; ch < c1; ++ch) {
        const int v0 = ch * p.ds, w = min(p.ds, p.D - v0);
        if (need_freq) {
            fill_freqs(freq_s, v0, w, p.pe == PE_SINUSOIDAL ? 10000.0f : p.rope_base, p.pe == PE_SINUSOIDAL ? p.D : p.rotary_dim);
            __syncthreads();
        }
        load_slice<T>(Qs, pitch, Qg, nq, rq_pad, i0, p.D, v0, w, p.pe, p.rotary_dim, true, freq_s, p.cos_cache, p.sin_cache);
        load_slice<T>(Ks, pitch, Kg, nk, rk_pad, j0, p.D, v0, w, p.pe, p.rotary_dim, pe_encodes_k(p.pe), freq_s,
                      p.cos_cache, p.sin_cache);
        __syncthreads();
        qk_dispatch(Qs, Ks, pitch, (w + 3) & ~3, nq, nk, acc);
        __syncthreads();
    }
    if (c0 < c1) emit_scores(p.S + bh * p.Lq * p.Lk, p.Lk, i0, j0, nq, nk, acc, p.nsplit > 1);
}

// ------------------------------------------------------------------------------------------------
// Two-pass path, pass 2: O[:, slice] = softmax(scale * S) * V[:, slice].  grid (ceil(D/dv), nqt, BH),
// dv <= 64.  Dynamic shared memory: Vs[64][dv+4] | Pt[64][68] | rowmax[64] | rowsum[64].
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(SD_THREADS) splitd_softmax_pv_kernel(const SplitDParams p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int dv = p.dv;
    const int v0 = blockIdx.x * dv, w = min(dv, p.D - v0), pitch = dv + 4;
    const int i0 = blockIdx.y * SD_TILE, nq = min(SD_TILE, p.Lq - i0);
    const long long bh = blockIdx.z;
    float *Vs = reinterpret_cast<float *>(smem_raw);
    float *Pt = Vs + SD_TILE * pitch;
    float *rowmax = Pt + SD_TILE * SD_PT_PITCH;
    float *rowsum = rowmax + SD_TILE;
    const float *Sg = p.S + (bh * p.Lq + i0) * p.Lk;
    const T *Vg = reinterpret_cast<const T *>(p.V) + bh * p.Lk * p.D;
    T *Og = reinterpret_cast<T *>(p.O) + (bh * p.Lq + i0) * p.D;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // row statistics over all keys (max, then sum of exp), one warp per row
    for (int i = warp; i < nq; i += SD_THREADS / 32) {
        const float *row = Sg + (long long)i * p.Lk;
        float m = -INFINITY;
        for (int j = lane; j < p.Lk; j += 32) m = fmaxf(m, __ldcg(row + j) * p.scale);
        m = warp_max(m);
        float t = 0.0f;
        for (int j = lane; j < p.Lk; j += 32) t += expf(__ldcg(row + j) * p.scale - m);
        t = warp_sum(t);
        if (lane == 0) { rowmax[i] = m; rowsum[i] = t; }
    }
    __syncthreads();

    const int ncol4 = (w + 3) >> 2;
    const int nunits = ((nq + 3) >> 2) * ncol4;   // <= 16 * 16 = 256: at most one unit per thread
    const int u = threadIdx.x;
    const int r0 = (u / ncol4) * 4, c4 = u % ncol4;
    float o[4][4];
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int c = 0; c < 4; ++c) o[r][c] = 0.0f;

    for (int j0 = 0; j0 < p.Lk; j0 += SD_TILE) {
        const int nk = min(SD_TILE, p.Lk - j0);
        load_slice<T>(Vs, pitch, Vg + (long long)j0 * p.D, nk, nk, 0, p.D, v0, w, PE_NONE, 0, false, nullptr, nullptr, nullptr);
        for (int idx = threadIdx.x; idx < SD_TILE * nk; idx += SD_THREADS) {
            const int i = idx / nk, j = idx - i * nk;   // consecutive threads -> consecutive keys: coalesced reads of S
            float pr = 0.0f;
            if (i < nq) pr = expf(__ldcg(Sg + (long long)i * p.Lk + j0 + j) * p.scale - rowmax[i]) / rowsum[i];
            Pt[j * SD_PT_PITCH + i] = pr;
        }
        __syncthreads();
        if (u < nunits) pv_unit(Pt, Vs, pitch, nk, r0, c4, o);
        __syncthreads();
    }
    if (u < nunits) store_unit<T>(Og, p.D, nq, w, v0, r0, c4, o);
}

}  // namespace b200attn
