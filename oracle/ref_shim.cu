/*
 * Shim that compiles the reference project's own translation units, where they lie in the
 * reference tree, into one shared library (oracle/_ref/libref_attn.so) with C-linkage wrappers
 * around its CPU oracles and its GPU launchers.  TEST INFRASTRUCTURE ONLY: used to pin the C
 * restatement in attn_oracle.c, as the "reference kernel" parity oracle on the GPU, and as the
 * CPU baseline that the benchmark reports.  No reference source is copied: the files are
 * #included by path (REF_ROOT is given on the compiler command line by oracle/build.py).
 *
 * Each reference file is a stand-alone program that re-defines the same helper names, so each is
 * wrapped in its own namespace and its main() is renamed.  Standard headers are included first,
 * outside any namespace, so that the includes inside the reference files become no-ops.
 */
#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <mma.h>
#include <cstdio>
#include <cmath>
#include <cstdlib>
#include <iostream>
#include <vector>

#define REF_STR2(x) #x
#define REF_STR(x) REF_STR2(x)
#define REF_FILE(rel) REF_STR(REF_ROOT/rel)

#define main ref_program_main

namespace ref_plain {
#include REF_FILE(final/attention.cu)
}
#undef CUDA_CHECK
namespace ref_rope {
#include REF_FILE(final/rope.cu)
}
#undef CUDA_CHECK
namespace ref_sinus {
#include REF_FILE(final/sinusoidal.cu)
}
#undef CUDA_CHECK
namespace ref_bf16 {
#include REF_FILE(kernels/attention_bf16_optimized_fused.cu)
}
#undef main

extern "C" {

/* final/attention.cu:228 */
void ref_attention_cpu(const float *Q, const float *K, const float *V, float *out,
                       int B, int H, int Lq, int Lk, int D) {
    ref_plain::attention_cpu(Q, K, V, out, B, H, Lq, Lk, D);
}
/* final/attention.cu:195 (device pointers; blocks until complete) */
void ref_attention_forward_optimized(const float *Q, const float *K, const float *V, float *out,
                                     int B, int H, int Lq, int Lk, int D) {
    ref_plain::attention_forward_optimized(Q, K, V, out, B, H, Lq, Lk, D);
}
/* final/rope.cu:20 */
void ref_precompute_rope_cache(float *c, float *s, int max_len, int rotary_dim, float base) {
    ref_rope::precompute_rope_cache(c, s, max_len, rotary_dim, base);
}
/* final/rope.cu:1439 */
void ref_attention_rope_cpu(const float *Q, const float *K, const float *V, float *out,
                            const float *c, const float *s, int B, int H, int Lq, int Lk, int D) {
    ref_rope::attention_rope_cpu(Q, K, V, out, c, s, B, H, Lq, Lk, D);
}
/* final/rope.cu:375 (raw K, on-the-fly angles) and :1209 (table driven); device pointers */
void ref_attention_forward_rope_fused_v2(const float *Q, const float *K, const float *V, float *out,
                                         int B, int H, int Lq, int Lk, int D) {
    ref_rope::attention_forward_rope_fused_v2(Q, K, V, out, B, H, Lq, Lk, D);
}
void ref_attention_forward_rope_fused(const float *Q, const float *K, const float *V, float *out,
                                      const float *c, const float *s,
                                      int B, int H, int Lq, int Lk, int D) {
    ref_rope::attention_forward_rope_fused(Q, K, V, out, c, s, B, H, Lq, Lk, D);
}
/* final/rope.cu:230 */
void ref_attention_forward_rope_fused_v7_hybrid(const float *Q, const float *Krot, const float *V,
                                                float *out, int B, int H, int Lq, int Lk, int D,
                                                int rotary_dim) {
    ref_rope::attention_forward_rope_fused_v7_hybrid(Q, Krot, V, out, B, H, Lq, Lk, D, rotary_dim);
}
/* final/sinusoidal.cu:838, :858 */
void ref_generate_sinusoidal_embeddings_cpu(float *sin_t, float *cos_t, int max_len, int D) {
    ref_sinus::generate_sinusoidal_embeddings_cpu(sin_t, cos_t, max_len, D);
}
void ref_attention_sinusoidal_cpu(const float *Q, const float *K, const float *V,
                                  const float *sin_t, const float *cos_t, float *out,
                                  int B, int H, int Lq, int Lk, int D) {
    ref_sinus::attention_sinusoidal_cpu(Q, K, V, sin_t, cos_t, out, B, H, Lq, Lk, D);
}
/* The reference has no host wrapper for the fused sinusoidal kernel; this is the launch its
 * test driver performs (final/sinusoidal.cu:1135-1137), followed by a device synchronise. */
int ref_attention_forward_sinusoidal_v5(const float *Q, const float *K, const float *V, float *out,
                                        int B, int H, int Lq, int Lk, int D) {
    float scale = 1.0f / sqrtf(static_cast<float>(D));
    dim3 grid(Lq, B * H);
    int smem = (64 + 32 + D) * (int)sizeof(float);
    ref_sinus::attention_fwd_kernel_sinusoidal_fused_v5<64><<<grid, 256, smem>>>(
        Q, K, V, out, B, H, Lq, Lk, D, scale);
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    return (int)e;
}
/* kernels/attention_bf16_optimized_fused.cu:493, :521 (device pointers to bf16) */
void ref_attention_forward_bf16(const void *Q, const void *K, const void *V, void *out,
                                int B, int H, int Lq, int Lk, int D) {
    ref_bf16::attention_forward_bf16((const __nv_bfloat16 *)Q, (const __nv_bfloat16 *)K,
                                     (const __nv_bfloat16 *)V, (__nv_bfloat16 *)out, B, H, Lq, Lk, D);
}
void ref_attention_forward_sinusoidal_bf16(const void *Q, const void *K, const void *V, void *out,
                                           int B, int H, int Lq, int Lk, int D) {
    ref_bf16::attention_forward_sinusoidal_bf16((const __nv_bfloat16 *)Q, (const __nv_bfloat16 *)K,
                                                (const __nv_bfloat16 *)V, (__nv_bfloat16 *)out,
                                                B, H, Lq, Lk, D);
}

} /* extern "C" */
