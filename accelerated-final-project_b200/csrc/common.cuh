// Shared device/host helpers for the b200attn kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#if defined(__CUDA_ARCH__) && (__CUDA_ARCH__ < 1000)
#error "b200attn is written for sm_100a only"
#endif

// The in-kernel cycle accounting and the bring-up exports exist only in builds made with
// -DB200ATTN_DEVTOOLS (the shipped library is built without it).
#ifndef B200ATTN_DEVTOOLS
#undef B200ATTN_SD_PROFILE
#undef B200ATTN_TC_PROFILE
#endif

namespace b200attn {

// Positional-encoding selector; values match enum b200attn_pe in include/b200attn.h.
enum PeKind : int { PE_NONE = 0, PE_ROPE_INTERLEAVED = 1, PE_ROPE_HALF = 2, PE_SINUSOIDAL = 3, PE_ROPE_Q_ONLY = 4, PE_ROPE_HALF_Q_ONLY = 5 };
__host__ __device__ __forceinline__ bool pe_pairs_halves(int pe) { return pe == PE_ROPE_HALF || pe == PE_ROPE_HALF_Q_ONLY; }
__host__ __device__ __forceinline__ bool pe_is_rope(int pe) { return pe == PE_ROPE_INTERLEAVED || pe == PE_ROPE_HALF || pe == PE_ROPE_Q_ONLY || pe == PE_ROPE_HALF_Q_ONLY; }
__host__ __device__ __forceinline__ bool pe_encodes_k(int pe) { return pe != PE_NONE && pe != PE_ROPE_Q_ONLY && pe != PE_ROPE_HALF_Q_ONLY; }

// Error bits a kernel may OR into its error word (read back by the host after the launch).
enum KernelErr : unsigned {
    KERR_HEAD_BARRIER_TIMEOUT = 1u,  // split-head_d: not every slice of a head arrived in time
    KERR_MBAR_TIMEOUT = 2u,          // a bounded mbarrier wait expired
    KERR_TMEM = 4u                   // tensor-memory allocation protocol failed
};

// Record kernel error bits: in the device error word (complete, OR-ed) and, when the host gave one,
// in a word of mapped pinned host memory, which the host can look at after a synchronisation
// without a device-to-host copy (any non-zero value there means "read the device word").
__device__ __forceinline__ void report_kernel_error(unsigned *err, unsigned *err_sys, unsigned bits) {
    atomicOr(err, bits);
    if (err_sys != nullptr) {
        *reinterpret_cast<volatile unsigned *>(err_sys) = bits;
        __threadfence_system();
    }
}

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- mbarrier (shared::cta) -------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_test_wait(uint64_t *bar, uint32_t parity) {   // one look, never suspends
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: returns false when `limit` polls went by without the phase completing.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, uint32_t limit) {
    if (mbar_test_wait(bar, parity)) return true;   // often the phase is long complete: try_wait costs ~80 clocks more even then
    for (uint32_t it = 0; it < limit; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if (it > 64) __nanosleep(32);
    }
    return false;
}

// ---- bulk async copy global -> shared (TMA, untiled): 16-byte aligned addresses, size % 16 == 0
__device__ __forceinline__ void bulk_g2s(void *smem_dst, const void *gsrc, uint32_t bytes, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            smem_u32(smem_dst)),
        "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// ---- element conversion -----------------------------------------------------------------------
__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }
__device__ __forceinline__ float to_f32(__half x) { return __half2float(x); }

template <typename T> struct OutCvt;
template <> struct OutCvt<float> {
    static __device__ __forceinline__ float one(float x) { return x; }
};
template <> struct OutCvt<__nv_bfloat16> {
    static __device__ __forceinline__ __nv_bfloat16 one(float x) { return __float2bfloat16_rn(x); }
};
template <> struct OutCvt<__half> {
    static __device__ __forceinline__ __half one(float x) { return __float2half_rn(x); }
};

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

}  // namespace b200attn
