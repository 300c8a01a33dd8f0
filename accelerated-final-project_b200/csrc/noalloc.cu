// b200attn_forward_static: fp32 forward for small problems that never allocates.
//
// Some callers cannot allocate device memory at the moment they need attention: code living inside
// a framework whose caching allocator owns the whole device and must not see foreign cudaMalloc
// calls, a latency-critical loop that cannot afford the implicit device synchronisation an
// allocation may cause, or a process that has handed its memory budget to something else.  The
// regular entry points of this library
// grow a per-device scratch with cudaMalloc on demand; this one uses a fixed scratch that is part
// of the library image instead (a file-scope __device__ array, so every GPU that loads the
// library holds B200ATTN_STATIC_SCRATCH_BYTES of it until the process exits).
//
// What it runs: the fused split-head_d kernel (splitd.cuh), fp32, no positional encoding, whose
// scratch is the Lq x Lk score matrix of every head plus two arrival counters per head and an
// error word.  Limits (checked, B200ATTN_ERR_TOO_LARGE otherwise): len_q, len_k <= 64,
// batch*heads <= number of SMs, batch*heads*len_q*len_k*4 + batch*heads*8 + 256 bytes within the
// array.
//
// First call on a device: resolves the device address of the array (cudaGetSymbolAddress) and
// raises the kernel's shared-memory limit; both are host-side set-up without allocation, but they
// are not stream operations, so make the first call on each device before starting a capture.
// Every call uses the same array and clears the part it needs on the caller's stream first; two
// calls that overlap on the GPU (different streams, no dependency) would race on it.
#include <cmath>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "../../include/b200attn.h"
#include "splitd.cuh"

namespace b200attn {

constexpr size_t kStaticScratchBytes = B200ATTN_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

struct StaticDev {
    bool ready = false;
    unsigned char *scratch = nullptr;   // DEVICE address of g_static_scratch on this device
    int sm_count = 0;
    size_t dyn_smem_max = 0;
};
static StaticDev g_static_dev[64];
static std::mutex g_static_mu;
static thread_local char t_static_err[256] = "";

static int static_fail(int status, const char *msg) {
    snprintf(t_static_err, sizeof t_static_err, "%s", msg);
    return status;
}

}  // namespace b200attn

using namespace b200attn;

extern "C" const char *b200attn_static_last_error(void) { return t_static_err; }

extern "C" int b200attn_forward_static(const float *Q, const float *K, const float *V, float *out, int B, int H, int Lq, int Lk,
                                       int D, void *stream) {
    if (!Q || !K || !V || !out || B <= 0 || H <= 0 || Lq <= 0 || Lk <= 0 || D <= 0)
        return static_fail(B200ATTN_ERR_INVALID_ARG, "b200attn_forward_static: NULL pointer or non-positive size");
    if (out == Q || out == K || out == V) return static_fail(B200ATTN_ERR_INVALID_ARG, "b200attn_forward_static: out aliases an input");
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return static_fail(B200ATTN_ERR_NO_DEVICE, "b200attn_forward_static: no CUDA device");
    StaticDev &sd = g_static_dev[dev];
    {
        std::lock_guard<std::mutex> lk(g_static_mu);
        if (!sd.ready) {
            // The array's name is a host-side handle here, not a device address: ask the runtime for
            // the address on the CURRENT device and give the kernel that.
            void *ptr = nullptr;
            cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
            if (e != cudaSuccess) return static_fail(B200ATTN_ERR_CUDA, cudaGetErrorString(e));
            int major = 0, smem_optin = 0;
            cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
            cudaDeviceGetAttribute(&sd.sm_count, cudaDevAttrMultiProcessorCount, dev);
            cudaDeviceGetAttribute(&smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
            if (major != 10) return static_fail(B200ATTN_ERR_NO_DEVICE, "b200attn_forward_static: sm_100 device required");
            cudaFuncAttributes fa;
            e = cudaFuncGetAttributes(&fa, splitd_fused_kernel<float>);
            if (e != cudaSuccess) return static_fail(B200ATTN_ERR_CUDA, cudaGetErrorString(e));
            sd.dyn_smem_max = (size_t)smem_optin - fa.sharedSizeBytes;
            e = cudaFuncSetAttribute(splitd_fused_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sd.dyn_smem_max);
            if (e != cudaSuccess) return static_fail(B200ATTN_ERR_CUDA, cudaGetErrorString(e));
            sd.scratch = static_cast<unsigned char *>(ptr);
            sd.ready = true;
        }
    }
    const long long BH = (long long)B * H;
    if (Lq > SD_TILE || Lk > SD_TILE) return static_fail(B200ATTN_ERR_TOO_LARGE, "b200attn_forward_static: len_q and len_k must be <= 64");
    if (BH > sd.sm_count) return static_fail(B200ATTN_ERR_TOO_LARGE, "b200attn_forward_static: batch*heads exceeds the number of SMs");
    // layout of the array: [error word, padded to 256 B][2*BH counters, padded to 256 B][BH*Lq*Lk scores]
    const size_t counters_bytes = (((size_t)2 * BH * sizeof(unsigned)) + 255) & ~(size_t)255;
    const size_t scores_bytes = (size_t)BH * Lq * Lk * sizeof(float);
    const size_t need = 256 + counters_bytes + scores_bytes;
    if (need > kStaticScratchBytes) return static_fail(B200ATTN_ERR_TOO_LARGE, "b200attn_forward_static: batch*heads*len_q*len_k exceeds the static scratch");

    // slice width as in the regular entry point: packed TMA tiles want ds a multiple of 4 with ds/4 odd
    const bool tma_ok = (D % 4 == 0) && ((((uintptr_t)Q | (uintptr_t)K | (uintptr_t)V) & 15) == 0);
    long long nsplit_max = sd.sm_count / BH;
    int ds = (int)((D + nsplit_max - 1) / nsplit_max);
    bool use_tma = tma_ok;
    if (use_tma) {
        ds = (ds + 3) & ~3;
        if (((ds >> 2) & 1) == 0) ds += 4;
        if (ds > 252) use_tma = false;
    }
    if (!use_tma) {
        ds = (ds + 7) & ~7;
        if (ds < 8) ds = 8;
    }
    const int nsplit = (D + ds - 1) / ds;
    const size_t smem = ((size_t)3 * SD_TILE * (ds + 4) + (size_t)SD_TILE * SD_PT_PITCH + ds / 2 + 4) * sizeof(float);
    if (smem > sd.dyn_smem_max) return static_fail(B200ATTN_ERR_TOO_LARGE, "b200attn_forward_static: head_d too large for one slice per SM");
    CUtensorMap tmQ, tmK, tmV;   // encoded on the host; no device allocation involved
    memset(&tmQ, 0, sizeof tmQ); memset(&tmK, 0, sizeof tmK); memset(&tmV, 0, sizeof tmV);
    if (use_tma && (!make_tmap_2d(&tmQ, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, Q, BH * Lq, D, ds, Lq, CU_TENSOR_MAP_SWIZZLE_NONE) ||
                    !make_tmap_2d(&tmK, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, K, BH * Lk, D, ds, Lk, CU_TENSOR_MAP_SWIZZLE_NONE) ||
                    !make_tmap_2d(&tmV, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, V, BH * Lk, D, ds, Lk, CU_TENSOR_MAP_SWIZZLE_NONE)))
        return static_fail(B200ATTN_ERR_CUDA, "b200attn_forward_static: cuTensorMapEncodeTiled failed");

    cudaStream_t st = (cudaStream_t)stream;
    // the array keeps whatever the last call left: clear the part this call reads before writing
    cudaError_t e = cudaMemsetAsync(sd.scratch, 0, need, st);
    if (e != cudaSuccess) return static_fail(B200ATTN_ERR_CUDA, cudaGetErrorString(e));
    SplitDParams p{};
    p.Q = Q; p.K = K; p.V = V; p.O = out;
    p.BH = BH; p.Lq = Lq; p.Lk = Lk; p.D = D;
    p.ds = ds; p.nsplit = nsplit;
    p.pe = PE_NONE; p.rotary_dim = D; p.rope_base = 10000.0f;
    p.scale = 1.0f / sqrtf((float)D);
    p.err = reinterpret_cast<unsigned *>(sd.scratch);
    p.err_sys = nullptr;
    p.counters = reinterpret_cast<unsigned *>(sd.scratch + 256);
    p.S = reinterpret_cast<float *>(sd.scratch + 256 + counters_bytes);
    p.spin_limit = 1u << 21;
    p.use_tma = use_tma ? 1 : 0;
    dim3 grid(nsplit, (unsigned)BH);
    void *kargs[] = {&tmQ, &tmK, &tmV, &p};
    e = cudaLaunchCooperativeKernel((const void *)splitd_fused_kernel<float>, grid, dim3(SD_THREADS), kargs, smem, st);
    if (e != cudaSuccess) return static_fail(B200ATTN_ERR_CUDA, cudaGetErrorString(e));
    return B200ATTN_OK;
}
