// Blackwell (sm_100a) building blocks used by the tensor-core kernels: tensor memory, tcgen05.mma
// with shared-memory descriptors, TMA tiled loads, cluster / distributed-shared-memory helpers.
// Every wait in this file is bounded.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace b200attn {

// ---- cluster ------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
// Address of the same shared-memory location in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_rank(uint32_t saddr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
    return r;
}
__device__ __forceinline__ void st_cluster_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
// Arrive (release, cluster scope) on an mbarrier that may live in another CTA of the cluster.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait on a barrier whose arrivals may come from the peer CTA.
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t *bar, uint32_t parity, uint32_t limit) {
    for (uint32_t it = 0; it < limit; ++it) {
        if (mbar_try_wait_cluster(bar, parity)) return true;
        if (it > 64) __nanosleep(32);
    }
    return false;
}
// Generic-proxy writes (st.shared / st.shared::cluster) -> visible to the async proxy (UMMA, TMA).
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }
// The same restricted to this CTA's shared memory / to the cluster's shared memory.  The unrestricted
// form also orders global memory between the proxies: it waits for the thread's global stores and for
// bulk copies in flight, which costs thousands of cycles inside a pipelined loop.
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_dsmem() { asm volatile("fence.proxy.async.shared::cluster;" ::: "memory"); }

// ---- TMA tiled load (no multicast) ----------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(void *smem_dst, const CUtensorMap *tmap, int x, int y, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
            smem_u32(smem_dst)),
        "l"(tmap), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void tma_load_3d(void *smem_dst, const CUtensorMap *tmap, int x, int y, int z, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(
            smem_u32(smem_dst)),
        "l"(tmap), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void tma_load_4d(void *smem_dst, const CUtensorMap *tmap, int x, int y, int z, int w, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(
            smem_u32(smem_dst)),
        "l"(tmap), "r"(x), "r"(y), "r"(z), "r"(w), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap *tmap) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// ---- tensor memory ------------------------------------------------------------------------------
// One full warp allocates `ncols` (power of two >= 32) columns; the base address lands in *slot.
__device__ __forceinline__ void tmem_alloc(uint32_t *slot, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// 32 lanes x 32 columns of 32-bit: thread i of the warp receives columns [col, col+32) of TMEM lane
// (lane_base + i); a warp may only touch the lane quadrant 32*(warp_id % 4).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
        "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
        "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]),
        "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ---- UMMA descriptors -----------------------------------------------------------------------------
// Shared-memory matrix descriptor (64 bit): start address >> 4 in bits [0,14), leading byte offset
// >> 4 in [16,30), stride byte offset >> 4 in [32,46), version 1 in [46,48), layout type in [61,64)
// (2 = 128-byte swizzle).
//
// K-major operand tile, 128-byte swizzle: rows of 64 bf16 (128 B) at a pitch of 128 B, groups of 8
// rows 1024 B apart (SBO); 1024-byte aligned.  A K=16 step inside the 64-wide row advances the start
// address by 32 B.
__device__ __forceinline__ uint64_t umma_desc_k_sw128(uint32_t saddr) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)2 << 61);
}
// MN-major operand tile, 128-byte swizzle: 64 MN-elements (128 B) contiguous per K row, groups of 8
// K rows 1024 B apart (SBO), the next 64 MN-elements `lbo_bytes` further (LBO).
__device__ __forceinline__ uint64_t umma_desc_mn_sw128(uint32_t saddr, uint32_t lbo_bytes) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo_bytes >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// MN-major operand tile of 32-bit elements (tf32): the only swizzled layout the tensor core takes for
// it is the 128-byte swizzle on 32-byte units (layout type 1; what TMA writes with
// CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B): 32 MN-elements (128 B) contiguous per K row, the 32-byte
// quarter q of K row r stored at quarter q ^ (r % 4), groups of 4 K rows `sbo_bytes` apart, the next
// 32 MN-elements `lbo_bytes` further.
__device__ __forceinline__ uint64_t umma_desc_mn_sw128_32b(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo_bytes >> 4) << 16) | ((uint64_t)(sbo_bytes >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)1 << 61);
}
// Instruction descriptor, kind::f16 with bf16 operands and fp32 accumulation: D format fp32 (bits
// [4,6) = 1), A/B format bf16 (bits [7,10) and [10,13) = 1), major bits 15/16 (0 = K-major,
// 1 = MN-major), N >> 3 in [17,23), M >> 4 in [24,29).
__host__ __device__ constexpr uint32_t umma_idesc_bf16(int M, int N, int a_mn_major, int b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)a_mn_major << 15) | ((uint32_t)b_mn_major << 16) |
           ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
// The same with the 16-bit operand format chosen at run time: fp16 (format code 0) or bf16 (1).
__host__ __device__ constexpr uint32_t umma_idesc_16(int M, int N, int a_mn_major, int b_mn_major, int f16) {
    return (1u << 4) | ((f16 ? 0u : 1u) << 7) | ((f16 ? 0u : 1u) << 10) | ((uint32_t)a_mn_major << 15) | ((uint32_t)b_mn_major << 16) |
           ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// The mbarrier receives one arrival when every MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// ---- the same for kind::tf32: fp32 containers of which the tensor core uses sign, exponent and the upper
// ten mantissa bits; fp32 accumulation.  A/B format code 2 (bits [7,10) and [10,13)); K = 8 per
// instruction (32 bytes of a K-major row, one 8-row group of an MN-major tile). ----
__host__ __device__ constexpr uint32_t umma_idesc_tf32(int M, int N, int a_mn_major, int b_mn_major) {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)a_mn_major << 15) | ((uint32_t)b_mn_major << 16) |
           ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
__device__ __forceinline__ void umma_tf32(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// ---- programmatic dependent launch: no-ops unless the kernel was launched with the attribute ---------
// Lets the next kernel of the stream, if it was launched as a programmatic dependent, start now.
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// Returns once the kernel this one programmatically depends on has completed and its writes are visible.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ---- TMA tiled store shared -> global (bulk async-group completion) ---------------------------------
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *tmap, const void *smem_src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(tmap), "r"(smem_u32(smem_src)),
                 "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// ... until the stores have read their shared-memory source (it may then be reused, or the CTA may exit)
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }

// Four fp32 additions to global memory in one L2 operation (16-byte aligned address).
__device__ __forceinline__ void red_add_v4(float *addr, float a, float b, float c, float d) {
    asm volatile("red.relaxed.gpu.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// ---- the same for a pair of CTAs working as one (cta_group::2): both CTAs of a 2-CTA cluster allocate
// together, the MMA is issued by one thread of the LEADER CTA (cluster rank 0) with M = 256 (128 rows
// from each CTA's A tile, into each CTA's own tensor memory) and the B tile split along N between
// the two CTAs' shared memories at the same offsets; a commit arrives on ONE mbarrier given by its
// shared::cluster address (so it may be the peer's); a bulk-tensor load may complete on the peer's
// mbarrier.  No multicast is used anywhere. ----
__device__ __forceinline__ void tmem_alloc_2cta(uint32_t *slot, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_2cta(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_bf16_2cta(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// one arrival on the mbarrier at this shared::cluster address when every MMA issued so far has completed
__device__ __forceinline__ void umma_commit_2cta(uint32_t cluster_addr) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr) : "memory");
}
// tiled load into THIS CTA's shared memory whose bytes are counted on the mbarrier at `mbar_cluster_addr`
__device__ __forceinline__ void tma_load_2d_2cta(void *smem_dst, const CUtensorMap *tmap, int x, int y, uint32_t mbar_cluster_addr) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
            smem_u32(smem_dst)),
        "l"(tmap), "r"(x), "r"(y), "r"(mbar_cluster_addr)
        : "memory");
}

// ---- host: tensor maps (the encoder is taken from the driver at run time; no -lcuda) -------------
typedef CUresult (*PFN_tmapEncodeTiled)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                         const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                         CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
inline PFN_tmapEncodeTiled tmap_encode_fn() {
    static PFN_tmapEncodeTiled fn = [] {
        void *f = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &qres) != cudaSuccess || qres != cudaDriverEntryPointSuccess)
            f = nullptr;
        return (PFN_tmapEncodeTiled)f;
    }();
    return fn;
}
// Tiled map over a row-major [rows][cols] matrix; box = [box_rows][box_cols]; out-of-range elements read as zero.
inline bool make_tmap_2d(CUtensorMap *m, CUtensorMapDataType dt, int esize, const void *base, long long rows, long long cols,
                         int box_cols, int box_rows, CUtensorMapSwizzle swz) {
    PFN_tmapEncodeTiled enc = tmap_encode_fn();
    if (!enc) return false;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)cols * esize};
    cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    return enc(m, dt, 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// 32-byte store (one full sector per thread; the address must be 32-byte aligned).  Row-per-thread
// epilogues write with this: a 16-byte store covers half a sector, and partial-sector writes make
// the L2 merge (or fetch) the other half.
__device__ __forceinline__ void st_global_v8(void *ptr, uint4 a, uint4 b) {
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(ptr), "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b.x),
                 "r"(b.y), "r"(b.z), "r"(b.w)
                 : "memory");
}

// Row-per-thread epilogues hold, per thread, 128 contiguous bytes of "their" row (w[0..31]).  Stored
// as they are, every store instruction of a warp touches 32 different cache lines.  This helper
// first transposes 4x4 blocks of 32-byte pieces among groups of four neighbouring lanes (= four
// neighbouring rows) with two butterfly rounds of shuffles, after which lane j of a group holds
// piece j of each of the group's rows, and every store instruction writes full 128-byte lines.
// `row0_ptr` is the address of the 128-byte segment in the row of the group's FIRST lane,
// `row_pitch` the distance between rows in bytes.  All 32 lanes must call it.
__device__ __forceinline__ void store_rows_128B_transposed(unsigned char *row0_ptr, size_t row_pitch, uint32_t (&w)[32], int lane) {
    const int j = lane & 3;
#pragma unroll
    for (int M = 2; M >= 1; M >>= 1) {
        const bool up = (j & M) != 0;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if (k & M) continue;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const uint32_t send = up ? w[8 * k + e] : w[8 * (k | M) + e];
                const uint32_t recv = __shfl_xor_sync(0xffffffffu, send, M);
                if (up) w[8 * k + e] = recv; else w[8 * (k | M) + e] = recv;
            }
        }
    }
    // slot m now holds piece j of the row of lane (group base + m)
#pragma unroll
    for (int m = 0; m < 4; ++m)
        st_global_v8(row0_ptr + (size_t)m * row_pitch + j * 32, make_uint4(w[8 * m], w[8 * m + 1], w[8 * m + 2], w[8 * m + 3]),
                     make_uint4(w[8 * m + 4], w[8 * m + 5], w[8 * m + 6], w[8 * m + 7]));
}

// The same where only the first `rows_valid` rows of the lane's group of four exist (<= 0: none): the
// trade is done by all lanes, the stores only for rows that exist.
__device__ __forceinline__ void store_rows_128B_transposed_if(unsigned char *row0_ptr, size_t row_pitch, uint32_t (&w)[32], int lane, int rows_valid) {
    const int j = lane & 3;
#pragma unroll
    for (int M = 2; M >= 1; M >>= 1) {
        const bool up = (j & M) != 0;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if (k & M) continue;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const uint32_t send = up ? w[8 * k + e] : w[8 * (k | M) + e];
                const uint32_t recv = __shfl_xor_sync(0xffffffffu, send, M);
                if (up) w[8 * k + e] = recv; else w[8 * (k | M) + e] = recv;
            }
        }
    }
#pragma unroll
    for (int m = 0; m < 4; ++m)
        if (m < rows_valid)
            st_global_v8(row0_ptr + (size_t)m * row_pitch + j * 32, make_uint4(w[8 * m], w[8 * m + 1], w[8 * m + 2], w[8 * m + 3]),
                         make_uint4(w[8 * m + 4], w[8 * m + 5], w[8 * m + 6], w[8 * m + 7]));
}

// A bf16 row-major [rows][cols] matrix seen as [cols/64 groups][rows][64 columns], so that ONE request
// fetches a box of `box_groups` 64-column groups x `box_rows` rows and lays it down as consecutive
// [box_rows x 128 B] slabs with the 128-byte swizzle: the shared-memory layout of a K-major tile
// wider than 64 elements, or of an MN-major operand, which otherwise takes one request per slab.
// (A bulk-tensor request costs the SM about 130 cycles whatever its size.)
inline bool make_tmap_grouped(CUtensorMap *m, const void *base, long long rows, long long cols, int box_rows, int box_groups) {
    PFN_tmapEncodeTiled enc = tmap_encode_fn();
    if (!enc || cols % 64 != 0) return false;
    cuuint64_t dims[3] = {64, (cuuint64_t)rows, (cuuint64_t)(cols / 64)};
    cuuint64_t strides[2] = {(cuuint64_t)cols * 2, 128};
    cuuint32_t box[3] = {64, (cuuint32_t)box_rows, (cuuint32_t)box_groups};
    cuuint32_t estr[3] = {1, 1, 1};
    return enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The same for `heads` matrices of [rows][cols] one after the other, with the head as a fourth coordinate: rows
// of a box beyond a head's last row read as zero instead of as the next head's rows.
inline bool make_tmap_grouped_heads(CUtensorMap *m, const void *base, long long heads, long long rows, long long cols, int box_rows, int box_groups) {
    PFN_tmapEncodeTiled enc = tmap_encode_fn();
    if (!enc || cols % 64 != 0) return false;
    cuuint64_t dims[4] = {64, (cuuint64_t)rows, (cuuint64_t)(cols / 64), (cuuint64_t)heads};
    cuuint64_t strides[3] = {(cuuint64_t)cols * 2, 128, (cuuint64_t)rows * (cuuint64_t)cols * 2};
    cuuint32_t box[4] = {64, (cuuint32_t)box_rows, (cuuint32_t)box_groups, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    return enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
}
// two values rounded to the 16-bit format of the call's tensors: fp16 or bf16
__device__ __forceinline__ uint32_t pack_16x2(float lo, float hi, bool f16) {
    if (f16) {
        __half2 v = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<uint32_t *>(&v);
    }
    return pack_bf16x2(lo, hi);
}
__device__ __forceinline__ uint16_t pack_16(float x, bool f16) {
    if (f16) { __half v = __float2half_rn(x); return *reinterpret_cast<uint16_t *>(&v); }
    __nv_bfloat16 v = __float2bfloat16_rn(x);
    return *reinterpret_cast<uint16_t *>(&v);
}

}  // namespace b200attn
