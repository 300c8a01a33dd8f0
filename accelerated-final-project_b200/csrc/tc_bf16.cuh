// bf16 attention forward on the 5th-generation tensor cores (tcgen05 + tensor memory + TMA).
//
// Why a CTA PAIR per query tile.  With head_d = 512 an fp32 output accumulator of 128 query rows
// fills all 512 columns of an SM's tensor memory, so the score tile S = Q K^T has nowhere to live
// on the same SM.  The work of one (batch-head, 128-query tile) is therefore split over a cluster
// of two CTAs that run different programs and execute the same number of tensor-core flops:
//
//   rank 0, "score CTA":  Q tile resident in shared memory (K-major, 128-byte swizzle), K streamed
//       by TMA in [128 keys x 64 columns] chunks, S = Q K^T into tensor memory (4 buffers of 128
//       columns), softmax warps read S with tcgen05.ld, keep the running max / sum per row in
//       registers and write P = exp2(scale*log2e*(S - m)) as bf16 straight into the OTHER CTA's
//       shared memory (distributed shared memory stores), in the swizzled K-major layout the PV
//       MMA wants.  The positional encoding is applied by transform warps to the Q tile once and
//       to every K chunk between its TMA arrival and its MMA (no separate pass over global memory).
//   rank 1, "output CTA": V streamed by TMA in [32 keys x head_d] stages (MN-major operand), the
//       accumulator O[128 x head_d] fp32 resident in tensor memory, O += P V; correction warps
//       rescale O only when the score CTA raised a row's reference max (lazy rescaling), and at
//       the end divide by the row sums and store bf16.
//
// All cross-role hand-offs are mbarriers; arrivals that cross the CTA boundary use cluster scope.
// Every wait is bounded: on expiry the role records KERR_MBAR_TIMEOUT and leaves its loop; all
// threads of both CTAs always reach the final cluster barrier, so neither CTA exits while its peer
// may still address its shared memory.
//
// Shapes taken here: bf16, head_d % 64 == 0, 64 <= head_d <= 512, len_q % 128 == 0,
// len_k % 128 == 0, encodings none / sinusoidal / interleaved RoPE (with or without K rotation).
// Everything else runs on the split-head_d kernels.
#pragma once

#include <atomic>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "../../include/b200attn.h"
#include "tc_common.cuh"

namespace b200attn {

constexpr int TC_THREADS = 448;   // warp 0 TMA, warp 1 MMA, warps 2-9 softmax (output CTA: 2-5 correction, 6 relay), warps 10-13 transform
constexpr int TC_BM = 128;        // query rows per tile
constexpr int TC_BN = 128;        // keys per block
constexpr int TC_VS = 32;         // keys per V stage
constexpr int TC_NK = 5;          // K chunk ring depth (score CTA)
constexpr int TC_NS = 4;          // S buffers in tensor memory (4 x 128 columns)
constexpr int TC_NP = 3;          // P buffers (output CTA shared memory)
constexpr int TC_NV = 3;          // V stage ring depth (output CTA)
constexpr int TC_NL = 8;          // row-sum slots in flight (the score CTA may run a few units ahead)
constexpr int TC_CHUNK_BYTES = TC_BM * 128;          // [128 rows x 64 bf16]
constexpr int TC_P_BYTES = TC_BM * TC_BN * 2;        // one P buffer
constexpr float TC_RESCALE_LOG2 = 8.0f;              // rescale O only when the max grew by > 2^8

struct TcParams {
    int Lq, Lk, D;
    int n_qtiles, n_blocks, n_chunks;   // Lq/128, Lk/128, D/64
    float scale_log2;                   // log2(e) / sqrt(D)
    int pe, rd;                         // PeKind; rotary_dim
    int rotate_k;                       // 0: K is taken as given (pre-rotated by the caller, or the encoded-K cache)
    int qt0, n_qt;                      // this launch covers query tiles [qt0, qt0 + n_qt) of every head
    long long n_units;                  // BH * n_qt units, dealt round-robin to the persistent clusters
    __nv_bfloat16 *k_store;             // optional: encoded K chunks are also written here ([BH*Lk][D])
    int sb_keys;                        // keys per score MMA tile: 256 (no encoding) or 128
    int k_stages, k_stage_bytes;        // K ring: 5 x 16 KB, or 3 x (16 KB K chunk + 16 KB encoding chunk)
    __nv_bfloat16 *O;
    unsigned *err;
    unsigned *err_sys;   // mirror flag in mapped host memory (may be null)
    unsigned spin_limit;
    float *debug_scores;                // optional: raw S of key block 0, [units][128][128]
};

struct TcBarriers {
    uint64_t q_full, q_empty;   // Q tile of the unit landed / was read by the unit's last score MMA
    uint64_t k_full[TC_NK], k_ready[TC_NK], k_empty[TC_NK];
    uint64_t s_full[TC_NS], s_empty[TC_NS];
    uint64_t p_empty[TC_NP];    // in the score CTA; arrived by the output CTA's relay warp
    uint64_t v_full[TC_NV], v_empty[TC_NV];
    uint64_t p_full[TC_NP];     // in the output CTA; arrived by the score CTA's softmax threads
    uint64_t pv_done[TC_NP];
    uint64_t corr_done[TC_NP];
    uint64_t l_full[TC_NL];     // row sums of unit (ui % TC_NL) have been sent
    uint64_t decided[2];        // score CTA: reference max of block t settled (t & 1)
};

// Positional encoding of one [128 rows x 64 columns] bf16 chunk in shared memory.  The encoding
// values arrive by TMA from a bf16 table in global memory as a tile of the SAME shape and swizzle,
// so element (row, col) of both tiles sits at the same byte offset and the transform is a plain
// element-wise pass over 1024 16-byte vectors (128 threads x 8), done with packed bf16x2 math:
//   sinusoidal: x += pe                                  (table: sin at even, cos at odd columns)
//   RoPE pairs: (xe, xo) -> (xe*c - xo*s, xe*s + xo*c)    (table: c at even, s at odd columns; c=1,
//                                                         s=0 beyond rotary_dim)
__device__ __forceinline__ uint32_t tc_pe_pair(uint32_t x, uint32_t t, bool sinus) {
    __nv_bfloat162 xv = *reinterpret_cast<__nv_bfloat162 *>(&x);
    __nv_bfloat162 r;
    if (sinus) {
        r = __hadd2(xv, *reinterpret_cast<__nv_bfloat162 *>(&t));
    } else {
        uint32_t cc = __byte_perm(t, 0, 0x1010);                  // (c, c)
        uint32_t ss = __byte_perm(t, 0, 0x3232) ^ 0x00008000u;    // (-s, s)
        uint32_t xs = __byte_perm(x, 0, 0x1032);                  // (xo, xe)
        r = __hfma2(*reinterpret_cast<__nv_bfloat162 *>(&xs), *reinterpret_cast<__nv_bfloat162 *>(&ss),
                    __hmul2(xv, *reinterpret_cast<__nv_bfloat162 *>(&cc)));
    }
    return *reinterpret_cast<uint32_t *>(&r);
}
__device__ __forceinline__ void tc_pe_chunk(unsigned char *tile, const unsigned char *pe_tile, bool sinus, int tid,
                                            __nv_bfloat16 *gdst = nullptr, int D = 0) {
    uint4 *x = reinterpret_cast<uint4 *>(tile);
    const uint4 *t = reinterpret_cast<const uint4 *>(pe_tile);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int o = tid + 128 * i;
        uint4 v = x[o];
        const uint4 w = t[o];
        v.x = tc_pe_pair(v.x, w.x, sinus);
        v.y = tc_pe_pair(v.y, w.y, sinus);
        v.z = tc_pe_pair(v.z, w.z, sinus);
        v.w = tc_pe_pair(v.w, w.w, sinus);
        x[o] = v;
        if (gdst != nullptr) {   // un-swizzle: piece o is row o/8, logical 16-byte column (o%8) ^ (row%8)
            const int r = o >> 3, q = (o & 7) ^ (r & 7);
            *reinterpret_cast<uint4 *>(gdst + (long long)r * D + q * 8) = v;
        }
    }
}

// Optional cycle accounting of the roles of cluster 0 (build with -DB200ATTN_TC_PROFILE).
#ifdef B200ATTN_TC_PROFILE
__device__ unsigned long long tc_prof[32];
#define TC_PROF_DECL long long pc_ = clock64(); unsigned long long pa_[8] = {0, 0, 0, 0, 0, 0, 0, 0}
#define TC_PROF(slot) do { const long long n_ = clock64(); pa_[(slot) & 7] += (unsigned long long)(n_ - pc_); pc_ = n_; } while (0)
#define TC_PROF_FLUSH(base, on) do { if ((on) && blockIdx.x < 2) for (int i_ = 0; i_ < 8; ++i_) tc_prof[(base) + i_] = pa_[i_]; } while (0)
#else
#define TC_PROF_DECL
#define TC_PROF(slot)
#define TC_PROF_FLUSH(base, on)
#endif

// A bounded wait that expired: record the error bit and, in bits 8.., which wait it was (the
// sites are numbered in source order), then leave the enclosing loop.
#define TC_FAIL_AT(site, cond)                                                     \
    if (cond) {                                                                    \
        report_kernel_error(p.err, p.err_sys, (unsigned)KERR_MBAR_TIMEOUT | (1u << (7 + (site)))); \
        failed = true;                                                             \
        break;                                                                     \
    }

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(TC_THREADS, 1)
tc_bf16_pair_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmPE, const TcParams p) {
    extern __shared__ unsigned char tc_smem_raw[];
    __shared__ TcBarriers bars;
    __shared__ uint32_t tmem_slot;
    __shared__ unsigned skip_flag;
    __shared__ float m_state[2][TC_BM];   // reference maxima of the rows, by unit parity

    // 1024-byte aligned base; identical offset in both CTAs of the cluster (same kernel, same layout)
    const uint32_t raw_addr = smem_u32(tc_smem_raw);
    unsigned char *smem = tc_smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);

    const uint32_t rank = cluster_ctarank();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // Persistent clusters: cluster k runs the units k, k + n_clusters, ...  Ring and barrier phases
    // run on through the units, so the score CTA starts the next unit (Q load, first score tiles,
    // softmax) while the output CTA is still finishing and storing the previous one.
    const int cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
    const int D = p.D, nch = p.n_chunks, T = p.n_blocks;
    const uint32_t lim = p.spin_limit;
    const bool has_pe = (p.pe != PE_NONE);
    const bool pe_k = has_pe && p.rotate_k;          // K chunks are encoded too (not for pre-rotated K)
    const int NKS = p.k_stages, KSB = p.k_stage_bytes;
    const int SB = p.sb_keys;                        // keys per score tile (one S buffer in tensor memory)
    const int HPS = SB / TC_BN;                      // 128-key blocks per score tile
    const int NSB = 512 / SB;                        // score tiles resident in tensor memory
    const int U = (T + HPS - 1) / HPS;               // score tiles per unit

    // ---- shared-memory carve-up ----
    // score CTA : [Q: nch chunks of 16 KB][K ring: k_stages stages of (K chunk [+ encoding chunk])][P staging: 8 x 4 KB]
    // output CTA: [P: TC_NP x 32 KB][V ring: TC_NV stages of TC_VS*D*2 B][alpha: TC_NP x 128 f32][lsum: TC_NL x 2 x 128 f32]
    unsigned char *q_smem = smem;
    unsigned char *k_smem = smem + (size_t)nch * TC_CHUNK_BYTES;
    unsigned char *stage_smem = k_smem + (size_t)p.k_stages * p.k_stage_bytes;   // 8 x 4 KB: P staging of the softmax warps
    unsigned char *p_smem = smem;
    unsigned char *v_smem = smem + (size_t)TC_NP * TC_P_BYTES;
    const int v_stage_bytes = TC_VS * D * 2;
    float *alpha_smem = reinterpret_cast<float *>(v_smem + (size_t)TC_NV * v_stage_bytes);
    float *lsum_smem = alpha_smem + TC_NP * TC_BM;

    if (threadIdx.x == 0) {
        mbar_init(&bars.q_full, 1);
        mbar_init(&bars.q_empty, 1);
        for (int i = 0; i < TC_NK; ++i) { mbar_init(&bars.k_full[i], 1); mbar_init(&bars.k_ready[i], 4); mbar_init(&bars.k_empty[i], 1); }
        for (int i = 0; i < TC_NS; ++i) { mbar_init(&bars.s_full[i], 1); mbar_init(&bars.s_empty[i], 4 * (p.sb_keys / TC_BN)); }
        for (int i = 0; i < TC_NV; ++i) { mbar_init(&bars.v_full[i], 1); mbar_init(&bars.v_empty[i], 1); }
        for (int i = 0; i < TC_NP; ++i) {
            mbar_init(&bars.p_empty[i], 1);
            mbar_init(&bars.p_full[i], 4);
            mbar_init(&bars.pv_done[i], 1);
            mbar_init(&bars.corr_done[i], 4);
        }
        for (int i = 0; i < TC_NL; ++i) mbar_init(&bars.l_full[i], p.n_blocks >= 2 ? 8 : 4);
        mbar_init(&bars.decided[0], 4);
        mbar_init(&bars.decided[1], 4);
        mbar_fence_init();
        tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
        if (p.pe != PE_NONE) tma_prefetch_desc(&tmPE);
    }
    if (warp == 0) tmem_alloc(&tmem_slot, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    // Once any cluster has reported an error the remaining clusters skip their work.  The score
    // CTA samples the error word and tells its peer, so that both CTAs take the same decision.
    cluster_arrive();   // both CTAs are running and have initialised their barriers
    cluster_wait();
    if (rank == 0 && threadIdx.x == 0) {
        const unsigned seen = *reinterpret_cast<volatile unsigned *>(p.err);
        skip_flag = seen;
        asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(map_to_rank(smem_u32(&skip_flag), 1)), "r"(seen) : "memory");
    }
    cluster_arrive();
    cluster_wait();

    bool failed = false;
    const bool skip = (skip_flag != 0);
    const long long n_units = p.n_units;

    if (skip) {
        // nothing: fall through to the common exit
    } else if (rank == 0) {
        // =============================== score CTA ===============================
        if (warp == 0) {
            if (lane == 0) {
                int it = 0, ui = 0;
                for (long long unit = cluster_id; unit < n_units && !failed; unit += n_clusters, ++ui) {
                    const int qt = p.qt0 + (int)(unit % p.n_qt);
                    const long long bh = unit / p.n_qt;
                    // the Q tile of the previous unit must have been read by its last score MMA
                    TC_FAIL_AT(1, !mbar_wait(&bars.q_empty, (ui & 1) ^ 1, lim));
                    mbar_expect_tx(&bars.q_full, (uint32_t)nch * TC_CHUNK_BYTES);
                    for (int c = 0; c < nch; ++c)
                        tma_load_2d(q_smem + (size_t)c * TC_CHUNK_BYTES, &tmQ, c * 64, (int)(bh * p.Lq + qt * TC_BM), &bars.q_full);
                    // With an encoding, the first nch ring slots of a unit carry the encoding rows of the
                    // QUERY tile (applied to the resident Q tile by the transform warps); after that every
                    // slot carries a K chunk and, if K is encoded too, its encoding chunk.
                    if (has_pe)
                        for (int c = 0; c < nch; ++c, ++it) {
                            const int s = it % NKS;
                            TC_FAIL_AT(2, !mbar_wait(&bars.k_empty[s], ((it / NKS) & 1) ^ 1, lim));
                            mbar_expect_tx(&bars.k_full[s], TC_CHUNK_BYTES);
                            tma_load_2d(k_smem + (size_t)s * KSB + TC_CHUNK_BYTES, &tmPE, c * 64, qt * TC_BM, &bars.k_full[s]);
                        }
                    for (int u = 0; u < U && !failed; ++u)
                        for (int c = 0; c < nch; ++c, ++it) {
                            const int s = it % NKS;
                            TC_FAIL_AT(3, !mbar_wait(&bars.k_empty[s], ((it / NKS) & 1) ^ 1, lim));
                            mbar_expect_tx(&bars.k_full[s], (uint32_t)SB * 128u + (pe_k ? TC_CHUNK_BYTES : 0));
                            tma_load_2d(k_smem + (size_t)s * KSB, &tmK, c * 64, (int)(bh * p.Lk + u * SB), &bars.k_full[s]);
                            if (pe_k) tma_load_2d(k_smem + (size_t)s * KSB + TC_CHUNK_BYTES, &tmPE, c * 64, u * SB, &bars.k_full[s]);
                        }
                }
            }
        } else if (warp == 1) {
            if (lane == 0) {
                const uint32_t idesc = umma_idesc_bf16(TC_BM, SB, 0, 0);
                int it = 0, ui = 0;
                uint32_t qph = 0;   // per-slot phase parity of k_ready when only the query phase uses it
                long long ug = 0;   // running score-tile counter
                TC_PROF_DECL;
                for (long long unit = cluster_id; unit < n_units && !failed; unit += n_clusters, ++ui) {
                    TC_FAIL_AT(4, !mbar_wait(&bars.q_full, ui & 1, lim));
                    if (has_pe)   // hand the ring slots of the query-encoding phase back once the transform warps are done with them
                        for (int c = 0; c < nch && !failed; ++c, ++it) {
                            const int s = it % NKS;
                            // k_ready[s] completes one phase per use by the transform warps: every ring use
                            // when K is encoded too, only these query-phase uses otherwise (tracked in qph)
                            const uint32_t par = pe_k ? ((it / NKS) & 1) : ((qph >> s) & 1);
                            qph ^= 1u << s;
                            TC_FAIL_AT(5, !mbar_wait(&bars.k_ready[s], par, lim));
                            mbar_arrive(&bars.k_empty[s]);
                        }
                    tc_fence_after();
                    for (int u = 0; u < U && !failed; ++u, ++ug) {
                        const int sb = (int)(ug % NSB);
                        TC_FAIL_AT(6, !mbar_wait(&bars.s_empty[sb], ((ug / NSB) & 1) ^ 1, lim));
                        tc_fence_after();
                        TC_PROF(4);
                        for (int c = 0; c < nch; ++c, ++it) {
                            const int s = it % NKS;
                            TC_PROF(5);
                            TC_FAIL_AT(7, !mbar_wait(pe_k ? &bars.k_ready[s] : &bars.k_full[s], (it / NKS) & 1, lim));
                            tc_fence_after();
                            TC_PROF(6);
                            const uint64_t da = umma_desc_k_sw128(smem_u32(q_smem + (size_t)c * TC_CHUNK_BYTES));
                            const uint64_t db = umma_desc_k_sw128(smem_u32(k_smem + (size_t)s * KSB));
#pragma unroll
                            for (int k = 0; k < 4; ++k)
                                umma_bf16(tmem + sb * SB, da + 2 * k, db + 2 * k, idesc, (c | k) != 0);
                            umma_commit(&bars.k_empty[s]);
                        }
                        if (failed) break;
                        umma_commit(&bars.s_full[sb]);
                        TC_PROF(5);
                    }
                    if (failed) break;
                    umma_commit(&bars.q_empty);   // the Q tile may be replaced once these MMAs have run
                }
                TC_PROF_FLUSH(8, true);
            }
        } else if (warp < 10) {
            // ---- softmax: two warpgroups (warps 2-5 and 6-9) take alternate key blocks; in each a
            // thread owns one query row.  The rows' reference maxima live in shared memory (m_state)
            // and are advanced strictly in block order: the group of block t waits for the decision
            // of block t-1, which the other group publishes through the `decided` barriers, right
            // after its (short) max pass, so the long exp/store passes of the two groups overlap.
            const int wg = (warp - 2) >> 2;
            const int n_groups = (T >= 2) ? 2 : 1;   // with a single key block per unit the second group has nothing to do
            const int row = 32 * (warp & 3) + lane;
            const uint32_t lane_addr = tmem + ((uint32_t)(32 * (warp & 3)) << 16);
            const uint32_t p_remote = map_to_rank(smem_u32(p_smem), 1);
            const uint32_t alpha_remote = map_to_rank(smem_u32(alpha_smem), 1);
            const uint32_t lsum_remote = map_to_rank(smem_u32(lsum_smem), 1);
            unsigned char *my_stage = stage_smem + (warp - 2) * 4096;   // 4 KB per softmax warp
            uint32_t r[32];
            int ui = 0;
            TC_PROF_DECL;
            for (long long unit = cluster_id; unit < n_units && !failed; unit += n_clusters, ++ui) {
                const long long tbase = (long long)ui * T, ubase = (long long)ui * U;   // running block / tile counters
                float *mst = m_state[ui & 1];
                float m_seen = -INFINITY, l = 0.0f;   // l is relative to m_seen
                int last = -1;
                // a score tile holds HPS blocks of 128 keys; with 256-key tiles the two groups work on the
                // two halves of the same tile, with 128-key tiles on alternate tiles
                const int t_end = U * HPS;
                for (int t = wg; t < t_end; t += 2) {
                    const long long tg = tbase + t, ug = ubase + t / HPS;
                    const int sb = (int)(ug % NSB), pb = (int)(tg % TC_NP);
                    TC_FAIL_AT(8, !mbar_wait(&bars.s_full[sb], (ug / NSB) & 1, lim));
                    if (t >= T) {   // padding half of the last tile: nothing to do but release it
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&bars.s_empty[sb]);
                        continue;
                    }
                    tc_fence_after();
                    TC_PROF(0);
                    const uint32_t ta = lane_addr + sb * SB + (t % HPS) * TC_BN;
                    float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        tmem_ld32(ta + c * 32, r);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            mx0 = fmaxf(mx0, __uint_as_float(r[j]));
                            mx1 = fmaxf(mx1, __uint_as_float(r[j + 1]));
                            mx2 = fmaxf(mx2, __uint_as_float(r[j + 2]));
                            mx3 = fmaxf(mx3, __uint_as_float(r[j + 3]));
                        }
#ifdef B200ATTN_DEVTOOLS
                        if (p.debug_scores != nullptr && t == 0) {
                            float *dbg = p.debug_scores + ((long long)unit * TC_BM + row) * TC_BN + c * 32;
                            for (int j = 0; j < 32; ++j) dbg[j] = __uint_as_float(r[j]);
                        }
#endif
                    }
                    const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
                    TC_PROF(1);
                    // decision for block t (needs the decision of block t-1 of this unit)
                    float m_new = mx, alpha = 1.0f;
                    if (t > 0) {
                        TC_FAIL_AT(9, !mbar_wait(&bars.decided[(tg - 1) & 1], ((tg - 1) >> 1) & 1, lim));
                        const float m_prev = mst[row];
                        if ((mx - m_prev) * p.scale_log2 > TC_RESCALE_LOG2) alpha = fast_exp2((m_prev - mx) * p.scale_log2);
                        else m_new = m_prev;
                    }
                    mst[row] = m_new;
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bars.decided[tg & 1]);
                    if (last >= 0 && m_new != m_seen) l *= fast_exp2((m_seen - m_new) * p.scale_log2);
                    m_seen = m_new;
                    TC_PROF(4);
                    TC_FAIL_AT(10, !mbar_wait_cluster(&bars.p_empty[pb], ((tg / TC_NP) & 1) ^ 1, lim));
                    TC_PROF(2);
                    const float msl = m_new * p.scale_log2;
                    // The block's probabilities go to the peer in two column blocks of 64 keys.  A warp
                    // first lays its 32 rows x 128 B out in its own 4 KB staging area (already in the
                    // swizzled layout of the destination), then copies it with lane-contiguous 16-byte
                    // remote stores, so that every remote store instruction covers 512 contiguous bytes.
                    const uint32_t pblk = p_remote + pb * TC_P_BYTES + (32 * (warp & 3)) * 128;
                    float l0 = 0.0f, l1 = 0.0f, l2 = 0.0f, l3 = 0.0f;
#pragma unroll
                    for (int cb = 0; cb < 2; ++cb) {
#pragma unroll
                        for (int ch = 0; ch < 2; ++ch) {
                            tmem_ld32(ta + (cb * 2 + ch) * 32, r);
                            tmem_ld_wait();
#pragma unroll
                            for (int g = 0; g < 4; ++g) {
                                float e[8];
#pragma unroll
                                for (int j = 0; j < 8; ++j) e[j] = fast_exp2(fmaf(__uint_as_float(r[8 * g + j]), p.scale_log2, -msl));
                                l0 += e[0] + e[4]; l1 += e[1] + e[5]; l2 += e[2] + e[6]; l3 += e[3] + e[7];
                                const int q = ch * 4 + g;   // 16-byte chunk index within the 64-key row
                                *reinterpret_cast<uint4 *>(my_stage + lane * 128 + ((q ^ (row & 7)) << 4)) =
                                    make_uint4(pack_bf16x2(e[0], e[1]), pack_bf16x2(e[2], e[3]), pack_bf16x2(e[4], e[5]), pack_bf16x2(e[6], e[7]));
                            }
                        }
                        __syncwarp();
#pragma unroll 4
                        for (int i = 0; i < 8; ++i) {
                            const uint4 v = *reinterpret_cast<const uint4 *>(my_stage + i * 512 + lane * 16);
                            st_cluster_v4(pblk + cb * (TC_BM * 128) + i * 512 + lane * 16, v.x, v.y, v.z, v.w);
                        }
                        __syncwarp();
                    }
                    l += (l0 + l1) + (l2 + l3);
                    tc_fence_before();
                    st_cluster_f32(alpha_remote + (pb * TC_BM + row) * 4, alpha);
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bars.s_empty[sb]);
                    last = t;
                    TC_PROF(3);
                    // hand the block over: every lane makes its stores visible to the peer's tensor core,
                    // one lane arrives for the warp (the other group computes meanwhile)
                    fence_proxy_async_dsmem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(map_to_rank(smem_u32(&bars.p_full[pb]), 1));
                    TC_PROF(5);
                }
                if (failed) break;
                // this group's part of the row sums, brought to the unit's final reference max.  A group
                // that did not take the last block waits for its decision first.  With a single key
                // block per unit the second group only releases the padding halves of the score tiles
                // and sends nothing.
                if (wg < n_groups) {
                    if (last != T - 1) {
                        const long long tl = tbase + T - 1;
                        TC_FAIL_AT(11, !mbar_wait(&bars.decided[tl & 1], (tl >> 1) & 1, lim));
                        const float m_fin = mst[row];
                        if (last >= 0 && m_fin != m_seen) l *= fast_exp2((m_seen - m_fin) * p.scale_log2);
                    }
                    const int ls = ui % TC_NL;
                    st_cluster_f32(lsum_remote + ((ls * 2 + wg) * TC_BM + row) * 4, l);
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(map_to_rank(smem_u32(&bars.l_full[ls]), 1));
                }
            }
            TC_PROF_FLUSH(0, threadIdx.x == 64);
        } else if (has_pe) {
            // ---- transform warps: encoding of the Q tile once per unit, then of every K chunk ----
            const int tid = threadIdx.x - 10 * 32;
            const bool sinus = (p.pe == PE_SINUSOIDAL);
            int it = 0, ui = 0;
            for (long long unit = cluster_id; unit < n_units && !failed; unit += n_clusters, ++ui) {
                const long long bh = unit / p.n_qt;
                TC_FAIL_AT(12, !mbar_wait(&bars.q_full, ui & 1, lim));
                for (int c = 0; c < nch; ++c, ++it) {
                    const int s = it % NKS;
                    TC_FAIL_AT(13, !mbar_wait(&bars.k_full[s], (it / NKS) & 1, lim));
                    tc_pe_chunk(q_smem + (size_t)c * TC_CHUNK_BYTES, k_smem + (size_t)s * KSB + TC_CHUNK_BYTES, sinus, tid);
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bars.k_ready[s]);
                }
                if (failed) break;
                if (pe_k) {
                    for (int t = 0; t < T && !failed; ++t)
                        for (int c = 0; c < nch; ++c, ++it) {
                            const int s = it % NKS;
                            TC_FAIL_AT(14, !mbar_wait(&bars.k_full[s], (it / NKS) & 1, lim));
                            unsigned char *kt = k_smem + (size_t)s * KSB;
                            __nv_bfloat16 *gd = p.k_store ? p.k_store + ((bh * p.Lk + (long long)t * TC_BN) * D + c * 64) : nullptr;
                            tc_pe_chunk(kt, kt + TC_CHUNK_BYTES, sinus, tid, gd, D);
                            fence_proxy_async_smem();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(&bars.k_ready[s]);
                        }
                } else {   // K comes encoded already and goes straight to the MMA; only the ring counter moves on
                    it += U * nch;
                }
            }
        }
    } else {
        // =============================== output CTA ===============================
        if (warp == 0) {
            if (lane == 0) {
                int it = 0;
                for (long long unit = cluster_id; unit < n_units && !failed; unit += n_clusters) {
                    const long long bh = unit / p.n_qt;
                    for (int t = 0; t < T && !failed; ++t)
                        for (int vs = 0; vs < TC_BN / TC_VS; ++vs, ++it) {
                            const int s = it % TC_NV;
                            TC_FAIL_AT(16, !mbar_wait(&bars.v_empty[s], ((it / TC_NV) & 1) ^ 1, lim));
                            mbar_expect_tx(&bars.v_full[s], (uint32_t)v_stage_bytes);
                            for (int g = 0; g < nch; ++g)
                                tma_load_2d(v_smem + (size_t)s * v_stage_bytes + (size_t)g * (TC_VS * 128), &tmV, g * 64,
                                            (int)(bh * p.Lk + t * TC_BN + vs * TC_VS), &bars.v_full[s]);
                        }
                }
            }
        } else if (warp == 1) {
            if (lane == 0) {
                int it = 0;
                long long tg = 0;   // running block counter
                TC_PROF_DECL;
                for (long long unit = cluster_id; unit < n_units && !failed; unit += n_clusters) {
                    for (int t = 0; t < T && !failed; ++t, ++tg) {
                        const int pb = (int)(tg % TC_NP);
                        TC_FAIL_AT(17, !mbar_wait_cluster(&bars.p_full[pb], (tg / TC_NP) & 1, lim));
                        TC_PROF(0);
                        TC_FAIL_AT(18, !mbar_wait(&bars.corr_done[pb], (tg / TC_NP) & 1, lim));
                        tc_fence_after();
                        TC_PROF(1);
                        for (int vs = 0; vs < TC_BN / TC_VS; ++vs, ++it) {
                            const int s = it % TC_NV;
                            TC_PROF(2);
                            TC_FAIL_AT(19, !mbar_wait(&bars.v_full[s], (it / TC_NV) & 1, lim));
                            tc_fence_after();
                            TC_PROF(3);
#pragma unroll
                            for (int kk = 0; kk < TC_VS / 16; ++kk) {
                                const int kg = vs * (TC_VS / 16) + kk;   // 16-key step within the block, 0..7
                                const uint64_t da = umma_desc_k_sw128(smem_u32(p_smem + (size_t)pb * TC_P_BYTES + (kg >> 2) * (TC_BM * 128))) + 2 * (kg & 3);
                                for (int n0 = 0; n0 < D; n0 += 256) {
                                    const int N = min(256, D - n0);
                                    const uint64_t db = umma_desc_mn_sw128(
                                        smem_u32(v_smem + (size_t)s * v_stage_bytes + (size_t)(n0 >> 6) * (TC_VS * 128) + kk * 2048), TC_VS * 128);
                                    umma_bf16(tmem + n0, da, db, umma_idesc_bf16(TC_BM, N, 0, 1), (t | kg) != 0);
                                }
                            }
                            umma_commit(&bars.v_empty[s]);
                        }
                        if (failed) break;
                        umma_commit(&bars.pv_done[pb]);
                        TC_PROF(2);
                    }
                }
                TC_PROF_FLUSH(16, true);
            }
        } else if (warp < 6) {
            // ---- correction + epilogue: one thread per query row ----
            const int row = 32 * (warp & 3) + lane;
            const uint32_t lane_addr = tmem + ((uint32_t)(32 * (warp & 3)) << 16);
            const int n_groups = (T >= 2) ? 2 : 1;
            uint32_t r[32];
            int ui = 0;
            long long tg = 0;
            for (long long unit = cluster_id; unit < n_units && !failed; unit += n_clusters, ++ui) {
                const int qt = p.qt0 + (int)(unit % p.n_qt);
                const long long bh = unit / p.n_qt;
                for (int t = 0; t < T; ++t, ++tg) {
                    const int pb = (int)(tg % TC_NP);
                    TC_FAIL_AT(20, !mbar_wait_cluster(&bars.p_full[pb], (tg / TC_NP) & 1, lim));
                    const float a = alpha_smem[pb * TC_BM + row];
                    if (t > 0 && __any_sync(0xffffffffu, a != 1.0f)) {
                        TC_FAIL_AT(21, !mbar_wait(&bars.pv_done[(tg - 1) % TC_NP], ((tg - 1) / TC_NP) & 1, lim));
                        tc_fence_after();
                        for (int c = 0; c < D / 32; ++c) {
                            tmem_ld32(lane_addr + c * 32, r);
                            tmem_ld_wait();
#pragma unroll
                            for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * a);
                            tmem_st32(lane_addr + c * 32, r);
                        }
                        tmem_st_wait();
                        tc_fence_before();
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bars.corr_done[pb]);
                }
                if (failed) break;
                // epilogue of the unit: O / row sum -> bf16 -> global.  The accumulator is free for the
                // next unit (whose first block overwrites it) only after these reads: the arrival on
                // corr_done for that block comes after this point in program order.
                const long long tl = tg - 1;
                TC_FAIL_AT(22, !mbar_wait(&bars.pv_done[tl % TC_NP], (tl / TC_NP) & 1, lim));
                tc_fence_after();
                const int ls = ui % TC_NL;
                TC_FAIL_AT(23, !mbar_wait_cluster(&bars.l_full[ls], (ui / TC_NL) & 1, lim));
                float lsum = lsum_smem[(ls * 2) * TC_BM + row];
                if (n_groups == 2) lsum += lsum_smem[(ls * 2 + 1) * TC_BM + row];
                const float inv = 1.0f / lsum;
                __nv_bfloat16 *orow = p.O + ((bh * p.Lq + qt * TC_BM + row) * (long long)D);
                for (int c = 0; c < D / 32; ++c) {
                    tmem_ld32(lane_addr + c * 32, r);
                    tmem_ld_wait();
                    uint4 o[4];
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        o[g].x = pack_bf16x2(__uint_as_float(r[8 * g + 0]) * inv, __uint_as_float(r[8 * g + 1]) * inv);
                        o[g].y = pack_bf16x2(__uint_as_float(r[8 * g + 2]) * inv, __uint_as_float(r[8 * g + 3]) * inv);
                        o[g].z = pack_bf16x2(__uint_as_float(r[8 * g + 4]) * inv, __uint_as_float(r[8 * g + 5]) * inv);
                        o[g].w = pack_bf16x2(__uint_as_float(r[8 * g + 6]) * inv, __uint_as_float(r[8 * g + 7]) * inv);
                    }
                    st_global_v8(orow + c * 32, o[0], o[1]);
                    st_global_v8(orow + c * 32 + 16, o[2], o[3]);
                }
                tc_fence_before();   // the accumulator reads are ordered before the corr_done arrival of the next unit
            }
        } else if (warp == 6) {
            // ---- relay: "PV of block t finished" -> the score CTA may overwrite that P buffer ----
            if (lane == 0) {
                long long tg = 0;
                for (long long unit = cluster_id; unit < n_units && !failed; unit += n_clusters)
                    for (int t = 0; t < T; ++t, ++tg) {
                        const int pb = (int)(tg % TC_NP);
                        TC_FAIL_AT(24, !mbar_wait(&bars.pv_done[pb], (tg / TC_NP) & 1, lim));
                        mbar_arrive_cluster(map_to_rank(smem_u32(&bars.p_empty[pb]), 0));
                    }
            }
        }
    }

    // a role that gave up lets copies and MMAs it may still have in flight drain before the CTA ends
    if (failed) for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    cluster_arrive();
    cluster_wait();
    if (warp == 0) tmem_dealloc(tmem, 512);
}
#undef TC_FAIL_AT

// ---- positional-encoding tables: [L][D] bf16, built on the device with the fp32 arithmetic of the
// reference CPU tables (final/sinusoidal.cu:838-855, final/rope.cu:20-40) and rounded once ----
__global__ void tc_build_pe_table(__nv_bfloat16 *table, int L, int D, int pe, int rd, float base) {
    const long long n = (long long)L * D;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const int pos = (int)(i / D), d = (int)(i % D);
        float v;
        if (pe == PE_SINUSOIDAL) {
            const float freq = 1.0f / powf(10000.0f, (2.0f * (float)(d / 2)) / (float)D);
            const float ang = (float)pos * freq;
            v = (d & 1) ? cosf(ang) : sinf(ang);
        } else if (d < rd) {
            const float freq = 1.0f / powf(base, (2.0f * (float)(d / 2)) / (float)rd);
            const float th = (float)pos * freq;
            v = (d & 1) ? sinf(th) : cosf(th);
        } else {
            v = (d & 1) ? 0.0f : 1.0f;   // columns beyond rotary_dim: identity rotation
        }
        table[i] = __float2bfloat16_rn(v);
    }
}

struct TcTables {
    struct Entry { int pe, L, D, rd; float base; __nv_bfloat16 *ptr; };
    static constexpr int kMax = 8;
    Entry e[kMax];
    int n = 0;
    __nv_bfloat16 *kcache = nullptr;   // encoded K of the current call (see tc_bf16_run)
    size_t kcache_bytes = 0;
    void release() {
        for (int i = 0; i < n; ++i) cudaFree(e[i].ptr);
        n = 0;
        if (kcache) cudaFree(kcache);
        kcache = nullptr;
        kcache_bytes = 0;
    }
    __nv_bfloat16 *get_kcache(size_t bytes) {
        if (bytes > kcache_bytes) {
            if (kcache) { cudaDeviceSynchronize(); cudaFree(kcache); }
            kcache = nullptr;
            kcache_bytes = 0;
            if (cudaMalloc(&kcache, bytes) != cudaSuccess) { (void)cudaGetLastError(); return nullptr; }
            kcache_bytes = bytes;
        }
        return kcache;
    }
    // Returns a device table with at least L rows for the key, building it on `st` when it is new.
    __nv_bfloat16 *get(int pe, int L, int D, int rd, float base, cudaStream_t st, std::atomic<unsigned long long> *launches, int *rows) {
        const int kind = (pe == PE_SINUSOIDAL) ? PE_SINUSOIDAL : PE_ROPE_INTERLEAVED;
        for (int i = 0; i < n; ++i)
            if (e[i].pe == kind && e[i].L >= L && e[i].D == D && e[i].rd == rd && e[i].base == base) { *rows = e[i].L; return e[i].ptr; }
        if (n == kMax) {   // evict everything once no kernel can still be reading a table
            cudaDeviceSynchronize();
            release();
        }
        __nv_bfloat16 *ptr = nullptr;
        if (cudaMalloc(&ptr, (size_t)L * D * sizeof(__nv_bfloat16)) != cudaSuccess) { (void)cudaGetLastError(); return nullptr; }
        tc_build_pe_table<<<296, 256, 0, st>>>(ptr, L, D, kind, rd, base);
        launches->fetch_add(1);
        e[n++] = Entry{kind, L, D, rd, base, ptr};
        *rows = L;
        return ptr;
    }
};

static thread_local char t_tc_error[256] = "";
inline const char *tc_bf16_error() { return t_tc_error; }

inline bool tc_bf16_supported(const b200attn_args &a, int rd) {
    if (a.dtype != B200ATTN_BF16) return false;
    if (a.head_d % 64 != 0 || a.head_d < 64 || a.head_d > 512) return false;
    if (a.len_q % TC_BM != 0 || a.len_k % TC_BN != 0) return false;
    if (pe_pairs_halves(a.pe)) return false;
    if (a.pe != B200ATTN_PE_NONE && a.pe != B200ATTN_PE_SINUSOIDAL && (rd % 8 != 0)) return false;
    if (a.cos_cache != nullptr) return false;
    if ((((uintptr_t)a.Q | (uintptr_t)a.K | (uintptr_t)a.V | (uintptr_t)a.out) & 15) != 0) return false;
    if (((uintptr_t)a.out & 31) != 0) return false;   // the epilogue stores 32 bytes at a time
    const long long BH = (long long)a.batch_sz * a.num_heads;
    if (BH * a.len_q >= (1ll << 31) || BH * a.len_k >= (1ll << 31)) return false;
    if (BH * (a.len_q / TC_BM) * 2 >= (1ll << 31)) return false;
    return true;
}

// 2-D bf16 tensor map over a [rows][D] row-major matrix with a [box_rows][64] box, 128-byte swizzle.
inline bool tc_make_map(CUtensorMap *m, const void *base, long long rows, int D, int box_rows) {
    return make_tmap_2d(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, rows, D, 64, box_rows, CU_TENSOR_MAP_SWIZZLE_128B);
}

inline size_t tc_smem_bytes(int D, bool has_pe) {
    (void)has_pe;
    const size_t ring = (size_t)2 * 2 * TC_CHUNK_BYTES + 8 * 4096;   // 2 stages of 32 KB (a 256-key K chunk, or a 128-key chunk + its encoding chunk) + P staging
    const size_t score = (size_t)(D / 64) * TC_CHUNK_BYTES + ring;
    const size_t outp = (size_t)TC_NP * TC_P_BYTES + (size_t)TC_NV * TC_VS * D * 2 + (size_t)(TC_NP + 2 * TC_NL) * TC_BM * sizeof(float);
    return (score > outp ? score : outp) + 1024;
}

// Returns B200ATTN_OK, -1 when the shape should run on the other path, or a status with tc_bf16_error() set.
inline int tc_bf16_run(const b200attn_args &a, int rd, float base, TcTables &tables, unsigned *err_dev, unsigned *err_sys, int sm_count,
                       unsigned spin_limit, cudaStream_t st, std::atomic<unsigned long long> *launches, float *debug_scores = nullptr) {
    const long long BH = (long long)a.batch_sz * a.num_heads;
    const int D = a.head_d;
    static std::mutex attr_mu;
    static bool attr_done[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    const size_t smem = tc_smem_bytes(D, a.pe != B200ATTN_PE_NONE);
    {
        std::lock_guard<std::mutex> lk(attr_mu);
        if (!attr_done[dev & 63]) {
            cudaFuncAttributes fa;
            if (cudaFuncGetAttributes(&fa, tc_bf16_pair_kernel) != cudaSuccess) { snprintf(t_tc_error, sizeof t_tc_error, "cudaFuncGetAttributes failed"); return B200ATTN_ERR_CUDA; }
            cudaDeviceProp prop;
            cudaGetDeviceProperties(&prop, dev);
            const size_t dyn_max = prop.sharedMemPerBlockOptin - fa.sharedSizeBytes;
            if (cudaFuncSetAttribute(tc_bf16_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn_max) != cudaSuccess) {
                snprintf(t_tc_error, sizeof t_tc_error, "cudaFuncSetAttribute(max dynamic shared memory) failed");
                return B200ATTN_ERR_CUDA;
            }
            attr_done[dev & 63] = true;
        }
    }
    TcParams p{};
    p.Lq = a.len_q; p.Lk = a.len_k; p.D = D;
    p.n_qtiles = a.len_q / TC_BM; p.n_blocks = a.len_k / TC_BN; p.n_chunks = D / 64;
    p.scale_log2 = 1.4426950408889634f / sqrtf((float)D);
    p.pe = a.pe == B200ATTN_PE_ROPE_Q_ONLY ? (int)PE_ROPE_INTERLEAVED : a.pe;
    p.rd = rd;
    p.rotate_k = (a.pe == B200ATTN_PE_ROPE_Q_ONLY) ? 0 : 1;
    p.O = (__nv_bfloat16 *)a.out;
    p.err = err_dev;
    p.err_sys = err_sys;
    p.spin_limit = spin_limit;
    p.debug_scores = debug_scores;
    p.k_stages = 2;   // two 32 KB stages measure the same as three; the third's 32 KB are the P staging
    p.k_stage_bytes = 2 * TC_CHUNK_BYTES;
    const bool has_pe = (a.pe != B200ATTN_PE_NONE);
    CUtensorMap tmQ, tmK128, tmK256, tmV, tmPE;
    if (!tc_make_map(&tmQ, a.Q, BH * a.len_q, D, TC_BM) || !tc_make_map(&tmK128, a.K, BH * a.len_k, D, 128) ||
        !tc_make_map(&tmK256, a.K, BH * a.len_k, D, 256) || !tc_make_map(&tmV, a.V, BH * a.len_k, D, TC_VS)) {
        snprintf(t_tc_error, sizeof t_tc_error, "cuTensorMapEncodeTiled failed");
        return B200ATTN_ERR_CUDA;
    }
    tmPE = tmK128;
    if (has_pe) {
        const int L = a.len_q > a.len_k ? a.len_q : a.len_k;
        int rows = 0;
        const __nv_bfloat16 *tab = tables.get(a.pe, L, D, rd, a.pe == B200ATTN_PE_SINUSOIDAL ? 10000.0f : base, st, launches, &rows);
        if (!tab) { snprintf(t_tc_error, sizeof t_tc_error, "could not allocate the positional-encoding table"); return B200ATTN_ERR_CUDA; }
        if (!tc_make_map(&tmPE, tab, rows, D, TC_BN)) { snprintf(t_tc_error, sizeof t_tc_error, "cuTensorMapEncodeTiled failed"); return B200ATTN_ERR_CUDA; }
    }
    auto launch = [&](const CUtensorMap &mK, int qt0, int n_qt) -> int {
        p.qt0 = qt0; p.n_qt = n_qt;
        const long long units = BH * n_qt;
        p.n_units = units;
        long long clusters = sm_count / 2;   // persistent: one cluster per SM pair, units dealt round-robin
        if (clusters > units) clusters = units;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)(2 * clusters));
        cfg.blockDim = dim3(TC_THREADS);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = st;
        cudaError_t e = cudaLaunchKernelEx(&cfg, tc_bf16_pair_kernel, tmQ, mK, tmV, tmPE, p);
        if (e != cudaSuccess) {
            snprintf(t_tc_error, sizeof t_tc_error, "tc_bf16_pair_kernel launch failed: %s", cudaGetErrorString(e));
            return B200ATTN_ERR_CUDA;
        }
        launches->fetch_add(1);
        return B200ATTN_OK;
    };
    const bool pe_k = has_pe && p.rotate_k;
    // Encoded-K cache.  When K carries an encoding and a head has several query tiles, the unit of
    // the head's FIRST query tile encodes K inside its K load (as every unit would) and, while the
    // encoded chunk is in registers, also writes it to a scratch copy; the units of the other query
    // tiles of that head then load the encoded K and run without the transform (second launch,
    // stream-ordered after the first).  The encoding is still applied once, inside a K load, by
    // the attention kernel itself; the scratch is as large as K.
    if (pe_k && p.n_qtiles >= 3) {
        const size_t kbytes = (size_t)BH * a.len_k * D * sizeof(__nv_bfloat16);
        __nv_bfloat16 *kc = tables.get_kcache(kbytes);
        CUtensorMap tmKc;
        if (kc != nullptr && tc_make_map(&tmKc, kc, BH * a.len_k, D, 256)) {
            p.sb_keys = 128; p.k_store = kc;
            int rc = launch(tmK128, 0, 1);
            if (rc) return rc;
            p.sb_keys = 256; p.k_store = nullptr; p.rotate_k = 0;
            return launch(tmKc, 1, p.n_qtiles - 1);
        }
    }
    p.k_store = nullptr;
    p.sb_keys = pe_k ? 128 : 256;
    return launch(pe_k ? tmK128 : tmK256, 0, p.n_qtiles);
}

}  // namespace b200attn
