// bf16 attention forward for FEW QUERIES AND MANY KEYS on the tensor cores: the decode / cross-attention
// regime (1-64 queries against a long K/V, e.g. a KV cache; named as the real workload of the fused-RoPE
// kernels in the reference's writeup.md:299-301).  The problem is bound by streaming K and V from HBM
// once, so the keys of a head are cut into splits that run on different SMs, each split keeps a running
// (max, sum, O) of its own and a second small kernel combines the splits:
//
//   dec_split_kernel    unit = (head, key split).  Q [<= 64 rows x head_d] is loaded once (M = 64 MMA rows);
//                       K and V arrive by TMA in chunks of 128 keys through two independent rings (a K stage
//                       is free again as soon as its score MMA has completed, not when the chunk's P V has);
//                       S = Q Kt (tcgen05, fp32 in tensor memory, double-buffered), one thread per query row
//                       takes the chunk maximum, writes P = exp2(S - max) as the bf16 A operand, O_c = P V
//                       (fresh accumulator per chunk, double-buffered) is folded into the row's running
//                       output in registers: O = O * 2^(m - m') + O_c * 2^(m_c - m'): no accumulator is ever
//                       rescaled in tensor memory.
//   dec_combine_kernel  out = sum_s 2^(m_s - m) O_s / sum_s 2^(m_s - m) l_s over the splits of a head.
//
// A positional encoding is applied inside the load: four transform warps encode every landed K chunk (and
// the Q tile once) in shared memory between TMA arrival and MMA, with the packed bf16 arithmetic and the
// L2-resident tables of the two-kernel path (positions: query row i -> i, key j -> j, as the reference
// kernels do, final/rope.cu:129, 307).  The *_Q_ONLY kinds take K as already rotated (b200attn_rope_k).
//
// Shapes taken here: bf16, head_d 64 or 128, len_q <= 64, any len_k > 64, 16-byte aligned tensors; rotate-half
// needs head_d 128 and rotary_dim == head_d.  Every wait is bounded.
#pragma once

#include "tc_wide.cuh"

namespace b200attn {

constexpr int DC_THREADS = 320;   // warp 0 TMA, warp 1 MMA, warps 2-5 softmax + running output, warps 6-9 transform
constexpr int DC_NK = 128;        // keys per chunk
constexpr int DC_MQ = 64;         // query rows of the MMA tile
constexpr int DC_QSLAB = DC_MQ * 128;   // [64 rows x 64 bf16]
constexpr int DC_KSLAB = DC_NK * 128;   // [128 keys x 64 bf16]
constexpr int DC_PBUF = 2 * DC_QSLAB;   // P [64 x 128 keys]: two atoms of 64 keys

struct DecParams {
    long long BH;
    int Lq, Lk, D, nch;        // nch = D / 64
    int nsplit, cps;           // key splits per head, chunks per split
    float scale_log2;          // log2(e) / sqrt(D)
    int table_kind;            // 0 none, 1 element-wise partner table (interleaved RoPE, sinusoidal), 2 rotate-half table
    int sinus, rotate_q, rotate_k;
    int f16;                   // the tensors are fp16 (no encoding then), else bf16
    const __nv_bfloat16 *tab;  // [>= max(64, 128 * ceil(Lk / 128))][D]
    float *part_O;             // [BH][nsplit][64][D] unnormalised outputs of the splits
    float *part_ml;            // [BH][nsplit][64][2] their (max in log2 units, sum)
    __nv_bfloat16 *O;          // [BH * Lq][D]; written here directly when nsplit == 1
    unsigned *err, *err_sys;
    unsigned spin_limit;
};

struct DcBars {
    uint64_t q_full, q_ready;
    uint64_t k_full[2], k_ready[2], k_free[2];
    uint64_t v_full[2], v_free[2];
    uint64_t s_full[2], p_full[2], o_full[2], o_free[2];
};

inline size_t dec_smem_bytes(int nch) { return (size_t)nch * DC_QSLAB + (size_t)4 * nch * DC_KSLAB + 2 * DC_PBUF + 1024; }

#define DC_FAIL_AT(site, cond)                                                                      \
    if (cond) {                                                                                     \
        report_kernel_error(p.err, p.err_sys, (unsigned)KERR_MBAR_TIMEOUT | (1u << (7 + (site))));  \
        failed = true;                                                                              \
        break;                                                                                      \
    }

// Encodes `rows` x (64 * nch) bf16 laid out as nch slabs [rows x 128 B] with the 128-byte swizzle, in place;
// row r has position pos0 + r.  128 threads.  The table values of eight pieces are requested before the first is
// used: with one fetch at a time a K chunk cost its transform warps eight L2 round trips in a row, more than the
// chunk's share of the HBM time.
// `landed` is called once, after the first eight fetches have been issued and before the tile is touched: the wait
// for the tile's TMA load goes there, so that the table values travel while the tile does.  Returns what it returned.
template <class Landed>
__device__ __forceinline__ bool dec_encode_tile(unsigned char *tile, int rows, int slab_bytes, int nch, int D, int pos0, int table_kind, bool sinus,
                                                const __nv_bfloat16 *tab, int tid, Landed landed) {
    const int per_slab = rows * 8;   // 16-byte pieces per slab
    constexpr int U = 8;
    bool waited = false;
    if (table_kind == 2) {
        const int half_slabs = nch >> 1, total = half_slabs * per_slab;
        for (int o0 = tid; o0 < total; o0 += 128 * U) {
            uint4 tc[U], ts[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int o = o0 + 128 * u;
                if (o < total) {
                    const int c = o / per_slab, w = o - c * per_slab, r = w >> 3, q = (w & 7) ^ (r & 7);
                    const __nv_bfloat16 *tp = tab + (long long)(pos0 + r) * D + c * 64 + q * 8;
                    tc[u] = tcw_ldg_here(tp);
                    ts[u] = tcw_ldg_here(tp + (D >> 1));
                }
            }
            if (!waited) { if (!landed()) return false; waited = true; }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int o = o0 + 128 * u;
                if (o < total) {
                    const int c = o / per_slab, w = o - c * per_slab;
                    uint4 *plo = reinterpret_cast<uint4 *>(tile + (size_t)c * slab_bytes + (size_t)w * 16);
                    uint4 *phi = reinterpret_cast<uint4 *>(tile + (size_t)(c + half_slabs) * slab_bytes + (size_t)w * 16);
                    uint4 lo = *plo, hi = *phi;
                    tcw_rotate(lo.x, hi.x, tc[u].x, ts[u].x);
                    tcw_rotate(lo.y, hi.y, tc[u].y, ts[u].y);
                    tcw_rotate(lo.z, hi.z, tc[u].z, ts[u].z);
                    tcw_rotate(lo.w, hi.w, tc[u].w, ts[u].w);
                    *plo = lo;
                    *phi = hi;
                }
            }
        }
    } else {
        const int total = nch * per_slab;
        for (int o0 = tid; o0 < total; o0 += 128 * U) {
            uint4 t[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int o = o0 + 128 * u;
                if (o < total) {
                    const int c = o / per_slab, w = o - c * per_slab, r = w >> 3, q = (w & 7) ^ (r & 7);
                    t[u] = tcw_ldg_here(tab + (long long)(pos0 + r) * D + c * 64 + q * 8);
                }
            }
            if (!waited) { if (!landed()) return false; waited = true; }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int o = o0 + 128 * u;
                if (o < total) {
                    const int c = o / per_slab, w = o - c * per_slab;
                    uint4 *px = reinterpret_cast<uint4 *>(tile + (size_t)c * slab_bytes + (size_t)w * 16);
                    uint4 v = *px;
                    v.x = tc_pe_pair(v.x, t[u].x, sinus);
                    v.y = tc_pe_pair(v.y, t[u].y, sinus);
                    v.z = tc_pe_pair(v.z, t[u].z, sinus);
                    v.w = tc_pe_pair(v.w, t[u].w, sinus);
                    *px = v;
                }
            }
        }
    }
    if (!waited) return landed();   // (an empty tile)
    return true;
}

template <int NCH>   // head_d / 64
__global__ void __launch_bounds__(DC_THREADS, 1)
dec_split_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                 const DecParams p) {
    extern __shared__ unsigned char dc_smem_raw[];
    __shared__ DcBars bars;
    __shared__ uint32_t tmem_slot;
    const uint32_t raw_addr = smem_u32(dc_smem_raw);
    unsigned char *smem = dc_smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int nch = NCH, D = 64 * NCH;
    const uint32_t lim = p.spin_limit;
    const int split = blockIdx.x;
    const long long bh = blockIdx.y;
    const int total_chunks = (p.Lk + DC_NK - 1) / DC_NK;
    const int c0 = split * p.cps, c1 = min(total_chunks, c0 + p.cps);
    const int n = c1 - c0;   // >= 1 by construction of the grid

    unsigned char *q_smem = smem;
    unsigned char *k_smem = q_smem + (size_t)nch * DC_QSLAB;          // 2 stages of nch slabs
    unsigned char *v_smem = k_smem + (size_t)2 * nch * DC_KSLAB;      // 2 stages of nch slabs
    unsigned char *p_smem = v_smem + (size_t)2 * nch * DC_KSLAB;      // 2 buffers
    const int kv_stage = nch * DC_KSLAB;

    if (threadIdx.x == 0) {
        mbar_init(&bars.q_full, 1);
        mbar_init(&bars.q_ready, 4);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&bars.k_full[i], 1); mbar_init(&bars.k_ready[i], 4); mbar_init(&bars.k_free[i], 1);
            mbar_init(&bars.v_full[i], 1); mbar_init(&bars.v_free[i], 1);
            mbar_init(&bars.s_full[i], 1); mbar_init(&bars.p_full[i], 4); mbar_init(&bars.o_full[i], 1); mbar_init(&bars.o_free[i], 4);
        }
        mbar_fence_init();
        tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
    }
    if (warp == 1) tmem_alloc(&tmem_slot, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    const uint32_t tmem_s = tmem, tmem_o = tmem + 256;   // S buffers at columns 0 / 128, output buffers at 256 / 384
    bool failed = false;
    const bool skip = (*reinterpret_cast<volatile unsigned *>(p.err) != 0);

    if (skip) {
        // fall through to the common exit
    } else if (warp == 0) {
        if (lane == 0) {
            mbar_expect_tx(&bars.q_full, (uint32_t)nch * (uint32_t)p.Lq * 128u);
            for (int c = 0; c < nch; ++c) tma_load_2d(q_smem + (size_t)c * DC_QSLAB, &tmQ, c * 64, (int)(bh * p.Lq), &bars.q_full);
            for (int t = 0; t < n; ++t) {
                const int st = t & 1;
                const int row0 = (int)(bh * p.Lk + (long long)(c0 + t) * DC_NK);
                DC_FAIL_AT(0, !mbar_wait(&bars.k_free[st], ((t >> 1) & 1) ^ 1, lim));
                mbar_expect_tx(&bars.k_full[st], (uint32_t)kv_stage);
                tma_load_3d(k_smem + (size_t)st * kv_stage, &tmK, 0, row0, 0, &bars.k_full[st]);
                DC_FAIL_AT(1, !mbar_wait(&bars.v_free[st], ((t >> 1) & 1) ^ 1, lim));
                mbar_expect_tx(&bars.v_full[st], (uint32_t)kv_stage);
                tma_load_3d(v_smem + (size_t)st * kv_stage, &tmV, 0, row0, 0, &bars.v_full[st]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t id_s = umma_idesc_16(DC_MQ, DC_NK, 0, 0, p.f16), id_o = umma_idesc_16(DC_MQ, D, 0, 1, p.f16);
            auto issue_scores = [&](int t) -> bool {
                const int st = t & 1;
                if (!mbar_wait(p.rotate_k ? &bars.k_ready[st] : &bars.k_full[st], (t >> 1) & 1, lim)) return false;
                tc_fence_after();
                for (int c = 0; c < nch; ++c) {
                    const uint64_t da = umma_desc_k_sw128(smem_u32(q_smem + (size_t)c * DC_QSLAB));
                    const uint64_t db = umma_desc_k_sw128(smem_u32(k_smem + (size_t)st * kv_stage + (size_t)c * DC_KSLAB));
#pragma unroll
                    for (int k = 0; k < 4; ++k) umma_bf16(tmem_s + st * DC_NK, da + 2 * k, db + 2 * k, id_s, (c | k) != 0);
                }
                umma_commit(&bars.k_free[st]);
                umma_commit(&bars.s_full[st]);
                return true;
            };
            do {
                DC_FAIL_AT(2, !mbar_wait(p.rotate_q ? &bars.q_ready : &bars.q_full, 0, lim));
                tc_fence_after();
                DC_FAIL_AT(3, !issue_scores(0));
                for (int t = 0; t < n; ++t) {
                    const int st = t & 1;
                    // the scores of the next chunk run under this chunk's softmax (its S buffer was read when P of chunk t-1 was published)
                    if (t + 1 < n) DC_FAIL_AT(4, !issue_scores(t + 1));
                    DC_FAIL_AT(5, !mbar_wait(&bars.p_full[st], (t >> 1) & 1, lim));
                    DC_FAIL_AT(6, !mbar_wait(&bars.v_full[st], (t >> 1) & 1, lim));
                    DC_FAIL_AT(7, !mbar_wait(&bars.o_free[st], ((t >> 1) & 1) ^ 1, lim));
                    tc_fence_after();
#pragma unroll
                    for (int kk = 0; kk < DC_NK / 16; ++kk) {
                        const uint64_t da = umma_desc_k_sw128(smem_u32(p_smem + (size_t)st * DC_PBUF + (size_t)(kk >> 2) * DC_QSLAB)) + 2 * (kk & 3);
                        const uint64_t db = umma_desc_mn_sw128(smem_u32(v_smem + (size_t)st * kv_stage + (size_t)kk * 2048), DC_KSLAB);
                        umma_bf16(tmem_o + st * 128, da, db, id_o, kk != 0);
                    }
                    umma_commit(&bars.v_free[st]);
                    umma_commit(&bars.o_full[st]);
                }
            } while (false);
        }
    } else if (warp < 6) {
        // ---- one thread per query row: row 16 q + lane sits in lane `lane` (< 16) of quadrant q = warp % 4 ----
        const int qd = warp & 3, row = 16 * qd + lane;
        const uint32_t lane_addr = ((uint32_t)(32 * qd) << 16);
        const bool active = lane < 16 && row < p.Lq;
        float m_run = -INFINITY, l_run = 0.0f, m_prev = -INFINITY, l_prev = 0.0f;
        float o_run[D];
#pragma unroll
        for (int j = 0; j < D; ++j) o_run[j] = 0.0f;
        uint32_t r[32];
        for (int t = 0; t < n && !failed; ++t) {
            const int st = t & 1;
            const int nvalid = min(DC_NK, p.Lk - (c0 + t) * DC_NK);
            DC_FAIL_AT(8, !mbar_wait(&bars.s_full[st], (t >> 1) & 1, lim));
            tc_fence_after();
            // pass 1: the chunk's row maximum
            float mx = -INFINITY;
            for (int g = 0; g < DC_NK / 32; ++g) {
                tmem_ld32(tmem_s + lane_addr + st * DC_NK + g * 32, r);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (g * 32 + j < nvalid) mx = fmaxf(mx, __uint_as_float(r[j]));
            }
            const float m_c = mx * p.scale_log2;
            // pass 2: P = exp2(S - max) as the bf16 A operand [64 rows x 128 keys], 16 keys per 32 bytes
            float l_c = 0.0f;
            unsigned char *prow = p_smem + (size_t)st * DC_PBUF + (row >> 3) * 1024 + (row & 7) * 128;
            for (int g = 0; g < DC_NK / 32; ++g) {
                tmem_ld32(tmem_s + lane_addr + st * DC_NK + g * 32, r);
                tmem_ld_wait();
                uint32_t w[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int k0 = g * 32 + 2 * j;
                    const float e0 = (k0 < nvalid) ? fast_exp2(fmaf(__uint_as_float(r[2 * j]), p.scale_log2, -m_c)) : 0.0f;
                    const float e1 = (k0 + 1 < nvalid) ? fast_exp2(fmaf(__uint_as_float(r[2 * j + 1]), p.scale_log2, -m_c)) : 0.0f;
                    l_c += e0 + e1;
                    w[j] = pack_16x2(e0, e1, p.f16 != 0);
                }
                if (lane < 16) {
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        const int piece = (g * 4 + q4) & 7, atom = (g * 4 + q4) >> 3;   // 8 keys per 16-byte piece, 8 pieces per atom row
                        *reinterpret_cast<uint4 *>(prow + (size_t)atom * DC_QSLAB + ((piece ^ (row & 7)) << 4)) =
                            make_uint4(w[4 * q4], w[4 * q4 + 1], w[4 * q4 + 2], w[4 * q4 + 3]);
                    }
                }
            }
            tc_fence_before();
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars.p_full[st]);
            // fold O_c = P V of the PREVIOUS chunk into the running output: its MMAs ran while this chunk's
            // softmax was computed, so this wait is over when it is reached
            if (t > 0) {
                const int sp = (t - 1) & 1;
                DC_FAIL_AT(9, !mbar_wait(&bars.o_full[sp], ((t - 1) >> 1) & 1, lim));
                tc_fence_after();
                const float m_new = fmaxf(m_run, m_prev);
                const float a = (m_run == -INFINITY) ? 0.0f : fast_exp2(m_run - m_new), b = fast_exp2(m_prev - m_new);
#pragma unroll
                for (int g = 0; g < D / 32; ++g) {
                    tmem_ld32(tmem_o + lane_addr + sp * 128 + g * 32, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; ++j) o_run[g * 32 + j] = fmaf(o_run[g * 32 + j], a, __uint_as_float(r[j]) * b);
                }
                l_run = fmaf(l_run, a, l_prev * b);
                m_run = m_new;
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars.o_free[sp]);
            }
            m_prev = m_c;
            l_prev = l_c;
        }
        if (!failed) {
            do {   // the last chunk
                const int sp = (n - 1) & 1;
                DC_FAIL_AT(12, !mbar_wait(&bars.o_full[sp], ((n - 1) >> 1) & 1, lim));
                tc_fence_after();
                const float m_new = fmaxf(m_run, m_prev);
                const float a = (m_run == -INFINITY) ? 0.0f : fast_exp2(m_run - m_new), b = fast_exp2(m_prev - m_new);
#pragma unroll
                for (int g = 0; g < D / 32; ++g) {
                    tmem_ld32(tmem_o + lane_addr + sp * 128 + g * 32, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; ++j) o_run[g * 32 + j] = fmaf(o_run[g * 32 + j], a, __uint_as_float(r[j]) * b);
                }
                l_run = fmaf(l_run, a, l_prev * b);
                m_run = m_new;
            } while (false);
        }
        if (!failed && active) {
            if (p.nsplit == 1) {
                const float inv = 1.0f / l_run;
                __nv_bfloat16 *orow = p.O + (bh * p.Lq + row) * (long long)D;
#pragma unroll
                for (int j = 0; j < D; j += 8) {
                    uint4 v;
                    v.x = pack_16x2(o_run[j] * inv, o_run[j + 1] * inv, p.f16 != 0);
                    v.y = pack_16x2(o_run[j + 2] * inv, o_run[j + 3] * inv, p.f16 != 0);
                    v.z = pack_16x2(o_run[j + 4] * inv, o_run[j + 5] * inv, p.f16 != 0);
                    v.w = pack_16x2(o_run[j + 6] * inv, o_run[j + 7] * inv, p.f16 != 0);
                    *reinterpret_cast<uint4 *>(orow + j) = v;
                }
            } else {
                float *po = p.part_O + ((bh * p.nsplit + split) * DC_MQ + row) * (long long)D;
#pragma unroll
                for (int j = 0; j < D; j += 4) *reinterpret_cast<float4 *>(po + j) = make_float4(o_run[j], o_run[j + 1], o_run[j + 2], o_run[j + 3]);
                float *pm = p.part_ml + ((bh * p.nsplit + split) * DC_MQ + row) * 2;
                pm[0] = m_run;
                pm[1] = l_run;
            }
        }
    } else if (p.rotate_q || p.rotate_k) {
        // ---- transform warps: the Q tile once, then every K chunk, encoded in place ----
        const int tid = threadIdx.x - 6 * 32;
        do {
            if (p.rotate_q) {
                DC_FAIL_AT(10, !dec_encode_tile(q_smem, DC_MQ, DC_QSLAB, nch, D, 0, p.table_kind, p.sinus != 0, p.tab, tid,
                                                [&]() { return mbar_wait(&bars.q_full, 0, lim); }));
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars.q_ready);
            }
            if (p.rotate_k) {
                for (int t = 0; t < n; ++t) {
                    const int st = t & 1;
                    DC_FAIL_AT(11, !dec_encode_tile(k_smem + (size_t)st * kv_stage, DC_NK, DC_KSLAB, nch, D, (c0 + t) * DC_NK, p.table_kind, p.sinus != 0, p.tab, tid,
                                                    [&]() { return mbar_wait(&bars.k_full[st], (t >> 1) & 1, lim); }));
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bars.k_ready[st]);
                }
            }
        } while (false);
    }

    if (failed) for (int i = 0; i < 2000; ++i) __nanosleep(1000);   // let copies and MMAs in flight drain
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 1) tmem_dealloc(tmem, 512);
}

// ---------------------------------------------------------------------------------------------------
// The same unit for AT MOST 32 QUERIES, transposed: St [128 keys x NQ] = K Qt and Ot [head_d x NQ] = Vt Pt
// (NQ = 16 or 32 query columns).  With the keys along the 128 tensor-memory lanes every softmax thread is
// busy (a row per query leaves 60 of 64 rows idle for 4 queries) and the work per chunk is NQ values per
// thread instead of 128.  The reference maximum of P is the RUNNING row maximum, the same for all
// threads, so each thread rescales what it holds itself: its partial row sums (one per key lane, reduced
// over the lanes once at the end of the split) and its row of the running Ot.
// ---------------------------------------------------------------------------------------------------
template <int N> __device__ __forceinline__ void dec_tmem_ld(uint32_t taddr, uint32_t (&r)[N]);
template <> __device__ __forceinline__ void dec_tmem_ld<32>(uint32_t taddr, uint32_t (&r)[32]) { tmem_ld32(taddr, r); }
template <> __device__ __forceinline__ void dec_tmem_ld<16>(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
          "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

template <int NCH, int NQ>   // head_d / 64; query columns (16 or 32)
__global__ void __launch_bounds__(DC_THREADS, 1)
dec_t_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
             const DecParams p) {
    extern __shared__ unsigned char dc_smem_raw[];
    __shared__ DcBars bars;
    __shared__ uint32_t tmem_slot;
    __shared__ float wmax[2][4][NQ];   // chunk maxima of the four softmax warps, double-buffered by chunk parity
    __shared__ float wsum[4][NQ];
    __shared__ uint64_t mx_full[2], sum_full;   // the four warps have written wmax[i] / wsum (bounded waits, like every other)
    const uint32_t raw_addr = smem_u32(dc_smem_raw);
    unsigned char *smem = dc_smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int nch = NCH, D = 64 * NCH;
    const uint32_t lim = p.spin_limit;
    const int split = blockIdx.x;
    const long long bh = blockIdx.y;
    const int total_chunks = (p.Lk + DC_NK - 1) / DC_NK;
    const int c0 = split * p.cps, c1 = min(total_chunks, c0 + p.cps);
    const int n = c1 - c0;

    unsigned char *q_smem = smem;
    unsigned char *k_smem = q_smem + (size_t)nch * DC_QSLAB;
    unsigned char *v_smem = k_smem + (size_t)2 * nch * DC_KSLAB;
    unsigned char *p_smem = v_smem + (size_t)2 * nch * DC_KSLAB;
    constexpr int kv_stage = nch * DC_KSLAB;

    if (threadIdx.x == 0) {
        mbar_init(&bars.q_full, 1);
        mbar_init(&bars.q_ready, 4);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&bars.k_full[i], 1); mbar_init(&bars.k_ready[i], 4); mbar_init(&bars.k_free[i], 1);
            mbar_init(&bars.v_full[i], 1); mbar_init(&bars.v_free[i], 1);
            mbar_init(&bars.s_full[i], 1); mbar_init(&bars.p_full[i], 4); mbar_init(&bars.o_full[i], 1); mbar_init(&bars.o_free[i], 4);
        }
        mbar_init(&mx_full[0], 4); mbar_init(&mx_full[1], 4); mbar_init(&sum_full, 4);
        mbar_fence_init();
        tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
    }
    if (warp == 1) tmem_alloc(&tmem_slot, 256);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    const uint32_t tmem_s = tmem, tmem_o = tmem + 128;   // St buffers at columns 0 / 64, Ot buffers at 128 / 192
    bool failed = false;
    const bool skip = (*reinterpret_cast<volatile unsigned *>(p.err) != 0);

    if (skip) {
        // fall through to the common exit
    } else if (warp == 0) {
        if (lane == 0) {
            mbar_expect_tx(&bars.q_full, (uint32_t)nch * (uint32_t)p.Lq * 128u);
            for (int c = 0; c < nch; ++c) tma_load_2d(q_smem + (size_t)c * DC_QSLAB, &tmQ, c * 64, (int)(bh * p.Lq), &bars.q_full);
            for (int t = 0; t < n; ++t) {
                const int st = t & 1;
                const int row0 = (int)(bh * p.Lk + (long long)(c0 + t) * DC_NK);
                DC_FAIL_AT(0, !mbar_wait(&bars.k_free[st], ((t >> 1) & 1) ^ 1, lim));
                mbar_expect_tx(&bars.k_full[st], (uint32_t)kv_stage);
                tma_load_3d(k_smem + (size_t)st * kv_stage, &tmK, 0, row0, 0, &bars.k_full[st]);
                DC_FAIL_AT(1, !mbar_wait(&bars.v_free[st], ((t >> 1) & 1) ^ 1, lim));
                mbar_expect_tx(&bars.v_full[st], (uint32_t)kv_stage);
                tma_load_3d(v_smem + (size_t)st * kv_stage, &tmV, 0, row0, 0, &bars.v_full[st]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t id_s = umma_idesc_16(DC_NK, NQ, 0, 0, p.f16), id_o = umma_idesc_16(D, NQ, 1, 0, p.f16);
            auto issue_scores = [&](int t) -> bool {
                const int st = t & 1;
                if (!mbar_wait(p.rotate_k ? &bars.k_ready[st] : &bars.k_full[st], (t >> 1) & 1, lim)) return false;
                tc_fence_after();
                for (int c = 0; c < nch; ++c) {
                    const uint64_t da = umma_desc_k_sw128(smem_u32(k_smem + (size_t)st * kv_stage + (size_t)c * DC_KSLAB));
                    const uint64_t db = umma_desc_k_sw128(smem_u32(q_smem + (size_t)c * DC_QSLAB));
#pragma unroll
                    for (int k = 0; k < 4; ++k) umma_bf16(tmem_s + st * 64, da + 2 * k, db + 2 * k, id_s, (c | k) != 0);
                }
                umma_commit(&bars.k_free[st]);
                umma_commit(&bars.s_full[st]);
                return true;
            };
            do {
                DC_FAIL_AT(2, !mbar_wait(p.rotate_q ? &bars.q_ready : &bars.q_full, 0, lim));
                tc_fence_after();
                DC_FAIL_AT(3, !issue_scores(0));
                for (int t = 0; t < n; ++t) {
                    const int st = t & 1;
                    if (t + 1 < n) DC_FAIL_AT(4, !issue_scores(t + 1));
                    DC_FAIL_AT(5, !mbar_wait(&bars.p_full[st], (t >> 1) & 1, lim));
                    DC_FAIL_AT(6, !mbar_wait(&bars.v_full[st], (t >> 1) & 1, lim));
                    DC_FAIL_AT(7, !mbar_wait(&bars.o_free[st], ((t >> 1) & 1) ^ 1, lim));
                    tc_fence_after();
#pragma unroll
                    for (int kk = 0; kk < DC_NK / 16; ++kk) {
                        const uint64_t da = umma_desc_mn_sw128(smem_u32(v_smem + (size_t)st * kv_stage + (size_t)kk * 2048), DC_KSLAB);
                        const uint64_t db = umma_desc_k_sw128(smem_u32(p_smem + (size_t)st * DC_PBUF + (size_t)(kk >> 2) * DC_QSLAB)) + 2 * (kk & 3);
                        umma_bf16(tmem_o + st * 64, da, db, id_o, kk != 0);
                    }
                    umma_commit(&bars.v_free[st]);
                    umma_commit(&bars.o_full[st]);
                }
            } while (false);
        }
    } else if (warp < 6) {
        // ---- key lane j = 32 (warp % 4) + lane of every chunk; the same thread owns row d of Ot (head_d 128:
        // d = j; head_d 64, an M = 64 accumulator: d = 16 (warp % 4) + lane for lane < 16) ----
        const int qd = warp & 3, j = 32 * qd + lane;
        const uint32_t lane_addr = ((uint32_t)(32 * qd) << 16);
        const int drow = (D == 128) ? j : 16 * qd + lane;
        const bool d_active = (D == 128) || lane < 16;
        float m_run[NQ], l_part[NQ], o_run[NQ];
#pragma unroll
        for (int q = 0; q < NQ; ++q) { m_run[q] = -INFINITY; l_part[q] = 0.0f; o_run[q] = 0.0f; }
        uint32_t r[NQ];
        for (int t = 0; t < n && !failed; ++t) {
            const int st = t & 1;
            const bool valid = (c0 + t) * DC_NK + j < p.Lk;
            DC_FAIL_AT(8, !mbar_wait(&bars.s_full[st], (t >> 1) & 1, lim));
            tc_fence_after();
            dec_tmem_ld<NQ>(tmem_s + lane_addr + st * 64, r);
            tmem_ld_wait();
            float sv[NQ], mx[NQ];
#pragma unroll
            for (int q = 0; q < NQ; ++q) { sv[q] = valid ? __uint_as_float(r[q]) * p.scale_log2 : -INFINITY; mx[q] = sv[q]; }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1)
#pragma unroll
                for (int q = 0; q < NQ; ++q) mx[q] = fmaxf(mx[q], __shfl_xor_sync(0xffffffffu, mx[q], o));
            if (lane < NQ) {   // lane q publishes the warp's maximum of query q
                float v = mx[0];
#pragma unroll
                for (int q = 1; q < NQ; ++q) v = (lane == q) ? mx[q] : v;
                wmax[t & 1][qd][lane] = v;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&mx_full[t & 1]);
            DC_FAIL_AT(13, !mbar_wait(&mx_full[t & 1], (t >> 1) & 1, lim));
            // new running maxima (the same in every thread), factors for what is held relative to the old ones
            float alpha[NQ];
            unsigned char *pbase = p_smem + (size_t)st * DC_PBUF + (size_t)(j >> 6) * DC_QSLAB + (j & 7) * 2;
            const int piece = (j & 63) >> 3;
#pragma unroll
            for (int q = 0; q < NQ; ++q) {
                const float mc = fmaxf(fmaxf(wmax[t & 1][0][q], wmax[t & 1][1][q]), fmaxf(wmax[t & 1][2][q], wmax[t & 1][3][q]));
                const float mn = fmaxf(m_run[q], mc);
                alpha[q] = (m_run[q] == -INFINITY) ? 0.0f : fast_exp2(m_run[q] - mn);
                m_run[q] = mn;
                const float e = valid ? fast_exp2(sv[q] - mn) : 0.0f;
                l_part[q] = fmaf(l_part[q], alpha[q], e);
                // Pt as the K-major B operand [NQ rows x 128 keys]: row q, key j
                *reinterpret_cast<uint16_t *>(pbase + (q >> 3) * 1024 + (q & 7) * 128 + ((piece ^ (q & 7)) << 4)) = pack_16(e, p.f16 != 0);
            }
            tc_fence_before();
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars.p_full[st]);
            // Ot of the previous chunk was computed relative to the maxima before this update
            if (t > 0) {
                const int sp = (t - 1) & 1;
                DC_FAIL_AT(9, !mbar_wait(&bars.o_full[sp], ((t - 1) >> 1) & 1, lim));
                tc_fence_after();
                dec_tmem_ld<NQ>(tmem_o + lane_addr + sp * 64, r);
                tmem_ld_wait();
#pragma unroll
                for (int q = 0; q < NQ; ++q) o_run[q] = (o_run[q] + __uint_as_float(r[q])) * alpha[q];
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars.o_free[sp]);
            } else {
#pragma unroll
                for (int q = 0; q < NQ; ++q) o_run[q] *= alpha[q];
            }
        }
        if (!failed) {
            do {
                const int sp = (n - 1) & 1;
                DC_FAIL_AT(12, !mbar_wait(&bars.o_full[sp], ((n - 1) >> 1) & 1, lim));
                tc_fence_after();
                dec_tmem_ld<NQ>(tmem_o + lane_addr + sp * 64, r);
                tmem_ld_wait();
#pragma unroll
                for (int q = 0; q < NQ; ++q) o_run[q] += __uint_as_float(r[q]);
                // row sums: over the 32 lanes, then over the four warps
#pragma unroll
                for (int o = 16; o > 0; o >>= 1)
#pragma unroll
                    for (int q = 0; q < NQ; ++q) l_part[q] += __shfl_xor_sync(0xffffffffu, l_part[q], o);
                if (lane < NQ) {
                    float v = l_part[0];
#pragma unroll
                    for (int q = 1; q < NQ; ++q) v = (lane == q) ? l_part[q] : v;
                    wsum[qd][lane] = v;
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&sum_full);
                DC_FAIL_AT(14, !mbar_wait(&sum_full, 0, lim));
                if (d_active) {
#pragma unroll
                    for (int q = 0; q < NQ; ++q) {
                        if (q >= p.Lq) break;
                        const float l = (wsum[0][q] + wsum[1][q]) + (wsum[2][q] + wsum[3][q]);
                        if (p.nsplit == 1) {
                            reinterpret_cast<uint16_t *>(p.O)[(bh * p.Lq + q) * (long long)D + drow] = pack_16(o_run[q] / l, p.f16 != 0);
                        } else {
                            p.part_O[((bh * p.nsplit + split) * DC_MQ + q) * (long long)D + drow] = o_run[q];
                            if (drow == 0) {
                                float *pm = p.part_ml + ((bh * p.nsplit + split) * DC_MQ + q) * 2;
                                pm[0] = m_run[q];
                                pm[1] = l;
                            }
                        }
                    }
                }
            } while (false);
        }
    } else if (p.rotate_q || p.rotate_k) {
        const int tid = threadIdx.x - 6 * 32;
        do {
            if (p.rotate_q) {
                DC_FAIL_AT(10, !dec_encode_tile(q_smem, DC_MQ, DC_QSLAB, nch, D, 0, p.table_kind, p.sinus != 0, p.tab, tid,
                                                [&]() { return mbar_wait(&bars.q_full, 0, lim); }));
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars.q_ready);
            }
            if (p.rotate_k) {
                for (int t = 0; t < n; ++t) {
                    const int st = t & 1;
                    DC_FAIL_AT(11, !dec_encode_tile(k_smem + (size_t)st * kv_stage, DC_NK, DC_KSLAB, nch, D, (c0 + t) * DC_NK, p.table_kind, p.sinus != 0, p.tab, tid,
                                                    [&]() { return mbar_wait(&bars.k_full[st], (t >> 1) & 1, lim); }));
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bars.k_ready[st]);
                }
            }
        } while (false);
    }

    if (failed) for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 1) tmem_dealloc(tmem, 256);
}
#undef DC_FAIL_AT

// out[bh][i][:] from the splits' (max, sum, O): grid (Lq, BH), one thread per output column pair.
__global__ void dec_combine_kernel(const DecParams p) {
    const int i = blockIdx.x;
    const long long bh = blockIdx.y;
    const float *ml = p.part_ml + (bh * p.nsplit * DC_MQ + i) * 2;
    float m = -INFINITY;
    for (int s = 0; s < p.nsplit; ++s) m = fmaxf(m, ml[(long long)s * DC_MQ * 2]);
    float l = 0.0f;
    for (int s = 0; s < p.nsplit; ++s) l += fast_exp2(ml[(long long)s * DC_MQ * 2] - m) * ml[(long long)s * DC_MQ * 2 + 1];
    const float inv = 1.0f / l;
    for (int d = 2 * threadIdx.x; d < p.D; d += 2 * blockDim.x) {
        float o0 = 0.0f, o1 = 0.0f;
        for (int s = 0; s < p.nsplit; ++s) {
            const float w = fast_exp2(ml[(long long)s * DC_MQ * 2] - m);
            const float2 v = *reinterpret_cast<const float2 *>(p.part_O + ((bh * p.nsplit + s) * DC_MQ + i) * (long long)p.D + d);
            o0 = fmaf(w, v.x, o0);
            o1 = fmaf(w, v.y, o1);
        }
        *reinterpret_cast<uint32_t *>(p.O + (bh * p.Lq + i) * (long long)p.D + d) = pack_16x2(o0 * inv, o1 * inv, p.f16 != 0);
    }
}

template <typename Kern>
inline bool dec_set_smem(Kern kern, size_t optin) {
    cudaFuncAttributes fa;
    return cudaFuncGetAttributes(&fa, kern) == cudaSuccess &&
           cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(optin - fa.sharedSizeBytes)) == cudaSuccess;
}

inline bool dec_supported(const b200attn_args &a, int rd) {
    if (a.dtype != B200ATTN_BF16 && !(a.dtype == B200ATTN_F16 && a.pe == B200ATTN_PE_NONE)) return false;   // the encodings are bf16 arithmetic
    if (a.head_d != 64 && a.head_d != 128) return false;
    if (a.len_q > DC_MQ || a.len_k <= 64) return false;   // short K runs on the split-head_d kernels
    if (a.cos_cache != nullptr && !pe_is_rope(a.pe)) return false;
    if (pe_pairs_halves(a.pe) && (rd != a.head_d || a.head_d != 128)) return false;   // the partner column lies 64 columns (one slab) away
    if (pe_is_rope(a.pe) && !pe_pairs_halves(a.pe) && rd % 2 != 0) return false;
    if ((((uintptr_t)a.Q | (uintptr_t)a.K | (uintptr_t)a.V | (uintptr_t)a.out) & 15) != 0) return false;
    const long long BH = (long long)a.batch_sz * a.num_heads;
    if (BH * ((long long)a.len_k + DC_NK) >= (1ll << 31) || BH > 65535) return false;
    return true;
}

// Returns B200ATTN_OK, -1 when the shape should run on another path (also when scratch could not be
// allocated: nothing has been launched then), or a status with tc_bf16_error() set.
inline int dec_run(const b200attn_args &a, int rd, float base, TcwScratch &sc, TcTables &tables, unsigned *err_dev, unsigned *err_sys, int sm_count,
                   unsigned spin_limit, cudaStream_t st, std::atomic<unsigned long long> *launches) {
    const long long BH = (long long)a.batch_sz * a.num_heads;
    const int D = a.head_d, Lq = a.len_q, Lk = a.len_k, nch = D / 64;
    static std::mutex attr_mu;
    static bool attr_done[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    {
        std::lock_guard<std::mutex> lk(attr_mu);
        if (!attr_done[dev & 63]) {
            cudaFuncAttributes fa;
            cudaDeviceProp prop;
            cudaGetDeviceProperties(&prop, dev);
            if (cudaFuncGetAttributes(&fa, dec_split_kernel<1>) != cudaSuccess ||
                cudaFuncSetAttribute(dec_split_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(prop.sharedMemPerBlockOptin - fa.sharedSizeBytes)) != cudaSuccess ||
                cudaFuncGetAttributes(&fa, dec_split_kernel<2>) != cudaSuccess ||
                cudaFuncSetAttribute(dec_split_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(prop.sharedMemPerBlockOptin - fa.sharedSizeBytes)) != cudaSuccess ||
                !dec_set_smem(dec_t_kernel<1, 16>, prop.sharedMemPerBlockOptin) || !dec_set_smem(dec_t_kernel<1, 32>, prop.sharedMemPerBlockOptin) ||
                !dec_set_smem(dec_t_kernel<2, 16>, prop.sharedMemPerBlockOptin) || !dec_set_smem(dec_t_kernel<2, 32>, prop.sharedMemPerBlockOptin)) {
                (void)cudaGetLastError();
                snprintf(t_tc_error, sizeof t_tc_error, "cudaFuncSetAttribute(max dynamic shared memory) failed");
                return B200ATTN_ERR_CUDA;
            }
            attr_done[dev & 63] = true;
        }
    }
    DecParams p{};
    p.BH = BH; p.Lq = Lq; p.Lk = Lk; p.D = D; p.nch = nch;
    const int total_chunks = (Lk + DC_NK - 1) / DC_NK;
    // splits: fill the SMs, but give a split at least two chunks of work
    int nsplit = (int)(sm_count / BH);
    if (nsplit > (total_chunks + 1) / 2) nsplit = (total_chunks + 1) / 2;
    if (nsplit < 1) nsplit = 1;
    p.cps = (total_chunks + nsplit - 1) / nsplit;
    p.nsplit = (total_chunks + p.cps - 1) / p.cps;   // no empty split
    p.scale_log2 = 1.4426950408889634f / sqrtf((float)D);
    p.rotate_q = a.pe != B200ATTN_PE_NONE ? 1 : 0;
    p.rotate_k = pe_encodes_k(a.pe) ? 1 : 0;
    p.sinus = a.pe == B200ATTN_PE_SINUSOIDAL ? 1 : 0;
    p.f16 = a.dtype == B200ATTN_F16 ? 1 : 0;
    p.table_kind = a.pe == B200ATTN_PE_NONE ? 0 : pe_pairs_halves(a.pe) ? 2 : 1;
    if (p.table_kind != 0) {
        const int Lt = total_chunks * DC_NK > DC_MQ ? total_chunks * DC_NK : DC_MQ;
        __nv_bfloat16 *tab = nullptr;
        if (a.cos_cache != nullptr) {
            tab = (__nv_bfloat16 *)sc.get(5, (size_t)Lt * D * 2);
            if (!tab) { snprintf(t_tc_error, sizeof t_tc_error, "could not allocate the cos/sin table"); return -1; }
            tcw_table_from_cache<<<296, 256, 0, st>>>(tab, Lt, D, rd, p.table_kind == 2 ? 1 : 0, Lq > Lk ? Lq : Lk, a.cos_cache, a.sin_cache);
            launches->fetch_add(1);
        } else if (p.table_kind == 2) {
            tab = tcw_half_table(sc, Lt, D, base, st, launches);
            if (!tab) { snprintf(t_tc_error, sizeof t_tc_error, "could not allocate the cos/sin table"); return -1; }
        } else {
            int rows = 0;
            tab = tables.get(a.pe, Lt, D, rd, a.pe == B200ATTN_PE_SINUSOIDAL ? 10000.0f : base, st, launches, &rows);
            if (!tab) { snprintf(t_tc_error, sizeof t_tc_error, "could not allocate the positional-encoding table"); return -1; }
        }
        p.tab = tab;
    }
    if (p.nsplit > 1) {
        p.part_O = (float *)sc.get(6, (size_t)BH * p.nsplit * DC_MQ * D * sizeof(float));
        p.part_ml = (float *)sc.get(7, (size_t)BH * p.nsplit * DC_MQ * 2 * sizeof(float));
        if (!p.part_O || !p.part_ml) { snprintf(t_tc_error, sizeof t_tc_error, "could not allocate the split scratch"); return -1; }
    }
    p.O = (__nv_bfloat16 *)a.out;
    p.err = err_dev; p.err_sys = err_sys; p.spin_limit = spin_limit;
    CUtensorMap tmQ, tmK, tmV;
    if (!tc_make_map(&tmQ, a.Q, BH * Lq, D, Lq) || !make_tmap_grouped(&tmK, a.K, BH * Lk, D, DC_NK, nch) ||
        !make_tmap_grouped(&tmV, a.V, BH * Lk, D, DC_NK, nch)) {
        snprintf(t_tc_error, sizeof t_tc_error, "cuTensorMapEncodeTiled failed");
        return B200ATTN_ERR_CUDA;
    }
    const dim3 grid((unsigned)p.nsplit, (unsigned)BH);
    const size_t smem = dec_smem_bytes(nch);
    // up to 32 queries: the transposed kernel (keys along the tensor-memory lanes); more: a row per query
    if (Lq <= 16) { if (nch == 1) dec_t_kernel<1, 16><<<grid, DC_THREADS, smem, st>>>(tmQ, tmK, tmV, p); else dec_t_kernel<2, 16><<<grid, DC_THREADS, smem, st>>>(tmQ, tmK, tmV, p); }
    else if (Lq <= 32) { if (nch == 1) dec_t_kernel<1, 32><<<grid, DC_THREADS, smem, st>>>(tmQ, tmK, tmV, p); else dec_t_kernel<2, 32><<<grid, DC_THREADS, smem, st>>>(tmQ, tmK, tmV, p); }
    else if (nch == 1) dec_split_kernel<1><<<grid, DC_THREADS, smem, st>>>(tmQ, tmK, tmV, p);
    else dec_split_kernel<2><<<grid, DC_THREADS, smem, st>>>(tmQ, tmK, tmV, p);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { snprintf(t_tc_error, sizeof t_tc_error, "dec_split_kernel launch failed: %s", cudaGetErrorString(e)); return B200ATTN_ERR_CUDA; }
    launches->fetch_add(1);
    if (p.nsplit > 1) {
        dec_combine_kernel<<<dim3((unsigned)Lq, (unsigned)BH), 64, 0, st>>>(p);
        e = cudaGetLastError();
        if (e != cudaSuccess) { snprintf(t_tc_error, sizeof t_tc_error, "dec_combine_kernel launch failed: %s", cudaGetErrorString(e)); return B200ATTN_ERR_CUDA; }
        launches->fetch_add(1);
    }
    return B200ATTN_OK;
}

}  // namespace b200attn
