// bf16 / fp16 attention forward for narrow heads (head_d 64, 128 or 256) as ONE kernel on the 5th-generation tensor
// cores: the scores never leave the SM.  (At these widths the two-kernel path of tc_wide.cuh is bound by the
// HBM round trip of its score scratch, whose bytes per FLOP grow as 1 / head_d.)  Same mathematics as the
// reference's bf16 forward, kernels/attention_bf16_optimized_fused.cu:493-505: softmax(Q K^T / sqrt(d)) V with
// fp32 scores, fp32 softmax statistics and fp32 accumulation.
//
// Both kernels are persistent and warp-specialised: one thread requests Q, K and V tiles by TMA through a ring of
// shared-memory stages in exactly the order the MMAs consume them; one thread per query tile issues the tcgen05
// MMAs; warpgroups of 128 threads - a thread per query row, which is a lane of tensor memory - do the online
// softmax and, at the end of a unit, the epilogue O / row sum -> 16 bit -> global.  Score tiles and output
// accumulators live in tensor memory (512 columns: the budget that shapes both layouts).
//   fa_kernel     head_d 64 / 128: units of (head, 256 query rows) = two query tiles, P through shared memory;
//   fa256_kernel  head_d 256: units of (head, 128 query rows), two score buffers, P through tensor memory.
// The ring position (stage, parity) of the loading and issuing threads is kept incrementally: a division by the
// run-time stage count cost such a thread some 400 clocks per wait and, at head_d 256, a sixth of the throughput.
//
// Sequence lengths of any size: the tensor maps have the head as a coordinate of their own, so that rows beyond a
// sequence read as zero; the columns of keys that do not exist are set to -inf before the softmax; output rows
// that do not exist are not stored.  Every wait is bounded; a wait that expires sets the error word.
#pragma once

#include "tc_bf16.cuh"
#include "rope_k.cuh"

namespace b200attn {

constexpr int FA_BM = 128;          // query rows per tile (two tiles per unit)
constexpr int FA_BN = 128;          // keys per tile
constexpr int FA_MAX_STAGES = 8;
constexpr float FA_RESCALE_LOG2 = 8.0f;   // the accumulator is rescaled when a row maximum grows by more than this (log2 units)

struct FaParams {
    int Lq, Lk, D;
    int nqp;                   // pairs of query tiles per head: ceil(ceil(Lq / 128) / 2)
    int nkt;                   // key tiles: ceil(Lk / 128)
    int nst;                   // ring stages (fa_kernel: [128 keys x head_d] each; fa256_kernel: 32 KB each)
    long long n_units;         // heads * nqp
    float scale_log2;          // log2(e) / sqrt(head_d)
    int f16;                   // the tensors are fp16, else bf16
    __nv_bfloat16 *O;          // [heads * Lq][D] (16-bit elements of the call's format)
    unsigned *err, *err_sys;
    unsigned spin_limit;
};

struct FaBars {   // fa256_kernel
    uint64_t kv_full[FA_MAX_STAGES], kv_empty[FA_MAX_STAGES];
    uint64_t q_full, q_empty;
    uint64_t s_full[2];        // S_t has been computed
    uint64_t p_full[2];        // P_t has been written (and O_t rescaled where needed)
    uint64_t o_done[2];        // the P V MMAs of tile t issued so far have completed
    uint64_t o_empty[2];       // the epilogue has read O_t
};

// D[tmem] (+)= A[tmem] * B[smem]: A [128 rows x 16] of 16-bit elements, a row per lane, two elements per 32-bit column
__device__ __forceinline__ void umma_16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
        "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

#define FA_FAIL_AT(site, cond)                                                                      \
    if (cond) {                                                                                     \
        report_kernel_error(p.err, p.err_sys, (unsigned)KERR_MBAR_TIMEOUT | (1u << (7 + (site))));  \
        failed = true;                                                                              \
        break;                                                                                      \
    }

// ---------------------------------------------------------------------------------------------------
// head_d 64 / 128: two query tiles of 128 rows per unit, one MMA-issuing thread and one softmax warpgroup per tile.
// Per key tile of 128 keys and query tile t:
//   - the issuer writes S_t = Q_t K_j^T (fp32, 128 columns of tensor memory) and commits to s_full;
//   - a softmax thread (one per query row) takes its whole score row into registers and says so (s_read): the
//     score MMAs of key tile j + 1 start then, under the softmax of tile j - the score tile is never the reason a
//     warpgroup waits;
//   - P = exp2(S * scale - reference) goes, as 16-bit values, to a shared-memory tile of its own (K-major, 128-byte
//     swizzle: what the MMA reads as its A operand) in two halves of 64 keys, handed over separately (p_half,
//     p_full), so that the first half of O_t += P V_j runs under the second half of the softmax;
//   - the accumulator O_t [128 x head_d] fp32 stays in tensor memory; it is only rescaled when a row's maximum has
//     grown by more than 2^8 since the reference maximum was set (the row sum carries the same reference, so the
//     result is exact; P stays far inside the 16-bit range): after the first tiles that almost never happens.
//   issuer t:  S_t = Q_t K_0^T | [s_read] S_t = Q_t K_j+1^T, [p_half] O_t += P_t[:, :64] V_j[:64], [p_full] O_t += P_t[:, 64:] V_j[64:] | ...
// Why this shape (measured on B200, B*H = 64, len 4096, head_d 128; TFLOP/s):
//   P written over its own score tile in tensor memory and read from there by the MMA, one issuer      860
//     (per key tile the chain softmax -> P V -> Q K^T -> softmax is serial for each query tile)
//   the same with an issuer per query tile                                                              790
//   key tiles of 64 keys, two score buffers per query tile, P in tensor memory; one / two issuers   630 / 800
//     (an MMA of N = 64 costs an issuing thread as much as one of N = 128: 100 to 140 clocks)
//   this layout, 352 threads, 168 registers per thread                                                 1020
//   ... with the softmax warpgroups taking over registers of warpgroup 0 (setmaxnreg, no spills)         1110
//   ... with a quarter / half of the exponentials as a cubic on the FMA pipe instead of ex2      1060 / 940
//   ... with a P buffer of 64 keys only (second half held in registers) and a fourth K / V stage         960
//   ... with ring stage and parity kept incrementally (a 64-bit division cost each wait ~400 clocks)    1150
//   ... with a non-suspending look before every barrier wait, and one wait per key tile for the P buffer   1200 - 1230
struct FaPairBars {
    uint64_t kv_full[FA_MAX_STAGES], kv_empty[FA_MAX_STAGES];   // kv_empty: one arrival per issuer
    uint64_t q_full, q_empty;                                   // q_empty: one arrival per issuer
    uint64_t s_full[2], s_read[2];      // per query tile: scores are there / are in the softmax threads' registers
    uint64_t p_half[2], p_full[2];      // the first / second 64 keys of P are in shared memory
    uint64_t o_done[2];                 // the MMAs over P (both halves) have completed
    uint64_t o_empty[2];
};
constexpr int FA_THREADS = 384;      // warpgroup 0: warp 0 loads, warps 1 and 2 issue the MMAs of query tile 0 / 1 (warp 3 idles); warpgroups 1, 2: softmax of tile 0 / 1
constexpr int FA_REGS_SMALL = 80, FA_REGS_LARGE = 208;   // registers per thread after the hand-over: 128 * 80 + 256 * 208 <= 384 * 168
constexpr uint32_t FA_P_BYTES = 128u * 128u * 2u;   // a P tile: [2 groups of 64 keys][128 rows][128 B]

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

template <bool F16>
__global__ void __launch_bounds__(FA_THREADS, 1)
fa_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, const FaParams p) {
    extern __shared__ unsigned char fa_smem_raw[];
    __shared__ FaPairBars bars;
    __shared__ uint32_t tmem_slot;
    const uint32_t raw_addr = smem_u32(fa_smem_raw);
    unsigned char *smem = fa_smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int D = p.D, nkt = p.nkt, nst = p.nst;
    const int ng = D >> 6;
    const uint32_t tile_bytes = (uint32_t)FA_BN * (uint32_t)D * 2u;   // a Q, K or V tile: [ng groups][128 rows][128 B]
    unsigned char *q_smem = smem;                                      // two Q tiles
    unsigned char *p_smem = smem + 2 * (size_t)tile_bytes;             // two P tiles
    unsigned char *ring = p_smem + 2 * (size_t)FA_P_BYTES;
    const uint32_t lim = p.spin_limit;

    if (threadIdx.x == 0) {
        for (int i = 0; i < FA_MAX_STAGES; ++i) { mbar_init(&bars.kv_full[i], 1); mbar_init(&bars.kv_empty[i], 2); }
        mbar_init(&bars.q_full, 1);
        mbar_init(&bars.q_empty, 2);
        for (int t = 0; t < 2; ++t) {
            mbar_init(&bars.s_full[t], 1); mbar_init(&bars.s_read[t], 4);
            mbar_init(&bars.p_half[t], 4); mbar_init(&bars.p_full[t], 4);
            mbar_init(&bars.o_done[t], 1);
            mbar_init(&bars.o_empty[t], 4);
        }
        mbar_fence_init();
        tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
    }
    if (warp == 0) tmem_alloc(&tmem_slot, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;        // S_t: columns [128 t, 128 t + 128); O_t: [256 + 128 t, ...)
    bool failed = false;
    const bool skip = (*reinterpret_cast<volatile unsigned *>(p.err) != 0);   // an earlier kernel of the call failed

    // the softmax threads hold a whole score row: they take over registers that the loading and issuing warps do not need
    // (each branch opens with its setmaxnreg, so that the compiler budgets the branch accordingly)
    if (skip) {
        // fall through to the common exit
    } else if (warp < 4) {
      asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(FA_REGS_SMALL));
      if (warp == 0) {
        if (lane == 0) {
            int s = 0;            // ring stage and the parity of its use (kept by hand: a division here costs the thread hundreds of clocks)
            uint32_t ph = 0;
            int ui = 0;
            bool ok = true;
            TC_PROF_DECL;
            auto load_kv = [&](const CUtensorMap *tm, int bh, int j) {
                TC_PROF(1);
                ok = ok && mbar_wait(&bars.kv_empty[s], ph ^ 1u, lim);
                TC_PROF(0);
                if (!ok) return;
                mbar_expect_tx(&bars.kv_full[s], tile_bytes);
                tma_load_4d(ring + (size_t)s * tile_bytes, tm, 0, j * FA_BN, 0, bh, &bars.kv_full[s]);
                if (++s == nst) { s = 0; ph ^= 1u; }
            };
            for (long long unit = blockIdx.x; unit < p.n_units && ok; unit += gridDim.x, ++ui) {
                const int bh = (int)(unit / p.nqp), qp = (int)(unit % p.nqp);
                ok = mbar_wait(&bars.q_empty, (uint32_t)(ui & 1) ^ 1u, lim);
                if (!ok) break;
                mbar_expect_tx(&bars.q_full, 2 * tile_bytes);
                tma_load_4d(q_smem, &tmQ, 0, qp * 2 * FA_BM, 0, bh, &bars.q_full);
                tma_load_4d(q_smem + tile_bytes, &tmQ, 0, qp * 2 * FA_BM + FA_BM, 0, bh, &bars.q_full);
                load_kv(&tmK, bh, 0);                     // the order of the issuers: K_0 | K_1, V_0 | K_2, V_1 | ...
                for (int j = 0; j < nkt && ok; ++j) {
                    if (j + 1 < nkt) load_kv(&tmK, bh, j + 1);
                    load_kv(&tmV, bh, j);
                }
            }
            if (!ok) { report_kernel_error(p.err, p.err_sys, (unsigned)KERR_MBAR_TIMEOUT | (1u << 7)); failed = true; }
            TC_PROF_FLUSH(8, true);
        }
      } else if (warp < 3) {
        if (lane == 0) {
            const int t = warp - 1;
            const uint32_t id_qk = umma_idesc_16(FA_BM, FA_BN, 0, 0, F16 ? 1 : 0), id_pv = umma_idesc_16(FA_BM, D, 0, 1, F16 ? 1 : 0);
            const uint32_t qa = smem_u32(q_smem + (size_t)t * tile_bytes), pa = smem_u32(p_smem + (size_t)t * FA_P_BYTES);
            const uint32_t t_s = tmem + t * 128, t_o = tmem + 256 + t * 128;
            int s = 0;             // ring stage and the parity of its use
            uint32_t ph = 0;
            uint32_t sc = 0;       // key tiles done so far: phase of the hand-offs with the softmax warps
            int ui = 0, lu = 0;    // units; units in which this query tile has rows (phase of o_empty)
            bool ok = true;
            TC_PROF_DECL;
            auto qk = [&](bool last) {   // S_t = Q_t K^T with the K tile at the ring position; then this issuer is done with the tile
                ok = ok && mbar_wait(&bars.kv_full[s], ph, lim);
                if (!ok) return;
                tc_fence_after();
                TC_PROF(1);
                const uint32_t ka = smem_u32(ring + (size_t)s * tile_bytes);
                for (int g = 0; g < ng; ++g) {
                    const uint64_t dq = umma_desc_k_sw128(qa + g * (FA_BM * 128)), dk = umma_desc_k_sw128(ka + g * (FA_BN * 128));
#pragma unroll
                    for (int k = 0; k < 4; ++k) umma_bf16(t_s, dq + 2 * k, dk + 2 * k, id_qk, (g | k) != 0);
                }
                umma_commit(&bars.s_full[t]);
                umma_commit(&bars.kv_empty[s]);
                if (last) umma_commit(&bars.q_empty);   // this issuer's last MMA of the unit that reads Q
                if (++s == nst) { s = 0; ph ^= 1u; }
                TC_PROF(2);
            };
            for (long long unit = blockIdx.x; unit < p.n_units && ok; unit += gridDim.x, ++ui) {
                ok = mbar_wait(&bars.q_full, (uint32_t)(ui & 1), lim);
                if (!ok) break;
                tc_fence_after();
                if (((int)(unit % p.nqp) * 2 + t) * FA_BM >= p.Lq) {
                    // the query tile lies beyond the sequence (an odd number of query tiles): nothing to compute, but the
                    // ring and the Q buffer are handed back in step with the other issuer - one arrival per landed tile
                    mbar_arrive(&bars.q_empty);
                    for (int i = 0; i < 2 * nkt && ok; ++i) {
                        ok = mbar_wait(&bars.kv_full[s], ph, lim);
                        if (!ok) break;
                        mbar_arrive(&bars.kv_empty[s]);
                        if (++s == nst) { s = 0; ph ^= 1u; }
                    }
                    continue;
                }
                qk(nkt == 1);   // (S_t is free: the wait for p_full of the previous unit's last tile came after its s_read)
                for (int j = 0; j < nkt && ok; ++j, ++sc) {
                    if (j + 1 < nkt) {
                        TC_PROF(7);
                        ok = mbar_wait(&bars.s_read[t], sc & 1u, lim);   // the scores of tile j are in registers
                        if (!ok) break;
                        TC_PROF(0);
                        tc_fence_after();
                        qk(j + 2 == nkt);
                        if (!ok) break;
                    }
                    ok = mbar_wait(&bars.kv_full[s], ph, lim);   // V_j
                    if (ok && j == 0) ok = mbar_wait(&bars.o_empty[t], (uint32_t)(lu & 1) ^ 1u, lim);   // the epilogue of the previous unit has read O_t
                    TC_PROF(3);
                    const uint32_t va = smem_u32(ring + (size_t)s * tile_bytes);
#pragma unroll
                    for (int h = 0; h < 2 && ok; ++h) {
                        ok = mbar_wait(h == 0 ? &bars.p_half[t] : &bars.p_full[t], sc & 1u, lim);
                        if (!ok) break;
                        tc_fence_after();
                        TC_PROF(4 + h);
                        const uint64_t dp = umma_desc_k_sw128(pa + h * (FA_BM * 128));
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            umma_bf16(t_o, dp + 2 * k, umma_desc_mn_sw128(va + (4 * h + k) * 2048, FA_BN * 128), id_pv, (j > 0 || h != 0 || k != 0) ? 1u : 0u);
                        if (h == 1) umma_commit(&bars.o_done[t]);
                        TC_PROF(6);
                    }
                    if (!ok) break;
                    umma_commit(&bars.kv_empty[s]);
                    if (++s == nst) { s = 0; ph ^= 1u; }
                }
                ++lu;
            }
            if (!ok) { report_kernel_error(p.err, p.err_sys, (unsigned)KERR_MBAR_TIMEOUT | (1u << 9)); failed = true; }
            TC_PROF_FLUSH(8 * t, t == 0);
        }
      }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(FA_REGS_LARGE));
        // ---- softmax and epilogue of query tile t; thread = query row (tensor-memory lane) ----
        const int t = (warp - 4) >> 2, q = warp & 3;
        const int row = 32 * q + lane;
        const uint32_t ts = tmem + ((uint32_t)(32 * q) << 16) + (uint32_t)t * 128u;   // S_t of this row
        const uint32_t to = tmem + ((uint32_t)(32 * q) << 16) + 256u + (uint32_t)t * 128u;
        const uint32_t prow = smem_u32(p_smem + (size_t)t * FA_P_BYTES) + (uint32_t)row * 128u;   // this row of P_t, first group of 64 keys
        const uint32_t sw = (uint32_t)(row & 7);
        const float sl2 = p.scale_log2;
        long long sc = 0;
        float m_ref = 0.0f, l = 0.0f;
        uint32_t r0[32], r1[32], r2[32], r3[32];
        TC_PROF_DECL;
        for (long long unit = blockIdx.x; unit < p.n_units && !failed; unit += gridDim.x) {
            const int bh = (int)(unit / p.nqp), qp = (int)(unit % p.nqp);
            if ((qp * 2 + t) * FA_BM >= p.Lq) continue;   // this query tile lies beyond the sequence: its issuer skips it too
            for (int j = 0; j < nkt; ++j, ++sc) {
                TC_PROF(6);
                FA_FAIL_AT(2, !mbar_wait(&bars.s_full[t], (uint32_t)(sc & 1), lim));
                tc_fence_after();
                TC_PROF(0);
                const int valid = min(FA_BN, p.Lk - j * FA_BN);   // real keys in this tile
                tmem_ld32(ts, r0);
                tmem_ld32(ts + 32, r1);
                tmem_ld32(ts + 64, r2);
                tmem_ld32(ts + 96, r3);
                tmem_ld_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars.s_read[t]);   // S_t may be overwritten
                TC_PROF(1);
                if (valid < FA_BN) {   // (the same for every thread) keys that do not exist: exp2(-inf) = 0
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        if (i >= valid) r0[i] = 0xff800000u;
                        if (32 + i >= valid) r1[i] = 0xff800000u;
                        if (64 + i >= valid) r2[i] = 0xff800000u;
                        if (96 + i >= valid) r3[i] = 0xff800000u;
                    }
                }
                float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    mx0 = fmaxf(mx0, __uint_as_float(r0[i])); mx1 = fmaxf(mx1, __uint_as_float(r1[i]));
                    mx2 = fmaxf(mx2, __uint_as_float(r2[i])); mx3 = fmaxf(mx3, __uint_as_float(r3[i]));
                }
                const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * sl2;
                if (j == 0) {
                    m_ref = mx;
                    l = 0.0f;
                } else {
                    // ---- rescale the accumulator where the maximum has outgrown its reference (rare) ----
                    const bool need = mx > m_ref + FA_RESCALE_LOG2;
                    if (__any_sync(0xffffffffu, need)) {
                        FA_FAIL_AT(3, !mbar_wait(&bars.o_done[t], (uint32_t)((sc - 1) & 1), lim));   // the previous P V of this tile is done
                        tc_fence_after();
                        const float m_new = need ? mx : m_ref;
                        const float f = fast_exp2(m_ref - m_new);
                        uint32_t w[16];
                        for (int c = 0; c < (D >> 4); ++c) {
                            tmem_ld16(to + 16 * c, w);
                            tmem_ld_wait();
#pragma unroll
                            for (int i = 0; i < 16; ++i) w[i] = __float_as_uint(__uint_as_float(w[i]) * f);
                            tmem_st16(to + 16 * c, w);
                        }
                        tmem_st_wait();
                        l *= f;
                        m_ref = m_new;
                    }
                }
                // ---- P = exp2(S * scale - reference) -> 16 bit -> this row of the shared-memory tile, 8 keys (16 bytes) at a time ----
                TC_PROF(2);
                float sum0 = 0.0f, sum1 = 0.0f;
                auto half = [&](const uint32_t (&a)[32], const uint32_t (&b)[32], uint32_t base) {
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        uint32_t pk[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int e = 8 * (c & 3) + 2 * i;
                            const float x0 = __uint_as_float(c < 4 ? a[e] : b[e]), x1 = __uint_as_float(c < 4 ? a[e + 1] : b[e + 1]);
                            const float e0 = fast_exp2(fmaf(x0, sl2, -m_ref)), e1 = fast_exp2(fmaf(x1, sl2, -m_ref));
                            sum0 += e0; sum1 += e1;
                            pk[i] = pack_16x2(e0, e1, F16);
                        }
                        st_shared_v4(base + ((((uint32_t)c) ^ sw) << 4), pk[0], pk[1], pk[2], pk[3]);
                    }
                };
                // the MMAs of the previous key tile have read P (its second half was handed over ~800 clocks ago: one wait
                // here, instead of one per half, is rarely a real wait and saves the cost of the second)
                if (sc > 0) FA_FAIL_AT(5, !mbar_wait(&bars.o_done[t], (uint32_t)((sc - 1) & 1), lim));
                TC_PROF(7);
                half(r0, r1, prow);
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars.p_half[t]);
                TC_PROF(3);
                TC_PROF(7);
                half(r2, r3, prow + FA_BM * 128);
                l += sum0 + sum1;
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars.p_full[t]);
                TC_PROF(4);
            }
            if (failed) break;
            // ---- epilogue of the unit: O_t / row sum -> 16 bit -> global; lanes trade pieces so that the stores cover full lines ----
            FA_FAIL_AT(4, !mbar_wait(&bars.o_done[t], (uint32_t)((sc - 1) & 1), lim));
            tc_fence_after();
            const float inv = 1.0f / l;
            const int qrow0 = qp * 2 * FA_BM + t * FA_BM;   // first query row of the tile within its head
            __nv_bfloat16 *orow = p.O + ((long long)bh * p.Lq + qrow0 + row) * (long long)D;
            unsigned char *row0 = reinterpret_cast<unsigned char *>(orow - (long long)(lane & 3) * D);
            for (int cp = 0; cp < ng; ++cp) {
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    tmem_ld32(to + cp * 64 + hh * 32, r0);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 16; ++i) r1[16 * hh + i] = pack_16x2(__uint_as_float(r0[2 * i]) * inv, __uint_as_float(r0[2 * i + 1]) * inv, F16);
                }
                store_rows_128B_transposed_if(row0 + cp * 128, (size_t)D * 2, r1, lane, p.Lq - (qrow0 + (row & ~3)));
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars.o_empty[t]);
            TC_PROF(5);
        }
        TC_PROF_FLUSH(16 + 8 * t, (threadIdx.x & 127) == 64);
    }

    if (failed) for (int i = 0; i < 2000; ++i) __nanosleep(1000);   // let copies and MMAs in flight drain
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 0) tmem_dealloc(tmem, 512);
}
// ---------------------------------------------------------------------------------------------------
// head_d 256: ONE query tile of 128 rows per unit.  The output accumulator [128 x 256] fp32 takes half of the tensor
// memory; the other half holds two score buffers, so that S_j+1 = Q K_j+1^T is computed while the softmax warps work
// on S_j.  P (16 bit) is written over the first 64 columns of its own score buffer and the P V MMA takes its A operand
// from tensor memory (umma_16_ts), so P never touches shared memory:   S_0 | S_1, O += P_0 V_0, S_2, O += P_1 V_1, S_3, ...   K and V pass through the ring
// in halves of 32 KB (K: 128 keys x 128 of the 256 columns; V: 64 keys x 256 columns) in exactly the order the MMA
// thread consumes them.  One softmax warpgroup (a thread per row) serves both buffers: its row statistics are one
// stream, and with 192 threads a thread may hold its 128 scores in registers.
constexpr int FB_THREADS = 192;     // warp 0: TMA, warp 1: MMA, warps 2-5: softmax and epilogue
constexpr int FB_D = 256;
constexpr int FB_STAGE = 32768;

template <bool F16>
__global__ void __launch_bounds__(FB_THREADS, 1)
fa256_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, const FaParams p) {
    extern __shared__ unsigned char fa_smem_raw[];
    __shared__ FaBars bars;
    __shared__ uint32_t tmem_slot;
    const uint32_t raw_addr = smem_u32(fa_smem_raw);
    unsigned char *smem = fa_smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nkt = p.nkt, nst = p.nst;
    unsigned char *q_smem = smem;                       // [4 groups][128 rows][128 B]
    unsigned char *ring = smem + 2 * FB_STAGE;
    const uint32_t lim = p.spin_limit;

    if (threadIdx.x == 0) {
        for (int i = 0; i < FA_MAX_STAGES; ++i) { mbar_init(&bars.kv_full[i], 1); mbar_init(&bars.kv_empty[i], 1); }
        mbar_init(&bars.q_full, 1);
        mbar_init(&bars.q_empty, 1);
        for (int t = 0; t < 2; ++t) { mbar_init(&bars.s_full[t], 1); mbar_init(&bars.p_full[t], 4); mbar_init(&bars.o_done[t], 1); mbar_init(&bars.o_empty[t], 4); }
        mbar_fence_init();
        tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
    }
    if (warp == 0) tmem_alloc(&tmem_slot, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;        // score buffer b: columns [128 b, 128 b + 128); O: [256, 512)
    bool failed = false;
    const bool skip = (*reinterpret_cast<volatile unsigned *>(p.err) != 0);

    if (skip) {
        // fall through to the common exit
    } else if (warp == 0) {
        if (lane == 0) {
            int s = 0;            // ring stage and the parity of its use (kept by hand: a division here costs the thread hundreds of clocks)
            uint32_t ph = 0;
            int ui = 0;
            auto load_k = [&](int bh, int j, bool &ok) {   // the two column halves of K tile j
                for (int h = 0; h < 2 && ok; ++h) {
                    ok = mbar_wait(&bars.kv_empty[s], ph ^ 1u, lim);
                    if (!ok) break;
                    mbar_expect_tx(&bars.kv_full[s], FB_STAGE);
                    tma_load_4d(ring + (size_t)s * FB_STAGE, &tmK, 0, j * FA_BN, 2 * h, bh, &bars.kv_full[s]);
                    if (++s == nst) { s = 0; ph ^= 1u; }
                }
            };
            auto load_v = [&](int bh, int j, bool &ok) {   // the two key halves of V tile j
                for (int h = 0; h < 2 && ok; ++h) {
                    ok = mbar_wait(&bars.kv_empty[s], ph ^ 1u, lim);
                    if (!ok) break;
                    mbar_expect_tx(&bars.kv_full[s], FB_STAGE);
                    tma_load_4d(ring + (size_t)s * FB_STAGE, &tmV, 0, j * FA_BN + 64 * h, 0, bh, &bars.kv_full[s]);
                    if (++s == nst) { s = 0; ph ^= 1u; }
                }
            };
            bool ok = true;
            for (long long unit = blockIdx.x; unit < p.n_units && ok; unit += gridDim.x, ++ui) {
                const int bh = (int)(unit / p.nqp), qt = (int)(unit % p.nqp);
                ok = mbar_wait(&bars.q_empty, (uint32_t)(ui & 1) ^ 1u, lim);
                if (!ok) break;
                mbar_expect_tx(&bars.q_full, 2 * FB_STAGE);
                tma_load_4d(q_smem, &tmQ, 0, qt * FA_BM, 0, bh, &bars.q_full);
                load_k(bh, 0, ok);                        // the order of the MMA thread: K_0 | K_1, V_0, K_2, V_1, ...
                for (int j = 0; j < nkt && ok; ++j) {
                    if (j + 1 < nkt) load_k(bh, j + 1, ok);
                    if (ok) load_v(bh, j, ok);
                }
            }
            if (!ok) { report_kernel_error(p.err, p.err_sys, (unsigned)KERR_MBAR_TIMEOUT | (1u << 7)); failed = true; }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t id_qk = umma_idesc_16(FA_BM, FA_BN, 0, 0, F16 ? 1 : 0), id_pv = umma_idesc_16(FA_BM, FB_D, 0, 1, F16 ? 1 : 0);
            int s = 0;                  // ring stage and the parity of its use
            uint32_t ph = 0;
            long long gt = 0;           // tiles issued so far (score buffer = tile & 1)
            int ui = 0;
            bool ok = true;
            const uint32_t qa = smem_u32(q_smem);
            auto qk = [&](long long g) {   // S_(g & 1) = Q K^T over the two column halves of the K tile
                const int b = (int)(g & 1);
                for (int h = 0; h < 2 && ok; ++h) {
                    ok = mbar_wait(&bars.kv_full[s], ph, lim);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t ka = smem_u32(ring + (size_t)s * FB_STAGE);
#pragma unroll
                    for (int k = 0; k < 8; ++k)
                        umma_bf16(tmem + b * 128, umma_desc_k_sw128(qa + (2 * h + (k >> 2)) * (FA_BM * 128)) + 2 * (k & 3),
                                  umma_desc_k_sw128(ka + (k >> 2) * (FA_BN * 128)) + 2 * (k & 3), id_qk, (h | k) != 0);
                    umma_commit(&bars.kv_empty[s]);
                    if (++s == nst) { s = 0; ph ^= 1u; }
                }
                umma_commit(&bars.s_full[b]);
            };
            auto pv = [&](long long g, bool acc) {   // O (+)= P V over the two key halves of the V tile; P in the first 64 columns of the score buffer
                const int b = (int)(g & 1);
                for (int h = 0; h < 2 && ok; ++h) {
                    ok = mbar_wait(&bars.kv_full[s], ph, lim);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t va = smem_u32(ring + (size_t)s * FB_STAGE);
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk)
                        umma_16_ts(tmem + 256, tmem + b * 128 + (4 * h + kk) * 8, umma_desc_mn_sw128(va + kk * 2048, 64 * 128), id_pv, (acc || h != 0 || kk != 0) ? 1u : 0u);
                    umma_commit(&bars.kv_empty[s]);
                    if (++s == nst) { s = 0; ph ^= 1u; }
                }
                umma_commit(&bars.o_done[b]);
            };
            for (long long unit = blockIdx.x; unit < p.n_units && ok; unit += gridDim.x, ++ui) {
                ok = mbar_wait(&bars.q_full, (uint32_t)(ui & 1), lim);
                if (!ok) break;
                tc_fence_after();
                qk(gt);
                for (int j = 0; j < nkt && ok; ++j) {
                    if (j + 1 < nkt) qk(gt + j + 1);
                    else umma_commit(&bars.q_empty);   // the unit's last score MMA has been issued
                    if (!ok) break;
                    if (j == 0) ok = mbar_wait(&bars.o_empty[0], (uint32_t)(ui & 1) ^ 1u, lim);   // the epilogue of the previous unit has read O
                    const long long g = gt + j;
                    ok = ok && mbar_wait(&bars.p_full[g & 1], (uint32_t)((g >> 1) & 1), lim);
                    if (!ok) break;
                    tc_fence_after();
                    pv(g, j > 0);
                }
                gt += nkt;
            }
            if (!ok) { report_kernel_error(p.err, p.err_sys, (unsigned)KERR_MBAR_TIMEOUT | (1u << 9)); failed = true; }
        }
    } else {
        // ---- softmax and epilogue; thread = query row (tensor-memory lane) ----
        const int q = warp & 3;
        const int row = 32 * q + lane;
        const uint32_t tl = tmem + ((uint32_t)(32 * q) << 16);
        const uint32_t to = tl + 256u;
        const float sl2 = p.scale_log2;
        long long gt = 0;
        float m_ref = 0.0f, l = 0.0f;
        uint32_t r0[32], r1[32], r2[32], r3[32];
        // The P V product of tile g arrives on o_done[g & 1].  The score MMA of tile g + 1 is issued before the P V MMA
        // of tile g, so these warps can be a tile ahead of the products; a wait by parity can only tell the current
        // phase of a barrier from the one before it, hence two barriers, each followed phase by phase: at the start
        // of tile g the product of tile g - 2 is certainly done (the MMAs complete in the order they were issued) and
        // is ticked off, which keeps every later wait within one phase of its barrier.
        long long seen[2] = {0, 0};   // phases of o_done[b] seen complete
        auto see_pv_done = [&](long long g) {   // true once the P V product of tile g (counted over the units) is done
            const int b = (int)(g & 1);
            while (seen[b] <= (g >> 1)) {
                if (!mbar_wait(&bars.o_done[b], (uint32_t)(seen[b] & 1), lim)) return false;
                ++seen[b];
            }
            return true;
        };
        for (long long unit = blockIdx.x; unit < p.n_units && !failed; unit += gridDim.x) {
            const int bh = (int)(unit / p.nqp), qt = (int)(unit % p.nqp);
            for (int j = 0; j < nkt; ++j, ++gt) {
                const uint32_t ts = tl + (uint32_t)(gt & 1) * 128u;
                FA_FAIL_AT(2, !mbar_wait(&bars.s_full[gt & 1], (uint32_t)((gt >> 1) & 1), lim));
                tc_fence_after();
                const int valid = min(FA_BN, p.Lk - j * FA_BN);
                if (gt >= 2) FA_FAIL_AT(5, !see_pv_done(gt - 2));   // (done long ago: ticked off)
                tmem_ld32(ts, r0);
                tmem_ld32(ts + 32, r1);
                tmem_ld32(ts + 64, r2);
                tmem_ld32(ts + 96, r3);
                tmem_ld_wait();
                if (valid < FA_BN) {   // (the same for every thread) keys that do not exist: exp2(-inf) = 0
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        if (i >= valid) r0[i] = 0xff800000u;
                        if (32 + i >= valid) r1[i] = 0xff800000u;
                        if (64 + i >= valid) r2[i] = 0xff800000u;
                        if (96 + i >= valid) r3[i] = 0xff800000u;
                    }
                }
                float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    mx0 = fmaxf(mx0, __uint_as_float(r0[i])); mx1 = fmaxf(mx1, __uint_as_float(r1[i]));
                    mx2 = fmaxf(mx2, __uint_as_float(r2[i])); mx3 = fmaxf(mx3, __uint_as_float(r3[i]));
                }
                const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * sl2;
                if (j == 0) {
                    m_ref = mx;
                    l = 0.0f;
                } else {
                    const bool need = mx > m_ref + FA_RESCALE_LOG2;
                    if (__any_sync(0xffffffffu, need)) {
                        FA_FAIL_AT(3, !see_pv_done(gt - 1));   // the previous P V is done
                        tc_fence_after();
                        const float m_new = need ? mx : m_ref;
                        const float f = fast_exp2(m_ref - m_new);
                        uint32_t w[32];
                        for (int c = 0; c < FB_D / 32; ++c) {
                            tmem_ld32(to + 32 * c, w);
                            tmem_ld_wait();
#pragma unroll
                            for (int i = 0; i < 32; ++i) w[i] = __float_as_uint(__uint_as_float(w[i]) * f);
                            tmem_st32(to + 32 * c, w);
                        }
                        tmem_st_wait();
                        l *= f;
                        m_ref = m_new;
                    }
                }
                float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float e0 = fast_exp2(fmaf(__uint_as_float(r0[2 * i]), sl2, -m_ref)), e1 = fast_exp2(fmaf(__uint_as_float(r0[2 * i + 1]), sl2, -m_ref));
                    sum0 += e0; sum1 += e1;
                    r0[i] = pack_16x2(e0, e1, F16);
                }
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float e0 = fast_exp2(fmaf(__uint_as_float(r1[2 * i]), sl2, -m_ref)), e1 = fast_exp2(fmaf(__uint_as_float(r1[2 * i + 1]), sl2, -m_ref));
                    sum0 += e0; sum1 += e1;
                    r0[16 + i] = pack_16x2(e0, e1, F16);
                }
                tmem_st32(ts, r0);
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float e0 = fast_exp2(fmaf(__uint_as_float(r2[2 * i]), sl2, -m_ref)), e1 = fast_exp2(fmaf(__uint_as_float(r2[2 * i + 1]), sl2, -m_ref));
                    sum0 += e0; sum1 += e1;
                    r2[i] = pack_16x2(e0, e1, F16);
                }
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float e0 = fast_exp2(fmaf(__uint_as_float(r3[2 * i]), sl2, -m_ref)), e1 = fast_exp2(fmaf(__uint_as_float(r3[2 * i + 1]), sl2, -m_ref));
                    sum0 += e0; sum1 += e1;
                    r2[16 + i] = pack_16x2(e0, e1, F16);
                }
                tmem_st32(ts + 32, r2);
                l += sum0 + sum1;
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars.p_full[gt & 1]);
            }
            if (failed) break;
            // ---- epilogue of the unit: O / row sum -> 16 bit -> global ----
            if (gt >= 2) FA_FAIL_AT(4, !see_pv_done(gt - 2));
            FA_FAIL_AT(4, !see_pv_done(gt - 1));
            tc_fence_after();
            const float inv = 1.0f / l;
            const int qrow0 = qt * FA_BM;
            __nv_bfloat16 *orow = p.O + ((long long)bh * p.Lq + qrow0 + row) * (long long)FB_D;
            unsigned char *row0 = reinterpret_cast<unsigned char *>(orow - (long long)(lane & 3) * FB_D);
            for (int cp = 0; cp < FB_D / 64; ++cp) {
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    tmem_ld32(to + cp * 64 + hh * 32, r0);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 16; ++i) r1[16 * hh + i] = pack_16x2(__uint_as_float(r0[2 * i]) * inv, __uint_as_float(r0[2 * i + 1]) * inv, F16);
                }
                store_rows_128B_transposed_if(row0 + cp * 128, (size_t)FB_D * 2, r1, lane, p.Lq - (qrow0 + (row & ~3)));
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars.o_empty[0]);
        }
    }

    if (failed) for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 0) tmem_dealloc(tmem, 512);
}

#undef FA_FAIL_AT

// ---- host side ------------------------------------------------------------------------------------
inline bool fa_supported(const b200attn_args &a) {
    if (a.dtype != B200ATTN_BF16 && a.dtype != B200ATTN_F16) return false;
    if (a.head_d != 64 && a.head_d != 128 && a.head_d != 256) return false;
    if (a.len_q <= 64) return false;   // few queries: the key-split kernels, or the split-head_d kernels
    if ((((uintptr_t)a.Q | (uintptr_t)a.K | (uintptr_t)a.V) & 15) != 0 || ((uintptr_t)a.out & 31) != 0) return false;
    const long long BH = (long long)a.batch_sz * a.num_heads;
    if (BH >= (1ll << 31) || BH * ((a.len_q + 255) / 256) >= (1ll << 40)) return false;
    return true;
}

// Returns B200ATTN_OK, -1 when the shape should run on another path (nothing has been launched then), or a
// status with tc_bf16_error() set.
inline int fa_run(const b200attn_args &a, unsigned *err_dev, unsigned *err_sys, int sm_count, unsigned spin_limit, cudaStream_t st,
                  std::atomic<unsigned long long> *launches) {
    const long long BH = (long long)a.batch_sz * a.num_heads;
    const int D = a.head_d, Lq = a.len_q, Lk = a.len_k;
    static std::mutex attr_mu;
    static size_t smem_max[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    {
        std::lock_guard<std::mutex> lk(attr_mu);
        if (smem_max[dev & 63] == 0) {
            cudaFuncAttributes fa, fb;
            cudaDeviceProp prop;
            cudaGetDeviceProperties(&prop, dev);
            // one limit for both kernels of this file: the opt-in maximum less the larger static allocation
            bool ok = cudaFuncGetAttributes(&fa, fa_kernel<false>) == cudaSuccess && cudaFuncGetAttributes(&fb, fa256_kernel<false>) == cudaSuccess;
            const size_t stat = ok ? (fa.sharedSizeBytes > fb.sharedSizeBytes ? fa.sharedSizeBytes : fb.sharedSizeBytes) : 0;
            const int dyn = ok ? (int)(prop.sharedMemPerBlockOptin - stat) : 0;
            ok = ok && cudaFuncSetAttribute(fa_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, dyn) == cudaSuccess &&
                 cudaFuncSetAttribute(fa_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, dyn) == cudaSuccess &&
                 cudaFuncSetAttribute(fa256_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, dyn) == cudaSuccess &&
                 cudaFuncSetAttribute(fa256_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, dyn) == cudaSuccess;
            if (!ok) { (void)cudaGetLastError(); snprintf(t_tc_error, sizeof t_tc_error, "cudaFuncSetAttribute(max dynamic shared memory) failed"); return B200ATTN_ERR_CUDA; }
            smem_max[dev & 63] = (size_t)dyn;
        }
    }
    if (D == FB_D) {
        // one query tile per unit, K and V through the ring in halves
        int nst = (int)((smem_max[dev & 63] - 1024 - 2 * FB_STAGE) / FB_STAGE);
        if (nst > FA_MAX_STAGES) nst = FA_MAX_STAGES;
        if (nst < 5) return -1;
        CUtensorMap tmQ, tmK, tmV;
        if (!make_tmap_grouped_heads(&tmQ, a.Q, BH, Lq, D, FA_BM, 4) || !make_tmap_grouped_heads(&tmK, a.K, BH, Lk, D, FA_BN, 2) ||
            !make_tmap_grouped_heads(&tmV, a.V, BH, Lk, D, 64, 4)) {
            snprintf(t_tc_error, sizeof t_tc_error, "cuTensorMapEncodeTiled failed");
            return -1;
        }
        FaParams p{};
        p.Lq = Lq; p.Lk = Lk; p.D = D;
        p.nqp = (Lq + FA_BM - 1) / FA_BM;   // query tiles per head
        p.nkt = (Lk + FA_BN - 1) / FA_BN;
        p.nst = nst;
        p.n_units = BH * p.nqp;
        p.scale_log2 = 1.4426950408889634f / sqrtf((float)D);
        p.f16 = a.dtype == B200ATTN_F16 ? 1 : 0;
        p.O = (__nv_bfloat16 *)a.out;
        p.err = err_dev; p.err_sys = err_sys; p.spin_limit = spin_limit;
        const unsigned grid = (unsigned)(p.n_units < sm_count ? p.n_units : sm_count);
        const size_t smem = (size_t)(2 + nst) * FB_STAGE + 1024;
        if (p.f16) fa256_kernel<true><<<grid, FB_THREADS, smem, st>>>(tmQ, tmK, tmV, p);
        else fa256_kernel<false><<<grid, FB_THREADS, smem, st>>>(tmQ, tmK, tmV, p);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) { snprintf(t_tc_error, sizeof t_tc_error, "fa256_kernel launch failed: %s", cudaGetErrorString(e)); return B200ATTN_ERR_CUDA; }
        launches->fetch_add(1);
        return B200ATTN_OK;
    }
    const size_t tb = (size_t)FA_BN * D * 2;
    int nst = (int)((smem_max[dev & 63] - 1024 - 2 * tb - 2 * (size_t)FA_P_BYTES) / tb);   // head_d 128: 3 stages; 64: 8
    if (nst > FA_MAX_STAGES) nst = FA_MAX_STAGES;
    if (nst < 3) return -1;
    CUtensorMap tmQ, tmK, tmV;
    if (!make_tmap_grouped_heads(&tmQ, a.Q, BH, Lq, D, FA_BM, D / 64) || !make_tmap_grouped_heads(&tmK, a.K, BH, Lk, D, FA_BN, D / 64) ||
        !make_tmap_grouped_heads(&tmV, a.V, BH, Lk, D, FA_BN, D / 64)) {
        snprintf(t_tc_error, sizeof t_tc_error, "cuTensorMapEncodeTiled failed");
        return -1;
    }
    FaParams p{};
    p.Lq = Lq; p.Lk = Lk; p.D = D;
    p.nqp = ((Lq + FA_BM - 1) / FA_BM + 1) / 2;
    p.nkt = (Lk + FA_BN - 1) / FA_BN;
    p.nst = nst;
    p.n_units = BH * p.nqp;
    p.scale_log2 = 1.4426950408889634f / sqrtf((float)D);
    p.f16 = a.dtype == B200ATTN_F16 ? 1 : 0;
    p.O = (__nv_bfloat16 *)a.out;
    p.err = err_dev; p.err_sys = err_sys; p.spin_limit = spin_limit;
    const unsigned grid = (unsigned)(p.n_units < sm_count ? p.n_units : sm_count);
    const size_t smem = 2 * tb + 2 * (size_t)FA_P_BYTES + (size_t)nst * tb + 1024;
    if (p.f16) fa_kernel<true><<<grid, FA_THREADS, smem, st>>>(tmQ, tmK, tmV, p);
    else fa_kernel<false><<<grid, FA_THREADS, smem, st>>>(tmQ, tmK, tmV, p);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { snprintf(t_tc_error, sizeof t_tc_error, "fa_kernel launch failed: %s", cudaGetErrorString(e)); return B200ATTN_ERR_CUDA; }
    launches->fetch_add(1);
    return B200ATTN_OK;
}

// Encoded copies for a call with a positional encoding: Q (and K, unless the caller keeps K encoded) is encoded once
// into a scratch copy - fp32 arithmetic of the reference tables, one rounding to the 16-bit format - and `b` becomes
// the same call on the copies without an encoding.  For the narrow heads of the kernel above, encoding K inside the
// operand load would repeat the work once per 256 query rows, while the copy costs a few per cent of the attention
// itself (0.27 GB of traffic against 0.65 ms of tensor-core work at B*H = 64, len 4096, head_d 128); the reference does
// the same in attention_forward_separate_rope, final/rope.cu:1379-1416.  Also what gives fp16 tensors with an encoding
// a tensor-core path at all (the in-load encodings of tc_wide.cuh are bf16 arithmetic).
// `q_copy`, `k_copy`: device scratch of the sizes of Q, K.
template <typename T>
inline int fa_encode_copies(const b200attn_args &a, int rd, float base, T *q_copy, T *k_copy, int sm_count, cudaStream_t st,
                            std::atomic<unsigned long long> *launches, b200attn_args *b) {
    RopeKParams rp{};
    rp.BH = (long long)a.batch_sz * a.num_heads;
    rp.D = a.head_d;
    rp.sinus = a.pe == B200ATTN_PE_SINUSOIDAL ? 1 : 0;
    rp.rd = rp.sinus ? a.head_d : rd;
    rp.half = pe_pairs_halves(a.pe) ? 1 : 0;
    rp.pos0 = 0;
    rp.base = rp.sinus ? 10000.0f : base;
    rp.cos_cache = rp.sinus ? nullptr : a.cos_cache;
    rp.sin_cache = rp.sinus ? nullptr : a.sin_cache;
    rp.X = a.Q; rp.Y = q_copy; rp.L = a.len_q;
    cudaError_t e = launch_rope_k<T>(rp, sm_count, st);
    launches->fetch_add(1);
    if (e == cudaSuccess && pe_encodes_k(a.pe)) {
        rp.X = a.K; rp.Y = k_copy; rp.L = a.len_k;
        e = launch_rope_k<T>(rp, sm_count, st);
        launches->fetch_add(1);
    }
    if (e != cudaSuccess) { snprintf(t_tc_error, sizeof t_tc_error, "encoding kernel launch failed: %s", cudaGetErrorString(e)); return B200ATTN_ERR_CUDA; }
    *b = a;
    b->Q = q_copy;
    if (pe_encodes_k(a.pe)) b->K = k_copy;
    b->pe = B200ATTN_PE_NONE;
    b->cos_cache = nullptr; b->sin_cache = nullptr;
    return B200ATTN_OK;
}

}  // namespace b200attn
