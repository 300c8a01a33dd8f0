// bf16 attention forward on the 5th-generation tensor cores as two persistent kernels per call, with
// the scores passing through a bf16 scratch in HBM.  It began as the path for wide heads (a 128-row
// fp32 output accumulator of a 1024-wide head is twice the tensor memory of an SM and the query tile
// is more shared memory than an SM has, so the one-kernel pipeline of tc_bf16.cuh does not fit) and
// measured faster than that pipeline on the narrow heads too, so it takes every shape it supports.
//
//   tcw_scores_kernel   S tiles [128 queries x 256 keys] = Q Kt, a K-loop over 64-wide chunks of
//                       head_d with both operands streamed by TMA through a 4-slot ring, the
//                       accumulator double-buffered in tensor memory (2 x 256 columns) so that the
//                       epilogue of one tile runs under the MMAs of the next.  The epilogue takes the
//                       row maximum of the tile and writes the scores in log2 units RELATIVE to that
//                       maximum as bf16 (values near the maximum, the ones that carry weight, are
//                       then small numbers and keep their precision) plus the maximum itself in fp32.
//   tcw_pv_kernel       per (head, query tile, block of <= 512 output columns): the global row
//                       maximum is the maximum of the tile maxima, so P = exp2(S - max) is final when
//                       it is computed (no running rescale of the accumulator).  A score block arrives
//                       by TMA in the swizzled K-major layout of the MMA's A operand and sixteen warps
//                       turn it into P in place; one thread issues O += P V with V streamed by TMA;
//                       the accumulator [128 x <=512] fp32 stays in tensor memory until the unit's
//                       epilogue divides by the row sums.
//
// A positional encoding (rotate-half or interleaved-pair RoPE, sinusoidal) is applied inside the
// operand load of the score kernel: the ring is filled two chunks at a time (rotate-half: chunks c
// and c + n_chunks/2), eight transform warps encode the two slots in shared memory between TMA
// arrival and MMA, and while the encoded pieces are in registers they are also written to a scratch
// copy.  The tiles that do this are one "diagonal" set per head that touches every query tile and
// every key tile once; a second launch computes all the other tiles from the encoded copies without
// any transform.
//
// Shapes taken here: bf16 (fp16 without an encoding), head_d % 64 == 0 (with an encoding: % 128; rotate-half:
// rotary_dim == head_d), any len_q, len_k <= 65536 (not both <= 64).  Lengths that are not multiples of the
// tiles: the operand tiles reach into the next head's rows (or read zeros behind the last head), whose
// scores land in rows and columns of S that nobody uses - S keeps whole 128-blocks per head -; the
// columns of keys that do not exist are written as -inf, V rows that do not exist read as zero (the head is a
// coordinate of the V map), and output rows that do not exist are not stored.  Every wait is bounded.
#pragma once

#include "tc_bf16.cuh"

namespace b200attn {

constexpr int TW_THREADS = 448;            // warp 0 TMA, warp 1 MMA, warps 2-5 epilogue, warps 6-13 transform
constexpr int TW_NST = 4;                  // operand ring depth
constexpr int TW_BM = 128;                 // query rows per score tile
constexpr int TW_BN = 256;                 // keys per score tile
constexpr int TW_QCHUNK = TW_BM * 128;     // [128 rows x 64 bf16]
constexpr int TW_KCHUNK = TW_BN * 128;     // [256 rows x 64 bf16]
constexpr int TW_STAGE = TW_QCHUNK + TW_KCHUNK;

struct TcwScoreParams {
    int Lq, Lk, D, nch;        // nch = D / 64
    int Lqp, Lkp;              // Lq and Lk rounded up to multiples of 128: rows per head and row pitch of S
    int nqt, nkt;              // ceil(Lq / 128), ceil(Lk / 256)
    int mode;                  // 0: every tile, operands as given; 1: the encoding tile set; 2: all other tiles
    int pe;                    // mode 1: PE_ROPE_HALF, PE_ROPE_INTERLEAVED or PE_SINUSOIDAL
    int rotate_k;              // mode 1: 0 = only Q carries the encoding
    int f16;                   // operands are fp16 (no encoding then), else bf16
    int tph;                   // tiles per head in this launch
    long long n_tiles;         // heads * tph
    float scale_log2;          // log2(e) / sqrt(D)
    __nv_bfloat16 *S;          // [heads * Lqp][Lkp]  scores, log2 units, relative to the tile's row maximum; -inf beyond Lk
    float *rowmax;             // [heads * Lqp][nkt] row maxima of the tiles, log2 units
    const __nv_bfloat16 *tab;  // mode 1: [>= max(Lqp, 256 * nkt)][D]; rotate-half: cos in columns [0, D/2), sin in [D/2, D);
                               // otherwise the layout of tc_build_pe_table (element-wise partner of the data)
    __nv_bfloat16 *q_store, *k_store;   // mode 1: rotated copies, [heads * Lq][D] and [heads * Lk][D]
    unsigned *err, *err_sys;
    unsigned spin_limit;
};

struct TwBars {
    uint64_t full[TW_NST], ready[TW_NST], empty[TW_NST];
    uint64_t acc_full[2], acc_empty[2];
};

// Optional cycle accounting (profiling builds only): -DB200ATTN_TC_PROFILE plus -DB200ATTN_PROF_WIDE=1
// (score kernel, launches of mode B200ATTN_PROF_MODE) or =2 (P V kernel).
#if defined(B200ATTN_TC_PROFILE) && defined(B200ATTN_PROF_WIDE)
#ifndef B200ATTN_PROF_MODE
#define B200ATTN_PROF_MODE 1
#endif
#define TWS_DECL TC_PROF_DECL
#define TWS(slot) do { if (B200ATTN_PROF_WIDE == 1) TC_PROF(slot); } while (0)
#define TWS_FLUSH(base, on) do { if (B200ATTN_PROF_WIDE == 1 && p.mode == B200ATTN_PROF_MODE) TC_PROF_FLUSH(base, on); } while (0)
#define TWP(slot) do { if (B200ATTN_PROF_WIDE == 2) TC_PROF(slot); } while (0)
#define TWP_FLUSH(base, on) do { if (B200ATTN_PROF_WIDE == 2) TC_PROF_FLUSH(base, on); } while (0)
#else
#define TWS_DECL
#define TWS(slot)
#define TWS_FLUSH(base, on)
#define TWP(slot)
#define TWP_FLUSH(base, on)
#endif

#define TW_FAIL_AT(site, cond)                                                                      \
    if (cond) {                                                                                     \
        report_kernel_error(p.err, p.err_sys, (unsigned)KERR_MBAR_TIMEOUT | (1u << (7 + (site))));  \
        failed = true;                                                                              \
        break;                                                                                      \
    }

// Tile j of a head for the three launch modes.  Mode 1 (the encoding launch) is a set of max(nqt, nkt)
// tiles that contains every query tile and every key tile; mode 2 is its complement.  With at least
// as many query tiles as key tiles, query tile q is paired with key tile a(q): q/2 where that
// reaches every key tile (then the 128 query rows have the positions of one half of the 256 key
// rows, and one set of table values serves both), else q mod nkt.
__host__ __device__ __forceinline__ int tcw_diag_kt(int q, int nqt, int nkt) {
    return (nqt >= 2 * nkt - 1) ? (q >> 1) % nkt : q % nkt;
}
__host__ __device__ __forceinline__ void tcw_tile_of(int mode, int j, int nqt, int nkt, int *qt, int *kt) {
    if (mode == 0) { *qt = j / nkt; *kt = j - *qt * nkt; }
    else if (nkt <= nqt) {
        if (mode == 1) { *qt = j; *kt = tcw_diag_kt(j, nqt, nkt); }
        else { const int q = j / (nkt - 1), r = j - q * (nkt - 1); *qt = q; *kt = (tcw_diag_kt(q, nqt, nkt) + 1 + r) % nkt; }
    } else {
        if (mode == 1) { *qt = j % nqt; *kt = j; }
        else { const int k = j / (nqt - 1), r = j - k * (nqt - 1); *kt = k; *qt = (k % nqt + 1 + r) % nqt; }
    }
}

// (lo, hi) -> (lo*c - hi*s, hi*c + lo*s) on packed bf16 pairs
__device__ __forceinline__ void tcw_rotate(uint32_t &lo, uint32_t &hi, uint32_t c, uint32_t s) {
    const __nv_bfloat162 l = *reinterpret_cast<__nv_bfloat162 *>(&lo), h = *reinterpret_cast<__nv_bfloat162 *>(&hi);
    const __nv_bfloat162 cc = *reinterpret_cast<__nv_bfloat162 *>(&c), ss = *reinterpret_cast<__nv_bfloat162 *>(&s);
    uint32_t ns_bits = s ^ 0x80008000u;
    const __nv_bfloat162 ns = *reinterpret_cast<__nv_bfloat162 *>(&ns_bits);
    __nv_bfloat162 nl = __hfma2(h, ns, __hmul2(l, cc));
    __nv_bfloat162 nh = __hfma2(l, ss, __hmul2(h, cc));
    lo = *reinterpret_cast<uint32_t *>(&nl);
    hi = *reinterpret_cast<uint32_t *>(&nh);
}

// A 16-byte read-only load that the compiler keeps where it is written (it would otherwise be free to
// sink a plain load down to its first use, which defeats a software pipeline of loads).
__device__ __forceinline__ uint4 tcw_ldg_here(const void *ptr) {
    uint4 v;
    asm volatile("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(ptr));
    return v;
}

// Epilogue of one accumulator row [<= 256 keys] of a score tile, by the row's thread: the maximum over the
// tile's real keys, then the scores in log2 units relative to it as bf16, 64 keys (128 bytes) at a time with
// neighbouring rows trading pieces so that the stores cover full lines.  Keys beyond the sequence (the tile's
// columns >= valid) are written as -inf up to the end of the last 128-key block that holds a real key: they
// weigh nothing in the P V kernel, which reads whole blocks.  `srow0` = the row's place in S minus
// (lane & 3) rows.  Returns the maximum (log2 units).
__device__ __forceinline__ float tcw_store_score_row(uint32_t ta, int valid, float scale_log2, unsigned char *srow0, size_t pitch_bytes, int lane) {
    uint32_t r[32], wds[32];
    const int nfull = valid >> 5, tail = valid & 31;
    float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
    for (int c = 0; c < nfull; ++c) {
        tmem_ld32(ta + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
            mx0 = fmaxf(mx0, __uint_as_float(r[j]));
            mx1 = fmaxf(mx1, __uint_as_float(r[j + 1]));
            mx2 = fmaxf(mx2, __uint_as_float(r[j + 2]));
            mx3 = fmaxf(mx3, __uint_as_float(r[j + 3]));
        }
    }
    if (tail) {
        tmem_ld32(ta + nfull * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
            mx0 = fmaxf(mx0, j < tail ? __uint_as_float(r[j]) : -INFINITY);
            mx1 = fmaxf(mx1, j + 1 < tail ? __uint_as_float(r[j + 1]) : -INFINITY);
            mx2 = fmaxf(mx2, j + 2 < tail ? __uint_as_float(r[j + 2]) : -INFINITY);
            mx3 = fmaxf(mx3, j + 3 < tail ? __uint_as_float(r[j + 3]) : -INFINITY);
        }
    }
    const float mt = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * scale_log2;
    const int npc = 2 * ((valid + 127) >> 7);   // 64-key pieces up to the end of the last block with a real key
    for (int cp = 0; cp < npc; ++cp) {
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            const int k0 = (2 * cp + hh) * 32;   // first key of this 32-column group (the same for the whole warp)
            if (k0 >= valid) {
#pragma unroll
                for (int q = 0; q < 16; ++q) wds[16 * hh + q] = 0xFF80FF80u;   // (-inf, -inf)
            } else {
                tmem_ld32(ta + k0, r);
                tmem_ld_wait();
                if (k0 + 32 <= valid) {
#pragma unroll
                    for (int q = 0; q < 16; ++q)
                        wds[16 * hh + q] = pack_bf16x2(fmaf(__uint_as_float(r[2 * q]), scale_log2, -mt), fmaf(__uint_as_float(r[2 * q + 1]), scale_log2, -mt));
                } else {
#pragma unroll
                    for (int q = 0; q < 16; ++q)
                        wds[16 * hh + q] = pack_bf16x2(k0 + 2 * q < valid ? fmaf(__uint_as_float(r[2 * q]), scale_log2, -mt) : -INFINITY,
                                                       k0 + 2 * q + 1 < valid ? fmaf(__uint_as_float(r[2 * q + 1]), scale_log2, -mt) : -INFINITY);
                }
            }
        }
        store_rows_128B_transposed(srow0 + cp * 128, pitch_bytes, wds, lane);
    }
    return mt;
}

__global__ void __launch_bounds__(TW_THREADS, 1)
tcw_scores_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK, const TcwScoreParams p) {
    extern __shared__ unsigned char tw_smem_raw[];
    __shared__ TwBars bars;
    __shared__ uint32_t tmem_slot;
    const uint32_t raw_addr = smem_u32(tw_smem_raw);
    unsigned char *smem = tw_smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nch = p.nch;
    const uint32_t lim = p.spin_limit;
    const bool encode = (p.mode == 1);
    const bool pair_half = encode && p.pe == PE_ROPE_HALF;   // ring slots (s, s+1) hold chunks (c, c + nch/2) instead of (2c, 2c+1)

    if (threadIdx.x == 0) {
        for (int i = 0; i < TW_NST; ++i) { mbar_init(&bars.full[i], 1); mbar_init(&bars.ready[i], 8); mbar_init(&bars.empty[i], 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(&bars.acc_full[i], 1); mbar_init(&bars.acc_empty[i], 4); }
        mbar_fence_init();
        tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK);
    }
    if (warp == 0) tmem_alloc(&tmem_slot, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    bool failed = false;
    const bool skip = (*reinterpret_cast<volatile unsigned *>(p.err) != 0);   // an earlier kernel of the call failed

    if (skip) {
        // fall through to the common exit
    } else if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            TWS_DECL;
            for (long long tile = blockIdx.x; tile < p.n_tiles && !failed; tile += gridDim.x) {
                const long long bh = tile / p.tph;
                int qt, kt;
                tcw_tile_of(p.mode, (int)(tile - bh * p.tph), p.nqt, p.nkt, &qt, &kt);
                for (int ci = 0; ci < nch; ++ci, ++it) {
                    // encoding tiles take the chunks in pairs (c, c + nch/2) on neighbouring ring slots
                    const int c = pair_half ? ((ci >> 1) + (ci & 1) * (nch >> 1)) : ci;
                    const int s = it % TW_NST;
                    TWS(0);
                    TW_FAIL_AT(0, !mbar_wait(&bars.empty[s], ((it / TW_NST) & 1) ^ 1, lim));
                    TWS(1);
                    unsigned char *st = smem + (size_t)s * TW_STAGE;
                    mbar_expect_tx(&bars.full[s], TW_STAGE);
                    tma_load_2d(st, &tmQ, c * 64, (int)(bh * p.Lq + qt * TW_BM), &bars.full[s]);
                    tma_load_2d(st + TW_QCHUNK, &tmK, c * 64, (int)(bh * p.Lk + kt * TW_BN), &bars.full[s]);
                }
            }
            TWS_FLUSH(0, true);
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_16(TW_BM, TW_BN, 0, 0, p.f16);
            int it = 0;
            long long tc = 0;
            TWS_DECL;
            for (long long tile = blockIdx.x; tile < p.n_tiles && !failed; tile += gridDim.x, ++tc) {
                const int ab = (int)(tc & 1);
                TWS(2);
                TW_FAIL_AT(1, !mbar_wait(&bars.acc_empty[ab], ((tc >> 1) & 1) ^ 1, lim));
                tc_fence_after();
                TWS(0);
                for (int ci = 0; ci < nch; ++ci, ++it) {
                    const int s = it % TW_NST;
                    TWS(2);
                    TW_FAIL_AT(2, !mbar_wait(encode ? &bars.ready[s] : &bars.full[s], (it / TW_NST) & 1, lim));
                    tc_fence_after();
                    TWS(1);
                    const uint64_t da = umma_desc_k_sw128(smem_u32(smem + (size_t)s * TW_STAGE));
                    const uint64_t db = umma_desc_k_sw128(smem_u32(smem + (size_t)s * TW_STAGE + TW_QCHUNK));
#pragma unroll
                    for (int k = 0; k < 4; ++k) umma_bf16(tmem + ab * TW_BN, da + 2 * k, db + 2 * k, idesc, (ci | k) != 0);
                    umma_commit(&bars.empty[s]);
                }
                if (failed) break;
                umma_commit(&bars.acc_full[ab]);
            }
            TWS_FLUSH(8, true);
        }
    } else if (warp < 6) {
        // ---- epilogue: one thread per query row of the tile ----
        const int row = 32 * (warp & 3) + lane;
        const uint32_t lane_addr = tmem + ((uint32_t)(32 * (warp & 3)) << 16);
        long long tc = 0;
        for (long long tile = blockIdx.x; tile < p.n_tiles && !failed; tile += gridDim.x, ++tc) {
            const long long bh = tile / p.tph;
            int qt, kt;
            tcw_tile_of(p.mode, (int)(tile - bh * p.tph), p.nqt, p.nkt, &qt, &kt);
            const int ab = (int)(tc & 1);
            TW_FAIL_AT(3, !mbar_wait(&bars.acc_full[ab], (tc >> 1) & 1, lim));
            tc_fence_after();
            const uint32_t ta = lane_addr + ab * TW_BN;
            const long long grow = bh * p.Lqp + (long long)qt * TW_BM + row;
            __nv_bfloat16 *srow = p.S + grow * p.Lkp + (long long)kt * TW_BN;
            const float mt = tcw_store_score_row(ta, min(TW_BN, p.Lk - kt * TW_BN), p.scale_log2,
                                                 reinterpret_cast<unsigned char *>(srow - (long long)(lane & 3) * p.Lkp), (size_t)p.Lkp * 2, lane);
            p.rowmax[grow * p.nkt + kt] = mt;
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars.acc_empty[ab]);
        }
    } else if (encode) {
        // ---- transform warps: encoding of the two chunks in ring slots (s, s+1) ----
        // rotate-half couples the two slots (chunks c and c + nch/2); the other encodings treat them
        // independently (chunks 2c and 2c+1), each piece with the table piece of the same row and column.
        // A thread owns 12 of the 3072 16-byte piece pairs of a step: 4 in the Q chunks and 8 in the K
        // chunks, each 32 rows below the last, all in the same logical column.  Where the query rows
        // have the positions of one half of the key rows (kt == qt / 2), Q piece i and K piece
        // i + 4 (qt & 1) use the same table values: the step then needs 8 table fetches, not 12.
        // The fetches run through four register slots, each refilled as soon as it has been used:
        // first half of a step = Q piece i and its twin K piece, then slot i takes the values of
        // the i-th remaining K piece; second half = those K pieces, then slot m takes the values of
        // Q piece m of the next step.  Every fetch so has half a step of work to land.
        const int tid = threadIdx.x - 6 * 32;   // 0..255
        const int npairs = nch >> 1;
        const int half = pair_half ? (p.D >> 1) : 64;   // column distance between the chunks of slots s and s+1
        const int cmul = pair_half ? 64 : 128;          // first column of the step's first chunk = c * cmul
        const bool sinus = (p.pe == PE_SINUSOIDAL);
        const bool rotate_k = (p.rotate_k != 0);
        const int r0 = tid >> 3;
        const int qcol = (tid & 7) ^ (r0 & 7);   // logical 16-byte column of all pieces of this thread
        struct Step { long long tile, bh; int qt, kt, c, h; bool valid, shared, store_q, store_k; };
        auto decode = [&](Step &s) {
            s.valid = s.tile < p.n_tiles;
            if (s.valid) {
                s.bh = s.tile / p.tph;
                const int j = (int)(s.tile - s.bh * p.tph);
                tcw_tile_of(p.mode, j, p.nqt, p.nkt, &s.qt, &s.kt);
                s.shared = rotate_k && (s.kt == (s.qt >> 1));          // query rows = half (qt & 1) of the key rows
                s.h = s.shared ? (s.qt & 1) : 0;
                if (p.nkt <= p.nqt) {
                    s.store_q = true;
                    // key tile kt is met by several query tiles: its first meeting stores it
                    s.store_k = rotate_k && ((p.nqt >= 2 * p.nkt - 1) ? ((s.qt & 1) == 0 && (s.qt >> 1) < p.nkt) : (s.qt < p.nkt));
                } else {
                    s.store_q = j < p.nqt;
                    s.store_k = rotate_k;
                }
            }
        };
        auto next_of = [&](const Step &s) {   // the step after s: next chunk pair, or the first of this CTA's next tile
            Step n = s;
            if (++n.c == npairs) { n.c = 0; n.tile += gridDim.x; decode(n); }
            return n;
        };
        auto tab_q = [&](const Step &s, int i) {
            return p.tab + (long long)(s.qt * TW_BM + 32 * i + r0) * p.D + s.c * cmul + qcol * 8;
        };
        auto tab_k = [&](const Step &s, int i) {   // i = 0..7
            return p.tab + (long long)(s.kt * TW_BN + 32 * i + r0) * p.D + s.c * cmul + qcol * 8;
        };
        auto encode_piece = [&](uint4 &lo, uint4 &hi, const uint4 &ta, const uint4 &tb) {
            if (pair_half) {
                tcw_rotate(lo.x, hi.x, ta.x, tb.x);
                tcw_rotate(lo.y, hi.y, ta.y, tb.y);
                tcw_rotate(lo.z, hi.z, ta.z, tb.z);
                tcw_rotate(lo.w, hi.w, ta.w, tb.w);
            } else {
                lo.x = tc_pe_pair(lo.x, ta.x, sinus); hi.x = tc_pe_pair(hi.x, tb.x, sinus);
                lo.y = tc_pe_pair(lo.y, ta.y, sinus); hi.y = tc_pe_pair(hi.y, tb.y, sinus);
                lo.z = tc_pe_pair(lo.z, ta.z, sinus); hi.z = tc_pe_pair(hi.z, tb.z, sinus);
                lo.w = tc_pe_pair(lo.w, ta.w, sinus); hi.w = tc_pe_pair(hi.w, tb.w, sinus);
            }
        };
        uint4 ta[4], tb[4];   // table values for the chunk in slot s (a) and in slot s+1 (b)
        Step cur;
        cur.tile = blockIdx.x; cur.bh = 0; cur.qt = 0; cur.kt = 0; cur.c = 0; cur.h = 0;
        cur.shared = false; cur.store_q = false; cur.store_k = false;
        decode(cur);
#pragma unroll
        for (int i = 0; i < 4; ++i) { ta[i] = make_uint4(0, 0, 0, 0); tb[i] = ta[i]; }
        if (cur.valid) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const __nv_bfloat16 *tp = tab_q(cur, i);
                ta[i] = tcw_ldg_here(tp);
                tb[i] = tcw_ldg_here(tp + half);
            }
        }
        int it = 0;
        TWS_DECL;
        for (long long n = 0; cur.valid && !failed; ++n, it += 2) {
            TWS(3);
            const Step nx = next_of(cur);
            const int s = it % TW_NST;
            TWS(0);
            TW_FAIL_AT(4, !mbar_wait(&bars.full[s], (it / TW_NST) & 1, lim));
            TW_FAIL_AT(5, !mbar_wait(&bars.full[s + 1], (it / TW_NST) & 1, lim));
            TWS(1);
            unsigned char *lo_st = smem + (size_t)s * TW_STAGE, *hi_st = lo_st + TW_STAGE;
            const long long qrow0 = cur.bh * p.Lq + (long long)cur.qt * TW_BM, krow0 = cur.bh * p.Lk + (long long)cur.kt * TW_BN;
            const int gcol = cur.c * cmul + qcol * 8;
            // ---- first half: Q piece i and, with K encoded, the K piece 4h + i ----
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                {
                    const size_t off = (size_t)(tid + 256 * i) * 16;
                    uint4 lo = *reinterpret_cast<uint4 *>(lo_st + off), hi = *reinterpret_cast<uint4 *>(hi_st + off);
                    encode_piece(lo, hi, ta[i], tb[i]);
                    *reinterpret_cast<uint4 *>(lo_st + off) = lo;
                    *reinterpret_cast<uint4 *>(hi_st + off) = hi;
                    if (cur.store_q && cur.qt * TW_BM + 32 * i + r0 < p.Lq) {
                        __nv_bfloat16 *g = p.q_store + (qrow0 + 32 * i + r0) * (long long)p.D + gcol;
                        *reinterpret_cast<uint4 *>(g) = lo;
                        *reinterpret_cast<uint4 *>(g + half) = hi;
                    }
                }
                if (rotate_k) {
                    const int ik = 4 * cur.h + i;   // K piece of the same positions when shared
                    uint4 ka = ta[i], kb = tb[i];
                    if (!cur.shared) {              // different positions: fetch the values now (not pipelined; rare shapes)
                        const __nv_bfloat16 *tp = tab_k(cur, ik);
                        ka = tcw_ldg_here(tp);
                        kb = tcw_ldg_here(tp + half);
                    }
                    const size_t off = (size_t)TW_QCHUNK + (size_t)(tid + 256 * ik) * 16;
                    uint4 lo = *reinterpret_cast<uint4 *>(lo_st + off), hi = *reinterpret_cast<uint4 *>(hi_st + off);
                    encode_piece(lo, hi, ka, kb);
                    *reinterpret_cast<uint4 *>(lo_st + off) = lo;
                    *reinterpret_cast<uint4 *>(hi_st + off) = hi;
                    const int krow = 32 * ik + r0;
                    if (cur.store_k && cur.kt * TW_BN + krow < p.Lk) {
                        __nv_bfloat16 *g = p.k_store + (krow0 + krow) * (long long)p.D + gcol;
                        *reinterpret_cast<uint4 *>(g) = lo;
                        *reinterpret_cast<uint4 *>(g + half) = hi;
                    }
                    // slot i next serves the i-th remaining K piece of this step
                    const __nv_bfloat16 *tp = tab_k(cur, 4 * (1 - cur.h) + i);
                    ta[i] = tcw_ldg_here(tp);
                    tb[i] = tcw_ldg_here(tp + half);
                } else if (nx.valid) {
                    const __nv_bfloat16 *tp = tab_q(nx, i);
                    ta[i] = tcw_ldg_here(tp);
                    tb[i] = tcw_ldg_here(tp + half);
                }
            }
            // ---- second half: the other four K pieces ----
            if (rotate_k) {
#pragma unroll
                for (int m = 0; m < 4; ++m) {
                    const int ik = 4 * (1 - cur.h) + m;
                    const size_t off = (size_t)TW_QCHUNK + (size_t)(tid + 256 * ik) * 16;
                    uint4 lo = *reinterpret_cast<uint4 *>(lo_st + off), hi = *reinterpret_cast<uint4 *>(hi_st + off);
                    encode_piece(lo, hi, ta[m], tb[m]);
                    *reinterpret_cast<uint4 *>(lo_st + off) = lo;
                    *reinterpret_cast<uint4 *>(hi_st + off) = hi;
                    const int krow = 32 * ik + r0;
                    if (cur.store_k && cur.kt * TW_BN + krow < p.Lk) {
                        __nv_bfloat16 *g = p.k_store + (krow0 + krow) * (long long)p.D + gcol;
                        *reinterpret_cast<uint4 *>(g) = lo;
                        *reinterpret_cast<uint4 *>(g + half) = hi;
                    }
                    if (nx.valid) {   // slot m next serves Q piece m of the next step
                        const __nv_bfloat16 *tp = tab_q(nx, m);
                        ta[m] = tcw_ldg_here(tp);
                        tb[m] = tcw_ldg_here(tp + half);
                    }
                }
            }
            TWS(2);
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) { mbar_arrive(&bars.ready[s]); mbar_arrive(&bars.ready[s + 1]); }
            cur = nx;
        }
        TWS_FLUSH(16, tid == 0);
    }

    if (failed) for (int i = 0; i < 2000; ++i) __nanosleep(1000);   // let copies and MMAs in flight drain
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 0) tmem_dealloc(tmem, 512);
}

// ---------------------------------------------------------------------------------------------------
// The same score GEMM with a [256 queries x 256 keys] tile per CTA: two accumulators of 128 rows
// (TMEM columns 0-255 and 256-511) share every K chunk, so an operand chunk pair is 64 KB for eight
// MMAs instead of 48 KB for four, i.e. two thirds of the L2 -> SM bytes per FLOP.  The accumulators
// cannot be double-buffered any more; instead they are staggered: accumulator 0 finishes (and is
// drained by warps 2-5) four MMAs before accumulator 1 (warps 6-9), and the next tile's MMAs into
// accumulator 0 start as soon as it is drained.  Used for launches without the transform (modes 0 and
// 2) when the query tiles pair up; mode 2 relies on both tiles of a pair having the same key tile in
// the encoding launch (tcw_diag_kt with q / 2).
constexpr int T2_THREADS = 320;            // warp 0 TMA, warp 1 MMA, warps 2-5 / 6-9 epilogue of accumulator 0 / 1
constexpr int T2_NST = 3;
constexpr int T2_QCHUNK = 2 * TW_QCHUNK;   // [256 rows x 64 bf16]
constexpr int T2_STAGE = T2_QCHUNK + TW_KCHUNK;

struct T2Bars {
    uint64_t full[T2_NST], empty[T2_NST];
    uint64_t acc_full[2], acc_empty[2];
};

// tile j of a head: query-tile pair qp and key tile kt
__host__ __device__ __forceinline__ void tcw_tile256_of(int mode, int j, int nkt, int *qp, int *kt) {
    if (mode == 0) { *qp = j / nkt; *kt = j - *qp * nkt; }
    else { const int q = j / (nkt - 1), r = j - q * (nkt - 1); *qp = q; *kt = (q % nkt + 1 + r) % nkt; }
}

__global__ void __launch_bounds__(T2_THREADS, 1)
tcw_scores256_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK, const TcwScoreParams p) {
    extern __shared__ unsigned char tw_smem_raw[];
    __shared__ T2Bars bars;
    __shared__ uint32_t tmem_slot;
    const uint32_t raw_addr = smem_u32(tw_smem_raw);
    unsigned char *smem = tw_smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nch = p.nch;
    const uint32_t lim = p.spin_limit;

    if (threadIdx.x == 0) {
        for (int i = 0; i < T2_NST; ++i) { mbar_init(&bars.full[i], 1); mbar_init(&bars.empty[i], 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(&bars.acc_full[i], 1); mbar_init(&bars.acc_empty[i], 4); }
        mbar_fence_init();
        tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK);
    }
    if (warp == 0) tmem_alloc(&tmem_slot, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    bool failed = false;
    const bool skip = (*reinterpret_cast<volatile unsigned *>(p.err) != 0);

    if (skip) {
        // fall through to the common exit
    } else if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            for (long long tile = blockIdx.x; tile < p.n_tiles && !failed; tile += gridDim.x) {
                const long long bh = tile / p.tph;
                int qp, kt;
                tcw_tile256_of(p.mode, (int)(tile - bh * p.tph), p.nkt, &qp, &kt);
                for (int ci = 0; ci < nch; ++ci, ++it) {
                    const int s = it % T2_NST;
                    TW_FAIL_AT(16, !mbar_wait(&bars.empty[s], ((it / T2_NST) & 1) ^ 1, lim));
                    unsigned char *st = smem + (size_t)s * T2_STAGE;
                    mbar_expect_tx(&bars.full[s], T2_STAGE);
                    tma_load_2d(st, &tmQ, ci * 64, (int)(bh * p.Lq + qp * 256), &bars.full[s]);
                    tma_load_2d(st + T2_QCHUNK, &tmK, ci * 64, (int)(bh * p.Lk + kt * TW_BN), &bars.full[s]);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_16(TW_BM, TW_BN, 0, 0, p.f16);
            int it = 0;
            long long tc = 0;
            for (long long tile = blockIdx.x; tile < p.n_tiles && !failed; tile += gridDim.x, ++tc) {
                for (int ci = 0; ci < nch; ++ci, ++it) {
                    const int s = it % T2_NST;
                    TW_FAIL_AT(17, !mbar_wait(&bars.full[s], (it / T2_NST) & 1, lim));
                    tc_fence_after();
                    const uint64_t da0 = umma_desc_k_sw128(smem_u32(smem + (size_t)s * T2_STAGE));
                    const uint64_t da1 = umma_desc_k_sw128(smem_u32(smem + (size_t)s * T2_STAGE + TW_QCHUNK));
                    const uint64_t db = umma_desc_k_sw128(smem_u32(smem + (size_t)s * T2_STAGE + T2_QCHUNK));
                    if (ci == 0) {   // the previous tile's rows 0-127 have been read out of accumulator 0
                        TW_FAIL_AT(18, !mbar_wait(&bars.acc_empty[0], (tc & 1) ^ 1, lim));
                        tc_fence_after();
                    }
#pragma unroll
                    for (int k = 0; k < 4; ++k) umma_bf16(tmem, da0 + 2 * k, db + 2 * k, idesc, (ci | k) != 0);
                    if (ci == nch - 1) umma_commit(&bars.acc_full[0]);
                    if (ci == 0) {
                        TW_FAIL_AT(19, !mbar_wait(&bars.acc_empty[1], (tc & 1) ^ 1, lim));
                        tc_fence_after();
                    }
#pragma unroll
                    for (int k = 0; k < 4; ++k) umma_bf16(tmem + TW_BN, da1 + 2 * k, db + 2 * k, idesc, (ci | k) != 0);
                    umma_commit(&bars.empty[s]);
                }
                if (failed) break;
                umma_commit(&bars.acc_full[1]);
            }
        }
    } else {
        // ---- epilogue: warps 2-5 read accumulator 0 (rows 0-127 of the tile), warps 6-9 accumulator 1 ----
        const int acc = warp >= 6 ? 1 : 0;
        const int row = 128 * acc + 32 * (warp & 3) + lane;
        const uint32_t ta = tmem + ((uint32_t)(32 * (warp & 3)) << 16) + acc * TW_BN;
        long long tc = 0;
        for (long long tile = blockIdx.x; tile < p.n_tiles && !failed; tile += gridDim.x, ++tc) {
            const long long bh = tile / p.tph;
            int qp, kt;
            tcw_tile256_of(p.mode, (int)(tile - bh * p.tph), p.nkt, &qp, &kt);
            TW_FAIL_AT(20, !mbar_wait(&bars.acc_full[acc], tc & 1, lim));
            tc_fence_after();
            const long long grow = bh * p.Lqp + (long long)qp * 256 + row;
            __nv_bfloat16 *srow = p.S + grow * p.Lkp + (long long)kt * TW_BN;
            const float mt = tcw_store_score_row(ta, min(TW_BN, p.Lk - kt * TW_BN), p.scale_log2,
                                                 reinterpret_cast<unsigned char *>(srow - (long long)(lane & 3) * p.Lkp), (size_t)p.Lkp * 2, lane);
            p.rowmax[grow * p.nkt + kt] = mt;
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars.acc_empty[acc]);
        }
    }

    if (failed) for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 0) tmem_dealloc(tmem, 512);
}

// ---------------------------------------------------------------------------------------------------
constexpr int TP_THREADS = 608;   // warp 0 V loads, warp 1 MMA, warps 2-17 softmax and the unit's epilogue, warp 18 S loads
constexpr int TP_VS = 64;         // keys per V stage
constexpr int TP_VW = 256;        // output columns per V stage (one MMA N): a stage is [64 keys x <= 256 columns], 32 KB
constexpr int TP_NV = 3;   // V stage ring depth (32 KB each; TP_NV + TP_NP <= 7 fits the shared memory;
                                        // measured on cfg 4 / cfg 5: 4 + 3 is 1 % faster than 3 + 4, 5 + 2 is 6 % slower)
constexpr int TP_NP = 4;   // score / P buffers (32 KB each)

struct TcwPvParams {
    int Lq, Lk, D;
    int DW, ndp;               // output columns per unit (<= 512, a multiple of 64) and units per query tile
    int nqt, nkt, nblk;        // ceil(Lq / 128), ceil(Lk / 256), ceil(Lk / 128): S has nqt * 128 rows per head, nblk * 128 columns
    long long n_units;         // heads * nqt * ndp
    const float *rowmax;       // as written by tcw_scores_kernel (the scores themselves come through the tensor map)
    int f16;                   // V, P and the output are fp16, else bf16 (the stored scores are bf16 either way)
    __nv_bfloat16 *O;          // [heads * Lq][D] (16-bit elements of the call's format)
    unsigned *err, *err_sys;
    unsigned spin_limit;
};

struct TpBars {
    uint64_t v_full[TP_NV], v_empty[TP_NV];
    uint64_t s_full[TP_NP];    // the score block has landed in the buffer
    uint64_t p_full[TP_NP];    // ... has been turned into P in place
    uint64_t p_empty[TP_NP];   // ... has been read by the block's last MMA
    uint64_t o_full, o_empty;
    uint64_t l_full;           // the sixteen softmax warps have written the unit's row sums
};

// The stored scores of a key block [128 rows x 128 keys] bf16 are loaded by TMA as two
// [128 x 64] boxes with the 128-byte swizzle, which is exactly the K-major operand layout the MMA
// wants for P: the softmax warps turn the block into P IN PLACE (exp2 is element-wise, every
// thread rewrites the 16-byte pieces it read), so no score ever passes through a register before
// it is needed and the P tile needs no second buffer.
__global__ void __launch_bounds__(TP_THREADS, 1)
tcw_pv_kernel(const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmS, const TcwPvParams p) {
    extern __shared__ unsigned char tw_smem_raw[];
    __shared__ TpBars bars;
    __shared__ uint32_t tmem_slot;
    __shared__ float l_smem[2][TW_BM];
    const uint32_t raw_addr = smem_u32(tw_smem_raw);
    unsigned char *smem = tw_smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
    unsigned char *p_smem = smem;                                   // TP_NP x 32 KB
    unsigned char *v_smem = smem + (size_t)TP_NP * TC_P_BYTES;      // TP_NV x 32 KB
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int DW = p.DW, nblk = p.nblk;
    const int v_stage_bytes = TP_VS * TP_VW * 2;   // ring pitch; a stage of the last column part may hold less
    const int nvw = (DW + TP_VW - 1) / TP_VW;      // column parts per 64 keys
    const uint32_t lim = p.spin_limit;

    if (threadIdx.x == 0) {
        for (int i = 0; i < TP_NV; ++i) { mbar_init(&bars.v_full[i], 1); mbar_init(&bars.v_empty[i], 1); }
        for (int i = 0; i < TP_NP; ++i) { mbar_init(&bars.s_full[i], 1); mbar_init(&bars.p_full[i], 16); mbar_init(&bars.p_empty[i], 1); }
        mbar_init(&bars.o_full, 1);
        mbar_init(&bars.o_empty, 16);
        mbar_init(&bars.l_full, 16);
        mbar_fence_init();
        tma_prefetch_desc(&tmV); tma_prefetch_desc(&tmS);
    }
    if (warp == 0) tmem_alloc(&tmem_slot, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    bool failed = false;
    const bool skip = (*reinterpret_cast<volatile unsigned *>(p.err) != 0);

    if (skip) {
        // fall through to the common exit
    } else if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            TWS_DECL;
            for (long long unit = blockIdx.x; unit < p.n_units && !failed; unit += gridDim.x) {
                const int dp = (int)(unit % p.ndp);
                const long long bh = unit / p.ndp / p.nqt;
                for (int t = 0; t < nblk && !failed; ++t)
                    for (int vs = 0; vs < TC_BN / TP_VS && !failed; ++vs)
                        for (int vw = 0; vw < nvw; ++vw, ++it) {
                            const int s = it % TP_NV;
                            const int ng = min(TP_VW, DW - vw * TP_VW) / 64;   // 64-column groups in this stage
                            TWP(1);
                            TW_FAIL_AT(8, !mbar_wait(&bars.v_empty[s], ((it / TP_NV) & 1) ^ 1, lim));
                            TWP(0);
                            // one request: [4 column groups][64 keys][64 columns]; groups beyond the unit's columns
                            // (ng < 4) are fetched too and never read
                            (void)ng;
                            mbar_expect_tx(&bars.v_full[s], (uint32_t)v_stage_bytes);
                            // (the head is a coordinate of its own: key rows beyond the sequence read as zero)
                            tma_load_4d(v_smem + (size_t)s * v_stage_bytes, &tmV, 0, t * TC_BN + vs * TP_VS, (dp * DW + vw * TP_VW) / 64, (int)bh,
                                        &bars.v_full[s]);
                        }
            }
            TWP_FLUSH(0, true);
        }
    } else if (warp == 18) {
        if (lane == 0) {
            long long tg = 0;
            TWS_DECL;
            for (long long unit = blockIdx.x; unit < p.n_units && !failed; unit += gridDim.x) {
                const long long rest = unit / p.ndp;   // = bh * nqt + qt: the row tile of the score matrix
                for (int t = 0; t < nblk; ++t, ++tg) {
                    const int pb = (int)(tg % TP_NP);
                    TWP(1);
                    TW_FAIL_AT(15, !mbar_wait(&bars.p_empty[pb], ((tg / TP_NP) & 1) ^ 1, lim));
                    TWP(0);
                    mbar_expect_tx(&bars.s_full[pb], TC_P_BYTES);
                    tma_load_3d(p_smem + (size_t)pb * TC_P_BYTES, &tmS, 0, (int)(rest * TW_BM), t * 2, &bars.s_full[pb]);   // [2 groups][128 rows][64 keys]
                }
            }
            TWP_FLUSH(4, true);
        }
    } else if (warp == 1) {
        if (lane == 0) {
            int it = 0, ui = 0;
            long long tg = 0;
            TWS_DECL;
            for (long long unit = blockIdx.x; unit < p.n_units && !failed; unit += gridDim.x, ++ui) {
                // the epilogue of the previous unit has read the accumulator
                TWP(3);
                TW_FAIL_AT(9, !mbar_wait(&bars.o_empty, (ui & 1) ^ 1, lim));
                tc_fence_after();
                TWP(0);
                for (int t = 0; t < nblk && !failed; ++t, ++tg) {
                    const int pb = (int)(tg % TP_NP);
                    TWP(3);
                    TW_FAIL_AT(10, !mbar_wait(&bars.p_full[pb], (tg / TP_NP) & 1, lim));
                    tc_fence_after();
                    TWP(1);
                    for (int vs = 0; vs < TC_BN / TP_VS && !failed; ++vs)
                        for (int vw = 0; vw < nvw; ++vw, ++it) {
                            const int s = it % TP_NV;
                            const int N = min(TP_VW, DW - vw * TP_VW);
                            TWP(3);
                            TW_FAIL_AT(11, !mbar_wait(&bars.v_full[s], (it / TP_NV) & 1, lim));
                            tc_fence_after();
                            TWP(2);
#pragma unroll
                            for (int kk = 0; kk < TP_VS / 16; ++kk) {
                                const int kg = vs * (TP_VS / 16) + kk;   // 16-key step within the block, 0..7
                                const uint64_t da = umma_desc_k_sw128(smem_u32(p_smem + (size_t)pb * TC_P_BYTES + (kg >> 2) * (TW_BM * 128))) + 2 * (kg & 3);
                                const uint64_t db = umma_desc_mn_sw128(smem_u32(v_smem + (size_t)s * v_stage_bytes + kk * 2048), TP_VS * 128);
                                umma_bf16(tmem + vw * TP_VW, da, db, umma_idesc_16(TW_BM, N, 0, 1, p.f16), (t | kg) != 0);
                            }
                            umma_commit(&bars.v_empty[s]);
                        }
                    if (failed) break;
                    umma_commit(&bars.p_empty[pb]);
                }
                if (failed) break;
                umma_commit(&bars.o_full);
            }
            TWP_FLUSH(8, true);
        }
    } else {
        // ---- softmax warps: warp w owns rows [8w, 8w+8) of every key block.  Eight lanes cover one
        // 128-byte row of a 64-key half (conflict-free 16-byte accesses), so a thread works on rows
        // 8w + lane/8 and 8w + 4 + lane/8, in both halves: four 16-byte pieces per block.  The offset
        // (tile maximum - row maximum) of row 8w + k for key tile j is kept in lane j % 32 of offs[k], for the 32
        // key tiles (8192 keys) the unit is working through; lane k of `tot` keeps the row maximum itself. ----
        const int w = warp - 2, rl = lane >> 3;
        int ui = 0;
        long long tg = 0;
        TWS_DECL;
        // lane j keeps (tile maximum - row maximum) of key tile j < 32 for each of the warp's eight rows
        auto load_stats = [&](long long g0, float (&oo)[8], float &tt) {
            tt = 0.0f;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const float m = lane < p.nkt ? __ldg(p.rowmax + (g0 + k) * p.nkt + lane) : -INFINITY;
                float mm = m;
                for (int j = lane + 32; j < p.nkt; j += 32) mm = fmaxf(mm, __ldg(p.rowmax + (g0 + k) * p.nkt + j));   // more than 8192 keys
                mm = warp_max(mm);
                oo[k] = m - mm;
                if (lane == k) tt = mm;
            }
        };
        // the same for the next 32 key tiles, from tile kt0 on
        auto next_stats = [&](long long g0, int kt0, float (&oo)[8], float tt) {
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const float m = kt0 + lane < p.nkt ? __ldg(p.rowmax + (g0 + k) * p.nkt + kt0 + lane) : -INFINITY;
                oo[k] = m - __shfl_sync(0xffffffffu, tt, k);
            }
        };
        auto grow0_of = [&](long long unit) {   // row of S and of the maxima: heads are nqt * 128 rows apart there
            return (unit / p.ndp) * (long long)TW_BM + 8 * w;
        };
        float offs[8], offsn[8], tot = 0.0f, totn = 0.0f;
        for (long long unit = blockIdx.x; unit < p.n_units && !failed; unit += gridDim.x, ++ui) {
            const int dp = (int)(unit % p.ndp);
            const long long rest = unit / p.ndp;
            const int qt = (int)(rest % p.nqt);
            const long long bh = rest / p.nqt;
            const long long grow0 = rest * (long long)TW_BM + 8 * w;
            // (the statistics of the unit were loaded while the previous unit was finishing)
            if (ui == 0) load_stats(grow0, offs, tot);
            float lA = 0.0f, lB = 0.0f, offA = 0.0f, offB = 0.0f;
            for (int t = 0; t < nblk; ++t, ++tg) {
                const int pb = (int)(tg % TP_NP);
                if ((t & 1) == 0) {   // a new 256-key tile: fetch this thread's two offsets
                    const int kt = t >> 1;
                    if (kt != 0 && (kt & 31) == 0) next_stats(grow0, kt, offs, tot);
                    float v[8];
#pragma unroll
                    for (int k = 0; k < 8; ++k) v[k] = __shfl_sync(0xffffffffu, offs[k], kt & 31);
                    offA = rl == 0 ? v[0] : rl == 1 ? v[1] : rl == 2 ? v[2] : v[3];
                    offB = rl == 0 ? v[4] : rl == 1 ? v[5] : rl == 2 ? v[6] : v[7];
                }
                TWP(3);
                TW_FAIL_AT(12, !mbar_wait(&bars.s_full[pb], (tg / TP_NP) & 1, lim));
                TWP(0);
                unsigned char *base = p_smem + (size_t)pb * TC_P_BYTES + (8 * w + rl) * 128 + (lane & 7) * 16;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    // i & 1: row A / row B (4 rows = 512 B further); i >> 1: the 64-key half (16 KB further)
                    uint4 *pp = reinterpret_cast<uint4 *>(base + (i & 1) * 512 + (i >> 1) * (TW_BM * 128));
                    const uint4 xv = *pp;
                    const float off = (i & 1) ? offB : offA;
                    const uint32_t x[4] = {xv.x, xv.y, xv.z, xv.w};
                    uint32_t o[4];
                    float sum = 0.0f;
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const float e0 = fast_exp2(__uint_as_float(x[q] << 16) + off);
                        const float e1 = fast_exp2(__uint_as_float(x[q] & 0xffff0000u) + off);
                        sum += e0 + e1;
                        o[q] = pack_16x2(e0, e1, p.f16 != 0);
                    }
                    if (i & 1) lB += sum; else lA += sum;
                    *pp = make_uint4(o[0], o[1], o[2], o[3]);
                }
                TWP(1);
                fence_proxy_async_smem();
                TWP(2);
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars.p_full[pb]);
            }
            if (failed) break;
            const bool have_next = unit + gridDim.x < p.n_units;
            if (have_next) load_stats(grow0_of(unit + gridDim.x), offsn, totn);   // lands while this unit drains
#pragma unroll
            for (int o = 4; o > 0; o >>= 1) {
                lA += __shfl_xor_sync(0xffffffffu, lA, o);
                lB += __shfl_xor_sync(0xffffffffu, lB, o);
            }
            if ((lane & 7) == 0) { l_smem[ui & 1][8 * w + rl] = lA; l_smem[ui & 1][8 * w + 4 + rl] = lB; }
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars.l_full);
            {
                // ---- epilogue of the unit: O / row sum -> bf16 -> global.  A warp may only read the
                // TMEM lane quadrant warp % 4; the four warps of a quadrant share its 32-column groups ----
                const int row = 32 * (warp & 3) + lane;
                const uint32_t lane_addr = tmem + ((uint32_t)(32 * (warp & 3)) << 16);
                TWP(4);
                TW_FAIL_AT(13, !mbar_wait(&bars.l_full, ui & 1, lim));
                TW_FAIL_AT(14, !mbar_wait(&bars.o_full, ui & 1, lim));
                tc_fence_after();
                TWP(5);
                const float inv = 1.0f / l_smem[ui & 1][row];
                __nv_bfloat16 *orow = p.O + (bh * p.Lq + (long long)qt * TW_BM + row) * (long long)p.D + dp * DW;
                uint32_t r[32], wds[32];
                // 64 output columns (128 bytes of the row) at a time; lanes trade pieces so that the
                // stores cover full lines
                unsigned char *row0 = reinterpret_cast<unsigned char *>(orow - (long long)(lane & 3) * p.D);
                for (int cp = (w >> 2); cp < DW / 64; cp += 4) {
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) {
                        tmem_ld32(lane_addr + cp * 64 + hh * 32, r);
                        tmem_ld_wait();
#pragma unroll
                        for (int q = 0; q < 16; ++q)
                            wds[16 * hh + q] = pack_16x2(__uint_as_float(r[2 * q]) * inv, __uint_as_float(r[2 * q + 1]) * inv, p.f16 != 0);
                    }
                    store_rows_128B_transposed_if(row0 + cp * 128, (size_t)p.D * 2, wds, lane, p.Lq - (qt * TW_BM + (row & ~3)));
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars.o_empty);
            }
            TWP(6);
            if (have_next) {
#pragma unroll
                for (int k = 0; k < 8; ++k) offs[k] = offsn[k];
                tot = totn;
            }
        }
        TWP_FLUSH(16, threadIdx.x == 64);
    }

    if (failed) for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 0) tmem_dealloc(tmem, 512);
}
#undef TW_FAIL_AT

// ---- host side ------------------------------------------------------------------------------------
// cos(pos * f_i) in columns [0, D/2) and sin(pos * f_i) in [D/2, D), f_i = base^(-2i/D): the fp32
// arithmetic of the reference's cos/sin caches (final/rope.cu:20-40), rounded once to bf16.
__global__ void tcw_build_half_table(__nv_bfloat16 *table, int L, int D, float base) {
    const long long n = (long long)L * D;
    const int half = D >> 1;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const int pos = (int)(i / D), d = (int)(i % D);
        const int f = d < half ? d : d - half;
        const float freq = 1.0f / powf(base, (2.0f * (float)f) / (float)D);
        const float th = (float)pos * freq;
        table[i] = __float2bfloat16_rn(d < half ? cosf(th) : sinf(th));
    }
}

// The same two table layouts filled from caller-supplied caches [cache_rows][rd] (value of pair i at columns
// 2i and 2i+1, final/rope.cu:20-40) instead of computed angles: half != 0 gives the rotate-half layout
// (needs rd == D), otherwise the element-wise partner layout of tc_build_pe_table (cos at even columns, sin
// at odd ones, identity beyond rd).  Rows beyond the cache are the identity rotation (no real key or query
// has those positions).
__global__ void tcw_table_from_cache(__nv_bfloat16 *table, int L, int D, int rd, int half, int cache_rows, const float *cos_cache,
                                     const float *sin_cache) {
    const long long n = (long long)L * D;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const int pos = (int)(i / D), d = (int)(i % D);
        float v;
        if (half) {
            const int f = d < (D >> 1) ? d : d - (D >> 1);
            v = d < (D >> 1) ? 1.0f : 0.0f;
            if (pos < cache_rows) v = d < (D >> 1) ? cos_cache[(long long)pos * rd + 2 * f] : sin_cache[(long long)pos * rd + 2 * f];
        } else {
            v = (d & 1) ? 0.0f : 1.0f;
            if (pos < cache_rows && d < rd) v = (d & 1) ? sin_cache[(long long)pos * rd + d] : cos_cache[(long long)pos * rd + d];
        }
        table[i] = __float2bfloat16_rn(v);
    }
}

// Optional per-kernel timing (b200attn_debug_kernel_times): while it is switched on, every launch of
// this path is bracketed by two events on its stream; the sums per kernel kind are collected after
// a synchronisation.  Kinds: 0 = score kernel, encoding launch; 1 = score kernel; 2 = P V kernel.
struct TcwTimer {
    static constexpr int kMax = 2048;
    bool on = false;
    int n = 0;
    cudaEvent_t ev[2 * kMax];
    int kind[kMax];
    bool have_events = false;
    void begin(int k, cudaStream_t st) {
        if (!on || n >= kMax) return;
        if (!have_events) { for (int i = 0; i < 2 * kMax; ++i) cudaEventCreate(&ev[i]); have_events = true; }
        kind[n] = k;
        cudaEventRecord(ev[2 * n], st);
    }
    void end(cudaStream_t st) {
        if (!on || n >= kMax) return;
        cudaEventRecord(ev[2 * n + 1], st);
        ++n;
    }
    // ms[0..2] = summed durations per kind, cnt[0..2] = launches per kind; clears the record
    void collect(double *ms, int *cnt) {
        for (int k = 0; k < 3; ++k) { ms[k] = 0.0; cnt[k] = 0; }
        for (int i = 0; i < n; ++i) {
            float t = 0.0f;
            if (cudaEventElapsedTime(&t, ev[2 * i], ev[2 * i + 1]) == cudaSuccess) { ms[kind[i]] += t; cnt[kind[i]]++; }
        }
        n = 0;
    }
};
inline TcwTimer &tcw_timer() { static TcwTimer t; return t; }

// Scratch of the wide path, kept per device and grown on demand.
struct TcwScratch {
    // S, rowmax, rotated Q, rotated K, table, table made from caller caches, key-split partial outputs, their (max, sum)
    void *buf[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    size_t bytes[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    int tab_L = 0, tab_D = 0;
    float tab_base = 0.0f;
    void *get(int i, size_t want) {
        if (want > bytes[i]) {
            if (buf[i]) { cudaDeviceSynchronize(); cudaFree(buf[i]); }
            buf[i] = nullptr; bytes[i] = 0;
            if (i == 4) tab_L = 0;
            if (cudaMalloc(&buf[i], want) != cudaSuccess) { (void)cudaGetLastError(); return nullptr; }
            bytes[i] = want;
        }
        return buf[i];
    }
    void release() {
        for (int i = 0; i < 8; ++i) { if (buf[i]) cudaFree(buf[i]); buf[i] = nullptr; bytes[i] = 0; }
        tab_L = 0;
    }
};

// The rotate-half cos/sin table [>= Lt][D] for `base`, kept between calls; nullptr when it cannot be allocated.
inline __nv_bfloat16 *tcw_half_table(TcwScratch &sc, int Lt, int D, float base, cudaStream_t st, std::atomic<unsigned long long> *launches) {
    const bool have = sc.buf[4] && sc.tab_L >= Lt && sc.tab_D == D && sc.tab_base == base;
    __nv_bfloat16 *tab = (__nv_bfloat16 *)(have ? sc.buf[4] : sc.get(4, (size_t)Lt * D * 2));
    if (!tab) return nullptr;
    if (!have) {
        if (sc.tab_L != 0) cudaDeviceSynchronize();   // no kernel may still be reading the table that is replaced
        tcw_build_half_table<<<296, 256, 0, st>>>(tab, Lt, D, base);
        launches->fetch_add(1);
        sc.tab_L = Lt; sc.tab_D = D; sc.tab_base = base;
    }
    return tab;
}

inline bool tcw_supported(const b200attn_args &a, int rd) {
    if (a.dtype != B200ATTN_BF16 && !(a.dtype == B200ATTN_F16 && a.pe == B200ATTN_PE_NONE)) return false;   // the encodings are bf16 arithmetic
    if (a.head_d % 64 != 0 || a.head_d < 64 || a.head_d > 8192) return false;
    if (a.len_q <= 64 && a.len_k <= 64) return false;   // short sequences: the split-head_d kernels
    if (a.len_k > 65536) return false;
    if (a.cos_cache != nullptr && !pe_is_rope(a.pe)) return false;
    if (pe_pairs_halves(a.pe)) { if (a.head_d % 128 != 0 || rd != a.head_d) return false; }
    else if (a.pe != B200ATTN_PE_NONE) { if (a.head_d % 128 != 0 || (a.pe != B200ATTN_PE_SINUSOIDAL && rd % 8 != 0)) return false; }
    if ((((uintptr_t)a.Q | (uintptr_t)a.K | (uintptr_t)a.V | (uintptr_t)a.out) & 15) != 0) return false;
    if (((uintptr_t)a.out & 31) != 0) return false;   // the epilogue stores 32 bytes at a time
    const long long BH = (long long)a.batch_sz * a.num_heads;
    if (BH * (a.len_q + 128) >= (1ll << 31) || BH * (a.len_k + 256) >= (1ll << 31)) return false;
    return true;
}

// Returns B200ATTN_OK, -1 when the shape should run on another path (also when the scratch could not be
// allocated: nothing has been launched then), or a status with tc_bf16_error() set.
inline int tcw_run(const b200attn_args &a, int rd, float base, TcwScratch &sc, TcTables &tables, unsigned *err_dev, unsigned *err_sys, int sm_count,
                   unsigned spin_limit, size_t score_scratch_cap, cudaStream_t st, std::atomic<unsigned long long> *launches) {
    const long long BH = (long long)a.batch_sz * a.num_heads;
    const int D = a.head_d, Lq = a.len_q, Lk = a.len_k;
    const bool encoded = (a.pe != B200ATTN_PE_NONE);              // any encoding: two score launches
    const bool pair_half = pe_pairs_halves(a.pe);
    const bool rotate_k = pe_encodes_k(a.pe);
    int ndp = 1;
    while (D % (64 * ndp) != 0 || D / ndp > 512) ++ndp;
    const int DW = D / ndp;
    // any lengths: S and the maxima are kept with both lengths rounded up to whole 128-blocks
    const int nqt = (Lq + TW_BM - 1) / TW_BM, nkt = (Lk + TW_BN - 1) / TW_BN, nblk = (Lk + TC_BN - 1) / TC_BN;
    const int Lqp = nqt * TW_BM, Lkp = nblk * TC_BN;
    const size_t smem_s = (size_t)TW_NST * TW_STAGE + 1024;
    const size_t smem_p = (size_t)TP_NP * TC_P_BYTES + (size_t)TP_NV * TP_VS * TP_VW * 2 + 1024;
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
            bool ok = cudaFuncGetAttributes(&fa, tcw_scores_kernel) == cudaSuccess &&
                      cudaFuncSetAttribute(tcw_scores_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(prop.sharedMemPerBlockOptin - fa.sharedSizeBytes)) == cudaSuccess;
            ok = ok && cudaFuncGetAttributes(&fa, tcw_scores256_kernel) == cudaSuccess &&
                 cudaFuncSetAttribute(tcw_scores256_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(prop.sharedMemPerBlockOptin - fa.sharedSizeBytes)) == cudaSuccess;
            ok = ok && cudaFuncGetAttributes(&fa, tcw_pv_kernel) == cudaSuccess &&
                 cudaFuncSetAttribute(tcw_pv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(prop.sharedMemPerBlockOptin - fa.sharedSizeBytes)) == cudaSuccess;
            if (!ok) { (void)cudaGetLastError(); snprintf(t_tc_error, sizeof t_tc_error, "cudaFuncSetAttribute(max dynamic shared memory) failed"); return B200ATTN_ERR_CUDA; }
            attr_done[dev & 63] = true;
        }
    }
    // heads per pass: the score scratch of one pass stays below a cap (default 2 GiB)
    const size_t cap = score_scratch_cap;
    const size_t s_head = (size_t)Lqp * Lkp * sizeof(__nv_bfloat16);
    long long G = (long long)(cap / s_head);
    if (G < 1) G = 1;
    if (G > BH) G = BH;
    __nv_bfloat16 *S = (__nv_bfloat16 *)sc.get(0, (size_t)G * s_head);
    float *rowmax = (float *)sc.get(1, (size_t)G * Lqp * nkt * sizeof(float));
    __nv_bfloat16 *qs = nullptr, *ks = nullptr, *tab = nullptr;
    if (!S || !rowmax) { snprintf(t_tc_error, sizeof t_tc_error, "could not allocate the score scratch"); return -1; }
    if (encoded) {
        qs = (__nv_bfloat16 *)sc.get(2, (size_t)G * Lq * D * 2);
        ks = (__nv_bfloat16 *)sc.get(3, (size_t)G * Lk * D * 2);
        const int Lt = (Lqp > nkt * TW_BN ? Lqp : nkt * TW_BN);
        if (!qs || !ks) { snprintf(t_tc_error, sizeof t_tc_error, "could not allocate the rotated-operand scratch"); return -1; }
        if (a.cos_cache != nullptr) {
            // the caller's angles: the table is rebuilt on every call (the caches may have changed)
            tab = (__nv_bfloat16 *)sc.get(5, (size_t)Lt * D * 2);
            if (!tab) { snprintf(t_tc_error, sizeof t_tc_error, "could not allocate the cos/sin table"); return -1; }
            tcw_table_from_cache<<<296, 256, 0, st>>>(tab, Lt, D, rd, pair_half ? 1 : 0, Lq > Lk ? Lq : Lk, a.cos_cache, a.sin_cache);
            launches->fetch_add(1);
        } else if (pair_half) {
            tab = tcw_half_table(sc, Lt, D, base, st, launches);
            if (!tab) { snprintf(t_tc_error, sizeof t_tc_error, "could not allocate the cos/sin table"); return -1; }
        } else {
            int rows = 0;
            tab = tables.get(a.pe, Lt, D, rd, a.pe == B200ATTN_PE_SINUSOIDAL ? 10000.0f : base, st, launches, &rows);
            if (!tab) { snprintf(t_tc_error, sizeof t_tc_error, "could not allocate the positional-encoding table"); return -1; }
        }
    }
    for (long long h0 = 0; h0 < BH; h0 += G) {
        const long long nh = (BH - h0 < G) ? BH - h0 : G;
        const __nv_bfloat16 *Qg = (const __nv_bfloat16 *)a.Q + h0 * Lq * D, *Kg = (const __nv_bfloat16 *)a.K + h0 * Lk * D;
        const __nv_bfloat16 *Vg = (const __nv_bfloat16 *)a.V + h0 * Lk * D;
        TcwScoreParams sp{};
        sp.Lq = Lq; sp.Lk = Lk; sp.Lqp = Lqp; sp.Lkp = Lkp; sp.D = D; sp.nch = D / 64; sp.nqt = nqt; sp.nkt = nkt;
        sp.scale_log2 = 1.4426950408889634f / sqrtf((float)D);
        sp.f16 = a.dtype == B200ATTN_F16 ? 1 : 0;
        sp.S = S; sp.rowmax = rowmax; sp.tab = tab; sp.q_store = qs; sp.k_store = ks;
        sp.pe = a.pe == B200ATTN_PE_ROPE_Q_ONLY ? (int)PE_ROPE_INTERLEAVED : a.pe == B200ATTN_PE_ROPE_HALF_Q_ONLY ? (int)PE_ROPE_HALF : a.pe;
        sp.rotate_k = rotate_k ? 1 : 0;
        sp.err = err_dev; sp.err_sys = err_sys; sp.spin_limit = spin_limit;
        // launches without the transform use the [256 x 256] tile kernel when the query tiles pair up
        // (and, for the complement of the encoding launch, when both tiles of a pair met the same key tile there)
        const bool big_ok = (nqt % 2 == 0);
        auto launch_scores = [&](const void *Qp, const void *Kp, int mode, int tph) -> int {
            if (tph <= 0) return B200ATTN_OK;
            const bool big = big_ok && (mode == 0 || (mode == 2 && nkt <= nqt && nqt >= 2 * nkt - 1));
            CUtensorMap tmQ, tmK;
            if (!tc_make_map(&tmQ, Qp, nh * Lq, D, big ? 256 : TW_BM) || !tc_make_map(&tmK, Kp, nh * Lk, D, TW_BN)) {
                snprintf(t_tc_error, sizeof t_tc_error, "cuTensorMapEncodeTiled failed");
                return B200ATTN_ERR_CUDA;
            }
            if (big) tph /= 2;   // tiles of two query tiles each
            sp.mode = mode; sp.tph = tph; sp.n_tiles = nh * tph;
            const unsigned grid = (unsigned)(sp.n_tiles < sm_count ? sp.n_tiles : sm_count);
            tcw_timer().begin(mode == 1 ? 0 : 1, st);
            if (big) tcw_scores256_kernel<<<grid, T2_THREADS, (size_t)T2_NST * T2_STAGE + 1024, st>>>(tmQ, tmK, sp);
            else tcw_scores_kernel<<<grid, TW_THREADS, smem_s, st>>>(tmQ, tmK, sp);
            tcw_timer().end(st);
            cudaError_t e = cudaGetLastError();
            if (e != cudaSuccess) { snprintf(t_tc_error, sizeof t_tc_error, "score kernel launch failed: %s", cudaGetErrorString(e)); return B200ATTN_ERR_CUDA; }
            launches->fetch_add(1);
            return B200ATTN_OK;
        };
        CUtensorMap tmV, tmS;
        const bool maps_ok = make_tmap_grouped_heads(&tmV, Vg, nh, Lk, D, TP_VS, TP_VW / 64) && make_tmap_grouped(&tmS, S, nh * Lqp, Lkp, TW_BM, 2);
        if (!maps_ok) { snprintf(t_tc_error, sizeof t_tc_error, "cuTensorMapEncodeTiled failed"); return h0 == 0 ? -1 : B200ATTN_ERR_CUDA; }
        int rc;
        if (encoded) {
            const int nA = nqt > nkt ? nqt : nkt;
            rc = launch_scores(Qg, Kg, 1, nA);
            if (rc == B200ATTN_OK) rc = launch_scores(qs, rotate_k ? (const void *)ks : (const void *)Kg, 2, nqt * nkt - nA);
        } else {
            rc = launch_scores(Qg, Kg, 0, nqt * nkt);
        }
        if (rc) return rc;
        TcwPvParams pp{};
        pp.Lq = Lq; pp.Lk = Lk; pp.D = D; pp.DW = DW; pp.ndp = ndp; pp.nqt = nqt; pp.nkt = nkt; pp.nblk = nblk;
        pp.n_units = nh * nqt * ndp;
        pp.f16 = a.dtype == B200ATTN_F16 ? 1 : 0;
        pp.rowmax = rowmax; pp.O = (__nv_bfloat16 *)a.out + h0 * Lq * D;
        pp.err = err_dev; pp.err_sys = err_sys; pp.spin_limit = spin_limit;
        tcw_timer().begin(2, st);
        {
            const unsigned grid = (unsigned)(pp.n_units < sm_count ? pp.n_units : sm_count);
            tcw_pv_kernel<<<grid, TP_THREADS, smem_p, st>>>(tmV, tmS, pp);
        }
        tcw_timer().end(st);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) { snprintf(t_tc_error, sizeof t_tc_error, "tcw_pv_kernel launch failed: %s", cudaGetErrorString(e)); return B200ATTN_ERR_CUDA; }
        launches->fetch_add(1);
    }
    return B200ATTN_OK;
}

}  // namespace b200attn
