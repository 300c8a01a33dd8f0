// fp32 attention forward for short sequences (len_q, len_k <= 64) and wide heads on the tensor cores:
// the split-head_d decomposition of splitd.cuh (a CTA owns a column slice of Q, K and V of one head,
// every input byte is read from HBM once) with both contractions done by tcgen05.mma.kind::tf32 on
// error-compensated operands, so that the result keeps fp32 accuracy.
//
// An fp32 value x is split into hi = x with the low 13 mantissa bits cleared (exactly representable
// as tf32) and the residual lo = x - hi (exact in fp32, at most 13 significant bits, of which the
// tensor core keeps 11).  A product a*b is taken as hi_a*hi_b + hi_a*lo_b + lo_a*hi_b (+ lo_a*lo_b, which is
// below 2^-22 |a b| and comes for free) with fp32 accumulation.  (Replaces the scalar loops of the reference
// kernel, final/attention.cu:120-142 and :169-181; the reference's own arithmetic is fp32 FMA, and the result
// here agrees with it to a few 1e-7.)
//
//   load      Q and K as 32-column "atoms" (128 bytes per row, 128-byte swizzle: the K-major operand
//             layout of the MMA) into landing slots, V as [keys x 32 columns] slabs with the 128-byte swizzle
//             on 32-byte units, the M-major operand layout of 32-bit elements.  A call on its own requests its
//             whole slice when the CTA starts (the bytes in flight per SM are what decides the HBM rate).  A
//             call of a batch, which runs beside its neighbours in the stream, takes a compact form: fewer
//             landing slots than atoms (a slot is requested again as soon as it has been split), and V lands
//             over the slots and stages when the score MMAs are done, under the wait for the other slices - a
//             CTA of the widest slice then takes half of an SM's shared memory, narrower ones a third.
//   split     six warps write each landed atom as Q hi | Q lo | K hi | K lo into an operand stage;
//   scores    one thread issues, per 8 columns, two MMAs of M = 64, N = 128 into one accumulator:
//             Q hi [K hi; K lo]^T and Q lo [K hi; K lo]^T (M = 64: the accumulator row r sits in tensor-memory
//             lane 32*(r/16) + r%16); a row's score is the sum of its two column halves;
//   reduce    the partial scores of the slices of a head are summed in an L2-resident scratch with
//             16-byte vector reductions; a per-head arrival counter tells when the sum is complete.
//             All CTAs of a call are resident together (the host sizes the grid and the shared memory for
//             that); the wait is bounded all the same and reports an error instead of hanging.
//   softmax   every slice CTA reads the 64 x 64 scores back, half a warp per row (shuffle max / sum);
//   output    O[:, slice]^T = V^T P^T per block of 128 output columns: V hi and V lo in turn as the M-major
//             A operand (M = 128: an output column per tensor-memory lane), [P hi | P lo] as one K-major B
//             operand of N = 128; the thread of a column adds a row's hi and lo halves and a warp stores 128
//             contiguous bytes of an output row.  P and V lo live where the atoms were; where that room is
//             short the contraction runs in two passes of 32 keys, V lo and P of the second pass replacing
//             those of the first.
//
// Consecutive independent calls overlap on the GPU (programmatic dependent launch: a call's kernel starts
// while the one before it is still running, and two or three CTAs share an SM).
// The score scratch is therefore a ring of ST_NBUF buffers: call n sums into buffer n % ST_NBUF; the last
// slice CTA of a head to have read the head's scores clears them (off the critical path, during P V) and
// bumps the buffer's generation counter; a later call that gets the same buffer first checks (at its
// start, long before it needs it) that the generation has reached what its predecessors must have left.
#pragma once

#include "tc_common.cuh"

namespace b200attn {

constexpr int ST_THREADS = 256;        // warp 0: TMA + arrival counter, warp 1: MMA, warps 2-7: split, warps 4-7: score read-out
constexpr int ST_SPLIT_THREADS = 192;
constexpr int ST_ATOM = 32;            // fp32 columns in a 128-byte swizzled row
constexpr int ST_SLAB = 64 * 128;      // [64 rows x 128 B]
constexpr int ST_CHUNK = 2 * ST_SLAB;  // the unit of the shared-memory layout: one atom of Q and of K as it lands, or two slabs of V
constexpr int ST_STAGE = 2 * ST_CHUNK; // an atom as the score MMAs take it: Q hi | Q lo | K hi | K lo
constexpr int ST_MAX_ATOMS = 8;        // widest slice: 256 columns (two blocks of 128 output columns)
constexpr int ST_MAX_SLOTS = 8;        // landing slots
constexpr int ST_NST = 2;              // operand stages (one in the most compact form)
constexpr int ST_NBUF = 8;             // score-scratch ring

struct SdtcParams {
    long long BH;
    int Lq, Lk, D;
    int apc;                 // atoms per slice
    int natoms;              // ceil(D / 32)
    int nsplit;              // slices per head
    int buf;                 // which buffer of the scratch ring this call sums into
    unsigned gen_expect;     // heads that earlier calls must have cleared in that buffer before it is used
    int tmem_cols;           // tensor-memory columns to allocate (128 or 256)
    int nr;                  // landing slots (16 KB each)
    int nst;                 // operand stages (32 KB each): 1 or 2
    int v_own;               // 1: V has shared memory of its own behind the stages and is requested at once;
                             // 0: V lands over the stages once the score MMAs are done
    int kc;                  // keys per pass of the P V contraction: 64 (one pass) or 32
    float scale;
    float *O;                // [B*H*Lq][D]
    float *S;                // [ST_NBUF][cap_bh][64][64] partial-score sums; all zero outside the heads in use
    unsigned *counters;      // [ST_NBUF][cap_bh][2]: read-out warps (four per slice) that have added their scores; slices that have read the sum
    unsigned *gen;           // [ST_NBUF] heads cleared so far, per buffer
    int cap_bh;              // heads each buffer has room for
    unsigned *err, *err_sys;
    unsigned spin_limit;
    unsigned wait_extra;     // 0; a test makes the head wait for arrivals that never come
#ifdef B200ATTN_DEVTOOLS
    float *dbg;              // bring-up dump of CTA (0, 0): see the ST_DBG sites
    unsigned long long *stamps;   // [CTAs][32] globaltimer at the ST_STAMP sites
#endif
};

struct StBars {
    uint64_t full[ST_MAX_SLOTS];            // slot c % nr: atom c of Q and K has landed
    uint64_t raw_free[ST_MAX_SLOTS];        // slot c % nr: the split warps have read atom c
    uint64_t ready[ST_NST], st_free[ST_NST];   // stage c % nst: operands written / read by the MMAs
    uint64_t v_full, s_full, o_full;
    uint64_t buf_ok;                        // the scratch buffer has been cleared by its previous users
};

// The kernel's barriers and flags live in the dynamic allocation too (no static shared memory), in the
// kilobyte that aligning the tiles to 1024 bytes leaves over.
struct StShared {
    StBars bars;
    uint32_t tmem_slot;
    unsigned s_fail;
};
static_assert(sizeof(StShared) <= 512, "the barriers have to fit the alignment slack");

// Shared memory of a CTA in units of 16 KB: landing slots | operand stages | V (v_own), + 1 KB (alignment of the
// tiles, barriers).
//   while the scores are computed   TMA lands atom c of Q and K in slot c % nr; the split warps write it as
//                                   Q hi | Q lo | K hi | K lo into stage c % nst (the slot is free again at once);
//   afterwards                      V (hi in place) in the last 2 * ceil(apc / 4) units - its own, requested when the
//                                   CTA starts, or the last of the stages and slots, requested when the last score
//                                   MMA is done;
//                                   everything below holds P of a pass and V lo of a pass.
inline int sdtc_vblocks(int apc) { return (apc + 3) / 4; }
inline int sdtc_units(int apc, int nr, int nst, int v_own) { return nr + 2 * nst + (v_own ? 2 * sdtc_vblocks(apc) : 0); }
inline size_t sdtc_smem_bytes(int apc, int nr, int nst, int v_own) { return (size_t)sdtc_units(apc, nr, nst, v_own) * ST_CHUNK + 1024; }
// P [hi | lo] of a pass is kc / 32 units, V lo of a pass the same per block of four atoms
inline bool sdtc_layout_ok(int apc, int nr, int nst, int v_own, int kc) {
    const int nb = sdtc_vblocks(apc);
    return nr >= 1 && nr <= ST_MAX_SLOTS && nst >= 1 && nst <= ST_NST && (1 + nb) * (kc / 32) <= sdtc_units(apc, nr, nst, v_own) - 2 * nb;
}

// x -> (x with the low 13 mantissa bits cleared, the exact remainder)
__device__ __forceinline__ void st_split4(const float4 x, float4 &hi, float4 &lo) {
    hi.x = __uint_as_float(__float_as_uint(x.x) & 0xffffe000u); lo.x = x.x - hi.x;
    hi.y = __uint_as_float(__float_as_uint(x.y) & 0xffffe000u); lo.y = x.y - hi.y;
    hi.z = __uint_as_float(__float_as_uint(x.z) & 0xffffe000u); lo.z = x.z - hi.z;
    hi.w = __uint_as_float(__float_as_uint(x.w) & 0xffffe000u); lo.w = x.w - hi.w;
}

// byte offset of fp32 element (row, col) of a [64 rows x 32 columns] slab in the 128-byte swizzle
__device__ __forceinline__ uint32_t st_swz(int row, int col) {
    return (uint32_t)((row >> 3) * 1024 + (row & 7) * 128 + ((((col >> 2) ^ (row & 7)) << 4)) + (col & 3) * 4);
}

// V hi in place and V lo (kc * 128 bytes per atom) for the key rows [k0, k0 + kc) of every atom, by the 192
// threads of the split warps; key rows [Lk, kpad) enter the contraction and are written as zero
__device__ __forceinline__ void st_split_v(unsigned char *v_hi, unsigned char *v_lo, int nat, int k0, int kc, int kpad, int Lk, int t) {
    const int sh = kc == 64 ? 9 : 8;   // 16-byte pieces per atom and pass: kc * 8
    for (int idx = t; idx < (nat << sh); idx += ST_SPLIT_THREADS) {
        const int a = idx >> sh, i = idx & ((1 << sh) - 1), row = k0 + (i >> 3);
        if (row < kpad) {
            float4 *ph = reinterpret_cast<float4 *>(v_hi + (size_t)a * ST_SLAB + (size_t)k0 * 128 + (size_t)i * 16);
            float4 hi = make_float4(0.f, 0.f, 0.f, 0.f), lo = hi;
            if (row < Lk) st_split4(*ph, hi, lo);
            *ph = hi;
            *reinterpret_cast<float4 *>(v_lo + ((size_t)idx << 4)) = lo;   // a * kc * 128 + i * 16
        }
    }
}

// 4 x 4 transpose across the four lanes of a quad: on entry x[r] belongs to (this lane's column, row r); on exit
// x[c] belongs to (column c of the quad, row = this lane's place in the quad)
__device__ __forceinline__ void st_quad_transpose(float &x0, float &x1, float &x2, float &x3, int lane) {
    const bool b0 = lane & 1, b1 = lane & 2;
    float r = __shfl_xor_sync(0xffffffffu, b0 ? x0 : x1, 1);
    if (b0) x0 = r; else x1 = r;
    r = __shfl_xor_sync(0xffffffffu, b0 ? x2 : x3, 1);
    if (b0) x2 = r; else x3 = r;
    r = __shfl_xor_sync(0xffffffffu, b1 ? x0 : x2, 2);
    if (b1) x0 = r; else x2 = r;
    r = __shfl_xor_sync(0xffffffffu, b1 ? x1 : x3, 2);
    if (b1) x1 = r; else x3 = r;
}

#ifdef B200ATTN_DEVTOOLS
#define ST_DBG(slot, expr) do { if (p.dbg && blockIdx.x == 0 && blockIdx.y == 0) { expr; } } while (0)
#define ST_STAMP(k) do { if (p.stamps) { unsigned long long t_; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_)); \
    p.stamps[((size_t)blockIdx.y * gridDim.x + blockIdx.x) * 32 + (k)] = t_; } } while (0)
#else
#define ST_DBG(slot, expr)
#define ST_STAMP(k)
#endif

#define ST_FAIL_AT(site, cond)                                                                       \
    if (cond) {                                                                                      \
        report_kernel_error(p.err, p.err_sys, (unsigned)KERR_MBAR_TIMEOUT | (1u << (7 + (site))));   \
        *reinterpret_cast<volatile unsigned *>(&s_fail) = 1u;                                        \
        failed = true;                                                                               \
        break;                                                                                       \
    }

__global__ void __launch_bounds__(ST_THREADS, 3)
sdtc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
            const SdtcParams p) {
    extern __shared__ __align__(256) unsigned char st_smem_raw[];
    if (threadIdx.x == 0) ST_STAMP(0);
    const uint32_t raw_addr = smem_u32(st_smem_raw);
    const uint32_t slack = (1024u - (raw_addr & 1023u)) & 1023u;   // 0, 256, 512 or 768
    unsigned char *smem = st_smem_raw + slack;
    const int nr = p.nr, nst = p.nst, nblk = (p.apc + 3) >> 2;
    const int units = nr + 2 * nst + (p.v_own ? 2 * nblk : 0);
    const size_t tile_bytes = (size_t)units * ST_CHUNK;
    // the 1 KB beyond the tiles is split into `slack` bytes before them and the rest behind them: the
    // barriers go where 512 bytes fit
    StShared &sh = *reinterpret_cast<StShared *>(slack >= 512 ? st_smem_raw : smem + tile_bytes);
    StBars &bars = sh.bars;
    uint32_t &tmem_slot = sh.tmem_slot;
    unsigned &s_fail = sh.s_fail;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int slice = blockIdx.x;
    const long long bh = blockIdx.y;
    const int Lq = p.Lq, Lk = p.Lk;
    // The slice of CTA s is the atoms s, s + nsplit, s + 2 nsplit, ...: at any moment the CTAs of a head
    // are then fetching neighbouring 128-byte pieces of the same rows, which DRAM serves from open pages.
    const int nat = (p.natoms - slice + p.nsplit - 1) / p.nsplit;   // >= 1: nsplit <= natoms
    auto atom_col = [&](int c) { return (slice + c * p.nsplit) * ST_ATOM; };
    const int kpad = (Lk + 7) & ~7;              // keys covered by the P V contraction (8 per MMA)
    const uint32_t lim = p.spin_limit;

    unsigned char *raw = smem;                                       // nr landing slots: Q [64 x 32] | K [64 x 32]
    unsigned char *stages = smem + (size_t)nr * ST_CHUNK;            // nst stages: Q hi | Q lo | K hi | K lo
    unsigned char *v_hi = smem + (size_t)(units - 2 * nblk) * ST_CHUNK;   // afterwards: slab a = V[:, atom a] [keys x 32 columns]
    // below V, once the score MMAs are done: P of a pass (per 32 keys: hi [64 x 32] | lo [64 x 32], one N = 128
    // operand) and V lo of a pass (kc keys of every atom)
    const int kc = p.kc, pslabs = kc >> 5;
    const uint32_t vlo_pitch = (uint32_t)kc * 128u;
    unsigned char *p_buf = smem;
    unsigned char *v_lo = smem + (size_t)pslabs * ST_CHUNK;

    float *S_cur = p.S + ((size_t)p.buf * p.cap_bh + bh) * 4096;
    unsigned *cnt_cur = p.counters + ((size_t)p.buf * p.cap_bh + bh) * 2;   // [0] arrivals, [1] readers

    // requests of thread 0
    auto load_atom = [&](int c, int r) {   // atom c into landing slot r = c % nr
        unsigned char *st = raw + (size_t)r * ST_CHUNK;
        mbar_expect_tx(&bars.full[r], (uint32_t)(Lq + Lk) * 128u);
        tma_load_2d(st, &tmQ, atom_col(c), (int)(bh * Lq), &bars.full[r]);
        tma_load_2d(st + ST_SLAB, &tmK, atom_col(c), (int)(bh * Lk), &bars.full[r]);
    };
    auto load_v = [&]() {
        for (int a = 0; a < nat; ++a) tma_load_2d(v_hi + (size_t)a * ST_SLAB, &tmV, atom_col(a), (int)(bh * Lk), &bars.v_full);
    };

    // one thread sets the barriers up and at once requests what has room: the first nr atoms of Q and K, then V
    // if it has room of its own (a second issuing thread, or V requested alongside, measured no faster): the
    // loads are in flight while the other warps allocate tensor memory and meet at the barrier below
    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
        for (int i = 0; i < ST_MAX_SLOTS; ++i) { mbar_init(&bars.full[i], 1); mbar_init(&bars.raw_free[i], 6); }
        for (int i = 0; i < ST_NST; ++i) { mbar_init(&bars.ready[i], 6); mbar_init(&bars.st_free[i], 1); }
        mbar_init(&bars.v_full, 1);
        mbar_init(&bars.s_full, 1);
        mbar_init(&bars.o_full, 1);
        mbar_init(&bars.buf_ok, 1);
        s_fail = 0u;
        mbar_fence_init();
        for (int c = 0; c < nat && c < nr; ++c) load_atom(c, c);
        mbar_expect_tx(&bars.v_full, (uint32_t)nat * (uint32_t)Lk * 128u);
        if (p.v_own) load_v();
    }
    if (warp == 1) tmem_alloc(&tmem_slot, (uint32_t)p.tmem_cols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    bool failed = false;
    if (threadIdx.x == 0) ST_STAMP(1);
    // a following call that was declared independent of this one may start its loads now
    grid_launch_dependents();

    if (warp == 0) {
        if (lane == 0) {
            // ---- the buffer of the scratch ring is clean once its earlier users have cleared their heads ----
            unsigned seen = 0;
            for (unsigned it = 0; it < lim; ++it) {
                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(p.gen + p.buf) : "memory");
                if ((int)(seen - p.gen_expect) >= 0) break;
                __nanosleep(100);
            }
            if ((int)(seen - p.gen_expect) < 0) {
                report_kernel_error(p.err, p.err_sys, (unsigned)KERR_HEAD_BARRIER_TIMEOUT | (1u << 20));
                *reinterpret_cast<volatile unsigned *>(&s_fail) = 1u;
            }
            mbar_arrive(&bars.buf_ok);
            // ---- the atoms beyond the landing slots follow as the split warps hand slots back; V lands over the
            // stages once the last score MMA has read them ----
            bool ok = true;
            // (slot and parity are counted along: a division by the run-time slot count costs a lone thread ~100 clocks)
            for (int c = nr, r = 0, par = 0; c < nat && ok; ++c) {
                ok = mbar_wait(&bars.raw_free[r], (uint32_t)par, lim);
                if (ok) load_atom(c, r);
                if (++r == nr) { r = 0; par ^= 1; }
            }
            if (ok && !p.v_own) {
                ok = mbar_wait(&bars.s_full, 0, lim);
                if (ok) load_v();
            }
            if (!ok) {
                report_kernel_error(p.err, p.err_sys, (unsigned)KERR_MBAR_TIMEOUT | (1u << 16));
                *reinterpret_cast<volatile unsigned *>(&s_fail) = 1u;
            }
            // ---- the head's scores are complete when every read-out warp of every slice has arrived ----
            const unsigned want = 4u * (unsigned)p.nsplit + p.wait_extra;
            seen = 0;
            for (unsigned it = 0; it < lim; ++it) {
                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(cnt_cur) : "memory");
                if (seen >= want) break;
                __nanosleep(20);
            }
            ST_STAMP(7);
            if (seen < want) {
                report_kernel_error(p.err, p.err_sys, (unsigned)KERR_HEAD_BARRIER_TIMEOUT);
                *reinterpret_cast<volatile unsigned *>(&s_fail) = 1u;
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- score MMAs: per 8 columns two M = 64, N = 128 MMAs into one accumulator, Q hi [K hi; K lo]^T and
            // Q lo [K hi; K lo]^T: a row's products with K hi in columns 0-63, with K lo in columns 64-127 ----
            const uint32_t id = umma_idesc_tf32(64, 128, 0, 0);
            for (int c = 0, j = 0, jph = 0; c < nat; ++c, jph ^= (j + 1 == nst), j = (j + 1 == nst) ? 0 : j + 1) {
                ST_FAIL_AT(2, !mbar_wait(&bars.ready[j], (uint32_t)jph, lim));
                if (c == nat - 1) ST_STAMP(18);
                tc_fence_after();
                const uint32_t sa = smem_u32(stages + (size_t)j * ST_STAGE);
                const uint64_t dq = umma_desc_k_sw128(sa), dk = umma_desc_k_sw128(sa + ST_CHUNK);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    umma_tf32(tmem, dq + 2 * k, dk + 2 * k, id, (c | k) != 0);
                    umma_tf32(tmem, dq + (ST_SLAB >> 4) + 2 * k, dk + 2 * k, id, 1u);
                }
                umma_commit(&bars.st_free[j]);
            }
            if (!failed) umma_commit(&bars.s_full);
            ST_STAMP(19);
        }
    } else {
        const int t = threadIdx.x - 64;   // 0..191
        // ---- hi / lo split of the landed Q and K atoms into an operand stage ----
        for (int c = 0, r = 0, rph = 0, j = 0, jph = 0; c < nat;
             ++c, rph ^= (r + 1 == nr), r = (r + 1 == nr) ? 0 : r + 1, jph ^= (j + 1 == nst), j = (j + 1 == nst) ? 0 : j + 1) {
            ST_FAIL_AT(3, !mbar_wait(&bars.full[r], (uint32_t)rph, lim));
            ST_FAIL_AT(7, !mbar_wait(&bars.st_free[j], (uint32_t)jph ^ 1u, lim));
            if (t == 0 && c == 0) ST_STAMP(2);
            if (t == 0 && c == nat - 1) ST_STAMP(3);
            const unsigned char *src = raw + (size_t)r * ST_CHUNK;
            unsigned char *dst = stages + (size_t)j * ST_STAGE;
            for (int idx = t; idx < 1024; idx += ST_SPLIT_THREADS) {
                const int part = idx >> 9, i = idx & 511;   // Q / K; 16-byte piece of the [64 x 128 B] slab
                if ((i >> 3) < (part ? Lk : Lq)) {
                    float4 hi, lo;
                    st_split4(*reinterpret_cast<const float4 *>(src + (size_t)idx * 16), hi, lo);
                    unsigned char *d = dst + (size_t)part * ST_CHUNK + (size_t)i * 16;
                    *reinterpret_cast<float4 *>(d) = hi;
                    *reinterpret_cast<float4 *>(d + ST_SLAB) = lo;
                }
            }
            if (t == 0 && c == nat - 1) ST_STAMP(16);
            ST_DBG(0, if (c == 0 && t < 64) { p.dbg[t] = reinterpret_cast<float *>(dst)[t]; p.dbg[64 + t] = reinterpret_cast<float *>(dst + ST_SLAB)[t];
                                              p.dbg[128 + t] = reinterpret_cast<float *>(dst + ST_CHUNK)[t]; p.dbg[192 + t] = reinterpret_cast<float *>(dst + ST_CHUNK + ST_SLAB)[t]; });
            fence_proxy_async_smem();
            if (t == 0 && c == nat - 1) ST_STAMP(17);
            __syncwarp();
            if (lane == 0) { mbar_arrive(&bars.ready[j]); mbar_arrive(&bars.raw_free[r]); }
        }
        failed = __any_sync(0xffffffffu, failed);   // the collective tensor-memory loads below need whole warps
        // ---- the score MMAs are done: the landing slots and the stages may be overwritten ----
        if (!failed) {
            do {
                ST_FAIL_AT(4, !mbar_wait(&bars.s_full, 0, lim));
                if (warp >= 4) ST_FAIL_AT(8, !mbar_wait(&bars.buf_ok, 0, lim));   // (checked at the start of the kernel: long over)
            } while (false);
            failed = __any_sync(0xffffffffu, failed) || (*reinterpret_cast<volatile unsigned *>(&s_fail) != 0u);
        }
        // ---- read-out of the partial scores (warps 4-7: one tensor-memory lane quadrant each; M = 64: row r is
        // in lane 32 (r / 16) + r % 16): a thread adds its row's two column halves and then adds the sums to the
        // head's scores in the scratch ----
        if (warp >= 4 && !failed) {
            if (threadIdx.x == 128) ST_STAMP(4);
            tc_fence_after();
            const int q = warp & 3;
            const uint32_t ta = tmem + ((uint32_t)(32 * q) << 16);
            const int row = 16 * q + lane;
            float *srow = S_cur + (size_t)row * 64;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                uint32_t r0[16], r1[16];
                tmem_ld16(ta + 16 * k, r0);
                tmem_ld16(ta + 64 + 16 * k, r1);
                tmem_ld_wait();
                ST_DBG(1, if (warp == 4 && k == 0 && lane < 2) { for (int jj = 0; jj < 16; ++jj) p.dbg[256 + lane * 64 + jj] = __uint_as_float(r0[jj]); });
                if (lane < 16 && row < Lq) {
#pragma unroll
                    for (int jj = 0; jj < 16; jj += 4)
                        red_add_v4(srow + 16 * k + jj, __uint_as_float(r0[jj]) + __uint_as_float(r1[jj]), __uint_as_float(r0[jj + 1]) + __uint_as_float(r1[jj + 1]),
                                   __uint_as_float(r0[jj + 2]) + __uint_as_float(r1[jj + 2]), __uint_as_float(r0[jj + 3]) + __uint_as_float(r1[jj + 3]));
                }
            }
            if (threadIdx.x == 128) ST_STAMP(5);
            tc_fence_before();
            __syncwarp();
            // release at gpu scope, cumulative over the warp's additions (ordered before it by the warp barrier)
            if (lane == 0) asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(cnt_cur) : "memory");
        }
        // ---- hi / lo split of V for the first pass of P V (all of V when there is one pass) ----
        if (!failed) {
            do {
                ST_FAIL_AT(5, !mbar_wait(&bars.v_full, 0, lim));
                if (t == 0) ST_STAMP(8);
                st_split_v(v_hi, v_lo, nat, 0, kc, kpad, Lk, t);
                fence_proxy_async_smem();
            } while (false);
        }
    }
    if (threadIdx.x == 64) ST_STAMP(9);
    __syncthreads();   // the head's scores are complete (or the wait gave up); V is split
    if (threadIdx.x == 0) ST_STAMP(10);
    failed = (*reinterpret_cast<volatile unsigned *>(&s_fail) != 0u);

    // ---- softmax of the head's scores: half a warp per row, four keys per lane (16-byte loads); the
    // probabilities stay in registers until the pass of P V that takes their keys ----
    constexpr int RPW = 4;   // row pairs per warp: warp w owns rows [8w, 8w + 8)
    const int cg = lane & 15, r2 = lane >> 4;
    float4 sv[RPW];
    if (!failed) {
#pragma unroll
        for (int k = 0; k < RPW; ++k) {
            const int i = 8 * warp + 2 * k + r2;
            sv[k] = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
            if (i < Lq && 4 * cg < Lk) sv[k] = __ldcg(reinterpret_cast<const float4 *>(S_cur + (size_t)i * 64) + cg);
        }
        float mx[RPW], tot[RPW];
#pragma unroll
        for (int k = 0; k < RPW; ++k) {
            sv[k].x = (4 * cg + 0 < Lk) ? sv[k].x * p.scale : -INFINITY;
            sv[k].y = (4 * cg + 1 < Lk) ? sv[k].y * p.scale : -INFINITY;
            sv[k].z = (4 * cg + 2 < Lk) ? sv[k].z * p.scale : -INFINITY;
            sv[k].w = (4 * cg + 3 < Lk) ? sv[k].w * p.scale : -INFINITY;
            mx[k] = fmaxf(fmaxf(sv[k].x, sv[k].y), fmaxf(sv[k].z, sv[k].w));
        }
#pragma unroll
        for (int o = 8; o > 0; o >>= 1)
#pragma unroll
            for (int k = 0; k < RPW; ++k) mx[k] = fmaxf(mx[k], __shfl_xor_sync(0xffffffffu, mx[k], o));
        if (threadIdx.x == 0 && mx[0] > -1e30f) ST_STAMP(6);
#pragma unroll
        for (int k = 0; k < RPW; ++k) {
            // arguments are <= 0 (2 ulp); masked keys give exp(-inf) = 0
            sv[k].x = __expf(sv[k].x - mx[k]); sv[k].y = __expf(sv[k].y - mx[k]);
            sv[k].z = __expf(sv[k].z - mx[k]); sv[k].w = __expf(sv[k].w - mx[k]);
            tot[k] = (sv[k].x + sv[k].y) + (sv[k].z + sv[k].w);
        }
#pragma unroll
        for (int o = 8; o > 0; o >>= 1)
#pragma unroll
            for (int k = 0; k < RPW; ++k) tot[k] += __shfl_xor_sync(0xffffffffu, tot[k], o);
#pragma unroll
        for (int k = 0; k < RPW; ++k) {
            const float inv = __frcp_rn(tot[k]);
            sv[k].x *= inv; sv[k].y *= inv; sv[k].z *= inv; sv[k].w *= inv;
        }
    }

    // ---- O[:, slice]^T = V^T P^T in passes of kc keys: per block of 128 output columns (four atoms) and 8 keys,
    // D[column][row | 64 + row] += Vhi^T [Phi | Plo]^T and += Vlo^T [Phi | Plo]^T - V is the M-major A operand
    // (M = 128: a column per tensor-memory lane), P hi and P lo are one K-major B operand of N = 128, and the sum
    // of a row's hi and lo halves is formed by the thread that stores it ----
    const int ksteps = kpad >> 3, kpc = kc >> 3;   // 8-key MMA steps in all and per pass
    const int npass = (ksteps + kpc - 1) / kpc;
    for (int h = 0; h < npass; ++h) {
        if (h > 0 && !failed) {
            // the MMAs of the previous pass have read their V lo and P: both are replaced
            do { ST_FAIL_AT(9, !mbar_wait(&bars.o_full, (h - 1) & 1, lim)); } while (false);
            if (threadIdx.x == 64) ST_STAMP(23);
            if (!failed && warp >= 2) st_split_v(v_hi, v_lo, nat, h * kc, kc, kpad, Lk, (int)threadIdx.x - 64);
            if (threadIdx.x == 64) ST_STAMP(24);
        }
        if (!failed) {
            const int ks = cg >> 3;                                  // which 32 keys this lane's four belong to
            const bool mine = (pslabs == 2) ? true : (ks == h);
            const uint32_t slab_off = (pslabs == 2) ? (uint32_t)ks * ST_CHUNK : 0u;
#pragma unroll
            for (int k = 0; k < RPW; ++k) {
                const int i = 8 * warp + 2 * k + r2;
                if (mine && i < Lq && 4 * cg < kpad) {
                    float4 hi, lo;
                    st_split4(sv[k], hi, lo);
                    const uint32_t off = slab_off + st_swz(i, 4 * (cg & 7));
                    *reinterpret_cast<float4 *>(p_buf + off) = hi;
                    *reinterpret_cast<float4 *>(p_buf + ST_SLAB + off) = lo;
                }
            }
            if (threadIdx.x == 0) ST_STAMP(h == 0 ? 20 : 25);
            fence_proxy_async_smem();
            if (threadIdx.x == 0) ST_STAMP(h == 0 ? 21 : 26);
        }
        tc_fence_before();
        __syncthreads();
        tc_fence_after();
        failed = (*reinterpret_cast<volatile unsigned *>(&s_fail) != 0u);
        ST_DBG(3, if (h == 0 && threadIdx.x < 64) { p.dbg[512 + threadIdx.x] = reinterpret_cast<float *>(p_buf)[threadIdx.x]; p.dbg[576 + threadIdx.x] = reinterpret_cast<float *>(v_hi)[threadIdx.x];
                                                    p.dbg[640 + threadIdx.x] = reinterpret_cast<float *>(v_lo)[threadIdx.x]; });
        if (threadIdx.x == 0) ST_STAMP(h == 0 ? 11 : 27);
        if (warp == 1 && lane == 0 && !failed) {
            const uint32_t idv = umma_idesc_tf32(128, 128, 1, 0);
            for (int kk = h * kpc; kk < ksteps && kk < (h + 1) * kpc; ++kk) {
                const int kl = kk - h * kpc;
                const uint64_t dp = umma_desc_k_sw128(smem_u32(p_buf + (size_t)(kl >> 2) * ST_CHUNK)) + 2 * (kl & 3);
                for (int b = 0; b < nblk; ++b) {
                    const uint64_t dv_hi = umma_desc_mn_sw128_32b(smem_u32(v_hi + (size_t)b * 4 * ST_SLAB + (size_t)kk * 1024), ST_SLAB, 512);
                    const uint64_t dv_lo = umma_desc_mn_sw128_32b(smem_u32(v_lo + (size_t)b * 4 * vlo_pitch + (size_t)kl * 1024), vlo_pitch, 512);
                    umma_tf32(tmem + b * 128, dv_hi, dp, idv, kk != 0);
                    umma_tf32(tmem + b * 128, dv_lo, dp, idv, 1u);
                }
            }
            umma_commit(&bars.o_full);
            ST_STAMP(h == 0 ? 22 : 28);
        }
        // ---- while P V runs: this slice has read the head's scores; the last slice to say so clears them and
        // the head's counters for the buffer's next user, then bumps the buffer's generation ----
        if (h == 0 && warp == 2 && !failed) {
            unsigned old = 0;
            if (lane == 0) asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(old) : "l"(cnt_cur + 1) : "memory");
            old = __shfl_sync(0xffffffffu, old, 0);
            if (old == (unsigned)p.nsplit - 1u) {
                float4 *z = reinterpret_cast<float4 *>(S_cur);
#pragma unroll 4
                for (int i = lane; i < 1024; i += 32) z[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (lane < 2) cnt_cur[lane] = 0u;
                __threadfence();
                __syncwarp();
                if (lane == 0) asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(p.gen + p.buf) : "memory");
            }
        }
    }
    if (!failed) {
        do {
            ST_FAIL_AT(6, !mbar_wait(&bars.o_full, (npass - 1) & 1, lim));
            if (threadIdx.x == 0) ST_STAMP(12);
            tc_fence_after();
            // The thread of tensor-memory lane 32 q + l of block b holds output column l of atom 4 b + q: its row n
            // is column n (P hi part) plus column 64 + n (P lo part).  The four lanes of a quad transpose 4 rows x 4
            // columns among themselves, so that a lane stores 16 bytes and a store instruction writes four whole
            // 128-byte lines.  One block: two warps per lane quadrant take 32 rows each; two blocks: a warp per
            // block and quadrant.
            const int q = warp & 3, b = (nblk == 2) ? (warp >> 2) : 0, a = 4 * b + q;
            const int n_lo = (nblk == 2) ? 0 : 32 * (warp >> 2), n_hi = (nblk == 2) ? 64 : n_lo + 32;
            if (a < nat) {
                const uint32_t ta = tmem + ((uint32_t)(32 * q) << 16) + (uint32_t)b * 128u;
                const int col0 = atom_col(a) + (lane & ~3);   // head_d is a multiple of 4: the four columns are inside or outside together
                float *obase = p.O + bh * Lq * (long long)p.D + col0;
                for (int n0 = n_lo; n0 < n_hi && n0 < Lq; n0 += 16) {
                    uint32_t rh[16], rl[16];
                    tmem_ld16(ta + n0, rh);
                    tmem_ld16(ta + 64 + n0, rl);
                    tmem_ld_wait();
                    if (threadIdx.x == 0 && n0 == 0) ST_STAMP(29);
                    float v[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(rh[j]) + __uint_as_float(rl[j]);
                    ST_DBG(4, if (warp == 0 && n0 == 0 && lane < 2) { for (int j = 0; j < 16; ++j) p.dbg[704 + lane * 32 + j] = v[j]; });
#pragma unroll
                    for (int t4 = 0; t4 < 4; ++t4) {
                        st_quad_transpose(v[4 * t4], v[4 * t4 + 1], v[4 * t4 + 2], v[4 * t4 + 3], lane);
                        const int row = n0 + 4 * t4 + (lane & 3);
                        if (row < Lq && col0 < p.D)
                            *reinterpret_cast<float4 *>(obase + (long long)row * p.D) = make_float4(v[4 * t4], v[4 * t4 + 1], v[4 * t4 + 2], v[4 * t4 + 3]);
                    }
                    if (threadIdx.x == 0 && n0 == 0) ST_STAMP(30);
                    if (threadIdx.x == 0 && n0 == 16) ST_STAMP(31);
                }
            }
        } while (false);
    }
    if (threadIdx.x == 0) ST_STAMP(13);
    failed = (*reinterpret_cast<volatile unsigned *>(&s_fail) != 0u);
    if (failed && threadIdx.x == 0) {
        // never leave while this CTA's own bulk copies or MMAs may still be in flight
        for (int i = 0; i < 200; ++i) __nanosleep(1000);
    }
    // A kernel launched as the programmatic dependent of the previous call must not complete before it
    // (the stream's order of completion is what later work in the stream relies on).
    if (threadIdx.x == 0) grid_dependency_wait();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 1) tmem_dealloc(tmem, (uint32_t)p.tmem_cols);
    if (threadIdx.x == 32) ST_STAMP(15);
}

#undef ST_FAIL_AT

}  // namespace b200attn
