// Host side of b200attn: the extern "C" layer declared in include/b200attn.h, argument validation,
// kernel selection, per-device workspace and the (batch, head) sharded launcher.
//
// The drop-in symbols mirror the reference launchers (final/attention.cu:195-221 and siblings):
// legacy default stream, blocking, exit(EXIT_FAILURE) on error.  Everything else goes through
// b200attn_forward_ex, which returns a status code instead.
#include <atomic>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <type_traits>
#include <vector>

#include "../../include/b200attn.h"
#include "splitd.cuh"
#include "splitd_tc.cuh"
#include "rope_k.cuh"
#include "synth.cuh"
#include "tc_bf16.cuh"
#include "tc_wide.cuh"
#include "dec.cuh"
#include "tc_fa.cuh"

namespace b200attn {

static thread_local std::string t_last_error;
static thread_local const char *t_last_path = "";
static std::atomic<unsigned long long> g_launches{0};

static int fail(int status, const char *fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    t_last_error = buf;
    return status;
}
#define CU_TRY(expr)                                                                                  \
    do {                                                                                              \
        cudaError_t e_ = (expr);                                                                      \
        if (e_ != cudaSuccess)                                                                        \
            return fail(B200ATTN_ERR_CUDA, "CUDA error %d (%s) at %s:%d: %s", (int)e_,                \
                        cudaGetErrorString(e_), __FILE__, __LINE__, #expr);                           \
    } while (0)

constexpr int kMaxDevices = 64;
constexpr int kSplitDMaxDs = 272;                      // widest slice whose Q,K,V tiles fit 227 KB
constexpr size_t kDefaultScratchCap = 1ull << 30;      // two-pass scores scratch per launch chunk

// Tensor maps are a function of (base address, shape, box) only; encoding one costs the host about a
// microsecond, which matters next to a kernel of a few microseconds, so they are kept.
struct TmapCache {
    struct alignas(64) Entry {
        CUtensorMap map;
        const void *base = nullptr;
        long long rows = 0;
        int cols = 0, box_rows = 0, swz = 0;
        bool valid = false;
    };
    static constexpr size_t kEntries = 4096;   // direct-mapped
    std::vector<Entry> e;
    // fp32 [rows][cols] matrix, box [box_rows x 32 columns], one of the 128-byte swizzles
    const CUtensorMap *get(const void *base, long long rows, int cols, int box_rows, CUtensorMapSwizzle swz) {
        if (e.empty()) e.resize(kEntries);
        size_t h = (size_t)((uintptr_t)base >> 4) * 0x9E3779B97F4A7C15ull;
        h ^= (size_t)rows * 0xC2B2AE3D27D4EB4Full + (size_t)cols * 1315423911u + (size_t)box_rows + ((size_t)swz << 40);
        Entry &x = e[(h >> 20) % kEntries];
        if (!(x.valid && x.base == base && x.rows == rows && x.cols == cols && x.box_rows == box_rows && x.swz == (int)swz)) {
            x.valid = make_tmap_2d(&x.map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, base, rows, cols, ST_ATOM, box_rows, swz);
            x.base = base; x.rows = rows; x.cols = cols; x.box_rows = box_rows; x.swz = (int)swz;
            if (!x.valid) return nullptr;
        }
        return &x.map;
    }
};

// Per-device state.  Guarded by `mu`: calls for one device are serialised on the host.
struct DeviceCtx {
    std::mutex mu;
    std::atomic<bool> ready{false};
    int sm_count = 0;
    int cc_major = 0;
    size_t max_smem_optin = 0;
    float *S = nullptr;            // scores scratch
    size_t S_bytes = 0;
    unsigned *counters = nullptr;  // 2 per head
    size_t counters_n = 0;
    unsigned *err_dev = nullptr;
    unsigned *err_host = nullptr;  // word of mapped pinned host memory: a kernel that reports an error also writes it here
    unsigned *err_host_dev = nullptr;   // the same word as the device sees it
    unsigned *err_bits = nullptr;  // pinned landing place for the device word when err_host says there is something to read
    bool scratch_dirty = false;    // a failed fused launch may have left S / counters non-zero
    bool attr_set[9] = {false, false, false, false, false, false, false, false, false};   // [kernel 0..2][fp32, bf16, fp16]
    size_t dyn_smem_max[9] = {0, 0, 0, 0, 0, 0, 0, 0, 0};
    void *stage[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};   // host-buffer entry point: two sets of Q,K,V,O chunk buffers
    size_t stage_bytes[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    cudaStream_t host_streams[3] = {nullptr, nullptr, nullptr};   // copy-in, compute, copy-out
    cudaEvent_t host_events[6] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    cudaStream_t shard_stream = nullptr;
    // tensor-core split-head_d path: double-buffered score scratch (see splitd_tc.cuh)
    float *sdtc_S = nullptr;
    unsigned *sdtc_cnt = nullptr;
    unsigned *sdtc_gen = nullptr;
    int sdtc_cap = 0;              // heads per buffer of the scratch ring
    unsigned sdtc_seq = 0;         // calls so far: call n uses buffer n % ST_NBUF
    unsigned sdtc_gen_expect[ST_NBUF] = {};   // heads the earlier users of each buffer will have cleared
    bool sdtc_attr = false;
    size_t sdtc_smem_max = 0;
    // the last enqueued call, when it was this kernel: a following call that is declared independent of it
    // (b200attn_forward_many) may be launched as its programmatic dependent
    bool prev_sdtc = false;
    cudaStream_t prev_stream = nullptr;
    uintptr_t prev_out_lo = 0, prev_out_hi = 0;
    // Calls for one device share scratch and tables.  When a call comes on another stream than the
    // call before it, it is made to wait (on the device) for everything enqueued on that stream so far.
    bool have_last_stream = false;
    cudaStream_t last_stream = nullptr;
    cudaEvent_t last_event = nullptr;
    TmapCache tmaps;
    TcTables tc_tables;            // positional-encoding tables of the tensor-core path
    TcwScratch tcw;                // scratch of the wide-head tensor-core path
};
static DeviceCtx g_ctx[kMaxDevices];

static int get_ctx(DeviceCtx **out, int *dev_out = nullptr) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(B200ATTN_ERR_NO_DEVICE, "no CUDA device: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= kMaxDevices) return fail(B200ATTN_ERR_NO_DEVICE, "device ordinal %d out of range", dev);
    DeviceCtx &c = g_ctx[dev];
    if (!c.ready.load(std::memory_order_acquire)) {
        std::lock_guard<std::mutex> lk(c.mu);
        if (!c.ready.load(std::memory_order_relaxed)) {
            cudaDeviceProp prop;
            CU_TRY(cudaGetDeviceProperties(&prop, dev));
            if (prop.major != 10)
                return fail(B200ATTN_ERR_NO_DEVICE, "device %d is sm_%d%d; this library runs on sm_100 only", dev,
                            prop.major, prop.minor);
            c.sm_count = prop.multiProcessorCount;
            c.cc_major = prop.major;
            c.max_smem_optin = prop.sharedMemPerBlockOptin;
            // on a failure nothing stays allocated, so that a retry does not leak
            unsigned *err_dev = nullptr, *err_host = nullptr, *err_host_dev = nullptr;
            cudaError_t e = cudaMalloc(&err_dev, sizeof(unsigned));
            if (e == cudaSuccess) e = cudaMemset(err_dev, 0, sizeof(unsigned));
            if (e == cudaSuccess) e = cudaHostAlloc(&err_host, 2 * sizeof(unsigned), cudaHostAllocMapped | cudaHostAllocPortable);
            if (e == cudaSuccess) e = cudaHostGetDevicePointer(reinterpret_cast<void **>(&err_host_dev), err_host, 0);
            if (e != cudaSuccess) {
                if (err_dev) cudaFree(err_dev);
                if (err_host) cudaFreeHost(err_host);
                (void)cudaGetLastError();
                return fail(B200ATTN_ERR_CUDA, "CUDA error %d (%s) while setting up device %d", (int)e, cudaGetErrorString(e), dev);
            }
            err_host[0] = err_host[1] = 0;
            c.err_dev = err_dev; c.err_host = err_host; c.err_bits = err_host + 1; c.err_host_dev = err_host_dev;
            c.ready.store(true, std::memory_order_release);
        }
    }
    *out = &c;
    if (dev_out) *dev_out = dev;
    return B200ATTN_OK;
}

static int ensure_scratch(DeviceCtx &c, size_t s_bytes, size_t n_counters, cudaStream_t st) {
    if (s_bytes > c.S_bytes) {
        if (c.S) CU_TRY(cudaFree(c.S));
        c.S = nullptr; c.S_bytes = 0;
        size_t want = s_bytes < (1u << 20) ? (1u << 20) : s_bytes;
        CU_TRY(cudaMalloc(&c.S, want));
        CU_TRY(cudaMemsetAsync(c.S, 0, want, st));
        c.S_bytes = want;
    }
    if (n_counters > c.counters_n) {
        if (c.counters) CU_TRY(cudaFree(c.counters));
        c.counters = nullptr; c.counters_n = 0;
        size_t want = n_counters < 4096 ? 4096 : n_counters;
        CU_TRY(cudaMalloc(&c.counters, want * sizeof(unsigned)));
        CU_TRY(cudaMemsetAsync(c.counters, 0, want * sizeof(unsigned), st));
        c.counters_n = want;
    }
    if (c.scratch_dirty) {
        if (c.S) CU_TRY(cudaMemsetAsync(c.S, 0, c.S_bytes, st));
        if (c.counters) CU_TRY(cudaMemsetAsync(c.counters, 0, c.counters_n * sizeof(unsigned), st));
        if (c.sdtc_S) {
            CU_TRY(cudaMemsetAsync(c.sdtc_S, 0, (size_t)ST_NBUF * c.sdtc_cap * 4096 * sizeof(float), st));
            CU_TRY(cudaMemsetAsync(c.sdtc_cnt, 0, (size_t)ST_NBUF * c.sdtc_cap * 2 * sizeof(unsigned), st));
            CU_TRY(cudaMemsetAsync(c.sdtc_gen, 0, ST_NBUF * sizeof(unsigned), st));
            for (int i = 0; i < ST_NBUF; ++i) c.sdtc_gen_expect[i] = 0;
        }
        CU_TRY(cudaMemsetAsync(c.err_dev, 0, sizeof(unsigned), st));
        c.scratch_dirty = false;
    }
    return B200ATTN_OK;
}

static size_t fused_smem_bytes(int ds) {
    return ((size_t)3 * SD_TILE * (ds + 4) + (size_t)SD_TILE * SD_PT_PITCH + ds / 2 + 4) * sizeof(float);
}

template <typename T> constexpr int type_slot() { return sizeof(T) == 4 ? 0 : std::is_same<T, __half>::value ? 2 : 1; }

template <typename Kern>
static int set_smem_attr(DeviceCtx &c, int slot, Kern kern) {
    if (!c.attr_set[slot]) {
        // the opt-in limit covers static + dynamic shared memory
        cudaFuncAttributes fa;
        CU_TRY(cudaFuncGetAttributes(&fa, kern));
        c.dyn_smem_max[slot] = c.max_smem_optin - fa.sharedSizeBytes;
        CU_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)c.dyn_smem_max[slot]));
        c.attr_set[slot] = true;
    }
    return B200ATTN_OK;
}

// Test hook (b200attn_debug_lost_arrival): the per-head barrier of the fused kernel expects this many
// arrivals more than there are slices, i.e. waits for a flag that nothing sets, with this poll limit.
static std::atomic<unsigned> g_test_wait_extra{0}, g_test_spin_limit{0};

// b200attn_set_option
static std::atomic<unsigned> g_spin_limit{1u << 21};
static std::atomic<long long> g_score_scratch_mb{2048};

static unsigned current_spin_limit() {
    if (unsigned t = g_test_spin_limit.load()) return t;
    return g_spin_limit.load();
}

// ---- split-head_d path --------------------------------------------------------------------------
template <typename T>
static int run_splitd(DeviceCtx &c, const b200attn_args &a, int rd, float base, cudaStream_t st) {
    const long long BH = (long long)a.batch_sz * a.num_heads;
    const int Lq = a.len_q, Lk = a.len_k, D = a.head_d;
    SplitDParams p{};
    p.Q = a.Q; p.K = a.K; p.V = a.V; p.O = a.out;
    p.BH = BH; p.Lq = Lq; p.Lk = Lk; p.D = D;
    p.pe = a.pe; p.rotary_dim = rd; p.rope_base = base;
    p.scale = 1.0f / sqrtf((float)D);
    p.cos_cache = a.cos_cache; p.sin_cache = a.sin_cache;
    p.err = c.err_dev;
    p.err_sys = c.err_host_dev;
    p.spin_limit = current_spin_limit();
    p.wait_extra = g_test_wait_extra.load();
    const bool aligned16 = ((((uintptr_t)a.Q | (uintptr_t)a.K | (uintptr_t)a.V) & 15) == 0);
    p.use_tma = (sizeof(T) == 4 && a.pe == B200ATTN_PE_NONE && D % 4 == 0 && aligned16) ? 1 : 0;

    // -- fused cooperative launch: whole heads co-resident, one CTA per slice --
    bool fused = !(a.flags & B200ATTN_FLAG_FORCE_TWO_PASS) && Lq <= SD_TILE && Lk <= SD_TILE;
    int ds = 0, nsplit = 0;
    size_t smem = 0;
    if (fused) {
        long long nsplit_max = c.sm_count / BH;
        if (nsplit_max < 1) fused = false;
        else {
            ds = (int)((D + nsplit_max - 1) / nsplit_max);
            if (p.use_tma) {
                // packed TMA tiles: slice width a multiple of 4 with ds/4 odd (16 rows then cover all
                // shared-memory banks) and within the 256-element box limit
                ds = (ds + 3) & ~3;
                if (((ds >> 2) & 1) == 0) ds += 4;
                if (ds > 252) p.use_tma = 0;
            }
            if (!p.use_tma) {
                ds = (ds + 7) & ~7;
                if (ds < 8) ds = 8;
            }
            if (ds > kSplitDMaxDs) fused = false;
            nsplit = (D + ds - 1) / ds;
            smem = fused_smem_bytes(ds);
            if (smem > c.max_smem_optin) fused = false;
        }
    }
    if (fused) {
        const int slot = type_slot<T>();
        int rc = set_smem_attr(c, slot, splitd_fused_kernel<T>);
        if (rc) return rc;
        if (smem > c.dyn_smem_max[slot]) fused = false;
    }
    if (fused) {
        int per_sm = 0;
        CU_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, splitd_fused_kernel<T>, SD_THREADS, smem));
        if ((long long)per_sm * c.sm_count < (long long)nsplit * BH || BH > 65535) fused = false;
    }
    if (fused) {
        int rc = ensure_scratch(c, (size_t)BH * Lq * Lk * sizeof(float), (size_t)2 * BH, st);
        if (rc) return rc;
        p.S = c.S; p.counters = c.counters; p.ds = ds; p.nsplit = nsplit;
        CUtensorMap tmQ, tmK, tmV;
        memset(&tmQ, 0, sizeof tmQ); memset(&tmK, 0, sizeof tmK); memset(&tmV, 0, sizeof tmV);
        if (p.use_tma) {
            if (!make_tmap_2d(&tmQ, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, a.Q, BH * Lq, D, ds, Lq, CU_TENSOR_MAP_SWIZZLE_NONE) ||
                !make_tmap_2d(&tmK, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, a.K, BH * Lk, D, ds, Lk, CU_TENSOR_MAP_SWIZZLE_NONE) ||
                !make_tmap_2d(&tmV, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, a.V, BH * Lk, D, ds, Lk, CU_TENSOR_MAP_SWIZZLE_NONE))
                return fail(B200ATTN_ERR_CUDA, "cuTensorMapEncodeTiled failed for the split-head_d slices");
        }
        dim3 grid(nsplit, (unsigned)BH);
        void *kargs[] = {&tmQ, &tmK, &tmV, &p};
        CU_TRY(cudaLaunchCooperativeKernel((const void *)splitd_fused_kernel<T>, grid, dim3(SD_THREADS), kargs, smem, st));
        g_launches.fetch_add(1);
        t_last_path = "splitd_fused";
        return B200ATTN_OK;
    }

    // -- two launches per chunk of heads: scores, then softmax + PV --
    // column chunks of <= 128; split a tile's chunks over several CTAs only when the grid would
    // otherwise leave SMs idle (few heads, short sequences, wide heads)
    ds = D <= 128 ? ((D + 7) & ~7) : 128;
    {
        const int nchunks = (D + ds - 1) / ds;
        const long long tiles = (long long)((Lq + SD_TILE - 1) / SD_TILE) * ((Lk + SD_TILE - 1) / SD_TILE) * BH;
        long long want = (2LL * c.sm_count + tiles - 1) / tiles;
        nsplit = (int)(want < 1 ? 1 : (want > nchunks ? nchunks : want));
        const int per = (nchunks + nsplit - 1) / nsplit;
        nsplit = (nchunks + per - 1) / per;   // no empty CTA
    }
    const int dv = D < 64 ? ((D + 7) & ~7) : 64;
    const int nqt = (Lq + SD_TILE - 1) / SD_TILE, nkt = (Lk + SD_TILE - 1) / SD_TILE;
    if ((long long)nqt * nkt > 65535) return fail(B200ATTN_ERR_TOO_LARGE, "len_q x len_k = %d x %d exceeds the split-head_d path's tiling limit", Lq, Lk);
    const size_t per_head = (size_t)Lq * Lk * sizeof(float);
    size_t cap = kDefaultScratchCap;
    if (per_head > cap) cap = per_head;
    long long chunk = (long long)(cap / per_head);
    if (chunk > BH) chunk = BH;
    if (chunk > 65535) chunk = 65535;
    int rc = ensure_scratch(c, (size_t)chunk * per_head, 0, st);
    if (rc) return rc;
    rc = set_smem_attr(c, 3 + type_slot<T>(), splitd_scores_kernel<T>);
    if (rc) return rc;
    rc = set_smem_attr(c, 6 + type_slot<T>(), splitd_softmax_pv_kernel<T>);
    if (rc) return rc;
    const size_t smem1 = ((size_t)2 * SD_TILE * (ds + 4) + ds / 2 + 4) * sizeof(float);
    const size_t smem2 = ((size_t)SD_TILE * (dv + 4) + (size_t)SD_TILE * SD_PT_PITCH + 2 * SD_TILE) * sizeof(float);
    const size_t esz = sizeof(T);
    for (long long bh0 = 0; bh0 < BH; bh0 += chunk) {
        const long long n = (BH - bh0 < chunk) ? (BH - bh0) : chunk;
        SplitDParams q = p;
        q.Q = (const char *)a.Q + (size_t)bh0 * Lq * D * esz;
        q.K = (const char *)a.K + (size_t)bh0 * Lk * D * esz;
        q.V = (const char *)a.V + (size_t)bh0 * Lk * D * esz;
        q.O = (char *)a.out + (size_t)bh0 * Lq * D * esz;
        q.BH = n; q.S = c.S; q.ds = ds; q.nsplit = nsplit; q.dv = dv; q.use_tma = 0;
        splitd_scores_kernel<T><<<dim3(nsplit, nqt * nkt, (unsigned)n), SD_THREADS, smem1, st>>>(q);
        CU_TRY(cudaGetLastError());
        splitd_softmax_pv_kernel<T><<<dim3((D + dv - 1) / dv, nqt, (unsigned)n), SD_THREADS, smem2, st>>>(q);
        CU_TRY(cudaGetLastError());
        g_launches.fetch_add(2);
        // the scratch must be all-zero again for the fused kernel
        CU_TRY(cudaMemsetAsync(c.S, 0, (size_t)n * per_head, st));
    }
    t_last_path = "splitd_two_pass";
    return B200ATTN_OK;
}

#ifdef B200ATTN_DEVTOOLS
static float *g_sdtc_dbg = nullptr;
static unsigned long long *g_sdtc_stamps = nullptr;
static long long g_sdtc_stamp_calls = 0;   // with B200ATTN_SDTC_STAMP_STRIDE set: call n writes at n * stride
#endif
// ---- split-head_d path on the tensor cores (fp32, no positional encoding, len <= 64) ---------------
// Slices are whole 32-column atoms; a head gets as many slices as the SM count allows.  Returns -1 when
// the shape belongs to the CUDA-core kernels (an encoding, an odd head_d, more heads than SMs, a slice
// wider than 256 columns).
// `independent_of_prev`: the caller declared this call independent of the one before it; `batched`: the call is
// one of a batch of such calls (it, or the next one, may run beside its neighbour).
static int run_sdtc(DeviceCtx &c, const b200attn_args &a, cudaStream_t st, bool independent_of_prev, bool batched) {
    const long long BH = (long long)a.batch_sz * a.num_heads;
    const int Lq = a.len_q, Lk = a.len_k, D = a.head_d;
    if (a.dtype != B200ATTN_F32 || a.pe != B200ATTN_PE_NONE || Lq > 64 || Lk > 64 || D % 4 != 0) return -1;
    if ((((uintptr_t)a.Q | (uintptr_t)a.K | (uintptr_t)a.V) & 15) != 0 || ((uintptr_t)a.out & 31) != 0) return -1;   // 32-byte output stores
    if (BH > c.sm_count || BH > 65535) return -1;
    const int natoms = (D + ST_ATOM - 1) / ST_ATOM;
    const int slots = (int)(c.sm_count / BH);
    int apc = (natoms + slots - 1) / slots;
#ifdef B200ATTN_DEVTOOLS
    if (const char *e = getenv("B200ATTN_SDTC_APC")) apc = atoi(e);
#endif
    if (apc > ST_MAX_ATOMS) return -1;
    const int nsplit = (natoms + apc - 1) / apc;
    // Overlap with the previous call: this call's inputs must not be that call's output.  (Two CTAs
    // share an SM up to half of its shared memory, i.e. with slices of up to 128 columns; the whole of this
    // call then runs beside the previous one.  Wider slices still gain the launch latency.)
    const size_t in_q = (size_t)BH * Lq * D * 4, in_k = (size_t)BH * Lk * D * 4;
    auto hits_prev_out = [&](const void *ptr, size_t n) { return (uintptr_t)ptr < c.prev_out_hi && (uintptr_t)ptr + n > c.prev_out_lo; };
    const bool overlap = independent_of_prev && c.prev_sdtc && c.prev_stream == st && !c.scratch_dirty &&
                         !hits_prev_out(a.Q, in_q) && !hits_prev_out(a.K, in_k) && !hits_prev_out(a.V, in_k);
    // Shared memory of a CTA in units of 16 KB: nr landing slots, nst operand stages of two units, and V either in
    // two units per block of its own (requested when the CTA starts) or over the stages.  A call on its own takes
    // what an SM has: two stages, V on its own, a landing slot per atom as far as they fit, P V in one pass.  A
    // call of a batch takes the form that lets the most CTAs share an SM - its neighbours in the stream run beside
    // it - (at most three: the registers); among equals the form listed first below.
    const int nb = sdtc_vblocks(apc), tmem_cols = 128 * nb;
    const size_t sm_bytes = (size_t)c.max_smem_optin + 1024;   // per SM; the system keeps 1 KB per CTA
    int nr = 0, nst = ST_NST, v_own = 1, kc = 64;
    if (batched || overlap) {
        int best = 0;
        for (int s2 = ST_NST; s2 >= 1; --s2)
            for (int vo = 1; vo >= 0; --vo)
                for (int r = apc < ST_MAX_SLOTS ? apc : ST_MAX_SLOTS; r >= 1; --r)
                    for (int k = 64; k >= 32; k -= 32) {
                        if (!sdtc_layout_ok(apc, r, s2, vo, k)) continue;
                        const size_t bytes = sdtc_smem_bytes(apc, r, s2, vo);
                        if (bytes > (size_t)c.max_smem_optin) continue;
                        int n = (int)(sm_bytes / (bytes + 1024));
                        if (n > 512 / tmem_cols) n = 512 / tmem_cols;
                        if (n > 3) n = 3;
                        if (n > best) { best = n; nr = r; nst = s2; v_own = vo; kc = k; }
                    }
    } else {
        const int room = (int)(((size_t)c.max_smem_optin - 1024) / ST_CHUNK) - 2 * ST_NST - 2 * nb;   // units left for landing slots
        nr = apc < room ? apc : room;
        if (nr > ST_MAX_SLOTS) nr = ST_MAX_SLOTS;
    }
#ifdef B200ATTN_DEVTOOLS
    if (const char *e = getenv("B200ATTN_SDTC_NR")) nr = atoi(e);
    if (const char *e = getenv("B200ATTN_SDTC_NST")) nst = atoi(e);
    if (const char *e = getenv("B200ATTN_SDTC_VOWN")) v_own = atoi(e);
    if (const char *e = getenv("B200ATTN_SDTC_KC")) kc = atoi(e);
    if (kc != 32 && kc != 64) return -1;
#endif
    if (nr < 1 || !sdtc_layout_ok(apc, nr, nst, v_own, kc)) return -1;
    size_t smem = sdtc_smem_bytes(apc, nr, nst, v_own);
    // The CTAs that fit an SM by shared memory must also fit it by tensor memory (512 columns): a CTA that had to
    // wait for columns held by CTAs that wait for its scores would never get them.  Ask for more shared memory
    // where that is not so by itself.
    {
        const size_t by_tmem = 512 / (size_t)tmem_cols;
        if (sm_bytes / (smem + 1024) > by_tmem) smem = sm_bytes / (by_tmem + 1);
    }
    if (!c.sdtc_attr) {
        cudaFuncAttributes fa;
        CU_TRY(cudaFuncGetAttributes(&fa, sdtc_kernel));
        c.sdtc_smem_max = c.max_smem_optin - fa.sharedSizeBytes;
        CU_TRY(cudaFuncSetAttribute(sdtc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)c.sdtc_smem_max));
        c.sdtc_attr = true;
    }
    if (smem > c.sdtc_smem_max) return -1;
    if (c.sdtc_S == nullptr) {
        const int cap = c.sm_count;
        CU_TRY(cudaMalloc(&c.sdtc_S, (size_t)ST_NBUF * cap * 4096 * sizeof(float)));
        CU_TRY(cudaMalloc(&c.sdtc_cnt, (size_t)ST_NBUF * cap * 2 * sizeof(unsigned)));
        CU_TRY(cudaMalloc(&c.sdtc_gen, ST_NBUF * sizeof(unsigned)));
        c.sdtc_cap = cap;
        c.scratch_dirty = true;   // cleared below, on this call's stream
    }
    if (c.scratch_dirty) {
        int rc = ensure_scratch(c, 0, 0, st);
        if (rc) return rc;
    }
    // (the four maps are copied before the next lookup can evict one: the cache is direct-mapped)
    CUtensorMap tmQ, tmK, tmV;
    const CUtensorMap *m;
    bool ok = (m = c.tmaps.get(a.Q, BH * Lq, D, Lq, CU_TENSOR_MAP_SWIZZLE_128B)) != nullptr;
    if (ok) { tmQ = *m; ok = (m = c.tmaps.get(a.K, BH * Lk, D, Lk, CU_TENSOR_MAP_SWIZZLE_128B)) != nullptr; }
    if (ok) { tmK = *m; ok = (m = c.tmaps.get(a.V, BH * Lk, D, Lk, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B)) != nullptr; }
    if (ok) tmV = *m;
    if (!ok) return fail(B200ATTN_ERR_CUDA, "cuTensorMapEncodeTiled failed for the split-head_d slices");
    SdtcParams p{};
    p.BH = BH; p.Lq = Lq; p.Lk = Lk; p.D = D;
    p.apc = apc; p.natoms = natoms; p.nsplit = nsplit;
    const int buf = (int)(c.sdtc_seq % ST_NBUF);
    p.buf = buf; p.gen_expect = c.sdtc_gen_expect[buf]; p.cap_bh = c.sdtc_cap; p.tmem_cols = tmem_cols; p.nr = nr; p.nst = nst; p.v_own = v_own; p.kc = kc;
    p.scale = 1.0f / sqrtf((float)D);
    p.O = (float *)a.out;
    p.S = c.sdtc_S; p.counters = c.sdtc_cnt; p.gen = c.sdtc_gen;
    p.err = c.err_dev; p.err_sys = c.err_host_dev;
    p.spin_limit = current_spin_limit();
    p.wait_extra = g_test_wait_extra.load();
#ifdef B200ATTN_DEVTOOLS
    p.dbg = g_sdtc_dbg;
    p.stamps = g_sdtc_stamps;
    if (g_sdtc_stamps != nullptr) {
        static const long long stride = getenv("B200ATTN_SDTC_STAMP_STRIDE") ? atoll(getenv("B200ATTN_SDTC_STAMP_STRIDE")) : 0;
        p.stamps += (g_sdtc_stamp_calls++) * stride;
    }
#endif
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)nsplit, (unsigned)BH);
    cfg.blockDim = dim3(ST_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = overlap ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    CU_TRY(cudaLaunchKernelEx(&cfg, sdtc_kernel, tmQ, tmK, tmV, p));
    c.sdtc_seq += 1;
    c.sdtc_gen_expect[buf] += (unsigned)BH;
    c.prev_sdtc = true;
    c.prev_stream = st;
    c.prev_out_lo = (uintptr_t)a.out;
    c.prev_out_hi = (uintptr_t)a.out + in_q;
    g_launches.fetch_add(1);
    t_last_path = "splitd_tc";
    return B200ATTN_OK;
}

// ---- validation + dispatch ----------------------------------------------------------------------
static int validate(const b200attn_args *a, int *rd_out, float *base_out) {
    if (a == nullptr) return fail(B200ATTN_ERR_INVALID_ARG, "args is NULL");
    if (a->struct_size != sizeof(b200attn_args))
        return fail(B200ATTN_ERR_INVALID_ARG, "args->struct_size is %zu, expected %zu", a->struct_size, sizeof(b200attn_args));
    if (!a->Q || !a->K || !a->V || !a->out) return fail(B200ATTN_ERR_INVALID_ARG, "Q, K, V and out must be non-NULL");
    if (a->batch_sz <= 0 || a->num_heads <= 0 || a->len_q <= 0 || a->len_k <= 0 || a->head_d <= 0)
        return fail(B200ATTN_ERR_INVALID_ARG, "batch_sz, num_heads, len_q, len_k, head_d must be positive (got %d,%d,%d,%d,%d)",
                    a->batch_sz, a->num_heads, a->len_q, a->len_k, a->head_d);
    if (a->dtype != B200ATTN_F32 && a->dtype != B200ATTN_BF16 && a->dtype != B200ATTN_F16) return fail(B200ATTN_ERR_INVALID_ARG, "unknown dtype %d", a->dtype);
    if (a->pe < B200ATTN_PE_NONE || a->pe > B200ATTN_PE_ROPE_HALF_Q_ONLY) return fail(B200ATTN_ERR_INVALID_ARG, "unknown pe kind %d", a->pe);
    const size_t esz = a->dtype == B200ATTN_F32 ? 4 : 2;   // bf16 and fp16 are both two bytes
    if (((uintptr_t)a->Q | (uintptr_t)a->K | (uintptr_t)a->V | (uintptr_t)a->out) & (esz - 1))
        return fail(B200ATTN_ERR_INVALID_ARG, "tensor pointers must be aligned to the element size");
    if (a->out == a->Q || a->out == a->K || a->out == a->V) return fail(B200ATTN_ERR_INVALID_ARG, "out must not alias an input");
    int rd = a->rotary_dim == 0 ? a->head_d : a->rotary_dim;
    const bool rope = pe_is_rope(a->pe);
    if (rope) {
        if (rd < 0 || rd > a->head_d || (rd & 1))
            return fail(B200ATTN_ERR_INVALID_ARG, "rotary_dim must be even and within [0, head_d] (got %d, head_d %d)", rd, a->head_d);
        if ((a->cos_cache == nullptr) != (a->sin_cache == nullptr))
            return fail(B200ATTN_ERR_INVALID_ARG, "cos_cache and sin_cache must be given together");
    } else {
        rd = a->head_d;
    }
    float base = a->rope_base == 0.0f ? 10000.0f : a->rope_base;
    if (!(base > 0.0f)) return fail(B200ATTN_ERR_INVALID_ARG, "rope_base must be positive");
    *rd_out = rd; *base_out = base;
    return B200ATTN_OK;
}

// To be called with the work of the call complete (its streams synchronised): kernels mirror an error
// into mapped host memory, so the common case is one host load and no device-to-host copy.
static int report_kernel_errors(DeviceCtx &c, const char *what) {
    if (*reinterpret_cast<volatile unsigned *>(c.err_host) == 0) return B200ATTN_OK;
    unsigned bits = *c.err_host;
    if (cudaMemcpy(c.err_bits, c.err_dev, sizeof(unsigned), cudaMemcpyDeviceToHost) == cudaSuccess) bits |= *c.err_bits;
    *c.err_host = 0;
    c.scratch_dirty = true;
    cudaMemset(c.err_dev, 0, sizeof(unsigned));   // the error is reported once; later launches start clean
    return fail(B200ATTN_ERR_KERNEL, "%s reported error bits 0x%x (bit 0: head barrier wait expired, bit 1: mbarrier wait expired, bits 8..31: which wait of the tensor-core kernel)", what, bits);
}

static int check_kernel_errors(DeviceCtx &c, cudaStream_t st, bool sync) {
    // asynchronous calls do not wait; an error of theirs is reported by the next call on this device
    if (!sync) return B200ATTN_OK;
    CU_TRY(cudaStreamSynchronize(st));
    return report_kernel_errors(c, "kernel");
}

static int forward_device(const b200attn_args *a, bool independent_of_prev = false, bool batched = false) {
    int rd; float base;
    int rc = validate(a, &rd, &base);
    if (rc) return rc;
    DeviceCtx *c;
    rc = get_ctx(&c);
    if (rc) return rc;
    std::lock_guard<std::mutex> lk(c->mu);
    cudaStream_t st = (cudaStream_t)a->stream;
    // an error left by an earlier asynchronous call is reported now
    if (*reinterpret_cast<volatile unsigned *>(c->err_host) != 0) {
        cudaDeviceSynchronize();   // let the failed work drain before the scratch is cleaned
        return report_kernel_errors(*c, "an earlier asynchronous call");
    }
    if (c->have_last_stream && c->last_stream != st) {
        if (!c->last_event) CU_TRY(cudaEventCreateWithFlags(&c->last_event, cudaEventDisableTiming));
        cudaError_t e = cudaEventRecord(c->last_event, c->last_stream);
        if (e == cudaSuccess) e = cudaStreamWaitEvent(st, c->last_event, 0);
        if (e != cudaSuccess) {   // the earlier stream is gone or unusable: order by waiting for the device
            (void)cudaGetLastError();
            CU_TRY(cudaDeviceSynchronize());
        }
    }
    c->last_stream = st;
    c->have_last_stream = true;
    bool done = false;
    const bool chain = independent_of_prev && c->prev_sdtc;
    c->prev_sdtc = false;   // set again by the kernel that supports being overlapped
    // bf16 on the tensor cores: the two-kernel path (scores, then P V) takes every shape it supports;
    // the one-kernel cluster pipeline takes the rest of its own shapes (and all of them when the call
    // asks for it with B200ATTN_FLAG_PREFER_ONE_KERNEL: the two are measured against each other that way).
    const bool tc_ok = (a->dtype == B200ATTN_BF16 || a->dtype == B200ATTN_F16) && !(a->flags & B200ATTN_FLAG_FORCE_GENERIC);
    const bool wide_ok = tc_ok && tcw_supported(*a, rd), pair_ok = tc_ok && tc_bf16_supported(*a, rd);
    const bool use_pair = pair_ok && (!wide_ok || (a->flags & B200ATTN_FLAG_PREFER_ONE_KERNEL));
    if (use_pair) {
        rc = tc_bf16_run(*a, rd, base, c->tc_tables, c->err_dev, c->err_host_dev, c->sm_count, current_spin_limit(), st, &g_launches);
        if (rc == B200ATTN_OK) { t_last_path = "tc_bf16"; done = true; }
        else if (rc != -1) return fail(rc, "%s", tc_bf16_error());
    }
    // few queries against many keys (decode, cross-attention): key splits on the tensor cores
    if (!done && tc_ok && dec_supported(*a, rd)) {
        rc = dec_run(*a, rd, base, c->tcw, c->tc_tables, c->err_dev, c->err_host_dev, c->sm_count, current_spin_limit(), st, &g_launches);
        if (rc == B200ATTN_OK) { t_last_path = "tc_decode"; done = true; }
        else if (rc != -1) return fail(rc, "%s", tc_bf16_error());
    }
    // A call with an encoding that runs on encoded copies of Q and K (the scratch of the two-kernel path's rotated
    // operands): the narrow-head kernel below, and fp16 tensors on the two-kernel path (whose in-load encodings
    // are bf16 arithmetic).
    b200attn_args enc;
    auto encode_copies = [&](b200attn_args *b) -> int {
        const size_t BHs = (size_t)a->batch_sz * a->num_heads;
        void *qc = c->tcw.get(2, BHs * a->len_q * a->head_d * 2);
        void *kc = pe_encodes_k(a->pe) ? c->tcw.get(3, BHs * a->len_k * a->head_d * 2) : nullptr;
        if (qc == nullptr || (pe_encodes_k(a->pe) && kc == nullptr)) return -1;
        return a->dtype == B200ATTN_F16 ? fa_encode_copies<__half>(*a, rd, base, (__half *)qc, (__half *)kc, c->sm_count, st, &g_launches, b)
                                        : fa_encode_copies<__nv_bfloat16>(*a, rd, base, (__nv_bfloat16 *)qc, (__nv_bfloat16 *)kc, c->sm_count, st, &g_launches, b);
    };
    // narrow heads, many queries: one kernel, the scores stay in tensor memory
    if (!done && tc_ok && !(a->flags & B200ATTN_FLAG_TWO_KERNELS) && fa_supported(*a)) {
        const b200attn_args *use = a;
        rc = B200ATTN_OK;
        if (a->pe != B200ATTN_PE_NONE) { rc = encode_copies(&enc); use = &enc; }
        if (rc == B200ATTN_OK) rc = fa_run(*use, c->err_dev, c->err_host_dev, c->sm_count, current_spin_limit(), st, &g_launches);
        if (rc == B200ATTN_OK) { t_last_path = "tc_fused"; done = true; }
        else if (rc != -1) return fail(rc, "%s", tc_bf16_error());
    }
    if (!done && tc_ok && !wide_ok && a->dtype == B200ATTN_F16 && a->pe != B200ATTN_PE_NONE) {
        b200attn_args plain = *a;
        plain.pe = B200ATTN_PE_NONE; plain.cos_cache = nullptr; plain.sin_cache = nullptr;
        if (tcw_supported(plain, plain.head_d)) {
            rc = encode_copies(&enc);
            if (rc == B200ATTN_OK)
                rc = tcw_run(enc, enc.head_d, base, c->tcw, c->tc_tables, c->err_dev, c->err_host_dev, c->sm_count, current_spin_limit(),
                             (size_t)g_score_scratch_mb.load() << 20, st, &g_launches);
            if (rc == B200ATTN_OK) { t_last_path = "tc_wide"; done = true; }
            else if (rc != -1) return fail(rc, "%s", tc_bf16_error());
        }
    }
    if (!done && wide_ok) {
        rc = tcw_run(*a, rd, base, c->tcw, c->tc_tables, c->err_dev, c->err_host_dev, c->sm_count, current_spin_limit(),
                     (size_t)g_score_scratch_mb.load() << 20, st, &g_launches);
        if (rc == B200ATTN_OK) { t_last_path = "tc_wide"; done = true; }
        else if (rc != -1) return fail(rc, "%s", tc_bf16_error());
        else if (pair_ok && !use_pair) {   // no room for the score scratch: the one-kernel pipeline needs none
            rc = tc_bf16_run(*a, rd, base, c->tc_tables, c->err_dev, c->err_host_dev, c->sm_count, current_spin_limit(), st, &g_launches);
            if (rc == B200ATTN_OK) { t_last_path = "tc_bf16"; done = true; }
            else if (rc != -1) return fail(rc, "%s", tc_bf16_error());
        }
    }
    if (!done && !(a->flags & (B200ATTN_FLAG_FORCE_GENERIC | B200ATTN_FLAG_FORCE_TWO_PASS))) {
        c->prev_sdtc = chain;
        rc = run_sdtc(*c, *a, st, independent_of_prev, batched);
        if (rc != B200ATTN_OK) c->prev_sdtc = false;
        if (rc == B200ATTN_OK) done = true;
        else if (rc != -1) return rc;
    }
    if (!done) {
        rc = (a->dtype == B200ATTN_F32) ? run_splitd<float>(*c, *a, rd, base, st)
           : (a->dtype == B200ATTN_F16) ? run_splitd<__half>(*c, *a, rd, base, st) : run_splitd<__nv_bfloat16>(*c, *a, rd, base, st);
        if (rc) return rc;
    }
    return check_kernel_errors(*c, st, !(a->flags & B200ATTN_FLAG_ASYNC));
}

static int ensure_stage(DeviceCtx &c, int i, size_t bytes) {
    if (bytes > c.stage_bytes[i]) {
        if (c.stage[i]) CU_TRY(cudaFree(c.stage[i]));
        c.stage[i] = nullptr; c.stage_bytes[i] = 0;
        CU_TRY(cudaMalloc(&c.stage[i], bytes));
        c.stage_bytes[i] = bytes;
    }
    return B200ATTN_OK;
}

static void legacy(const void *Q, const void *K, const void *V, void *out, int B, int H, int Lq, int Lk, int D, int dtype,
                   int pe, int rd, const float *cc, const float *sc) {
    b200attn_args a{};
    a.struct_size = sizeof a;
    a.Q = Q; a.K = K; a.V = V; a.out = out;
    a.batch_sz = B; a.num_heads = H; a.len_q = Lq; a.len_k = Lk; a.head_d = D;
    a.dtype = dtype; a.pe = pe; a.rotary_dim = rd; a.cos_cache = cc; a.sin_cache = sc;
    a.flags = B200ATTN_FLAG_ASYNC;   // the one wait of the call is the device-wide one below
    int rc = forward_device(&a);
    if (rc == B200ATTN_OK) {
        // the reference launchers end with cudaDeviceSynchronize (final/attention.cu:220)
        cudaError_t e = cudaDeviceSynchronize();
        if (e != cudaSuccess) rc = fail(B200ATTN_ERR_CUDA, "CUDA error %d (%s) at %s:%d", (int)e, cudaGetErrorString(e), __FILE__, __LINE__);
        DeviceCtx *c;
        if (rc == B200ATTN_OK && get_ctx(&c) == B200ATTN_OK) {
            std::lock_guard<std::mutex> lk(c->mu);
            rc = report_kernel_errors(*c, "kernel");
        }
    }
    if (rc != B200ATTN_OK) {
        fprintf(stderr, "b200attn: %s\n", t_last_error.c_str());
        exit(EXIT_FAILURE);
    }
}

}  // namespace b200attn

using namespace b200attn;

extern "C" {

void attention_forward_optimized(const float *Q, const float *K, const float *V, float *out, int B, int H, int Lq, int Lk, int D) {
    legacy(Q, K, V, out, B, H, Lq, Lk, D, B200ATTN_F32, B200ATTN_PE_NONE, 0, nullptr, nullptr);
}
void attention_forward_bf16(const void *Q, const void *K, const void *V, void *out, int B, int H, int Lq, int Lk, int D) {
    legacy(Q, K, V, out, B, H, Lq, Lk, D, B200ATTN_BF16, B200ATTN_PE_NONE, 0, nullptr, nullptr);
}
void attention_forward_rope_fused_v2(const float *Q, const float *K, const float *V, float *out, int B, int H, int Lq, int Lk, int D) {
    legacy(Q, K, V, out, B, H, Lq, Lk, D, B200ATTN_F32, B200ATTN_PE_ROPE_INTERLEAVED, D, nullptr, nullptr);
}
void attention_forward_rope_fused(const float *Q, const float *K, const float *V, float *out, const float *cos_cache,
                                  const float *sin_cache, int B, int H, int Lq, int Lk, int D) {
    if (!cos_cache || !sin_cache) {
        fprintf(stderr, "b200attn: attention_forward_rope_fused needs cos_cache and sin_cache\n");
        exit(EXIT_FAILURE);
    }
    legacy(Q, K, V, out, B, H, Lq, Lk, D, B200ATTN_F32, B200ATTN_PE_ROPE_INTERLEAVED, D, cos_cache, sin_cache);
}
void attention_forward_rope_fused_v7_hybrid(const float *Q, const float *Kr, const float *V, float *out, int B, int H, int Lq,
                                            int Lk, int D, int rotary_dim) {
    // the reference rotates the columns d < rotary_dim (final/rope.cu:129-149): none when it is 0
    legacy(Q, Kr, V, out, B, H, Lq, Lk, D, B200ATTN_F32, rotary_dim == 0 ? B200ATTN_PE_NONE : B200ATTN_PE_ROPE_Q_ONLY, rotary_dim, nullptr, nullptr);
}
void attention_forward_rope_bf16(const void *Q, const void *K, const void *V, void *out, int B, int H, int Lq, int Lk, int D) {
    legacy(Q, K, V, out, B, H, Lq, Lk, D, B200ATTN_BF16, B200ATTN_PE_ROPE_INTERLEAVED, D, nullptr, nullptr);
}
void attention_forward_rope_bf16_v7(const void *Q, const void *Kr, const void *V, void *out, int B, int H, int Lq, int Lk, int D,
                                    int rotary_dim) {
    legacy(Q, Kr, V, out, B, H, Lq, Lk, D, B200ATTN_BF16, rotary_dim == 0 ? B200ATTN_PE_NONE : B200ATTN_PE_ROPE_Q_ONLY, rotary_dim, nullptr, nullptr);
}
void attention_forward_sinusoidal_fused(const float *Q, const float *K, const float *V, float *out, int B, int H, int Lq, int Lk, int D) {
    legacy(Q, K, V, out, B, H, Lq, Lk, D, B200ATTN_F32, B200ATTN_PE_SINUSOIDAL, 0, nullptr, nullptr);
}
void attention_forward_sinusoidal_bf16(const void *Q, const void *K, const void *V, void *out, int B, int H, int Lq, int Lk, int D) {
    legacy(Q, K, V, out, B, H, Lq, Lk, D, B200ATTN_BF16, B200ATTN_PE_SINUSOIDAL, 0, nullptr, nullptr);
}

int b200attn_forward_ex(const b200attn_args *args) { return forward_device(args); }

#ifdef B200ATTN_DEVTOOLS
// Bring-up aid (development builds only): runs the one-kernel tensor-core pipeline and also returns the
// raw scores Q K^T of key block 0, [B*H*(Lq/128)][128][128] fp32, for checking the first MMA stage.
int b200attn_debug_tc_scores(const b200attn_args *a, float *scores_dev) {
    int rd; float base;
    int rc = validate(a, &rd, &base);
    if (rc) return rc;
    DeviceCtx *c;
    rc = get_ctx(&c);
    if (rc) return rc;
    if (!tc_bf16_supported(*a, rd)) return fail(B200ATTN_ERR_INVALID_ARG, "shape not taken by the tensor-core kernel");
    std::lock_guard<std::mutex> lk(c->mu);
    rc = tc_bf16_run(*a, rd, base, c->tc_tables, c->err_dev, c->err_host_dev, c->sm_count, current_spin_limit(), (cudaStream_t)a->stream, &g_launches, scores_dev);
    if (rc) return fail(rc, "%s", tc_bf16_error());
    return check_kernel_errors(*c, (cudaStream_t)a->stream, true);
}

void b200attn_debug_sdtc_dump(float *dev_buf) { g_sdtc_dbg = dev_buf; }
void b200attn_debug_sdtc_stamps(unsigned long long *dev_buf) { g_sdtc_stamps = dev_buf; g_sdtc_stamp_calls = 0; }

#ifdef B200ATTN_SD_PROFILE
int b200attn_debug_sd_stamps(unsigned long long *out, int n) {
    return (int)cudaMemcpyFromSymbol(out, sd_stamps, (size_t)n * sizeof(unsigned long long));
}
#endif

#ifdef B200ATTN_TC_PROFILE
int b200attn_debug_tc_prof(unsigned long long *out32, int reset) {
    if (reset) { unsigned long long z[32] = {}; return (int)cudaMemcpyToSymbol(tc_prof, z, sizeof z); }
    return (int)cudaMemcpyFromSymbol(out32, tc_prof, 32 * sizeof(unsigned long long));
}
#endif
#endif  // B200ATTN_DEVTOOLS

int b200attn_forward_many(const b200attn_args *args, int n) {
    if (args == nullptr || n < 0) return fail(B200ATTN_ERR_INVALID_ARG, "b200attn_forward_many: NULL args or negative n");
    for (int i = 0; i < n; ++i) {
        // the entries are independent problems by contract: entry i may overlap the tail of entry i - 1
        const bool beside_prev = i > 0 && !(args[i].flags & B200ATTN_FLAG_NO_OVERLAP);
        const bool beside_next = i + 1 < n && !(args[i + 1].flags & B200ATTN_FLAG_NO_OVERLAP);
        int rc = forward_device(&args[i], beside_prev, beside_prev || beside_next);
        if (rc) return rc;
    }
    return B200ATTN_OK;
}

int b200attn_forward_host(const b200attn_args *h) {
    int rd; float base;
    int rc = validate(h, &rd, &base);
    if (rc) return rc;
    if (h->cos_cache || h->sin_cache) return fail(B200ATTN_ERR_INVALID_ARG, "b200attn_forward_host takes no cos/sin caches");
    DeviceCtx *c;
    rc = get_ctx(&c);
    if (rc) return rc;
    const size_t esz = h->dtype == B200ATTN_F32 ? 4 : 2;
    const long long BH = (long long)h->batch_sz * h->num_heads;
    const size_t q1 = (size_t)h->len_q * h->head_d * esz, k1 = (size_t)h->len_k * h->head_d * esz;   // bytes per (b,h) slice
    // (batch, head) slices are independent and contiguous, so the problem is cut into chunks of heads
    // and copy-in, compute and copy-out of consecutive chunks overlap on three streams (two buffer
    // sets).  Small problems go through in one chunk.
    long long chunk = BH;
    const size_t per_head = 2 * q1 + 2 * k1;
    if ((size_t)BH * per_head > ((size_t)64 << 20)) {
        chunk = (long long)((((size_t)256 << 20) + per_head - 1) / per_head);   // about 256 MiB of traffic per chunk
        if (chunk < 1) chunk = 1;
        if (chunk * 4 > BH) chunk = (BH + 3) / 4;                                // at least four chunks in flight
        if (chunk < 1) chunk = 1;
    }
    const long long nchunks = (BH + chunk - 1) / chunk;
    {
        std::lock_guard<std::mutex> lk(c->mu);
        if (!c->host_streams[0]) {
            for (int i = 0; i < 3; ++i) CU_TRY(cudaStreamCreateWithFlags(&c->host_streams[i], cudaStreamNonBlocking));
            for (int i = 0; i < 6; ++i) CU_TRY(cudaEventCreateWithFlags(&c->host_events[i], cudaEventDisableTiming));
        }
        const int nbuf = nchunks > 1 ? 2 : 1;
        for (int sset = 0; sset < nbuf; ++sset) {
            if ((rc = ensure_stage(*c, 4 * sset + 0, (size_t)chunk * q1)) || (rc = ensure_stage(*c, 4 * sset + 1, (size_t)chunk * k1)) ||
                (rc = ensure_stage(*c, 4 * sset + 2, (size_t)chunk * k1)) || (rc = ensure_stage(*c, 4 * sset + 3, (size_t)chunk * q1)))
                return rc;
        }
    }
    cudaStream_t s_in = c->host_streams[0], s_run = c->host_streams[1], s_out = c->host_streams[2];
    cudaEvent_t *ev_in = &c->host_events[0], *ev_run = &c->host_events[2], *ev_out = &c->host_events[4];   // [2] each, by buffer set
    for (long long ci = 0; ci < nchunks; ++ci) {
        const int sset = (int)(ci & 1);
        const long long h0 = ci * chunk, n = (BH - h0 < chunk) ? (BH - h0) : chunk;
        void *dq = c->stage[4 * sset + 0], *dk = c->stage[4 * sset + 1], *dv = c->stage[4 * sset + 2], *dout = c->stage[4 * sset + 3];
        // the inputs of this buffer set may be overwritten once the chunk two steps back has been computed
        if (ci >= 2) CU_TRY(cudaStreamWaitEvent(s_in, ev_run[sset], 0));
        CU_TRY(cudaMemcpyAsync(dq, (const char *)h->Q + (size_t)h0 * q1, (size_t)n * q1, cudaMemcpyHostToDevice, s_in));
        CU_TRY(cudaMemcpyAsync(dk, (const char *)h->K + (size_t)h0 * k1, (size_t)n * k1, cudaMemcpyHostToDevice, s_in));
        CU_TRY(cudaMemcpyAsync(dv, (const char *)h->V + (size_t)h0 * k1, (size_t)n * k1, cudaMemcpyHostToDevice, s_in));
        CU_TRY(cudaEventRecord(ev_in[sset], s_in));
        CU_TRY(cudaStreamWaitEvent(s_run, ev_in[sset], 0));
        if (ci >= 2) CU_TRY(cudaStreamWaitEvent(s_run, ev_out[sset], 0));   // the output buffer has been copied out
        b200attn_args d = *h;
        d.Q = dq; d.K = dk; d.V = dv; d.out = dout;
        d.batch_sz = 1; d.num_heads = (int)n;
        d.stream = s_run;
        d.flags = (h->flags | B200ATTN_FLAG_ASYNC);
        rc = forward_device(&d);
        if (rc) { cudaDeviceSynchronize(); return rc; }
        CU_TRY(cudaEventRecord(ev_run[sset], s_run));
        CU_TRY(cudaStreamWaitEvent(s_out, ev_run[sset], 0));
        CU_TRY(cudaMemcpyAsync((char *)h->out + (size_t)h0 * q1, dout, (size_t)n * q1, cudaMemcpyDeviceToHost, s_out));
        CU_TRY(cudaEventRecord(ev_out[sset], s_out));
    }
    CU_TRY(cudaStreamWaitEvent(s_out, ev_run[(nchunks - 1) & 1], 0));
    CU_TRY(cudaStreamSynchronize(s_out));
    CU_TRY(cudaStreamSynchronize(s_in));
    CU_TRY(cudaStreamSynchronize(s_run));
    return report_kernel_errors(*c, "kernel");
}

void b200attn_shard_ranges(long long total, int n, long long *begin, long long *count) {
    if (n <= 0) return;
    const long long q = total / n, r = total % n;
    long long at = 0;
    for (int g = 0; g < n; ++g) {
        count[g] = q + (g < r ? 1 : 0);
        begin[g] = at;
        at += count[g];
    }
}

int b200attn_forward_sharded(const b200attn_args *proto, int n, const int *devices, const void *const *Q, const void *const *K,
                             const void *const *V, void *const *out, const int *bh_count) {
    if (!proto || n <= 0 || !devices || !Q || !K || !V || !out || !bh_count)
        return fail(B200ATTN_ERR_INVALID_ARG, "b200attn_forward_sharded: NULL argument or n_devices <= 0");
    int prev = 0;
    CU_TRY(cudaGetDevice(&prev));
    int status = B200ATTN_OK;
    std::vector<cudaStream_t> streams(n, nullptr);
    // launch everywhere first, wait afterwards
    for (int g = 0; g < n && status == B200ATTN_OK; ++g) {
        if (bh_count[g] <= 0) continue;
        cudaError_t e = cudaSetDevice(devices[g]);
        if (e != cudaSuccess) {
            status = fail(B200ATTN_ERR_CUDA, "cudaSetDevice(%d): %s", devices[g], cudaGetErrorString(e));
            (void)cudaGetLastError();   // the failure is reported through the status; do not leave it pending
            break;
        }
        DeviceCtx *c;
        if ((status = get_ctx(&c))) break;
        if (!c->shard_stream) {
            e = cudaStreamCreateWithFlags(&c->shard_stream, cudaStreamNonBlocking);
            if (e != cudaSuccess) { status = fail(B200ATTN_ERR_CUDA, "cudaStreamCreate: %s", cudaGetErrorString(e)); break; }
        }
        streams[g] = c->shard_stream;
        b200attn_args a = *proto;
        a.Q = Q[g]; a.K = K[g]; a.V = V[g]; a.out = out[g];
        a.batch_sz = 1; a.num_heads = bh_count[g];
        a.stream = c->shard_stream;
        a.flags |= B200ATTN_FLAG_ASYNC;
        status = forward_device(&a);
    }
    for (int g = 0; g < n; ++g) {
        if (!streams[g]) continue;
        cudaSetDevice(devices[g]);
        DeviceCtx &c = g_ctx[devices[g]];
        cudaError_t e = cudaStreamSynchronize(streams[g]);
        if (e != cudaSuccess && status == B200ATTN_OK) status = fail(B200ATTN_ERR_CUDA, "device %d: %s", devices[g], cudaGetErrorString(e));
        if (c.ready && *reinterpret_cast<volatile unsigned *>(c.err_host) != 0) {
            char what[32];
            snprintf(what, sizeof what, "device %d: kernel", devices[g]);
            std::lock_guard<std::mutex> lk(c.mu);
            const int rc = report_kernel_errors(c, what);
            if (status == B200ATTN_OK) status = rc;
        }
    }
    cudaSetDevice(prev);
    return status;
}

// Failure detection can be exercised without faulting anything: with extra > 0 the next fused
// split-head_d launches wait (at most spin_limit polls) for arrivals that never come, give up, and
// report B200ATTN_ERR_KERNEL through the normal error path.  (0, 0) restores normal operation.
void b200attn_debug_lost_arrival(unsigned extra, unsigned spin_limit) {
    g_test_wait_extra.store(extra);
    g_test_spin_limit.store(spin_limit);
}

// Per-kernel timing of the two-kernel bf16 path.  enable = 1 / 0 switches the recording on / off
// (single-threaded use, one device); with out != NULL the call synchronises the device and returns
// the summed milliseconds of [encoding score launches, score launches, P V launches] in out[0..2]
// and the launch counts in out[3..5], clearing the record.
int b200attn_debug_kernel_times(int enable, double *out) {
    TcwTimer &t = tcw_timer();
    if (out != nullptr) {
        if (cudaDeviceSynchronize() != cudaSuccess) return B200ATTN_ERR_CUDA;
        int cnt[3];
        t.collect(out, cnt);
        for (int k = 0; k < 3; ++k) out[3 + k] = (double)cnt[k];
    }
    t.on = (enable != 0);
    return B200ATTN_OK;
}

// Host copy of the tile enumeration of the two-kernel bf16 path, for tests (no GPU needed).  big = 0:
// tile j of a head in launch `mode` (0 all tiles, 1 encoding launch, 2 its complement) -> (query tile,
// key tile); big = 1: the 256-row variant -> (query-tile pair, key tile).  Returns the number of tiles
// per head of that launch, or -1 when the launch does not exist for the shape.
int b200attn_debug_tile_of(int big, int mode, int j, int nqt, int nkt, int *qt, int *kt) {
    if (nqt <= 0 || nkt <= 0 || mode < 0 || mode > 2) return -1;
    const int nA = nqt > nkt ? nqt : nkt;
    int count = mode == 0 ? nqt * nkt : mode == 1 ? nA : nqt * nkt - nA;
    if (big) {
        if (mode == 1 || nqt % 2 != 0) return -1;
        if (mode == 2 && !(nkt <= nqt && nqt >= 2 * nkt - 1)) return -1;
        count /= 2;
        if (j >= 0 && j < count) tcw_tile256_of(mode, j, nkt, qt, kt);
    } else if (j >= 0 && j < count) {
        tcw_tile_of(mode, j, nqt, nkt, qt, kt);
    }
    return count;
}

int b200attn_rope_k(const void *X, void *X_rot, int batch_sz, int num_heads, int len, int head_d, int dtype, int pairing,
                    int rotary_dim, float rope_base, int pos0, const float *cos_cache, const float *sin_cache, void *stream) {
    if (!X || !X_rot || batch_sz <= 0 || num_heads <= 0 || len <= 0 || head_d <= 0 || pos0 < 0)
        return fail(B200ATTN_ERR_INVALID_ARG, "b200attn_rope_k: NULL pointer, non-positive size or negative position");
    if (dtype != B200ATTN_F32 && dtype != B200ATTN_BF16 && dtype != B200ATTN_F16) return fail(B200ATTN_ERR_INVALID_ARG, "unknown dtype %d", dtype);
    if (pairing != B200ATTN_PE_ROPE_INTERLEAVED && pairing != B200ATTN_PE_ROPE_HALF)
        return fail(B200ATTN_ERR_INVALID_ARG, "b200attn_rope_k: pairing must be B200ATTN_PE_ROPE_INTERLEAVED or B200ATTN_PE_ROPE_HALF");
    const int rd = rotary_dim == 0 ? head_d : rotary_dim;
    if (rd < 0 || rd > head_d || (rd & 1)) return fail(B200ATTN_ERR_INVALID_ARG, "rotary_dim must be even and within [0, head_d] (got %d, head_d %d)", rd, head_d);
    if ((cos_cache == nullptr) != (sin_cache == nullptr)) return fail(B200ATTN_ERR_INVALID_ARG, "cos_cache and sin_cache must be given together");
    const float base = rope_base == 0.0f ? 10000.0f : rope_base;
    if (!(base > 0.0f)) return fail(B200ATTN_ERR_INVALID_ARG, "rope_base must be positive");
    const size_t esz = dtype == B200ATTN_F32 ? 4 : 2;
    if (((uintptr_t)X | (uintptr_t)X_rot) & (esz - 1)) return fail(B200ATTN_ERR_INVALID_ARG, "tensor pointers must be aligned to the element size");
    DeviceCtx *c;
    int rc = get_ctx(&c);
    if (rc) return rc;
    RopeKParams p{};
    p.X = X; p.Y = X_rot;
    p.BH = (long long)batch_sz * num_heads; p.L = len; p.D = head_d; p.rd = rd;
    p.half = pairing == B200ATTN_PE_ROPE_HALF ? 1 : 0;
    p.pos0 = pos0; p.base = base; p.cos_cache = cos_cache; p.sin_cache = sin_cache;
    cudaError_t e = dtype == B200ATTN_F32 ? launch_rope_k<float>(p, c->sm_count, (cudaStream_t)stream)
                    : dtype == B200ATTN_F16 ? launch_rope_k<__half>(p, c->sm_count, (cudaStream_t)stream)
                                            : launch_rope_k<__nv_bfloat16>(p, c->sm_count, (cudaStream_t)stream);
    if (e != cudaSuccess) return fail(B200ATTN_ERR_CUDA, "CUDA error %d (%s) launching the rotation kernel", (int)e, cudaGetErrorString(e));
    g_launches.fetch_add(1);
    return B200ATTN_OK;
}

int b200attn_set_option(int option, long long value) {
    switch (option) {
    case B200ATTN_OPT_SCORE_SCRATCH_MB:
        if (value < 1) return fail(B200ATTN_ERR_INVALID_ARG, "the score scratch cap must be at least 1 MiB");
        g_score_scratch_mb.store(value);
        return B200ATTN_OK;
    case B200ATTN_OPT_SPIN_LIMIT:
        if (value < 1 || value > 0x7fffffffLL) return fail(B200ATTN_ERR_INVALID_ARG, "the poll limit must be in [1, 2^31)");
        g_spin_limit.store((unsigned)value);
        return B200ATTN_OK;
    default:
        return fail(B200ATTN_ERR_INVALID_ARG, "unknown option %d", option);
    }
}

const char *b200attn_last_error(void) { return t_last_error.c_str(); }
const char *b200attn_last_path(void) { return t_last_path; }
unsigned long long b200attn_launch_count(void) { return g_launches.load(); }
const char *b200attn_version(void) { return "b200attn 0.1 (sm_100a)"; }

void b200attn_release_workspace(void) {
    int prev = 0;
    if (cudaGetDevice(&prev) != cudaSuccess) return;
    for (int dev = 0; dev < kMaxDevices; ++dev) {
        DeviceCtx &c = g_ctx[dev];
        if (!c.ready) continue;
        std::lock_guard<std::mutex> lk(c.mu);
        cudaSetDevice(dev);
        cudaDeviceSynchronize();
        if (c.S) cudaFree(c.S);
        c.S = nullptr; c.S_bytes = 0;
        if (c.counters) cudaFree(c.counters);
        c.counters = nullptr; c.counters_n = 0;
        if (c.sdtc_S) cudaFree(c.sdtc_S);
        if (c.sdtc_cnt) cudaFree(c.sdtc_cnt);
        if (c.sdtc_gen) cudaFree(c.sdtc_gen);
        c.sdtc_S = nullptr; c.sdtc_cnt = nullptr; c.sdtc_gen = nullptr; c.sdtc_cap = 0; c.sdtc_seq = 0;
        for (int i = 0; i < ST_NBUF; ++i) c.sdtc_gen_expect[i] = 0;
        for (int i = 0; i < 8; ++i) { if (c.stage[i]) cudaFree(c.stage[i]); c.stage[i] = nullptr; c.stage_bytes[i] = 0; }
        c.tc_tables.release();
        c.tcw.release();
        c.prev_sdtc = false;
    }
    cudaSetDevice(prev);
}

int b200attn_synth_fill(void *dst, long long n, unsigned long long seed, unsigned long long tensor_id, long long index0,
                        int dist, int dtype, void *stream) {
    if (!dst || n < 0 || (dist != 0 && dist != 1) || (dtype != B200ATTN_F32 && dtype != B200ATTN_BF16))
        return fail(B200ATTN_ERR_INVALID_ARG, "b200attn_synth_fill: bad argument");
    if (n == 0) return B200ATTN_OK;
    DeviceCtx *c;
    int rc = get_ctx(&c);
    if (rc) return rc;
    launch_synth_fill(dst, n, seed, tensor_id, index0, dist, dtype, c->sm_count, (cudaStream_t)stream);
    CU_TRY(cudaGetLastError());
    g_launches.fetch_add(1);
    return B200ATTN_OK;
}

}  // extern "C"
