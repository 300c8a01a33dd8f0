/*
 * b200attn — scaled-dot-product attention forward for NVIDIA B200 (sm_100a), C ABI.
 *
 * The library is a drop-in for the host launchers of agoel2005/accelerated-final-project: the
 * first group of functions below has the names, argument order, argument meaning and error
 * behaviour of those launchers (each comment cites the reference definition it replaces, path
 * relative to the reference tree).  The second group is this library's own extended interface
 * (status codes instead of exit(), streams, positional-encoding selector, host-buffer and
 * multi-GPU entry points).
 *
 * Conventions of the drop-in group (taken from the reference, QUICKSTART.md:67-84,132-172 and
 * final/attention.cu:195-221):
 *   - all tensors are dense row-major [B,H,L,D]: idx = ((b*H+h)*L + i)*D + d; K and V share Lk;
 *   - pointers are DEVICE pointers on the current device, caller-owned, 16-byte aligned;
 *     `out` is written in full and must not alias an input;
 *   - scale = 1/sqrtf(head_d); non-causal; no mask; positions are the row indices 0..L-1;
 *   - the call runs on the legacy default stream and returns after the work has completed;
 *   - on a CUDA error or an invalid argument the call prints a message to stderr and calls
 *     exit(EXIT_FAILURE), as the reference's CUDA_CHECK does (final/attention.cu:12-21).
 *   - bf16 tensors are arrays of 16-bit bfloat16 (__nv_bfloat16), passed as void pointers.
 *
 * There is no CPU fallback: without a CUDA device the calls fail.
 */
#ifndef B200ATTN_H
#define B200ATTN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------------------------------ */
/* Drop-in entry points                                                                        */
/* ------------------------------------------------------------------------------------------ */

/* fp32 forward.  Replaces attention_forward_optimized, final/attention.cu:195-221 (declared
 * extern "C" by its external caller, final/benchmark_pytorch_comparison.cu:22-24). */
void attention_forward_optimized(const float *Q, const float *K, const float *V, float *out,
                                 int batch_sz, int num_heads, int len_q, int len_k, int head_d);

/* bf16 in/out; the products accumulate in fp32 and the row maxima, exponentials' sums and the final
 * division are fp32.  On the default tensor-core path the scores pass through a bf16 scratch (stored
 * relative to the fp32 maximum of their 256-key tile) and a positional encoding is applied to the bf16
 * operands with a single rounding.  Replaces attention_forward_bf16,
 * kernels/attention_bf16_optimized_fused.cu:493-505. */
void attention_forward_bf16(const void *Q, const void *K, const void *V, void *out,
                            int batch_sz, int num_heads, int len_q, int len_k, int head_d);

/* fp32, RoPE fused into the Q/K load: raw K, full rotation (rotary_dim = head_d), interleaved
 * pairs (2i,2i+1), theta 10000, angles computed in-kernel.  Replaces
 * attention_forward_rope_fused_v2, final/rope.cu:375-391. */
void attention_forward_rope_fused_v2(const float *Q, const float *K, const float *V, float *out,
                                     int batch_sz, int num_heads, int len_q, int len_k, int head_d);

/* fp32, RoPE fused, angles taken from caller-supplied device caches of shape [max(Lq,Lk), head_d]
 * in the layout of precompute_rope_cache (final/rope.cu:20-40: the value of pair i is stored at
 * columns 2i and 2i+1).  Replaces attention_forward_rope_fused, final/rope.cu:1209-1238. */
void attention_forward_rope_fused(const float *Q, const float *K, const float *V, float *out,
                                  const float *cos_cache, const float *sin_cache,
                                  int batch_sz, int num_heads, int len_q, int len_k, int head_d);

/* fp32 "hybrid": Q is rotated in the load (interleaved pairs, first rotary_dim columns), K is
 * taken as already rotated by the caller.  Replaces attention_forward_rope_fused_v7_hybrid,
 * final/rope.cu:230-247. */
void attention_forward_rope_fused_v7_hybrid(const float *Q, const float *K_rotated, const float *V,
                                            float *out, int batch_sz, int num_heads, int len_q,
                                            int len_k, int head_d, int rotary_dim);

/* bf16, RoPE of raw Q and raw K fused (full rotation, interleaved pairs, theta 10000).  Replaces
 * attention_forward_rope_bf16, kernels/attention_bf16_all_kernels.cu:451-466. */
void attention_forward_rope_bf16(const void *Q, const void *K, const void *V, void *out,
                                 int batch_sz, int num_heads, int len_q, int len_k, int head_d);

/* bf16 hybrid (Q rotated in the load, K pre-rotated).  Replaces the 10-argument overload
 * attention_forward_rope_bf16 of kernels/attention_bf16_optimized_fused.cu:507-519; renamed
 * because C has no overloading. */
void attention_forward_rope_bf16_v7(const void *Q, const void *K_rotated, const void *V, void *out,
                                    int batch_sz, int num_heads, int len_q, int len_k, int head_d,
                                    int rotary_dim);

/* fp32, additive sinusoidal encoding fused into the Q/K load: PE[p,2i] = sin(p*f_i),
 * PE[p,2i+1] = cos(p*f_i), f_i = 10000^(-2i/head_d), added to Q and K (not V) in fp32.  The
 * reference has no host wrapper for this path; this replaces the direct launch of
 * attention_fwd_kernel_sinusoidal_fused_v5 at final/sinusoidal.cu:1135-1137 (kernel :84-234). */
void attention_forward_sinusoidal_fused(const float *Q, const float *K, const float *V, float *out,
                                        int batch_sz, int num_heads, int len_q, int len_k, int head_d);

/* bf16 variant of the above.  Replaces attention_forward_sinusoidal_bf16,
 * kernels/attention_bf16_optimized_fused.cu:521-533. */
void attention_forward_sinusoidal_bf16(const void *Q, const void *K, const void *V, void *out,
                                       int batch_sz, int num_heads, int len_q, int len_k, int head_d);

/* ------------------------------------------------------------------------------------------ */
/* Extended interface                                                                          */
/* ------------------------------------------------------------------------------------------ */

enum b200attn_status {
    B200ATTN_OK = 0,
    B200ATTN_ERR_INVALID_ARG = 1,   /* null pointer, non-positive size, alignment, unsupported combination */
    B200ATTN_ERR_CUDA = 2,          /* a CUDA runtime/driver call failed; see b200attn_last_error() */
    B200ATTN_ERR_NO_DEVICE = 3,     /* no usable sm_100 device */
    B200ATTN_ERR_KERNEL = 4,        /* a kernel reported an internal error (bounded wait expired) */
    B200ATTN_ERR_TOO_LARGE = 5      /* a fixed-capacity entry point was given a problem beyond its limit */
};

/* B200ATTN_F16 (IEEE half in and out, fp32 accumulation) has no launcher of its own in the reference's
 * final/ tree; it covers what kernels/attention_kernel_fp16.cu:194 (attention_forward_fp16) does.  Without a
 * positional encoding it runs on the tensor cores for the shapes the bf16 paths take; with one, on the
 * CUDA-core kernels. */
enum b200attn_dtype { B200ATTN_F32 = 0, B200ATTN_BF16 = 1, B200ATTN_F16 = 2 };

/* Positional encoding applied to Q and K inside the load (no separate pass). */
enum b200attn_pe {
    B200ATTN_PE_NONE = 0,
    B200ATTN_PE_ROPE_INTERLEAVED = 1, /* pairs (2i, 2i+1), final/rope.cu:138-149 */
    B200ATTN_PE_ROPE_HALF = 2,        /* pairs (i, i + rotary_dim/2) ("rotate-half") */
    B200ATTN_PE_SINUSOIDAL = 3,       /* additive, final/sinusoidal.cu:143-161 */
    B200ATTN_PE_ROPE_Q_ONLY = 4,      /* interleaved on Q only; K is pre-rotated, final/rope.cu:102-228 */
    B200ATTN_PE_ROPE_HALF_Q_ONLY = 5  /* rotate-half on Q only; K is pre-rotated (e.g. by b200attn_rope_k) */
};

enum b200attn_flags {
    B200ATTN_FLAG_ASYNC = 1,          /* enqueue only; do not synchronise the stream */
    B200ATTN_FLAG_FORCE_GENERIC = 2,  /* use the CUDA-core split-head_d kernels even where a tensor-core kernel applies */
    B200ATTN_FLAG_FORCE_TWO_PASS = 4, /* split-head_d path: two launches instead of one fused launch */
    B200ATTN_FLAG_PREFER_ONE_KERNEL = 8, /* bf16: where both tensor-core paths take the shape, run the one-kernel cluster pipeline */
    B200ATTN_FLAG_NO_OVERLAP = 16,    /* b200attn_forward_many: start this entry only after the previous one has completed */
    B200ATTN_FLAG_TWO_KERNELS = 32    /* bf16 / fp16, head_d 64, 128 or 256: run the two-kernel path where the one-kernel narrow-head path would run (the two are measured against each other that way) */
};

typedef struct b200attn_args {
    size_t struct_size;      /* sizeof(b200attn_args) */
    const void *Q, *K, *V;   /* device pointers, [B,H,Lq,D] / [B,H,Lk,D] */
    void *out;               /* device pointer, [B,H,Lq,D] */
    int batch_sz, num_heads, len_q, len_k, head_d;
    int dtype;               /* enum b200attn_dtype */
    int pe;                  /* enum b200attn_pe */
    int rotary_dim;          /* RoPE kinds: even, <= head_d; 0 means head_d */
    float rope_base;         /* RoPE kinds: theta; 0 means 10000 */
    const float *cos_cache;  /* optional (all RoPE kinds): device [max(Lq,Lk), rotary_dim] caches */
    const float *sin_cache;  /*   in the precompute_rope_cache layout; NULL = angles computed by the library */
    void *stream;            /* cudaStream_t; NULL = legacy default stream */
    unsigned flags;          /* enum b200attn_flags */
} b200attn_args;

/* The general entry point: validates, launches on args->stream, synchronises that stream unless
 * B200ATTN_FLAG_ASYNC is set.  Never exits the process.  Thread-compatible per device: calls for
 * one device must not overlap in time on different host threads.  Calls for one device share scratch
 * and tables: a call on another stream than the previous call of that device is ordered, on the
 * device, after everything enqueued on the previous call's stream (so asynchronous calls on several
 * streams are safe but do not run concurrently). */
int b200attn_forward_ex(const b200attn_args *args);

/* Enqueues n INDEPENDENT problems (args[i] for i < n) in one call; stops at the first failure.
 * Each entry is handled as by b200attn_forward_ex (give them B200ATTN_FLAG_ASYNC to enqueue them back
 * to back without a host synchronisation in between), with one difference: because no entry may read
 * what another entry of the same call writes, the library lets consecutive entries on one stream
 * overlap on the GPU (entry i starts loading its inputs while entry i-1 is finishing; an entry whose
 * Q, K or V overlaps the previous entry's `out` is simply not overlapped). */
int b200attn_forward_many(const b200attn_args *args, int n);

/* Same computation with HOST buffers (pageable or pinned): copies Q, K, V to device staging
 * buffers owned by the library, runs the forward, copies `out` back, and returns when `out` is
 * complete.  The device-side fields `stream` and B200ATTN_FLAG_ASYNC are ignored. */
int b200attn_forward_host(const b200attn_args *args_with_host_pointers);

/* (batch, head) data-parallel launcher for the GPUs of one box: entry g of each pointer array is a
 * device pointer ON devices[g] holding that device's contiguous range of flat (b*H+h) slices,
 * bh_count[g] of them (slices are contiguous L*D slabs, so no repacking and no collective is
 * involved).  All devices are launched before any is waited for; returns after all completed.
 * `proto` supplies everything except Q/K/V/out/batch_sz/num_heads/stream. */
int b200attn_forward_sharded(const b200attn_args *proto, int n_devices, const int *devices,
                             const void *const *Q, const void *const *K, const void *const *V,
                             void *const *out, const int *bh_count);

/* Splits B*H slices over n parts as evenly as possible: part g gets [begin[g], begin[g]+count[g]). */
void b200attn_shard_ranges(long long total_bh, int n_parts, long long *begin, long long *count);

/* Message for the last non-OK status returned on the calling thread ("" if none). */
const char *b200attn_last_error(void);

/* Name of the kernel path the last successful b200attn_forward_ex on this thread used:
 * "splitd_tc" (fp32, short sequences, tensor cores with error-compensated tf32), "splitd_fused" and
 * "splitd_two_pass" (CUDA cores), "tc_wide" (bf16 on the tensor cores: score kernel, then P V kernel),
 * "tc_fused" (bf16 / fp16, head_d 64, 128 or 256, more than 64 queries: one kernel, scores in tensor
 * memory; an encoding is applied to copies of Q and K first), "tc_bf16" (bf16 on the tensor cores, one-kernel
 * cluster pipeline) or "tc_decode" (bf16, up to 64 queries against a long K/V: key splits on the tensor cores
 * plus a combine kernel). */
const char *b200attn_last_path(void);

/* Number of kernel launches issued by this library in this process so far. */
unsigned long long b200attn_launch_count(void);

/* Frees the per-device scratch and staging buffers the library holds. */
void b200attn_release_workspace(void);

/* Library version string. */
const char *b200attn_version(void);

/* "Rotate once and keep it": X_rot = RoPE(X) for a device tensor X [B,H,len,head_d] (fp32, bf16 or fp16), the
 * first rotary_dim columns rotated and the rest copied; row l of every (b,h) slice has position pos0 + l
 * (pos0 > 0 when keys are appended to a cache).  A KV-cache caller rotates K with this once and then calls
 * attention with a *_Q_ONLY encoding.  pairing is B200ATTN_PE_ROPE_INTERLEAVED or B200ATTN_PE_ROPE_HALF;
 * rotary_dim 0 means head_d; rope_base 0 means 10000; cos_cache / sin_cache are optional device caches
 * [>= pos0 + len][rotary_dim] in the precompute_rope_cache layout (NULL: angles computed with the fp32
 * arithmetic of that function, final/rope.cu:20-40).  X_rot may be X (in place).  Enqueued on `stream`, not
 * waited for.  Replaces rope_kernel, final/rope.cu:1240-1280, as used by attention_forward_separate_rope
 * (final/rope.cu:1379-1416); that kernel takes the position modulo 64 (:1257), this one does not. */
int b200attn_rope_k(const void *X, void *X_rot, int batch_sz, int num_heads, int len, int head_d, int dtype, int pairing,
                    int rotary_dim, float rope_base, int pos0, const float *cos_cache, const float *sin_cache, void *stream);

/* Process-wide settings (they apply to calls made after the change). */
enum b200attn_option {
    B200ATTN_OPT_SCORE_SCRATCH_MB = 1, /* bf16 two-kernel path: cap, in MiB, of the score scratch of one pass over the heads (default 2048) */
    B200ATTN_OPT_SPIN_LIMIT = 2        /* polls after which a wait inside a kernel gives up and reports B200ATTN_ERR_KERNEL (default 2^21) */
};
int b200attn_set_option(int option, long long value);

/* Measurement and test hooks (no counterpart in the reference).
 * b200attn_debug_kernel_times: enable = 1 / 0 switches per-launch CUDA-event timing of the bf16
 *   two-kernel path on / off (single-threaded use, one device); with out != NULL the call first
 *   synchronises the device and returns the summed milliseconds of [encoding score launches, score
 *   launches, P V launches] in out[0..2] and the launch counts in out[3..5], clearing the record.
 * b200attn_debug_lost_arrival: failure detection without a fault.  With extra > 0 the per-head barrier
 *   of the fp32 split-head_d kernels waits (at most spin_limit polls) for arrivals that never come, gives
 *   up, and the call reports B200ATTN_ERR_KERNEL; (0, 0) restores normal operation.
 * b200attn_debug_tile_of: host copy of the tile enumeration of the bf16 two-kernel path (big = 0: tile j
 *   of a head in launch `mode` -> query tile, key tile; big = 1: the 256-row variant); returns the number
 *   of tiles per head of that launch or -1 when the launch does not exist for the shape.  Needs no GPU. */
int b200attn_debug_kernel_times(int enable, double *out);
void b200attn_debug_lost_arrival(unsigned extra, unsigned spin_limit);
int b200attn_debug_tile_of(int big, int mode, int j, int nqt, int nkt, int *qt, int *kt);

/* fp32 forward without positional encoding that never allocates device memory: its scratch is a
 * fixed array inside the library image (B200ATTN_STATIC_SCRATCH_BYTES per GPU, held from library
 * load to process exit).  For callers that cannot call cudaMalloc when they need attention: code
 * living under a framework allocator that owns the device, or a latency-critical loop that cannot
 * afford the implicit synchronisation of an allocation.
 * No counterpart in the reference (its launcher needs no scratch).  Device pointers as for
 * attention_forward_optimized; the work is enqueued on `stream` and NOT waited for.  Limits:
 * len_q, len_k <= 64, batch_sz*num_heads <= SM count,
 * 256 + round_up(8*batch_sz*num_heads, 256) + 4*batch_sz*num_heads*len_q*len_k bytes within the
 * static scratch, and a head's column slices must fit one per SM: with
 * s = floor(SM count / (batch_sz*num_heads)) slices per head, ceil(head_d / s) <= about 270 columns
 * (e.g. 148 heads of head_d 8192 are refused); beyond them the call returns B200ATTN_ERR_TOO_LARGE
 * and does nothing.  The first
 * call on a device does host-side set-up (symbol address, shared-memory limit): make it before any
 * stream capture.  All calls share the one array, so calls that overlap on the GPU race; the kernel's
 * error word is not read back (check the output, or use b200attn_forward_ex).  Message of the last
 * failure on this thread: b200attn_static_last_error(). */
#define B200ATTN_STATIC_SCRATCH_BYTES 1048576u
int b200attn_forward_static(const float *Q, const float *K, const float *V, float *out, int batch_sz, int num_heads,
                            int len_q, int len_k, int head_d, void *stream);
const char *b200attn_static_last_error(void);

/* Fills a device buffer with the synthetic inputs the tests and the benchmark use: element i gets
 * a value drawn from splitmix64(seed*2^40 + tensor_id*2^36 + index0 + i); dist 0 = uniform[-1,1),
 * 1 = normal(0,1) by Box-Muller; stored as fp32 or rounded to bf16. */
int b200attn_synth_fill(void *dst, long long n, unsigned long long seed, unsigned long long tensor_id,
                        long long index0, int dist, int dtype, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* B200ATTN_H */
