/*
 * CPU oracle for the attention-forward path.  TEST INFRASTRUCTURE ONLY: this file is the checker
 * the CUDA library is compared against; nothing the library ships links, loads or calls it.
 *
 * Every function restates, in plain C with 64-bit indexing, the arithmetic of one CPU routine of
 * the reference project (paths are relative to the reference tree):
 *
 *   oracle_attention_f32            final/attention.cu:228-283   (attention_cpu)
 *   oracle_rope_cache               final/rope.cu:20-40          (precompute_rope_cache)
 *   oracle_apply_rope_interleaved   final/rope.cu:1418-1437      (apply_rope_cpu)
 *   oracle_attention_rope_f32       final/rope.cu:1439-1499      (attention_rope_cpu)
 *   oracle_sinusoidal_tables        final/sinusoidal.cu:838-855  (generate_sinusoidal_embeddings_cpu)
 *   oracle_attention_sinusoidal_f32 final/sinusoidal.cu:858-928  (attention_sinusoidal_cpu)
 *
 * Parity is pinned: tests compare these functions with the reference's own CPU routines compiled
 * from the reference tree (oracle/_ref) and with the reference's golden SDPA vectors.
 *
 * The order of floating-point operations follows the reference exactly (sequential fp32 sums,
 * probabilities divided by the row sum before the PV product) so the restatement is bit-identical
 * to the reference CPU code when both are built without fast-math.
 *
 * Layout everywhere: dense row-major [B,H,L,D], idx = ((b*H+h)*L + i)*D + d.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef long long i64;

/* ---- pe kinds shared with the library header (include/b200attn.h) ---- */
enum {
    ORACLE_PE_NONE = 0,
    ORACLE_PE_ROPE_INTERLEAVED = 1, /* pairs (2i,2i+1): final/rope.cu:138-149 */
    ORACLE_PE_ROPE_HALF = 2,        /* pairs (i,i+rd/2): rotate-half pairing */
    ORACLE_PE_SINUSOIDAL = 3,       /* additive: final/sinusoidal.cu:143-161 */
    ORACLE_PE_ROPE_Q_ONLY = 4       /* interleaved on Q only, K given pre-rotated: final/rope.cu:102-228 */
};

/* One (b,h) slice of naive attention; q,k,v,o point at the slice.  final/attention.cu:243-280 */
static void attention_slice(const float *q, const float *k, const float *v, float *o,
                            int len_q, int len_k, int head_d, float *scores) {
    const float scale = 1.0f / sqrtf((float)head_d);
    for (int i = 0; i < len_q; i++) {
        const float *qi = q + (i64)i * head_d;
        float max_s = -INFINITY;
        for (int j = 0; j < len_k; j++) {
            const float *kj = k + (i64)j * head_d;
            float s = 0.0f;
            for (int d = 0; d < head_d; d++) s += qi[d] * kj[d];
            s *= scale;
            scores[j] = s;
            max_s = fmaxf(max_s, s);
        }
        float total = 0.0f;
        for (int j = 0; j < len_k; j++) {
            scores[j] = expf(scores[j] - max_s);
            total += scores[j];
        }
        for (int j = 0; j < len_k; j++) scores[j] /= total;
        float *oi = o + (i64)i * head_d;
        for (int d = 0; d < head_d; d++) {
            float r = 0.0f;
            for (int j = 0; j < len_k; j++) r += scores[j] * v[(i64)j * head_d + d];
            oi[d] = r;
        }
    }
}

/* final/attention.cu:228-283 */
void oracle_attention_f32(const float *Q, const float *K, const float *V, float *out,
                          int B, int H, int Lq, int Lk, int D) {
    float *scores = (float *)malloc(sizeof(float) * (size_t)(Lk > 0 ? Lk : 1));
    for (i64 bh = 0; bh < (i64)B * H; bh++)
        attention_slice(Q + bh * Lq * D, K + bh * Lk * D, V + bh * Lk * D, out + bh * Lq * D,
                        Lq, Lk, D, scores);
    free(scores);
}

/* final/rope.cu:20-40: cache[pos*rd + 2i] = cache[pos*rd + 2i+1] = cos/sin(pos * base^(-2i/rd)) */
void oracle_rope_cache(float *cos_cache, float *sin_cache, int max_len, int rotary_dim, float base) {
    for (int pos = 0; pos < max_len; pos++)
        for (int i = 0; i < rotary_dim / 2; i++) {
            float freq = 1.0f / powf(base, (2.0f * i) / rotary_dim);
            float theta = pos * freq;
            float c = cosf(theta), s = sinf(theta);
            cos_cache[(i64)pos * rotary_dim + 2 * i] = c;
            cos_cache[(i64)pos * rotary_dim + 2 * i + 1] = c;
            sin_cache[(i64)pos * rotary_dim + 2 * i] = s;
            sin_cache[(i64)pos * rotary_dim + 2 * i + 1] = s;
        }
}

/* final/rope.cu:1418-1437, generalised to rotary_dim <= head_d (the tail is copied, as the
 * reference GPU prologue does at final/rope.cu:152-154).  cache row stride = rotary_dim. */
void oracle_apply_rope_interleaved(const float *in, float *out, const float *cos_cache,
                                   const float *sin_cache, int len, int head_d, int rotary_dim) {
    for (int pos = 0; pos < len; pos++) {
        const float *x = in + (i64)pos * head_d;
        float *y = out + (i64)pos * head_d;
        for (int d = 0; d < rotary_dim; d += 2) {
            float xe = x[d], xo = x[d + 1];
            float c = cos_cache[(i64)pos * rotary_dim + d];
            float s = sin_cache[(i64)pos * rotary_dim + d];
            y[d] = xe * c - xo * s;
            y[d + 1] = xe * s + xo * c;
        }
        for (int d = rotary_dim; d < head_d; d++) y[d] = x[d];
    }
}

/* Rotate-half pairing: pair i couples columns (i, i+rd/2) with the angle of pair i.  Equal to the
 * interleaved rotation under the column permutation X'[2i]=X[i], X'[2i+1]=X[i+rd/2]. */
void oracle_apply_rope_half(const float *in, float *out, const float *cos_cache,
                            const float *sin_cache, int len, int head_d, int rotary_dim) {
    const int half = rotary_dim / 2;
    for (int pos = 0; pos < len; pos++) {
        const float *x = in + (i64)pos * head_d;
        float *y = out + (i64)pos * head_d;
        for (int i = 0; i < half; i++) {
            float xe = x[i], xo = x[i + half];
            float c = cos_cache[(i64)pos * rotary_dim + 2 * i];
            float s = sin_cache[(i64)pos * rotary_dim + 2 * i];
            y[i] = xe * c - xo * s;
            y[i + half] = xe * s + xo * c;
        }
        for (int d = rotary_dim; d < head_d; d++) y[d] = x[d];
    }
}

/* final/sinusoidal.cu:838-855 */
void oracle_sinusoidal_tables(float *sin_table, float *cos_table, int max_len, int head_d) {
    const float base = 10000.0f;
    for (int pos = 0; pos < max_len; pos++)
        for (int i = 0; i < head_d; i++) {
            float freq = 1.0f / powf(base, (2.0f * (i / 2)) / (float)head_d);
            float angle = pos * freq;
            sin_table[(i64)pos * head_d + i] = sinf(angle);
            cos_table[(i64)pos * head_d + i] = cosf(angle);
        }
}

/* Adds PE[p,2i]=sin, PE[p,2i+1]=cos in fp32: final/sinusoidal.cu:885-897 */
static void add_sinusoidal(const float *in, float *out, const float *sin_table,
                           const float *cos_table, int len, int head_d) {
    for (int pos = 0; pos < len; pos++)
        for (int d = 0; d < head_d; d++) {
            float pe = (d % 2 == 0) ? sin_table[(i64)pos * head_d + d] : cos_table[(i64)pos * head_d + d];
            out[(i64)pos * head_d + d] = in[(i64)pos * head_d + d] + pe;
        }
}

/*
 * General entry: attention with a positional encoding applied to Q and K of every (b,h) slice,
 * positions 0..L-1 (final/rope.cu:129,307).  For ROPE kinds the cos/sin caches are built with
 * oracle_rope_cache(max(Lq,Lk), rotary_dim, base); for SINUSOIDAL with oracle_sinusoidal_tables.
 * pe = ROPE_INTERLEAVED with rotary_dim == D reproduces attention_rope_cpu (final/rope.cu:1439-1499),
 * pe = SINUSOIDAL reproduces attention_sinusoidal_cpu (final/sinusoidal.cu:858-928).
 * bh_begin/bh_end select a range of flat (b*H+h) slices (all of them: 0, B*H) so that callers can
 * fan slices out over host threads or evaluate a sample of a large problem.
 */
int oracle_attention_pe_f32(const float *Q, const float *K, const float *V, float *out,
                            int B, int H, int Lq, int Lk, int D,
                            int pe, int rotary_dim, float base, i64 bh_begin, i64 bh_end) {
    const int Lmax = Lq > Lk ? Lq : Lk;
    float *scores = (float *)malloc(sizeof(float) * (size_t)(Lk > 0 ? Lk : 1));
    float *qt = NULL, *kt = NULL, *ta = NULL, *tb = NULL;
    if (pe != ORACLE_PE_NONE) {
        qt = (float *)malloc(sizeof(float) * (size_t)Lq * D);
        kt = (float *)malloc(sizeof(float) * (size_t)Lk * D);
        if (pe == ORACLE_PE_SINUSOIDAL) {
            ta = (float *)malloc(sizeof(float) * (size_t)Lmax * D);
            tb = (float *)malloc(sizeof(float) * (size_t)Lmax * D);
            oracle_sinusoidal_tables(ta, tb, Lmax, D);
        } else {
            ta = (float *)malloc(sizeof(float) * (size_t)Lmax * rotary_dim);
            tb = (float *)malloc(sizeof(float) * (size_t)Lmax * rotary_dim);
            oracle_rope_cache(ta, tb, Lmax, rotary_dim, base);
        }
    }
    (void)B; (void)H;
    for (i64 bh = bh_begin; bh < bh_end; bh++) {
        const float *q = Q + bh * Lq * D, *k = K + bh * Lk * D, *v = V + bh * Lk * D;
        float *o = out + bh * Lq * D;
        switch (pe) {
        case ORACLE_PE_NONE:
            attention_slice(q, k, v, o, Lq, Lk, D, scores);
            continue;
        case ORACLE_PE_ROPE_INTERLEAVED:
            oracle_apply_rope_interleaved(q, qt, ta, tb, Lq, D, rotary_dim);
            oracle_apply_rope_interleaved(k, kt, ta, tb, Lk, D, rotary_dim);
            break;
        case ORACLE_PE_ROPE_HALF:
            oracle_apply_rope_half(q, qt, ta, tb, Lq, D, rotary_dim);
            oracle_apply_rope_half(k, kt, ta, tb, Lk, D, rotary_dim);
            break;
        case ORACLE_PE_ROPE_Q_ONLY:
            oracle_apply_rope_interleaved(q, qt, ta, tb, Lq, D, rotary_dim);
            memcpy(kt, k, sizeof(float) * (size_t)Lk * D);
            break;
        case ORACLE_PE_SINUSOIDAL:
            add_sinusoidal(q, qt, ta, tb, Lq, D);
            add_sinusoidal(k, kt, ta, tb, Lk, D);
            break;
        default:
            free(scores); free(qt); free(kt); free(ta); free(tb);
            return -1;
        }
        attention_slice(qt, kt, v, o, Lq, Lk, D, scores);
    }
    free(scores); free(qt); free(kt); free(ta); free(tb);
    return 0;
}

/* final/rope.cu:1439-1499 with caller-supplied caches of row stride D (full rotation). */
void oracle_attention_rope_f32(const float *Q, const float *K, const float *V, float *out,
                               const float *cos_cache, const float *sin_cache,
                               int B, int H, int Lq, int Lk, int D) {
    float *scores = (float *)malloc(sizeof(float) * (size_t)(Lk > 0 ? Lk : 1));
    float *qt = (float *)malloc(sizeof(float) * (size_t)Lq * D);
    float *kt = (float *)malloc(sizeof(float) * (size_t)Lk * D);
    for (i64 bh = 0; bh < (i64)B * H; bh++) {
        oracle_apply_rope_interleaved(Q + bh * Lq * D, qt, cos_cache, sin_cache, Lq, D, D);
        oracle_apply_rope_interleaved(K + bh * Lk * D, kt, cos_cache, sin_cache, Lk, D, D);
        attention_slice(qt, kt, V + bh * Lk * D, out + bh * Lq * D, Lq, Lk, D, scores);
    }
    free(scores); free(qt); free(kt);
}

/* final/sinusoidal.cu:858-928 with caller-supplied tables. */
void oracle_attention_sinusoidal_f32(const float *Q, const float *K, const float *V,
                                     const float *sin_table, const float *cos_table, float *out,
                                     int B, int H, int Lq, int Lk, int D) {
    float *scores = (float *)malloc(sizeof(float) * (size_t)(Lk > 0 ? Lk : 1));
    float *qt = (float *)malloc(sizeof(float) * (size_t)Lq * D);
    float *kt = (float *)malloc(sizeof(float) * (size_t)Lk * D);
    for (i64 bh = 0; bh < (i64)B * H; bh++) {
        add_sinusoidal(Q + bh * Lq * D, qt, sin_table, cos_table, Lq, D);
        add_sinusoidal(K + bh * Lk * D, kt, sin_table, cos_table, Lk, D);
        attention_slice(qt, kt, V + bh * Lk * D, out + bh * Lq * D, Lq, Lk, D, scores);
    }
    free(scores); free(qt); free(kt);
}

/*
 * Sampled evaluation for problems too large to run in full on a CPU: computes the output rows
 * (bh[r], row[r]) for r < n_rows into out_rows[r*D .. r*D+D).  The K slice of a (b,h) is
 * transformed once per distinct bh (rows must be grouped by bh).  Same arithmetic as
 * oracle_attention_pe_f32 for those rows.
 */
int oracle_attention_pe_rows_f32(const float *Q, const float *K, const float *V, float *out_rows,
                                 int Lq, int Lk, int D, int pe, int rotary_dim, float base,
                                 const i64 *bh, const int *row, int n_rows) {
    const int Lmax = Lq > Lk ? Lq : Lk;
    float *scores = (float *)malloc(sizeof(float) * (size_t)Lk);
    float *qt = (float *)malloc(sizeof(float) * (size_t)D);
    float *kt = NULL, *ta = NULL, *tb = NULL;
    int tstride = 0;
    if (pe != ORACLE_PE_NONE) {
        kt = (float *)malloc(sizeof(float) * (size_t)Lk * D);
        tstride = (pe == ORACLE_PE_SINUSOIDAL) ? D : rotary_dim;
        ta = (float *)malloc(sizeof(float) * (size_t)Lmax * tstride);
        tb = (float *)malloc(sizeof(float) * (size_t)Lmax * tstride);
        if (pe == ORACLE_PE_SINUSOIDAL) oracle_sinusoidal_tables(ta, tb, Lmax, D);
        else oracle_rope_cache(ta, tb, Lmax, rotary_dim, base);
    }
    i64 cur = -1;
    for (int r = 0; r < n_rows; r++) {
        const float *k = K + bh[r] * Lk * D, *v = V + bh[r] * Lk * D;
        const float *q = Q + (bh[r] * Lq + row[r]) * D;
        const float *kk = k, *qq = q;
        if (pe != ORACLE_PE_NONE) {
            if (cur != bh[r]) {
                cur = bh[r];
                if (pe == ORACLE_PE_ROPE_INTERLEAVED) oracle_apply_rope_interleaved(k, kt, ta, tb, Lk, D, rotary_dim);
                else if (pe == ORACLE_PE_ROPE_HALF) oracle_apply_rope_half(k, kt, ta, tb, Lk, D, rotary_dim);
                else if (pe == ORACLE_PE_SINUSOIDAL) add_sinusoidal(k, kt, ta, tb, Lk, D);
                else memcpy(kt, k, sizeof(float) * (size_t)Lk * D);
            }
            const float *ca = ta + (i64)row[r] * tstride, *cb = tb + (i64)row[r] * tstride;
            if (pe == ORACLE_PE_ROPE_HALF) oracle_apply_rope_half(q, qt, ca, cb, 1, D, rotary_dim);
            else if (pe == ORACLE_PE_SINUSOIDAL) add_sinusoidal(q, qt, ca, cb, 1, D);
            else oracle_apply_rope_interleaved(q, qt, ca, cb, 1, D, rotary_dim);
            kk = kt; qq = qt;
        }
        attention_slice(qq, kk, v, out_rows + (i64)r * D, 1, Lk, D, scores);
    }
    free(scores); free(qt); free(kt); free(ta); free(tb);
    return 0;
}

/* ---- bf16 helpers: round-to-nearest-even fp32 -> bf16 bits and back (NaN kept quiet) ---- */
uint16_t oracle_f32_to_bf16(float f) {
    uint32_t u; memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
float oracle_bf16_to_f32(uint16_t h) {
    uint32_t u = (uint32_t)h << 16; float f; memcpy(&f, &u, 4); return f;
}
void oracle_round_to_bf16(const float *in, uint16_t *out, i64 n) {
    for (i64 i = 0; i < n; i++) out[i] = oracle_f32_to_bf16(in[i]);
}
void oracle_bf16_upcast(const uint16_t *in, float *out, i64 n) {
    for (i64 i = 0; i < n; i++) out[i] = oracle_bf16_to_f32(in[i]);
}

/*
 * Synthetic inputs: counter-based generator, identical in C, numpy and the library's device fill.
 *   u64 = splitmix64(seed*2^40 + tensor_id*2^36 + linear_index)
 *   uniform[-1,1):  -1 + 2 * (u64 >> 40) / 2^24
 *   normal(0,1):    Box-Muller on u1 = ((u64 >> 40) + 1) / 2^24, u2 = ((u64 >> 16) & 0xffffff) / 2^24
 */
static inline uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}
void oracle_fill_uniform(float *out, i64 n, uint64_t seed, uint64_t tensor_id, i64 index0) {
    for (i64 i = 0; i < n; i++) {
        uint64_t u = splitmix64((seed << 40) + (tensor_id << 36) + (uint64_t)(index0 + i));
        out[i] = -1.0f + 2.0f * ((float)(u >> 40) * (1.0f / 16777216.0f));
    }
}
void oracle_fill_normal(float *out, i64 n, uint64_t seed, uint64_t tensor_id, i64 index0) {
    for (i64 i = 0; i < n; i++) {
        uint64_t u = splitmix64((seed << 40) + (tensor_id << 36) + (uint64_t)(index0 + i));
        float u1 = ((float)(u >> 40) + 1.0f) * (1.0f / 16777216.0f);
        float u2 = (float)((u >> 16) & 0xffffffu) * (1.0f / 16777216.0f);
        out[i] = sqrtf(-2.0f * logf(u1)) * cosf(6.28318530717958647692f * u2);
    }
}
