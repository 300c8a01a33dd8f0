// C++ parity driver in the shape of the reference's own test programs (final/attention.cu:333-529,
// final/rope.cu:1544, final/sinusoidal.cu:981): host buffers filled from srand(42)/rand() in the
// reference's order, device buffers from cudaMalloc, the drop-in launchers called exactly as the
// reference's main() calls its own, results compared with the CPU oracle.  Links the library through
// include/b200attn.h only; the oracle (oracle/attn_oracle.c) is the checker.  Exit code 0 = all passed.
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "b200attn.h"

extern "C" {
void oracle_attention_f32(const float *, const float *, const float *, float *, int, int, int, int, int);
int oracle_attention_pe_f32(const float *, const float *, const float *, float *, int, int, int, int, int, int, int, float,
                            long long, long long);
}

static void init_random(std::vector<float> &v) {   // final/attention.cu:290-294
    for (auto &x : v) x = -1.0f + 2.0f * (rand() / (float)RAND_MAX);
}

// the reference's AND-of-failures rule (final/attention.cu:296-331) with this library's fp32 tolerance
static bool check(const std::vector<float> &got, const std::vector<float> &want, const char *what) {
    float max_abs = 0.0f;
    long bad = 0;
    for (size_t i = 0; i < got.size(); ++i) {
        const float ad = fabsf(got[i] - want[i]), rd = ad / (fabsf(want[i]) + 1e-8f);
        if (!(ad <= max_abs)) max_abs = ad;
        if (ad > 1e-4f && rd > 1e-3f) ++bad;
    }
    const bool ok = bad == 0 && max_abs <= 1e-4f;
    printf("  %-58s max abs diff %.3g  %s\n", what, max_abs, ok ? "PASSED" : "FAILED");
    return ok;
}

typedef void (*launcher_t)(const float *, const float *, const float *, float *, int, int, int, int, int);

static bool run(const char *name, launcher_t fn, int pe, int B, int H, int Lq, int Lk, int D) {
    const size_t nq = (size_t)B * H * Lq * D, nk = (size_t)B * H * Lk * D;
    std::vector<float> Q(nq), K(nk), V(nk), out(nq), want(nq);
    init_random(Q); init_random(K); init_random(V);
    float *dQ, *dK, *dV, *dO;
    if (cudaMalloc(&dQ, nq * 4) || cudaMalloc(&dK, nk * 4) || cudaMalloc(&dV, nk * 4) || cudaMalloc(&dO, nq * 4)) return false;
    cudaMemcpy(dQ, Q.data(), nq * 4, cudaMemcpyHostToDevice);
    cudaMemcpy(dK, K.data(), nk * 4, cudaMemcpyHostToDevice);
    cudaMemcpy(dV, V.data(), nk * 4, cudaMemcpyHostToDevice);
    fn(dQ, dK, dV, dO, B, H, Lq, Lk, D);   // blocking, like the reference launcher
    cudaMemcpy(out.data(), dO, nq * 4, cudaMemcpyDeviceToHost);
    if (pe == 0) oracle_attention_f32(Q.data(), K.data(), V.data(), want.data(), B, H, Lq, Lk, D);
    else oracle_attention_pe_f32(Q.data(), K.data(), V.data(), want.data(), B, H, Lq, Lk, D, pe, D, 10000.0f, 0, (long long)B * H);
    cudaFree(dQ); cudaFree(dK); cudaFree(dV); cudaFree(dO);
    char what[160];
    snprintf(what, sizeof what, "%s bs=%d nh=%d lq=%d lk=%d hdim=%d", name, B, H, Lq, Lk, D);
    return check(out, want, what);
}

int main() {
    srand(42);
    bool ok = true;
    // final/attention.cu:488-522
    const int plain[][4] = {{1, 1, 4, 8}, {1, 2, 8, 16}, {2, 4, 32, 32}, {2, 8, 64, 64}, {1, 4, 16, 64}, {2, 8, 64, 128},
                            {1, 4, 64, 512}, {1, 4, 64, 2048}, {1, 2, 32, 4096}, {1, 1, 16, 8192}};
    for (auto &s : plain) ok &= run("attention_forward_optimized", attention_forward_optimized, 0, s[0], s[1], s[2], s[2], s[3]);
    ok &= run("attention_forward_optimized (cross)", attention_forward_optimized, 0, 1, 2, 16, 32, 32);   // :496
    // final/rope.cu:1917-1928 (interleaved pairs, full rotation = pe kind 1)
    const int rope[][4] = {{1, 1, 4, 8}, {1, 2, 8, 16}, {2, 4, 32, 32}, {1, 4, 16, 64}, {1, 4, 64, 128}, {1, 4, 64, 512}, {1, 4, 64, 2048}};
    for (auto &s : rope) ok &= run("attention_forward_rope_fused_v2", attention_forward_rope_fused_v2, 1, s[0], s[1], s[2], s[2], s[3]);
    // final/sinusoidal.cu:1270-1276 (pe kind 3)
    const int sinus[][4] = {{1, 4, 64, 512}, {1, 4, 64, 2048}, {1, 2, 32, 4096}};
    for (auto &s : sinus) ok &= run("attention_forward_sinusoidal_fused", attention_forward_sinusoidal_fused, 3, s[0], s[1], s[2], s[2], s[3]);
    printf(ok ? "ALL TESTS PASSED\n" : "SOME TESTS FAILED\n");
    return ok ? 0 : 1;
}
