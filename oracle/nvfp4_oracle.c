/* CPU oracle for the NVFP4 weight path in plain C -- TEST INFRASTRUCTURE, not product code.
 *
 * Only tests, the smoke check and the benchmark's CPU-baseline leg load this library; the CUDA
 * library never links or calls it.  Parity status: PINNED -- tests/test_oracle_c.py checks
 * every function here against the vectors the reference's own Python code produced
 * (tests/golden/), bit for bit for codes/scales/global scale.
 *
 * Restates:
 *   quantiser   reference tools/requant_dense_nvfp4.py:28-68 (tables, quant_block), :209-215 (gs)
 *   dequantiser reference ref/gen_moe.py:20-30, include/nvfp4.cuh:3-7, 30-35
 *   gemv/gemm   reference kernels/gemv.cu:246-322 (what is computed; sums are fp64 here)
 *   MoE block   reference kernels/moe.cu:126-156 (route), :253-258 (SwiGLU clamps), :584-597
 *               (fixed-order combine); ref/gen_moe.py:62-96
 *
 * Build: make -C oracle   (gcc -O2 -fopenmp -shared; no fast-math: fp32 steps must stay IEEE)
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static const float kE2M1[8] = {0.f, .5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
static const float kE2M1Mid[7] = {.25f, .75f, 1.25f, 1.75f, 2.5f, 3.5f, 5.f};
static float g_e4m3[256];
static float g_e4m3_mid[126];
static int g_init = 0;

/* fp8-e4m3 code -> fp32, built from the fields so that it is exact (nvfp4.cuh:30-35). */
static float e4m3_decode(int v) {
    const int s = v >> 7, e = (v >> 3) & 0xF, m = v & 7;
    float r = e == 0 ? (float)m * (1.f / 8.f) * (1.f / 64.f)
                     : (1.f + (float)m * (1.f / 8.f)) * ldexpf(1.f, e - 7);
    return s ? -r : r;
}

static void init_tables(void) {
    if (g_init) return;
    for (int i = 0; i < 256; ++i) g_e4m3[i] = e4m3_decode(i);
    for (int i = 0; i < 126; ++i) g_e4m3_mid[i] = (g_e4m3[i + 1] + g_e4m3[i]) / 2.f;
    g_init = 1;
}

int oracle_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

static inline float bf16_to_f32(uint16_t b) {
    uint32_t u = (uint32_t)b << 16; float f; memcpy(&f, &u, 4); return f;
}

/* fp32(2688 / max(amax, 1e-12)), quotient in double (requant_dense_nvfp4.py:209-215). */
float oracle_global_scale(const uint16_t* w_bf16, size_t n) {
    float amax = 0.f;
    for (size_t i = 0; i < n; ++i) { const float a = fabsf(bf16_to_f32(w_bf16[i])); if (a > amax) amax = a; }
    double d = (double)amax; if (d < 1e-12) d = 1e-12;
    return (float)((448.0 * 6.0) / d);
}

/* number of table mid-points strictly below s == numpy searchsorted(side='left'):
 * a value that sits exactly on a mid-point takes the LOWER code. */
static inline int count_below(const float* mid, int n, float s) {
    int lo = 0, hi = n;                       /* first index with mid[i] >= s */
    while (lo < hi) { const int m = (lo + hi) >> 1; if (mid[m] < s) lo = m + 1; else hi = m; }
    return lo;
}

/* quant_block (requant_dense_nvfp4.py:53-68): every step in fp32, IEEE division. */
void oracle_quantize(const uint16_t* w_bf16, int rows, int K, float gs, uint8_t* packed, uint8_t* scale) {
    init_tables();
    const int G = K / 16;
    #pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; ++r) {
        for (int g = 0; g < G; ++g) {
            float v[16], amax = 0.f;
            for (int j = 0; j < 16; ++j) {
                v[j] = bf16_to_f32(w_bf16[(size_t)r * K + g * 16 + j]);
                const float a = fabsf(v[j]); if (a > amax) amax = a;
            }
            const float t = amax / 6.0f;
            float s = t * gs;
            if (s < 0.f) s = 0.f; if (s > 448.f) s = 448.f;
            const int code = count_below(g_e4m3_mid, 126, s);
            float eff = g_e4m3[code] / gs;
            if (!(eff > 1e-30f)) eff = 1e-30f;
            uint8_t idx[16];
            for (int j = 0; j < 16; ++j) {
                const float q = v[j] / eff;
                int c = count_below(kE2M1Mid, 7, fabsf(q));
                if (signbit(q) && c != 0) c |= 8;
                idx[j] = (uint8_t)c;
            }
            scale[(size_t)r * G + g] = (uint8_t)code;
            for (int j = 0; j < 8; ++j)
                packed[(size_t)r * (K / 2) + g * 8 + j] = (uint8_t)(idx[2 * j] | (idx[2 * j + 1] << 4));
        }
    }
}

/* w = e2m1(nib) * (e4m3(scale) / gs), the product order of ref/gen_moe.py:29. */
void oracle_dequant(const uint8_t* packed, const uint8_t* scale, float gs, int N, int K, float* out) {
    init_tables();
    #pragma omp parallel for schedule(static)
    for (int n = 0; n < N; ++n)
        for (int k = 0; k < K; ++k) {
            const uint8_t b = packed[(size_t)n * (K / 2) + (k >> 1)];
            const int nib = (k & 1) ? (b >> 4) : (b & 15);
            const float v = (nib & 8) ? -kE2M1[nib & 7] : kE2M1[nib & 7];
            out[(size_t)n * K + k] = v * (g_e4m3[scale[(size_t)n * (K / 16) + (k >> 4)]] / gs);
        }
}

/* y[M,N] (double) = x[M,K] . dequant(W)^T with fp64 accumulation. */
void oracle_gemm(const float* x, const uint8_t* packed, const uint8_t* scale, float gs,
                 int M, int N, int K, double* y) {
    init_tables();
    #pragma omp parallel for schedule(static)
    for (int n = 0; n < N; ++n) {
        for (int m = 0; m < M; ++m) {
            double acc = 0.0;
            for (int g = 0; g < K / 16; ++g) {
                const float sc = g_e4m3[scale[(size_t)n * (K / 16) + g]] / gs;
                for (int j = 0; j < 16; ++j) {
                    const int k = g * 16 + j;
                    const uint8_t b = packed[(size_t)n * (K / 2) + (k >> 1)];
                    const int nib = (k & 1) ? (b >> 4) : (b & 15);
                    const float v = (nib & 8) ? -kE2M1[nib & 7] : kE2M1[nib & 7];
                    acc += (double)(v * sc) * (double)x[(size_t)m * K + k];
                }
            }
            y[(size_t)m * N + n] = acc;
        }
    }
}

/* Router for one token: sigmoid, rank by score+bias with strict '>' (lowest index wins a tie),
 * weights = unbiased scores / (1e-20 + sum) * scaling  (kernels/moe.cu:126-156). */
void oracle_route(const double* logits, const float* bias, int E, int topk, float scaling,
                  int norm_prob, int32_t* sel, float* wts) {
    float* score = (float*)malloc(sizeof(float) * E);
    float* choice = (float*)malloc(sizeof(float) * E);
    for (int i = 0; i < E; ++i) { score[i] = (float)(1.0 / (1.0 + exp(-logits[i]))); choice[i] = score[i] + bias[i]; }
    for (int k = 0; k < topk; ++k) {
        int bi = -1; float bv = -1e30f;
        for (int i = 0; i < E; ++i) if (choice[i] > bv) { bv = choice[i]; bi = i; }
        sel[k] = bi; wts[k] = score[bi]; choice[bi] = -1e30f;
    }
    float d = 1.f;
    if (norm_prob) { d = 1e-20f; for (int k = 0; k < topk; ++k) d += wts[k]; }
    for (int k = 0; k < topk; ++k) wts[k] = wts[k] / d * scaling;
    free(score); free(choice);
}

/* One SwiGLU expert for one token: y[H] (double) += w * down(silu(min(g,L)) * clamp(u,+-L)). */
void oracle_expert(const float* x, int H, int I,
                   const uint8_t* gp, const uint8_t* gsc, float ggs,
                   const uint8_t* up, const uint8_t* usc, float ugs,
                   const uint8_t* dp, const uint8_t* dsc, float dgs,
                   float limit, double weight, double* y) {
    double* g = (double*)malloc(sizeof(double) * I);
    double* u = (double*)malloc(sizeof(double) * I);
    float* act = (float*)malloc(sizeof(float) * I);
    double* o = (double*)malloc(sizeof(double) * H);
    oracle_gemm(x, gp, gsc, ggs, 1, I, H, g);
    oracle_gemm(x, up, usc, ugs, 1, I, H, u);
    for (int i = 0; i < I; ++i) {
        double a = g[i] < limit ? g[i] : limit;
        double b = u[i] < -limit ? -limit : (u[i] > limit ? limit : u[i]);
        act[i] = (float)(a / (1.0 + exp(-a)) * b);
    }
    oracle_gemm(act, dp, dsc, dgs, 1, H, I, o);
    for (int h = 0; h < H; ++h) y[h] += weight * o[h];
    free(g); free(u); free(act); free(o);
}
