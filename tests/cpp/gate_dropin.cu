// gate_dropin.cu -- a gate in the style of the reference's tests/gate_nvfp4.cu and
// tests/gate_gemv_multi.cu, written against THIS repository's include/gemv.h and include/moe.h
// and linked with libb200nvfp4.so: what a reference caller would see after the swap.
//   1. quantise seeded bf16 weights on the GPU (C ABI), dequantise on the host (format definition)
//   2. gemv vs host dequant-then-matvec (rel-L2 <= 1e-3), gemv == gemm(M=1) and gemm rows == gemv
//      (memcmp), fused group == separate gemvs (memcmp) with poison-filled outputs
//   3. a small MoE layer through glm5::moe_forward_batch vs glm5::moe_forward per token (memcmp)
// Exit code 0 only if everything passes.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include "gemv.h"
#include "moe.h"
#include "b200_nvfp4.h"

using namespace glm5;
#define CU(x) do { cudaError_t e_ = (x); if (e_) { fprintf(stderr, "cuda %s:%d %s\n", __FILE__, __LINE__, cudaGetErrorString(e_)); exit(2); } } while (0)

static unsigned lcg = 12345u;
static float urand() { lcg = lcg * 1664525u + 1013904223u; return (float)((int)(lcg >> 8) % 2001 - 1000) / 1000.f; }

struct DevW { uint8_t* p; uint8_t* s; float* g; int N, K; std::vector<float> deq; };

static float e4m3(uint8_t v) { int e = (v >> 3) & 15, m = v & 7; float r = e ? (1.f + m / 8.f) * std::ldexp(1.f, e - 7) : m / 512.f; return (v & 0x80) ? -r : r; }

static DevW make_weight(int N, int K) {
    std::vector<__nv_bfloat16> h((size_t)N * K);
    for (auto& v : h) v = __float2bfloat16(urand() * 0.05f);
    __nv_bfloat16* d; CU(cudaMalloc(&d, h.size() * 2)); CU(cudaMemcpy(d, h.data(), h.size() * 2, cudaMemcpyHostToDevice));
    DevW W{}; W.N = N; W.K = K;
    CU(cudaMalloc(&W.p, (size_t)N * K / 2)); CU(cudaMalloc(&W.s, (size_t)N * K / 16)); CU(cudaMalloc(&W.g, 4));
    if (b200_nvfp4_quantize(d, N, K, W.p, W.s, W.g, nullptr, 0)) exit(3);
    CU(cudaDeviceSynchronize()); CU(cudaFree(d));
    std::vector<uint8_t> p((size_t)N * K / 2), s((size_t)N * K / 16); float g;
    CU(cudaMemcpy(p.data(), W.p, p.size(), cudaMemcpyDeviceToHost)); CU(cudaMemcpy(s.data(), W.s, s.size(), cudaMemcpyDeviceToHost));
    CU(cudaMemcpy(&g, W.g, 4, cudaMemcpyDeviceToHost));
    static const float lut[8] = {0.f, .5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
    W.deq.resize((size_t)N * K);
    for (int n = 0; n < N; ++n) for (int k = 0; k < K; ++k) {
        const uint8_t b = p[(size_t)n * K / 2 + k / 2]; const int nib = (k & 1) ? b >> 4 : b & 15;
        W.deq[(size_t)n * K + k] = (nib & 8 ? -lut[nib & 7] : lut[nib & 7]) * (e4m3(s[(size_t)n * K / 16 + k / 16]) / g);
    }
    return W;
}

int main() {
    int fails = 0;
    const int shapes[][2] = {{1000, 4096}, {64, 1536}, {130, 128}, {33, 48}};
    for (auto& sh : shapes) {
        const int N = sh[0], K = sh[1], M = 4;
        DevW W = make_weight(N, K);
        std::vector<float> hx((size_t)M * K); for (auto& v : hx) v = urand();
        float *dx, *y1, *ym; CU(cudaMalloc(&dx, hx.size() * 4)); CU(cudaMalloc(&y1, N * 4)); CU(cudaMalloc(&ym, (size_t)M * N * 4));
        CU(cudaMemcpy(dx, hx.data(), hx.size() * 4, cudaMemcpyHostToDevice));
        CU(cudaMemset(y1, 0xA5, N * 4)); CU(cudaMemset(ym, 0x5A, (size_t)M * N * 4));
        const WRef Wq(W.p, W.s, W.g);
        gemv(y1, Wq, dx, N, K, GEMV_BF16, 0);
        gemm(ym, Wq, dx, M, N, K, GEMV_BF16, 0);
        CU(cudaDeviceSynchronize());
        std::vector<float> h1(N), hm((size_t)M * N);
        CU(cudaMemcpy(h1.data(), y1, N * 4, cudaMemcpyDeviceToHost)); CU(cudaMemcpy(hm.data(), ym, hm.size() * 4, cudaMemcpyDeviceToHost));
        double num = 0, den = 0;
        for (int n = 0; n < N; ++n) { double r = 0; for (int k = 0; k < K; ++k) r += (double)W.deq[(size_t)n * K + k] * hx[k]; num += (h1[n] - r) * (h1[n] - r); den += r * r; }
        const double rel = std::sqrt(num / (den + 1e-30));
        int bad = memcmp(h1.data(), hm.data(), N * 4) != 0;
        for (int m = 1; m < M; ++m) {
            gemv(y1, Wq, dx + (size_t)m * K, N, K, GEMV_BF16, 0); CU(cudaDeviceSynchronize());
            CU(cudaMemcpy(h1.data(), y1, N * 4, cudaMemcpyDeviceToHost));
            bad += memcmp(h1.data(), hm.data() + (size_t)m * N, N * 4) != 0;
        }
        const bool ok = rel <= 1e-3 && bad == 0 && den > 0;
        printf("gemv/gemm  N=%5d K=%5d  rel %.2e  rows-vs-gemv %s  %s\n", N, K, rel, bad ? "DIFFER" : "bit-identical", ok ? "PASS" : "FAIL");
        fails += !ok;
    }
    {   // fused group, shared x and per-job x
        const int K = 4096, Ns[3] = {512, 64, 32};
        DevW W[3]; for (int i = 0; i < 3; ++i) W[i] = make_weight(Ns[i], K);
        std::vector<float> hx((size_t)3 * K); for (auto& v : hx) v = urand();
        float* dx; CU(cudaMalloc(&dx, hx.size() * 4)); CU(cudaMemcpy(dx, hx.data(), hx.size() * 4, cudaMemcpyHostToDevice));
        for (int shared = 1; shared >= 0; --shared) {
            float *ya, *yb; CU(cudaMalloc(&ya, 608 * 4)); CU(cudaMalloc(&yb, 608 * 4));
            CU(cudaMemset(ya, 0xA5, 608 * 4)); CU(cudaMemset(yb, 0x5A, 608 * 4));
            GemvJob jobs[3]; int off = 0;
            for (int i = 0; i < 3; ++i) {
                const float* xi = dx + (size_t)(shared ? 0 : i) * K;
                gemv(ya + off, WRef(W[i].p, W[i].s, W[i].g), xi, Ns[i], K, GEMV_BF16, 0);
                jobs[i].y = yb + off; jobs[i].W = WRef(W[i].p, W[i].s, W[i].g); jobs[i].x = xi; jobs[i].N = Ns[i];
                off += Ns[i];
            }
            gemv_multi(jobs, 3, K, GEMV_BF16, 0);
            CU(cudaDeviceSynchronize());
            std::vector<float> a(608), b(608);
            CU(cudaMemcpy(a.data(), ya, 608 * 4, cudaMemcpyDeviceToHost)); CU(cudaMemcpy(b.data(), yb, 608 * 4, cudaMemcpyDeviceToHost));
            int nz = 0; for (float v : a) nz += v != 0.f;
            const bool ok = memcmp(a.data(), b.data(), 608 * 4) == 0 && nz > 304;
            printf("gemv_multi %s x  %s\n", shared ? "shared " : "per-job", ok ? "PASS bit-identical" : "FAIL");
            fails += !ok;
        }
    }
    {   // MoE: batch of 3 tokens == 3 single-token calls, bit for bit
        const int H = 512, I = 256, E = 8, TK = 2, M = 3;
        moe_set_geometry(H, I, 2.5f, 10.f, true);
        std::vector<Nvfp4Mat> tab((E + 1) * 3);
        for (int e = 0; e <= E; ++e) {
            DevW g = make_weight(I, H), u = make_weight(I, H), d = make_weight(H, I);
            tab[e * 3] = {g.p, g.s, g.g}; tab[e * 3 + 1] = {u.p, u.s, u.g}; tab[e * 3 + 2] = {d.p, d.s, d.g};
            if (!nvfp4_check_align(tab[e * 3], "expert")) fails++;
        }
        Nvfp4Mat* dtab; CU(cudaMalloc(&dtab, tab.size() * sizeof(Nvfp4Mat))); CU(cudaMemcpy(dtab, tab.data(), tab.size() * sizeof(Nvfp4Mat), cudaMemcpyHostToDevice));
        std::vector<__nv_bfloat16> hr((size_t)E * H); for (auto& v : hr) v = __float2bfloat16(urand() * 0.2f);
        std::vector<float> hb(E), hx((size_t)M * H); for (auto& v : hb) v = urand() * 0.1f; for (auto& v : hx) v = urand();
        __nv_bfloat16* dr; float *db, *dx, *y, *y1, *wts, *ws; int32_t* sel;
        CU(cudaMalloc(&dr, hr.size() * 2)); CU(cudaMemcpy(dr, hr.data(), hr.size() * 2, cudaMemcpyHostToDevice));
        CU(cudaMalloc(&db, E * 4)); CU(cudaMemcpy(db, hb.data(), E * 4, cudaMemcpyHostToDevice));
        CU(cudaMalloc(&dx, hx.size() * 4)); CU(cudaMemcpy(dx, hx.data(), hx.size() * 4, cudaMemcpyHostToDevice));
        CU(cudaMalloc(&y, (size_t)M * H * 4)); CU(cudaMalloc(&y1, (size_t)M * H * 4)); CU(cudaMalloc(&wts, M * TK * 4)); CU(cudaMalloc(&sel, M * TK * 4));
        MoeLayer L{}; L.router_w = WRef((const void*)dr); L.router_bias = db; L.experts = dtab; L.shared = dtab + E * 3; L.n_expert = E; L.topk = TK;
        b200_moe_layer bl{{dr, nullptr, nullptr, nullptr}, db, (const b200_nvfp4_mat*)dtab, (const b200_nvfp4_mat*)(dtab + E * 3), E, TK, H, I, 2.5f, 10.f, 1};
        CU(cudaMalloc(&ws, b200_moe_workspace_bytes(&bl, M)));
        moe_forward_batch(dx, L, y, sel, wts, ws, M, 0);
        for (int m = 0; m < M; ++m) moe_forward(dx + (size_t)m * H, L, y1 + (size_t)m * H, sel, wts, ws, 0);
        CU(cudaDeviceSynchronize());
        std::vector<float> a((size_t)M * H), b((size_t)M * H);
        CU(cudaMemcpy(a.data(), y, a.size() * 4, cudaMemcpyDeviceToHost)); CU(cudaMemcpy(b.data(), y1, b.size() * 4, cudaMemcpyDeviceToHost));
        int nz = 0; for (float v : a) nz += v != 0.f;
        const bool ok = memcmp(a.data(), b.data(), a.size() * 4) == 0 && nz > (int)a.size() / 2;
        printf("moe_forward_batch rows == moe_forward  %s\n", ok ? "PASS bit-identical" : "FAIL");
        fails += !ok;
        // the same after moe_prepare (tensor-core experts): still row == single call bit for bit, and
        // close to the CUDA-core result
        if (moe_prepare(L)) {
            moe_forward_batch(dx, L, y, sel, wts, ws, M, 0);
            for (int m = 0; m < M; ++m) moe_forward(dx + (size_t)m * H, L, y1 + (size_t)m * H, sel, wts, ws, 0);
            CU(cudaDeviceSynchronize());
            std::vector<float> c((size_t)M * H), d((size_t)M * H);
            CU(cudaMemcpy(c.data(), y, c.size() * 4, cudaMemcpyDeviceToHost)); CU(cudaMemcpy(d.data(), y1, d.size() * 4, cudaMemcpyDeviceToHost));
            double num = 0, den = 0;
            for (size_t i = 0; i < c.size(); ++i) { num += (double)(c[i] - a[i]) * (c[i] - a[i]); den += (double)a[i] * a[i]; }
            const bool ok2 = memcmp(c.data(), d.data(), c.size() * 4) == 0 && memcmp(c.data(), a.data(), c.size() * 4) != 0 && num <= 1e-6 * den;
            printf("prepared layer: rows == single calls, rel-L2 to CUDA-core %.2e  %s\n", sqrt(num / (den + 1e-30)), ok2 ? "PASS" : "FAIL");
            fails += !ok2;
            moe_release(L);
        } else { printf("moe_prepare refused the gate's geometry  FAIL\n"); fails++; }
    }
    unsigned st = 0; b200_nvfp4_device_status(&st, 0);
    if (st) { printf("device status %08x\n", st); fails++; }
    printf("gate_dropin: %s\n", fails ? "FAIL" : "PASS");
    return fails ? 1 : 0;
}
