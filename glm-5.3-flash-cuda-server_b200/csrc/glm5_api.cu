// glm5_api.cu -- the reference's C++ entry points (namespace glm5, include/gemv.h and
// include/moe.h of this repository) as thin forwards to the C ABI, so that the reference's
// callers link against libb200nvfp4.so unchanged.  Error behaviour follows the reference:
// misuse prints a message and aborts (reference kernels/gemv.cu:373, src/engine.cu:32-33).
#include "gemv.h"
#include "moe.h"
#include "b200_nvfp4.h"
#include <cstdio>
#include <cstdlib>

namespace glm5 {

static_assert(sizeof(Nvfp4Mat) == sizeof(b200_nvfp4_mat), "expert tables are shared with the C ABI as they are");
static_assert((int)GEMV_MULTI_MAX == (int)B200_GEMV_MULTI_MAX, "job limit");

static void must(int rc, const char* what) {
    if (rc) { fprintf(stderr, "glm5::%s: %s\n", what, b200_nvfp4_strerror(rc)); abort(); }
}
static b200_wref cw(const WRef& w) { return b200_wref{w.p, w.packed, w.scale, w.gscale}; }

void gemv(float* y, const WRef& W, const float* x, int N, int K, int dtype, cudaStream_t s) {
    const b200_wref w = cw(W);
    must(b200_nvfp4_gemm(y, &w, x, 1, N, K, dtype, s), "gemv");
}
void gemm(float* y, const WRef& W, const float* x, int M, int N, int K, int dtype, cudaStream_t s) {
    const b200_wref w = cw(W);
    must(b200_nvfp4_gemm(y, &w, x, M, N, K, dtype, s), "gemm");
}
void gemm_multi(const GemvJob* jobs, int n, int M, int K, int dtype, cudaStream_t s) {
    if (n < 1) return;
    if (n > GEMV_MULTI_MAX || M > B200_GEMV_M_MAX) {           // correct, not fused
        for (int i = 0; i < n; ++i) gemm(jobs[i].y, jobs[i].W, jobs[i].x, M, jobs[i].N, K, dtype, s);
        return;
    }
    b200_gemv_job j[B200_GEMV_MULTI_MAX];
    for (int i = 0; i < n; ++i) j[i] = b200_gemv_job{jobs[i].y, cw(jobs[i].W), jobs[i].x, jobs[i].N};
    must(b200_nvfp4_gemv_multi(j, n, M, K, dtype, s), "gemv_multi");
}
void gemv_multi(const GemvJob* jobs, int n, int K, int dtype, cudaStream_t s) { gemm_multi(jobs, n, 1, K, dtype, s); }
size_t split_workspace_bytes(int M, int K) { return b200_nvfp4_split_workspace_bytes(M, K); }
void gemm_ws(float* y, const WRef& W, const float* x, int M, int N, int K, int dtype, void* ws, cudaStream_t s) {
    const b200_wref w = cw(W);
    must(b200_nvfp4_gemm_ws(y, &w, x, M, N, K, dtype, ws, s), "gemm_ws");
}
void gemm_multi_ws(const GemvJob* jobs, int n, int M, int K, int dtype, void* ws, cudaStream_t s) {
    if (n < 1) return;
    if (n > GEMV_MULTI_MAX || M > B200_GEMV_M_MAX) { gemm_multi(jobs, n, M, K, dtype, s); return; }
    b200_gemv_job j[B200_GEMV_MULTI_MAX];
    for (int i = 0; i < n; ++i) j[i] = b200_gemv_job{jobs[i].y, cw(jobs[i].W), jobs[i].x, jobs[i].N};
    must(b200_nvfp4_gemv_multi_ws(j, n, M, K, dtype, ws, s), "gemm_multi_ws");
}
void exact_prefill(bool on) { must(b200_nvfp4_set_option(B200_OPT_PREFILL_FP4, on ? 0 : 1), "exact_prefill"); }
size_t gemm_bf16_workspace_bytes(int M, int K) { return b200_nvfp4_gemm_bf16_workspace_bytes(M, K); }
void gemm_bf16(float* y, const WRef& W, const void* x_bf16, int M, int N, int K, void* ws, cudaStream_t s) {
    const b200_wref w = cw(W);
    must(b200_nvfp4_gemm_bf16(y, &w, x_bf16, M, N, K, ws, s), "gemm_bf16");
}
size_t dense_mlp_workspace_bytes(int M, int hidden, int inter) { return b200_dense_mlp_workspace_bytes(M, hidden, inter); }
void dense_mlp_nvfp4(const float* x, const WRef& gate, const WRef& up, const WRef& down, int hidden, int inter,
                     float limit, float* y, void* ws, int M, cudaStream_t s) {
    const b200_wref g = cw(gate), u = cw(up), d = cw(down);
    must(b200_dense_mlp(x, &g, &u, &d, hidden, inter, limit, y, ws, M, s), "dense_mlp_nvfp4");
}
void f32_to_bf16(void* dst, const float* src, size_t n, cudaStream_t s) { must(b200_f32_to_bf16(dst, src, n, s), "f32_to_bf16"); }
void f32_from_bf16_dev(float* dst, const void* src, size_t n, cudaStream_t s) { must(b200_bf16_to_f32(dst, src, n, s), "f32_from_bf16_dev"); }

// reference include/glm5_config.h:20, 84-91
static struct { int hidden = 4096, inter = 2048; float scale = 2.5f, limit = 10.f; int norm = 1; } g_geo;

void moe_set_geometry(int hidden, int inter, float routed_scale, float swiglu_limit, bool norm_topk) {
    g_geo.hidden = hidden; g_geo.inter = inter; g_geo.scale = routed_scale; g_geo.limit = swiglu_limit; g_geo.norm = norm_topk ? 1 : 0;
}
static b200_moe_layer cl(const MoeLayer& L) {
    return b200_moe_layer{cw(L.router_w), L.router_bias, reinterpret_cast<const b200_nvfp4_mat*>(L.experts),
                          reinterpret_cast<const b200_nvfp4_mat*>(L.shared), L.n_expert, L.topk,
                          g_geo.hidden, g_geo.inter, g_geo.scale, g_geo.limit, g_geo.norm};
}
size_t moe_batch_workspace_floats(int M) {
    MoeLayer d{}; d.n_expert = 144; d.topk = 8;                // the reference's N_ROUTED_EXPERT / N_EXPERT_PER_TOK
    const b200_moe_layer l = cl(d);
    return (b200_moe_workspace_bytes(&l, M) + 3) / 4;
}
size_t moe_workspace_floats() { return moe_batch_workspace_floats(1); }
bool nvfp4_check_align(const Nvfp4Mat& m, const char* what) {
    // the reference's floor (kernels/moe.cu:628-636): 4-byte aligned packed bytes and global scale; every kernel
    // of this library runs from there (the 16-byte fast paths are chosen per tensor, on the device where needed)
    if (((uintptr_t)m.packed & 3) || ((uintptr_t)m.gscale & 3)) {
        fprintf(stderr, "nvfp4: %s needs 4-byte aligned packed bytes and global scale (packed=%p scale=%p gscale=%p)\n",
                what, (const void*)m.packed, (const void*)m.scale, (const void*)m.gscale);
        return false;
    }
    return true;
}
void moe_route_batch(const float* x, const MoeLayer& L, int32_t* sel, float* wts, float* logits, int M, cudaStream_t s) {
    const b200_moe_layer l = cl(L);
    must(b200_moe_route(x, &l, sel, wts, logits, M, s), "moe_route");
}
void moe_route(const float* x, const MoeLayer& L, int32_t* sel, float* wts, float* logits, cudaStream_t s) {
    moe_route_batch(x, L, sel, wts, logits, 1, s);
}
bool moe_prepare(const MoeLayer& L) {
    b200_moe_layer l = cl(L);
    const int rc = b200_moe_prepare(&l);
    if (rc == B200_ENOTIMPL) return false;
    must(rc, "moe_prepare");
    return true;
}
void moe_release(const MoeLayer& L) { b200_moe_layer l = cl(L); (void)b200_moe_release(&l); }

void moe_forward_batch(const float* x, const MoeLayer& L, float* y, int32_t* sel, float* wts, float* ws, int M, cudaStream_t s) {
    const b200_moe_layer l = cl(L);
    must(b200_moe_forward(x, &l, y, sel, wts, ws, M, s), "moe_forward");
}
void moe_forward(const float* x, const MoeLayer& L, float* y, int32_t* sel, float* wts, float* ws, cudaStream_t s) {
    moe_forward_batch(x, L, y, sel, wts, ws, 1, s);
}

}  // namespace glm5
