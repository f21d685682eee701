// C-callable doors into the REFERENCE's own CUDA kernels -- TEST INFRASTRUCTURE, not product.
//
// This file holds no algorithm.  oracle/Makefile compiles it together with the reference's
// kernels/gemv.cu, kernels/moe.cu and kernels/dprof.cu (read in place from the reference
// checkout, never copied) into oracle/_ref/libref_kernels.so, so that GPU tests can compare
// this library's results with the reference kernels on identical device buffers, and the
// benchmark can time "the kernel to beat" on the same GPU.  Entry points mirror
// reference include/gemv.h:29,56,75 and include/moe.h:28-45.
#include <cuda_runtime.h>
#include <cstdint>
#include "gemv.h"
#include "moe.h"
#include "glm5_config.h"

extern "C" {

void ref_gemm_nvfp4(float* y, const uint8_t* packed, const uint8_t* scale, const float* gs,
                    const float* x, int M, int N, int K, cudaStream_t s) {
    glm5::gemm(y, glm5::WRef(packed, scale, gs), x, M, N, K, glm5::GEMV_BF16, s);
}

void ref_gemm_bf16(float* y, const void* w, const float* x, int M, int N, int K, cudaStream_t s) {
    glm5::gemm(y, glm5::WRef(w), x, M, N, K, glm5::GEMV_BF16, s);
}

// jobs: n entries of {y, packed, scale, gs, x} pointers and N, all sharing K (n <= 4).
void ref_gemv_multi(float* const* y, const uint8_t* const* packed, const uint8_t* const* scale,
                    const float* const* gs, const float* const* x, const int* N, int n, int K,
                    cudaStream_t s) {
    glm5::GemvJob jobs[glm5::GEMV_MULTI_MAX];
    for (int i = 0; i < n && i < glm5::GEMV_MULTI_MAX; ++i)
        jobs[i] = glm5::GemvJob{y[i], glm5::WRef(packed[i], scale[i], gs[i]), x[i], N[i]};
    glm5::gemv_multi(jobs, n, K, glm5::GEMV_BF16, s);
}

int ref_moe_hidden() { return glm5::HIDDEN; }
int ref_moe_inter() { return glm5::MOE_INTER; }
int ref_moe_experts() { return glm5::N_ROUTED_EXPERT; }
int ref_moe_topk() { return glm5::N_EXPERT_PER_TOK; }
size_t ref_moe_workspace_floats(int M) { return glm5::moe_batch_workspace_floats(M); }

// experts / shared: DEVICE arrays of {packed, scale, gscale} pointer triples (3*E and 3 entries).
void ref_moe_forward(const float* x, const void* router_bf16, const float* bias,
                     const void* experts, const void* shared, int n_expert, int topk,
                     float* y, int32_t* sel, float* wts, float* ws, int M, cudaStream_t s) {
    glm5::MoeLayer L;
    L.router_w = glm5::WRef(router_bf16);
    L.router_bias = bias;
    L.experts = static_cast<const glm5::Nvfp4Mat*>(experts);
    L.shared = static_cast<const glm5::Nvfp4Mat*>(shared);
    L.n_expert = n_expert;
    L.topk = topk;
    glm5::moe_forward_batch(x, L, y, sel, wts, ws, M, s);
}

}  // extern "C"
