// gemv.h -- source-compatible replacement for the reference's include/gemv.h (namespace glm5),
// implemented by libb200nvfp4.so.  Same types, same free functions, same argument meaning:
//   WRef (reference include/gemv.h:16-26), GemvJob (:50-55), gemv (:29), gemv_multi (:56),
//   f32_to_bf16 / f32_from_bf16_dev (:61-62), gemm (:75).
// Differences, all additive: GEMV_MULTI_MAX is 8 (was 4), and gemm_multi runs a fused group at
// M <= 8 rows.  Misuse aborts with a message, as the reference does (kernels/gemv.cu:373).
#pragma once
#include <cuda_runtime.h>
#include <cstddef>
#include <cstdint>

namespace glm5 {

enum { GEMV_F32 = 0, GEMV_BF16 = 1 };
enum { GEMV_MULTI_MAX = 8 };

// A weight matrix: a plain row-major [N, K] buffer of the call's dtype, or an NVFP4 triple.
// When `packed` is set the triple is used and dtype is ignored.  A bare pointer converts
// implicitly and means "plain buffer", so code that assigns pointers keeps compiling.
struct WRef {
    const void*    p      = nullptr;
    const uint8_t* packed = nullptr;   // [N, K/2], low nibble = even k
    const uint8_t* scale  = nullptr;   // [N, K/16], fp8-e4m3
    const float*   gscale = nullptr;   // [1]
    WRef() = default;
    WRef(const void* q) : p(q) {}                                   // NOLINT(google-explicit-constructor)
    WRef(std::nullptr_t) {}
    WRef(const uint8_t* pk, const uint8_t* sc, const float* gs) : packed(pk), scale(sc), gscale(gs) {}
    bool nvfp4() const { return packed != nullptr; }
};

struct GemvJob {
    float*       y = nullptr;
    WRef         W;
    const float* x = nullptr;
    int          N = 0;
};

// y[N] = W[N,K] . x[K]; x, y fp32.
void gemv(float* y, const WRef& W, const float* x, int N, int K, int dtype, cudaStream_t s);
// y[M,N] = x[M,K] . W^T; row m of the result is bit-identical to gemv of row m.
void gemm(float* y, const WRef& W, const float* x, int M, int N, int K, int dtype, cudaStream_t s);
// n independent gemvs sharing K and dtype in one launch; bit-identical to n gemv calls.
void gemv_multi(const GemvJob* jobs, int n, int K, int dtype, cudaStream_t s);
// The same with M <= 8 rows per job (x is [M,K], y is [M,N]).  Not in the reference.
void gemm_multi(const GemvJob* jobs, int n, int M, int K, int dtype, cudaStream_t s);
// Not in the reference: gemm / gemm_multi with `ws` = split_workspace_bytes(M, K) bytes of device
// scratch (256-byte aligned, not shared with a call that may overlap this one).  The M activation
// rows are then prepared for the tensor cores once per call instead of once per thread block:
// from 3 rows on this is faster (8 rows: 18 us instead of 26 us for the six sibling products; a
// 128-row prefill chunk: 2.2x), and the results are the same bits.
// From 16 rows on gemm_ws runs the wide tensor-core GEMM (weights read once per 256 rows, activations
// quantised to NVFP4 per token: a few per cent from the exact product) unless exact_prefill(true) was called.
size_t split_workspace_bytes(int M, int K);
void gemm_ws(float* y, const WRef& W, const float* x, int M, int N, int K, int dtype, void* ws, cudaStream_t s);
void gemm_multi_ws(const GemvJob* jobs, int n, int M, int K, int dtype, void* ws, cudaStream_t s);
void exact_prefill(bool on);
// Not in the reference: the wide GEMM on bf16 activations, y[M,N] f32 = x[M,K] bf16 . W^T (W NVFP4);
// ws = gemm_bf16_workspace_bytes(M, K) bytes.
size_t gemm_bf16_workspace_bytes(int M, int K);
void gemm_bf16(float* y, const WRef& W, const void* x_bf16, int M, int N, int K, void* ws, cudaStream_t s);
// The dense-layer MLP (reference kernels/layer.cu:235-254) on NVFP4 weights gate, up [inter, hidden] and
// down [hidden, inter]: ws = dense_mlp_workspace_bytes(M, hidden, inter) bytes.
size_t dense_mlp_workspace_bytes(int M, int hidden, int inter);
void dense_mlp_nvfp4(const float* x, const WRef& gate, const WRef& up, const WRef& down, int hidden, int inter,
                     float limit, float* y, void* ws, int M, cudaStream_t s);

void f32_to_bf16(void* dst, const float* src, size_t n, cudaStream_t s);
void f32_from_bf16_dev(float* dst, const void* src, size_t n, cudaStream_t s);

}  // namespace glm5
