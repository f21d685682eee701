// b200_internal.h -- declarations shared by the library's translation units (not installed).
#pragma once
#include <cuda_runtime.h>
#include <algorithm>
#include <cstdint>
#include <cstddef>
#include "b200_nvfp4.h"

namespace b200 {

// Number of SMs of the current device (cached per device index).
int sm_count();
// cudaGetLastError() after a launch: 0, or B200_ELAUNCH with the runtime's text on stderr.
int check_launch(const char* what);
int launch_failed(const char* what);
// Device address of the status word that bounded waits write to (null if the query failed).
unsigned int* device_status_ptr();
// 1 if the caller declared weight buffers immutable while kernels run (B200_OPT_STABLE_WEIGHTS).
int stable_weights_option();

// One launch's worth of NVFP4 gemv jobs as the kernels see them.  task0 is the index of the
// job's first row tile in the launch's flat tile list (general kernel only).
struct GemvJobDev {
    float* y; const uint8_t* P; const uint8_t* S; const float* gs; const float* x;
    int N; int task0;
};
struct GemvParams {
    GemvJobDev j[B200_GEMV_MULTI_MAX];
    int n_jobs, total_tasks, K;
};

// gemv.cu
int nvfp4_multi(const b200_gemv_job* jobs, int n, int M, int K, cudaStream_t s, void* split_ws);
int dense_gemm(float* y, const void* W, const float* x, int M, int N, int K, int dtype, cudaStream_t s);
int nvfp4_math_mode();

// gemv_tma.cu: single-row (M = 1) bulk-copy pipelined kernel; returns B200_ENOTIMPL when the
// shapes / alignments it needs do not hold, and the caller then uses the general kernel.
int nvfp4_multi_tma(const GemvParams& p, cudaStream_t s);
// gemv_umma.cu: single-row tensor-core (tcgen05 block-scaled) kernel; same contract.
int nvfp4_multi_umma(const GemvParams& p, int M, cudaStream_t s);
size_t umma_presplit_bytes(int M, int K);
int nvfp4_multi_umma_ws(const GemvParams& p, int M, void* ws, cudaStream_t s);
// One job of the tensor-core kernel: x [M, K], y [M, N].  x2 != nullptr: the activations are the
// clamped SwiGLU of two vectors, x = silu(min(x, limit)) * clamp(x2, -limit, limit) (the MoE down
// projection reads the gate and up products directly).  mw, ms: CUtensorMap of packed weights and
// of scales in GLOBAL memory (job-table launches); nullptr = the maps passed as kernel parameters.
// bimg != nullptr: the activation rows were already split into their B image (K/256 x 8 KB, rows at a
// stride of 8) and digit weights gam[M*8] by k_split_rows; x and x2 are then not read.
struct UmJob { float* y; const float* x; const float* x2; const float* gs; const void* mw; const void* ms;
               const unsigned char* bimg; const float* gam; int N; int M; int task0; int pad; };
// One unit of k_split_rows: M rows of x (SwiGLU with x2 when x2 != nullptr) -> bimg, gam.  M = 0: nothing.
struct SplitJob { const float* x; const float* x2; unsigned char* bimg; float* gam; int M; int pad; };
int umma_split_launch(const SplitJob* jobs, int n_jobs, int K, float limit, cudaStream_t s);
bool umma_shape_ok(int K);
// moe_umma.cu: the experts of a prepared layer on the tensor-core kernel; B200_ENOTIMPL = not applicable.
size_t moe_umma_ws_bytes(const b200_moe_layer* L, int M);
struct MoePlan;
int moe_umma_plan_args(const float* x, const b200_moe_layer* L, void* scratch, int M, MoePlan* q, int* R_gu, int* R_d);
int moe_umma_experts(const float* x, const b200_moe_layer* L, float* y, const int32_t* sel, const float* wts,
                     void* scratch, int M, cudaStream_t s, bool planned);
int umma_encode_maps(void* out_w, void* out_s, const void* P, const void* S, int N, int K, int R);    // two 128-byte maps, host memory
int umma_table_launch(const UmJob* table, int n_jobs, int N, int K, int R, float limit, int max_m, cudaStream_t s);

}  // namespace b200
