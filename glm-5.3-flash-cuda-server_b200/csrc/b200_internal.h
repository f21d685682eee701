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
// 1 if calls with scratch and >= 16 activation rows may quantise the activations to NVFP4 (B200_OPT_PREFILL_FP4).
int prefill_fp4_option();
constexpr int PREFILL_MIN_ROWS = 16;

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

// tmap.cu: TMA tensor map of a u8 matrix [rows, row_bytes] with box [box_bytes x box_rows] (128B-swizzled or
// plain), written to `out` (128 bytes, host memory).  cached: remember the encoded map (weights).
bool tmap_available();
bool tmap_u8_2d(void* out, const void* base, size_t rows, size_t row_bytes, int box_bytes, int box_rows, bool swz, bool cached);
bool scale_box(int K, int* box, int* swz);

// common.cu: byte accounting (b200_nvfp4_set_byte_credit).  credit(): host-known counts; the grouped MoE paths
// add their job counts on the device to credit_counters()[0] (gate and up jobs) and [1] (down jobs), each job
// being one pass over one expert matrix; geometry of the last grouped call is remembered for the flush.
void credit(int kind, double bytes);
bool credit_on();
unsigned long long* credit_counters();
void credit_grouped_geometry(int hidden, int inter);

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
                     void* scratch, int M, cudaStream_t s, bool planned, int wide);
// moe.cu: b200_moe_experts with the choice between the exact experts and the wide GEMM made by the caller
// (wide = 1 / 0), or by the row count (-1): an expert-parallel rank decides by the tokens of ALL ranks.
int moe_experts_mode(const float* x, const b200_moe_layer* L, float* y, const int32_t* sel, const float* wts,
                     void* ws, int M, cudaStream_t s, int wide);
int umma_encode_maps(void* out_w, void* out_s, const void* P, const void* S, int N, int K, int R);    // two 128-byte maps, host memory
int umma_table_launch(const UmJob* table, int n_jobs, int N, int K, int R, float limit, int max_m, cudaStream_t s);

// gemm_mxf4.cu: the wide GEMM with both operands in NVFP4 (activations quantised per token first).
// One job: `rows` activation rows, starting at row `row0` of the quantised activation buffer, against one
// weight matrix of N rows; y[m * ldy + n].  gs_x points at the job's first per-token global scale.
// mw, ms: tensor maps of the weight in GLOBAL memory (table launches; box height = the launch's R).
struct GxJob { float* y; const float* gs_w; const float* gs_x; const void* mw; const void* ms; int row0; int rows; int N; int ldy; };
size_t gemm_mxf4_ws_bytes(int M, int K);
bool gemm_mxf4_shape_ok(int K);
int gemm_mxf4_dense(float* y, const b200_wref* W, const void* x, int x_kind, int M, int N, int K, void* ws, cudaStream_t s);
int quant_act_launch(int mode, const void* x, const void* x2, float limit, const int* src_row, const int* m_dev, int M,
                     int rows_launch, int K, unsigned char* xq, unsigned char* sfb, size_t sfb_rows, float* gsx, cudaStream_t s);
int gemm_mxf4_table(const GxJob* table, int max_jobs, long expected_jobs, int NT, int N, int K, int R, const unsigned char* xq, size_t x_rows,
                    const unsigned char* sfb, size_t sfb_rows, cudaStream_t s);

// gemm_f16w.cu: the exact wide GEMM (weights dequantised to fp16 in the kernel, tcgen05 kind::f16).
size_t gemm_f16w_ws_bytes(int M, int K);
int gemm_f16w_dense(float* y, const b200_wref* W, const void* x, int x_kind, int M, int N, int K, void* ws, cudaStream_t s);

}  // namespace b200
