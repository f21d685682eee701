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

// gemv.cu
int nvfp4_multi(const b200_gemv_job* jobs, int n, int M, int K, cudaStream_t s);
int dense_gemm(float* y, const void* W, const float* x, int M, int N, int K, int dtype, cudaStream_t s);
int nvfp4_math_mode();

}  // namespace b200
