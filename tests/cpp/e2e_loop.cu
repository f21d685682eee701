// e2e_loop.cu -- the host loop of the benchmark's end-to-end leg, in C++ against the C ABI: what an engine
// written like the reference's (src/engine.cu: one host thread, one stream, the result read every step)
// does around a fused sibling-gemv call.  Per step: copy the activation rows from pinned host memory,
// b200_nvfp4_gemv_multi on the step's weight copy, copy the outputs back to pinned host memory, wait.
// Built as a small shared library so that bench.py can hand it device / pinned pointers and read the time.
#include <chrono>
#include <cuda_runtime.h>
#include "b200_nvfp4.h"

extern "C" double e2e_gemv_multi_loop(const b200_gemv_job* jobs, int copies, int n, int M, int K,
                                      const float* x_host, float* x_dev, size_t x_bytes,
                                      const float* y_dev, float* y_host, size_t y_bytes,
                                      int steps, int warmup, cudaStream_t s, int* rc_out) {
    int rc = 0;
    auto step = [&](int i) {
        if (cudaMemcpyAsync(x_dev, x_host, x_bytes, cudaMemcpyHostToDevice, s) != cudaSuccess) rc = -1;
        if (int r = b200_nvfp4_gemv_multi(jobs + (size_t)(i % copies) * n, n, M, K, B200_BF16, s)) rc = r;
        if (cudaMemcpyAsync(y_host, y_dev, y_bytes, cudaMemcpyDeviceToHost, s) != cudaSuccess) rc = -1;
        if (cudaStreamSynchronize(s) != cudaSuccess) rc = -1;      // the caller reads the result every step
    };
    for (int i = 0; i < warmup; ++i) step(i);
    const auto t0 = std::chrono::steady_clock::now();
    for (int i = 0; i < steps; ++i) step(i);
    const double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count() / (steps > 0 ? steps : 1);
    if (rc_out) *rc_out = rc;
    return ms;
}
