// e2e_loop.cu -- the host loop of the benchmark's end-to-end leg, in C++ against the C ABI: what an engine
// written like the reference's (src/engine.cu: one host thread, one stream, the result read every step)
// does around a fused sibling-gemv call.  Per step: copy the activation rows from pinned host memory,
// b200_nvfp4_gemv_multi on the step's weight copy, copy the outputs back to pinned host memory (the three
// captured once per weight copy and replayed as one graph launch), wait.
// Built as a small shared library so that bench.py can hand it device / pinned pointers and read the time.
#include <chrono>
#include <cuda_runtime.h>
#include "b200_nvfp4.h"

extern "C" double e2e_gemv_multi_loop(const b200_gemv_job* jobs, int copies, int n, int M, int K,
                                      const float* x_host, float* x_dev, size_t x_bytes,
                                      const float* y_dev, float* y_host, size_t y_bytes,
                                      int steps, int warmup, cudaStream_t s, int* rc_out) {
    int rc = 0;
    auto enqueue = [&](int i) {
        if (cudaMemcpyAsync(x_dev, x_host, x_bytes, cudaMemcpyHostToDevice, s) != cudaSuccess) rc = -1;
        if (int r = b200_nvfp4_gemv_multi(jobs + (size_t)(i % copies) * n, n, M, K, B200_BF16, s)) rc = r;
        if (cudaMemcpyAsync(y_host, y_dev, y_bytes, cudaMemcpyDeviceToHost, s) != cudaSuccess) rc = -1;
    };
    // The three operations of a step as ONE graph launch per step (one graph per weight copy, built before the
    // timed region): what a decode loop that replays captured steps does.  The copies from and to pinned host
    // memory are nodes of the graph, so they run every step inside the timed region; if capture is not possible
    // the step falls back to three stream calls.
    constexpr int MAX_COPIES = 64;
    cudaGraphExec_t exec[MAX_COPIES] = {};
    bool graphs = copies >= 1 && copies <= MAX_COPIES;
    if (graphs) {
        enqueue(0);                                               // outside capture first: one-time set-up inside the library
        if (cudaStreamSynchronize(s) != cudaSuccess) rc = -1;
        for (int c = 0; c < copies && graphs; ++c) {
            cudaGraph_t g = nullptr;
            if (cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal) != cudaSuccess) { graphs = false; break; }
            enqueue(c);
            if (cudaStreamEndCapture(s, &g) != cudaSuccess || !g || rc != 0) { graphs = false; rc = 0; if (g) cudaGraphDestroy(g); break; }
            if (cudaGraphInstantiate(&exec[c], g, 0) != cudaSuccess) graphs = false;
            cudaGraphDestroy(g);
        }
        if (!graphs) cudaGetLastError();
    }
    auto step = [&](int i) {
        if (graphs) { if (cudaGraphLaunch(exec[i % copies], s) != cudaSuccess) rc = -1; }
        else enqueue(i);
        if (cudaStreamSynchronize(s) != cudaSuccess) rc = -1;      // the caller reads the result every step
    };
    for (int i = 0; i < warmup; ++i) step(i);
    const auto t0 = std::chrono::steady_clock::now();
    for (int i = 0; i < steps; ++i) step(i);
    const double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count() / (steps > 0 ? steps : 1);
    for (int c = 0; c < MAX_COPIES; ++c) if (exec[c]) cudaGraphExecDestroy(exec[c]);
    if (rc_out) *rc_out = rc;
    return ms;
}
