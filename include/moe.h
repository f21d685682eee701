// moe.h -- source-compatible replacement for the reference's include/moe.h (namespace glm5),
// implemented by libb200nvfp4.so: Nvfp4Mat (:13-17), MoeLayer (:19-26), moe_workspace_floats /
// moe_batch_workspace_floats / nvfp4_check_align (:28-30), moe_forward / moe_route (:32-35),
// moe_forward_batch / moe_route_batch (:41-45).
// The reference compiles the layer geometry in (hidden 4096, inter 2048, scale 2.5, clamp 10,
// renormalised gates; include/glm5_config.h:20, 84-91).  Here those are the defaults of a
// process-wide setting that moe_set_geometry changes, e.g. to inter = 1536.
#pragma once
#include <cuda_runtime.h>
#include <cstddef>
#include <cstdint>
#include "gemv.h"

namespace glm5 {

struct Nvfp4Mat {
    const uint8_t* packed;   // [out, in/2], low nibble = even column
    const uint8_t* scale;    // [out, in/16], fp8-e4m3
    const float*   gscale;   // [1]
};

struct MoeLayer {
    WRef            router_w;      // bf16 [n_expert, hidden]
    const float*    router_bias;   // fp32 [n_expert]
    const Nvfp4Mat* experts;       // DEVICE array of 3*n_expert: [3e] gate, [3e+1] up, [3e+2] down
    const Nvfp4Mat* shared;        // DEVICE array of 3
    int n_expert;
    int topk;
};

// Not in the reference: layer geometry used by every call below (defaults = reference constants).
// This is the ONE piece of process-wide state behind this header (MoeLayer has no room for it and the
// reference's callers do not pass it): set it once, before moe_workspace_floats /
// moe_batch_workspace_floats are asked for a size -- a workspace sized under one geometry is too small
// for a larger one, and the calls cannot check that (ws carries no size).  Callers that need several
// geometries in one process use the C ABI, whose b200_moe_layer carries the geometry per layer.
void moe_set_geometry(int hidden, int inter, float routed_scale, float swiglu_limit, bool norm_topk);
// Not in the reference: once per layer after its tables are built (src/engine.cu:168-195 is the
// place), so that moe_forward* run their experts on the tensor-core kernels.
// Synchronous (reads the tables back); false = the layer's geometry or alignment does not suit
// them and it keeps the CUDA-core kernels.  moe_release drops what moe_prepare built.
bool moe_prepare(const MoeLayer& L);
void moe_release(const MoeLayer& L);

size_t moe_workspace_floats();
size_t moe_batch_workspace_floats(int M);
// true if the fast expert kernels can read this tensor (16-byte aligned packed, 2-byte aligned
// scale, 4-byte aligned gscale); prints what is wrong otherwise.  The reference's floor was 4 bytes.
bool nvfp4_check_align(const Nvfp4Mat& m, const char* what);

void moe_forward(const float* x, const MoeLayer& L, float* y, int32_t* sel, float* wts, float* ws,
                 cudaStream_t s);
void moe_route(const float* x, const MoeLayer& L, int32_t* sel, float* wts, float* logits, cudaStream_t s);
void moe_forward_batch(const float* x, const MoeLayer& L, float* y, int32_t* sel, float* wts, float* ws,
                       int M, cudaStream_t s);
void moe_route_batch(const float* x, const MoeLayer& L, int32_t* sel, float* wts, float* logits, int M,
                     cudaStream_t s);

}  // namespace glm5
