// dense_mlp.cu -- the dense-layer MLP as one call: y = down( silu(min(gate x, L)) * clamp(up x, -L, L) ).
// Replaces the reference's dense_mlp / dense_mlp_batch (kernels/layer.cu:235-254: two gemvs, the
// elementwise k_swiglu_clamped :201-208, a third gemv).  Here gate and up run as ONE fused two-job launch
// (they share x), then the clamped SwiGLU, then down; from 16 rows on (and with the prefill option on)
// the three products run on the wide tensor-core GEMM instead.
#include "b200_internal.h"

namespace b200 {

__global__ void k_swiglu_clamped(float* __restrict__ out, const float* __restrict__ gate, const float* __restrict__ up,
                                 size_t n4, float limit) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n4) return;
    const float4 a = reinterpret_cast<const float4*>(gate)[i], b = reinterpret_cast<const float4*>(up)[i];
    auto f = [&](float g, float u) {
        g = fminf(g, limit);                                        // upper clamp only
        u = fminf(fmaxf(u, -limit), limit);
        return (g / (1.f + __expf(-g))) * u;
    };
    reinterpret_cast<float4*>(out)[i] = make_float4(f(a.x, b.x), f(a.y, b.y), f(a.z, b.z), f(a.w, b.w));
}

static size_t up256(size_t v) { return (v + 255) / 256 * 256; }

}  // namespace b200

using namespace b200;

extern "C" size_t b200_dense_mlp_workspace_bytes(int M, int hidden, int inter) {
    if (M < 1 || hidden < 1 || inter < 1) return 0;
    return 2 * up256((size_t)M * inter * 4) + b200_nvfp4_split_workspace_bytes(M, std::max(hidden, inter));
}

extern "C" int b200_dense_mlp(const float* x, const b200_wref* gate, const b200_wref* up, const b200_wref* down,
                              int hidden, int inter, float limit, float* y, void* ws, int M, b200_stream stream) {
    if (!x || !gate || !up || !down || !y || !ws || M < 1 || hidden < 1 || inter < 1) return B200_EINVAL;
    if (!gate->packed || !up->packed || !down->packed) return B200_EINVAL;      // the NVFP4 path; plain weights go through b200_nvfp4_gemm
    if ((inter & 3) || (hidden & 15) || (inter & 15)) return B200_ESHAPE;
    if ((uintptr_t)ws & 255) return B200_EALIGN;
    float* g = static_cast<float*>(ws);
    float* u = reinterpret_cast<float*>(static_cast<char*>(ws) + up256((size_t)M * inter * 4));
    void* split = static_cast<char*>(ws) + 2 * up256((size_t)M * inter * 4);
    if (M <= B200_GEMV_M_MAX) {
        const b200_gemv_job jobs[2] = {{g, *gate, x, inter}, {u, *up, x, inter}};
        if (int rc = b200_nvfp4_gemv_multi_ws(jobs, 2, M, hidden, B200_BF16, split, stream)) return rc;
    } else {
        if (int rc = b200_nvfp4_gemm_ws(g, gate, x, M, inter, hidden, B200_BF16, split, stream)) return rc;
        if (int rc = b200_nvfp4_gemm_ws(u, up, x, M, inter, hidden, B200_BF16, split, stream)) return rc;
    }
    const size_t n4 = (size_t)M * inter / 4;
    k_swiglu_clamped<<<(unsigned)((n4 + 255) / 256), 256, 0, stream>>>(g, g, u, n4, limit);
    if (int rc = check_launch("k_swiglu_clamped")) return rc;
    return b200_nvfp4_gemm_ws(y, down, g, M, hidden, inter, B200_BF16, split, stream);
}
