// quant_core.cuh -- one 16-group of the bit-exact NVFP4 quantiser (shared by the weight quantiser and
// the per-token activation quantiser of the block-scaled GEMM).
//
// Bit-exact with the reference's numpy quantiser (tools/requant_dense_nvfp4.py:53-68 quant_block):
// every step is one IEEE fp32 operation in the reference's order (__fdiv_rn / __fmul_rn, so that
// the compiler cannot fuse or reorder them), and code selection is numpy's searchsorted(mid, v) =
// "number of mid-points strictly below v", so a value exactly on a mid-point takes the LOWER code
// (the hardware converters round such ties to even, which is why they are not used here).
#pragma once
#include "nvfp4_decode.cuh"

namespace b200 {

// fp32(2688 / max(amax, 1e-12)) with the quotient taken in double (reference :215).
__device__ __forceinline__ float nvfp4_global_scale(float amax) {
    double d = (double)amax;
    if (!(d >= 1e-12)) d = 1e-12;
    return (float)((448.0 * 6.0) / d);
}

// Largest e4m3 code (0..126) whose value is <= s, for 0 <= s <= 448, from the float's fields.
__device__ __forceinline__ int e4m3_floor_code(float s) {
    if (s < 0.015625f) return (int)(s * 512.f);              // subnormal codes: value = m / 512
    const uint32_t b = __float_as_uint(s);
    return (int)((((b >> 23) - 120u) << 3) | ((b >> 20) & 7u));
}

__device__ __forceinline__ int e2m1_index(float a) {          // #{mid < a}, mids of the e2m1 grid
    return (a > 0.25f) + (a > 0.75f) + (a > 1.25f) + (a > 1.75f) + (a > 2.5f) + (a > 3.5f) + (a > 5.0f);
}

// One 16-group: scale code and sixteen e2m1 codes, fp32 IEEE operations in the reference's order.
__device__ __forceinline__ void quantize_group(const float (&v)[16], float gs, uint32_t& lo, uint32_t& hi, int& code) {
    float amax = 0.f;
    #pragma unroll
    for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(v[j]));
    float s = __fmul_rn(__fdiv_rn(amax, 6.0f), gs);
    s = fminf(fmaxf(s, 0.f), 448.f);
    code = e4m3_floor_code(s);
    if (code < 126) {
        const float mid = __fmul_rn(__fadd_rn(e4m3_to_f32(code + 1), e4m3_to_f32(code)), 0.5f);
        code += (mid < s) ? 1 : 0;
    }
    const float eff = fmaxf(__fdiv_rn(e4m3_to_f32(code), gs), 1e-30f);
    lo = 0; hi = 0;
    #pragma unroll
    for (int j = 0; j < 16; ++j) {
        const float q = __fdiv_rn(v[j], eff);
        uint32_t c = (uint32_t)e2m1_index(fabsf(q));
        if (c != 0 && (__float_as_uint(q) >> 31)) c |= 8u;
        if (j < 8) lo |= c << (4 * j); else hi |= c << (4 * (j - 8));
    }
}
}  // namespace b200
