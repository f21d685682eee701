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

// One 16-group: scale code and sixteen e2m1 codes, bit for bit what the reference's fp32 operations give.
//
// The reference computes q = fl(v / eff) per element and counts the e2m1 mid-points strictly below |q|.
// A correctly rounded division per element is what made this kernel instruction-bound, so the count is
// taken without dividing: fl(|v| / eff) > mid  <=>  |v| / eff > mid + ulp(mid)/2 in real arithmetic (all
// seven mid-points have even mantissas, so an exact tie rounds back down to the mid-point)  <=>
// |v| > eff * (mid + ulp(mid)/2), and that product of a 24-bit and a 25-bit number is exact in double.
// Rounded DOWN to fp32 it is a threshold t with  |v| > t  <=>  the reference's comparison, for every fp32 v
// (an infinity exceeds every threshold, a NaN none: as v / eff would).  Seven thresholds per group, then
// seven comparisons per element.
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
    // mid-points 0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5 plus half an ulp of their binade (2^-26 .. 2^-22)
    const double de = (double)eff;
    const float t0 = __double2float_rd(de * (0.25 + 0x1p-26)), t1 = __double2float_rd(de * (0.75 + 0x1p-25)),
                t2 = __double2float_rd(de * (1.25 + 0x1p-24)), t3 = __double2float_rd(de * (1.75 + 0x1p-24)),
                t4 = __double2float_rd(de * (2.5 + 0x1p-23)), t5 = __double2float_rd(de * (3.5 + 0x1p-23)),
                t6 = __double2float_rd(de * (5.0 + 0x1p-22));
    lo = 0; hi = 0;
    #pragma unroll
    for (int j = 0; j < 16; ++j) {
        const float a = fabsf(v[j]);
        uint32_t c = (uint32_t)((a > t0) + (a > t1) + (a > t2) + (a > t3) + (a > t4) + (a > t5) + (a > t6));
        if (c != 0 && (__float_as_uint(v[j]) >> 31)) c |= 8u;
        if (j < 8) lo |= c << (4 * j); else hi |= c << (4 * (j - 8));
    }
}

// The same group for bf16 inputs, two elements per instruction.  u[j] holds elements 2j (low half) and 2j+1 as
// they lie in memory.  A bf16 magnitude a exceeds an fp32 threshold t >= 0 exactly when it exceeds t rounded DOWN
// to bf16 (a is on the bf16 grid: the next grid point above floor(t) is above t), so the seven comparisons run on
// packed bf16 pairs; each answers 1.0 or 0.0, and their sum on top of 128.0 is the bf16 number 0x4300 + count
// (a step of 1 at that exponent), so the count is read off the low three bits.  Bit for bit quantize_group.
__device__ __forceinline__ void quantize_group_bf16(const uint32_t (&u)[8], float gs, uint32_t& lo, uint32_t& hi, int& code) {
    uint32_t a[8];
    #pragma unroll
    for (int j = 0; j < 8; ++j) a[j] = u[j] & 0x7fff7fffu;
    // amax: magnitudes order like their bit patterns, per 16-bit half
    uint32_t m = a[0];
    #pragma unroll
    for (int j = 1; j < 8; ++j) m = __vmaxu2(m, a[j]);
    const uint32_t mh = max(m & 0xffffu, m >> 16);
    // a NaN in the group: the float maximum of the reference's code ignores it unless... keep fp32 semantics: fmaxf drops NaNs
    float amax = 0.f;
    if (mh <= 0x7f80u) amax = __uint_as_float(mh << 16);
    else {
        #pragma unroll
        for (int j = 0; j < 8; ++j) {
            amax = fmaxf(amax, __uint_as_float(a[j] << 16));
            amax = fmaxf(amax, __uint_as_float(a[j] & 0xffff0000u));
        }
    }
    float s = __fmul_rn(__fdiv_rn(amax, 6.0f), gs);
    s = fminf(fmaxf(s, 0.f), 448.f);
    code = e4m3_floor_code(s);
    if (code < 126) {
        const float mid = __fmul_rn(__fadd_rn(e4m3_to_f32(code + 1), e4m3_to_f32(code)), 0.5f);
        code += (mid < s) ? 1 : 0;
    }
    const float eff = fmaxf(__fdiv_rn(e4m3_to_f32(code), gs), 1e-30f);
    const double de = (double)eff;
    auto thr = [&](double mid_plus) -> __nv_bfloat162 {
        const uint32_t b = __float_as_uint(__double2float_rd(de * mid_plus)) >> 16;      // truncation = rounding down (t >= 0)
        const uint32_t p = b | (b << 16);
        return *reinterpret_cast<const __nv_bfloat162*>(&p);
    };
    const __nv_bfloat162 t0 = thr(0.25 + 0x1p-26), t1 = thr(0.75 + 0x1p-25), t2 = thr(1.25 + 0x1p-24), t3 = thr(1.75 + 0x1p-24),
                         t4 = thr(2.5 + 0x1p-23), t5 = thr(3.5 + 0x1p-23), t6 = thr(5.0 + 0x1p-22);
    const uint32_t base_bits = 0x43004300u;                                                  // 128.0 | 128.0
    const __nv_bfloat162 base = *reinterpret_cast<const __nv_bfloat162*>(&base_bits);
    lo = 0; hi = 0;
    #pragma unroll
    for (int j = 0; j < 8; ++j) {
        const __nv_bfloat162 av = *reinterpret_cast<const __nv_bfloat162*>(&a[j]);
        __nv_bfloat162 c = __hadd2(base, __hgt2(av, t0));
        c = __hadd2(c, __hgt2(av, t1)); c = __hadd2(c, __hgt2(av, t2)); c = __hadd2(c, __hgt2(av, t3));
        c = __hadd2(c, __hgt2(av, t4)); c = __hadd2(c, __hgt2(av, t5)); c = __hadd2(c, __hgt2(av, t6));
        uint32_t ci = *reinterpret_cast<const uint32_t*>(&c) & 0x00070007u;                  // two counts
        const uint32_t nz = (ci + 0x00070007u) & 0x00080008u;                                // 8 where the count is not 0
        ci |= (u[j] >> 12) & nz;                                                             // the sign bit, on non-zero codes only
        const uint32_t byte = (ci | (ci >> 12)) & 0xffu;                                     // low nibble = even element
        if (j < 4) lo |= byte << (8 * j); else hi |= byte << (8 * (j - 4));
    }
}
}  // namespace b200
