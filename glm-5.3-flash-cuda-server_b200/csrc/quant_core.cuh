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
// packed bf16 pairs; each answers 1.0 or 0.0.  Summed on top of 128.0, plus 8.0 where the element is negative and
// its count is not zero, they give the bf16 number 0x4300 + code (a step of 1 at that exponent): the e2m1 code is
// the low byte.  Comparisons, sums and the sign all run on the half-precision pipe; the integer pipe only takes
// the magnitudes and gathers the bytes.  Bit for bit quantize_group.
__device__ __forceinline__ void quantize_group_bf16(const uint32_t (&u)[8], float gs, uint32_t& lo, uint32_t& hi, int& code) {
    auto bf2 = [](uint32_t v) { return *reinterpret_cast<const __nv_bfloat162*>(&v); };
    auto bits = [](__nv_bfloat162 v) { return *reinterpret_cast<const uint32_t*>(&v); };
    __nv_bfloat162 a[8];
    #pragma unroll
    for (int j = 0; j < 8; ++j) a[j] = bf2(u[j] & 0x7fff7fffu);
    // amax: __hmax2 returns the other operand when one is a NaN, as fmaxf does
    __nv_bfloat162 m = a[0];
    #pragma unroll
    for (int j = 1; j < 8; ++j) m = __hmax2(m, a[j]);
    const uint32_t mb = bits(m);
    const float amax = fmaxf(fmaxf(0.f, __uint_as_float(mb << 16)), __uint_as_float(mb & 0xffff0000u));
    float s = __fmul_rn(__fdiv_rn(amax, 6.0f), gs);
    s = fminf(fmaxf(s, 0.f), 448.f);
    code = e4m3_floor_code(s);
    if (code < 126) {
        const float mid = __fmul_rn(__fadd_rn(e4m3_to_f32(code + 1), e4m3_to_f32(code)), 0.5f);
        code += (mid < s) ? 1 : 0;
    }
    const float eff = fmaxf(__fdiv_rn(e4m3_to_f32(code), gs), 1e-30f);
    const double de = (double)eff;
    auto thr = [&](double mid_plus) {
        const uint32_t b = __float_as_uint(__double2float_rd(de * mid_plus));      // truncation to bf16 = rounding down (t >= 0)
        return bf2(__byte_perm(b, b, 0x3232));                                     // the high half in both halves
    };
    const __nv_bfloat162 t0 = thr(0.25 + 0x1p-26), t1 = thr(0.75 + 0x1p-25), t2 = thr(1.25 + 0x1p-24), t3 = thr(1.75 + 0x1p-24),
                         t4 = thr(2.5 + 0x1p-23), t5 = thr(3.5 + 0x1p-23), t6 = thr(5.0 + 0x1p-22);
    const __nv_bfloat162 base = bf2(0x43004300u), eight = bf2(0x41004100u), zero = bf2(0u);      // 128.0, 8.0, 0.0
    uint32_t n[8];
    #pragma unroll
    for (int j = 0; j < 8; ++j) {
        const __nv_bfloat162 r0 = __hgt2(a[j], t0);
        __nv_bfloat162 c = __hadd2(base, r0);
        c = __hadd2(c, __hgt2(a[j], t1)); c = __hadd2(c, __hgt2(a[j], t2)); c = __hadd2(c, __hgt2(a[j], t3));
        c = __hadd2(c, __hgt2(a[j], t4)); c = __hadd2(c, __hgt2(a[j], t5)); c = __hadd2(c, __hgt2(a[j], t6));
        c = __hfma2(__hmul2(__hlt2(bf2(u[j]), zero), r0), eight, c);                // + 8 for a negative element with a non-zero count
        n[j] = bits(c);                                                             // byte 0: code of element 2j, byte 2: of element 2j+1
    }
    // low nibbles = even elements, high nibbles = odd elements
    const uint32_t e_lo = __byte_perm(__byte_perm(n[0], n[1], 0x0040), __byte_perm(n[2], n[3], 0x0040), 0x5410);
    const uint32_t o_lo = __byte_perm(__byte_perm(n[0], n[1], 0x0062), __byte_perm(n[2], n[3], 0x0062), 0x5410);
    const uint32_t e_hi = __byte_perm(__byte_perm(n[4], n[5], 0x0040), __byte_perm(n[6], n[7], 0x0040), 0x5410);
    const uint32_t o_hi = __byte_perm(__byte_perm(n[4], n[5], 0x0062), __byte_perm(n[6], n[7], 0x0062), 0x5410);
    lo = e_lo | (o_lo << 4);
    hi = e_hi | (o_hi << 4);
}
}  // namespace b200
