// nvfp4_decode.cuh -- device-side NVFP4 primitives for sm_100a.
//
// Format (reference include/nvfp4.cuh:3-7): packed [N,K/2] u8 with the LOW nibble holding the
// even k, scale [N,K/16] u8 fp8-e4m3, gscale [1] f32;
//     w = e2m1(nibble) * e4m3(scale) / gscale.
// Replaces the reference's fp8e4m3 / e2m1x2 / e4m3x2 / e2m1x8 inlines (include/nvfp4.cuh:30-66).
//
// Why the arithmetic here is packed fp16 and not fp32: at ~6.5 TB/s a B200 must retire ~11.6e12
// weights/s, and the chip issues ~35e12 lane-instructions/s, so a decode+MAC sequence may cost
// at most ~2 instructions per weight.  Turning every weight into an fp32 register (one
// half->float conversion each, on the 64-lane conversion pipe) does not fit; consuming the
// hardware unpack's half2 result directly does:
//   cvt.rn.f16x2.e2m1x2   one instruction per 2 weights (exact: all e2m1 values are fp16 numbers)
//   fma.rn.f16x2          one instruction per 2 MACs, in chains of at most 8 inside one 16-group
//   fma.rn.f32.f16        folds a chain into the fp32 accumulator times the group's e4m3 scale
//                         (e4m3 -> f16 is exact; f16*f16 is exact in fp32)
// Activations are pre-scaled by a power of two per row so that chains cannot overflow fp16.
#pragma once
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cstdint>

namespace b200 {

// Exact e4m3 -> fp32 from the bit fields (positive and negative codes, subnormals included).
__host__ __device__ __forceinline__ float e4m3_to_f32(uint32_t v) {
    const uint32_t e = (v >> 3) & 0xF, m = v & 7;
#ifdef __CUDA_ARCH__
    const float mag = e == 0 ? (float)m * (1.f / 512.f) : __uint_as_float(((e + 120u) << 23) | (m << 20));
#else
    union { uint32_t u; float f; } c; c.u = ((e + 120u) << 23) | (m << 20);
    const float mag = e == 0 ? (float)m * (1.f / 512.f) : c.f;
#endif
    return (v & 0x80) ? -mag : mag;
}

// Two e4m3 scale bytes (low byte = first group) -> half2 bits, one hardware instruction.
__device__ __forceinline__ uint32_t e4m3x2_to_h2(uint16_t two) {
    uint32_t r;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(r) : "h"(two));
    return r;
}

// Four packed bytes (8 weights, k ascending) -> 4 half2 {even k, odd k}.
__device__ __forceinline__ void e2m1x8_to_h2(uint32_t w, uint32_t (&h)[4]) {
    asm("{\n"
        " .reg .b8 b0, b1, b2, b3;\n"
        " mov.b32 {b0, b1, b2, b3}, %4;\n"
        " cvt.rn.f16x2.e2m1x2 %0, b0;\n"
        " cvt.rn.f16x2.e2m1x2 %1, b1;\n"
        " cvt.rn.f16x2.e2m1x2 %2, b2;\n"
        " cvt.rn.f16x2.e2m1x2 %3, b3;\n"
        "}" : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3]) : "r"(w));
}

__device__ __forceinline__ uint32_t hmul2_u(uint32_t a, uint32_t b) {
    uint32_t d; asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d;
}
__device__ __forceinline__ uint32_t hfma2_u(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d; asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c)); return d;
}
__device__ __forceinline__ uint32_t hadd2_u(uint32_t a, uint32_t b) {
    uint32_t d; asm("add.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d;
}

// acc += lo(h2)*s + hi(h2)*s with the products and the sums in fp32 (s is one f16).
__device__ __forceinline__ float fold_h2(float acc, uint32_t h2, uint16_t s) {
    asm("{\n .reg .b16 l, h;\n mov.b32 {l, h}, %1;\n"
        " fma.rn.f32.f16 %0, l, %2, %0;\n fma.rn.f32.f16 %0, h, %2, %0;\n}"
        : "+f"(acc) : "r"(h2), "h"(s));
    return acc;
}

// acc += w.lo*x.lo + w.hi*x.hi, fp16 inputs, fp32 products and sums.
__device__ __forceinline__ float mac2_f32(float acc, uint32_t w2, uint32_t x2) {
    asm("{\n .reg .b16 wl, wh, xl, xh;\n mov.b32 {wl, wh}, %1;\n mov.b32 {xl, xh}, %2;\n"
        " fma.rn.f32.f16 %0, wl, xl, %0;\n fma.rn.f32.f16 %0, wh, xh, %0;\n}"
        : "+f"(acc) : "r"(w2), "r"(x2));
    return acc;
}

// One 16-weight group: 8 packed bytes (wa = k 0..7, wb = k 8..15) against 8 half2 of x.
// MATH 0: one fp16x2 chain of 8 (first link a multiply), folded into fp32 with the scale.
// MATH 1: sixteen f16*f16 -> fp32 MACs, then one fp32 FMA with the scale.
template <int MATH>
__device__ __forceinline__ float group_dot(float acc, uint32_t wa, uint32_t wb, const uint32_t* x,
                                           uint16_t sc_h) {
    uint32_t h[4], g[4];
    e2m1x8_to_h2(wa, h);
    e2m1x8_to_h2(wb, g);
    if (MATH == 0) {
        uint32_t c0 = hmul2_u(h[0], x[0]);
        uint32_t c1 = hmul2_u(g[0], x[4]);
        c0 = hfma2_u(h[1], x[1], c0); c1 = hfma2_u(g[1], x[5], c1);
        c0 = hfma2_u(h[2], x[2], c0); c1 = hfma2_u(g[2], x[6], c1);
        c0 = hfma2_u(h[3], x[3], c0); c1 = hfma2_u(g[3], x[7], c1);
        acc = fold_h2(acc, c0, sc_h);
        acc = fold_h2(acc, c1, sc_h);
        return acc;
    } else {
        float t = 0.f;
        #pragma unroll
        for (int j = 0; j < 4; ++j) t = mac2_f32(t, h[j], x[j]);
        #pragma unroll
        for (int j = 0; j < 4; ++j) t = mac2_f32(t, g[j], x[4 + j]);
        return fmaf(t, __half2float(__ushort_as_half(sc_h)), acc);
    }
}

// Streaming 16-byte / 4-byte / 2-byte global loads that do not allocate in L1: weights are
// read exactly once per launch.
__device__ __forceinline__ uint4 ldg_stream_v4(const void* p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
    return r;
}
__device__ __forceinline__ uint32_t ldg_stream_u32(const void* p) {
    uint32_t r; asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(r) : "l"(p)); return r;
}
__device__ __forceinline__ uint16_t ldg_stream_u16(const void* p) {
    uint16_t r; asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(r) : "l"(p)); return r;
}

__device__ __forceinline__ float warp_sum(float v) {
    #pragma unroll
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
    #pragma unroll
    for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// ---- activation staging ---------------------------------------------------------------------
// x (fp32, one row of K values) -> shared memory as fp16, scaled by a power of two chosen from
// the row's amax so that amax lands in [256, 512): an 8-long fp16 chain of |w| <= 6 stays below
// 8*6*512 = 24576 < 65504, and values down to amax*2^-23 keep full fp16 precision.  Layout:
// 16-byte chunks (8 halves); chunk i is stored at i ^ ((i >> 3) & 7) so that the 4 chunks a
// lane reads for one 32-weight unit (stride 64 B between lanes) fall in distinct banks.
__host__ __device__ __forceinline__ int xs_chunks(int K) { return ((K + 63) >> 6) << 3; }   // padded to 8
__device__ __forceinline__ int xs_swz(int i) { return i ^ ((i >> 3) & 7); }

// Power-of-two scale for a row with the given amax (1 for amax == 0 or non-finite).
__device__ __forceinline__ float row_pow2_scale(float amax) {
    if (!(amax > 0.f) || !(amax < 3.0e38f)) return 1.f;
    int e; frexpf(amax, &e);                       // amax = f * 2^e, f in [0.5, 1)
    int s = 9 - e;                                  // amax * 2^s in [256, 512)
    s = s < -120 ? -120 : (s > 120 ? 120 : s);
    return __uint_as_float((uint32_t)(s + 127) << 23);
}

}  // namespace b200
