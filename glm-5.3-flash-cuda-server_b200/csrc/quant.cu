// quant.cu -- bf16 -> NVFP4 quantiser and NVFP4 -> fp32 dequantiser for sm_100a.
//
// Bit-exact with the reference's numpy quantiser (tools/requant_dense_nvfp4.py:53-68 quant_block,
// :209-215 global scale).  What "bit-exact" forces here:
//   * every step is one IEEE fp32 operation in the reference's order (amax/6, *gs, clip,
//     e4m3(code)/gs, w/eff): no FMA contraction, no approximate division -- the expressions use
//     __fdiv_rn / __fmul_rn so the compiler cannot fuse or reorder them;
//   * code selection is numpy's searchsorted(mid, v) = "number of mid-points strictly below v",
//     so a value exactly on a mid-point takes the LOWER code; the hardware converters round such
//     ties to even, which is why cvt.rn.satfinite.e2m1x2 / e4m3x2 are not used here;
//   * the global scale is a double-precision quotient rounded once to fp32.
// HBM-bound: 2 B read and 0.5625 B written per weight; one thread owns one 16-group (32 B in,
// 8 B + 1 B out), consecutive threads own consecutive groups, so every access is coalesced.
#include "b200_internal.h"
#include "nvfp4_decode.cuh"
#include "quant_core.cuh"

namespace b200 {

// amax over the tensor.  Non-negative floats order like their bit patterns, so an unsigned
// atomicMax on the bits is an exact, order-independent float max.
__global__ void __launch_bounds__(256)
k_amax_bf16(const uint4* __restrict__ w, size_t n_vec, const __nv_bfloat16* __restrict__ tail,
            size_t n_tail, uint32_t* __restrict__ out_bits) {
    float a = 0.f;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    // packed: |x| as bit patterns, __hmax2 (which, like fmaxf, returns the other operand when one is a NaN)
    uint32_t mbits = 0u;
    auto fold = [&](const uint4& v) {
        const uint32_t u[4] = {v.x, v.y, v.z, v.w};
        #pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t x = u[j] & 0x7fff7fffu;
            const __nv_bfloat162 r = __hmax2(*reinterpret_cast<const __nv_bfloat162*>(&mbits), *reinterpret_cast<const __nv_bfloat162*>(&x));
            mbits = *reinterpret_cast<const uint32_t*>(&r);
        }
    };
    for (; i + 7 * stride < n_vec; i += 8 * stride) {           // eight loads in flight per thread
        uint4 v[8];
        #pragma unroll
        for (int q = 0; q < 8; ++q) v[q] = w[i + q * stride];
        #pragma unroll
        for (int q = 0; q < 8; ++q) fold(v[q]);
    }
    for (; i < n_vec; i += stride) fold(w[i]);
    a = fmaxf(fmaxf(0.f, __uint_as_float(mbits << 16)), __uint_as_float(mbits & 0xffff0000u));
    if (blockIdx.x == 0)
        for (size_t i = threadIdx.x; i < n_tail; i += blockDim.x) a = fmaxf(a, fabsf(__bfloat162float(tail[i])));
    a = warp_max(a);
    if ((threadIdx.x & 31) == 0 && a > 0.f) atomicMax(out_bits, __float_as_uint(a));
}

// In place: amax bits -> gs = fp32(2688 / max(amax, 1e-12)), quotient in double.
__global__ void k_finish_gs(float* gs) {
    double d = (double)gs[0];
    if (!(d >= 1e-12)) d = 1e-12;
    gs[0] = (float)((448.0 * 6.0) / d);
}

__device__ __forceinline__ void unpack_bf16x16(const uint4& a, const uint4& b, float (&v)[16]) {
    const uint32_t u[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    #pragma unroll
    for (int j = 0; j < 8; ++j) {
        v[2 * j] = __uint_as_float(u[j] << 16);
        v[2 * j + 1] = __uint_as_float(u[j] & 0xffff0000u);
    }
}
__device__ __forceinline__ void store_group(uint8_t* packed, uint8_t* scale, size_t g, uint32_t lo, uint32_t hi, int code, bool vec_out) {
    if (vec_out) {
        reinterpret_cast<uint2*>(packed)[g] = make_uint2(lo, hi);
    } else {
        #pragma unroll
        for (int j = 0; j < 4; ++j) { packed[8 * g + j] = (uint8_t)(lo >> (8 * j)); packed[8 * g + 4 + j] = (uint8_t)(hi >> (8 * j)); }
    }
    scale[g] = (uint8_t)code;
}

__global__ void __launch_bounds__(256)
k_quantize(const __nv_bfloat16* __restrict__ w, size_t n_groups, const float* __restrict__ gsp,
           uint8_t* __restrict__ packed, uint8_t* __restrict__ scale, bool vec_in, bool vec_out) {
    const float gs = gsp[0];
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    size_t g = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (vec_in) {
        const uint4* wv = reinterpret_cast<const uint4*>(w);
        // Two groups per trip: four loads in flight, two chains.  The tensor is walked from its END: the amax pass
        // that ran just before read it front to back, so its tail is what the L2 still holds.
        for (; g + stride < n_groups; g += 2 * stride) {
            const size_t ga = n_groups - 1 - g, gb = n_groups - 1 - (g + stride);
            const uint4 a0 = wv[2 * ga], b0 = wv[2 * ga + 1], a1 = wv[2 * gb], b1 = wv[2 * gb + 1];
            const uint32_t u0[8] = {a0.x, a0.y, a0.z, a0.w, b0.x, b0.y, b0.z, b0.w}, u1[8] = {a1.x, a1.y, a1.z, a1.w, b1.x, b1.y, b1.z, b1.w};
            uint32_t lo0, hi0, lo1, hi1; int c0, c1;
            quantize_group_bf16(u0, gs, lo0, hi0, c0);
            quantize_group_bf16(u1, gs, lo1, hi1, c1);
            store_group(packed, scale, ga, lo0, hi0, c0, vec_out);
            store_group(packed, scale, gb, lo1, hi1, c1, vec_out);
        }
    }
    for (; g < n_groups; g += stride) {
        const size_t gr = vec_in ? n_groups - 1 - g : g;
        float v[16];
        if (vec_in) {
            unpack_bf16x16(reinterpret_cast<const uint4*>(w)[2 * gr], reinterpret_cast<const uint4*>(w)[2 * gr + 1], v);
        } else {
            #pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = __bfloat162float(w[16 * gr + j]);
        }
        uint32_t lo, hi; int code;
        quantize_group(v, gs, lo, hi, code);
        store_group(packed, scale, gr, lo, hi, code, vec_out);
    }
}

// out[n,k] = e2m1(nib) * (e4m3(scale) / gs): the operation order of reference
// ref/gen_moe.py:29, so results compare bit for bit.
__global__ void __launch_bounds__(256)
k_dequantize(float* __restrict__ out, const uint8_t* __restrict__ packed, const uint8_t* __restrict__ scale,
             const float* __restrict__ gsp, size_t n_groups) {
    const float gs = gsp[0];
    for (size_t g = (size_t)blockIdx.x * blockDim.x + threadIdx.x; g < n_groups;
         g += (size_t)gridDim.x * blockDim.x) {
        const float sc = __fdiv_rn(e4m3_to_f32(scale[g]), gs);
        #pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint32_t b = packed[8 * g + j];
            const float mag[8] = {0.f, .5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
            const float l = mag[b & 7], h = mag[(b >> 4) & 7];
            out[16 * g + 2 * j] = __fmul_rn((b & 8) ? -l : l, sc);
            out[16 * g + 2 * j + 1] = __fmul_rn((b & 0x80) ? -h : h, sc);
        }
    }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_nvfp4_quantize(const void* w_bf16, int N, int K, uint8_t* packed, uint8_t* scale,
                                   float* gscale, const float* gscale_in, b200_stream stream) {
    if (N < 0 || K <= 0 || (!gscale && !gscale_in)) return B200_EINVAL;
    if (N > 0 && (!w_bf16 || !packed || !scale)) return B200_EINVAL;      // N == 0: only gscale is written
    if (K & 15) return B200_ESHAPE;
    if (((uintptr_t)w_bf16 & 1) || (gscale && ((uintptr_t)gscale & 3))) return B200_EALIGN;
    const size_t n = (size_t)N * K;
    const int grid_cap = sm_count() * 8;
    const float* gs = gscale_in;
    if (!gscale_in) {
        if (cudaMemsetAsync(gscale, 0, 4, stream) != cudaSuccess) return launch_failed("quantize: memset");
        if (n) {
            const bool al = ((uintptr_t)w_bf16 & 15) == 0;
            const size_t n_vec = al ? n / 8 : 0, n_tail = n - n_vec * 8;
            const int grid = (int)std::min<size_t>((n_vec + 255) / 256 + 1, grid_cap);
            k_amax_bf16<<<grid, 256, 0, stream>>>(static_cast<const uint4*>(w_bf16), n_vec,
                static_cast<const __nv_bfloat16*>(w_bf16) + n_vec * 8, n_tail, reinterpret_cast<uint32_t*>(gscale));
            if (int rc = check_launch("k_amax_bf16")) return rc;
        }
        k_finish_gs<<<1, 1, 0, stream>>>(gscale);
        if (int rc = check_launch("k_finish_gs")) return rc;
        gs = gscale;
    }
    if (n == 0) return B200_OK;
    const size_t groups = n / 16;
    const int grid = (int)std::min<size_t>((groups + 255) / 256, grid_cap);
    k_quantize<<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(w_bf16), groups, gs, packed, scale,
                                         ((uintptr_t)w_bf16 & 15) == 0, ((uintptr_t)packed & 7) == 0);
    return check_launch("k_quantize");
}

extern "C" int b200_nvfp4_dequantize(float* out, const b200_nvfp4_mat* W, int N, int K, b200_stream stream) {
    if (!out || !W || !W->packed || !W->scale || !W->gscale || N < 0 || K <= 0) return B200_EINVAL;
    if (K & 15) return B200_ESHAPE;
    const size_t groups = (size_t)N * K / 16;
    if (groups == 0) return B200_OK;
    const int grid = (int)std::min<size_t>((groups + 255) / 256, sm_count() * 8);
    k_dequantize<<<grid, 256, 0, stream>>>(out, W->packed, W->scale, W->gscale, groups);
    return check_launch("k_dequantize");
}
