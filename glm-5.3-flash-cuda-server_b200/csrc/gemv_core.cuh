// gemv_core.cuh -- the block- and warp-level building blocks shared by the NVFP4 gemv kernel and
// the MoE expert kernels: activation staging into shared memory and the R-rows-per-warp inner
// loop.  The arithmetic order inside warp_rows is what fixes a row's result bit for bit, so
// every kernel that must agree with the gemv (reference invariant "gemv_multi == gemv ==
// gemm row", include/gemv.h:41-44, 65-71) goes through this one copy.
#pragma once
#include "nvfp4_decode.cuh"

namespace b200 {

constexpr int GEMV_THREADS = 256;
constexpr int GEMV_WARPS = GEMV_THREADS / 32;

// ---- activation staging (block-wide) ----------------------------------------------------------
// x: nrows rows of K fp32 values, row stride K.  xs: nrows * xs_chunks(K) 16-byte chunks.
// inv_s[r] receives 1 / (the row's power-of-two scale).  red: nrows * GEMV_WARPS floats.
__device__ __forceinline__ void stage_x(const float* __restrict__ x, int nrows, int K, uint4* xs,
                                        float* inv_s, float* red) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nchunk = K >> 3, stride = xs_chunks(K);
    const bool v4 = (((uintptr_t)x) & 15) == 0;
    for (int m = 0; m < nrows; ++m) {
        const float* xr = x + (size_t)m * K;
        float a = 0.f;
        if (v4) {
            for (int i = tid; i < (K >> 2); i += GEMV_THREADS) {
                const float4 v = reinterpret_cast<const float4*>(xr)[i];
                a = fmaxf(a, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
            }
        } else {
            for (int i = tid; i < K; i += GEMV_THREADS) a = fmaxf(a, fabsf(xr[i]));
        }
        a = warp_max(a);
        if (lane == 0) red[m * GEMV_WARPS + warp] = a;
    }
    __syncthreads();
    for (int m = 0; m < nrows; ++m) {
        float a = 0.f;
        #pragma unroll
        for (int w = 0; w < GEMV_WARPS; ++w) a = fmaxf(a, red[m * GEMV_WARPS + w]);
        const float sc = row_pow2_scale(a);
        if (tid == 0) inv_s[m] = 1.f / sc;
        const float* xr = x + (size_t)m * K;
        for (int i = tid; i < nchunk; i += GEMV_THREADS) {
            float f[8];
            if (v4) {
                const float4 u = reinterpret_cast<const float4*>(xr)[2 * i];
                const float4 v = reinterpret_cast<const float4*>(xr)[2 * i + 1];
                f[0] = u.x; f[1] = u.y; f[2] = u.z; f[3] = u.w; f[4] = v.x; f[5] = v.y; f[6] = v.z; f[7] = v.w;
            } else {
                #pragma unroll
                for (int j = 0; j < 8; ++j) f[j] = xr[8 * i + j];
            }
            uint4 o;
            __half2 h;
            h = __floats2half2_rn(f[0] * sc, f[1] * sc); o.x = *reinterpret_cast<uint32_t*>(&h);
            h = __floats2half2_rn(f[2] * sc, f[3] * sc); o.y = *reinterpret_cast<uint32_t*>(&h);
            h = __floats2half2_rn(f[4] * sc, f[5] * sc); o.z = *reinterpret_cast<uint32_t*>(&h);
            h = __floats2half2_rn(f[6] * sc, f[7] * sc); o.w = *reinterpret_cast<uint32_t*>(&h);
            xs[(size_t)m * stride + xs_swz(i)] = o;
        }
    }
    __syncthreads();
}

// ---- R rows x M activation rows, one warp -----------------------------------------------------
struct RowPtr { const uint8_t* p; const uint8_t* s; };

// ANY = false: rows are 16-byte aligned (packed) and 2-byte aligned (scales), checked by the host.
// ANY = true: rows may sit at the format's floor -- packed bytes 4-byte aligned, scales at any address
// (the reference guarantees no more: kernels/moe.cu:167-174) -- which only the device can see for expert
// tables that live in device memory; the branch is warp-uniform and the values loaded are the same.
template <int R, bool ANY = false>
__device__ __forceinline__ void load_step(const RowPtr (&rows)[R], int c, uint4 (&w)[R], uint16_t (&s)[R]) {
    #pragma unroll
    for (int r = 0; r < R; ++r) {
        const uint8_t* pp = rows[r].p + (size_t)c * 16;
        const uint8_t* ps = rows[r].s + (size_t)c * 2;
        if (!ANY || (((uintptr_t)pp & 15) == 0)) w[r] = ldg_stream_v4(pp);
        else w[r] = make_uint4(ldg_stream_u32(pp), ldg_stream_u32(pp + 4), ldg_stream_u32(pp + 8), ldg_stream_u32(pp + 12));
        if (!ANY || (((uintptr_t)ps & 1) == 0)) s[r] = ldg_stream_u16(ps);
        else s[r] = (uint16_t)((uint32_t)__ldg(ps) | ((uint32_t)__ldg(ps + 1) << 8));
    }
}

template <int M, int R, int MATH, bool ANY = false>
__device__ __forceinline__ void warp_rows(const RowPtr (&rows)[R], int K, const uint4* xs,
                                          float (&acc)[R][M], int lane) {
    const int nch = K >> 5, stride = xs_chunks(K);
    uint4 wc[R]; uint16_t sc[R];
    int c = lane;
    if (c < nch) load_step<R, ANY>(rows, c, wc, sc);
    for (; c < nch; c += 32) {
        uint4 wn[R]; uint16_t sn[R];
        if (c + 32 < nch) load_step<R, ANY>(rows, c + 32, wn, sn);
        #pragma unroll
        for (int m = 0; m < M; ++m) {
            uint32_t xr[16];
            const uint4* xp = xs + (size_t)m * stride;
            #pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint4 v = xp[xs_swz(4 * c + j)];
                xr[4 * j] = v.x; xr[4 * j + 1] = v.y; xr[4 * j + 2] = v.z; xr[4 * j + 3] = v.w;
            }
            #pragma unroll
            for (int r = 0; r < R; ++r) {
                const uint32_t s2 = e4m3x2_to_h2(sc[r]);
                acc[r][m] = group_dot<MATH>(acc[r][m], wc[r].x, wc[r].y, xr, (uint16_t)(s2 & 0xffffu));
                acc[r][m] = group_dot<MATH>(acc[r][m], wc[r].z, wc[r].w, xr + 8, (uint16_t)(s2 >> 16));
            }
        }
        if (c + 32 < nch) {
            #pragma unroll
            for (int r = 0; r < R; ++r) { wc[r] = wn[r]; sc[r] = sn[r]; }
        }
    }
}

// Same loop with a separate staged activation row per weight row (the MoE down projection,
// where each slot's expert multiplies its own intermediate vector).  xr_base[r] points at the
// staged row for weight row r.
template <int R, int MATH, bool ANY = false>
__device__ __forceinline__ void warp_rows_own_x(const RowPtr (&rows)[R], int K,
                                                const uint4* const (&xr_base)[R], float (&acc)[R],
                                                int lane) {
    const int nch = K >> 5;
    uint4 wc[R]; uint16_t sc[R];
    int c = lane;
    if (c < nch) load_step<R, ANY>(rows, c, wc, sc);
    for (; c < nch; c += 32) {
        uint4 wn[R]; uint16_t sn[R];
        if (c + 32 < nch) load_step<R, ANY>(rows, c + 32, wn, sn);
        #pragma unroll
        for (int r = 0; r < R; ++r) {
            uint32_t xr[16];
            #pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint4 v = xr_base[r][xs_swz(4 * c + j)];
                xr[4 * j] = v.x; xr[4 * j + 1] = v.y; xr[4 * j + 2] = v.z; xr[4 * j + 3] = v.w;
            }
            const uint32_t s2 = e4m3x2_to_h2(sc[r]);
            acc[r] = group_dot<MATH>(acc[r], wc[r].x, wc[r].y, xr, (uint16_t)(s2 & 0xffffu));
            acc[r] = group_dot<MATH>(acc[r], wc[r].z, wc[r].w, xr + 8, (uint16_t)(s2 >> 16));
        }
        if (c + 32 < nch) {
            #pragma unroll
            for (int r = 0; r < R; ++r) { wc[r] = wn[r]; sc[r] = sn[r]; }
        }
    }
}

}  // namespace b200
