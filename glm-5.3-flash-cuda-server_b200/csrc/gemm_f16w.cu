// gemm_f16w.cu -- the EXACT wide GEMM: y[M,N] = x[M,K] . W[N,K]^T with NVFP4 weights dequantised inside the
// kernel to fp16 and multiplied on tcgen05.mma kind::f16 (fp32 accumulation in TMEM).
//
// Why it is exact: e2m1(w) * e4m3(scale) has at most six significant bits and an exponent between 2^-10 and
// 2^11, so it is an fp16 number; a bf16 activation has eight significant bits and, scaled per token by a
// power of two so that the token's maximum lies in [2^13, 2^14), is an fp16 number too (elements more than
// 2^-27 below the token's maximum lose bits: far below any tolerance).  fp16 x fp16 products are exact in
// fp32, so the only rounding is the fp32 accumulation -- the semantics of the reference's fp32-activation
// gemm (kernels/gemv.cu:246-329), which the block-scaled FP4 x FP4 path cannot give.  f32 activations are
// rounded to fp16 once per element (2^-12 relative, rel-L2 of a product about 1.4e-4).
// The reference reads W once per 4 rows (kernels/gemv.cu:369-396); here W crosses HBM once per call and the
// decode cost is paid once per weight and CTA, not once per weight and row.
//
// One CTA of 16 warps per (128 weight rows, job of up to NT activation rows); K in super-steps of 256 (one TMA
// box of packed weights) = two half-steps of 128 (what the fp16 operand buffers hold).
//   warp 0      TMA: per super-step the packed weights [128 B x 128 rows] (128B-swizzled) and their scale bytes
//               [16 B x 128 rows] into one slot of a ring
//   warp 3      TMA: per half-step two boxes [128 B x NT rows] of the fp16 activations (64 k each)
//   warps 4-11  converters: per half-step 128 rows x 128 k: cvt.rn.f16x2.e2m1x2, times the group's scale
//               (e4m3 -> f16, exact), stored as the K-major 128B-swizzled fp16 tile the MMA reads; several
//               operand buffers, so that the conversion runs ahead of the MMAs
//   warp 1      MMA issuer: 8 tcgen05.mma.kind::f16 (K = 16 each) per half-step, tcgen05.commit frees
//               the operand buffer, the activation slot and (every second half-step) the packed slot
//   warp 2      TMEM allocation;  warps 12-15  epilogue: D[128 rows, NT tokens] * 2^e[token] / gs_w -> y
// Barriers are per step and used once (K <= 16384: 64 super-steps, 128 half-steps); every wait is bounded.
// No cluster launch, no multicast.
#include "b200_internal.h"
#include "nvfp4_decode.cuh"
#include "tma_pipe.cuh"
#include <cuda.h>
#include <cuda_fp16.h>
#include <cstdio>

namespace b200 {

constexpr int GF_THREADS = 512;
constexpr int GF_CONV = 256;
constexpr int GF_MAX_SUPER = 64, GF_MAX_HALF = 128;          // K <= 16384
constexpr uint32_t GF_P_BYTES = 16384 + 2048;                // a super-step: packed weights 128 rows x 128 B, then their scales 128 rows x 16 B
constexpr uint32_t GF_A16_BYTES = 32768;                     // fp16 operand of a half-step: 2 k-blocks x [128 rows x 128 B]

struct GfParams {
    float* y; const float* gs_w; const float* rowscale;      // rowscale[m] = 2^e of token m (NaN for a non-finite token)
    unsigned int* status;
    int M, N, K, n_jobs, sp, sb, na, prefetch_before_wait;      // ring slots: packed, activations, fp16 operand buffers
};

__device__ __forceinline__ void gf_tma_2d(uint32_t dst, const void* map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 :: "r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ uint64_t gf_desc(uint32_t saddr) {      // K-major, 128B-swizzled, 8-row groups 1024 B apart
    return (uint64_t)((saddr >> 4) & 0x3FFF) | ((uint64_t)(1024u >> 4) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}

template <int NT>
__global__ void __launch_bounds__(GF_THREADS, 1)
k_gemm_f16w(const __grid_constant__ GfParams p, const __grid_constant__ CUtensorMap map_x,
            const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_s) {
    constexpr uint32_t B_BYTES = 2u * NT * 128u;             // activations of a half-step: 2 k-blocks x [NT rows x 128 B]
    extern __shared__ __align__(1024) unsigned char smem[];
    __shared__ uint64_t fullP[GF_MAX_SUPER], fullB[GF_MAX_HALF], a16_full[GF_MAX_HALF], done16[GF_MAX_HALF], done_bar;
    __shared__ uint32_t tmem_base_s;
    __shared__ float sx[NT];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int K = p.K, nsup = K >> 8, nhalf = K >> 7;
    const int tile_n = (int)blockIdx.x / p.n_jobs, ji = (int)blockIdx.x - tile_n * p.n_jobs;
    const int rown0 = tile_n * 128, m0 = ji * NT, rows = min(NT, p.M - m0);

    unsigned char* ringP = smem + ((1024u - (smem_u32(smem) & 1023u)) & 1023u);
    unsigned char* a16 = ringP + (size_t)p.sp * GF_P_BYTES;          // na operand buffers
    unsigned char* ringB = a16 + (size_t)p.na * GF_A16_BYTES;

    pdl_launch_dependents();
    for (int i = tid; i < nsup; i += GF_THREADS) mbar_init(smem_u32(&fullP[i]), 1);
    for (int i = tid; i < nhalf; i += GF_THREADS) {
        mbar_init(smem_u32(&fullB[i]), 1);
        mbar_init(smem_u32(&a16_full[i]), GF_CONV / 32);
        mbar_init(smem_u32(&done16[i]), 1);
    }
    if (tid == 0) mbar_init(smem_u32(&done_bar), 1);
    mbar_fence_init();
    if (warp == 2) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_u32(&tmem_base_s)), "r"(NT < 32 ? 32 : NT));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmem_base_s;

    if (warp == 0) {
        // ---- packed weights and their scales: lane l issues super-steps l, l + 32, .. ----
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" :: "l"(&map_w) : "memory");
            asm volatile("prefetch.tensormap [%0];" :: "l"(&map_s) : "memory");
        }
        if (!p.prefetch_before_wait) pdl_wait();
        for (int g = lane; g < nsup; g += 32) {
            // the slot is free once the operand of the second half-step of the super-step that held it has been
            // converted (a16_full), not only multiplied: the MMAs never read the packed bytes
            if (g >= p.sp) mbar_wait_spin(smem_u32(&a16_full[2 * (g - p.sp) + 1]), 0, p.status, 21);
            const uint32_t bar = smem_u32(&fullP[g]), dst = smem_u32(ringP) + (uint32_t)(g % p.sp) * GF_P_BYTES;
            mbar_expect_tx(bar, GF_P_BYTES);
            gf_tma_2d(dst, &map_w, g * 128, rown0, bar);
            gf_tma_2d(dst + 16384, &map_s, g * 16, rown0, bar);                  // the super-step's 16 scale bytes of every row
        }
        __syncwarp();
    } else if (warp == 3) {
        // ---- activations: lane l issues half-steps l, l + 32, .. ----
        if (lane == 0) asm volatile("prefetch.tensormap [%0];" :: "l"(&map_x) : "memory");
        pdl_wait();                                  // they come from the conversion launch
        for (int h = lane; h < nhalf; h += 32) {
            if (h >= p.sb) mbar_wait_spin(smem_u32(&done16[h - p.sb]), 0, p.status, 22);
            const uint32_t bar = smem_u32(&fullB[h]), dst = smem_u32(ringB) + (uint32_t)(h % p.sb) * B_BYTES;
            mbar_expect_tx(bar, B_BYTES);
            gf_tma_2d(dst, &map_x, (2 * h) * 128, m0, bar);
            gf_tma_2d(dst + NT * 128u, &map_x, (2 * h + 1) * 128, m0, bar);
        }
        __syncwarp();
        // asynchronous commit arrivals must have landed before the CTA's shared memory is handed on
        for (int h = max(0, nhalf - 32) + lane; h < nhalf; h += 32) mbar_wait_spin(smem_u32(&done16[h]), 0, p.status, 23);
        __syncwarp();
    } else if (warp == 1) {
        // ---- MMA issuer ----
        const uint32_t idesc = (1u << 4) | ((uint32_t)(NT >> 3) << 17) | ((128u >> 4) << 24);     // D f32, A and B f16, K-major
        const uint64_t dA0 = gf_desc(smem_u32(a16)), dB0 = gf_desc(smem_u32(ringB));
        for (int h = 0; h < nhalf; ++h) {
            mbar_wait_spin(smem_u32(&a16_full[h]), 0, p.status, 24);
            mbar_wait_spin(smem_u32(&fullB[h]), 0, p.status, 25);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (lane == 0) {
                const uint64_t oA = (uint64_t)(((uint32_t)(h % p.na) * GF_A16_BYTES) >> 4), oB = (uint64_t)(((uint32_t)(h % p.sb) * B_BYTES) >> 4);
                #pragma unroll
                for (int kb = 0; kb < 2; ++kb) {
                    #pragma unroll
                    for (int k16 = 0; k16 < 4; ++k16) {
                        const uint64_t da = dA0 + oA + (uint64_t)(kb * (16384 >> 4)) + k16 * 2;
                        const uint64_t db = dB0 + oB + (uint64_t)(kb * ((NT * 128) >> 4)) + k16 * 2;
                        asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                                     " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                                     :: "r"(tmem), "l"(da), "l"(db), "r"(idesc), "r"((uint32_t)((h | kb | k16) != 0)) : "memory");
                    }
                }
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(smem_u32(&done16[h])) : "memory");
            }
            __syncwarp();
        }
        if (lane == 0) asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(smem_u32(&done_bar)) : "memory");
        __syncwarp();
    } else if (warp >= 4 && warp < 12) {
        // ---- converters: thread -> (weight row r, k-block kb of the half-step) ----
        const int t = tid - 128, r = t & 127, kb = t >> 7;      // a quarter-warp = 8 consecutive rows: conflict-free swizzled accesses
        for (int h = 0; h < nhalf; ++h) {
            const int g = h >> 1, half = h & 1;
            mbar_wait_spin(smem_u32(&fullP[g]), 0, p.status, 27);
            if (h >= p.na) mbar_wait_spin(smem_u32(&done16[h - p.na]), 0, p.status, 28);      // the operand buffer is free again
            const unsigned char* pk = ringP + (size_t)(g % p.sp) * GF_P_BYTES + (size_t)r * 128;
            const int j0 = half * 4 + kb * 2;
            const uint4 w0 = *reinterpret_cast<const uint4*>(pk + (((j0) ^ (r & 7)) << 4));
            const uint4 w1 = *reinterpret_cast<const uint4*>(pk + (((j0 + 1) ^ (r & 7)) << 4));
            const uint32_t sc4 = *reinterpret_cast<const uint32_t*>(ringP + (size_t)(g % p.sp) * GF_P_BYTES + 16384 + r * 16 + half * 8 + kb * 4);      // four group scales
            const uint32_t s01 = e4m3x2_to_h2((uint16_t)(sc4 & 0xffffu)), s23 = e4m3x2_to_h2((uint16_t)(sc4 >> 16));
            const uint32_t sc[4] = {__byte_perm(s01, s01, 0x1010), __byte_perm(s01, s01, 0x3232), __byte_perm(s23, s23, 0x1010), __byte_perm(s23, s23, 0x3232)};
            const uint32_t w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
            unsigned char* dst = a16 + (size_t)(h % p.na) * GF_A16_BYTES + (size_t)kb * 16384 + (size_t)r * 128;
            #pragma unroll
            for (int q = 0; q < 8; ++q) {            // word q: weights 8q .. 8q+7 of the k-block, group q / 2
                uint32_t hh[4];
                e2m1x8_to_h2(w[q], hh);
                const uint32_t s2 = sc[q >> 1];
                const uint4 o = make_uint4(hmul2_u(hh[0], s2), hmul2_u(hh[1], s2), hmul2_u(hh[2], s2), hmul2_u(hh[3], s2));
                *reinterpret_cast<uint4*>(dst + ((q ^ (r & 7)) << 4)) = o;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // generic-proxy stores -> the MMA's async-proxy reads
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&a16_full[h]));
        }
    } else if (warp >= 12) {
        // ---- epilogue ----
        const int te = tid - 384, q4 = warp & 3;
        pdl_wait();
        if (te < NT) sx[te] = te < rows ? p.rowscale[m0 + te] / p.gs_w[0] : 0.f;
        named_sync(1, 128);
        mbar_wait_spin(smem_u32(&done_bar), 0, p.status, 29);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tq = tmem + ((uint32_t)(q4 * 32) << 16);
        const int row = rown0 + q4 * 32 + lane;
        #pragma unroll 1
        for (int c0 = 0; c0 < NT; c0 += 16) {
            if (c0 >= rows) break;
            uint32_t d[16];
            asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                         : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]), "=r"(d[4]), "=r"(d[5]), "=r"(d[6]), "=r"(d[7]),
                           "=r"(d[8]), "=r"(d[9]), "=r"(d[10]), "=r"(d[11]), "=r"(d[12]), "=r"(d[13]), "=r"(d[14]), "=r"(d[15])
                         : "r"(tq + (uint32_t)c0));
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (row < p.N) {
                #pragma unroll
                for (int j = 0; j < 16; ++j)
                    if (c0 + j < rows) p.y[(size_t)(m0 + c0 + j) * p.N + row] = __uint_as_float(d[j]) * sx[c0 + j];
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 2) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem), "r"(NT < 32 ? 32 : NT));
}

// One CTA per activation row: x (bf16 when !F32, else f32) -> fp16 row scaled by a power of two so that the
// row's maximum lies in [2^13, 2^14); rowscale[m] = the inverse of that factor (NaN if the row holds an
// infinity or a NaN, so that its outputs become NaN).
template <bool F32>
__global__ void __launch_bounds__(256)
k_act_f16(const void* __restrict__ xin, int K, __half* __restrict__ xh, float* __restrict__ rowscale) {
    __shared__ uint32_t red[8];
    const int row = blockIdx.x, tid = threadIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    auto ld = [&](int i) -> float {
        return F32 ? static_cast<const float*>(xin)[(size_t)row * K + i] : __bfloat162float(static_cast<const __nv_bfloat16*>(xin)[(size_t)row * K + i]);
    };
    uint32_t ai = 0u;
    for (int i = tid; i < K; i += 256) ai = max(ai, __float_as_uint(ld(i)) & 0x7fffffffu);
    #pragma unroll
    for (int o = 16; o; o >>= 1) ai = max(ai, __shfl_xor_sync(0xffffffffu, ai, o));
    if ((tid & 31) == 0) red[tid >> 5] = ai;
    __syncthreads();
    ai = red[0];
    #pragma unroll
    for (int w = 1; w < 8; ++w) ai = max(ai, red[w]);
    const bool bad = ai >= 0x7f800000u;
    int e = (int)(ai >> 23) - 127;                   // floor(log2(amax)) for normal numbers
    if (ai < 0x00800000u) e = -126;
    const float down = __uint_as_float((uint32_t)min(127 + 13 - e, 254) << 23);           // 2^(13 - e)
    const float sc = (ai == 0u || bad) ? 1.f : down;
    if (tid == 0) rowscale[row] = bad ? __uint_as_float(0x7fc00000u) : 1.f / sc;
    for (int i = tid; i < K; i += 256) xh[(size_t)row * K + i] = __float2half_rn(ld(i) * sc);
}

static size_t up256(size_t v) { return (v + 255) / 256 * 256; }

size_t gemm_f16w_ws_bytes(int M, int K) {
    if (M < 1 || K < 256) return 256;
    return up256((size_t)M * K * 2) + up256((size_t)M * 4);
}

template <int NT>
static int gf_launch(GfParams& p, const CUtensorMap& mx, const CUtensorMap& mw, const CUtensorMap& ms, int grid, cudaStream_t s) {
    auto kern = k_gemm_f16w<NT>;
    static int attr_cache[64][2] = {};
    static bool ready[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return launch_failed("gemm_f16w: cudaGetDevice");
    if (dev < 0 || dev >= 64) dev = 0;
    int* ac = attr_cache[dev];
    if (!ac[1]) {
        cudaFuncAttributes fa;
        int oi = 0;
        if (cudaFuncGetAttributes(&fa, kern) != cudaSuccess ||
            cudaDeviceGetAttribute(&oi, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess) return launch_failed("gemm_f16w: attributes");
        ac[0] = oi; ac[1] = (int)fa.sharedSizeBytes + 1;
    }
    const size_t static_smem = (size_t)ac[1] - 1, room = (size_t)ac[0] - static_smem - 2048;
    const int nsup = p.K / 256, nhalf = p.K / 128;
    const size_t b_slot = 2 * (size_t)NT * 128;
    // Shared memory: two fp16 operand buffers and three packed slots, the rest for the activation ring
    // (measured: ring depths beyond these change nothing -- the kernel is bound by the conversion).
    p.na = 2; p.sp = std::min(nsup, 3); p.sb = std::min(nhalf, 8);
    auto need = [&] { return (size_t)p.na * GF_A16_BYTES + (size_t)p.sb * b_slot + (size_t)p.sp * GF_P_BYTES; };
    while (need() > room && p.sb > 2) --p.sb;
    while (need() > room && p.sp > 2) --p.sp;
    if (need() > room) return B200_ENOTIMPL;
    p.na = std::min(p.na, nhalf);
    const size_t smem = need() + 1024;
    if (!ready[dev]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(ac[0] - static_smem)) != cudaSuccess)
            return launch_failed("gemm_f16w: cudaFuncSetAttribute");
        ready[dev] = true;
    }
    cudaLaunchConfig_t lc{};
    lc.gridDim = dim3(grid); lc.blockDim = dim3(GF_THREADS); lc.dynamicSmemBytes = smem; lc.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = at; lc.numAttrs = 1;
    if (cudaLaunchKernelEx(&lc, kern, p, mx, mw, ms) != cudaSuccess) return launch_failed("k_gemm_f16w");
    return check_launch("k_gemm_f16w");
}

// y[M, N] = x[M, K] . W^T with exact products.  x_kind 0: bf16, 1: f32.  ws: gemm_f16w_ws_bytes(M, K).
int gemm_f16w_dense(float* y, const b200_wref* W, const void* x, int x_kind, int M, int N, int K, void* ws, cudaStream_t s) {
    if (!y || !W || !W->packed || !W->scale || !W->gscale || !x || !ws || M < 1 || N < 1) return B200_EINVAL;
    if ((K & 255) || K < 256 || K > 16384 || !tmap_available()) return B200_ENOTIMPL;
    if (((uintptr_t)W->packed & 15) || ((uintptr_t)W->scale & 15) || ((uintptr_t)x & 15) || ((uintptr_t)ws & 255)) return B200_ENOTIMPL;
    __half* xh = static_cast<__half*>(ws);
    float* rowscale = reinterpret_cast<float*>(static_cast<char*>(ws) + up256((size_t)M * K * 2));
    // The conversion of a 128-row weight tile costs a CTA 9-12 us of the SFU pipe (cvt.e2m1x2 runs there), so it
    // is shared by as many tokens as one accumulator holds; 64-token tiles were measured slower from 65 rows on.
    const int NT = M <= 64 ? 64 : 128, n_jobs = (M + NT - 1) / NT, tiles_n = (N + 127) / 128;
    GfParams p{};
    p.y = y; p.gs_w = W->gscale; p.rowscale = rowscale; p.status = device_status_ptr();
    if (!p.status) return B200_ENOTIMPL;
    p.M = M; p.N = N; p.K = K; p.n_jobs = n_jobs; p.prefetch_before_wait = stable_weights_option();
    CUtensorMap mx, mw, ms;
    if (!tmap_u8_2d(&mw, W->packed, (size_t)N, (size_t)K / 2, 128, 128, true, true) ||
        !tmap_u8_2d(&ms, W->scale, (size_t)N, (size_t)K / 16, 16, 128, false, true) ||
        !tmap_u8_2d(&mx, xh, (size_t)M, (size_t)K * 2, 128, NT, true, true)) return B200_ENOTIMPL;
    credit(B200_CREDIT_GEMM, (double)n_jobs * N * K * 0.5625);
    {
        cudaLaunchConfig_t lc{};
        lc.gridDim = dim3(M); lc.blockDim = dim3(256); lc.stream = s;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[0].val.programmaticStreamSerializationAllowed = 1;
        lc.attrs = at; lc.numAttrs = 1;
        const cudaError_t e = x_kind ? cudaLaunchKernelEx(&lc, k_act_f16<true>, x, K, xh, rowscale)
                                     : cudaLaunchKernelEx(&lc, k_act_f16<false>, x, K, xh, rowscale);
        if (e != cudaSuccess) return launch_failed("k_act_f16");
        if (int rc = check_launch("k_act_f16")) return rc;
    }
    return NT == 64 ? gf_launch<64>(p, mx, mw, ms, tiles_n * n_jobs, s) : gf_launch<128>(p, mx, mw, ms, tiles_n * n_jobs, s);
}

}  // namespace b200

using namespace b200;

extern "C" size_t b200_nvfp4_gemm_bf16_exact_workspace_bytes(int M, int K) { return gemm_f16w_ws_bytes(M, K); }

extern "C" int b200_nvfp4_gemm_bf16_exact(float* y, const b200_wref* W, const void* x_bf16, int M, int N, int K,
                                          void* ws, b200_stream stream) {
    if (!y || !W || !x_bf16 || !ws || M < 1 || N < 1 || K < 1 || !W->packed) return B200_EINVAL;
    if (K & 15) return B200_ESHAPE;
    if ((uintptr_t)ws & 255) return B200_EALIGN;
    return gemm_f16w_dense(y, W, x_bf16, 0, M, N, K, ws, stream);
}
