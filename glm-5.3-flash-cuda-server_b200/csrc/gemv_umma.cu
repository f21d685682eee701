// gemv_umma.cu -- NVFP4 gemv (one activation row) on the 5th-generation tensor cores:
// tcgen05.mma kind::mxf4nvf4 (block-16, UE4M3 scales), TMEM accumulators, TMA tile loads.
//
// Why tensor cores for a matrix-VECTOR product: the CUDA-core formulation is capped by the
// conversion pipe (cvt.rn.f16x2.e2m1x2 issues once per ~3 cycles per scheduler: 24e12 weights/s
// chip-wide against the 11.6e12 that 6.5 TB/s of HBM delivers, before a single load, barrier or
// reduction).  tcgen05.mma reads the packed e2m1 bytes and the e4m3 scale bytes exactly as the
// format stores them, so the SM does no decode work at all and the kernel is a pure stream.
//
// How fp32-activation accuracy is kept although both MMA operands are FP4: the activation row is
// written as EIGHT FP4 columns.  Per 16-group g, x = gamma * s_g * v with s_g an e4m3 scale
// (rounded up so |v| < 4) and v rounded to 16 fractional bits: v = sign * sum_t d_t 4^-t with
// base-4 digits d_t in {0,1,2,3}, all of which e2m1 represents exactly.  Column t of the B
// operand holds the digits d_t (same block scales s_g for every column); the MMA's N = 8 columns
// come for free, and the epilogue adds the columns as y = (sum_t gamma 4^-t D[:,t]) / gscale.
// Rounding error per activation <= 2^-17 of 4 s_g, i.e. < 1e-5 of the group's amax -- thirty
// times finer than fp16 staging -- and products and sums inside the MMA are exact / fp32.
//
// Per CTA (one per SM): rows [r0, r0+R) of one job, R <= 128 a multiple of 8.
//   warp 0      TMA producer: per 256-k stage one box [128 B x R rows] of packed weights
//               (SWIZZLE_128B, K-major UMMA operand layout) and one box [16 B x R rows] of scales
//   warps 2-5   split the activation row into the B image (once), then per stage rearrange the
//               R x 16 scale bytes into the four 512-byte scale atoms tcgen05.cp expects, and at
//               the end read the accumulators (tcgen05.ld) and write y
//   warp 1      TMEM allocation; one thread issues, per stage, 8 tcgen05.cp (scales -> TMEM) and
//               4 tcgen05.mma (K = 64 each), then tcgen05.commit frees the stage
// Every mbarrier wait is bounded (tma_pipe.cuh).  No cluster launch, no multicast.
#include "b200_internal.h"
#include "nvfp4_decode.cuh"
#include "tma_pipe.cuh"
#include <cuda.h>
#include <cstdio>
#include <cstdlib>

namespace b200 {

constexpr int UM_THREADS = 192;                    // 6 warps
constexpr int UM_NB = 8;                           // MMA N = digits per activation
constexpr int UM_MAX_STAGES = 14;
constexpr int UM_TMEM_COLS = 128;                  // D [0,8) | SFA slots [32,64) | SFB slots [64,96)

struct UmJob { float* y; const float* gs; int N; int task0; };
struct UmParams {
    UmJob j[B200_GEMV_MULTI_MAX];
    const float* x;
    unsigned int* status;
    int n_jobs, K, R, stages, prefetch_before_wait;
    uint32_t stage_bytes, a_bytes;                 // per stage: A tile | raw scales | 4 scale atoms
};
struct UmMaps { CUtensorMap w[B200_GEMV_MULTI_MAX]; CUtensorMap s[B200_GEMV_MULTI_MAX]; };

__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr, uint32_t sbo_bytes, uint32_t layout) {
    // start address >> 4 | LBO (unused here) | SBO >> 4 | version 1 | layout type (2 = SWIZZLE_128B, 0 = none)
    return (uint64_t)((saddr >> 4) & 0x3FFF) | ((uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)(layout & 7) << 61);
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 :: "r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(bar) : "memory");
}

// e4m3 code (0..126) of the smallest representable value >= v (v >= 0); 126 (448) if v is larger.
__device__ __forceinline__ uint32_t e4m3_ceil_code(float v) {
    uint16_t two;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(two) : "f"(0.f), "f"(v));     // low byte <- v
    uint32_t c = two & 0xFFu;
    if (e4m3_to_f32(c) < v && c < 126u) ++c;
    return c;
}

__global__ void __launch_bounds__(UM_THREADS, 1)
k_gemv_umma(const __grid_constant__ UmParams p, const __grid_constant__ UmMaps maps) {
    extern __shared__ __align__(1024) unsigned char smem[];
    __shared__ uint64_t full_bar[UM_MAX_STAGES], sf_bar[UM_MAX_STAGES], empty_bar[UM_MAX_STAGES], done_bar;
    __shared__ uint32_t tmem_base_s;
    __shared__ float gam[UM_NB], red[8];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int K = p.K, nst = (K + 255) >> 8;       // 256-k stages along K
    // which job / rows
    int ji = 0;
    #pragma unroll
    for (int q = 1; q < B200_GEMV_MULTI_MAX; ++q) if (q < p.n_jobs && (int)blockIdx.x >= p.j[q].task0) ji = q;
    const UmJob J = p.j[ji];
    const int row0 = ((int)blockIdx.x - J.task0) * p.R;
    const int valid = min(p.R, J.N - row0);
    unsigned char* ring = smem + ((1024u - (smem_u32(smem) & 1023u)) & 1023u);      // SWIZZLE_128B tiles need 1 KB alignment
    unsigned char* bimg = ring + (size_t)p.stages * p.stage_bytes;          // nst tiles of 1 KB
    unsigned char* sfb = bimg + (size_t)nst * 1024;                          // K/64 atoms at 128 B stride (+384 tail)

    pdl_launch_dependents();
    if (tid == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1); mbar_init(smem_u32(&sf_bar[s]), 128); mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        mbar_init(smem_u32(&done_bar), 1);
        mbar_fence_init();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_u32(&tmem_base_s)), "r"(UM_TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_base_s;

    if (warp == 0) {
        // ---- TMA producer ----
        if (lane == 0) {
            if (!p.prefetch_before_wait) pdl_wait();
            const uint32_t bytes = (uint32_t)p.R * 128u + (uint32_t)p.R * 16u;
            for (int it = 0; it < nst; ++it) {
                const int s = it % p.stages;
                if (it >= p.stages) mbar_wait(smem_u32(&empty_bar[s]), ((it / p.stages) - 1) & 1, p.status, 1);
                const uint32_t bar = smem_u32(&full_bar[s]);
                const uint32_t dst = smem_u32(ring + (size_t)s * p.stage_bytes);
                mbar_expect_tx(bar, bytes);
                tma_load_2d(dst, &maps.w[ji], it * 128, row0, bar);
                tma_load_2d(dst + p.a_bytes, &maps.s[ji], it * 16, row0, bar);
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer ----
        pdl_wait();
        named_sync(2, 160);                          // B image, scale atoms of x and gam[] are ready
        if (lane == 0) {
            const uint32_t idesc = (1u << 7) | (1u << 10) | ((uint32_t)(UM_NB >> 3) << 17) | ((128u >> 4) << 24);
            for (int it = 0; it < nst; ++it) {
                const int s = it % p.stages, slot = it & 1;
                mbar_wait(smem_u32(&sf_bar[s]), (it / p.stages) & 1, p.status, 3);
                tc_fence_after();
                const uint32_t st = smem_u32(ring + (size_t)s * p.stage_bytes);
                const int nkb = min(4, (K - it * 256) >> 6);
                for (int kb = 0; kb < nkb; ++kb) {
                    const uint64_t da = umma_desc(st + p.a_bytes + (uint32_t)p.R * 16u + kb * 512, 128, 0);
                    const uint64_t db = umma_desc(smem_u32(sfb) + (it * 4 + kb) * 128, 128, 0);
                    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" :: "r"(tmem + 32 + slot * 16 + kb * 4), "l"(da));
                    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" :: "r"(tmem + 64 + slot * 16 + kb * 4), "l"(db));
                }
                for (int kb = 0; kb < nkb; ++kb) {
                    const uint64_t da = umma_desc(st + kb * 32, 1024, 2);
                    const uint64_t db = umma_desc(smem_u32(bimg) + it * 1024 + kb * 32, 1024, 2);
                    const uint32_t acc = (it | kb) != 0;
                    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                                 " tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n}"
                                 :: "r"(tmem), "l"(da), "l"(db), "r"(idesc), "r"(acc),
                                    "r"(tmem + 32 + slot * 16 + kb * 4), "r"(tmem + 64 + slot * 16 + kb * 4) : "memory");
                }
                tc_commit(smem_u32(&empty_bar[s]));
            }
            tc_commit(smem_u32(&done_bar));
        }
    } else {
        // ---- warps 2..5: activation split, per-stage scale rearrangement, epilogue ----
        const int t4 = tid - 64;                     // 0..127
        pdl_wait();
        const float* x = p.x;
        // global amax of x
        float a = 0.f;
        for (int i = t4; i < (K >> 2); i += 128) {
            const float4 v = reinterpret_cast<const float4*>(x)[i];
            a = fmaxf(a, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
        }
        a = warp_max(a);
        if (lane == 0) red[warp - 2] = a;
        named_sync(1, 128);
        a = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
        // gamma: x = gamma * s_g * v with s_g <= 448 and |v| < 4
        const float gamma = (a > 0.f && a < 3.0e38f) ? a * (1.0f / (448.f * 3.99f)) : 1.f;
        if (t4 < UM_NB) gam[t4] = gamma * __uint_as_float((uint32_t)(127 - 2 * t4) << 23);      // gamma * 4^-t
        for (int i = t4; i < 384; i += 128) sfb[(size_t)(K >> 6) * 128 + i] = 0;                  // tail the last atom reads
        for (int g = t4; g < (K >> 4); g += 128) {
            float v[16];
            #pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float4 f = reinterpret_cast<const float4*>(x)[g * 4 + q];
                v[4 * q] = f.x; v[4 * q + 1] = f.y; v[4 * q + 2] = f.z; v[4 * q + 3] = f.w;
            }
            float am = 0.f;
            #pragma unroll
            for (int q = 0; q < 16; ++q) am = fmaxf(am, fabsf(v[q]));
            const uint32_t code = e4m3_ceil_code(am / (gamma * 3.99f));
            const float sdec = e4m3_to_f32(code);
            const float inv = sdec > 0.f ? 16384.f / (gamma * sdec) : 0.f;
            uint32_t lo[UM_NB], hi[UM_NB];
            #pragma unroll
            for (int t = 0; t < UM_NB; ++t) { lo[t] = 0; hi[t] = 0; }
            #pragma unroll
            for (int q = 0; q < 16; ++q) {
                int iq = __float2int_rn(v[q] * inv);
                const uint32_t sgn = iq < 0 ? 8u : 0u;
                uint32_t m = (uint32_t)min(abs(iq), 65535);
                #pragma unroll
                for (int t = 0; t < UM_NB; ++t) {
                    const uint32_t d = (m >> (2 * (UM_NB - 1 - t))) & 3u;       // digit of weight 4^-t
                    const uint32_t c = d ? ((d << 1) - (d == 3u) + sgn) : 0u;     // e2m1 code of +-d: 1->2, 2->4, 3->5
                    if (q < 8) lo[t] |= c << (4 * q); else hi[t] |= c << (4 * (q - 8));
                }
            }
            // B image: tile (256 k) = g / 16, row t, 16-byte chunk (g % 16) / 2 swizzled with the row, half g % 2
            const int tile = g >> 4, ch = (g & 15) >> 1, hf = g & 1;
            #pragma unroll
            for (int t = 0; t < UM_NB; ++t)
                *reinterpret_cast<uint2*>(bimg + tile * 1024 + t * 128 + ((ch ^ t) << 4) + hf * 8) = make_uint2(lo[t], hi[t]);
            // scale atoms of x: K-block g / 4, scale index g % 4, same byte for all 8 columns
            #pragma unroll
            for (int n = 0; n < UM_NB; ++n) sfb[(size_t)(g >> 2) * 128 + n * 16 + (g & 3)] = (uint8_t)code;
        }
        fence_async_smem();
        named_sync(2, 160);                          // with the MMA warp
        // per stage: row r's 16 scale bytes -> 4 atoms
        for (int it = 0; it < nst; ++it) {
            const int s = it % p.stages;
            mbar_wait(smem_u32(&full_bar[s]), (it / p.stages) & 1, p.status, 2);
            unsigned char* st = ring + (size_t)s * p.stage_bytes + p.a_bytes;
            if (t4 < p.R) {
                const uint4 v = *reinterpret_cast<const uint4*>(st + t4 * 16);
                unsigned char* at = st + (size_t)p.R * 16 + (t4 & 31) * 16 + (t4 >> 5) * 4;
                *reinterpret_cast<uint32_t*>(at) = v.x;
                *reinterpret_cast<uint32_t*>(at + 512) = v.y;
                *reinterpret_cast<uint32_t*>(at + 1024) = v.z;
                *reinterpret_cast<uint32_t*>(at + 1536) = v.w;
            }
            fence_async_smem();
            mbar_arrive(smem_u32(&sf_bar[s]));
        }
        // epilogue
        mbar_wait(smem_u32(&done_bar), 0, p.status, 4);
        tc_fence_after();
        uint32_t d[8];
        const int q4 = warp & 3;                     // TMEM lane quadrant this warp may read
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                     : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]), "=r"(d[4]), "=r"(d[5]), "=r"(d[6]), "=r"(d[7])
                     : "r"(tmem + ((uint32_t)(q4 * 32) << 16)));
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        const int r = q4 * 32 + lane;
        if (r < valid) {
            float acc = 0.f;
            #pragma unroll
            for (int t = UM_NB - 1; t >= 0; --t) acc = fmaf(__uint_as_float(d[t]), gam[t], acc);     // small terms first
            J.y[row0 + r] = acc / J.gs[0];
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem), "r"(UM_TMEM_COLS));
}

// ---- host side ---------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) p = nullptr;
        return (EncodeTiledFn)p;
    }();
    return fn;
}
// u8 matrix [rows, row_bytes]; box [box_bytes x box_rows].
static bool make_map(CUtensorMap* m, const void* base, int rows, size_t row_bytes, int box_bytes, int box_rows, bool swz) {
    const cuuint64_t dims[2] = {(cuuint64_t)row_bytes, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
    const cuuint32_t box[2] = {(cuuint32_t)box_bytes, (cuuint32_t)box_rows};
    const cuuint32_t es[2] = {1, 1};
    return encode_fn()(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, es,
                       CU_TENSOR_MAP_INTERLEAVE_NONE, swz ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                       CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Conditions: M = 1, one activation row shared by all jobs, K % 64 == 0 and K <= 16384, 16-byte
// aligned tensors and activation, K/16 a multiple of 16 (scale row pitch for TMA).
int nvfp4_multi_umma(const GemvParams& g, cudaStream_t s) {
    const int K = g.K;
    if ((K & 255) || K > 16384 || !encode_fn()) return B200_ENOTIMPL;
    int total = 0;
    for (int i = 0; i < g.n_jobs; ++i) {
        if (g.j[i].x != g.j[0].x || ((uintptr_t)g.j[i].P & 15) || ((uintptr_t)g.j[i].S & 15)) return B200_ENOTIMPL;
        total += g.j[i].N;
    }
    if (((uintptr_t)g.j[0].x & 15) || total < 256) return B200_ENOTIMPL;
    const int nsm = sm_count();
    int R = 128;
    for (int r = 8; r <= 128; r += 8) {
        int tasks = 0;
        for (int i = 0; i < g.n_jobs; ++i) tasks += (g.j[i].N + r - 1) / r;
        if (tasks <= nsm) { R = r; break; }
    }
    static UmMaps maps;                              // one host thread at a time calls in
    UmParams p{};
    p.x = g.j[0].x; p.n_jobs = g.n_jobs; p.K = K; p.R = R;
    int tasks = 0;
    for (int i = 0; i < g.n_jobs; ++i) {
        p.j[i] = UmJob{g.j[i].y, g.j[i].gs, g.j[i].N, tasks};
        tasks += (g.j[i].N + R - 1) / R;
        if (!make_map(&maps.w[i], g.j[i].P, g.j[i].N, (size_t)K / 2, 128, R, true) ||
            !make_map(&maps.s[i], g.j[i].S, g.j[i].N, (size_t)K / 16, 16, R, false)) return B200_ENOTIMPL;
    }
    for (int i = g.n_jobs; i < B200_GEMV_MULTI_MAX; ++i) { p.j[i] = p.j[0]; p.j[i].task0 = 0x7fffffff; maps.w[i] = maps.w[0]; maps.s[i] = maps.s[0]; }
    p.a_bytes = (uint32_t)R * 128u;
    p.stage_bytes = ((p.a_bytes + (uint32_t)R * 16u + 2048u) + 1023u) & ~1023u;
    const int nst = K / 256;
    const size_t fixed = (size_t)nst * 1024 + (size_t)(K / 64) * 128 + 384;
    cudaFuncAttributes fa;
    int dev = 0, optin = 0;
    if (cudaFuncGetAttributes(&fa, k_gemv_umma) != cudaSuccess || cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess) return launch_failed("gemv_umma: attributes");
    const size_t room = (size_t)optin - fa.sharedSizeBytes - 1024;        // 1 KB: alignment of the dynamic part
    if (fixed + 2 * (size_t)p.stage_bytes > room) return B200_ENOTIMPL;
    p.stages = (int)std::min<size_t>(std::min(UM_MAX_STAGES, nst), (room - fixed) / p.stage_bytes);
    p.status = device_status_ptr();
    if (!p.status) return B200_ENOTIMPL;
    p.prefetch_before_wait = stable_weights_option();
    const size_t smem = (size_t)p.stages * p.stage_bytes + fixed + 1024;
    static bool ready = false;
    if (!ready) {
        if (cudaFuncSetAttribute(k_gemv_umma, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(room + 1024)) != cudaSuccess)
            return launch_failed("gemv_umma: cudaFuncSetAttribute");
        ready = true;
    }
    cudaLaunchConfig_t lc{};
    lc.gridDim = dim3(tasks); lc.blockDim = dim3(UM_THREADS); lc.dynamicSmemBytes = smem; lc.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = at; lc.numAttrs = 1;
    if (cudaLaunchKernelEx(&lc, k_gemv_umma, p, maps) != cudaSuccess) return launch_failed("k_gemv_umma");
    return check_launch("k_gemv_umma");
}

}  // namespace b200
