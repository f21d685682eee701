// gemv_tma.cu -- NVFP4 gemv, one activation row, as a bulk-copy (TMA) pipeline for sm_100a.
//
// Why a second kernel: a [12288 x 4096] NVFP4 matrix is 28 MB, ~190 KB per SM and ~4.4 us at HBM
// speed; a kernel whose warps fetch their own rows through registers spends longer than that
// ramping up and draining.  Here the grid is ONE CTA per SM that uses at most half of the SM
// (shared memory, registers, threads), each owning a contiguous range of rows.  A producer
// thread asks for the range tile by tile: a tile of 8 rows is two bulk copies (packed bytes,
// scale bytes -- contiguous because rows are) into a ring of shared-memory stages, each guarded
// by a full/empty mbarrier pair (5 x 18 KB at K = 4096).  Eight consumer warps work on a landed
// tile in pairs of rows: four warps per tile, two tiles in progress, the two rows of a warp
// interleaved instruction by instruction so that two warps per scheduler keep the pipes busy.
// The other half of the SM is left for the NEXT kernel of the stream (see "Launch overlap"):
// while this launch computes, its successor is already resident and streaming its weights, so
// HBM never idles between launches.
//
// The activation row lives in REGISTERS: lane l always works on 16-byte chunks l, l+32, ... of
// a row, so it needs the same K/32 activation values for every row; they are staged through
// shared memory once (fp16, power-of-two scaled, same rule as the general kernel) and kept.
//
// Launch overlap: the kernel is launched with programmatic stream serialisation and releases
// its dependents at once, so the next kernel in the stream gets its CTAs resident as soon as
// this one's exit.  It executes griddepcontrol.wait before it touches anything an upstream
// kernel may have written (x, gscale, y).  Weights are model state; with the "weights are
// stable" option the producer starts the weight copies BEFORE that wait, which hides the whole
// ramp behind the previous kernel's tail.  The option is off by default because it is only
// valid if no kernel still running on the stream writes those weight buffers.
//
// A row's arithmetic (chunk order per lane, group_dot, xor-shuffle tree, final scaling) is the
// same sequence the general kernel executes, so both produce identical bits and the reference's
// "gemv == gemm row == fused group" invariants hold across the two kernels.
#include "b200_internal.h"
#include "gemv_core.cuh"
#include "tma_pipe.cuh"
#include <cstdlib>

namespace b200 {

constexpr int GT_WARPS = 8;                        // consumer warps = rows per tile
constexpr int GT_THREADS = (GT_WARPS + 1) * 32;    // + one producer warp
constexpr int GT_MAX_STAGES = 16;

struct TmaCfg {
    int total_rows, stages, prefetch_before_wait;
    uint32_t stage_bytes, packed_bytes;            // per stage; scales start at packed_bytes
    unsigned int* status;
    unsigned long long* trace;                     // B200_TRACE builds only: 32 timestamps per CTA
};

#ifdef B200_TRACE
__device__ __forceinline__ unsigned long long gtime() { unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t; }
#define TRACE(cfg, slot) do { if ((cfg).trace && (threadIdx.x & 31) == 0 && (threadIdx.x == 0 || threadIdx.x == GT_WARPS * 32) && (slot) < 32) (cfg).trace[blockIdx.x * 32 + (slot)] = gtime(); } while (0)
#else
#define TRACE(cfg, slot) do { } while (0)
#endif

// Row range of CTA c and the walk over its tiles.  Producer and consumers run the same walk.
struct TileWalk {
    int r, end, job, job_start;
    __device__ TileWalk(int total, int cta, int ncta) {
        r = (int)(((long long)total * cta) / ncta);
        end = (int)(((long long)total * (cta + 1)) / ncta);
        job = 0; job_start = 0;
    }
    // Next tile: job index, first row inside the job, row count (<= GT_WARPS).  False at the end.
    __device__ bool next(const GemvParams& p, int& j, int& row0, int& n) {
        if (r >= end) return false;
        while (r >= job_start + p.j[job].N) { job_start += p.j[job].N; ++job; }
        j = job; row0 = r - job_start;
        n = min(GT_WARPS, min(end - r, p.j[job].N - row0));
        r += n;
        return true;
    }
};

struct Producer {
    TileWalk w; int t;
    __device__ Producer(int total, int cta, int ncta) : w(total, cta, ncta), t(0) {}
    // Issues tiles until `limit` tiles are out (or the range ends).  Returns false at the end.
    __device__ bool issue(const GemvParams& p, const TmaCfg& cfg, unsigned char* ring, uint64_t* full_bar,
                          uint64_t* empty_bar, int limit) {
        const int K = p.K;
        int j, row0, n;
        while (t < limit) {
            if (!w.next(p, j, row0, n)) return false;
            const int s = t % cfg.stages;
            if (t >= cfg.stages) mbar_wait(smem_u32(&empty_bar[s]), ((t / cfg.stages) - 1) & 1, cfg.status, 1);
            const uint32_t pb = (uint32_t)n * (K >> 1), sb = (uint32_t)n * (K >> 4);
            const uint32_t bar = smem_u32(&full_bar[s]);
            const uint32_t dst = smem_u32(ring + (size_t)s * cfg.stage_bytes);
            mbar_expect_tx(bar, pb + sb);
            bulk_g2s(dst, p.j[j].P + (size_t)row0 * (K >> 1), pb, bar);
            bulk_g2s(dst + cfg.packed_bytes, p.j[j].S + (size_t)row0 * (K >> 4), sb, bar);
            ++t;
            TRACE(cfg, 17 + t);
        }
        return true;
    }
};

template <int NJ, int MATH>
__global__ void __launch_bounds__(GT_THREADS, 2)
k_gemv_tma(const __grid_constant__ GemvParams p, const __grid_constant__ TmaCfg cfg) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ uint64_t full_bar[GT_MAX_STAGES], empty_bar[GT_MAX_STAGES];
    __shared__ float inv_s[1];
    __shared__ float inv_gs[B200_GEMV_MULTI_MAX];
    __shared__ float red[GT_WARPS];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int K = p.K, nch = K >> 5;
    uint4* xs = reinterpret_cast<uint4*>(smem);                      // staged activation row
    unsigned char* ring = smem + (size_t)xs_chunks(K) * 16;

    TRACE(cfg, tid == 0 ? 0 : 16);
    pdl_launch_dependents();                        // the next kernel may start taking free SM slots

    if (warp == GT_WARPS) {
        // ---- producer: barriers, then the first ring-full of tiles, then refills ----
        Producer pr(cfg.total_rows, blockIdx.x, gridDim.x);
        bool more = true;
        if (lane == 0) {
            for (int s = 0; s < cfg.stages; ++s) { mbar_init(smem_u32(&full_bar[s]), 1); mbar_init(smem_u32(&empty_bar[s]), GT_WARPS / 2); }
            mbar_fence_init();
            TRACE(cfg, 17);
            if (!cfg.prefetch_before_wait) pdl_wait();
            more = pr.issue(p, cfg, ring, full_bar, empty_bar, cfg.stages);
        }
        __syncthreads();                            // publishes the barrier initialisation
        if (lane == 0 && more) pr.issue(p, cfg, ring, full_bar, empty_bar, 0x7fffffff);
        return;
    }

    // ---- consumers ----
    pdl_wait();                                     // x, gscale, y belong to upstream kernels until here
    TRACE(cfg, 1);
    {
        // One pass over x: each thread keeps its values in registers across the amax reduction
        // (a second trip to global memory would cost another full memory latency here).
        const float* x = p.j[0].x;
        if (tid < p.n_jobs) inv_gs[tid] = 1.f / p.j[tid].gs[0];
        constexpr int XV = (NJ * 128 + GT_WARPS * 32 - 1) / (GT_WARPS * 32);   // 8-float units per thread
        float4 xu[XV][2];
        float a = 0.f;
        #pragma unroll
        for (int q = 0; q < XV; ++q) {
            const int i = tid + q * GT_WARPS * 32;
            if (i < (K >> 3)) {
                xu[q][0] = reinterpret_cast<const float4*>(x)[2 * i];
                xu[q][1] = reinterpret_cast<const float4*>(x)[2 * i + 1];
            } else { xu[q][0] = make_float4(0.f, 0.f, 0.f, 0.f); xu[q][1] = xu[q][0]; }
            const float4 u = xu[q][0], v = xu[q][1];
            a = fmaxf(a, fmaxf(fmaxf(fabsf(u.x), fabsf(u.y)), fmaxf(fabsf(u.z), fabsf(u.w))));
            a = fmaxf(a, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
        }
        a = warp_max(a);
        if (lane == 0) red[warp] = a;
        named_sync(1, GT_WARPS * 32);
        a = 0.f;
        #pragma unroll
        for (int w = 0; w < GT_WARPS; ++w) a = fmaxf(a, red[w]);
        const float sc = row_pow2_scale(a);
        if (tid == 0) inv_s[0] = 1.f / sc;
        #pragma unroll
        for (int q = 0; q < XV; ++q) {
            const int i = tid + q * GT_WARPS * 32;
            if (i < (K >> 3)) {
                const float4 u = xu[q][0], v = xu[q][1];
                uint4 o; __half2 h;
                h = __floats2half2_rn(u.x * sc, u.y * sc); o.x = *reinterpret_cast<uint32_t*>(&h);
                h = __floats2half2_rn(u.z * sc, u.w * sc); o.y = *reinterpret_cast<uint32_t*>(&h);
                h = __floats2half2_rn(v.x * sc, v.y * sc); o.z = *reinterpret_cast<uint32_t*>(&h);
                h = __floats2half2_rn(v.z * sc, v.w * sc); o.w = *reinterpret_cast<uint32_t*>(&h);
                xs[xs_swz(i)] = o;
            }
        }
    }
    __syncthreads();                                // staged x visible; barriers initialised
    uint32_t xr[NJ][16];
    #pragma unroll
    for (int jj = 0; jj < NJ; ++jj) {
        const int c = lane + 32 * jj;
        #pragma unroll
        for (int q = 0; q < 4; ++q) {
            uint4 v = make_uint4(0, 0, 0, 0);
            if (c < nch) v = xs[xs_swz(4 * c + q)];
            xr[jj][4 * q] = v.x; xr[jj][4 * q + 1] = v.y; xr[jj][4 * q + 2] = v.z; xr[jj][4 * q + 3] = v.w;
        }
    }
    const float xinv = inv_s[0];
    TRACE(cfg, 2);

    // Warp w works on tiles t with t % 2 == w / 4, rows 2*(w%4) and 2*(w%4)+1 of the tile.
    const int half = warp >> 2, r0 = (warp & 3) * 2;
    TileWalk w(cfg.total_rows, blockIdx.x, gridDim.x);
    int j, row0, n, t = 0;
    while (w.next(p, j, row0, n)) {
        if ((t & 1) == half) {
            const int s = t % cfg.stages;
            mbar_wait(smem_u32(&full_bar[s]), (t / cfg.stages) & 1, cfg.status, 2);
            if (r0 < n) {
                const unsigned char* st = ring + (size_t)s * cfg.stage_bytes;
                const uint4* wa = reinterpret_cast<const uint4*>(st + (size_t)r0 * (K >> 1));
                const uint4* wb = reinterpret_cast<const uint4*>(st + (size_t)(r0 + 1) * (K >> 1));
                const uint16_t* sa = reinterpret_cast<const uint16_t*>(st + cfg.packed_bytes + (size_t)r0 * (K >> 4));
                const uint16_t* sb = reinterpret_cast<const uint16_t*>(st + cfg.packed_bytes + (size_t)(r0 + 1) * (K >> 4));
                float acc0 = 0.f, acc1 = 0.f;
                #pragma unroll
                for (int jj = 0; jj < NJ; ++jj) {
                    const int c = lane + 32 * jj;
                    if (c < nch) {
                        const uint4 va = wa[c], vb = wb[c];
                        const uint32_t s2a = e4m3x2_to_h2(sa[c]), s2b = e4m3x2_to_h2(sb[c]);
                        acc0 = group_dot<MATH>(acc0, va.x, va.y, xr[jj], (uint16_t)(s2a & 0xffffu));
                        acc1 = group_dot<MATH>(acc1, vb.x, vb.y, xr[jj], (uint16_t)(s2b & 0xffffu));
                        acc0 = group_dot<MATH>(acc0, va.z, va.w, xr[jj] + 8, (uint16_t)(s2a >> 16));
                        acc1 = group_dot<MATH>(acc1, vb.z, vb.w, xr[jj] + 8, (uint16_t)(s2b >> 16));
                    }
                }
                #pragma unroll
                for (int o = 16; o; o >>= 1) {
                    acc0 += __shfl_xor_sync(0xffffffffu, acc0, o);
                    acc1 += __shfl_xor_sync(0xffffffffu, acc1, o);
                }
                if (lane == 0) {
                    const float k = inv_gs[j];
                    p.j[j].y[row0 + r0] = acc0 * xinv * k;
                    if (r0 + 1 < n) p.j[j].y[row0 + r0 + 1] = acc1 * xinv * k;
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&empty_bar[s]));
            TRACE(cfg, 3 + t < 15 ? 3 + t : 14);
        }
        ++t;
    }
    TRACE(cfg, 15);
}

#ifdef B200_TRACE
unsigned long long* g_trace = nullptr;
#endif

// Opt in to the largest dynamic shared-memory size the device allows for this kernel
// (the per-block opt-in limit minus the kernel's static shared memory), once.
template <typename Kern>
static int allow_big_smem(Kern kern, size_t need) {
    cudaFuncAttributes fa;
    int dev = 0, optin = 0;
    if (cudaFuncGetAttributes(&fa, kern) != cudaSuccess || cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess)
        return launch_failed("gemv_tma: attribute query");
    const size_t room = (size_t)optin - fa.sharedSizeBytes;
    if (need > room) return B200_ENOTIMPL;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)room) != cudaSuccess)
        return launch_failed("gemv_tma: cudaFuncSetAttribute");
    return B200_OK;
}

template <int NJ, int MATH>
static int launch_tma_math(const GemvParams& p, const TmaCfg& cfg, size_t smem, int grid, cudaStream_t s) {
    static bool ready_all[64] = {};                 // the attribute is per device
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    if (!ready_all[dev]) {
        if (int rc = allow_big_smem(k_gemv_tma<NJ, MATH>, smem)) return rc;
        ready_all[dev] = true;
    }
    cudaLaunchConfig_t lc{};
    lc.gridDim = dim3(grid); lc.blockDim = dim3(GT_THREADS); lc.dynamicSmemBytes = smem; lc.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = at; lc.numAttrs = 1;
    if (cudaLaunchKernelEx(&lc, k_gemv_tma<NJ, MATH>, p, cfg) != cudaSuccess) return launch_failed("k_gemv_tma");
    return check_launch("k_gemv_tma");
}

template <int NJ>
static int launch_tma(const GemvParams& p, const TmaCfg& cfg, size_t smem, int grid, cudaStream_t s) {
    return nvfp4_math_mode() ? launch_tma_math<NJ, 1>(p, cfg, smem, grid, s)
                             : launch_tma_math<NJ, 0>(p, cfg, smem, grid, s);
}

// Conditions: one activation row shared by every job; K a multiple of 256 (so that a tile's
// scale bytes are a 16-byte multiple) and at most 4096 (activation registers); packed and scale
// tensors 16-byte aligned; activation 16-byte aligned.
int nvfp4_multi_tma(const GemvParams& p, cudaStream_t s) {
    const int K = p.K;
    if ((K & 255) || K > 4096) return B200_ENOTIMPL;
    int total = 0;
    for (int i = 0; i < p.n_jobs; ++i) {
        const GemvJobDev& j = p.j[i];
        if (j.x != p.j[0].x) return B200_ENOTIMPL;
        if (((uintptr_t)j.P & 15) || ((uintptr_t)j.S & 15)) return B200_ENOTIMPL;
        total += j.N;
    }
    if (((uintptr_t)p.j[0].x & 15) || total < GT_WARPS * 16) return B200_ENOTIMPL;
    TmaCfg cfg{};
    cfg.total_rows = total;
    cfg.packed_bytes = (uint32_t)GT_WARPS * (K >> 1);
    cfg.stage_bytes = cfg.packed_bytes + (uint32_t)GT_WARPS * (K >> 4);
    const size_t xbytes = (size_t)xs_chunks(K) * 16;
    // two CTAs per SM: each gets half of the SM's shared memory minus static and reserved parts
    const size_t budget = (size_t)(227 * 1024) / 2 - 2048 - xbytes;
    const int grid = std::min(sm_count(), (total + GT_WARPS - 1) / GT_WARPS);
    const int tiles_per_cta = ((total + grid - 1) / grid + GT_WARPS - 1) / GT_WARPS + 1;
    cfg.stages = (int)std::min<size_t>(std::min(GT_MAX_STAGES, tiles_per_cta), budget / cfg.stage_bytes);
    if (cfg.stages < 2) return B200_ENOTIMPL;
    cfg.status = device_status_ptr();
    if (!cfg.status) return B200_ENOTIMPL;
    cfg.prefetch_before_wait = stable_weights_option();
    cfg.trace = nullptr;
#ifdef B200_TRACE
    { static unsigned long long* tb = nullptr; if (!tb) cudaMalloc(&tb, 1024 * 32 * 8); cfg.trace = tb; g_trace = tb; }
#endif
    const size_t smem = xbytes + (size_t)cfg.stages * cfg.stage_bytes;
    const int nch = K >> 5, nj = (nch + 31) / 32;
    switch (nj) {
        case 1: return launch_tma<1>(p, cfg, smem, grid, s);
        case 2: return launch_tma<2>(p, cfg, smem, grid, s);
        case 3: return launch_tma<3>(p, cfg, smem, grid, s);
        default: return launch_tma<4>(p, cfg, smem, grid, s);
    }
}

}  // namespace b200

#ifdef B200_TRACE
extern "C" int b200_debug_trace(unsigned long long* host_out, int n_cta) {
    if (!b200::g_trace) return 1;
    return cudaMemcpy(host_out, b200::g_trace, (size_t)n_cta * 32 * 8, cudaMemcpyDeviceToHost) != cudaSuccess;
}
#endif
