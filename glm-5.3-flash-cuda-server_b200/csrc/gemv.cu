// gemv.cu -- NVFP4 / bf16 / f32 matrix-vector and skinny (M <= 8) matrix-matrix products for
// sm_100a, CUDA-core path.  Replaces the reference's kernels/gemv.cu (gemv :456-465, gemm
// :369-396 and :649-701, gemv_multi :404-435, converters :470-488).
//
// Shape of the NVFP4 kernel (k_gemv_nvfp4):
//   * a block stages the activation rows once in shared memory as fp16 (power-of-two scaled,
//     bank-swizzled), then its 8 warps each own R consecutive weight rows;
//   * a lane reads one 16-byte packed chunk (32 weights = two 16-groups) and the matching two
//     e4m3 scale bytes per row per step, with the next step's loads issued before the current
//     step's arithmetic, so 2*R*16 B per lane are always in flight;
//   * arithmetic is packed fp16 chains folded into fp32 accumulators (see nvfp4_decode.cuh);
//   * one launch serves up to 8 independent jobs that share K and M: the jobs' row tiles form
//     one flat task list that the grid strides over, so a 32-row sibling does not cost a launch
//     or an almost-empty block row.
// Results do not depend on the grid size, on M, or on which job list a matrix came in with: a
// row's accumulation order is fixed by (K, lane), nothing else.
#include "b200_internal.h"
#include "gemv_core.cuh"
#include <cstdio>
#include <cstdlib>

namespace b200 {

template <int M, int R, int MATH>
__global__ void __launch_bounds__(GEMV_THREADS)
k_gemv_nvfp4(const __grid_constant__ GemvParams p) {
    extern __shared__ uint4 xs[];
    __shared__ float inv_s[M];
    __shared__ float red[M * GEMV_WARPS];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int K = p.K;
    const float* staged = nullptr;
    for (int task = blockIdx.x; task < p.total_tasks; task += gridDim.x) {
        int ji = 0;
        #pragma unroll
        for (int q = 1; q < B200_GEMV_MULTI_MAX; ++q) if (q < p.n_jobs && task >= p.j[q].task0) ji = q;
        const GemvJobDev& J = p.j[ji];
        if (J.x != staged) {
            if (staged) __syncthreads();           // nobody may still be reading the old rows
            stage_x(J.x, M, K, xs, inv_s, red);
            staged = J.x;
        }
        const int row0 = (task - J.task0) * (GEMV_WARPS * R) + warp * R;
        if (row0 >= J.N) continue;
        RowPtr rows[R];
        #pragma unroll
        for (int r = 0; r < R; ++r) {
            const int n = min(row0 + r, J.N - 1);  // a short last tile re-reads its last row
            rows[r].p = J.P + (size_t)n * (K >> 1);
            rows[r].s = J.S + (size_t)n * (K >> 4);
        }
        float acc[R][M];
        #pragma unroll
        for (int r = 0; r < R; ++r)
            #pragma unroll
            for (int m = 0; m < M; ++m) acc[r][m] = 0.f;
        warp_rows<M, R, MATH>(rows, K, xs, acc, lane);
        const float ig = 1.f / J.gs[0];
        #pragma unroll
        for (int r = 0; r < R; ++r)
            #pragma unroll
            for (int m = 0; m < M; ++m) {
                const float v = warp_sum(acc[r][m]);
                if (lane == 0 && row0 + r < J.N) J.y[(size_t)m * J.N + row0 + r] = v * inv_s[m] * ig;
            }
    }
}

// ---- generic NVFP4 fallback -------------------------------------------------------------------
// Any K % 16 == 0 and any 4-byte-aligned tensor (the floor the reference's loader guarantees,
// kernels/moe.cu:167-174): one warp per row, 4-byte weight loads, activations read as fp32
// from global memory, fp32 arithmetic.  Slow and exact; used when the fast kernel's 16-byte
// alignment or shared-memory conditions do not hold.
template <int M>
__global__ void __launch_bounds__(GEMV_THREADS)
k_gemv_nvfp4_generic(const __grid_constant__ GemvParams p) {
    const int lane = threadIdx.x & 31;
    const int K = p.K, units = K >> 3;
    const int wid = blockIdx.x * GEMV_WARPS + (threadIdx.x >> 5), nw = gridDim.x * GEMV_WARPS;
    for (int ji = 0; ji < p.n_jobs; ++ji) {
        const GemvJobDev& J = p.j[ji];
        const float ig = 1.f / J.gs[0];
        for (int n = wid; n < J.N; n += nw) {
            const uint8_t* P = J.P + (size_t)n * (K >> 1);
            const uint8_t* S = J.S + (size_t)n * (K >> 4);
            float acc[M];
            #pragma unroll
            for (int m = 0; m < M; ++m) acc[m] = 0.f;
            for (int u = lane; u < units; u += 32) {
                const uint32_t w = *reinterpret_cast<const uint32_t*>(P + 4 * (size_t)u);
                const float sc = e4m3_to_f32(S[u >> 1]);
                uint32_t h[4];
                e2m1x8_to_h2(w, h);
                float wf[8];
                #pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h[j]));
                    wf[2 * j] = f.x; wf[2 * j + 1] = f.y;
                }
                #pragma unroll
                for (int m = 0; m < M; ++m) {
                    const float* xr = J.x + (size_t)m * K + 8 * (size_t)u;
                    float t = 0.f;
                    #pragma unroll
                    for (int j = 0; j < 8; ++j) t = fmaf(wf[j], xr[j], t);
                    acc[m] = fmaf(t, sc, acc[m]);
                }
            }
            #pragma unroll
            for (int m = 0; m < M; ++m) {
                const float v = warp_sum(acc[m]);
                if (lane == 0) J.y[(size_t)m * J.N + n] = v * ig;
            }
        }
    }
}

// ---- bf16 / f32 weights -------------------------------------------------------------------------
// One warp per output row, fp32 arithmetic throughout.  On the hot path this serves only the
// MoE router ([n_expert, hidden] bf16, reference kernels/moe.cu:647), whose logits decide the
// expert ranking and therefore stay in full fp32.  VEC: 16-byte weight loads, legal only when
// the base and the row stride are 16-byte aligned (the reference's vec16_ok rule,
// kernels/gemv.cu:188-192).
template <int M, bool BF16, bool VEC>
__global__ void __launch_bounds__(GEMV_THREADS)
k_gemm_dense(float* __restrict__ y, const void* __restrict__ W, const float* __restrict__ x,
             int N, int K) {
    const int lane = threadIdx.x & 31;
    const int n = blockIdx.x * GEMV_WARPS + (threadIdx.x >> 5);
    if (n >= N) return;
    float acc[M];
    #pragma unroll
    for (int m = 0; m < M; ++m) acc[m] = 0.f;
    constexpr int EPV = BF16 ? 8 : 4;              // elements per 16-byte vector
    int k0 = 0;
    if (VEC) {
        const int nv = K / EPV;
        const uint4* Wr = reinterpret_cast<const uint4*>(
            static_cast<const char*>(W) + (size_t)n * K * (BF16 ? 2 : 4));
        #pragma unroll 4                             // four weight loads in flight; the sums keep their order
        for (int i = lane; i < nv; i += 32) {
            const uint4 raw = Wr[i];
            float wf[EPV];
            if (BF16) {
                const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&raw);
                #pragma unroll
                for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(b[j]); wf[2 * j] = f.x; wf[2 * j + 1] = f.y; }
            } else {
                wf[0] = __uint_as_float(raw.x); wf[1] = __uint_as_float(raw.y);
                wf[2] = __uint_as_float(raw.z); wf[3] = __uint_as_float(raw.w);
            }
            #pragma unroll
            for (int m = 0; m < M; ++m) {
                const float* xr = x + (size_t)m * K + (size_t)i * EPV;
                #pragma unroll
                for (int j = 0; j < EPV; ++j) acc[m] = fmaf(wf[j], xr[j], acc[m]);
            }
        }
        k0 = nv * EPV;
    }
    for (int k = k0 + lane; k < K; k += 32) {
        const float w = BF16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(W)[(size_t)n * K + k])
                             : static_cast<const float*>(W)[(size_t)n * K + k];
        #pragma unroll
        for (int m = 0; m < M; ++m) acc[m] = fmaf(w, x[(size_t)m * K + k], acc[m]);
    }
    #pragma unroll
    for (int m = 0; m < M; ++m) {
        const float v = warp_sum(acc[m]);
        if (lane == 0) y[(size_t)m * N + n] = v;
    }
}

// The same product for few output rows (the MoE router: 144 x 4096): one CTA per row, the row's K
// split over 256 threads so that every weight load of the kernel is in flight at once, then a
// fixed-order reduction (lanes by shuffle, the eight warps in warp order).  bf16 weights, 16-byte
// aligned rows.
template <int M>
__global__ void __launch_bounds__(GEMV_THREADS)
k_gemm_dense_row(float* __restrict__ y, const __nv_bfloat16* __restrict__ W, const float* __restrict__ x, int N, int K) {
    __shared__ float part[GEMV_WARPS][M];
    const int n = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint4* Wr = reinterpret_cast<const uint4*>(W + (size_t)n * K);
    float acc[M];
    #pragma unroll
    for (int m = 0; m < M; ++m) acc[m] = 0.f;
    for (int i = threadIdx.x; i < (K >> 3); i += GEMV_THREADS) {
        const uint4 raw = Wr[i];
        const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&raw);
        float wf[8];
        #pragma unroll
        for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(b[j]); wf[2 * j] = f.x; wf[2 * j + 1] = f.y; }
        #pragma unroll
        for (int m = 0; m < M; ++m) {
            const float* xr = x + (size_t)m * K + (size_t)i * 8;
            #pragma unroll
            for (int j = 0; j < 8; ++j) acc[m] = fmaf(wf[j], xr[j], acc[m]);
        }
    }
    #pragma unroll
    for (int m = 0; m < M; ++m) {
        const float v = warp_sum(acc[m]);
        if (lane == 0) part[warp][m] = v;
    }
    __syncthreads();
    if (threadIdx.x < M) {
        float v = 0.f;
        #pragma unroll
        for (int w = 0; w < GEMV_WARPS; ++w) v += part[w][threadIdx.x];
        y[(size_t)threadIdx.x * N + n] = v;
    }
}

// The same product for MANY activation rows in one launch (the router logits of a prefill chunk): a CTA
// takes ET weight rows x up to 8 activation rows.  Every (weight row, activation row) pair is computed
// exactly as k_gemm_dense_row computes it -- same split of K over the threads, same FMA order, same
// reduction order -- so a token's logits, and with them its expert selection, do not depend on how many
// tokens were routed together.  Each thread keeps its slice of the 8 activation rows in registers and
// reuses it for the ET weight rows.
template <int ET>
__global__ void __launch_bounds__(GEMV_THREADS)
k_gemm_dense_rows(float* __restrict__ y, const __nv_bfloat16* __restrict__ W, const float* __restrict__ x, int M, int N, int K) {
    constexpr int TM = 8;
    __shared__ float part[GEMV_WARPS][ET][TM];
    const int n0 = blockIdx.x * ET, m0 = blockIdx.y * TM, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int mv = min(TM, M - m0);
    float acc[ET][TM];
    #pragma unroll
    for (int e = 0; e < ET; ++e)
        #pragma unroll
        for (int m = 0; m < TM; ++m) acc[e][m] = 0.f;
    for (int i = threadIdx.x; i < (K >> 3); i += GEMV_THREADS) {
        float xr[TM][8];
        #pragma unroll
        for (int m = 0; m < TM; ++m) {
            if (m < mv) {
                const float4* xp = reinterpret_cast<const float4*>(x + (size_t)(m0 + m) * K + (size_t)i * 8);
                const float4 a = xp[0], b = xp[1];
                xr[m][0] = a.x; xr[m][1] = a.y; xr[m][2] = a.z; xr[m][3] = a.w; xr[m][4] = b.x; xr[m][5] = b.y; xr[m][6] = b.z; xr[m][7] = b.w;
            } else {
                #pragma unroll
                for (int j = 0; j < 8; ++j) xr[m][j] = 0.f;
            }
        }
        #pragma unroll
        for (int e = 0; e < ET; ++e) {
            if (n0 + e >= N) break;
            const uint4 raw = reinterpret_cast<const uint4*>(W + (size_t)(n0 + e) * K)[i];
            const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&raw);
            float wf[8];
            #pragma unroll
            for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(b[j]); wf[2 * j] = f.x; wf[2 * j + 1] = f.y; }
            #pragma unroll
            for (int m = 0; m < TM; ++m) {
                #pragma unroll
                for (int j = 0; j < 8; ++j) acc[e][m] = fmaf(wf[j], xr[m][j], acc[e][m]);
            }
        }
    }
    #pragma unroll
    for (int e = 0; e < ET; ++e)
        #pragma unroll
        for (int m = 0; m < TM; ++m) {
            const float v = warp_sum(acc[e][m]);
            if (lane == 0) part[warp][e][m] = v;
        }
    __syncthreads();
    if (threadIdx.x < ET * TM) {
        const int e = threadIdx.x / TM, m = threadIdx.x - e * TM;
        if (n0 + e < N && m < mv) {
            float v = 0.f;
            #pragma unroll
            for (int w = 0; w < GEMV_WARPS; ++w) v += part[w][e][m];
            y[(size_t)(m0 + m) * N + n0 + e] = v;
        }
    }
}

__global__ void k_f32_to_bf16(__nv_bfloat16* d, const float* s, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) d[i] = __float2bfloat16(s[i]);
}
__global__ void k_bf16_to_f32(float* d, const __nv_bfloat16* s, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) d[i] = __bfloat162float(s[i]);
}

// ---- host side ---------------------------------------------------------------------------------
template <int M> struct RowsFor { static constexpr int v = M <= 2 ? 4 : 2; };

int nvfp4_math_mode() {
    static const int mode = [] {
        const char* e = getenv("B200_NVFP4_MATH");
        return (e && *e == '1') ? 1 : 0;
    }();
    return mode;
}

template <int M, int MATH>
static int launch_fast(const GemvParams& p, size_t smem, cudaStream_t s) {
    constexpr int R = RowsFor<M>::v;
    auto kern = k_gemv_nvfp4<M, R, MATH>;
    struct PerDevice { size_t smem_cfg = 0, occ_smem = (size_t)-1; int occ = 0; };
    static PerDevice cache[64];                      // the function attribute and the occupancy are per device
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    PerDevice& c = cache[dev];
    if (smem > 48 * 1024 && smem > c.smem_cfg) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return launch_failed("gemv: cudaFuncSetAttribute");
        c.smem_cfg = smem;
    }
    if (c.occ_smem != smem) {
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&c.occ, kern, GEMV_THREADS, smem) != cudaSuccess || c.occ < 1)
            return launch_failed("gemv: occupancy query");
        c.occ_smem = smem;
    }
    const int grid = std::min(p.total_tasks, sm_count() * c.occ);
    kern<<<grid, GEMV_THREADS, smem, s>>>(p);
    return check_launch("k_gemv_nvfp4");
}

template <int M>
static int launch_m(const GemvParams& p, bool fast, size_t smem, cudaStream_t s) {
    if (!fast) {
        int rows = 0;
        for (int i = 0; i < p.n_jobs; ++i) rows = std::max(rows, p.j[i].N);
        const int grid = std::min((rows + GEMV_WARPS - 1) / GEMV_WARPS, sm_count() * 8);
        k_gemv_nvfp4_generic<M><<<grid, GEMV_THREADS, 0, s>>>(p);
        return check_launch("k_gemv_nvfp4_generic");
    }
    return nvfp4_math_mode() ? launch_fast<M, 1>(p, smem, s) : launch_fast<M, 0>(p, smem, s);
}

// B200_NVFP4_GENERAL=1 keeps every shape on the general kernel (used by tests that compare the
// two kernels bit for bit, and for profiling).
static bool force_general() {
    const char* e = getenv("B200_NVFP4_GENERAL");
    return e && *e == '1';
}

// The tensor-core kernel (gemv_umma.cu) takes every shape it can; B200_NVFP4_UMMA=0 keeps it off
// (used by tests that compare the kernels with one another, and for profiling).
static bool use_umma() {
    const char* e = getenv("B200_NVFP4_UMMA");
    return !(e && *e == '0');
}

int rows_per_tile(int M) { return GEMV_WARPS * (M <= 2 ? 4 : 2); }

// Validates, decides fast vs generic, builds the flat task list, launches.  n in 1..8, M in 1..8.
int nvfp4_multi(const b200_gemv_job* jobs, int n, int M, int K, cudaStream_t s, void* split_ws) {
    if (!jobs || n < 1 || n > B200_GEMV_MULTI_MAX || M < 1 || M > B200_GEMV_M_MAX) return B200_EINVAL;
    if (K <= 0 || (K & 15)) return B200_ESHAPE;
    GemvParams p{};
    p.n_jobs = n; p.K = K;
    const size_t smem1 = (size_t)xs_chunks(K) * 16, smem = (size_t)M * smem1;
    if (smem > 200 * 1024 && smem1 <= 200 * 1024 && M > 1) {
        // The staged activations of all M rows do not fit shared memory: take the rows in chunks
        // that do, so that which kernel computes a row never depends on M (a gemm row must equal
        // the gemv of that row bit for bit).
        const int mc = (int)(200 * 1024 / smem1);
        for (int done = 0; done < M; done += mc) {
            b200_gemv_job sub[B200_GEMV_MULTI_MAX];
            for (int i = 0; i < n; ++i) {
                sub[i] = jobs[i];
                sub[i].y = jobs[i].y + (size_t)done * jobs[i].N;
                sub[i].x = jobs[i].x + (size_t)done * K;
            }
            if (int rc = nvfp4_multi(sub, n, std::min(mc, M - done), K, s, nullptr)) return rc;
        }
        return B200_OK;
    }
    bool fast = (K & 31) == 0 && smem <= 200 * 1024;
    int tasks = 0;
    const int tile = rows_per_tile(M);
    for (int i = 0; i < n; ++i) {
        const b200_gemv_job& j = jobs[i];
        if (!j.y || !j.x || !j.W.packed || !j.W.scale || !j.W.gscale || j.N <= 0) return B200_EINVAL;
        if (((uintptr_t)j.W.packed & 3) || ((uintptr_t)j.W.gscale & 3) || ((uintptr_t)j.x & 3) ||
            ((uintptr_t)j.y & 3)) return B200_EALIGN;
        if (((uintptr_t)j.W.packed & 15) || ((uintptr_t)j.W.scale & 1)) fast = false;
        p.j[i] = GemvJobDev{j.y, j.W.packed, j.W.scale, j.W.gscale, j.x, j.N, tasks};
        tasks += (j.N + tile - 1) / tile;
    }
    for (int i = n; i < B200_GEMV_MULTI_MAX; ++i) { p.j[i] = p.j[0]; p.j[i].N = 0; p.j[i].task0 = 0x7fffffff; }
    p.total_tasks = tasks;
    if (use_umma() && !force_general()) {            // checks its own conditions; they do not depend on M
        if (split_ws && M > 2) {                         // activations split once into the caller's scratch (pays from 3 rows on)
            const int rc = nvfp4_multi_umma_ws(p, M, split_ws, s);
            if (rc != B200_ENOTIMPL) return rc;
        }
        const int rc = nvfp4_multi_umma(p, M, s);
        if (rc != B200_ENOTIMPL) return rc;
    }
    if (M == 1 && fast && !force_general()) {
        const int rc = nvfp4_multi_tma(p, s);
        if (rc != B200_ENOTIMPL) return rc;
    }
    switch (M) {
        case 1: return launch_m<1>(p, fast, smem, s);
        case 2: return launch_m<2>(p, fast, smem, s);
        case 3: return launch_m<3>(p, fast, smem, s);
        case 4: return launch_m<4>(p, fast, smem, s);
        case 5: return launch_m<5>(p, fast, smem, s);
        case 6: return launch_m<6>(p, fast, smem, s);
        case 7: return launch_m<7>(p, fast, smem, s);
        default: return launch_m<8>(p, fast, smem, s);
    }
}

template <int M>
static int launch_dense(float* y, const void* W, const float* x, int N, int K, int dtype, cudaStream_t s) {
    const int grid = (N + GEMV_WARPS - 1) / GEMV_WARPS;
    const int eb = dtype == B200_F32 ? 4 : 2;
    const bool vec = (((uintptr_t)W & 15) == 0) && ((((size_t)K * eb) & 15) == 0);
    if (dtype == B200_BF16 && vec && N <= 2048 && K >= 2048) {       // few rows: latency-bound, one CTA per row
        k_gemm_dense_row<M><<<N, GEMV_THREADS, 0, s>>>(y, static_cast<const __nv_bfloat16*>(W), x, N, K);
        return check_launch("k_gemm_dense_row");
    }
    if (dtype == B200_F32) {
        if (vec) k_gemm_dense<M, false, true><<<grid, GEMV_THREADS, 0, s>>>(y, W, x, N, K);
        else     k_gemm_dense<M, false, false><<<grid, GEMV_THREADS, 0, s>>>(y, W, x, N, K);
    } else {
        if (vec) k_gemm_dense<M, true, true><<<grid, GEMV_THREADS, 0, s>>>(y, W, x, N, K);
        else     k_gemm_dense<M, true, false><<<grid, GEMV_THREADS, 0, s>>>(y, W, x, N, K);
    }
    return check_launch("k_gemm_dense");
}

int dense_gemm(float* y, const void* W, const float* x, int M, int N, int K, int dtype, cudaStream_t s) {
    if (!y || !W || !x || M < 1 || N < 1 || K < 1) return B200_EINVAL;
    if (dtype != B200_F32 && dtype != B200_BF16) return B200_EINVAL;
    if (M > 8 && dtype == B200_BF16 && N <= 2048 && K >= 2048 && !(K & 7) && !((uintptr_t)W & 15) && !((uintptr_t)x & 15)) {
        // many rows against a small bf16 matrix (router logits of a prefill chunk): one launch, same bits per row
        constexpr int ET = 4;
        k_gemm_dense_rows<ET><<<dim3((N + ET - 1) / ET, (M + 7) / 8), GEMV_THREADS, 0, s>>>(y, static_cast<const __nv_bfloat16*>(W), x, M, N, K);
        return check_launch("k_gemm_dense_rows");
    }
    for (int done = 0; done < M;) {
        const int c = std::min(M - done, 8);
        float* yc = y + (size_t)done * N;
        const float* xc = x + (size_t)done * K;
        int rc;
        switch (c) {
            case 1: rc = launch_dense<1>(yc, W, xc, N, K, dtype, s); break;
            case 2: rc = launch_dense<2>(yc, W, xc, N, K, dtype, s); break;
            case 3: rc = launch_dense<3>(yc, W, xc, N, K, dtype, s); break;
            case 4: rc = launch_dense<4>(yc, W, xc, N, K, dtype, s); break;
            case 5: rc = launch_dense<5>(yc, W, xc, N, K, dtype, s); break;
            case 6: rc = launch_dense<6>(yc, W, xc, N, K, dtype, s); break;
            case 7: rc = launch_dense<7>(yc, W, xc, N, K, dtype, s); break;
            default: rc = launch_dense<8>(yc, W, xc, N, K, dtype, s); break;
        }
        if (rc) return rc;
        done += c;
    }
    return B200_OK;
}

}  // namespace b200

using namespace b200;

extern "C" int b200_nvfp4_gemm(float* y, const b200_wref* W, const float* x, int M, int N, int K,
                               int dtype, b200_stream stream) {
    if (!W || M < 1) return B200_EINVAL;
    if (!W->packed) {
        // one pass per 8 rows, or a single one through the many-row kernel (same conditions as dense_gemm)
        const bool one = M > 8 && dtype == B200_BF16 && N <= 2048 && K >= 2048;
        credit(B200_CREDIT_GEMM, (double)(one ? 1 : (M + 7) / 8) * N * K * (dtype == B200_F32 ? 4.0 : 2.0));
        return dense_gemm(y, W->p, x, M, N, K, dtype, stream);
    }
    credit(B200_CREDIT_GEMM, (double)((M + B200_GEMV_M_MAX - 1) / B200_GEMV_M_MAX) * N * K * 0.5625);
    for (int done = 0; done < M;) {
        const int c = std::min(M - done, (int)B200_GEMV_M_MAX);
        b200_gemv_job j{y + (size_t)done * N, *W, x + (size_t)done * K, N};
        const int rc = nvfp4_multi(&j, 1, c, K, stream, nullptr);
        if (rc) return rc;
        done += c;
    }
    return B200_OK;
}

extern "C" size_t b200_nvfp4_split_workspace_bytes(int M, int K) {
    if (M < 1 || K < 256) return 256;
    return std::max(std::max((umma_presplit_bytes(M, K) + 255) / 256 * 256, gemm_mxf4_ws_bytes(M, K)), M >= PREFILL_MIN_ROWS ? gemm_f16w_ws_bytes(M, K) : (size_t)0);
}

extern "C" int b200_nvfp4_gemm_ws(float* y, const b200_wref* W, const float* x, int M, int N, int K,
                                  int dtype, void* ws, b200_stream stream) {
    if (!W || M < 1) return B200_EINVAL;
    if (!W->packed || !ws || M < 3 || !use_umma() || force_general()) return b200_nvfp4_gemm(y, W, x, M, N, K, dtype, stream);
    if ((uintptr_t)ws & 255) return B200_EALIGN;
    if (M >= PREFILL_MIN_ROWS) {
        // prefill widths: W once per call.  NVFP4 activations on the block-scaled MMA, or (option off) exact
        // products on the f16 MMA with the weights dequantised inside the kernel
        const int rc = prefill_fp4_option() ? gemm_mxf4_dense(y, W, x, 1, M, N, K, ws, stream)
                                            : gemm_f16w_dense(y, W, x, 1, M, N, K, ws, stream);
        if (rc != B200_ENOTIMPL) return rc;
    }
    credit(B200_CREDIT_GEMM, (double)((M + B200_GEMV_M_MAX - 1) / B200_GEMV_M_MAX) * N * K * 0.5625);
    // every row at once: one split launch, then one pass over the weights per 8 rows
    b200_gemv_job j{y, *W, x, N};
    GemvParams p{};
    if (!j.y || !j.x || !W->scale || !W->gscale || N <= 0 || K <= 0 || (K & 15)) return B200_EINVAL;
    p.n_jobs = 1; p.K = K;
    p.j[0] = GemvJobDev{j.y, W->packed, W->scale, W->gscale, j.x, N, 0};
    for (int i = 1; i < B200_GEMV_MULTI_MAX; ++i) { p.j[i] = p.j[0]; p.j[i].N = 0; p.j[i].task0 = 0x7fffffff; }
    const int rc = nvfp4_multi_umma_ws(p, M, ws, stream);
    if (rc != B200_ENOTIMPL) return rc;
    for (int done = 0; done < M;) {                   // as b200_nvfp4_gemm, whose bytes were credited above
        const int c = std::min(M - done, (int)B200_GEMV_M_MAX);
        b200_gemv_job jj{y + (size_t)done * N, *W, x + (size_t)done * K, N};
        if (int r2 = nvfp4_multi(&jj, 1, c, K, stream, nullptr)) return r2;
        done += c;
    }
    return B200_OK;
}

extern "C" int b200_nvfp4_gemv_multi_ws(const b200_gemv_job* jobs, int n, int M, int K, int dtype,
                                        void* ws, b200_stream stream) {
    if (!jobs || n < 1 || n > B200_GEMV_MULTI_MAX || M < 1 || M > B200_GEMV_M_MAX) return B200_EINVAL;
    if (ws && ((uintptr_t)ws & 255)) return B200_EALIGN;
    for (int i = 0; i < n; ++i)
        if (!jobs[i].W.packed) return b200_nvfp4_gemv_multi(jobs, n, M, K, dtype, stream);
    if (credit_on()) {
        double b = 0.0;
        for (int i = 0; i < n; ++i) b += (double)jobs[i].N * K * 0.5625;
        credit(B200_CREDIT_GEMM, b);
    }
    return nvfp4_multi(jobs, n, M, K, stream, ws);
}

extern "C" int b200_nvfp4_gemv_multi(const b200_gemv_job* jobs, int n, int M, int K, int dtype,
                                     b200_stream stream) {
    if (!jobs || n < 1 || n > B200_GEMV_MULTI_MAX || M < 1 || M > B200_GEMV_M_MAX) return B200_EINVAL;
    bool all_q = true;
    for (int i = 0; i < n; ++i) all_q = all_q && jobs[i].W.packed != nullptr;
    if (all_q && credit_on()) {
        double b = 0.0;
        for (int i = 0; i < n; ++i) b += (double)jobs[i].N * K * 0.5625;
        credit(B200_CREDIT_GEMM, b);
    }
    if (all_q) return nvfp4_multi(jobs, n, M, K, stream, nullptr);
    for (int i = 0; i < n; ++i) {                  // mixed or plain weights: correct, not fused
        const int rc = b200_nvfp4_gemm(jobs[i].y, &jobs[i].W, jobs[i].x, M, jobs[i].N, K, dtype, stream);
        if (rc) return rc;
    }
    return B200_OK;
}

extern "C" int b200_f32_to_bf16(void* dst, const float* src, size_t n, b200_stream stream) {
    if (!dst || !src) return B200_EINVAL;
    if (n == 0) return B200_OK;
    k_f32_to_bf16<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>((__nv_bfloat16*)dst, src, n);
    return check_launch("k_f32_to_bf16");
}

extern "C" int b200_bf16_to_f32(float* dst, const void* src, size_t n, b200_stream stream) {
    if (!dst || !src) return B200_EINVAL;
    if (n == 0) return B200_OK;
    k_bf16_to_f32<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(dst, (const __nv_bfloat16*)src, n);
    return check_launch("k_bf16_to_f32");
}
