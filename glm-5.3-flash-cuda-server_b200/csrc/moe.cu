// moe.cu -- MoE block for sm_100a: sigmoid router with bias-ranked top-k, routed + shared NVFP4
// SwiGLU experts, gate-weighted sum.  Replaces the reference's kernels/moe.cu (k_route :126-156,
// k_expert_act :175-259, k_expert_down :270-327, k_down_combine :584-597, entry points :602-740).
//
// Launches per layer: router logits (bf16 gemm), k_route, k_expert_act, k_expert_down.
//   k_expert_act   one warp owns two intermediate indices o, o+1 of one (token, slot): the gate
//                  and up rows of both stream together (4 rows x 2 steps in flight per lane),
//                  and the clamped SwiGLU is applied before anything is written.
//   k_expert_down  one warp owns one hidden row of one token and walks the slots three at a
//                  time, each slot against its own staged intermediate vector; the gate
//                  weight, 1/gscale and the staging scale are folded per slot at lane level and
//                  the warp is reduced once, in a fixed order -- so the per-slot partial buffer
//                  and the separate combine launch of the reference are gone, and results are
//                  identical from run to run (no atomics).
// Geometry (hidden, inter, top-k, scale, clamp) is per layer at run time.
#include "b200_internal.h"
#include "gemv_core.cuh"
#include "moe_plan.cuh"
#include <cstdio>

namespace b200 {

constexpr int ROUTE_MAXC = 16;        // candidates per lane -> n_expert <= 512
constexpr int MOE_MAX_SLOTS = 17;     // topk <= 16, plus the shared expert

struct MoeArgs {
    const float* x; float* y; const int32_t* sel; const float* wts; float* act;
    const b200_nvfp4_mat* experts; const b200_nvfp4_mat* shared;
    int M, H, I, E, topk, ns;
    float limit;
};

// One warp per token.  Ranking value = sigmoid(logit) + bias, gate value = sigmoid(logit);
// among equal ranking values the lowest expert index wins, as in the reference's serial scan
// with a strict '>' (kernels/moe.cu:146-152).
template <int C>                                   // candidates per lane: n_expert <= 32 * C
__global__ void __launch_bounds__(32)
k_route(int32_t* __restrict__ sel, float* __restrict__ wts, const float* __restrict__ logits,
        const float* __restrict__ bias, int E, int K, float scaling, int norm_prob, const __grid_constant__ MoePlan plan) {
    const int tok = blockIdx.x, lane = threadIdx.x;
    logits += (size_t)tok * E; sel += (size_t)tok * K; wts += (size_t)tok * K;
    // Ranking values as unsigned keys that order like the floats (0 = not a candidate: padding, a NaN, anything
    // at or below -1e30, or already taken), so that a round is two warp reductions -- the largest key, then the
    // lowest expert index among the lanes that hold it -- instead of five rounds of three shuffles.
    float score[C];
    uint32_t key[C];
    #pragma unroll
    for (int j = 0; j < C; ++j) {
        const int i = lane + 32 * j;
        score[j] = 0.f; key[j] = 0u;
        if (i < E) {
            score[j] = 1.f / (1.f + __expf(-logits[i]));
            const float c = score[j] + bias[i];
            const uint32_t u = __float_as_uint(c);
            if (c > -1e30f) key[j] = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
        }
    }
    uint32_t lk = 0u; int lj = 0; float ls = 0.f;   // this lane's best candidate: key, slot, gate value (lowest slot among equals)
    auto local_best = [&]() {
        lk = 0u; lj = 0; ls = 0.f;
        #pragma unroll
        for (int j = 0; j < C; ++j) if (key[j] > lk) { lk = key[j]; lj = j; ls = score[j]; }
    };
    local_best();
    float my_w = 0.f;                              // lane k keeps the k-th gate
    int my_e = 0;                                  // ... and the k-th expert
    for (int k = 0; k < K; ++k) {
        const uint32_t gmax = __reduce_max_sync(0xffffffffu, lk);
        int bi = 0; float bs = 0.f;                // fewer than K candidates: expert 0 with gate 0, as the serial scan would leave it
        if (gmax) {
            bi = (int)__reduce_min_sync(0xffffffffu, lk == gmax ? (uint32_t)(lane + 32 * lj) : 0x7fffffffu);
            bs = __shfl_sync(0xffffffffu, ls, bi & 31);
        }
        if (lane == (bi & 31)) {
            #pragma unroll
            for (int j = 0; j < C; ++j) if (j == (bi >> 5)) key[j] = 0u;
            local_best();
        }
        if (lane == k) { my_w = bs; my_e = bi; }
        if (lane == 0) sel[k] = bi;
    }
    float d = 1.f;
    if (norm_prob) {
        d = 1e-20f;
        for (int k = 0; k < K; ++k) d += __shfl_sync(0xffffffffu, my_w, k);
    }
    if (lane < K) wts[lane] = my_w / d * scaling;
    // job records of the tensor-core experts for this token's pairs (prepared layers only)
    if (plan.j1 && lane < plan.ns) moe_plan_pair(plan, tok, lane, my_e);
}

template <int MATH>
__global__ void __launch_bounds__(GEMV_THREADS)
k_expert_act(const __grid_constant__ MoeArgs a, int tiles, int total_tasks) {
    extern __shared__ uint4 xs[];
    __shared__ float inv_s[1];
    __shared__ float red[GEMV_WARPS];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int staged = -1;
    for (int task = blockIdx.x; task < total_tasks; task += gridDim.x) {
        const int m = task / (a.ns * tiles), rem = task - m * (a.ns * tiles);
        const int slot = rem / tiles, tile = rem - slot * tiles;
        if (m != staged) {
            if (staged >= 0) __syncthreads();
            stage_x(a.x + (size_t)m * a.H, 1, a.H, xs, inv_s, red);
            staged = m;
        }
        const int o0 = tile * (GEMV_WARPS * 2) + warp * 2;
        if (o0 >= a.I) continue;
        const b200_nvfp4_mat* mats;
        if (slot < a.topk) {
            int e = a.sel[(size_t)m * a.topk + slot];
            e = e < 0 ? 0 : (e >= a.E ? a.E - 1 : e);
            mats = a.experts + (size_t)e * 3;
        } else mats = a.shared;
        const b200_nvfp4_mat G = mats[0], U = mats[1];
        const int o1 = min(o0 + 1, a.I - 1);
        const size_t pr = (size_t)a.H >> 1, sr = (size_t)a.H >> 4;
        RowPtr rows[4] = {{G.packed + o0 * pr, G.scale + o0 * sr}, {U.packed + o0 * pr, U.scale + o0 * sr},
                          {G.packed + o1 * pr, G.scale + o1 * sr}, {U.packed + o1 * pr, U.scale + o1 * sr}};
        float acc[4][1] = {{0.f}, {0.f}, {0.f}, {0.f}};
        warp_rows<1, 4, MATH, true>(rows, a.H, xs, acc, lane);
        const float kg = inv_s[0] / G.gscale[0], ku = inv_s[0] / U.gscale[0];
        #pragma unroll
        for (int q = 0; q < 2; ++q) {
            float g = warp_sum(acc[2 * q][0]) * kg, u = warp_sum(acc[2 * q + 1][0]) * ku;
            if (lane == 0 && o0 + q < a.I) {
                g = fminf(g, a.limit);
                u = fminf(fmaxf(u, -a.limit), a.limit);
                a.act[((size_t)m * a.ns + slot) * a.I + o0 + q] = (g / (1.f + __expf(-g))) * u;
            }
        }
    }
}

template <int MATH>
__global__ void __launch_bounds__(GEMV_THREADS)
k_expert_down(const __grid_constant__ MoeArgs a, int tiles, int total_tasks) {
    extern __shared__ uint4 xs[];
    __shared__ float inv_s[MOE_MAX_SLOTS];
    __shared__ float red[MOE_MAX_SLOTS * GEMV_WARPS];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int stride = xs_chunks(a.I);
    int staged = -1;
    for (int task = blockIdx.x; task < total_tasks; task += gridDim.x) {
        const int m = task / tiles, tile = task - m * tiles;
        if (m != staged) {
            if (staged >= 0) __syncthreads();
            stage_x(a.act + (size_t)m * a.ns * a.I, a.ns, a.I, xs, inv_s, red);
            staged = m;
        }
        const int h = tile * GEMV_WARPS + warp;
        if (h >= a.H) continue;
        const size_t pr = (size_t)a.I >> 1, sr = (size_t)a.I >> 4;
        float tot = 0.f;
        for (int s0 = 0; s0 < a.ns; s0 += 3) {
            RowPtr rows[3]; const uint4* xb[3]; float coef[3];
            #pragma unroll
            for (int q = 0; q < 3; ++q) {
                const int slot = min(s0 + q, a.ns - 1);
                const b200_nvfp4_mat* mats;
                float w = 1.f;
                if (slot < a.topk) {
                    int e = a.sel[(size_t)m * a.topk + slot];
                    e = e < 0 ? 0 : (e >= a.E ? a.E - 1 : e);
                    mats = a.experts + (size_t)e * 3;
                    w = a.wts[(size_t)m * a.topk + slot];
                } else mats = a.shared;
                const b200_nvfp4_mat D = mats[2];
                rows[q].p = D.packed + h * pr; rows[q].s = D.scale + h * sr;
                xb[q] = xs + (size_t)slot * stride;
                coef[q] = (s0 + q < a.ns) ? w * inv_s[slot] / D.gscale[0] : 0.f;
            }
            float acc[3] = {0.f, 0.f, 0.f};
            warp_rows_own_x<3, MATH, true>(rows, a.I, xb, acc, lane);
            tot = fmaf(acc[0], coef[0], tot);
            tot = fmaf(acc[1], coef[1], tot);
            tot = fmaf(acc[2], coef[2], tot);
        }
        tot = warp_sum(tot);
        if (lane == 0) a.y[(size_t)m * a.H + h] = tot;
    }
}

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

static int check_layer(const b200_moe_layer* L, int M) {
    if (!L || M < 1) return B200_EINVAL;
    if (!L->experts || L->n_expert < 1 || L->topk < 1 || L->topk > 16 || L->topk > L->n_expert) return B200_EINVAL;
    if (L->n_expert > 32 * ROUTE_MAXC) return B200_ELIMIT;
    if (L->hidden <= 0 || L->inter <= 0 || (L->hidden & 31) || (L->inter & 31)) return B200_ESHAPE;
    if ((size_t)xs_chunks(L->hidden) * 16 > 200 * 1024 ||
        (size_t)(L->topk + 1) * xs_chunks(L->inter) * 16 > 200 * 1024) return B200_ELIMIT;
    return B200_OK;
}

template <typename Kern>
static int grid_for(Kern kern, size_t smem, int tasks, int* grid) {
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return launch_failed("moe: cudaFuncSetAttribute");
    int occ = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, GEMV_THREADS, smem) != cudaSuccess || occ < 1)
        return launch_failed("moe: occupancy query");
    *grid = std::min(tasks, sm_count() * occ);
    return B200_OK;
}

static int experts_forward(const float* x, const b200_moe_layer* L, float* y, const int32_t* sel,
                           const float* wts, float* act, int M, cudaStream_t s, bool allow_tensor_path, bool planned = false, int wide = -1) {
    if (allow_tensor_path) {                             // prepared layers (moe_umma.cu)
        const int rc = moe_umma_experts(x, L, y, sel, wts, act, M, s, planned, wide);
        if (rc != B200_ENOTIMPL) return rc;
    }
    credit(B200_CREDIT_MOE_ACT, (double)M * (L->topk + (L->shared ? 1 : 0)) * 2.0 * L->inter * L->hidden * 0.5625);
    credit(B200_CREDIT_MOE_DOWN, (double)M * (L->topk + (L->shared ? 1 : 0)) * 1.0 * L->inter * L->hidden * 0.5625);
    MoeArgs a{};
    a.x = x; a.y = y; a.sel = sel; a.wts = wts; a.act = act;
    a.experts = L->experts; a.shared = L->shared;
    a.M = M; a.H = L->hidden; a.I = L->inter; a.E = L->n_expert; a.topk = L->topk;
    a.ns = L->topk + (L->shared ? 1 : 0);
    a.limit = L->swiglu_limit;
    const int math = nvfp4_math_mode();
    {
        const int tiles = (a.I + GEMV_WARPS * 2 - 1) / (GEMV_WARPS * 2), tasks = M * a.ns * tiles;
        const size_t smem = (size_t)xs_chunks(a.H) * 16;
        int grid = 0;
        if (math) {
            if (int rc = grid_for(k_expert_act<1>, smem, tasks, &grid)) return rc;
            k_expert_act<1><<<grid, GEMV_THREADS, smem, s>>>(a, tiles, tasks);
        } else {
            if (int rc = grid_for(k_expert_act<0>, smem, tasks, &grid)) return rc;
            k_expert_act<0><<<grid, GEMV_THREADS, smem, s>>>(a, tiles, tasks);
        }
        if (int rc = check_launch("k_expert_act")) return rc;
    }
    {
        const int tiles = (a.H + GEMV_WARPS - 1) / GEMV_WARPS, tasks = M * tiles;
        const size_t smem = (size_t)a.ns * xs_chunks(a.I) * 16;
        int grid = 0;
        if (math) {
            if (int rc = grid_for(k_expert_down<1>, smem, tasks, &grid)) return rc;
            k_expert_down<1><<<grid, GEMV_THREADS, smem, s>>>(a, tiles, tasks);
        } else {
            if (int rc = grid_for(k_expert_down<0>, smem, tasks, &grid)) return rc;
            k_expert_down<0><<<grid, GEMV_THREADS, smem, s>>>(a, tiles, tasks);
        }
        if (int rc = check_launch("k_expert_down")) return rc;
    }
    return B200_OK;
}

}  // namespace b200

using namespace b200;

// Workspace: logits f32 [M, E] | scratch of the experts, each part 256-byte aligned.  The scratch is
// act f32 [M, topk+1, inter] for the CUDA-core experts; the tensor-core path (up to 8 tokens) wants
// more (moe_umma.cu), and the size covers whichever of the two a call may take.
static size_t legacy_workspace_bytes(const b200_moe_layer* L, int M) {
    return align_up((size_t)M * L->n_expert * 4, 256) + align_up((size_t)M * (L->topk + 1) * L->inter * 4, 256);
}
extern "C" size_t b200_moe_workspace_bytes(const b200_moe_layer* L, int M) {
    if (!L || M < 1) return 0;
    size_t scratch = align_up((size_t)M * (L->topk + 1) * L->inter * 4, 256);
    scratch = std::max(scratch, moe_umma_ws_bytes(L, M));
    return align_up((size_t)M * L->n_expert * 4, 256) + scratch;
}

static int route_launch(const float* x, const b200_moe_layer* L, int32_t* sel, float* wts, float* logits, int M,
                        cudaStream_t stream, const MoePlan& plan) {
    if (int rc = check_layer(L, M)) return rc;
    if (!x || !sel || !wts || !logits || !L->router_bias) return B200_EINVAL;
    if (int rc = b200_nvfp4_gemm(logits, &L->router_w, x, M, L->n_expert, L->hidden, B200_BF16, stream)) return rc;
    if (L->n_expert <= 128)
        k_route<4><<<M, 32, 0, stream>>>(sel, wts, logits, L->router_bias, L->n_expert, L->topk, L->routed_scale, L->norm_topk, plan);
    else if (L->n_expert <= 256)
        k_route<8><<<M, 32, 0, stream>>>(sel, wts, logits, L->router_bias, L->n_expert, L->topk, L->routed_scale, L->norm_topk, plan);
    else
        k_route<ROUTE_MAXC><<<M, 32, 0, stream>>>(sel, wts, logits, L->router_bias, L->n_expert, L->topk, L->routed_scale, L->norm_topk, plan);
    return check_launch("k_route");
}

extern "C" int b200_moe_route(const float* x, const b200_moe_layer* L, int32_t* sel, float* wts,
                              float* logits, int M, b200_stream stream) {
    return route_launch(x, L, sel, wts, logits, M, stream, MoePlan{});
}

int b200::moe_experts_mode(const float* x, const b200_moe_layer* L, float* y, const int32_t* sel, const float* wts,
                           void* ws, int M, cudaStream_t stream, int wide) {
    if (int rc = check_layer(L, M)) return rc;
    if (!x || !y || !sel || !wts || !ws) return B200_EINVAL;
    if ((uintptr_t)ws & 15) return B200_EALIGN;
    float* act = reinterpret_cast<float*>(static_cast<char*>(ws) + align_up((size_t)M * L->n_expert * 4, 256));
    return experts_forward(x, L, y, sel, wts, act, M, stream, true, false, wide);
}

extern "C" int b200_moe_experts(const float* x, const b200_moe_layer* L, float* y, const int32_t* sel,
                                const float* wts, void* ws, int M, b200_stream stream) {
    return moe_experts_mode(x, L, y, sel, wts, ws, M, stream, -1);
}

extern "C" int b200_moe_forward(const float* x, const b200_moe_layer* L, float* y, int32_t* sel,
                                float* wts, void* ws, int M, b200_stream stream) {
    if (int rc = check_layer(L, M)) return rc;
    if (!x || !y || !sel || !wts || !ws) return B200_EINVAL;
    if ((uintptr_t)ws & 15) return B200_EALIGN;
    float* logits = static_cast<float*>(ws);
    float* act = reinterpret_cast<float*>(static_cast<char*>(ws) + align_up((size_t)M * L->n_expert * 4, 256));
    // On a prepared layer the router kernel also writes the job records of the tensor-core experts.
    MoePlan plan{};
    int R_gu = 0, R_d = 0;
    const bool planned = moe_umma_plan_args(x, L, act, M, &plan, &R_gu, &R_d) == B200_OK;
    if (!planned) plan = MoePlan{};
    if (int rc = route_launch(x, L, sel, wts, logits, M, stream, plan)) return rc;
    return experts_forward(x, L, y, sel, wts, act, M, stream, true, planned);
}

// ---- allocation-free variant -------------------------------------------------------------------
// b200_moe_forward needs a workspace (router logits + the experts' intermediate activations),
// and normally the caller allocates it from b200_moe_workspace_bytes.  Some hosts of this
// library cannot do that.  The reference engine sizes its one workspace buffer at start-up from
// ITS moe_workspace_floats(); once this library sits behind the old header the engine may be
// running with a buffer of the old size, and it has no moment at which it could get a new one:
// the MoE block runs between decode steps, where a cudaMalloc would synchronise the device and
// stall the token loop, and under stream capture an allocation is not legal at all.  For those
// callers the scratch lives inside the library, in the array below, which every GPU that loads
// the library holds until the process exits.
//
// Limit: B200_MOE_STATIC_WS_BYTES (1 MiB) -- enough for 14 tokens at the reference geometry
// (144 experts, top-8 + shared, inter 2048: 74 304 B per token).  Larger requests are refused.
// The array is shared by every call on the device and keeps the previous call's bytes.  Nothing
// in it has to start at zero: every byte a launch reads was written earlier by the same call
// (logits by the router launch, activations by the gate/up launch), so it is never cleared.
// Two calls whose kernels overlap on the GPU (different streams without an ordering between
// them) would write the same scratch at once and corrupt each other: order them.
constexpr size_t B200_MOE_STATIC_WS_BYTES = 1u << 20;
static __device__ __align__(256) unsigned char g_moe_static_ws[B200_MOE_STATIC_WS_BYTES];

// Device address of the array for the CURRENT device.  In host code the array's name is only a
// handle; the address a kernel can use comes from cudaGetSymbolAddress, once per device.
static int moe_static_ws_ptr(void** out) {
    static void* cache[64] = {nullptr};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return b200::launch_failed("moe_forward_static: cudaGetDevice");
    if (!cache[dev]) {
        void* ptr = nullptr;
        const cudaError_t e = cudaGetSymbolAddress((void**)&ptr, g_moe_static_ws);
        if (e != cudaSuccess || !ptr) {
            fprintf(stderr, "b200_nvfp4: cudaGetSymbolAddress(static MoE workspace) failed: %s\n", cudaGetErrorString(e));
            return B200_ELAUNCH;
        }
        cache[dev] = ptr;
    }
    *out = cache[dev];
    return B200_OK;
}

extern "C" size_t b200_moe_static_ws_limit(void) { return B200_MOE_STATIC_WS_BYTES; }

extern "C" int b200_moe_forward_static(const float* x, const b200_moe_layer* L, float* y, int32_t* sel,
                                       float* wts, int M, b200_stream stream) {
    if (int rc = check_layer(L, M)) return rc;
    const size_t need = legacy_workspace_bytes(L, M);    // this entry point always runs the CUDA-core experts
    if (need > B200_MOE_STATIC_WS_BYTES) {
        fprintf(stderr, "b200_nvfp4: b200_moe_forward_static needs %zu bytes of scratch for M=%d, the built-in "
                        "workspace holds %zu; use b200_moe_forward with a caller-allocated workspace\n",
                need, M, B200_MOE_STATIC_WS_BYTES);
        return B200_ELIMIT;
    }
    if (!x || !y || !sel || !wts) return B200_EINVAL;
    void* ws = nullptr;
    if (int rc = moe_static_ws_ptr(&ws)) return rc;
    float* logits = static_cast<float*>(ws);
    if (int rc = b200_moe_route(x, L, sel, wts, logits, M, stream)) return rc;
    float* act = reinterpret_cast<float*>(static_cast<char*>(ws) + align_up((size_t)M * L->n_expert * 4, 256));
    return experts_forward(x, L, y, sel, wts, act, M, stream, false);
}
