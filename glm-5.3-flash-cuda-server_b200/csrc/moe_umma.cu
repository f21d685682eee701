// moe_umma.cu -- the MoE experts on the tensor-core gemv kernel (gemv_umma.cu), once
// b200_moe_prepare() has been called for the layer.
//
// The expert tables of a layer live in device memory and the router picks experts on the device,
// but a TMA tensor map has to be encoded on the host.  b200_moe_prepare therefore reads the
// layer's tables once, encodes the six maps of every expert (gate, up, down: packed weights and
// scales) and keeps them in device memory; at run time a small kernel turns (token, slot) pairs
// into job records that point at the maps of the selected experts.
//
// Launches per layer: router logits, k_route, k_moe_plan, gate+up products of all pairs (one
// tensor-core launch), down products (one tensor-core launch; it reads the two products and
// applies the clamped SwiGLU while it splits its activation vector), k_moe_combine.
// Up to 8 tokens every (token, slot) pair is its own single-row job, the shared expert included
// (its weights are read once from HBM and then from L2).  Beyond 8 tokens the pairs are sorted by
// expert on the device and an expert's rows run in chunks of up to 8, each chunk split into its
// FP4 digit image once (k_split_rows).  Either way a row is computed on its own: a token's result
// does not depend on what else is in the batch, bit for bit.  The gate-weighted sum runs over
// the slots in slot order.
#include "b200_internal.h"
#include "moe_plan.cuh"
#include "tma_pipe.cuh"
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

namespace b200 {

constexpr int MU_MAX_TOKENS = 8;
// Fewest tokens for which the (token, slot) pairs are sorted by expert, so that every distinct expert
// (and the shared expert) is streamed once for up to 8 rows instead of once per pair (the reference's
// gathered kernels, kernels/moe.cu:353-581).  Below it every pair is its own job.  B200_MOE_GROUP_MIN
// overrides it for experiments.
static int group_min_tokens() {
    static const int v = [] { const char* e = getenv("B200_MOE_GROUP_MIN"); const int n = e ? atoi(e) : 0; return n >= 2 ? n : MU_MAX_TOKENS + 1; }();
    return v;
}

struct Prepared {
    const b200_nvfp4_mat* experts; const b200_nvfp4_mat* shared;     // key
    int E, H, I;
    unsigned char* maps;          // device: [(E + 1) experts][3 matrices][w, s] x 128 bytes, shared expert last; then the same again
                                  // with boxes 128 rows tall, for the wide GEMM (MU_GX_MAPS bytes further on)
    int R_gu, R_d;
    int device;
};
static std::vector<Prepared> g_prepared;
static std::mutex g_prepared_mu;

// A COPY of the layer's entry, taken under the lock (the table may grow or an entry be released by another
// thread right after).  The device memory behind `maps` stays valid until b200_moe_release, which the
// caller must not run while calls on that layer are still queued.
static bool find_prepared(const b200_moe_layer* L, Prepared* out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) return false;
    std::lock_guard<std::mutex> lk(g_prepared_mu);
    for (const Prepared& p : g_prepared)
        if (p.maps && p.experts == L->experts && p.shared == L->shared && p.E == L->n_expert && p.H == L->hidden && p.I == L->inter && p.device == dev) {
            if (out) *out = p;
            return true;
        }
    return false;
}

// Box height for n_jobs jobs of N rows: fewest waves of CTAs over the SMs, each wave costing its
// rows plus a fixed part (activation split, pipeline fill and drain) worth about 40 rows.
static int pick_rows(int n_jobs, int N) {
    int best = 128; long best_cost = -1;
    for (int R = 128; R >= 32; R -= 8) {
        const long tasks = (long)n_jobs * ((N + R - 1) / R), waves = (tasks + sm_count() - 1) / sm_count();
        const long cost = waves * (R + 40);
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = R; }
    }
    return best;
}

__global__ void k_moe_plan(const __grid_constant__ MoePlan q, const int32_t* __restrict__ sel, int M) {
    const int pair = blockIdx.x * blockDim.x + threadIdx.x;
    if (pair >= M * q.ns) return;
    const int m = pair / q.ns, slot = pair - m * q.ns;
    moe_plan_pair(q, m, slot, slot < q.topk ? sel[(size_t)m * q.topk + slot] : 0);
}

// y[m, h] = sum over the routed slots in slot order of wts[m, k] * part[row(m, k), h], plus the shared expert's
// row.  row(m, k) = m * ns + k, or posof[m * ns + k] when the rows were grouped by expert.
__global__ void k_moe_combine(float* __restrict__ y, const float* __restrict__ part, const float* __restrict__ wts,
                              const int* __restrict__ posof, int M, int topk, int ns, int H) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;          // float4 index
    const int per = H >> 2;
    if (i >= M * per) return;
    const int m = i / per, h4 = i - m * per;
    const float4* p = reinterpret_cast<const float4*>(part) + h4;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k = 0; k < topk; ++k) {
        const float w = wts[(size_t)m * topk + k];
        const int row = posof ? posof[m * ns + k] : m * ns + k;
        const float4 v = p[(size_t)row * per];
        acc.x = fmaf(w, v.x, acc.x); acc.y = fmaf(w, v.y, acc.y); acc.z = fmaf(w, v.z, acc.z); acc.w = fmaf(w, v.w, acc.w);
    }
    if (ns > topk) {
        const int row = posof ? posof[m * ns + topk] : m * ns + topk;
        const float4 v = p[(size_t)row * per];
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    reinterpret_cast<float4*>(y)[i] = acc;
}

// ---- more than 8 tokens: rows grouped by expert ---------------------------------------------------
// One CTA sorts the (token, slot) pairs by expert (counting sort; the order inside an expert's
// group is whatever the atomics give, which is harmless: every row is computed on its own) and
// writes one job per expert and chunk of up to 8 rows, so that an expert's weights are read once
// per 8 rows that chose it.  Job slots beyond the ones needed get N = 0 and their CTAs return at once.
constexpr int MG_MAX_GROUPS = 513;                   // n_expert <= 512, plus the shared expert

__global__ void __launch_bounds__(1024)
k_moe_group(const __grid_constant__ MoePlan q, const int32_t* __restrict__ sel, int* __restrict__ posof,
            const float* __restrict__ xg, SplitJob* __restrict__ s1, SplitJob* __restrict__ s2,
            unsigned char* __restrict__ img1, unsigned char* __restrict__ img2, float* __restrict__ gam1,
            float* __restrict__ gam2, int M, int max_jobs, unsigned long long* __restrict__ credit_jobs) {
    __shared__ int cnt[MG_MAX_GROUPS], off[MG_MAX_GROUPS], jstart[MG_MAX_GROUPS], cursor[MG_MAX_GROUPS];
    __shared__ int total_jobs;
    const int G = q.E + 1, pairs = M * q.ns;
    for (int e = threadIdx.x; e < G; e += blockDim.x) { cnt[e] = 0; cursor[e] = 0; }
    __syncthreads();
    auto group_of = [&](int p) {
        const int m = p / q.ns, slot = p - m * q.ns;
        if (slot >= q.topk) return q.E;
        const int e = sel[(size_t)m * q.topk + slot];
        return e < 0 ? 0 : (e >= q.E ? q.E - 1 : e);
    };
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) atomicAdd(&cnt[group_of(p)], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int o = 0, j = 0;
        for (int e = 0; e < G; ++e) { off[e] = o; jstart[e] = j; o += cnt[e]; j += (cnt[e] + 7) >> 3; }
        total_jobs = j;
        if (credit_jobs) { atomicAdd(&credit_jobs[0], 2ull * j); atomicAdd(&credit_jobs[1], (unsigned long long)j); }   // passes over expert matrices: gate + up, down
    }
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = group_of(p);
        posof[p] = off[e] + atomicAdd(&cursor[e], 1);
    }
    for (int e = threadIdx.x; e < G; e += blockDim.x) {
        const b200_nvfp4_mat* mats = e < q.E ? q.experts + (size_t)e * 3 : q.shared;
        const unsigned char* mp = q.maps + (size_t)e * 6 * 128;
        for (int c = 0; c * 8 < cnt[e]; ++c) {
            const int idx = jstart[e] + c, rows = min(8, cnt[e] - 8 * c);
            const size_t pos0 = (size_t)off[e] + 8 * c;
            float* g = q.gbuf + pos0 * q.I;
            float* u = q.ubuf + pos0 * q.I;
            // the chunk's rows are split once (k_split_rows) for all the CTAs of its jobs
            unsigned char* b1 = img1 + (size_t)idx * (q.H >> 8) * 8192;
            unsigned char* b2 = img2 + (size_t)idx * (q.I >> 8) * 8192;
            float* ga1 = gam1 + (size_t)idx * 64;
            float* ga2 = gam2 + (size_t)idx * 64;
            s1[idx] = SplitJob{xg + pos0 * q.H, nullptr, b1, ga1, rows, 0};
            s2[idx] = SplitJob{g, u, b2, ga2, rows, 0};
            q.j1[2 * idx] = UmJob{g, nullptr, nullptr, mats[0].gscale, mp, mp + 128, b1, ga1, q.I, rows, 0, 0};
            q.j1[2 * idx + 1] = UmJob{u, nullptr, nullptr, mats[1].gscale, mp + 256, mp + 384, b1, ga1, q.I, rows, 0, 0};
            q.j2[idx] = UmJob{q.part + pos0 * q.H, nullptr, nullptr, mats[2].gscale, mp + 512, mp + 640, b2, ga2, q.H, rows, 0, 0};
        }
    }
    for (int idx = total_jobs + threadIdx.x; idx < max_jobs; idx += blockDim.x) {
        const UmJob none{nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, 0, 0, 0, 0};
        q.j1[2 * idx] = none; q.j1[2 * idx + 1] = none; q.j2[idx] = none;
        s1[idx] = SplitJob{nullptr, nullptr, nullptr, nullptr, 0, 0}; s2[idx] = s1[idx];
    }
}

// xg[posof[p], :] = x[token of pair p, :]
__global__ void k_moe_gather(float* __restrict__ xg, const float* __restrict__ x, const int* __restrict__ posof,
                             int pairs, int ns, int H) {
    const int per = H >> 2;
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)pairs * per) return;
    const int p = (int)(i / per), h4 = (int)(i - (size_t)p * per);
    reinterpret_cast<float4*>(xg)[(size_t)posof[p] * per + h4] = reinterpret_cast<const float4*>(x)[(size_t)(p / ns) * per + h4];
}

static size_t up256(size_t v) { return (v + 255) / 256 * 256; }

static int grouped_max_jobs(const b200_moe_layer* L, int M) { return (M * (L->topk + 1) + 7) / 8 + L->n_expert + 1; }

// Scratch of the tensor-core path behind the logits.  Up to 8 tokens: job tables | gate products |
// up products | down products, one row per (token, slot) pair.  More: pair positions | job tables |
// gathered activations | gate | up | down products, rows grouped by expert.
static size_t moe_gx_ws_bytes(const b200_moe_layer* L, int M);
size_t moe_umma_ws_bytes(const b200_moe_layer* L, int M) {
    const size_t ns = (size_t)L->topk + 1, pairs = (size_t)M * ns;
    size_t small = 0;
    if (M <= MU_MAX_TOKENS)
        small = std::max(moe_gx_ws_bytes(L, M), up256(pairs * 3 * sizeof(UmJob)) + 2 * up256(pairs * L->inter * 4) + up256(pairs * L->hidden * 4));
    const size_t mj = (size_t)grouped_max_jobs(L, M);
    return std::max(std::max(small, moe_gx_ws_bytes(L, M)), up256(pairs * 4) + up256(mj * 3 * sizeof(UmJob)) + 2 * up256(mj * sizeof(SplitJob)) + 2 * up256(mj * 64 * 4) +
           up256(mj * (L->hidden >> 8) * 8192) + up256(mj * (L->inter >> 8) * 8192) +
           2 * up256(pairs * L->hidden * 4) + 2 * up256(pairs * L->inter * 4));
}

// Fills `q` for a call on a prepared layer.  B200_ENOTIMPL: not prepared, too many tokens, or an
// unaligned activation -> the caller runs the CUDA-core experts.
int moe_umma_plan_args(const float* x, const b200_moe_layer* L, void* scratch, int M, MoePlan* q, int* R_gu, int* R_d) {
    if (M > MU_MAX_TOKENS || M >= group_min_tokens() || ((uintptr_t)x & 15)) return B200_ENOTIMPL;
    Prepared Pc;
    if (!find_prepared(L, &Pc)) return B200_ENOTIMPL;
    const Prepared* P = &Pc;
    const int ns = L->topk + (L->shared ? 1 : 0), pairs = M * ns, H = L->hidden, I = L->inter;
    char* w = static_cast<char*>(scratch);
    q->j1 = reinterpret_cast<UmJob*>(w);
    q->j2 = q->j1 + (size_t)2 * pairs;
    w += up256((size_t)M * (L->topk + 1) * 3 * sizeof(UmJob));
    q->gbuf = reinterpret_cast<float*>(w); w += up256((size_t)M * (L->topk + 1) * I * 4);
    q->ubuf = reinterpret_cast<float*>(w); w += up256((size_t)M * (L->topk + 1) * I * 4);
    q->part = reinterpret_cast<float*>(w);
    q->experts = L->experts; q->shared = L->shared; q->maps = P->maps; q->x = x;
    q->topk = L->topk; q->ns = ns; q->E = L->n_expert; q->H = H; q->I = I;
    *R_gu = P->R_gu; *R_d = P->R_d;
    return B200_OK;
}

// More than 8 tokens on a prepared layer.
static int moe_umma_grouped(const float* x, const b200_moe_layer* L, float* y, const int32_t* sel, const float* wts,
                            void* scratch, int M, cudaStream_t s) {
    if (((uintptr_t)x & 15) || L->n_expert + 1 > MG_MAX_GROUPS) return B200_ENOTIMPL;
    Prepared Pc;
    if (!find_prepared(L, &Pc)) return B200_ENOTIMPL;
    const Prepared* P = &Pc;
    const int ns = L->topk + (L->shared ? 1 : 0), pairs = M * ns, H = L->hidden, I = L->inter;
    const int max_jobs = grouped_max_jobs(L, M);
    const size_t np = (size_t)M * (L->topk + 1);     // the sizes the workspace was laid out with
    char* w = static_cast<char*>(scratch);
    int* posof = reinterpret_cast<int*>(w); w += up256(np * 4);
    MoePlan q{};
    q.j1 = reinterpret_cast<UmJob*>(w); q.j2 = q.j1 + (size_t)2 * max_jobs; w += up256((size_t)max_jobs * 3 * sizeof(UmJob));
    SplitJob* s1 = reinterpret_cast<SplitJob*>(w); w += up256((size_t)max_jobs * sizeof(SplitJob));
    SplitJob* s2 = reinterpret_cast<SplitJob*>(w); w += up256((size_t)max_jobs * sizeof(SplitJob));
    float* gam1 = reinterpret_cast<float*>(w); w += up256((size_t)max_jobs * 64 * 4);
    float* gam2 = reinterpret_cast<float*>(w); w += up256((size_t)max_jobs * 64 * 4);
    unsigned char* img1 = reinterpret_cast<unsigned char*>(w); w += up256((size_t)max_jobs * (H >> 8) * 8192);
    unsigned char* img2 = reinterpret_cast<unsigned char*>(w); w += up256((size_t)max_jobs * (I >> 8) * 8192);
    float* xg = reinterpret_cast<float*>(w); w += up256(np * H * 4);
    q.part = reinterpret_cast<float*>(w); w += up256(np * H * 4);
    q.gbuf = reinterpret_cast<float*>(w); w += up256(np * I * 4);
    q.ubuf = reinterpret_cast<float*>(w);
    q.experts = L->experts; q.shared = L->shared; q.maps = P->maps; q.x = x;
    q.topk = L->topk; q.ns = ns; q.E = L->n_expert; q.H = H; q.I = I;
    if (credit_on()) credit_grouped_geometry(H, I);
    k_moe_group<<<1, 1024, 0, s>>>(q, sel, posof, xg, s1, s2, img1, img2, gam1, gam2, M, max_jobs, credit_on() ? credit_counters() : nullptr);
    if (int rc = check_launch("k_moe_group")) return rc;
    const size_t n4 = (size_t)pairs * (H >> 2);
    k_moe_gather<<<(unsigned)((n4 + 255) / 256), 256, 0, s>>>(xg, x, posof, pairs, ns, H);
    if (int rc = check_launch("k_moe_gather")) return rc;
    if (int rc = umma_split_launch(s1, max_jobs, H, 0.f, s)) return rc;
    if (int rc = umma_table_launch(q.j1, 2 * max_jobs, I, H, P->R_gu, 0.f, 8, s)) return rc == B200_ENOTIMPL ? B200_ELAUNCH : rc;
    if (int rc = umma_split_launch(s2, max_jobs, I, L->swiglu_limit, s)) return rc;
    if (int rc = umma_table_launch(q.j2, max_jobs, H, I, P->R_d, L->swiglu_limit, 8, s)) return rc == B200_ENOTIMPL ? B200_ELAUNCH : rc;
    const int y4 = M * (H >> 2);
    k_moe_combine<<<(y4 + 255) / 256, 256, 0, s>>>(y, q.part, wts, posof, M, q.topk, ns, H);
    return check_launch("k_moe_combine");
}

// ---- 16 tokens and more: rows grouped by expert, both GEMM operands in NVFP4 -----------------------
// Same counting sort as k_moe_group, but the jobs are those of the wide GEMM (gemm_mxf4.cu): one job
// per expert and chunk of up to NT rows, so that an expert's weights are read once per NT rows that
// chose it (the passes of 8 rows above re-read them NT/8 times).  src_row[pos] = token of the pair
// sorted to position pos: the activation quantiser gathers with it.
__global__ void __launch_bounds__(1024)
k_moe_group_gx(const __grid_constant__ MoePlan q, const int32_t* __restrict__ sel, int* __restrict__ posof,
               int* __restrict__ src_row, GxJob* __restrict__ j1, GxJob* __restrict__ j2,
               const float* __restrict__ gsx1, const float* __restrict__ gsx2, int M, int NT, int max_jobs,
               unsigned long long* __restrict__ credit_jobs) {
    __shared__ int cnt[MG_MAX_GROUPS], off[MG_MAX_GROUPS], jstart[MG_MAX_GROUPS], cursor[MG_MAX_GROUPS];
    __shared__ int total_jobs;
    pdl_wait();
    const int G = q.E + 1, pairs = M * q.ns;
    for (int e = threadIdx.x; e < G; e += blockDim.x) { cnt[e] = 0; cursor[e] = 0; }
    __syncthreads();
    auto group_of = [&](int p) {
        const int m = p / q.ns, slot = p - m * q.ns;
        if (slot >= q.topk) return q.E;
        const int e = sel[(size_t)m * q.topk + slot];
        return e < 0 ? 0 : (e >= q.E ? q.E - 1 : e);
    };
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) atomicAdd(&cnt[group_of(p)], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int o = 0, j = 0;
        for (int e = 0; e < G; ++e) { off[e] = o; jstart[e] = j; o += cnt[e]; j += (cnt[e] + NT - 1) / NT; }
        total_jobs = j;
        if (credit_jobs) { atomicAdd(&credit_jobs[0], 2ull * j); atomicAdd(&credit_jobs[1], (unsigned long long)j); }   // passes over expert matrices: gate + up, down
    }
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = group_of(p), pos = off[e] + atomicAdd(&cursor[e], 1);
        posof[p] = pos;
        src_row[pos] = p / q.ns;
    }
    for (int e = threadIdx.x; e < G; e += blockDim.x) {
        const b200_nvfp4_mat* mats = e < q.E ? q.experts + (size_t)e * 3 : q.shared;
        const unsigned char* mp = q.maps + (size_t)(q.E + 1) * 6 * 128 + (size_t)e * 6 * 128;     // the 128-row boxes
        for (int c = 0; c * NT < cnt[e]; ++c) {
            const int idx = jstart[e] + c, rows = min(NT, cnt[e] - NT * c), pos0 = off[e] + NT * c;
            j1[2 * idx] = GxJob{q.gbuf + (size_t)pos0 * q.I, mats[0].gscale, gsx1 + pos0, mp, mp + 128, pos0, rows, q.I, q.I};
            j1[2 * idx + 1] = GxJob{q.ubuf + (size_t)pos0 * q.I, mats[1].gscale, gsx1 + pos0, mp + 256, mp + 384, pos0, rows, q.I, q.I};
            j2[idx] = GxJob{q.part + (size_t)pos0 * q.H, mats[2].gscale, gsx2 + pos0, mp + 512, mp + 640, pos0, rows, q.H, q.H};
        }
    }
    for (int idx = total_jobs + threadIdx.x; idx < max_jobs; idx += blockDim.x) {
        const GxJob none{nullptr, nullptr, nullptr, nullptr, nullptr, 0, 0, 0, 0};
        j1[2 * idx] = none; j1[2 * idx + 1] = none; j2[idx] = none;
    }
}

// Token tile of the grouped wide GEMM: narrow while few rows share an expert (a job's cost is its
// expert's weights whatever its width, and narrow tiles keep more stages in flight).
static int gx_tile(int M) { return M <= 64 ? 32 : (M <= 256 ? 64 : 128); }
static int gx_max_jobs(const b200_moe_layer* L, int M) { return (M * (L->topk + 1)) / gx_tile(M) + L->n_expert + 1; }

static size_t moe_gx_ws_bytes(const b200_moe_layer* L, int M) {
    const size_t np = (size_t)M * (L->topk + 1), mj = (size_t)gx_max_jobs(L, M), padrows = np + 256;
    const size_t H = L->hidden, I = L->inter;
    return 2 * up256(np * 4) + up256(mj * 3 * sizeof(GxJob)) +
           up256(np * (H / 2)) + up256(padrows * (H / 16)) + up256(np * 4) +          // quantised token rows
           up256(np * (I / 2)) + up256(padrows * (I / 16)) + up256(np * 4) +          // quantised SwiGLU rows
           2 * up256(np * I * 4) + up256(np * H * 4);                                 // gate, up, down products
}

static int moe_gx_grouped(const float* x, const b200_moe_layer* L, float* y, const int32_t* sel, const float* wts,
                          void* scratch, int M, cudaStream_t s) {
    if (((uintptr_t)x & 15) || L->n_expert + 1 > MG_MAX_GROUPS || !gemm_mxf4_shape_ok(L->hidden) || !gemm_mxf4_shape_ok(L->inter)) return B200_ENOTIMPL;
    Prepared Pc;
    if (!find_prepared(L, &Pc)) return B200_ENOTIMPL;
    const Prepared* P = &Pc;
    const int ns = L->topk + (L->shared ? 1 : 0), pairs = M * ns, H = L->hidden, I = L->inter;
    const int NT = gx_tile(M), max_jobs = gx_max_jobs(L, M);
    const size_t np = (size_t)M * (L->topk + 1), padrows = np + 256;
    char* w = static_cast<char*>(scratch);
    int* posof = reinterpret_cast<int*>(w); w += up256(np * 4);
    int* src_row = reinterpret_cast<int*>(w); w += up256(np * 4);
    GxJob* j1 = reinterpret_cast<GxJob*>(w); GxJob* j2 = j1 + (size_t)2 * max_jobs; w += up256((size_t)max_jobs * 3 * sizeof(GxJob));
    unsigned char* xq1 = reinterpret_cast<unsigned char*>(w); w += up256(np * (H / 2));
    unsigned char* sf1 = reinterpret_cast<unsigned char*>(w); w += up256(padrows * (H / 16));
    float* gs1 = reinterpret_cast<float*>(w); w += up256(np * 4);
    unsigned char* xq2 = reinterpret_cast<unsigned char*>(w); w += up256(np * (I / 2));
    unsigned char* sf2 = reinterpret_cast<unsigned char*>(w); w += up256(padrows * (I / 16));
    float* gs2 = reinterpret_cast<float*>(w); w += up256(np * 4);
    MoePlan q{};
    q.gbuf = reinterpret_cast<float*>(w); w += up256(np * I * 4);
    q.ubuf = reinterpret_cast<float*>(w); w += up256(np * I * 4);
    q.part = reinterpret_cast<float*>(w);
    q.experts = L->experts; q.shared = L->shared; q.maps = P->maps; q.x = x;
    q.topk = L->topk; q.ns = ns; q.E = L->n_expert; q.H = H; q.I = I;
    if (credit_on()) credit_grouped_geometry(H, I);
    k_moe_group_gx<<<1, 1024, 0, s>>>(q, sel, posof, src_row, j1, j2, gs1, gs2, M, NT, max_jobs, credit_on() ? credit_counters() : nullptr);
    if (int rc = check_launch("k_moe_group_gx")) return rc;
    if (int rc = quant_act_launch(1, x, nullptr, 0.f, src_row, nullptr, pairs, pairs, H, xq1, sf1, padrows, gs1, s)) return rc;
    // jobs the table is likely to hold: every expert that can be hit once, plus the extra chunks of busy experts
    const long expect = std::min<long>(L->n_expert, (long)M * L->topk) + (L->shared ? 1 : 0) + pairs / NT;
    if (int rc = gemm_mxf4_table(j1, 2 * max_jobs, 2 * expect, NT, I, H, 128, xq1, (size_t)pairs, sf1, padrows, s)) return rc == B200_ENOTIMPL ? B200_ELAUNCH : rc;
    if (int rc = quant_act_launch(2, q.gbuf, q.ubuf, L->swiglu_limit, nullptr, nullptr, pairs, pairs, I, xq2, sf2, padrows, gs2, s)) return rc;
    if (int rc = gemm_mxf4_table(j2, max_jobs, expect, NT, H, I, 128, xq2, (size_t)pairs, sf2, padrows, s)) return rc == B200_ENOTIMPL ? B200_ELAUNCH : rc;
    const int y4 = M * (H >> 2);
    k_moe_combine<<<(y4 + 255) / 256, 256, 0, s>>>(y, q.part, wts, posof, M, q.topk, ns, H);
    return check_launch("k_moe_combine");
}

// The experts of a call on a prepared layer.  planned: the job tables were already written (by the router).
int moe_umma_experts(const float* x, const b200_moe_layer* L, float* y, const int32_t* sel, const float* wts,
                     void* scratch, int M, cudaStream_t s, bool planned, int wide) {
    // wide: 1 = the grouped wide GEMM whatever M, 0 = never, -1 = by this call's row count
    if (wide < 0) wide = M >= PREFILL_MIN_ROWS && prefill_fp4_option();
    if (wide) {                                                    // prefill widths: an expert's weights once per up to 128 rows
        const int rc = moe_gx_grouped(x, L, y, sel, wts, scratch, M, s);
        if (rc != B200_ENOTIMPL) return rc;
    }
    if (M >= group_min_tokens()) return moe_umma_grouped(x, L, y, sel, wts, scratch, M, s);
    MoePlan q{};
    int R_gu = 0, R_d = 0;
    if (int rc = moe_umma_plan_args(x, L, scratch, M, &q, &R_gu, &R_d)) return rc;
    const int pairs = M * q.ns;
    credit(B200_CREDIT_MOE_ACT, (double)pairs * 2.0 * q.I * q.H * 0.5625);      // every pair streams its expert (reference kernels/moe.cu:719-722)
    credit(B200_CREDIT_MOE_DOWN, (double)pairs * 1.0 * q.I * q.H * 0.5625);
    if (!planned) {
        k_moe_plan<<<(pairs + 127) / 128, 128, 0, s>>>(q, sel, M);
        if (int rc = check_launch("k_moe_plan")) return rc;
    }
    if (int rc = umma_table_launch(q.j1, 2 * pairs, q.I, q.H, R_gu, 0.f, 1, s)) return rc == B200_ENOTIMPL ? B200_ELAUNCH : rc;
    if (int rc = umma_table_launch(q.j2, pairs, q.H, q.I, R_d, L->swiglu_limit, 1, s)) return rc == B200_ENOTIMPL ? B200_ELAUNCH : rc;
    const int n4 = M * (q.H >> 2);
    k_moe_combine<<<(n4 + 255) / 256, 256, 0, s>>>(y, q.part, wts, nullptr, M, q.topk, q.ns, q.H);
    return check_launch("k_moe_combine");
}

}  // namespace b200

using namespace b200;

extern "C" int b200_moe_prepare(const b200_moe_layer* L) {
    if (!L || !L->experts || L->n_expert < 1 || L->hidden <= 0 || L->inter <= 0) return B200_EINVAL;
    if (find_prepared(L, nullptr)) return B200_OK;
    if (!umma_shape_ok(L->hidden) || !umma_shape_ok(L->inter) || (L->hidden & 3)) return B200_ENOTIMPL;
    const int E = L->n_expert, nexp = E + 1;
    std::vector<b200_nvfp4_mat> mats((size_t)nexp * 3);
    if (cudaMemcpy(mats.data(), L->experts, (size_t)E * 3 * sizeof(b200_nvfp4_mat), cudaMemcpyDeviceToHost) != cudaSuccess)
        return launch_failed("moe_prepare: expert table copy");
    if (L->shared) {
        if (cudaMemcpy(mats.data() + (size_t)E * 3, L->shared, 3 * sizeof(b200_nvfp4_mat), cudaMemcpyDeviceToHost) != cudaSuccess)
            return launch_failed("moe_prepare: shared expert table copy");
    } else {
        for (int q = 0; q < 3; ++q) mats[(size_t)E * 3 + q] = mats[q];       // never selected: ns == topk
    }
    Prepared P{};
    P.experts = L->experts; P.shared = L->shared; P.E = E; P.H = L->hidden; P.I = L->inter;
    const int ns = L->topk + (L->shared ? 1 : 0);
    P.R_gu = pick_rows(2 * ns, L->inter);
    P.R_d = pick_rows(ns, L->hidden);
    std::vector<unsigned char> host((size_t)nexp * 12 * 128);
    for (int e = 0; e < nexp; ++e) {
        const b200_nvfp4_mat* m = &mats[(size_t)e * 3];
        unsigned char* o = host.data() + (size_t)e * 6 * 128;
        if (umma_encode_maps(o, o + 128, m[0].packed, m[0].scale, L->inter, L->hidden, P.R_gu) ||
            umma_encode_maps(o + 256, o + 384, m[1].packed, m[1].scale, L->inter, L->hidden, P.R_gu) ||
            umma_encode_maps(o + 512, o + 640, m[2].packed, m[2].scale, L->hidden, L->inter, P.R_d)) return B200_ENOTIMPL;
        o += (size_t)nexp * 6 * 128;                     // the wide GEMM's boxes: always 128 rows
        if (umma_encode_maps(o, o + 128, m[0].packed, m[0].scale, L->inter, L->hidden, 128) ||
            umma_encode_maps(o + 256, o + 384, m[1].packed, m[1].scale, L->inter, L->hidden, 128) ||
            umma_encode_maps(o + 512, o + 640, m[2].packed, m[2].scale, L->hidden, L->inter, 128)) return B200_ENOTIMPL;
    }
    if (cudaGetDevice(&P.device) != cudaSuccess) return launch_failed("moe_prepare: cudaGetDevice");
    if (cudaMalloc(&P.maps, host.size()) != cudaSuccess) return launch_failed("moe_prepare: cudaMalloc");
    if (cudaMemcpy(P.maps, host.data(), host.size(), cudaMemcpyHostToDevice) != cudaSuccess) { cudaFree(P.maps); return launch_failed("moe_prepare: upload"); }
    std::lock_guard<std::mutex> lk(g_prepared_mu);
    for (Prepared& q : g_prepared)
        if (!q.maps) { q = P; return B200_OK; }          // a released slot
    g_prepared.push_back(P);
    return B200_OK;
}

extern "C" int b200_moe_release(const b200_moe_layer* L) {
    if (!L) return B200_EINVAL;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) return B200_ELAUNCH;
    std::lock_guard<std::mutex> lk(g_prepared_mu);
    for (Prepared& p : g_prepared)
        if (p.experts == L->experts && p.shared == L->shared && p.device == dev && p.maps) {
            cudaFree(p.maps);                            // waits for the device: queued launches on this layer have finished
            p.maps = nullptr; p.experts = nullptr; p.shared = nullptr; p.E = -1;   // the slot is free for the next prepare
            return B200_OK;
        }
    return B200_EINVAL;
}
