// moe_umma.cu -- the MoE experts on the tensor-core gemv kernel (gemv_umma.cu), for decode batches
// of up to 8 tokens, once b200_moe_prepare() has been called for the layer.
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
// Every (token, slot) pair is its own single-row job, the shared expert included (its weights
// are read once from HBM and then from L2): a token's result does not depend on what else is
// in the batch, bit for bit.  The gate-weighted sum runs over the slots in slot order.
#include "b200_internal.h"
#include "moe_plan.cuh"
#include <cstdio>
#include <cstring>
#include <mutex>
#include <vector>

namespace b200 {

constexpr int MU_MAX_TOKENS = 8;

struct Prepared {
    const b200_nvfp4_mat* experts; const b200_nvfp4_mat* shared;     // key
    int E, H, I;
    unsigned char* maps;          // device: [(E + 1) experts][3 matrices][w, s] x 128 bytes; shared expert last
    int R_gu, R_d;
    int device;
};
static std::vector<Prepared> g_prepared;
static std::mutex g_prepared_mu;

static const Prepared* find_prepared(const b200_moe_layer* L) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
    std::lock_guard<std::mutex> lk(g_prepared_mu);
    for (const Prepared& p : g_prepared)
        if (p.experts == L->experts && p.shared == L->shared && p.E == L->n_expert && p.H == L->hidden && p.I == L->inter && p.device == dev)
            return &p;                                   // entries are never removed or moved while in use: see release
    return nullptr;
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

// y[m, h] = sum over the routed slots in slot order of wts[m, k] * part[m, k, h], plus the shared expert's row.
__global__ void k_moe_combine(float* __restrict__ y, const float* __restrict__ part, const float* __restrict__ wts,
                              int M, int topk, int ns, int H) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;          // float4 index
    const int per = H >> 2;
    if (i >= M * per) return;
    const int m = i / per, h4 = i - m * per;
    const float4* p = reinterpret_cast<const float4*>(part + (size_t)m * ns * H) + h4;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k = 0; k < topk; ++k) {
        const float w = wts[(size_t)m * topk + k];
        const float4 v = p[(size_t)k * per];
        acc.x = fmaf(w, v.x, acc.x); acc.y = fmaf(w, v.y, acc.y); acc.z = fmaf(w, v.z, acc.z); acc.w = fmaf(w, v.w, acc.w);
    }
    if (ns > topk) {
        const float4 v = p[(size_t)topk * per];
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    reinterpret_cast<float4*>(y)[i] = acc;
}

static size_t up256(size_t v) { return (v + 255) / 256 * 256; }

// Scratch of the tensor-core path behind the logits: job tables | gate products | up products | down products.
size_t moe_umma_ws_bytes(const b200_moe_layer* L, int M) {
    const size_t ns = (size_t)L->topk + 1, pairs = (size_t)M * ns;
    return up256(pairs * 3 * sizeof(UmJob)) + 2 * up256(pairs * L->inter * 4) + up256(pairs * L->hidden * 4);
}

// Fills `q` for a call on a prepared layer.  B200_ENOTIMPL: not prepared, too many tokens, or an
// unaligned activation -> the caller runs the CUDA-core experts.
int moe_umma_plan_args(const float* x, const b200_moe_layer* L, void* scratch, int M, MoePlan* q, int* R_gu, int* R_d) {
    if (M > MU_MAX_TOKENS || ((uintptr_t)x & 15)) return B200_ENOTIMPL;
    const Prepared* P = find_prepared(L);
    if (!P) return B200_ENOTIMPL;
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

// The experts of a planned call.  planned: the job tables were already written (by the router).
int moe_umma_experts(const float* x, const b200_moe_layer* L, float* y, const int32_t* sel, const float* wts,
                     void* scratch, int M, cudaStream_t s, bool planned) {
    MoePlan q{};
    int R_gu = 0, R_d = 0;
    if (int rc = moe_umma_plan_args(x, L, scratch, M, &q, &R_gu, &R_d)) return rc;
    const int pairs = M * q.ns;
    if (!planned) {
        k_moe_plan<<<(pairs + 127) / 128, 128, 0, s>>>(q, sel, M);
        if (int rc = check_launch("k_moe_plan")) return rc;
    }
    if (int rc = umma_table_launch(q.j1, 2 * pairs, q.I, q.H, R_gu, 0.f, s)) return rc == B200_ENOTIMPL ? B200_ELAUNCH : rc;
    if (int rc = umma_table_launch(q.j2, pairs, q.H, q.I, R_d, L->swiglu_limit, s)) return rc == B200_ENOTIMPL ? B200_ELAUNCH : rc;
    const int n4 = M * (q.H >> 2);
    k_moe_combine<<<(n4 + 255) / 256, 256, 0, s>>>(y, q.part, wts, M, q.topk, q.ns, q.H);
    return check_launch("k_moe_combine");
}

}  // namespace b200

using namespace b200;

extern "C" int b200_moe_prepare(const b200_moe_layer* L) {
    if (!L || !L->experts || L->n_expert < 1 || L->hidden <= 0 || L->inter <= 0) return B200_EINVAL;
    if (find_prepared(L)) return B200_OK;
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
    std::vector<unsigned char> host((size_t)nexp * 6 * 128);
    for (int e = 0; e < nexp; ++e) {
        const b200_nvfp4_mat* m = &mats[(size_t)e * 3];
        unsigned char* o = host.data() + (size_t)e * 6 * 128;
        if (umma_encode_maps(o, o + 128, m[0].packed, m[0].scale, L->inter, L->hidden, P.R_gu) ||
            umma_encode_maps(o + 256, o + 384, m[1].packed, m[1].scale, L->inter, L->hidden, P.R_gu) ||
            umma_encode_maps(o + 512, o + 640, m[2].packed, m[2].scale, L->hidden, L->inter, P.R_d)) return B200_ENOTIMPL;
    }
    if (cudaGetDevice(&P.device) != cudaSuccess) return launch_failed("moe_prepare: cudaGetDevice");
    if (cudaMalloc(&P.maps, host.size()) != cudaSuccess) return launch_failed("moe_prepare: cudaMalloc");
    if (cudaMemcpy(P.maps, host.data(), host.size(), cudaMemcpyHostToDevice) != cudaSuccess) { cudaFree(P.maps); return launch_failed("moe_prepare: upload"); }
    std::lock_guard<std::mutex> lk(g_prepared_mu);
    g_prepared.reserve(4096);                            // pointers into the vector stay valid
    if (g_prepared.size() >= 4096) { cudaFree(P.maps); return B200_ELIMIT; }
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
            cudaFree(p.maps); p.maps = nullptr; p.experts = nullptr; p.shared = nullptr; p.E = -1;   // slot stays, never matches again
            return B200_OK;
        }
    return B200_EINVAL;
}
