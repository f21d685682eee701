// moe_plan.cuh -- job records of the tensor-core MoE path for one (token, slot) pair.
#pragma once
#include "b200_internal.h"

namespace b200 {

// Where the job tables, the per-expert tensor maps and the intermediate buffers of one call live.
// j1 == nullptr: no plan wanted.
struct MoePlan {
    UmJob* j1; UmJob* j2;                          // gate/up jobs [2 * pairs], down jobs [pairs]
    const b200_nvfp4_mat* experts; const b200_nvfp4_mat* shared;
    const unsigned char* maps;                     // [(E + 1) experts][gate w,s | up w,s | down w,s] x 128 bytes
    const float* x; float* gbuf; float* ubuf; float* part;
    int topk, ns, E, H, I;
};

// Pair (token m, slot): slot < topk is routed expert e, slot == topk the shared expert.
__device__ __forceinline__ void moe_plan_pair(const MoePlan& q, int m, int slot, int e) {
    const int pair = m * q.ns + slot;
    const b200_nvfp4_mat* mats = q.shared;
    if (slot < q.topk) { e = e < 0 ? 0 : (e >= q.E ? q.E - 1 : e); mats = q.experts + (size_t)e * 3; }
    else e = q.E;                                  // the shared expert's maps come last
    const unsigned char* mp = q.maps + (size_t)e * 6 * 128;
    const float* xm = q.x + (size_t)m * q.H;
    float* g = q.gbuf + (size_t)pair * q.I;
    float* u = q.ubuf + (size_t)pair * q.I;
    q.j1[2 * pair] = UmJob{g, xm, nullptr, mats[0].gscale, mp, mp + 128, nullptr, nullptr, q.I, 1, 0, 0};
    q.j1[2 * pair + 1] = UmJob{u, xm, nullptr, mats[1].gscale, mp + 256, mp + 384, nullptr, nullptr, q.I, 1, 0, 0};
    q.j2[pair] = UmJob{q.part + (size_t)pair * q.H, g, u, mats[2].gscale, mp + 512, mp + 640, nullptr, nullptr, q.H, 1, 0, 0};
}

}  // namespace b200
