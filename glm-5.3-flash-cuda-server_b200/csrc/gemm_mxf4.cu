// gemm_mxf4.cu -- the wide (prefill / batched, M >= 16) NVFP4 GEMM: y[M,N] = x[M,K] . W[N,K]^T on
// tcgen05.mma kind::mxf4nvf4.block_scale.block16 with BOTH operands in NVFP4.
//
// The weights are used exactly as the format stores them (packed e2m1 bytes and e4m3 block
// scales, read through TMA).  The activations are quantised to NVFP4 first, one token at a time,
// by k_quant_act: the reference's own quant_block rule (tools/requant_dense_nvfp4.py:53-68) with a
// per-token global scale 2688 / amax(token), so that a token's result never depends on the rest of
// its batch.  That costs about 9 % per-element activation error; results are therefore judged against
// deq(W) . deq(quant(x)), and the library keeps the exact small-batch kernels (gemv_umma.cu) for
// callers that want fp32-activation accuracy.  The reference streams W once per chunk of 4 rows
// (kernels/gemv.cu:369-396); here W is read ONCE for up to 256 rows.
//
// One CTA per (tile of R <= 128 weight rows, job of up to NT activation rows); K walked in steps of
// 256.  The accumulator D[128 weight rows (lanes), NT tokens (columns)] stays in TMEM for the whole K.
//   warp 0      TMA producer: the tile's weight scale rows once (slabs [R x 128 B]); per step one
//               128B-swizzled box of packed weights [128 B x R], one of packed activations
//               [128 B x NT] and the step's activation scales (one contiguous NT x 16 B chunk: the
//               quantiser writes them step-major) into a ring of stages.  Lane l issues steps l, l+32, ..
//   warp 1      MMA issuer: four tcgen05.mma (K = 64 each, N = NT) per step, tcgen05.commit frees the stage
//   warp 2      allocates / frees TMEM
//   warps 4-11  two groups of four warps (one per TMEM lane quadrant) on alternate steps move the
//               step's scales into TMEM with tcgen05.st (lane r % 32, column r / 32: the layout the
//               block-scaled MMA reads): 16 columns for the weights' 128 x 16 scale bytes, NT/8 for the
//               activations'.  Afterwards each group reads half of the accumulator columns, applies
//               1 / (gs_w * gs_x[token]) and writes y (lanes = consecutive n: coalesced).
// Barriers full/sf/empty are per step and used once (K <= 16384: at most 64 steps).  Every wait is
// bounded (tma_pipe.cuh).  No cluster launch, no multicast.
#include "b200_internal.h"
#include "quant_core.cuh"
#include "tma_pipe.cuh"
#include <cuda.h>
#include <cstdio>
#include <cstdlib>

namespace b200 {

constexpr int GX_THREADS = 384;
constexpr int GX_MOVERS = 256;
constexpr int GX_MAX_STEPS = 64;                   // K <= 16384
constexpr int GX_MAX_STAGES = 8;
constexpr int GX_MAX_SLABS = 16;                   // scale slabs per CTA (a slab covers 8 steps, or a whole tile when K/16 < 128)
constexpr int GX_TMEM_COLS = 512;                  // accumulator [0, NT) | scale slots from column 256
constexpr int GX_COL_SF = 256;
constexpr uint32_t GX_A_BYTES = 16384;             // the MMA always reads 128 rows x 128 B of a stage

struct GxParams {
    const GxJob* table;                            // jobs in global memory (written by an earlier kernel), or nullptr:
    GxJob one;                                     // ... job j = activation rows [j * NT, j * NT + NT) of `one`
    const unsigned char* sfb;                      // activation scales [K/256][sfb_rows][16]
    size_t sfb_rows;
    unsigned int* status;
    int n_jobs, K, R, prefetch_before_wait;
    int sa, sb, ssf;                               // slots of the weight ring, of the activation ring, and of the scale slots in TMEM (ssf <= sb)
    uint32_t a_slot;                               // bytes of a weight slot: R x 128 rounded up to 1 KB (the MMA reads 16 KB from its start)
    int sc_box, sc_swz;
    int T;                                         // consecutive weight-row tiles per CTA (T * NT <= 256 accumulator columns, T * K/256 <= 64 steps)
    int sps, nslot;                                // steps per scale slab; slots of the slab ring
    int nacc;                                      // accumulators per tile (1, 2 or 4): k-block it adds into accumulator it % nacc
};

__device__ __forceinline__ void gx_tma_2d(uint32_t dst, const void* map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 :: "r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ uint64_t gx_desc(uint32_t saddr) {
    // K-major operand tile, 128B-swizzled: start address >> 4 | SBO = 1024 B (8 rows) | version 1 | SWIZZLE_128B
    return (uint64_t)((saddr >> 4) & 0x3FFF) | ((uint64_t)(1024u >> 4) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
__device__ __forceinline__ void gx_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void gx_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void gx_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(bar) : "memory");
}

// tcgen05.st of 4*CB registers (32x32b): register i goes to column i of the warp's lane quadrant.
template <int N> struct GxSt;
template <> struct GxSt<4> {
    static __device__ __forceinline__ void st(uint32_t a, const uint32_t* r) {
        asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1,%2,%3,%4};"
                     :: "r"(a), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]) : "memory");
    }
};
template <> struct GxSt<8> {
    static __device__ __forceinline__ void st(uint32_t a, const uint32_t* r) {
        asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                     :: "r"(a), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]) : "memory");
    }
};
template <> struct GxSt<16> {
    static __device__ __forceinline__ void st(uint32_t a, const uint32_t* r) {
        asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                     :: "r"(a), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
    }
};
template <> struct GxSt<32> {
    static __device__ __forceinline__ void st(uint32_t a, const uint32_t* r) {
        asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
                     "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
                     :: "r"(a), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
                        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
                        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]) : "memory");
    }
};

template <int NT>
__global__ void __launch_bounds__(GX_THREADS, 1)
k_gemm_mxf4(const __grid_constant__ GxParams p, const __grid_constant__ CUtensorMap map_x,
            const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_s) {
    constexpr int CB = NT / 32;                    // TMEM columns the activation scales of one 64-k block fill
    constexpr int CBS = CB < 4 ? 4 : CB;           // ... and the columns between two blocks (scale addresses stay multiples of 4)
    constexpr int SLOT = 16 + 4 * CBS;             // TMEM columns of one step's scales
    constexpr uint32_t B_BYTES = NT * 128u;
    extern __shared__ __align__(1024) unsigned char smem[];
    __shared__ uint64_t full_bar[GX_MAX_STEPS], sf_bar[GX_MAX_STEPS], empty_bar[GX_MAX_STEPS], slab_bar[GX_MAX_SLABS], done_bar;
    __shared__ uint32_t tmem_base_s;
    __shared__ float sx[NT];                       // 1 / (gs_w * gs_x[token]) of the job's rows
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int K = p.K, nst = K >> 8, R = p.R;

    GxJob J;
    const int chunk = (int)blockIdx.x / p.n_jobs, ji = (int)blockIdx.x - chunk * p.n_jobs;
    const void* mw = &map_w;
    const void* ms = &map_s;
    if (p.table) {
        pdl_wait();                                // the table is written by an earlier kernel of the stream
        J = p.table[ji];
        if (J.rows <= 0) return;                   // an unused slot: the whole CTA leaves before it owns anything
        mw = J.mw; ms = J.ms;
    } else {
        J = p.one;
        J.row0 = ji * NT;
        J.rows = min(NT, J.rows - J.row0);
        J.y += (size_t)J.row0 * J.ldy;
        J.gs_x += J.row0;
    }
    // Jobs of a table launch with few rows load (and multiply) only a 32- or 64-row box of activations: an
    // expert that three tokens chose should not pull a 128-row tile through L2 at every step.  In table
    // mode the two weight-map parameters are unused and carry the activation maps with the smaller boxes.
    int nb = NT;
    const void* mx = &map_x;
    if (p.table) {
        if (NT > 32 && J.rows <= 32) { nb = 32; mx = &map_w; }
        else if (NT > 64 && J.rows <= 64) { nb = 64; mx = &map_s; }
    }
    // this CTA's consecutive tiles of R weight rows: [tile0, tile0 + ntile)
    const int tile0 = chunk * p.T, ntile = min(p.T, (J.N + R - 1) / R - tile0);
    if (ntile <= 0) return;
    const int nsteps = ntile * nst;                // step g: tile g / nst, 256-k block g % nst
    const int sps = p.sps;                         // steps one scale slab covers; slab j = steps [j * sps, (j + 1) * sps)
    const uint32_t slab_bytes = (uint32_t)R * (uint32_t)p.sc_box;

    unsigned char* ringA = smem + ((1024u - (smem_u32(smem) & 1023u)) & 1023u);  // sa slots of packed weights
    unsigned char* ringB = ringA + (size_t)p.sa * p.a_slot;                     // sb slots of packed activations
    unsigned char* scl = ringB + (size_t)p.sb * B_BYTES;                        // ring of weight-scale slabs [R x sc_box], 1 KB aligned (swizzle)
    unsigned char* sfbs = scl + (size_t)p.nslot * slab_bytes;                   // per activation slot NT x 16 B of activation scales

    pdl_launch_dependents();
    if (warp >= 4) {
        const int i = tid - 128;
        if (i < nsteps) mbar_init(smem_u32(&full_bar[i]), 1);
        else if (i >= 64 && i < 64 + nsteps) mbar_init(smem_u32(&sf_bar[i - 64]), 128);
        else if (i >= 128 && i < 128 + nsteps) mbar_init(smem_u32(&empty_bar[i - 128]), 1);
        else if (i >= 192 && i < 192 + GX_MAX_SLABS) mbar_init(smem_u32(&slab_bar[i - 192]), 1);
        else if (i == 255) mbar_init(smem_u32(&done_bar), p.nacc >= 2 ? 2 : 1);
        mbar_fence_init();
    }
    if (warp == 2) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_u32(&tmem_base_s)), "r"(GX_TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    gx_fence_before();
    __syncthreads();
    gx_fence_after();
    const uint32_t tmem = tmem_base_s;

    if (warp == 0) {
        // ---- TMA producer: lane l issues steps l, l + 32, .. (and the scale slab that starts with such a step) ----
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" :: "l"(mw) : "memory");
            asm volatile("prefetch.tensormap [%0];" :: "l"(ms) : "memory");
            asm volatile("prefetch.tensormap [%0];" :: "l"(mx) : "memory");
        }
        if (!p.prefetch_before_wait) pdl_wait();
        const uint32_t full0 = smem_u32(&full_bar[0]), empty0 = smem_u32(&empty_bar[0]), slab0 = smem_u32(&slab_bar[0]);
        const uint32_t step_bytes = (uint32_t)R * 128u + (uint32_t)nb * 128u + (uint32_t)nb * 16u;
        int t = lane / nst, it = lane - t * nst;
        const int spt = nst / sps;                 // slabs per tile
        for (int g = lane; g < nsteps; g += 32) {
            const int rown0 = (tile0 + t) * R;
            const int js = p.sc_swz ? (it >> 3) : 0;                 // slab of this step within its tile
            if ((p.sc_swz ? (it & 7) : it) == 0) {
                // the slab of scale rows that steps [g, g + sps) read; its slot is free once the MMAs of the
                // last step of the slab that held it have completed (their scale movers are then done as well)
                const int j = t * spt + js;
                if (j >= p.nslot) mbar_wait_spin(empty0 + ((j - p.nslot + 1) * sps - 1) * 8, 0, p.status, 8);
                mbar_expect_tx(slab0 + j * 8, slab_bytes);
                gx_tma_2d(smem_u32(scl) + (uint32_t)(j % p.nslot) * slab_bytes, ms, js * p.sc_box, rown0, slab0 + j * 8);
            }
            // The weights stream from HBM and get the deep ring; the activations come from L2 and share a
            // short ring with the step's scale slot in TMEM.  Both loads of a step signal one barrier.
            const int sA = g % p.sa, sB = g % p.sb;
            if (g >= p.sa) mbar_wait_spin(empty0 + (g - p.sa) * 8, 0, p.status, 9);
            const uint32_t bar = full0 + g * 8;
            mbar_expect_tx(bar, step_bytes);
            gx_tma_2d(smem_u32(ringA) + (uint32_t)sA * p.a_slot, mw, it * 128, rown0, bar);     // weights may be read early (stable weights)
            pdl_wait();                                                           // the activations come from the quantiser launch
            if (g >= p.sb) mbar_wait_spin(empty0 + (g - p.sb) * 8, 0, p.status, 7);
            gx_tma_2d(smem_u32(ringB) + (uint32_t)sB * B_BYTES, mx, it * 128, J.row0, bar);
            bulk_g2s(smem_u32(sfbs) + (uint32_t)sB * NT * 16u, p.sfb + ((size_t)it * p.sfb_rows + (size_t)J.row0) * 16, (uint32_t)nb * 16u, bar);
            it += 32; while (it >= nst) { it -= nst; ++t; }
        }
        __syncwarp();
        // The tcgen05.commit arrivals on empty_bar are asynchronous: wait for the last one of every
        // stage, or the CTA could exit with an arrival in flight that lands in the next CTA's shared memory.
        for (int g = max(0, nsteps - p.sa) + lane; g < nsteps; g += 32)
            mbar_wait_spin(empty0 + g * 8, 0, p.status, 10);
        __syncwarp();
    } else if (warp == 1 || (warp == 3 && p.nacc >= 2)) {
        // ---- MMA issuers: the whole warp walks the loop, lane 0 issues ----
        // A chain of MMAs into one accumulator runs at the latency of an MMA, not at its issue rate, and
        // that latency (about 110 cycles) exceeds the execution time of an MMA narrower than 256 columns.
        // So a tile has nacc accumulators -- k-block `it` adds into accumulator it % nacc, the epilogue adds
        // them up in a fixed order -- and with two or more of them two warps issue: warp 1 the even
        // k-blocks, warp 3 the odd ones (different accumulators, so no order between the warps matters).
        const int mwi = warp == 1 ? 0 : 1, two = p.nacc >= 2;
        const uint32_t idesc = (1u << 7) | (1u << 10) | ((uint32_t)(nb >> 3) << 17) | ((128u >> 4) << 24);
        const uint64_t dA0 = gx_desc(smem_u32(ringA)), dB0 = gx_desc(smem_u32(ringB));
        const uint32_t sf0 = smem_u32(&sf_bar[0]), empty0 = smem_u32(&empty_bar[0]);
        int sA = 0, sB = 0, sF = 0, t = 0, it = 0;
        for (int g = 0; g < nsteps; ++g) {
            if (!two || (it & 1) == mwi) {
                mbar_wait_spin(sf0 + g * 8, 0, p.status, 11);
                gx_fence_after();
                if (lane == 0) {
                    const uint32_t slot = tmem + GX_COL_SF + (uint32_t)sF * SLOT;
                    const uint64_t soA = (uint64_t)(((uint32_t)sA * p.a_slot) >> 4), soB = (uint64_t)(((uint32_t)sB * B_BYTES) >> 4);
                    const uint32_t tD = tmem + (uint32_t)((t * p.nacc + (it & (p.nacc - 1))) * NT);
                    const uint32_t first = it < p.nacc ? 0u : 1u;           // the first k-block of an accumulator starts it
                    #pragma unroll
                    for (int kb = 0; kb < 4; ++kb) {
                        asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                                     " tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n}"
                                     :: "r"(tD), "l"(dA0 + soA + kb * 2), "l"(dB0 + soB + kb * 2), "r"(idesc),
                                        "r"(kb ? 1u : first), "r"(slot + kb * 4), "r"(slot + 16 + kb * CBS) : "memory");
                    }
                    gx_commit(empty0 + g * 8);
                }
                __syncwarp();
            }
            if (++sA == p.sa) sA = 0;
            if (++sB == p.sb) sB = 0;
            if (++sF == p.ssf) sF = 0;
            if (++it == nst) { it = 0; ++t; }
        }
        if (lane == 0) gx_commit(smem_u32(&done_bar));
        __syncwarp();
    } else if (warp >= 4) {
        // ---- scale movers, then epilogue ----
        const int tm = tid - 128, grp = tm >> 7, q4 = warp & 3;
        const uint32_t tq = tmem + ((uint32_t)(q4 * 32) << 16);
        pdl_wait();
        if (tm < NT) sx[tm] = tm < J.rows ? 1.0f / (J.gs_w[0] * J.gs_x[tm]) : 0.f;
        named_sync(1, GX_MOVERS);
        const uint32_t full0 = smem_u32(&full_bar[0]), sf0 = smem_u32(&sf_bar[0]), slab0 = smem_u32(&slab_bar[0]);
        const uint32_t empty0 = smem_u32(&empty_bar[0]);
        int s = grp % p.sb, sf = grp % p.ssf;
        int t = grp / nst, it = grp - t * nst;
        const int spt = nst / sps;
        for (int g = grp; g < nsteps; g += 2) {
            const int js = p.sc_swz ? (it >> 3) : 0, is = p.sc_swz ? (it & 7) : it;     // slab within the tile, step within the slab
            const int j = t * spt + js, valid = J.N - (tile0 + t) * R;    // weight rows of this tile that exist (may exceed R)
            mbar_wait_spin(slab0 + j * 8, 0, p.status, 12);
            mbar_wait_spin(full0 + g * 8, 0, p.status, 13);
            // the scale slot in TMEM is free once the MMAs of the step that used it last have completed
            // (implied by full[g] when there are as many slots as activation slots)
            if (p.ssf < p.sb && g >= p.ssf) mbar_wait_spin(empty0 + (g - p.ssf) * 8, 0, p.status, 6);
            // weights: lane l holds rows l, l+32, l+64, l+96, 16 bytes each = four 64-k blocks x four scales;
            // block kb of row 32c + l goes to column kb*4 + c
            const unsigned char* sl = scl + (size_t)(j % p.nslot) * slab_bytes;
            uint32_t ra[16];
            #pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int r = lane + 32 * c;
                uint32_t off;
                if (p.sc_swz) off = (uint32_t)r * 128u + (uint32_t)((is ^ (r & 7)) << 4);
                else off = (uint32_t)r * (uint32_t)p.sc_box + (uint32_t)is * 16u;
                const uint4 v = (r < R && r < valid) ? *reinterpret_cast<const uint4*>(sl + off) : make_uint4(0u, 0u, 0u, 0u);
                ra[c] = v.x; ra[4 + c] = v.y; ra[8 + c] = v.z; ra[12 + c] = v.w;
            }
            // activations: lane l holds tokens l, l+32, ..; block kb of token 32c + l goes to column 16 + kb*CBS + c
            uint32_t rb[4 * CBS];
            const unsigned char* sb = sfbs + (size_t)s * NT * 16;
            #pragma unroll
            for (int c = 0; c < CBS; ++c) {
                const uint4 v = (c < CB && 32 * c < nb) ? *reinterpret_cast<const uint4*>(sb + (size_t)(lane + 32 * c) * 16) : make_uint4(0u, 0u, 0u, 0u);
                rb[c] = v.x; rb[CBS + c] = v.y; rb[2 * CBS + c] = v.z; rb[3 * CBS + c] = v.w;
            }
            const uint32_t slot = tq + GX_COL_SF + (uint32_t)sf * SLOT;
            GxSt<16>::st(slot, ra);
            GxSt<4 * CBS>::st(slot + 16, rb);
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            gx_fence_before();
            mbar_arrive(sf0 + g * 8);
            s += 2; while (s >= p.sb) s -= p.sb;
            sf += 2; while (sf >= p.ssf) sf -= p.ssf;
            it += 2; while (it >= nst) { it -= nst; ++t; }
        }
        // epilogue: group grp takes columns [grp * NT/2, (grp + 1) * NT/2) of every tile
        mbar_wait_spin(smem_u32(&done_bar), 0, p.status, 14);
        gx_fence_after();
        const int r = q4 * 32 + lane;
        #pragma unroll 1
        for (int te = 0; te < ntile; ++te) {
            const int row = (tile0 + te) * R + r;
            const bool ok = r < R && row < J.N;
            #pragma unroll 1
            for (int c0 = grp * (NT / 2); c0 < (grp + 1) * (NT / 2); c0 += 16) {
                if (c0 >= J.rows) break;             // warp-uniform: the remaining tokens do not exist
                float d[16];
                #pragma unroll 1
                for (int a = 0; a < p.nacc; ++a) {
                    uint32_t v[16];
                    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                                   "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                                 : "r"(tq + (uint32_t)((te * p.nacc + a) * NT + c0)));
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    #pragma unroll
                    for (int j = 0; j < 16; ++j) d[j] = a == 0 ? __uint_as_float(v[j]) : d[j] + __uint_as_float(v[j]);     // accumulators in index order
                    if (a + 1 < p.nacc && (a + 1) >= nst) break;     // fewer k-blocks than accumulators: the rest were never started
                }
                if (ok) {
                    #pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if (c0 + j < J.rows) J.y[(size_t)(c0 + j) * J.ldy + row] = d[j] * sx[c0 + j];
                }
            }
        }
    }
    gx_fence_before();
    __syncthreads();
    if (warp == 2) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem), "r"(GX_TMEM_COLS));
}

// ---- per-token activation quantiser -------------------------------------------------------------
// One CTA per activation row.  MODE 0: bf16 rows; 1: f32 rows; 2: f32 rows of the clamped SwiGLU
// silu(min(g, limit)) * clamp(u, -limit, limit) of two product vectors (the MoE down projection's input).
// src_row != nullptr: output row r is input row src_row[r] (gathers token rows into expert order).
// Output: packed [*, K/2] codes, scales step-major [K/256][sfb_rows][16], gsx[r] = 2688 / amax(row r).
// Rows in [M, rows_total) only get zero scales (they pad the last tile of a dense call).
template <int MODE>
__global__ void __launch_bounds__(256)
k_quant_act(const void* __restrict__ xin, const void* __restrict__ xin2, float limit, const int* __restrict__ src_row,
            const int* __restrict__ m_dev, int M, int K, unsigned char* __restrict__ xq, unsigned char* __restrict__ sfb,
            size_t sfb_rows, float* __restrict__ gsx) {
    __shared__ uint32_t red[8];
    const int row = blockIdx.x, tid = threadIdx.x, groups = K >> 4;
    pdl_launch_dependents();
    pdl_wait();
    if (m_dev) M = m_dev[0];                        // row count decided on the device (rows grouped by expert)
    if (row >= M) {
        if (m_dev) return;
        for (int st = tid; st < (K >> 8); st += 256)
            *reinterpret_cast<uint4*>(sfb + ((size_t)st * sfb_rows + row) * 16) = make_uint4(0u, 0u, 0u, 0u);
        return;
    }
    const size_t src = src_row ? (size_t)src_row[row] : (size_t)row;
    auto load = [&](int g, float (&v)[16]) {
        if (MODE == 0) {
            const uint4* r = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(xin) + src * K) + 2 * g;
            const uint4 a = r[0], b = r[1];
            const uint32_t u[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
            #pragma unroll
            for (int j = 0; j < 8; ++j) { v[2 * j] = __uint_as_float(u[j] << 16); v[2 * j + 1] = __uint_as_float(u[j] & 0xffff0000u); }
        } else {
            const float4* r = reinterpret_cast<const float4*>(static_cast<const float*>(xin) + src * K) + 4 * g;
            const float4* r2 = MODE == 2 ? reinterpret_cast<const float4*>(static_cast<const float*>(xin2) + src * K) + 4 * g : nullptr;
            #pragma unroll
            for (int q = 0; q < 4; ++q) {
                float4 a = r[q];
                if (MODE == 2) {
                    const float4 u = r2[q];
                    const float gg[4] = {fminf(a.x, limit), fminf(a.y, limit), fminf(a.z, limit), fminf(a.w, limit)};
                    const float uu[4] = {fminf(fmaxf(u.x, -limit), limit), fminf(fmaxf(u.y, -limit), limit),
                                         fminf(fmaxf(u.z, -limit), limit), fminf(fmaxf(u.w, -limit), limit)};
                    a = make_float4((gg[0] / (1.f + __expf(-gg[0]))) * uu[0], (gg[1] / (1.f + __expf(-gg[1]))) * uu[1],
                                    (gg[2] / (1.f + __expf(-gg[2]))) * uu[2], (gg[3] / (1.f + __expf(-gg[3]))) * uu[3]);
                }
                v[4 * q] = a.x; v[4 * q + 1] = a.y; v[4 * q + 2] = a.z; v[4 * q + 3] = a.w;
            }
        }
    };
    float first[16];
    // maximum over the bit patterns of |x| (they order like the values; an infinity or a NaN wins instead of
    // being dropped): a row that holds one gets a NaN global scale, and with it NaN outputs
    uint32_t ai = 0u;
    for (int g = tid; g < groups; g += 256) {
        float v[16];
        load(g, v);
        #pragma unroll
        for (int j = 0; j < 16; ++j) { ai = max(ai, __float_as_uint(v[j]) & 0x7fffffffu); if (g == tid) first[j] = v[j]; }
    }
    #pragma unroll
    for (int o = 16; o; o >>= 1) ai = max(ai, __shfl_xor_sync(0xffffffffu, ai, o));
    if ((tid & 31) == 0) red[tid >> 5] = ai;
    __syncthreads();
    ai = red[0];
    #pragma unroll
    for (int w = 1; w < 8; ++w) ai = max(ai, red[w]);
    const float gs = ai >= 0x7f800000u ? __uint_as_float(0x7fc00000u) : nvfp4_global_scale(__uint_as_float(ai));
    if (tid == 0) gsx[row] = gs;
    for (int g = tid; g < groups; g += 256) {
        float v[16];
        if (g == tid) {
            #pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = first[j];
        } else load(g, v);
        uint32_t lo, hi; int code;
        quantize_group(v, gs, lo, hi, code);
        reinterpret_cast<uint2*>(xq + (size_t)row * (K >> 1))[g] = make_uint2(lo, hi);
        sfb[((size_t)(g >> 4) * sfb_rows + row) * 16 + (g & 15)] = (unsigned char)code;
    }
}

// ---- host side ---------------------------------------------------------------------------------
static int gx_accumulators(int NT);
static size_t up256(size_t v) { return (v + 255) / 256 * 256; }

size_t gemm_mxf4_ws_bytes(int M, int K) {
    if (M < 1 || K < 256) return 256;
    const size_t rows = ((size_t)M + 255) / 256 * 256;
    return up256(rows * (size_t)(K / 2)) + up256(rows * (size_t)(K / 16)) + up256(rows * 4);
}

bool gemm_mxf4_shape_ok(int K) {
    int b, z;
    return !(K & 255) && K >= 256 && K <= 16384 && scale_box(K, &b, &z) && tmap_available();
}

int quant_act_launch(int mode, const void* x, const void* x2, float limit, const int* src_row, const int* m_dev, int M,
                     int rows_launch, int K, unsigned char* xq, unsigned char* sfb, size_t sfb_rows, float* gsx, cudaStream_t s) {
    if (rows_launch < 1) return B200_OK;
    cudaLaunchConfig_t lc{};
    lc.gridDim = dim3(rows_launch); lc.blockDim = dim3(256); lc.dynamicSmemBytes = 0; lc.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = at; lc.numAttrs = 1;
    cudaError_t e;
    if (mode == 0) e = cudaLaunchKernelEx(&lc, k_quant_act<0>, x, x2, limit, src_row, m_dev, M, K, xq, sfb, sfb_rows, gsx);
    else if (mode == 1) e = cudaLaunchKernelEx(&lc, k_quant_act<1>, x, x2, limit, src_row, m_dev, M, K, xq, sfb, sfb_rows, gsx);
    else e = cudaLaunchKernelEx(&lc, k_quant_act<2>, x, x2, limit, src_row, m_dev, M, K, xq, sfb, sfb_rows, gsx);
    if (e != cudaSuccess) return launch_failed("k_quant_act");
    return check_launch("k_quant_act");
}

// Shared memory and stage count of a launch; false if not even two stages fit.
template <int NT>
static int gx_launch_t(GxParams& p, const CUtensorMap& mx, const CUtensorMap& mw, const CUtensorMap& ms, int grid, cudaStream_t s) {
    auto kern = k_gemm_mxf4<NT>;
    static int attr_cache[64][2] = {};               // [device] = {optin, static bytes + 1}
    static bool ready[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return launch_failed("gemm_mxf4: cudaGetDevice");
    if (dev < 0 || dev >= 64) dev = 0;
    int* ac = attr_cache[dev];
    if (!ac[1]) {
        cudaFuncAttributes fa;
        int oi = 0;
        if (cudaFuncGetAttributes(&fa, kern) != cudaSuccess ||
            cudaDeviceGetAttribute(&oi, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess) return launch_failed("gemm_mxf4: attributes");
        ac[0] = oi; ac[1] = (int)fa.sharedSizeBytes + 1;
    }
    const size_t static_smem = (size_t)ac[1] - 1;
    const size_t room = (size_t)ac[0] - static_smem - 2048;        // 1 KB alignment slack + 1 KB system reserve
    const int nst = p.K / 256;
    p.sps = p.sc_swz ? 8 : nst;
    const int slabs = p.T * (nst / p.sps);
    p.nacc = gx_accumulators(NT);
    if (p.T < 1 || p.T * p.nacc * NT > GX_COL_SF || p.T * nst > GX_MAX_STEPS || slabs > GX_MAX_SLABS) return B200_ENOTIMPL;
    p.nslot = std::min(slabs, 3);
    const int nsteps = p.T * nst;
    p.a_slot = ((uint32_t)p.R * 128u + 1023u) & ~1023u;
    // Ring depths: a step is in flight from the moment its loads are issued until its MMAs complete, and both
    // the weights (HBM) and the activations (L2, but requested by every CTA at once) take a microsecond or
    // more to arrive, so the shallower of the two rings bounds the step rate.  Take the split of the shared
    // memory that makes the shallower ring as deep as possible (ties: the deeper weight ring).
    const size_t b_slot = (size_t)NT * 128 + (size_t)NT * 16, slab_sz = (size_t)p.nslot * p.R * p.sc_box;
    p.sa = 0; p.sb = 0;
    for (int sb = std::min(nsteps, 16); sb >= 1; --sb) {
        const size_t fx = slab_sz + (size_t)sb * b_slot;
        if (fx + (size_t)p.a_slot + GX_A_BYTES > room) continue;
        const int sa = (int)std::min<size_t>((room - fx - GX_A_BYTES) / p.a_slot + 1, (size_t)std::min(nsteps, 16));
        if (std::min(sa, sb) > std::min(p.sa, p.sb) || (std::min(sa, sb) == std::min(p.sa, p.sb) && sa > p.sa)) { p.sa = sa; p.sb = sb; }
    }
    if (const char* e = getenv("B200_GX_RINGS")) {       // tuning aid: "sa,sb" replaces the choice above when it fits
        int ua = 0, ub = 0;
        if (sscanf(e, "%d,%d", &ua, &ub) == 2 && ua >= 1 && ub >= 1 && ub <= 16 && ua <= 16) {
            ua = std::min(ua, nsteps); ub = std::min(ub, nsteps);
            if (slab_sz + (size_t)ub * b_slot + (size_t)(ua - 1) * p.a_slot + GX_A_BYTES <= room) { p.sa = ua; p.sb = ub; }
        }
    }
    if (p.sa < 1 || (std::min(p.sa, p.sb) < 2 && nsteps > 1)) return B200_ENOTIMPL;
    p.ssf = std::min(p.sb, (GX_TMEM_COLS - GX_COL_SF) / (16 + 4 * std::max(NT / 32, 4)));
    const size_t fixed = slab_sz + (size_t)p.sb * b_slot;
    // the MMA reads 16 KB from the start of a weight slot whatever R: keep that inside the allocation for the last slot
    size_t smem = (size_t)p.sa * p.a_slot + fixed + 1024;
    if (smem < (size_t)(p.sa - 1) * p.a_slot + GX_A_BYTES + 1024) smem = (size_t)(p.sa - 1) * p.a_slot + GX_A_BYTES + 1024;
    if (!ready[dev]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(ac[0] - static_smem)) != cudaSuccess)
            return launch_failed("gemm_mxf4: cudaFuncSetAttribute");
        ready[dev] = true;
    }
    cudaLaunchConfig_t lc{};
    lc.gridDim = dim3(grid); lc.blockDim = dim3(GX_THREADS); lc.dynamicSmemBytes = smem; lc.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = at; lc.numAttrs = 1;
    if (cudaLaunchKernelEx(&lc, kern, p, mx, mw, ms) != cudaSuccess) return launch_failed("k_gemm_mxf4");
    return check_launch("k_gemm_mxf4");
}

static int gx_launch(int NT, GxParams& p, const CUtensorMap& mx, const CUtensorMap& mw, const CUtensorMap& ms, int grid, cudaStream_t s) {
    switch (NT) {
        case 32: return gx_launch_t<32>(p, mx, mw, ms, grid, s);
        case 64: return gx_launch_t<64>(p, mx, mw, ms, grid, s);
        case 128: return gx_launch_t<128>(p, mx, mw, ms, grid, s);
        default: return gx_launch_t<256>(p, mx, mw, ms, grid, s);
    }
}

// Token tile for M activation rows against N weight rows: as narrow as covers M up to 128; beyond
// that 256 columns per CTA unless the narrower tile still fits one wave of CTAs.
static int pick_nt(int M, int N) {
    if (M <= 32) return 32;
    if (M <= 64) return 64;
    if (M <= 128) return 128;
    const int tiles_n = (N + 127) / 128, nsm = sm_count();
    return tiles_n * ((M + 127) / 128) <= nsm ? 128 : 256;
}

// Accumulators per tile.  The kernel can split a tile's k-blocks over 2 or 4 accumulators issued by two
// warps (independent MMA chains); measured on B200 that buys nothing -- the steps are paced by the arrival
// of the weight tiles, not by the MMA chain -- and it costs TMEM columns that are better spent on more tiles
// per CTA, so one accumulator per tile it is.  B200_GX_NACC=2|4 switches the split on for experiments.
static int gx_accumulators(int NT) {
    static const int forced = [] { const char* e = getenv("B200_GX_NACC"); return e ? atoi(e) : 1; }();
    if ((forced == 2 || forced == 4) && forced * NT <= GX_COL_SF) return forced;
    return 1;
}

// Consecutive weight-row tiles per CTA: as many as the accumulator columns (T * NT <= 256), the per-step
// barriers (T * K/256 <= 64) and the scale slabs allow while the launch still has a CTA for every SM.  A
// CTA pays its set-up (TMEM, barriers, descriptors, pipeline fill and drain) once for all its tiles.
static int pick_tiles_per_cta(int NT, int K, int tiles_n, long jobs) {
    int box = 0, swz = 0;
    scale_box(K, &box, &swz);
    const int nst = K / 256, slabs_per_tile = swz ? nst / 8 : 1, nsm = sm_count();
    int best = 1;
    for (int T = 2; T <= tiles_n && T * gx_accumulators(NT) * NT <= GX_COL_SF && T * nst <= GX_MAX_STEPS && T * slabs_per_tile <= GX_MAX_SLABS; ++T)
        if (jobs * ((tiles_n + T - 1) / T) >= nsm) best = T;
    return best;
}

// Dense: y[M, N] = quant(x)[M, K] . W^T.  x_kind 0: bf16, 1: f32.  ws: gemm_mxf4_ws_bytes(M, K).
int gemm_mxf4_dense(float* y, const b200_wref* W, const void* x, int x_kind, int M, int N, int K, void* ws, cudaStream_t s) {
    if (!y || !W || !W->packed || !W->scale || !W->gscale || !x || !ws || M < 1 || N < 1) return B200_EINVAL;
    if (!gemm_mxf4_shape_ok(K)) return B200_ENOTIMPL;
    if (((uintptr_t)W->packed & 15) || ((uintptr_t)W->scale & 15) || ((uintptr_t)x & 15) || ((uintptr_t)ws & 255)) return B200_ENOTIMPL;
    const int NT = pick_nt(M, N), n_jobs = (M + NT - 1) / NT, nsm = sm_count();
    // weight rows per CTA: with one token tile the kernel is bandwidth-bound and wants every SM busy (the
    // smallest multiple of 8 whose tiles still fit the SMs); with several, the MMA is always 128 rows tall.
    int R = 128;
    if (n_jobs == 1)
        for (int r = 8; r <= 128; r += 8) if ((N + r - 1) / r <= nsm) { R = r; break; }
    const size_t rows = ((size_t)M + 255) / 256 * 256;
    unsigned char* xq = static_cast<unsigned char*>(ws);
    unsigned char* sfb = xq + up256(rows * (size_t)(K / 2));
    float* gsx = reinterpret_cast<float*>(sfb + up256(rows * (size_t)(K / 16)));
    GxParams p{};
    p.table = nullptr;
    p.one = GxJob{y, W->gscale, gsx, nullptr, nullptr, 0, M, N, N};
    p.sfb = sfb; p.sfb_rows = rows;
    p.status = device_status_ptr();
    if (!p.status) return B200_ENOTIMPL;
    p.n_jobs = n_jobs; p.K = K; p.R = R; p.prefetch_before_wait = stable_weights_option();
    if (!scale_box(K, &p.sc_box, &p.sc_swz)) return B200_ENOTIMPL;
    CUtensorMap mx, mw, ms;
    if (!tmap_u8_2d(&mw, W->packed, (size_t)N, (size_t)K / 2, 128, R, true, true) ||
        !tmap_u8_2d(&ms, W->scale, (size_t)N, (size_t)K / 16, p.sc_box, R, p.sc_swz != 0, true) ||
        !tmap_u8_2d(&mx, xq, (size_t)M, (size_t)K / 2, 128, NT, true, true)) return B200_ENOTIMPL;
    credit(B200_CREDIT_GEMM, (double)n_jobs * N * K * 0.5625);      // W streams once per token tile (the later tiles mostly from L2)
    if (int rc = quant_act_launch(x_kind ? 1 : 0, x, nullptr, 0.f, nullptr, nullptr, M, n_jobs * NT, K, xq, sfb, rows, gsx, s)) return rc;
    const int tiles_n = (N + R - 1) / R;
    p.T = pick_tiles_per_cta(NT, K, tiles_n, n_jobs);
    return gx_launch(NT, p, mx, mw, ms, (tiles_n + p.T - 1) / p.T * n_jobs, s);
}

// Jobs from a table in device memory (rows grouped by expert); expected_jobs: how many of the max_jobs slots
// are likely to hold a job (decides how many tiles a CTA takes).  Every job's weight maps were encoded
// with box height R and N weight rows; the activation rows of all jobs live in one quantised buffer
// (xq [x_rows, K/2], scales sfb [K/256][sfb_rows][16]).
int gemm_mxf4_table(const GxJob* table, int max_jobs, long expected_jobs, int NT, int N, int K, int R, const unsigned char* xq, size_t x_rows,
                    const unsigned char* sfb, size_t sfb_rows, cudaStream_t s) {
    if (!gemm_mxf4_shape_ok(K)) return B200_ENOTIMPL;
    GxParams p{};
    p.table = table;
    p.sfb = sfb; p.sfb_rows = sfb_rows;
    p.status = device_status_ptr();
    if (!p.status) return B200_ENOTIMPL;
    p.n_jobs = max_jobs; p.K = K; p.R = R; p.prefetch_before_wait = 0;
    if (!scale_box(K, &p.sc_box, &p.sc_swz)) return B200_ENOTIMPL;
    CUtensorMap mx, mx32, mx64;                      // activation boxes of NT, 32 and 64 rows (jobs with few rows take the small ones)
    if (!tmap_u8_2d(&mx, xq, x_rows, (size_t)K / 2, 128, NT, true, true) ||
        !tmap_u8_2d(&mx32, xq, x_rows, (size_t)K / 2, 128, 32, true, true) ||
        !tmap_u8_2d(&mx64, xq, x_rows, (size_t)K / 2, 128, 64, true, true)) return B200_ENOTIMPL;
    const int tiles_n = (N + R - 1) / R;
    p.T = pick_tiles_per_cta(NT, K, tiles_n, std::max(1L, expected_jobs));
    return gx_launch(NT, p, mx, mx32, mx64, (tiles_n + p.T - 1) / p.T * max_jobs, s);
}

}  // namespace b200

using namespace b200;

extern "C" size_t b200_nvfp4_gemm_bf16_workspace_bytes(int M, int K) { return gemm_mxf4_ws_bytes(M, K); }

extern "C" int b200_nvfp4_gemm_bf16(float* y, const b200_wref* W, const void* x_bf16, int M, int N, int K,
                                    void* ws, b200_stream stream) {
    if (!y || !W || !x_bf16 || !ws || M < 1 || N < 1 || K < 1) return B200_EINVAL;
    if (!W->packed) return B200_EINVAL;
    if (K & 15) return B200_ESHAPE;
    if ((uintptr_t)ws & 255) return B200_EALIGN;
    return gemm_mxf4_dense(y, W, x_bf16, 0, M, N, K, ws, stream);
}

extern "C" int b200_nvfp4_quantize_tokens(const void* x, int x_is_f32, int M, int K, uint8_t* packed,
                                          uint8_t* scale_step_major, float* gs, b200_stream stream) {
    if (!x || !packed || !scale_step_major || !gs || M < 1 || K < 1) return B200_EINVAL;
    if (K & 255) return B200_ESHAPE;
    if (((uintptr_t)x & 15) || ((uintptr_t)packed & 7) || ((uintptr_t)scale_step_major & 15) || ((uintptr_t)gs & 3)) return B200_EALIGN;
    return quant_act_launch(x_is_f32 ? 1 : 0, x, nullptr, 0.f, nullptr, nullptr, M, M, K, packed, scale_step_major, (size_t)M, gs, stream);
}
