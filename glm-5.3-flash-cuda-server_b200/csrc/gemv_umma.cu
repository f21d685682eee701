// gemv_umma.cu -- NVFP4 gemv / small-batch gemm (1..8 activation rows) on the 5th-generation tensor cores:
// tcgen05.mma kind::mxf4nvf4 (block-16, UE4M3 scales), TMEM accumulators.
//
// Why tensor cores for a matrix-VECTOR product: the CUDA-core formulation is capped by the
// conversion pipe (cvt.rn.f16x2.e2m1x2 issues once per ~3 cycles per scheduler: 24e12 weights/s
// chip-wide against the 11.6e12 that 6.5 TB/s of HBM delivers, before a single load, barrier or
// reduction).  tcgen05.mma reads the packed e2m1 bytes and the e4m3 scale bytes exactly as the
// format stores them, so the SM does no decode work at all and the kernel is a pure stream.
//
// How fp32-activation accuracy is kept although both MMA operands are FP4: the activation row is
// written as EIGHT FP4 columns.  x = gamma * v with gamma = amax(x) / 3.99, so |v| < 4, and v is
// rounded to 14 fractional bits: v = sign * sum_t d_t 4^-t, t = 0..7, with base-4 digits d_t in
// {0,1,2,3}, all of which e2m1 represents exactly.  Column t of the B operand holds the digits
// d_t; its block scales are the constant 1.0, written to TMEM once.  The MMA's N = 8 columns come
// for free (an MMA of M = 128 costs ~55 cycles for any N <= 96, measured), and the epilogue adds
// them: y = (sum_t gamma 4^-t D[:,t]) / gscale.  Rounding error per activation <= 2^-15 gamma =
// 7.7e-6 amax(x): measured rel-L2 of a product 1.6e-5, forty times finer than fp16 staging;
// products and sums inside the MMA are exact / fp32.
//
// Per CTA (one per SM): T consecutive tiles of R rows of one job (R <= 128 a multiple of 8; T = 1
// for a plain gemv, up to 8 for the MoE job-table launches), K walked in steps of 256.
//   warp 0      TMA producer.  First the CTA's scale rows, as slabs [R rows x 128 B] (128B-swizzled,
//               so 32 lanes reading one 16-byte column of 32 consecutive rows hit different banks);
//               then per step one box [128 B x R rows] of packed weights (SWIZZLE_128B, the K-major
//               operand layout the MMA reads) into a ring of stages.  Lane l issues steps l, l+32, ..:
//               one thread issuing tensor loads back to back gets one out every ~0.35 us (measured).
//   warp 1      L2 prefetch of the steps the ring cannot take at once; warps 2-3 idle
//   warps 4-7   MMA issuers: warp w takes every fourth step: 4 tcgen05.mma (K = 64 each) into the
//               accumulator of the step's k-block (k-block % 4: the summation order of a row never
//               depends on tiling), then a tcgen05.commit frees the stage
//   warps 8-15  workers: split the activation rows into the B image (once per CTA); then, in two
//               groups of four warps (one warp per TMEM lane quadrant) taking alternate steps, move
//               the step's R x 16 scale bytes from shared memory to the stage's scale columns in
//               TMEM (tcgen05.st: lane r % 32, column r / 32, the layout the block-scaled MMA reads);
//               the first group finally reads the accumulators and writes y
// Up to 8 activation rows per job: row m is columns 8m..8m+7 of the MMA's N = 8M, so every row is
// computed exactly as if it were alone (a gemm row equals its gemv bit for bit).
// Barriers: full[step], sf[step] and empty[step] are used once each, so that no waiter ever has
// to tell phases apart (a parity wait cannot tell "two phases behind" from "ready").  In the
// single-thread roles the whole warp walks the loop and waits (a lone lane whose 31 siblings are
// parked at the closing barrier is scheduled rarely: measured 20 % slower).  Before it exits a CTA
// waits for the last tcgen05.commit arrival of every stage: an arrival still in flight would land
// in the shared memory of the next CTA on that SM.
// Prologue without a CTA-wide barrier: warp 0 initialises the barriers of its own loads and requests the
// slabs and the first four stages at once; the MMA warps initialise the other barriers, allocate TMEM and
// arrive at named barrier 3, where only the producer waits; the workers go straight to the dependency
// wait and the activation loads, and learn of everything else at named barrier 2.
//
// Decode kernel with RESIDENT scales (RES: up to four activation rows, one tile per CTA, K <= 7424 for one
// row, 6912 for two, 5888 for three or four): TMEM has room for the scales of every step at once, so the MMA
// warps (idle until the activations are split) move them all as soon as the slabs have landed -- with weights
// declared stable that is before the dependency wait.  They transpose a step's 4 x 4 words in registers into
// [k-block][32 rows][16 B] and the tensor core copies that to TMEM (tcgen05.cp 32x128b.warpx4, issued by the lane
// that issues the step's MMAs, so the two are ordered without a wait).  The slabs and their transposed copy lie
// under the last stages of the ring, which are requested once a tcgen05.commit says the copies are done.  For
// the decode shapes (K = 4096, R <= 96, one row) the ring then holds the CTA's whole tile: every weight byte is
// requested before the first MMA, and after the activation split the MMAs run at issue speed.
// Every mbarrier wait is bounded (tma_pipe.cuh).  No cluster launch, no multicast.
#include "b200_internal.h"
#include "nvfp4_decode.cuh"
#include "tma_pipe.cuh"
#include <cuda.h>
#include <cstdio>
#include <cstdlib>

namespace b200 {

#define UM_WAIT mbar_wait_spin

constexpr int UM_LOAD_WARPS = 4;
constexpr int UM_MMA_WARPS = 4;
constexpr int UM_WORKERS = 256;
constexpr int UM_LOADERS = 32 * UM_LOAD_WARPS;
constexpr int UM_THREADS = UM_LOADERS + 32 * UM_MMA_WARPS + UM_WORKERS;
constexpr int UM_NB = 8;                           // MMA N = digits per activation
constexpr int UM_MAX_M = 8;                        // activation rows per job (MMA N = 8 * M <= 64)
constexpr int UM_MAX_STAGES = 12;                  // TMEM holds one 16-column scale slot per stage
constexpr int UM_MAX_STEPS = 64;                   // K <= 16384
constexpr int UM_TMEM_COLS = 512;                  // D0..D3 [0,256), 64 each | unit scales [256,260) | weight scales from 272, 16 columns per slot
constexpr int UM_COL_SB = 256, UM_COL_SF = 272;
// Decode kernel with resident scales, up to UM_RES_MAX_M activation rows: accumulators D0..D3 at a stride of a columns
// (8 for one row, 16 for two, 32 for three or four) | unit scales [4a, 4a + 4) | step g's scales [4a + 16 + 16 g, ..).
constexpr int UM_RES_MAX_M = 4;
static inline int um_res_acc_stride(int M) { return M <= 1 ? 8 : (M == 2 ? 16 : 32); }
static inline int um_res_steps(int M) { return (UM_TMEM_COLS - (4 * um_res_acc_stride(M) + 16)) / 16; }      // 29 / 27 / 23 steps


struct UmParams {
    UmJob j[B200_GEMV_MULTI_MAX];
    const UmJob* table;                            // != nullptr: jobs live in global memory, tiles_per_job CTAs each
    unsigned int* status;
    float limit;                                   // SwiGLU clamp for jobs with x2
    int n_jobs, K, R, stages, prefetch_before_wait, max_m, tiles_per_job;
    int dry_run;                                   // host only: stop before the launch (does the shape fit?)
    int T;                                         // consecutive row tiles of one job per CTA (T * max_m <= 8, T * K/256 <= 64)
    uint32_t stage_bytes;                          // per stage: the A tile, R x 128 bytes rounded up to 1 KB
    int sc_box, sc_swz;                            // scale slab: box width in bytes (128 swizzled, or K/16 plain)
    uint32_t bimg_off, scl_off, tsc_off;           // shared-memory offsets of the B image, of the scale slabs and (resident scales) of their transposed copy from the (1 KB aligned) ring
    int ov_first;                                  // resident scales: stages from this one on share their bytes with the scale slabs or the transposed copy
    int early;                                     // stages requested by the producer before it waits for the other barriers (-1: not even the slabs)
    int acc_stride;                                // resident scales: TMEM columns between the four accumulators
    int require_res;                               // host only: refuse the launch unless it takes the resident-scales kernel
};


struct UmMaps { CUtensorMap w[B200_GEMV_MULTI_MAX]; CUtensorMap s[B200_GEMV_MULTI_MAX]; };

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 :: "r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr, uint32_t sbo_bytes, uint32_t layout) {
    // start address >> 4 | LBO (unused here) | SBO >> 4 | version 1 | layout type (2 = SWIZZLE_128B, 0 = none)
    return (uint64_t)((saddr >> 4) & 0x3FFF) | ((uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)(layout & 7) << 61);
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(bar) : "memory");
}
// Splits M activation rows x[M, K] (the clamped SwiGLU of x and x2 when x2 != nullptr) into the B image
// `bimg` ([K/256 steps][stride_m rows][8 digits][128 B], 128B-swizzled; shared or global memory) and
// writes gam[m*8 + t] = gamma_m 4^-t.  256 threads (t4 = 0..255) call it together; `red` is shared
// scratch [UM_MAX_M][8]; named barrier 1 is used among the 256.
template <bool SINGLE>
__device__ __forceinline__ void split_rows(const float* x, const float* x2, float lim, int M, int K, int stride_m,
                                           unsigned char* bimg, float* gam, float (*red)[8], int t4) {
    const int lane = t4 & 31;
    auto ldx = [&](const float4* row, const float4* row2, int i) -> float4 {
        float4 v = row[i];
        if (row2) {
            const float4 u = row2[i];
            const float g[4] = {fminf(v.x, lim), fminf(v.y, lim), fminf(v.z, lim), fminf(v.w, lim)};
            const float w[4] = {fminf(fmaxf(u.x, -lim), lim), fminf(fmaxf(u.y, -lim), lim), fminf(fmaxf(u.z, -lim), lim), fminf(fmaxf(u.w, -lim), lim)};
            v = make_float4((g[0] / (1.f + __expf(-g[0]))) * w[0], (g[1] / (1.f + __expf(-g[1]))) * w[1],
                            (g[2] / (1.f + __expf(-g[2]))) * w[2], (g[3] / (1.f + __expf(-g[3]))) * w[3]);
        }
        return v;
    };
    // Pass A: amax of every activation row.  For M == 1 this thread's first 16-group stays in
    // registers for pass B (for K <= 4096 that is all of its work: one trip to memory, not two).
    float4 xv[4];
    auto ab = [](float f) { return __float_as_uint(f) & 0x7fffffffu; };
    if (!SINGLE && M >= 2 && M <= 4) {
        // Two to four rows: the loads of all rows are issued before any row's maximum is reduced (one trip to
        // memory for the pass instead of one per row).
        uint32_t am[4] = {0u, 0u, 0u, 0u};
        for (int i = t4 * 4; i < (K >> 2); i += UM_WORKERS * 4) {
            #pragma unroll
            for (int m = 0; m < 4; ++m) {
                if (m < M) {
                    const float4* xr = reinterpret_cast<const float4*>(x + (size_t)m * K);
                    const float4* xr2 = x2 ? reinterpret_cast<const float4*>(x2 + (size_t)m * K) : nullptr;
                    #pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const float4 v = ldx(xr, xr2, i + q);
                        am[m] = max(am[m], max(max(ab(v.x), ab(v.y)), max(ab(v.z), ab(v.w))));
                    }
                }
            }
        }
        #pragma unroll
        for (int m = 0; m < 4; ++m) {
            if (m < M) {
                uint32_t a = am[m];
                #pragma unroll
                for (int o = 16; o; o >>= 1) a = max(a, __shfl_xor_sync(0xffffffffu, a, o));
                if (lane == 0) red[m][t4 >> 5] = __uint_as_float(a);
            }
        }
    } else
    for (int m = 0; m < M; ++m) {
        const float4* xr = reinterpret_cast<const float4*>(x + (size_t)m * K);
        const float4* xr2 = x2 ? reinterpret_cast<const float4*>(x2 + (size_t)m * K) : nullptr;
        // The maximum is taken over the bit patterns of |x|: they order like the values, and an infinity or
        // a NaN (patterns from 0x7f800000 up) wins the maximum instead of being dropped as fmaxf would.
        uint32_t a = 0u;
        for (int i = t4 * 4; i < (K >> 2); i += UM_WORKERS * 4) {
            #pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float4 v = ldx(xr, xr2, i + q);
                if ((SINGLE || M == 1) && i == t4 * 4) xv[q] = v;
                a = max(a, max(max(ab(v.x), ab(v.y)), max(ab(v.z), ab(v.w))));
            }
        }
        #pragma unroll
        for (int o = 16; o; o >>= 1) a = max(a, __shfl_xor_sync(0xffffffffu, a, o));
        if (lane == 0) red[m][t4 >> 5] = __uint_as_float(a);
    }
    named_sync(1, UM_WORKERS);
    // Pass B: x = gamma * v with |v| < 4; v is kept to 14 fractional bits
    auto row_inv = [&](int m) -> float {
        uint32_t ai = 0u;
        #pragma unroll
        for (int w = 0; w < 8; ++w) ai = max(ai, __float_as_uint(red[m][w]));
        const float a = __uint_as_float(ai);
        // a row with an infinity or a NaN in it yields NaN for every output of that row (the fp32 kernels of
        // the reference propagate non-finite activations too; digits cannot carry them)
        const float gamma = ai >= 0x7f800000u ? __uint_as_float(0x7fc00000u) : (a > 0.f ? a * (1.0f / 3.99f) : 1.f);
        if (t4 < UM_NB) gam[m * UM_NB + t4] = gamma * __uint_as_float((uint32_t)(127 - 2 * t4) << 23);      // gamma * 4^-t
        return 16384.f / gamma;
    };
    // 16 activations of row m (group g) -> 16 words of eight e2m1 codes (nibble j = digit of weight
    // 4^-(7-j)), then two 8x8 nibble transposes so that each digit's 16 codes are contiguous.
    auto split_group = [&](int m, int g, float inv, bool cached) {
        const float4* xr = reinterpret_cast<const float4*>(x + (size_t)m * K);
        const float4* xr2 = x2 ? reinterpret_cast<const float4*>(x2 + (size_t)m * K) : nullptr;
        uint32_t W[16];
        #pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
            const float4 f = cached ? xv[q4] : ldx(xr, xr2, g * 4 + q4);
            const float v[4] = {f.x, f.y, f.z, f.w};
            #pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int iq = __float2int_rn(v[e] * inv);
                uint32_t mm = (uint32_t)min(abs(iq), 65535);
                mm = (mm | (mm << 8)) & 0x00FF00FFu;
                mm = (mm | (mm << 4)) & 0x0F0F0F0Fu;
                mm = (mm | (mm << 2)) & 0x33333333u;                    // one base-4 digit per nibble
                const uint32_t b1 = (mm >> 1) & 0x11111111u, b0 = mm & 0x11111111u;
                uint32_t c = (mm << 1) - (b1 & b0);                        // e2m1 code of the digit: 0,2,4,5
                if (iq < 0) c |= (b1 | b0) << 3;                           // sign on the non-zero digits
                W[q4 * 4 + e] = c;
            }
        }
        #pragma unroll
        for (int h = 0; h < 16; h += 8) {
            #pragma unroll
            for (int r = 0; r < 8; r += 2) { const uint32_t t = ((W[h + r] >> 4) ^ W[h + r + 1]) & 0x0F0F0F0Fu; W[h + r] ^= t << 4; W[h + r + 1] ^= t; }
            #pragma unroll
            for (int r = 0; r < 8; ++r) if (!(r & 2)) { const uint32_t t = ((W[h + r] >> 8) ^ W[h + r + 2]) & 0x00FF00FFu; W[h + r] ^= t << 8; W[h + r + 2] ^= t; }
            #pragma unroll
            for (int r = 0; r < 4; ++r) { const uint32_t t = ((W[h + r] >> 16) ^ W[h + r + 4]) & 0x0000FFFFu; W[h + r] ^= t << 16; W[h + r + 4] ^= t; }
        }
        // W[j] (j < 8): codes of digit 7-j for activations 0..7; W[8 + j]: for activations 8..15.
        // B image: step (256 k) = g / 16, atom m (8 rows of 128 B), row t, 16-byte chunk (g % 16) / 2
        // swizzled with the row, half g % 2
        const int tile = g >> 4, ch = (g & 15) >> 1, hf = g & 1;
        unsigned char* at = bimg + ((size_t)tile * stride_m + m) * 1024 + hf * 8;
        #pragma unroll
        for (int t = 0; t < UM_NB; ++t)
            *reinterpret_cast<uint2*>(at + t * 128 + ((ch ^ t) << 4)) = make_uint2(W[7 - t], W[15 - t]);
    };
    if (SINGLE || M == 1) {
        const float inv = row_inv(0);
        for (int g = t4; g < (K >> 4); g += UM_WORKERS) split_group(0, g, inv, g == t4);
    } else {
        // two rows per trip: two independent dependency chains for the scheduler to interleave
        for (int m = 0; m < M; m += 2) {
            const bool two = m + 1 < M;
            const float inv0 = row_inv(m), inv1 = two ? row_inv(m + 1) : 0.f;
            for (int g = t4; g < (K >> 4); g += UM_WORKERS) {
                split_group(m, g, inv0, false);
                if (two) split_group(m + 1, g, inv1, false);
            }
        }
    }
}

// GEN = false: the decode hot path (one activation row, one tile per CTA, jobs in the parameters,
// plain activations) with the general loops folded away at compile time.
template <bool GEN, bool RES>
__global__ void __launch_bounds__(UM_THREADS, 1)
k_gemv_umma(const __grid_constant__ UmParams p, const __grid_constant__ UmMaps maps) {
    static_assert(!(GEN && RES), "resident scales are a decode-kernel mode");
    const int COL_ACC = RES ? p.acc_stride : 64, COL_SB = RES ? 4 * p.acc_stride : UM_COL_SB, COL_SF = RES ? 4 * p.acc_stride + 16 : UM_COL_SF;
    extern __shared__ __align__(1024) unsigned char smem[];
    __shared__ uint64_t full_bar[UM_MAX_STEPS], sf_bar[UM_MAX_STEPS], empty_bar[UM_MAX_STEPS], done_bar, sc_bar, bi_bar, scd_bar;
    __shared__ uint32_t tmem_base_s;
    __shared__ float gam[UM_MAX_M][UM_NB], red[UM_MAX_M][8];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int K = p.K, nst = K >> 8;               // 256-k steps along K
    // which job / rows
    int ji = 0;
    UmJob J;
    const int T = GEN ? p.T : 1;
    if (GEN && p.table) {
        pdl_wait();                                  // the table is written by an earlier kernel of the stream
        const int per_job = p.tiles_per_job / T;     // CTAs per job (the host makes T divide tiles_per_job)
        ji = (int)blockIdx.x / per_job;
        J = p.table[ji];
        if (J.N <= 0) return;                        // an unused slot of the table: the whole CTA leaves
        J.task0 = ji * per_job;
    } else {
        #pragma unroll
        for (int q = 1; q < B200_GEMV_MULTI_MAX; ++q) if (q < p.n_jobs && (int)blockIdx.x >= p.j[q].task0) ji = q;
        J = p.j[ji];
        J.mw = &maps.w[ji]; J.ms = &maps.s[ji];
    }
    const int row0 = ((int)blockIdx.x - J.task0) * p.R * T;      // first row of the CTA's T tiles
    const int nsteps = T * nst;                      // step g: tile g / nst, 256-k block g % nst
    const int M = GEN ? J.M : (RES ? p.max_m : 1);   // the resident-scales kernel takes up to four rows (all jobs the same number)
    unsigned char* ring = smem + ((1024u - (smem_u32(smem) & 1023u)) & 1023u);      // SWIZZLE_128B tiles need 1 KB alignment
    unsigned char* bimg = ring + p.bimg_off;        // nst tiles of max_m KB: [step][row m][digit t][128 B]
    unsigned char* scl = ring + p.scl_off;          // all scale rows of the CTA: per tile, slabs [R x sc_box]

    pdl_launch_dependents();
    // ---- TMA producer, part one (warp 0): with weights declared stable, the scale slabs and every stage that
    // waits for nothing are requested before anything else happens in the CTA -- before the TMEM allocation and
    // the CTA-wide barrier, on barriers this warp initialises itself.  Lane l issues steps l, l + 32, ...
    const uint32_t full0 = smem_u32(&full_bar[0]), ring0 = smem_u32(ring);
    const int n_early = p.prefetch_before_wait ? min(min(p.stages, p.ov_first), p.early) : 0;
    const bool early_scales = p.prefetch_before_wait && p.early >= 0;
    auto issue_scales = [&]() {
        // All scale rows of the CTA, in slabs [R rows x sc_box bytes]: one tensor load per slab instead of one
        // [R x 16 B] box per step (a box costs the TMA unit ~1 ns per row whatever the row's width).  128-byte
        // slabs are stored 128B-swizzled, so that 32 lanes reading the same 16-byte column of 32 consecutive
        // rows hit different banks.
        const int nslab = (K >> 4) / p.sc_box;
        const uint32_t slab_bytes = (uint32_t)p.R * (uint32_t)(K >> 4);     // one tile's scale rows
        if (lane == 0) mbar_expect_tx(smem_u32(&sc_bar), slab_bytes * (uint32_t)T);
        __syncwarp();
        for (int q = lane; q < T * nslab; q += 32) {
            const int t = q / nslab, sl = q - t * nslab;
            tma_load_2d(smem_u32(scl) + (uint32_t)t * slab_bytes + (uint32_t)sl * (uint32_t)p.R * (uint32_t)p.sc_box,
                        (const CUtensorMap*)J.ms, sl * p.sc_box, row0 + t * p.R, smem_u32(&sc_bar));
        }
    };
    auto issue_stage = [&](int g) {
        const int s = g % p.stages, t = g / nst, it = g - t * nst;
        const uint32_t bar = full0 + g * 8, dst = ring0 + (uint32_t)s * p.stage_bytes;
        mbar_expect_tx(bar, (uint32_t)p.R * 128u);
        tma_load_2d(dst, (const CUtensorMap*)J.mw, it * 128, row0 + t * p.R, bar);
    };
    if (warp == 0) {
        for (int i = lane; i < nsteps; i += 32) mbar_init(full0 + i * 8, 1);
        if (lane == 0) mbar_init(smem_u32(&sc_bar), 1);
        mbar_fence_init();
        __syncwarp();
        if (early_scales) {
            issue_scales();
            for (int g = lane; g < n_early; g += 32) issue_stage(g);
        }
    }
    // No CTA-wide barrier in the prologue: the workers go straight to the dependency wait and the activation
    // loads (the longest chain of the kernel); the MMA warps initialise the other barriers and allocate TMEM,
    // and meet the producer at named barrier 3; the workers learn of all that at named barrier 2.
    const bool mma_warp = warp >= UM_LOAD_WARPS && warp < UM_LOAD_WARPS + UM_MMA_WARPS;
    if (mma_warp) {
        const int i = tid - UM_LOADERS;
        for (int k = i; k < nsteps; k += 32 * UM_MMA_WARPS) {
            mbar_init(smem_u32(&sf_bar[k]), 128);
            mbar_init(smem_u32(&empty_bar[k]), 1);
        }
        if (i == 0) mbar_init(smem_u32(&done_bar), UM_MMA_WARPS);
        if (i == 1) mbar_init(smem_u32(&scd_bar), UM_MMA_WARPS);
        mbar_fence_init();
        if (warp == UM_LOAD_WARPS) {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_u32(&tmem_base_s)), "r"(UM_TMEM_COLS));
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
        }
        tc_fence_before();
    }
    // The producer waits at barrier 3 for the MMA warps' initialisations; they only arrive there (the
    // producer has nothing they need) and meet among themselves at barrier 4 for the TMEM address.
    if (warp == 0) named_sync(3, 32 + 32 * UM_MMA_WARPS);
    if (mma_warp) {
        asm volatile("bar.arrive 3, %0;" :: "r"(32 + 32 * UM_MMA_WARPS) : "memory");
        named_sync(4, 32 * UM_MMA_WARPS);
    }
    uint32_t tmem = 0u, tq = 0u;                     // TMEM base; the lane quadrant this warp may access (set once the role knows the base)
    // Weight scales, shared memory -> TMEM.  Lane l holds rows l, l+32, l+64, l+96: 16 bytes each = four
    // k-blocks x four scales; k-block kb of row 32c + l goes to column kb*4 + c.  Within a group of four
    // warps each warp writes its own TMEM lane quadrant (the MMA wants the 32-lane block in all four).
    const uint32_t slab_bytes = (uint32_t)p.R * (uint32_t)(K >> 4);     // one tile's scale rows
    auto load_scales = [&](int t, int it, uint4 (&v)[4]) {
        const unsigned char* sl = scl + (uint32_t)t * slab_bytes;
        const int valid = J.N - (row0 + t * p.R);            // rows of this tile that exist (may exceed R)
        #pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int r = lane + 32 * c;
            uint32_t off;
            if (p.sc_swz) off = (uint32_t)(it >> 3) * (uint32_t)p.R * 128u + (uint32_t)r * 128u + (uint32_t)(((it & 7) ^ (r & 7)) << 4);
            else off = (uint32_t)r * (uint32_t)p.sc_box + (uint32_t)it * 16u;
            v[c] = (r < p.R && r < valid) ? *reinterpret_cast<const uint4*>(sl + off) : make_uint4(0u, 0u, 0u, 0u);
        }
    };
    auto store_scales = [&](uint32_t slot, const uint4 (&v)[4]) {
        asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                     :: "r"(tq + COL_SF + slot * 16u),
                        "r"(v[0].x), "r"(v[1].x), "r"(v[2].x), "r"(v[3].x), "r"(v[0].y), "r"(v[1].y), "r"(v[2].y), "r"(v[3].y),
                        "r"(v[0].z), "r"(v[1].z), "r"(v[2].z), "r"(v[3].z), "r"(v[0].w), "r"(v[1].w), "r"(v[2].w), "r"(v[3].w) : "memory");
    };

    if (warp < UM_LOAD_WARPS) {
        // ---- TMA producer, part two: warp 0; lane l issues the loads of steps l, l + 32, ... ----
        // One thread issuing tensor loads back to back gets one out every ~0.35 us (measured), so
        // the steps are dealt to the lanes: each lane waits for its own stage and issues on its own.
        if (warp == 0) {
            const uint32_t empty0 = smem_u32(&empty_bar[0]);
            if (!early_scales) {
                if (lane == 0) { asm volatile("prefetch.tensormap [%0];" :: "l"(J.mw) : "memory");
                                 asm volatile("prefetch.tensormap [%0];" :: "l"(J.ms) : "memory"); }
                if (!p.prefetch_before_wait) pdl_wait();
                issue_scales();
            }
            for (int g = lane; g < nsteps; g += 32) {
                if (g < n_early) continue;
                if (g >= p.stages) UM_WAIT(empty0 + (g - p.stages) * 8, 0, p.status, 1);      // the step that had this stage is done
                else if (RES && g % p.stages >= p.ov_first) UM_WAIT(smem_u32(&scd_bar), 0, p.status, 8);   // the slabs under this stage are in TMEM
                issue_stage(g);
            }
            __syncwarp();
            // Tail: the tcgen05.commit arrivals on empty_bar are asynchronous.  Wait for the last one
            // of every stage, or the CTA could exit with an arrival still in flight and it would
            // land on whatever the next CTA keeps at that shared-memory address.
            for (int g = max(0, nsteps - p.stages) + lane; g < nsteps; g += 32)
                UM_WAIT(empty0 + g * 8, 0, p.status, 5);
            __syncwarp();
        }
        else if (warp == 1 && !GEN) {
            // L2 prefetch of the steps the ring cannot take at once (legal before the upstream kernel
            // has finished: L2 is the point of coherence).  Only on the single-tile path: a prefetch
            // costs the TMA unit as much as a load, and a multi-tile CTA would queue dozens of them.
            for (int g = (RES ? min(p.stages, p.ov_first) : p.stages) + lane; g < nsteps; g += 32) {
                const int t = g / nst, it = g - t * nst;
                asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];"
                             :: "l"(J.mw), "r"(it * 128), "r"(row0 + t * p.R) : "memory");
            }
        }
    } else if (warp < UM_LOAD_WARPS + UM_MMA_WARPS) {
        // ---- MMA issuers: warp w takes the steps g with g % 4 == w ----
        tc_fence_after();
        tmem = tmem_base_s;
        tq = tmem + ((uint32_t)((warp & 3) * 32) << 16);
        {
            // unit block scales of the activation digits (e4m3 1.0), once: each warp its own lane quadrant
            const uint32_t one = 0x38383838u;
            asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %1, %1, %1};" :: "r"(tq + COL_SB), "r"(one) : "memory");
        }
        if (RES) {
            // Resident scales: every step has its own TMEM slot, and these four warps (one per lane quadrant)
            // have nothing else to do until the activations are split: they move all the scales, needing
            // only the slabs.  After that the slabs' shared memory belongs to the ring (scd_bar).
            UM_WAIT(smem_u32(&sc_bar), 0, p.status, 6);
            // Warp w takes its own MMA steps g = w, w + 4, ...  A step's scales are [R rows][4 k-blocks x 4 B] in
            // the slab; the tensor core's copy (tcgen05.cp 32x128b.warpx4) wants, per k-block, 32 rows of 16 B
            // where row l holds the 4-byte scales of weight rows l, l+32, l+64, l+96: it writes them to TMEM
            // lane l, columns 0..3, in all four lane quadrants -- the layout the block-scaled MMA reads.  Lane
            // l transposes its 4 x 4 words in registers; the copies are issued by the lane that issues the
            // step's MMAs later (same thread: they execute in order), and a commit tells the producer when
            // the shared memory under them is free.
            unsigned char* tsc = ring + p.tsc_off;         // [step][k-block][32 rows][16 B]
            const int me = warp - UM_LOAD_WARPS;
            for (int g = me; g < nsteps; g += UM_MMA_WARPS) {
                uint4 v[4];
                load_scales(0, g, v);
                uint4* o = reinterpret_cast<uint4*>(tsc + (size_t)g * 2048 + (size_t)lane * 16);
                o[0] = make_uint4(v[0].x, v[1].x, v[2].x, v[3].x);
                o[32] = make_uint4(v[0].y, v[1].y, v[2].y, v[3].y);
                o[64] = make_uint4(v[0].z, v[1].z, v[2].z, v[3].z);
                o[96] = make_uint4(v[0].w, v[1].w, v[2].w, v[3].w);
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) {
                for (int g = me; g < nsteps; g += UM_MMA_WARPS) {
                    #pragma unroll
                    for (int kb = 0; kb < 4; ++kb) {
                        // 32 rows x 16 B, contiguous: four 8-row core matrices 128 B apart, no swizzle
                        const uint64_t sd = umma_desc(smem_u32(tsc) + (uint32_t)g * 2048u + (uint32_t)kb * 512u, 128, 0) | ((uint64_t)(128 >> 4) << 16);
                        asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;"
                                     :: "r"(tmem + COL_SF + (uint32_t)g * 16u + (uint32_t)kb * 4u), "l"(sd) : "memory");
                    }
                }
                tc_commit(smem_u32(&scd_bar));
            }
            __syncwarp();
        }
        // General kernel: these warps are idle while the workers split the activations, so they move the scales of
        // the steps of the ring's first round (a slot each, free at this point); the workers take over from there.
        const int npre = RES ? 0 : (min(nsteps, p.stages) & ~1);       // even: the two worker groups keep their parity
        if (!RES && npre > 0) {
            UM_WAIT(smem_u32(&sc_bar), 0, p.status, 6);
            int t = 0, it = 0;
            for (int g = 0; g < npre; ++g) {
                uint4 v[4];
                load_scales(t, it, v);
                store_scales((uint32_t)g, v);
                if (++it == nst) { it = 0; ++t; }
            }
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        tc_fence_before();
        for (int g = 0; g < npre; ++g) mbar_arrive(smem_u32(&sf_bar[g]));
        if (RES && warp - UM_LOAD_WARPS < nsteps)        // this warp's first step: its weights are awaited now rather than after the barrier
            UM_WAIT(full0 + (warp - UM_LOAD_WARPS) * 8, 0, p.status, 3);
        const int me = warp - UM_LOAD_WARPS;
        const uint32_t idesc = (1u << 7) | (1u << 10) | ((uint32_t)M << 17) | ((128u >> 4) << 24);     // N = 8 M
        const uint64_t dA0 = umma_desc(smem_u32(ring), 1024, 2), dB0 = umma_desc(smem_u32(bimg), 1024, 2);
        const uint32_t tSB = tmem + COL_SB;
        const uint32_t sf0 = smem_u32(&sf_bar[0]), empty0 = smem_u32(&empty_bar[0]);
        named_sync(2, 32 * UM_MMA_WARPS + UM_WORKERS);   // B image, unit and weight scales and gam[] are ready
        tc_fence_after();
        {
            int s = me % p.stages;
            int t = me / nst, it = me - t * nst;                       // tile and k-block of step g, kept without divisions
            for (int g = me; g < nsteps; g += UM_MMA_WARPS) {          // whole warp waits, lane 0 issues
                const uint32_t tsf = tmem + COL_SF + (uint32_t)(RES ? g : s) * 16u;
                // accumulator it % 4 of tile t: fixed by the k-block alone, so that the summation order of a
                // row does not depend on which tile of the CTA it is in (or on how many tiles a CTA takes)
                const uint32_t tD = tmem + (uint32_t)((it & 3) * COL_ACC + t * 8 * M);
                const uint64_t dA = dA0 + (((uint32_t)s * p.stage_bytes) >> 4), dB = dB0 + (uint32_t)(it * p.max_m) * 64u;
                const uint32_t acc0 = it >= 4;                          // the first k-block of an accumulator starts it
                UM_WAIT((RES ? full0 : sf0) + g * 8, 0, p.status, 3);      // resident scales: only the step's weights are awaited
                if (!RES && g < npre) UM_WAIT(full0 + g * 8, 0, p.status, 2);   // scales moved ahead of the weights: wait for those too
                tc_fence_after();
                if (lane == 0) {
                    #pragma unroll
                    for (int kb = 0; kb < 4; ++kb) {                           // K % 256 == 0: always four 64-k blocks
                        asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                                     " tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n}"
                                     :: "r"(tD), "l"(dA + kb * 2), "l"(dB + kb * 2), "r"(idesc), "r"(kb ? 1u : acc0),
                                        "r"(tsf + kb * 4), "r"(tSB) : "memory");
                    }
                    tc_commit(empty0 + g * 8);
                }
                __syncwarp();
                s += UM_MMA_WARPS; while (s >= p.stages) s -= p.stages;
                it += UM_MMA_WARPS; while (it >= nst) { it -= nst; ++t; }
            }
            if (lane == 0) tc_commit(smem_u32(&done_bar));
            __syncwarp();
        }
    } else {
        // ---- workers: activation split, then per-step scale copies; the first four warps also the epilogue ----
        const int t4 = tid - UM_LOADERS - 32 * UM_MMA_WARPS;      // 0..255
        const int q4 = warp & 3;
        pdl_wait();
        const float gsv = J.gs[0];
        if (GEN && J.bimg) {
            // The B image was split once for all CTAs of the job by k_split_rows: copy it in.
            const uint32_t total = (uint32_t)nst * (uint32_t)p.max_m * 1024u;
            if (t4 == 0) { mbar_init(smem_u32(&bi_bar), 1); mbar_fence_init(); mbar_expect_tx(smem_u32(&bi_bar), total); }
            named_sync(1, UM_WORKERS);
            for (uint32_t o = (uint32_t)t4 * 16384u; o < total; o += UM_WORKERS * 16384u)
                bulk_g2s(smem_u32(bimg) + o, J.bimg + o, min(16384u, total - o), smem_u32(&bi_bar));
            if (t4 < M * UM_NB) (&gam[0][0])[t4] = J.gam[t4];
            UM_WAIT(smem_u32(&bi_bar), 0, p.status, 7);
        } else {
            if (!GEN && M == 1) split_rows<true>(J.x, nullptr, p.limit, 1, K, p.max_m, bimg, &gam[0][0], red, t4);
            else split_rows<false>(J.x, GEN ? J.x2 : nullptr, p.limit, M, K, p.max_m, bimg, &gam[0][0], red, t4);
        }
        fence_async_smem();
        tc_fence_before();
        named_sync(2, 32 * UM_MMA_WARPS + UM_WORKERS);   // with the MMA warps
        tc_fence_after();
        tmem = tmem_base_s;
        tq = tmem + ((uint32_t)(q4 * 32) << 16);
        if (!RES) {
            // The first four worker warps take the even steps, the other four the odd ones; a step's scales
            // go to the TMEM slot of its stage.
            const uint32_t full0 = smem_u32(&full_bar[0]), sf0 = smem_u32(&sf_bar[0]);
            const int grp = t4 >> 7;
            const int g0 = (min(nsteps, p.stages) & ~1) + grp;        // the MMA warps moved the steps before that
            int s = g0 % p.stages;
            UM_WAIT(smem_u32(&sc_bar), 0, p.status, 6);
            // Software-pipelined: the next step's scale bytes are read from shared memory while this
            // step's tcgen05.st is in flight.
            int rt = g0 / nst, rit = g0 - rt * nst;                    // tile and k-block of the next step to read
            auto read_scales = [&](int g, uint4 (&v)[4]) {
                // full[g] also says that the MMAs that last read this stage's scale slot are done
                UM_WAIT(full0 + g * 8, 0, p.status, 2);
                const int t = rt, it = rit;
                rit += 2; while (rit >= nst) { rit -= nst; ++rt; }
                load_scales(t, it, v);
            };
            uint4 v[4], vn[4];
            if (g0 < nsteps) read_scales(g0, v);
            for (int g = g0; g < nsteps; g += 2) {
                store_scales((uint32_t)s, v);
                if (g + 2 < nsteps) read_scales(g + 2, vn);
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                tc_fence_before();
                mbar_arrive(sf0 + g * 8);
                s += 2; while (s >= p.stages) s -= p.stages;
                #pragma unroll
                for (int c = 0; c < 4; ++c) v[c] = vn[c];
            }
        }
        if (t4 < 128) {
            // epilogue
            UM_WAIT(smem_u32(&done_bar), 0, p.status, 4);
            tc_fence_after();
            const int r = q4 * 32 + lane;
            for (int t = 0; t < T; ++t) {
                const int row = row0 + t * p.R + r;
                for (int m = 0; m < M; ++m) {
                    // tile t, activation row m: columns t*8M + m*8 .. +7 of each of the four accumulators
                    uint32_t d[4][8];
                    #pragma unroll
                    for (int w = 0; w < 4; ++w)
                        asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                                     : "=r"(d[w][0]), "=r"(d[w][1]), "=r"(d[w][2]), "=r"(d[w][3]), "=r"(d[w][4]), "=r"(d[w][5]), "=r"(d[w][6]), "=r"(d[w][7])
                                     : "r"(tq + (uint32_t)(w * COL_ACC + t * 8 * M + m * 8)));
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (r < p.R && row < J.N) {
                        float acc = 0.f;
                        #pragma unroll
                        for (int dg = UM_NB - 1; dg >= 0; --dg) {          // small terms first
                            float dsum = __uint_as_float(d[0][dg]);
                            #pragma unroll
                            for (int w = 1; w < 4; ++w) if (w < nst) dsum += __uint_as_float(d[w][dg]);   // accumulators that had a k-block
                            acc = fmaf(dsum, gam[m][dg], acc);
                        }
                        J.y[(size_t)m * J.N + row] = acc / gsv;
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == UM_LOAD_WARPS) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem), "r"(UM_TMEM_COLS));
}


// Pre-split activations of a gemm: chunk c (rows 8c..8c+7) has its image at img + c * chunk_bytes
// (rows at `stride`) and its digit weights at gam + c * 64.
struct PreSplit { unsigned char* img; float* gam; size_t chunk_bytes; int stride; int chunk; bool dry_run; };

// One CTA per activation row of x [M, K].
__global__ void __launch_bounds__(UM_WORKERS)
k_split_x(const float* __restrict__ x, int K, int stride, unsigned char* __restrict__ img, size_t chunk_bytes, float* __restrict__ gam) {
    __shared__ float red[UM_MAX_M][8];
    pdl_wait();
    const int m = blockIdx.x, c = m / UM_MAX_M, r = m - c * UM_MAX_M;
    split_rows<false>(x + (size_t)m * K, nullptr, 0.f, 1, K, stride, img + (size_t)c * chunk_bytes + (size_t)r * 1024,
                      gam + (size_t)c * UM_MAX_M * UM_NB + r * UM_NB, red, (int)threadIdx.x);
}

// ---- host side ---------------------------------------------------------------------------------
// u8 matrix [rows, row_bytes]; box [box_bytes x box_rows]; maps of weights are remembered (tmap.cu).
static bool make_map(CUtensorMap* m, const void* base, int rows, size_t row_bytes, int box_bytes, int box_rows, bool swz) {
    return tmap_u8_2d(m, base, (size_t)rows, row_bytes, box_bytes, box_rows, swz, true);
}

// Conditions: M = 1 (one activation row shared by all jobs), K % 256 == 0 and K <= 16384, 16-byte
// aligned tensors and activation, at least 256 rows in total.
static int umma_launch(const GemvParams& g, int M, int m0, cudaStream_t s, const PreSplit* pre, bool require_res = false);
static int umma_finish_launch(UmParams& p, const UmMaps& maps, int tasks, cudaStream_t s);

// Rows of the activations are taken in chunks that fit the shared memory (the B image takes M KB
// per 256 k); every chunk size computes each row with the same arithmetic, so results do not
// depend on how the rows were chunked.
int nvfp4_multi_umma(const GemvParams& g, int M, cudaStream_t s) {
    if (M < 1) return B200_ENOTIMPL;
    int done = 0, cap = UM_MAX_M;                    // cap: the chunk size the first launch settled on
    while (done < M) {
        int mc = std::min(cap, M - done), rc = umma_launch(g, mc, done, s, nullptr);
        while (rc == B200_ENOTIMPL && done == 0 && mc > 1) { mc /= 2; rc = umma_launch(g, mc, done, s, nullptr); }
        if (rc != B200_OK) return rc;                // ENOTIMPL only before anything was launched
        cap = mc; done += mc;
    }
    return B200_OK;
}

// The same with the activation rows split beforehand, once, into caller-supplied scratch: one
// k_split_x launch for all M rows, then one pass per 8 rows whose CTAs copy their image in instead
// of each splitting the rows again.  All jobs must share one activation matrix.
size_t umma_presplit_bytes(int M, int K) {
    const size_t chunks = ((size_t)M + UM_MAX_M - 1) / UM_MAX_M, stride = (size_t)std::min(M, UM_MAX_M);
    return chunks * (size_t)(K / 256) * stride * 1024 + chunks * UM_MAX_M * UM_NB * 4;
}
int nvfp4_multi_umma_ws(const GemvParams& g, int M, void* ws, cudaStream_t s) {
    const int K = g.K;
    if (M < 2 || !ws || ((uintptr_t)ws & 255) || (K & 255) || K > 16384) return B200_ENOTIMPL;
    for (int i = 0; i < g.n_jobs; ++i) if (g.j[i].x != g.j[0].x) return B200_ENOTIMPL;
    if ((uintptr_t)g.j[0].x & 15) return B200_ENOTIMPL;
    // Up to four rows: one launch of the resident-scales kernel, which splits the rows itself (the same digits,
    // so the same bits as the split-once path below), instead of a split launch and a product launch.
    if (M <= UM_RES_MAX_M) {
        const int rc = umma_launch(g, M, 0, s, nullptr, true);
        if (rc != B200_ENOTIMPL) return rc;
    }
    PreSplit pre{};
    pre.stride = std::min(M, UM_MAX_M);
    pre.chunk_bytes = (size_t)(K / 256) * pre.stride * 1024;
    const int chunks = (M + UM_MAX_M - 1) / UM_MAX_M;
    pre.img = static_cast<unsigned char*>(ws);
    pre.gam = reinterpret_cast<float*>(pre.img + (size_t)chunks * pre.chunk_bytes);
    // does a pass fit at all?  (asked before anything is launched, so that the caller can fall back)
    {
        pre.dry_run = true;
        const int probe = umma_launch(g, std::min(M, UM_MAX_M), 0, s, &pre);
        pre.dry_run = false;
        if (probe != B200_OK) return probe;
    }
    k_split_x<<<M, UM_WORKERS, 0, s>>>(g.j[0].x, K, pre.stride, pre.img, pre.chunk_bytes, pre.gam);
    if (int rc = check_launch("k_split_x")) return rc;
    for (int done = 0; done < M; done += UM_MAX_M) {
        pre.chunk = done / UM_MAX_M;
        if (int rc = umma_launch(g, std::min(UM_MAX_M, M - done), done, s, &pre)) return rc == B200_ENOTIMPL ? B200_ELAUNCH : rc;
    }
    return B200_OK;
}

// One launch: activation rows [m0, m0 + M) of every job.
static int umma_launch(const GemvParams& g, int M, int m0, cudaStream_t s, const PreSplit* pre, bool require_res) {
    const int K = g.K;
    if ((K & 255) || K > 16384 || !tmap_available()) return B200_ENOTIMPL;
    if (M < 1 || M > UM_MAX_M) return B200_ENOTIMPL;
    for (int i = 0; i < g.n_jobs; ++i)
        if (((uintptr_t)g.j[i].x & 15) || ((uintptr_t)g.j[i].P & 15) || ((uintptr_t)g.j[i].S & 15)) return B200_ENOTIMPL;
    const int nsm = sm_count();
    int R = 128;
    for (int r = 8; r <= 128; r += 8) {
        int tasks = 0;
        for (int i = 0; i < g.n_jobs; ++i) tasks += (g.j[i].N + r - 1) / r;
        if (tasks <= nsm) { R = r; break; }
    }
    static thread_local UmMaps maps;                 // copied into the launch; one per host thread
    UmParams p{};
    p.n_jobs = g.n_jobs; p.K = K; p.R = R; p.max_m = pre ? pre->stride : M; p.T = 1;
    p.dry_run = pre && pre->dry_run;
    p.require_res = require_res ? 1 : 0;
    if (!scale_box(K, &p.sc_box, &p.sc_swz)) return B200_ENOTIMPL;
    {
        // More tiles than SMs even at R = 128 (a vocabulary projection, a fused pair of wide projections): a CTA
        // takes T consecutive tiles of R rows, so that it splits the activations and fills its pipeline once.
        // (R, T) by estimated time: a wave of CTAs costs its rows plus a fixed part worth about 40 rows; a last
        // wave that fills only part of the SMs runs faster per CTA, but not below 0.4 of a full wave's time.
        // Same limits as the job-table launches; the results do not depend on R or T.
        long tiles128 = 0;
        for (int i = 0; i < g.n_jobs; ++i) tiles128 += (g.j[i].N + 127) / 128;
        // Up to two waves of single tiles stay as they are: one tile per CTA keeps the resident-scales kernel, whose
        // fixed part is half the general kernel's, and the second wave starts SM by SM as the first one drains
        // (two fused [12288 x 4096] projections: 192 single tiles 17 us, 96 CTAs of two tiles 22 us, measured).
        if (tiles128 > 2 * nsm) {
            const int nst = K / 256;
            double best = -1.0;
            for (int T = 1; T * p.max_m <= 8 && T * nst <= UM_MAX_STEPS; ++T)
                for (int r = 32; r <= 128; r += 8) {
                    if ((size_t)T * r * (K / 16) + (size_t)nst * p.max_m * 1024 + 4 * (((size_t)r * 128 + 1023) & ~(size_t)1023) > 200 * 1024) continue;
                    long ctas = 0;
                    for (int i = 0; i < g.n_jobs; ++i) ctas += ((g.j[i].N + r - 1) / r + T - 1) / T;
                    const long full = ctas / nsm, rem = ctas - full * nsm;
                    const double rows = (double)r * T;
                    const double cost = full * (rows + 40.0) + (rem ? rows * std::max((double)rem / nsm, 0.4) + 40.0 : 0.0);
                    if (best < 0.0 || cost < best - 1e-9 || (cost < best + 1e-9 && r > R)) { best = cost; R = r; p.T = T; }
                }
            p.R = R;
        }
    }
    int tasks = 0;
    for (int i = 0; i < g.n_jobs; ++i) {
        p.j[i] = UmJob{g.j[i].y + (size_t)m0 * g.j[i].N, g.j[i].x + (size_t)m0 * K, nullptr, g.j[i].gs, nullptr, nullptr,
                       pre ? pre->img + (size_t)pre->chunk * pre->chunk_bytes : nullptr,
                       pre ? pre->gam + (size_t)pre->chunk * UM_MAX_M * UM_NB : nullptr, g.j[i].N, M, tasks, 0};
        tasks += ((g.j[i].N + R - 1) / R + p.T - 1) / p.T;
        if (!make_map(&maps.w[i], g.j[i].P, g.j[i].N, (size_t)K / 2, 128, R, true) ||
            !make_map(&maps.s[i], g.j[i].S, g.j[i].N, (size_t)K / 16, p.sc_box, R, p.sc_swz != 0)) return B200_ENOTIMPL;
    }
    for (int i = g.n_jobs; i < B200_GEMV_MULTI_MAX; ++i) { p.j[i] = p.j[0]; p.j[i].task0 = 0x7fffffff; maps.w[i] = maps.w[0]; maps.s[i] = maps.s[0]; }
    return umma_finish_launch(p, maps, tasks, s);
}

// Everything after the jobs are known: shared-memory budget, stage count, launch.
static int umma_finish_launch(UmParams& p, const UmMaps& maps, int tasks, cudaStream_t s) {
    const int K = p.K, R = p.R, M = p.max_m;
    p.stage_bytes = ((uint32_t)R * 128u + 1023u) & ~1023u;
    const int nst = K / 256;
    size_t fixed = (size_t)nst * M * 1024 + (size_t)p.T * R * (K / 16);      // B image | scale slabs of the T tiles
    // The MMA is always 128 rows tall: it reads 16 KB from the start of a stage even when only R
    // rows were loaded (the extra accumulator rows are never stored).  Keep that read inside the
    // allocation for the last stage as well.
    if (p.stage_bytes + fixed < 16384) fixed = 16384 - p.stage_bytes;
    const bool presplit = p.table == nullptr && p.j[0].bimg != nullptr;
    const bool res = p.table == nullptr && !presplit && p.T == 1 && p.max_m <= UM_RES_MAX_M && nst <= um_res_steps(p.max_m);
    const bool gen = !res && (p.table != nullptr || p.max_m != 1 || p.T != 1);
    if (p.require_res && !res) return B200_ENOTIMPL;
    p.acc_stride = um_res_acc_stride(p.max_m);
    const int var = gen ? 0 : res ? 2 : 1;
    auto kern = gen ? k_gemv_umma<true, false> : res ? k_gemv_umma<false, true> : k_gemv_umma<false, false>;
    // static shared memory of the kernel and the device's opt-in limit: asked once per device and variant
    static int attr_cache[64][3][2] = {};            // [device][variant] = {optin, static bytes + 1}
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return launch_failed("gemv_umma: cudaGetDevice");
    int* ac = attr_cache[dev >= 0 && dev < 64 ? dev : 0][var];
    if (!ac[1]) {
        cudaFuncAttributes fa;
        int oi = 0;
        if (cudaFuncGetAttributes(&fa, kern) != cudaSuccess ||
            cudaDeviceGetAttribute(&oi, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess) return launch_failed("gemv_umma: attributes");
        ac[0] = oi; ac[1] = (int)fa.sharedSizeBytes + 1;
    }
    const int optin = ac[0];
    const size_t static_smem = (size_t)ac[1] - 1;
    const size_t room = (size_t)optin - static_smem - 2048;    // 1 KB alignment slack + 1 KB system reserve
    if (fixed + 2 * (size_t)p.stage_bytes > room) return B200_ENOTIMPL;
    const int nsteps = p.T * nst;
    size_t total;                                    // dynamic shared memory from the aligned ring base
    if (res) {
        // Ring | transposed scales | slabs | B image when everything fits; otherwise the transposed scales and
        // the slabs lie under the last stages of the ring (which wait until the scales are in TMEM), so that the
        // ring is as deep as the SM allows.
        const size_t bimg = (size_t)nst * M * 1024, sc = ((size_t)R * (K / 16) + 1023) & ~(size_t)1023, tsc = (size_t)nsteps * 2048;
        if ((size_t)nsteps * p.stage_bytes + tsc + sc + bimg <= room) {
            p.stages = nsteps; p.tsc_off = (uint32_t)nsteps * p.stage_bytes; p.ov_first = nsteps;
            p.scl_off = p.tsc_off + (uint32_t)tsc;
            p.bimg_off = p.scl_off + (uint32_t)sc;
        } else {
            p.stages = (int)std::min<size_t>(nsteps, (room - bimg) / p.stage_bytes);
            const size_t ring = std::max((size_t)p.stages * p.stage_bytes, tsc + sc);
            p.scl_off = (uint32_t)(ring - sc); p.tsc_off = p.scl_off - (uint32_t)tsc;
            p.ov_first = (int)(p.tsc_off / p.stage_bytes);
            p.bimg_off = (uint32_t)ring;
        }
        total = std::max((size_t)p.bimg_off + bimg, (size_t)(p.stages - 1) * p.stage_bytes + 16384);
        if (total > room || (p.stages < 3 && p.stages < nsteps)) return B200_ENOTIMPL;
    } else {
        p.stages = (int)std::min<size_t>(std::min(UM_MAX_STAGES, nsteps), (room - fixed) / p.stage_bytes);
        // The scale warps look two steps ahead before they release a step: with a ring of two that
        // would wait for itself.
        if (p.stages < 3 && p.stages < nsteps) return B200_ENOTIMPL;
        p.bimg_off = (uint32_t)p.stages * p.stage_bytes;
        p.scl_off = p.bimg_off + (uint32_t)nst * (uint32_t)M * 1024u;
        p.ov_first = p.stages;
        total = (size_t)p.stages * p.stage_bytes + fixed;
    }
    p.status = device_status_ptr();
    if (!p.status) return B200_ENOTIMPL;
    p.prefetch_before_wait = stable_weights_option();
    // Measured on the decode shapes (six siblings, K = 4096, 16 stages resident): 4 stages at once 7.1-7.3 us per
    // launch, 2: 7.5, 0: 7.7, 8: 7.9, all 16: 8.1-8.4.  A flood of requests from every SM at once delays what
    // each SM needs first (its scale slabs, the activation row); pacing later requests by earlier arrivals was
    // slower still (a window of 4 stages: 8.2, of 6: 7.5).
    p.early = 4;
    if (p.dry_run) return B200_OK;
    const size_t smem = total + 1024;
    static bool ready_all[64][3] = {};               // the attribute is per device
    bool* ready = ready_all[dev >= 0 && dev < 64 ? dev : 0];
    if (!ready[var]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(optin - static_smem)) != cudaSuccess)
            return launch_failed("gemv_umma: cudaFuncSetAttribute");
        ready[var] = true;
    }
    cudaLaunchConfig_t lc{};
    lc.gridDim = dim3(tasks); lc.blockDim = dim3(UM_THREADS); lc.dynamicSmemBytes = smem; lc.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = at; lc.numAttrs = 1;
    if (cudaLaunchKernelEx(&lc, kern, p, maps) != cudaSuccess) return launch_failed("k_gemv_umma");
    return check_launch("k_gemv_umma");
}

// ---- activation rows split once for many CTAs ------------------------------------------------------
__global__ void __launch_bounds__(UM_WORKERS)
k_split_rows(const SplitJob* __restrict__ jobs, int K, float limit) {
    __shared__ float red[UM_MAX_M][8];
    pdl_wait();
    const SplitJob j = jobs[blockIdx.x];
    if (j.M <= 0) return;
    split_rows<false>(j.x, j.x2, limit, j.M, K, UM_MAX_M, j.bimg, j.gam, red, (int)threadIdx.x);
}

int umma_split_launch(const SplitJob* jobs, int n_jobs, int K, float limit, cudaStream_t s) {
    k_split_rows<<<n_jobs, UM_WORKERS, 0, s>>>(jobs, K, limit);
    return check_launch("k_split_rows");
}

// ---- job-table launches (the MoE experts) ---------------------------------------------------------
bool umma_shape_ok(int K) { int b, z; return !(K & 255) && K <= 16384 && scale_box(K, &b, &z) && tmap_available(); }

int umma_encode_maps(void* out_w, void* out_s, const void* P, const void* S, int N, int K, int R) {
    int box = 0, swz = 0;
    if (!umma_shape_ok(K) || !scale_box(K, &box, &swz) || ((uintptr_t)P & 15) || ((uintptr_t)S & 15)) return B200_ENOTIMPL;
    if (!tmap_u8_2d(out_w, P, (size_t)N, (size_t)K / 2, 128, R, true, false) ||
        !tmap_u8_2d(out_s, S, (size_t)N, (size_t)K / 16, box, R, swz != 0, false)) return B200_ENOTIMPL;
    return B200_OK;
}

// n_jobs jobs of N weight rows and up to max_m activation rows each, described by `table` (device memory, filled by an earlier
// kernel of the stream); every job's tensor maps were encoded with box height R.
int umma_table_launch(const UmJob* table, int n_jobs, int N, int K, int R, float limit, int max_m, cudaStream_t s) {
    static UmMaps none{};                            // unused in table mode, still a kernel parameter
    UmParams p{};
    p.table = table; p.limit = limit; p.n_jobs = n_jobs; p.K = K; p.R = R; p.max_m = max_m;
    p.tiles_per_job = (N + R - 1) / R;
    if (!scale_box(K, &p.sc_box, &p.sc_swz)) return B200_ENOTIMPL;
    // Tiles per CTA: as many as still leave every SM a CTA.  A CTA splits its activation row and
    // fills its pipeline once, whatever its number of tiles.  Limits: 64 steps (barriers), 8 tiles
    // (accumulator columns), and the tiles' scale rows must fit beside four stages.
    const int nst = K / 256, nsm = sm_count();
    p.T = 1;
    for (int T = 2; T * max_m <= 8; ++T) {
        if (p.tiles_per_job % T || T * nst > UM_MAX_STEPS) continue;
        if ((size_t)T * R * (K / 16) + (size_t)nst * 1024 + 4 * (((size_t)R * 128 + 1023) & ~(size_t)1023) > 200 * 1024) continue;
        if ((long)n_jobs * (p.tiles_per_job / T) >= nsm - nsm / 16) p.T = T;
    }
    return umma_finish_launch(p, none, n_jobs * (p.tiles_per_job / p.T), s);
}

}  // namespace b200

