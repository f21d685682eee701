// ep.cu -- expert-parallel MoE layer: the experts of one layer sharded over the GPUs of one node,
// host side in C++ behind the C ABI, exchange over NCCL.
//
// The reference is single-GPU (all 144 experts behind one device-side table, src/engine.cu:168-195);
// this is the multi-GPU form of the same block (kernels/moe.cu:669-740: route, experts, fixed-order
// gate sum :584-597).  One process per GPU.  Rank r owns experts [r*E/G, (r+1)*E/G); router, bias and
// the shared expert are replicated; tokens are data-parallel.  Per call, on every rank:
//   1. route the rank's own tokens (b200_moe_route)                                 -> sel, wts
//   2. k_ep_plan: count the (token, slot) pairs per destination rank, give every pair a position in
//      the send order (grouped by destination); k_ep_pack: token rows as bf16 + the local expert id
//      in a 16-byte trailer, one message row per pair
//   3. counts: one ncclAllGather of the G send counts; a one-thread kernel publishes the G x G matrix
//      to pinned host memory; the host waits for it (bounded) -- the one host wait of the call:
//      NCCL's point-to-point calls take their sizes from the host
//   4. dispatch: ONE group of ncclSend/ncclRecv, rows and ids in the same message, into a local
//      receive buffer (a rank's own pairs are copied device to device)
//   5. the received rows through this rank's experts (b200_moe_experts on the local shard: rows
//      grouped by expert, the wide tensor-core GEMM from 16 rows on)
//   6. combine: the reverse group returns one f32 output row per pair
//   7. y[t] = sum over slots in slot order of wts[t,k] * out[pair(t,k)] + shared(x[t])
// The shared expert does not depend on routing: it runs on a second stream, forked at entry and
// joined before step 7, so it overlaps the exchange.
// Remote data only ever arrives through NCCL into buffers this rank owns; no kernel here is given
// a peer's memory, and nothing uses multicast.  NCCL is bound at run time (dlopen), so the library
// loads without it as long as no expert-parallel context is created.
#include "b200_internal.h"
#include <nccl.h>
#include <dlfcn.h>
#include <chrono>
#include <cstdio>
#include <cstring>
#include <new>

namespace b200 {

struct NcclApi {
    ncclResult_t (*GetUniqueId)(ncclUniqueId*);
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int);
    ncclResult_t (*CommDestroy)(ncclComm_t);
    ncclResult_t (*CommAbort)(ncclComm_t);
    ncclResult_t (*GroupStart)();
    ncclResult_t (*GroupEnd)();
    ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t);
    ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t);
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t);
    const char* (*GetErrorString)(ncclResult_t);
    bool ok;
};

static const NcclApi* nccl_api() {
    static NcclApi api = [] {
        NcclApi a{};
        // dlopen by soname returns the copy the process already holds (e.g. the one a framework brought) if any
        void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!h) { fprintf(stderr, "b200_nvfp4: cannot load libnccl.so.2: %s\n", dlerror()); return a; }
        auto sym = [&](const char* n) { void* p = dlsym(h, n); if (!p) fprintf(stderr, "b200_nvfp4: %s missing in libnccl\n", n); return p; };
        a.GetUniqueId = (decltype(a.GetUniqueId))sym("ncclGetUniqueId");
        a.CommInitRank = (decltype(a.CommInitRank))sym("ncclCommInitRank");
        a.CommDestroy = (decltype(a.CommDestroy))sym("ncclCommDestroy");
        a.CommAbort = (decltype(a.CommAbort))sym("ncclCommAbort");
        a.GroupStart = (decltype(a.GroupStart))sym("ncclGroupStart");
        a.GroupEnd = (decltype(a.GroupEnd))sym("ncclGroupEnd");
        a.Send = (decltype(a.Send))sym("ncclSend");
        a.Recv = (decltype(a.Recv))sym("ncclRecv");
        a.AllGather = (decltype(a.AllGather))sym("ncclAllGather");
        a.GetErrorString = (decltype(a.GetErrorString))sym("ncclGetErrorString");
        a.ok = a.GetUniqueId && a.CommInitRank && a.CommDestroy && a.CommAbort && a.GroupStart && a.GroupEnd && a.Send &&
               a.Recv && a.AllGather && a.GetErrorString;
        return a;
    }();
    return api.ok ? &api : nullptr;
}

constexpr int EP_MAX_WORLD = 16;
constexpr int EP_TRAILER = 16;                     // bytes after the bf16 row: int32 local expert id, 12 spare

// One CTA.  dest(pair) = sel / experts_per_rank; send_pos[pair] = offset of its destination + a cursor.
// The order inside a destination's group is whatever the atomics give; every row is computed on its
// own and finds its way back through send_pos, so results do not depend on it.
__global__ void __launch_bounds__(1024)
k_ep_plan(const int32_t* __restrict__ sel, int pairs, int epr, int world, int* __restrict__ counts, int* __restrict__ send_pos) {
    __shared__ int cnt[EP_MAX_WORLD], off[EP_MAX_WORLD], cur[EP_MAX_WORLD];
    if (threadIdx.x < EP_MAX_WORLD) { cnt[threadIdx.x] = 0; cur[threadIdx.x] = 0; }
    __syncthreads();
    auto dest = [&](int p) { const int d = sel[p] / epr; return d < 0 ? 0 : (d >= world ? world - 1 : d); };
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) atomicAdd(&cnt[dest(p)], 1);
    __syncthreads();
    if (threadIdx.x == 0) { int o = 0; for (int g = 0; g < world; ++g) { off[g] = o; o += cnt[g]; counts[g] = cnt[g]; } }
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) { const int g = dest(p); send_pos[p] = off[g] + atomicAdd(&cur[g], 1); }
}

// One message row per pair: H bf16 values of the token, then the trailer.
__global__ void k_ep_pack(const float* __restrict__ x, const int32_t* __restrict__ sel, const int* __restrict__ send_pos,
                          unsigned char* __restrict__ send, int pairs, int topk, int H, int epr, size_t row_bytes) {
    const int per = H >> 3;                          // 8 values (16 bytes of bf16) per thread
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)pairs * (per + 1)) return;
    const int p = (int)(i / (per + 1)), c = (int)(i - (size_t)p * (per + 1));
    unsigned char* row = send + (size_t)send_pos[p] * row_bytes;
    if (c == per) {
        const int e = sel[p];
        *reinterpret_cast<int4*>(row + (size_t)H * 2) = make_int4(e - (e / epr) * epr, p, 0, 0);
        return;
    }
    const float4* src = reinterpret_cast<const float4*>(x + (size_t)(p / topk) * H) + 2 * c;
    const float4 a = src[0], b = src[1];
    __nv_bfloat162 o[4] = {__floats2bfloat162_rn(a.x, a.y), __floats2bfloat162_rn(a.z, a.w),
                           __floats2bfloat162_rn(b.x, b.y), __floats2bfloat162_rn(b.z, b.w)};
    reinterpret_cast<uint4*>(row)[c] = *reinterpret_cast<uint4*>(o);
}

// Received message rows -> f32 rows + expert ids for the local expert call.
__global__ void k_ep_unpack(const unsigned char* __restrict__ recv, float* __restrict__ rows, int32_t* __restrict__ eid,
                            int* __restrict__ touched, int R, int H, int n_local, size_t row_bytes) {
    const int per = H >> 3;
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)R * (per + 1)) return;
    const int r = (int)(i / (per + 1)), c = (int)(i - (size_t)r * (per + 1));
    const unsigned char* row = recv + (size_t)r * row_bytes;
    if (c == per) {
        const int e = reinterpret_cast<const int*>(row + (size_t)H * 2)[0];
        eid[r] = e < 0 ? 0 : (e >= n_local ? n_local - 1 : e);
        touched[eid[r]] = 1;                         // statistics only: which local experts this call reads
        return;
    }
    const uint4 v = reinterpret_cast<const uint4*>(row)[c];
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
    float4* dst = reinterpret_cast<float4*>(rows + (size_t)r * H) + 2 * c;
    dst[0] = make_float4(__uint_as_float(u[0] << 16), __uint_as_float(u[0] & 0xffff0000u), __uint_as_float(u[1] << 16), __uint_as_float(u[1] & 0xffff0000u));
    dst[1] = make_float4(__uint_as_float(u[2] << 16), __uint_as_float(u[2] & 0xffff0000u), __uint_as_float(u[3] << 16), __uint_as_float(u[3] & 0xffff0000u));
}

// The G x G count matrix to pinned host memory, then the sequence number the host waits for.
__global__ void k_ep_publish(const int* __restrict__ all_counts, int n, volatile int* host, int seq) {
    for (int i = 0; i < n; ++i) host[1 + i] = all_counts[i];
    __threadfence_system();
    host[0] = seq;
}

// y[t] = sum_k wts[t,k] * back[send_pos[t*topk + k]] (slot order) + shared[t]
__global__ void k_ep_combine(float* __restrict__ y, const float* __restrict__ back, const float* __restrict__ wts,
                             const int* __restrict__ send_pos, const float* __restrict__ shared, int T, int topk, int H) {
    const int per = H >> 2;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= T * per) return;
    const int t = i / per, h4 = i - t * per;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k = 0; k < topk; ++k) {
        const float w = wts[(size_t)t * topk + k];
        const float4 v = reinterpret_cast<const float4*>(back)[(size_t)send_pos[t * topk + k] * per + h4];
        acc.x = fmaf(w, v.x, acc.x); acc.y = fmaf(w, v.y, acc.y); acc.z = fmaf(w, v.z, acc.z); acc.w = fmaf(w, v.w, acc.w);
    }
    if (shared) {
        const float4 v = reinterpret_cast<const float4*>(shared)[(size_t)t * per + h4];
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    reinterpret_cast<float4*>(y)[i] = acc;
}

__global__ void k_ep_fill(float* ones, int32_t* zeros, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) { ones[i] = 1.f; zeros[i] = 0; }
}

}  // namespace b200

using namespace b200;

struct b200_ep {
    int rank, world, E, epr, topk, H, I, max_tokens, max_rows;
    b200_moe_layer router, local, shared;
    bool has_shared;
    ncclComm_t comm;
    const NcclApi* api;
    size_t row_bytes;
    // device
    float* logits; int* counts; int* all_counts; int* send_pos;
    unsigned char* send_buf; unsigned char* recv_buf;
    float* rows; int32_t* eid; float* ones; int32_t* zeros; int* touched;
    float* out_rows; float* back; float* shared_out;
    void* ws_local; void* ws_shared;
    // host
    volatile int* host_counts;                       // pinned: [0] sequence number, [1 ..] G x G counts
    cudaStream_t side; cudaEvent_t ev_fork, ev_join;
    cudaEvent_t ev_t[6];                             // timing: call start, dispatch start/end, combine start/end, call end
    int seq;
    b200_ep_stats stats;
};

static int ep_nccl(const b200_ep* ep, ncclResult_t r, const char* what) {
    if (r == ncclSuccess) return B200_OK;
    fprintf(stderr, "b200_nvfp4: %s: %s\n", what, ep->api->GetErrorString(r));
    return B200_ECOMM;
}

extern "C" int b200_ep_unique_id(void* id128) {
    if (!id128) return B200_EINVAL;
    const NcclApi* api = nccl_api();
    if (!api) return B200_ECOMM;
    static_assert(sizeof(ncclUniqueId) == 128, "NCCL unique id size");
    ncclUniqueId id;
    if (api->GetUniqueId(&id) != ncclSuccess) return B200_ECOMM;
    memcpy(id128, &id, 128);
    return B200_OK;
}

extern "C" int b200_ep_destroy(b200_ep* ep) {
    if (!ep) return B200_EINVAL;
    cudaDeviceSynchronize();
    if (ep->comm) ep->api->CommDestroy(ep->comm);
    void* dev[] = {ep->touched, ep->logits, ep->counts, ep->all_counts, ep->send_pos, ep->send_buf, ep->recv_buf, ep->rows, ep->eid, ep->ones,
                   ep->zeros, ep->out_rows, ep->back, ep->shared_out, ep->ws_local, ep->ws_shared};
    for (void* p : dev) if (p) cudaFree(p);
    if (ep->host_counts) cudaFreeHost((void*)ep->host_counts);
    if (ep->side) cudaStreamDestroy(ep->side);
    if (ep->ev_fork) cudaEventDestroy(ep->ev_fork);
    if (ep->ev_join) cudaEventDestroy(ep->ev_join);
    for (cudaEvent_t e : ep->ev_t) if (e) cudaEventDestroy(e);
    delete ep;
    return B200_OK;
}

extern "C" int b200_ep_create(b200_ep** out, const void* id128, int rank, int world, const b200_moe_layer* router,
                              const b200_moe_layer* local, const b200_moe_layer* shared, int max_tokens) {
    if (!out || !router || !local || world < 1 || world > EP_MAX_WORLD || rank < 0 || rank >= world || max_tokens < 1) return B200_EINVAL;
    if (world > 1 && !id128) return B200_EINVAL;
    if (router->n_expert % world || local->n_expert != router->n_expert / world || local->topk != 1) return B200_EINVAL;
    if (local->hidden != router->hidden || (router->hidden & 7)) return B200_ESHAPE;
    if (shared && (shared->n_expert != 1 || shared->topk != 1 || shared->hidden != router->hidden)) return B200_EINVAL;
    b200_ep* ep = new (std::nothrow) b200_ep();
    if (!ep) return B200_ELIMIT;
    memset(ep, 0, sizeof(*ep));
    ep->rank = rank; ep->world = world; ep->E = router->n_expert; ep->epr = ep->E / world; ep->topk = router->topk;
    ep->H = router->hidden; ep->I = local->inter; ep->max_tokens = max_tokens;
    ep->max_rows = world * max_tokens * ep->topk;       // every pair of every rank could land here
    ep->router = *router; ep->local = *local; ep->has_shared = shared != nullptr;
    if (shared) ep->shared = *shared;
    ep->row_bytes = (size_t)ep->H * 2 + EP_TRAILER;
    const size_t pairs = (size_t)max_tokens * ep->topk, H = ep->H, R = ep->max_rows;
    bool ok = true;
    auto alloc = [&](void* p, size_t bytes) { ok = ok && cudaMalloc((void**)p, bytes ? bytes : 256) == cudaSuccess; };
    alloc(&ep->logits, (size_t)max_tokens * ep->E * 4);
    alloc(&ep->counts, EP_MAX_WORLD * 4);
    alloc(&ep->all_counts, EP_MAX_WORLD * EP_MAX_WORLD * 4);
    alloc(&ep->send_pos, pairs * 4);
    alloc(&ep->send_buf, pairs * ep->row_bytes);
    alloc(&ep->recv_buf, R * ep->row_bytes);
    alloc(&ep->rows, R * H * 4);
    alloc(&ep->eid, R * 4);
    alloc(&ep->touched, (size_t)ep->epr * 4);
    const size_t n1 = std::max(R, (size_t)max_tokens);
    alloc(&ep->ones, n1 * 4);
    alloc(&ep->zeros, n1 * 4);
    alloc(&ep->out_rows, R * H * 4);
    alloc(&ep->back, pairs * H * 4);
    alloc(&ep->ws_local, b200_moe_workspace_bytes(&ep->local, (int)R));
    if (shared) {
        alloc(&ep->shared_out, (size_t)max_tokens * H * 4);
        alloc(&ep->ws_shared, b200_moe_workspace_bytes(&ep->shared, max_tokens));
    }
    ok = ok && cudaHostAlloc((void**)&ep->host_counts, (1 + EP_MAX_WORLD * EP_MAX_WORLD) * 4, cudaHostAllocMapped) == cudaSuccess;
    ok = ok && cudaStreamCreateWithFlags(&ep->side, cudaStreamNonBlocking) == cudaSuccess;
    ok = ok && cudaEventCreateWithFlags(&ep->ev_fork, cudaEventDisableTiming) == cudaSuccess;
    ok = ok && cudaEventCreateWithFlags(&ep->ev_join, cudaEventDisableTiming) == cudaSuccess;
    for (cudaEvent_t& e : ep->ev_t) ok = ok && cudaEventCreate(&e) == cudaSuccess;
    if (!ok) { launch_failed("b200_ep_create: allocation"); b200_ep_destroy(ep); return B200_ELIMIT; }
    ep->host_counts[0] = 0;
    k_ep_fill<<<(unsigned)((n1 + 255) / 256), 256>>>(ep->ones, ep->zeros, (int)n1);
    if (cudaDeviceSynchronize() != cudaSuccess) { launch_failed("b200_ep_create: fill"); b200_ep_destroy(ep); return B200_ELAUNCH; }
    if (world > 1) {
        ep->api = nccl_api();
        if (!ep->api) { b200_ep_destroy(ep); return B200_ECOMM; }
        ncclUniqueId id;
        memcpy(&id, id128, 128);
        if (int rc = ep_nccl(ep, ep->api->CommInitRank(&ep->comm, world, id, rank), "ncclCommInitRank")) { ep->comm = nullptr; b200_ep_destroy(ep); return rc; }
    }
    *out = ep;
    return B200_OK;
}

// Synchronises the device (it reads back which local experts the last call touched): call it outside timed regions.
extern "C" int b200_ep_last_stats(const b200_ep* ep, b200_ep_stats* out) {
    if (!ep || !out) return B200_EINVAL;
    *out = ep->stats;
    int flags[512] = {0};
    const int n = std::min(ep->epr, 512);
    if (cudaDeviceSynchronize() != cudaSuccess || cudaMemcpy(flags, ep->touched, (size_t)n * 4, cudaMemcpyDeviceToHost) != cudaSuccess)
        return launch_failed("b200_ep_last_stats");
    out->local_experts_touched = 0;
    for (int i = 0; i < n; ++i) out->local_experts_touched += flags[i] != 0;
    float ms = 0.f;
    out->plan_us = cudaEventElapsedTime(&ms, ep->ev_t[0], ep->ev_t[1]) == cudaSuccess ? ms * 1e3f : -1.f;
    out->dispatch_us = cudaEventElapsedTime(&ms, ep->ev_t[1], ep->ev_t[2]) == cudaSuccess ? ms * 1e3f : -1.f;
    out->experts_us = cudaEventElapsedTime(&ms, ep->ev_t[2], ep->ev_t[3]) == cudaSuccess ? ms * 1e3f : -1.f;
    out->combine_us = cudaEventElapsedTime(&ms, ep->ev_t[3], ep->ev_t[4]) == cudaSuccess ? ms * 1e3f : -1.f;
    out->total_us = cudaEventElapsedTime(&ms, ep->ev_t[0], ep->ev_t[5]) == cudaSuccess ? ms * 1e3f : -1.f;
    return B200_OK;
}

extern "C" int b200_ep_forward(b200_ep* ep, const float* x, float* y, int32_t* sel, float* wts, int T, b200_stream stream) {
    if (!ep || !x || !y || !sel || !wts || T < 1) return B200_EINVAL;
    if (T > ep->max_tokens) return B200_ELIMIT;
    if (((uintptr_t)x & 15) || ((uintptr_t)y & 15)) return B200_EALIGN;
    const int G = ep->world, topk = ep->topk, H = ep->H, pairs = T * topk;
    cudaStream_t s = stream;
    // exact experts or the wide GEMM: decided by the tokens of ALL ranks, so that G ranks on T tokens compute
    // every row the way one GPU on the same T tokens does
    const int wide = (long)T * G >= PREFILL_MIN_ROWS && prefill_fp4_option();
    cudaEventRecord(ep->ev_t[0], s);
    // the shared expert only needs x: fork it onto the side stream now
    if (ep->has_shared) {
        if (cudaEventRecord(ep->ev_fork, s) != cudaSuccess || cudaStreamWaitEvent(ep->side, ep->ev_fork, 0) != cudaSuccess) return launch_failed("b200_ep_forward: fork");
        if (int rc = moe_experts_mode(x, &ep->shared, ep->shared_out, ep->zeros, ep->ones, ep->ws_shared, T, ep->side, wide)) return rc;
        if (cudaEventRecord(ep->ev_join, ep->side) != cudaSuccess) return launch_failed("b200_ep_forward: join record");
    }
    if (int rc = b200_moe_route(x, &ep->router, sel, wts, ep->logits, T, s)) return rc;
    k_ep_plan<<<1, 1024, 0, s>>>(sel, pairs, ep->epr, G, ep->counts, ep->send_pos);
    if (int rc = check_launch("k_ep_plan")) return rc;
    {
        const size_t n = (size_t)pairs * ((H >> 3) + 1);
        k_ep_pack<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(x, sel, ep->send_pos, ep->send_buf, pairs, topk, H, ep->epr, ep->row_bytes);
        if (int rc = check_launch("k_ep_pack")) return rc;
    }
    int scnt[EP_MAX_WORLD] = {0}, rcnt[EP_MAX_WORLD] = {0}, soff[EP_MAX_WORLD + 1] = {0}, roff[EP_MAX_WORLD + 1] = {0};
    if (G == 1) {
        scnt[0] = rcnt[0] = pairs;
    } else {
        if (int rc = ep_nccl(ep, ep->api->AllGather(ep->counts, ep->all_counts, (size_t)G, ncclInt32, ep->comm, s), "ncclAllGather(counts)")) return rc;
        const int seq = ++ep->seq;
        k_ep_publish<<<1, 1, 0, s>>>(ep->all_counts, G * G, ep->host_counts, seq);
        if (int rc = check_launch("k_ep_publish")) return rc;
        // The one host wait of the call: the sizes of the exchange.  Bounded: a peer that never joins
        // the collective leaves the sequence number unchanged, and the call gives up.
        const auto t0 = std::chrono::steady_clock::now();
        while (ep->host_counts[0] != seq) {
            if (std::chrono::steady_clock::now() - t0 > std::chrono::seconds(20)) {
                fprintf(stderr, "b200_nvfp4: b200_ep_forward: rank %d waited 20 s for the exchange sizes; aborting the communicator\n", ep->rank);
                ep->api->CommAbort(ep->comm); ep->comm = nullptr;
                return B200_ETIMEOUT;
            }
        }
        for (int g = 0; g < G; ++g) { scnt[g] = ep->host_counts[1 + ep->rank * G + g]; rcnt[g] = ep->host_counts[1 + g * G + ep->rank]; }
    }
    for (int g = 0; g < G; ++g) { soff[g + 1] = soff[g] + scnt[g]; roff[g + 1] = roff[g] + rcnt[g]; }
    const int R = roff[G];
    if (soff[G] != pairs || R > ep->max_rows) return B200_ECOMM;
    const size_t rb = ep->row_bytes;
    // dispatch
    cudaEventRecord(ep->ev_t[1], s);
    if (scnt[ep->rank] &&
        cudaMemcpyAsync(ep->recv_buf + (size_t)roff[ep->rank] * rb, ep->send_buf + (size_t)soff[ep->rank] * rb,
                        (size_t)scnt[ep->rank] * rb, cudaMemcpyDeviceToDevice, s) != cudaSuccess) return launch_failed("b200_ep_forward: local dispatch copy");
    if (G > 1) {
        if (int rc = ep_nccl(ep, ep->api->GroupStart(), "ncclGroupStart")) return rc;
        for (int g = 0; g < G; ++g) {
            if (g == ep->rank) continue;
            ncclResult_t r1 = ncclSuccess, r2 = ncclSuccess;
            if (scnt[g]) r1 = ep->api->Send(ep->send_buf + (size_t)soff[g] * rb, (size_t)scnt[g] * rb, ncclUint8, g, ep->comm, s);
            if (rcnt[g]) r2 = ep->api->Recv(ep->recv_buf + (size_t)roff[g] * rb, (size_t)rcnt[g] * rb, ncclUint8, g, ep->comm, s);
            if (r1 != ncclSuccess || r2 != ncclSuccess) { ep->api->GroupEnd(); return ep_nccl(ep, r1 != ncclSuccess ? r1 : r2, "ncclSend/ncclRecv(dispatch)"); }
        }
        if (int rc = ep_nccl(ep, ep->api->GroupEnd(), "ncclGroupEnd(dispatch)")) return rc;
    }
    cudaEventRecord(ep->ev_t[2], s);
    // this rank's experts on what arrived
    if (cudaMemsetAsync(ep->touched, 0, (size_t)ep->epr * 4, s) != cudaSuccess) return launch_failed("b200_ep_forward: memset");
    if (R) {
        const size_t n = (size_t)R * ((H >> 3) + 1);
        k_ep_unpack<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(ep->recv_buf, ep->rows, ep->eid, ep->touched, R, H, ep->epr, rb);
        if (int rc = check_launch("k_ep_unpack")) return rc;
        if (int rc = moe_experts_mode(ep->rows, &ep->local, ep->out_rows, ep->eid, ep->ones, ep->ws_local, R, s, wide)) return rc;
    }
    // combine
    cudaEventRecord(ep->ev_t[3], s);
    const size_t ob = (size_t)H * 4;
    if (scnt[ep->rank] &&
        cudaMemcpyAsync(reinterpret_cast<unsigned char*>(ep->back) + (size_t)soff[ep->rank] * ob,
                        reinterpret_cast<unsigned char*>(ep->out_rows) + (size_t)roff[ep->rank] * ob,
                        (size_t)scnt[ep->rank] * ob, cudaMemcpyDeviceToDevice, s) != cudaSuccess) return launch_failed("b200_ep_forward: local combine copy");
    if (G > 1) {
        if (int rc = ep_nccl(ep, ep->api->GroupStart(), "ncclGroupStart")) return rc;
        for (int g = 0; g < G; ++g) {
            if (g == ep->rank) continue;
            ncclResult_t r1 = ncclSuccess, r2 = ncclSuccess;
            if (rcnt[g]) r1 = ep->api->Send(ep->out_rows + (size_t)roff[g] * H, (size_t)rcnt[g] * H, ncclFloat32, g, ep->comm, s);
            if (scnt[g]) r2 = ep->api->Recv(ep->back + (size_t)soff[g] * H, (size_t)scnt[g] * H, ncclFloat32, g, ep->comm, s);
            if (r1 != ncclSuccess || r2 != ncclSuccess) { ep->api->GroupEnd(); return ep_nccl(ep, r1 != ncclSuccess ? r1 : r2, "ncclSend/ncclRecv(combine)"); }
        }
        if (int rc = ep_nccl(ep, ep->api->GroupEnd(), "ncclGroupEnd(combine)")) return rc;
    }
    cudaEventRecord(ep->ev_t[4], s);
    if (ep->has_shared && cudaStreamWaitEvent(s, ep->ev_join, 0) != cudaSuccess) return launch_failed("b200_ep_forward: join");
    const int n4 = T * (H >> 2);
    k_ep_combine<<<(n4 + 255) / 256, 256, 0, s>>>(y, ep->back, wts, ep->send_pos, ep->has_shared ? ep->shared_out : nullptr, T, topk, H);
    if (int rc = check_launch("k_ep_combine")) return rc;
    cudaEventRecord(ep->ev_t[5], s);
    ep->stats.tokens = T; ep->stats.recv_rows = R; ep->stats.sent_remote_rows = pairs - scnt[ep->rank];
    ep->stats.recv_remote_rows = R - rcnt[ep->rank];
    ep->stats.dispatch_bytes_out = (unsigned long long)ep->stats.sent_remote_rows * rb;
    ep->stats.combine_bytes_in = (unsigned long long)ep->stats.sent_remote_rows * ob;
    return B200_OK;
}
