// common.cu -- error reporting and cached device attributes.
#include "b200_internal.h"
#include "tma_pipe.cuh"
#include <cstdio>
#include <cstdlib>

namespace b200 {

int sm_count() {
    static int cache[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cache[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cache[dev] = n;
    }
    return cache[dev];
}

// Written by a kernel whose bounded wait ran out (see tma_pipe.cuh); read by
// b200_nvfp4_device_status.  One word per device that loads the library.
__device__ unsigned int g_device_status[2] = {0, 0};   // [0] first failure, [1] OR of (1 << site) over all failures

unsigned int* device_status_ptr() {
    static unsigned int* cache[64] = {nullptr};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (!cache[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_device_status) != cudaSuccess) return nullptr;
        cache[dev] = static_cast<unsigned int*>(p);
    }
    return cache[dev];
}

static int g_stable_weights = -1;
int stable_weights_option() {
    if (g_stable_weights < 0) {
        const char* e = getenv("B200_STABLE_WEIGHTS");
        g_stable_weights = (e && *e == '1') ? 1 : 0;
    }
    return g_stable_weights;
}
void set_stable_weights(int v) { g_stable_weights = v ? 1 : 0; }

// 1 (default): calls that carry scratch and 16 or more activation rows take the wide tensor-core GEMM,
// which quantises the activations to NVFP4; 0: every call keeps fp32-activation accuracy.
static int g_prefill_fp4 = -1;
int prefill_fp4_option() {
    if (g_prefill_fp4 < 0) {
        const char* e = getenv("B200_PREFILL_FP4");
        g_prefill_fp4 = (e && *e == '0') ? 0 : 1;
    }
    return g_prefill_fp4;
}

// ---- byte accounting ---------------------------------------------------------------------------------
static b200_byte_credit_fn g_credit_fn = nullptr;
static void* g_credit_user = nullptr;
static double g_grouped_matrix_bytes = 0.0;         // bytes of one expert matrix of the last grouped MoE call
__device__ unsigned long long g_credit_jobs[2] = {0ull, 0ull};

bool credit_on() { return g_credit_fn != nullptr; }
void credit(int kind, double bytes) { if (g_credit_fn) g_credit_fn(kind, bytes, g_credit_user); }
void credit_grouped_geometry(int hidden, int inter) { g_grouped_matrix_bytes = (double)hidden * inter * 0.5625; }
unsigned long long* credit_counters() {
    static unsigned long long* cache[64] = {nullptr};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (!cache[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_credit_jobs) != cudaSuccess) return nullptr;
        cache[dev] = static_cast<unsigned long long*>(p);
    }
    return cache[dev];
}

int launch_failed(const char* what) {
    const cudaError_t e = cudaGetLastError();
    fprintf(stderr, "b200_nvfp4: %s failed: %s\n", what, cudaGetErrorString(e));
    return B200_ELAUNCH;
}

int check_launch(const char* what) {
    const cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) return B200_OK;
    fprintf(stderr, "b200_nvfp4: launch of %s failed: %s\n", what, cudaGetErrorString(e));
    return B200_ELAUNCH;
}

}  // namespace b200

extern "C" const char* b200_nvfp4_strerror(int code) {
    switch (code) {
        case B200_OK: return "ok";
        case B200_EINVAL: return "invalid argument";
        case B200_ESHAPE: return "unsupported shape (K must be a multiple of 16)";
        case B200_EALIGN: return "pointer not 4-byte aligned";
        case B200_ELAUNCH: return "CUDA launch failed";
        case B200_ELIMIT: return "size beyond the documented maximum";
        case B200_ENOTIMPL: return "not implemented";
        case B200_ETIMEOUT: return "a bounded wait ran out";
        case B200_ECOMM: return "NCCL missing or failed";
        default: return "unknown error";
    }
}

extern "C" int b200_nvfp4_version(void) { return 200; }

extern "C" int b200_nvfp4_set_byte_credit(b200_byte_credit_fn fn, void* user) {
    b200::g_credit_fn = fn; b200::g_credit_user = user;
    return B200_OK;
}

extern "C" int b200_nvfp4_flush_byte_credit(int credit) {
    unsigned long long* p = b200::credit_counters();
    if (!p) return B200_ELAUNCH;
    unsigned long long jobs[2] = {0ull, 0ull};
    if (cudaMemcpy(jobs, p, sizeof jobs, cudaMemcpyDeviceToHost) != cudaSuccess || cudaMemset(p, 0, sizeof jobs) != cudaSuccess)
        return b200::launch_failed("flush_byte_credit");
    if (credit) {
        b200::credit(B200_CREDIT_MOE_ACT, (double)jobs[0] * b200::g_grouped_matrix_bytes);
        b200::credit(B200_CREDIT_MOE_DOWN, (double)jobs[1] * b200::g_grouped_matrix_bytes);
    }
    return B200_OK;
}

extern "C" int b200_nvfp4_set_option(int option, int value) {
    if (option == B200_OPT_STABLE_WEIGHTS) { b200::set_stable_weights(value); return B200_OK; }
    if (option == B200_OPT_PREFILL_FP4) { b200::g_prefill_fp4 = value ? 1 : 0; return B200_OK; }
    return B200_EINVAL;
}

// One thread waits, with the library's bounded wait, on a barrier that nobody ever arrives at: the wait gives
// up after its limit (about a second), records site 15 in the status word, and the kernel returns.
__global__ void k_selftest_wait(unsigned int* status) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) { b200::mbar_init(b200::smem_u32(&bar), 1); b200::mbar_fence_init(); }
    __syncthreads();
    if (threadIdx.x == 0) b200::mbar_wait(b200::smem_u32(&bar), 0, status, 15);
}

extern "C" int b200_nvfp4_selftest_bounded_wait(b200_stream stream) {
    unsigned int* p = b200::device_status_ptr();
    if (!p) return B200_ELAUNCH;
    k_selftest_wait<<<1, 32, 0, stream>>>(p);
    return b200::check_launch("k_selftest_wait");
}

extern "C" int b200_nvfp4_device_status(unsigned int* out, int clear) {
    if (!out) return B200_EINVAL;
    unsigned int* p = b200::device_status_ptr();
    if (!p) return B200_ELAUNCH;
    unsigned int both[2] = {0, 0};
    if (cudaMemcpy(both, p, sizeof(both), cudaMemcpyDeviceToHost) != cudaSuccess) return b200::launch_failed("device_status read");
    *out = both[0];
    if (both[0]) fprintf(stderr, "b200_nvfp4: device status: first failure %08x, sites mask %08x\n", both[0], both[1]);
    if (clear && both[0] && cudaMemset(p, 0, sizeof(both)) != cudaSuccess) return b200::launch_failed("device_status clear");
    return B200_OK;
}
