// common.cu -- error reporting and cached device attributes.
#include "b200_internal.h"
#include <cstdio>

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
        default: return "unknown error";
    }
}

extern "C" int b200_nvfp4_version(void) { return 100; }
