// Status codes, error text and device bookkeeping shared by every entry point.
#include "common.cuh"

#include <cstdarg>
#include <cstring>

namespace jg {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

}  // namespace jg

extern "C" {

int jg_version(void) { return 100; }

const char* jg_status_string(int status) {
    switch (status) {
        case JG_OK: return "ok";
        case JG_EINVAL: return "invalid argument";
        case JG_ESHAPE: return "shape mismatch or size beyond int32 indexing";
        case JG_EWORKSPACE: return "workspace missing or too small";
        case JG_ECUDA: return "CUDA runtime error";
        case JG_ETIMEOUT: return "bounded device-side wait ran out";
        case JG_EUNSUPPORTED: return "not supported by this build";
        default: return "unknown status";
    }
}

const char* jg_last_error(void) { return jg::g_err; }

int jg_set_device(int device) {
    JG_CHECK_ARG(device >= 0, JG_EINVAL, "device %d < 0", device);
    JG_CUDA(cudaSetDevice(device));
    return JG_OK;
}

}  // extern "C"
