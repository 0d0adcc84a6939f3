// Shared helpers for the sm_100a kernels and their C-ABI entry points.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>
#include <cstddef>
#include <cstdio>

#include "../../include/jgb200.h"

namespace jg {

constexpr int kWarp = 32;
constexpr unsigned kFull = 0xffffffffu;

// Thread-local detail text behind jg_last_error().
void set_error(const char* fmt, ...);

// Number of SMs of the current device (cached per device).
int sm_count();

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// Carves 256-byte aligned pieces out of a caller-owned workspace.
struct Carver {
    char* base;
    size_t used = 0;
    explicit Carver(void* p) : base(static_cast<char*>(p)) {}
    template <class T>
    T* take(size_t count) {
        used = align_up(used, 256);
        T* r = reinterpret_cast<T*>(base ? base + used : nullptr);
        used += count * sizeof(T);
        return r;
    }
    size_t total() const { return align_up(used, 256); }
};

#define JG_CHECK_ARG(cond, code, ...)          \
    do {                                       \
        if (!(cond)) {                         \
            ::jg::set_error(__VA_ARGS__);      \
            return (code);                     \
        }                                      \
    } while (0)

#define JG_CUDA(expr)                                                                  \
    do {                                                                               \
        cudaError_t _e = (expr);                                                       \
        if (_e != cudaSuccess) {                                                       \
            ::jg::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e),    \
                            __FILE__, __LINE__);                                       \
            return JG_ECUDA;                                                           \
        }                                                                              \
    } while (0)

// Launch check that does not synchronise: reports configuration errors only.
#define JG_LAUNCH_CHECK() JG_CUDA(cudaGetLastError())

__device__ __forceinline__ int lane_id() { return threadIdx.x & 31; }

// Streaming (read-once) loads: keep L2 for the gathered feature rows.
__device__ __forceinline__ int ld_stream(const int* p) { return __ldcs(p); }
__device__ __forceinline__ float ld_stream(const float* p) { return __ldcs(p); }

}  // namespace jg
