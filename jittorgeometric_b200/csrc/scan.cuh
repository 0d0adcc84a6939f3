// Device-wide exclusive scan of int32 (three small kernels), shared by the conversion and the
// partition code.  Everything here has internal linkage: each translation unit gets its own copy.
#pragma once
#include "common.cuh"

namespace jg {

// ------------------------------------------------------------------------------- device scan
constexpr int kScanThreads = 512;
constexpr int kScanItems = 8;
constexpr int kScanTile = kScanThreads * kScanItems;

static __device__ __forceinline__ int block_exclusive_scan(int v, int* total, int* s_warp /*[32]*/) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    int inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        int t = __shfl_up_sync(kFull, inc, o);
        if (lane >= o) inc += t;
    }
    if (lane == 31) s_warp[wid] = inc;
    __syncthreads();
    if (wid == 0) {
        const int nw = blockDim.x >> 5;
        int w = lane < nw ? s_warp[lane] : 0;
        int winc = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            int t = __shfl_up_sync(kFull, winc, o);
            if (lane >= o) winc += t;
        }
        s_warp[lane] = winc - w;  // exclusive prefix of warp sums
        if (lane == 31) *total = winc;
    }
    __syncthreads();
    const int r = s_warp[wid] + inc - v;
    __syncthreads();
    return r;
}

static __global__ void __launch_bounds__(kScanThreads) scan_reduce_kernel(const int* __restrict__ in, int64_t n, int* __restrict__ sums) {
    __shared__ int s_warp[32];
    __shared__ int s_total;
    const int64_t base = (int64_t)blockIdx.x * kScanTile;
    int v = 0;
#pragma unroll
    for (int i = 0; i < kScanItems; i++) {
        const int64_t p = base + (int64_t)i * kScanThreads + threadIdx.x;
        if (p < n) v += in[p];
    }
    block_exclusive_scan(v, &s_total, s_warp);
    if (threadIdx.x == 0) sums[blockIdx.x] = s_total;
}

// One block: exclusive scan of `m` block sums in place.
static __global__ void __launch_bounds__(1024) scan_sums_kernel(int* sums, int64_t m) {
    __shared__ int s_warp[32];
    __shared__ int s_total;
    int carry = 0;
    for (int64_t base = 0; base < m; base += 1024) {
        const int64_t p = base + threadIdx.x;
        const int v = p < m ? sums[p] : 0;
        const int ex = block_exclusive_scan(v, &s_total, s_warp);
        if (p < m) sums[p] = carry + ex;
        carry += s_total;
        __syncthreads();
    }
}

static __global__ void __launch_bounds__(kScanThreads) scan_apply_kernel(const int* __restrict__ in, int* __restrict__ out, int64_t n,
                                                                  const int* __restrict__ sums) {
    __shared__ int s_warp[32];
    __shared__ int s_total;
    const int64_t base = (int64_t)blockIdx.x * kScanTile + (int64_t)threadIdx.x * kScanItems;
    int v[kScanItems];
    int local = 0;
#pragma unroll
    for (int i = 0; i < kScanItems; i++) {
        v[i] = (base + i < n) ? in[base + i] : 0;
        local += v[i];
    }
    int ex = block_exclusive_scan(local, &s_total, s_warp) + sums[blockIdx.x];
#pragma unroll
    for (int i = 0; i < kScanItems; i++) {
        if (base + i < n) out[base + i] = ex;
        ex += v[i];
    }
}

static size_t scan_temp_ints(int64_t n) { return (size_t)((n + kScanTile - 1) / kScanTile) + 1; }

// Exclusive scan of n int32 (in place allowed).  `sums` holds scan_temp_ints(n) ints.
static int exclusive_scan(const int* in, int* out, int64_t n, int* sums, cudaStream_t st) {
    if (n <= 0) return JG_OK;
    const int64_t blocks = (n + kScanTile - 1) / kScanTile;
    scan_reduce_kernel<<<(unsigned)blocks, kScanThreads, 0, st>>>(in, n, sums);
    JG_LAUNCH_CHECK();
    scan_sums_kernel<<<1, 1024, 0, st>>>(sums, blocks);
    JG_LAUNCH_CHECK();
    scan_apply_kernel<<<(unsigned)blocks, kScanThreads, 0, st>>>(in, out, n, sums);
    JG_LAUNCH_CHECK();
    return JG_OK;
}


}  // namespace jg
