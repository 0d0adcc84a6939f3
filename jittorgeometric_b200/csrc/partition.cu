// Compact halo of the 1-D row partition (sm_100a).
//
// With skewed degrees most remote feature rows are never referenced by a given shard (on the
// scale-21 R-MAT workload a rank needs 59 / 50 / 41 % of the remote rows at 2 / 4 / 8 shards), so
// exchanging whole shards moves rows nobody reads.  These kernels build, once per graph, the map
// from global source ids to positions in a packed halo buffer (ordered by global id, hence grouped
// by owner), the per-owner lists of needed rows, and, per aggregation, gather the rows another rank
// asked for into a send buffer.  They replace, on device, what the reference's offline partitioner
// computes with Python loops (partition/distchunk_manager.py:100-157) and the whole-block broadcast
// of ops/distspmm.py:31-39.
#include "common.cuh"
#include "scan.cuh"

namespace jg {

// Rows inside [lo, hi) are the shard's own and are not marked.
__global__ void mark_rows_kernel(const int32_t* __restrict__ idx, int64_t nnz, int32_t lo, int32_t hi,
                                 int* __restrict__ flag) {
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < nnz; e += (int64_t)gridDim.x * blockDim.x) {
        const int32_t s = idx[e];
        if (s < lo || s >= hi) flag[s] = 1;   // benign race: every writer stores the same value
    }
}

// own rows -> idx - lo, remote rows -> base + slot in the packed halo buffer
__global__ void remap_kernel(const int32_t* __restrict__ idx, const int* __restrict__ pos, int64_t nnz, int32_t lo,
                             int32_t hi, int32_t base, int32_t* __restrict__ out) {
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < nnz; e += (int64_t)gridDim.x * blockDim.x) {
        const int32_t s = idx[e];
        out[e] = (s >= lo && s < hi) ? s - lo : base + pos[s];
    }
}

// needed[pos[g]] = g for every marked global id g (ascending, because pos is an exclusive scan)
__global__ void list_marked_kernel(const int* __restrict__ flag, const int* __restrict__ pos, int64_t n,
                                   int32_t* __restrict__ needed) {
    for (int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; g < n; g += (int64_t)gridDim.x * blockDim.x)
        if (flag[g]) needed[pos[g]] = (int32_t)g;
}

// out[i,:] = x[rows[i] - rebase,:]: one warp per row, 128-bit copies when the width allows.
__global__ void __launch_bounds__(256) gather_rows_kernel(float* __restrict__ out, const float* __restrict__ x,
                                                          const int32_t* __restrict__ rows, int64_t n_rows, int64_t f,
                                                          int32_t rebase, int vec) {
    const int lane = lane_id();
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t i = warp; i < n_rows; i += n_warps) {
        const float* src = x + (size_t)(rows[i] - rebase) * f;
        float* dst = out + (size_t)i * f;
        if (vec) {
            for (int64_t c = lane; c < f / 4; c += 32)
                __stcs(reinterpret_cast<float4*>(dst) + c, __ldg(reinterpret_cast<const float4*>(src) + c));
        } else {
            for (int64_t c = lane; c < f; c += 32) dst[c] = __ldg(src + c);
        }
    }
}

struct HaloMapWs {
    int* flag;
    int* sums;
    size_t bytes;
};
static HaloMapWs carve_halo_map(void* ws, int64_t n) {
    Carver c(ws);
    HaloMapWs v;
    v.flag = c.take<int>(n + 1);
    v.sums = c.take<int>(scan_temp_ints(n + 1));
    v.bytes = c.total();
    return v;
}

}  // namespace jg

using namespace jg;

extern "C" {

size_t jg_halo_map_workspace_bytes(int64_t n_global) {
    if (n_global < 0) return 0;
    return carve_halo_map(nullptr, n_global).bytes;
}

int jg_halo_map_build(const int32_t* halo_idx, int64_t nnz, int64_t n_global, int32_t lo, int32_t hi, int32_t base,
                      int32_t* pos, int32_t* needed, int32_t* remapped_idx, void* workspace, size_t workspace_bytes,
                      jg_stream_t stream) {
    JG_CHECK_ARG(nnz >= 0 && n_global >= 0 && lo <= hi, JG_EINVAL, "halo_map_build: bad size or range");
    JG_CHECK_ARG(pos && (nnz == 0 || (halo_idx && needed && remapped_idx)), JG_EINVAL, "halo_map_build: null pointer");
    JG_CHECK_ARG(n_global < INT32_MAX && nnz <= INT32_MAX, JG_ESHAPE, "halo_map_build: sizes beyond int32");
    JG_CHECK_ARG(workspace && workspace_bytes >= jg_halo_map_workspace_bytes(n_global), JG_EWORKSPACE,
                 "halo_map_build: workspace too small");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    HaloMapWs ws = carve_halo_map(workspace, n_global);
    const int grid = sm_count() * 8;
    JG_CUDA(cudaMemsetAsync(ws.flag, 0, sizeof(int) * (size_t)(n_global + 1), st));
    if (nnz > 0) {
        mark_rows_kernel<<<grid, 256, 0, st>>>(halo_idx, nnz, lo, hi, ws.flag);
        JG_LAUNCH_CHECK();
    }
    int rc = exclusive_scan(ws.flag, reinterpret_cast<int*>(pos), n_global + 1, ws.sums, st);
    if (rc != JG_OK) return rc;
    if (nnz > 0) {
        list_marked_kernel<<<grid, 256, 0, st>>>(ws.flag, reinterpret_cast<const int*>(pos), n_global, needed);
        JG_LAUNCH_CHECK();
        remap_kernel<<<grid, 256, 0, st>>>(halo_idx, reinterpret_cast<const int*>(pos), nnz, lo, hi, base, remapped_idx);
        JG_LAUNCH_CHECK();
    }
    return JG_OK;
}

int jg_gather_rows_f32(float* out, const float* x, const int32_t* rows, int64_t n_rows, int64_t f, int32_t rebase,
                       jg_stream_t stream) {
    JG_CHECK_ARG(n_rows >= 0 && f >= 0, JG_EINVAL, "gather_rows: negative size");
    if (n_rows == 0 || f == 0) return JG_OK;
    JG_CHECK_ARG(out && x && rows, JG_EINVAL, "gather_rows: null pointer");
    const int vec = (f % 4 == 0) && ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(x)) % 16 == 0);
    int64_t blocks = (n_rows * 32 + 255) / 256;
    const int64_t cap = (int64_t)sm_count() * 8;
    if (blocks > cap) blocks = cap;
    gather_rows_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(out, x, rows, n_rows, f, rebase, vec);
    JG_LAUNCH_CHECK();
    return JG_OK;
}

}  // extern "C"
