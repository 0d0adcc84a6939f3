// Neighbour sampling for mini-batch training (sm_100a): the device side of the reference's
// layer-wise sampler (examples/minibatch_example.py:232-362) and of its four operators
//   gpuinitco         ops/cpp/gpuinitco_op.cc:37-52          per-destination sample counts
//   sampleprocessing  ops/cpp/sampleprocessing_op.cc:38-176  draw up to `fanout` in-edges per destination
//   csctocsr          ops/cpp/csctocsr_op.cc:26-172          sampled CSC -> CSR over explicit id lists
//   getweight         ops/cpp/getweight_op.cc:37-187         1 / (sqrt(out-degree) * sqrt(in-degree))
// The reference's kernels use one thread per destination (sampling), an O(sources * edges) count
// loop and a one-thread prefix sum (csctocsr); here sampling is one warp per destination with a
// counter-based generator (the draw depends only on seed and destination id, not on scheduling),
// csctocsr is the library's stable radix sort, and degrees are integer atomics (exact).
#include "common.cuh"
#include "scan.cuh"

namespace jg {

// ---- counter-based generator: 64-bit mix of (seed, destination id, draw number)
__device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
// uniform integer in [0, bound) from one 64-bit draw (multiply-high; the bias is below 2^-32 for
// bounds that fit in int32)
__device__ __forceinline__ int draw_below(unsigned long long seed, int vertex, int k, int bound) {
    const unsigned long long r = mix64(mix64(seed ^ ((unsigned long long)(unsigned)vertex << 32)) + (unsigned long long)k);
    return (int)__umul64hi(r, (unsigned long long)bound);
}

__global__ void sample_counts_kernel(const int32_t* __restrict__ dst, int64_t n_dst, const int32_t* __restrict__ g_off,
                                     int32_t fanout, int32_t* __restrict__ out) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_dst; i += (int64_t)gridDim.x * blockDim.x) {
        const int32_t v = dst[i];
        const int32_t deg = g_off[v + 1] - g_off[v];
        out[i] = (fanout < 0 || deg < fanout) ? deg : fanout;
    }
}

// One warp per destination.  deg <= fanout (or fanout < 0): the in-edge list is copied in its stored
// order, as the reference does.  Otherwise `fanout` DISTINCT positions of the list are drawn with
// Floyd's algorithm: for j = deg - fanout .. deg - 1 draw t in [0, j]; take t unless it was taken
// before, else take j.  The picks sit in shared memory and the membership test runs across the lanes.
constexpr int kSampleWarps = 8;
constexpr int kMaxFanout = 1024;   // the limit of the reference's CUDA sampler (sampleprocessing_op.cc:143-144)
__global__ void __launch_bounds__(kSampleWarps * 32) sample_neighbors_kernel(const int32_t* __restrict__ dst, int64_t n_dst,
                                                                             const int32_t* __restrict__ layer_off,
                                                                             const int32_t* __restrict__ g_off,
                                                                             const int32_t* __restrict__ g_idx, int32_t fanout,
                                                                             unsigned long long seed, int32_t* __restrict__ out,
                                                                             int64_t capacity, int* __restrict__ error) {
    extern __shared__ int s_picks[];   // [kSampleWarps][fanout]
    const int lane = lane_id();
    const int warp = threadIdx.x >> 5;
    int* picks = s_picks + (size_t)warp * (fanout > 0 ? fanout : 0);
    const int64_t n_warps = (int64_t)gridDim.x * kSampleWarps;
    for (int64_t i = (int64_t)blockIdx.x * kSampleWarps + warp; i < n_dst; i += n_warps) {
        const int32_t v = dst[i];
        const int32_t start = g_off[v], deg = g_off[v + 1] - start;
        const int64_t pos = layer_off[i];
        const int32_t room = layer_off[i + 1] - layer_off[i];
        const int32_t want = (fanout < 0 || deg < fanout) ? deg : fanout;
        if (room != want || pos < 0 || pos + want > capacity) {   // offsets that do not belong to this (dst, fanout)
            if (lane == 0) atomicExch(error, 1);
            continue;
        }
        if (want == deg) {
            for (int k = lane; k < deg; k += 32) out[pos + k] = g_idx[start + k];
            continue;
        }
        for (int k = 0; k < fanout; k++) {
            const int j = deg - fanout + k;
            const int t = draw_below(seed, v, k, j + 1);
            bool seen = false;
            for (int q = lane; q < k; q += 32) seen |= picks[q] == t;
            const int pick = __any_sync(kFull, seen) ? j : t;
            __syncwarp();
            if (lane == 0) picks[k] = pick;
            __syncwarp();
        }
        for (int k = lane; k < fanout; k += 32) out[pos + k] = g_idx[start + picks[k]];
        __syncwarp();
    }
}

// out[j] = values[i] (or i when values is null) for every entry j of column i; one warp per column
__global__ void expand_columns_kernel(const int32_t* __restrict__ off, int64_t n_cols, const int32_t* __restrict__ values,
                                      int32_t* __restrict__ out) {
    const int lane = lane_id();
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t i = warp; i < n_cols; i += n_warps) {
        const int32_t s = off[i], e = off[i + 1];
        const int32_t val = values ? values[i] : (int32_t)i;
        for (int32_t j = s + lane; j < e; j += 32) out[j] = val;
    }
}

__global__ void fill_i32_kernel(int32_t* p, int32_t v, int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) p[i] = v;
}
// where[ids[i]] = i (when an id is listed twice the larger position wins, as in the reference's
// sequential loop, csctocsr_op.cc:44-46)
__global__ void index_of_ids_kernel(const int32_t* __restrict__ ids, int64_t n, int32_t* __restrict__ where) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        atomicMax(&where[ids[i]], (int32_t)i);
}
// sort key of every CSC entry: the row its source id maps to, or n_src (a bucket that is cut off
// afterwards) when the id is not listed
__global__ void source_rows_kernel(const int32_t* __restrict__ row_idx, int64_t n_edges, const int32_t* __restrict__ where,
                                   int64_t id_range, int32_t n_src, int32_t* __restrict__ key) {
    for (int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; j < n_edges; j += (int64_t)gridDim.x * blockDim.x) {
        const int32_t id = row_idx[j];
        const int32_t r = (id >= 0 && id < id_range) ? where[id] : -1;
        key[j] = r >= 0 ? r : n_src;
    }
}
__global__ void copy_offsets_kernel(const int32_t* __restrict__ in, int64_t n, int32_t* __restrict__ out, int64_t* kept) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        out[i] = in[i];
        if (i == n - 1 && kept) *kept = in[i];
    }
}

// integer degrees, then weights: both exact, so the result equals the reference's sequential loop
__global__ void sample_degrees_kernel(const int32_t* __restrict__ dst_ids, int64_t n_dst, const int32_t* __restrict__ off,
                                      const int32_t* __restrict__ row_idx, int32_t* __restrict__ ins, int32_t* __restrict__ outs) {
    const int lane = lane_id();
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t i = warp; i < n_dst; i += n_warps) {
        const int32_t s = off[i], e = off[i + 1];
        if (lane == 0 && e > s) atomicAdd(&ins[dst_ids[i]], e - s);
        for (int32_t j = s + lane; j < e; j += 32) atomicAdd(&outs[row_idx[j]], 1);
    }
}
__global__ void degree_weights_kernel(const int32_t* __restrict__ dst_ids, int64_t n_dst, const int32_t* __restrict__ off,
                                      const int32_t* __restrict__ row_idx, const int32_t* __restrict__ ins,
                                      const int32_t* __restrict__ outs, float* __restrict__ w) {
    const int lane = lane_id();
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t i = warp; i < n_dst; i += n_warps) {
        const int32_t s = off[i], e = off[i + 1];
        if (e <= s) continue;
        const float root_in = __fsqrt_rn((float)ins[dst_ids[i]]);
        for (int32_t j = s + lane; j < e; j += 32)
            w[j] = __fdiv_rn(1.0f, __fmul_rn(__fsqrt_rn((float)outs[row_idx[j]]), root_in));
    }
}

static unsigned grid_for(int64_t items, int per_block) {
    int64_t b = (items + per_block - 1) / per_block;
    const int64_t cap = (int64_t)sm_count() * 8;
    if (b > cap) b = cap;
    return (unsigned)(b > 0 ? b : 1);
}

struct CscToCsrWs {
    int32_t* where;
    int32_t* ei;      // [2, E]: row key, column value
    int32_t* off;     // [n_src + 2]
    float* w;         // [E] weights written by the sort (all ones, unused)
    void* convert;
    size_t convert_bytes;
    size_t bytes;
};
static CscToCsrWs carve_csc_to_csr(void* ws, int64_t n_src, int64_t n_edges, int64_t id_range) {
    Carver c(ws);
    CscToCsrWs v;
    v.where = c.take<int32_t>((size_t)id_range);
    v.ei = c.take<int32_t>((size_t)(2 * n_edges));
    v.off = c.take<int32_t>((size_t)(n_src + 2));
    v.w = c.take<float>((size_t)n_edges);
    v.convert_bytes = jg_convert_workspace_bytes(n_edges, n_src + 1);
    v.convert = c.take<char>(v.convert_bytes);
    v.bytes = c.total();
    return v;
}

}  // namespace jg

using namespace jg;

extern "C" {

size_t jg_sample_counts_workspace_bytes(int64_t n_dst) {
    if (n_dst < 0) return 0;
    Carver c(nullptr);
    c.take<int>((size_t)(n_dst + 1));
    c.take<int>(scan_temp_ints(n_dst + 1));
    return c.total();
}

int jg_sample_counts(const int32_t* dst, int64_t n_dst, const int32_t* g_off, int32_t fanout, int cumulative, int32_t* out,
                     void* workspace, size_t workspace_bytes, jg_stream_t stream) {
    JG_CHECK_ARG(n_dst >= 0 && n_dst < INT32_MAX, JG_EINVAL, "sample_counts: bad size");
    JG_CHECK_ARG(out && (n_dst == 0 || (dst && g_off)), JG_EINVAL, "sample_counts: null pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (!cumulative) {   // the reference operator: out[0] = 0, out[i+1] = count of destination i
        JG_CUDA(cudaMemsetAsync(out, 0, sizeof(int32_t), st));
        if (n_dst > 0) {
            sample_counts_kernel<<<grid_for(n_dst, 256), 256, 0, st>>>(dst, n_dst, g_off, fanout, out + 1);
            JG_LAUNCH_CHECK();
        }
        return JG_OK;
    }
    JG_CHECK_ARG(workspace && workspace_bytes >= jg_sample_counts_workspace_bytes(n_dst), JG_EWORKSPACE,
                 "sample_counts: workspace too small");
    Carver c(workspace);
    int* counts = c.take<int>((size_t)(n_dst + 1));
    int* sums = c.take<int>(scan_temp_ints(n_dst + 1));
    JG_CUDA(cudaMemsetAsync(counts + n_dst, 0, sizeof(int), st));
    if (n_dst > 0) {
        sample_counts_kernel<<<grid_for(n_dst, 256), 256, 0, st>>>(dst, n_dst, g_off, fanout, counts);
        JG_LAUNCH_CHECK();
    }
    return exclusive_scan(counts, reinterpret_cast<int*>(out), n_dst + 1, sums, st);
}

int jg_sample_neighbors(const int32_t* dst, int64_t n_dst, const int32_t* layer_off, const int32_t* g_off, const int32_t* g_idx,
                        int32_t fanout, uint64_t seed, int32_t* layer_idx, int64_t layer_capacity, int32_t* error_flag,
                        jg_stream_t stream) {
    JG_CHECK_ARG(n_dst >= 0 && layer_capacity >= 0, JG_EINVAL, "sample_neighbors: negative size");
    JG_CHECK_ARG(error_flag, JG_EINVAL, "sample_neighbors: null error flag");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    JG_CUDA(cudaMemsetAsync(error_flag, 0, sizeof(int32_t), st));
    if (n_dst == 0) return JG_OK;
    JG_CHECK_ARG(dst && layer_off && g_off && (layer_capacity == 0 || (g_idx && layer_idx)), JG_EINVAL,
                 "sample_neighbors: null pointer");
    if (fanout > kMaxFanout) {
        set_error("sample_neighbors: fanout %d beyond %d (the limit of the reference's CUDA sampler as well)", fanout, kMaxFanout);
        return JG_EUNSUPPORTED;
    }
    const size_t smem = (size_t)kSampleWarps * (size_t)(fanout > 0 ? fanout : 0) * sizeof(int);
    sample_neighbors_kernel<<<grid_for(n_dst, kSampleWarps), kSampleWarps * 32, smem, st>>>(
        dst, n_dst, layer_off, g_off, g_idx, fanout, (unsigned long long)seed, layer_idx, layer_capacity, error_flag);
    JG_LAUNCH_CHECK();
    return JG_OK;
}

int jg_expand_columns(const int32_t* off, int64_t n_cols, const int32_t* values, int32_t* out, jg_stream_t stream) {
    JG_CHECK_ARG(n_cols >= 0, JG_EINVAL, "expand_columns: negative size");
    if (n_cols == 0) return JG_OK;
    JG_CHECK_ARG(off && out, JG_EINVAL, "expand_columns: null pointer");
    expand_columns_kernel<<<grid_for(n_cols * 32, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(off, n_cols, values, out);
    JG_LAUNCH_CHECK();
    return JG_OK;
}

size_t jg_csc_to_csr_workspace_bytes(int64_t n_src, int64_t n_edges, int64_t id_range) {
    if (n_src < 0 || n_edges < 0 || id_range < 0) return 0;
    return carve_csc_to_csr(nullptr, n_src, n_edges, id_range).bytes;
}

int jg_csc_to_csr(const int32_t* col_off, const int32_t* row_idx, int64_t n_dst, int64_t n_edges, const int32_t* dst_ids,
                  const int32_t* src_ids, int64_t n_src, int64_t id_range, int32_t* row_off, int32_t* col_idx, int64_t* kept,
                  void* workspace, size_t workspace_bytes, jg_stream_t stream) {
    JG_CHECK_ARG(n_dst >= 0 && n_edges >= 0 && n_src >= 0 && id_range >= 0, JG_EINVAL, "csc_to_csr: negative size");
    JG_CHECK_ARG(row_off && kept && col_off, JG_EINVAL, "csc_to_csr: null pointer");
    JG_CHECK_ARG(n_edges == 0 || (row_idx && col_idx), JG_EINVAL, "csc_to_csr: null index array");
    JG_CHECK_ARG(n_src == 0 || src_ids, JG_EINVAL, "csc_to_csr: null source ids");
    JG_CHECK_ARG(n_edges < INT32_MAX - 1 && n_src < INT32_MAX - 1 && id_range < INT32_MAX, JG_ESHAPE, "csc_to_csr: sizes beyond int32");
    JG_CHECK_ARG(workspace && workspace_bytes >= jg_csc_to_csr_workspace_bytes(n_src, n_edges, id_range), JG_EWORKSPACE,
                 "csc_to_csr: workspace too small");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    CscToCsrWs ws = carve_csc_to_csr(workspace, n_src, n_edges, id_range);
    if (id_range > 0) {
        fill_i32_kernel<<<grid_for(id_range, 256), 256, 0, st>>>(ws.where, -1, id_range);
        JG_LAUNCH_CHECK();
    }
    if (n_src > 0) {
        index_of_ids_kernel<<<grid_for(n_src, 256), 256, 0, st>>>(src_ids, n_src, ws.where);
        JG_LAUNCH_CHECK();
    }
    if (n_edges > 0) {
        source_rows_kernel<<<grid_for(n_edges, 256), 256, 0, st>>>(row_idx, n_edges, ws.where, id_range, (int32_t)n_src, ws.ei);
        JG_LAUNCH_CHECK();
        expand_columns_kernel<<<grid_for(n_dst * 32, 256), 256, 0, st>>>(col_off, n_dst, dst_ids, ws.ei + n_edges);
        JG_LAUNCH_CHECK();
    }
    // stable sort by row key; entries of unlisted sources land in row n_src and are cut off
    int rc = jg_coo_to_compressed(ws.ei, nullptr, n_edges, n_src + 1, 0, 0, col_idx, ws.off, ws.w, ws.convert, ws.convert_bytes,
                                  stream);
    if (rc != JG_OK) return rc;
    copy_offsets_kernel<<<grid_for(n_src + 1, 256), 256, 0, st>>>(ws.off, n_src + 1, row_off, kept);
    JG_LAUNCH_CHECK();
    return JG_OK;
}

size_t jg_degree_weights_workspace_bytes(int64_t vtx_size) {
    if (vtx_size < 0) return 0;
    Carver c(nullptr);
    c.take<int32_t>((size_t)(2 * vtx_size));
    return c.total();
}

int jg_degree_weights(int64_t vtx_size, const int32_t* dst_ids, int64_t n_dst, const int32_t* col_off, const int32_t* row_idx,
                      int64_t n_edges, float* out_w, void* workspace, size_t workspace_bytes, jg_stream_t stream) {
    JG_CHECK_ARG(vtx_size >= 0 && n_dst >= 0 && n_edges >= 0, JG_EINVAL, "degree_weights: negative size");
    if (n_dst == 0 || n_edges == 0) return JG_OK;
    JG_CHECK_ARG(dst_ids && col_off && row_idx && out_w, JG_EINVAL, "degree_weights: null pointer");
    JG_CHECK_ARG(workspace && workspace_bytes >= jg_degree_weights_workspace_bytes(vtx_size), JG_EWORKSPACE,
                 "degree_weights: workspace too small");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    Carver c(workspace);
    int32_t* ins = c.take<int32_t>((size_t)(2 * vtx_size));
    int32_t* outs = ins + vtx_size;
    JG_CUDA(cudaMemsetAsync(ins, 0, sizeof(int32_t) * (size_t)(2 * vtx_size), st));
    sample_degrees_kernel<<<grid_for(n_dst * 32, 256), 256, 0, st>>>(dst_ids, n_dst, col_off, row_idx, ins, outs);
    JG_LAUNCH_CHECK();
    degree_weights_kernel<<<grid_for(n_dst * 32, 256), 256, 0, st>>>(dst_ids, n_dst, col_off, row_idx, ins, outs, out_w);
    JG_LAUNCH_CHECK();
    return JG_OK;
}

}  // extern "C"
