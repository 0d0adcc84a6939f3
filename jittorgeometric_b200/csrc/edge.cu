// Per-edge operators of the attention path, as individually callable ops (sm_100a):
//   scatter_to_edge   msg[e,:] = x[src(e),:] or x[dst(e),:]      (ops/cpp/scattertoedge_op.cc:35-141)
//   edge_to_vertex    out[v,:] = sum of msg rows per destination / source (ops/cpp/edgetovertex_op.cc:27-95)
//   edge_softmax      per-destination softmax of per-edge scores, forward and backward
//                     (ops/cpp/edgesoftmax_op.cc:36-120, ops/cpp/edgesoftmaxbackward_op.cc:27-54)
// Edges are in CSC order: segment v = [off[v], off[v+1]) holds the in-edges of destination v and
// idx[e] is the source of edge e.  All four are pure bandwidth kernels (one pass over an [E, C]
// array); the fused attention kernel in gat.cu makes the [E, C] temporaries unnecessary, these
// exist for API parity.
#include "common.cuh"

namespace jg {

constexpr int kEdgeBlock = 256;

// Row (segment owner) of edge e: the v with off[v] <= e < off[v+1], searched in [lo, hi].
__device__ __forceinline__ int32_t owner_of(const int32_t* __restrict__ off, int32_t lo, int32_t hi, int32_t e) {
    while (lo < hi) {  // largest v with off[v] <= e
        const int32_t mid = lo + (hi - lo + 1) / 2;
        if (off[mid] <= e) lo = mid; else hi = mid - 1;
    }
    return lo;
}

// One warp copies node rows onto 32 consecutive edges at a time.  G lanes share a row (G * 16 bytes per
// step), 32 / G rows are copied side by side and four such steps are in flight, so a 256-byte row does
// not leave half the warp idle behind one dependent load.
__global__ void __launch_bounds__(kEdgeBlock) scatter_to_edge_kernel(float* __restrict__ out, const float* __restrict__ x,
                                                                     const int32_t* __restrict__ idx,
                                                                     const int32_t* __restrict__ off, int64_t n, int64_t E,
                                                                     int64_t C, int flag, int lanes_per_row) {
    const int lane = lane_id();
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const bool vec = lanes_per_row > 0;   // 0: width or pointers that 16-byte accesses cannot take
    const int G = vec ? lanes_per_row : 32, sub = lane / G, gl = lane % G, R = 32 / G;
    for (int64_t e0 = warp * 32; e0 < E; e0 += n_warps * 32) {
        const int64_t e = e0 + lane;
        int32_t node = 0;
        if (flag == 0) {
            if (e < E) node = idx[e];
        } else {
            // rows of the tile's first and last edge bound every lane's search
            const int32_t last = (int32_t)((e0 + 31) < (E - 1) ? (e0 + 31) : (E - 1));
            const int32_t r_first = owner_of(off, 0, (int32_t)n - 1, (int32_t)e0);
            const int32_t r_last = owner_of(off, r_first, (int32_t)n - 1, last);
            if (e < E) node = owner_of(off, r_first, r_last, (int32_t)e);
        }
        const int cnt = (E - e0) < 32 ? (int)(E - e0) : 32;
        if (vec) {
            constexpr int U = 4;
            const int64_t chunks = C / 4;
            for (int k0 = 0; k0 < cnt; k0 += R * U) {
                int32_t src[U];
#pragma unroll
                for (int u = 0; u < U; u++) src[u] = __shfl_sync(kFull, node, (k0 + u * R + sub) & 31);
                for (int64_t c = gl; c < chunks; c += G) {
                    float4 v[U];
#pragma unroll
                    for (int u = 0; u < U; u++) {
                        const int k = k0 + u * R + sub;
                        v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (k < cnt) v[u] = __ldg(reinterpret_cast<const float4*>(x + (size_t)src[u] * C) + c);
                    }
#pragma unroll
                    for (int u = 0; u < U; u++) {
                        const int k = k0 + u * R + sub;
                        if (k < cnt) __stcs(reinterpret_cast<float4*>(out + (size_t)(e0 + k) * C) + c, v[u]);
                    }
                }
            }
        } else {
            for (int k = 0; k < cnt; k++) {
                const int32_t src = __shfl_sync(kFull, node, k);
                const float* xr = x + (size_t)src * C;
                float* o = out + (size_t)(e0 + k) * C;
                for (int64_t c = lane; c < C; c += 32) o[c] = __ldg(xr + c);
            }
        }
    }
}

// out[v,:] = sum of msg[e,:] over the in-edges of v, ascending e (flag 1): one warp per destination.
__global__ void __launch_bounds__(kEdgeBlock) edge_to_vertex_dst_kernel(float* __restrict__ out, const float* __restrict__ msg,
                                                                        const int32_t* __restrict__ off, int64_t n, int64_t C) {
    const int lane = lane_id();
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t v = warp; v < n; v += n_warps) {
        const int32_t s = off[v], e = off[v + 1];
        for (int64_t c = lane; c < C; c += 32) {
            float acc = 0.f;
            int32_t j = s;
            for (; j + 4 <= e; j += 4) {  // four independent loads in flight, added in order
                const float a0 = __ldcs(msg + (size_t)j * C + c), a1 = __ldcs(msg + (size_t)(j + 1) * C + c);
                const float a2 = __ldcs(msg + (size_t)(j + 2) * C + c), a3 = __ldcs(msg + (size_t)(j + 3) * C + c);
                acc = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(acc, a0), a1), a2), a3);
            }
            for (; j < e; j++) acc = __fadd_rn(acc, __ldcs(msg + (size_t)j * C + c));
            out[(size_t)v * C + c] = acc;
        }
    }
}

// out[idx[e],:] += msg[e,:] (flag 0): scatter by source.  Float atomics, as the reference's CUDA
// kernel does (ops/cpp/edgetovertex_op.cc:69); out must be zeroed by the launcher.
__global__ void __launch_bounds__(kEdgeBlock) edge_to_vertex_src_kernel(float* __restrict__ out, const float* __restrict__ msg,
                                                                        const int32_t* __restrict__ idx, int64_t E, int64_t C) {
    const int64_t total = E * C;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t e = i / C, c = i - e * C;
        atomicAdd(out + (size_t)idx[e] * C + c, __ldcs(msg + i));
    }
}

__global__ void zero_kernel(float* p, int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) p[i] = 0.f;
}

// ------------------------------------------------------------------------------- edge softmax
// x, y are [E, H] row-major; the softmax runs over each segment separately for every column.
// HP = H when H is a power of two <= 32: a lane then always meets the same column (its flat
// index modulo H is lane % H) and columns are reduced with xor-shuffles over offsets >= H.
template <int HP>
__device__ __forceinline__ float reduce_same_column_max(float v) {
#pragma unroll
    for (int o = 16; o >= HP; o >>= 1) v = fmaxf(v, __shfl_xor_sync(kFull, v, o));
    return v;
}
template <int HP>
__device__ __forceinline__ float reduce_same_column_sum(float v) {
#pragma unroll
    for (int o = 16; o >= HP; o >>= 1) v += __shfl_xor_sync(kFull, v, o);
    return v;
}

// Segments of kSoftmaxHub edges or more are left to the block-per-segment kernels below: one warp
// walking tens of thousands of entries alone would be the tail of the whole launch.
constexpr int kSoftmaxHub = 2048;
// The backward pass has no exponentials and a cheap block-wide sum, and a block that owns a segment finds it in
// L2 on its second sweep (far fewer segments are in flight than with a warp each): measured on the attention
// workload 0.77 ms with the forward's threshold, 0.57 ms with this one.  The forward's block role pays a
// four-column (maximum, sum) merge with exponentials per segment and was slower below 2048 edges (1.0 vs 0.58 ms).
constexpr int kSoftmaxBwdHub = 384;
// 128-bit forward kernel: its block role makes three sweeps (maxima, sums, values) with plain block
// reductions, the second and third out of L2, and takes the same segments as the backward's.
constexpr int kSoftmaxFwdVecHub = 384;

// Running (maximum, sum of exp(x - maximum)) of the elements a lane has met; merging two such states
// rescales the one with the smaller maximum.  An empty state is (-inf, 0).
struct MaxSum {
    float m, s;
    __device__ __forceinline__ void add4(float a0, float a1, float a2, float a3) {
        const float m4 = fmaxf(fmaxf(a0, a1), fmaxf(a2, a3));
        if (m4 > m) {
            s *= expf(m - m4);   // m = -inf at the start: the empty sum scales to 0
            m = m4;
        }
        s += (expf(a0 - m) + expf(a1 - m)) + (expf(a2 - m) + expf(a3 - m));
    }
    __device__ __forceinline__ void add(float a) {
        if (a > m) {
            s *= expf(m - a);
            m = a;
        }
        s += expf(a - m);
    }
    __device__ __forceinline__ void merge(float m2, float s2) {
        const float mn = fmaxf(m, m2);
        const float f1 = (m == -INFINITY) ? 0.f : expf(m - mn);
        const float f2 = (m2 == -INFINITY) ? 0.f : expf(m2 - mn);
        s = s * f1 + s2 * f2;
        m = mn;
    }
};

// Two passes per segment: (maximum, sum) in one sweep with four loads in flight per lane, then the
// normalised values (the second sweep finds the segment in cache).
template <int HP>
__global__ void __launch_bounds__(kEdgeBlock) edge_softmax_fwd_kernel(float* __restrict__ y, const float* __restrict__ x,
                                                                      const int32_t* __restrict__ off, int64_t n) {
    const int lane = lane_id();
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t v = warp; v < n; v += n_warps) {
        if (off[v + 1] - off[v] >= kSoftmaxHub) continue;
        const int64_t s = (int64_t)off[v] * HP, e = (int64_t)off[v + 1] * HP;
        if (s >= e) continue;
        MaxSum st = {-INFINITY, 0.f};
        int64_t i = s + lane;
        for (; i + 96 < e; i += 128) st.add4(x[i], x[i + 32], x[i + 64], x[i + 96]);
        for (; i < e; i += 32) st.add(x[i]);
#pragma unroll
        for (int o = 16; o >= HP; o >>= 1) {   // lanes of the same column; both partners end with the same state
            const float m2 = __shfl_xor_sync(kFull, st.m, o), s2 = __shfl_xor_sync(kFull, st.s, o);
            if (lane & o) {
                MaxSum other = {m2, s2};
                other.merge(st.m, st.s);
                st = other;
            } else {
                st.merge(m2, s2);
            }
        }
        const float mx = st.m, inv = 1.f / st.s;
        i = s + lane;
        for (; i + 96 < e; i += 128) {
            const float a0 = x[i], a1 = x[i + 32], a2 = x[i + 64], a3 = x[i + 96];
            y[i] = expf(a0 - mx) * inv; y[i + 32] = expf(a1 - mx) * inv;
            y[i + 64] = expf(a2 - mx) * inv; y[i + 96] = expf(a3 - mx) * inv;
        }
        for (; i < e; i += 32) y[i] = expf(x[i] - mx) * inv;
    }
}

// Block-wide reductions over the threads that meet the same column (thread t always meets column
// t % HP because the block size is a multiple of HP): inside a warp by shuffles, across the warps
// through shared memory in warp order.
template <int HP, bool IS_MAX>
__device__ __forceinline__ float block_same_column(float v, float* s_buf /*[kEdgeBlock]*/) {
    v = IS_MAX ? reduce_same_column_max<HP>(v) : reduce_same_column_sum<HP>(v);
    __syncthreads();
    s_buf[threadIdx.x] = v;
    __syncthreads();
    float r = s_buf[threadIdx.x & 31];
#pragma unroll
    for (int w = 1; w < kEdgeBlock / 32; w++) {
        const float o = s_buf[w * 32 + (threadIdx.x & 31)];
        r = IS_MAX ? fmaxf(r, o) : r + o;
    }
    return r;
}

// One block per long segment, the same two sweeps as the warp kernel: running (maximum, sum) with four
// loads in flight per thread, merged across the block in thread order, then the normalised values.
template <int HP>
__global__ void __launch_bounds__(kEdgeBlock) edge_softmax_fwd_hub_kernel(float* __restrict__ y, const float* __restrict__ x,
                                                                          const int32_t* __restrict__ off, int64_t n) {
    __shared__ float s_m[kEdgeBlock], s_s[kEdgeBlock];
    const int lane = threadIdx.x & 31;
    for (int64_t v = blockIdx.x; v < n; v += gridDim.x) {
        if (off[v + 1] - off[v] < kSoftmaxHub) continue;   // block-uniform
        const int64_t s = (int64_t)off[v] * HP, e = (int64_t)off[v + 1] * HP;
        MaxSum st = {-INFINITY, 0.f};
        int64_t i = s + threadIdx.x;
        for (; i + 3 * kEdgeBlock < e; i += 4 * kEdgeBlock)
            st.add4(x[i], x[i + kEdgeBlock], x[i + 2 * kEdgeBlock], x[i + 3 * kEdgeBlock]);
        for (; i < e; i += kEdgeBlock) st.add(x[i]);
#pragma unroll
        for (int o = 16; o >= HP; o >>= 1) {   // lanes of the same column inside the warp
            const float m2 = __shfl_xor_sync(kFull, st.m, o), s2 = __shfl_xor_sync(kFull, st.s, o);
            if (lane & o) {
                MaxSum other = {m2, s2};
                other.merge(st.m, st.s);
                st = other;
            } else {
                st.merge(m2, s2);
            }
        }
        __syncthreads();
        s_m[threadIdx.x] = st.m;
        s_s[threadIdx.x] = st.s;
        __syncthreads();
        MaxSum all = {s_m[lane], s_s[lane]};     // warps in order: every thread ends with the same state per column
#pragma unroll
        for (int w = 1; w < kEdgeBlock / 32; w++) all.merge(s_m[w * 32 + lane], s_s[w * 32 + lane]);
        const float mx = all.m, inv = 1.f / all.s;
        i = s + threadIdx.x;
        for (; i + 3 * kEdgeBlock < e; i += 4 * kEdgeBlock) {
            const float a0 = x[i], a1 = x[i + kEdgeBlock], a2 = x[i + 2 * kEdgeBlock], a3 = x[i + 3 * kEdgeBlock];
            y[i] = expf(a0 - mx) * inv; y[i + kEdgeBlock] = expf(a1 - mx) * inv;
            y[i + 2 * kEdgeBlock] = expf(a2 - mx) * inv; y[i + 3 * kEdgeBlock] = expf(a3 - mx) * inv;
        }
        for (; i < e; i += kEdgeBlock) y[i] = expf(x[i] - mx) * inv;
    }
}

// 128-bit form of the two kernels above for H = 4, 8, 16, 32 (16-byte aligned x and y): a lane
// carries the four columns of one float4 (column group lane % (H/4)), so four times the bytes are in
// flight per lane for the same number of requests.  Same two sweeps, same merge order per column.
__device__ __forceinline__ void merge_lanes(MaxSum& st, int lane, int o) {
    const float m2 = __shfl_xor_sync(kFull, st.m, o), s2 = __shfl_xor_sync(kFull, st.s, o);
    if (lane & o) {
        MaxSum other = {m2, s2};
        other.merge(st.m, st.s);
        st = other;
    } else {
        st.merge(m2, s2);
    }
}

__device__ __forceinline__ float4 softmax_values(const float4& a, const float (&mx)[4], const float (&inv)[4]) {
    return make_float4(expf(a.x - mx[0]) * inv[0], expf(a.y - mx[1]) * inv[1], expf(a.z - mx[2]) * inv[2], expf(a.w - mx[3]) * inv[3]);
}

template <int HP>
__device__ __forceinline__ void softmax_fwd_vec_warps(float4* __restrict__ y, const float4* __restrict__ x,
                                                      const int32_t* __restrict__ off, int64_t n, int block, int n_blocks) {
    constexpr int Q = HP / 4;
    const int lane = lane_id();
    const int64_t warp = ((int64_t)block * blockDim.x + threadIdx.x) >> 5;
    const int64_t n_warps = ((int64_t)n_blocks * blockDim.x) >> 5;
    for (int64_t v = warp; v < n; v += n_warps) {
        if (off[v + 1] - off[v] >= kSoftmaxFwdVecHub) continue;
        const int64_t s = (int64_t)off[v] * Q, e = (int64_t)off[v + 1] * Q;
        if (s >= e) continue;
        MaxSum st[4] = {{-INFINITY, 0.f}, {-INFINITY, 0.f}, {-INFINITY, 0.f}, {-INFINITY, 0.f}};
        int64_t i = s + lane;
        for (; i + 96 < e; i += 128) {
            const float4 a0 = x[i], a1 = x[i + 32], a2 = x[i + 64], a3 = x[i + 96];
            st[0].add4(a0.x, a1.x, a2.x, a3.x); st[1].add4(a0.y, a1.y, a2.y, a3.y);
            st[2].add4(a0.z, a1.z, a2.z, a3.z); st[3].add4(a0.w, a1.w, a2.w, a3.w);
        }
        for (; i < e; i += 32) {
            const float4 a = x[i];
            st[0].add(a.x); st[1].add(a.y); st[2].add(a.z); st[3].add(a.w);
        }
#pragma unroll
        for (int o = 16; o >= Q; o >>= 1) {
#pragma unroll
            for (int c = 0; c < 4; c++) merge_lanes(st[c], lane, o);
        }
        float mx[4], inv[4];
#pragma unroll
        for (int c = 0; c < 4; c++) { mx[c] = st[c].m; inv[c] = 1.f / st[c].s; }
        i = s + lane;
        for (; i + 96 < e; i += 128) {
            const float4 a0 = x[i], a1 = x[i + 32], a2 = x[i + 64], a3 = x[i + 96];
            __stcs(y + i, softmax_values(a0, mx, inv)); __stcs(y + i + 32, softmax_values(a1, mx, inv));
            __stcs(y + i + 64, softmax_values(a2, mx, inv)); __stcs(y + i + 96, softmax_values(a3, mx, inv));
        }
        for (; i < e; i += 32) __stcs(y + i, softmax_values(x[i], mx, inv));
    }
}

// Four per-thread values reduced over the threads of the block that meet the same columns (thread t carries the
// columns of float4 number t % Q): shuffles inside the warp, one pass through shared memory across the warps
// (in warp order), two barriers for all four values.
template <int Q, bool IS_MAX>
__device__ __forceinline__ void block_same_columns4(float (&v)[4], float (*s_buf)[kEdgeBlock]) {
#pragma unroll
    for (int c = 0; c < 4; c++) v[c] = IS_MAX ? reduce_same_column_max<Q>(v[c]) : reduce_same_column_sum<Q>(v[c]);
    __syncthreads();
#pragma unroll
    for (int c = 0; c < 4; c++) s_buf[c][threadIdx.x] = v[c];
    __syncthreads();
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int c = 0; c < 4; c++) {
        float r = s_buf[c][lane];
#pragma unroll
        for (int w = 1; w < kEdgeBlock / 32; w++) {
            const float o = s_buf[c][w * 32 + lane];
            r = IS_MAX ? fmaxf(r, o) : r + o;
        }
        v[c] = r;
    }
}

// Block role of the 128-bit forward kernel: a block owns a segment and sweeps it three times - column maxima,
// sums of exp(x - maximum), normalised values.  Only the first sweep comes from DRAM: with a block per segment
// few segments are in flight and the other two find theirs in L2.  The reductions are plain maxima and sums
// (no rescaling exponentials), two barriers each.
template <int HP>
__device__ __forceinline__ void softmax_fwd_vec_block(float4* __restrict__ y, const float4* __restrict__ x,
                                                      const int32_t* __restrict__ off, int64_t n, int block, int n_blocks,
                                                      float (*s_buf)[kEdgeBlock]) {
    constexpr int Q = HP / 4;
    for (int64_t v = block; v < n; v += n_blocks) {
        if (off[v + 1] - off[v] < kSoftmaxFwdVecHub) continue;   // block-uniform
        const int64_t s = (int64_t)off[v] * Q, e = (int64_t)off[v + 1] * Q;
        float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
        int64_t i = s + threadIdx.x;
        for (; i + 3 * kEdgeBlock < e; i += 4 * kEdgeBlock) {
            const float4 a0 = x[i], a1 = x[i + kEdgeBlock], a2 = x[i + 2 * kEdgeBlock], a3 = x[i + 3 * kEdgeBlock];
            mx[0] = fmaxf(mx[0], fmaxf(fmaxf(a0.x, a1.x), fmaxf(a2.x, a3.x)));
            mx[1] = fmaxf(mx[1], fmaxf(fmaxf(a0.y, a1.y), fmaxf(a2.y, a3.y)));
            mx[2] = fmaxf(mx[2], fmaxf(fmaxf(a0.z, a1.z), fmaxf(a2.z, a3.z)));
            mx[3] = fmaxf(mx[3], fmaxf(fmaxf(a0.w, a1.w), fmaxf(a2.w, a3.w)));
        }
        for (; i < e; i += kEdgeBlock) {
            const float4 a = x[i];
            mx[0] = fmaxf(mx[0], a.x); mx[1] = fmaxf(mx[1], a.y); mx[2] = fmaxf(mx[2], a.z); mx[3] = fmaxf(mx[3], a.w);
        }
        block_same_columns4<Q, true>(mx, s_buf);
        float sm[4] = {0.f, 0.f, 0.f, 0.f};
        i = s + threadIdx.x;
        for (; i + 3 * kEdgeBlock < e; i += 4 * kEdgeBlock) {
            const float4 a0 = x[i], a1 = x[i + kEdgeBlock], a2 = x[i + 2 * kEdgeBlock], a3 = x[i + 3 * kEdgeBlock];
            sm[0] += (expf(a0.x - mx[0]) + expf(a1.x - mx[0])) + (expf(a2.x - mx[0]) + expf(a3.x - mx[0]));
            sm[1] += (expf(a0.y - mx[1]) + expf(a1.y - mx[1])) + (expf(a2.y - mx[1]) + expf(a3.y - mx[1]));
            sm[2] += (expf(a0.z - mx[2]) + expf(a1.z - mx[2])) + (expf(a2.z - mx[2]) + expf(a3.z - mx[2]));
            sm[3] += (expf(a0.w - mx[3]) + expf(a1.w - mx[3])) + (expf(a2.w - mx[3]) + expf(a3.w - mx[3]));
        }
        for (; i < e; i += kEdgeBlock) {
            const float4 a = x[i];
            sm[0] += expf(a.x - mx[0]); sm[1] += expf(a.y - mx[1]); sm[2] += expf(a.z - mx[2]); sm[3] += expf(a.w - mx[3]);
        }
        block_same_columns4<Q, false>(sm, s_buf);
        float inv[4];
#pragma unroll
        for (int c = 0; c < 4; c++) inv[c] = 1.f / sm[c];
        i = s + threadIdx.x;
        for (; i + 3 * kEdgeBlock < e; i += 4 * kEdgeBlock) {
            const float4 a0 = x[i], a1 = x[i + kEdgeBlock], a2 = x[i + 2 * kEdgeBlock], a3 = x[i + 3 * kEdgeBlock];
            __stcs(y + i, softmax_values(a0, mx, inv)); __stcs(y + i + kEdgeBlock, softmax_values(a1, mx, inv));
            __stcs(y + i + 2 * kEdgeBlock, softmax_values(a2, mx, inv)); __stcs(y + i + 3 * kEdgeBlock, softmax_values(a3, mx, inv));
        }
        for (; i < e; i += kEdgeBlock) __stcs(y + i, softmax_values(x[i], mx, inv));
    }
}

// ONE launch for both roles: the first `hub_blocks` blocks take the long segments (a block each, scheduled
// first), the others the short ones (a warp each), so the long segments' tail runs beside the bulk of the
// work instead of after it.
template <int HP>
__global__ void __launch_bounds__(kEdgeBlock) edge_softmax_fwd_vec_kernel(float4* __restrict__ y, const float4* __restrict__ x,
                                                                          const int32_t* __restrict__ off, int64_t n, int hub_blocks) {
    __shared__ float s_buf[4][kEdgeBlock];
    if ((int)blockIdx.x < hub_blocks)
        softmax_fwd_vec_block<HP>(y, x, off, n, (int)blockIdx.x, hub_blocks, s_buf);
    else
        softmax_fwd_vec_warps<HP>(y, x, off, n, (int)blockIdx.x - hub_blocks, (int)gridDim.x - hub_blocks);
}

// Any H: one (segment, column) pair per warp pass, strided access.
__global__ void __launch_bounds__(kEdgeBlock) edge_softmax_fwd_any_kernel(float* __restrict__ y, const float* __restrict__ x,
                                                                          const int32_t* __restrict__ off, int64_t n, int64_t H) {
    const int lane = lane_id();
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t t = warp; t < n * H; t += n_warps) {
        const int64_t v = t / H, h = t - v * H;
        const int64_t s = off[v], e = off[v + 1];
        if (s >= e) continue;
        float mx = -INFINITY;
        for (int64_t j = s + lane; j < e; j += 32) mx = fmaxf(mx, x[j * H + h]);
        mx = reduce_same_column_max<1>(mx);
        float sum = 0.f;
        for (int64_t j = s + lane; j < e; j += 32) sum += expf(x[j * H + h] - mx);
        sum = reduce_same_column_sum<1>(sum);
        for (int64_t j = s + lane; j < e; j += 32) y[j * H + h] = expf(x[j * H + h] - mx) / sum;
    }
}

// dx = y*g - y*dot, dot = sum over the segment of y*g.
template <int HP>
__global__ void __launch_bounds__(kEdgeBlock) edge_softmax_bwd_kernel(float* __restrict__ dx, const float* __restrict__ g,
                                                                      const float* __restrict__ y,
                                                                      const int32_t* __restrict__ off, int64_t n) {
    const int lane = lane_id();
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t v = warp; v < n; v += n_warps) {
        if (off[v + 1] - off[v] >= kSoftmaxBwdHub) continue;
        const int64_t s = (int64_t)off[v] * HP, e = (int64_t)off[v + 1] * HP;
        float dot = 0.f;
        int64_t i = s + lane;
        for (; i + 96 < e; i += 128) {   // eight independent loads in flight, added in order
            const float p0 = y[i] * g[i], p1 = y[i + 32] * g[i + 32], p2 = y[i + 64] * g[i + 64], p3 = y[i + 96] * g[i + 96];
            dot = (((dot + p0) + p1) + p2) + p3;
        }
        for (; i < e; i += 32) dot += y[i] * g[i];
        dot = reduce_same_column_sum<HP>(dot);
        for (i = s + lane; i < e; i += 32) dx[i] = __fsub_rn(__fmul_rn(y[i], g[i]), __fmul_rn(y[i], dot));
    }
}

template <int HP>
__global__ void __launch_bounds__(kEdgeBlock) edge_softmax_bwd_hub_kernel(float* __restrict__ dx, const float* __restrict__ g,
                                                                          const float* __restrict__ y,
                                                                          const int32_t* __restrict__ off, int64_t n) {
    __shared__ float s_buf[kEdgeBlock];
    for (int64_t v = blockIdx.x; v < n; v += gridDim.x) {
        if (off[v + 1] - off[v] < kSoftmaxBwdHub) continue;   // block-uniform
        const int64_t s = (int64_t)off[v] * HP, e = (int64_t)off[v + 1] * HP;
        float dot = 0.f;
        int64_t i = s + threadIdx.x;
        for (; i + 3 * kEdgeBlock < e; i += 4 * kEdgeBlock) {   // eight independent loads in flight, added in order
            const float p0 = y[i] * g[i], p1 = y[i + kEdgeBlock] * g[i + kEdgeBlock];
            const float p2 = y[i + 2 * kEdgeBlock] * g[i + 2 * kEdgeBlock], p3 = y[i + 3 * kEdgeBlock] * g[i + 3 * kEdgeBlock];
            dot = (((dot + p0) + p1) + p2) + p3;
        }
        for (; i < e; i += kEdgeBlock) dot += y[i] * g[i];
        dot = block_same_column<HP, false>(dot, s_buf);
        i = s + threadIdx.x;
        for (; i + 3 * kEdgeBlock < e; i += 4 * kEdgeBlock) {
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const float yy = y[i + u * kEdgeBlock], gg = g[i + u * kEdgeBlock];
                dx[i + u * kEdgeBlock] = __fsub_rn(__fmul_rn(yy, gg), __fmul_rn(yy, dot));
            }
        }
        for (; i < e; i += kEdgeBlock) dx[i] = __fsub_rn(__fmul_rn(y[i], g[i]), __fmul_rn(y[i], dot));
    }
}

// 128-bit forms for H = 4, 8, 16, 32 (16-byte aligned operands): a lane carries the four columns of a float4.
__device__ __forceinline__ float4 softmax_grad(const float4& yy, const float4& gg, const float (&dot)[4]) {
    return make_float4(__fsub_rn(__fmul_rn(yy.x, gg.x), __fmul_rn(yy.x, dot[0])), __fsub_rn(__fmul_rn(yy.y, gg.y), __fmul_rn(yy.y, dot[1])),
                       __fsub_rn(__fmul_rn(yy.z, gg.z), __fmul_rn(yy.z, dot[2])), __fsub_rn(__fmul_rn(yy.w, gg.w), __fmul_rn(yy.w, dot[3])));
}
__device__ __forceinline__ void dot_add(float (&dot)[4], const float4& yy, const float4& gg) {
    dot[0] += yy.x * gg.x; dot[1] += yy.y * gg.y; dot[2] += yy.z * gg.z; dot[3] += yy.w * gg.w;
}

template <int HP>
__device__ __forceinline__ void softmax_bwd_vec_warps(float4* __restrict__ dx, const float4* __restrict__ g,
                                                      const float4* __restrict__ y, const int32_t* __restrict__ off, int64_t n,
                                                      int block, int n_blocks) {
    constexpr int Q = HP / 4;
    const int lane = lane_id();
    const int64_t warp = ((int64_t)block * blockDim.x + threadIdx.x) >> 5;
    const int64_t n_warps = ((int64_t)n_blocks * blockDim.x) >> 5;
    for (int64_t v = warp; v < n; v += n_warps) {
        if (off[v + 1] - off[v] >= kSoftmaxBwdHub) continue;
        const int64_t s = (int64_t)off[v] * Q, e = (int64_t)off[v + 1] * Q;
        float dot[4] = {0.f, 0.f, 0.f, 0.f};
        int64_t i = s + lane;
        for (; i + 32 < e; i += 64) {   // four independent 16-byte loads in flight, added in order
            const float4 y0 = y[i], g0 = g[i], y1 = y[i + 32], g1 = g[i + 32];
            dot_add(dot, y0, g0);
            dot_add(dot, y1, g1);
        }
        for (; i < e; i += 32) dot_add(dot, y[i], g[i]);
#pragma unroll
        for (int c = 0; c < 4; c++) dot[c] = reduce_same_column_sum<Q>(dot[c]);
        i = s + lane;
        for (; i + 32 < e; i += 64) {
            const float4 y0 = y[i], g0 = g[i], y1 = y[i + 32], g1 = g[i + 32];
            __stcs(dx + i, softmax_grad(y0, g0, dot));
            __stcs(dx + i + 32, softmax_grad(y1, g1, dot));
        }
        for (; i < e; i += 32) __stcs(dx + i, softmax_grad(y[i], g[i], dot));
    }
}

template <int HP>
__device__ __forceinline__ void softmax_bwd_vec_block(float4* __restrict__ dx, const float4* __restrict__ g,
                                                      const float4* __restrict__ y, const int32_t* __restrict__ off, int64_t n,
                                                      int block, int n_blocks, float* s_buf) {
    constexpr int Q = HP / 4;
    for (int64_t v = block; v < n; v += n_blocks) {
        if (off[v + 1] - off[v] < kSoftmaxBwdHub) continue;   // block-uniform
        const int64_t s = (int64_t)off[v] * Q, e = (int64_t)off[v + 1] * Q;
        float dot[4] = {0.f, 0.f, 0.f, 0.f};
        int64_t i = s + threadIdx.x;
        for (; i + 3 * kEdgeBlock < e; i += 4 * kEdgeBlock) {   // eight loads in flight per thread, added in order
            float4 yy[4], gg[4];
#pragma unroll
            for (int u = 0; u < 4; u++) { yy[u] = y[i + u * kEdgeBlock]; gg[u] = g[i + u * kEdgeBlock]; }
#pragma unroll
            for (int u = 0; u < 4; u++) dot_add(dot, yy[u], gg[u]);
        }
        for (; i + kEdgeBlock < e; i += 2 * kEdgeBlock) {
            const float4 y0 = y[i], g0 = g[i], y1 = y[i + kEdgeBlock], g1 = g[i + kEdgeBlock];
            dot_add(dot, y0, g0);
            dot_add(dot, y1, g1);
        }
        for (; i < e; i += kEdgeBlock) dot_add(dot, y[i], g[i]);
#pragma unroll
        for (int c = 0; c < 4; c++) dot[c] = block_same_column<Q, false>(dot[c], s_buf);
        i = s + threadIdx.x;
        for (; i + 3 * kEdgeBlock < e; i += 4 * kEdgeBlock) {
            float4 yy[4], gg[4];
#pragma unroll
            for (int u = 0; u < 4; u++) { yy[u] = y[i + u * kEdgeBlock]; gg[u] = g[i + u * kEdgeBlock]; }
#pragma unroll
            for (int u = 0; u < 4; u++) __stcs(dx + i + u * kEdgeBlock, softmax_grad(yy[u], gg[u], dot));
        }
        for (; i + kEdgeBlock < e; i += 2 * kEdgeBlock) {
            const float4 y0 = y[i], g0 = g[i], y1 = y[i + kEdgeBlock], g1 = g[i + kEdgeBlock];
            __stcs(dx + i, softmax_grad(y0, g0, dot));
            __stcs(dx + i + kEdgeBlock, softmax_grad(y1, g1, dot));
        }
        for (; i < e; i += kEdgeBlock) __stcs(dx + i, softmax_grad(y[i], g[i], dot));
    }
}

template <int HP>
__global__ void __launch_bounds__(kEdgeBlock) edge_softmax_bwd_vec_kernel(float4* __restrict__ dx, const float4* __restrict__ g,
                                                                          const float4* __restrict__ y,
                                                                          const int32_t* __restrict__ off, int64_t n, int hub_blocks) {
    __shared__ float s_buf[kEdgeBlock];
    if ((int)blockIdx.x < hub_blocks)
        softmax_bwd_vec_block<HP>(dx, g, y, off, n, (int)blockIdx.x, hub_blocks, s_buf);
    else
        softmax_bwd_vec_warps<HP>(dx, g, y, off, n, (int)blockIdx.x - hub_blocks, (int)gridDim.x - hub_blocks);
}

__global__ void __launch_bounds__(kEdgeBlock) edge_softmax_bwd_any_kernel(float* __restrict__ dx, const float* __restrict__ g,
                                                                          const float* __restrict__ y,
                                                                          const int32_t* __restrict__ off, int64_t n, int64_t H) {
    const int lane = lane_id();
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t t = warp; t < n * H; t += n_warps) {
        const int64_t v = t / H, h = t - v * H;
        const int64_t s = off[v], e = off[v + 1];
        float dot = 0.f;
        for (int64_t j = s + lane; j < e; j += 32) dot += y[j * H + h] * g[j * H + h];
        dot = reduce_same_column_sum<1>(dot);
        for (int64_t j = s + lane; j < e; j += 32)
            dx[j * H + h] = __fsub_rn(__fmul_rn(y[j * H + h], g[j * H + h]), __fmul_rn(y[j * H + h], dot));
    }
}

// Structure check: offsets start at 0, never decrease, end at nnz; every index lies in [0, n_in).
// Violations are counted per kind in report[0..3]; nothing is dereferenced through a bad value.
__global__ void validate_segments_kernel(const int32_t* __restrict__ idx, const int32_t* __restrict__ off, int64_t n_out,
                                         int64_t n_in, int64_t nnz, int32_t* __restrict__ report) {
    const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    if (t == 0) {
        if (off[0] != 0) atomicAdd(&report[0], 1);
        if (off[n_out] != nnz) atomicAdd(&report[1], 1);
    }
    for (int64_t v = t; v < n_out; v += stride)
        if (off[v + 1] < off[v]) atomicAdd(&report[2], 1);
    for (int64_t e = t; e < nnz; e += stride)
        if (idx[e] < 0 || idx[e] >= n_in) atomicAdd(&report[3], 1);
}

static int grid_for_warps(int64_t warps_wanted) {
    const int64_t max_blocks = (int64_t)sm_count() * 8;
    int64_t blocks = (warps_wanted * 32 + kEdgeBlock - 1) / kEdgeBlock;
    if (blocks < 1) blocks = 1;
    return (int)(blocks < max_blocks ? blocks : max_blocks);
}

// blocks of the block-per-segment kernels: they scan all segments for the long ones
static int hub_blocks(int64_t n_nodes) {
    const int64_t cap = (int64_t)sm_count() * 8;
    return (int)(n_nodes < cap ? (n_nodes > 0 ? n_nodes : 1) : cap);
}

}  // namespace jg

using namespace jg;

extern "C" {

int jg_scatter_to_edge_f32(float* out, const float* x, const int32_t* idx, const int32_t* off, int64_t n_nodes,
                           int64_t n_edges, int64_t c, int flag, jg_stream_t stream) {
    JG_CHECK_ARG(n_nodes >= 0 && n_edges >= 0 && c >= 0, JG_EINVAL, "scatter_to_edge: negative size");
    JG_CHECK_ARG(flag == 0 || flag == 1, JG_EINVAL, "scatter_to_edge: flag must be 0 (source) or 1 (destination)");
    if (n_edges == 0 || c == 0) return JG_OK;
    JG_CHECK_ARG(out && x && idx && off, JG_EINVAL, "scatter_to_edge: null pointer");
    JG_CHECK_ARG(n_nodes > 0, JG_ESHAPE, "scatter_to_edge: edges without nodes");
    JG_CHECK_ARG(n_edges <= INT32_MAX && n_nodes < INT32_MAX, JG_ESHAPE, "scatter_to_edge: sizes beyond int32");
    int lanes_per_row = 0;
    if (c % 4 == 0 && (reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(x)) % 16 == 0) {
        lanes_per_row = 1;
        while (lanes_per_row < 32 && lanes_per_row * 4 < c) lanes_per_row *= 2;
    }
    scatter_to_edge_kernel<<<grid_for_warps((n_edges + 31) / 32), kEdgeBlock, 0, static_cast<cudaStream_t>(stream)>>>(
        out, x, idx, off, n_nodes, n_edges, c, flag, lanes_per_row);
    JG_LAUNCH_CHECK();
    return JG_OK;
}

int jg_edge_to_vertex_f32(float* out, const float* msg, const int32_t* idx, const int32_t* off, int64_t n_nodes,
                          int64_t n_edges, int64_t c, int flag, jg_stream_t stream) {
    JG_CHECK_ARG(n_nodes >= 0 && n_edges >= 0 && c >= 0, JG_EINVAL, "edge_to_vertex: negative size");
    JG_CHECK_ARG(flag == 0 || flag == 1, JG_EINVAL, "edge_to_vertex: flag must be 0 (source) or 1 (destination)");
    if (n_nodes == 0 || c == 0) return JG_OK;
    JG_CHECK_ARG(out && off, JG_EINVAL, "edge_to_vertex: null out/off");
    JG_CHECK_ARG(n_edges == 0 || (msg && idx), JG_EINVAL, "edge_to_vertex: null msg/idx");
    JG_CHECK_ARG(n_edges <= INT32_MAX && n_nodes < INT32_MAX, JG_ESHAPE, "edge_to_vertex: sizes beyond int32");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (flag == 1) {
        edge_to_vertex_dst_kernel<<<grid_for_warps(n_nodes), kEdgeBlock, 0, st>>>(out, msg, off, n_nodes, c);
        JG_LAUNCH_CHECK();
    } else {
        zero_kernel<<<grid_for_warps((n_nodes * c + 31) / 32), kEdgeBlock, 0, st>>>(out, n_nodes * c);
        JG_LAUNCH_CHECK();
        if (n_edges > 0) {
            edge_to_vertex_src_kernel<<<grid_for_warps((n_edges * c + 31) / 32), kEdgeBlock, 0, st>>>(out, msg, idx, n_edges, c);
            JG_LAUNCH_CHECK();
        }
    }
    return JG_OK;
}

int jg_edge_softmax_fwd_f32(float* y, const float* x, const int32_t* off, int64_t n_nodes, int64_t n_edges, int64_t h,
                            jg_stream_t stream) {
    JG_CHECK_ARG(n_nodes >= 0 && n_edges >= 0 && h >= 0, JG_EINVAL, "edge_softmax: negative size");
    if (n_edges == 0 || h == 0 || n_nodes == 0) return JG_OK;
    JG_CHECK_ARG(y && x && off, JG_EINVAL, "edge_softmax: null pointer");
    JG_CHECK_ARG(n_edges * h <= (int64_t)INT32_MAX * 32, JG_ESHAPE, "edge_softmax: sizes too large");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int grid = grid_for_warps(n_nodes);
    const int hub_grid = hub_blocks(n_nodes);
    if ((h == 4 || h == 8 || h == 16 || h == 32) && (reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) % 16 == 0) {
        float4* y4 = reinterpret_cast<float4*>(y);
        const float4* x4 = reinterpret_cast<const float4*>(x);
#define JG_SOFTMAX_VEC(HP) edge_softmax_fwd_vec_kernel<HP><<<hub_grid + grid, kEdgeBlock, 0, st>>>(y4, x4, off, n_nodes, hub_grid)
        if (h == 4) { JG_SOFTMAX_VEC(4); }
        else if (h == 8) { JG_SOFTMAX_VEC(8); }
        else if (h == 16) { JG_SOFTMAX_VEC(16); }
        else { JG_SOFTMAX_VEC(32); }
#undef JG_SOFTMAX_VEC
        JG_LAUNCH_CHECK();
        return JG_OK;
    }
    switch (h) {
        case 1: edge_softmax_fwd_kernel<1><<<grid, kEdgeBlock, 0, st>>>(y, x, off, n_nodes);
                edge_softmax_fwd_hub_kernel<1><<<hub_grid, kEdgeBlock, 0, st>>>(y, x, off, n_nodes); break;
        case 2: edge_softmax_fwd_kernel<2><<<grid, kEdgeBlock, 0, st>>>(y, x, off, n_nodes);
                edge_softmax_fwd_hub_kernel<2><<<hub_grid, kEdgeBlock, 0, st>>>(y, x, off, n_nodes); break;
        case 4: edge_softmax_fwd_kernel<4><<<grid, kEdgeBlock, 0, st>>>(y, x, off, n_nodes);
                edge_softmax_fwd_hub_kernel<4><<<hub_grid, kEdgeBlock, 0, st>>>(y, x, off, n_nodes); break;
        case 8: edge_softmax_fwd_kernel<8><<<grid, kEdgeBlock, 0, st>>>(y, x, off, n_nodes);
                edge_softmax_fwd_hub_kernel<8><<<hub_grid, kEdgeBlock, 0, st>>>(y, x, off, n_nodes); break;
        case 16: edge_softmax_fwd_kernel<16><<<grid, kEdgeBlock, 0, st>>>(y, x, off, n_nodes);
                edge_softmax_fwd_hub_kernel<16><<<hub_grid, kEdgeBlock, 0, st>>>(y, x, off, n_nodes); break;
        case 32: edge_softmax_fwd_kernel<32><<<grid, kEdgeBlock, 0, st>>>(y, x, off, n_nodes);
                edge_softmax_fwd_hub_kernel<32><<<hub_grid, kEdgeBlock, 0, st>>>(y, x, off, n_nodes); break;
        default: edge_softmax_fwd_any_kernel<<<grid_for_warps(n_nodes * h), kEdgeBlock, 0, st>>>(y, x, off, n_nodes, h);
    }
    JG_LAUNCH_CHECK();
    return JG_OK;
}

int jg_edge_softmax_bwd_f32(float* dx, const float* grad, const float* y, const int32_t* off, int64_t n_nodes,
                            int64_t n_edges, int64_t h, jg_stream_t stream) {
    JG_CHECK_ARG(n_nodes >= 0 && n_edges >= 0 && h >= 0, JG_EINVAL, "edge_softmax_bwd: negative size");
    if (n_edges == 0 || h == 0 || n_nodes == 0) return JG_OK;
    JG_CHECK_ARG(dx && grad && y && off, JG_EINVAL, "edge_softmax_bwd: null pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int grid = grid_for_warps(n_nodes);
    const int hub_grid = hub_blocks(n_nodes);
    if ((h == 4 || h == 8 || h == 16 || h == 32) &&
        (reinterpret_cast<uintptr_t>(dx) | reinterpret_cast<uintptr_t>(grad) | reinterpret_cast<uintptr_t>(y)) % 16 == 0) {
        float4* d4 = reinterpret_cast<float4*>(dx);
        const float4* g4 = reinterpret_cast<const float4*>(grad);
        const float4* y4 = reinterpret_cast<const float4*>(y);
#define JG_SOFTMAX_BWD_VEC(HP) edge_softmax_bwd_vec_kernel<HP><<<hub_grid + grid, kEdgeBlock, 0, st>>>(d4, g4, y4, off, n_nodes, hub_grid)
        if (h == 4) { JG_SOFTMAX_BWD_VEC(4); }
        else if (h == 8) { JG_SOFTMAX_BWD_VEC(8); }
        else if (h == 16) { JG_SOFTMAX_BWD_VEC(16); }
        else { JG_SOFTMAX_BWD_VEC(32); }
#undef JG_SOFTMAX_BWD_VEC
        JG_LAUNCH_CHECK();
        return JG_OK;
    }
    switch (h) {
        case 1: edge_softmax_bwd_kernel<1><<<grid, kEdgeBlock, 0, st>>>(dx, grad, y, off, n_nodes);
                 edge_softmax_bwd_hub_kernel<1><<<hub_grid, kEdgeBlock, 0, st>>>(dx, grad, y, off, n_nodes); break;
        case 2: edge_softmax_bwd_kernel<2><<<grid, kEdgeBlock, 0, st>>>(dx, grad, y, off, n_nodes);
                 edge_softmax_bwd_hub_kernel<2><<<hub_grid, kEdgeBlock, 0, st>>>(dx, grad, y, off, n_nodes); break;
        case 4: edge_softmax_bwd_kernel<4><<<grid, kEdgeBlock, 0, st>>>(dx, grad, y, off, n_nodes);
                 edge_softmax_bwd_hub_kernel<4><<<hub_grid, kEdgeBlock, 0, st>>>(dx, grad, y, off, n_nodes); break;
        case 8: edge_softmax_bwd_kernel<8><<<grid, kEdgeBlock, 0, st>>>(dx, grad, y, off, n_nodes);
                 edge_softmax_bwd_hub_kernel<8><<<hub_grid, kEdgeBlock, 0, st>>>(dx, grad, y, off, n_nodes); break;
        case 16: edge_softmax_bwd_kernel<16><<<grid, kEdgeBlock, 0, st>>>(dx, grad, y, off, n_nodes);
                 edge_softmax_bwd_hub_kernel<16><<<hub_grid, kEdgeBlock, 0, st>>>(dx, grad, y, off, n_nodes); break;
        case 32: edge_softmax_bwd_kernel<32><<<grid, kEdgeBlock, 0, st>>>(dx, grad, y, off, n_nodes);
                 edge_softmax_bwd_hub_kernel<32><<<hub_grid, kEdgeBlock, 0, st>>>(dx, grad, y, off, n_nodes); break;
        default: edge_softmax_bwd_any_kernel<<<grid_for_warps(n_nodes * h), kEdgeBlock, 0, st>>>(dx, grad, y, off, n_nodes, h);
    }
    JG_LAUNCH_CHECK();
    return JG_OK;
}


/* Checks a CSR/CSC structure before it is handed to the gather kernels (which trust it).
 * Synchronises the stream.  workspace: 16 bytes. */
int jg_validate_segments(const int32_t* idx, const int32_t* off, int64_t n_out, int64_t n_in, int64_t nnz,
                         void* workspace, size_t workspace_bytes, jg_stream_t stream) {
    JG_CHECK_ARG(n_out >= 0 && n_in >= 0 && nnz >= 0, JG_EINVAL, "validate_segments: negative size");
    JG_CHECK_ARG(off && (nnz == 0 || idx), JG_EINVAL, "validate_segments: null pointer");
    JG_CHECK_ARG(workspace && workspace_bytes >= 16, JG_EWORKSPACE, "validate_segments: workspace of 16 bytes needed");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int32_t* report = static_cast<int32_t*>(workspace);
    JG_CUDA(cudaMemsetAsync(report, 0, 16, st));
    validate_segments_kernel<<<grid_for_warps((n_out + nnz + 31) / 32 + 1), kEdgeBlock, 0, st>>>(idx, off, n_out, n_in, nnz, report);
    JG_LAUNCH_CHECK();
    int32_t host[4] = {0, 0, 0, 0};
    JG_CUDA(cudaMemcpyAsync(host, report, 16, cudaMemcpyDeviceToHost, st));
    JG_CUDA(cudaStreamSynchronize(st));
    if (host[0] || host[1] || host[2] || host[3]) {
        set_error("bad structure: off[0] != 0: %d, off[n] != nnz: %d, decreasing offsets: %d, indices outside [0, %lld): %d",
                  host[0], host[1], host[2], (long long)n_in, host[3]);
        return JG_EINVAL;
    }
    return JG_OK;
}

}  // extern "C"
