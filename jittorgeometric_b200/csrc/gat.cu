// Fused attention aggregation over CSC in-edges (sm_100a): logits, per-destination softmax and
// weighted multi-head aggregation in ONE pass, replacing the reference's six-launch pipeline with
// three [E, C] temporaries (nn/conv/gat_conv.py:67-83: ScatterToEdge x2, concat, matmul,
// leaky_relu, EdgeSoftmax, multiply, ScatterToVertex).
//
//   h      [n, H*D]  transformed node features (after the layer's ReLU)
//   logit(e,hd) = leaky_relu( a_src[hd] . h[src(e),hd,:] + a_dst[hd] . h[dst(e),hd,:] )
//   alpha  = softmax of the logits over the in-edges of each destination, per head
//   out[v,hd,:] = sum_e alpha(e,hd) * h[src(e),hd,:]
//
// One warp per destination (a whole CTA for destinations with 4096 or more in-edges, its warps
// taking alternate tiles and their partial states merged in warp order).  G = C/4 lanes cover one source row with a 128-bit load each, 32/G
// edges are processed side by side.  The source score is recomputed from the gathered row (four
// FMAs and a shuffle) instead of being fetched from a second array: that saves one 32-byte sector
// per edge, and the row has to be read anyway.  The softmax is the running-maximum ("online")
// form, so each source row is read exactly once; lane groups and hub pieces are merged with the
// usual (max, sum, accumulator) rule in a fixed order, so results are run-to-run identical.
// Bound: L2/LSU bandwidth when h fits in L2 (the 233k-node workload: h = 59.6 MB), HBM otherwise;
// per edge one 4 B index and one C*4 B row.
#include "common.cuh"

namespace jg {

constexpr int kGatBlock = 256;
constexpr int kHubBucket = 13;   // degree buckets 13..32: at least 2^12 = 4096 in-edges, walked by a whole CTA

struct GatArgs {
    float* out;
    float* lse;        // [n, H] log2-domain log-sum-exp of each destination's logits, or null
    const float* h;
    const float* a_src;
    const float* a_dst;
    const int32_t* idx;
    const int32_t* off;
    int64_t n;
    float slope;
    unsigned long long* ticket;
    const int32_t* order;      // destinations in processing order (longest segments first), or null
    const int32_t* hub_count;  // [1] how many leading entries of `order` have >= 4096 in-edges
};

// ---- processing order: destinations bucketed by floor(log2(degree)), largest bucket first, so the
// longest segments start earliest and the grid does not end on one warp walking a hub alone.
struct GatPlanView {
    int32_t* counts;   // [64] bucket sizes, then bucket cursors
    int32_t* order;    // [n]
};
__device__ __forceinline__ int degree_bucket(int32_t deg) { return deg <= 0 ? 0 : 32 - __clz(deg); }  // 0..32

__global__ void gat_plan_count_kernel(const int32_t* __restrict__ off, int64_t n, int32_t* counts) {
    __shared__ int s_cnt[33];
    if (threadIdx.x < 33) s_cnt[threadIdx.x] = 0;
    __syncthreads();
    for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < n; v += (int64_t)gridDim.x * blockDim.x)
        atomicAdd(&s_cnt[degree_bucket(off[v + 1] - off[v])], 1);
    __syncthreads();
    if (threadIdx.x < 33 && s_cnt[threadIdx.x]) atomicAdd(&counts[threadIdx.x], s_cnt[threadIdx.x]);
}
// one thread: bucket start positions, largest bucket first
__global__ void gat_plan_starts_kernel(int32_t* counts) {
    int run = 0;
    for (int b = 32; b >= 0; b--) {
        const int c = counts[b];
        counts[b] = run;
        run += c;
        if (b == kHubBucket) counts[40] = run;   // destinations with at least 4096 in-edges
    }
}
__global__ void gat_plan_fill_kernel(const int32_t* __restrict__ off, int64_t n, int32_t* cursors, int32_t* order) {
    for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < n; v += (int64_t)gridDim.x * blockDim.x)
        order[atomicAdd(&cursors[degree_bucket(off[v + 1] - off[v])], 1)] = (int32_t)v;
}

// Segments of 4096 or more entries ("hubs", the first counts[40] entries of `order`) are cut into
// pieces of kGatPiece entries so that a segment of millions of entries is shared by many CTAs:
// piece_start[i] = number of pieces of the hubs before hub i, counts[41] = total.  One block.
constexpr int kGatPiece = 8192;
// floats per piece partial: C column sums, then H score sums padded to a multiple of four so that
// every partial starts on a 16-byte boundary (the column sums are stored as float4)
__host__ __device__ constexpr int piece_stride(int c, int heads) { return c + ((heads + 3) & ~3); }
__global__ void __launch_bounds__(1024) gat_plan_pieces_kernel(const int32_t* __restrict__ off, const int32_t* __restrict__ order,
                                                               int32_t* counts, int32_t* __restrict__ piece_start) {
    __shared__ int s_warp[32];
    __shared__ int s_carry;
    const int n_hub = counts[40];
    if (threadIdx.x == 0) s_carry = 0;
    __syncthreads();
    for (int base = 0; base < n_hub; base += 1024) {
        const int i = base + threadIdx.x;
        int mine = 0;
        if (i < n_hub) {
            const int32_t v = order[i];
            mine = (off[v + 1] - off[v] + kGatPiece - 1) / kGatPiece;
        }
        int incl = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(kFull, incl, o);
            if ((threadIdx.x & 31) >= o) incl += t;
        }
        if ((threadIdx.x & 31) == 31) s_warp[threadIdx.x >> 5] = incl;
        __syncthreads();
        if (threadIdx.x < 32) {
            int w = s_warp[threadIdx.x];
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int t = __shfl_up_sync(kFull, w, o);
                if (threadIdx.x >= o) w += t;
            }
            s_warp[threadIdx.x] = w;
        }
        __syncthreads();
        const int before = s_carry + ((threadIdx.x >> 5) ? s_warp[(threadIdx.x >> 5) - 1] : 0) + incl - mine;
        if (i < n_hub) piece_start[i] = before;
        __syncthreads();
        if (threadIdx.x == 1023) s_carry = before + mine;
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        piece_start[n_hub] = s_carry;
        counts[41] = s_carry;
    }
}

__device__ __forceinline__ float dot4(const float4& a, const float4& b) {
    return fmaf(a.w, b.w, fmaf(a.z, b.z, fmaf(a.y, b.y, a.x * b.x)));
}

struct Softmax4 {
    float m, l;
    float4 acc;
    __device__ __forceinline__ void init() {
        m = -INFINITY;
        l = 0.f;
        acc = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    // one more term with logit z (log2 units) and value row x.  The running maximum rises only a
    // handful of times per segment, so the rescale sits behind a branch and the common path is one
    // exp2 and four FMAs.
    __device__ __forceinline__ void push(float z, const float4& x) {
        if (z > m) {
            const float sc = exp2f(m - z);   // m = -inf at the start: everything accumulated (nothing) scales to 0
            l *= sc;
            acc.x *= sc; acc.y *= sc; acc.z *= sc; acc.w *= sc;
            m = z;
        }
        const float p = exp2f(z - m);
        l += p;
        acc.x = fmaf(p, x.x, acc.x);
        acc.y = fmaf(p, x.y, acc.y);
        acc.z = fmaf(p, x.z, acc.z);
        acc.w = fmaf(p, x.w, acc.w);
    }
    // merge another partial state (either may be empty: m == -inf, l == 0)
    __device__ __forceinline__ void merge(float m2, float l2, const float4& a2) {
        const float mn = fmaxf(m, m2);
        const float s1 = (m == -INFINITY) ? 0.f : exp2f(m - mn);
        const float s2 = (m2 == -INFINITY) ? 0.f : exp2f(m2 - mn);
        l = l * s1 + l2 * s2;
        acc.x = acc.x * s1 + a2.x * s2;
        acc.y = acc.y * s1 + a2.y * s2;
        acc.z = acc.z * s1 + a2.z * s2;
        acc.w = acc.w * s1 + a2.w * s2;
        m = mn;
    }
};

// G lanes per row (C = 4*G), DL = D/4 lanes per head; both powers of two, DL <= G <= 32.
// Walks the 32-edge tiles first_tile, first_tile + tile_stride, ... of segment [s, e).
template <int G, int DL>
__device__ __forceinline__ void gat_walk(const GatArgs& a, int32_t s, int32_t e, int first_tile, int tile_stride,
                                         const float4& as4, float sd, const char* hb, Softmax4& st) {
    constexpr int EPS = 32 / G;
    constexpr int C = 4 * G;
    constexpr int B = 4;  // steps per batch
    const int lane = lane_id();
    const int sub = lane / G;
    for (int64_t j0 = (int64_t)s + 32 * (int64_t)first_tile; j0 < e; j0 += 32 * (int64_t)tile_stride) {
        int my_idx = 0;
        if (j0 + lane < e) my_idx = ld_stream(a.idx + j0 + lane);
        const int cnt = (int)((e - j0) < 32 ? (e - j0) : 32);
        for (int tt = 0; tt < cnt; tt += EPS * B) {
            float4 x[B];
            bool ok[B];
#pragma unroll
            for (int u = 0; u < B; u++) {
                const int k = tt + u * EPS + sub;
                const int src = __shfl_sync(kFull, my_idx, k & 31);
                ok[u] = k < cnt;
                x[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (ok[u]) x[u] = __ldg(reinterpret_cast<const float4*>(hb + (size_t)(unsigned)src * (C * 4)));
            }
#pragma unroll
            for (int u = 0; u < B; u++) {
                float ss = dot4(x[u], as4);
#pragma unroll
                for (int o = 1; o < DL; o <<= 1) ss += __shfl_xor_sync(kFull, ss, o);
                float z = ss + sd;
                z = fmaxf(z, z * a.slope);   // leaky_relu for a slope in [0, 1]
                if (ok[u]) st.push(z, x[u]);
            }
        }
    }
}

// Merges the lane groups that took alternate edges (fixed order) and writes the output row.
template <int G, int DL>
__device__ __forceinline__ void gat_finish(const GatArgs& a, int64_t v, Softmax4& st) {
    constexpr int C = 4 * G;
    const int lane = lane_id();
    const int sub = lane / G, fl = lane % G;
#pragma unroll
    for (int o = G; o < 32; o <<= 1) {
        const float m2 = __shfl_xor_sync(kFull, st.m, o);
        const float l2 = __shfl_xor_sync(kFull, st.l, o);
        float4 a2;
        a2.x = __shfl_xor_sync(kFull, st.acc.x, o);
        a2.y = __shfl_xor_sync(kFull, st.acc.y, o);
        a2.z = __shfl_xor_sync(kFull, st.acc.z, o);
        a2.w = __shfl_xor_sync(kFull, st.acc.w, o);
        // both partners apply the merge in the same operand order, so they agree bit for bit
        if (lane & o) {
            Softmax4 other;
            other.m = m2; other.l = l2; other.acc = a2;
            other.merge(st.m, st.l, st.acc);
            st = other;
        } else {
            st.merge(m2, l2, a2);
        }
    }
    if (sub == 0) {
        const float inv = st.l > 0.f ? 1.f / st.l : 0.f;
        __stcs(reinterpret_cast<float4*>(a.out + (size_t)v * C) + fl,
               make_float4(st.acc.x * inv, st.acc.y * inv, st.acc.z * inv, st.acc.w * inv));
        if (a.lse && fl % DL == 0) a.lse[(size_t)v * (G / DL) + fl / DL] = st.l > 0.f ? st.m + log2f(st.l) : 0.f;
    }
}

template <int G, int DL>
__global__ void __launch_bounds__(kGatBlock) gat_aggregate_kernel(GatArgs a) {
    constexpr int C = 4 * G;
    constexpr int W = kGatBlock / 32;
    __shared__ float s_state[W][32][6];
    __shared__ unsigned long long s_ticket;
    const int lane = lane_id();
    const int warp = threadIdx.x / 32;
    const int fl = lane % G;
    // attention vectors scaled by log2(e): the positive factor commutes with leaky_relu, and the
    // softmax can then use exp2 directly
    constexpr float kLog2e = 1.4426950408889634f;
    float4 as4 = __ldg(reinterpret_cast<const float4*>(a.a_src) + fl);
    float4 ad4 = __ldg(reinterpret_cast<const float4*>(a.a_dst) + fl);
    as4.x *= kLog2e; as4.y *= kLog2e; as4.z *= kLog2e; as4.w *= kLog2e;
    ad4.x *= kLog2e; ad4.y *= kLog2e; ad4.z *= kLog2e; ad4.w *= kLog2e;
    const char* hb = reinterpret_cast<const char*>(a.h) + fl * 16;
    const int64_t n_hub = a.order ? (int64_t)a.hub_count[0] : 0;

    // ---- hubs: one CTA per destination, its warps take alternate 32-edge tiles
    for (;;) {
        __syncthreads();
        if (threadIdx.x == 0) s_ticket = atomicAdd(a.ticket + 1, 1ull);
        __syncthreads();
        const unsigned long long t = s_ticket;
        if ((int64_t)t >= n_hub) break;
        const int64_t v = a.order[t];
        const int32_t s = a.off[v], e = a.off[v + 1];
        const float4 hv = __ldg(reinterpret_cast<const float4*>(hb + (size_t)v * (C * 4)));
        float sd = dot4(hv, ad4);
#pragma unroll
        for (int o = 1; o < DL; o <<= 1) sd += __shfl_xor_sync(kFull, sd, o);
        Softmax4 st;
        st.init();
        gat_walk<G, DL>(a, s, e, warp, W, as4, sd, hb, st);
        float* mine = s_state[warp][lane];
        mine[0] = st.m; mine[1] = st.l; mine[2] = st.acc.x; mine[3] = st.acc.y; mine[4] = st.acc.z; mine[5] = st.acc.w;
        __syncthreads();
        if (warp == 0) {
            for (int w = 1; w < W; w++) {   // fixed order: warp 0's state, then 1, 2, ...
                const float* o = s_state[w][lane];
                st.merge(o[0], o[1], make_float4(o[2], o[3], o[4], o[5]));
            }
            gat_finish<G, DL>(a, v, st);
        }
    }
    // ---- everything else: one warp per destination
    for (;;) {
        unsigned long long t = 0;
        if (lane == 0) t = atomicAdd(a.ticket, 1ull);
        t = __shfl_sync(kFull, t, 0) + (unsigned long long)n_hub;
        if ((int64_t)t >= a.n) break;
        const int64_t v = a.order ? (int64_t)a.order[t] : (int64_t)t;
        const int32_t s = a.off[v], e = a.off[v + 1];
        const float4 hv = __ldg(reinterpret_cast<const float4*>(hb + (size_t)v * (C * 4)));
        float sd = dot4(hv, ad4);
#pragma unroll
        for (int o = 1; o < DL; o <<= 1) sd += __shfl_xor_sync(kFull, sd, o);
        Softmax4 st;
        st.init();
        gat_walk<G, DL>(a, s, e, 0, 1, as4, sd, hb, st);
        gat_finish<G, DL>(a, v, st);
    }
}

// Persistent grid, but never more warps than segments: every warp takes at least one ticket, and on a
// small graph (a sampled mini-batch) a full grid would mostly queue on the ticket counter.
static unsigned gat_grid(int64_t n_segments, int blocks_per_sm) {
    int64_t blocks = (n_segments + kGatBlock / 32 - 1) / (kGatBlock / 32);
    const int64_t full = (int64_t)sm_count() * blocks_per_sm;
    if (blocks > full) blocks = full;
    return (unsigned)(blocks > 0 ? blocks : 1);
}

template <int G, int DL>
static int launch_gat(const GatArgs& a, cudaStream_t st) {
    static int blocks_per_sm = 0;
    auto kern = gat_aggregate_kernel<G, DL>;
    if (blocks_per_sm == 0) {
        int b = 0;
        JG_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&b, kern, kGatBlock, 0));
        blocks_per_sm = b > 0 ? b : 1;
    }
    kern<<<gat_grid(a.n, blocks_per_sm), kGatBlock, 0, st>>>(a);
    JG_LAUNCH_CHECK();
    return JG_OK;
}

template <int G>
static int launch_gat_g(int dl, const GatArgs& a, cudaStream_t st) {
    switch (dl) {
        case 1: return launch_gat<G, 1>(a, st);
        case 2: if constexpr (G >= 2) return launch_gat<G, 2>(a, st); break;
        case 4: if constexpr (G >= 4) return launch_gat<G, 4>(a, st); break;
        case 8: if constexpr (G >= 8) return launch_gat<G, 8>(a, st); break;
        case 16: if constexpr (G >= 16) return launch_gat<G, 16>(a, st); break;
        case 32: if constexpr (G >= 32) return launch_gat<G, 32>(a, st); break;
    }
    return JG_EUNSUPPORTED;
}

// ------------------------------------------------------------------------------ backward
// With alpha(e) = exp2(z2(e) - lse2[v]) rebuilt from the saved log-sum-exp, g = grad_out and
// delta[v,hd] = g[v,hd,:] . out[v,hd,:] (= sum_e alpha(e) * dalpha(e)):
//   dalpha(e) = g[v,hd,:] . h[src(e),hd,:]
//   dpre(e)   = alpha(e) * (dalpha(e) - delta[v,hd]) * (pre(e) > 0 ? 1 : slope)
//   d_dst[v,hd] = sum over in-edges of v of dpre(e)           (pass 1, by destination over CSC)
//   d_src[u,hd] = sum over out-edges of u of dpre(e)          (pass 2, by source over the transpose)
//   grad_h[u,hd,:] = sum over out-edges alpha(e) * g[dst(e),hd,:] + d_src[u,hd]*a_src[hd] + d_dst[u,hd]*a_dst[hd]
//   grad_a_src[hd,:] = sum_u d_src[u,hd] * h[u,hd,:],  grad_a_dst likewise with d_dst   (pass 3)
// Every sum is a gather in a fixed order: no atomics on data, run-to-run identical results.
struct GatBwdArgs {
    float* grad_h;
    const float* grad_out;
    const float* out;
    const float* lse;
    const float* h;
    const float* a_src;
    const float* a_dst;
    const int32_t* idx;        // CSC: sources of each destination's in-edges
    const int32_t* off;
    const int32_t* idx_t;      // transpose: destinations of each source's out-edges
    const int32_t* off_t;
    int64_t n;
    float slope;
    unsigned long long* ticket;   // [4]
    const int32_t* order;
    const int32_t* hub_count;
    const int32_t* order_t;
    const int32_t* hub_count_t;
    float4* info;     // [n, H]: (a_dst . h[v] in log2 units, lse2[v], delta[v], 0)
    float* d_dst;     // [n, H]
    float* d_src;     // [n, H]
    const int32_t* piece_start_t;   // pieces of the hub sources (see gat_plan_pieces_kernel)
    const int32_t* n_pieces_t;      // [1]
    float* piece_partial;           // [pieces, piece_stride] partial sums of multi-piece hubs
};

template <int DL>
__device__ __forceinline__ void reduce_head2(float& a, float& b) {
#pragma unroll
    for (int o = 1; o < DL; o <<= 1) {
        a += __shfl_xor_sync(kFull, a, o);
        b += __shfl_xor_sync(kFull, b, o);
    }
}

// pass 1 walk: sum of dpre over tiles first_tile, first_tile + tile_stride, ... of [s, e)
template <int G, int DL>
__device__ __forceinline__ float gat_bwd_dst_walk(const GatBwdArgs& a, int32_t s, int32_t e, int first_tile, int tile_stride,
                                                  const float4& as4, float sd, const float4& gv, float lse2, float delta,
                                                  const char* hb) {
    constexpr int EPS = 32 / G;
    constexpr int C = 4 * G;
    constexpr int B = 4;
    const int lane = lane_id();
    const int sub = lane / G;
    float acc = 0.f;
    for (int64_t j0 = (int64_t)s + 32 * (int64_t)first_tile; j0 < e; j0 += 32 * (int64_t)tile_stride) {
        int my_idx = 0;
        if (j0 + lane < e) my_idx = ld_stream(a.idx + j0 + lane);
        const int cnt = (int)((e - j0) < 32 ? (e - j0) : 32);
        for (int tt = 0; tt < cnt; tt += EPS * B) {
            float4 x[B];
            bool ok[B];
#pragma unroll
            for (int u = 0; u < B; u++) {
                const int k = tt + u * EPS + sub;
                const int src = __shfl_sync(kFull, my_idx, k & 31);
                ok[u] = k < cnt;
                x[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (ok[u]) x[u] = __ldg(reinterpret_cast<const float4*>(hb + (size_t)(unsigned)src * (C * 4)));
            }
#pragma unroll
            for (int u = 0; u < B; u++) {
                float ss = dot4(x[u], as4);
                float da = dot4(x[u], gv);
                reduce_head2<DL>(ss, da);
                const float pre = ss + sd;
                const float z = fmaxf(pre, pre * a.slope);
                const float t = exp2f(z - lse2) * (da - delta);
                if (ok[u]) acc += pre > 0.f ? t : t * a.slope;
            }
        }
    }
    return acc;
}

template <int G, int DL>
__global__ void __launch_bounds__(kGatBlock) gat_backward_dst_kernel(GatBwdArgs a) {
    constexpr int C = 4 * G;
    constexpr int H = G / DL;
    constexpr int W = kGatBlock / 32;
    __shared__ float s_part[W][32];
    __shared__ unsigned long long s_ticket;
    const int lane = lane_id();
    const int warp = threadIdx.x / 32;
    const int fl = lane % G;
    constexpr float kLog2e = 1.4426950408889634f;
    float4 as4 = __ldg(reinterpret_cast<const float4*>(a.a_src) + fl);
    float4 ad4 = __ldg(reinterpret_cast<const float4*>(a.a_dst) + fl);
    as4.x *= kLog2e; as4.y *= kLog2e; as4.z *= kLog2e; as4.w *= kLog2e;
    ad4.x *= kLog2e; ad4.y *= kLog2e; ad4.z *= kLog2e; ad4.w *= kLog2e;
    const char* hb = reinterpret_cast<const char*>(a.h) + fl * 16;
    const int64_t n_hub = a.order ? (int64_t)a.hub_count[0] : 0;

    auto own = [&](int64_t v, float& sd, float4& gv, float& lse2, float& delta) {
        const float4 hv = __ldg(reinterpret_cast<const float4*>(hb + (size_t)v * (C * 4)));
        gv = __ldg(reinterpret_cast<const float4*>(a.grad_out + (size_t)v * C) + fl);
        const float4 ov = __ldg(reinterpret_cast<const float4*>(a.out + (size_t)v * C) + fl);
        sd = dot4(hv, ad4);
        delta = dot4(gv, ov);
        reduce_head2<DL>(sd, delta);
        lse2 = __ldg(a.lse + (size_t)v * H + fl / DL);
    };
    auto finish = [&](int64_t v, float acc, float sd, float lse2, float delta) {
        // lane groups took alternate edges: butterfly sum (both partners add the same two values)
#pragma unroll
        for (int o = G; o < 32; o <<= 1) acc += __shfl_xor_sync(kFull, acc, o);
        if (lane < G && fl % DL == 0) {
            a.d_dst[(size_t)v * H + fl / DL] = acc;
            a.info[(size_t)v * H + fl / DL] = make_float4(sd, lse2, delta, 0.f);
        }
    };

    for (;;) {   // hubs: one CTA per destination
        __syncthreads();
        if (threadIdx.x == 0) s_ticket = atomicAdd(a.ticket + 1, 1ull);
        __syncthreads();
        const unsigned long long t = s_ticket;
        if ((int64_t)t >= n_hub) break;
        const int64_t v = a.order[t];
        float sd, lse2, delta;
        float4 gv;
        own(v, sd, gv, lse2, delta);
        float acc = gat_bwd_dst_walk<G, DL>(a, a.off[v], a.off[v + 1], warp, W, as4, sd, gv, lse2, delta, hb);
        s_part[warp][lane] = acc;
        __syncthreads();
        if (warp == 0) {
            for (int w = 1; w < W; w++) acc += s_part[w][lane];   // fixed order
            finish(v, acc, sd, lse2, delta);
        }
    }
    for (;;) {   // one warp per destination
        unsigned long long t = 0;
        if (lane == 0) t = atomicAdd(a.ticket, 1ull);
        t = __shfl_sync(kFull, t, 0) + (unsigned long long)n_hub;
        if ((int64_t)t >= a.n) break;
        const int64_t v = a.order ? (int64_t)a.order[t] : (int64_t)t;
        float sd, lse2, delta;
        float4 gv;
        own(v, sd, gv, lse2, delta);
        const float acc = gat_bwd_dst_walk<G, DL>(a, a.off[v], a.off[v + 1], 0, 1, as4, sd, gv, lse2, delta, hb);
        finish(v, acc, sd, lse2, delta);
    }
}

struct GatSrcAcc {
    float s;
    float4 g;
};

// pass 2 walk over the out-edges of one source
template <int G, int DL>
__device__ __forceinline__ void gat_bwd_src_walk(const GatBwdArgs& a, int32_t s, int32_t e, int first_tile, int tile_stride,
                                                 const float4& hu, float ss, const char* gb, const float4* info,
                                                 GatSrcAcc& acc) {
    constexpr int EPS = 32 / G;
    constexpr int C = 4 * G;
    constexpr int H = G / DL;
    constexpr int B = 4;
    const int lane = lane_id();
    const int sub = lane / G;
    for (int64_t j0 = (int64_t)s + 32 * (int64_t)first_tile; j0 < e; j0 += 32 * (int64_t)tile_stride) {
        int my_idx = 0;
        if (j0 + lane < e) my_idx = ld_stream(a.idx_t + j0 + lane);
        const int cnt = (int)((e - j0) < 32 ? (e - j0) : 32);
        for (int tt = 0; tt < cnt; tt += EPS * B) {
            float4 gq[B], inf[B];
            bool ok[B];
#pragma unroll
            for (int u = 0; u < B; u++) {
                const int k = tt + u * EPS + sub;
                const int dst = __shfl_sync(kFull, my_idx, k & 31);
                ok[u] = k < cnt;
                gq[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                inf[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (ok[u]) {
                    gq[u] = __ldg(reinterpret_cast<const float4*>(gb + (size_t)(unsigned)dst * (C * 4)));
                    inf[u] = __ldg(info + (size_t)(unsigned)dst * H);
                }
            }
#pragma unroll
            for (int u = 0; u < B; u++) {
                float da = dot4(hu, gq[u]);
#pragma unroll
                for (int o = 1; o < DL; o <<= 1) da += __shfl_xor_sync(kFull, da, o);
                const float pre = ss + inf[u].x;
                const float z = fmaxf(pre, pre * a.slope);
                const float alpha = ok[u] ? exp2f(z - inf[u].y) : 0.f;
                const float t = alpha * (da - inf[u].z);
                acc.s += pre > 0.f ? t : t * a.slope;
                acc.g.x = fmaf(alpha, gq[u].x, acc.g.x);
                acc.g.y = fmaf(alpha, gq[u].y, acc.g.y);
                acc.g.z = fmaf(alpha, gq[u].z, acc.g.z);
                acc.g.w = fmaf(alpha, gq[u].w, acc.g.w);
            }
        }
    }
}

template <int G, int DL>
__global__ void __launch_bounds__(kGatBlock) gat_backward_src_kernel(GatBwdArgs a) {
    constexpr int C = 4 * G;
    constexpr int H = G / DL;
    constexpr int W = kGatBlock / 32;
    __shared__ float s_part[W][32][5];
    __shared__ unsigned long long s_ticket;
    const int lane = lane_id();
    const int warp = threadIdx.x / 32;
    const int fl = lane % G;
    constexpr float kLog2e = 1.4426950408889634f;
    const float4 as_raw = __ldg(reinterpret_cast<const float4*>(a.a_src) + fl);
    const float4 as4 = make_float4(as_raw.x * kLog2e, as_raw.y * kLog2e, as_raw.z * kLog2e, as_raw.w * kLog2e);
    const char* hb = reinterpret_cast<const char*>(a.h) + fl * 16;
    const char* gb = reinterpret_cast<const char*>(a.grad_out) + fl * 16;
    const float4* info = a.info + fl / DL;
    const int64_t n_hub = a.order_t ? (int64_t)a.hub_count_t[0] : 0;

    auto own = [&](int64_t u, float4& hu, float& ss) {
        hu = __ldg(reinterpret_cast<const float4*>(hb + (size_t)u * (C * 4)));
        ss = dot4(hu, as4);
#pragma unroll
        for (int o = 1; o < DL; o <<= 1) ss += __shfl_xor_sync(kFull, ss, o);
    };
    auto fold = [&](GatSrcAcc& acc) {   // lane groups took alternate edges: butterfly sums
#pragma unroll
        for (int o = G; o < 32; o <<= 1) {
            acc.s += __shfl_xor_sync(kFull, acc.s, o);
            acc.g.x += __shfl_xor_sync(kFull, acc.g.x, o);
            acc.g.y += __shfl_xor_sync(kFull, acc.g.y, o);
            acc.g.z += __shfl_xor_sync(kFull, acc.g.z, o);
            acc.g.w += __shfl_xor_sync(kFull, acc.g.w, o);
        }
    };
    auto finish = [&](int64_t u, const GatSrcAcc& acc) {
        if (lane < G) {
            const float4 ad_raw = __ldg(reinterpret_cast<const float4*>(a.a_dst) + fl);
            const float dd = a.d_dst[(size_t)u * H + fl / DL];
            float4 r;
            r.x = acc.g.x + acc.s * as_raw.x + dd * ad_raw.x;
            r.y = acc.g.y + acc.s * as_raw.y + dd * ad_raw.y;
            r.z = acc.g.z + acc.s * as_raw.z + dd * ad_raw.z;
            r.w = acc.g.w + acc.s * as_raw.w + dd * ad_raw.w;
            __stcs(reinterpret_cast<float4*>(a.grad_h + (size_t)u * C) + fl, r);
            if (fl % DL == 0) a.d_src[(size_t)u * H + fl / DL] = acc.s;
        }
    };

    // hub sources: one CTA per piece of kGatPiece out-edges
    const int64_t n_piece = a.order_t ? (int64_t)a.n_pieces_t[0] : 0;
    __shared__ int s_hub;
    for (;;) {
        __syncthreads();
        if (threadIdx.x == 0) {
            const unsigned long long t = atomicAdd(a.ticket + 3, 1ull);
            s_ticket = t;
            if ((int64_t)t < n_piece) {   // the hub whose piece range holds t: last i with piece_start[i] <= t
                int lo = 0, hi = (int)n_hub;
                while (hi - lo > 1) {
                    const int mid = (lo + hi) >> 1;
                    if ((unsigned long long)a.piece_start_t[mid] <= t) lo = mid; else hi = mid;
                }
                s_hub = lo;
            }
        }
        __syncthreads();
        const unsigned long long t = s_ticket;
        if ((int64_t)t >= n_piece) break;
        const int hub = s_hub;
        const int first = a.piece_start_t[hub];
        const int pieces = a.piece_start_t[hub + 1] - first;
        const int64_t u = a.order_t[hub];
        const int64_t s0 = (int64_t)a.off_t[u] + (int64_t)((int)t - first) * kGatPiece;
        const int64_t e_all = a.off_t[u + 1];
        const int64_t e0 = s0 + kGatPiece < e_all ? s0 + kGatPiece : e_all;
        float4 hu;
        float ss;
        own(u, hu, ss);
        GatSrcAcc acc = {0.f, make_float4(0.f, 0.f, 0.f, 0.f)};
        gat_bwd_src_walk<G, DL>(a, (int32_t)s0, (int32_t)e0, warp, W, hu, ss, gb, info, acc);
        float* mine = s_part[warp][lane];
        mine[0] = acc.s; mine[1] = acc.g.x; mine[2] = acc.g.y; mine[3] = acc.g.z; mine[4] = acc.g.w;
        __syncthreads();
        if (warp == 0) {
            for (int w = 1; w < W; w++) {   // fixed order
                const float* o = s_part[w][lane];
                acc.s += o[0]; acc.g.x += o[1]; acc.g.y += o[2]; acc.g.z += o[3]; acc.g.w += o[4];
            }
            fold(acc);
            if (pieces == 1) {
                finish(u, acc);
            } else if (lane < G) {   // partial of this piece; gat_backward_src_fixup_kernel adds the pieces up
                float* dst = a.piece_partial + (size_t)t * piece_stride(C, H);
                reinterpret_cast<float4*>(dst)[fl] = acc.g;
                if (fl % DL == 0) dst[C + fl / DL] = acc.s;
            }
        }
    }
    for (;;) {   // one warp per source
        unsigned long long t = 0;
        if (lane == 0) t = atomicAdd(a.ticket + 2, 1ull);
        t = __shfl_sync(kFull, t, 0) + (unsigned long long)n_hub;
        if ((int64_t)t >= a.n) break;
        const int64_t u = a.order_t ? (int64_t)a.order_t[t] : (int64_t)t;
        float4 hu;
        float ss;
        own(u, hu, ss);
        GatSrcAcc acc = {0.f, make_float4(0.f, 0.f, 0.f, 0.f)};
        gat_bwd_src_walk<G, DL>(a, a.off_t[u], a.off_t[u + 1], 0, 1, hu, ss, gb, info, acc);
        fold(acc);
        finish(u, acc);
    }
}

// Sums the piece partials of every multi-piece hub source in piece order and writes its rows.
// One block per hub (grid-stride), one thread per column.
__global__ void __launch_bounds__(128) gat_backward_src_fixup_kernel(GatBwdArgs a, int c, int d) {
    const int heads = c / d;
    const int n_hub = a.hub_count_t[0];
    const int col = threadIdx.x;
    if (col >= c) return;
    const int head = col / d;
    for (int hub = blockIdx.x; hub < n_hub; hub += gridDim.x) {
        const int first = a.piece_start_t[hub];
        const int pieces = a.piece_start_t[hub + 1] - first;
        if (pieces <= 1) continue;
        const int64_t u = a.order_t[hub];
        float g = 0.f, sc = 0.f;
        for (int p = 0; p < pieces; p++) {
            const float* src = a.piece_partial + (size_t)(first + p) * piece_stride(c, heads);
            g += src[col];
            sc += src[c + head];
        }
        const float dd = a.d_dst[(size_t)u * heads + head];
        a.grad_h[(size_t)u * c + col] = g + sc * a.a_src[col] + dd * a.a_dst[col];
        if (col % d == 0) a.d_src[(size_t)u * heads + head] = sc;
    }
}

// pass 3: partial[b][0][c] = sum over the block's rows of d_src[r, c/D] * h[r, c]; [b][1][c] with d_dst.
// Rows are dealt to (block, slot) round-robin and summed in ascending order; slots and blocks are
// then combined in index order, so the result does not depend on scheduling.
constexpr int kScoreGradThreads = 256;
__global__ void __launch_bounds__(kScoreGradThreads) gat_score_grad_partial_kernel(const float* __restrict__ h,
                                                                                   const float* __restrict__ d_src,
                                                                                   const float* __restrict__ d_dst, int64_t n,
                                                                                   int c, int d, float* __restrict__ partial) {
    __shared__ float s_a[kScoreGradThreads], s_b[kScoreGradThreads];
    const int slots = kScoreGradThreads / c;
    const int col = threadIdx.x % c, slot = threadIdx.x / c;
    const int heads = c / d;
    float acc_s = 0.f, acc_d = 0.f;
    if (slot < slots) {
        for (int64_t r = (int64_t)blockIdx.x * slots + slot; r < n; r += (int64_t)gridDim.x * slots) {
            const float x = h[(size_t)r * c + col];
            acc_s = fmaf(d_src[(size_t)r * heads + col / d], x, acc_s);
            acc_d = fmaf(d_dst[(size_t)r * heads + col / d], x, acc_d);
        }
    }
    s_a[threadIdx.x] = acc_s;
    s_b[threadIdx.x] = acc_d;
    __syncthreads();
    if (threadIdx.x < c) {
        for (int k = 1; k < slots; k++) {
            acc_s += s_a[k * c + col];
            acc_d += s_b[k * c + col];
        }
        partial[((size_t)blockIdx.x * 2 + 0) * c + col] = acc_s;
        partial[((size_t)blockIdx.x * 2 + 1) * c + col] = acc_d;
    }
}

__global__ void gat_score_grad_final_kernel(const float* __restrict__ partial, int blocks, int c, float* __restrict__ grad_a_src,
                                            float* __restrict__ grad_a_dst) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= 2 * c) return;
    const int which = t / c, col = t % c;
    float acc = 0.f;
    for (int b = 0; b < blocks; b++) acc += partial[((size_t)b * 2 + which) * c + col];
    (which ? grad_a_dst : grad_a_src)[col] = acc;
}

struct GatBwdWs {
    unsigned long long* ticket;
    float4* info;
    float* d_dst;
    float* d_src;
    float* partial;
    float* piece_partial;
    int blocks;
    size_t bytes;
};
// upper bound on the pieces of all hubs: every hub has at least 4096 entries, every piece but a
// hub's last is full
static int64_t max_pieces(int64_t n_edges) { return n_edges / kGatPiece + n_edges / 4096 + 1; }

static GatBwdWs carve_gat_bwd(void* ws, int64_t n, int64_t n_edges, int64_t heads, int64_t c, int blocks) {
    Carver cv(ws);
    GatBwdWs v;
    v.piece_partial = cv.take<float>((size_t)max_pieces(n_edges) * (size_t)piece_stride((int)c, (int)heads));
    v.ticket = cv.take<unsigned long long>(4);
    v.info = cv.take<float4>((size_t)n * heads);
    v.d_dst = cv.take<float>((size_t)n * heads);
    v.d_src = cv.take<float>((size_t)n * heads);
    v.partial = cv.take<float>((size_t)blocks * 2 * c);
    v.blocks = blocks;
    v.bytes = cv.total();
    return v;
}
constexpr int kScoreGradBlocks = 296;   // two per SM on a 148-SM part; only sets the partial count

template <int G, int DL>
static int launch_gat_bwd(const GatBwdArgs& a, cudaStream_t st) {
    static int bps_dst = 0, bps_src = 0;
    auto k1 = gat_backward_dst_kernel<G, DL>;
    auto k2 = gat_backward_src_kernel<G, DL>;
    if (bps_dst == 0) {
        int b = 0;
        JG_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&b, k1, kGatBlock, 0));
        bps_dst = b > 0 ? b : 1;
        JG_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&b, k2, kGatBlock, 0));
        bps_src = b > 0 ? b : 1;
    }
    k1<<<gat_grid(a.n, bps_dst), kGatBlock, 0, st>>>(a);
    JG_LAUNCH_CHECK();
    k2<<<gat_grid(a.n, bps_src), kGatBlock, 0, st>>>(a);
    JG_LAUNCH_CHECK();
    if (a.order_t) {
        gat_backward_src_fixup_kernel<<<sm_count() * 2, 128, 0, st>>>(a, 4 * G, 4 * DL);
        JG_LAUNCH_CHECK();
    }
    return JG_OK;
}

template <int G>
static int launch_gat_bwd_g(int dl, const GatBwdArgs& a, cudaStream_t st) {
    switch (dl) {
        case 1: return launch_gat_bwd<G, 1>(a, st);
        case 2: if constexpr (G >= 2) return launch_gat_bwd<G, 2>(a, st); break;
        case 4: if constexpr (G >= 4) return launch_gat_bwd<G, 4>(a, st); break;
        case 8: if constexpr (G >= 8) return launch_gat_bwd<G, 8>(a, st); break;
        case 16: if constexpr (G >= 16) return launch_gat_bwd<G, 16>(a, st); break;
        case 32: if constexpr (G >= 32) return launch_gat_bwd<G, 32>(a, st); break;
    }
    return JG_EUNSUPPORTED;
}

}  // namespace jg

using namespace jg;

extern "C" {

size_t jg_gat_plan_bytes(int64_t n_nodes) {
    if (n_nodes < 0) return 0;
    Carver c(nullptr);
    c.take<int32_t>(64);
    c.take<int32_t>(n_nodes);
    c.take<int32_t>(n_nodes + 1);
    return c.total();
}

int jg_gat_plan_build(const int32_t* off, int64_t n_nodes, void* plan, size_t plan_bytes, jg_stream_t stream) {
    JG_CHECK_ARG(off && plan && n_nodes >= 0, JG_EINVAL, "gat_plan_build: bad argument");
    JG_CHECK_ARG(plan_bytes >= jg_gat_plan_bytes(n_nodes), JG_EWORKSPACE, "gat_plan_build: plan buffer too small");
    JG_CHECK_ARG(n_nodes < INT32_MAX, JG_ESHAPE, "gat_plan_build: sizes beyond int32");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    Carver c(plan);
    int32_t* counts = c.take<int32_t>(64);
    int32_t* order = c.take<int32_t>(n_nodes);
    int32_t* piece_start = c.take<int32_t>(n_nodes + 1);
    JG_CUDA(cudaMemsetAsync(counts, 0, 64 * sizeof(int32_t), st));
    if (n_nodes == 0) return JG_OK;
    const int grid = sm_count() * 4;
    gat_plan_count_kernel<<<grid, 256, 0, st>>>(off, n_nodes, counts);
    JG_LAUNCH_CHECK();
    gat_plan_starts_kernel<<<1, 1, 0, st>>>(counts);
    JG_LAUNCH_CHECK();
    gat_plan_fill_kernel<<<grid, 256, 0, st>>>(off, n_nodes, counts, order);
    JG_LAUNCH_CHECK();
    gat_plan_pieces_kernel<<<1, 1024, 0, st>>>(off, order, counts, piece_start);
    JG_LAUNCH_CHECK();
    return JG_OK;
}

size_t jg_gat_aggregate_workspace_bytes(int64_t n_nodes, int64_t n_edges, int64_t heads, int64_t dim) {
    (void)n_nodes; (void)n_edges; (void)heads; (void)dim;
    return 256;
}

int jg_gat_aggregate_supported(int64_t heads, int64_t dim) {
    if (heads <= 0 || dim <= 0 || dim % 4) return 0;
    const int64_t g = heads * dim / 4, dl = dim / 4;
    auto pow2 = [](int64_t v) { return v > 0 && (v & (v - 1)) == 0; };
    return pow2(g) && pow2(dl) && g <= 32;
}

int jg_gat_aggregate_f32(float* out, float* lse, const float* h, const float* a_src, const float* a_dst, const int32_t* idx,
                         const int32_t* off, int64_t n_nodes, int64_t n_edges, int64_t heads, int64_t dim, float slope,
                         const void* plan, void* workspace, size_t workspace_bytes, jg_stream_t stream) {
    JG_CHECK_ARG(n_nodes >= 0 && n_edges >= 0 && heads > 0 && dim > 0, JG_EINVAL, "gat_aggregate: bad size");
    if (n_nodes == 0) return JG_OK;
    JG_CHECK_ARG(out && h && a_src && a_dst && off, JG_EINVAL, "gat_aggregate: null pointer");
    JG_CHECK_ARG(n_edges == 0 || idx, JG_EINVAL, "gat_aggregate: null idx");
    JG_CHECK_ARG(n_edges <= INT32_MAX && n_nodes < INT32_MAX, JG_ESHAPE, "gat_aggregate: sizes beyond int32");
    if (!jg_gat_aggregate_supported(heads, dim)) {
        set_error("gat_aggregate: heads*dim/4 and dim/4 must be powers of two with heads*dim <= 128 (got %lld x %lld)",
                  (long long)heads, (long long)dim);
        return JG_EUNSUPPORTED;
    }
    JG_CHECK_ARG((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(h) | reinterpret_cast<uintptr_t>(a_src) |
                  reinterpret_cast<uintptr_t>(a_dst)) % 16 == 0, JG_EINVAL, "gat_aggregate: pointers must be 16-byte aligned");
    JG_CHECK_ARG(slope >= 0.f && slope <= 1.f, JG_EINVAL, "gat_aggregate: slope must lie in [0, 1]");
    JG_CHECK_ARG(workspace && workspace_bytes >= 256, JG_EWORKSPACE, "gat_aggregate: workspace missing");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    GatArgs a = {out, lse, h, a_src, a_dst, idx, off, n_nodes, slope, static_cast<unsigned long long*>(workspace), nullptr, nullptr};
    if (plan) {
        Carver c(const_cast<void*>(plan));
        a.hub_count = c.take<int32_t>(64) + 40;
        a.order = c.take<int32_t>(n_nodes);
    }
    JG_CUDA(cudaMemsetAsync(a.ticket, 0, 2 * sizeof(unsigned long long), st));
    const int g = (int)(heads * dim / 4), dl = (int)(dim / 4);
    switch (g) {
        case 1: return launch_gat_g<1>(dl, a, st);
        case 2: return launch_gat_g<2>(dl, a, st);
        case 4: return launch_gat_g<4>(dl, a, st);
        case 8: return launch_gat_g<8>(dl, a, st);
        case 16: return launch_gat_g<16>(dl, a, st);
        case 32: return launch_gat_g<32>(dl, a, st);
    }
    return JG_EUNSUPPORTED;
}

size_t jg_gat_backward_workspace_bytes(int64_t n_nodes, int64_t n_edges, int64_t heads, int64_t dim) {
    if (n_nodes < 0 || n_edges < 0 || heads <= 0 || dim <= 0) return 0;
    return carve_gat_bwd(nullptr, n_nodes, n_edges, heads, heads * dim, kScoreGradBlocks).bytes;
}

int jg_gat_backward_f32(float* grad_h, float* grad_a_src, float* grad_a_dst, const float* grad_out, const float* out,
                        const float* lse, const float* h, const float* a_src, const float* a_dst, const int32_t* idx,
                        const int32_t* off, const int32_t* idx_t, const int32_t* off_t, int64_t n_nodes, int64_t n_edges,
                        int64_t heads, int64_t dim, float slope, const void* plan, const void* plan_t, void* workspace,
                        size_t workspace_bytes, jg_stream_t stream) {
    JG_CHECK_ARG(n_nodes >= 0 && n_edges >= 0 && heads > 0 && dim > 0, JG_EINVAL, "gat_backward: bad size");
    JG_CHECK_ARG(grad_a_src && grad_a_dst, JG_EINVAL, "gat_backward: null pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int64_t c = heads * dim;
    if (n_nodes == 0) {
        JG_CUDA(cudaMemsetAsync(grad_a_src, 0, sizeof(float) * (size_t)c, st));
        JG_CUDA(cudaMemsetAsync(grad_a_dst, 0, sizeof(float) * (size_t)c, st));
        return JG_OK;
    }
    JG_CHECK_ARG(grad_h && grad_out && out && lse && h && a_src && a_dst && off && off_t, JG_EINVAL,
                 "gat_backward: null pointer");
    JG_CHECK_ARG(n_edges == 0 || (idx && idx_t), JG_EINVAL, "gat_backward: null idx");
    JG_CHECK_ARG(n_edges <= INT32_MAX && n_nodes < INT32_MAX, JG_ESHAPE, "gat_backward: sizes beyond int32");
    if (!jg_gat_aggregate_supported(heads, dim)) {
        set_error("gat_backward: heads*dim/4 and dim/4 must be powers of two with heads*dim <= 128 (got %lld x %lld)",
                  (long long)heads, (long long)dim);
        return JG_EUNSUPPORTED;
    }
    JG_CHECK_ARG((reinterpret_cast<uintptr_t>(grad_h) | reinterpret_cast<uintptr_t>(grad_out) | reinterpret_cast<uintptr_t>(out) |
                  reinterpret_cast<uintptr_t>(h) | reinterpret_cast<uintptr_t>(a_src) | reinterpret_cast<uintptr_t>(a_dst)) % 16 == 0,
                 JG_EINVAL, "gat_backward: pointers must be 16-byte aligned");
    JG_CHECK_ARG(slope >= 0.f && slope <= 1.f, JG_EINVAL, "gat_backward: slope must lie in [0, 1]");
    JG_CHECK_ARG(workspace && workspace_bytes >= jg_gat_backward_workspace_bytes(n_nodes, n_edges, heads, dim), JG_EWORKSPACE,
                 "gat_backward: workspace too small");
    GatBwdWs ws = carve_gat_bwd(workspace, n_nodes, n_edges, heads, c, kScoreGradBlocks);
    GatBwdArgs a = {};
    a.grad_h = grad_h; a.grad_out = grad_out; a.out = out; a.lse = lse; a.h = h; a.a_src = a_src; a.a_dst = a_dst;
    a.idx = idx; a.off = off; a.idx_t = idx_t; a.off_t = off_t; a.n = n_nodes; a.slope = slope;
    a.ticket = ws.ticket; a.info = ws.info; a.d_dst = ws.d_dst; a.d_src = ws.d_src;
    if (plan) {
        Carver cv(const_cast<void*>(plan));
        a.hub_count = cv.take<int32_t>(64) + 40;
        a.order = cv.take<int32_t>(n_nodes);
    }
    if (plan_t) {
        Carver cv(const_cast<void*>(plan_t));
        a.hub_count_t = cv.take<int32_t>(64) + 40;
        a.n_pieces_t = a.hub_count_t + 1;
        a.order_t = cv.take<int32_t>(n_nodes);
        a.piece_start_t = cv.take<int32_t>(n_nodes + 1);
        a.piece_partial = ws.piece_partial;
    }
    JG_CUDA(cudaMemsetAsync(a.ticket, 0, 4 * sizeof(unsigned long long), st));
    const int g = (int)(c / 4), dl = (int)(dim / 4);
    int rc = JG_EUNSUPPORTED;
    switch (g) {
        case 1: rc = launch_gat_bwd_g<1>(dl, a, st); break;
        case 2: rc = launch_gat_bwd_g<2>(dl, a, st); break;
        case 4: rc = launch_gat_bwd_g<4>(dl, a, st); break;
        case 8: rc = launch_gat_bwd_g<8>(dl, a, st); break;
        case 16: rc = launch_gat_bwd_g<16>(dl, a, st); break;
        case 32: rc = launch_gat_bwd_g<32>(dl, a, st); break;
    }
    if (rc != JG_OK) return rc;
    gat_score_grad_partial_kernel<<<ws.blocks, kScoreGradThreads, 0, st>>>(h, ws.d_src, ws.d_dst, n_nodes, (int)c, (int)dim,
                                                                          ws.partial);
    JG_LAUNCH_CHECK();
    gat_score_grad_final_kernel<<<1, 256, 0, st>>>(ws.partial, ws.blocks, (int)c, grad_a_src, grad_a_dst);
    JG_LAUNCH_CHECK();
    return JG_OK;
}

}  // extern "C"
