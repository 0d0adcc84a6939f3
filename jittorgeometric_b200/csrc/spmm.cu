// Weighted segment aggregation (CSC forward / CSR backward SpMM) for sm_100a.
//
//   out[v,:] = sum_{j in [off[v], off[v+1])} w[j] * x[idx[j],:]
//
// Replaces the reference's AggregateOp (ops/cpp/aggregate_op.cc:26-105) and the
// cuSPARSE SpMM behind SpmmCsr/SpmmCoo (ops/spmmcsr.py:31, ops/spmmcoo.py:34).
//
// Work decomposition.  A "work id" is either one piece (<= chunk entries) of a
// hub row listed in the plan, or one ordinary row.  A persistent grid of warps
// pulls ids eight at a time from a global ticket counter (hub pieces first, so
// the longest items start earliest).  One warp owns one id: it reads 32 indices
// and weights with one coalesced load each (the next tile, which may already
// belong to the next row, is prefetched), stages them in shared memory as
// (index, weight) pairs so that each entry costs one 64-bit broadcast load, and
// gathers feature rows with 128-bit loads, a batch of rows in flight per lane.
// Full batches run without predicates: the kernel is sensitive to instruction
// issue as well as to memory latency (about 8-12 instructions per entry).
// Memory-bound: per nonzero one 4 B index, one 4 B weight and one F*4 B row.
//
// Determinism.  Each output row is produced by exactly one warp (or, for a hub
// row, by a fixed-order sum of its pieces' partial rows held in scratch), so
// results do not depend on which warp ran which id.  No atomics touch data; the
// only atomic is the ticket counter.
#include "common.cuh"

namespace jg {

struct PlanHeader {
    int32_t n_hubs;
    int32_t n_items;
    int32_t chunk;
    int32_t max_hubs;
    int32_t max_items;
    int32_t pad[3];
};

struct PlanView {
    PlanHeader* hdr;
    int32_t* hub_row;    // [max_hubs] row id of each hub
    int32_t* hub_first;  // [max_hubs] first partial slot of each hub
    int32_t* item_hub;   // [max_items] hub index of each piece
    int32_t* item_k;     // [max_items] piece number within its hub
};

static inline int64_t plan_max_hubs(int64_t nnz, int32_t chunk) { return nnz / ((int64_t)chunk + 1) + 1; }
static inline int64_t plan_max_items(int64_t nnz, int32_t chunk) {
    return nnz / chunk + plan_max_hubs(nnz, chunk) + 1;
}

static PlanView plan_view(void* plan, int64_t nnz, int32_t chunk, size_t* bytes) {
    Carver c(plan);
    PlanView v;
    v.hdr = c.take<PlanHeader>(1);
    v.hub_row = c.take<int32_t>(plan_max_hubs(nnz, chunk));
    v.hub_first = c.take<int32_t>(plan_max_hubs(nnz, chunk));
    v.item_hub = c.take<int32_t>(plan_max_items(nnz, chunk));
    v.item_k = c.take<int32_t>(plan_max_items(nnz, chunk));
    if (bytes) *bytes = c.total();
    return v;
}

__global__ void plan_build_kernel(const int32_t* __restrict__ off, int64_t n, PlanView p, int32_t chunk) {
    for (int64_t v = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; v < n;
         v += (int64_t)gridDim.x * blockDim.x) {
        int32_t deg = off[v + 1] - off[v];
        if (deg > chunk) {
            int32_t pieces = (deg + chunk - 1) / chunk;
            int32_t h = atomicAdd(&p.hdr->n_hubs, 1);
            int32_t first = atomicAdd(&p.hdr->n_items, pieces);
            p.hub_row[h] = (int32_t)v;
            p.hub_first[h] = first;
            for (int32_t k = 0; k < pieces; k++) {
                p.item_hub[first + k] = h;
                p.item_k[first + k] = k;
            }
        }
    }
}

constexpr int kGrab = 8;      // most work ids taken per ticket (AggArgs::grab: fewer when the work is short)
constexpr int kBlock = 256;   // threads per CTA

struct AggArgs {
    float* out;
    const float* x;
    const int32_t* idx;
    const int32_t* off;
    const float* w;
    int64_t n_out;
    int64_t f;
    const PlanHeader* hdr;  // null: no plan
    const int32_t* hub_row;
    const int32_t* hub_first;
    const int32_t* item_hub;
    const int32_t* item_k;
    float* partial;
    unsigned long long* ticket;
    int accumulate;  // 1: add the aggregated row to what `out` already holds (old + sum)
    int64_t max_items;  // host-side upper bound on the plan's pieces (sizes the grid)
    const float* bias;  // epilogue on finished output rows: + bias[column] (null: none) ...
    int relu;           // ... then max(., 0)
    int ordered;        // 1: every row must be summed in stored order (no lane groups taking alternate entries)
    int reserve_ctas;   // CTA slots of the persistent grid left free for a kernel that runs beside this one
    int grab;           // work ids per ticket, 1..kGrab (set by the launcher from the amount of work)
};


// Exact mode rounds multiply and add separately, as the reference CPU loop does; the fused
// mode uses one FMA per term.
template <bool EXACT>
__device__ __forceinline__ void axpy4(float4& a, const float4& v, float w) {
    if (EXACT) {
        a.x = __fadd_rn(__fmul_rn(v.x, w), a.x);
        a.y = __fadd_rn(__fmul_rn(v.y, w), a.y);
        a.z = __fadd_rn(__fmul_rn(v.z, w), a.z);
        a.w = __fadd_rn(__fmul_rn(v.w, w), a.w);
    } else {
        a.x = fmaf(v.x, w, a.x);
        a.y = fmaf(v.y, w, a.y);
        a.z = fmaf(v.z, w, a.z);
        a.w = fmaf(v.w, w, a.w);
    }
}

// Vector-width kernel (F = 4*G*VPL).  G lanes cover one feature row, 32/G entries are gathered
// side by side, B steps per batch.
// EPI compiles in the bias/ReLU epilogue (a separate instantiation, so the plain kernel is untouched).
// FULL: the row is exactly 4*G*VPL floats wide (everything about the width folds at compile time).
// !FULL: any 16-byte-aligned width up to that; lanes whose columns lie beyond it sit out.
template <int G, int VPL, int B, int MINB, bool EXACT, bool EPI, bool FULL>
__global__ void __launch_bounds__(kBlock, MINB) aggregate_rows_kernel(AggArgs a) {
    constexpr int EPS = 32 / G;
    const int F = FULL ? 4 * G * VPL : (int)a.f;
    __shared__ int2 s_tile[kBlock / 32][32];
    const int lane = lane_id();
    const int sub = lane / G;
    const int fl = lane % G;
    bool qok[VPL];
#pragma unroll
    for (int q = 0; q < VPL; q++) qok[q] = FULL || (fl + q * G) * 4 < F;
    int2* tile = s_tile[threadIdx.x / 32];
    const char* xb = reinterpret_cast<const char*>(a.x) + fl * 16;
    const int64_t n_items = a.hdr ? a.hdr->n_items : 0;
    const int chunk = a.hdr ? a.hdr->chunk : 0x7fffffff;
    const int64_t total = n_items + a.n_out;
    const int grab = a.grab;
    for (;;) {
        unsigned long long base = 0;
        if (lane == 0) base = atomicAdd(a.ticket, (unsigned long long)grab);
        base = __shfl_sync(kFull, base, 0);
        if ((int64_t)base >= total) break;
        const int64_t row0 = (int64_t)base - n_items;
        int32_t offv = 0;
        {
            const int64_t r = row0 + lane;
            if (lane <= grab && r >= 0 && r <= a.n_out) offv = a.off[r];
        }
        int32_t pf_pos = -1;  // position of the prefetched tile
        int32_t pf_lim = -1;  // ... which holds entries below this bound only
        int pf_idx = 0;
        float pf_w = 0.f;
#pragma unroll 1
        for (int i = 0; i < grab; i++) {
            const int64_t id = (int64_t)base + i;
            if (id >= total) break;
            int32_t s, e, lim;
            float* dst;
            const bool add_old = a.accumulate && id >= n_items;
            if (id < n_items) {
                const int h = a.item_hub[id];
                const int k = a.item_k[id];
                const int row = a.hub_row[h];
                const int32_t rs = a.off[row], re = a.off[row + 1];
                s = rs + k * chunk;
                e = min(re, s + chunk);
                lim = re;  // the next piece of the same hub continues where this one ends
                dst = a.partial + (size_t)(a.hub_first[h] + k) * F;
            } else {
                s = __shfl_sync(kFull, offv, i);
                e = __shfl_sync(kFull, offv, i + 1);
                if (e - s > chunk) continue;  // hub row: its pieces are separate work ids
                // entries of the following rows of this grab are contiguous with this row's
                const int64_t left = a.n_out - row0;
                const int last = left < grab ? (int)left : grab;
                lim = __shfl_sync(kFull, offv, last);
                dst = a.out + (size_t)(id - n_items) * F;
            }
            if (lim != pf_lim) pf_pos = -1;  // a tile prefetched under another bound is not reusable
            pf_lim = lim;
            float4 acc[VPL];
#pragma unroll
            for (int q = 0; q < VPL; q++) acc[q] = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int32_t j0 = s; j0 < e; j0 += 32) {
                int cur_idx = pf_idx;
                float cur_w = pf_w;
                if (pf_pos != j0) {
                    cur_idx = 0;
                    cur_w = 0.f;
                    if (j0 + lane < lim) {
                        cur_idx = ld_stream(a.idx + j0 + lane);
                        cur_w = ld_stream(a.w + j0 + lane);
                    }
                }
                // next tile: the rest of this row, or the start of the next row of the grab
                pf_pos = min(j0 + 32, e);
                pf_idx = 0;
                pf_w = 0.f;
                if (pf_pos + lane < lim) {
                    pf_idx = ld_stream(a.idx + pf_pos + lane);
                    pf_w = ld_stream(a.w + pf_pos + lane);
                }
                __syncwarp();
                tile[lane] = make_int2(cur_idx, __float_as_int(cur_w));
                __syncwarp();
                const int cnt = min(32, e - j0);
                int t = 0;
                for (; t + EPS * B <= cnt; t += EPS * B) {  // full batches: no predicates
                    float4 v[B][VPL];
                    float wv[B];
#pragma unroll
                    for (int u = 0; u < B; u++) {
                        const int2 p = tile[t + u * EPS + sub];
                        wv[u] = __int_as_float(p.y);
                        const float4* g = reinterpret_cast<const float4*>(xb + (size_t)(unsigned)p.x * (size_t)(F * 4));
#pragma unroll
                        for (int q = 0; q < VPL; q++) v[u][q] = qok[q] ? __ldg(g + q * G) : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
#pragma unroll
                    for (int u = 0; u < B; u++)
#pragma unroll
                        for (int q = 0; q < VPL; q++) axpy4<EXACT>(acc[q], v[u][q], wv[u]);
                }
                if (t < cnt) {  // last, partial batch
                    // Four or more entries per step (rows of at most 32 columns): steps whose entries all lie beyond the
                    // row are skipped by a warp-uniform test - most rows of a power-law graph are shorter than one
                    // step, and for them seven of the eight steps are empty (F = 32: -6 % time).  With one or two
                    // entries per step the same test measured 5 % SLOWER (it breaks up the batch of loads), so it is
                    // compiled in for the narrow instantiation only.
                    float4 v[B][VPL];
                    float wv[B];
#pragma unroll
                    for (int u = 0; u < B; u++) {
                        const int k = t + u * EPS + sub;
                        wv[u] = 0.f;
#pragma unroll
                        for (int q = 0; q < VPL; q++) v[u][q] = make_float4(0.f, 0.f, 0.f, 0.f);
                        if ((EPS < 4 || t + u * EPS < cnt) && k < cnt) {
                            const int2 p = tile[k];
                            wv[u] = __int_as_float(p.y);
                            const float4* g = reinterpret_cast<const float4*>(xb + (size_t)(unsigned)p.x * (size_t)(F * 4));
#pragma unroll
                            for (int q = 0; q < VPL; q++)
                                if (qok[q]) v[u][q] = __ldg(g + q * G);
                        }
                    }
#pragma unroll
                    for (int u = 0; u < B; u++) {
                        if (EPS < 4 || t + u * EPS < cnt) {
#pragma unroll
                            for (int q = 0; q < VPL; q++) axpy4<EXACT>(acc[q], v[u][q], wv[u]);
                        }
                    }
                }
            }
            if (EPS > 1) {
#pragma unroll
                for (int o = G; o < 32; o <<= 1)
#pragma unroll
                    for (int q = 0; q < VPL; q++) {
                        acc[q].x += __shfl_xor_sync(kFull, acc[q].x, o);
                        acc[q].y += __shfl_xor_sync(kFull, acc[q].y, o);
                        acc[q].z += __shfl_xor_sync(kFull, acc[q].z, o);
                        acc[q].w += __shfl_xor_sync(kFull, acc[q].w, o);
                    }
            }
            if (sub == 0) {
                float4* o = reinterpret_cast<float4*>(dst) + fl;
#pragma unroll
                for (int q = 0; q < VPL; q++) {
                    if (!qok[q]) continue;
                    if (add_old) {
                        const float4 old = o[q * G];
                        acc[q].x = __fadd_rn(old.x, acc[q].x);
                        acc[q].y = __fadd_rn(old.y, acc[q].y);
                        acc[q].z = __fadd_rn(old.z, acc[q].z);
                        acc[q].w = __fadd_rn(old.w, acc[q].w);
                    }
                    if (EPI && id >= n_items) {   // a finished output row (pieces of hub rows get theirs in the fix-up)
                        if (a.bias) {
                            const float4 b4 = __ldg(reinterpret_cast<const float4*>(a.bias) + fl + q * G);
                            acc[q].x += b4.x; acc[q].y += b4.y; acc[q].z += b4.z; acc[q].w += b4.w;
                        }
                        if (a.relu) {
                            acc[q].x = fmaxf(acc[q].x, 0.f); acc[q].y = fmaxf(acc[q].y, 0.f);
                            acc[q].z = fmaxf(acc[q].z, 0.f); acc[q].w = fmaxf(acc[q].w, 0.f);
                        }
                    }
                    __stcs(o + q * G, acc[q]);
                }
            }
        }
    }
}

// Any feature width: lanes stride over columns with scalar loads, up to 256 columns per sweep.
template <int Q>
__device__ __forceinline__ void warp_segment_any(const AggArgs& a, int32_t s, int32_t e, float* dst, bool add_old, bool final_row) {
    constexpr int UNROLL = Q <= 2 ? 8 : 4;
    const int lane = lane_id();
    const int64_t F = a.f;
    for (int64_t c0 = 0; c0 < F; c0 += 32 * Q) {
        float acc[Q];
#pragma unroll
        for (int q = 0; q < Q; q++) acc[q] = 0.f;
        for (int32_t j0 = s; j0 < e; j0 += 32) {
            const int cnt = min(32, e - j0);
            int cur_idx = 0;
            float cur_w = 0.f;
            if (j0 + lane < e) {
                cur_idx = ld_stream(a.idx + j0 + lane);
                cur_w = ld_stream(a.w + j0 + lane);
            }
            for (int t = 0; t < cnt; t += UNROLL) {
                float v[UNROLL][Q];
                float wv[UNROLL];
#pragma unroll
                for (int u = 0; u < UNROLL; u++) {
                    const int k = t + u;
                    const int src = __shfl_sync(kFull, cur_idx, k & 31);
                    wv[u] = __shfl_sync(kFull, cur_w, k & 31);
                    const float* p = a.x + (size_t)src * F + c0 + lane;
#pragma unroll
                    for (int q = 0; q < Q; q++)
                        v[u][q] = (k < cnt && c0 + q * 32 + lane < F) ? __ldg(p + q * 32) : 0.f;
                    if (k >= cnt) wv[u] = 0.f;
                }
#pragma unroll
                for (int u = 0; u < UNROLL; u++)
#pragma unroll
                    for (int q = 0; q < Q; q++) acc[q] = __fadd_rn(__fmul_rn(v[u][q], wv[u]), acc[q]);
            }
        }
#pragma unroll
        for (int q = 0; q < Q; q++)
            if (c0 + q * 32 + lane < F) {
                float v = add_old ? __fadd_rn(dst[c0 + q * 32 + lane], acc[q]) : acc[q];
                if (final_row) {
                    if (a.bias) v += __ldg(a.bias + c0 + q * 32 + lane);
                    if (a.relu) v = fmaxf(v, 0.f);
                }
                dst[c0 + q * 32 + lane] = v;
            }
    }
}

// Any feature width: one warp per work id, column-strided scalar loads, Q * 32 columns per sweep
// (Q = 2 or 4 for widths up to 64 or 128, so that narrow odd widths do not pay for empty sweeps).
template <int Q>
__global__ void __launch_bounds__(kBlock) aggregate_any_kernel(AggArgs a) {
    const int lane = lane_id();
    const int64_t n_items = a.hdr ? a.hdr->n_items : 0;
    const int chunk = a.hdr ? a.hdr->chunk : 0x7fffffff;
    const int64_t total = n_items + a.n_out;
    const int64_t F = a.f;
    const int grab = a.grab;
    for (;;) {
        unsigned long long base = 0;
        if (lane == 0) base = atomicAdd(a.ticket, (unsigned long long)grab);
        base = __shfl_sync(kFull, base, 0);
        if ((int64_t)base >= total) break;
        // offsets of up to kGrab consecutive ordinary rows with one coalesced read
        const int64_t row0 = (int64_t)base - n_items;
        int32_t offv = 0;
        {
            const int64_t r = row0 + lane;
            if (lane <= grab && r >= 0 && r <= a.n_out) offv = a.off[r];
        }
#pragma unroll 1
        for (int i = 0; i < grab; i++) {
            const int64_t id = (int64_t)base + i;
            if (id >= total) break;
            int32_t s, e;
            float* dst;
            if (id < n_items) {
                const int h = a.item_hub[id];
                const int k = a.item_k[id];
                const int row = a.hub_row[h];
                const int32_t rs = a.off[row], re = a.off[row + 1];
                s = rs + k * chunk;
                e = min(re, s + chunk);
                dst = a.partial + (size_t)(a.hub_first[h] + k) * F;
            } else {
                // lane i of this grab holds off[row], lane i+1 holds off[row+1]
                const int64_t row = id - n_items;
                s = __shfl_sync(kFull, offv, i);
                e = __shfl_sync(kFull, offv, i + 1);
                if (e - s > chunk) continue;  // hub row: its pieces are separate work ids
                dst = a.out + (size_t)row * F;
            }
            warp_segment_any<Q>(a, s, e, dst, a.accumulate && id >= n_items, id >= n_items);
        }
    }
}

// Narrow feature widths (F <= G <= 32, any alignment): G lanes own one work id (an output row or a
// piece of a hub row), so 32/G of them are walked side by side, each in its own stored order with
// separately rounded multiply and add - the result of a row is bit-identical to the sequential
// reference loop.  The G lanes fetch G consecutive (index, weight) entries with one coalesced load
// each and hand them round with width-G shuffles; lane c gathers column c of every source row.
// All groups run the trip count of the longest of their segments, with predicates, so the shuffles
// stay convergent.  The last layer of a GCN (a handful of classes) is this shape.
template <int G>
__global__ void __launch_bounds__(kBlock) aggregate_narrow_kernel(AggArgs a) {
    constexpr int R = 32 / G;          // work ids per warp step
    constexpr int ROUNDS = 4;          // steps per ticket
    const int lane = lane_id();
    const int grp = lane / G, c = lane % G;
    const int64_t n_items = a.hdr ? a.hdr->n_items : 0;
    const int chunk = a.hdr ? a.hdr->chunk : 0x7fffffff;
    const int64_t total = n_items + a.n_out;
    const int F = (int)a.f;
    const bool col_ok = c < F;
    for (;;) {
        unsigned long long base = 0;
        if (lane == 0) base = atomicAdd(a.ticket, (unsigned long long)(R * ROUNDS));
        base = __shfl_sync(kFull, base, 0);
        if ((int64_t)base >= total) break;
#pragma unroll 1
        for (int round = 0; round < ROUNDS; round++) {
            const int64_t id = (int64_t)base + round * R + grp;
            int32_t s = 0, e = 0;
            float* dst = nullptr;
            bool final_row = false;
            if (id < total) {
                if (id < n_items) {
                    const int h = a.item_hub[id];
                    const int k = a.item_k[id];
                    const int row = a.hub_row[h];
                    const int32_t rs = a.off[row], re = a.off[row + 1];
                    s = rs + k * chunk;
                    e = min(re, s + chunk);
                    dst = a.partial + (size_t)(a.hub_first[h] + k) * F;
                } else {
                    const int64_t row = id - n_items;
                    s = a.off[row];
                    e = a.off[row + 1];
                    if (e - s > chunk) {   // hub row: its pieces are separate work ids
                        e = s;
                    } else {
                        dst = a.out + (size_t)row * F;
                        final_row = true;
                    }
                }
            }
            const int len = e - s;
            int maxlen = len;
#pragma unroll
            for (int o = G; o < 32; o <<= 1) maxlen = max(maxlen, __shfl_xor_sync(kFull, maxlen, o));
            if (G < 32 && (int64_t)base + round * R >= total) break;   // warp-uniform: nothing left in this ticket
            float acc = 0.f;
            for (int j = 0; j < maxlen; j += G) {
                int my_idx = 0;
                float my_w = 0.f;
                if (j + c < len) {
                    my_idx = ld_stream(a.idx + s + j + c);
                    my_w = ld_stream(a.w + s + j + c);
                }
#pragma unroll
                for (int k0 = 0; k0 < G; k0 += 4) {
                    float v[4], wv[4];
                    bool ok[4];
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        const int k = k0 + u;
                        const int src = __shfl_sync(kFull, my_idx, k, G);
                        wv[u] = __shfl_sync(kFull, my_w, k, G);
                        ok[u] = j + k < len;
                        v[u] = 0.f;
                        if (ok[u] && col_ok) v[u] = __ldg(a.x + (size_t)(unsigned)src * F + c);
                    }
#pragma unroll
                    for (int u = 0; u < 4; u++)
                        if (ok[u]) acc = __fadd_rn(__fmul_rn(v[u], wv[u]), acc);
                }
            }
            if (dst && col_ok) {
                float v = acc;
                if (final_row) {
                    if (a.accumulate) v = __fadd_rn(dst[c], v);
                    if (a.bias) v += __ldg(a.bias + c);
                    if (a.relu) v = fmaxf(v, 0.f);
                }
                dst[c] = v;
            }
        }
    }
}

// Adds the partial rows of every hub in piece order and writes the hub's output row: one thread per
// (hub, column), consecutive threads on consecutive columns.
__global__ void __launch_bounds__(kBlock) hub_fixup_kernel(AggArgs a) {
    const int64_t n_hubs = a.hdr->n_hubs;
    const int chunk = a.hdr->chunk;
    const int64_t F = a.f;
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < n_hubs * F; t += (int64_t)gridDim.x * blockDim.x) {
        const int64_t h = t / F, c = t - h * F;
        const int row = a.hub_row[h];
        const int deg = a.off[row + 1] - a.off[row];
        const int pieces = (deg + chunk - 1) / chunk;
        const float* p = a.partial + (size_t)a.hub_first[h] * F + c;
        float acc = p[0];
        for (int k = 1; k < pieces; k++) acc = __fadd_rn(acc, p[(size_t)k * F]);
        float* o = a.out + (size_t)row * F + c;
        float v = a.accumulate ? __fadd_rn(*o, acc) : acc;
        if (a.bias) v += __ldg(a.bias + c);
        if (a.relu) v = fmaxf(v, 0.f);
        *o = v;
    }
}

// Persistent grid: as many CTAs as fit on the device, but no more than the work can feed.  Every warp
// takes at least one ticket (an atomic on one address) to learn that nothing is left, so on a small
// graph a full grid of some ten thousand warps would spend its time queueing on that counter.
template <class K>
static int launch_persistent(K kern, int* blocks_per_sm, const AggArgs& a, cudaStream_t st) {
    if (*blocks_per_sm == 0) {
        int b = 0;
        JG_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&b, kern, kBlock, 0));
        *blocks_per_sm = b > 0 ? b : 1;
    }
    int64_t full = (int64_t)sm_count() * *blocks_per_sm;
    if (a.reserve_ctas > 0) full = full - a.reserve_ctas > sm_count() ? full - a.reserve_ctas : sm_count();
    // Tickets of eight ids keep the atomic rare on a large graph; when a warp would see fewer than about
    // two dozen tickets the tail (the last warps still walking their eight rows while the rest of the
    // device idles) dominates, so the tickets get smaller: a shard of 262 k rows ran at half the per-entry
    // speed of the whole graph with eight ids per ticket.
    AggArgs b = a;
    const int64_t ids = a.n_out + a.max_items;
    int64_t g = ids / (full * (kBlock / 32) * 24);
    b.grab = g < 1 ? 1 : (g > kGrab ? kGrab : (int)g);
    const int64_t grabs = (ids + b.grab - 1) / b.grab;
    int64_t blocks = (grabs + kBlock / 32 - 1) / (kBlock / 32);
    if (blocks > full) blocks = full;
    if (blocks < 1) blocks = 1;
    kern<<<(unsigned)blocks, kBlock, 0, st>>>(b);
    JG_LAUNCH_CHECK();
    return JG_OK;
}

template <int G, int VPL, int B, int MINB, bool EXACT>
static int launch_rows(const AggArgs& a, cudaStream_t st) {
    static int bps[4] = {0, 0, 0, 0};
    const bool epi = a.bias || a.relu;
    if (a.f == 4 * G * VPL) {
        if (epi) return launch_persistent(aggregate_rows_kernel<G, VPL, B, MINB, EXACT, true, true>, &bps[0], a, st);
        return launch_persistent(aggregate_rows_kernel<G, VPL, B, MINB, EXACT, false, true>, &bps[1], a, st);
    }
    // a narrower 16-byte-aligned width on the same lane layout (the epilogue variant serves both cases)
    return launch_persistent(aggregate_rows_kernel<G, VPL, B, MINB, EXACT, true, false>, &bps[2], a, st);
}

// Picks the kernel for a feature width: the vector kernel for the 128-bit-aligned widths it is
// specialised for, the column-strided kernel for everything else.
static int dispatch_aggregate(const AggArgs& a, cudaStream_t st) {
    const int64_t f = a.f;
    const bool vec_ok = (f % 4 == 0) && ((reinterpret_cast<uintptr_t>(a.x) | reinterpret_cast<uintptr_t>(a.out) |
                                          reinterpret_cast<uintptr_t>(a.partial)) % 16 == 0);
    // widths up to 64 normally put two or four entries of a row side by side in one warp and add the
    // lane groups' partial sums at the end; an ordered sum takes the narrow kernel (F <= 32) or the
    // 128-column layout with idle lanes (F <= 64) instead
    // (the lane groups' partial sums are added at the end, so these two layouts differ from the sequential
    // sum by rounding anyway: they use one fused multiply-add per term, half the arithmetic instructions
    // of the separately rounded form, in a kernel that is bound by instruction issue at these widths)
    if (vec_ok && f == 32 && !a.ordered) return launch_rows<8, 1, 8, 4, false>(a, st);
    if (vec_ok && f > 32 && f <= 64 && !a.ordered) return launch_rows<16, 1, 8, 4, false>(a, st);
    if (vec_ok && f > 32 && f <= 64) return launch_rows<32, 1, 8, 4, true>(a, st);
    if (vec_ok && f > 64 && f <= 128) return launch_rows<32, 1, 8, 4, true>(a, st);
    if (vec_ok && f > 128 && f <= 256) return launch_rows<32, 2, 4, 4, true>(a, st);
    if (vec_ok && f > 256 && f <= 512) return launch_rows<32, 4, 2, 3, true>(a, st);
    if (f <= 32) {   // narrow rows (any alignment): several rows per warp
        static int nb4 = 0, nb8 = 0, nb16 = 0, nb32 = 0;
        if (f <= 4) return launch_persistent(aggregate_narrow_kernel<4>, &nb4, a, st);
        if (f <= 8) return launch_persistent(aggregate_narrow_kernel<8>, &nb8, a, st);
        if (f <= 16) return launch_persistent(aggregate_narrow_kernel<16>, &nb16, a, st);
        return launch_persistent(aggregate_narrow_kernel<32>, &nb32, a, st);
    }
    static int any2 = 0, any4 = 0, any8 = 0;
    if (f <= 64) return launch_persistent(aggregate_any_kernel<2>, &any2, a, st);
    if (f <= 128) return launch_persistent(aggregate_any_kernel<4>, &any4, a, st);
    return launch_persistent(aggregate_any_kernel<8>, &any8, a, st);
}

}  // namespace jg

using namespace jg;

extern "C" {

size_t jg_spmm_plan_bytes(int64_t n_out, int64_t nnz, int32_t chunk) {
    if (n_out < 0 || nnz < 0 || chunk <= 0) return 0;
    size_t bytes = 0;
    plan_view(nullptr, nnz, chunk, &bytes);
    return bytes;
}

int jg_spmm_plan_build(const int32_t* off, int64_t n_out, int64_t nnz, int32_t chunk, void* plan,
                       size_t plan_bytes, jg_stream_t stream) {
    JG_CHECK_ARG(off && plan, JG_EINVAL, "plan_build: null pointer");
    JG_CHECK_ARG(n_out >= 0 && nnz >= 0 && chunk > 0, JG_EINVAL, "plan_build: bad sizes");
    JG_CHECK_ARG(n_out < INT32_MAX && nnz <= INT32_MAX, JG_ESHAPE, "plan_build: sizes beyond int32");
    size_t need = 0;
    PlanView v = plan_view(plan, nnz, chunk, &need);
    JG_CHECK_ARG(plan_bytes >= need, JG_EWORKSPACE, "plan_build: plan buffer %zu < %zu", plan_bytes, need);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    PlanHeader h = {0, 0, chunk, (int32_t)plan_max_hubs(nnz, chunk), (int32_t)plan_max_items(nnz, chunk), {0, 0, 0}};
    JG_CUDA(cudaMemcpyAsync(v.hdr, &h, sizeof(h), cudaMemcpyHostToDevice, st));
    if (n_out > 0) {
        int grid = (int)((n_out + 255) / 256);
        if (grid > sm_count() * 16) grid = sm_count() * 16;
        plan_build_kernel<<<grid, 256, 0, st>>>(off, n_out, v, chunk);
        JG_LAUNCH_CHECK();
    }
    return JG_OK;
}

size_t jg_aggregate_workspace_bytes(int64_t n_out, int64_t nnz, int64_t f, int32_t chunk) {
    (void)n_out;
    Carver c(nullptr);
    c.take<unsigned long long>(1);
    if (chunk > 0 && nnz > 0 && f > 0) c.take<float>((size_t)plan_max_items(nnz, chunk) * (size_t)f);
    return c.total();
}

static int aggregate_impl(float* out, const float* x, const int32_t* idx, const int32_t* off,
                          const float* w, int64_t n_out, int64_t n_in, int64_t f, int64_t nnz,
                          const void* plan, int32_t chunk, void* workspace, size_t workspace_bytes,
                          jg_stream_t stream, int accumulate, const float* bias = nullptr, int relu = 0, int ordered = 0,
                          int reserve_ctas = 0) {
    JG_CHECK_ARG(n_out >= 0 && n_in >= 0 && f >= 0 && nnz >= 0, JG_EINVAL, "aggregate: negative size");
    if (n_out == 0 || f == 0) return JG_OK;
    JG_CHECK_ARG(out && off, JG_EINVAL, "aggregate: null out/off");
    JG_CHECK_ARG(nnz == 0 || (x && idx && w), JG_EINVAL, "aggregate: null x/idx/w with nnz > 0");
    JG_CHECK_ARG(n_out < INT32_MAX && n_in <= INT32_MAX && nnz <= INT32_MAX, JG_ESHAPE,
                 "aggregate: sizes beyond int32 indexing");
    JG_CHECK_ARG(!plan || chunk > 0, JG_EINVAL, "aggregate: a plan needs the chunk it was built with");
    JG_CHECK_ARG(workspace, JG_EWORKSPACE, "aggregate: workspace is null");
    const size_t need = jg_aggregate_workspace_bytes(n_out, nnz, f, plan ? chunk : 0);
    JG_CHECK_ARG(workspace_bytes >= need, JG_EWORKSPACE, "aggregate: workspace %zu < %zu", workspace_bytes, need);
    cudaStream_t st = static_cast<cudaStream_t>(stream);

    AggArgs a = {};
    a.out = out; a.x = x; a.idx = idx; a.off = off; a.w = w; a.n_out = n_out; a.f = f;
    a.accumulate = accumulate;
    a.bias = bias;
    a.relu = relu;
    a.ordered = ordered;
    a.reserve_ctas = reserve_ctas;
    JG_CHECK_ARG(!bias || f % 4 != 0 || reinterpret_cast<uintptr_t>(bias) % 16 == 0, JG_EINVAL,
                 "aggregate: bias must be 16-byte aligned");
    Carver c(workspace);
    a.ticket = c.take<unsigned long long>(1);
    if (plan) {
        PlanView v = plan_view(const_cast<void*>(plan), nnz, chunk, nullptr);
        a.hdr = v.hdr; a.hub_row = v.hub_row; a.hub_first = v.hub_first;
        a.item_hub = v.item_hub; a.item_k = v.item_k;
        a.partial = c.take<float>((size_t)plan_max_items(nnz, chunk) * (size_t)f);
        a.max_items = plan_max_items(nnz, chunk);
    }
    JG_CUDA(cudaMemsetAsync(a.ticket, 0, sizeof(unsigned long long), st));

    int rc = dispatch_aggregate(a, st);
    if (rc != JG_OK) return rc;
    if (plan) {
        hub_fixup_kernel<<<sm_count() * 2, kBlock, 0, st>>>(a);
        JG_LAUNCH_CHECK();
    }
    return JG_OK;
}


int jg_aggregate_f32(float* out, const float* x, const int32_t* idx, const int32_t* off,
                     const float* w, int64_t n_out, int64_t n_in, int64_t f, int64_t nnz,
                     const void* plan, int32_t chunk, void* workspace, size_t workspace_bytes,
                     jg_stream_t stream) {
    return aggregate_impl(out, x, idx, off, w, n_out, n_in, f, nnz, plan, chunk, workspace, workspace_bytes, stream, 0);
}

int jg_aggregate_add_f32(float* out, const float* x, const int32_t* idx, const int32_t* off,
                         const float* w, int64_t n_out, int64_t n_in, int64_t f, int64_t nnz,
                         const void* plan, int32_t chunk, void* workspace, size_t workspace_bytes,
                         jg_stream_t stream) {
    return aggregate_impl(out, x, idx, off, w, n_out, n_in, f, nnz, plan, chunk, workspace, workspace_bytes, stream, 1);
}

int jg_aggregate_ordered_f32(float* out, const float* x, const int32_t* idx, const int32_t* off, const float* w,
                             int64_t n_out, int64_t n_in, int64_t f, int64_t nnz, const void* plan, int32_t chunk,
                             void* workspace, size_t workspace_bytes, jg_stream_t stream) {
    return aggregate_impl(out, x, idx, off, w, n_out, n_in, f, nnz, plan, chunk, workspace, workspace_bytes, stream, 0, nullptr,
                          0, 1);
}

int jg_aggregate_bias_act_f32(float* out, const float* x, const int32_t* idx, const int32_t* off, const float* w,
                              const float* bias, int relu, int64_t n_out, int64_t n_in, int64_t f, int64_t nnz,
                              const void* plan, int32_t chunk, void* workspace, size_t workspace_bytes, jg_stream_t stream) {
    return aggregate_impl(out, x, idx, off, w, n_out, n_in, f, nnz, plan, chunk, workspace, workspace_bytes, stream, 0, bias,
                          relu ? 1 : 0);
}

int jg_aggregate_opts_f32(float* out, const float* x, const int32_t* idx, const int32_t* off, const float* w,
                          const float* bias, int relu, int accumulate, int ordered, int reserve_ctas, int64_t n_out,
                          int64_t n_in, int64_t f, int64_t nnz, const void* plan, int32_t chunk, void* workspace,
                          size_t workspace_bytes, jg_stream_t stream) {
    JG_CHECK_ARG(!(accumulate && (bias || relu)), JG_EINVAL, "aggregate_opts: the epilogue cannot be combined with accumulate");
    JG_CHECK_ARG(!(accumulate && ordered), JG_EINVAL, "aggregate_opts: ordered cannot be combined with accumulate");
    JG_CHECK_ARG(reserve_ctas >= 0, JG_EINVAL, "aggregate_opts: negative reserve");
    return aggregate_impl(out, x, idx, off, w, n_out, n_in, f, nnz, plan, chunk, workspace, workspace_bytes, stream,
                          accumulate ? 1 : 0, bias, relu ? 1 : 0, ordered ? 1 : 0, reserve_ctas);
}

// ------------------------------------------------------------------------------------------
// Aggregation without any allocation.
//
// Some callers cannot hand this library a workspace: a host program that is not allowed to call
// cudaMalloc once it is running (an inference server whose memory pool is fixed at start-up, a
// plugin loaded into a process that owns the allocator, code running where a device allocation
// would force a synchronisation it cannot afford).  For them the scratch of the aggregation
// (ticket counter, hub plan, partial rows of split hub rows) lives in one fixed array that is part
// of the library image on every GPU that loads it, kStaticScratchBytes long.
namespace jg {

constexpr size_t kStaticScratchBytes = size_t(32) << 20;  // 32 MiB per GPU, held until exit
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// Device address of g_static_scratch per device.  In host code the array's name is only a
// stand-in for the symbol, so the address a kernel may use has to be asked for, once per device,
// with that device current.
static unsigned char* g_static_ptr[64] = {nullptr};

static int static_scratch(unsigned char** out) {
    int dev = 0;
    JG_CUDA(cudaGetDevice(&dev));
    JG_CHECK_ARG(dev >= 0 && dev < 64, JG_EUNSUPPORTED, "device index %d beyond 63", dev);
    if (!g_static_ptr[dev]) {
        void* p = nullptr;
        JG_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
        g_static_ptr[dev] = static_cast<unsigned char*>(p);
    }
    *out = g_static_ptr[dev];
    return JG_OK;
}

// Start-of-call state of the shared array: ticket at zero, empty plan with this call's piece length.
__global__ void static_scratch_init_kernel(unsigned long long* ticket, PlanHeader* hdr, int32_t chunk, int32_t max_hubs,
                                           int32_t max_items) {
    *ticket = 0ull;
    PlanHeader h = {0, 0, chunk, max_hubs, max_items, {0, 0, 0}};
    *hdr = h;
}

// Bytes of scratch one call needs when hub rows are cut into `chunk`-entry pieces.
static size_t static_need(int64_t nnz, int64_t f, int32_t chunk) {
    size_t plan_bytes = 0;
    plan_view(nullptr, nnz, chunk, &plan_bytes);
    Carver c(nullptr);
    c.take<unsigned long long>(1);
    c.take<unsigned char>(plan_bytes);
    c.take<float>((size_t)plan_max_items(nnz, chunk) * (size_t)f);
    return c.total();
}

}  // namespace jg

size_t jg_aggregate_static_capacity_bytes(void) { return jg::kStaticScratchBytes; }

int jg_aggregate_f32_static(float* out, const float* x, const int32_t* idx, const int32_t* off,
                            const float* w, int64_t n_out, int64_t n_in, int64_t f, int64_t nnz,
                            jg_stream_t stream) {
    JG_CHECK_ARG(n_out >= 0 && n_in >= 0 && f >= 0 && nnz >= 0, JG_EINVAL, "aggregate_static: negative size");
    if (n_out == 0 || f == 0) return JG_OK;
    JG_CHECK_ARG(out && off, JG_EINVAL, "aggregate_static: null out/off");
    JG_CHECK_ARG(nnz == 0 || (x && idx && w), JG_EINVAL, "aggregate_static: null x/idx/w with nnz > 0");
    JG_CHECK_ARG(n_out < INT32_MAX && n_in <= INT32_MAX && nnz <= INT32_MAX, JG_ESHAPE,
                 "aggregate_static: sizes beyond int32 indexing");
    // Piece length: 1024 entries, doubled until plan and partial rows fit the fixed array.
    int32_t chunk = 1024;
    while (static_need(nnz, f, chunk) > kStaticScratchBytes && chunk < (1 << 20)) chunk *= 2;
    const size_t need = static_need(nnz, f, chunk);
    JG_CHECK_ARG(need <= kStaticScratchBytes, JG_EWORKSPACE,
                 "aggregate_static: nnz=%lld at width %lld needs %zu bytes of scratch even with %d-entry pieces; "
                 "the built-in scratch holds %zu (use jg_aggregate_f32 with a caller-owned workspace)",
                 (long long)nnz, (long long)f, need, chunk, kStaticScratchBytes);
    unsigned char* base = nullptr;
    int rc = static_scratch(&base);
    if (rc != JG_OK) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);

    size_t plan_bytes = 0;
    plan_view(nullptr, nnz, chunk, &plan_bytes);
    Carver c(base);
    AggArgs a = {};
    a.out = out; a.x = x; a.idx = idx; a.off = off; a.w = w; a.n_out = n_out; a.f = f;
    a.ticket = c.take<unsigned long long>(1);
    PlanView v = plan_view(c.take<unsigned char>(plan_bytes), nnz, chunk, nullptr);
    a.hdr = v.hdr; a.hub_row = v.hub_row; a.hub_first = v.hub_first; a.item_hub = v.item_hub; a.item_k = v.item_k;
    a.partial = c.take<float>((size_t)plan_max_items(nnz, chunk) * (size_t)f);
    a.max_items = plan_max_items(nnz, chunk);

    // The array keeps whatever the previous call left: the two words that must start at zero
    // (ticket, plan counters) are rewritten here; everything else is written before it is read.
    // Both are written by a one-thread kernel from its arguments: no host memory is referenced once
    // this function has returned.
    static_scratch_init_kernel<<<1, 1, 0, st>>>(a.ticket, v.hdr, chunk, (int32_t)plan_max_hubs(nnz, chunk),
                                                (int32_t)plan_max_items(nnz, chunk));
    JG_LAUNCH_CHECK();
    {
        int grid = (int)((n_out + 255) / 256);
        if (grid > sm_count() * 16) grid = sm_count() * 16;
        plan_build_kernel<<<grid, 256, 0, st>>>(off, n_out, v, chunk);
        JG_LAUNCH_CHECK();
    }
    rc = dispatch_aggregate(a, st);
    if (rc != JG_OK) return rc;
    hub_fixup_kernel<<<sm_count() * 2, kBlock, 0, st>>>(a);
    JG_LAUNCH_CHECK();
    return JG_OK;
}

}  // extern "C"
