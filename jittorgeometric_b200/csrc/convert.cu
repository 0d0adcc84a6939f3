// COO -> CSR / CSC conversion with optional fused gcn_norm, for sm_100a.
//
// Replaces the reference's host-side, single-thread counting sorts
// (ops/cpp/cootocsr_op.cc:24-57, ops/cpp/cootocsc_op.cc:23-53) and the tensor-level
// gcn_norm / add_remaining_self_loops (nn/conv/gcn_conv.py:18-37, utils/loop.py:120-134).
//
// Layout contract (bit-exact with the reference): entry i of the COO list lands at
// off[key_i] + #{j < i : key_j == key_i}, i.e. a STABLE sort on the row key; with gcn_norm the
// list is the input with (v,v) entries removed followed by one loop per node in node order.
//
// Method: stable least-significant-digit radix sort, 8 bits per pass, ceil(bits(n)/8) passes,
// carrying (key, other index, weight).  Each pass = per-tile digit histogram, one device-wide
// exclusive scan of the [tile][digit] count matrix in digit-major order, and a stable scatter: ranks inside a tile come from
// warp match masks in element order, elements are staged in shared memory in digit order and
// written out in coalesced runs.  The first pass reads the caller's COO directly (self-loop
// removal and the appended loops are folded into it: removed entries are simply never counted),
// the last pass writes the caller's output arrays.  Offsets are found from the sorted keys by
// boundary detection; nothing uses floating-point atomics, so results are run-to-run identical.
// HBM-bound: about 28 bytes per entry and pass (4 histogram read, 12 read, 12 write).
#include "common.cuh"
#include "scan.cuh"

namespace jg {

constexpr int kSortThreads = 256;
constexpr int kSortItems = 8;
constexpr int kSortTile = kSortThreads * kSortItems;  // 2048 entries per tile
constexpr int kSortWarps = kSortThreads / 32;
constexpr int kRadix = 256;

// ------------------------------------------------------------------------------- digit-major scan
// The per-tile digit counts live as matrix[tile][digit] (rows of 256 counts, written and read
// coalesced).  The scatter needs, for every (digit, tile), the number of entries with a smaller
// digit anywhere plus the entries with the same digit in earlier tiles: an exclusive scan in
// digit-major order.  It is done column-wise, thread d walking column d, so every access is a
// coalesced row: chunk sums, one block that scans chunks and digits, then a walk down each chunk.
constexpr int kChunkTiles = 128;

__global__ void __launch_bounds__(kRadix) colscan_chunk_sums(const int* __restrict__ matrix, int64_t n_tiles,
                                                             int* __restrict__ chunk_sums) {
    const int64_t t0 = (int64_t)blockIdx.x * kChunkTiles;
    const int64_t t1 = t0 + kChunkTiles < n_tiles ? t0 + kChunkTiles : n_tiles;
    int sum = 0;
    for (int64_t t = t0; t < t1; t++) sum += matrix[t * kRadix + threadIdx.x];
    chunk_sums[(int64_t)blockIdx.x * kRadix + threadIdx.x] = sum;
}

__global__ void __launch_bounds__(kRadix) colscan_chunks(int* __restrict__ chunk_sums, int64_t n_chunks) {
    __shared__ int s_warp[32];
    __shared__ int s_total;
    int run = 0;
    for (int64_t c = 0; c < n_chunks; c++) {          // exclusive prefix of this digit's chunk sums
        const int v = chunk_sums[c * kRadix + threadIdx.x];
        chunk_sums[c * kRadix + threadIdx.x] = run;
        run += v;
    }
    const int base = block_exclusive_scan(run, &s_total, s_warp);   // entries with a smaller digit
    for (int64_t c = 0; c < n_chunks; c++) chunk_sums[c * kRadix + threadIdx.x] += base;
}

__global__ void __launch_bounds__(kRadix) colscan_apply(int* __restrict__ matrix, int64_t n_tiles,
                                                        const int* __restrict__ chunk_sums) {
    const int64_t t0 = (int64_t)blockIdx.x * kChunkTiles;
    const int64_t t1 = t0 + kChunkTiles < n_tiles ? t0 + kChunkTiles : n_tiles;
    int run = chunk_sums[(int64_t)blockIdx.x * kRadix + threadIdx.x];
    for (int64_t t = t0; t < t1; t++) {
        const int v = matrix[t * kRadix + threadIdx.x];
        matrix[t * kRadix + threadIdx.x] = run;
        run += v;
    }
}

// ------------------------------------------------------------------------------- sort passes
// Where a pass reads its elements from.
struct SortSrc {
    // mode 0: SoA buffers (key, idx, w) of `count` entries
    const int32_t* key;
    const int32_t* idx;
    const float* w;
    // mode 1: the caller's COO list (first pass)
    const int32_t* coo_src;
    const int32_t* coo_dst;
    const float* coo_w;       // null: unit weights
    const float* loop_w;      // weight of the appended loop of node v (null: 1)
    int64_t e0;               // input entries
    int64_t n_loops;          // appended loops (0 or n)
    int by;                   // 0: key = source, 1: key = destination
    int drop_loops;           // skip (v,v) input entries
    int mode;
    int64_t count;            // positions of the (virtual) list, an upper bound when dcount is set
    const unsigned long long* dcount;  // device-resident element count (mode 0 after a dropping pass)
};

struct Elem {
    int32_t key, idx;
    float w;
    bool valid;
};

// An element is fetched in two steps so that a tile's loads can all be issued before anything looks at a
// loaded value: load_raw only loads (what it returns is not inspected), finish_elem derives key, index and
// validity.  With the two fused, the self-loop test of the first pass (a == b) made every element wait for
// its own loads before the next element's were issued, and every element re-read the device-side count.
struct Raw {
    int32_t a, b;
    float w;
};

__device__ __forceinline__ int64_t list_count(const SortSrc& s) { return s.dcount ? (int64_t)*s.dcount : s.count; }

__device__ __forceinline__ Raw load_raw(const SortSrc& s, int64_t p, int64_t count) {
    Raw r;
    r.a = 0; r.b = 0; r.w = 1.f;
    if (p >= count) return r;
    if (s.mode == 0) {
        r.a = s.key[p]; r.b = s.idx[p];
        if (s.w) r.w = s.w[p];
    } else if (s.mode == 2) {
        // mirrored list: position 2i is edge i as given, 2i + 1 the same edge reversed
        const int64_t i = p >> 1;
        r.a = s.coo_src[i]; r.b = s.coo_dst[i];
        if (s.coo_w) r.w = s.coo_w[i];
    } else if (p < s.e0) {
        r.a = s.coo_src[p]; r.b = s.coo_dst[p];
        if (s.coo_w) r.w = s.coo_w[p];
    } else {
        const int32_t v = (int32_t)(p - s.e0);
        r.a = v; r.b = v;
        if (s.loop_w) r.w = s.loop_w[v];
    }
    return r;
}

__device__ __forceinline__ Elem finish_elem(const SortSrc& s, int64_t p, int64_t count, const Raw& r) {
    Elem e;
    e.valid = p < count;
    e.key = 0; e.idx = 0; e.w = r.w;
    if (!e.valid) { e.w = 0.f; return e; }
    if (s.mode == 0) {
        e.key = r.a; e.idx = r.b;
    } else if (s.mode == 2) {
        e.key = (p & 1) ? r.b : r.a;
        e.idx = (p & 1) ? r.a : r.b;
    } else if (p < s.e0) {
        e.key = s.by == 0 ? r.a : r.b;
        e.idx = s.by == 0 ? r.b : r.a;
        if (s.drop_loops && r.a == r.b) e.valid = false;
    } else {
        e.key = r.a; e.idx = r.a;
    }
    return e;
}

// digit of an element for this pass: from the key, or (canonical order passes) from the index
__device__ __forceinline__ int digit_of(const Elem& e, int shift, int from_idx) {
    return ((from_idx ? e.idx : e.key) >> shift) & (kRadix - 1);
}

// SORTED: the source is a sorted buffer (mode 0); a separate instantiation, so that the register needs of the
// first pass's element loader do not lower the occupancy of the other passes.
template <bool SORTED>
__global__ void __launch_bounds__(kSortThreads) sort_hist_kernel(SortSrc s, int shift, int from_idx, int* __restrict__ matrix,
                                                                 int64_t n_tiles) {
    __shared__ int s_hist[kRadix];
    s_hist[threadIdx.x] = 0;
    __syncthreads();
    const int64_t base = (int64_t)blockIdx.x * kSortTile;
    if (SORTED) {
        // sorted-buffer passes: only the array the digit comes from is read (half the bytes of a full element)
        const int32_t* from = from_idx ? s.idx : s.key;
        const int64_t count = s.dcount ? (int64_t)*s.dcount : s.count;
        int32_t v[kSortItems];
#pragma unroll
        for (int i = 0; i < kSortItems; i++) {
            const int64_t p = base + (int64_t)i * kSortThreads + threadIdx.x;
            v[i] = p < count ? from[p] : -1;
        }
#pragma unroll
        for (int i = 0; i < kSortItems; i++)
            if (v[i] >= 0) atomicAdd(&s_hist[(v[i] >> shift) & (kRadix - 1)], 1);
    } else {
        const int64_t count = list_count(s);
        Raw raw[kSortItems];
#pragma unroll
        for (int i = 0; i < kSortItems; i++) raw[i] = load_raw(s, base + (int64_t)i * kSortThreads + threadIdx.x, count);   // all loads in flight
#pragma unroll
        for (int i = 0; i < kSortItems; i++) {
            const Elem e = finish_elem(s, base + (int64_t)i * kSortThreads + threadIdx.x, count, raw[i]);
            if (e.valid) atomicAdd(&s_hist[digit_of(e, shift, from_idx)], 1);
        }
    }
    __syncthreads();
    matrix[(int64_t)blockIdx.x * kRadix + threadIdx.x] = s_hist[threadIdx.x];   // [tile][digit]: one coalesced row
    (void)n_tiles;
}

struct SortDst {
    int32_t* key;   // may be null on the last pass when keys are not needed
    int32_t* idx;
    float* w;
};

// Stable scatter of one tile.  Element order inside the tile is (warp, round, lane), which is the
// order of the source list because warp w reads one contiguous range of 32 * kSortItems entries.
// HAS_W = false: every weight is 1 (no input weights), so the sort moves (key, index) pairs only and
// the caller writes the weights afterwards; a third less traffic per pass.
template <bool HAS_W>
__global__ void __launch_bounds__(kSortThreads, 4) sort_scatter_kernel(SortSrc s, SortDst d, int shift, int from_idx,
                                                                    const int* __restrict__ matrix, int64_t n_tiles) {
    extern __shared__ __align__(16) unsigned char smem[];
    int* s_whist = reinterpret_cast<int*>(smem);                       // [kSortWarps][kRadix]
    int* s_gbase = s_whist + kSortWarps * kRadix;                      // [kRadix] global offset of a digit for this tile
    int* s_scan = s_gbase + kRadix;                                    // [32]
    int2* s_pair = reinterpret_cast<int2*>(s_scan + 32);               // [kSortTile] (key, index): one 8-byte access per element
    float* s_w = reinterpret_cast<float*>(s_pair + kSortTile);         // [kSortTile]
    __shared__ int s_total;

    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int tile_first = matrix[(int64_t)blockIdx.x * kRadix + threadIdx.x];   // this tile's global start of digit `threadIdx.x`: fetched first, needed last
    for (int i = threadIdx.x; i < kSortWarps * kRadix; i += kSortThreads) s_whist[i] = 0;
    __syncthreads();

    const int64_t wbase = (int64_t)blockIdx.x * kSortTile + (int64_t)wid * (32 * kSortItems);
    Elem el[kSortItems];
    int dig[kSortItems];
    int rank[kSortItems];
    int* my_hist = s_whist + wid * kRadix;
    const unsigned lt_mask = (1u << lane) - 1u;
    // every load of the tile first (independent, all in flight), the ranking rounds after them: with the load
    // inside the round each of the eight rounds waited for its own memory latency behind the warp barriers
    {
        const int64_t count = list_count(s);
        Raw raw[kSortItems];
#pragma unroll
        for (int r = 0; r < kSortItems; r++) raw[r] = load_raw(s, wbase + r * 32 + lane, count);
#pragma unroll
        for (int r = 0; r < kSortItems; r++) el[r] = finish_elem(s, wbase + r * 32 + lane, count, raw[r]);
    }
#pragma unroll
    for (int r = 0; r < kSortItems; r++) {
        dig[r] = el[r].valid ? digit_of(el[r], shift, from_idx) : kRadix;  // kRadix: not an element
        const unsigned peers = __match_any_sync(kFull, dig[r]);
        int before = 0;
        if (el[r].valid) before = my_hist[dig[r]];
        __syncwarp();
        rank[r] = before + __popc(peers & lt_mask);
        if (el[r].valid && (peers & lt_mask) == 0) my_hist[dig[r]] = before + __popc(peers);
        __syncwarp();
    }
    __syncthreads();
    // one thread per digit: exclusive prefix over warps, tile total
    {
        // per warp and digit: first tile slot of that warp's elements of the digit (digit start + the earlier
        // warps' counts), so that staging needs one look-up per element
        const int dgt = threadIdx.x;
        int cnt_w[kSortWarps];
        int run = 0;
#pragma unroll
        for (int w = 0; w < kSortWarps; w++) {
            cnt_w[w] = s_whist[w * kRadix + dgt];
            run += cnt_w[w];
        }
        const int start = block_exclusive_scan(run, &s_total, s_scan);
        int at = start;
#pragma unroll
        for (int w = 0; w < kSortWarps; w++) {
            s_whist[w * kRadix + dgt] = at;
            at += cnt_w[w];
        }
        s_gbase[dgt] = tile_first - start;  // global position = gbase + tile slot
        (void)n_tiles;
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < kSortItems; r++) {
        if (el[r].valid) {
            const int q = my_hist[dig[r]] + rank[r];
            s_pair[q] = make_int2(el[r].key, el[r].idx);
            if (HAS_W) s_w[q] = el[r].w;
        }
    }
    __syncthreads();
    const int total = s_total;
    for (int q = threadIdx.x; q < total; q += kSortThreads) {
        const int2 e = s_pair[q];
        const int64_t g = (int64_t)s_gbase[((from_idx ? e.y : e.x) >> shift) & (kRadix - 1)] + q;   // the digit again, from the element
        if (d.key) d.key[g] = e.x;
        d.idx[g] = e.y;
        if (HAS_W) d.w[g] = s_w[q];
    }
}

constexpr size_t kScatterSmem = sizeof(int) * (kSortWarps * kRadix + kRadix + 32) +
                                sizeof(int2) * kSortTile + sizeof(float) * kSortTile;

// ------------------------------------------------------------------------------- small kernels
// off[k] = first position whose key is >= k, for k in [0, n]; keys sorted, E entries.
__global__ void offsets_from_sorted_keys(const int32_t* __restrict__ key, int64_t E_host,
                                         const unsigned long long* __restrict__ dcount, int64_t n, int32_t* __restrict__ off) {
    // four positions per thread: one 16-byte load of their keys (when aligned) and the key before them
    const int64_t E = dcount ? (int64_t)*dcount : E_host;
    const int64_t j0 = 4 * ((int64_t)blockIdx.x * blockDim.x + threadIdx.x);
    if (j0 > E) return;
    int64_t prev = j0 == 0 ? -1 : key[j0 - 1];
    int32_t k4[4];
    if (j0 + 4 <= E && reinterpret_cast<uintptr_t>(key) % 16 == 0) {
        const int4 v = *reinterpret_cast<const int4*>(key + j0);
        k4[0] = v.x; k4[1] = v.y; k4[2] = v.z; k4[3] = v.w;
    } else {
#pragma unroll
        for (int i = 0; i < 4; i++) k4[i] = j0 + i < E ? key[j0 + i] : 0;
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int64_t j = j0 + i;
        if (j > E) break;
        const int64_t hi = j == E ? n : k4[i];
        for (int64_t k = prev + 1; k <= hi; k++) off[k] = (int32_t)j;
        prev = hi;
    }
}

__global__ void set_count_kernel(unsigned long long* p, unsigned long long v) { *p = v; }

// Valid-entry count of the first pass (input entries that are not (v,v), plus loops).
__global__ void count_kept_kernel(const int32_t* __restrict__ src, const int32_t* __restrict__ dst, int64_t e0,
                                  unsigned long long* __restrict__ kept) {
    unsigned long long c = 0;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < e0; i += (int64_t)gridDim.x * blockDim.x)
        c += src[i] != dst[i];
#pragma unroll
    for (int o = 16; o; o >>= 1) c += __shfl_xor_sync(kFull, c, o);
    if ((threadIdx.x & 31) == 0 && c) atomicAdd(kept, c);
}

// Weight of the loop appended for node v: the fill value, or the weight of the LAST (v,v) input
// entry (an indexed assignment keeps the last write, utils/loop.py:131-133).
__global__ void last_loop_index_kernel(const int32_t* __restrict__ src, const int32_t* __restrict__ dst, int64_t e0,
                                       int* __restrict__ last) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < e0; i += (int64_t)gridDim.x * blockDim.x)
        if (src[i] == dst[i]) atomicMax(&last[src[i]], (int)i);
}
__global__ void loop_weight_kernel(const int* __restrict__ last, const float* __restrict__ w, float fill, int64_t n,
                                   float* __restrict__ loop_w) {
    const int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (v < n) loop_w[v] = last[v] >= 0 ? (w ? w[last[v]] : 1.f) : fill;
}

// deg[v] = sum of the raw weights of column v in list order (sequential fp32 adds, the order a
// host scatter-add takes); dis = deg^-1/2 correctly rounded through double.
__global__ void degree_kernel(const int32_t* __restrict__ off, const float* __restrict__ w, int64_t n, int unit,
                              float* __restrict__ dis) {
    const int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (v >= n) return;
    const int32_t s = off[v], e = off[v + 1];
    float deg = 0.f;
    if (unit) {
        deg = (float)(e - s);  // exact while the count stays below 2^24, as sequential adds of 1.0f are
        if (e - s > (1 << 24)) {
            deg = 0.f;
            for (int32_t j = s; j < e; j++) deg = __fadd_rn(deg, 1.f);
        }
    } else {
        for (int32_t j = s; j < e; j++) deg = __fadd_rn(deg, w[j]);
    }
    dis[v] = (float)(1.0 / sqrt((double)deg));
}

// w'[j] = (dis[source] * w[j]) * dis[destination]  (nn/conv/gcn_conv.py:37); key is the segment
// owner, idx the other endpoint; key_is_dst tells which is which.
__global__ void norm_weight_kernel(const int32_t* __restrict__ key, const int32_t* __restrict__ idx, float* __restrict__ w,
                                   const float* __restrict__ dis, const unsigned long long* __restrict__ dcount,
                                   int key_is_dst, int unit) {
    const int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= (int64_t)*dcount) return;
    const int32_t k = key[j], o = idx[j];
    const float ds = dis[key_is_dst ? o : k], dd = dis[key_is_dst ? k : o];
    w[j] = __fmul_rn(__fmul_rn(ds, unit ? 1.f : w[j]), dd);   // unit: the sort did not carry the (all-one) weights
}

// Four entries per thread (16-byte loads and store; all three arrays 16-byte aligned): with one entry per
// thread the pass was bound by occupancy times a chain of three dependent latencies (count, endpoints, dis).
__global__ void __launch_bounds__(256) norm_weight_vec_kernel(const int32_t* __restrict__ key, const int32_t* __restrict__ idx,
                                                              float* __restrict__ w, const float* __restrict__ dis,
                                                              const unsigned long long* __restrict__ dcount, int key_is_dst, int unit) {
    const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t count = (int64_t)*dcount;
    const int64_t j = 4 * t;
    if (j >= count) return;
    if (j + 4 <= count) {
        const int4 k = reinterpret_cast<const int4*>(key)[t], o = reinterpret_cast<const int4*>(idx)[t];
        float4 v = unit ? make_float4(1.f, 1.f, 1.f, 1.f) : reinterpret_cast<const float4*>(w)[t];
        const int4 a = key_is_dst ? o : k, b = key_is_dst ? k : o;     // a: sources, b: destinations
        const float s0 = dis[a.x], s1 = dis[a.y], s2 = dis[a.z], s3 = dis[a.w];
        const float d0 = dis[b.x], d1 = dis[b.y], d2 = dis[b.z], d3 = dis[b.w];
        v.x = __fmul_rn(__fmul_rn(s0, v.x), d0); v.y = __fmul_rn(__fmul_rn(s1, v.y), d1);
        v.z = __fmul_rn(__fmul_rn(s2, v.z), d2); v.w = __fmul_rn(__fmul_rn(s3, v.w), d3);
        reinterpret_cast<float4*>(w)[t] = v;
    } else {
        for (int64_t i = j; i < count; i++) {
            const int32_t kk = key[i], oo = idx[i];
            const float ds = dis[key_is_dst ? oo : kk], dd = dis[key_is_dst ? kk : oo];
            w[i] = __fmul_rn(__fmul_rn(ds, unit ? 1.f : w[i]), dd);
        }
    }
}

static int launch_norm_weights(const int32_t* key, const int32_t* idx, float* w, const float* dis, const unsigned long long* dcount,
                               int key_is_dst, int unit, int64_t cap, cudaStream_t st) {
    if (cap <= 0) return JG_OK;
    if ((reinterpret_cast<uintptr_t>(key) | reinterpret_cast<uintptr_t>(idx) | reinterpret_cast<uintptr_t>(w)) % 16 == 0)
        norm_weight_vec_kernel<<<(unsigned)(((cap + 3) / 4 + 255) / 256), 256, 0, st>>>(key, idx, w, dis, dcount, key_is_dst, unit);
    else
        norm_weight_kernel<<<(unsigned)((cap + 255) / 256), 256, 0, st>>>(key, idx, w, dis, dcount, key_is_dst, unit);
    JG_LAUNCH_CHECK();
    return JG_OK;
}

// keep[i] = 1 for input entries that are not (v,v)
__global__ void keep_flags_kernel(const int32_t* __restrict__ src, const int32_t* __restrict__ dst, int64_t e0,
                                  int* __restrict__ keep) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < e0) keep[i] = src[i] != dst[i];
}

// Normalised COO list in the reference's order: kept entries in input order, then one loop per node.
__global__ void write_norm_coo_kernel(const int32_t* __restrict__ src, const int32_t* __restrict__ dst,
                                      const float* __restrict__ w, const float* __restrict__ loop_w,
                                      const int* __restrict__ pos, const float* __restrict__ dis, int64_t e0, int64_t n,
                                      const unsigned long long* __restrict__ total, int32_t* __restrict__ out_src,
                                      int32_t* __restrict__ out_dst, float* __restrict__ out_w) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t kept = (int64_t)*total - n;
    if (i < e0) {
        const int32_t a = src[i], b = dst[i];
        if (a != b) {
            const int64_t p = pos[i];
            out_src[p] = a;
            out_dst[p] = b;
            out_w[p] = __fmul_rn(__fmul_rn(dis[a], w ? w[i] : 1.f), dis[b]);
        }
    } else if (i < e0 + n) {
        const int32_t v = (int32_t)(i - e0);
        out_src[kept + v] = v;
        out_dst[kept + v] = v;
        out_w[kept + v] = __fmul_rn(__fmul_rn(dis[v], loop_w ? loop_w[v] : 1.f), dis[v]);
    }
}

// add_self_loops = false: entry i keeps its place, w' = (dis[src] * w) * dis[dst]
__global__ void norm_coo_plain_kernel(const int32_t* __restrict__ src, const int32_t* __restrict__ dst,
                                      const float* __restrict__ w, const float* __restrict__ dis, int64_t e0,
                                      int32_t* __restrict__ out_src, int32_t* __restrict__ out_dst, float* __restrict__ out_w) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= e0) return;
    const int32_t a = src[i], b = dst[i];
    out_src[i] = a;
    out_dst[i] = b;
    out_w[i] = __fmul_rn(__fmul_rn(dis[a], w ? w[i] : 1.f), dis[b]);
}

// ---- symmetrise + dedupe: first entry of every run of equal (row, col) pairs survives
__global__ void first_of_run_kernel(const int32_t* __restrict__ key, const int32_t* __restrict__ idx, int64_t m,
                                    int* __restrict__ flag) {
    const int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (j < m) flag[j] = (j == 0) || key[j] != key[j - 1] || idx[j] != idx[j - 1];
    if (j == m) flag[j] = 0;
}
__global__ void compact_runs_kernel(const int32_t* __restrict__ key, const int32_t* __restrict__ idx,
                                    const float* __restrict__ w, const int* __restrict__ pos, int64_t m,
                                    int32_t* __restrict__ out_src, int32_t* __restrict__ out_dst,
                                    float* __restrict__ out_w, int64_t* __restrict__ out_count) {
    const int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (j < m) {
        const bool first = (j == 0) || key[j] != key[j - 1] || idx[j] != idx[j - 1];
        if (first) {
            const int p = pos[j];
            out_src[p] = key[j];
            out_dst[p] = idx[j];
            out_w[p] = w[j];
        }
    }
    if (j == m) *out_count = pos[m];
}

// ---- 1-D row partition: split a shard's in-edges into interior (source owned) and halo (remote)
__global__ void interior_flags_kernel(const int32_t* __restrict__ idx, int64_t nnz, int32_t lo, int32_t hi,
                                      int* __restrict__ flag) {
    const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e < nnz) flag[e] = idx[e] >= lo && idx[e] < hi;
    if (e == nnz) flag[e] = 0;
}

// pos[e] = number of interior entries before e (exclusive scan of the flags, nnz + 1 entries).
__global__ void split_write_kernel(const int32_t* __restrict__ idx, const float* __restrict__ w,
                                   const int* __restrict__ pos, int64_t nnz, int32_t lo, int32_t hi,
                                   int32_t* __restrict__ int_idx, float* __restrict__ int_w,
                                   int32_t* __restrict__ halo_idx, float* __restrict__ halo_w) {
    const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= nnz) return;
    const int32_t s = idx[e];
    const int p = pos[e];
    if (s >= lo && s < hi) {
        int_idx[p] = s - lo;     // interior sources are addressed inside the shard's own rows
        int_w[p] = w[e];
    } else {
        halo_idx[e - p] = s;     // halo sources keep their global id
        halo_w[e - p] = w[e];
    }
}

__global__ void split_offsets_kernel(const int32_t* __restrict__ off, const int* __restrict__ pos, int64_t n_rows,
                                     int32_t* __restrict__ int_off, int32_t* __restrict__ halo_off,
                                     int64_t* __restrict__ counts) {
    const int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (v > n_rows) return;
    const int32_t o = off[v];
    const int p = pos[o];
    int_off[v] = p;
    halo_off[v] = o - p;
    if (v == n_rows) {
        counts[0] = p;
        counts[1] = o - p;
    }
}

__global__ void fill_int_kernel(int* p, int v, int64_t n) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] = v;
}

// ------------------------------------------------------------------------------- host driver
static int bits_for(int64_t n) {
    int b = 1;
    while (b < 31 && ((int64_t)1 << b) < n) b++;
    return b;
}

struct ConvertWs {
    int32_t *key[2], *idx[2];
    float* w[2];
    int* matrix;
    int* scan_sums;
    float* dis;
    float* loop_w;
    int* last_loop;
    unsigned long long* kept;
    size_t bytes;
};

static ConvertWs carve_convert(void* ws, int64_t cap, int64_t n) {
    Carver c(ws);
    ConvertWs v;
    for (int b = 0; b < 2; b++) {
        v.key[b] = c.take<int32_t>(cap);
        v.idx[b] = c.take<int32_t>(cap);
        v.w[b] = c.take<float>(cap);
    }
    const int64_t tiles = (cap + kSortTile - 1) / kSortTile + 1;
    v.matrix = c.take<int>((size_t)tiles * kRadix);
    v.scan_sums = c.take<int>((size_t)((tiles + kChunkTiles - 1) / kChunkTiles + 1) * kRadix);
    v.dis = c.take<float>(n + 1);
    v.loop_w = c.take<float>(n + 1);
    v.last_loop = c.take<int>(n + 1);
    v.kept = c.take<unsigned long long>(1);
    v.bytes = c.total();
    return v;
}

// Sorts the (virtual) list described by `first` into (keys, out_idx, out_w), stable on the key;
// canonical additionally orders the entries of one key by their index.  `kept` (device) is the
// element count after a first pass that drops entries, or null when first.count is exact.
// *sorted_key receives the buffer holding the sorted keys.
// carry_w = false (all weights are 1): out_w is left untouched, the caller fills it.
static int radix_sort(SortSrc first, int64_t n, int canonical, const unsigned long long* kept, ConvertWs& ws,
                      int32_t* out_idx, float* out_w, int32_t** sorted_key, cudaStream_t st, bool carry_w = true) {
    static bool attr_set[64] = {false};
    int dev = 0;
    JG_CUDA(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        JG_CUDA(cudaFuncSetAttribute(sort_scatter_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kScatterSmem));
        JG_CUDA(cudaFuncSetAttribute(sort_scatter_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kScatterSmem));
        attr_set[dev] = true;
    }
    const int bits = bits_for(n);
    const int key_passes = (bits + 7) / 8;
    const int total_passes = canonical ? 2 * key_passes : key_passes;
    const int64_t tiles = (first.count + kSortTile - 1) / kSortTile;  // upper bound for every pass
    SortSrc src = first;
    int cur = 0;
    *sorted_key = ws.key[0];
    if (tiles == 0) return JG_OK;
    for (int p = 0; p < total_passes; p++) {
        const int from_idx = canonical && p < key_passes;
        const int shift = 8 * (canonical && !from_idx ? p - key_passes : p);
        if (src.mode == 0)
            sort_hist_kernel<true><<<(unsigned)tiles, kSortThreads, 0, st>>>(src, shift, from_idx, ws.matrix, tiles);
        else
            sort_hist_kernel<false><<<(unsigned)tiles, kSortThreads, 0, st>>>(src, shift, from_idx, ws.matrix, tiles);
        JG_LAUNCH_CHECK();
        {
            const int64_t chunks = (tiles + kChunkTiles - 1) / kChunkTiles;
            colscan_chunk_sums<<<(unsigned)chunks, kRadix, 0, st>>>(ws.matrix, tiles, ws.scan_sums);
            JG_LAUNCH_CHECK();
            colscan_chunks<<<1, kRadix, 0, st>>>(ws.scan_sums, chunks);
            JG_LAUNCH_CHECK();
            colscan_apply<<<(unsigned)chunks, kRadix, 0, st>>>(ws.matrix, tiles, ws.scan_sums);
            JG_LAUNCH_CHECK();
        }
        const bool last = p == total_passes - 1;
        SortDst dst;
        dst.key = ws.key[cur];
        dst.idx = last ? out_idx : ws.idx[cur];
        dst.w = carry_w ? (last ? out_w : ws.w[cur]) : nullptr;
        if (carry_w)
            sort_scatter_kernel<true><<<(unsigned)tiles, kSortThreads, kScatterSmem, st>>>(src, dst, shift, from_idx, ws.matrix, tiles);
        else
            sort_scatter_kernel<false><<<(unsigned)tiles, kSortThreads, kScatterSmem, st>>>(src, dst, shift, from_idx, ws.matrix, tiles);
        JG_LAUNCH_CHECK();
        *sorted_key = dst.key;
        SortSrc nxt = {};
        nxt.mode = 0;
        nxt.key = dst.key; nxt.idx = dst.idx; nxt.w = dst.w;
        nxt.count = first.count;
        nxt.dcount = kept;
        src = nxt;
        cur ^= 1;
    }
    return JG_OK;
}

static inline unsigned blocks_for(int64_t n, int threads) { return (unsigned)((n + threads - 1) / threads); }

}  // namespace jg

using namespace jg;

extern "C" {

size_t jg_convert_workspace_bytes(int64_t n_edges, int64_t n_nodes) {
    if (n_edges < 0 || n_nodes < 0) return 0;
    return carve_convert(nullptr, n_edges + n_nodes, n_nodes).bytes;
}

int jg_coo_to_compressed(const int32_t* edge_index, const float* w, int64_t n_edges, int64_t n_nodes, int by,
                         int canonical, int32_t* out_idx, int32_t* out_off, float* out_w, void* workspace,
                         size_t workspace_bytes, jg_stream_t stream) {
    JG_CHECK_ARG(n_edges >= 0 && n_nodes >= 0, JG_EINVAL, "coo_to_compressed: negative size");
    JG_CHECK_ARG(by == 0 || by == 1, JG_EINVAL, "coo_to_compressed: by must be 0 (source) or 1 (destination)");
    JG_CHECK_ARG(out_off, JG_EINVAL, "coo_to_compressed: null offsets");
    JG_CHECK_ARG(n_edges == 0 || (edge_index && out_idx && out_w), JG_EINVAL, "coo_to_compressed: null array");
    JG_CHECK_ARG(n_edges <= INT32_MAX - 1 && n_nodes < INT32_MAX, JG_ESHAPE, "coo_to_compressed: sizes beyond int32");
    JG_CHECK_ARG(workspace && workspace_bytes >= jg_convert_workspace_bytes(n_edges, n_nodes), JG_EWORKSPACE,
                 "coo_to_compressed: workspace %zu < %zu", workspace_bytes, jg_convert_workspace_bytes(n_edges, n_nodes));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    ConvertWs ws = carve_convert(workspace, n_edges + n_nodes, n_nodes);
    SortSrc first = {};
    first.mode = 1;
    first.coo_src = edge_index;
    first.coo_dst = edge_index + n_edges;
    first.coo_w = w;
    first.e0 = n_edges;
    first.by = by;
    first.count = n_edges;
    int32_t* skey = nullptr;
    const bool carry_w = w != nullptr;
    int rc = radix_sort(first, n_nodes, canonical, nullptr, ws, out_idx, out_w, &skey, st, carry_w);
    if (rc != JG_OK) return rc;
    if (!carry_w && n_edges > 0) {   // no input weights: every output weight is 1.0f
        fill_int_kernel<<<blocks_for(n_edges, 256), 256, 0, st>>>(reinterpret_cast<int*>(out_w), 0x3f800000, n_edges);
        JG_LAUNCH_CHECK();
    }
    offsets_from_sorted_keys<<<blocks_for((n_edges + 4) / 4, 256), 256, 0, st>>>(skey, n_edges, nullptr, n_nodes, out_off);
    JG_LAUNCH_CHECK();
    return JG_OK;
}

int jg_gcn_norm_compressed(const int32_t* edge_index, const float* w, int64_t n_edges, int64_t n_nodes, float fill,
                           int add_self_loops, int canonical, int32_t* csc_idx, int32_t* csc_off, float* csc_w,
                           int32_t* csr_idx, int32_t* csr_off, float* csr_w, int64_t* out_count, void* workspace,
                           size_t workspace_bytes, jg_stream_t stream) {
    JG_CHECK_ARG(n_edges >= 0 && n_nodes >= 0, JG_EINVAL, "gcn_norm_compressed: negative size");
    JG_CHECK_ARG(csc_idx && csc_off && csc_w && out_count, JG_EINVAL, "gcn_norm_compressed: CSC outputs and count are required");
    JG_CHECK_ARG((csr_idx && csr_off && csr_w) || (!csr_idx && !csr_off && !csr_w), JG_EINVAL,
                 "gcn_norm_compressed: CSR outputs must be all given or all null");
    JG_CHECK_ARG(n_edges == 0 || edge_index, JG_EINVAL, "gcn_norm_compressed: null edge_index");
    JG_CHECK_ARG(n_edges + n_nodes <= INT32_MAX - 1, JG_ESHAPE, "gcn_norm_compressed: sizes beyond int32");
    JG_CHECK_ARG(workspace && workspace_bytes >= jg_convert_workspace_bytes(n_edges, n_nodes), JG_EWORKSPACE,
                 "gcn_norm_compressed: workspace %zu < %zu", workspace_bytes, jg_convert_workspace_bytes(n_edges, n_nodes));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int64_t cap = n_edges + n_nodes;
    ConvertWs ws = carve_convert(workspace, cap, n_nodes);
    const int32_t* src = edge_index;
    const int32_t* dst = edge_index + n_edges;
    const int grid = sm_count() * 8;

    // entries that survive: non-loop input entries + one loop per node; without self-loops the list as given
    set_count_kernel<<<1, 1, 0, st>>>(ws.kept, (unsigned long long)(add_self_loops ? n_nodes : n_edges));
    JG_LAUNCH_CHECK();
    if (n_edges > 0 && add_self_loops) {
        count_kept_kernel<<<grid, 256, 0, st>>>(src, dst, n_edges, ws.kept);
        JG_LAUNCH_CHECK();
    }
    const bool unit = (w == nullptr) && (fill == 1.0f || !add_self_loops);
    const float* loop_w = nullptr;
    if (!unit && n_nodes > 0 && add_self_loops) {
        fill_int_kernel<<<blocks_for(n_nodes, 256), 256, 0, st>>>(ws.last_loop, -1, n_nodes);
        JG_LAUNCH_CHECK();
        if (n_edges > 0) {
            last_loop_index_kernel<<<grid, 256, 0, st>>>(src, dst, n_edges, ws.last_loop);
            JG_LAUNCH_CHECK();
        }
        loop_weight_kernel<<<blocks_for(n_nodes, 256), 256, 0, st>>>(ws.last_loop, w, fill, n_nodes, ws.loop_w);
        JG_LAUNCH_CHECK();
        loop_w = ws.loop_w;
    }
    SortSrc first = {};
    first.mode = 1;
    first.coo_src = src; first.coo_dst = dst; first.coo_w = w; first.loop_w = loop_w;
    first.e0 = n_edges;
    first.n_loops = add_self_loops ? n_nodes : 0;
    first.drop_loops = add_self_loops ? 1 : 0;
    first.count = add_self_loops ? cap : n_edges;

    // destination-major (CSC), raw weights; degrees and dis from its segments
    int32_t* skey = nullptr;
    first.by = 1;
    int rc = radix_sort(first, n_nodes, canonical, ws.kept, ws, csc_idx, csc_w, &skey, st, !unit);
    if (rc != JG_OK) return rc;
    offsets_from_sorted_keys<<<blocks_for((cap + 4) / 4, 256), 256, 0, st>>>(skey, 0, ws.kept, n_nodes, csc_off);
    JG_LAUNCH_CHECK();
    if (n_nodes > 0) {
        degree_kernel<<<blocks_for(n_nodes, 256), 256, 0, st>>>(csc_off, csc_w, n_nodes, unit ? 1 : 0, ws.dis);
        JG_LAUNCH_CHECK();
    }
    rc = launch_norm_weights(skey, csc_idx, csc_w, ws.dis, ws.kept, 1, unit ? 1 : 0, cap, st);
    if (rc != JG_OK) return rc;
    if (csr_idx) {
        bool weights_done = false;
        if (canonical) {
            // The canonical CSC list is ordered by (destination, source); ONE stable sort of it by source gives
            // (source, destination), the canonical CSR, in half the passes of sorting the input again by both
            // keys.  The normalised weight of an entry is the same number in both formats, so it travels with
            // the entry (unit weights are not carried at all and are written afterwards, as for the CSC).
            SortSrc from_csc = {};
            from_csc.mode = 0;
            from_csc.key = csc_idx;                 // source of every entry, the new key
            from_csc.idx = skey;                    // its destination (the sorted keys of the CSC sort)
            from_csc.w = unit ? nullptr : csc_w;
            from_csc.count = first.count;
            from_csc.dcount = ws.kept;
            rc = radix_sort(from_csc, n_nodes, 0, ws.kept, ws, csr_idx, csr_w, &skey, st, !unit);
            weights_done = !unit;
        } else {
            first.by = 0;
            rc = radix_sort(first, n_nodes, canonical, ws.kept, ws, csr_idx, csr_w, &skey, st, !unit);
        }
        if (rc != JG_OK) return rc;
        offsets_from_sorted_keys<<<blocks_for((cap + 4) / 4, 256), 256, 0, st>>>(skey, 0, ws.kept, n_nodes, csr_off);
        JG_LAUNCH_CHECK();
        if (!weights_done) {
            rc = launch_norm_weights(skey, csr_idx, csr_w, ws.dis, ws.kept, 0, unit ? 1 : 0, cap, st);
            if (rc != JG_OK) return rc;
        }
    }
    JG_CUDA(cudaMemcpyAsync(out_count, ws.kept, sizeof(unsigned long long), cudaMemcpyDeviceToDevice, st));
    return JG_OK;
}


struct NormCooWs {
    void* convert;
    size_t convert_bytes;
    int32_t* tmp_idx;
    int32_t* tmp_off;
    float* tmp_w;
    int* pos;
    int* pos_sums;
    int64_t* count;
    size_t bytes;
};

static NormCooWs carve_norm_coo(void* ws, int64_t n_edges, int64_t n_nodes) {
    Carver c(ws);
    NormCooWs v;
    v.convert_bytes = jg_convert_workspace_bytes(n_edges, n_nodes);
    v.convert = c.take<unsigned char>(v.convert_bytes);
    v.tmp_idx = c.take<int32_t>(n_edges + n_nodes);
    v.tmp_off = c.take<int32_t>(n_nodes + 1);
    v.tmp_w = c.take<float>(n_edges + n_nodes);
    v.pos = c.take<int>(n_edges + 1);
    v.pos_sums = c.take<int>(scan_temp_ints(n_edges + 1));
    v.count = c.take<int64_t>(1);
    v.bytes = c.total();
    return v;
}

size_t jg_gcn_norm_coo_workspace_bytes(int64_t n_edges, int64_t n_nodes) {
    if (n_edges < 0 || n_nodes < 0) return 0;
    return carve_norm_coo(nullptr, n_edges, n_nodes).bytes;
}

int jg_gcn_norm_coo(const int32_t* edge_index, const float* w, int64_t n_edges, int64_t n_nodes, float fill,
                    int add_self_loops, int32_t* out_src, int32_t* out_dst, float* out_w, int64_t* out_count,
                    void* workspace, size_t workspace_bytes, jg_stream_t stream) {
    JG_CHECK_ARG(n_edges >= 0 && n_nodes >= 0, JG_EINVAL, "gcn_norm_coo: negative size");
    JG_CHECK_ARG(out_count, JG_EINVAL, "gcn_norm_coo: null count");
    JG_CHECK_ARG(n_edges + n_nodes == 0 || (out_src && out_dst && out_w), JG_EINVAL, "gcn_norm_coo: null output");
    JG_CHECK_ARG(n_edges == 0 || edge_index, JG_EINVAL, "gcn_norm_coo: null edge_index");
    JG_CHECK_ARG(workspace && workspace_bytes >= jg_gcn_norm_coo_workspace_bytes(n_edges, n_nodes), JG_EWORKSPACE,
                 "gcn_norm_coo: workspace %zu < %zu", workspace_bytes, jg_gcn_norm_coo_workspace_bytes(n_edges, n_nodes));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    NormCooWs nw = carve_norm_coo(workspace, n_edges, n_nodes);
    // degrees come from the destination-major order (sequential sums in list order); its arrays are scratch here
    int rc = jg_gcn_norm_compressed(edge_index, w, n_edges, n_nodes, fill, add_self_loops, 0, nw.tmp_idx, nw.tmp_off,
                                    nw.tmp_w, nullptr, nullptr, nullptr, out_count, nw.convert, nw.convert_bytes, stream);
    if (rc != JG_OK) return rc;
    ConvertWs ws = carve_convert(nw.convert, n_edges + n_nodes, n_nodes);  // dis, loop_w and kept live there
    const bool unit = (w == nullptr) && fill == 1.0f;
    if (!add_self_loops) {   // the list as given, every weight scaled by the two degrees
        if (n_edges > 0) {
            norm_coo_plain_kernel<<<blocks_for(n_edges, 256), 256, 0, st>>>(edge_index, edge_index + n_edges, w, ws.dis,
                                                                            n_edges, out_src, out_dst, out_w);
            JG_LAUNCH_CHECK();
        }
        return JG_OK;
    }
    if (n_edges > 0) {
        keep_flags_kernel<<<blocks_for(n_edges, 256), 256, 0, st>>>(edge_index, edge_index + n_edges, n_edges, nw.pos);
        JG_LAUNCH_CHECK();
        rc = exclusive_scan(nw.pos, nw.pos, n_edges, nw.pos_sums, st);
        if (rc != JG_OK) return rc;
    }
    if (n_edges + n_nodes > 0) {
        write_norm_coo_kernel<<<blocks_for(n_edges + n_nodes, 256), 256, 0, st>>>(
            edge_index, edge_index + n_edges, w, unit ? nullptr : ws.loop_w, nw.pos, ws.dis, n_edges, n_nodes, ws.kept,
            out_src, out_dst, out_w);
        JG_LAUNCH_CHECK();
    }
    return JG_OK;
}


size_t jg_partition_split_workspace_bytes(int64_t nnz) {
    if (nnz < 0) return 0;
    Carver c(nullptr);
    c.take<int>(nnz + 1);
    c.take<int>(scan_temp_ints(nnz + 1));
    return c.total();
}

int jg_partition_split(const int32_t* idx, const int32_t* off, const float* w, int64_t n_rows, int64_t nnz, int32_t lo,
                       int32_t hi, int32_t* int_idx, int32_t* int_off, float* int_w, int32_t* halo_idx,
                       int32_t* halo_off, float* halo_w, int64_t* out_counts, void* workspace, size_t workspace_bytes,
                       jg_stream_t stream) {
    JG_CHECK_ARG(n_rows >= 0 && nnz >= 0 && lo <= hi, JG_EINVAL, "partition_split: bad sizes");
    JG_CHECK_ARG(off && int_off && halo_off && out_counts, JG_EINVAL, "partition_split: null offsets/counts");
    JG_CHECK_ARG(nnz == 0 || (idx && w && int_idx && int_w && halo_idx && halo_w), JG_EINVAL, "partition_split: null array");
    JG_CHECK_ARG(nnz < INT32_MAX && n_rows < INT32_MAX, JG_ESHAPE, "partition_split: sizes beyond int32");
    JG_CHECK_ARG(workspace && workspace_bytes >= jg_partition_split_workspace_bytes(nnz), JG_EWORKSPACE,
                 "partition_split: workspace too small");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    Carver c(workspace);
    int* pos = c.take<int>(nnz + 1);
    int* sums = c.take<int>(scan_temp_ints(nnz + 1));
    interior_flags_kernel<<<blocks_for(nnz + 1, 256), 256, 0, st>>>(idx, nnz, lo, hi, pos);
    JG_LAUNCH_CHECK();
    int rc = exclusive_scan(pos, pos, nnz + 1, sums, st);
    if (rc != JG_OK) return rc;
    if (nnz > 0) {
        split_write_kernel<<<blocks_for(nnz, 256), 256, 0, st>>>(idx, w, pos, nnz, lo, hi, int_idx, int_w, halo_idx, halo_w);
        JG_LAUNCH_CHECK();
    }
    split_offsets_kernel<<<blocks_for(n_rows + 1, 256), 256, 0, st>>>(off, pos, n_rows, int_off, halo_off, out_counts);
    JG_LAUNCH_CHECK();
    return JG_OK;
}


struct UndirectedWs {
    void* convert;
    size_t convert_bytes;
    int32_t* idx;
    float* w;
    int* pos;
    int* pos_sums;
    size_t bytes;
};

static UndirectedWs carve_undirected(void* ws, int64_t n_edges, int64_t n_nodes) {
    Carver c(ws);
    UndirectedWs v;
    v.convert_bytes = jg_convert_workspace_bytes(2 * n_edges, n_nodes);
    v.convert = c.take<unsigned char>(v.convert_bytes);
    v.idx = c.take<int32_t>(2 * n_edges + 1);
    v.w = c.take<float>(2 * n_edges + 1);
    v.pos = c.take<int>(2 * n_edges + 1);
    v.pos_sums = c.take<int>(scan_temp_ints(2 * n_edges + 1));
    v.bytes = c.total();
    return v;
}

size_t jg_to_undirected_workspace_bytes(int64_t n_edges, int64_t n_nodes) {
    if (n_edges < 0 || n_nodes < 0) return 0;
    return carve_undirected(nullptr, n_edges, n_nodes).bytes;
}

int jg_to_undirected(const int32_t* edge_index, const float* attr, int64_t n_edges, int64_t n_nodes, int32_t* out_src,
                     int32_t* out_dst, float* out_attr, int64_t* out_count, void* workspace, size_t workspace_bytes,
                     jg_stream_t stream) {
    JG_CHECK_ARG(n_edges >= 0 && n_nodes >= 0, JG_EINVAL, "to_undirected: negative size");
    JG_CHECK_ARG(out_count, JG_EINVAL, "to_undirected: null count");
    JG_CHECK_ARG(n_edges == 0 || (edge_index && out_src && out_dst && out_attr), JG_EINVAL, "to_undirected: null array");
    JG_CHECK_ARG(2 * n_edges <= INT32_MAX - 1 && n_nodes < INT32_MAX, JG_ESHAPE, "to_undirected: sizes beyond int32");
    JG_CHECK_ARG(workspace && workspace_bytes >= jg_to_undirected_workspace_bytes(n_edges, n_nodes), JG_EWORKSPACE,
                 "to_undirected: workspace too small");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int64_t m = 2 * n_edges;
    UndirectedWs uw = carve_undirected(workspace, n_edges, n_nodes);
    ConvertWs ws = carve_convert(uw.convert, m + n_nodes, n_nodes);
    SortSrc first = {};
    first.mode = 2;
    first.coo_src = edge_index;
    first.coo_dst = edge_index + n_edges;
    first.coo_w = attr;
    first.count = m;
    int32_t* skey = nullptr;
    int rc = radix_sort(first, n_nodes, 1, nullptr, ws, uw.idx, uw.w, &skey, st);   // by (row, col), stable
    if (rc != JG_OK) return rc;
    first_of_run_kernel<<<blocks_for(m + 1, 256), 256, 0, st>>>(skey, uw.idx, m, uw.pos);
    JG_LAUNCH_CHECK();
    rc = exclusive_scan(uw.pos, uw.pos, m + 1, uw.pos_sums, st);
    if (rc != JG_OK) return rc;
    compact_runs_kernel<<<blocks_for(m + 1, 256), 256, 0, st>>>(skey, uw.idx, uw.w, uw.pos, m, out_src, out_dst, out_attr,
                                                                 out_count);
    JG_LAUNCH_CHECK();
    return JG_OK;
}

}  // extern "C"
