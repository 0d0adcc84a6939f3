// Halo exchange of the 1-D row partition by direct loads from peer memory over NVLink (sm_100a).
//
// Replaces the reference's P rounds of pickled host MPI.bcast of whole feature blocks
// (ops/distspmm.py:31-39, utils/distributed_utils.py:66-74).  Every rank keeps its feature rows in
// a buffer its peers have mapped (one process per GPU, symmetric allocation) and each rank PULLS
// the distinct remote rows its in-edges reference straight out of their owners' buffers into its
// local halo rows: no pack step, no send buffer, no collective kernel.
//
// Ordering is by epoch words, not barriers.  A rank's flag block holds, per buffer slot, one
// "ready" and one "done" word per peer:
//   * jg_halo_post (owner, after its feature rows are written): stores the epoch into
//     ready[slot][owner] of every rank's flag block with release semantics at system scope;
//   * the pull kernel acquires ready[slot][q] in its own flag block before the first load from
//     owner q, and when its last block has landed stores the epoch into done[slot][puller] of every
//     owner's flag block;
//   * jg_halo_wait (owner, before it overwrites its rows): acquires done[slot][q] of every peer.
// Every wait is bounded by a time limit; a wait that runs out writes a code to an error word the
// host can read and the kernel returns after draining the copies it has in flight.  Nothing traps.
//
// The pull itself: one warp per CTA drives a ring of shared-memory stages with bulk asynchronous
// copies (cp.async.bulk): every lane issues row-sized copies peer -> shared memory that complete on
// the stage's mbarrier, and one bulk store moves the stage (consecutive halo rows) to local memory.
// A CTA is 32 threads and a few registers, so the kernel runs beside an aggregation kernel that has
// been told to leave a few CTA slots free (jg_aggregate_opts_f32, reserve_ctas) - that is how the
// exchange of one feature width hides under the aggregation of another.  No load uses cluster
// multicast.  Widths whose rows are not multiples of 16 bytes take a plain-load kernel.
#include "common.cuh"

#include <cuda_fp16.h>

namespace jg {

constexpr int kMaxRanks = 16;
constexpr int kFlagSlots = 16;
constexpr int kPullStages = 4;
constexpr uint32_t kPullSpins = 1u << 22;   // bounded mbarrier wait on a copy in flight

__host__ __device__ inline size_t flag_index(int slot, int kind, int rank) {
    return ((size_t)slot * 2 + (size_t)kind) * kMaxRanks + (size_t)rank;
}

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint64_t global_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Waits until *p has reached `epoch` (wrap-around compare); false when `limit_ns` ran out.
__device__ __forceinline__ bool wait_epoch(const uint32_t* p, uint32_t epoch, uint64_t limit_ns) {
    if ((int32_t)(ld_acquire_sys(p) - epoch) >= 0) return true;
    const uint64_t t0 = global_ns();
    for (;;) {
        if ((int32_t)(ld_acquire_sys(p) - epoch) >= 0) return true;
        if (global_ns() - t0 > limit_ns) return false;
        __nanosleep(256);
    }
}

__device__ __forceinline__ void report(int32_t* error, int32_t code) {
    if (error) {
        *reinterpret_cast<volatile int32_t*>(error) = code;
        __threadfence_system();
    }
}

struct PeerTable {
    const void* x[kMaxRanks];       // every rank's feature buffer (own rows first), as mapped here
    uint32_t* flags[kMaxRanks];     // every rank's flag block, as mapped here
    int64_t seg_begin[kMaxRanks + 1];  // halo slots [seg_begin[q], seg_begin[q+1]) hold rows owned by rank q
    int64_t seg_end[kMaxRanks];        // this call fetches the slots [seg_begin[q], seg_end[q]) (a part of the segment, or all of it)
    int32_t lo[kMaxRanks];          // first global row id of rank q
    int32_t order[kMaxRanks];       // the peers in the order this rank visits them (rank+1, rank+2, ...)
    int32_t n_blocks[kMaxRanks];    // blocks of rows_per_block halo slots in rank q's segment
};

struct PullArgs {
    unsigned char* halo;     // local halo rows [n_halo, row_bytes]
    const int32_t* needed;   // [n_halo] global ids, ascending (grouped by owner)
    PeerTable t;
    int32_t world, rank;
    uint32_t row_bytes;
    int32_t rows_per_block;
    int32_t max_blocks;      // largest n_blocks over the peers
    uint32_t* my_flags;
    int32_t slot;
    uint32_t epoch;
    unsigned int* counter;   // local word, zero between calls: CTAs that have finished
    int32_t* error;
    uint64_t wait_ns;
};

__global__ void halo_post_kernel(PeerTable t, int world, int rank, int slot, int kind, uint32_t epoch) {
    const int q = threadIdx.x;
    if (q < world) {
        __threadfence_system();   // the rows written before this kernel are visible before the word is
        st_release_sys(t.flags[q] + flag_index(slot, kind, rank), epoch);
    }
}

__global__ void halo_wait_kernel(const uint32_t* my_flags, int world, int rank, int slot, int kind, uint32_t epoch,
                                 int32_t* error, uint64_t wait_ns) {
    const int q = threadIdx.x;
    if (q < world && q != rank) {
        if (!wait_epoch(my_flags + flag_index(slot, kind, q), epoch, wait_ns)) report(error, 0x200 + q);
    }
}

__device__ __forceinline__ uint32_t xsmem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ bool xmbar_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = xsmem_u32(bar);
    for (uint32_t spin = 0; spin < kPullSpins; spin++) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
        if (spin > 32) __nanosleep(spin > 4096 ? 512 : 64);
    }
    return false;
}

// Virtual block v -> (owner, first halo slot, rows).  Blocks are dealt to the peers in turn, so a
// rank reads from all its peers at once and every owner serves all its readers at once.
__device__ __forceinline__ bool decode_block(const PullArgs& a, int64_t v, int& q, int64_t& r0, int& cnt) {
    const int n_peers = a.world - 1;
    const int j = (int)(v % n_peers);
    const int64_t lb = v / n_peers;
    q = a.t.order[j];
    if (lb >= a.t.n_blocks[q]) return false;
    r0 = a.t.seg_begin[q] + lb * a.rows_per_block;
    const int64_t left = a.t.seg_end[q] - r0;
    cnt = left < a.rows_per_block ? (int)left : a.rows_per_block;
    return true;
}

// The next block a producer warp will request, with this lane's row ids already loaded: the ids of
// block b + 1 are fetched while the copies of block b are being issued, so a lane never sits through a
// dependent id load per row (that chain, about 2 us per row and lane, was the limit of the first version).
constexpr int kMaxIdsPerLane = 8;   // rows_per_block <= 256
struct BlockCursor {
    int64_t v;
    bool have;
    int q, cnt;
    int64_t r0;
    int32_t ids[kMaxIdsPerLane];
};
__device__ __forceinline__ void cursor_advance(const PullArgs& a, BlockCursor& c, int64_t total_v, int lane) {
    c.have = false;
    while (c.v < total_v && !c.have) {
        c.have = decode_block(a, c.v, c.q, c.r0, c.cnt);
        c.v += gridDim.x;
    }
    if (c.have) {
#pragma unroll
        for (int j = 0; j < kMaxIdsPerLane; j++) {
            const int i = lane + 32 * j;
            c.ids[j] = i < c.cnt ? __ldg(a.needed + c.r0 + i) : 0;
        }
    }
}
// Requests the rows of the cursor's block: one bulk copy per row, completing on `bar`.
__device__ __forceinline__ void cursor_issue(const PullArgs& a, const BlockCursor& c, uint32_t dst0, uint32_t bar, int lane) {
    if (lane == 0)
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"((uint32_t)c.cnt * a.row_bytes) : "memory");
    const unsigned char* base = static_cast<const unsigned char*>(a.t.x[c.q]);
    const int32_t lo = a.t.lo[c.q];
#pragma unroll
    for (int j = 0; j < kMaxIdsPerLane; j++) {
        const int i = lane + 32 * j;
        if (i < c.cnt) {
            const unsigned char* src = base + (size_t)(c.ids[j] - lo) * a.row_bytes;
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                         ::"r"(dst0 + (uint32_t)i * a.row_bytes), "l"(src), "r"(a.row_bytes), "r"(bar) : "memory");
        }
    }
}

// When the last CTA of a pull has finished, every owner learns that this rank has read its rows.
__device__ __forceinline__ void finish_pull(const PullArgs& a, bool ok) {
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        // low half: CTAs that have finished; high half: CTAs that gave up
        const unsigned int done = atomicAdd(a.counter, ok ? 1u : 0x10001u);
        if ((done & 0xffffu) == gridDim.x - 1) {
            *a.counter = 0u;
            __threadfence_system();
            if (ok && (done >> 16) == 0)
                for (int q = 0; q < a.world; q++)
                    st_release_sys(a.t.flags[q] + flag_index(a.slot, 1, a.rank), a.epoch);
        }
    }
}

__global__ void __launch_bounds__(32) halo_pull_bulk_kernel(PullArgs a, uint32_t stage_bytes, int n_stages) {
    extern __shared__ __align__(128) unsigned char smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + (size_t)n_stages * stage_bytes);
    const int lane = threadIdx.x;
    if (lane == 0) {
        for (int s = 0; s < n_stages; s++)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(xsmem_u32(&full[s])));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    const int64_t total_v = (int64_t)a.max_blocks * (a.world - 1);
    int64_t v_cons = blockIdx.x;
    uint32_t it_load = 0, it_cons = 0, ready_mask = 0;
    bool ok = true;
    BlockCursor cur;
    cur.v = blockIdx.x;
    cursor_advance(a, cur, total_v, lane);

    auto issue_next = [&]() -> bool {
        if (!cur.have) return false;
        const int q = cur.q;
        if (!((ready_mask >> q) & 1u)) {   // first touch of this owner: its rows must have been posted
            int r = 1;
            if (lane == 0) r = wait_epoch(a.my_flags + flag_index(a.slot, 0, q), a.epoch, a.wait_ns) ? 1 : 0;
            r = __shfl_sync(kFull, r, 0);
            if (!r) {
                if (lane == 0) report(a.error, 0x100 + q);
                ok = false;
                return false;
            }
            ready_mask |= 1u << q;
            asm volatile("fence.proxy.async;" ::: "memory");   // the acquire orders generic accesses; the copies below are asynchronous-proxy reads
        }
        const int s = (int)(it_load % (uint32_t)n_stages);
        cursor_issue(a, cur, xsmem_u32(smem + (size_t)s * stage_bytes), xsmem_u32(&full[s]), lane);
        it_load++;
        cursor_advance(a, cur, total_v, lane);
        return true;
    };

    for (int j = 0; j < n_stages - 1; j++)
        if (!issue_next()) break;
    while (ok) {
        int q = 0, cnt = 0;
        int64_t r0 = 0;
        bool found = false;
        while (v_cons < total_v && !found) {
            found = decode_block(a, v_cons, q, r0, cnt);
            v_cons += gridDim.x;
        }
        if (!found) break;
        if (it_cons >= 1) {   // the stage the next load goes to was stored by the previous round: its read must be over
            if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            __syncwarp();
        }
        issue_next();
        if (!ok || it_cons >= it_load) break;
        const int s = (int)(it_cons % (uint32_t)n_stages);
        if (!xmbar_wait(&full[s], (it_cons / (uint32_t)n_stages) & 1u)) {
            if (lane == 0) report(a.error, 0x300);
            ok = false;
            it_cons++;     // this copy is given up; the drain below waits for the later ones only
            break;
        }
        if (lane == 0) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                         ::"l"(a.halo + (size_t)r0 * a.row_bytes), "r"(xsmem_u32(smem + (size_t)s * stage_bytes)),
                           "r"((uint32_t)cnt * a.row_bytes) : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
        it_cons++;
    }
    // copies still in flight into this CTA's shared memory must land before it exits
    for (uint32_t it = it_cons; it < it_load; it++)
        xmbar_wait(&full[it % (uint32_t)n_stages], (it / (uint32_t)n_stages) & 1u);
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    finish_pull(a, ok);
}

// Half-width payload: the owners keep an fp16 copy of their rows, the puller fetches those (half the
// NVLink bytes) and widens them to fp32 on the way into its halo rows.  fp16 rather than bf16: its
// unit roundoff (2^-11) keeps every aggregated element within 5e-4 of the fp32 result relative to the
// sum of absolute terms, bf16 (2^-8) does not stay within 2e-3 on rows with few in-edges.  Warp 0
// issues the bulk copies as above; warps 1-4 turn every landed stage into fp32 rows with 16-byte loads
// from shared memory and coalesced 16-byte stores, and hand the stage back through a second mbarrier.
struct HalfCtl {
    int abort;        // the producer gave up ...
    uint32_t issued;  // ... after this many blocks, which still land and are still converted
};

__global__ void __launch_bounds__(160) halo_pull_half_kernel(PullArgs a, uint32_t stage_bytes, int n_stages) {
    extern __shared__ __align__(128) unsigned char smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + (size_t)n_stages * stage_bytes);
    uint64_t* empty = full + kPullStages;
    volatile HalfCtl* ctl = reinterpret_cast<volatile HalfCtl*>(empty + kPullStages);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) {
        for (int s = 0; s < n_stages; s++) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(xsmem_u32(&full[s])));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 4;" ::"r"(xsmem_u32(&empty[s])));
        }
        ctl->abort = 0;
        ctl->issued = 0xffffffffu;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const int64_t total_v = (int64_t)a.max_blocks * (a.world - 1);
    const uint32_t dst_row_bytes = a.row_bytes * 2;     // fp32 rows on this side
    if (warp == 0) {
        uint32_t it = 0, ready_mask = 0;
        bool ok = true;
        BlockCursor cur;
        cur.v = blockIdx.x;
        cursor_advance(a, cur, total_v, lane);
        while (ok && cur.have) {
            const int q = cur.q;
            if (!((ready_mask >> q) & 1u)) {
                int r = 1;
                if (lane == 0) r = wait_epoch(a.my_flags + flag_index(a.slot, 0, q), a.epoch, a.wait_ns) ? 1 : 0;
                r = __shfl_sync(kFull, r, 0);
                if (!r) {
                    if (lane == 0) report(a.error, 0x100 + q);
                    ok = false;
                    break;
                }
                ready_mask |= 1u << q;
                asm volatile("fence.proxy.async;" ::: "memory");
            }
            const int s = (int)(it % (uint32_t)n_stages);
            if (it >= (uint32_t)n_stages && !xmbar_wait(&empty[s], ((it / (uint32_t)n_stages) - 1u) & 1u)) {
                if (lane == 0) report(a.error, 0x300);
                ok = false;
                break;
            }
            cursor_issue(a, cur, xsmem_u32(smem + (size_t)s * stage_bytes), xsmem_u32(&full[s]), lane);
            it++;
            cursor_advance(a, cur, total_v, lane);
        }
        if (!ok && lane == 0) {
            ctl->issued = it;
            __threadfence_block();
            ctl->abort = 1;
        }
    } else {
        int64_t v = blockIdx.x;
        uint32_t it = 0;
        const int t = threadIdx.x - 32;    // 0..127
        for (;;) {
            int q = 0, cnt = 0;
            int64_t r0 = 0;
            bool found = false;
            while (v < total_v && !found) {
                found = decode_block(a, v, q, r0, cnt);
                v += gridDim.x;
            }
            if (!found) break;
            const int s = (int)(it % (uint32_t)n_stages);
            const uint32_t addr = xsmem_u32(&full[s]);
            const uint32_t parity = (it / (uint32_t)n_stages) & 1u;
            bool landed = false;
            for (uint32_t spin = 0; spin < kPullSpins; spin++) {
                uint32_t done;
                asm volatile(
                    "{\n\t.reg .pred p;\n\t"
                    "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                    "selp.u32 %0, 1, 0, p;\n\t}"
                    : "=r"(done) : "r"(addr), "r"(parity) : "memory");
                if (done) { landed = true; break; }
                if (ctl->abort && it >= ctl->issued) break;      // this block was never requested
                if (spin > 32) __nanosleep(spin > 4096 ? 512 : 64);
            }
            if (!landed) break;
            const uint4* src = reinterpret_cast<const uint4*>(smem + (size_t)s * stage_bytes);
            float4* dst = reinterpret_cast<float4*>(a.halo + (size_t)r0 * dst_row_bytes);
            const int n16 = (int)(((uint32_t)cnt * a.row_bytes) >> 4);    // 16-byte groups of 8 fp16 values
            for (int e = t; e < n16; e += 128) {
                const uint4 raw = src[e];
                const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
                const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
                const float2 c = __half22float2(*reinterpret_cast<const __half2*>(&raw.z));
                const float2 dd = __half22float2(*reinterpret_cast<const __half2*>(&raw.w));
                dst[2 * e] = make_float4(a.x, a.y, b.x, b.y);
                dst[2 * e + 1] = make_float4(c.x, c.y, dd.x, dd.y);
            }
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(xsmem_u32(&empty[s])) : "memory");
            it++;
        }
    }
    __syncthreads();
    finish_pull(a, ctl->abort == 0);
}

// fp32 -> fp16 (round to nearest even, values beyond the fp16 range saturate at +-65504) of the rows an
// owner offers to its readers.
__device__ __forceinline__ float clamp_half(float v) { return fminf(fmaxf(v, -65504.f), 65504.f); }
__global__ void __launch_bounds__(256) rows_to_half_kernel(__half* __restrict__ out, const float* __restrict__ x, int64_t n4) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
        const float4 v = __ldcs(reinterpret_cast<const float4*>(x) + i);
        __half2 a = __floats2half2_rn(clamp_half(v.x), clamp_half(v.y)), b = __floats2half2_rn(clamp_half(v.z), clamp_half(v.w));
        uint2 packed;
        packed.x = *reinterpret_cast<uint32_t*>(&a);
        packed.y = *reinterpret_cast<uint32_t*>(&b);
        reinterpret_cast<uint2*>(out)[i] = packed;
    }
}

// Plain loads from peer memory.  Bulk copies are issued at a fixed rate per SM whatever their size (about
// 18 million a second on this part), so rows shorter than 1 KB are fetched faster by ordinary
// 16-byte loads with many of them in flight: G lanes share a row (G * 16 bytes per step), 32 / G rows are
// walked side by side, four steps unrolled.  HALF: the source rows are fp16 and are widened to fp32 here.
// Rows that are not multiples of 16 bytes fall back to 4-byte loads, one warp per row.
template <bool HALF>
__global__ void __launch_bounds__(256) halo_pull_rows_kernel(PullArgs a, int lanes_per_row) {
    __shared__ int s_ok;
    const int lane = lane_id(), warp = threadIdx.x / 32;
    const int64_t total_v = (int64_t)a.max_blocks * (a.world - 1);
    uint32_t ready_mask = 0;
    bool ok = true;
    const bool vec = lanes_per_row > 0;       // 0: rows or pointers that 16-byte accesses cannot take
    const uint32_t dst_row_bytes = HALF ? a.row_bytes * 2 : a.row_bytes;
    const int G = vec ? lanes_per_row : 32, sub = lane / G, gl = lane % G, rows_per_step = 32 / G;
    const uint32_t chunks = a.row_bytes / 16;     // 16-byte pieces of a source row
    for (int64_t v = blockIdx.x; v < total_v && ok; v += gridDim.x) {
        int q = 0, cnt = 0;
        int64_t r0 = 0;
        if (!decode_block(a, v, q, r0, cnt)) continue;
        if (!((ready_mask >> q) & 1u)) {
            if (threadIdx.x == 0) {
                s_ok = wait_epoch(a.my_flags + flag_index(a.slot, 0, q), a.epoch, a.wait_ns) ? 1 : 0;
                if (!s_ok) report(a.error, 0x100 + q);
            }
            __syncthreads();
            const int r = s_ok;
            __syncthreads();
            if (!r) { ok = false; break; }
            ready_mask |= 1u << q;
        }
        const unsigned char* base = static_cast<const unsigned char*>(a.t.x[q]);
        const int32_t lo = a.t.lo[q];
        if (vec) {
            constexpr int U = 4;
            for (int i0 = warp * rows_per_step * U; i0 < cnt; i0 += 8 * rows_per_step * U) {
                int32_t id[U];
#pragma unroll
                for (int u = 0; u < U; u++) {
                    const int i = i0 + u * rows_per_step + sub;
                    id[u] = i < cnt ? __ldg(a.needed + r0 + i) : lo;
                }
                for (uint32_t c = gl; c < chunks; c += G) {
                    uint4 val[U];
#pragma unroll
                    for (int u = 0; u < U; u++) {
                        const int i = i0 + u * rows_per_step + sub;
                        val[u] = make_uint4(0, 0, 0, 0);
                        if (i < cnt) val[u] = *reinterpret_cast<const uint4*>(base + (size_t)(id[u] - lo) * a.row_bytes + (size_t)c * 16);
                    }
#pragma unroll
                    for (int u = 0; u < U; u++) {
                        const int i = i0 + u * rows_per_step + sub;
                        if (i >= cnt) continue;
                        unsigned char* dst = a.halo + (size_t)(r0 + i) * dst_row_bytes;
                        if (HALF) {
                            const float2 p0 = __half22float2(*reinterpret_cast<const __half2*>(&val[u].x));
                            const float2 p1 = __half22float2(*reinterpret_cast<const __half2*>(&val[u].y));
                            const float2 p2 = __half22float2(*reinterpret_cast<const __half2*>(&val[u].z));
                            const float2 p3 = __half22float2(*reinterpret_cast<const __half2*>(&val[u].w));
                            reinterpret_cast<float4*>(dst)[2 * c] = make_float4(p0.x, p0.y, p1.x, p1.y);
                            reinterpret_cast<float4*>(dst)[2 * c + 1] = make_float4(p2.x, p2.y, p3.x, p3.y);
                        } else {
                            reinterpret_cast<uint4*>(dst)[c] = val[u];
                        }
                    }
                }
            }
        } else {
            const uint32_t words = a.row_bytes / 4;
            for (int i = warp; i < cnt; i += 8) {
                const int32_t id = __ldg(a.needed + r0 + i);
                const unsigned char* src = base + (size_t)(id - lo) * a.row_bytes;
                unsigned char* dst = a.halo + (size_t)(r0 + i) * a.row_bytes;
                for (uint32_t c = lane; c < words; c += 32)
                    reinterpret_cast<float*>(dst)[c] = reinterpret_cast<const float*>(src)[c];
            }
        }
    }
    finish_pull(a, ok);
}

static int fill_table(PeerTable* t, int world, void* const* peer_x, void* const* peer_flags, const int64_t* seg_begin,
                      const int32_t* lo) {
    for (int q = 0; q < world; q++) {
        t->x[q] = peer_x ? peer_x[q] : nullptr;
        t->flags[q] = static_cast<uint32_t*>(peer_flags[q]);
        if (seg_begin) {
            t->seg_begin[q] = seg_begin[q];
            t->seg_end[q] = seg_begin[q + 1];
        }
        if (lo) t->lo[q] = lo[q];
    }
    if (seg_begin) t->seg_begin[world] = seg_begin[world];
    return JG_OK;
}

}  // namespace jg

using namespace jg;

extern "C" {

size_t jg_halo_flag_bytes(void) { return sizeof(uint32_t) * kFlagSlots * 2 * kMaxRanks; }
int jg_halo_max_ranks(void) { return kMaxRanks; }
int jg_halo_flag_slots(void) { return kFlagSlots; }

int jg_halo_post(void* const* peer_flags_host, int world, int rank, int slot, int kind, uint32_t epoch, jg_stream_t stream) {
    JG_CHECK_ARG(peer_flags_host && world >= 1 && world <= kMaxRanks && rank >= 0 && rank < world, JG_EINVAL,
                 "halo_post: bad rank/world (at most %d ranks)", kMaxRanks);
    JG_CHECK_ARG(slot >= 0 && slot < kFlagSlots && (kind == 0 || kind == 1), JG_EINVAL, "halo_post: bad slot or kind");
    PeerTable t = {};
    fill_table(&t, world, nullptr, peer_flags_host, nullptr, nullptr);
    halo_post_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(t, world, rank, slot, kind, epoch);
    JG_LAUNCH_CHECK();
    return JG_OK;
}

int jg_halo_wait(const void* my_flags, int world, int rank, int slot, int kind, uint32_t epoch, int32_t* error,
                 int64_t wait_ns, jg_stream_t stream) {
    JG_CHECK_ARG(my_flags && world >= 1 && world <= kMaxRanks && rank >= 0 && rank < world, JG_EINVAL, "halo_wait: bad rank/world");
    JG_CHECK_ARG(slot >= 0 && slot < kFlagSlots && (kind == 0 || kind == 1) && wait_ns > 0, JG_EINVAL, "halo_wait: bad slot, kind or limit");
    halo_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const uint32_t*>(my_flags), world, rank, slot,
                                                                      kind, epoch, error, (uint64_t)wait_ns);
    JG_LAUNCH_CHECK();
    return JG_OK;
}

static int halo_pull_impl(void* halo, const int32_t* needed, void* const* peer_x_host, void* const* peer_flags_host,
                          const int64_t* seg_begin_host, const int64_t* part_begin_host, const int64_t* part_end_host,
                          const int32_t* lo_host, int world, int rank, int64_t row_bytes, int slot, uint32_t epoch, void* counter,
                          int32_t* error, int64_t wait_ns, int max_ctas, int plain, int src_half, jg_stream_t stream) {
    JG_CHECK_ARG(world >= 1 && world <= kMaxRanks && rank >= 0 && rank < world, JG_EINVAL, "halo_pull: bad rank/world");
    JG_CHECK_ARG(peer_x_host && peer_flags_host && seg_begin_host && lo_host && counter, JG_EINVAL, "halo_pull: null table");
    JG_CHECK_ARG(slot >= 0 && slot < kFlagSlots && wait_ns > 0, JG_EINVAL, "halo_pull: bad slot or limit");
    JG_CHECK_ARG(row_bytes > 0 && row_bytes % 4 == 0 && row_bytes < (int64_t(1) << 24), JG_ESHAPE, "halo_pull: row bytes must be a multiple of 4");
    JG_CHECK_ARG(seg_begin_host[world] >= 0 && seg_begin_host[rank + 1] == seg_begin_host[rank], JG_EINVAL,
                 "halo_pull: a rank's own segment must be empty");
    JG_CHECK_ARG((part_begin_host == nullptr) == (part_end_host == nullptr), JG_EINVAL, "halo_pull: part bounds come in pairs");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    PullArgs a = {};
    a.halo = static_cast<unsigned char*>(halo);
    a.needed = needed;
    fill_table(&a.t, world, peer_x_host, peer_flags_host, seg_begin_host, lo_host);
    int64_t n_halo = 0;          // rows this call fetches
    for (int q = 0; q < world; q++) {
        if (part_begin_host) {
            JG_CHECK_ARG(part_begin_host[q] >= seg_begin_host[q] && part_begin_host[q] <= part_end_host[q] &&
                             part_end_host[q] <= seg_begin_host[q + 1], JG_EINVAL, "halo_pull: a part must lie inside its owner's segment");
            a.t.seg_begin[q] = part_begin_host[q];
            a.t.seg_end[q] = part_end_host[q];
        }
        n_halo += a.t.seg_end[q] - a.t.seg_begin[q];
    }
    a.world = world; a.rank = rank; a.row_bytes = (uint32_t)row_bytes;
    a.my_flags = a.t.flags[rank];
    a.slot = slot; a.epoch = epoch;
    a.counter = static_cast<unsigned int*>(counter);
    a.error = error; a.wait_ns = (uint64_t)wait_ns;
    if (world == 1 || n_halo == 0) {
        // nothing to fetch: the owners still learn that this rank is done with the epoch
        halo_post_kernel<<<1, 32, 0, st>>>(a.t, world, rank, slot, 1, epoch);
        JG_LAUNCH_CHECK();
        return JG_OK;
    }
    JG_CHECK_ARG(halo && needed, JG_EINVAL, "halo_pull: null halo/needed");
    // about 16 KB per stage, whole multiples of 32 rows
    int64_t rpb = (16384 / row_bytes) / 32 * 32;
    if (rpb < 32) rpb = 32;
    if (rpb > 32 * kMaxIdsPerLane) rpb = 32 * kMaxIdsPerLane;
    a.rows_per_block = (int32_t)rpb;
    int64_t total_blocks = 0;
    a.max_blocks = 0;
    for (int j = 0; j < world - 1; j++) a.t.order[j] = (rank + 1 + j) % world;
    for (int q = 0; q < world; q++) {
        const int64_t rows = a.t.seg_end[q] - a.t.seg_begin[q];
        JG_CHECK_ARG(rows >= 0, JG_EINVAL, "halo_pull: segment bounds must not decrease");
        const int64_t nb = (rows + rpb - 1) / rpb;
        a.t.n_blocks[q] = (int32_t)nb;
        total_blocks += nb;
        if (nb > a.max_blocks) a.max_blocks = (int32_t)nb;
    }
    const size_t stage_bytes = (size_t)rpb * (size_t)row_bytes;
    int n_stages = kPullStages;
    while (n_stages > 2 && (size_t)n_stages * stage_bytes > 200 * 1024) n_stages--;
    const bool bulk = !plain && row_bytes % 16 == 0 && (size_t)n_stages * stage_bytes <= 200 * 1024 &&
                      (reinterpret_cast<uintptr_t>(halo) % 16 == 0);
    int64_t grid = total_blocks;
    if (max_ctas <= 0) max_ctas = 2 * sm_count();   // nothing runs beside this pull: two warps' worth of requests per SM
    if (max_ctas > 0xffff) max_ctas = 0xffff;
    // bulk copies pay off from 1 KB rows on; shorter rows take the plain-load kernel
    const bool use_bulk = bulk && row_bytes >= 1024;
    int lanes_per_row = 1;
    while (lanes_per_row < 32 && lanes_per_row * 16 < row_bytes) lanes_per_row *= 2;
    {
        uintptr_t bits = reinterpret_cast<uintptr_t>(halo) | (uintptr_t)row_bytes;
        for (int q = 0; q < world; q++) bits |= reinterpret_cast<uintptr_t>(peer_x_host[q]);
        if (bits % 16 != 0) lanes_per_row = 0;
    }
    if (grid > 0xffff) grid = 0xffff;
    if (src_half) {
        JG_CHECK_ARG(lanes_per_row > 0, JG_EUNSUPPORTED,
                     "halo_pull: the fp16 payload needs rows that are multiples of 16 bytes (width %% 8 == 0)");
        if (!use_bulk) {
            if (grid > 4 * (int64_t)max_ctas) grid = 4 * (int64_t)max_ctas;
            halo_pull_rows_kernel<true><<<(unsigned)grid, 256, 0, st>>>(a, lanes_per_row);
            JG_LAUNCH_CHECK();
            return JG_OK;
        }
        if (grid > max_ctas) grid = max_ctas;
        const size_t smem = (size_t)n_stages * stage_bytes + sizeof(uint64_t) * 2 * kPullStages + sizeof(HalfCtl) + 128;
        static size_t attr_half[64] = {0};
        int dev = 0;
        JG_CUDA(cudaGetDevice(&dev));
        if (dev >= 0 && dev < 64 && attr_half[dev] < smem) {
            JG_CUDA(cudaFuncSetAttribute(halo_pull_half_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(208 * 1024)));
            attr_half[dev] = 208 * 1024;
        }
        halo_pull_half_kernel<<<(unsigned)grid, 160, smem, st>>>(a, (uint32_t)stage_bytes, n_stages);
        JG_LAUNCH_CHECK();
        return JG_OK;
    }
    if (use_bulk) {
        bool aligned = true;
        for (int q = 0; q < world; q++) aligned = aligned && (reinterpret_cast<uintptr_t>(peer_x_host[q]) % 16 == 0);
        JG_CHECK_ARG(aligned, JG_EINVAL, "halo_pull: peer buffers must be 16-byte aligned");
        if (grid > max_ctas) grid = max_ctas;
        const size_t smem = (size_t)n_stages * stage_bytes + sizeof(uint64_t) * kPullStages + 128;
        static size_t attr_done[64] = {0};
        int dev = 0;
        JG_CUDA(cudaGetDevice(&dev));
        if (dev >= 0 && dev < 64 && attr_done[dev] < smem) {
            JG_CUDA(cudaFuncSetAttribute(halo_pull_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(208 * 1024)));
            attr_done[dev] = 208 * 1024;
        }
        halo_pull_bulk_kernel<<<(unsigned)grid, 32, smem, st>>>(a, (uint32_t)stage_bytes, n_stages);
    } else {
        // 256-thread CTAs: up to four per SM slot the caller granted
        if (grid > 4 * (int64_t)max_ctas) grid = 4 * (int64_t)max_ctas;
        halo_pull_rows_kernel<false><<<(unsigned)grid, 256, 0, st>>>(a, lanes_per_row);
    }
    JG_LAUNCH_CHECK();
    return JG_OK;
}

int jg_halo_pull(void* halo, const int32_t* needed, void* const* peer_x_host, void* const* peer_flags_host,
                 const int64_t* seg_begin_host, const int32_t* lo_host, int world, int rank, int64_t row_bytes, int slot,
                 uint32_t epoch, void* counter, int32_t* error, int64_t wait_ns, int max_ctas, int plain, int src_half,
                 jg_stream_t stream) {
    return halo_pull_impl(halo, needed, peer_x_host, peer_flags_host, seg_begin_host, nullptr, nullptr, lo_host, world, rank,
                          row_bytes, slot, epoch, counter, error, wait_ns, max_ctas, plain, src_half, stream);
}

int jg_halo_pull_part(void* halo, const int32_t* needed, void* const* peer_x_host, void* const* peer_flags_host,
                      const int64_t* seg_begin_host, const int64_t* part_begin_host, const int64_t* part_end_host,
                      const int32_t* lo_host, int world, int rank, int64_t row_bytes, int slot, uint32_t epoch, void* counter,
                      int32_t* error, int64_t wait_ns, int max_ctas, int plain, int src_half, jg_stream_t stream) {
    JG_CHECK_ARG(part_begin_host && part_end_host, JG_EINVAL, "halo_pull_part: null part bounds");
    return halo_pull_impl(halo, needed, peer_x_host, peer_flags_host, seg_begin_host, part_begin_host, part_end_host, lo_host,
                          world, rank, row_bytes, slot, epoch, counter, error, wait_ns, max_ctas, plain, src_half, stream);
}

int jg_rows_to_half(void* out, const float* x, int64_t n_values, jg_stream_t stream) {
    JG_CHECK_ARG(n_values >= 0 && n_values % 4 == 0, JG_ESHAPE, "rows_to_half: the value count must be a multiple of 4");
    if (n_values == 0) return JG_OK;
    JG_CHECK_ARG(out && x && reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 8 == 0, JG_EINVAL,
                 "rows_to_half: null or misaligned pointer");
    int64_t blocks = (n_values / 4 + 255) / 256;
    const int64_t cap = (int64_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    rows_to_half_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<__half*>(out), x, n_values / 4);
    JG_LAUNCH_CHECK();
    return JG_OK;
}

}  // extern "C"
