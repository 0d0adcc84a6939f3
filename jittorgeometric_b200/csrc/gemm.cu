// Dense feature transform  H = act(X * W + b)  on the 5th-generation tensor cores (sm_100a).
//
// Replaces the `x @ self.weight` of the reference layers (nn/conv/gcn_conv.py:95,
// nn/conv/gat_conv.py:86), which Jittor hands to cuBLAS.  It is the only tensor-core kernel of
// the path; shapes are skinny (K, M <= a few hundred, N in the millions), so the bound is HBM
// (read X once, write H once) and the point of tcgen05 is to keep the SMs out of the way.
//
//   X  [N, K]  fp32 row-major      (A operand, K-major)
//   Wt [M, K]  fp32 row-major      (B operand, K-major: the layer weight transposed once)
//   H  [N, M]  fp32                (TF32 products, fp32 accumulation in TMEM)
//
// One CTA per SM, persistent over 128-row tiles.  Warp 0 (one lane) is the TMA producer: 128x32
// tiles of X and Mx32 tiles of Wt land in a 4-stage shared-memory ring with the 128-byte swizzle
// (cp.async.bulk.tensor, CTA-local, no cluster multicast; out-of-range rows and the K tail are
// zero-filled by TMA).  When K is not a multiple of 4 (row pitch not a multiple of 16 bytes, which
// TMA cannot address) warp 0 fills the ring with plain coalesced loads in the same layout.  Warp 1 (one lane) issues tcgen05.mma.kind::tf32 (128 x M x 8 per
// instruction) into one of two TMEM accumulators and commits ring slots / accumulators to
// mbarriers.  Warps 2-9 are the epilogue: tcgen05.ld of the accumulator quadrant their warp id
// gives them access to, bias and ReLU fused, each warp's 32x32 block staged in shared memory and
// written to H by a bulk tensor store (TMA), overlapping the next tile's MMAs.  Every mbarrier wait is bounded; a wait that runs out sets an error word that
// the host reads, and the CTA still frees its TMEM and exits.
#include "common.cuh"

#include <cuda.h>
#include <cuda_fp16.h>
#include <cstring>

namespace jg {

constexpr int kGemmThreads = 416;   // 13 warps: producer, MMA, 8 epilogue, 3 more plain-load producers
constexpr int kEpiWarps = 8;
constexpr int kPlainWarps = 4;      // warps 0, 10, 11, 12 when operands are fetched by plain loads
constexpr int kTileM = 128;         // rows of X per tile
constexpr int kTileK = 32;          // tf32 elements per 128-byte swizzle row
constexpr int kStages = 4;
constexpr uint32_t kWaitSpins = 1u << 22;  // bounded mbarrier wait (about a second with back-off)

struct GemmParams {
    float* out;
    const float* bias;
    int64_t n_rows;
    int32_t k, m;       // reduction length, output width
    int32_t m_pad;      // TMEM columns per accumulator (power of two >= 32)
    int32_t relu;
    int32_t n_tiles, k_blocks;
    int32_t* error;
    const float* x;     // plain-load producer only (rows whose pitch TMA cannot take)
    const float* wt;
    int32_t plain_loads;
    int32_t tma_store;   // epilogue stages 32x32 blocks in shared memory and stores them by TMA
    int32_t ldo;         // row pitch of the output in floats (the full width when m is one column tile of it)
    int32_t col_base;    // first output column of this tile (out, bias and wt already point at it)
    __half* out_half;    // optional second copy of the result in fp16 (same shape and pitch in elements), or null
    uint32_t wait_spins; // limit of every mbarrier wait (kWaitSpins; the time-out test entry shortens it)
    int32_t withhold;    // time-out test entry only: the producer skips this fill of the ring (-1: none)
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Bounded wait for the phase with the given parity; false when it ran out.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint32_t spins = kWaitSpins) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t spin = 0; spin < spins; spin++) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
        if (spin > 64) __nanosleep(spin > 4096 ? 256 : 32);
    }
    return false;
}

// 4-byte asynchronous global->shared copy; valid == false writes zeros.
__device__ __forceinline__ void cp_async4(uint32_t smem_dst, const float* src, bool valid) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(smem_dst), "l"(src), "r"(valid ? 4 : 0) : "memory");
}

// 8-byte variant (row pitch and base a multiple of 8 bytes): half the requests per tile.
__device__ __forceinline__ void cp_async8(uint32_t smem_dst, const float* src, bool valid) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(smem_dst), "l"(src), "r"(valid ? 8 : 0) : "memory");
}

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(smem_dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}

// Shared-memory matrix descriptor: K-major tile, 128-byte swizzle, rows 128 B apart, 8-row groups
// 1024 B apart (stride byte offset), descriptor version 1.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    return (uint64_t)((smem_addr >> 4) & 0x3FFF) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}

__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; i++) v[i] = __uint_as_float(r[i]);
}

// 32 accumulator columns of this lane's row: two 16-column loads in flight, one wait.  The second
// load is skipped (zeros) when it would reach past the accumulator's columns.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32], bool second) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    if (second) {
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
            : "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
              "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
            : "r"(taddr + 16));
    } else {
#pragma unroll
        for (int i = 16; i < 32; i++) r[i] = 0;
    }
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; i++) v[i] = __uint_as_float(r[i]);
}

struct GemmSmem {
    uint64_t full[kStages], empty[kStages];
    uint64_t acc_full[2], acc_empty[2];
    uint32_t tmem_base;
    int32_t abort;
};

__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tf32_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                 const __grid_constant__ CUtensorMap map_out, const __grid_constant__ CUtensorMap map_half, GemmParams p) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // ring first (1024-byte aligned stages), control block after it
    unsigned char* ring = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t a_bytes = kTileM * kTileK * 4;                    // 16 KB
    const uint32_t b_rows = (uint32_t)((p.m + 15) / 16 * 16);   // MMA N: a multiple of 16 when M = 128
    const uint32_t b_bytes = ((b_rows * kTileK * 4) + 1023) / 1024 * 1024;
    const uint32_t stage_bytes = a_bytes + b_bytes;
    unsigned char* slabs = ring + kStages * stage_bytes;                 // 4 KB per epilogue warp (TMA-store epilogue)
    unsigned char* hslabs = slabs + (p.tma_store ? kEpiWarps * 4096 : 0);   // 2 KB per epilogue warp (fp16 copy)
    GemmSmem* ctl = reinterpret_cast<GemmSmem*>(hslabs + (p.out_half ? kEpiWarps * 2048 : 0));
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; s++) {
            mbar_init(&ctl->full[s], p.plain_loads ? 32 * kPlainWarps : 1);   // one arrival per producer lane, or the TMA lane's
            mbar_init(&ctl->empty[s], 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(&ctl->acc_full[b], 1);
            mbar_init(&ctl->acc_empty[b], kEpiWarps);   // one arrival per epilogue warp
        }
        ctl->abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 2) {  // TMEM: two accumulators of m_pad columns
        const uint32_t cols = (uint32_t)(2 * p.m_pad);
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctl->tmem_base)), "r"(cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = ctl->tmem_base;
    volatile int32_t* abort_flag = &ctl->abort;

    if ((warp == 0 || warp >= 10) && p.plain_loads) {
        const uint32_t pw = warp == 0 ? 0u : (uint32_t)(warp - 9);   // producer index 0..3: rows pw, pw + 4, ...
        // ---------------------------------------------------------------- plain-load producer
        // For K not a multiple of 4 the row pitch is not a multiple of 16 bytes and TMA cannot
        // address the matrix.  Four warps then fill the ring themselves (one warp cannot keep enough
        // requests in flight): per row and k-block one
        // coalesced 128-byte read (cp.async, 4 bytes per lane) lands in shared memory in the same
        // 128-byte swizzle TMA would have produced (16-byte chunk c of row r at chunk c ^ (r & 7)).
        // Each lane's arrival on the slot's barrier fires when its copies have landed; the MMA
        // lane orders them before the tensor core's asynchronous proxy with a proxy fence.
        uint32_t it = 0;
        const uint32_t chunk_off = (uint32_t)(lane >> 2), in_chunk = (uint32_t)(lane & 3) * 4;
        bool ok = true;
        for (int tile = blockIdx.x; tile < p.n_tiles && ok && !*abort_flag; tile += gridDim.x) {
            for (int kb = 0; kb < p.k_blocks; kb++, it++) {
                const int s = it % kStages;
                const uint32_t round = it / kStages;
                if (round > 0 && !mbar_wait(&ctl->empty[s], (round - 1) & 1, p.wait_spins)) { ok = false; break; }
                const uint32_t a_dst = smem_u32(ring + s * stage_bytes);
                const int64_t row0 = (int64_t)tile * kTileM;
                // Everything that does not change from row to row is worked out once per k-block: a lane's rows are
                // r = r_first + 8 j (8-byte form) or r = pw + 4 j (4-byte form), so r & 7 - the swizzle term - is fixed
                // (or alternates between two values), the destination advances by whole 1024-byte groups and the
                // source by a fixed number of rows.  The loop body is one copy and two additions; the first version
                // recomputed addresses, swizzle and bounds per copy (about 50 instructions each) and the four producer
                // warps, not memory, set the pace (602 -> 64 on 233 k rows: 0.45 ms).
                const bool full_tile = row0 + kTileM <= p.n_rows;
                if (p.plain_loads == 2) {
                    // even K: a lane copies two neighbouring values, a half-warp one 128-byte row segment, a
                    // warp two rows per instruction
                    const uint32_t half = (uint32_t)lane >> 4, hl = (uint32_t)lane & 15u;
                    const int kc = kb * kTileK + 2 * (int)hl;
                    const bool kin2 = kc < p.k;
                    const uint32_t r_first = 2 * pw + half;                       // 0..7 = r & 7 for all of this lane's rows
                    const uint32_t lane_off = r_first * 128 + (((hl >> 1) ^ r_first) << 4) + (hl & 1u) * 8u;
                    const int64_t step = 8 * (int64_t)p.k;
                    {
                        const uint32_t dst = a_dst + lane_off;
                        const float* src = p.x + (row0 + r_first) * p.k + kc;
                        if (full_tile && kin2) {
#pragma unroll
                            for (int j = 0; j < kTileM / 8; j++) cp_async8(dst + j * 1024, src + j * step, true);
                        } else {
#pragma unroll
                            for (int j = 0; j < kTileM / 8; j++) {
                                const bool in = kin2 && row0 + r_first + 8 * j < p.n_rows;
                                cp_async8(dst + j * 1024, in ? src + j * step : p.x, in);
                            }
                        }
                    }
                    {
                        const uint32_t dst = a_dst + a_bytes + lane_off;
                        const float* src = p.wt + (int64_t)r_first * p.k + kc;
                        const int groups = (int)b_rows / 8;
                        for (int j = 0; j < groups; j++) {
                            const bool in = kin2 && (int)(r_first + 8 * j) < p.m;
                            cp_async8(dst + j * 1024, in ? src + j * step : p.wt, in);
                        }
                    }
                    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(&ctl->full[s])) : "memory");
                    continue;
                }
                const int kcol = kb * kTileK + lane;
                const bool kin = kcol < p.k;
                // asynchronous 4-byte copies straight into shared memory (zero-filled outside the
                // matrix): nothing waits here, the barrier counts the copies as they land.  Rows r = pw + 4 j:
                // r & 7 is pw for even j and pw + 4 for odd j.
                const uint32_t off_even = pw * 128 + ((chunk_off ^ pw) << 4) + in_chunk;
                const uint32_t off_odd = (pw + 4) * 128 + ((chunk_off ^ (pw + 4)) << 4) + in_chunk;
                const int64_t step = 8 * (int64_t)p.k;
                {
                    const float* src_even = p.x + (row0 + pw) * p.k + kcol;
                    const float* src_odd = src_even + 4 * (int64_t)p.k;
                    if (full_tile && kin) {
#pragma unroll
                        for (int j = 0; j < kTileM / 8; j++) {
                            cp_async4(a_dst + off_even + j * 1024, src_even + j * step, true);
                            cp_async4(a_dst + off_odd + j * 1024, src_odd + j * step, true);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < kTileM / 8; j++) {
                            const bool in_e = kin && row0 + pw + 8 * j < p.n_rows, in_o = kin && row0 + pw + 4 + 8 * j < p.n_rows;
                            cp_async4(a_dst + off_even + j * 1024, in_e ? src_even + j * step : p.x, in_e);
                            cp_async4(a_dst + off_odd + j * 1024, in_o ? src_odd + j * step : p.x, in_o);
                        }
                    }
                }
                {
                    const uint32_t b_dst = a_dst + a_bytes;
                    const float* src_even = p.wt + (int64_t)pw * p.k + kcol;
                    const float* src_odd = src_even + 4 * (int64_t)p.k;
                    const int groups = (int)b_rows / 8;
                    for (int j = 0; j < groups; j++) {
                        const bool in_e = kin && (int)(pw + 8 * j) < p.m, in_o = kin && (int)(pw + 4 + 8 * j) < p.m;
                        cp_async4(b_dst + off_even + j * 1024, in_e ? src_even + j * step : p.wt, in_e);
                        cp_async4(b_dst + off_odd + j * 1024, in_o ? src_odd + j * step : p.wt, in_o);
                    }
                }
                asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(&ctl->full[s])) : "memory");
            }
        }
        if (!ok) *abort_flag = 1;
    } else if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0) {
            uint32_t it = 0;
            for (int tile = blockIdx.x; tile < p.n_tiles && !*abort_flag; tile += gridDim.x) {
                for (int kb = 0; kb < p.k_blocks; kb++, it++) {
                    const int s = it % kStages;
                    const uint32_t round = it / kStages;
                    if (round > 0 && !mbar_wait(&ctl->empty[s], (round - 1) & 1, p.wait_spins)) { *abort_flag = 1; break; }
                    if ((int32_t)it == p.withhold) continue;   // test entry: this fill never arrives, its consumer's wait runs out
                    unsigned char* a_dst = ring + s * stage_bytes;
                    mbar_expect_tx(&ctl->full[s], a_bytes + b_rows * kTileK * 4);
                    tma_load_2d(a_dst, &map_x, kb * kTileK, tile * kTileM, &ctl->full[s]);
                    tma_load_2d(a_dst + a_bytes, &map_w, kb * kTileK, 0, &ctl->full[s]);
                }
            }
        }
    } else if (warp >= 10) {
        // spare producer warps: idle when TMA feeds the ring
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            // instruction descriptor: D fp32, A/B tf32, both K-major, N = b_rows, M = 128
            const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((b_rows >> 3) << 17) | ((kTileM >> 4) << 24);
            uint32_t it = 0, local_tile = 0;
            for (int tile = blockIdx.x; tile < p.n_tiles && !*abort_flag; tile += gridDim.x, local_tile++) {
                const int b = local_tile & 1;
                const uint32_t use = local_tile >> 1;
                if (use > 0 && !mbar_wait(&ctl->acc_empty[b], (use - 1) & 1, p.wait_spins)) { *abort_flag = 1; break; }
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + (uint32_t)(b * p.m_pad);
                bool ok = true;
                for (int kb = 0; kb < p.k_blocks; kb++, it++) {
                    const int s = it % kStages;
                    if (!mbar_wait(&ctl->full[s], (it / kStages) & 1, p.wait_spins)) { ok = false; break; }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // plain-load producer: generic-proxy writes
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(ring + s * stage_bytes);
                    const uint64_t da = umma_desc(a_addr), db = umma_desc(a_addr + a_bytes);
#pragma unroll
                    for (int k = 0; k < kTileK / 8; k++)   // 8 tf32 = 32 bytes per instruction: +2 in 16-byte units
                        umma_tf32(tmem_d, da + 2 * k, db + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    umma_commit(&ctl->empty[s]);            // slot free once these MMAs have read it
                }
                if (!ok) { *abort_flag = 1; break; }
                umma_commit(&ctl->acc_full[b]);             // accumulator complete
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue (warps 2..9)
        // A warp may read the TMEM lanes 32*(warp % 4) .. +31; two warps share a quadrant and take
        // alternate 32-column chunks.
        const int quad = warp & 3;
        const int half = (warp - 2) >> 2;
        const bool full_chunks = (p.m % 32) == 0 && (p.ldo % 4) == 0;   // 16-byte stores need 16-byte aligned row starts
        uint32_t local_tile = 0;
        for (int tile = blockIdx.x; tile < p.n_tiles && !*abort_flag; tile += gridDim.x, local_tile++) {
            const int b = local_tile & 1;
            if (!mbar_wait(&ctl->acc_full[b], (local_tile >> 1) & 1, p.wait_spins)) { *abort_flag = 1; break; }
            tc_fence_after();
            const int64_t row = (int64_t)tile * kTileM + quad * 32 + lane;
            const uint32_t taddr = tmem_base + (uint32_t)(b * p.m_pad) + ((uint32_t)(quad * 32) << 16);
            for (int c0 = half * 32; c0 < p.m; c0 += 64) {
                float v[32];
                tmem_ld32(taddr + (uint32_t)c0, v, c0 + 16 < (int)b_rows);
                if (p.tma_store) {
                    // bias / ReLU, then the warp's 32x32 block goes to its slab in the 128-byte swizzle
                    // (16-byte chunk c of row r at chunk c ^ (r & 7)) and leaves as ONE bulk tensor store:
                    // full 128-byte row segments instead of 32 scattered 16-byte stores per instruction.
                    if (p.bias) {
#pragma unroll
                        for (int i = 0; i < 32; i++)
                            if (c0 + i < p.m) v[i] += __ldg(p.bias + c0 + i);
                    }
                    if (p.relu) {
#pragma unroll
                        for (int i = 0; i < 32; i++) v[i] = fmaxf(v[i], 0.f);
                    }
                    unsigned char* slab = slabs + (warp - 2) * 4096;
                    if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // previous store has read the slab
                    __syncwarp();
#pragma unroll
                    for (int c = 0; c < 8; c++)
                        *reinterpret_cast<float4*>(slab + lane * 128 + ((c ^ (lane & 7)) << 4)) =
                            make_float4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
                    unsigned char* hslab = hslabs + (warp - 2) * 2048;
                    if (p.out_half) {
                        // the fp16 copy a partitioned aggregation offers to its peers: the same 32x32 block as 64-byte
                        // rows in the 64-byte swizzle (16-byte chunk c of row r at chunk c ^ ((r >> 1) & 3)), stored
                        // by a second bulk tensor store; values beyond the fp16 range saturate
#pragma unroll
                        for (int c = 0; c < 4; c++) {
                            uint4 pk;
                            __half2 h0 = __floats2half2_rn(fminf(fmaxf(v[8 * c], -65504.f), 65504.f), fminf(fmaxf(v[8 * c + 1], -65504.f), 65504.f));
                            __half2 h1 = __floats2half2_rn(fminf(fmaxf(v[8 * c + 2], -65504.f), 65504.f), fminf(fmaxf(v[8 * c + 3], -65504.f), 65504.f));
                            __half2 h2 = __floats2half2_rn(fminf(fmaxf(v[8 * c + 4], -65504.f), 65504.f), fminf(fmaxf(v[8 * c + 5], -65504.f), 65504.f));
                            __half2 h3 = __floats2half2_rn(fminf(fmaxf(v[8 * c + 6], -65504.f), 65504.f), fminf(fmaxf(v[8 * c + 7], -65504.f), 65504.f));
                            pk.x = *reinterpret_cast<uint32_t*>(&h0); pk.y = *reinterpret_cast<uint32_t*>(&h1);
                            pk.z = *reinterpret_cast<uint32_t*>(&h2); pk.w = *reinterpret_cast<uint32_t*>(&h3);
                            *reinterpret_cast<uint4*>(hslab + lane * 64 + ((c ^ ((lane >> 1) & 3)) << 4)) = pk;
                        }
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) {
                        asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
                                     ::"l"(&map_out), "r"(p.col_base + c0), "r"(tile * kTileM + quad * 32), "r"(smem_u32(slab)) : "memory");
                        if (p.out_half)
                            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
                                         ::"l"(&map_half), "r"(p.col_base + c0), "r"(tile * kTileM + quad * 32), "r"(smem_u32(hslab)) : "memory");
                        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    }
                } else if (row < p.n_rows) {
                    float* o = p.out + row * p.ldo + c0;
                    if (p.bias) {
#pragma unroll
                        for (int i = 0; i < 32; i++)
                            if (full_chunks || c0 + i < p.m) v[i] += __ldg(p.bias + c0 + i);
                    }
                    if (p.relu) {
#pragma unroll
                        for (int i = 0; i < 32; i++) v[i] = fmaxf(v[i], 0.f);
                    }
                    if (full_chunks) {
#pragma unroll
                        for (int i = 0; i < 8; i++)
                            __stcs(reinterpret_cast<float4*>(o) + i, make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]));
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; i++)
                            if (c0 + i < p.m) o[i] = v[i];
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctl->acc_empty[b]);
        }
        if (p.tma_store && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // stores have landed
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 2) {
        const uint32_t cols = (uint32_t)(2 * p.m_pad);
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(cols) : "memory");
    }
    if (threadIdx.x == 0 && *abort_flag) {   // plain store: the word may live in pinned host memory
        *reinterpret_cast<volatile int32_t*>(p.error) = 1;
        __threadfence_system();
    }
}

// cuTensorMapEncodeTiled through the runtime's driver entry point lookup: no link-time
// dependency on the driver library.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// 2-D fp16 tensor [rows, cols] row-major, box [32 rows, 32 columns] = 64-byte rows, 64-byte swizzle (stores only).
static int make_map_half(CUtensorMap* map, const void* base, int64_t rows, int64_t cols) {
    EncodeTiledFn enc = encode_tiled_fn();
    JG_CHECK_ARG(enc, JG_ECUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    cuuint32_t box[2] = {32, 32};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    JG_CHECK_ARG(r == CUDA_SUCCESS, JG_ECUDA, "cuTensorMapEncodeTiled (fp16) failed with code %d", (int)r);
    return JG_OK;
}

// 2-D fp32 tensor [rows, cols] row-major, box [box_rows, 32 columns], 128-byte swizzle, zero fill
// on loads / clipping on stores outside the tensor.
static int make_map(CUtensorMap* map, const float* base, int64_t rows, int64_t cols, int box_rows, int atom32 = 0) {
    EncodeTiledFn enc = encode_tiled_fn();
    JG_CHECK_ARG(enc, JG_ECUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)cols * 4};
    cuuint32_t box[2] = {(cuuint32_t)kTileK, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box, elem,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    JG_CHECK_ARG(r == CUDA_SUCCESS, JG_ECUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
    return JG_OK;
}

// ------------------------------------------------------------------------------------------
// Weight gradient  gw[K, M] = x^T * g = sum over the rows n of x[n, :]^T g[n, :]  on the tensor cores.
//
// The reduction runs over the ROWS, so both operands are "MN-major" for the MMA: in x [n, K] the
// feature index (the M of the instruction) is the contiguous one, in g [n, M] the output column (its
// N).  32-bit MN-major operands take the 128-byte swizzle with 32-byte atoms (the plain 128-byte
// swizzle with both major bits set returned all zeros on a B200), so the TMA maps of this kernel use
// CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B.  A box of 64 rows x 32 columns lands as 64 lines of 128 bytes:
// 32 consecutive MN elements per line, 4 lines per K atom, two atoms (512 bytes apart: the stride
// byte offset) per K = 8 instruction, and the 32-column blocks that make up the 128 features (or the
// M columns) one box (8192 bytes: the leading byte offset) apart; both major bits set in the
// instruction descriptor.  One CTA owns a tile of 128 features and one slice of the rows, accumulates
// [128, M] in TMEM over its slice and writes it to partial[slice]; a second kernel adds the slices in
// order (no atomics: results repeat exactly).  Same bounded mbarrier waits as the transform.
constexpr int kTnRows = 64;          // rows (the reduction dimension) per stage
constexpr int kTnThreads = 192;      // warp 0: TMA producer, warp 1: MMA, warps 2-5: epilogue

struct TnParams {
    float* partial;      // [slices][k][m]
    int64_t n_rows;
    int32_t k, m;        // features (rows of gw), columns of g and gw
    int32_t m_blocks;    // 32-column boxes of g per stage
    int32_t n_pad;       // MMA N (m rounded up to 16) and TMEM columns (power of two >= 32)
    int32_t tmem_cols;
    int32_t blocks_per_slice;   // stages of kTnRows rows per slice
    int32_t stages;
    int32_t* error;
};

// MN-major operand of 32-bit elements: 128-byte swizzle with 32-byte atoms (layout type 1), whose K atom
// is 4 lines: stride byte offset 512 between the two atoms of one K = 8 step.
__device__ __forceinline__ uint64_t umma_desc_mn(uint32_t smem_addr, uint32_t lbo_bytes) {
    return (uint64_t)((smem_addr >> 4) & 0x3FFF) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16) | (32ull << 32) | (1ull << 46) |
           (1ull << 61);
}

__global__ void __launch_bounds__(kTnThreads, 1)
gemm_tn_tf32_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_g, TnParams p) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* ring = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t box_bytes = kTnRows * 128;                         // 8 KB
    const uint32_t a_bytes = 4 * box_bytes;                           // 128 features
    const uint32_t stage_bytes = a_bytes + (uint32_t)p.m_blocks * box_bytes;
    GemmSmem* ctl = reinterpret_cast<GemmSmem*>(ring + (size_t)p.stages * stage_bytes);
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int slice = blockIdx.x, ftile = blockIdx.y;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; s++) {
            mbar_init(&ctl->full[s], 1);
            mbar_init(&ctl->empty[s], 1);
        }
        mbar_init(&ctl->acc_full[0], 1);
        ctl->abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 2) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctl->tmem_base)), "r"((uint32_t)p.tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = ctl->tmem_base;
    volatile int32_t* abort_flag = &ctl->abort;
    const int64_t blk0 = (int64_t)slice * p.blocks_per_slice;
    const int64_t n_blocks_total = (p.n_rows + kTnRows - 1) / kTnRows;
    int64_t my_blocks = n_blocks_total - blk0;
    if (my_blocks > p.blocks_per_slice) my_blocks = p.blocks_per_slice;
    if (my_blocks < 0) my_blocks = 0;

    if (warp == 0) {
        if (lane == 0) {
            for (int64_t it = 0; it < my_blocks && !*abort_flag; it++) {
                const int s = (int)(it % p.stages);
                const uint32_t round = (uint32_t)(it / p.stages);
                if (round > 0 && !mbar_wait(&ctl->empty[s], (round - 1) & 1)) { *abort_flag = 1; break; }
                unsigned char* dst = ring + (size_t)s * stage_bytes;
                mbar_expect_tx(&ctl->full[s], stage_bytes);
                const int row = (int)((blk0 + it) * kTnRows);
                for (int j = 0; j < 4; j++) tma_load_2d(dst + j * box_bytes, &map_x, ftile * 128 + j * 32, row, &ctl->full[s]);
                for (int j = 0; j < p.m_blocks; j++) tma_load_2d(dst + a_bytes + j * box_bytes, &map_g, j * 32, row, &ctl->full[s]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && my_blocks > 0) {
            // D fp32, A/B tf32, both MN-major, N = n_pad, M = 128
            const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | (1u << 15) | (1u << 16) | (((uint32_t)p.n_pad >> 3) << 17) | ((128u >> 4) << 24);
            bool ok = true;
            for (int64_t it = 0; it < my_blocks; it++) {
                const int s = (int)(it % p.stages);
                if (!mbar_wait(&ctl->full[s], (uint32_t)(it / p.stages) & 1)) { ok = false; break; }
                tc_fence_after();
                const uint32_t a_addr = smem_u32(ring + (size_t)s * stage_bytes);
                const uint64_t da = umma_desc_mn(a_addr, box_bytes), db = umma_desc_mn(a_addr + a_bytes, box_bytes);
#pragma unroll
                for (int ks = 0; ks < kTnRows / 8; ks++)   // 8 rows = 1024 bytes per K step: +64 in 16-byte units
                    umma_tf32(tmem_base, da + 64 * ks, db + 64 * ks, idesc, (it > 0 || ks > 0) ? 1u : 0u);
                umma_commit(&ctl->empty[s]);
            }
            if (!ok) *abort_flag = 1;
            umma_commit(&ctl->acc_full[0]);
        }
    } else {
        // epilogue: warp w reads TMEM lanes 32*(w % 4) .. +31 = features ftile*128 + 32*(w % 4) + lane
        const int quad = warp & 3;
        const int64_t feat = (int64_t)ftile * 128 + quad * 32 + lane;
        float* out = p.partial + ((size_t)slice * p.k + (size_t)feat) * p.m;
        if (my_blocks > 0) {
            if (!mbar_wait(&ctl->acc_full[0], 0)) *abort_flag = 1;
            tc_fence_after();
            if (!*abort_flag) {
                for (int c0 = 0; c0 < p.m; c0 += 32) {
                    float v[32];
                    tmem_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)c0, v, c0 + 16 < p.n_pad);
                    if (feat < p.k) {
#pragma unroll
                        for (int i = 0; i < 32; i++)
                            if (c0 + i < p.m) out[c0 + i] = v[i];
                    }
                }
            }
        } else if (feat < p.k) {
            for (int c = 0; c < p.m; c++) out[c] = 0.f;   // a slice beyond the last row contributes nothing
        }
        tc_fence_before();
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 2)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)p.tmem_cols) : "memory");
    if (threadIdx.x == 0 && *abort_flag) {
        *reinterpret_cast<volatile int32_t*>(p.error) = 1;
        __threadfence_system();
    }
}

// 2-D fp32 tensor [rows, cols] row-major, box [kTnRows rows, 32 columns], 128-byte swizzle, zero fill.
static int make_map_rows(CUtensorMap* map, const float* base, int64_t rows, int64_t cols) { return make_map(map, base, rows, cols, kTnRows, 1); }

// gw[k, m] = sum_s partial[s]: defined with the fp32 product (gemm_f32.cu).
int reduce_slices(float* c, const float* partial, int64_t M, int64_t N, int slices, cudaStream_t st);

}  // namespace jg

using namespace jg;

extern "C" {

int jg_gemm_tf32_supported(int64_t n_rows, int64_t k, int64_t m) {
    return n_rows > 0 && k > 0 && m > 0 && m <= 4096 && k < (1 << 20) && n_rows < ((int64_t)1 << 31) * 64;
}

size_t jg_gemm_tf32_workspace_bytes(void) { return 256; }

// Set only inside jg_gemm_tf32_timeout_selftest (one thread, for the duration of its call).
static thread_local uint32_t g_test_wait_spins = kWaitSpins;
static thread_local int32_t g_test_withhold = -1;

// One column tile (at most 256 output columns) of the product.
static int gemm_tile(float* out, const float* x, const float* wt, const float* bias, int64_t n_rows, int64_t k, int64_t m,
                     int64_t m_total, int64_t col_base, int relu, int32_t* error, cudaStream_t st, __half* out_half = nullptr) {
    // TMA needs 16-byte aligned bases and row pitches; anything else goes through the plain-load producer
    const bool plain = (k % 4 != 0) || ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(wt)) % 16 != 0);
    const int b_rows = (int)((m + 15) / 16 * 16);
    CUtensorMap map_x, map_w;
    memset(&map_x, 0, sizeof(map_x));
    memset(&map_w, 0, sizeof(map_w));
    if (!plain) {
        int rc = make_map(&map_x, x, n_rows, k, kTileM);
        if (rc != JG_OK) return rc;
        rc = make_map(&map_w, wt, m, k, b_rows);
        if (rc != JG_OK) return rc;
    }
    GemmParams p = {};
    // plain loads: 8-byte copies when every row starts on an 8-byte boundary, else 4-byte copies
    const bool pairs = (k % 2 == 0) && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(wt)) % 8 == 0);
    p.x = x; p.wt = wt; p.plain_loads = plain ? (pairs ? 2 : 1) : 0;
    // TMA store needs a 16-byte row pitch for the output
    p.tma_store = (m_total % 4 == 0 && m % 4 == 0) ? 1 : 0;
    CUtensorMap map_out;
    memset(&map_out, 0, sizeof(map_out));
    if (p.tma_store) {
        int rc2 = make_map(&map_out, out - col_base, n_rows, m_total, 32);
        if (rc2 != JG_OK) return rc2;
    }
    p.out = out; p.bias = bias; p.n_rows = n_rows; p.k = (int32_t)k; p.m = (int32_t)m; p.relu = relu;
    p.ldo = (int32_t)m_total; p.col_base = (int32_t)col_base;
    p.out_half = out_half;
    CUtensorMap map_half;
    memset(&map_half, 0, sizeof(map_half));
    if (out_half) {
        JG_CHECK_ARG(p.tma_store, JG_ESHAPE, "gemm_tf32: the fp16 copy needs an output width that is a multiple of 8");
        int rc3 = make_map_half(&map_half, out_half - col_base, n_rows, m_total);
        if (rc3 != JG_OK) return rc3;
    }
    int pad = 32;
    while (pad < b_rows) pad *= 2;
    p.m_pad = pad;
    p.n_tiles = (int32_t)((n_rows + kTileM - 1) / kTileM);
    p.k_blocks = (int32_t)((k + kTileK - 1) / kTileK);
    p.error = error;
    p.wait_spins = g_test_wait_spins;
    p.withhold = g_test_withhold;
    const size_t a_bytes = kTileM * kTileK * 4;
    const size_t b_bytes = ((size_t)b_rows * kTileK * 4 + 1023) / 1024 * 1024;
    const size_t smem = 1024 + kStages * (a_bytes + b_bytes) + (p.tma_store ? kEpiWarps * 4096 : 0) +
                        (out_half ? kEpiWarps * 2048 : 0) + sizeof(GemmSmem) + 64;
    static size_t attr_done[64] = {0};
    int dev = 0;
    JG_CUDA(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && attr_done[dev] < smem) {
        JG_CUDA(cudaFuncSetAttribute(gemm_tf32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(227 * 1024)));
        attr_done[dev] = 227 * 1024;
    }
    int grid = sm_count();
    if (grid > p.n_tiles) grid = p.n_tiles;
    gemm_tf32_kernel<<<grid, kGemmThreads, smem, st>>>(map_x, map_w, map_out, map_half, p);
    JG_LAUNCH_CHECK();
    return JG_OK;
}

static int gemm_impl(float* out, void* out_half, const float* x, const float* wt, const float* bias, int64_t n_rows, int64_t k,
                     int64_t m, int relu, void* workspace, size_t workspace_bytes, jg_stream_t stream, bool clear_error = true) {
    JG_CHECK_ARG(n_rows >= 0 && k > 0 && m > 0, JG_EINVAL, "gemm_tf32: bad size");
    JG_CHECK_ARG(!out_half || (m % 8 == 0 && reinterpret_cast<uintptr_t>(out_half) % 16 == 0), JG_ESHAPE,
                 "gemm_tf32: the fp16 copy needs a width that is a multiple of 8 and a 16-byte aligned buffer");
    if (n_rows == 0) return JG_OK;
    JG_CHECK_ARG(out && x && wt, JG_EINVAL, "gemm_tf32: null pointer");
    if (!jg_gemm_tf32_supported(n_rows, k, m)) {
        set_error("gemm_tf32: needs m <= 4096 (got k=%lld, m=%lld)", (long long)k, (long long)m);
        return JG_EUNSUPPORTED;
    }
    JG_CHECK_ARG(reinterpret_cast<uintptr_t>(out) % 16 == 0, JG_EINVAL, "gemm_tf32: out must be 16-byte aligned");
    JG_CHECK_ARG(workspace && workspace_bytes >= 256, JG_EWORKSPACE, "gemm_tf32: workspace missing");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int32_t* error = static_cast<int32_t*>(workspace);
    if (clear_error) JG_CUDA(cudaMemsetAsync(error, 0, sizeof(int32_t), st));
    // wider outputs: one launch per tile of 256 columns (x is read once per tile); 128 columns when the fp16
    // copy needs its own staging slabs in shared memory
    const int64_t tile_w = out_half ? 128 : 256;
    for (int64_t cb = 0; cb < m; cb += tile_w) {
        const int64_t mt = m - cb < tile_w ? m - cb : tile_w;
        int rc = gemm_tile(out + cb, x, wt + cb * k, bias ? bias + cb : nullptr, n_rows, k, mt, m, cb, relu, error, st,
                           out_half ? static_cast<__half*>(out_half) + cb : nullptr);
        if (rc != JG_OK) return rc;
    }
    return JG_OK;
}

int jg_gemm_tf32(float* out, const float* x, const float* wt, const float* bias, int64_t n_rows, int64_t k, int64_t m,
                 int relu, void* workspace, size_t workspace_bytes, jg_stream_t stream) {
    return gemm_impl(out, nullptr, x, wt, bias, n_rows, k, m, relu, workspace, workspace_bytes, stream);
}

int jg_gemm_tf32_dual(float* out, void* out_half, const float* x, const float* wt, const float* bias, int64_t n_rows, int64_t k,
                      int64_t m, int relu, void* workspace, size_t workspace_bytes, jg_stream_t stream) {
    return gemm_impl(out, out_half, x, wt, bias, n_rows, k, m, relu, workspace, workspace_bytes, stream, false);
}

/* Failure-path self-test: the same kernel as jg_gemm_tf32, but the producer leaves out fill number
 * `withhold` of every CTA's ring and every wait gives up after `wait_spins` polls.  The consumer's bounded
 * wait runs out, the CTAs free their TMEM and return, the error word is set: jg_gemm_tf32_status then
 * reports JG_ETIMEOUT.  `out` is left partly written.  Needs the TMA producer (k % 4 == 0, aligned x and
 * wt).  Nothing traps and the context stays usable. */
int jg_gemm_tf32_timeout_selftest(float* out, const float* x, const float* wt, int64_t n_rows, int64_t k, int64_t m,
                                  int32_t withhold, uint32_t wait_spins, void* workspace, size_t workspace_bytes, jg_stream_t stream) {
    JG_CHECK_ARG(k % 4 == 0 && (reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(wt)) % 16 == 0, JG_EINVAL,
                 "gemm_tf32_timeout_selftest: needs the TMA producer (k %% 4 == 0, 16-byte aligned operands)");
    JG_CHECK_ARG(withhold >= 0 && wait_spins >= 128 && wait_spins <= kWaitSpins, JG_EINVAL, "gemm_tf32_timeout_selftest: bad hook values");
    g_test_wait_spins = wait_spins;
    g_test_withhold = withhold;
    const int rc = gemm_impl(out, nullptr, x, wt, nullptr, n_rows, k, m, 0, workspace, workspace_bytes, stream);
    g_test_wait_spins = kWaitSpins;
    g_test_withhold = -1;
    return rc;
}

static int tn_slices(int64_t n_rows, int64_t k) {
    const int64_t tiles = (k + 127) / 128;
    const int64_t blocks = (n_rows + kTnRows - 1) / kTnRows;
    int64_t s = (sm_count() + tiles - 1) / tiles;        // about one CTA per SM
    if (s > (blocks + 3) / 4) s = (blocks + 3) / 4;      // at least four stages of rows per slice
    return s < 1 ? 1 : (int)s;
}

int jg_gemm_tn_tf32_supported(int64_t n_rows, int64_t k, int64_t m) {
    return n_rows > 0 && k > 0 && m > 0 && m <= 256 && k % 4 == 0 && m % 4 == 0 && n_rows < ((int64_t)1 << 31) - kTnRows;
}

size_t jg_gemm_tn_tf32_workspace_bytes(int64_t n_rows, int64_t k, int64_t m) {
    if (!jg_gemm_tn_tf32_supported(n_rows, k, m)) return 0;
    return 256 + align_up((size_t)tn_slices(n_rows, k) * (size_t)k * (size_t)m * sizeof(float), 256);
}

int jg_gemm_tn_tf32(float* gw, const float* x, const float* g, int64_t n_rows, int64_t k, int64_t m, int32_t* error,
                    void* workspace, size_t workspace_bytes, jg_stream_t stream) {
    JG_CHECK_ARG(gw && x && g && error, JG_EINVAL, "gemm_tn_tf32: null pointer");
    if (!jg_gemm_tn_tf32_supported(n_rows, k, m)) {
        set_error("gemm_tn_tf32: needs k %% 4 == 0, m %% 4 == 0, m <= 256 (got k=%lld, m=%lld)", (long long)k, (long long)m);
        return JG_EUNSUPPORTED;
    }
    JG_CHECK_ARG((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(g)) % 16 == 0, JG_EINVAL, "gemm_tn_tf32: operands must be 16-byte aligned");
    const size_t need = jg_gemm_tn_tf32_workspace_bytes(n_rows, k, m);
    JG_CHECK_ARG(workspace && workspace_bytes >= need, JG_EWORKSPACE, "gemm_tn_tf32: workspace %zu < %zu", workspace_bytes, need);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    CUtensorMap map_x, map_g;
    memset(&map_x, 0, sizeof(map_x));
    memset(&map_g, 0, sizeof(map_g));
    int rc = make_map_rows(&map_x, x, n_rows, k);
    if (rc != JG_OK) return rc;
    rc = make_map_rows(&map_g, g, n_rows, m);
    if (rc != JG_OK) return rc;
    TnParams p = {};
    p.partial = reinterpret_cast<float*>(static_cast<unsigned char*>(workspace) + 256);
    p.n_rows = n_rows; p.k = (int32_t)k; p.m = (int32_t)m;
    p.m_blocks = (int32_t)((m + 31) / 32);
    p.n_pad = (int32_t)((m + 15) / 16 * 16);
    int cols = 32;
    while (cols < p.n_pad) cols *= 2;
    p.tmem_cols = cols;
    const int slices = tn_slices(n_rows, k);
    const int64_t blocks = (n_rows + kTnRows - 1) / kTnRows;
    p.blocks_per_slice = (int32_t)((blocks + slices - 1) / slices);
    const size_t stage_bytes = (size_t)(4 + p.m_blocks) * kTnRows * 128;
    int stages = kStages;
    while (stages > 2 && (size_t)stages * stage_bytes > 200 * 1024) stages--;
    p.stages = stages;
    p.error = error;
    const size_t smem = 1024 + (size_t)stages * stage_bytes + sizeof(GemmSmem) + 64;
    static size_t attr_done[64] = {0};
    int dev = 0;
    JG_CUDA(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && attr_done[dev] < smem) {
        JG_CUDA(cudaFuncSetAttribute(gemm_tn_tf32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(227 * 1024)));
        attr_done[dev] = 227 * 1024;
    }
    dim3 grid((unsigned)slices, (unsigned)((k + 127) / 128));
    gemm_tn_tf32_kernel<<<grid, kTnThreads, smem, st>>>(map_x, map_g, p);
    JG_LAUNCH_CHECK();
    return reduce_slices(gw, p.partial, k, m, slices, st);
}

/* Reads the error word a finished jg_gemm_tf32 call left in its workspace (synchronises the
 * stream): JG_OK, or JG_ETIMEOUT when a bounded wait inside the kernel ran out. */
int jg_gemm_tf32_status(const void* workspace, jg_stream_t stream) {
    JG_CHECK_ARG(workspace, JG_EINVAL, "gemm_tf32_status: null workspace");
    int32_t err = 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    JG_CUDA(cudaMemcpyAsync(&err, workspace, sizeof(err), cudaMemcpyDeviceToHost, st));
    JG_CUDA(cudaStreamSynchronize(st));
    if (err) {
        set_error("gemm_tf32: a bounded wait inside the kernel ran out");
        return JG_ETIMEOUT;
    }
    return JG_OK;
}

}  // extern "C"
