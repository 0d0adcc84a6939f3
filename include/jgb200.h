/* jgb200 - C ABI of the B200 (sm_100a) message-passing kernels.
 *
 * Drop-in boundary for the operator layer of JittorGeometric
 * (jittor_geometric/ops/*.py -> jittor_geometric/ops/cpp/*_op.cc): every entry
 * point below replaces one native operator of that layer and is what a binding
 * (ctypes, cffi, a Jittor custom op) would call.
 *
 * Conventions
 *   - all pointers are DEVICE pointers unless the name ends in _host;
 *   - indices int32, values fp32, dense matrices row-major and contiguous;
 *   - `off` arrays have n+1 entries, segment v = [off[v], off[v+1]);
 *   - the caller owns every buffer, including the workspace whose size the
 *     matching *_workspace_bytes() call reports; the library allocates nothing
 *     and keeps no per-call state;
 *   - every call is asynchronous on `stream` (a cudaStream_t passed as void*);
 *   - the return value is JG_OK or a negative jg_status; jg_last_error() gives
 *     the detail text for the calling thread.  Nothing exits or traps.
 */
#ifndef JGB200_H
#define JGB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* jg_stream_t; /* cudaStream_t */

enum jg_status {
    JG_OK = 0,
    JG_EINVAL = -1,       /* null pointer, negative size, bad flag */
    JG_ESHAPE = -2,       /* sizes that do not fit together or exceed int32 indexing */
    JG_EWORKSPACE = -3,   /* workspace missing or too small */
    JG_ECUDA = -4,        /* a CUDA runtime call failed */
    JG_ETIMEOUT = -5,     /* a bounded device-side wait ran out */
    JG_EUNSUPPORTED = -6  /* valid request this build does not implement */
};

int jg_version(void);
const char* jg_status_string(int status);
const char* jg_last_error(void);
/* Makes `device` current for the library's CUDA runtime on the calling thread. */
int jg_set_device(int device);

/* ------------------------------------------------------------------ aggregation
 * Weighted segment aggregation  out[v,:] = sum_{j in seg(v)} w[j] * x[idx[j],:].
 * Replaces AggregateOp (ops/cpp/aggregate_op.cc:26-105; Python wrapper
 * ops/aggregateWithWeight.py:19-41): called with the CSC arrays it is the forward
 * pass, with the CSR arrays the backward pass.  It is also the kernel behind the
 * cuSPARSE-backed SpmmCsr/SpmmCoo (ops/spmmcsr.py:21-44, ops/spmmcoo.py:19-45).
 * For f < 32 and f > 64 multiply and add are rounded separately and the terms of a row
 * are added in ascending j, so rows of at most `chunk` entries reproduce the
 * reference CPU loop bit for bit; for 32 <= f <= 64 two or four entries are taken side
 * by side with fused multiply-adds and their partial sums added at the end
 * (rounding-level difference; use jg_aggregate_ordered_f32 where the order matters).  Longer rows are split into
 * `chunk`-sized pieces whose partial sums are added in piece order.  No atomics touch
 * `out`.  Any f >= 1 is accepted: f <= 32 runs several rows per warp, 16-byte-aligned
 * widths up to 512 use 128-bit gathers, other widths column-strided scalar loads.
 *
 * The hub plan lists the rows longer than `chunk`; it depends only on `off` and
 * is reusable across calls; pass the `chunk` it was built with.  plan == NULL
 * (chunk ignored) processes every row unsplit.
 * `out` need not be zeroed: every row is written.  x has n_in rows, out n_out. */
size_t jg_spmm_plan_bytes(int64_t n_out, int64_t nnz, int32_t chunk);
int jg_spmm_plan_build(const int32_t* off, int64_t n_out, int64_t nnz, int32_t chunk, void* plan,
                       size_t plan_bytes, jg_stream_t stream);
size_t jg_aggregate_workspace_bytes(int64_t n_out, int64_t nnz, int64_t f, int32_t chunk);
int jg_aggregate_f32(float* out, const float* x, const int32_t* idx, const int32_t* off,
                     const float* w, int64_t n_out, int64_t n_in, int64_t f, int64_t nnz,
                     const void* plan, int32_t chunk, void* workspace, size_t workspace_bytes,
                     jg_stream_t stream);

/* Structure check for the arrays the gather kernels trust: off[0] == 0, offsets non-decreasing,
 * off[n_out] == nnz, every idx in [0, n_in).  Returns JG_EINVAL with the violation counts in
 * jg_last_error(); synchronises the stream; workspace of 16 bytes.  The reference has no such
 * check (a bad index there reads out of bounds, ops/cpp/aggregate_op.cc:45-58); here it is what a
 * debug build or a cautious caller runs once per graph instead of a memory sanitizer. */
int jg_validate_segments(const int32_t* idx, const int32_t* off, int64_t n_out, int64_t n_in, int64_t nnz,
                         void* workspace, size_t workspace_bytes, jg_stream_t stream);

/* Same aggregation, added to what `out` already holds: out[v,:] = out[v,:] + sum_j w[j]*x[idx[j],:]
 * (the sum is formed first, then added).  Used by the partitioned path, where the rows gathered
 * from other shards are aggregated after the shard's own rows - the place where the reference
 * adds the per-source-rank results (ops/distspmm.py:39, `result = result + output`). */
int jg_aggregate_add_f32(float* out, const float* x, const int32_t* idx, const int32_t* off,
                         const float* w, int64_t n_out, int64_t n_in, int64_t f, int64_t nnz,
                         const void* plan, int32_t chunk, void* workspace, size_t workspace_bytes,
                         jg_stream_t stream);

/* The same aggregation with every row that is not split by the plan summed strictly in stored order
 * at EVERY width (jg_aggregate_f32 does so for f < 32 and f > 64 only; in between it lets lane groups
 * take alternate entries, which is faster and differs by rounding).  With idx = 0, 1, 2, ... and
 * unit weights over an [n_edges, f] message matrix this is the per-destination sum of
 * edgetovertex (ops/cpp/edgetovertex_op.cc:27-57), bit-identical to its sequential loop. */
int jg_aggregate_ordered_f32(float* out, const float* x, const int32_t* idx, const int32_t* off, const float* w,
                             int64_t n_out, int64_t n_in, int64_t f, int64_t nnz, const void* plan, int32_t chunk,
                             void* workspace, size_t workspace_bytes, jg_stream_t stream);

/* The same aggregation with the layer's epilogue fused into the store of every finished row:
 * out[v,:] = act(sum + bias), bias [f] or NULL, relu != 0 clamps at zero.  Replaces the separate
 * elementwise passes of `out = out + self.bias` and `nn.relu(...)` that follow the aggregation in the
 * reference layers (nn/conv/gcn_conv.py:100-101, examples/gcn_example.py:76-77), each a read and a
 * write of the whole [n_out, f] matrix. */
int jg_aggregate_bias_act_f32(float* out, const float* x, const int32_t* idx, const int32_t* off, const float* w,
                              const float* bias, int relu, int64_t n_out, int64_t n_in, int64_t f, int64_t nnz,
                              const void* plan, int32_t chunk, void* workspace, size_t workspace_bytes, jg_stream_t stream);

/* The aggregation with every option of the entry points above in one call (bias/relu epilogue,
 * accumulate, ordered) plus `reserve_ctas`: that many CTA slots of the persistent grid are left free, so
 * that a small kernel on another stream - the halo pull of the next exchange, jg_halo_pull - finds room
 * to run beside it.  The reference runs its P exchange rounds and SpMMs strictly one after another
 * (ops/distspmm.py:31-39). */
int jg_aggregate_opts_f32(float* out, const float* x, const int32_t* idx, const int32_t* off, const float* w,
                          const float* bias, int relu, int accumulate, int ordered, int reserve_ctas, int64_t n_out,
                          int64_t n_in, int64_t f, int64_t nnz, const void* plan, int32_t chunk, void* workspace,
                          size_t workspace_bytes, jg_stream_t stream);

/* ------------------------------------------------------------------ 1-D row partition
 * Splits the in-edge structure of one shard (destination rows [lo, hi) of the graph, `idx`
 * holding GLOBAL source ids) into interior entries (source inside [lo, hi), ids rebased to the
 * shard) and halo entries (source owned by another shard, ids kept global), each keeping the
 * order of the input within a row.  Replaces the per-source-rank sub-CSR construction of the
 * reference's offline partitioner (partition/distchunk_manager.py:100-106,
 * examples/dist_gcn/dist_partition.py:122-158), on device.  Output arrays need room for nnz
 * entries (offsets n_rows + 1); out_counts[0..1] (device, int64) receive the two entry counts. */
size_t jg_partition_split_workspace_bytes(int64_t nnz);
int jg_partition_split(const int32_t* idx, const int32_t* off, const float* w, int64_t n_rows, int64_t nnz, int32_t lo,
                       int32_t hi, int32_t* int_idx, int32_t* int_off, float* int_w, int32_t* halo_idx,
                       int32_t* halo_off, float* halo_w, int64_t* out_counts, void* workspace, size_t workspace_bytes,
                       jg_stream_t stream);

/* Compact halo.  jg_halo_map_build takes entries of a shard with GLOBAL source ids (all of them, or
 * only the halo entries from jg_partition_split) and the shard's own row range [lo, hi), and
 * produces: pos[n_global + 1], the exclusive scan of "remote row g is referenced" (pos[g] = slot of
 * row g in a packed halo buffer ordered by global id, pos[n_global] = number of distinct remote rows
 * needed); needed[pos[n_global]], those rows ascending (grouped by owner, since owners hold
 * contiguous ranges); remapped_idx[nnz]: own rows become idx - lo, remote rows base + pos[idx]
 * (base = where the halo rows start in the buffer the aggregation will read; lo = hi = base = 0
 * re-addresses pure halo entries into the packed buffer alone).  jg_gather_rows_f32 packs out[i,:] = x[rows[i] - rebase,:], the kernel a rank
 * uses to fill the send buffer with the rows another rank asked for.  Together they replace the
 * whole-block broadcast of the reference (ops/distspmm.py:31-39) by an exchange of referenced rows
 * only. */
size_t jg_halo_map_workspace_bytes(int64_t n_global);
int jg_halo_map_build(const int32_t* halo_idx, int64_t nnz, int64_t n_global, int32_t lo, int32_t hi, int32_t base,
                      int32_t* pos, int32_t* needed, int32_t* remapped_idx, void* workspace, size_t workspace_bytes,
                      jg_stream_t stream);
int jg_gather_rows_f32(float* out, const float* x, const int32_t* rows, int64_t n_rows, int64_t f, int32_t rebase,
                       jg_stream_t stream);

/* Halo exchange by direct loads from peer memory (one process per GPU, NVLink).  Replaces the P
 * rounds of host-staged MPI.bcast of whole feature blocks (ops/distspmm.py:31-39,
 * utils/distributed_utils.py:66-74): every rank keeps its feature rows in a buffer all ranks have
 * mapped and pulls the distinct remote rows it references (`needed`, from jg_halo_map_build) out of
 * their owners' buffers into its own halo rows.
 *
 * Flag block: jg_halo_flag_bytes() bytes per rank, zeroed once, mapped by every rank; it holds one
 * "ready" (kind 0) and one "done" (kind 1) epoch word per buffer slot (< jg_halo_flag_slots()) and
 * rank (< jg_halo_max_ranks()).  Arrays named *_host are HOST arrays of `world` device pointers (the
 * peers' buffers as mapped in this process, this rank's own included) or of per-rank values.
 *   jg_halo_post   writes `epoch` into word (slot, kind, rank) of EVERY rank's flag block, after all
 *                  earlier work of `stream` (kind 0: "my rows of this slot are written").
 *   jg_halo_pull   for every peer q waits (at most wait_ns) for ready word (slot, q) >= epoch in this
 *                  rank's flag block, then copies rows needed[seg_begin[q] .. seg_begin[q+1]) -
 *                  global ids, row id - lo[q] inside peer q's buffer - to halo rows of the same
 *                  positions; when everything has landed it posts done word (slot, rank) = epoch to
 *                  every rank.  Rows are row_bytes long (a multiple of 4; multiples of 16 use bulk
 *                  asynchronous copies through shared memory, one warp per CTA, at most max_ctas
 *                  CTAs; plain != 0 forces the plain-load kernel).  `counter` is 4 zeroed bytes of
 *                  device memory owned by the caller, zero again when the call has finished.
 *   jg_halo_wait   waits (at most wait_ns) until word (slot, kind, q) >= epoch for every peer q in
 *                  this rank's flag block (kind 1: "every peer has read my rows, I may overwrite them").
 * A wait that runs out stores a code in *error (a device-accessible int32, e.g. pinned host memory:
 * 0x100 + q ready word of rank q, 0x200 + q done word of rank q, 0x300 a copy that never landed) and the
 * kernel returns; nothing traps and the context stays usable.  No load uses cluster multicast. */
size_t jg_halo_flag_bytes(void);
int jg_halo_max_ranks(void);
int jg_halo_flag_slots(void);
int jg_halo_post(void* const* peer_flags_host, int world, int rank, int slot, int kind, uint32_t epoch, jg_stream_t stream);
int jg_halo_wait(const void* my_flags, int world, int rank, int slot, int kind, uint32_t epoch, int32_t* error,
                 int64_t wait_ns, jg_stream_t stream);
int jg_halo_pull(void* halo, const int32_t* needed, void* const* peer_x_host, void* const* peer_flags_host,
                 const int64_t* seg_begin_host, const int32_t* lo_host, int world, int rank, int64_t row_bytes, int slot,
                 uint32_t epoch, void* counter, int32_t* error, int64_t wait_ns, int max_ctas, int plain, int src_half,
                 jg_stream_t stream);
/* The same pull for a PART of every owner's segment: halo slots [part_begin_host[q], part_end_host[q]) inside
 * [seg_begin_host[q], seg_begin_host[q+1]).  An owner that produces its rows block after block (a transform
 * that follows an aggregation of a row range) posts one epoch word per block (its own `slot` each), and its
 * readers fetch the rows of a block while the owner computes the next one.  No counterpart in the reference,
 * whose broadcast moves whole blocks of every rank (ops/distspmm.py:31-39). */
int jg_halo_pull_part(void* halo, const int32_t* needed, void* const* peer_x_host, void* const* peer_flags_host,
                      const int64_t* seg_begin_host, const int64_t* part_begin_host, const int64_t* part_end_host,
                      const int32_t* lo_host, int world, int rank, int64_t row_bytes, int slot, uint32_t epoch, void* counter,
                      int32_t* error, int64_t wait_ns, int max_ctas, int plain, int src_half, jg_stream_t stream);
/* Half-width payload of the exchange: jg_rows_to_half rounds n_values fp32 values (a multiple of 4) to
 * fp16 (values beyond +-65504 saturate), the copy of its rows an owner offers; jg_halo_pull with
 * src_half != 0 then reads rows of row_bytes = 2 * width bytes (a multiple of 16) from the peers' fp16
 * buffers and widens them to fp32 halo rows of 2 * row_bytes.  Every aggregated element stays within
 * 5e-4 of the fp32 exchange relative to its sum of absolute terms: for the workloads whose tolerance is
 * 2e-3 (a TF32/bf16 transform feeds the aggregation).  The fp32 exchange is bit-exact. */
int jg_rows_to_half(void* out, const float* x, int64_t n_values, jg_stream_t stream);

/* ------------------------------------------------------------------ conversion
 * COO -> CSR (by = 0, rows keyed by source) or CSC (by = 1, columns keyed by destination).
 * Replaces CootocsrOp / CootocscOp (ops/cpp/cootocsr_op.cc:24-57, ops/cpp/cootocsc_op.cc:23-53;
 * Python wrappers ops/cootocsr.py:28-35, ops/cootocsc.py:29-36).  edge_index is [2, n_edges]
 * row-major (all sources, then all destinations).  Entry i lands at
 * off[key_i] + #{j < i : key_j == key_i}: the reference's stable order, bit for bit.
 * canonical != 0 orders the entries of one row by their index instead.  w == NULL means unit
 * weights.  Outputs: out_idx[n_edges], out_off[n_nodes + 1], out_w[n_edges]. */
size_t jg_convert_workspace_bytes(int64_t n_edges, int64_t n_nodes);
int jg_coo_to_compressed(const int32_t* edge_index, const float* w, int64_t n_edges, int64_t n_nodes, int by,
                         int canonical, int32_t* out_idx, int32_t* out_off, float* out_w, void* workspace,
                         size_t workspace_bytes, jg_stream_t stream);

/* gcn_norm fused with the conversion: replaces gcn_norm + add_remaining_self_loops
 * (nn/conv/gcn_conv.py:18-37, utils/loop.py:120-134) followed by cootocsc / cootocsr, without
 * materialising the normalised COO list.  (v,v) input entries are dropped, one loop per node is
 * appended in node order (weight `fill`, or the weight of the node's last (v,v) input entry),
 * deg = weighted in-degree, w' = (deg^-1/2[src] * w) * deg^-1/2[dst].  Output arrays need room for
 * n_edges + n_nodes entries; the actual entry count is written to *out_count (device, int64).
 * The CSR triple may be NULL (all three) when only the CSC is wanted.  add_self_loops == 0
 * (the reference's add_self_loops=False, nn/conv/gcn_conv.py:25) normalises the list as given:
 * nothing is dropped or appended, and a node without in-edges has deg^-1/2 = inf, as there. */
int jg_gcn_norm_compressed(const int32_t* edge_index, const float* w, int64_t n_edges, int64_t n_nodes, float fill,
                           int add_self_loops, int canonical, int32_t* csc_idx, int32_t* csc_off, float* csc_w,
                           int32_t* csr_idx, int32_t* csr_off, float* csr_w, int64_t* out_count, void* workspace,
                           size_t workspace_bytes, jg_stream_t stream);

/* gcn_norm as a COO list, for callers that want the reference's intermediate
 * (nn/conv/gcn_conv.py:18-37): out_src/out_dst/out_w (room for n_edges + n_nodes entries each)
 * receive the kept entries in input order followed by one loop per node; *out_count (device,
 * int64) the entry count.  Same weights as jg_gcn_norm_compressed. */
size_t jg_gcn_norm_coo_workspace_bytes(int64_t n_edges, int64_t n_nodes);
int jg_gcn_norm_coo(const int32_t* edge_index, const float* w, int64_t n_edges, int64_t n_nodes, float fill,
                    int add_self_loops, int32_t* out_src, int32_t* out_dst, float* out_w, int64_t* out_count,
                    void* workspace, size_t workspace_bytes, jg_stream_t stream);

/* Symmetrise and deduplicate a COO list: replaces ToundirectedOp (ops/cpp/toundirected_op.cc:33-63;
 * wrapper ops/toundirected.py:16-22).  Every edge is mirrored, the 2 * n_edges entries are sorted
 * by (row, col) and one entry per distinct pair is kept - the first in mirrored-list order (edge i
 * as given, then reversed, for i = 0, 1, ...); the reference sorts with an unstable sort and leaves
 * that choice unspecified.  Outputs need room for 2 * n_edges entries; *out_count (device, int64)
 * receives the entry count. */
size_t jg_to_undirected_workspace_bytes(int64_t n_edges, int64_t n_nodes);
int jg_to_undirected(const int32_t* edge_index, const float* attr, int64_t n_edges, int64_t n_nodes, int32_t* out_src,
                     int32_t* out_dst, float* out_attr, int64_t* out_count, void* workspace, size_t workspace_bytes,
                     jg_stream_t stream);

/* ------------------------------------------------------------------ per-edge operators
 * Edges are in CSC order (segment v = in-edges of destination v, idx[e] = source of edge e).
 *
 * jg_scatter_to_edge_f32 replaces ScattertoedgeOp (ops/cpp/scattertoedge_op.cc:35-141; wrapper
 * ops/scatterToEdge.py:22-51): out[e,:] = x[idx[e],:] (flag 0, "src") or x[v,:] for e in segment v
 * (flag 1, "dst").  out is [n_edges, c]; every row is written.
 *
 * jg_edge_to_vertex_f32 replaces EdgetovertexOp (ops/cpp/edgetovertex_op.cc:27-95; wrapper
 * ops/scatterToVertex.py:23-50): flag 1: out[v,:] = sum of msg rows of segment v, ascending e;
 * flag 0: out[idx[e],:] += msg[e,:] (float atomics, as the reference's CUDA kernel).  Every out row
 * is written (zeros where nothing lands).
 *
 * jg_edge_softmax_fwd_f32 / _bwd_f32 replace EdgesoftmaxOp / EdgesoftmaxbackwardOp
 * (ops/cpp/edgesoftmax_op.cc:36-120, ops/cpp/edgesoftmaxbackward_op.cc:27-54; wrapper
 * ops/edgesoftmax.py:62-80): x, y, grad, dx are [n_edges, h]; each column is normalised over each
 * segment with the maximum subtracted (the reference's CPU recipe; h = 1 is the reference's own
 * shape).  Backward: dx = y*g - y*sum_segment(y*g).  Empty segments write nothing. */
int jg_scatter_to_edge_f32(float* out, const float* x, const int32_t* idx, const int32_t* off, int64_t n_nodes,
                           int64_t n_edges, int64_t c, int flag, jg_stream_t stream);
int jg_edge_to_vertex_f32(float* out, const float* msg, const int32_t* idx, const int32_t* off, int64_t n_nodes,
                          int64_t n_edges, int64_t c, int flag, jg_stream_t stream);
int jg_edge_softmax_fwd_f32(float* y, const float* x, const int32_t* off, int64_t n_nodes, int64_t n_edges, int64_t h,
                            jg_stream_t stream);
int jg_edge_softmax_bwd_f32(float* dx, const float* grad, const float* y, const int32_t* off, int64_t n_nodes,
                            int64_t n_edges, int64_t h, jg_stream_t stream);

/* Fused attention aggregation: the edge phase of GATConv.execute (nn/conv/gat_conv.py:60-83) in
 * one pass over CSC - logits leaky_relu(a_src.h[src] + a_dst.h[dst]), per-destination softmax,
 * weighted sum of source rows - with `heads` independent heads of width `dim` (heads = 1 is the
 * reference layer: a_src / a_dst are the two halves of its [2C, 1] attention vector).
 * h and out are [n_nodes, heads*dim]; a_src, a_dst are [heads, dim].  Supported shapes are
 * reported by jg_gat_aggregate_supported (heads*dim/4 and dim/4 powers of two, heads*dim <= 128);
 * others return JG_EUNSUPPORTED and are served by the per-edge operators above.
 * `plan` (optional, from jg_gat_plan_build; depends only on `off`) lists the destinations longest
 * segment first, which keeps the grid from ending on one warp that walks a hub alone.  `lse` may be
 * NULL; otherwise it receives [n_nodes, heads] values for jg_gat_backward_f32. */
size_t jg_gat_plan_bytes(int64_t n_nodes);
int jg_gat_plan_build(const int32_t* off, int64_t n_nodes, void* plan, size_t plan_bytes, jg_stream_t stream);
size_t jg_gat_aggregate_workspace_bytes(int64_t n_nodes, int64_t n_edges, int64_t heads, int64_t dim);
int jg_gat_aggregate_supported(int64_t heads, int64_t dim);
int jg_gat_aggregate_f32(float* out, float* lse, const float* h, const float* a_src, const float* a_dst, const int32_t* idx,
                         const int32_t* off, int64_t n_nodes, int64_t n_edges, int64_t heads, int64_t dim, float slope,
                         const void* plan, void* workspace, size_t workspace_bytes, jg_stream_t stream);

/* Backward of the fused attention aggregation (the reference differentiates the six operators one
 * by one: ops/scatterToEdge.py:42-46, ops/edgesoftmax.py:69-74, ops/scatterToVertex.py:41-45).
 * `lse` [n_nodes, heads] is what the forward wrote when given a non-NULL `lse` (log-sum-exp of each
 * destination's logits, base 2); `out` is the forward result, `grad_out` its gradient.  Outputs:
 * grad_h [n_nodes, heads*dim], grad_a_src and grad_a_dst [heads, dim].  (idx, off) is the CSC the
 * forward used; (idx_t, off_t) is the same edge set grouped by SOURCE (for every source the
 * destinations of its out-edges), e.g. from jg_coo_to_compressed.  `plan` / `plan_t` (optional) are
 * jg_gat_plan_build over `off` / `off_t`; with `plan_t` a source with millions of out-edges is cut
 * into pieces shared by many thread blocks.  Three gather passes (by destination, by source, a
 * column reduction), no atomics on data: results are run-to-run identical. */
size_t jg_gat_backward_workspace_bytes(int64_t n_nodes, int64_t n_edges, int64_t heads, int64_t dim);
int jg_gat_backward_f32(float* grad_h, float* grad_a_src, float* grad_a_dst, const float* grad_out, const float* out,
                        const float* lse, const float* h, const float* a_src, const float* a_dst, const int32_t* idx,
                        const int32_t* off, const int32_t* idx_t, const int32_t* off_t, int64_t n_nodes, int64_t n_edges,
                        int64_t heads, int64_t dim, float slope, const void* plan, const void* plan_t, void* workspace,
                        size_t workspace_bytes, jg_stream_t stream);

/* ------------------------------------------------------------------ neighbour sampling
 * Device side of the reference's layer-wise mini-batch sampler (examples/minibatch_example.py:232-362).
 *
 * jg_sample_counts replaces gpuinitco_op.gpuinitco(dst_size, fanout, dst, layer_off, global_off)
 * (ops/gpuinitco.py:30-36, ops/cpp/gpuinitco_op.cc:37-52): with cumulative == 0 it writes what that
 * kernel writes, out[0] = 0 and out[i+1] = min(in-degree of dst[i], fanout) (counts); with
 * cumulative != 0 it writes the running sum the sampler needs (examples/minibatch_example.py:253-262),
 * out[n_dst] = total.  fanout < 0 means "all neighbours".  The workspace is only used when cumulative.
 *
 * jg_sample_neighbors replaces sampleprocessing_op.sampleprocessing(fanout, dst, layer_off, layer_idx,
 * global_off, global_idx) (ops/sampleprocessing.py:28-35, ops/cpp/sampleprocessing_op.cc:38-176): column
 * i of the layer receives all in-edges of dst[i] in stored order when there are at most `fanout` of
 * them, else `fanout` entries from distinct positions of its in-edge list.  The draw is a pure
 * function of (seed, dst[i], fanout): the same call gives the same sample.  fanout <= 1024 (the
 * reference's CUDA limit); error_flag[0] is set to 1 if layer_off does not hold the running sums of
 * jg_sample_counts for this (dst, fanout) or exceeds layer_capacity (nothing is written there).
 *
 * jg_expand_columns: out[j] = values[i] (i itself when values is NULL) for every entry j of column i.
 *
 * jg_csc_to_csr replaces csctocsr_op.csctocsr(col_off, row_idx, row_off, col_idx, dst, src)
 * (ops/csctocsr.py:27-34, ops/cpp/csctocsr_op.cc:26-80): row r of the result belongs to src_ids[r],
 * column values are dst_ids[column], entries whose source id is not listed are dropped, entries of a
 * row keep the CSC traversal order (bit-exact with the reference's CPU body).  id_range bounds every
 * id in src_ids (ids in row_idx outside [0, id_range) count as unlisted); col_idx needs room for
 * n_edges entries; kept[0] receives the number of entries written.
 *
 * jg_degree_weights replaces getweight_op.getweight(vtx_size, dst, src, col_off, row_idx, w)
 * (ops/getweight.py:29-37, ops/cpp/getweight_op.cc:37-84): w[j] = 1 / (sqrtf(out-degree of the
 * entry's source) * sqrtf(in-degree of dst_ids[column])), degrees counted over this structure;
 * bit-exact with the reference's CPU body. */
size_t jg_sample_counts_workspace_bytes(int64_t n_dst);
int jg_sample_counts(const int32_t* dst, int64_t n_dst, const int32_t* g_off, int32_t fanout, int cumulative, int32_t* out,
                     void* workspace, size_t workspace_bytes, jg_stream_t stream);
int jg_sample_neighbors(const int32_t* dst, int64_t n_dst, const int32_t* layer_off, const int32_t* g_off, const int32_t* g_idx,
                        int32_t fanout, uint64_t seed, int32_t* layer_idx, int64_t layer_capacity, int32_t* error_flag,
                        jg_stream_t stream);
int jg_expand_columns(const int32_t* off, int64_t n_cols, const int32_t* values, int32_t* out, jg_stream_t stream);
size_t jg_csc_to_csr_workspace_bytes(int64_t n_src, int64_t n_edges, int64_t id_range);
int jg_csc_to_csr(const int32_t* col_off, const int32_t* row_idx, int64_t n_dst, int64_t n_edges, const int32_t* dst_ids,
                  const int32_t* src_ids, int64_t n_src, int64_t id_range, int32_t* row_off, int32_t* col_idx, int64_t* kept,
                  void* workspace, size_t workspace_bytes, jg_stream_t stream);
size_t jg_degree_weights_workspace_bytes(int64_t vtx_size);
int jg_degree_weights(int64_t vtx_size, const int32_t* dst_ids, int64_t n_dst, const int32_t* col_off, const int32_t* row_idx,
                      int64_t n_edges, float* out_w, void* workspace, size_t workspace_bytes, jg_stream_t stream);

/* ------------------------------------------------------------------ dense feature transform
 * out[n_rows, m] = act(x[n_rows, k] * W + bias) with TF32 products and fp32 accumulation on the
 * tcgen05 tensor cores; replaces the `x @ self.weight` (+ bias, + ReLU) of the reference layers
 * (nn/conv/gcn_conv.py:95,100-101, nn/conv/gat_conv.py:86-87).  `wt` is the weight TRANSPOSED,
 * [m, k] row-major; bias may be NULL; relu != 0 clamps at zero.  Supported when m <= 256
 * (jg_gemm_tf32_supported); other shapes return JG_EUNSUPPORTED.  Operands are fetched by TMA when
 * k % 4 == 0 and x, wt are 16-byte aligned, by plain loads otherwise.  The workspace
 * (jg_gemm_tf32_workspace_bytes) receives an error word: jg_gemm_tf32_status synchronises the
 * stream and returns JG_ETIMEOUT if a bounded wait inside the kernel ran out. */
int jg_gemm_tf32_supported(int64_t n_rows, int64_t k, int64_t m);
size_t jg_gemm_tf32_workspace_bytes(void);
int jg_gemm_tf32(float* out, const float* x, const float* wt, const float* bias, int64_t n_rows, int64_t k, int64_t m,
                 int relu, void* workspace, size_t workspace_bytes, jg_stream_t stream);
int jg_gemm_tf32_status(const void* workspace, jg_stream_t stream);
/* Failure-path self-test of the transform (no counterpart in the reference, whose kernels have no waits):
 * the same kernel, but every CTA's producer leaves out ring fill number `withhold` and every wait gives
 * up after `wait_spins` polls (128 .. 2^22).  The consumer's bounded wait runs out, the CTAs free their
 * TMEM and return, and jg_gemm_tf32_status on the same workspace reports JG_ETIMEOUT; nothing traps
 * and the next call on the device runs normally.  `out` is left partly written.  Needs k % 4 == 0 and
 * 16-byte aligned x, wt. */
int jg_gemm_tf32_timeout_selftest(float* out, const float* x, const float* wt, int64_t n_rows, int64_t k, int64_t m,
                                  int32_t withhold, uint32_t wait_spins, void* workspace, size_t workspace_bytes, jg_stream_t stream);
/* The same transform, optionally writing a second copy of the result in fp16 (out_half [n_rows, m] or NULL;
 * m % 8 == 0, values beyond +-65504 saturate) from the same epilogue: the copy a row-partitioned
 * aggregation offers to its peers (jg_halo_pull with src_half), without a separate conversion pass over
 * the result.  The reference broadcasts the fp32 product itself (ops/distspmm.py:31-39).
 * The error word (first 4 bytes of `workspace`) is STICKY here: the call does not clear it, a kernel whose
 * bounded wait ran out stores 1 with a plain store, so the word may live in pinned host memory that the
 * host polls without synchronising (and clears itself). */
int jg_gemm_tf32_dual(float* out, void* out_half, const float* x, const float* wt, const float* bias, int64_t n_rows, int64_t k,
                      int64_t m, int relu, void* workspace, size_t workspace_bytes, jg_stream_t stream);

/* Weight gradient gw[k, m] = x^T * g (x [n_rows, k], g [n_rows, m], both row-major) on the tensor cores, TF32
 * products: the product Jittor's autograd forms for `x @ self.weight` (nn/conv/gcn_conv.py:95).  The
 * reduction runs over the rows, so both operands are MN-major for tcgen05; the rows are cut into slices,
 * one CTA per (slice, 128 features), and the slices' partial results are added in a fixed order.
 * Supported when k % 4 == 0, m % 4 == 0 and m <= 256 (jg_gemm_tn_tf32_supported); other shapes take
 * jg_gemm_f32.  `error` is a sticky word as in jg_gemm_tf32_dual. */
int jg_gemm_tn_tf32_supported(int64_t n_rows, int64_t k, int64_t m);
size_t jg_gemm_tn_tf32_workspace_bytes(int64_t n_rows, int64_t k, int64_t m);
int jg_gemm_tn_tf32(float* gw, const float* x, const float* g, int64_t n_rows, int64_t k, int64_t m, int32_t* error,
                    void* workspace, size_t workspace_bytes, jg_stream_t stream);

/* Dense product in full fp32 on the CUDA cores: c[M, N] (row pitch ldc) = op(A) * op(B) (+ bias[N], ReLU),
 * operands addressed by strides, A(i,l) = a[i*sa0 + l*sa1], B(l,j) = b[l*sb0 + j*sb1], so that x @ W,
 * g @ W^T and x^T @ g are one kernel.  Serves what the tensor-core transform does not: the fp32 opt-out of
 * the layers (the reference's `x @ self.weight` in fp32, nn/conv/gcn_conv.py:95), the weight gradient
 * x^T g of its backward, and shapes jg_gemm_tf32 refuses.  A long reduction is cut into slices whose
 * partial results are added in a fixed order (workspace from jg_gemm_f32_workspace_bytes; may be 0). */
size_t jg_gemm_f32_workspace_bytes(int64_t M, int64_t N, int64_t K);
int jg_gemm_f32(float* c, const float* a, const float* b, const float* bias, int64_t M, int64_t N, int64_t K, int64_t sa0,
                int64_t sa1, int64_t sb0, int64_t sb1, int64_t ldc, int relu, void* workspace, size_t workspace_bytes,
                jg_stream_t stream);

/* Aggregation for callers that cannot allocate.  No counterpart in the reference: this entry
 * point exists for hosts that must not call cudaMalloc (or any allocating routine) once they
 * run - a serving process with a memory pool fixed at start-up, a plugin inside a process that
 * owns the device allocator - and therefore cannot provide the workspace jg_aggregate_f32
 * asks for.  Same result contract as jg_aggregate_f32; the scratch (ticket counter, hub plan,
 * partial rows of split hub rows) is a fixed array of jg_aggregate_static_capacity_bytes()
 * (32 MiB) inside the library image, resident on every GPU that loads the library until the
 * process exits.  The caller still passes inputs and outputs; nothing is allocated or freed.
 *   - Hub rows are cut into pieces of 1024 entries, doubled until plan and partial rows fit
 *     the array; if they cannot fit, JG_EWORKSPACE is returned with the sizes in
 *     jg_last_error() and nothing is launched.
 *   - The first call on each device looks up the array's device address; make that first call
 *     outside any stream capture, with the device current.
 *   - Every call on a device shares the one array (it keeps the previous call's contents; the
 *     words that must start at zero are cleared by each call).  Calls that overlap on the GPU -
 *     different streams, or different host threads - race on it: serialise them. */
size_t jg_aggregate_static_capacity_bytes(void);
int jg_aggregate_f32_static(float* out, const float* x, const int32_t* idx, const int32_t* off,
                            const float* w, int64_t n_out, int64_t n_in, int64_t f, int64_t nnz,
                            jg_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* JGB200_H */
