"""Host-side mirror of ``jittor_geometric.ops`` (jittor_geometric/ops/__init__.py:5-18).

Same names, argument order and meaning as the reference operators, with
``torch.Tensor`` on a CUDA device in place of ``jittor.Var``.  Every operator
calls a hand-written sm_100a kernel through the C ABI of ``libjgb200.so``; there
is no CPU or eager fallback for any of them.
"""
import ctypes
import os

import torch

from ._lib import check, lib, ptr, stream_for, workspace
from .data import CSC, CSR

__all__ = ["aggregateWithWeight", "aggregate_bias_act", "segment_aggregate", "SpmmPlan", "cootocsr", "cootocsc", "gcn_norm_csc_csr",
           "SpmmCsr", "SpmmCoo", "ScatterToEdge", "ScatterToVertex", "EdgeSoftmax", "gat_aggregate",
           "gat_aggregate_supported", "gcn_norm_coo", "linear_tf32", "check_transform_status", "linear_tf32_autograd", "linear_tf32_supported", "matmul_f32", "linear_f32_autograd", "linear_nt", "weight_grad_tf32", "toUndirected", "validate_structure"]

DEFAULT_CHUNK = int(os.environ.get("JG_SPMM_CHUNK", "1024"))
SMALL_GRAPH_NNZ = 1 << 20
SMALL_GRAPH_CHUNK = int(os.environ.get("JG_SPMM_SMALL_CHUNK", "64"))
FEW_ROWS = 1 << 19
FEW_ROWS_CHUNK = int(os.environ.get("JG_SPMM_FEW_ROWS_CHUNK", "256"))


def _as_i32(t, name):
    """int32 view of an index tensor; int64 input is range-checked and narrowed
    (the reference's cuSPARSE path accepts both widths, tests/test_spmmcsr.py:14-15)."""
    if t.dtype == torch.int32:
        return t.contiguous()
    if t.dtype == torch.int64:
        if t.numel() and int(t.max()) > 2**31 - 1:
            raise RuntimeError(f"{name}: value beyond int32")
        return t.to(torch.int32).contiguous()
    raise RuntimeError(f"{name}: expected an int32 index tensor, got {t.dtype}")


def _as_f32(t, name):
    if t.dtype != torch.float32:
        raise RuntimeError(f"{name}: expected float32, got {t.dtype}")
    return t.contiguous()


def validate_structure(idx, off, n_in):
    """Raises if a CSR/CSC structure is malformed (offsets not starting at 0, decreasing, not ending
    at the entry count, or an index outside ``[0, n_in)``).  The aggregation kernels trust their
    inputs; with ``JG_DEBUG_CHECKS=1`` every aggregation call runs this first."""
    idx, off = _as_i32(idx, "indices"), _as_i32(off, "offset")
    ws = workspace(16, idx.device if idx.numel() else off.device)
    check(lib().jg_validate_segments(ptr(idx), ptr(off), off.numel() - 1, int(n_in), idx.numel(), ptr(ws), ws.numel(),
                                     stream_for(off)), "jg_validate_segments")


def default_chunk(nnz, n_out=None):
    """Piece length for hub rows.  On a small graph the longest row is the critical path of the whole
    aggregation (one warp walks it while the rest of the GPU idles), so rows are cut much shorter
    there; on a large graph long pieces keep the number of partial rows small.  In between - many
    nonzeros but few output rows, e.g. one shard of an 8-way partition - a 1024-entry row is still a
    quarter of a millisecond of one warp's time against a kernel of a millisecond or two: 256."""
    if nnz < SMALL_GRAPH_NNZ:
        return min(DEFAULT_CHUNK, SMALL_GRAPH_CHUNK)
    if n_out is not None and n_out < FEW_ROWS:
        return min(DEFAULT_CHUNK, FEW_ROWS_CHUNK)
    return DEFAULT_CHUNK


class SpmmPlan:
    """Hub plan of one offset array: the rows longer than ``chunk`` entries, split
    into pieces so that no warp owns more than ``chunk`` entries.  Depends only
    on the offsets; build once per graph and reuse."""

    def __init__(self, off, nnz, chunk=None):
        self.n_out = off.numel() - 1
        chunk = default_chunk(nnz, self.n_out) if chunk is None else int(chunk)
        self.chunk = chunk
        self.nnz = int(nnz)
        self.off_ptr = off.data_ptr()
        nbytes = lib().jg_spmm_plan_bytes(self.n_out, self.nnz, chunk)
        self.buf = workspace(nbytes, off.device)
        check(lib().jg_spmm_plan_build(ptr(off), self.n_out, self.nnz, chunk, ptr(self.buf),
                                       self.buf.numel(), stream_for(off)), "jg_spmm_plan_build")


def _plan_of(holder, off, nnz):
    """Plan cached on a CSC/CSR container (rebuilt if its offsets tensor changed)."""
    if holder is None:
        return SpmmPlan(off, nnz)
    plan = getattr(holder, "_jg_plan", None)
    if plan is None or plan.off_ptr != off.data_ptr() or plan.nnz != nnz or plan.chunk != default_chunk(nnz, off.numel() - 1):
        plan = SpmmPlan(off, nnz)
        holder._jg_plan = plan
    return plan


def segment_aggregate(x, idx, off, w, n_out=None, plan=None, out=None, accumulate=False, bias=None, relu=False,
                      ordered=False, reserve_ctas=0):
    """out[v,:] = sum_{j in [off[v], off[v+1])} w[j] * x[idx[j],:]  (fp32).

    The one kernel behind aggregateWithWeight (forward over CSC, backward over
    CSR), SpmmCsr and SpmmCoo.  ``plan`` is an :class:`SpmmPlan` of ``off`` or
    ``None`` to process every row unsplit.  ``accumulate=True`` adds the result to ``out``.
    ``bias`` / ``relu`` fuse the layer epilogue ``act(sum + bias)`` into the store of every row
    (forward only, not together with ``accumulate``).  ``ordered=True`` sums every unsplit row
    strictly in stored order at every width (the default does for widths below 32 and above 64).
    ``reserve_ctas`` leaves that many CTA slots of the persistent grid free for a kernel on another
    stream (the halo pull of the next exchange)."""
    x = _as_f32(x, "x")
    if x.dim() != 2:
        raise RuntimeError("x: expected a 2-D feature matrix")
    idx, off, w = _as_i32(idx, "indices"), _as_i32(off, "offset"), _as_f32(w, "edge_weight")
    n_out = off.numel() - 1 if n_out is None else int(n_out)
    if off.numel() != n_out + 1:
        raise RuntimeError(f"offset has {off.numel()} entries, expected {n_out + 1}")
    nnz = idx.numel()
    if w.numel() != nnz:
        raise RuntimeError(f"edge_weight has {w.numel()} entries, indices {nnz}")
    n_in, f = x.shape
    if os.environ.get("JG_DEBUG_CHECKS") == "1":
        validate_structure(idx, off, n_in)
    if f > 32 and f % 4 and out is None and not accumulate:
        # rows that do not start on 16-byte boundaries can only be gathered with scalar loads, several
        # times slower than the vector kernel: pad the width to a multiple of four (one extra pass over
        # x) and hand back the first f columns of the padded result (a strided view)
        pad = 4 - f % 4
        xp = torch.nn.functional.pad(x, (0, pad))
        bp = None if bias is None else torch.nn.functional.pad(_as_f32(bias, "bias"), (0, pad))
        return segment_aggregate(xp, idx, off, w, n_out=n_out, plan=plan, bias=bp, relu=relu, ordered=ordered,
                                 reserve_ctas=reserve_ctas)[:, :f]
    if out is None:
        if accumulate:
            raise RuntimeError("accumulate=True needs the tensor to add to (out=)")
        out = torch.empty((n_out, f), dtype=torch.float32, device=x.device)
    chunk = plan.chunk if plan is not None else 0
    ws = workspace(lib().jg_aggregate_workspace_bytes(n_out, nnz, f, chunk), x.device)
    if reserve_ctas:
        b = None if bias is None else _as_f32(bias, "bias")
        if b is not None and b.numel() != f:
            raise RuntimeError(f"bias has {b.numel()} entries, the feature width is {f}")
        check(lib().jg_aggregate_opts_f32(ptr(out), ptr(x), ptr(idx), ptr(off), ptr(w), ptr(b), 1 if relu else 0,
                                          1 if accumulate else 0, 1 if ordered else 0, int(reserve_ctas), n_out, n_in, f, nnz,
                                          ptr(plan.buf) if plan is not None else None, chunk, ptr(ws), ws.numel(),
                                          stream_for(x)), "jg_aggregate_opts_f32")
        return out
    if bias is not None or relu:
        if accumulate:
            raise RuntimeError("segment_aggregate: the fused epilogue cannot be combined with accumulate=True")
        b = None if bias is None else _as_f32(bias, "bias")
        if b is not None and b.numel() != f:
            raise RuntimeError(f"bias has {b.numel()} entries, the feature width is {f}")
        check(lib().jg_aggregate_bias_act_f32(ptr(out), ptr(x), ptr(idx), ptr(off), ptr(w), ptr(b), 1 if relu else 0, n_out, n_in,
                                              f, nnz, ptr(plan.buf) if plan is not None else None, chunk, ptr(ws), ws.numel(),
                                              stream_for(x)), "jg_aggregate_bias_act_f32")
        return out
    if ordered and accumulate:
        raise RuntimeError("segment_aggregate: ordered=True cannot be combined with accumulate=True")
    fn = lib().jg_aggregate_add_f32 if accumulate else (lib().jg_aggregate_ordered_f32 if ordered else lib().jg_aggregate_f32)
    check(fn(ptr(out), ptr(x), ptr(idx), ptr(off), ptr(w), n_out, n_in, f, nnz,
                                 ptr(plan.buf) if plan is not None else None, chunk, ptr(ws), ws.numel(),
                                 stream_for(x)), "jg_aggregate_f32")
    return out


class _AggregateFunc(torch.autograd.Function):
    """execute/grad pairing of AggregateFunc (ops/aggregateWithWeight.py:19-41)."""

    @staticmethod
    def forward(ctx, x, csc, csr, edge_weight):
        ctx.csr = csr
        ctx.weight = edge_weight
        w = edge_weight if isinstance(edge_weight, torch.Tensor) else csc.edge_weight
        nnz = csc.row_indices.numel()
        return segment_aggregate(x, csc.row_indices, csc.column_offset, w,
                                 plan=_plan_of(csc, csc.column_offset, nnz))

    @staticmethod
    def backward(ctx, grad_output):
        csr = ctx.csr
        w = ctx.weight if isinstance(ctx.weight, torch.Tensor) else csr.edge_weight
        nnz = csr.column_indices.numel()
        g = segment_aggregate(grad_output.contiguous(), csr.column_indices, csr.row_offset, w,
                              plan=_plan_of(csr, csr.row_offset, nnz))
        return g, None, None, None


def aggregateWithWeight(x, csc, csr, weight=None):
    """Weighted neighbour aggregation of the vertex embedding matrix ``x`` over the
    graph given as CSC (forward) and CSR (backward)
    (ops/aggregateWithWeight.py:53-55).  ``weight`` overrides the containers'
    edge weights for both directions, as in the reference."""
    return _AggregateFunc.apply(x, csc, csr, weight)


class _AggregateBiasAct(torch.autograd.Function):
    """``act(A x + b)`` with the epilogue fused into the aggregation's store; backward masks the
    gradient with the saved output, sums it for the bias and aggregates it over the CSR."""

    @staticmethod
    def forward(ctx, x, bias, csc, csr, relu):
        out = segment_aggregate(x, csc.row_indices, csc.column_offset, csc.edge_weight,
                                plan=_plan_of(csc, csc.column_offset, csc.row_indices.numel()), bias=bias, relu=relu)
        ctx.csr, ctx.relu, ctx.has_bias = csr, relu, bias is not None
        if relu:
            ctx.save_for_backward(out)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        g = grad_output
        if ctx.relu:
            (out,) = ctx.saved_tensors
            g = g * (out > 0)
        g = g.contiguous()
        csr = ctx.csr
        gx = None
        if ctx.needs_input_grad[0]:
            gx = segment_aggregate(g, csr.column_indices, csr.row_offset, csr.edge_weight,
                                   plan=_plan_of(csr, csr.row_offset, csr.column_indices.numel()))
        gb = g.sum(0) if ctx.has_bias and ctx.needs_input_grad[1] else None
        return gx, gb, None, None, None


def aggregate_bias_act(x, csc, csr, bias=None, relu=False):
    """``act(aggregateWithWeight(x, csc, csr) + bias)`` in one kernel: what the reference computes
    with separate elementwise passes after the aggregation (nn/conv/gcn_conv.py:96-101 and the
    ``nn.relu`` of examples/gcn_example.py:76)."""
    if bias is None and not relu:
        return aggregateWithWeight(x, csc, csr)
    return _AggregateBiasAct.apply(x, bias, csc, csr, bool(relu))


def _edge_index(edge_index):
    ei = _as_i32(edge_index, "edge_index")
    if ei.dim() != 2 or ei.shape[0] != 2:
        raise RuntimeError("edge_index: expected shape [2, E]")
    return ei


def _compress(edge_index, edge_weight, v_num, by, sorted):
    ei = _edge_index(edge_index)
    E = ei.shape[1]
    w = None if edge_weight is None else _as_f32(edge_weight, "edge_weight")
    if w is not None and w.numel() != E:
        raise RuntimeError(f"edge_weight has {w.numel()} entries, edge_index {E}")
    v_num = int(v_num)
    dev = ei.device
    idx = torch.empty(E, dtype=torch.int32, device=dev)
    off = torch.empty(v_num + 1, dtype=torch.int32, device=dev)
    ow = torch.empty(E, dtype=torch.float32, device=dev)
    ws = workspace(lib().jg_convert_workspace_bytes(E, v_num), dev)
    check(lib().jg_coo_to_compressed(ptr(ei), ptr(w), E, v_num, by, 1 if sorted else 0, ptr(idx), ptr(off), ptr(ow),
                                     ptr(ws), ws.numel(), stream_for(ei)), "jg_coo_to_compressed")
    return idx, off, ow


def cootocsr(edge_index, edge_weight, v_num, sorted=False):
    """COO -> CSR (ops/cootocsr.py:28-35): rows keyed by source, entries of a row in COO
    order (the reference's stable layout); ``sorted=True`` orders them by column instead."""
    idx, off, w = _compress(edge_index, edge_weight, v_num, 0, sorted)
    return CSR(idx, off, w)


def cootocsc(edge_index, edge_weight, v_num, sorted=False):
    """COO -> CSC (ops/cootocsc.py:29-36): columns keyed by destination."""
    idx, off, w = _compress(edge_index, edge_weight, v_num, 1, sorted)
    return CSC(idx, off, w)


def gcn_norm_csc_csr(edge_index, edge_weight, num_nodes, improved=False, want_csr=True, sorted=False,
                     add_self_loops=True):
    """``gcn_norm`` (nn/conv/gcn_conv.py:18-37) fused with ``cootocsc`` / ``cootocsr``: returns
    ``(CSC, CSR)`` of the self-looped, symmetrically normalised graph without building the
    normalised COO list (``CSR`` is ``None`` when ``want_csr`` is false)."""
    ei = _edge_index(edge_index)
    E0 = ei.shape[1]
    n = int(num_nodes)
    w = None if edge_weight is None else _as_f32(edge_weight, "edge_weight")
    dev = ei.device
    cap = E0 + n
    mk_i = lambda m: torch.empty(m, dtype=torch.int32, device=dev)
    mk_f = lambda m: torch.empty(m, dtype=torch.float32, device=dev)
    csc = (mk_i(cap), mk_i(n + 1), mk_f(cap))
    csr = (mk_i(cap), mk_i(n + 1), mk_f(cap)) if want_csr else (None, None, None)
    count = torch.zeros(1, dtype=torch.int64, device=dev)
    ws = workspace(lib().jg_convert_workspace_bytes(E0, n), dev)
    check(lib().jg_gcn_norm_compressed(ptr(ei), ptr(w), E0, n, 2.0 if improved else 1.0, 1 if add_self_loops else 0,
                                       1 if sorted else 0,
                                       ptr(csc[0]), ptr(csc[1]), ptr(csc[2]), ptr(csr[0]), ptr(csr[1]), ptr(csr[2]),
                                       ptr(count), ptr(ws), ws.numel(), stream_for(ei)), "jg_gcn_norm_compressed")
    E = int(count.item())  # one synchronisation per graph: the entry count sizes the views
    out_csc = CSC(csc[0][:E], csc[1], csc[2][:E])
    out_csr = CSR(csr[0][:E], csr[1], csr[2][:E]) if want_csr else None
    return out_csc, out_csr


def gcn_norm_coo(edge_index, edge_weight, num_nodes, improved=False, add_self_loops=True):
    """``gcn_norm`` (nn/conv/gcn_conv.py:18-37) as the reference returns it: the COO list with
    (v,v) entries removed, one loop per node appended, and symmetric-normalised weights;
    ``add_self_loops=False`` normalises the list as given."""
    ei = _edge_index(edge_index)
    E0, n, dev = ei.shape[1], int(num_nodes), ei.device
    w = None if edge_weight is None else _as_f32(edge_weight, "edge_weight")
    cap = E0 + n
    out = torch.empty((2, cap), dtype=torch.int32, device=dev)
    ow = torch.empty(cap, dtype=torch.float32, device=dev)
    count = torch.zeros(1, dtype=torch.int64, device=dev)
    ws = workspace(lib().jg_gcn_norm_coo_workspace_bytes(E0, n), dev)
    check(lib().jg_gcn_norm_coo(ptr(ei), ptr(w), E0, n, 2.0 if improved else 1.0, 1 if add_self_loops else 0,
                                ptr(out[0]), ptr(out[1]), ptr(ow),
                                ptr(count), ptr(ws), ws.numel(), stream_for(ei)), "jg_gcn_norm_coo")
    E = int(count.item())
    return out[:, :E].contiguous(), ow[:E]


def toUndirected(edge_index, edge_attr, num_nodes):
    """Mirror every edge, sort by (row, col) and drop duplicate pairs (ops/toundirected.py:16-22).
    Returns ``(new_edge_index [2, M], new_edge_attr [M])``."""
    ei = _edge_index(edge_index)
    E, dev = ei.shape[1], ei.device
    attr = _as_f32(edge_attr, "edge_attr")
    if attr.numel() != E:
        raise RuntimeError(f"edge_attr has {attr.numel()} entries, edge_index {E}")
    n = int(num_nodes) if num_nodes is not None else (int(ei.max()) + 1 if E else 0)
    out = torch.empty((2, max(2 * E, 1)), dtype=torch.int32, device=dev)
    oa = torch.empty(max(2 * E, 1), dtype=torch.float32, device=dev)
    count = torch.zeros(1, dtype=torch.int64, device=dev)
    ws = workspace(lib().jg_to_undirected_workspace_bytes(E, n), dev)
    check(lib().jg_to_undirected(ptr(ei), ptr(attr), E, n, ptr(out[0]), ptr(out[1]), ptr(oa), ptr(count), ptr(ws),
                                 ws.numel(), stream_for(ei)), "jg_to_undirected")
    m = int(count.item())
    return out[:, :m].contiguous(), oa[:m]


# ------------------------------------------------------------------------------ SpMM front ends
def _csr_rows(csr):
    """Source of every CSR entry (row ids expanded from the offsets)."""
    off = _as_i32(csr.row_offset, "row_offset")
    n = off.numel() - 1
    out = torch.empty(csr.column_indices.numel(), dtype=torch.int32, device=off.device)
    if out.numel():
        check(lib().jg_expand_columns(ptr(off), n, None, ptr(out), stream_for(off)), "jg_expand_columns")
    return out


def _transposed_of(csr, n_cols=None):
    """CSC of the same matrix, built on device once and cached on the CSR object: the
    destination-major structure an atomics-free ``A^T x`` needs.  ``n_cols`` is the column count
    of a rectangular block (default: square)."""
    key = (csr.column_indices.data_ptr(), csr.row_offset.data_ptr(),
           0 if csr.edge_weight is None else csr.edge_weight.data_ptr(), n_cols)
    cached = getattr(csr, "_jg_transposed", None)
    if cached is None or cached[0] != key:
        n = csr.row_offset.numel() - 1 if n_cols is None else int(n_cols)
        ei = torch.stack([_csr_rows(csr), _as_i32(csr.column_indices, "column_indices")])
        cached = (key, cootocsc(ei, csr.edge_weight, n))
        csr._jg_transposed = cached
    return cached[1]


class _SpmmCsrFunc(torch.autograd.Function):
    """execute/grad pairing of SpmmCsrFunc (ops/spmmcsr.py:21-39).  The reference's grad applies the
    SAME operator (same trans_A) to grad_output, which is the true gradient only for a symmetric
    matrix; that behaviour is kept."""

    @staticmethod
    def forward(ctx, x, csr, trans_A, trans_B):
        if trans_B:
            raise RuntimeError("SpmmCsr: trans_B=True is not supported (the reference never passes it)")
        ctx.csr, ctx.trans_A = csr, trans_A
        return _spmm_csr(x, csr, trans_A)

    @staticmethod
    def backward(ctx, grad_output):
        return _spmm_csr(grad_output.contiguous(), ctx.csr, ctx.trans_A), None, None, None


def _spmm_csr(x, csr, trans_A):
    if trans_A:
        t = _transposed_of(csr)
        return segment_aggregate(x, t.row_indices, t.column_offset, t.edge_weight,
                                 plan=_plan_of(t, t.column_offset, t.row_indices.numel()))
    return segment_aggregate(x, csr.column_indices, csr.row_offset, csr.edge_weight,
                             plan=_plan_of(csr, csr.row_offset, csr.column_indices.numel()))


def SpmmCsr(x, csr, trans_A=True, trans_B=False):
    """``op(A) @ x`` for a CSR matrix (ops/spmmcsr.py:42-44).  With the default ``trans_A=True`` and
    a source-keyed CSR this is out[dst] = sum w * x[src], the same result as
    ``aggregateWithWeight`` over the CSC."""
    return _SpmmCsrFunc.apply(x, csr, trans_A, trans_B)


class _SpmmCooFunc(torch.autograd.Function):
    """SpmmCooFunc (ops/spmmcoo.py:19-41); its grad calls the operator with default flags."""

    @staticmethod
    def forward(ctx, x, edge_index, edge_weight, trans_A, trans_B):
        if trans_B:
            raise RuntimeError("SpmmCoo: trans_B=True is not supported (the reference never passes it)")
        n = x.shape[0]
        fwd = cootocsc(edge_index, edge_weight, n) if trans_A else cootocsr(edge_index, edge_weight, n)
        ctx.n, ctx.ei, ctx.w = n, edge_index, edge_weight
        idx = fwd.row_indices if trans_A else fwd.column_indices
        off = fwd.column_offset if trans_A else fwd.row_offset
        return segment_aggregate(x, idx, off, fwd.edge_weight, plan=SpmmPlan(off, idx.numel()))

    @staticmethod
    def backward(ctx, grad_output):
        t = cootocsr(ctx.ei, ctx.w, ctx.n)
        g = segment_aggregate(grad_output.contiguous(), t.column_indices, t.row_offset, t.edge_weight,
                              plan=SpmmPlan(t.row_offset, t.column_indices.numel()))
        return g, None, None, None, None


def SpmmCoo(x, edge_index, edge_weight, trans_A=True, trans_B=False):
    """``op(A) @ x`` for a COO matrix whose rows are ``edge_index[0]`` (ops/spmmcoo.py:43-45)."""
    return _SpmmCooFunc.apply(x, edge_index, edge_weight, trans_A, trans_B)


# ------------------------------------------------------------------------------ per-edge operators
def _scatter_to_edge(x, csc, flag):
    x = _as_f32(x, "x")
    idx, off = _as_i32(csc.row_indices, "row_indices"), _as_i32(csc.column_offset, "column_offset")
    E, n, c = idx.numel(), off.numel() - 1, x.shape[1]
    out = torch.empty((E, c), dtype=torch.float32, device=x.device)
    check(lib().jg_scatter_to_edge_f32(ptr(out), ptr(x), ptr(idx), ptr(off), n, E, c, flag, stream_for(x)),
          "jg_scatter_to_edge_f32")
    return out


def _edge_to_vertex(msg, csc, flag):
    msg = _as_f32(msg, "msg")
    idx, off = _as_i32(csc.row_indices, "row_indices"), _as_i32(csc.column_offset, "column_offset")
    E, n, c = idx.numel(), off.numel() - 1, msg.shape[1]
    if msg.shape[0] != E:
        raise RuntimeError(f"edge tensor has {msg.shape[0]} rows, the graph {E} edges")
    if flag == 1 and E > 0 and (c <= 32 or c % 4 == 0):
        # the per-destination sum is an aggregation of the message rows with identity indices and unit
        # weights: the aggregation kernel brings vector loads, eight rows in flight per lane and hub
        # rows cut into pieces, and its ordered variant keeps the reference's summation order
        ident = getattr(csc, "_jg_identity", None)
        if ident is None or ident[0].numel() != E or ident[0].device != msg.device:
            ident = (torch.arange(E, dtype=torch.int32, device=msg.device), torch.ones(E, dtype=torch.float32, device=msg.device))
            csc._jg_identity = ident
        plan = getattr(csc, "_jg_plan_ordered", None)         # long pieces: only real hubs lose the stored order
        if plan is None or plan.off_ptr != off.data_ptr() or plan.nnz != E:
            plan = SpmmPlan(off, E, chunk=DEFAULT_CHUNK)
            csc._jg_plan_ordered = plan
        return segment_aggregate(msg, ident[0], off, ident[1], n_out=n, plan=plan, ordered=True)
    out = torch.empty((n, c), dtype=torch.float32, device=msg.device)
    check(lib().jg_edge_to_vertex_f32(ptr(out), ptr(msg), ptr(idx), ptr(off), n, E, c, flag, stream_for(msg)),
          "jg_edge_to_vertex_f32")
    return out


class _ScatterToEdgeFunc(torch.autograd.Function):
    """ScatterToEdgeFunc (ops/scatterToEdge.py:22-46): backward is edge_to_vertex with the same flag."""

    @staticmethod
    def forward(ctx, x, csc, flow):
        ctx.csc, ctx.flag = csc, (0 if flow == "src" else 1)
        return _scatter_to_edge(x, csc, ctx.flag)

    @staticmethod
    def backward(ctx, grad_output):
        return _edge_to_vertex(grad_output.contiguous(), ctx.csc, ctx.flag), None, None


def ScatterToEdge(x, csc, flow):
    """Node rows copied onto edges in CSC order: ``flow="src"`` takes each edge's source row,
    anything else its destination row (ops/scatterToEdge.py:49-51)."""
    return _ScatterToEdgeFunc.apply(x, csc, flow)


class _ScatterToVertexFunc(torch.autograd.Function):
    """ScatterToVertexFunc (ops/scatterToVertex.py:23-46): always sums per destination, whatever
    ``flow`` says; backward copies the destination's gradient row onto its in-edges."""

    @staticmethod
    def forward(ctx, x, csc, flow):
        ctx.csc = csc
        return _edge_to_vertex(x, csc, 1)

    @staticmethod
    def backward(ctx, grad_output):
        return _scatter_to_edge(grad_output.contiguous(), ctx.csc, 1), None, None


def ScatterToVertex(x, csc, flow):
    return _ScatterToVertexFunc.apply(x, csc, flow)


def _edge_softmax(x, off, bwd_y=None):
    shape = x.shape
    x2 = _as_f32(x, "x").reshape(shape[0], -1)
    E, h = x2.shape
    n = off.numel() - 1
    out = torch.empty_like(x2)     # every edge lies in exactly one segment, so every element is written
    if bwd_y is None:
        check(lib().jg_edge_softmax_fwd_f32(ptr(out), ptr(x2), ptr(off), n, E, h, stream_for(x2)), "jg_edge_softmax_fwd_f32")
    else:
        y2 = bwd_y.reshape(E, h).contiguous()
        check(lib().jg_edge_softmax_bwd_f32(ptr(out), ptr(x2), ptr(y2), ptr(off), n, E, h, stream_for(x2)),
              "jg_edge_softmax_bwd_f32")
    return out.reshape(shape)


class _EdgeSoftmaxFunc(torch.autograd.Function):
    """EdgeSoftmaxFunc (ops/edgesoftmax.py:62-74)."""

    @staticmethod
    def forward(ctx, x, csc):
        off = _as_i32(csc.column_offset, "column_offset")
        if x.shape[0] != csc.row_indices.numel():
            raise RuntimeError(f"x has {x.shape[0]} rows, the graph {csc.row_indices.numel()} edges")
        y = _edge_softmax(x, off)
        ctx.off = off
        ctx.save_for_backward(y)
        return y

    @staticmethod
    def backward(ctx, grad_output):
        (y,) = ctx.saved_tensors
        return _edge_softmax(grad_output.contiguous(), ctx.off, bwd_y=y), None


def EdgeSoftmax(x, csc):
    """Softmax of per-edge scores over the in-edges of every destination
    (ops/edgesoftmax.py:78-80).  ``x`` is ``[E]`` or ``[E, 1]`` as in the reference, or ``[E, H]``
    for H independent heads."""
    return _EdgeSoftmaxFunc.apply(x, csc)


def gat_aggregate_supported(heads, dim):
    return bool(lib().jg_gat_aggregate_supported(int(heads), int(dim)))


def _gat_plan(holder, attr, off, n, like):
    plan = getattr(holder, attr, None)
    if plan is None or plan[0] != off.data_ptr():
        buf = workspace(lib().jg_gat_plan_bytes(n), like.device)
        check(lib().jg_gat_plan_build(ptr(off), n, ptr(buf), buf.numel(), stream_for(like)), "jg_gat_plan_build")
        plan = (off.data_ptr(), buf)
        setattr(holder, attr, plan)
    return plan[1]


def _gat_forward(h, a_src, a_dst, csc, heads, slope, want_lse):
    n, c = h.shape
    dim = c // heads
    idx, off = _as_i32(csc.row_indices, "row_indices"), _as_i32(csc.column_offset, "column_offset")
    if off.numel() != n + 1:
        raise RuntimeError("gat_aggregate: column_offset does not match h")
    out = torch.empty_like(h)
    lse = torch.empty((n, heads), dtype=torch.float32, device=h.device) if want_lse else None
    plan = _gat_plan(csc, "_jg_gat_plan", off, n, h)
    ws = workspace(lib().jg_gat_aggregate_workspace_bytes(n, idx.numel(), heads, dim), h.device)
    check(lib().jg_gat_aggregate_f32(ptr(out), ptr(lse), ptr(h), ptr(a_src), ptr(a_dst), ptr(idx), ptr(off), n, idx.numel(),
                                     heads, dim, float(slope), ptr(plan), ptr(ws), ws.numel(), stream_for(h)),
          "jg_gat_aggregate_f32")
    return out, lse


def _by_source(csc):
    """The edges of a CSC grouped by source (for every source the destinations of its out-edges),
    built on device once and cached on the container."""
    view = getattr(csc, "_jg_by_source_view", None)
    if view is None or view.column_indices.data_ptr() != csc.row_indices.data_ptr():
        view = CSR(csc.row_indices, csc.column_offset, csc.edge_weight)
        csc._jg_by_source_view = view
    return _transposed_of(view)


class _GatAggregate(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, a_src, a_dst, csc, heads, slope):
        out, lse = _gat_forward(h, a_src, a_dst, csc, heads, slope, True)
        ctx.save_for_backward(h, a_src, a_dst, out, lse)
        ctx.csc, ctx.heads, ctx.slope = csc, heads, slope
        return out

    @staticmethod
    def backward(ctx, grad_out):
        h, a_src, a_dst, out, lse = ctx.saved_tensors
        csc, heads = ctx.csc, ctx.heads
        n, c = h.shape
        dim = c // heads
        g = _as_f32(grad_out, "grad_out")
        t = _by_source(csc)
        idx, off = _as_i32(csc.row_indices, "row_indices"), _as_i32(csc.column_offset, "column_offset")
        idx_t, off_t = t.row_indices, t.column_offset
        grad_h = torch.empty_like(h)
        grad_as, grad_ad = torch.empty_like(a_src), torch.empty_like(a_dst)
        plan = _gat_plan(csc, "_jg_gat_plan", off, n, h)
        plan_t = _gat_plan(t, "_jg_gat_plan", off_t, n, h)
        ws = workspace(lib().jg_gat_backward_workspace_bytes(n, idx.numel(), heads, dim), h.device)
        check(lib().jg_gat_backward_f32(ptr(grad_h), ptr(grad_as), ptr(grad_ad), ptr(g), ptr(out), ptr(lse), ptr(h), ptr(a_src),
                                        ptr(a_dst), ptr(idx), ptr(off), ptr(idx_t), ptr(off_t), n, idx.numel(), heads, dim,
                                        float(ctx.slope), ptr(plan), ptr(plan_t), ptr(ws), ws.numel(), stream_for(h)),
              "jg_gat_backward_f32")
        return grad_h, grad_as, grad_ad, None, None, None


def gat_aggregate(h, a_src, a_dst, csc, heads, slope=0.2):
    """Fused edge phase of the attention layer (nn/conv/gat_conv.py:60-83): logits, per-destination
    softmax and weighted aggregation in one pass.  ``h`` is ``[N, heads*dim]``; ``a_src`` and
    ``a_dst`` are ``[heads, dim]``.  Differentiable in ``h``, ``a_src`` and ``a_dst`` (fused
    backward: two gather passes and a column reduction, no ``[E, C]`` temporaries)."""
    h = _as_f32(h, "h")
    n, c = h.shape
    heads = int(heads)
    dim = c // heads
    shape_s, shape_d = a_src.shape, a_dst.shape
    a_src, a_dst = _as_f32(a_src, "a_src").reshape(-1), _as_f32(a_dst, "a_dst").reshape(-1)
    if a_src.numel() != c or a_dst.numel() != c or dim * heads != c:
        raise RuntimeError("gat_aggregate: a_src/a_dst must hold heads*dim values")
    if torch.is_grad_enabled() and (h.requires_grad or a_src.requires_grad or a_dst.requires_grad):
        return _GatAggregate.apply(h, a_src, a_dst, csc, heads, float(slope))
    return _gat_forward(h, a_src, a_dst, csc, heads, slope, False)[0]


# ------------------------------------------------------------------------------ dense transform
def linear_tf32_supported(n_rows, k, m):
    return bool(lib().jg_gemm_tf32_supported(int(n_rows), int(k), int(m)))


_tf32_status = {}      # device index -> pinned host word a transform kernel sets when a bounded wait ran out


def _tf32_status_word(device):
    idx = device.index if device.index is not None else torch.cuda.current_device()
    word = _tf32_status.get(idx)
    if word is None:
        word = torch.zeros(64, dtype=torch.int32).pin_memory()
        _tf32_status[idx] = word
    return word


def check_transform_status(device=None, synchronize=False):
    """Raises if a ``linear_tf32`` kernel on ``device`` gave up on a bounded wait (its output is then
    not valid).  The kernels report through a word in pinned host memory, so the check costs nothing;
    it runs at the start of every ``linear_tf32`` call, and a training loop may call it (with
    ``synchronize=True`` for a definitive answer) before the optimiser step."""
    words = _tf32_status.items() if device is None else [(None, _tf32_status_word(torch.device(device)))]
    if synchronize:
        torch.cuda.synchronize()
    for _, word in list(words):
        if int(word[0]):
            word[0] = 0
            raise RuntimeError("jg_gemm_tf32: a bounded wait inside the kernel ran out [JG_ETIMEOUT]; the result of "
                               "that transform is not valid")


def linear_tf32(x, weight, bias=None, relu=False, weight_t=None, check_status=False, out=None, out_half=None):
    """``act(x @ weight + bias)`` on the tcgen05 tensor cores (TF32 products, fp32 accumulation):
    the dense feature transform of the layers (nn/conv/gcn_conv.py:95, nn/conv/gat_conv.py:86).
    ``weight`` is ``[k, m]`` as the layers store it; ``weight_t`` may carry its cached transpose.
    Forward only.  ``out`` receives the result in place (e.g. the feature buffer of a partitioned
    aggregation); ``out_half`` additionally receives an fp16 copy from the same epilogue (the half-width
    halo payload of :class:`dist.ShardedGraph`).  ``check_status=True`` synchronises and raises if a bounded wait in the kernel
    ran out."""
    x = _as_f32(x, "x")
    n, k = x.shape
    m = weight.shape[1]
    wt = weight_t if weight_t is not None else _as_f32(weight, "weight").t().contiguous()
    b = None if bias is None else _as_f32(bias, "bias")
    if out is None:
        out = torch.empty((n, m), dtype=torch.float32, device=x.device)
    elif out.shape != (n, m) or out.dtype != torch.float32 or not out.is_contiguous():
        raise RuntimeError(f"out: expected a contiguous float32 [{n}, {m}] tensor")
    word = _tf32_status_word(x.device)
    if int(word[0]):                       # an earlier transform on this device gave up: its consumers must not carry on
        check_transform_status(x.device)
    st = stream_for(x)
    if out_half is not None and (out_half.dtype != torch.float16 or out_half.shape[1] != m or out_half.shape[0] < n
                                 or not out_half.is_contiguous()):
        raise RuntimeError(f"out_half: expected a contiguous float16 tensor of at least [{n}, {m}]")
    check(lib().jg_gemm_tf32_dual(ptr(out), ptr(out_half), ptr(x), ptr(wt), ptr(b), n, k, m, 1 if relu else 0,
                                  ctypes.c_void_p(word.data_ptr()), 256, st), "jg_gemm_tf32_dual")
    if check_status:
        check_transform_status(x.device, synchronize=True)
    return out


def matmul_f32(a, b, trans_a=False, trans_b=False, bias=None, relu=False):
    """``act(op(a) @ op(b) + bias)`` in full fp32 on the library's own CUDA-core kernel (no vendor GEMM):
    the fp32 opt-out of the layers' transform, the weight gradient ``x^T g`` and the shapes
    ``linear_tf32`` does not take.  ``a`` and ``b`` are 2-D and contiguous; the transposes are taken by
    stride, nothing is copied."""
    a, b = _as_f32(a, "a"), _as_f32(b, "b")
    M, K = (a.shape[1], a.shape[0]) if trans_a else a.shape
    K2, N = (b.shape[1], b.shape[0]) if trans_b else b.shape
    if K != K2:
        raise RuntimeError(f"matmul_f32: inner sizes differ ({K} and {K2})")
    sa0, sa1 = (1, a.shape[1]) if trans_a else (a.shape[1], 1)
    sb0, sb1 = (1, b.shape[1]) if trans_b else (b.shape[1], 1)
    bb = None if bias is None else _as_f32(bias, "bias")
    out = torch.empty((M, N), dtype=torch.float32, device=a.device)
    ws = workspace(lib().jg_gemm_f32_workspace_bytes(M, N, K), a.device)
    check(lib().jg_gemm_f32(ptr(out), ptr(a), ptr(b), ptr(bb), M, N, K, sa0, sa1, sb0, sb1, N, 1 if relu else 0, ptr(ws),
                            ws.numel(), stream_for(a)), "jg_gemm_f32")
    return out


class _LinearF32(torch.autograd.Function):
    """``act(x @ weight)`` in fp32 with its backward, every product on :func:`matmul_f32`."""

    @staticmethod
    def forward(ctx, x, weight, relu):
        out = matmul_f32(x, weight, relu=relu)
        ctx.relu = relu
        ctx.save_for_backward(x, weight, out if relu else None)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        x, weight, out = ctx.saved_tensors
        g = _relu_mask(grad_output, out) if ctx.relu else grad_output.contiguous()
        gx = matmul_f32(g, weight, trans_b=True) if ctx.needs_input_grad[0] else None
        gw = matmul_f32(x, g, trans_a=True) if ctx.needs_input_grad[1] else None
        return gx, gw, None


def linear_f32_autograd(x, weight, relu=False):
    """The layers' transform in fp32 (``tf32=False``), usable in training."""
    return _LinearF32.apply(_as_f32(x, "x"), _as_f32(weight, "weight"), bool(relu))


def weight_grad_tf32(x, g):
    """``x^T @ g`` (the weight gradient of ``x @ W``) on the tensor cores with TF32 products when the shape
    allows (widths multiples of 4, at most 256 output columns), else in fp32 on the CUDA cores."""
    x, g = _as_f32(x, "x"), _as_f32(g, "g")
    n, k = x.shape
    m = g.shape[1]
    if g.shape[0] != n:
        raise RuntimeError("weight_grad_tf32: x and g need the same number of rows")
    if not lib().jg_gemm_tn_tf32_supported(n, k, m) or (x.data_ptr() | g.data_ptr()) % 16:
        return matmul_f32(x, g, trans_a=True)
    word = _tf32_status_word(x.device)
    if int(word[0]):
        check_transform_status(x.device)
    out = torch.empty((k, m), dtype=torch.float32, device=x.device)
    ws = workspace(lib().jg_gemm_tn_tf32_workspace_bytes(n, k, m), x.device)
    check(lib().jg_gemm_tn_tf32(ptr(out), ptr(x), ptr(g), n, k, m, ctypes.c_void_p(word.data_ptr()), ptr(ws), ws.numel(),
                                stream_for(x)), "jg_gemm_tn_tf32")
    return out


class _LinearNT(torch.autograd.Function):
    """``x @ weight^T + bias`` for a weight stored ``[out, in]`` (the layout of a ``Linear`` layer):
    TF32 forward and input gradient on the tensor-core kernel when asked for, everything else on the fp32
    kernel; the bias gradient is a column sum."""

    @staticmethod
    def forward(ctx, x, weight, bias, tf32):
        ctx.tf32 = tf32
        ctx.has_bias = bias is not None
        ctx.save_for_backward(x, weight)
        if tf32 and linear_tf32_supported(x.shape[0], x.shape[1], weight.shape[0]):
            return linear_tf32(x, weight.t(), bias=bias, weight_t=weight.contiguous())
        return matmul_f32(x, weight, trans_b=True, bias=bias)

    @staticmethod
    def backward(ctx, grad_output):
        x, weight = ctx.saved_tensors
        g = grad_output.contiguous()
        gx = gw = gb = None
        if ctx.needs_input_grad[0]:
            if ctx.tf32 and linear_tf32_supported(g.shape[0], g.shape[1], weight.shape[1]):
                gx = linear_tf32(g, weight, weight_t=weight.t().contiguous())
            else:
                gx = matmul_f32(g, weight)
        if ctx.needs_input_grad[1]:
            gw = weight_grad_tf32(g, x) if ctx.tf32 else matmul_f32(g, x, trans_a=True)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            gb = g.sum(0)
        return gx, gw, gb, None


def linear_nt(x, weight, bias=None, tf32=True):
    """``x @ weight^T + bias`` with ``weight`` stored ``[out, in]``; differentiable."""
    return _LinearNT.apply(_as_f32(x, "x"), _as_f32(weight, "weight"), bias, bool(tf32))


def _relu_mask(grad, out):
    """``grad * (out > 0)``: the gradient through a fused ReLU, from the saved output."""
    return (grad * (out > 0)).contiguous()


class _LinearTF32(torch.autograd.Function):
    """``act(x @ weight)`` through the tcgen05 kernel with a backward: ``grad_x = g @ weight^T`` runs
    on the same kernel (its transposed operand is the weight itself); ``grad_weight = x^T @ g`` is a
    reduction over the rows and runs on its own tensor-core kernel (MN-major operands, sliced over the
    rows, fixed-order sum of the slices) or, for widths that are not multiples of 4, on the fp32 kernel."""

    @staticmethod
    def forward(ctx, x, weight, relu):
        out = linear_tf32(x, weight, relu=relu)
        ctx.relu = relu
        ctx.save_for_backward(x, weight, out if relu else None)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        x, weight, out = ctx.saved_tensors
        g = _relu_mask(grad_output, out) if ctx.relu else grad_output.contiguous()
        gx = gw = None
        if ctx.needs_input_grad[0]:
            if linear_tf32_supported(g.shape[0], g.shape[1], weight.shape[0]):
                gx = linear_tf32(g, weight.t(), weight_t=weight.contiguous())
            else:
                gx = matmul_f32(g, weight, trans_b=True)
        if ctx.needs_input_grad[1]:
            gw = weight_grad_tf32(x, g)
        return gx, gw, None


def linear_tf32_autograd(x, weight, relu=False):
    """:func:`linear_tf32` usable in training (TF32 products in forward and backward)."""
    return _LinearTF32.apply(_as_f32(x, "x"), _as_f32(weight, "weight"), bool(relu))

