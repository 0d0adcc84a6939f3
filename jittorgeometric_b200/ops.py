"""Host-side mirror of ``jittor_geometric.ops`` (jittor_geometric/ops/__init__.py:5-18).

Same names, argument order and meaning as the reference operators, with
``torch.Tensor`` on a CUDA device in place of ``jittor.Var``.  Every operator
calls a hand-written sm_100a kernel through the C ABI of ``libjgb200.so``; there
is no CPU, eager or library fallback.
"""
import os

import torch

from . import _lib
from ._lib import check, lib, ptr, stream_for, workspace
from .data import CSC, CSR

__all__ = ["aggregateWithWeight", "segment_aggregate", "SpmmPlan", "cootocsr", "cootocsc", "gcn_norm_csc_csr"]

DEFAULT_CHUNK = int(os.environ.get("JG_SPMM_CHUNK", "1024"))


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


class SpmmPlan:
    """Hub plan of one offset array: the rows longer than ``chunk`` entries, split
    into pieces so that no warp owns more than ``chunk`` entries.  Depends only
    on the offsets; build once per graph and reuse."""

    def __init__(self, off, nnz, chunk=None):
        chunk = DEFAULT_CHUNK if chunk is None else int(chunk)
        self.chunk = chunk
        self.n_out = off.numel() - 1
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
    if plan is None or plan.off_ptr != off.data_ptr() or plan.nnz != nnz or plan.chunk != DEFAULT_CHUNK:
        plan = SpmmPlan(off, nnz)
        holder._jg_plan = plan
    return plan


def segment_aggregate(x, idx, off, w, n_out=None, plan=None, out=None):
    """out[v,:] = sum_{j in [off[v], off[v+1])} w[j] * x[idx[j],:]  (fp32).

    The one kernel behind aggregateWithWeight (forward over CSC, backward over
    CSR), SpmmCsr and SpmmCoo.  ``plan`` is an :class:`SpmmPlan` of ``off`` or
    ``None`` to process every row unsplit."""
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
    if out is None:
        out = torch.empty((n_out, f), dtype=torch.float32, device=x.device)
    chunk = plan.chunk if plan is not None else 0
    ws = workspace(lib().jg_aggregate_workspace_bytes(n_out, nnz, f, chunk), x.device)
    check(lib().jg_aggregate_f32(ptr(out), ptr(x), ptr(idx), ptr(off), ptr(w), n_out, n_in, f, nnz,
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


def gcn_norm_csc_csr(edge_index, edge_weight, num_nodes, improved=False, want_csr=True, sorted=False):
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
    check(lib().jg_gcn_norm_compressed(ptr(ei), ptr(w), E0, n, 2.0 if improved else 1.0, 1 if sorted else 0,
                                       ptr(csc[0]), ptr(csc[1]), ptr(csc[2]), ptr(csr[0]), ptr(csr[1]), ptr(csr[2]),
                                       ptr(count), ptr(ws), ws.numel(), stream_for(ei)), "jg_gcn_norm_compressed")
    E = int(count.item())  # one synchronisation per graph: the entry count sizes the views
    out_csc = CSC(csc[0][:E], csc[1], csc[2][:E])
    out_csr = CSR(csr[0][:E], csr[1], csr[2][:E]) if want_csr else None
    return out_csc, out_csr
