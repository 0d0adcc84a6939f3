"""Neighbour sampling for mini-batch training, on device.

Mirrors the four sampling operators of ``jittor_geometric.ops`` (ops/gpuinitco.py,
ops/sampleprocessing.py, ops/csctocsr.py, ops/getweight.py: same names, argument order and
results) and the layer-wise sampler built on them in the reference's mini-batch example
(examples/minibatch_example.py:119-400: ``SampledSubgraph``, ``LayerSampGraph``, ``sample_one``,
``NeighborLoader``).  Where the example loops over nodes in Python (the merged adjacency
dictionary, examples/minibatch_example.py:300-340) everything here stays on the GPU: distinct ids
and the global-to-local map come from a mark/scan/list pass, the merged CSC from the library's
stable radix sort.  There is no CPU path.
"""
import torch

from . import ops
from ._lib import check, lib, ptr, stream_for, workspace
from .data import CSC, CSR

__all__ = ["gpuinitco", "sampleprocessing", "csctocsr", "getweight", "from_nodes", "to_nodes", "layer_offsets", "LayerSampGraph", "SampledSubgraph",
           "sample_layers", "build_subgraph", "sample_one", "NeighborLoader"]

_i32 = ops._as_i32


def _counts(dst, g_off, fanout, cumulative):
    dst, g_off = _i32(dst, "csc_layer_dst"), _i32(g_off, "csc_global_column_offset")
    n = dst.numel()
    out = torch.empty(n + 1, dtype=torch.int32, device=dst.device)
    ws = workspace(lib().jg_sample_counts_workspace_bytes(n), dst.device)
    check(lib().jg_sample_counts(ptr(dst), n, ptr(g_off), int(fanout), 1 if cumulative else 0, ptr(out), ptr(ws), ws.numel(),
                                 stream_for(dst)), "jg_sample_counts")
    return out


def gpuinitco(dst_size, fanout_i, csc_layer_dst, csc_global_column_offset):
    """``out[0] = 0``, ``out[i+1] = min(in-degree of dst[i], fanout)`` (ops/gpuinitco.py:30-36): per
    destination COUNTS, exactly what the reference kernel writes.  :func:`layer_offsets` gives the
    running sums the sampler needs."""
    if int(dst_size) != csc_layer_dst.numel():
        raise RuntimeError(f"gpuinitco: dst_size {dst_size} but {csc_layer_dst.numel()} destinations")
    return _counts(csc_layer_dst, csc_global_column_offset, fanout_i, False)


def layer_offsets(fanout_i, csc_layer_dst, csc_global_column_offset):
    """Column offsets of a sampled layer: running sum of ``min(in-degree, fanout)``
    (examples/minibatch_example.py:253-262); ``fanout < 0`` keeps every neighbour."""
    return _counts(csc_layer_dst, csc_global_column_offset, fanout_i, True)


def sampleprocessing(fanout_i, csc_layer_dst, csc_layer_column_offset, csc_global_column_offset, csc_global_row_indices,
                     seed=0, total=None):
    """Source ids of the sampled in-edges of every destination, column after column
    (ops/sampleprocessing.py:28-35).  A destination with at most ``fanout_i`` in-edges keeps all of
    them in stored order; otherwise ``fanout_i`` are drawn from distinct positions of its list.  The
    draw is a pure function of ``(seed, destination id, fanout)``.  ``total`` (the last offset) saves
    the device read the reference also makes (``column_offset[-1].item()``)."""
    dst = _i32(csc_layer_dst, "csc_layer_dst")
    off = _i32(csc_layer_column_offset, "csc_layer_column_offset")
    g_off = _i32(csc_global_column_offset, "csc_global_column_offset")
    g_idx = _i32(csc_global_row_indices, "csc_global_row_indices")
    if off.numel() != dst.numel() + 1:
        raise RuntimeError("sampleprocessing: column_offset must have one more entry than dst")
    unchecked = total is not None
    total = int(off[-1].item()) if total is None else int(total)
    out = torch.empty(total, dtype=torch.int32, device=dst.device)
    flag = torch.empty(1, dtype=torch.int32, device=dst.device)
    check(lib().jg_sample_neighbors(ptr(dst), dst.numel(), ptr(off), ptr(g_off), ptr(g_idx), int(fanout_i), int(seed) & (2**64 - 1),
                                    ptr(out), total, ptr(flag), stream_for(dst)), "jg_sample_neighbors")
    if not unchecked and int(flag.item()):
        raise RuntimeError("sampleprocessing: column_offset does not match min(in-degree, fanout) of the destinations")
    return out


def csctocsr(column_offset, row_indices, dst, src):
    """CSC -> CSR over explicit id lists (ops/csctocsr.py:27-34): returns
    ``(row_offset, column_indices)``; row ``r`` belongs to ``src[r]``, column values are ``dst``
    ids, entries whose source is not in ``src`` are dropped, rows keep the CSC traversal order."""
    off, idx = _i32(column_offset, "column_offset"), _i32(row_indices, "row_indices")
    dst, src = _i32(dst, "dst"), _i32(src, "src")
    if off.numel() != dst.numel() + 1:
        raise RuntimeError("csctocsr: column_offset must have one more entry than dst")
    dev = off.device
    n_src, E = src.numel(), idx.numel()
    id_range = int(src.max().item()) + 1 if n_src else 0
    row_off = torch.empty(n_src + 1, dtype=torch.int32, device=dev)
    col_idx = torch.empty(max(E, 1), dtype=torch.int32, device=dev)
    kept = torch.zeros(1, dtype=torch.int64, device=dev)
    ws = workspace(lib().jg_csc_to_csr_workspace_bytes(n_src, E, id_range), dev)
    check(lib().jg_csc_to_csr(ptr(off), ptr(idx), dst.numel(), E, ptr(dst), ptr(src), n_src, id_range, ptr(row_off), ptr(col_idx),
                              ptr(kept), ptr(ws), ws.numel(), stream_for(off)), "jg_csc_to_csr")
    return row_off, col_idx[: int(kept.item())]


def _square_csr(column_offset, row_indices, n):
    """``csctocsr`` with ``dst = src = arange(n)`` and every id listed: nothing is dropped, so no
    device read is needed for the entry count."""
    off, idx = _i32(column_offset, "column_offset"), _i32(row_indices, "row_indices")
    dev, E = off.device, idx.numel()
    ids = torch.arange(n, dtype=torch.int32, device=dev)
    row_off = torch.empty(n + 1, dtype=torch.int32, device=dev)
    col_idx = torch.empty(max(E, 1), dtype=torch.int32, device=dev)
    kept = torch.zeros(1, dtype=torch.int64, device=dev)
    ws = workspace(lib().jg_csc_to_csr_workspace_bytes(n, E, n), dev)
    check(lib().jg_csc_to_csr(ptr(off), ptr(idx), n, E, ptr(ids), ptr(ids), n, n, ptr(row_off), ptr(col_idx), ptr(kept), ptr(ws),
                              ws.numel(), stream_for(off)), "jg_csc_to_csr")
    return row_off, col_idx[:E]


def getweight(vtx_size, csc_layer_dst, csc_layer_src, csc_layer_column_offset, csc_layer_row_indices):
    """``w = 1 / (sqrt(out-degree[src]) * sqrt(in-degree[dst]))`` per entry, degrees counted over the
    given structure (ops/getweight.py:29-37).  ``csc_layer_src`` is accepted and unused, as in the
    reference body."""
    dst = _i32(csc_layer_dst, "csc_layer_dst")
    off, idx = _i32(csc_layer_column_offset, "csc_layer_column_offset"), _i32(csc_layer_row_indices, "csc_layer_row_indices")
    E = idx.numel()
    w = torch.empty(E, dtype=torch.float32, device=off.device)
    ws = workspace(lib().jg_degree_weights_workspace_bytes(int(vtx_size)), off.device)
    check(lib().jg_degree_weights(int(vtx_size), ptr(dst), dst.numel(), ptr(off), ptr(idx), E, ptr(w), ptr(ws), ws.numel(),
                                  stream_for(off)), "jg_degree_weights")
    return w


def from_nodes(csc, nodes):
    """In-neighbours of every node of ``nodes``, list after list, duplicates kept
    (ops/saparse_ops.py:9-40; a Python loop over the nodes there, one full-copy sampling pass here)."""
    if csc is None:
        raise ValueError("CSC structure must be provided.")
    off = layer_offsets(-1, nodes, csc.column_offset)
    return sampleprocessing(-1, nodes, off, csc.column_offset, csc.row_indices)


def to_nodes(csr, nodes):
    """Out-neighbours of every node of ``nodes``, list after list (ops/saparse_ops.py:43-73)."""
    if csr is None:
        raise ValueError("CSR structure must be provided.")
    off = layer_offsets(-1, nodes, csr.row_offset)
    return sampleprocessing(-1, nodes, off, csr.row_offset, csr.column_indices)


def _expand(off, values, total):
    out = torch.empty(total, dtype=torch.int32, device=off.device)
    if total == 0:
        return out
    check(lib().jg_expand_columns(ptr(off), off.numel() - 1, ptr(values), ptr(out), stream_for(off)), "jg_expand_columns")
    return out


def _distinct(ids, n_global):
    """``(sorted distinct ids, position of every input id in that list)`` by mark / scan / list on
    device: what ``jt.unique`` plus the ``global2local`` table do in the reference
    (examples/minibatch_example.py:283-295)."""
    ids = _i32(ids, "ids")
    m, dev = ids.numel(), ids.device
    pos = torch.empty(n_global + 1, dtype=torch.int32, device=dev)
    listed = torch.empty(max(min(m, n_global), 1), dtype=torch.int32, device=dev)
    local = torch.empty(max(m, 1), dtype=torch.int32, device=dev)
    ws = workspace(lib().jg_halo_map_workspace_bytes(n_global), dev)
    # an empty "own" range: every id is listed
    check(lib().jg_halo_map_build(ptr(ids), m, n_global, 0, 0, 0, ptr(pos), ptr(listed), ptr(local), ptr(ws), ws.numel(),
                                  stream_for(ids)), "jg_halo_map_build")
    count = int(pos[n_global].item())
    return listed[:count], local[:m]


class LayerSampGraph:
    """One sampled layer (examples/minibatch_example.py:182-189): destinations, their column
    offsets, the sampled source ids and the distinct sources."""

    def __init__(self, dst=None, column_offset=None, row_indices=None, src=None):
        self.dst, self.column_offset, self.row_indices, self.src = dst, column_offset, row_indices, src


class SampledSubgraph:
    """The merged local graph of one mini-batch (examples/minibatch_example.py:119-178)."""

    def __init__(self):
        self.layers = 0
        self.fanout = []
        self.layer_graph = []
        self.X = None
        self.target_lab = None
        self.column_offset = self.row_indices = self.row_offset = self.column_indices = None
        self.csc_edge_weight = self.csr_edge_weight = None
        self.csc = self.csr = None
        self.local2global = None
        self.num_nodes = 0
        self.num_edges = 0

    def build_csc_csr(self):
        self.csc = CSC(self.row_indices, self.column_offset, self.csc_edge_weight)
        self.csr = CSR(self.column_indices, self.row_offset, self.csr_edge_weight)


def sample_layers(fanout, sample_nids, csc_global_column_offset, csc_global_row_indices, seed=0):
    """Layer-wise sampling (examples/minibatch_example.py:237-279): layer 0 samples the in-edges of
    the batch, layer i those of layer i-1's distinct sources.  The reference shuffles each layer's
    destinations; here they stay sorted (the order only fixes the column order of intermediate
    layers, which the merged graph does not keep)."""
    g_off = _i32(csc_global_column_offset, "csc_global_column_offset")
    g_idx = _i32(csc_global_row_indices, "csc_global_row_indices")
    n_global = g_off.numel() - 1
    layers = []
    dst = _i32(sample_nids, "sample_nids")
    for i, f in enumerate(fanout):
        off = layer_offsets(f, dst, g_off)
        total = int(off[-1].item())
        idx = sampleprocessing(f, dst, off, g_off, g_idx, seed=(int(seed) << 8) + i, total=total)
        src, _ = _distinct(idx, n_global)
        layers.append(LayerSampGraph(dst, off, idx, src))
        dst = src
    return layers


def build_subgraph(layers, n_global):
    """Merges sampled layers into one local graph (examples/minibatch_example.py:281-358): local ids
    are positions in the sorted list of all touched nodes; column ``v`` of the merged CSC holds the
    entries of ``v`` from layer 0, then layer 1, ... in their sampled order; the CSR keeps the CSC
    traversal order inside its rows; weights are ``getweight`` of the merged graph."""
    ssg = SampledSubgraph()
    ssg.layer_graph = list(layers)
    ssg.layers = len(layers)
    pieces = []
    for lay in layers:
        pieces += [lay.dst, lay.row_indices]
    sizes = [p.numel() for p in pieces]
    local2global, local = _distinct(torch.cat(pieces), n_global)
    parts = list(torch.split(local, sizes))
    n = local2global.numel()
    srcs, dsts = [], []
    for k, lay in enumerate(layers):
        dst_local, src_local = parts[2 * k].contiguous(), parts[2 * k + 1]
        srcs.append(src_local)
        dsts.append(_expand(lay.column_offset, dst_local, lay.row_indices.numel()))
    ei = torch.stack([torch.cat(srcs), torch.cat(dsts)])
    csc = ops.cootocsc(ei, None, n)                      # stable: layer order, then sampled order
    ssg.local2global, ssg.num_nodes, ssg.num_edges = local2global, n, ei.shape[1]
    ssg.column_offset, ssg.row_indices = csc.column_offset, csc.row_indices
    ssg.row_offset, ssg.column_indices = _square_csr(ssg.column_offset, ssg.row_indices, n)
    ids = torch.arange(n, dtype=torch.int32, device=ei.device)
    ssg.csc_edge_weight = getweight(n, ids, ids, ssg.column_offset, ssg.row_indices)
    ssg.csr_edge_weight = getweight(n, ids, ids, ssg.row_offset, ssg.column_indices)
    ssg.build_csc_csr()
    return ssg


def _gather_rows(x, rows):
    x = ops._as_f32(x, "feature")
    out = torch.empty((rows.numel(), x.shape[1]), dtype=torch.float32, device=x.device)
    check(lib().jg_gather_rows_f32(ptr(out), ptr(x), ptr(rows), rows.numel(), x.shape[1], 0, stream_for(x)), "jg_gather_rows_f32")
    return out


def sample_one(fanout, csc_global_column_offset, csc_global_row_indices, sample_nids, global_feature=None, global_target=None,
               seed=0):
    """One mini-batch (examples/minibatch_example.py:232-362): sampled layers, merged local CSC/CSR
    with ``getweight`` weights, and the feature / label rows of the touched nodes."""
    layers = sample_layers(fanout, sample_nids, csc_global_column_offset, csc_global_row_indices, seed)
    ssg = build_subgraph(layers, csc_global_column_offset.numel() - 1)
    ssg.fanout = list(fanout)
    if global_feature is not None:
        ssg.X = _gather_rows(global_feature, ssg.local2global)
    if global_target is not None:
        ssg.target_lab = global_target[ssg.local2global.long()]
    return ssg


class NeighborLoader:
    """Batches of seed nodes, each turned into a :class:`SampledSubgraph`
    (examples/minibatch_example.py:365-400).  ``reset()`` reshuffles the seeds with a generator
    seeded from ``seed`` and the epoch count, so a run can be repeated exactly."""

    def __init__(self, nids, fanout, batch_size, csc_col_off, csc_row_idx, global_feature=None, global_target=None, seed=0):
        self.nids = _i32(nids, "nids")
        self.fanout, self.batch_size = list(fanout), int(batch_size)
        self.csc_col_off, self.csc_row_idx = csc_col_off, csc_row_idx
        self.global_feature, self.global_target = global_feature, global_target
        self.seed, self.epoch = int(seed), 0
        self.batch_ids = []

    def reset(self):
        gen = torch.Generator(device=self.nids.device).manual_seed(self.seed * 1000003 + self.epoch)
        self.epoch += 1
        shuffled = self.nids[torch.randperm(self.nids.numel(), generator=gen, device=self.nids.device)]
        self.batch_ids = [shuffled[i: i + self.batch_size] for i in range(0, shuffled.numel(), self.batch_size)]

    def __len__(self):
        return len(self.batch_ids)

    def __iter__(self):
        for k, batch in enumerate(self.batch_ids):
            yield sample_one(self.fanout, self.csc_col_off, self.csc_row_idx, batch.contiguous(), self.global_feature,
                             self.global_target, seed=(self.seed * 7919 + self.epoch) * 100003 + k)
