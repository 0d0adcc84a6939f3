"""Partition file -> per-rank chunks, and their on-disk format.

Mirrors the reference's offline partitioner (partition/distchunk_manager.py:47-189,
examples/dist_gcn/dist_partition.py:122-158, data/distchunk.py:7-108): nodes are renumbered so that
every part is a contiguous id range, every rank gets the edges whose DESTINATION it owns as CSR, CSC
and one sub-CSR per source rank, plus its rows of the features, labels and masks.  The reference
does this with numpy, scipy and Python loops over every node and edge and pickles each chunk; here
the renumbering and the conversions run on the GPU through the library's radix sort, and a chunk is
saved as a directory of ``.npy`` files plus a small ``meta.json`` that can be memory-mapped back.
"""
import json
import os

import numpy as np
import torch

from . import ops
from ._lib import check, lib, ptr, stream_for
from .data import CSC, CSR

__all__ = ["DistChunk", "load_partition", "partition_to_chunks", "chunks_save", "distributed_file"]

FORMAT_VERSION = 1


def load_partition(path):
    """Part id of every node from a ``.npy`` file or from the text file METIS-style tools write (one
    part id per line, node i on line i) -> ``int32`` numpy array.  The reference stores the same
    vector pickled (partition/distchunk_manager.py:40-44); pickles are not read here."""
    if str(path).endswith(".npy"):
        part = np.load(path)
    else:
        part = np.loadtxt(path, dtype=np.int64, ndmin=1)
    if part.ndim != 1 or (part.size and part.min() < 0):
        raise ValueError("partition: expected one non-negative part id per node")
    return part.astype(np.int32)


def distributed_file(rank, nparts, file_dir=None):
    """Path of rank ``rank``'s chunk (data/distchunk.py:103-108; same name, here a directory)."""
    return None if file_dir is None else os.path.join(file_dir, f"subgraph_{nparts}_of_{rank}")


class DistChunk:
    """One rank's share of a partitioned graph (data/distchunk.py:7-66), fields named as there.

    ``edge_index`` is ``[2, E]`` with renumbered global source ids and LOCAL destination ids, sorted
    by (source, destination); ``offset`` holds the ``chunks + 1`` part boundaries; ``CSR`` has one
    row per global source and local destinations as columns, ``CSC`` one column per local destination
    and global sources as rows; ``chunk_CSR[q]`` is the part of ``CSR`` whose rows rank ``q`` owns.
    """

    ARRAYS = ("edge_index", "edge_weight", "offset", "local_feature", "local_label", "local_train_mask", "local_val_mask",
              "local_test_mask", "csr_column_indices", "csr_row_offset", "csr_edge_weight", "csc_row_indices",
              "csc_column_offset", "csc_edge_weight")

    def __init__(self, chunks, chunk_id, v_num, global_v_num, edge_index, offset, edge_weight=None, local_train_mask=None,
                 local_val_mask=None, local_test_mask=None, local_feature=None, local_label=None, num_classes=None):
        self.chunks, self.chunk_id, self.v_num, self.global_v_num = int(chunks), int(chunk_id), int(v_num), int(global_v_num)
        self.edge_index, self.edge_weight, self.offset = edge_index, edge_weight, offset
        self.local_masks = {"train": local_train_mask, "val": local_val_mask, "test": local_test_mask}
        self.local_feature, self.local_label, self.num_classes = local_feature, local_label, num_classes
        self.CSR = self.CSC = None
        self.chunk_CSR = []

    def set_csr(self, column_indices, row_offset, edge_weight=None):
        self.CSR = CSR(column_indices, row_offset, edge_weight)

    def set_csc(self, row_indices, column_offset, edge_weight=None):
        self.CSC = CSC(row_indices, column_offset, edge_weight)

    def set_chunk_csrs(self):
        """``chunk_CSR[q]``: the rows of ``CSR`` that rank ``q`` owns, offsets rebased
        (examples/dist_gcn/dist_partition.py:122-158; there a Python loop over every node and edge,
        here slices, because the renumbering made every rank's rows contiguous)."""
        bounds = [int(b) for b in self.offset.tolist()]
        ro, ci, w = self.CSR.row_offset, self.CSR.column_indices, self.CSR.edge_weight
        starts = ro[torch.as_tensor(bounds, device=ro.device, dtype=torch.long)].tolist()
        self.chunk_CSR = []
        for q in range(self.chunks):
            s, e = starts[q], starts[q + 1]
            self.chunk_CSR.append(CSR(ci[s:e], (ro[bounds[q]: bounds[q + 1] + 1] - s), None if w is None else w[s:e]))
        return self.chunk_CSR

    # ---- row partition and the optimised exchange path
    def row_partition(self):
        from .dist import RowPartition
        return RowPartition(self.global_v_num, self.chunks, bounds=self.offset.tolist())

    def sharded_graph(self, **kwargs):
        """The compact-halo aggregation of this rank (``dist.ShardedGraph``) over the chunk's CSC;
        collective, like the constructor it calls."""
        from .dist import ShardedGraph
        w = self.CSC.edge_weight
        if w is None:
            w = torch.ones(self.CSC.row_indices.numel(), dtype=torch.float32, device=self.CSC.row_indices.device)
        return ShardedGraph(self.row_partition(), self.chunk_id, self.CSC.row_indices, self.CSC.column_offset, w, **kwargs)

    # ---- on-disk format: a directory with meta.json and one .npy per array
    def _arrays(self):
        out = {"edge_index": self.edge_index, "edge_weight": self.edge_weight, "offset": self.offset,
               "local_feature": self.local_feature, "local_label": self.local_label,
               "local_train_mask": self.local_masks["train"], "local_val_mask": self.local_masks["val"],
               "local_test_mask": self.local_masks["test"]}
        if self.CSR is not None:
            out.update(csr_column_indices=self.CSR.column_indices, csr_row_offset=self.CSR.row_offset,
                       csr_edge_weight=self.CSR.edge_weight)
        if self.CSC is not None:
            out.update(csc_row_indices=self.CSC.row_indices, csc_column_offset=self.CSC.column_offset,
                       csc_edge_weight=self.CSC.edge_weight)
        return {k: v for k, v in out.items() if v is not None}

    def save(self, file_path):
        """Writes the chunk under directory ``file_path`` (data/distchunk.py:86-92 pickles the object
        instead).  ``chunk_CSR`` is not stored: it is a set of slices of ``CSR``, rebuilt on load."""
        os.makedirs(file_path, exist_ok=True)
        names = []
        for name, t in self._arrays().items():
            a = t.detach().cpu().numpy() if isinstance(t, torch.Tensor) else np.asarray(t)
            np.save(os.path.join(file_path, name + ".npy"), np.ascontiguousarray(a))
            names.append(name)
        meta = {"format": FORMAT_VERSION, "chunks": self.chunks, "chunk_id": self.chunk_id, "v_num": self.v_num,
                "global_v_num": self.global_v_num, "num_classes": self.num_classes, "arrays": names}
        tmp = os.path.join(file_path, "meta.json.tmp")
        with open(tmp, "w") as f:
            json.dump(meta, f)
        os.replace(tmp, os.path.join(file_path, "meta.json"))       # written last: a chunk without it is incomplete

    @staticmethod
    def load(file_path, device=None, mmap=True):
        """Reads a chunk written by :meth:`save`.  With ``mmap`` the arrays are memory-mapped (pages
        are read when touched, or streamed to ``device`` when one is given)."""
        with open(os.path.join(file_path, "meta.json")) as f:
            meta = json.load(f)
        if meta.get("format") != FORMAT_VERSION:
            raise RuntimeError(f"{file_path}: unknown chunk format {meta.get('format')!r}")
        got = {}
        for name in meta["arrays"]:
            if name not in DistChunk.ARRAYS:
                raise RuntimeError(f"{file_path}: unexpected array {name!r}")
            a = np.load(os.path.join(file_path, name + ".npy"), mmap_mode="r" if mmap else None, allow_pickle=False)
            t = _from_memmap(a) if mmap else torch.from_numpy(a)
            got[name] = t.to(device) if device is not None else t
        c = DistChunk(meta["chunks"], meta["chunk_id"], meta["v_num"], meta["global_v_num"], got.get("edge_index"),
                      got.get("offset"), got.get("edge_weight"), got.get("local_train_mask"), got.get("local_val_mask"),
                      got.get("local_test_mask"), got.get("local_feature"), got.get("local_label"), meta.get("num_classes"))
        if "csr_row_offset" in got:
            c.set_csr(got["csr_column_indices"], got["csr_row_offset"], got.get("csr_edge_weight"))
            c.set_chunk_csrs()
        if "csc_column_offset" in got:
            c.set_csc(got["csc_row_indices"], got["csc_column_offset"], got.get("csc_edge_weight"))
        return c


def _from_memmap(a):
    import warnings
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")           # torch warns that the mapped array is read-only
        return torch.from_numpy(a)


def chunks_save(chunks, output_dir):
    """Every chunk to ``output_dir/subgraph_{P}_of_{rank}`` (partition/distchunk_manager.py:185-189)."""
    for c in chunks:
        c.save(distributed_file(c.chunk_id, c.chunks, output_dir))


def _expand(off, total):
    out = torch.empty(total, dtype=torch.int32, device=off.device)
    if total == 0:
        return out
    check(lib().jg_expand_columns(ptr(off), off.numel() - 1, None, ptr(out), stream_for(off)), "jg_expand_columns")
    return out


def partition_to_chunks(partition, edge_index, num_nodes, num_parts, edge_weight=None, global_feature=None,
                        global_masks=None, global_label=None, num_classes=None):
    """Chunks of a partitioned graph (partition/distchunk_manager.py:47-157), built on device.

    ``partition[i]`` is the part of node ``i``.  Nodes are renumbered part after part; inside a part
    they keep their original order (the reference's ``np.argsort`` leaves that order unspecified).
    Rank ``p`` receives the edges whose destination it owns.  Entries of a CSR row / CSC column are
    ordered by index as scipy orders them; duplicate edges are kept as separate entries, where scipy
    would add their weights.  All inputs and results are CUDA tensors.
    """
    n, P = int(num_nodes), int(num_parts)
    part = ops._as_i32(torch.as_tensor(partition), "partition")
    dev = edge_index.device
    part = part.to(dev)
    if part.numel() != n:
        raise RuntimeError(f"partition has {part.numel()} entries, the graph {n} nodes")
    if n and int(part.max()) >= P:
        raise RuntimeError("partition: part id beyond num_parts")
    # stable sort of the node ids by part: rows of a CSR keyed by part id
    by_part = ops.cootocsr(torch.stack([part, torch.arange(n, dtype=torch.int32, device=dev)]), None, P)
    order, offset = by_part.column_indices, by_part.row_offset            # new id -> old id, part boundaries
    remap = torch.empty(n, dtype=torch.int32, device=dev)
    remap[order.long()] = torch.arange(n, dtype=torch.int32, device=dev)  # old id -> new id
    ei = ops._edge_index(edge_index)
    ei = torch.stack([remap[ei[0].long()], remap[ei[1].long()]])
    w = None if edge_weight is None else ops._as_f32(edge_weight, "edge_weight")
    # one canonical CSC of the renumbered graph; a rank's chunk is a range of its columns
    g_csc = ops.cootocsc(ei, w, n, sorted=True)
    bounds = offset.tolist()
    col_starts = g_csc.column_offset[offset.long()].tolist()
    masks = list(global_masks) if global_masks is not None else []
    masks += [None] * (3 - len(masks))
    take = lambda t, s, e: None if t is None else t.to(dev)[order[s:e].long()]
    chunks = []
    for p in range(P):
        s, e = bounds[p], bounds[p + 1]
        cs, ce = col_starts[p], col_starts[p + 1]
        rows = g_csc.row_indices[cs:ce].contiguous()
        col_off = (g_csc.column_offset[s: e + 1] - cs).contiguous()
        cw = None if w is None else g_csc.edge_weight[cs:ce].contiguous()
        local_dst = _expand(col_off, ce - cs)
        csr = ops.cootocsr(torch.stack([rows, local_dst]), cw, n, sorted=True)    # rows: all global sources
        src_sorted = _expand(csr.row_offset, ce - cs)
        chunk = DistChunk(P, p, e - s, n, torch.stack([src_sorted, csr.column_indices]), offset,
                          None if w is None else csr.edge_weight, take(masks[0], s, e), take(masks[1], s, e),
                          take(masks[2], s, e), take(global_feature, s, e), take(global_label, s, e), num_classes)
        chunk.set_csr(csr.column_indices, csr.row_offset, None if w is None else csr.edge_weight)
        chunk.set_csc(rows, col_off, cw)
        chunk.set_chunk_csrs()
        chunks.append(chunk)
    return chunks
