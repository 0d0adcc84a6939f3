"""Generates the committed golden vectors (``tests/golden/*.npz``).

Inputs are the hand-written graphs of the reference's own smoke scripts
(jittor_geometric/tests/test_*.py, which print but never assert) plus one seeded
citation-graph-shaped instance; outputs come from the reference's OWN CPU
operator bodies compiled by ``oracle/Makefile`` (``impl="ref"``), so this script
needs a reference checkout at build time.  Run from the repository root:

    python tests/golden/make_golden.py
"""
import hashlib
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle as O  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))
I = "ref"


def save(name, **arrays):
    np.savez_compressed(os.path.join(OUT, name + ".npz"), **arrays)
    print(name, {k: v.shape for k, v in arrays.items()})


def main():
    O.build()
    assert O.have_ref(), "reference CPU library missing: golden vectors need it"

    # tests/test_csr.py:16-18
    ei = np.array([[0, 0, 1, 1, 2], [1, 2, 2, 3, 3]], np.int32)
    w = np.array([1, 2, 3, 4, 5], np.float32)
    ci, ro, cw = O.coo_to_csr(ei, w, 4, I)
    ri, co, sw = O.coo_to_csc(ei, w, 4, I)
    save("ref_test_csr", edge_index=ei, edge_weight=w, n=np.int64(4), column_indices=ci, row_offset=ro,
         csr_weight=cw, row_indices=ri, column_offset=co, csc_weight=sw)

    # tests/test_mp_spmm.py:14-27
    x = np.array([[3, 2, 1, 0, 5, 0, 1, 0, 2, 0], [1, 0, 2, 3, 0, 4, 0, 5, 1, 0],
                  [0, 6, 0, 0, 7, 0, 8, 0, 9, 0], [4, 0, 0, 1, 0, 5, 0, 0, 0, 6],
                  [0, 0, 3, 0, 4, 0, 2, 1, 0, 0], [7, 0, 2, 0, 3, 0, 4, 5, 0, 6],
                  [1, 3, 0, 2, 0, 0, 4, 5, 6, 0], [0, 8, 0, 0, 7, 1, 0, 9, 2, 0],
                  [9, 0, 6, 0, 0, 2, 0, 0, 1, 3], [0, 1, 0, 4, 0, 0, 6, 0, 5, 7]], np.float32)
    ei = np.array([[0, 0, 1, 1, 2, 2, 3, 4, 4, 5, 5, 7, 8], [1, 2, 2, 3, 3, 4, 5, 8, 9, 5, 8, 9, 9]], np.int32)
    w = np.array([1, 2, 3, 4, 5, 3, 5, 1, 2, 3, 2, 3, 2], np.float32)
    ci, ro, cw = O.coo_to_csr(ei, w, 10, I)
    ri, co, sw = O.coo_to_csc(ei, w, 10, I)
    y = O.aggregate(x, ri, co, sw, impl=I)         # forward (CSC) == SpmmCsr(x, csr) == SpmmCoo
    gy = O.aggregate(x, ci, ro, cw, impl=I)        # backward kernel (CSR) on the same matrix
    save("ref_test_mp_spmm", x=x, edge_index=ei, edge_weight=w, n=np.int64(10), column_indices=ci,
         row_offset=ro, csr_weight=cw, row_indices=ri, column_offset=co, csc_weight=sw, out_csc=y, out_csr=gy)

    # tests/test_aggregate.py:43-54 (its offsets describe 3 vertices; the first three rows of x
    # are used, and the weight literals are the five the script spells out)
    x = np.array([[3, 2, 1], [3, 2, 1], [3, 2, 1]], np.float32)
    ri, co = np.array([0, 0, 1, 2], np.int32), np.array([0, 1, 3, 4], np.int32)
    sw = np.array([1.0, 2.0, 3, 0, 4.0], np.float32)[:4]
    ci, ro = np.array([0, 1, 1, 2], np.int32), np.array([0, 2, 3, 4], np.int32)
    cw = np.array([3.0, 1.0, 4, 0, 2.0], np.float32)[:4]
    save("ref_test_aggregate", x=x, row_indices=ri, column_offset=co, csc_weight=sw, column_indices=ci,
         row_offset=ro, csr_weight=cw, out_fwd=O.aggregate(x, ri, co, sw, impl=I),
         out_bwd=O.aggregate(x, ci, ro, cw, impl=I))

    # tests/test_edgesoftmax.py:19-25, plus a gradient vector for the backward op
    xs = np.array([1, 2, 3, 4], np.float32)
    ys = O.edge_softmax(xs, co, I)
    g = np.array([0.5, -1.0, 2.0, 0.25], np.float32)
    save("ref_test_edgesoftmax", x=xs, row_indices=ri, column_offset=co, out=ys, grad=g,
         grad_in=O.edge_softmax_backward(g, ys, co, I))

    # tests/test_scatter_to_edge.py:14-20 and tests/test_edgetovertex.py:20-26
    xv = np.array([[1, 1, 1], [2, 2, 2], [3, 3, 3]], np.float32)
    xe = np.array([[1, 1, 1], [2, 2, 2], [3, 3, 3], [3, 2, 1]], np.float32)
    save("ref_test_scatter", x_vertex=xv, x_edge=xe, row_indices=ri, column_offset=co,
         to_edge_src=O.scatter_to_edge(xv, ri, co, 0, I), to_edge_dst=O.scatter_to_edge(xv, ri, co, 1, I),
         to_vertex_dst=O.edge_to_vertex(xe, ri, co, 1, I), to_vertex_src=O.edge_to_vertex(xe, ri, co, 0, I))

    # tests/test_undirected.py:12-16
    ei = np.array([[0, 1, 1], [2, 0, 2]], np.int32)
    ea = np.array([1, 3, 2], np.float32)
    nei, nea = O.to_undirected(ei, ea, 3, I)
    save("ref_test_undirected", edge_index=ei, edge_attr=ea, new_edge_index=nei, new_edge_attr=nea)

    # tests/test_spmmcsr.py:13-17 (int64 indices there) and tests/test_spmmcoo.py:15-17.  Both go
    # through cuSPARSE in the reference with trans_A=True, i.e. out[dst] += w * x[src]; the CPU
    # aggregate over the transposed structure is the stated equivalent (tests/test_mp_spmm.py:28-36).
    x3 = np.array([[3, 2, 1], [3, 2, 1], [3, 2, 1]], np.float32)
    ci, ro = np.array([0, 1, 1, 2], np.int64), np.array([0, 2, 3, 4], np.int64)
    cw = np.array([3, 1, 4, 2], np.float32)
    src = np.repeat(np.arange(3), np.diff(ro)).astype(np.int32)
    tri, tco, tw = O.coo_to_csc(np.stack([src, ci.astype(np.int32)]), cw, 3, I)
    x4 = np.array([[3, 2, 1], [4, 2, 2], [1, 2, 3]], np.float32)
    ei = np.array([[0, 0, 1, 2], [1, 2, 2, 1]], np.int32)
    ew = np.ones(4, np.float32)
    cri, cco, cw2 = O.coo_to_csc(ei, ew, 3, I)
    save("ref_test_spmm", csr_x=x3, column_indices=ci, row_offset=ro, csr_weight=cw,
         csr_out=O.aggregate(x3, tri, tco, tw, impl=I), coo_x=x4, edge_index=ei, edge_weight=ew,
         coo_out=O.aggregate(x4, cri, cco, cw2, impl=I))

    # Seeded citation-graph-shaped instance: 2708 nodes, 5278 undirected edges, gcn_norm weights.
    import torch  # noqa: F401  (generator lives in the package)
    from jittorgeometric_b200 import synth
    ei = synth.preferential_attachment(2708, 5278, seed=20261125).numpy()
    nei, nw = O.gcn_norm(ei, None, 2708)
    ci, ro, cw = O.coo_to_csr(nei, nw, 2708, I)
    ri, co, sw = O.coo_to_csc(nei, nw, 2708, I)
    rng = np.random.default_rng(20261125)
    x7 = rng.standard_normal((2708, 7)).astype(np.float32)
    x256 = rng.standard_normal((2708, 256)).astype(np.float32)
    y7 = O.aggregate(x7, ri, co, sw, impl=I)
    y256 = O.aggregate(x256, ri, co, sw, impl=I)
    save("citation_2708", edge_index=ei, norm_edge_index=nei, norm_weight=nw, column_indices=ci, row_offset=ro,
         csr_weight=cw, row_indices=ri, column_offset=co, csc_weight=sw, x7=x7, y7=y7,
         x256_seed=np.int64(20261125), y256_rows=y256[::97].copy(),
         y256_sha256=np.frombuffer(hashlib.sha256(y256.tobytes()).digest(), np.uint8))


def sampling():
    """Golden vectors of the neighbour-sampling operators (compiled reference bodies)."""
    O.build()
    assert O.have_ref(), "reference CPU library missing: golden vectors need it"
    ids4 = np.arange(4, dtype=np.int32)
    # tests/test_csctocsr.py:25-35
    co, ri = np.array([0, 0, 1, 2, 4], np.int32), np.array([0, 0, 1, 2], np.int32)
    ro, ci = O.csc_to_csr(co, ri, ids4, ids4, I)
    # tests/test_getweight.py:25-33
    gco, gri = np.array([0, 1, 2, 3, 4], np.int32), np.array([0, 0, 1, 2], np.int32)
    gw = O.get_weight(4, ids4, ids4, gco, gri, I)
    # tests/test_sampleprocessing.py:34-40: every in-degree is at most the fanout (3), so the body copies
    # every list in stored order; layer offsets are the running sums of the degrees
    s_goff = np.array([0, 3, 6, 8, 10, 12, 14, 16, 17, 18, 19], np.int32)
    s_gidx = np.array([1, 2, 3, 2, 3, 4, 0, 5, 1, 6, 2, 7, 3, 8, 4, 9, 5, 6, 7], np.int32)
    s_dst = np.array([3, 0, 9, 5, 1], np.int32)
    s_off = np.concatenate([[0], np.cumsum(O.sample_counts(s_dst, s_goff, 3)[1:])]).astype(np.int32)
    s_out = O.sample_reference(3, s_dst, s_off, s_goff, s_gidx)
    # a seeded layer over explicit id lists: 300 destinations and 1500 listed sources out of 4000 ids
    rng = np.random.default_rng(20261125 + 7)
    l_off = np.concatenate([[0], np.cumsum(rng.integers(0, 12, size=300))]).astype(np.int32)
    l_idx = rng.integers(0, 4000, size=l_off[-1]).astype(np.int32)
    l_dst = rng.permutation(4000)[:300].astype(np.int32)
    l_src = rng.permutation(4000)[:1500].astype(np.int32)
    l_ro, l_ci = O.csc_to_csr(l_off, l_idx, l_dst, l_src, I)
    l_w = O.get_weight(4000, l_dst, l_src, l_off, l_idx, I)
    save("ref_test_sampling", csr_in_column_offset=co, csr_in_row_indices=ri, csr_row_offset=ro, csr_column_indices=ci,
         w_column_offset=gco, w_row_indices=gri, w_out=gw, counts_dst=ids4,
         counts_global_offset=np.array([0, 1, 3, 4, 5], np.int32), counts_out=np.array([0, 1, 2, 1, 1], np.int32),
         s_global_offset=s_goff, s_global_indices=s_gidx, s_dst=s_dst, s_layer_offset=s_off, s_out=s_out,
         l_column_offset=l_off, l_row_indices=l_idx, l_dst=l_dst, l_src=l_src, l_row_offset=l_ro,
         l_column_indices=l_ci, l_weight=l_w)


def partition():
    """Golden vectors of the offline partitioner: the reference's OWN ``DistChunkManager.partition_to_chunk``
    (partition/distchunk_manager.py:47-157) and ``set_chunks_csrs`` (examples/dist_gcn/dist_partition.py:122-158),
    loaded from the checkout and run on numpy inputs.  Their modules import Jittor and pymetis at the
    top, which are not installed; both are replaced by stand-ins that only hold attributes (the two
    functions themselves use numpy and scipy), so what runs is the reference's code unmodified."""
    import ast
    import importlib.util
    import pickle
    import tempfile
    import types
    ref_root = os.environ.get("JG_REFERENCE_ROOT", "/root/reference")

    class Holder:                       # stands in for DistChunk / CSR: keeps what it is given
        def __init__(self, *a, **kw):
            self.__dict__.update(kw)
            self.chunk_CSR = []

        def set_csr(self, column_indices, row_offset, edge_weight=None):
            self.CSR = Holder(column_indices=column_indices, row_offset=row_offset, edge_weight=edge_weight)

        def set_csc(self, row_indices, column_offset, edge_weight=None):
            self.CSC = Holder(row_indices=row_indices, column_offset=column_offset, edge_weight=edge_weight)

    jt = types.ModuleType("jittor")
    jt.Var = type("Var", (), {})
    jt.array = lambda a: np.asarray(a)
    jt.gc = lambda: None
    data_mod = types.ModuleType("jittor_geometric.data")
    data_mod.DistChunk, data_mod.CSR, data_mod.CSC = Holder, Holder, Holder
    pkg = types.ModuleType("jittor_geometric")
    pkg.data = data_mod
    metis = types.ModuleType("pymetis")
    metis.part_graph = None
    saved = {k: sys.modules.get(k) for k in ("jittor", "jittor_geometric", "jittor_geometric.data", "pymetis")}
    sys.modules.update({"jittor": jt, "jittor_geometric": pkg, "jittor_geometric.data": data_mod, "pymetis": metis})
    try:
        spec = importlib.util.spec_from_file_location(
            "ref_distchunk_manager", os.path.join(ref_root, "jittor_geometric", "partition", "distchunk_manager.py"))
        mgr_mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mgr_mod)
        # the two functions of the example script, without running the script itself
        src = open(os.path.join(ref_root, "examples", "dist_gcn", "dist_partition.py")).read()
        tree = ast.parse(src)
        keep = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name in ("compute_chunk_id", "set_chunks_csrs")]
        ns = {"np": np, "jt": jt, "tqdm": lambda it, **kw: it, "CSR": Holder}
        exec(compile(ast.Module(body=keep, type_ignores=[]), "dist_partition.py", "exec"), ns)
    finally:
        for k, v in saved.items():
            if v is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = v

    rng = np.random.default_rng(41)
    n, P, E = 60, 3, 400
    pairs = np.unique(rng.integers(0, n, size=(E, 2)), axis=0)          # distinct edges: scipy would add duplicates up
    edge_index = pairs.T.astype(np.int64)
    w = rng.random(edge_index.shape[1]).astype(np.float32)
    part = rng.integers(0, P, size=n).astype(np.int64)
    part[:P] = np.arange(P)
    feature = rng.standard_normal((n, 5)).astype(np.float32)
    label = np.arange(n)                                                # the local labels reveal the node order inside a part
    with tempfile.TemporaryDirectory() as tmp:
        pf = os.path.join(tmp, "partition.bin")
        with open(pf, "wb") as f:
            pickle.dump(part, f)
        chunks = mgr_mod.DistChunkManager().partition_to_chunk(pf, edge_index.copy(), n, P, edge_weight=w.copy(),
                                                               global_feature=feature, global_masks=[None, None, None],
                                                               global_label=label, num_classes=3)
    ns["set_chunks_csrs"](chunks, P)
    out = dict(edge_index=edge_index, edge_weight=w, partition=part, feature=feature, n=np.int64(n), parts=np.int64(P))
    for p, c in enumerate(chunks):
        out.update({f"p{p}_edge_index": np.asarray(c.edge_index), f"p{p}_edge_weight": np.asarray(c.edge_weight),
                    f"p{p}_offset": np.asarray(c.offset), f"p{p}_label": np.asarray(c.local_label),
                    f"p{p}_feature": np.asarray(c.local_feature),
                    f"p{p}_csr_indices": np.asarray(c.CSR.column_indices), f"p{p}_csr_indptr": np.asarray(c.CSR.row_offset),
                    f"p{p}_csr_data": np.asarray(c.CSR.edge_weight),
                    f"p{p}_csc_indices": np.asarray(c.CSC.row_indices), f"p{p}_csc_indptr": np.asarray(c.CSC.column_offset),
                    f"p{p}_csc_data": np.asarray(c.CSC.edge_weight)})
        for q, sub in enumerate(c.chunk_CSR):
            out.update({f"p{p}_chunk{q}_indices": np.asarray(sub.column_indices), f"p{p}_chunk{q}_indptr": np.asarray(sub.row_offset),
                        f"p{p}_chunk{q}_data": np.asarray(sub.edge_weight)})
    save("ref_partition", **out)


if __name__ == "__main__":
    if sys.argv[1:] == ["sampling"]:
        sampling()
    elif sys.argv[1:] == ["partition"]:
        partition()
    else:
        main()
        sampling()
