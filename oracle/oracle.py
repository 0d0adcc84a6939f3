"""TEST INFRASTRUCTURE ONLY: numpy/ctypes front end of the CPU checkers.

Every function takes and returns numpy arrays (int32 indices, fp32 values).
``impl="port"`` runs this repository's C restatement, ``impl="ref"`` runs the
reference's own compiled CPU body.  Pure-Python pieces of the reference
(``gcn_norm``, layer compositions) are restated in numpy here, each citing the
reference file it follows.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_PORT_SO = os.path.join(_HERE, "libjgoracle.so")
_REF_SO = os.path.join(_HERE, "_ref", "libjgref.so")

_port = None
_ref = None

c_i32p = ctypes.POINTER(ctypes.c_int32)
c_f32p = ctypes.POINTER(ctypes.c_float)


def build(quiet=True):
    """Compile the checkers (``make -C oracle``).  The reference library is only
    rebuilt where a reference checkout exists; elsewhere a prebuilt one is kept."""
    env = dict(os.environ)
    if "JG_REFERENCE_ROOT" in env:
        env["REF"] = env["JG_REFERENCE_ROOT"]
    r = subprocess.run(["make", "-C", _HERE], capture_output=True, text=True, env=env)
    if r.returncode != 0:
        raise RuntimeError("oracle build failed:\n" + r.stdout + r.stderr)
    if not quiet:
        print(r.stdout)


def _ip(a):
    return a.ctypes.data_as(c_i32p)


def _fp(a):
    return a.ctypes.data_as(c_f32p) if a is not None else None


def port_lib():
    global _port
    if _port is None:
        if not os.path.exists(_PORT_SO):
            build()
        _port = ctypes.CDLL(_PORT_SO)
        _port.orc_gcn_norm.restype = ctypes.c_int64
        _port.orc_to_undirected.restype = ctypes.c_int64
    return _port


def have_ref():
    return os.path.exists(_REF_SO)


def ref_lib():
    global _ref
    if _ref is None:
        if not have_ref():
            raise RuntimeError("reference CPU library not built (oracle/_ref/libjgref.so)")
        _ref = ctypes.CDLL(_REF_SO)
        _ref.ref_toundirected.restype = ctypes.c_long
    return _ref


def _i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


L = ctypes.c_int64


# --------------------------------------------------------------------- conversion
def _compress(edge_index, w, n, by, impl):
    ei = _i32(edge_index)
    assert ei.ndim == 2 and ei.shape[0] == 2
    E = ei.shape[1]
    w = _f32(w)
    off = np.zeros(n + 1, np.int32)
    idx = np.zeros(E, np.int32)
    ow = np.zeros(E, np.float32)
    if impl == "ref":
        fn = ref_lib().ref_cootocsr if by == 0 else ref_lib().ref_cootocsc
        fn(_ip(ei), _fp(w), ctypes.c_long(E), ctypes.c_int(n), _ip(idx), _ip(off), _fp(ow))
    else:
        key, other = (ei[0], ei[1]) if by == 0 else (ei[1], ei[0])
        key, other = _i32(key), _i32(other)
        port_lib().orc_coo_compress(_ip(key), _ip(other), _fp(w), L(E), ctypes.c_int32(n),
                                    _ip(off), _ip(idx), _fp(ow))
    return idx, off, ow


def coo_to_csr(edge_index, w, n, impl="port"):
    """-> (column_indices, row_offset, edge_weight); rows keyed by source."""
    return _compress(edge_index, w, n, 0, impl)


def coo_to_csc(edge_index, w, n, impl="port"):
    """-> (row_indices, column_offset, edge_weight); columns keyed by destination."""
    return _compress(edge_index, w, n, 1, impl)


def sort_within_rows(idx, off, w):
    """Canonical form: entries of every segment ordered by index (stable)."""
    idx2, w2 = idx.copy(), w.copy()
    n = len(off) - 1
    seg = np.repeat(np.arange(n, dtype=np.int64), np.diff(off).astype(np.int64))
    order = np.lexsort((idx.astype(np.int64), seg))
    return idx2[order], w2[order], order


# --------------------------------------------------------------------- aggregation
def aggregate(x, idx, off, w, n_out=None, impl="port"):
    """out[v,:] = sum_{j in seg(v)} w[j] * x[idx[j],:] in the reference's fp32 order."""
    x, idx, off, w = _f32(x), _i32(idx), _i32(off), _f32(w)
    n_out = len(off) - 1 if n_out is None else n_out
    f = x.shape[1]
    out = np.zeros((n_out, f), np.float32)
    if impl == "ref":
        # the reference body takes its row count from x, so x must have n_out rows
        assert x.shape[0] == n_out, "reference aggregate is square only"
        ref_lib().ref_aggregate(_fp(out), _fp(x), _ip(idx), _ip(off), _fp(w), ctypes.c_long(n_out),
                                ctypes.c_long(f), ctypes.c_long(len(idx)))
    else:
        port_lib().orc_aggregate(_fp(out), _fp(x), _ip(idx), _ip(off), _fp(w), L(n_out), L(f))
    return out


def aggregate_f64(x, idx, off, w, n_out=None):
    """float64 truth and the per-element sum of |w*x| used as the error scale."""
    import scipy.sparse as sp
    n_out = len(off) - 1 if n_out is None else n_out
    A = sp.csr_matrix((w.astype(np.float64), idx.astype(np.int64), off.astype(np.int64)),
                      shape=(n_out, x.shape[0]))
    Aabs = sp.csr_matrix((np.abs(w).astype(np.float64), idx.astype(np.int64), off.astype(np.int64)),
                         shape=(n_out, x.shape[0]))
    x64 = x.astype(np.float64)
    return A @ x64, Aabs @ np.abs(x64)


# --------------------------------------------------------------------- edge ops
def edge_softmax(x, off, impl="port"):
    x, off = _f32(x), _i32(off)
    n = len(off) - 1
    out = np.zeros_like(x)
    if impl == "ref":
        assert x.ndim == 1 or x.shape[1] == 1, "reference softmax is one scalar per edge"
        idx = np.zeros(x.shape[0], np.int32)
        ref_lib().ref_edgesoftmax(_fp(out), _fp(x), _ip(idx), _ip(off), ctypes.c_long(n),
                                  ctypes.c_long(x.shape[0]))
    else:
        H = 1 if x.ndim == 1 else x.shape[1]
        port_lib().orc_edge_softmax(_fp(out), _fp(x), _ip(off), L(n), L(H))
    return out


def edge_softmax_backward(grad, y, off, impl="port"):
    grad, y, off = _f32(grad), _f32(y), _i32(off)
    n = len(off) - 1
    out = np.zeros_like(grad)
    if impl == "ref":
        idx = np.zeros(grad.shape[0], np.int32)
        ref_lib().ref_edgesoftmax_backward(_fp(out), _fp(grad), _fp(y), _ip(idx), _ip(off),
                                           ctypes.c_long(n), ctypes.c_long(grad.shape[0]))
    else:
        H = 1 if grad.ndim == 1 else grad.shape[1]
        port_lib().orc_edge_softmax_backward(_fp(out), _fp(grad), _fp(y), _ip(off), L(n), L(H))
    return out


def scatter_to_edge(x, idx, off, flag, impl="port"):
    x, idx, off = _f32(x), _i32(idx), _i32(off)
    n, f, E = len(off) - 1, x.shape[1], len(idx)
    out = np.zeros((E, f), np.float32)
    if impl == "ref":
        ref_lib().ref_scattertoedge(_fp(out), _fp(x), _ip(idx), _ip(off), ctypes.c_long(n),
                                    ctypes.c_long(f), ctypes.c_long(E), ctypes.c_int(flag))
    else:
        port_lib().orc_scatter_to_edge(_fp(out), _fp(x), _ip(idx), _ip(off), L(n), L(f),
                                       ctypes.c_int(flag))
    return out


def edge_to_vertex(msg, idx, off, flag, impl="port"):
    msg, idx, off = _f32(msg), _i32(idx), _i32(off)
    n, f, E = len(off) - 1, msg.shape[1], len(idx)
    out = np.zeros((n, f), np.float32)
    if impl == "ref":
        ref_lib().ref_edgetovertex(_fp(out), _fp(msg), _ip(idx), _ip(off), ctypes.c_long(n),
                                   ctypes.c_long(f), ctypes.c_long(E), ctypes.c_int(flag))
    else:
        port_lib().orc_edge_to_vertex(_fp(out), _fp(msg), _ip(idx), _ip(off), L(n), L(f),
                                      ctypes.c_int(flag))
    return out


def to_undirected(edge_index, attr, n, impl="port"):
    ei, attr = _i32(edge_index), _f32(attr)
    E = ei.shape[1]
    if impl == "ref":
        nei = np.zeros((2, 2 * E), np.int32)
        na = np.zeros(2 * E, np.float32)
        m = ref_lib().ref_toundirected(_ip(ei), _fp(attr), ctypes.c_long(E), ctypes.c_int(n), _ip(nei),
                                       _fp(na))
        # the body writes [2, m] row-major into the front of the buffer
        flat = nei.reshape(-1)
        return np.stack([flat[:m], flat[m:2 * m]]).copy(), na[:m].copy()
    s, d = _i32(ei[0]), _i32(ei[1])
    os_, od, oa = np.zeros(2 * E, np.int32), np.zeros(2 * E, np.int32), np.zeros(2 * E, np.float32)
    m = port_lib().orc_to_undirected(_ip(s), _ip(d), _fp(attr), L(E), _ip(os_), _ip(od), _fp(oa))
    return np.stack([os_[:m], od[:m]]), oa[:m].copy()


# --------------------------------------------------------------------- neighbour sampling
def sample_counts(dst, g_off, fanout):
    """``gpuinitco`` (ops/gpuinitco.py:30-36): ``out[i+1] = min(deg(dst[i]), fanout)``, ``out[0] = 0``
    (counts, not a running sum, as the reference kernel writes them)."""
    dst, g_off = _i32(dst), _i32(g_off)
    out = np.zeros(len(dst) + 1, np.int32)
    port_lib().orc_sample_counts(_ip(dst), L(len(dst)), _ip(g_off), ctypes.c_int32(fanout), _ip(out))
    return out


def csc_to_csr(col_off, row_idx, dst_ids, src_ids, impl="port"):
    """``csctocsr`` (ops/csctocsr.py:27-34) -> ``(row_offset, column_indices)``."""
    col_off, row_idx, dst_ids, src_ids = _i32(col_off), _i32(row_idx), _i32(dst_ids), _i32(src_ids)
    E = len(row_idx)
    ro, ci = np.zeros(len(src_ids) + 1, np.int32), np.zeros(E, np.int32)
    if impl == "ref":
        ref_lib().ref_csctocsr(_ip(col_off), _ip(row_idx), ctypes.c_long(len(dst_ids)), ctypes.c_long(E), _ip(dst_ids),
                               _ip(src_ids), ctypes.c_long(len(src_ids)), _ip(ro), _ip(ci))
    else:
        max_id = int(max(src_ids.max(initial=0), row_idx.max(initial=0)))
        port_lib().orc_csc_to_csr.restype = ctypes.c_int64
        port_lib().orc_csc_to_csr(_ip(col_off), _ip(row_idx), L(len(dst_ids)), _ip(dst_ids), _ip(src_ids), L(len(src_ids)),
                                  ctypes.c_int32(max_id), _ip(ro), _ip(ci))
    return ro, ci[: ro[-1]].copy()


def get_weight(vtx_size, dst_ids, src_ids, col_off, row_idx, impl="port"):
    """``getweight`` (ops/getweight.py:29-37)."""
    dst_ids, src_ids, col_off, row_idx = _i32(dst_ids), _i32(src_ids), _i32(col_off), _i32(row_idx)
    w = np.zeros(len(row_idx), np.float32)
    if impl == "ref":
        ref_lib().ref_getweight(ctypes.c_int(vtx_size), _ip(dst_ids), ctypes.c_long(len(dst_ids)), _ip(src_ids),
                                ctypes.c_long(len(src_ids)), _ip(col_off), _ip(row_idx), ctypes.c_long(len(row_idx)), _fp(w))
    else:
        port_lib().orc_get_weight(ctypes.c_int32(vtx_size), _ip(dst_ids), L(len(dst_ids)), _ip(col_off), _ip(row_idx), _fp(w))
    return w


def sample_reference(fanout, dst, layer_off, g_off, g_idx, seed=1):
    """The reference's own CPU sampler (ops/cpp/sampleprocessing_op.cc:38-90; draws with ``rand()``)."""
    dst, layer_off, g_off, g_idx = _i32(dst), _i32(layer_off), _i32(g_off), _i32(g_idx)
    out = np.zeros(int(layer_off[-1]), np.int32)
    ref_lib().ref_sampleprocessing(ctypes.c_int(fanout), _ip(dst), ctypes.c_long(len(dst)), _ip(layer_off), _ip(out),
                                   ctypes.c_long(len(out)), _ip(g_off), ctypes.c_long(len(g_off) - 1), _ip(g_idx),
                                   ctypes.c_long(len(g_idx)), ctypes.c_uint(seed))
    return out


def check_sample(fanout, dst, layer_off, layer_idx, g_off, g_idx):
    """What every valid sample satisfies (the draw itself is random in the reference): column i
    holds ``min(deg, fanout)`` entries; all of the destination's in-edges in their stored order when
    ``deg <= fanout`` (or ``fanout < 0``), else ``fanout`` entries taken from DISTINCT positions of
    its in-edge list.  Returns an error string or ``None``."""
    for i, v in enumerate(dst):
        nb = g_idx[g_off[v]: g_off[v + 1]]
        got = layer_idx[layer_off[i]: layer_off[i + 1]]
        want_n = len(nb) if fanout < 0 else min(len(nb), fanout)
        if len(got) != want_n:
            return f"column {i}: {len(got)} entries, expected {want_n}"
        if want_n == len(nb):
            if not np.array_equal(got, nb):
                return f"column {i}: full copy differs"
        else:
            pool = {}
            for x in nb:
                pool[int(x)] = pool.get(int(x), 0) + 1
            for x in got:
                if pool.get(int(x), 0) == 0:
                    return f"column {i}: {int(x)} drawn more often than it occurs"
                pool[int(x)] -= 1
    return None


# --------------------------------------------------------------------- gcn_norm
def gcn_norm(edge_index, w, n, add_self_loops=True):
    """C restatement of gcn_norm + add_remaining_self_loops
    (nn/conv/gcn_conv.py:18-37, utils/loop.py:120-134) -> (edge_index[2,E], w[E]).  A node without
    in-edges has degree 0 and deg^-1/2 = inf there, as in the reference (its ``masked_fill`` result
    is discarded, nn/conv/gcn_conv.py:36); this only arises with ``add_self_loops=False``."""
    ei = _i32(edge_index)
    E0 = ei.shape[1]
    s, d = _i32(ei[0]), _i32(ei[1])
    w = None if w is None else _f32(w)
    os_, od, ow = np.zeros(E0 + n, np.int32), np.zeros(E0 + n, np.int32), np.zeros(E0 + n, np.float32)
    E = port_lib().orc_gcn_norm(_ip(s), _ip(d), _fp(w), L(E0), ctypes.c_int32(n), _ip(os_), _ip(od),
                                _fp(ow), ctypes.c_int(1 if add_self_loops else 0))
    return np.stack([os_[:E], od[:E]]), ow[:E].copy()


def gcn_norm_numpy(edge_index, w, n):
    """The same recipe written with numpy array operations, mirroring the
    reference's tensor-level code line by line (nn/conv/gcn_conv.py:24-37,
    utils/loop.py:120-134); used to cross-check the C restatement."""
    ei = _i32(edge_index)
    w = np.ones(ei.shape[1], np.float32) if w is None else _f32(w)
    row, col = ei[0], ei[1]
    mask = row != col
    loop_index = np.arange(n, dtype=np.int32)
    new_ei = np.concatenate([ei[:, mask], np.stack([loop_index, loop_index])], axis=1)
    loop_w = np.ones(n, np.float32)
    inv = ~mask
    if inv.any():
        loop_w[row[inv]] = w[inv]
    new_w = np.concatenate([w[mask], loop_w])
    deg = np.zeros(n, np.float32)
    np.add.at(deg, new_ei[1], new_w)  # sequential, list order
    with np.errstate(divide="ignore"):
        dis = np.power(deg, np.float32(-0.5)).astype(np.float32)
    out_w = (dis[new_ei[0]] * new_w) * dis[new_ei[1]]
    return new_ei, out_w.astype(np.float32)


# --------------------------------------------------------------------- layers
def glorot(shape, rng):
    """U(-s, s), s = sqrt(6 / (fan_in + fan_out)) (nn/inits.py:19-22)."""
    s = np.sqrt(6.0 / (shape[-2] + shape[-1]))
    return rng.uniform(-s, s, size=shape).astype(np.float32)


def gat_aggregate(h, a_src, a_dst, idx, off, H, D, slope=0.2):
    """Edge phase of the attention layer (nn/conv/gat_conv.py:67-83), H heads."""
    h, a_src, a_dst = _f32(h), _f32(a_src), _f32(a_dst)
    idx, off = _i32(idx), _i32(off)
    n = len(off) - 1
    out = np.zeros((n, H * D), np.float32)
    port_lib().orc_gat_aggregate(_fp(out), _fp(h), _fp(a_src), _fp(a_dst), _ip(idx), _ip(off), L(n),
                                 L(H), L(D), ctypes.c_float(slope))
    return out


def gat_unfused(h, a, idx, off, impl="port"):
    """The reference's own single-head pipeline, op by op (nn/conv/gat_conv.py:67-83):
    ScatterToEdge src/dst, concat, @ a, leaky_relu, EdgeSoftmax, multiply, ScatterToVertex."""
    e_s = scatter_to_edge(h, idx, off, 0, impl)
    e_d = scatter_to_edge(h, idx, off, 1, impl)
    cat = np.concatenate([e_s, e_d], axis=1)
    m = (cat @ _f32(a).reshape(-1, 1)).astype(np.float32)
    m = np.where(m > 0, m, np.float32(0.2) * m).astype(np.float32)
    alpha = edge_softmax(m.reshape(-1), off, impl).reshape(-1, 1)
    msg = (cat[:, : h.shape[1]] * alpha).astype(np.float32)
    return edge_to_vertex(msg, idx, off, 1, impl)


def gat_unfused_backward(h, a, idx, off, grad_out, impl="port"):
    """Gradients of :func:`gat_unfused` with respect to ``h`` and ``a``, composed from the reference's
    own backward pairings: ScatterToVertex.grad = scatter_to_edge by destination
    (ops/scatterToVertex.py:41-45), EdgeSoftmax.grad = edgesoftmaxbackward (ops/edgesoftmax.py:69-74),
    ScatterToEdge.grad = edge_to_vertex with the same flag (ops/scatterToEdge.py:42-46); the dense
    steps (concat, @ a, leaky_relu, multiply) differentiated with numpy.  Returns ``(grad_h, grad_a)``."""
    h, a, g = _f32(h), _f32(a).reshape(-1), _f32(grad_out)
    c = h.shape[1]
    e_s = scatter_to_edge(h, idx, off, 0, impl)
    e_d = scatter_to_edge(h, idx, off, 1, impl)
    cat = np.concatenate([e_s, e_d], axis=1)
    pre = (cat @ a.reshape(-1, 1)).astype(np.float32).reshape(-1)
    m = np.where(pre > 0, pre, np.float32(0.2) * pre).astype(np.float32)
    alpha = edge_softmax(m, off, impl)
    g_msg = scatter_to_edge(g, idx, off, 1, impl)                       # d out[v] / d msg[e] = 1 for e in seg(v)
    g_alpha = (g_msg * e_s).sum(1).astype(np.float32)
    g_es = (g_msg * alpha.reshape(-1, 1)).astype(np.float32)
    g_m = edge_softmax_backward(g_alpha, alpha, off, impl)
    g_pre = np.where(pre > 0, g_m, np.float32(0.2) * g_m).astype(np.float32)
    g_cat = g_pre.reshape(-1, 1) * a.reshape(1, -1)
    grad_a = (cat * g_pre.reshape(-1, 1)).sum(0).astype(np.float32)
    g_es = (g_es + g_cat[:, :c]).astype(np.float32)
    g_ed = g_cat[:, c:].astype(np.float32)
    grad_h = edge_to_vertex(g_es, idx, off, 0, impl) + edge_to_vertex(g_ed, idx, off, 1, impl)
    return grad_h.astype(np.float32), grad_a


def gcn_layer(x, W, b, csc, impl="port"):
    """GCNConv.execute (nn/conv/gcn_conv.py:94-102): (x @ W) aggregated over CSC, plus bias."""
    idx, off, w = csc
    h = (_f32(x) @ _f32(W)).astype(np.float32)
    out = aggregate(h, idx, off, w, impl=impl)
    return out + b if b is not None else out
