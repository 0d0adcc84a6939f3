"""GPU parity of COO->CSR/CSC conversion and the fused gcn_norm against the CPU checker:
indices, offsets and entry order bit-exact; normalised weights within a few ulp."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
G = os.path.join(os.path.dirname(__file__), "golden")


def load(name):
    return dict(np.load(os.path.join(G, name + ".npz")))


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.cpu().numpy()


def ulp_diff(a, b):
    return int(np.abs(a.view(np.int32).astype(np.int64) - b.view(np.int32).astype(np.int64)).max()) if a.size else 0


@pytest.mark.parametrize("name", ["ref_test_csr", "ref_test_mp_spmm"])
def test_reference_smoke_inputs(cuda, name):
    d = load(name)
    n = int(d["n"])
    csr = cuda.cootocsr(dev(d["edge_index"]), dev(d["edge_weight"]), n)
    csc = cuda.cootocsc(dev(d["edge_index"]), dev(d["edge_weight"]), n)
    assert np.array_equal(host(csr.column_indices), d["column_indices"])
    assert np.array_equal(host(csr.row_offset), d["row_offset"])
    assert np.array_equal(host(csr.edge_weight), d["csr_weight"])
    assert np.array_equal(host(csc.row_indices), d["row_indices"])
    assert np.array_equal(host(csc.column_offset), d["column_offset"])
    assert np.array_equal(host(csc.edge_weight), d["csc_weight"])


@pytest.mark.parametrize("n,E", [(1, 0), (1, 5), (3, 0), (200, 1), (256, 5000), (257, 5000), (5000, 70000),
                                 (70000, 300000), (1 << 17, 1 << 20)])
def test_stable_order_bit_exact(cuda, oracle, n, E):
    rng = np.random.default_rng(n * 7 + E)
    # skewed keys: duplicates, hubs and empty rows all occur
    ei = np.minimum((rng.random((2, E)) ** 3 * n).astype(np.int32), n - 1)
    w = rng.standard_normal(E).astype(np.float32)
    for by, fn, ofn in ((0, cuda.cootocsr, oracle.coo_to_csr), (1, cuda.cootocsc, oracle.coo_to_csc)):
        got = fn(dev(ei), dev(w), n)
        idx, off, ow = ofn(ei, w, n)
        g_idx, g_off = (got.column_indices, got.row_offset) if by == 0 else (got.row_indices, got.column_offset)
        assert np.array_equal(host(g_off), off)
        assert np.array_equal(host(g_idx), idx)
        assert np.array_equal(host(got.edge_weight), ow)


def test_canonical_order(cuda, oracle):
    rng = np.random.default_rng(9)
    n, E = 3000, 60000
    ei = rng.integers(0, n, size=(2, E)).astype(np.int32)
    w = rng.standard_normal(E).astype(np.float32)
    got = cuda.cootocsr(dev(ei), dev(w), n, sorted=True)
    idx, off, ow = oracle.coo_to_csr(ei, w, n)
    cidx, cw, _ = oracle.sort_within_rows(idx, off, ow)
    assert np.array_equal(host(got.row_offset), off)
    assert np.array_equal(host(got.column_indices), cidx)
    assert np.array_equal(host(got.edge_weight), cw)       # equal (row, col) pairs keep list order


@pytest.mark.parametrize("n,E,weighted", [(300, 4000, False), (300, 4000, True), (40000, 500000, False), (40000, 500000, True),
                                          (70000, 300000, True)])
def test_gcn_norm_sorted_columns(cuda, oracle, n, E, weighted):
    """``sorted=True``: both formats with the columns of every row in ascending order.  The CSR is built from
    the finished CSC list by one stable sort (equal pairs keep list order, weights travel with their
    entries); it must equal the reference's conversion of the normalised list, sorted inside its rows."""
    rng = np.random.default_rng(3 * n + E + weighted)
    ei = rng.integers(0, n, size=(2, E)).astype(np.int32)
    ei[:, : E // 50] = ei[:, E // 50: 2 * (E // 50)]            # repeated (source, destination) pairs
    w = rng.standard_normal(E).astype(np.float32) ** 2 + 0.1 if weighted else None
    csc, csr = cuda.gcn_norm_csc_csr(dev(ei), None if w is None else dev(w), n, sorted=True)
    nei, nw = oracle.gcn_norm(ei, w, n)
    for got, conv in ((csc, oracle.coo_to_csc), (csr, oracle.coo_to_csr)):
        idx, off, ow = conv(nei, nw, n)
        cidx, cw, _ = oracle.sort_within_rows(idx, off, ow)
        g_idx = got.row_indices if hasattr(got, "row_indices") else got.column_indices
        g_off = got.column_offset if hasattr(got, "column_offset") else got.row_offset
        assert np.array_equal(host(g_off), off)
        assert np.array_equal(host(g_idx), cidx)
        # the degree of a node is a sequential fp32 sum over its column in LIST order, and the sorted list is
        # in another order than the input list the reference sums over: a few ulp on weighted graphs
        gw = host(got.edge_weight)
        assert np.abs(gw - cw).max() <= 2e-6 * np.abs(cw).max() and (ulp_diff(gw, cw) <= 4 or weighted)
    # the CSR's weights were carried with their entries, not recomputed: the two formats hold the same numbers
    a = np.stack([np.repeat(np.arange(n), np.diff(host(csc.column_offset))), host(csc.row_indices), host(csc.edge_weight).view(np.int32)])
    b = np.stack([host(csr.column_indices), np.repeat(np.arange(n), np.diff(host(csr.row_offset))), host(csr.edge_weight).view(np.int32)])
    key_a = np.lexsort((a[2], a[1], a[0])); key_b = np.lexsort((b[2], b[1], b[0]))
    assert np.array_equal(a[:, key_a], b[:, key_b])


def check_gcn(cuda, oracle, ei, w, n, improved=False):
    csc, csr = cuda.gcn_norm_csc_csr(dev(ei), None if w is None else dev(w), n, improved=improved)
    if improved:
        pytest.skip("improved=True is checked by test_improved_fill only")
    nei, nw = oracle.gcn_norm(ei, w, n)
    for got, (idx, off, ow) in ((csc, oracle.coo_to_csc(nei, nw, n)), (csr, oracle.coo_to_csr(nei, nw, n))):
        g_idx = got.row_indices if hasattr(got, "row_indices") else got.column_indices
        g_off = got.column_offset if hasattr(got, "column_offset") else got.row_offset
        assert np.array_equal(host(g_off), off)
        assert np.array_equal(host(g_idx), idx)
        gw = host(got.edge_weight)
        assert ulp_diff(gw, ow) <= 4      # deg^-1/2: correctly rounded here, libm powf in the checker
    return csc, csr


def test_gcn_norm_citation_graph(cuda, oracle):
    d = load("citation_2708")
    csc, csr = check_gcn(cuda, oracle, d["edge_index"], None, 2708)
    assert np.array_equal(host(csc.row_indices), d["row_indices"])
    assert np.array_equal(host(csr.column_indices), d["column_indices"])
    assert csc.row_indices.numel() == 10556 + 2708
    frac_exact = float((host(csc.edge_weight) == d["csc_weight"]).mean())
    assert frac_exact > 0.95


@pytest.mark.parametrize("n,E,weighted", [(1, 0, False), (5, 3, True), (300, 4000, False), (300, 4000, True),
                                          (40000, 500000, False), (40000, 500000, True)])
def test_gcn_norm_random(cuda, oracle, n, E, weighted):
    rng = np.random.default_rng(n + E + weighted)
    ei = np.minimum((rng.random((2, E)) ** 2 * n).astype(np.int32), n - 1)   # includes (v,v) entries and duplicates
    w = (rng.random(E).astype(np.float32) + 0.1) if weighted else None
    check_gcn(cuda, oracle, ei, w, n)


def test_existing_loops_keep_last_weight(cuda, oracle):
    ei = np.array([[0, 1, 1, 2, 1], [1, 1, 2, 0, 1]], np.int32)
    w = np.array([1.0, 5.0, 2.0, 3.0, 7.0], np.float32)
    csc, _ = check_gcn(cuda, oracle, ei, w, 3)
    assert csc.row_indices.numel() == 3 + 3


def test_runs_are_identical(cuda):
    rng = np.random.default_rng(4)
    n, E = 20000, 400000
    ei = dev(rng.integers(0, n, size=(2, E)).astype(np.int32))
    w = dev(rng.random(E).astype(np.float32))
    a, _ = cuda.gcn_norm_csc_csr(ei, w, n)
    b, _ = cuda.gcn_norm_csc_csr(ei, w, n)
    assert torch.equal(a.row_indices, b.row_indices) and torch.equal(a.edge_weight, b.edge_weight)


def test_bad_arguments(cuda):
    with pytest.raises(RuntimeError):
        cuda.cootocsr(torch.zeros((3, 4), dtype=torch.int32, device="cuda"), torch.zeros(4, device="cuda"), 5)
    with pytest.raises(RuntimeError):
        cuda.cootocsr(torch.zeros((2, 4), dtype=torch.int32, device="cuda"), torch.zeros(3, device="cuda"), 5)


def test_to_undirected(cuda, oracle):
    d = load("ref_test_undirected")
    gei, ga = cuda.toUndirected(dev(d["edge_index"]), dev(d["edge_attr"]), 3)
    assert np.array_equal(host(gei), d["new_edge_index"])
    assert np.array_equal(host(ga), d["new_edge_attr"])
    rng = np.random.default_rng(12)
    for n, E in ((1, 3), (50, 0), (300, 5000), (70000, 400000)):
        ei = np.minimum((rng.random((2, E)) ** 2 * n).astype(np.int32), max(n - 1, 0))
        a = rng.standard_normal(E).astype(np.float32)
        gei, ga = cuda.toUndirected(dev(ei), dev(a), n)
        wei, wa = oracle.to_undirected(ei, a, n, "port")         # first of every duplicate run survives
        assert np.array_equal(host(gei), wei) and np.array_equal(host(ga), wa)
        if oracle.have_ref() and E:
            rei, _ = oracle.to_undirected(ei, a, n, "ref")       # the reference's indices (its attribute choice is unspecified)
            assert np.array_equal(host(gei), rei)
