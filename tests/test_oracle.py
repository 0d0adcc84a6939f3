"""CPU-only: the plain-C restatement must reproduce the golden vectors (which were
produced by the reference's own compiled CPU bodies) bit for bit, and must agree
with those bodies live wherever the compiled reference library is present."""
import os

import numpy as np
import pytest

G = os.path.join(os.path.dirname(__file__), "golden")


def load(name):
    return dict(np.load(os.path.join(G, name + ".npz")))


def impls(oracle):
    return ["port", "ref"] if oracle.have_ref() else ["port"]


def test_conversion_goldens(oracle):
    for impl in impls(oracle):
        for name in ("ref_test_csr", "ref_test_mp_spmm"):
            d = load(name)
            n = int(d["n"])
            ci, ro, cw = oracle.coo_to_csr(d["edge_index"], d["edge_weight"], n, impl)
            ri, co, sw = oracle.coo_to_csc(d["edge_index"], d["edge_weight"], n, impl)
            for got, key in ((ci, "column_indices"), (ro, "row_offset"), (cw, "csr_weight"),
                             (ri, "row_indices"), (co, "column_offset"), (sw, "csc_weight")):
                assert np.array_equal(got, d[key]), (impl, name, key)
    d = load("ref_test_csr")
    assert d["row_offset"].tolist() == [0, 2, 4, 5, 5]


def test_aggregate_goldens(oracle):
    for impl in impls(oracle):
        d = load("ref_test_mp_spmm")
        assert np.array_equal(oracle.aggregate(d["x"], d["row_indices"], d["column_offset"], d["csc_weight"], impl=impl), d["out_csc"])
        assert np.array_equal(oracle.aggregate(d["x"], d["column_indices"], d["row_offset"], d["csr_weight"], impl=impl), d["out_csr"])
        d = load("ref_test_aggregate")
        assert np.array_equal(oracle.aggregate(d["x"], d["row_indices"], d["column_offset"], d["csc_weight"], impl=impl), d["out_fwd"])
        assert np.array_equal(oracle.aggregate(d["x"], d["column_indices"], d["row_offset"], d["csr_weight"], impl=impl), d["out_bwd"])
        d = load("citation_2708")
        assert np.array_equal(oracle.aggregate(d["x7"], d["row_indices"], d["column_offset"], d["csc_weight"], impl=impl), d["y7"])


def test_aggregate_matches_float64_truth(oracle):
    d = load("citation_2708")
    y = oracle.aggregate(d["x7"], d["row_indices"], d["column_offset"], d["csc_weight"])
    truth, scale = oracle.aggregate_f64(d["x7"], d["row_indices"], d["column_offset"], d["csc_weight"])
    assert (np.abs(y - truth) / (scale + 1e-30)).max() <= 1e-5


def test_edge_ops_goldens(oracle):
    for impl in impls(oracle):
        d = load("ref_test_edgesoftmax")
        y = oracle.edge_softmax(d["x"], d["column_offset"], impl)
        assert np.array_equal(y, d["out"])
        assert np.array_equal(oracle.edge_softmax_backward(d["grad"], y, d["column_offset"], impl), d["grad_in"])
        d = load("ref_test_scatter")
        assert np.array_equal(oracle.scatter_to_edge(d["x_vertex"], d["row_indices"], d["column_offset"], 0, impl), d["to_edge_src"])
        assert np.array_equal(oracle.scatter_to_edge(d["x_vertex"], d["row_indices"], d["column_offset"], 1, impl), d["to_edge_dst"])
        assert np.array_equal(oracle.edge_to_vertex(d["x_edge"], d["row_indices"], d["column_offset"], 1, impl), d["to_vertex_dst"])
        assert np.array_equal(oracle.edge_to_vertex(d["x_edge"], d["row_indices"], d["column_offset"], 0, impl), d["to_vertex_src"])
        d = load("ref_test_undirected")
        nei, _ = oracle.to_undirected(d["edge_index"], d["edge_attr"], 3, impl)
        assert np.array_equal(nei, d["new_edge_index"])
    d = load("ref_test_edgesoftmax")
    assert abs(float(d["out"][1] + d["out"][2]) - 1.0) < 1e-6


def test_multihead_softmax_is_per_column(oracle):
    rng = np.random.default_rng(3)
    off = np.array([0, 3, 3, 10, 11], np.int32)
    x = rng.standard_normal((11, 4)).astype(np.float32)
    y = oracle.edge_softmax(x, off)
    for h in range(4):
        assert np.array_equal(y[:, h], oracle.edge_softmax(x[:, h].copy(), off))


def test_gcn_norm_golden_and_numpy(oracle):
    d = load("citation_2708")
    ei, w = oracle.gcn_norm(d["edge_index"], None, 2708)
    assert np.array_equal(ei, d["norm_edge_index"]) and np.array_equal(w, d["norm_weight"])
    assert ei.shape[1] == 10556 + 2708
    assert np.array_equal(ei[:, -2708:], np.stack([np.arange(2708)] * 2))  # loops appended last, in node order
    ei2, w2 = oracle.gcn_norm_numpy(d["edge_index"], None, 2708)
    assert np.array_equal(ei, ei2)
    ulp = np.abs(w.view(np.int32).astype(np.int64) - w2.view(np.int32).astype(np.int64)).max()
    assert ulp <= 8  # numpy's float32 power and libm's powf differ in the last bits


def test_gcn_norm_existing_loops_keep_their_weight(oracle):
    ei = np.array([[0, 1, 1, 2], [1, 1, 2, 0]], np.int32)
    w = np.array([1.0, 5.0, 2.0, 3.0], np.float32)
    nei, nw = oracle.gcn_norm(ei, w, 3)
    assert nei.tolist() == [[0, 1, 2, 0, 1, 2], [1, 2, 0, 0, 1, 2]]
    nei2, nw2 = oracle.gcn_norm_numpy(ei, w, 3)
    assert np.array_equal(nei, nei2) and np.allclose(nw, nw2, rtol=1e-6)
    # degree of node 1 = w(0->1) + loop weight 5
    assert np.isclose(nw[4], 5.0 / 6.0, rtol=1e-6)


@pytest.mark.parametrize("n,E,f", [(1, 0, 3), (7, 0, 4), (50, 400, 5), (300, 9000, 33)])
def test_port_equals_compiled_reference_on_random_graphs(oracle, n, E, f):
    if not oracle.have_ref():
        pytest.skip("compiled reference bodies not present")
    rng = np.random.default_rng(n * 1000 + E)
    ei = rng.integers(0, n, size=(2, E)).astype(np.int32)
    w = rng.standard_normal(E).astype(np.float32)
    for fn in (oracle.coo_to_csr, oracle.coo_to_csc):
        for a, b in zip(fn(ei, w, n, "port"), fn(ei, w, n, "ref")):
            assert np.array_equal(a, b)
    idx, off, cw = oracle.coo_to_csc(ei, w, n)
    x = rng.standard_normal((n, f)).astype(np.float32)
    assert np.array_equal(oracle.aggregate(x, idx, off, cw, impl="port"), oracle.aggregate(x, idx, off, cw, impl="ref"))
    sc = (rng.standard_normal(E) * 4).astype(np.float32)
    y = oracle.edge_softmax(sc, off, "port")
    assert np.array_equal(y, oracle.edge_softmax(sc, off, "ref"))
    g = rng.standard_normal(E).astype(np.float32)
    assert np.array_equal(oracle.edge_softmax_backward(g, y, off, "port"), oracle.edge_softmax_backward(g, y, off, "ref"))
    m = rng.standard_normal((E, f)).astype(np.float32)
    for flag in (0, 1):
        assert np.array_equal(oracle.scatter_to_edge(x, idx, off, flag, "port"), oracle.scatter_to_edge(x, idx, off, flag, "ref"))
        assert np.array_equal(oracle.edge_to_vertex(m, idx, off, flag, "port"), oracle.edge_to_vertex(m, idx, off, flag, "ref"))


def test_fused_gat_restatement_equals_unfused_reference_pipeline(oracle):
    rng = np.random.default_rng(11)
    n, E, C = 200, 3000, 8
    ei = rng.integers(0, n, size=(2, E)).astype(np.int32)
    nei, nw = oracle.gcn_norm(ei, None, n)
    idx, off, _ = oracle.coo_to_csc(nei, nw, n)
    h = np.maximum(rng.standard_normal((n, C)), 0).astype(np.float32)
    a = (rng.standard_normal(2 * C) * 0.3).astype(np.float32)
    impl = "ref" if oracle.have_ref() else "port"
    unfused = oracle.gat_unfused(h, a, idx, off, impl)
    fused = oracle.gat_aggregate(h, a[:C].reshape(1, C), a[C:].reshape(1, C), idx, off, 1, C)
    assert np.abs(unfused - fused).max() <= 2e-6


def test_sampling_checkers_on_the_reference_fixtures(oracle):
    """gpuinitco / csctocsr / getweight inputs of the reference's own tests (tests/test_gpuinitco.py:15-22,
    tests/test_csctocsr.py:25-35, tests/test_getweight.py:25-48) with the outputs those files state; the C
    restatement against the compiled reference bodies on the same inputs and on a random case."""
    ids = np.arange(4, dtype=np.int32)
    assert oracle.sample_counts(ids, np.array([0, 1, 3, 4, 5]), 2).tolist() == [0, 1, 2, 1, 1]
    impls = ["port", "ref"] if oracle.have_ref() else ["port"]
    for impl in impls:
        ro, ci = oracle.csc_to_csr(np.array([0, 0, 1, 2, 4]), np.array([0, 0, 1, 2]), ids, ids, impl)
        assert ro.tolist() == [0, 2, 3, 4, 4] and ci.tolist() == [1, 2, 3, 3]
        w = oracle.get_weight(4, ids, ids, np.array([0, 1, 2, 3, 4]), np.array([0, 0, 1, 2]), impl)
        assert np.abs(w - np.array([2 ** -0.5, 2 ** -0.5, 1, 1])).max() <= 1e-7
    rng = np.random.default_rng(0)
    n = 300
    dst = rng.integers(0, n, size=4000)
    off = np.concatenate([[0], np.cumsum(np.bincount(dst, minlength=n))]).astype(np.int32)
    idx = rng.integers(0, n, size=4000).astype(np.int32)
    ids = np.arange(n, dtype=np.int32)
    if oracle.have_ref():
        a, b = oracle.csc_to_csr(off, idx, ids, ids, "port"), oracle.csc_to_csr(off, idx, ids, ids, "ref")
        assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])
        assert np.array_equal(oracle.get_weight(n, ids, ids, off, idx, "port"), oracle.get_weight(n, ids, ids, off, idx, "ref"))
        some = rng.permutation(n)[:40].astype(np.int32)
        l_off = oracle.sample_counts(some, off, 6).cumsum().astype(np.int32)
        drawn = oracle.sample_reference(6, some, l_off, off, idx, seed=5)
        assert oracle.check_sample(6, some, l_off, drawn, off, idx) is None
    # the property checker rejects a sample that repeats a position
    bad_off = np.array([0, 2], np.int32)
    assert oracle.check_sample(2, np.array([0]), bad_off, np.array([7, 7]), np.array([0, 3]), np.array([7, 8, 9])) is not None


def test_sampling_golden_vectors(oracle):
    """Committed outputs of the compiled reference bodies for the sampling operators: the C
    restatement reproduces them (and so does the compiled reference where it is built)."""
    d = dict(np.load(os.path.join(G, "ref_test_sampling.npz")))
    ids4 = np.arange(4, dtype=np.int32)
    impls = ["port", "ref"] if oracle.have_ref() else ["port"]
    for impl in impls:
        ro, ci = oracle.csc_to_csr(d["csr_in_column_offset"], d["csr_in_row_indices"], ids4, ids4, impl)
        assert np.array_equal(ro, d["csr_row_offset"]) and np.array_equal(ci, d["csr_column_indices"])
        assert np.array_equal(oracle.get_weight(4, ids4, ids4, d["w_column_offset"], d["w_row_indices"], impl), d["w_out"])
        ro, ci = oracle.csc_to_csr(d["l_column_offset"], d["l_row_indices"], d["l_dst"], d["l_src"], impl)
        assert np.array_equal(ro, d["l_row_offset"]) and np.array_equal(ci, d["l_column_indices"])
        assert np.array_equal(oracle.get_weight(4000, d["l_dst"], d["l_src"], d["l_column_offset"], d["l_row_indices"], impl),
                              d["l_weight"])
    assert np.array_equal(oracle.sample_counts(d["counts_dst"], d["counts_global_offset"], 2), d["counts_out"])
    # every degree is within the fanout: the sample is the in-edge lists in stored order
    want = np.concatenate([d["s_global_indices"][d["s_global_offset"][v]: d["s_global_offset"][v + 1]] for v in d["s_dst"]])
    assert np.array_equal(d["s_out"], want)
    assert oracle.check_sample(3, d["s_dst"], d["s_layer_offset"], d["s_out"], d["s_global_offset"], d["s_global_indices"]) is None


def test_attention_backward_composition(oracle):
    """The reference's backward pairings composed into the gradient of its attention pipeline agree with
    float64 autograd of the same formula (torch on the CPU)."""
    import torch
    rng = np.random.default_rng(12)
    n, c = 60, 8
    dst = rng.integers(0, n, size=500)
    src = rng.integers(0, n, size=500)
    order = np.argsort(dst, kind="stable")
    idx = src[order].astype(np.int32)
    off = np.concatenate([[0], np.cumsum(np.bincount(dst, minlength=n))]).astype(np.int32)
    h = rng.standard_normal((n, c)).astype(np.float32)
    a = (rng.standard_normal(2 * c) * 0.4).astype(np.float32)
    g = rng.standard_normal((n, c)).astype(np.float32)
    impls = ["port", "ref"] if oracle.have_ref() else ["port"]
    ht, at = torch.from_numpy(h).double().requires_grad_(True), torch.from_numpy(a).double().requires_grad_(True)
    seg = torch.from_numpy(np.repeat(np.arange(n), np.diff(off)))
    e_s, e_d = ht[torch.from_numpy(idx).long()], ht[seg]
    m = torch.nn.functional.leaky_relu(torch.cat([e_s, e_d], 1) @ at, 0.2)
    top = torch.full((n,), -float("inf"), dtype=torch.float64).scatter_reduce(0, seg, m, "amax")
    p = torch.exp(m - top[seg])
    alpha = p / torch.zeros(n, dtype=torch.float64).index_add(0, seg, p)[seg]
    out = torch.zeros((n, c), dtype=torch.float64).index_add(0, seg, e_s * alpha.unsqueeze(1))
    out.backward(torch.from_numpy(g).double())
    for impl in impls:
        fwd = oracle.gat_unfused(h, a, idx, off, impl)
        assert np.abs(fwd - out.detach().numpy()).max() <= 1e-5
        gh, ga = oracle.gat_unfused_backward(h, a, idx, off, g, impl)
        assert np.abs(gh - ht.grad.numpy()).max() <= 2e-5 * np.abs(ht.grad.numpy()).max()
        assert np.abs(ga - at.grad.numpy()).max() <= 2e-5 * np.abs(at.grad.numpy()).max()


def test_sampling_restatement_against_reference_randomised(oracle):
    """Property test (hypothesis): the C restatement of csctocsr / getweight equals the compiled reference
    bodies on random small structures, including empty columns, unlisted sources and repeated ids."""
    if not oracle.have_ref():
        pytest.skip("compiled reference bodies not available")
    from hypothesis import given, settings, strategies as st

    @settings(max_examples=60, deadline=None)
    @given(st.integers(0, 2**31 - 1))
    def run(seed):
        rng = np.random.default_rng(seed)
        n_dst, universe = int(rng.integers(1, 12)), int(rng.integers(1, 30))
        off = np.concatenate([[0], np.cumsum(rng.integers(0, 5, size=n_dst))]).astype(np.int32)
        idx = rng.integers(0, universe, size=off[-1]).astype(np.int32)
        dst = rng.integers(0, universe, size=n_dst).astype(np.int32)
        src = rng.permutation(universe)[: int(rng.integers(0, universe + 1))].astype(np.int32)
        a, b = oracle.csc_to_csr(off, idx, dst, src, "port"), oracle.csc_to_csr(off, idx, dst, src, "ref")
        assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])
        if off[-1]:
            w1 = oracle.get_weight(universe, dst, src, off, idx, "port")
            w2 = oracle.get_weight(universe, dst, src, off, idx, "ref")
            assert np.array_equal(w1, w2)

    run()
