"""GPU parity of the per-edge operators, the fused attention kernel, the SpMM front ends and the
layer shims against the CPU checker."""
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
    return t.detach().cpu().numpy()


def random_csc(rng, n, E, hubs=0, hub_deg=0):
    dst = rng.integers(0, n, size=E)
    if hubs:
        dst = np.concatenate([dst, np.repeat(rng.integers(0, n, size=hubs), hub_deg)])
    src = rng.integers(0, n, size=len(dst))
    order = np.argsort(dst, kind="stable")
    off = np.concatenate([[0], np.cumsum(np.bincount(dst, minlength=n))]).astype(np.int32)
    return src[order].astype(np.int32), off


def softmax64(x, off):
    x = x.astype(np.float64)
    out = np.zeros_like(x)
    for v in range(len(off) - 1):
        s, e = off[v], off[v + 1]
        if e > s:
            z = np.exp(x[s:e] - x[s:e].max(0, keepdims=True))
            out[s:e] = z / z.sum(0, keepdims=True)
    return out


def test_reference_smoke_inputs(cuda):
    d = load("ref_test_scatter")
    csc = cuda.CSC(dev(d["row_indices"]), dev(d["column_offset"]), None)
    assert np.array_equal(host(cuda.ScatterToEdge(dev(d["x_vertex"]), csc, "src")), d["to_edge_src"])
    assert np.array_equal(host(cuda.ScatterToEdge(dev(d["x_vertex"]), csc, "dst")), d["to_edge_dst"])
    assert np.array_equal(host(cuda.ScatterToVertex(dev(d["x_edge"]), csc, "src")), d["to_vertex_dst"])
    d = load("ref_test_edgesoftmax")
    csc = cuda.CSC(dev(d["row_indices"]), dev(d["column_offset"]), None)
    x = dev(d["x"]).requires_grad_(True)
    y = cuda.EdgeSoftmax(x, csc)
    assert np.abs(host(y) - d["out"]).max() <= 1e-6
    y.backward(dev(d["grad"]))
    assert np.abs(host(x.grad) - d["grad_in"]).max() <= 1e-6


@pytest.mark.parametrize("c", [1, 3, 8, 64, 100])
def test_scatter_and_gather(cuda, oracle, c):
    rng = np.random.default_rng(c)
    n = 900
    idx, off = random_csc(rng, n, 12000, hubs=2, hub_deg=700)
    E = len(idx)
    csc = cuda.CSC(dev(idx), dev(off), None)
    x = rng.standard_normal((n, c)).astype(np.float32)
    m = rng.standard_normal((E, c)).astype(np.float32)
    for flow, flag in (("src", 0), ("dst", 1)):
        assert np.array_equal(host(cuda.ScatterToEdge(dev(x), csc, flow)), oracle.scatter_to_edge(x, idx, off, flag))
    assert np.array_equal(host(cuda.ScatterToVertex(dev(m), csc, "src")), oracle.edge_to_vertex(m, idx, off, 1))
    # backward pairings: gather-by-source scatters back by source (atomics: tolerance), gather-by-dst sums per dst
    xs = dev(x).requires_grad_(True)
    cuda.ScatterToEdge(xs, csc, "src").backward(dev(m))
    want = oracle.edge_to_vertex(m, idx, off, 0)
    scale = oracle.edge_to_vertex(np.abs(m), idx, off, 0)
    assert (np.abs(host(xs.grad) - want) / (scale + 1e-30)).max() <= 1e-5
    xd = dev(x).requires_grad_(True)
    cuda.ScatterToEdge(xd, csc, "dst").backward(dev(m))
    assert np.array_equal(host(xd.grad), oracle.edge_to_vertex(m, idx, off, 1))
    ms = dev(m).requires_grad_(True)
    cuda.ScatterToVertex(ms, csc, "src").backward(dev(x))
    assert np.array_equal(host(ms.grad), oracle.scatter_to_edge(x, idx, off, 1))


@pytest.mark.parametrize("h", [1, 2, 3, 4, 8, 16, 32])
def test_edge_softmax(cuda, oracle, h):
    rng = np.random.default_rng(10 + h)
    n = 600
    idx, off = random_csc(rng, n, 9000, hubs=2, hub_deg=3000)
    E = len(idx)
    csc = cuda.CSC(dev(idx), dev(off), None)
    x = (rng.standard_normal((E, h)) * 4).astype(np.float32)
    x[:5] += 90.0    # the reference's CUDA kernel overflows here; the CPU recipe (max subtracted) does not
    xt = dev(x if h > 1 else x[:, 0]).requires_grad_(True)
    y = cuda.EdgeSoftmax(xt, csc)
    want = oracle.edge_softmax(x, off)
    got = host(y).reshape(E, h)
    assert np.isfinite(got).all()
    # float64 truth: the reference's sequential fp32 sum over a 3000-edge segment carries its own
    # rounding error (the kernel sums the same terms in another order), so the bar is 1e-6 beyond
    # the reference recipe's own distance from the truth
    truth = softmax64(x, off)
    ref_err = np.abs(want - truth).max()
    assert np.abs(got - truth).max() <= 1e-6 + ref_err
    assert np.abs(got - want).max() <= 1e-6 + 2 * ref_err
    seg = np.repeat(np.arange(n), np.diff(off))
    sums = np.zeros((n, h)); np.add.at(sums, seg, got)
    assert np.abs(sums[np.diff(off) > 0] - 1).max() <= 1e-5
    g = rng.standard_normal((E, h)).astype(np.float32)
    y.backward(dev(g if h > 1 else g[:, 0]))
    want_g = oracle.edge_softmax_backward(g, want, off)
    # same bar for the backward: float64 truth, plus the distance of the reference's own sequential
    # fp32 recipe from it (long segments are summed in another order here)
    t64 = truth * g - truth * np.add.reduceat(truth * g, off[:-1][np.diff(off) > 0])[np.cumsum(np.diff(off) > 0)[seg] - 1]
    ref_err_g = np.abs(want_g - t64).max()
    got_g = host(xt.grad).reshape(E, h)
    assert np.abs(got_g - t64).max() <= 2e-6 + ref_err_g
    assert np.abs(got_g - want_g).max() <= 2e-6 + 2 * ref_err_g


@pytest.mark.parametrize("heads,dim", [(1, 8), (1, 64), (8, 8), (2, 16), (4, 4), (1, 128), (16, 8)])
def test_fused_attention(cuda, oracle, heads, dim):
    rng = np.random.default_rng(heads * 100 + dim)
    n, c = 700, heads * dim
    idx, off = random_csc(rng, n, 9000, hubs=2, hub_deg=2500)
    idx[off[1:][np.diff(off) > 0] - 1] = np.arange(n)[np.diff(off) > 0]   # a self-loop in every non-empty column
    csc = cuda.CSC(dev(idx), dev(off), None)
    hfeat = np.maximum(rng.standard_normal((n, c)), 0).astype(np.float32)
    a_src = (rng.standard_normal((heads, dim)) * 0.5).astype(np.float32)
    a_dst = (rng.standard_normal((heads, dim)) * 0.5).astype(np.float32)
    assert cuda.gat_aggregate_supported(heads, dim)
    got = host(cuda.gat_aggregate(dev(hfeat), dev(a_src), dev(a_dst), csc, heads))
    want = oracle.gat_aggregate(hfeat, a_src, a_dst, idx, off, heads, dim)
    scale = np.abs(hfeat).max() + 1e-30     # outputs are convex combinations of source rows
    assert np.abs(got - want).max() / scale <= 1e-5
    again = host(cuda.gat_aggregate(dev(hfeat), dev(a_src), dev(a_dst), csc, heads))
    assert np.array_equal(got, again)


def test_fused_attention_hub_destinations(cuda, oracle):
    """Destinations with 4096 or more in-edges take the path where a whole thread block shares one
    segment; 9000- and 20000-edge hubs, next to ordinary and empty destinations."""
    rng = np.random.default_rng(77)
    n, heads, dim = 3000, 8, 8
    dst = np.concatenate([rng.integers(10, n, size=20000), np.full(9000, 3), np.full(20000, 1500), np.full(4096, 7)])
    src = rng.integers(0, n, size=len(dst))
    order = np.argsort(dst, kind="stable")
    idx = src[order].astype(np.int32)
    off = np.concatenate([[0], np.cumsum(np.bincount(dst, minlength=n))]).astype(np.int32)
    csc = cuda.CSC(dev(idx), dev(off), None)
    hfeat = np.maximum(rng.standard_normal((n, heads * dim)), 0).astype(np.float32)
    a_src = (rng.standard_normal((heads, dim)) * 0.5).astype(np.float32)
    a_dst = (rng.standard_normal((heads, dim)) * 0.5).astype(np.float32)
    got = host(cuda.gat_aggregate(dev(hfeat), dev(a_src), dev(a_dst), csc, heads))
    want = oracle.gat_aggregate(hfeat, a_src, a_dst, idx, off, heads, dim)
    assert np.abs(got - want).max() / np.abs(hfeat).max() <= 1e-5
    assert not got[0].any() and not got[9].any()          # destinations without in-edges
    assert np.array_equal(got, host(cuda.gat_aggregate(dev(hfeat), dev(a_src), dev(a_dst), csc, heads)))


def test_fused_attention_equals_reference_pipeline(cuda, oracle):
    """Single head: the fused kernel against the reference's own op-by-op pipeline run on the CPU."""
    rng = np.random.default_rng(5)
    n, c = 400, 8
    ei = rng.integers(0, n, size=(2, 5000)).astype(np.int32)
    nei, nw = oracle.gcn_norm(ei, None, n)
    idx, off, _ = oracle.coo_to_csc(nei, nw, n)
    hfeat = np.maximum(rng.standard_normal((n, c)), 0).astype(np.float32)
    a = (rng.standard_normal(2 * c) * 0.3).astype(np.float32)
    impl = "ref" if oracle.have_ref() else "port"
    want = oracle.gat_unfused(hfeat, a, idx, off, impl)
    csc = cuda.CSC(dev(idx), dev(off), None)
    got = host(cuda.gat_aggregate(dev(hfeat), dev(a[:c]), dev(a[c:]), csc, 1))
    assert np.abs(got - want).max() <= 1e-5 * (np.abs(hfeat).max() + 1)


def test_fused_attention_backward_equals_reference_pairings(cuda, oracle):
    """Single head: gradients of the fused kernel against the reference's own backward pairings
    (ScatterToVertex.grad, EdgeSoftmax.grad, ScatterToEdge.grad) composed on the CPU."""
    rng = np.random.default_rng(15)
    n, c = 500, 8
    ei = rng.integers(0, n, size=(2, 6000)).astype(np.int32)
    nei, nw = oracle.gcn_norm(ei, None, n)
    idx, off, _ = oracle.coo_to_csc(nei, nw, n)
    hfeat = rng.standard_normal((n, c)).astype(np.float32)
    a = (rng.standard_normal(2 * c) * 0.3).astype(np.float32)
    g = rng.standard_normal((n, c)).astype(np.float32)
    impl = "ref" if oracle.have_ref() else "port"
    want_h, want_a = oracle.gat_unfused_backward(hfeat, a, idx, off, g, impl)
    csc = cuda.CSC(dev(idx), dev(off), None)
    h, a_s, a_d = dev(hfeat).requires_grad_(True), dev(a[:c]).requires_grad_(True), dev(a[c:]).requires_grad_(True)
    cuda.gat_aggregate(h, a_s, a_d, csc, 1).backward(dev(g))
    assert np.abs(host(h.grad) - want_h).max() <= 2e-5 * np.abs(want_h).max()
    got_a = np.concatenate([host(a_s.grad).reshape(-1), host(a_d.grad).reshape(-1)])
    assert np.abs(got_a - want_a).max() <= 2e-5 * np.abs(want_a).max()


def test_gat_layer_fused_and_unfused_agree(cuda):
    from jittorgeometric_b200 import nn
    torch.manual_seed(0)
    rng = np.random.default_rng(6)
    n = 500
    idx, off = random_csc(rng, n, 6000)
    csc = cuda.CSC(dev(idx), dev(off), None)
    layer = nn.GATConv(40, 64, 0, heads=8, tf32=False).cuda()
    x = torch.randn(n, 40, device="cuda")
    with torch.no_grad():
        fused = layer(x, csc)
        unfused = layer.propagate_unfused(torch.relu(x @ layer.weight), csc)
    assert (fused - unfused).abs().max().item() <= 1e-5 * (unfused.abs().max().item() + 1)
    # training: the fused backward against autograd through the per-edge operators
    target = torch.randn(n, 64, device="cuda")
    grads = []
    for fused in (True, False):
        layer.fused = fused
        layer.zero_grad()
        xg = x.clone().requires_grad_(True)
        (layer(xg, csc) * target).sum().backward()
        grads.append((xg.grad, layer.weight.grad.clone(), layer.edge_weight.grad.clone()))
    for a, b in zip(*grads):
        assert (a - b).abs().max().item() <= 2e-4 * (b.abs().max().item() + 1e-30)


def attention_truth(h, a_src, a_dst, idx, off, slope=0.2):
    """Differentiable float64 restatement of the edge phase with plain tensor operations."""
    n, heads, dim = h.shape[0], a_src.shape[0], a_src.shape[1]
    seg = torch.repeat_interleave(torch.arange(n, device=h.device), (off[1:] - off[:-1]).long())
    e_s, e_d = h[idx.long()].view(-1, heads, dim), h[seg].view(-1, heads, dim)
    m = torch.nn.functional.leaky_relu((e_s * a_src).sum(-1) + (e_d * a_dst).sum(-1), slope)
    top = torch.full((n, heads), -float("inf"), dtype=h.dtype, device=h.device).scatter_reduce(
        0, seg.view(-1, 1).expand(-1, heads), m, "amax")
    p = torch.exp(m - top[seg])
    alpha = p / torch.zeros((n, heads), dtype=h.dtype, device=h.device).index_add(0, seg, p)[seg]
    return torch.zeros_like(h).index_add(0, seg, (e_s * alpha.unsqueeze(-1)).reshape(-1, heads * dim))


@pytest.mark.parametrize("heads,dim", [(8, 8), (1, 64), (1, 8), (2, 4), (4, 16), (1, 128), (1, 4)])
def test_fused_attention_backward(cuda, heads, dim):
    """Gradients of the fused kernel with respect to h, a_src and a_dst against float64 autograd;
    hubs on both sides (destinations and sources with thousands of edges), empty rows, negative and
    positive logits (both branches of the leaky slope), identical results on a second run."""
    rng = np.random.default_rng(1000 + heads * 10 + dim)
    n, c = 2500, heads * dim
    dst = np.concatenate([rng.integers(10, n, size=30000), np.full(9000, 3), np.full(5000, 1500),
                          rng.integers(10, n, size=25000)])
    # source 42 has more than two pieces of 8192 out-edges, source 1500 a single piece
    src = np.concatenate([rng.integers(0, n, size=30000 + 9000 + 5000), np.full(20000, 42), np.full(5000, 1500)])
    order = np.argsort(dst, kind="stable")
    idx = src[order].astype(np.int32)
    off = np.concatenate([[0], np.cumsum(np.bincount(dst, minlength=n))]).astype(np.int32)
    csc = cuda.CSC(dev(idx), dev(off), None)
    h0 = rng.standard_normal((n, c)).astype(np.float32)
    a0 = (rng.standard_normal((2, heads, dim)) * 0.5).astype(np.float32)
    g0 = rng.standard_normal((n, c)).astype(np.float32)

    def run():
        h, a_s, a_d = dev(h0).requires_grad_(True), dev(a0[0]).requires_grad_(True), dev(a0[1]).requires_grad_(True)
        out = cuda.gat_aggregate(h, a_s, a_d, csc, heads)
        out.backward(dev(g0))
        return host(out), host(h.grad), host(a_s.grad), host(a_d.grad)

    got = run()
    hd, asd, add_ = dev(h0).double().requires_grad_(True), dev(a0[0]).double().requires_grad_(True), dev(a0[1]).double().requires_grad_(True)
    want_out = attention_truth(hd, asd, add_, dev(idx), dev(off))
    want_out.backward(dev(g0).double())
    want = (host(want_out), host(hd.grad), host(asd.grad), host(add_.grad))
    for name, a, b in zip(("out", "grad_h", "grad_a_src", "grad_a_dst"), got, want):
        assert a.shape == b.shape, name
        assert np.abs(a - b).max() <= 2e-5 * np.abs(b).max() + 1e-30, name
    again = run()
    for a, b in zip(got, again):
        assert np.array_equal(a, b)


def test_spmm_front_ends(cuda, oracle):
    d = load("ref_test_mp_spmm")
    csr = cuda.CSR(dev(d["column_indices"]), dev(d["row_offset"]), dev(d["csr_weight"]))
    x = dev(d["x"])
    assert np.array_equal(host(cuda.SpmmCsr(x, csr)), d["out_csc"])               # trans_A=True: A^T x
    assert np.array_equal(host(cuda.SpmmCsr(x, csr, trans_A=False)), d["out_csr"])
    assert np.array_equal(host(cuda.SpmmCoo(x, dev(d["edge_index"]), dev(d["edge_weight"]))), d["out_csc"])
    d = load("ref_test_spmm")
    csr = cuda.CSR(dev(d["column_indices"]), dev(d["row_offset"]), dev(d["csr_weight"]))   # int64, as the reference test
    assert np.array_equal(host(cuda.SpmmCsr(dev(d["csr_x"]), csr)), d["csr_out"])
    assert np.array_equal(host(cuda.SpmmCoo(dev(d["coo_x"]), dev(d["edge_index"]), dev(d["edge_weight"]))), d["coo_out"])


def test_gcn_norm_coo_list(cuda, oracle):
    from jittorgeometric_b200 import nn
    rng = np.random.default_rng(8)
    n, E = 3000, 40000
    ei = np.minimum((rng.random((2, E)) ** 2 * n).astype(np.int32), n - 1)
    for w in (None, rng.random(E).astype(np.float32) + 0.1):
        gei, gw = nn.gcn_norm(dev(ei), None if w is None else dev(w), n)
        wei, ww = oracle.gcn_norm(ei, w, n)
        assert np.array_equal(host(gei), wei)
        assert np.abs(host(gw).view(np.int32).astype(np.int64) - ww.view(np.int32).astype(np.int64)).max() <= 4


def test_gcn_norm_without_self_loops(cuda, oracle):
    """``gcn_norm(add_self_loops=False)`` (nn/conv/gcn_conv.py:18-37): the list as given, weights scaled by
    the weighted in-degrees; also through the fused conversion."""
    from jittorgeometric_b200 import nn
    rng = np.random.default_rng(9)
    n, E = 2000, 30000
    ei = np.minimum((rng.random((2, E)) ** 2 * n).astype(np.int32), n - 1)
    ei[1, :n] = np.arange(n)                                   # every node has an in-edge: finite weights
    for w in (None, rng.random(E).astype(np.float32) + 0.1):
        gei, gw = nn.gcn_norm(dev(ei), None if w is None else dev(w), n, add_self_loops=False)
        wei, ww = oracle.gcn_norm(ei, w, n, add_self_loops=False)
        assert np.array_equal(host(gei), ei) and np.array_equal(wei, ei)
        assert np.abs(host(gw).view(np.int32).astype(np.int64) - ww.view(np.int32).astype(np.int64)).max() <= 4
        csc, csr = cuda.gcn_norm_csc_csr(dev(ei), None if w is None else dev(w), n, add_self_loops=False)
        ri, co, cw = oracle.coo_to_csc(wei, ww, n)
        assert np.array_equal(host(csc.row_indices), ri) and np.array_equal(host(csc.column_offset), co)
        assert np.abs(host(csc.edge_weight).view(np.int32).astype(np.int64) - cw.view(np.int32).astype(np.int64)).max() <= 4
        ci, ro, rw = oracle.coo_to_csr(wei, ww, n)
        assert np.array_equal(host(csr.column_indices), ci) and np.array_equal(host(csr.row_offset), ro)


def test_gcn_layers_on_citation_graph(cuda, oracle):
    """Two-layer GCN forward + loss + backward on the 2708-node instance (layers 1433 -> 256 -> 7, fp32
    transform): the forward and all five gradients (both weights, both biases, the input) against
    float64 and against the reference recipe (numpy fp32 products + the checker's aggregation)."""
    from jittorgeometric_b200 import nn, synth
    d = load("citation_2708")
    n = 2708
    csc, csr = cuda.gcn_norm_csc_csr(dev(d["edge_index"]), None, n)
    x = synth.sparse_binary_features(n, 1433, 18, seed=3).numpy()
    torch.manual_seed(1)
    c1, c2 = nn.GCNConv(1433, 256, tf32=False).cuda(), nn.GCNConv(256, 7, tf32=False).cuda()
    with torch.no_grad():                                       # non-zero biases, so that their path is exercised
        c1.bias.copy_(torch.linspace(-0.05, 0.05, 256)); c2.bias.copy_(torch.linspace(-0.1, 0.1, 7))
    labels = torch.randint(7, (n,), generator=torch.Generator().manual_seed(2)).cuda()
    xt = dev(x).requires_grad_(True)
    out = c2(torch.relu(c1(xt, csc, csr)), csc, csr)
    loss = torch.nn.functional.cross_entropy(out, labels)
    loss.backward()
    ci, co, cw = host(csc.row_indices), host(csc.column_offset), host(csc.edge_weight)
    ri, ro, rw = host(csr.column_indices), host(csr.row_offset), host(csr.edge_weight)
    W1, b1, W2, b2, lab = host(c1.weight), host(c1.bias), host(c2.weight), host(c2.bias), host(labels)

    # float64 truth by dense autograd
    A = torch.zeros((n, n), dtype=torch.float64)
    A.index_put_((torch.from_numpy(np.repeat(np.arange(n), np.diff(co))), torch.from_numpy(ci.astype(np.int64))),
                 torch.from_numpy(cw.astype(np.float64)), accumulate=True)
    P = [torch.from_numpy(a.astype(np.float64)).requires_grad_(True) for a in (x, W1, b1, W2, b2)]
    h64 = torch.relu(A @ (P[0] @ P[1]) + P[2])
    z64 = A @ (h64 @ P[3]) + P[4]
    l64 = torch.nn.functional.cross_entropy(z64, torch.from_numpy(lab))
    g64 = [g.numpy() for g in torch.autograd.grad(l64, P)]
    # error scale of the forward: the same network on absolute values
    Aabs = A.abs()
    s1 = Aabs @ (torch.from_numpy(np.abs(x).astype(np.float64)) @ P[1].detach().abs()) + P[2].detach().abs()
    s2 = (Aabs @ (s1 @ P[3].detach().abs()) + P[4].detach().abs()).numpy()
    assert (np.abs(host(out) - z64.detach().numpy()) / s2).max() <= 1e-5
    assert abs(float(loss.detach()) - float(l64.detach())) <= 1e-5 * abs(float(l64.detach()))

    # the reference recipe in fp32: numpy products, the checker's aggregation (CSC forward, CSR backward)
    h1 = oracle.aggregate((x @ W1).astype(np.float32), ci, co, cw) + b1
    hr = np.maximum(h1, 0)
    z = oracle.aggregate((hr @ W2).astype(np.float32), ci, co, cw) + b2
    p = np.exp(z - z.max(1, keepdims=True)); p /= p.sum(1, keepdims=True)
    gz = p.copy(); gz[np.arange(n), lab] -= 1; gz /= n
    g2 = oracle.aggregate(gz.astype(np.float32), ri, ro, rw)
    gh1 = ((g2 @ W2.T) * (h1 > 0)).astype(np.float32)
    g1 = oracle.aggregate(gh1, ri, ro, rw)
    want = {"x": g1 @ W1.T, "W1": x.T @ g1, "b1": gh1.sum(0), "W2": hr.T @ g2, "b2": gz.sum(0)}
    have = {"x": host(xt.grad), "W1": host(c1.weight.grad), "b1": host(c1.bias.grad), "W2": host(c2.weight.grad),
            "b2": host(c2.bias.grad)}
    truth = dict(zip(("x", "W1", "b1", "W2", "b2"), g64))
    assert np.abs(host(out) - z).max() <= 1e-5 * np.abs(z).max()
    for name in ("x", "W1", "b1", "W2", "b2"):
        top = np.abs(truth[name]).max()
        assert have[name].shape == truth[name].shape, name
        assert np.abs(have[name] - truth[name]).max() <= 1e-5 * top, (name, "vs float64")
        assert np.abs(have[name] - want[name]).max() <= 2e-5 * top, (name, "vs the reference recipe in fp32")


def test_sgconv_appnp_against_checker(cuda, oracle):
    """``SGConv`` (nn/conv/sg_conv.py:62-70) and ``APPNP`` (nn/conv/appnp_conv.py:42-52) against the same
    compositions built from the CPU checker's aggregation."""
    from jittorgeometric_b200 import nn
    d = load("citation_2708")
    n = 2708
    csc, csr = cuda.gcn_norm_csc_csr(dev(d["edge_index"]), None, n)
    ci, co, cw = host(csc.row_indices), host(csc.column_offset), host(csc.edge_weight)
    f = np.random.default_rng(4).standard_normal((n, 16)).astype(np.float32)
    _, scale = oracle.aggregate_f64(np.abs(f), ci, co, cw)
    with torch.no_grad():
        torch.manual_seed(3)
        sg = nn.SGConv(16, 5, K=2, tf32=False).cuda()
        a2 = oracle.aggregate(oracle.aggregate(f, ci, co, cw), ci, co, cw)
        want = a2 @ host(sg.lin.weight).T + host(sg.lin.bias)
        assert np.abs(host(sg(dev(f), csc, csr)) - want).max() <= 1e-5 * (np.abs(a2).max() * 16 + 1)
        sg.lin.tf32 = True                                       # the default: TF32 products on the tensor cores
        assert np.abs(host(sg(dev(f), csc, csr)) - want).max() <= 2e-3 * (np.abs(a2).max() * 16 + 1)
        ap = nn.APPNP(K=3, alpha=0.1)
        want = f
        for _ in range(3):
            want = oracle.aggregate(want, ci, co, cw) * np.float32(0.9) + np.float32(0.1) * f
        assert (np.abs(host(ap(dev(f), csc, csr)) - want) / (scale + np.abs(f) + 1e-30)).max() <= 1e-5


def test_gatconv_takes_the_reference_constructor_call(cuda, oracle):
    """The reference's own call, ``GATConv(num_features, 128, e_num, cached=True, normalize=...)``
    (examples/gat_example.py:96-99, nn/conv/gat_conv.py:27-30): ``e_num`` is accepted and unused, the
    layer is single-head, and its forward equals the reference's op-by-op pipeline."""
    from jittorgeometric_b200 import nn
    d = load("citation_2708")
    n = 2708
    csc = cuda.cootocsc(dev(d["edge_index"]), None, n)
    e_num = d["edge_index"].shape[1]
    torch.manual_seed(5)
    conv1 = nn.GATConv(64, 128, e_num, cached=True, normalize=True).cuda()
    conv2 = nn.GATConv(128, 7, e_num, cached=True, normalize=True).cuda()
    assert conv1.heads == 1 and conv2.heads == 1 and conv1.tf32
    x = np.random.default_rng(6).standard_normal((n, 64)).astype(np.float32)
    with torch.no_grad():
        y1 = conv1(dev(x), csc)
        y2 = conv2(torch.relu(y1), csc)
    assert y1.shape == (n, 128) and y2.shape == (n, 7)
    ri, co = host(csc.row_indices), host(csc.column_offset)
    h = np.maximum(x @ host(conv1.weight), 0).astype(np.float32)
    want = oracle.gat_unfused(h, host(conv1.edge_weight)[:, 0], ri, co)
    assert np.abs(host(y1) - want).max() <= 2e-3 * np.abs(want).max()          # default transform: TF32 products on tcgen05
    conv1.tf32 = False                                                          # fp32 transform: the 1e-5 bar
    with torch.no_grad():
        y1 = conv1(dev(x), csc)
    assert np.abs(host(y1) - want).max() <= 1e-5 * np.abs(want).max() + 1e-6
    with pytest.raises(TypeError):
        nn.GATConv(64, 128)                                    # e_num is positional and required, as in the reference
