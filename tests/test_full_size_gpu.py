"""Full-size workloads checked through size-independent properties (the CPU checker cannot finish
these sizes in seconds): conversion at 268 M edges, SpMM at 125 M nonzeros, attention at 114.6 M
edges.  Needs about 20 GB of device memory."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _big_enough():
    return torch.cuda.is_available() and torch.cuda.get_device_properties(0).total_memory > 60e9


@pytest.fixture(scope="module")
def conv24(cuda):
    if not _big_enough():
        pytest.skip("needs a large GPU")
    from jittorgeometric_b200 import synth
    ei, n = synth.rmat_coo_shuffled(24, 16, 20261125 + 3, device="cuda")
    csc, csr = cuda.gcn_norm_csc_csr(ei, None, n)
    return ei, n, csc, csr


def test_conversion_scale24_properties(cuda, oracle, conv24):
    ei, n, csc, csr = conv24
    src, dst = ei[0].long(), ei[1].long()
    keep = src != dst
    E = int(keep.sum()) + n
    for idx, off, key_in, other_in in ((csc.row_indices, csc.column_offset, dst, src),
                                       (csr.column_indices, csr.row_offset, src, dst)):
        assert idx.numel() == E and int(off[0]) == 0 and int(off[-1]) == E
        deg = off[1:] - off[:-1]
        assert int(deg.min()) >= 1                                   # every node has its loop
        want_deg = torch.bincount(key_in[keep], minlength=n) + 1
        assert torch.equal(deg.long(), want_deg)                     # offsets = histogram of the keys
        last = idx[(off[1:] - 1).long()]
        assert torch.equal(last.long(), torch.arange(n, device="cuda"))   # the appended loop closes every row
        # the multiset of (key, other) pairs is preserved: two order-independent checksums
        rows = torch.repeat_interleave(torch.arange(n, device="cuda"), deg.long())
        got1 = int((rows * 1000003 + idx.long()).sum() % (2**61 - 1))
        k2 = torch.cat([key_in[keep], torch.arange(n, device="cuda")])
        o2 = torch.cat([other_in[keep], torch.arange(n, device="cuda")])
        assert got1 == int((k2 * 1000003 + o2).sum() % (2**61 - 1))
        got2 = int(((rows ^ (idx.long() << 7)) % 998244353).sum())
        assert got2 == int(((k2 ^ (o2 << 7)) % 998244353).sum())
    # stable order inside rows: 200 random rows against the sequential CPU checker
    rng = np.random.default_rng(0)
    pick = rng.integers(0, n, size=200)
    src_h, dst_h = ei[0].cpu().numpy(), ei[1].cpu().numpy()
    off_h = csc.column_offset.cpu().numpy()
    idx_h = csc.row_indices.cpu().numpy()
    for v in pick:
        sel = (dst_h == v) & (src_h != v)
        want = np.concatenate([src_h[sel], [v]])
        assert np.array_equal(idx_h[off_h[v]:off_h[v + 1]], want)
    # weights: 1/sqrt(deg[src]*deg[dst]) within a few ulp
    deg_f = (csc.column_offset[1:] - csc.column_offset[:-1]).double()
    rows = torch.repeat_interleave(torch.arange(n, device="cuda"), (csc.column_offset[1:] - csc.column_offset[:-1]).long())
    want_w = (1.0 / torch.sqrt(deg_f[csc.row_indices.long()] * deg_f[rows])).float()
    assert torch.allclose(csc.edge_weight, want_w, rtol=5e-7, atol=0)


def test_conversion_scale24_is_reproducible(cuda, conv24):
    ei, n, csc, _ = conv24
    again, _ = cuda.gcn_norm_csc_csr(ei, None, n, want_csr=False)
    assert torch.equal(again.row_indices, csc.row_indices) and torch.equal(again.edge_weight, csc.edge_weight)


def test_spmm_scale21_linearity_and_row_sums(cuda):
    if not _big_enough():
        pytest.skip("needs a large GPU")
    from jittorgeometric_b200 import synth
    ei, n = synth.rmat_graph(21, 32, 20261125 + 1, device="cuda")
    csc, _ = cuda.gcn_norm_csc_csr(ei, None, n, want_csr=False)
    nnz = csc.row_indices.numel()
    plan = cuda.ops.SpmmPlan(csc.column_offset, nnz)
    agg = lambda x: cuda.ops.segment_aggregate(x, csc.row_indices, csc.column_offset, csc.edge_weight, plan=plan)
    g = torch.Generator(device="cuda").manual_seed(1)
    for f in (32, 128):
        x = torch.randn((n, f), device="cuda", generator=g)
        y = torch.randn((n, f), device="cuda", generator=g)
        ax, ay, axy = agg(x), agg(y), agg(x + 2 * y)
        scale = agg(x.abs() + 2 * y.abs()) + 1e-30               # sum |w x| bound (weights are positive)
        assert float(((axy - (ax + 2 * ay)).abs() / scale).max()) <= 1e-5
        assert torch.equal(agg(x), ax)                             # run-to-run identical
    # constant features: every output row is the row sum of the weights, hub rows included
    ones = torch.ones((n, 32), device="cuda")
    rs = agg(ones)
    seg = torch.repeat_interleave(torch.arange(n, device="cuda"), (csc.column_offset[1:] - csc.column_offset[:-1]).long())
    want = torch.zeros(n, device="cuda", dtype=torch.float64).index_add_(0, seg, csc.edge_weight.double())
    assert float((rs[:, 0].double() - want).abs().max() / want.abs().max()) <= 1e-5
    assert torch.equal(rs[:, 0], rs[:, 31])


def test_attention_full_size_convexity(cuda):
    if not _big_enough():
        pytest.skip("needs a large GPU")
    from jittorgeometric_b200 import synth
    n, H, D = 232965, 8, 8
    rows, off = synth.lognormal_degree_csc(n, 114_600_000, 20261125 + 3, device="cuda")
    csc = cuda.CSC(rows, off, None)
    g = torch.Generator(device="cuda").manual_seed(2)
    a_src = torch.randn((H, D), device="cuda", generator=g) * 0.3
    a_dst = torch.randn((H, D), device="cuda", generator=g) * 0.3
    # constant rows: attention weights sum to one, so the output equals the constant
    c = torch.rand(H * D, device="cuda", generator=g) + 0.5
    h = c.repeat(n, 1).contiguous()
    out = cuda.gat_aggregate(h, a_src, a_dst, csc, H)
    # numerator and denominator are fp32 sums of up to ~60 000 terms each (the largest segments);
    # their rounding errors do not cancel exactly: a few 1e-5 relative, as a sequential fp32 sum has
    assert float(((out - c).abs() / c).max()) <= 1e-4
    # general rows: every output lies inside the range of the source rows of its segment (here: global range)
    h = torch.relu(torch.randn((n, H * D), device="cuda", generator=g))
    out = cuda.gat_aggregate(h, a_src, a_dst, csc, H)
    assert torch.isfinite(out).all()
    assert float(out.min()) >= -1e-6 and float(out.max()) <= float(h.max()) * (1 + 1e-5)
    assert torch.equal(out, cuda.gat_aggregate(h, a_src, a_dst, csc, H))
