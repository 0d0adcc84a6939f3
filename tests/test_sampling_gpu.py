"""GPU parity of the neighbour-sampling operators and the mini-batch sampler against the CPU
checker: deterministic parts (counts, full copies, CSC->CSR, weights, the merged subgraph) bit-exact,
the random draw through the properties every valid sample has."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.detach().cpu().numpy()


def random_csc(rng, n, E, hub=None):
    dst = rng.integers(0, n, size=E)
    if hub:
        dst = np.concatenate([dst, np.full(hub, 5)])
    src = rng.integers(0, n, size=len(dst))
    order = np.argsort(dst, kind="stable")
    off = np.concatenate([[0], np.cumsum(np.bincount(dst, minlength=n))]).astype(np.int32)
    return src[order].astype(np.int32), off


def test_reference_fixtures(cuda, oracle):
    """The inputs of the reference's own operator tests (tests/test_gpuinitco.py:15-22,
    tests/test_csctocsr.py:25-35, tests/test_getweight.py:25-33) and the outputs they state."""
    from jittorgeometric_b200 import sampling as S
    ids = np.arange(4, dtype=np.int32)
    got = host(S.gpuinitco(4, 2, dev(ids), dev(np.array([0, 1, 3, 4, 5], np.int32))))
    assert got.tolist() == [0, 1, 2, 1, 1]
    ro, ci = S.csctocsr(dev(np.array([0, 0, 1, 2, 4], np.int32)), dev(np.array([0, 0, 1, 2], np.int32)), dev(ids), dev(ids))
    assert host(ro).tolist() == [0, 2, 3, 4, 4] and host(ci).tolist() == [1, 2, 3, 3]
    w = host(S.getweight(4, dev(ids), dev(ids), dev(np.array([0, 1, 2, 3, 4], np.int32)), dev(np.array([0, 0, 1, 2], np.int32))))
    want = np.array([1 / np.sqrt(2.0), 1 / np.sqrt(2.0), 1.0, 1.0], np.float32)
    assert np.array_equal(w, oracle.get_weight(4, ids, ids, np.array([0, 1, 2, 3, 4]), np.array([0, 0, 1, 2])))
    assert np.abs(w - want).max() <= 1e-7


@pytest.mark.parametrize("fanout", [3, 10, 40, -1, 1024])
def test_sampling_counts_and_draws(cuda, oracle, fanout):
    from jittorgeometric_b200 import sampling as S
    rng = np.random.default_rng(fanout + 5)
    n = 3000
    g_idx, g_off = random_csc(rng, n, 40000, hub=5000)
    dst = rng.permutation(n)[:1200].astype(np.int32)
    dst[0] = 5                                                    # the hub: 5000 or more in-edges
    counts = host(S.gpuinitco(len(dst), fanout, dev(dst), dev(g_off)))
    if fanout >= 0:
        assert np.array_equal(counts, oracle.sample_counts(dst, g_off, fanout))
    off = host(S.layer_offsets(fanout, dev(dst), dev(g_off)))
    deg = g_off[dst + 1] - g_off[dst]
    want = deg if fanout < 0 else np.minimum(deg, fanout)
    assert np.array_equal(off, np.concatenate([[0], np.cumsum(want)]).astype(np.int32))
    got = host(S.sampleprocessing(fanout, dev(dst), dev(off), dev(g_off), dev(g_idx), seed=11))
    assert oracle.check_sample(fanout, dst, off, got, g_off, g_idx) is None
    again = host(S.sampleprocessing(fanout, dev(dst), dev(off), dev(g_off), dev(g_idx), seed=11))
    assert np.array_equal(got, again)                             # same seed, same sample
    if 0 <= fanout < deg.max():
        other = host(S.sampleprocessing(fanout, dev(dst), dev(off), dev(g_off), dev(g_idx), seed=12))
        assert not np.array_equal(got, other)
        assert oracle.check_sample(fanout, dst, off, other, g_off, g_idx) is None
    if oracle.have_ref() and fanout >= 0:                         # the reference's own sampler passes the same check
        ref = oracle.sample_reference(fanout, dst, off, g_off, g_idx)
        assert oracle.check_sample(fanout, dst, off, ref, g_off, g_idx) is None


def test_sampling_rejects_foreign_offsets(cuda):
    from jittorgeometric_b200 import sampling as S
    g_idx, g_off = random_csc(np.random.default_rng(1), 50, 600)
    dst = np.arange(20, dtype=np.int32)
    off = host(S.layer_offsets(3, dev(dst), dev(g_off)))
    with pytest.raises(RuntimeError):
        S.sampleprocessing(5, dev(dst), dev(off), dev(g_off), dev(g_idx))      # offsets were built for fanout 3
    with pytest.raises(RuntimeError):
        S.sampleprocessing(2000, dev(dst), dev(off), dev(g_off), dev(g_idx))   # beyond the supported fanout


def test_draws_are_uniform(cuda):
    """One destination with 40 in-edges, fanout 8, 4000 seeds: every position is drawn in about a
    fifth of the samples (binomial standard deviation 25 draws; the bound is more than five of them)."""
    from jittorgeometric_b200 import sampling as S
    g_off = np.array([0, 40], np.int32)
    g_idx = np.arange(40, dtype=np.int32)
    dst = np.zeros(1, np.int32)
    off = dev(np.array([0, 8], np.int32))
    hits = np.zeros(40)
    for seed in range(4000):
        got = host(S.sampleprocessing(8, dev(dst), off, dev(g_off), dev(g_idx), seed=seed, total=8))
        assert len(set(got.tolist())) == 8
        hits[got] += 1
    assert np.abs(hits - 800).max() < 140


def test_csc_to_csr_over_id_lists(cuda, oracle):
    """Arbitrary destination ids, a source list that misses some ids (their entries are dropped),
    stable order inside rows: bit-exact with the checker and with the reference's CPU body."""
    from jittorgeometric_b200 import sampling as S
    rng = np.random.default_rng(3)
    n_dst, universe = 400, 5000
    row_idx, off = random_csc(rng, n_dst, 6000)
    row_idx = rng.integers(0, universe, size=len(row_idx)).astype(np.int32)
    dst_ids = rng.permutation(universe)[:n_dst].astype(np.int32)
    src_ids = rng.permutation(universe)[:3000].astype(np.int32)            # about 40 % of the entries have no row
    ro, ci = S.csctocsr(dev(off), dev(row_idx), dev(dst_ids), dev(src_ids))
    want_ro, want_ci = oracle.csc_to_csr(off, row_idx, dst_ids, src_ids)
    assert np.array_equal(host(ro), want_ro) and np.array_equal(host(ci), want_ci)
    assert 0 < len(want_ci) < len(row_idx)
    if oracle.have_ref():
        ref_ro, ref_ci = oracle.csc_to_csr(off, row_idx, dst_ids, src_ids, "ref")
        assert np.array_equal(want_ro, ref_ro) and np.array_equal(want_ci, ref_ci)
    ro, ci = S.csctocsr(dev(np.zeros(1, np.int32)), dev(np.zeros(0, np.int32)), dev(np.zeros(0, np.int32)), dev(src_ids[:5]))
    assert host(ro).tolist() == [0] * 6 and ci.numel() == 0


def test_degree_weights(cuda, oracle):
    from jittorgeometric_b200 import sampling as S
    rng = np.random.default_rng(4)
    n = 2000
    idx, off = random_csc(rng, n, 30000, hub=4000)
    ids = np.arange(n, dtype=np.int32)
    got = host(S.getweight(n, dev(ids), dev(ids), dev(off), dev(idx)))
    assert np.array_equal(got, oracle.get_weight(n, ids, ids, off, idx))
    if oracle.have_ref():
        assert np.array_equal(got, oracle.get_weight(n, ids, ids, off, idx, "ref"))
    # a layer: 300 destinations with their own ids
    dst = rng.permutation(n)[:300].astype(np.int32)
    l_off = np.concatenate([[0], np.cumsum(rng.integers(0, 9, size=300))]).astype(np.int32)
    l_idx = rng.integers(0, n, size=l_off[-1]).astype(np.int32)
    got = host(S.getweight(n, dev(dst), dev(ids), dev(l_off), dev(l_idx)))
    assert np.array_equal(got, oracle.get_weight(n, dst, ids, l_off, l_idx))


def merge_layers_numpy(layers):
    """The reference's merge of sampled layers into one local graph, restated with its own
    dictionary loops (examples/minibatch_example.py:281-340)."""
    all_nodes = np.unique(np.concatenate([np.concatenate([d, idx]) for d, off, idx in layers]))
    g2l = -np.ones(all_nodes.max() + 1, np.int64)
    g2l[all_nodes] = np.arange(len(all_nodes))
    adj = {}
    for d, off, idx in layers:
        for i, v in enumerate(g2l[d]):
            adj.setdefault(int(v), []).extend(g2l[idx[off[i]: off[i + 1]]].tolist())
    col_off, rows = [0], []
    for v in range(len(all_nodes)):
        rows.extend(adj.get(v, []))
        col_off.append(len(rows))
    return all_nodes.astype(np.int32), np.array(col_off, np.int32), np.array(rows, np.int32)


def test_sampled_subgraph_equals_reference_merge(cuda, oracle):
    from jittorgeometric_b200 import sampling as S
    rng = np.random.default_rng(8)
    n = 5000
    g_idx, g_off = random_csc(rng, n, 60000, hub=3000)
    batch = rng.permutation(n)[:256].astype(np.int32)
    layers = S.sample_layers([10, 5], dev(batch), dev(g_off), dev(g_idx), seed=3)
    assert len(layers) == 2 and np.array_equal(host(layers[1].dst), np.unique(host(layers[0].row_indices)))
    ssg = S.build_subgraph(layers, n)
    l2g, col_off, rows = merge_layers_numpy([(host(l.dst), host(l.column_offset), host(l.row_indices)) for l in layers])
    assert np.array_equal(host(ssg.local2global), l2g) and ssg.num_nodes == len(l2g)
    assert np.array_equal(host(ssg.column_offset), col_off) and np.array_equal(host(ssg.row_indices), rows)
    ids = np.arange(len(l2g), dtype=np.int32)
    want_ro, want_ci = oracle.csc_to_csr(col_off, rows, ids, ids)
    assert np.array_equal(host(ssg.row_offset), want_ro) and np.array_equal(host(ssg.column_indices), want_ci)
    assert np.array_equal(host(ssg.csc_edge_weight), oracle.get_weight(len(l2g), ids, ids, col_off, rows))
    assert np.array_equal(host(ssg.csr_edge_weight), oracle.get_weight(len(l2g), ids, ids, want_ro, want_ci))


def test_neighbor_loader_trains_a_layer(cuda):
    """Mini-batches from the loader feed the aggregation layers: every seed node is visited once per
    epoch, the same seed repeats the epoch, and a GCN layer runs forward and backward on a batch."""
    from jittorgeometric_b200 import nn, sampling as S
    rng = np.random.default_rng(9)
    n, f = 4000, 32
    g_idx, g_off = random_csc(rng, n, 50000)
    feat = torch.randn(n, f, device="cuda")
    label = torch.randint(0, 4, (n,), device="cuda")
    seeds = dev(rng.permutation(n)[:1000].astype(np.int32))

    def epoch(seed):
        loader = S.NeighborLoader(seeds, [8, 4], 256, dev(g_off), dev(g_idx), feat, label, seed=seed)
        loader.reset()
        return loader, list(loader)

    loader, batches = epoch(1)
    assert len(loader) == 4 and len(batches) == 4
    seen = torch.cat([b.layer_graph[0].dst for b in batches])
    assert np.array_equal(np.sort(host(seen)), np.sort(host(seeds)))
    _, again = epoch(1)
    for a, b in zip(batches, again):
        assert torch.equal(a.row_indices, b.row_indices) and torch.equal(a.local2global, b.local2global)
        assert torch.equal(a.X, feat[a.local2global.long()]) and torch.equal(a.target_lab, label[a.local2global.long()])
    ssg = batches[0]
    layer = nn.GCNConv(f, 4).cuda()
    out = layer(ssg.X, ssg.csc, ssg.csr)
    loss = torch.nn.functional.cross_entropy(out, ssg.target_lab)
    loss.backward()
    assert torch.isfinite(loss) and torch.isfinite(layer.weight.grad).all() and layer.weight.grad.abs().sum() > 0


def test_sampling_edge_cases(cuda):
    """No destinations, destinations without in-edges, fanout 0: nothing is drawn and nothing breaks."""
    from jittorgeometric_b200 import sampling as S
    g_off = np.array([0, 0, 3, 3, 5], np.int32)              # nodes 0 and 2 have no in-edges
    g_idx = np.array([0, 2, 3, 1, 1], np.int32)
    empty = dev(np.zeros(0, np.int32))
    assert host(S.layer_offsets(3, empty, dev(g_off))).tolist() == [0]
    assert S.sampleprocessing(3, empty, dev(np.zeros(1, np.int32)), dev(g_off), dev(g_idx)).numel() == 0
    dst = np.array([0, 1, 2, 3], np.int32)
    off = host(S.layer_offsets(2, dev(dst), dev(g_off)))
    assert off.tolist() == [0, 0, 2, 2, 4]
    got = host(S.sampleprocessing(2, dev(dst), dev(off), dev(g_off), dev(g_idx), seed=4))
    assert set(got[:2]) <= {0, 2, 3} and len(set(got[:2])) == 2 and got[2:].tolist() == [1, 1]
    off0 = host(S.layer_offsets(0, dev(dst), dev(g_off)))
    assert off0.tolist() == [0, 0, 0, 0, 0]
    assert S.sampleprocessing(0, dev(dst), dev(off0), dev(g_off), dev(g_idx)).numel() == 0
    # a batch whose seeds have no in-edges at all: the subgraph is the seeds themselves, no entries
    ssg = S.sample_one([5, 5], dev(g_off), dev(g_idx), dev(np.array([0, 2], np.int32)))
    assert ssg.num_nodes == 2 and ssg.num_edges == 0 and host(ssg.column_offset).tolist() == [0, 0, 0]
    assert host(ssg.local2global).tolist() == [0, 2]


def test_sampling_golden_vectors(cuda):
    """The committed outputs of the reference's own compiled CPU bodies (tests/golden/ref_test_sampling.npz)."""
    import os
    from jittorgeometric_b200 import sampling as S
    d = dict(np.load(os.path.join(os.path.dirname(__file__), "golden", "ref_test_sampling.npz")))
    ro, ci = S.csctocsr(dev(d["l_column_offset"]), dev(d["l_row_indices"]), dev(d["l_dst"]), dev(d["l_src"]))
    assert np.array_equal(host(ro), d["l_row_offset"]) and np.array_equal(host(ci), d["l_column_indices"])
    w = S.getweight(4000, dev(d["l_dst"]), dev(d["l_src"]), dev(d["l_column_offset"]), dev(d["l_row_indices"]))
    assert np.array_equal(host(w), d["l_weight"])
    off = S.layer_offsets(3, dev(d["s_dst"]), dev(d["s_global_offset"]))
    assert np.array_equal(host(off), d["s_layer_offset"])
    got = S.sampleprocessing(3, dev(d["s_dst"]), off, dev(d["s_global_offset"]), dev(d["s_global_indices"]))
    assert np.array_equal(host(got), d["s_out"])
    assert host(S.gpuinitco(4, 2, dev(d["counts_dst"]), dev(d["counts_global_offset"]))).tolist() == d["counts_out"].tolist()


def test_from_nodes_and_to_nodes(cuda):
    """The inputs of the reference's tests/test_fromtonodes.py:12-26: neighbour lists concatenated in the
    order of the given nodes, duplicates kept."""
    col_offset, row_indices = dev(np.array([0, 2, 4, 5, 6, 7], np.int32)), dev(np.array([0, 3, 1, 4, 0, 4, 2], np.int32))
    row_offset, col_indices = dev(np.array([0, 2, 3, 4, 5, 7], np.int32)), dev(np.array([0, 2, 1, 4, 0, 1, 3], np.int32))
    nodes = dev(np.array([1, 2, 2, 4], np.int32))
    assert host(cuda.from_nodes(cuda.CSC(row_indices, col_offset, None), nodes)).tolist() == [1, 4, 0, 0, 2]
    assert host(cuda.to_nodes(cuda.CSR(col_indices, row_offset, None), nodes)).tolist() == [1, 4, 4, 1, 3]
    with pytest.raises(ValueError):
        cuda.from_nodes(None, nodes)
