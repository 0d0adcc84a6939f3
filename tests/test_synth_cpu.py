"""The per-shard graph generator of the multi-GPU benchmark against the whole-graph path: every
rank must end up with exactly its rows of the graph one GPU builds."""
import numpy as np
import torch


def test_shard_builder_equals_rows_of_the_whole_graph(oracle):
    from jittorgeometric_b200 import synth
    scale, ef, seed = 10, 8, 77
    ei, n = synth.rmat_graph(scale, ef, seed)
    nei, nw = oracle.gcn_norm(ei.numpy(), None, n)             # self-loops + normalisation, the reference's list order
    ri, co, cw = oracle.coo_to_csc(nei, nw, n)                 # the reference's stable CSC
    bounds = [0, 300, 700, n]
    shards = [synth.rmat_shard_csc(scale, ef, seed, lo, hi) for lo, hi in zip(bounds[:-1], bounds[1:])]
    deg = torch.cat([s[2] for s in shards])                    # what the ranks all-gather
    assert np.array_equal(deg.numpy(), np.diff(co))
    for (lo, hi), (idx, off, _) in zip(zip(bounds[:-1], bounds[1:]), shards):
        s, e = co[lo], co[hi]
        assert np.array_equal(idx.numpy(), ri[s:e])
        assert np.array_equal(off.numpy(), co[lo:hi + 1] - co[lo])
        w = synth.gcn_weights(idx, off, deg, lo).numpy()
        assert np.abs(w.view(np.int32).astype(np.int64) - cw[s:e].view(np.int32).astype(np.int64)).max() <= 4


def test_edge_stream_is_the_same_in_batches_and_whole():
    from jittorgeometric_b200 import synth
    a = synth.rmat_edges(8, 5000, 3, batch=1 << 24)
    b = [torch.cat(t) for t in zip(*synth.rmat_edge_batches(8, 5000, 3, batch=1 << 24))]
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
