"""Host side of the partitioned-graph format: explicit partition bounds, the chunk directory format
(save, memory-mapped load) and an uneven two-rank aggregation over gloo with the CPU checker as the
compute backend."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def reference_chunks(partition, edge_index, n, P, w, order=None):
    """Restatement of the reference partitioner (partition/distchunk_manager.py:63-157) with numpy and
    scipy, the node order inside a part pinned to the original order (``kind="stable"``) unless
    ``order`` gives it.  Pinned against the reference's own function by
    ``test_restatement_equals_the_reference_partitioner``."""
    from scipy.sparse import csc_matrix, csr_matrix
    order = np.argsort(partition, kind="stable") if order is None else order
    remap = np.zeros(n, np.int64)
    remap[order] = np.arange(n)
    ei = np.stack([remap[edge_index[0]], remap[edge_index[1]]])
    srt = np.lexsort((ei[1], ei[0]))
    ei, w = ei[:, srt], w[srt]
    offset = np.concatenate([[0], np.cumsum(np.bincount(partition, minlength=P))])
    out = []
    for p in range(P):
        s, e = offset[p], offset[p + 1]
        sel = (ei[1] >= s) & (ei[1] < e)
        cei, cw = ei[:, sel].copy(), w[sel]
        cei[1] -= s
        csr = csr_matrix((cw, (cei[0], cei[1])), shape=(n, e - s))
        csc = csc_matrix((cw, (cei[0], cei[1])), shape=(n, e - s))
        out.append(dict(edge_index=cei, edge_weight=cw, offset=offset, order=order, csr=csr, csc=csc, range=(s, e)))
    return out


def make_partitioned(seed, n, E, P):
    rng = np.random.default_rng(seed)
    pairs = np.unique(rng.integers(0, n, size=(E, 2)), axis=0)          # no duplicate edges: scipy would add them up
    edge_index = pairs.T.astype(np.int64)
    w = rng.random(edge_index.shape[1]).astype(np.float32)
    partition = rng.integers(0, P, size=n).astype(np.int32)
    partition[:P] = np.arange(P)                                          # no empty part
    return partition, edge_index, w


def chunk_from_reference(ref, p, P, n, feature):
    from jittorgeometric_b200.partition import DistChunk
    t = lambda a, dt: torch.from_numpy(np.ascontiguousarray(a).astype(dt))
    r = ref[p]
    s, e = r["range"]
    c = DistChunk(P, p, e - s, n, t(r["edge_index"], np.int32), t(r["offset"], np.int32), t(r["edge_weight"], np.float32),
                  local_feature=t(feature[r["order"]][s:e], np.float32), local_label=t(np.arange(s, e), np.int64), num_classes=3)
    c.set_csr(t(r["csr"].indices, np.int32), t(r["csr"].indptr, np.int32), t(r["csr"].data, np.float32))
    c.set_csc(t(r["csc"].indices, np.int32), t(r["csc"].indptr, np.int32), t(r["csc"].data, np.float32))
    c.set_chunk_csrs()
    return c


def test_chunk_directory_round_trip(tmp_path):
    from jittorgeometric_b200.partition import DistChunk, chunks_save, distributed_file, load_partition
    n, P = 60, 3
    partition, edge_index, w = make_partitioned(1, n, 400, P)
    feature = np.random.default_rng(2).standard_normal((n, 5)).astype(np.float32)
    ref = reference_chunks(partition, edge_index, n, P, w)
    chunks = [chunk_from_reference(ref, p, P, n, feature) for p in range(P)]
    chunks_save(chunks, str(tmp_path))
    for p in range(P):
        path = distributed_file(p, P, str(tmp_path))
        assert os.path.basename(path) == f"subgraph_{P}_of_{p}" and os.path.exists(os.path.join(path, "meta.json"))
        for mmap in (True, False):
            back = DistChunk.load(path, mmap=mmap)
            a = chunks[p]
            assert (back.chunks, back.chunk_id, back.v_num, back.global_v_num, back.num_classes) == (P, p, a.v_num, n, 3)
            for x, y in [(back.edge_index, a.edge_index), (back.edge_weight, a.edge_weight), (back.offset, a.offset),
                         (back.local_feature, a.local_feature), (back.local_label, a.local_label),
                         (back.CSR.column_indices, a.CSR.column_indices), (back.CSR.row_offset, a.CSR.row_offset),
                         (back.CSC.row_indices, a.CSC.row_indices), (back.CSC.edge_weight, a.CSC.edge_weight)]:
                assert torch.equal(x, y)
            assert back.local_masks["train"] is None
            # the per-source-rank blocks are slices of the CSR: together they hold every entry once
            assert sum(c.column_indices.numel() for c in back.chunk_CSR) == a.CSR.column_indices.numel()
            for q in range(P):
                lo, hi = int(a.offset[q]), int(a.offset[q + 1])
                blk = ref[p]["csr"][lo:hi]
                assert np.array_equal(back.chunk_CSR[q].row_offset.numpy(), blk.indptr)
                assert np.array_equal(back.chunk_CSR[q].column_indices.numpy(), blk.indices)
    # partition vectors: .npy and one-id-per-line text
    np.save(tmp_path / "part.npy", partition)
    np.savetxt(tmp_path / "graph.part.3", partition, fmt="%d")
    assert np.array_equal(load_partition(str(tmp_path / "part.npy")), partition)
    assert np.array_equal(load_partition(str(tmp_path / "graph.part.3")), partition)
    # an unknown format number and a stray array name are refused
    import json
    meta_path = os.path.join(distributed_file(0, P, str(tmp_path)), "meta.json")
    meta = json.load(open(meta_path))
    json.dump(dict(meta, format=99), open(meta_path, "w"))
    with pytest.raises(RuntimeError):
        DistChunk.load(distributed_file(0, P, str(tmp_path)))
    json.dump(dict(meta, arrays=meta["arrays"] + ["surprise"]), open(meta_path, "w"))
    with pytest.raises(RuntimeError):
        DistChunk.load(distributed_file(0, P, str(tmp_path)))


def test_explicit_bounds():
    from jittorgeometric_b200.dist import RowPartition
    p = RowPartition(10, 3, bounds=[0, 2, 9, 10])
    assert [p.n_local(r) for r in range(3)] == [2, 7, 1]
    assert [p.owner(v) for v in (0, 1, 2, 8, 9)] == [0, 0, 1, 1, 2]
    for bad in ([0, 5, 10], [0, 6, 4, 10], [1, 2, 3, 10], [0, 2, 3, 9]):
        with pytest.raises(ValueError):
            RowPartition(10, 3, bounds=bad)


def uneven_worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch.distributed as dist
    from test_dist_cpu import OracleBackend
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        n, f = 80, 4
        partition, edge_index, w = make_partitioned(5, n, 900, world)
        feature = np.random.default_rng(6).standard_normal((n, f)).astype(np.float32)
        ref = reference_chunks(partition, edge_index, n, world, w)
        chunk = chunk_from_reference(ref, rank, world, n, feature)
        g = chunk.sharded_graph(backend=OracleBackend())
        y = g.aggregate(chunk.local_feature)
        q.put((rank, 0, y.numpy(), None))
    except Exception as exc:
        q.put((rank, -1, None, repr(exc)))
        raise
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_chunks_drive_the_partitioned_aggregation(oracle):
    """Chunks with uneven part sizes feed ``ShardedGraph`` through explicit bounds; the result is the
    whole-graph aggregation in the renumbered node order."""
    world = 2
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=uneven_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = [q.get(timeout=90) for _ in range(world)]
    for p in procs:
        p.join(timeout=30)
    assert all(g[1] == 0 for g in got), [g[3] for g in got if g[1] != 0]
    n, f = 80, 4
    partition, edge_index, w = make_partitioned(5, n, 900, world)
    feature = np.random.default_rng(6).standard_normal((n, f)).astype(np.float64)
    A = np.zeros((n, n))
    np.add.at(A, (edge_index[1], edge_index[0]), w.astype(np.float64))      # y[dst] += w * x[src]
    want = A @ feature
    order = np.argsort(partition, kind="stable")
    offset = np.concatenate([[0], np.cumsum(np.bincount(partition, minlength=world))])
    for rank, _, y, _ in got:
        assert np.abs(y - want[order][offset[rank]: offset[rank + 1]]).max() <= 1e-4


def chunk_training_worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch.distributed as dist
    from jittorgeometric_b200 import dist as jd
    from test_dist_cpu import OracleBackend
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        n, f, classes, partition, edge_index, w, feature, labels = symmetric_problem(world)
        ref = reference_chunks(partition, edge_index, n, world, w)
        chunk = chunk_from_reference(ref, rank, world, n, feature)
        s, e = ref[rank]["range"]
        local_labels = torch.from_numpy(labels[ref[rank]["order"]][s:e].copy())
        g = chunk.sharded_graph(backend=OracleBackend())
        mgr = jd.DistributedManager()
        model = jd.ShardedGCN(f, 6, classes, layers=2, manager=mgr, seed=7)
        opt = torch.optim.SGD(model.parameters(), lr=0.3)
        mask = torch.ones(e - s, dtype=torch.bool)
        losses = [jd.sharded_training_step(model, g, chunk.local_feature, local_labels, mask, opt, mgr) for _ in range(2)]
        q.put((rank, 0, [p.detach().numpy().copy() for p in model.weights], losses))
    except Exception as exc:
        q.put((rank, -1, repr(exc), None))
        raise
    finally:
        dist.destroy_process_group()


def symmetric_problem(world):
    rng = np.random.default_rng(31)
    n, f, classes = 70, 5, 3
    a = rng.integers(0, n, size=260)
    b = rng.integers(0, n, size=260)
    keep = a != b
    pairs = np.unique(np.stack([np.minimum(a, b)[keep], np.maximum(a, b)[keep]], 1), axis=0)
    wv = (rng.random(len(pairs)) * 0.2).astype(np.float32)
    edge_index = np.concatenate([pairs.T, pairs.T[::-1]], axis=1).astype(np.int64)      # both directions: a symmetric matrix
    w = np.concatenate([wv, wv])
    partition = rng.integers(0, world, size=n).astype(np.int32)
    partition[:world] = np.arange(world)
    feature = rng.standard_normal((n, f)).astype(np.float32)
    labels = rng.integers(0, classes, size=n).astype(np.int64)
    return n, f, classes, partition, edge_index, w, feature, labels


@pytest.mark.timeout(180)
def test_training_on_chunks_of_a_partition_file(oracle):
    """Partition vector -> chunks -> compact-halo aggregation -> two SGD steps on three uneven ranks:
    losses and weights equal dense float64 training on the whole (renumbered) graph."""
    from jittorgeometric_b200 import dist as jd
    world = 3
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=chunk_training_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = [q.get(timeout=150) for _ in range(world)]
    for p in procs:
        p.join(timeout=30)
    assert all(g[1] == 0 for g in got), [g[2] for g in got if g[1] != 0]
    n, f, classes, partition, edge_index, w, feature, labels = symmetric_problem(world)
    A = np.zeros((n, n))
    np.add.at(A, (edge_index[1], edge_index[0]), w.astype(np.float64))
    A = torch.from_numpy(A)
    ref = jd.ShardedGCN(f, 6, classes, layers=2, manager=None, seed=7)
    W = [p.detach().double().requires_grad_(True) for p in ref.weights]
    X, L = torch.from_numpy(feature).double(), torch.from_numpy(labels)
    want_losses = []
    for _ in range(2):
        h = X
        for wt in W:
            h = (A @ h) @ wt
        loss = torch.nn.functional.nll_loss(torch.log_softmax(h, dim=1), L)
        grads = torch.autograd.grad(loss, W)
        want_losses.append(float(loss.detach()))
        W = [(wt - 0.3 * g).detach().requires_grad_(True) for wt, g in zip(W, grads)]
    for rank, _, weights, losses in got:
        assert np.allclose(losses, want_losses, rtol=1e-4, atol=1e-5)
        for have, want in zip(weights, W):
            assert np.abs(have - want.detach().numpy()).max() <= 1e-4


def test_restatement_equals_the_reference_partitioner():
    """``tests/golden/ref_partition.npz`` holds what the reference's own ``partition_to_chunk`` and
    ``set_chunks_csrs`` produced (run from the checkout by tests/golden/make_golden.py).  The numpy
    restatement above, given the node order the reference's ``argsort`` chose, reproduces every array;
    and ``DistChunk.set_chunk_csrs`` (slices) equals the reference's per-node loop."""
    from jittorgeometric_b200.partition import DistChunk
    g = dict(np.load(os.path.join(ROOT, "tests", "golden", "ref_partition.npz")))
    n, P = int(g["n"]), int(g["parts"])
    order = np.concatenate([g[f"p{p}_label"] for p in range(P)])         # labels were arange(n): the order the reference chose
    assert np.array_equal(np.sort(order), np.arange(n))
    assert np.array_equal(g["partition"][order], np.sort(g["partition"]))
    ref = reference_chunks(g["partition"], g["edge_index"], n, P, g["edge_weight"], order=order)
    t = lambda a, dt: torch.from_numpy(np.ascontiguousarray(a).astype(dt))
    for p in range(P):
        r = ref[p]
        assert np.array_equal(r["edge_index"], g[f"p{p}_edge_index"])
        assert np.array_equal(r["edge_weight"], g[f"p{p}_edge_weight"])
        assert np.array_equal(r["offset"], g[f"p{p}_offset"])
        assert np.array_equal(g["feature"][order][r["range"][0]: r["range"][1]], g[f"p{p}_feature"])
        for kind in ("csr", "csc"):
            assert np.array_equal(r[kind].indices, g[f"p{p}_{kind}_indices"])
            assert np.array_equal(r[kind].indptr, g[f"p{p}_{kind}_indptr"])
            assert np.array_equal(r[kind].data, g[f"p{p}_{kind}_data"])
        s, e = r["range"]
        c = DistChunk(P, p, e - s, n, t(r["edge_index"], np.int32), t(r["offset"], np.int32), t(r["edge_weight"], np.float32))
        c.set_csr(t(g[f"p{p}_csr_indices"], np.int32), t(g[f"p{p}_csr_indptr"], np.int32), t(g[f"p{p}_csr_data"], np.float32))
        for q, sub in enumerate(c.set_chunk_csrs()):
            assert np.array_equal(sub.column_indices.numpy(), g[f"p{p}_chunk{q}_indices"])
            assert np.array_equal(sub.row_offset.numpy(), g[f"p{p}_chunk{q}_indptr"])
            assert np.array_equal(sub.edge_weight.numpy(), g[f"p{p}_chunk{q}_data"])
