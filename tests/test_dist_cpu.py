"""CPU ranks over gloo (world size 2 and 3): the row partition, interior/halo split, shard
exchange and accumulate order of the partitioned aggregation, with the CPU checker standing in
for the kernels.  The result must equal the single-shard aggregation."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class OracleBackend:
    """numpy/oracle stand-in for the CUDA backend (tests only)."""

    def __init__(self):
        import oracle
        self.O = oracle

    def split(self, idx, off, w, lo, hi):
        idx, off, w = idx.numpy(), off.numpy(), w.numpy()
        inside = (idx >= lo) & (idx < hi)
        seg = np.repeat(np.arange(len(off) - 1), np.diff(off))
        def part(mask, rebase):
            o = np.concatenate([[0], np.cumsum(np.bincount(seg[mask], minlength=len(off) - 1))]).astype(np.int32)
            return torch.from_numpy((idx[mask] - rebase).astype(np.int32)), torch.from_numpy(o), torch.from_numpy(w[mask])
        return part(inside, lo), part(~inside, 0)

    def halo_map(self, halo_idx, n_global, bounds, lo=0, hi=0, base=0):
        idx = halo_idx.numpy()
        own = (idx >= lo) & (idx < hi)
        needed = np.unique(idx[~own])
        remapped = np.where(own, idx - lo, base + np.searchsorted(needed, idx)).astype(np.int32)
        counts = [int(((needed >= bounds[q]) & (needed < bounds[q + 1])).sum()) for q in range(len(bounds) - 1)]
        return torch.from_numpy(needed.astype(np.int32)), torch.from_numpy(remapped), counts

    def gather_rows(self, x, rows, rebase, out):
        out[: rows.numel()] = x[(rows.long() - rebase)]
        return out

    def plan(self, off, nnz):
        return None

    def aggregate(self, x, idx, off, w, n_out, plan, out=None, accumulate=False):
        y = torch.from_numpy(self.O.aggregate(x.numpy(), idx.numpy(), off.numpy(), w.numpy(), n_out=n_out))
        if accumulate:
            out += y
            return out
        return y


def make_graph(seed, n, E, f):
    rng = np.random.default_rng(seed)
    dst = rng.integers(0, n, size=E)
    src = rng.integers(0, n, size=E)
    order = np.argsort(dst, kind="stable")
    off = np.concatenate([[0], np.cumsum(np.bincount(dst, minlength=n))]).astype(np.int32)
    w = rng.standard_normal(E).astype(np.float32)
    x = rng.standard_normal((n, f)).astype(np.float32)
    return src[order].astype(np.int32), off, w[order], x


def worker(rank, world, port, n, E, f, q, mode):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    from jittorgeometric_b200 import dist as jd
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        idx, off, w, x = make_graph(7, n, E, f)
        part = jd.RowPartition(n, world)
        lo, hi = part.range(rank)
        l_idx, l_off, l_w = jd.shard_rows(torch.from_numpy(idx), torch.from_numpy(off), torch.from_numpy(w), part, rank)
        g = jd.ShardedGraph(part, rank, l_idx, l_off, l_w, backend=OracleBackend(), mode=mode)
        y = g.aggregate(torch.from_numpy(x[lo:hi].copy()))
        # two exchanges in flight before either aggregation is finished
        xa, xb = torch.from_numpy(x[lo:hi].copy()), torch.from_numpy(np.ascontiguousarray(x[lo:hi, :2]))
        pa, pb = g.start(xa), g.start(xb)
        try:                                                    # a second exchange of a width still in flight would share its buffers
            g.start(xa)
            raise AssertionError("a second start of the same width must raise")
        except RuntimeError as exc:
            assert "already in flight" in str(exc)
        ya, yb = g.finish(pa), g.finish(pb)
        assert torch.equal(ya, y) and torch.equal(yb, g.aggregate(xb))
        if mode == "overlap":
            # interior and halo together hold every entry of the shard exactly once
            assert g.interior[0].numel() + g.halo[0].numel() == l_idx.numel()
            assert g.interior[0].numel() == 0 or int(g.interior[0].max()) < hi - lo
            assert g.halo[0].numel() == 0 or int(g.halo[0].max()) < g.n_halo
        else:
            assert g.merged[0].numel() == l_idx.numel()
            assert l_idx.numel() == 0 or int(g.merged[0].max()) < (hi - lo) + g.n_halo
        # only referenced remote rows travel, each once; requests and deliveries agree
        assert g.n_halo == g.needed.numel() <= n - (hi - lo)
        assert all(lo <= int(v) < hi for v in g.send_rows.tolist())
        y_again = g.aggregate(torch.from_numpy(x[lo:hi].copy()))
        assert torch.equal(y, y_again)
        q.put((rank, lo, hi, y.numpy()))
    except Exception as exc:  # surface the failure in the parent instead of a queue timeout
        q.put((rank, -1, -1, repr(exc)))
        raise
    finally:
        dist.destroy_process_group()


def grad_worker(rank, world, port, n, f, q):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    from jittorgeometric_b200 import dist as jd
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        idx, off, w, x, gy = make_symmetric(3, n, f)
        part = jd.RowPartition(n, world)
        lo, hi = part.range(rank)
        g = jd.ShardedGraph(part, rank, *jd.shard_rows(torch.from_numpy(idx), torch.from_numpy(off), torch.from_numpy(w), part, rank),
                            backend=OracleBackend())
        xl = torch.from_numpy(x[lo:hi].copy()).requires_grad_(True)
        y = g.aggregate(xl)
        y.backward(torch.from_numpy(gy[lo:hi].copy()))
        q.put((rank, lo, hi, xl.grad.numpy()))
    except Exception as exc:
        q.put((rank, -1, -1, repr(exc)))
        raise
    finally:
        dist.destroy_process_group()


def make_symmetric(seed, n, f):
    rng = np.random.default_rng(seed)
    a = rng.integers(0, n, size=4 * n)
    b = rng.integers(0, n, size=4 * n)
    wv = rng.random(4 * n).astype(np.float32)
    src = np.concatenate([a, b]); dst = np.concatenate([b, a]); w = np.concatenate([wv, wv])
    order = np.argsort(dst, kind="stable")
    off = np.concatenate([[0], np.cumsum(np.bincount(dst, minlength=n))]).astype(np.int32)
    return (src[order].astype(np.int32), off, w[order], rng.standard_normal((n, f)).astype(np.float32),
            rng.standard_normal((n, f)).astype(np.float32))


@pytest.mark.timeout(120)
def test_partitioned_backward_on_a_symmetric_graph(oracle):
    """grad_x = A^T grad_y; for a symmetric A the same partitioned aggregation gives it."""
    world, n, f = 2, 90, 4
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=grad_worker, args=(r, world, port, n, f, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = [q.get(timeout=90) for _ in range(world)]
    for p in procs:
        p.join(timeout=30)
    assert all(g[1] >= 0 for g in got), [g[3] for g in got if g[1] < 0]
    idx, off, w, x, gy = make_symmetric(3, n, f)
    # true gradient: transpose aggregation, computed densely in float64
    A = np.zeros((n, n))
    seg = np.repeat(np.arange(n), np.diff(off))
    np.add.at(A, (seg, idx), w.astype(np.float64))
    want = A.T @ gy.astype(np.float64)
    for rank, lo, hi, gx in got:
        assert np.abs(gx - want[lo:hi]).max() <= 1e-4


def free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.mark.parametrize("world,n,mode", [(2, 101, "merged"), (3, 64, "merged"), (3, 64, "overlap")])
@pytest.mark.timeout(120)
def test_partitioned_aggregation_equals_single_shard(oracle, world, n, mode):
    E, f = 1500, 5
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=worker, args=(r, world, port, n, E, f, q, mode)) for r in range(world)]
    for p in procs:
        p.start()
    got = [q.get(timeout=90) for _ in range(world)]
    for p in procs:
        p.join(timeout=30)
    assert all(g[1] >= 0 for g in got), [g[3] for g in got if g[1] < 0]
    assert all(p.exitcode == 0 for p in procs)
    idx, off, w, x = make_graph(7, n, E, f)
    want = oracle.aggregate(x, idx, off, w)
    _, scale = oracle.aggregate_f64(x, idx, off, w)
    for rank, lo, hi, y in got:
        assert y.shape == (hi - lo, f)
        assert (np.abs(y - want[lo:hi]) / (scale[lo:hi] + 1e-30)).max() <= 1e-5
        if mode == "merged":      # every row is summed in the order the unpartitioned graph sums it
            assert np.array_equal(y, want[lo:hi])


def train_worker(rank, world, port, n, f, hidden, classes, steps, q):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    from jittorgeometric_b200 import dist as jd
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        idx, off, w, x, _ = make_symmetric(5, n, f)
        labels, mask = make_labels(5, n, classes)
        part = jd.RowPartition(n, world)
        lo, hi = part.range(rank)
        g = jd.ShardedGraph(part, rank, *jd.shard_rows(torch.from_numpy(idx), torch.from_numpy(off), torch.from_numpy(w), part, rank),
                            backend=OracleBackend())
        mgr = jd.DistributedManager()
        assert mgr.broadcast_args({"lr": 0.5} if rank == 0 else None) == {"lr": 0.5}
        model = jd.ShardedGCN(f, hidden, classes, layers=2, manager=mgr, seed=100 + rank)   # differing draws: the broadcast must win
        opt = torch.optim.SGD(model.parameters(), lr=0.5)
        losses = [jd.sharded_training_step(model, g, torch.from_numpy(x[lo:hi].copy()), torch.from_numpy(labels[lo:hi].copy()),
                                           torch.from_numpy(mask[lo:hi].copy()), opt, mgr) for _ in range(steps)]
        # parameter averaging of the reference's manager: make the ranks differ, then average
        with torch.no_grad():
            model.weights[0].add_(float(rank))
        mgr.synchronize_model_parameters(model)
        q.put((rank, 0, 0, [p.detach().numpy().copy() for p in model.weights], losses))
    except Exception as exc:
        q.put((rank, -1, -1, repr(exc), None))
        raise
    finally:
        dist.destroy_process_group()


def make_labels(seed, n, classes):
    rng = np.random.default_rng(seed + 1000)
    return rng.integers(0, classes, size=n).astype(np.int64), rng.random(n) < 0.6


@pytest.mark.timeout(180)
def test_partitioned_training_equals_single_process(oracle):
    """Two ranks, gradients summed over the ranks: weights and losses after three SGD steps equal
    dense float64 training on the whole graph."""
    from jittorgeometric_b200 import dist as jd
    world, n, f, hidden, classes, steps = 2, 90, 6, 5, 3, 3
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=train_worker, args=(r, world, port, n, f, hidden, classes, steps, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = [q.get(timeout=150) for _ in range(world)]
    for p in procs:
        p.join(timeout=30)
    assert all(g[1] >= 0 for g in got), [g[3] for g in got if g[1] < 0]
    idx, off, w, x, _ = make_symmetric(5, n, f)
    labels, mask = make_labels(5, n, classes)
    A = np.zeros((n, n))
    np.add.at(A, (np.repeat(np.arange(n), np.diff(off)), idx), w.astype(np.float64))
    A = torch.from_numpy(A)
    ref = jd.ShardedGCN(f, hidden, classes, layers=2, manager=None, seed=100)      # rank 0's draw
    W = [p.detach().double().requires_grad_(True) for p in ref.weights]
    X, L, M = torch.from_numpy(x).double(), torch.from_numpy(labels), torch.from_numpy(mask)
    want_losses = []
    for _ in range(steps):
        h = X
        for wt in W:
            h = (A @ h) @ wt
        loss = torch.nn.functional.nll_loss(torch.log_softmax(h, dim=1)[M], L[M])
        grads = torch.autograd.grad(loss, W)
        want_losses.append(float(loss.detach()))
        W = [(wt - 0.5 * g).detach().requires_grad_(True) for wt, g in zip(W, grads)]
    for rank, _, _, weights, losses in got:
        assert np.allclose(losses, want_losses, rtol=1e-4, atol=1e-5)
        # the first matrix was shifted by the rank and averaged: mean shift (world - 1) / 2
        assert np.abs(weights[0] - (W[0].detach().numpy() + (world - 1) / 2)).max() <= 1e-4
        assert np.abs(weights[1] - W[1].detach().numpy()).max() <= 1e-4


def spmm_rounds_worker(rank, world, port, n, f, q):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    import oracle as O
    from jittorgeometric_b200 import dist as jd
    from jittorgeometric_b200.data import CSR
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        idx, off, w, x, gy = make_symmetric(9, n, f)
        part = jd.RowPartition(n, world)
        lo, hi = part.range(rank)
        seg = np.repeat(np.arange(n), np.diff(off))
        mine = (seg >= lo) & (seg < hi)
        csr_list = []
        for s_rank in range(world):
            s_lo, s_hi = part.range(s_rank)
            sel = mine & (idx >= s_lo) & (idx < s_hi)
            ei = np.stack([idx[sel] - s_lo, seg[sel] - lo]).astype(np.int32)
            ci, ro, cw = O.coo_to_csr(ei, w[sel], s_hi - s_lo)
            csr_list.append(CSR(torch.from_numpy(ci), torch.from_numpy(ro), torch.from_numpy(cw)))

        def one_round(fb, csr, local_vnum, out):
            # op(A)^T product of one source rank's block with the CPU checker: CSR rows are sources
            ci, ro, cw = csr.column_indices.numpy(), csr.row_offset.numpy(), csr.edge_weight.numpy()
            rows = np.repeat(np.arange(len(ro) - 1), np.diff(ro)).astype(np.int32)
            ti, to, tw = O.coo_to_csc(np.stack([rows, ci]).astype(np.int32), cw, local_vnum)
            y = torch.from_numpy(O.aggregate(fb.numpy(), ti, to, tw, n_out=local_vnum))
            return y if out is None else out + y

        xl = torch.from_numpy(x[lo:hi].copy()).requires_grad_(True)
        y = jd.DistSpmm(jd.DistributedManager(), xl, csr_list, hi - lo, aggregate=one_round)
        y.backward(torch.from_numpy(gy[lo:hi].copy()))
        q.put((rank, lo, hi, y.detach().numpy(), xl.grad.numpy()))
    except Exception as exc:
        q.put((rank, -1, -1, repr(exc), None))
        raise
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_broadcast_rounds_forward_and_backward(oracle):
    """The reference-shaped DistSpmm (one broadcast round per source rank) on two CPU ranks:
    forward equals the whole-graph aggregation, backward follows the reference's rule."""
    world, n, f = 2, 70, 3
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=spmm_rounds_worker, args=(r, world, port, n, f, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = [q.get(timeout=90) for _ in range(world)]
    for p in procs:
        p.join(timeout=30)
    assert all(g[1] >= 0 for g in got), [g[3] for g in got if g[1] < 0]
    idx, off, w, x, gy = make_symmetric(9, n, f)
    A = np.zeros((n, n))
    np.add.at(A, (np.repeat(np.arange(n), np.diff(off)), idx), w.astype(np.float64))
    for rank, lo, hi, y, gx in got:
        assert np.abs(y - (A @ x.astype(np.float64))[lo:hi]).max() <= 1e-4
        assert np.abs(gx - (A.T @ gy.astype(np.float64))[lo:hi]).max() <= 1e-4


def test_row_partition_bounds():
    from jittorgeometric_b200.dist import RowPartition
    p = RowPartition(10, 4)
    assert p.pad == 3 and p.bounds == [0, 3, 6, 9, 10]
    assert [p.n_local(r) for r in range(4)] == [3, 3, 3, 1]
    assert p.owner(9) == 3 and p.owner(0) == 0
    p = RowPartition(8, 8)
    assert p.bounds == list(range(9))
    p = RowPartition(3, 4)       # more ranks than rows: trailing ranks own nothing
    assert [p.n_local(r) for r in range(4)] == [1, 1, 1, 0]
    with pytest.raises(ValueError):
        RowPartition(5, 0)


def silent_worker(rank, world, port, n, E, f, q):
    """Rank ``world - 1`` builds its graph and then never starts the exchange."""
    sys.path.insert(0, ROOT)
    import time
    import torch.distributed as dist
    from jittorgeometric_b200 import dist as jd
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        idx, off, w, x = make_graph(7, n, E, f)
        part = jd.RowPartition(n, world)
        lo, hi = part.range(rank)
        shard = jd.shard_rows(torch.from_numpy(idx), torch.from_numpy(off), torch.from_numpy(w), part, rank)
        g = jd.ShardedGraph(part, rank, *shard, backend=OracleBackend(), transport=jd.CollectiveTransport(timeout_s=3.0))
        if rank == world - 1:
            time.sleep(8.0)                                     # the failure: this rank never posts its halo rows
            q.put((rank, "silent", 0.0))
            return
        t0 = time.perf_counter()
        try:
            g.aggregate(torch.from_numpy(x[lo:hi].copy()))
            q.put((rank, "finished", time.perf_counter() - t0))
        except jd.ExchangeTimeout as exc:
            q.put((rank, "timeout", time.perf_counter() - t0))
    except Exception as exc:
        q.put((rank, repr(exc), -1.0))
    finally:
        # no destroy_process_group: its shutdown handshake would wait for the ranks that gave up
        q.close()
        q.join_thread()
        os._exit(0)


@pytest.mark.timeout(120)
def test_a_rank_that_never_posts_its_halo_ends_in_a_timeout_not_a_hang(oracle):
    """Failure detection on the host (three gloo ranks, one silent): the others' bounded wait for
    the exchange raises ``ExchangeTimeout`` after the transport's limit instead of hanging."""
    world, n, E, f = 3, 64, 1500, 5
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=silent_worker, args=(r, world, port, n, E, f, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = sorted(q.get(timeout=60) for _ in range(world))
    for p in procs:
        p.join(timeout=30)
    assert got[world - 1][1] == "silent"
    for rank, what, secs in got[: world - 1]:
        assert what == "timeout", got
        assert 2.0 <= secs <= 7.5, got


def test_row_blocks_cover_the_rows_in_whole_tiles():
    """``part_rows``: the row blocks of a block-wise exchange start on multiples of 128 rows (the transform's
    tile), cover every row once, and every rank derives the same boundaries for every owner."""
    from jittorgeometric_b200.dist import part_rows
    for n_local in (0, 1, 127, 128, 129, 1000, 8388608, 8388609, 12345677):
        for parts in (1, 2, 3, 4, 7):
            rows = part_rows(n_local, parts)
            assert len(rows) == parts + 1 and rows[0] == 0 and rows[-1] == n_local
            assert all(a <= b for a, b in zip(rows[:-1], rows[1:]))
            assert all(r % 128 == 0 or r == n_local for r in rows)
            sizes = [b - a for a, b in zip(rows[:-1], rows[1:])]
            assert sum(sizes) == n_local
