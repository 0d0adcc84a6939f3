"""GPU side of the partitioned aggregation: the split and accumulate kernels with the ranks of a
partition emulated one after another on one GPU (the exchange replaced by a local copy), and the
real NCCL path as child processes when the box has at least two GPUs."""
import os
import socket
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def make_graph(seed, n, E, f, hubs=3, hub_deg=3000):
    rng = np.random.default_rng(seed)
    dst = np.concatenate([rng.integers(0, n, size=E), np.repeat(rng.integers(0, n, size=hubs), hub_deg)])
    src = rng.integers(0, n, size=len(dst))
    order = np.argsort(dst, kind="stable")
    off = np.concatenate([[0], np.cumsum(np.bincount(dst, minlength=n))]).astype(np.int32)
    w = rng.standard_normal(len(dst)).astype(np.float32)
    x = rng.standard_normal((n, f)).astype(np.float32)
    return src[order].astype(np.int32), off, w[order], x


class Loopback:
    """Stands in for the process group when the ranks of a partition are emulated one after another
    on one GPU: requests and row segments are handed over by plain copies."""

    def __init__(self):
        self.graphs, self.features = [], []

    def send_buffer(self, rows, f, like):
        return torch.empty((max(rows, 1), f), dtype=like.dtype, device=like.device)

    def wire(self):
        world = len(self.graphs)
        matrix = [list(g.recv_counts) for g in self.graphs]
        for q, g in enumerate(self.graphs):
            parts = []
            for r, h in enumerate(self.graphs):
                s0 = h.recv_offset[q]
                parts.append(h.needed[s0:s0 + h.recv_counts[q]])
            g.apply_setup(matrix, torch.cat(parts) if parts else g.needed[:0])

    def exchange(self, g, send, recv, f):
        for q, h in enumerate(self.graphs):
            n = g.recv_counts[q]
            if q == g.rank or n == 0:
                continue
            packed = torch.empty((max(h.n_send, 1), f), device=recv.device)
            h.backend.gather_rows(self.features[q], h.send_rows, h.lo, packed)
            src0 = g.peer_send_offset[q]
            recv[g.recv_offset[q]:g.recv_offset[q] + n] = packed[src0:src0 + n]

        class Done:
            def wait(self):
                pass

            def release(self):
                pass
        return Done()


@pytest.mark.parametrize("mode", ["merged", "overlap"])
@pytest.mark.parametrize("world,n,f", [(2, 5001, 128), (4, 4096, 32), (8, 3000, 7)])
def test_emulated_ranks_on_one_gpu(cuda, oracle, world, n, f, mode):
    from jittorgeometric_b200 import dist as jd
    idx, off, w, x = make_graph(world, n, 60000, f)
    want = oracle.aggregate(x, idx, off, w)
    _, scale = oracle.aggregate_f64(x, idx, off, w)
    part = jd.RowPartition(n, world)
    t = lambda a: torch.from_numpy(a).cuda()
    idx_t, off_t, w_t = t(idx), t(off), t(w)
    whole = cuda.ops.segment_aggregate(t(x), idx_t, off_t, w_t, plan=cuda.ops.SpmmPlan(off_t, len(idx))).cpu().numpy()
    loop = Loopback()
    for rank in range(world):
        lo, hi = part.range(rank)
        loop.graphs.append(jd.ShardedGraph(part, rank, *jd.shard_rows(idx_t, off_t, w_t, part, rank), transport=loop,
                                           setup=False, mode=mode))
        loop.features.append(t(x[lo:hi].copy()))
    loop.wire()
    for rank, g in enumerate(loop.graphs):
        lo, hi = part.range(rank)
        s, e = off[lo], off[hi]
        loc = idx[s:e]
        inside = (loc >= lo) & (loc < hi)
        needed = np.unique(loc[~inside])
        # compact halo: the distinct remote rows, ascending, grouped by owner
        assert np.array_equal(g.needed.cpu().numpy(), needed)
        assert g.recv_counts == [int(((needed >= part.bounds[q]) & (needed < part.bounds[q + 1])).sum()) for q in range(world)]
        if mode == "overlap":
            # split: order inside a row preserved, interior ids rebased, halo entries re-addressed
            assert np.array_equal(g.interior[0].cpu().numpy(), loc[inside] - lo)
            seg = np.repeat(np.arange(hi - lo), np.diff(off[lo:hi + 1]))
            assert np.array_equal(np.diff(g.interior[1].cpu().numpy()), np.bincount(seg[inside], minlength=hi - lo))
            assert np.array_equal(np.diff(g.halo[1].cpu().numpy()), np.bincount(seg[~inside], minlength=hi - lo))
            assert np.array_equal(needed[g.halo[0].cpu().numpy()], loc[~inside])
        else:
            # one structure over [own rows | packed halo rows], entries in their original places
            m = g.merged[0].cpu().numpy()
            assert np.array_equal(m[inside], loc[inside] - lo)
            assert np.array_equal(needed[m[~inside] - (hi - lo)], loc[~inside])
        y = g.aggregate(loop.features[rank]).cpu().numpy()
        assert (np.abs(y - want[lo:hi]) / (scale[lo:hi] + 1e-30)).max() <= 1e-5
        assert np.array_equal(y, g.aggregate(loop.features[rank]).cpu().numpy())
        if mode == "merged":                              # every row summed exactly as the unpartitioned kernel sums it
            assert np.array_equal(y, whole[lo:hi])
        # layer epilogue: fused into the kernel's store (merged) or applied afterwards (overlap)
        bias = torch.linspace(-1, 1, f, device="cuda")
        z = g.aggregate(loop.features[rank], bias=bias, relu=True)
        assert torch.equal(z, torch.relu(torch.from_numpy(y).cuda() + bias))


def build_emulated(jd, world, n, f, E=60000, seed=None, mode="merged", **kw):
    idx, off, w, x = make_graph(world if seed is None else seed, n, E, f)
    part = jd.RowPartition(n, world)
    t = lambda a: torch.from_numpy(a).cuda()
    idx_t, off_t, w_t = t(idx), t(off), t(w)
    emu = jd.EmulatedRanks(world, **kw)
    graphs = [jd.ShardedGraph(part, r, *jd.shard_rows(idx_t, off_t, w_t, part, r), transport=emu.transport(r), setup=False,
                              mode=mode) for r in range(world)]
    emu.wire(graphs)
    for r, g in enumerate(graphs):                       # every rank's rows are in place before the first exchange
        lo, hi = part.range(r)
        g.feature_buffer(f).copy_(t(x[lo:hi].copy()))
    return (idx, off, w, x), part, emu, graphs


@pytest.mark.parametrize("world,n,f,parts", [(2, 5001, 128, 2), (4, 4096, 64, 4), (3, 2500, 256, 3), (8, 3000, 32, 2), (2, 300, 16, 4)])
def test_block_wise_exchange_and_row_range_aggregation(cuda, oracle, world, n, f, parts):
    """Rows offered and fetched block after block (one epoch word per block, ``jg_halo_pull_part``) land exactly
    where the whole-segment exchange puts them and give the same aggregation bit for bit; the aggregation of
    row ranges (what produces the blocks of the next layer) equals the whole one row for row."""
    from jittorgeometric_b200 import dist as jd
    (idx, off, w, x), part, emu, graphs = build_emulated(jd, world, n, f, E=20 * n)
    want = oracle.aggregate(x, idx, off, w)
    _, scale = oracle.aggregate_f64(x, idx, off, w)
    for r, g in enumerate(graphs):
        lo, hi = part.range(r)
        whole = g.aggregate(g.feature_buffer(f)).cpu().numpy()
        halo_whole = emu.buffer(f, r)[g.n_local: g.n_local + g.n_halo].clone()
        emu.buffer(f, r)[g.n_local:].zero_()
        # the blocks of every owner partition its segment of the needed rows
        tables = g.part_tables(parts)
        for q in range(world):
            assert tables[0][0][q] == g.recv_offset[q] and tables[-1][1][q] == g.recv_offset[q] + g.recv_counts[q]
            for c in range(parts - 1):
                assert tables[c][1][q] == tables[c + 1][0][q]
        handles = []
        for c in range(parts):
            handles.append(g.start_part(f, c, parts))
            if c < parts - 1:                    # later blocks have not arrived yet
                end = max(tables[c][1])
                later = [(tables[c2][0][q], tables[c2][1][q]) for c2 in range(c + 1, parts) for q in range(world)]
                torch.cuda.synchronize()
                for a, b in later:
                    assert not emu.buffer(f, r)[g.n_local + a: g.n_local + b].any()
        y = g.finish_parts(f, handles).cpu().numpy()
        emu.transport(r).check()
        assert torch.equal(emu.buffer(f, r)[g.n_local: g.n_local + g.n_halo], halo_whole)
        assert np.array_equal(y, whole)
        assert (np.abs(y - want[lo:hi]) / (scale[lo:hi] + 1e-30)).max() <= 1e-5
        # row ranges of one aggregation
        pending = g.start(g.feature_buffer(f))
        pending[2].wait()
        rows = jd.part_rows(g.n_local, parts)
        pieces = [g.aggregate_rows(pending, rows[c], rows[c + 1]) for c in range(parts) if rows[c + 1] > rows[c]]
        g.done(pending)
        got = torch.cat(pieces).cpu().numpy()
        assert got.shape == whole.shape
        assert (np.abs(got - want[lo:hi]) / (scale[lo:hi] + 1e-30)).max() <= 1e-5
        short = np.diff(off[lo: hi + 1]) <= 256            # rows no plan splits: the same sum whatever the range
        assert np.array_equal(got[short], whole[short])


@pytest.mark.parametrize("mode", ["merged", "overlap"])
@pytest.mark.parametrize("world,n,f,plain", [(2, 5001, 128, False), (4, 4096, 32, False), (8, 3000, 7, False), (3, 2500, 256, False),
                                             (4, 4096, 64, True), (2, 40000, 512, False)])
def test_direct_exchange_with_emulated_ranks(cuda, oracle, world, n, f, plain, mode):
    """The peer-load exchange (epoch words, bulk-copy pull kernel, plain-load pull kernel for rows that
    are not multiples of 16 bytes) with all ranks of the partition on one GPU, against the CPU checker
    and bit for bit against the unpartitioned kernel."""
    from jittorgeometric_b200 import dist as jd
    (idx, off, w, x), part, emu, graphs = build_emulated(jd, world, n, f, E=20 * n, mode=mode, plain=plain)
    want = oracle.aggregate(x, idx, off, w)
    _, scale = oracle.aggregate_f64(x, idx, off, w)
    t = lambda a: torch.from_numpy(a).cuda()
    whole = cuda.ops.segment_aggregate(t(x), t(idx), t(off), t(w), plan=cuda.ops.SpmmPlan(t(off), len(idx))).cpu().numpy()
    for r, g in enumerate(graphs):
        lo, hi = part.range(r)
        xr = g.feature_buffer(f)
        y = g.aggregate(xr).cpu().numpy()
        emu.transport(r).check()
        # the halo rows that landed are exactly the referenced remote rows
        halo = emu.buffer(f, r)[g.n_local: g.n_local + g.n_halo].cpu().numpy()
        assert np.array_equal(halo, x[g.needed.cpu().numpy()])
        assert (np.abs(y - want[lo:hi]) / (scale[lo:hi] + 1e-30)).max() <= 1e-5
        if mode == "merged":
            assert np.array_equal(y, whole[lo:hi])
        y2 = g.aggregate(t(x[lo:hi].copy())).cpu().numpy()          # rows handed over in another tensor: copied in, next epoch
        assert np.array_equal(y, y2)
    # two widths in flight on one rank; the same width twice raises
    g = graphs[0]
    lo, hi = part.range(0)
    f2 = 16 if f > 16 else 4
    for r, h in enumerate(graphs):
        a, b = part.range(r)
        h.feature_buffer(f2).copy_(t(np.ascontiguousarray(x[a:b, :f2])))
    pa, pb = g.start(g.feature_buffer(f)), g.start(g.feature_buffer(f2))
    with pytest.raises(RuntimeError, match="already in flight"):
        g.start(g.feature_buffer(f))
    ya, yb = g.finish(pa), g.finish(pb, relu=True)
    torch.cuda.synchronize()
    want2 = oracle.aggregate(np.ascontiguousarray(x[:, :f2]), idx, off, w)
    _, scale2 = oracle.aggregate_f64(np.ascontiguousarray(x[:, :f2]), idx, off, w)
    assert (np.abs(ya.cpu().numpy() - want[lo:hi]) / (scale[lo:hi] + 1e-30)).max() <= 1e-5
    assert (np.abs(yb.cpu().numpy() - np.maximum(want2[lo:hi], 0)) / (scale2[lo:hi] + 1e-30)).max() <= 1e-5


@pytest.mark.parametrize("world,n,f", [(2, 5001, 128), (4, 4096, 64), (8, 3000, 8), (2, 6000, 256), (2, 4000, 512)])
def test_half_width_halo_payload(cuda, oracle, world, n, f):
    """fp16 halo payload: what lands is the fp16 rounding of the remote rows, the rank's own rows stay
    fp32, the aggregation equals the unpartitioned kernel on exactly that mixed input and stays within
    5e-4 (fp16 unit roundoff 2^-11) of the fp32 result."""
    from jittorgeometric_b200 import dist as jd
    (idx, off, w, x), part, emu, graphs = build_emulated(jd, world, n, f, E=20 * n)
    t = lambda a: torch.from_numpy(a).cuda()
    x16 = t(x).to(torch.float16).float().cpu().numpy()          # round to nearest even
    _, scale = oracle.aggregate_f64(x, idx, off, w)
    want_full = oracle.aggregate(x, idx, off, w)
    for r, g in enumerate(graphs):
        g.halo_half = True
        lo, hi = part.range(r)
        y = g.aggregate(g.feature_buffer(f)).cpu().numpy()
        emu.transport(r).check()
        halo = emu.buffer(f, r)[g.n_local: g.n_local + g.n_halo].cpu().numpy()
        assert np.array_equal(halo, x16[g.needed.cpu().numpy()])
        mixed = x16.copy(); mixed[lo:hi] = x[lo:hi]
        whole = cuda.ops.segment_aggregate(t(mixed), t(idx), t(off), t(w), plan=cuda.ops.SpmmPlan(t(off), len(idx))).cpu().numpy()
        assert np.array_equal(y, whole[lo:hi])
        assert (np.abs(y - want_full[lo:hi]) / (scale[lo:hi] + 1e-30)).max() <= 5e-4


def test_exchange_wait_runs_out_and_reports(cuda):
    """Failure path of the exchange without any fault: a peer that never posts its rows.  The pull's
    bounded wait runs out after the (short) limit, the kernel returns, the host raises ExchangeTimeout
    with the silent rank's number, and the same context then runs a normal exchange."""
    from jittorgeometric_b200 import dist as jd
    (idx, off, w, x), part, emu, graphs = build_emulated(jd, 2, 3000, 64, wait_ms=20.0)
    g, tr = graphs[0], emu.transport(0)
    tr.post_for_peers = False                      # rank 1 stays silent
    y = g.aggregate(g.feature_buffer(64))
    torch.cuda.synchronize()                       # returns: the kernel gave up after 20 ms instead of spinning on
    with pytest.raises(jd.ExchangeTimeout, match="rank 1 never posted"):
        tr.check()
    tr.post_for_peers = True
    y = g.aggregate(g.feature_buffer(64))
    torch.cuda.synchronize()
    tr.check()
    t = lambda a: torch.from_numpy(a).cuda()
    whole = cuda.ops.segment_aggregate(t(x), t(idx), t(off), t(w), plan=cuda.ops.SpmmPlan(t(off), len(idx)))
    assert torch.equal(y, whole[: g.n_local])
    # the done-word wait of an owner whose reader never reports
    lib = __import__("jittorgeometric_b200._lib", fromlist=["lib"])
    err = torch.zeros(1, dtype=torch.int32).pin_memory()
    import ctypes
    lib.check(lib.lib().jg_halo_wait(lib.ptr(emu.flags[0]), 2, 0, 5, 1, 7, ctypes.c_void_p(err.data_ptr()), 5_000_000,
                                     lib.stream_for(emu.flags[0])), "jg_halo_wait")
    torch.cuda.synchronize()
    assert int(err[0]) == 0x200 + 1


def test_accumulate_mode(cuda, oracle):
    idx, off, w, x = make_graph(1, 2000, 30000, 64)
    t = lambda a: torch.from_numpy(a).cuda()
    base = np.random.default_rng(0).standard_normal((2000, 64)).astype(np.float32)
    for chunk in (None, 256):
        plan = cuda.ops.SpmmPlan(t(off), len(idx), chunk) if chunk else None
        out = t(base.copy())
        cuda.ops.segment_aggregate(t(x), t(idx), t(off), t(w), plan=plan, out=out, accumulate=True)
        fresh = cuda.ops.segment_aggregate(t(x), t(idx), t(off), t(w), plan=plan)
        assert np.array_equal(out.cpu().numpy(), base + fresh.cpu().numpy())     # old + sum, one rounding


def nccl_worker(rank, world, port, n, E, f, q, exchange):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    from jittorgeometric_b200 import dist as jd
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    import datetime
    os.environ["TORCH_SYMM_MEM_DISABLE_MULTICAST"] = "1"
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank), timeout=datetime.timedelta(seconds=90))
    try:
        idx, off, w, x = make_graph(11, n, E, f)
        part = jd.RowPartition(n, world)
        lo, hi = part.range(rank)
        t = lambda a: torch.from_numpy(a).cuda()
        g = jd.ShardedGraph(part, rank, *jd.shard_rows(t(idx), t(off), t(w), part, rank), exchange=exchange,
                            mode="overlap" if exchange == "nccl" else "merged")
        y = g.aggregate(t(x[lo:hi].copy()))
        y2 = g.aggregate(t(x[lo:hi].copy()))          # second exchange reuses the shard buffers
        torch.cuda.synchronize()
        assert torch.equal(y, y2)
        # two aggregations of different widths started before either is finished (pipelined exchanges)
        xa, xb = t(x[lo:hi].copy()), t(np.ascontiguousarray(x[lo:hi, :64]))
        pa, pb = g.start(xa), g.start(xb)
        ya, yb = g.finish(pa), g.finish(pb, relu=True)
        torch.cuda.synchronize()
        assert torch.equal(ya, y) and torch.equal(yb, torch.relu(g.aggregate(xb)))
        if g.direct:
            # block-wise exchange between real ranks: rows written and offered block after block, twice
            # (the second round reuses the blocks' epoch words), then a whole-segment exchange again
            buf = g.feature_buffer(f)
            rows = jd.part_rows(g.n_local, 3)
            for _ in range(2):
                buf = g.feature_buffer(f)                      # waits for the readers of the previous round
                handles = []
                for c in range(3):
                    buf[rows[c]: rows[c + 1]].copy_(t(x[lo + rows[c]: lo + rows[c + 1]].copy()))
                    handles.append(g.start_part(f, c, 3, ctas=0 if c == 2 else 32))
                yp = g.finish_parts(f, handles)
                torch.cuda.synchronize()
                g.transport.check()
                assert torch.equal(yp, y)
            assert torch.equal(g.aggregate(t(x[lo:hi].copy())), y)
        # the reference-shaped API: one sub-CSR per source rank, one broadcast round each
        import oracle as O
        import jittorgeometric_b200 as jg
        seg = np.repeat(np.arange(n), np.diff(off))
        mine = (seg >= lo) & (seg < hi)
        csr_list = []
        for src_rank in range(world):
            s_lo, s_hi = part.range(src_rank)
            sel = mine & (idx >= s_lo) & (idx < s_hi)
            ei = np.stack([idx[sel] - s_lo, seg[sel] - lo]).astype(np.int32)      # rows: sources of that rank, columns: local destinations
            ci, ro, cw = O.coo_to_csr(ei, w[sel], s_hi - s_lo)
            csr_list.append(jg.CSR(t(ci), t(ro), t(cw)))
        xl = t(x[lo:hi].copy()).requires_grad_(True)
        z = jd.DistSpmm(jd.DistributedManager(), xl, csr_list, hi - lo)
        z.backward(t(x[lo:hi].copy()) * 0.5)          # the reference's rule: the same rounds on the gradient
        torch.cuda.synchronize()
        q.put((rank, lo, hi, y.cpu().numpy(), z.detach().cpu().numpy(), xl.grad.cpu().numpy()))
    except Exception as exc:
        q.put((rank, -1, -1, repr(exc)))
        raise
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("exchange", ["nccl", "peer"])
@pytest.mark.timeout(300)
def test_nccl_ranks(cuda, oracle, exchange):
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    import torch.multiprocessing as mp
    n, E, f = 40000, 600000, 128
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=nccl_worker, args=(r, world, port, n, E, f, q, exchange)) for r in range(world)]
    for p in procs:
        p.start()
    got = [q.get(timeout=240) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    assert all(g[1] >= 0 for g in got), [g[3] for g in got if g[1] < 0]
    idx, off, w, x = make_graph(11, n, E, f)
    want = oracle.aggregate(x, idx, off, w)
    _, scale = oracle.aggregate_f64(x, idx, off, w)
    for rank, lo, hi, y, z, gx in got:
        assert (np.abs(y - want[lo:hi]) / (scale[lo:hi] + 1e-30)).max() <= 1e-5
        assert (np.abs(z - want[lo:hi]) / (scale[lo:hi] + 1e-30)).max() <= 1e-5
        assert (np.abs(gx - 0.5 * want[lo:hi]) / (scale[lo:hi] + 1e-30)).max() <= 1e-5


def make_symmetric(seed, n, f, per_node=6):
    rng = np.random.default_rng(seed)
    a = rng.integers(0, n, size=per_node * n)
    b = rng.integers(0, n, size=per_node * n)
    wv = (rng.random(per_node * n) / per_node).astype(np.float32)
    src = np.concatenate([a, b]); dst = np.concatenate([b, a]); w = np.concatenate([wv, wv])
    order = np.argsort(dst, kind="stable")
    off = np.concatenate([[0], np.cumsum(np.bincount(dst, minlength=n))]).astype(np.int32)
    return src[order].astype(np.int32), off, w[order], rng.standard_normal((n, f)).astype(np.float32)


def train_worker(rank, world, port, n, f, hidden, classes, steps, q):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    from jittorgeometric_b200 import dist as jd
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    import datetime
    os.environ["TORCH_SYMM_MEM_DISABLE_MULTICAST"] = "1"
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank), timeout=datetime.timedelta(seconds=90))
    try:
        idx, off, w, x = make_symmetric(21, n, f)
        rng = np.random.default_rng(22)
        labels, mask = rng.integers(0, classes, size=n).astype(np.int64), rng.random(n) < 0.5
        part = jd.RowPartition(n, world)
        lo, hi = part.range(rank)
        t = lambda a: torch.from_numpy(a).cuda()
        g = jd.ShardedGraph(part, rank, *jd.shard_rows(t(idx), t(off), t(w), part, rank), exchange="nccl", mode="merged")
        mgr = jd.DistributedManager()
        model = jd.ShardedGCN(f, hidden, classes, layers=2, manager=mgr, device="cuda", seed=300 + rank, tf32=False)
        opt = torch.optim.SGD(model.parameters(), lr=0.5)
        losses = [jd.sharded_training_step(model, g, t(x[lo:hi].copy()), t(labels[lo:hi].copy()), t(mask[lo:hi].copy()), opt, mgr)
                  for _ in range(steps)]
        torch.cuda.synchronize()
        q.put((rank, 0, 0, [p.detach().cpu().numpy() for p in model.weights], losses))
    except Exception as exc:
        q.put((rank, -1, -1, repr(exc), None))
        raise
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_nccl_training_step(cuda):
    """Graph-parallel training (halo exchange forward and backward, weight gradients summed over
    the ranks) equals dense float64 training of the same model on the whole graph."""
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    import torch.multiprocessing as mp
    from jittorgeometric_b200 import dist as jd
    n, f, hidden, classes, steps = 3000, 32, 16, 5, 3
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=train_worker, args=(r, world, port, n, f, hidden, classes, steps, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = [q.get(timeout=240) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    assert all(g[1] >= 0 for g in got), [g[3] for g in got if g[1] < 0]
    idx, off, w, x = make_symmetric(21, n, f)
    rng = np.random.default_rng(22)
    labels, mask = rng.integers(0, classes, size=n).astype(np.int64), rng.random(n) < 0.5
    A = np.zeros((n, n))
    np.add.at(A, (np.repeat(np.arange(n), np.diff(off)), idx), w.astype(np.float64))
    A = torch.from_numpy(A)
    ref = jd.ShardedGCN(f, hidden, classes, layers=2, manager=None, seed=300)
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
        for have, want in zip(weights, W):
            assert np.abs(have - want.detach().numpy()).max() <= 1e-4


def test_training_step_on_one_gpu(cuda):
    """``ShardedGCN`` + ``sharded_training_step`` on the device kernels with a one-rank process group
    (the whole graph is the rank's shard): three SGD steps equal dense float64 training.  The
    multi-rank version of the same check needs two GPUs (``test_nccl_training_step``) or CPU ranks
    (tests/test_dist_cpu.py)."""
    import torch.distributed as dist
    from jittorgeometric_b200 import dist as jd
    n, f, hidden, classes, steps = 3000, 32, 16, 5, 3
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=0, world_size=1)
    try:
        idx, off, w, x = make_symmetric(21, n, f)
        rng = np.random.default_rng(22)
        labels, mask = rng.integers(0, classes, size=n).astype(np.int64), rng.random(n) < 0.5
        t = lambda a: torch.from_numpy(a).cuda()
        part = jd.RowPartition(n, 1)
        g = jd.ShardedGraph(part, 0, t(idx), t(off), t(w), exchange="nccl", mode="merged")
        mgr = jd.DistributedManager()
        model = jd.ShardedGCN(f, hidden, classes, layers=2, manager=mgr, device="cuda", seed=300, tf32=False)
        opt = torch.optim.SGD(model.parameters(), lr=0.5)
        losses = [jd.sharded_training_step(model, g, t(x), t(labels), t(mask), opt, mgr) for _ in range(steps)]
        torch.cuda.synchronize()
        weights = [p.detach().cpu().numpy() for p in model.weights]
    finally:
        dist.destroy_process_group()
    A = np.zeros((n, n))
    np.add.at(A, (np.repeat(np.arange(n), np.diff(off)), idx), w.astype(np.float64))
    A = torch.from_numpy(A)
    ref = jd.ShardedGCN(f, hidden, classes, layers=2, manager=None, seed=300)
    W = [p.detach().double().requires_grad_(True) for p in ref.weights]
    X, L, M = torch.from_numpy(x).double(), torch.from_numpy(labels), torch.from_numpy(mask)
    for k in range(steps):
        h = X
        for wt in W:
            h = (A @ h) @ wt
        loss = torch.nn.functional.nll_loss(torch.log_softmax(h, dim=1)[M], L[M])
        grads = torch.autograd.grad(loss, W)
        assert abs(losses[k] - float(loss.detach())) <= 1e-4 * abs(float(loss.detach())) + 1e-5
        W = [(wt - 0.5 * gr).detach().requires_grad_(True) for wt, gr in zip(W, grads)]
    for have, want in zip(weights, W):
        assert np.abs(have - want.detach().numpy()).max() <= 1e-4
