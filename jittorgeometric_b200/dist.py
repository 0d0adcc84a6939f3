"""1-D destination-row partition of the aggregation across the GPUs of one box.

The reference's graph-parallel path (examples/dist_gcn/dist_gcn.py:73-88, ops/distspmm.py:16-61)
gives every rank the in-edges of its own destination rows, split offline into one sub-CSR per
source rank, and runs P rounds of host-staged pickled ``MPI.bcast`` + cuSPARSE.  Here each rank

* owns a contiguous range of destination rows and the matching rows of the feature matrix
  (:class:`RowPartition`; equal ranges of ``ceil(N / P)`` rows, which balances edges when vertex
  ids carry no degree order),
* splits its in-edges on device into interior entries (source row owned, read from the rank's own
  shard) and halo entries (source row remote),
* brings the other ranks' feature shards over NVLink into a local buffer laid out by global row
  id - copy-engine pulls from peer memory (:class:`PeerExchange`) or one NCCL all-gather - while
  the interior aggregation runs, then aggregates the halo entries from that buffer and adds them
  to the same output rows (fixed order: interior, then halo, so results are run-to-run
  identical).  Kernels only ever gather from local memory.

One process per GPU; ``torch.distributed`` supplies the communicator.  The compute backend is
pluggable so the partition and exchange logic can be exercised by CPU ranks over ``gloo``.
"""
import os

import torch
import torch.distributed as dist

from . import ops
from ._lib import check, lib, ptr, stream_for, workspace
from .data import CSC, CSR


class RowPartition:
    """Contiguous destination-row ranges: rank q owns rows [q * pad, min((q + 1) * pad, n))."""

    def __init__(self, n, world):
        if world < 1:
            raise ValueError("world size must be positive")
        self.n, self.world = int(n), int(world)
        self.pad = (self.n + self.world - 1) // self.world if self.n else 0
        self.bounds = [min(q * self.pad, self.n) for q in range(self.world + 1)]

    def range(self, rank):
        return self.bounds[rank], self.bounds[rank + 1]

    def n_local(self, rank):
        lo, hi = self.range(rank)
        return hi - lo

    def owner(self, row):
        return min(int(row) // self.pad, self.world - 1) if self.pad else 0


class DeviceBackend:
    """The CUDA library: interior/halo split and aggregation kernels."""

    def split(self, idx, off, w, lo, hi):
        nnz, n_rows, dev = idx.numel(), off.numel() - 1, idx.device
        mk_i = lambda m: torch.empty(max(m, 1), dtype=torch.int32, device=dev)
        mk_f = lambda m: torch.empty(max(m, 1), dtype=torch.float32, device=dev)
        ii, io, iw = mk_i(nnz), mk_i(n_rows + 1), mk_f(nnz)
        hi_, ho, hw = mk_i(nnz), mk_i(n_rows + 1), mk_f(nnz)
        counts = torch.zeros(2, dtype=torch.int64, device=dev)
        ws = workspace(lib().jg_partition_split_workspace_bytes(nnz), dev)
        check(lib().jg_partition_split(ptr(idx), ptr(off), ptr(w), n_rows, nnz, int(lo), int(hi), ptr(ii), ptr(io),
                                       ptr(iw), ptr(hi_), ptr(ho), ptr(hw), ptr(counts), ptr(ws), ws.numel(),
                                       stream_for(idx)), "jg_partition_split")
        ni, nh = (int(v) for v in counts.tolist())
        return (ii[:ni].clone(), io[: n_rows + 1], iw[:ni].clone()), (hi_[:nh].clone(), ho[: n_rows + 1], hw[:nh].clone())

    def plan(self, off, nnz):
        return ops.SpmmPlan(off, nnz)

    def aggregate(self, x, idx, off, w, n_out, plan, out=None, accumulate=False):
        return ops.segment_aggregate(x, idx, off, w, n_out=n_out, plan=plan, out=out, accumulate=accumulate)


class PeerExchange:
    """Shard exchange by peer-to-peer copies over NVLink, driven by the copy engines.

    An NCCL all-gather runs as a kernel, and the aggregation kernels are persistent grids that
    fill every SM: whichever starts first keeps the other waiting, so nothing overlaps.  Here every
    rank publishes its shard in a buffer its peers can map (``torch.distributed`` symmetric
    memory) and pulls the P-1 remote shards into its local gather buffer with plain device-to-device
    copies on a side stream; those are DMA transfers that need no SM, so they proceed underneath
    the interior aggregation, and the halo entries of each source rank are aggregated as soon as
    that rank's shard has arrived (one event per pull).  Two small barriers order the exchange: one
    after the shard is published (before anyone pulls), one after the pulls (before the shard may be
    overwritten).
    """

    BARRIER_TIMEOUT_MS = 20000

    def __init__(self, part, rank, group=None):
        import torch.distributed._symmetric_memory as symm
        self._symm = symm
        self.part, self.rank = part, rank
        self.group = group if group is not None else dist.group.WORLD
        self.sides = [torch.cuda.Stream() for _ in range(max(1, int(os.environ.get("JG_PEER_STREAMS", "1"))))]
        self._bufs = {}

    def buffer(self, f, device):
        """The rank's publishable feature shard of width ``f`` (``pad`` rows; write features here to
        skip one copy per aggregation)."""
        entry = self._bufs.get(f)
        if entry is None:
            t = self._symm.empty((self.part.pad, f), dtype=torch.float32, device=device)
            t.zero_()
            hdl = self._symm.rendezvous(t, self.group.group_name)
            entry = (t, hdl)
            self._bufs[f] = entry
        return entry

    def start(self, xp, full):
        f = xp.shape[1]
        buf, hdl = self.buffer(f, xp.device)
        if xp.data_ptr() != buf.data_ptr():
            buf.copy_(xp)
        hdl.barrier(channel=0, timeout_ms=self.BARRIER_TIMEOUT_MS)       # every shard is published
        cur = torch.cuda.current_stream()
        pad, world = self.part.pad, self.part.world
        events = {}
        for k, q in enumerate(self.order()):
            side = self.sides[k % len(self.sides)]                       # two pulls in flight
            if k < len(self.sides):
                side.wait_stream(cur)
            with torch.cuda.stream(side):
                peer = hdl.get_buffer(q, (pad, f), torch.float32)
                full[q * pad:(q + 1) * pad].copy_(peer)
                events[q] = side.record_event()
        return _PeerHandle(self, hdl, cur, events)

    def order(self):
        """Peers in the order their shards are pulled: staggered so that no two ranks start on the
        same peer."""
        return [(self.rank + step) % self.part.world for step in range(1, self.part.world)]


class _PeerHandle:
    def __init__(self, ex, hdl, cur, events):
        self.ex, self.hdl, self.cur, self.events = ex, hdl, cur, events

    def wait_peer(self, q):
        """Orders later work on the calling stream after the shard of rank ``q`` has arrived."""
        self.cur.wait_event(self.events[q])

    def wait(self):
        for side in self.ex.sides:
            self.cur.wait_stream(side)
        self.hdl.barrier(channel=1, timeout_ms=PeerExchange.BARRIER_TIMEOUT_MS)   # every pull has finished


class ShardedGraph:
    """One rank's share of a row-partitioned graph: the in-edges of its destination rows.

    ``idx`` holds GLOBAL source ids, ``off`` the offsets of the rank's own rows (CSC of the shard).
    """

    def __init__(self, part, rank, idx, off, w, backend=None, group=None, exchange="nccl"):
        self.part, self.rank, self.group = part, rank, group
        self.backend = backend or DeviceBackend()
        self.exchange = PeerExchange(part, rank, group) if exchange == "peer" else None
        self.lo, self.hi = part.range(rank)
        self.n_local = self.hi - self.lo
        if off.numel() != self.n_local + 1:
            raise RuntimeError(f"offsets describe {off.numel() - 1} rows, the rank owns {self.n_local}")
        self.interior, self.halo = self.backend.split(idx, off, w, self.lo, self.hi)
        self.interior_plan = self.backend.plan(self.interior[1], self.interior[0].numel())
        self.halo_plan = self.backend.plan(self.halo[1], self.halo[0].numel())
        # Optional (JG_HALO_PIPELINE=1): halo entries grouped by the rank that owns their source row
        # (ids rebased to that rank's shard), in pull order, so that each group can be aggregated as
        # soon as its shard has arrived.  Off by default: on 4 GPUs the aggregation kernels running
        # underneath the remaining pulls slowed both down (16.7 ms against 10.4 ms per sweep).
        self.halo_groups = []
        if self.exchange is not None and os.environ.get("JG_HALO_PIPELINE", "0") == "1":
            rest = self.halo
            for q in self.exchange.order():
                q_lo, q_hi = part.range(q)
                mine, rest = self.backend.split(rest[0], rest[1], rest[2], q_lo, q_hi)
                self.halo_groups.append((q, mine, self.backend.plan(mine[1], mine[0].numel())))
        self._full = {}

    def _gather_buffer(self, f, like):
        key = (f, like.device, like.dtype)
        buf = self._full.get(key)
        if buf is None:
            buf = torch.empty((self.part.world * self.part.pad, f), dtype=like.dtype, device=like.device)
            self._full[key] = buf
        return buf

    def _padded(self, x):
        if x.shape[0] == self.part.pad:
            return x
        if x.shape[0] != self.n_local:
            raise RuntimeError(f"x has {x.shape[0]} rows, the rank owns {self.n_local}")
        xp = torch.zeros((self.part.pad, x.shape[1]), dtype=x.dtype, device=x.device)
        xp[: self.n_local] = x
        return xp

    def aggregate(self, x, gather=None):
        """``y[v] = sum_{(u -> v)} w * x_global[u]`` for the rank's own rows ``v``.

        ``x`` holds the rank's rows of the feature matrix (``n_local`` rows, or ``pad`` rows with
        a zero tail).  ``gather(shard, full)`` fills ``full`` with every rank's padded shard and
        returns a handle whose ``wait()`` orders later work after it; the default is the
        copy-engine peer exchange (``exchange="peer"``) or an asynchronous
        ``all_gather_into_tensor`` on the process group (``exchange="nccl"``)."""
        f = x.shape[1]
        xp = self._padded(x)
        full = self._gather_buffer(f, xp)
        if gather is None and self.exchange is not None:
            handle = self.exchange.start(xp, full)
        elif gather is None:
            handle = dist.all_gather_into_tensor(full, xp, group=self.group, async_op=True)
        else:
            handle = gather(xp, full)
        # the rank's own rows while the shards travel
        y = self.backend.aggregate(xp, self.interior[0], self.interior[1], self.interior[2], self.n_local,
                                   self.interior_plan)
        if self.halo_groups and hasattr(handle, "wait_peer"):
            pad = self.part.pad
            for q, grp, plan in self.halo_groups:
                handle.wait_peer(q)
                if grp[0].numel():
                    self.backend.aggregate(full[q * pad:(q + 1) * pad], grp[0], grp[1], grp[2], self.n_local, plan,
                                           out=y, accumulate=True)
            handle.wait()
            return y
        if handle is not None:
            handle.wait()
        if self.halo[0].numel():
            self.backend.aggregate(full, self.halo[0], self.halo[1], self.halo[2], self.n_local, self.halo_plan,
                                   out=y, accumulate=True)
        return y


def shard_rows(idx, off, w, part, rank):
    """Cuts the rows of one rank out of a full CSC (global ids): helper for benchmarks and tests
    that build the whole graph on every rank and keep only their share."""
    lo, hi = part.range(rank)
    s, e = int(off[lo]), int(off[hi])
    return idx[s:e].contiguous(), (off[lo: hi + 1] - off[lo]).contiguous(), w[s:e].contiguous()


# ------------------------------------------------------------------------------ reference API mirror
class DistributedManager:
    """``rank`` / ``size`` / ``broadcast`` of the reference's manager
    (utils/distributed_utils.py:8-74) on a ``torch.distributed`` group: device-to-device NCCL
    broadcast instead of pickled host ``MPI.bcast``."""

    def __init__(self, group=None):
        self.group = group
        self.rank = dist.get_rank(group)
        self.size = dist.get_world_size(group)

    def broadcast(self, x, src, rows=None):
        """Every rank receives rank ``src``'s tensor; ``rows`` is the row count of that tensor when
        ranks hold different numbers of rows."""
        if self.rank == src:
            buf = x.contiguous()
        else:
            n = x.shape[0] if rows is None else rows
            buf = torch.empty((n,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.broadcast(buf, src=dist.get_global_rank(self.group, src) if self.group is not None else src, group=self.group)
        return buf


def DistSpmm(dist_mgr, x, csr_list, local_vnum, trans_A=True, trans_B=False, aggregate=None):
    """``sum_src op(A_src) @ x_src`` (ops/distspmm.py:16-61): ``csr_list[src]`` holds the edges from
    the rows of rank ``src`` (its CSR rows) to this rank's ``local_vnum`` destinations (its
    columns).  One broadcast round per source rank, as in the reference; forward only.  The
    optimised single-exchange path is :meth:`ShardedGraph.aggregate`."""
    if trans_B or not trans_A:
        raise RuntimeError("DistSpmm: only trans_A=True, trans_B=False (the reference's call) is supported")
    result = None
    for src in range(dist_mgr.size):
        csr = csr_list[src]
        v_src = csr.row_offset.numel() - 1
        fb = dist_mgr.broadcast(x, src, rows=v_src)
        t = ops._transposed_of(csr, n_cols=local_vnum)
        plan = ops._plan_of(t, t.column_offset, t.row_indices.numel())
        if result is None:
            result = ops.segment_aggregate(fb, t.row_indices, t.column_offset, t.edge_weight, n_out=local_vnum, plan=plan)
        else:
            ops.segment_aggregate(fb, t.row_indices, t.column_offset, t.edge_weight, n_out=local_vnum, plan=plan,
                                  out=result, accumulate=True)
    return result
