"""1-D destination-row partition of the aggregation across the GPUs of one box.

The reference's graph-parallel path (examples/dist_gcn/dist_gcn.py:73-88, ops/distspmm.py:16-61)
gives every rank the in-edges of its own destination rows, split offline into one sub-CSR per
source rank, and runs P rounds of host-staged pickled ``MPI.bcast`` + cuSPARSE.  Here each rank

* owns a contiguous range of destination rows and the matching rows of the feature matrix
  (:class:`RowPartition`; equal ranges of ``ceil(N / P)`` rows, which balances edges when vertex
  ids carry no degree order),
* splits its in-edges on device into interior entries (source row owned, read from the rank's own
  shard) and halo entries (source row remote),
* finds, once per graph, the distinct remote rows its halo entries reference (with skewed degrees
  a minority of all remote rows) and tells their owners; per aggregation every rank packs the rows
  its peers asked for and the packed segments travel over NVLink into a local halo buffer -
  copy-engine pulls from peer memory (:class:`PeerTransport`) or one NCCL all-to-all
  (:class:`CollectiveTransport`) - while the interior aggregation runs; the halo entries are then
  aggregated from that buffer and added to the same output rows (fixed order: interior, then
  halo, so results are run-to-run identical).  Kernels only ever gather from local memory.

One process per GPU; ``torch.distributed`` supplies the communicator.  The compute backend is
pluggable so the partition and exchange logic can be exercised by CPU ranks over ``gloo``.
"""
import torch
import torch.distributed as dist

from . import ops
from ._lib import check, lib, ptr, stream_for, workspace


class RowPartition:
    """Contiguous destination-row ranges.  By default rank q owns rows
    [q * pad, min((q + 1) * pad, n)) with ``pad = ceil(n / world)``; ``bounds`` (``world + 1``
    non-decreasing values from 0 to n) gives the ranges explicitly, e.g. the offsets of a
    partition file after the nodes have been reordered by part
    (partition/distchunk_manager.py:88-93)."""

    def __init__(self, n, world, bounds=None):
        if world < 1:
            raise ValueError("world size must be positive")
        self.n, self.world = int(n), int(world)
        self.pad = (self.n + self.world - 1) // self.world if self.n else 0
        if bounds is None:
            self.bounds = [min(q * self.pad, self.n) for q in range(self.world + 1)]
        else:
            self.bounds = [int(b) for b in bounds]
            if (len(self.bounds) != self.world + 1 or self.bounds[0] != 0 or self.bounds[-1] != self.n
                    or any(a > b for a, b in zip(self.bounds[:-1], self.bounds[1:]))):
                raise ValueError(f"bounds must be {self.world + 1} non-decreasing values from 0 to {self.n}")

    def range(self, rank):
        return self.bounds[rank], self.bounds[rank + 1]

    def n_local(self, rank):
        lo, hi = self.range(rank)
        return hi - lo

    def owner(self, row):
        import bisect
        return min(max(bisect.bisect_right(self.bounds, int(row)) - 1, 0), self.world - 1)


class DeviceBackend:
    """The CUDA library: interior/halo split, halo map, row packing and aggregation kernels."""

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

    def halo_map(self, halo_idx, n_global, bounds, lo=0, hi=0, base=0):
        """Distinct remote rows a shard references: ``(needed ids ascending, indices re-addressed -
        own rows [lo, hi) to ``idx - lo``, remote rows to ``base`` + slot in the packed halo buffer -
        and the rows needed from every owner)``."""
        nnz, dev = halo_idx.numel(), halo_idx.device
        pos = torch.empty(n_global + 1, dtype=torch.int32, device=dev)
        needed = torch.empty(max(min(nnz, n_global), 1), dtype=torch.int32, device=dev)
        remapped = torch.empty(max(nnz, 1), dtype=torch.int32, device=dev)
        ws = workspace(lib().jg_halo_map_workspace_bytes(n_global), dev)
        check(lib().jg_halo_map_build(ptr(halo_idx), nnz, n_global, int(lo), int(hi), int(base), ptr(pos), ptr(needed),
                                      ptr(remapped), ptr(ws), ws.numel(), stream_for(halo_idx)), "jg_halo_map_build")
        at = pos[torch.tensor(bounds, device=dev, dtype=torch.long)].tolist()
        counts = [at[q + 1] - at[q] for q in range(len(bounds) - 1)]
        return needed[: at[-1]].clone(), remapped[:nnz].clone(), counts

    def gather_rows(self, x, rows, rebase, out):
        n = rows.numel()
        check(lib().jg_gather_rows_f32(ptr(out), ptr(x), ptr(rows), n, x.shape[1], int(rebase), stream_for(x)),
              "jg_gather_rows_f32")
        return out

    def plan(self, off, nnz):
        return ops.SpmmPlan(off, nnz)

    def aggregate(self, x, idx, off, w, n_out, plan, out=None, accumulate=False, bias=None, relu=False):
        return ops.segment_aggregate(x, idx, off, w, n_out=n_out, plan=plan, out=out, accumulate=accumulate, bias=bias,
                                     relu=relu)


class _Done:
    def wait(self):
        pass

    def release(self):
        pass


class _WorkHandle:
    """An asynchronous ``torch.distributed`` collective."""

    def __init__(self, work):
        self.work = work

    def wait(self):
        self.work.wait()

    def release(self):
        pass


class CollectiveTransport:
    """Row exchange with ``torch.distributed`` collectives (NCCL on GPUs, gloo on CPU ranks):
    one ``all_to_all_single`` with per-peer row counts."""

    def __init__(self, group=None):
        self.group = group

    def send_buffer(self, rows, f, like):
        return torch.empty((max(rows, 1), f), dtype=like.dtype, device=like.device)

    # set-up collectives: the matrix of request counts and the requested row ids
    def all_gather_counts(self, g, counts):
        if g.part.world == 1:
            return [counts.tolist()]
        out = [torch.empty_like(counts) for _ in range(g.part.world)]
        dist.all_gather(out, counts, group=self.group)
        return [t.tolist() for t in out]

    def all_to_all_ids(self, g, needed, recv_counts, send_counts):
        if g.part.world == 1:
            return needed[:0]
        out = torch.empty(max(sum(send_counts), 1), dtype=needed.dtype, device=needed.device)
        src = needed if needed.numel() else torch.empty(1, dtype=needed.dtype, device=needed.device)
        dist.all_to_all_single(out[: sum(send_counts)], src[: sum(recv_counts)], output_split_sizes=list(send_counts),
                               input_split_sizes=list(recv_counts), group=self.group)
        return out[: sum(send_counts)]

    def exchange(self, g, send, recv, f):
        if g.part.world == 1:
            return _Done()
        send_split = [int(c) for c in g.send_counts]
        recv_split = [int(c) for c in g.recv_counts]
        return _WorkHandle(dist.all_to_all_single(recv[: sum(recv_split)], send[: sum(send_split)],
                                                  output_split_sizes=recv_split, input_split_sizes=send_split,
                                                  group=self.group, async_op=True))


class PeerTransport(CollectiveTransport):
    """Row exchange by peer-to-peer copies over NVLink, driven by the copy engines.

    An NCCL collective runs as a kernel, and the aggregation kernels are persistent grids that
    fill every SM: whichever starts first keeps the other waiting, so nothing overlaps.  Here every
    rank packs the rows its peers asked for into a buffer the peers can map (``torch.distributed``
    symmetric memory) and each rank pulls its segments with plain device-to-device copies on a side
    stream; those are DMA transfers that need no SM, so they proceed underneath the interior
    aggregation.  Two small barriers order the exchange: one after the buffers are packed (before
    anyone pulls), one after the pulls (before a buffer may be packed again).
    """

    BARRIER_TIMEOUT_MS = 20000

    def __init__(self, group=None):
        import torch.distributed._symmetric_memory as symm
        self._symm = symm
        self.group = group                                                # set-up collectives
        self.symm_group = group if group is not None else dist.group.WORLD
        self.side = torch.cuda.Stream()
        self._bufs = {}

    def send_buffer(self, rows, f, like):
        """Symmetric buffer of ``rows`` x ``f`` (the same shape on every rank)."""
        rows = max(rows, 1)
        entry = self._bufs.get((rows, f))
        if entry is None:
            t = self._symm.empty((rows, f), dtype=torch.float32, device=like.device)
            hdl = self._symm.rendezvous(t, self.symm_group.group_name)
            entry = (t, hdl)
            self._bufs[(rows, f)] = entry
        return entry[0]

    def exchange(self, g, send, recv, f):
        hdl = self._bufs[(send.shape[0], f)][1]
        hdl.barrier(channel=0, timeout_ms=self.BARRIER_TIMEOUT_MS)       # every send buffer is packed
        cur = torch.cuda.current_stream()
        self.side.wait_stream(cur)
        world, rank = g.part.world, g.rank
        with torch.cuda.stream(self.side):
            for step in range(1, world):
                q = (rank + step) % world                                  # staggered: no two ranks start on the same peer
                n = int(g.recv_counts[q])
                if n == 0:
                    continue
                peer = hdl.get_buffer(q, tuple(send.shape), torch.float32)
                src0 = int(g.peer_send_offset[q])                          # where rank q packed the rows meant for this rank
                dst0 = int(g.recv_offset[q])
                recv[dst0:dst0 + n].copy_(peer[src0:src0 + n])
            landed = torch.cuda.Event()
            landed.record(self.side)
        return _PeerHandle(hdl, landed)


class _PeerHandle:
    """``wait``: the current stream waits for THIS exchange's pulls (an event, so that pulls of later
    exchanges already queued on the side stream are not waited for).  ``release``: the barrier that
    tells every rank its send buffer has been read and may be packed again; it is issued after the
    aggregation has been queued, so no rank idles in it before its own kernel starts."""

    def __init__(self, hdl, landed):
        self.hdl, self.landed = hdl, landed

    def wait(self):
        torch.cuda.current_stream().wait_event(self.landed)

    def release(self):
        self.hdl.barrier(channel=1, timeout_ms=PeerTransport.BARRIER_TIMEOUT_MS)   # every pull has finished


class ShardedGraph:
    """One rank's share of a row-partitioned graph: the in-edges of its destination rows.

    ``idx`` holds GLOBAL source ids, ``off`` the offsets of the rank's own rows (CSC of the shard).
    Construction is collective (every rank of the group builds its graph at the same time): the
    ranks tell each other which rows they need.
    """

    def __init__(self, part, rank, idx, off, w, backend=None, group=None, exchange="nccl", transport=None,
                 setup=True, mode="merged"):
        self.part, self.rank, self.group = part, rank, group
        self.backend = backend or DeviceBackend()
        self.lo, self.hi = part.range(rank)
        self.n_local = self.hi - self.lo
        if off.numel() != self.n_local + 1:
            raise RuntimeError(f"offsets describe {off.numel() - 1} rows, the rank owns {self.n_local}")
        if transport is None:
            transport = PeerTransport(group) if exchange == "peer" else CollectiveTransport(group)
        self.transport = transport
        if mode not in ("merged", "overlap"):
            raise ValueError("mode must be 'merged' or 'overlap'")
        self.mode = mode
        if mode == "overlap":
            # own-source entries aggregated while the halo rows travel, halo entries added afterwards
            self.interior, halo = self.backend.split(idx, off, w, self.lo, self.hi)
            self.interior_plan = self.backend.plan(self.interior[1], self.interior[0].numel())
            # compact halo: distinct remote rows, ascending (= grouped by owner), and the halo entries
            # re-addressed into the packed buffer those rows will arrive in
            self.needed, halo_idx, self.recv_counts = self.backend.halo_map(halo[0], part.n, part.bounds)
            self.halo = (halo_idx, halo[1], halo[2])
            self.halo_plan = self.backend.plan(self.halo[1], self.halo[0].numel())
        else:
            # one aggregation over one buffer [own rows | packed halo rows]: every entry keeps its
            # place in its row, so each row is summed in exactly the order the unpartitioned graph
            # sums it, once, with no second pass over the output
            self.needed, m_idx, self.recv_counts = self.backend.halo_map(idx, part.n, part.bounds, self.lo, self.hi,
                                                                         self.n_local)
            self.merged = (m_idx, off, w)
            self.merged_plan = self.backend.plan(off, idx.numel())
        self.recv_offset = [sum(self.recv_counts[:q]) for q in range(part.world)]
        self.n_halo = sum(self.recv_counts)
        self._recv = {}
        if setup:
            self._setup_requests()

    # ---- set-up: who sends which rows to whom
    def _setup_requests(self):
        dev = self.needed.device
        counts = torch.tensor(self.recv_counts, dtype=torch.int64, device=dev)
        matrix = self.transport.all_gather_counts(self, counts)           # matrix[r][q] = rows rank r needs from rank q
        send_counts = [int(matrix[r][self.rank]) for r in range(self.part.world)]
        send_rows = self.transport.all_to_all_ids(self, self.needed, self.recv_counts, send_counts)
        self.apply_setup(matrix, send_rows)

    def apply_setup(self, matrix, send_rows):
        """``matrix[r][q]`` = rows rank r needs from rank q; ``send_rows`` = the global ids of this
        rank's rows its peers asked for, grouped by requesting rank in rank order."""
        world = self.part.world
        self.count_matrix = matrix
        self.send_counts = [int(matrix[r][self.rank]) for r in range(world)]
        self.send_offset = [sum(self.send_counts[:r]) for r in range(world)]
        # in rank q's send buffer the rows for rank r start after those for ranks 0..r-1
        self.peer_send_offset = [sum(int(matrix[r2][q]) for r2 in range(self.rank)) for q in range(world)]
        self.n_send = sum(self.send_counts)
        self.max_send = max(sum(int(matrix[r][q]) for r in range(world)) for q in range(world))
        self.send_rows = send_rows

    # ---- per aggregation
    def feature_buffer(self, f, like):
        """Where a caller should write the rank's feature rows to save a copy per aggregation (the
        head of the buffer the merged aggregation reads); any tensor with ``n_local`` rows works."""
        if self.mode == "merged":
            return self._recv_buffer(f, like)[: self.n_local]
        return torch.empty((self.n_local, f), dtype=like.dtype, device=like.device)

    def _recv_buffer(self, f, like):
        buf = self._recv.get(f)
        if buf is None:
            rows = self.n_halo + (self.n_local if self.mode == "merged" else 0)
            buf = torch.empty((max(rows, 1), f), dtype=like.dtype, device=like.device)
            self._recv[f] = buf
        return buf

    def aggregate(self, x, bias=None, relu=False):
        """``y[v] = sum_{(u -> v)} w * x_global[u]`` for the rank's own rows ``v``; ``x`` holds the
        rank's ``n_local`` rows of the feature matrix (extra rows are ignored).  With autograd the
        gradient is the same aggregation applied to the incoming gradient, which is the true
        gradient for a symmetric matrix (the normalised adjacency of an undirected graph) - the
        rule the reference's ``DistSpmmFunc.grad`` follows (ops/distspmm.py:42-57).  ``bias`` / ``relu``
        apply ``act(y + bias)``; without autograd and in the merged schedule they are fused into the
        aggregation kernel's store."""
        if torch.is_grad_enabled() and x.requires_grad:
            y = _ShardedAggregate.apply(x, self)
        elif bias is not None or relu:
            return self._aggregate(x, bias, relu)
        else:
            return self._aggregate(x)
        if bias is not None:
            y = y + bias
        return torch.relu(y) if relu else y

    def _aggregate(self, x, bias=None, relu=False):
        return self.finish(self.start(x), bias, relu)

    def start(self, x):
        """First half of an aggregation: packs the rows the peers asked for and starts the exchange.
        Several aggregations may be started before the first is finished; their exchanges then run
        underneath the aggregation kernels of the earlier ones.  Forward only."""
        if x.shape[0] < self.n_local:
            raise RuntimeError(f"x has {x.shape[0]} rows, the rank owns {self.n_local}")
        f = x.shape[1]
        buf = self._recv_buffer(f, x)
        send = self.transport.send_buffer(self.max_send, f, x)
        if self.n_send:
            self.backend.gather_rows(x, self.send_rows, self.lo, send)       # rows the peers asked for
        if self.mode == "merged":
            handle = self.transport.exchange(self, send, buf[self.n_local:], f)
            if x.data_ptr() != buf.data_ptr():
                buf[: self.n_local].copy_(x[: self.n_local])
        else:
            handle = self.transport.exchange(self, send, buf, f)
        return (x, buf, handle)

    def finish(self, pending, bias=None, relu=False):
        """Second half: waits for the halo rows of ``pending`` (from :meth:`start`) and aggregates."""
        x, buf, handle = pending
        if self.mode == "merged":
            handle.wait()
            if bias is not None or relu:
                y = self.backend.aggregate(buf, self.merged[0], self.merged[1], self.merged[2], self.n_local,
                                           self.merged_plan, bias=bias, relu=relu)
            else:
                y = self.backend.aggregate(buf, self.merged[0], self.merged[1], self.merged[2], self.n_local,
                                           self.merged_plan)
            handle.release()
            return y
        # the rank's own rows while the halo rows travel
        y = self.backend.aggregate(x, self.interior[0], self.interior[1], self.interior[2], self.n_local,
                                   self.interior_plan)
        handle.wait()
        if self.halo[0].numel():
            self.backend.aggregate(buf, self.halo[0], self.halo[1], self.halo[2], self.n_local, self.halo_plan,
                                   out=y, accumulate=True)
        handle.release()
        if bias is not None:
            y += bias
        return y.relu_() if relu else y


class _ShardedAggregate(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, graph):
        ctx.graph = graph
        return graph._aggregate(x.detach())

    @staticmethod
    def backward(ctx, grad_output):
        return ctx.graph._aggregate(grad_output.contiguous()), None


def shard_rows(idx, off, w, part, rank):
    """Cuts the rows of one rank out of a full CSC (global ids): helper for benchmarks and tests
    that build the whole graph on every rank and keep only their share."""
    lo, hi = part.range(rank)
    s, e = int(off[lo]), int(off[hi])
    return idx[s:e].contiguous(), (off[lo: hi + 1] - off[lo]).contiguous(), w[s:e].contiguous()


# ------------------------------------------------------------------------------ reference API mirror
class DistributedManager:
    """``rank`` / ``size`` / ``broadcast`` / parameter synchronisation of the reference's manager
    (utils/distributed_utils.py:8-74) on a ``torch.distributed`` group: device-to-device
    collectives (NCCL on GPUs) instead of pickled host ``MPI.bcast`` / ``MPI.Allreduce``."""

    def __init__(self, group=None):
        self.group = group
        self.rank = dist.get_rank(group)
        self.size = dist.get_world_size(group)

    def _global(self, rank):
        return dist.get_global_rank(self.group, rank) if self.group is not None else rank

    def broadcast(self, x, src, rows=None):
        """Every rank receives rank ``src``'s tensor; ``rows`` is the row count of that tensor when
        ranks hold different numbers of rows."""
        if self.rank == src:
            buf = x.contiguous()
        else:
            n = x.shape[0] if rows is None else rows
            buf = torch.empty((n,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.broadcast(buf, src=self._global(src), group=self.group)
        return buf

    def broadcast_args(self, args):
        """Rank 0's Python object on every rank (utils/distributed_utils.py:30-31)."""
        box = [args]
        dist.broadcast_object_list(box, src=self._global(0), group=self.group)
        return box[0]

    @staticmethod
    def _tensors(model):
        return list(model.parameters()) if hasattr(model, "parameters") else list(model)

    def _bucket_all_reduce(self, tensors, async_op=False):
        """One all-reduce over the concatenation of ``tensors`` (a launch per tensor would be
        latency-bound for the handful of small weight matrices of a GNN)."""
        flat = torch.cat([t.detach().reshape(-1) for t in tensors]) if tensors else None
        work = dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=self.group, async_op=async_op) if tensors else None
        return flat, work

    @staticmethod
    def _unpack(flat, tensors, scale, into):
        at = 0
        for t in tensors:
            n = t.numel()
            into(t).copy_((flat[at: at + n] * scale).view_as(t))
            at += n

    def synchronize_model_parameters(self, model):
        """Replaces every parameter by its mean over the ranks
        (utils/distributed_utils.py:33-37)."""
        self.finalize_synchronization(self.synchronize_model_parameters_non_blocking(model))

    def synchronize_model_parameters_non_blocking(self, model):
        """Starts the averaging and returns a handle for :meth:`finalize_synchronization`
        (utils/distributed_utils.py:39-57)."""
        tensors = self._tensors(model)
        flat, work = self._bucket_all_reduce(tensors, async_op=True)
        return (tensors, flat, work)

    def finalize_synchronization(self, requests):
        tensors, flat, work = requests
        if work is not None:
            work.wait()
        if flat is not None:
            with torch.no_grad():
                self._unpack(flat, tensors, 1.0 / self.size, lambda t: t.data)

    def all_reduce_gradients(self, model, scale=1.0):
        """Sums the ``.grad`` of every parameter over the ranks (times ``scale``).  With a loss that
        is a sum over the rank's own nodes divided by a global count, this is the exact gradient of
        the whole-graph loss, so every rank takes the same optimiser step.  The reference's example
        never combines gradients (examples/dist_gcn/dist_gcn.py:144-170 steps on the local loss);
        it only offers the parameter averaging above."""
        tensors = [p for p in self._tensors(model) if p.grad is not None]
        flat, _ = self._bucket_all_reduce([p.grad for p in tensors])
        if flat is not None:
            self._unpack(flat, tensors, scale, lambda t: t.grad)


def _device_round(fb, csr, local_vnum, out=None):
    t = ops._transposed_of(csr, n_cols=local_vnum)
    plan = ops._plan_of(t, t.column_offset, t.row_indices.numel())
    return ops.segment_aggregate(fb, t.row_indices, t.column_offset, t.edge_weight, n_out=local_vnum, plan=plan,
                                 out=out, accumulate=out is not None)


def _dist_spmm_rounds(dist_mgr, x, csr_list, local_vnum, one_round):
    result = None
    for src in range(dist_mgr.size):
        v_src = csr_list[src].row_offset.numel() - 1
        fb = dist_mgr.broadcast(x, src, rows=v_src)
        result = one_round(fb, csr_list[src], local_vnum, result)
    return result


class _DistSpmmFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dist_mgr, csr_list, local_vnum, one_round):
        ctx.args = (dist_mgr, csr_list, local_vnum, one_round)
        return _dist_spmm_rounds(dist_mgr, x.detach().contiguous(), csr_list, local_vnum, one_round)

    @staticmethod
    def backward(ctx, grad_output):
        # the reference's rule (ops/distspmm.py:42-57): the same rounds on the incoming gradient,
        # which is the true gradient when the whole matrix is symmetric
        dist_mgr, csr_list, local_vnum, one_round = ctx.args
        if grad_output.shape[0] != local_vnum:
            raise RuntimeError("DistSpmm backward: gradient rows differ from local_vnum")
        return _dist_spmm_rounds(dist_mgr, grad_output.contiguous(), csr_list, local_vnum, one_round), None, None, None, None


def DistSpmm(dist_mgr, x, csr_list, local_vnum, trans_A=True, trans_B=False, aggregate=None):
    """``sum_src op(A_src) @ x_src`` (ops/distspmm.py:16-61): ``csr_list[src]`` holds the edges from
    the rows of rank ``src`` (its CSR rows) to this rank's ``local_vnum`` destinations (its
    columns).  One broadcast round per source rank, as in the reference, forward and backward.
    ``aggregate(fb, csr, local_vnum, out)`` replaces the device kernel of one round (CPU ranks in
    tests).  The optimised single-exchange path is :meth:`ShardedGraph.aggregate`."""
    if trans_B or not trans_A:
        raise RuntimeError("DistSpmm: only trans_A=True, trans_B=False (the reference's call) is supported")
    one_round = aggregate or _device_round
    if torch.is_grad_enabled() and x.requires_grad:
        return _DistSpmmFn.apply(x, dist_mgr, csr_list, local_vnum, one_round)
    return _dist_spmm_rounds(dist_mgr, x, csr_list, local_vnum, one_round)


class ShardedGCN(torch.nn.Module):
    """The model of the reference's graph-parallel example (examples/dist_gcn/dist_gcn.py:46-88):
    ``layers`` rounds of ``h <- (A_hat h) W`` with Glorot weights drawn on rank 0 and broadcast, then
    ``log_softmax``.  ``A_hat h`` is :meth:`ShardedGraph.aggregate` (one compact halo exchange per
    layer) instead of ``P`` broadcast rounds.  ``relu=True`` adds the activation between layers that
    the single-GPU example has and the graph-parallel one omits."""

    def __init__(self, in_channels, hidden_channels, out_channels, layers=2, manager=None, relu=False,
                 device=None, seed=0):
        super().__init__()
        widths = [in_channels] + [hidden_channels] * (layers - 1) + [out_channels]
        gen = torch.Generator().manual_seed(seed)
        self.weights = torch.nn.ParameterList()
        for a, b in zip(widths[:-1], widths[1:]):
            bound = (6.0 / (a + b)) ** 0.5                      # nn/inits.py:19-22
            w = (torch.rand((a, b), generator=gen) * 2 - 1) * bound
            self.weights.append(torch.nn.Parameter(w.to(device) if device is not None else w))
        self.relu = relu
        self.manager = manager
        self.sync_parameters()

    def sync_parameters(self):
        """Rank 0's weights on every rank (examples/dist_gcn/dist_gcn.py:63-70)."""
        if self.manager is None or self.manager.size == 1:
            return
        with torch.no_grad():
            for w in self.weights:
                w.copy_(self.manager.broadcast(w.data, 0))

    def forward(self, x, graph):
        h = x
        last = len(self.weights) - 1
        for i, w in enumerate(self.weights):
            h = graph.aggregate(h) @ w
            if self.relu and i != last:
                h = torch.relu(h)
        return torch.log_softmax(h, dim=1)


def sharded_training_step(model, graph, x, labels, mask, optimizer, manager, sync="gradients"):
    """One optimiser step on a row-partitioned graph; returns the whole-graph training loss.

    ``sync="gradients"``: the loss is the negative log-likelihood summed over the rank's masked
    nodes and divided by the global number of masked nodes; weight gradients are summed over the
    ranks before the step, so the result equals single-process training on the whole graph.
    ``sync="parameters"``: every rank steps on its local mean loss and the weights are averaged
    afterwards (the reference manager's ``synchronize_model_parameters``).  ``sync="none"``:
    local steps only, what the reference's example does."""
    optimizer.zero_grad(set_to_none=True)
    pred = model(x, graph)
    picked = pred[mask]
    nll = -picked.gather(1, labels[mask].long().view(-1, 1)).sum()
    count = torch.tensor([float(picked.shape[0])], device=x.device)
    if sync == "gradients":
        dist.all_reduce(count, group=manager.group)
        loss = nll / count.clamp(min=1.0)
        loss.backward()
        manager.all_reduce_gradients(model)
        optimizer.step()
        total = loss.detach().clone().view(1)
        dist.all_reduce(total, group=manager.group)
        return float(total)
    loss = nll / count.clamp(min=1.0)
    loss.backward()
    optimizer.step()
    if sync == "parameters":
        manager.synchronize_model_parameters(model)
    elif sync != "none":
        raise ValueError(f"sync must be 'gradients', 'parameters' or 'none', got {sync!r}")
    return float(loss.detach())
