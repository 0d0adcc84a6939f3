"""1-D destination-row partition of the aggregation across the GPUs of one box.

The reference's graph-parallel path (examples/dist_gcn/dist_gcn.py:73-88, ops/distspmm.py:16-61)
gives every rank the in-edges of its own destination rows, split offline into one sub-CSR per
source rank, and runs P rounds of host-staged pickled ``MPI.bcast`` + cuSPARSE.  Here each rank

* owns a contiguous range of destination rows and the matching rows of the feature matrix
  (:class:`RowPartition`; equal ranges of ``ceil(N / P)`` rows, which balances edges when vertex
  ids carry no degree order),
* finds, once per graph, the distinct remote rows its in-edges reference (with skewed degrees a
  minority of all remote rows) and re-addresses its entries into one buffer ``[own rows | halo rows]``,
* per aggregation fetches those rows into the halo part and runs ONE aggregation over the buffer,
  every row summed exactly as the unpartitioned kernel sums it (``mode="merged"``); or aggregates
  the entries with owned sources while the halo rows travel and adds the rest afterwards
  (``mode="overlap"``).

Transports.  :class:`DirectTransport` (GPUs): every rank keeps its feature rows in a buffer all
ranks have mapped and PULLS the rows it needs straight out of their owners' buffers with a small
kernel of bulk asynchronous copies over NVLink - no pack step, no send buffer, no barrier; epoch
words with bounded waits order producers and readers, and the pull of one feature width runs beside
the aggregation of another.  :class:`CollectiveTransport`: owners pack the requested rows and one
``all_to_all_single`` moves them (NCCL, or gloo for CPU ranks in tests).

One process per GPU; ``torch.distributed`` supplies the communicator.  The compute backend is
pluggable so the partition and exchange logic can be exercised by CPU ranks over ``gloo``.
"""
import os

import ctypes

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


def part_rows(n_local, parts):
    """Boundaries of ``parts`` blocks of a rank's ``n_local`` rows: equal blocks rounded up to multiples of
    128 rows (the tile of the dense transform).  Every rank computes the same boundaries for every owner."""
    step = -(-int(n_local) // int(parts)) if n_local else 0
    step = -(-step // 128) * 128
    return [min(int(n_local), c * step) for c in range(int(parts))] + [int(n_local)]


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

    def aggregate(self, x, idx, off, w, n_out, plan, out=None, accumulate=False, bias=None, relu=False, reserve_ctas=0):
        return ops.segment_aggregate(x, idx, off, w, n_out=n_out, plan=plan, out=out, accumulate=accumulate, bias=bias,
                                     relu=relu, reserve_ctas=reserve_ctas)


class ExchangeTimeout(RuntimeError):
    """A bounded wait of the halo exchange ran out (``JG_ETIMEOUT``): a peer never posted its rows,
    never finished reading this rank's, or never joined the collective."""


class _Done:
    def wait(self):
        pass

    def release(self):
        pass


class _WorkHandle:
    """An asynchronous ``torch.distributed`` collective; ``timeout_s`` bounds the wait."""

    def __init__(self, work, timeout_s=None):
        self.work, self.timeout_s = work, timeout_s

    def wait(self):
        if self.timeout_s is None:
            self.work.wait()
            return
        import datetime
        try:
            done = self.work.wait(datetime.timedelta(seconds=self.timeout_s))
        except RuntimeError as exc:
            raise ExchangeTimeout(f"halo exchange: a peer did not take part within {self.timeout_s} s ({exc})") from exc
        if done is False:
            raise ExchangeTimeout(f"halo exchange: a peer did not take part within {self.timeout_s} s")

    def release(self):
        pass


class CollectiveTransport:
    """Row exchange with ``torch.distributed`` collectives (NCCL on GPUs, gloo on CPU ranks):
    one ``all_to_all_single`` with per-peer row counts."""

    def __init__(self, group=None, timeout_s=None):
        self.group = group
        self.timeout_s = timeout_s       # None: the process group's own timeout

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
                                                  group=self.group, async_op=True), self.timeout_s)


class _Slot:
    """One feature width's buffer ``[own rows | halo rows]`` as every rank has mapped it."""

    def __init__(self, index, buf, ptrs):
        self.index, self.buf = index, buf
        self.ptrs = (ctypes.c_void_p * len(ptrs))(*[int(p) for p in ptrs])
        self.epoch = 0           # exchanges started on this buffer
        self.acquired = 0        # epoch whose readers have been waited for
        self.buf16 = None        # fp16 copy of the own rows offered to the readers (half-width payload)
        self.ptrs16 = None
        self.part_flags = {}     # number of row blocks -> flag slots of a block-wise exchange
        self.last_flags = [index]   # flag slots the last exchange used (the words `acquire` waits on)


class DirectTransport(CollectiveTransport):
    """Halo rows pulled straight out of their owners' feature buffers over NVLink.

    Every rank writes its feature rows into the head of a buffer that all ranks have mapped
    (``torch.distributed`` symmetric memory is only the allocator and the address exchange) and
    fetches the remote rows it references with ``jg_halo_pull``: bulk asynchronous copies, one warp
    per CTA, no SM time to speak of, so the pull of the next feature width runs beside the current
    aggregation kernel (which leaves ``pull_ctas`` CTA slots free for it).  Producers and readers are
    ordered by epoch words in a mapped flag block: ``post`` after the rows are written, the pull
    acquires its owners' words before the first load and reports back when everything has landed,
    and ``acquire`` makes a rank wait for its readers before it overwrites its rows.  Every wait
    is bounded (``wait_ms``); one that runs out is reported through an error word in pinned host
    memory and raised as :class:`ExchangeTimeout` at the next call - nothing traps or hangs.
    No NCCL kernel is involved and nothing uses multicast.
    """

    direct = True

    def __init__(self, group=None, pull_ctas=48, wait_ms=2000.0, plain=False, device=None):
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm
        self._symm = symm
        self.group = group
        self.symm_group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if self.world > lib().jg_halo_max_ranks():
            raise RuntimeError(f"DirectTransport serves at most {lib().jg_halo_max_ranks()} ranks")
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        self.pull_ctas, self.wait_ns, self.plain = int(pull_ctas), int(wait_ms * 1e6), bool(plain)
        self.side = torch.cuda.Stream(device=self.device, priority=-1)
        self.profile = False
        self._slots = {}
        self._next_flag = 0
        words = lib().jg_halo_flag_bytes() // 4
        self._flags = symm.empty((words,), dtype=torch.int32, device=self.device)
        self._flags.zero_()
        hdl = symm.rendezvous(self._flags, self.symm_group.group_name)
        self._flag_ptrs = (ctypes.c_void_p * self.world)(*[int(p) for p in hdl.buffer_ptrs])
        self._counter = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._error = torch.zeros(1, dtype=torch.int32).pin_memory()
        torch.cuda.synchronize(self.device)
        dist.barrier(group=group)                     # every flag block is zero before anyone posts

    # ---- errors
    def check(self):
        """Raises :class:`ExchangeTimeout` if a bounded wait of an earlier exchange ran out."""
        code = int(self._error[0])
        if code:
            self._error[0] = 0
            what = {0x100: "never posted its rows", 0x200: "never finished reading this rank's rows"}.get(code & 0xf00,
                                                                                                      "a row copy never landed")
            raise ExchangeTimeout(f"halo exchange on rank {self.rank}: rank {code & 0xff} {what} "
                                  f"within {self.wait_ns / 1e6:.0f} ms [JG_ETIMEOUT, code {code:#x}]")

    # ---- buffers
    def _slot(self, g, f):
        slot = self._slots.get(f)
        if slot is None:
            buf = self._symm.empty((max(g.buffer_rows, 1), f), dtype=torch.float32, device=self.device)
            hdl = self._symm.rendezvous(buf, self.symm_group.group_name)
            slot = _Slot(self._take_flags(1)[0], buf, hdl.buffer_ptrs)
            self._slots[f] = slot
        return slot

    def _take_flags(self, count):
        """``count`` unused flag slots (every rank asks in the same order, so they agree on the numbers)."""
        if self._next_flag + count > lib().jg_halo_flag_slots():
            raise RuntimeError(f"DirectTransport has {lib().jg_halo_flag_slots()} flag slots (one per feature width, "
                               "one more per row block of a block-wise exchange)")
        got = list(range(self._next_flag, self._next_flag + count))
        self._next_flag += count
        return got

    def feature_buffer(self, g, f):
        """The rank's buffer for width ``f`` (``[own rows | halo rows]``; collective on first use:
        every rank must ask for its widths in the same order)."""
        return self._slot(g, f).buf

    def acquire(self, g, f):
        """Queues, on the current stream, the wait for every peer to have finished reading the rows
        of the last exchange of width ``f``: call it before overwriting the head of the buffer."""
        slot = self._slot(g, f)
        if slot.epoch > slot.acquired and self.world > 1:
            for flag in slot.last_flags:
                check(lib().jg_halo_wait(ptr(self._flags), self.world, self.rank, flag, 1, slot.epoch, self._eptr(),
                                         self.wait_ns, stream_for(slot.buf)), "jg_halo_wait")
        slot.acquired = slot.epoch

    def _eptr(self):
        return ctypes.c_void_p(self._error.data_ptr())

    def half_buffer(self, g, f):
        """The fp16 copy of the rank's rows that the peers read when ``g.halo_half`` is set (collective on
        first use).  A producer that writes it together with the fp32 rows (``ops.linear_tf32(out_half=)``)
        passes ``half_ready=True`` to ``start`` and saves the conversion pass."""
        slot = self._slot(g, f)
        if slot.buf16 is None:
            slot.buf16 = self._symm.empty((max(g.part.pad, 1), f), dtype=torch.float16, device=self.device)
            hdl = self._symm.rendezvous(slot.buf16, self.symm_group.group_name)
            slot.ptrs16 = (ctypes.c_void_p * self.world)(*[int(p) for p in hdl.buffer_ptrs])
        return slot.buf16

    def begin(self, g, f, half_ready=False):
        """The rank's rows of width ``f`` are in place (written by work already queued on the current
        stream): tells the peers and starts pulling this rank's halo rows on the side stream."""
        self.check()
        slot = self._slot(g, f)
        slot.epoch += 1
        slot.last_flags = [slot.index]
        st = stream_for(slot.buf)
        half = bool(getattr(g, "halo_half", False))
        if half:
            self.half_buffer(g, f)
            if not half_ready:
                check(lib().jg_rows_to_half(ptr(slot.buf16), ptr(slot.buf), g.n_local * f, st), "jg_rows_to_half")
        check(lib().jg_halo_post(self._flag_ptrs, self.world, self.rank, slot.index, 0, slot.epoch, st), "jg_halo_post")
        cur = torch.cuda.current_stream(self.device)
        self.side.wait_stream(cur)
        seg, los = self._tables(g)
        halo_ptr = ctypes.c_void_p(slot.buf.data_ptr() + g.n_local * f * 4)
        begun = None
        if self.profile:                      # timing events around the pull (benchmarks: where a step's time goes)
            begun = torch.cuda.Event(enable_timing=True)
            begun.record(self.side)
        check(lib().jg_halo_pull(halo_ptr, ptr(g.needed), slot.ptrs16 if half else slot.ptrs, self._flag_ptrs, seg, los,
                                 self.world, self.rank, (2 if half else 4) * f, slot.index, slot.epoch, ptr(self._counter),
                                 self._eptr(), self.wait_ns, self.pull_ctas, 1 if self.plain else 0, 1 if half else 0,
                                 ctypes.c_void_p(self.side.cuda_stream)), "jg_halo_pull")
        landed = torch.cuda.Event(enable_timing=self.profile)
        landed.record(self.side)
        return _DirectHandle(self, landed, begun)

    def begin_part(self, g, f, c, parts, half_ready=False, ctas=None):
        """Block ``c`` of ``parts`` (:func:`part_rows`) of the rank's rows of width ``f`` is in place: tells the
        peers and starts pulling the halo rows that lie in block ``c`` of THEIR owners.  A rank that produces
        its rows block after block (an aggregation of a row range followed by its transform) calls this after
        every block, in order, so the rows of a block travel while the next one is computed; every block has its
        own epoch words.  ``ctas``: CTA slots for the pull (default ``pull_ctas``; 0 = nothing runs beside it)."""
        self.check()
        slot = self._slot(g, f)
        flags = slot.part_flags.get(parts)
        if flags is None:
            flags = slot.part_flags[parts] = self._take_flags(parts)
        if c == 0:
            slot.epoch += 1
            slot.last_flags = flags
        st = stream_for(slot.buf)
        half = bool(getattr(g, "halo_half", False))
        rows = part_rows(g.n_local, parts)
        if half:
            self.half_buffer(g, f)
            if not half_ready and rows[c + 1] > rows[c]:
                check(lib().jg_rows_to_half(ptr(slot.buf16[rows[c]:]), ptr(slot.buf[rows[c]:]), (rows[c + 1] - rows[c]) * f, st),
                      "jg_rows_to_half")
        check(lib().jg_halo_post(self._flag_ptrs, self.world, self.rank, flags[c], 0, slot.epoch, st), "jg_halo_post")
        self.side.wait_stream(torch.cuda.current_stream(self.device))
        seg, los = self._tables(g)
        begins, ends = g.part_tables(parts)[c]
        halo_ptr = ctypes.c_void_p(slot.buf.data_ptr() + g.n_local * f * 4)
        check(lib().jg_halo_pull_part(halo_ptr, ptr(g.needed), slot.ptrs16 if half else slot.ptrs, self._flag_ptrs, seg, begins,
                                      ends, los, self.world, self.rank, (2 if half else 4) * f, flags[c], slot.epoch,
                                      ptr(self._counter), self._eptr(), self.wait_ns, self.pull_ctas if ctas is None else int(ctas),
                                      1 if self.plain else 0, 1 if half else 0, ctypes.c_void_p(self.side.cuda_stream)),
              "jg_halo_pull_part")
        landed = torch.cuda.Event()
        landed.record(self.side)
        return _DirectHandle(self, landed)

    def _tables(self, g):
        tables = getattr(g, "_pull_tables", None)
        if tables is None:                       # per-graph constants of the pull, built once
            tables = ((ctypes.c_int64 * (self.world + 1))(*([int(v) for v in g.recv_offset] + [int(g.n_halo)])),
                      (ctypes.c_int32 * self.world)(*[int(g.part.bounds[q]) for q in range(self.world)]))
            g._pull_tables = tables
        return tables


class EmulatedRanks:
    """The direct exchange with every rank of a partition living on ONE GPU in one process (no
    process group): each emulated rank has its own flag block and feature buffers in local memory,
    and the "peer" pointers are simply the other ranks' buffers.  It runs the real kernels
    (``jg_halo_post`` / ``jg_halo_pull``, epoch words included) where only one GPU is available.
    Kernels that wait for one another must not run as separate launches on one GPU, so a rank's
    exchange first posts the ready words of ALL emulated ranks (their rows must already be in their
    buffers: write every rank's ``feature_buffer`` before the first ``start``); ``acquire`` does not
    wait.  ``transport(rank)`` is what ``ShardedGraph(transport=...)`` takes."""

    def __init__(self, world, device=None, wait_ms=1000.0, plain=False, pull_ctas=48):
        self.world = int(world)
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        words = lib().jg_halo_flag_bytes() // 4
        self.flags = [torch.zeros(words, dtype=torch.int32, device=self.device) for _ in range(self.world)]
        self.flag_ptrs = (ctypes.c_void_p * self.world)(*[t.data_ptr() for t in self.flags])
        self.buffers = {}            # f -> [tensor per rank]
        self._flag_of = {}           # (f, parts) -> first flag slot
        self._next_flag = 0
        self.rows = [0] * self.world
        self.views = [_EmulatedRank(self, r, wait_ms, plain, pull_ctas) for r in range(self.world)]

    def transport(self, rank):
        return self.views[rank]

    def wire(self, graphs):
        """What the set-up collectives do between real ranks: every emulated rank learns the matrix of
        request counts (``graphs[r]`` built with ``transport=self.transport(r), setup=False``)."""
        matrix = [list(g.recv_counts) for g in graphs]
        for r, g in enumerate(graphs):
            g.apply_setup(matrix, None)
            self.rows[r] = g.n_local + g.n_halo

    def buffer(self, f, rank):
        bufs = self.buffers.get(f)
        if bufs is None:
            bufs = [torch.zeros((max(self.rows[r], 1), f), dtype=torch.float32, device=self.device) for r in range(self.world)]
            self.buffers[f] = bufs
        return bufs[rank]

    def slot_index(self, f, parts=1):
        """First of the ``parts`` flag slots of width ``f`` (1: the whole-segment exchange)."""
        key = (f, parts)
        if key not in self._flag_of:
            if self._next_flag + parts > lib().jg_halo_flag_slots():
                raise RuntimeError("too many flag slots")
            self._flag_of[key] = self._next_flag
            self._next_flag += parts
        return self._flag_of[key]


class _EmulatedRank(CollectiveTransport):
    direct = True

    def __init__(self, owner, rank, wait_ms, plain, pull_ctas):
        self.owner, self.rank, self.world = owner, rank, owner.world
        self.group = None
        self.wait_ns, self.plain, self.pull_ctas = int(wait_ms * 1e6), bool(plain), int(pull_ctas)
        self.epochs = {}
        self.post_for_peers = True       # tests of the time-out path switch this off: nobody posts, the wait runs out
        self._counter = torch.zeros(1, dtype=torch.int32, device=owner.device)
        self._error = torch.zeros(1, dtype=torch.int32).pin_memory()

    check = DirectTransport.check
    _eptr = DirectTransport._eptr

    def all_gather_counts(self, g, counts):
        raise RuntimeError("emulated ranks are wired by hand: ShardedGraph(setup=False) + apply_setup")

    def feature_buffer(self, g, f):
        return self.owner.buffer(f, self.rank)

    def acquire(self, g, f):
        pass

    def half_buffer(self, g, f):
        raise RuntimeError("emulated ranks convert on every exchange: no persistent fp16 buffer")

    def begin(self, g, f, half_ready=False):
        self.check()
        buf = self.feature_buffer(g, f)
        slot = self.owner.slot_index(f)
        epoch = self.epochs.get(f, 0) + 1
        self.epochs[f] = epoch
        st = stream_for(buf)
        half = bool(getattr(g, "halo_half", False))
        posters = range(self.world) if self.post_for_peers else [self.rank]
        sources = []
        for q in range(self.world):
            xq = self.owner.buffer(f, q)
            if half:                                  # every emulated owner's fp16 copy, made on its behalf
                n_q = g.part.n_local(q)
                x16 = torch.empty((max(n_q, 1), f), dtype=torch.float16, device=xq.device)
                check(lib().jg_rows_to_half(ptr(x16), ptr(xq), n_q * f, st), "jg_rows_to_half")
                xq = x16
            sources.append(xq)
        for q in posters:
            check(lib().jg_halo_post(self.owner.flag_ptrs, self.world, q, slot, 0, epoch, st), "jg_halo_post")
        ptrs = (ctypes.c_void_p * self.world)(*[t.data_ptr() for t in sources])
        seg = (ctypes.c_int64 * (self.world + 1))(*([int(v) for v in g.recv_offset] + [int(g.n_halo)]))
        los = (ctypes.c_int32 * self.world)(*[int(g.part.bounds[q]) for q in range(self.world)])
        check(lib().jg_halo_pull(ptr(buf[g.n_local:]), ptr(g.needed), ptrs, self.owner.flag_ptrs, seg, los, self.world,
                                 self.rank, (2 if half else 4) * f, slot, epoch, ptr(self._counter), self._eptr(), self.wait_ns,
                                 self.pull_ctas, 1 if self.plain else 0, 1 if half else 0, st), "jg_halo_pull")
        for t in sources:
            t.record_stream(torch.cuda.current_stream())
        return _Done()

    def begin_part(self, g, f, c, parts, half_ready=False, ctas=None):
        """Block ``c`` of a block-wise exchange (see :meth:`DirectTransport.begin_part`); the emulated owners'
        words for the block are posted here on their behalf, fp32 payload only."""
        self.check()
        if getattr(g, "halo_half", False):
            raise RuntimeError("emulated ranks exchange blocks in fp32 only")
        buf = self.feature_buffer(g, f)
        first = self.owner.slot_index(f, parts)
        if c == 0:
            self.epochs[(f, parts)] = self.epochs.get((f, parts), 0) + 1
        epoch = self.epochs[(f, parts)]
        st = stream_for(buf)
        for q in (range(self.world) if self.post_for_peers else [self.rank]):
            check(lib().jg_halo_post(self.owner.flag_ptrs, self.world, q, first + c, 0, epoch, st), "jg_halo_post")
        ptrs = (ctypes.c_void_p * self.world)(*[self.owner.buffer(f, q).data_ptr() for q in range(self.world)])
        seg = (ctypes.c_int64 * (self.world + 1))(*([int(v) for v in g.recv_offset] + [int(g.n_halo)]))
        los = (ctypes.c_int32 * self.world)(*[int(g.part.bounds[q]) for q in range(self.world)])
        begins, ends = g.part_tables(parts)[c]
        check(lib().jg_halo_pull_part(ptr(buf[g.n_local:]), ptr(g.needed), ptrs, self.owner.flag_ptrs, seg, begins, ends, los,
                                      self.world, self.rank, 4 * f, first + c, epoch, ptr(self._counter), self._eptr(), self.wait_ns,
                                      self.pull_ctas if ctas is None else int(ctas), 1 if self.plain else 0, 0, st),
              "jg_halo_pull_part")
        return _Done()


class _DirectHandle:
    def __init__(self, transport, landed, begun=None):
        self.transport, self.landed, self.begun = transport, landed, begun

    def wait(self):
        torch.cuda.current_stream().wait_event(self.landed)

    def release(self):
        pass


class ShardedGraph:
    """One rank's share of a row-partitioned graph: the in-edges of its destination rows.

    ``idx`` holds GLOBAL source ids, ``off`` the offsets of the rank's own rows (CSC of the shard).
    Construction is collective (every rank of the group builds its graph at the same time): the
    ranks tell each other which rows they need.  ``exchange``: ``"direct"`` (alias ``"peer"``) pulls
    halo rows out of peer memory (:class:`DirectTransport`), ``"nccl"`` packs and runs one all-to-all
    (:class:`CollectiveTransport`, also what CPU ranks use over gloo).
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
            transport = DirectTransport(group) if exchange in ("direct", "peer") else CollectiveTransport(group)
        self.transport = transport
        self.direct = bool(getattr(transport, "direct", False))
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
        self.buffer_rows = self.n_local + self.n_halo
        self._recv = {}
        self._inflight = set()
        # direct transport only: halo rows travel as fp16 (half the NVLink bytes; values beyond +-65504 saturate)
        # and are widened to fp32 on arrival; the rank's own rows stay fp32.  For workloads whose tolerance is
        # 2e-3 (a TF32/bf16 transform feeds the aggregation); widths must be multiples of 8.
        self.halo_half = False
        if setup:
            self._setup_requests()

    # ---- set-up: who sends which rows to whom
    def _setup_requests(self):
        dev = self.needed.device
        counts = torch.tensor(self.recv_counts, dtype=torch.int64, device=dev)
        matrix = self.transport.all_gather_counts(self, counts)           # matrix[r][q] = rows rank r needs from rank q
        send_counts = [int(matrix[r][self.rank]) for r in range(self.part.world)]
        # the owners only need the requested ids when they pack rows for their readers
        send_rows = None if self.direct else self.transport.all_to_all_ids(self, self.needed, self.recv_counts, send_counts)
        self.apply_setup(matrix, send_rows)

    def apply_setup(self, matrix, send_rows):
        """``matrix[r][q]`` = rows rank r needs from rank q; ``send_rows`` = the global ids of this
        rank's rows its peers asked for, grouped by requesting rank in rank order (``None`` when
        readers fetch rows themselves)."""
        world = self.part.world
        self.count_matrix = matrix
        self.send_counts = [int(matrix[r][self.rank]) for r in range(world)]
        self.send_offset = [sum(self.send_counts[:r]) for r in range(world)]
        # in rank q's send buffer the rows for rank r start after those for ranks 0..r-1
        self.peer_send_offset = [sum(int(matrix[r2][q]) for r2 in range(self.rank)) for q in range(world)]
        self.n_send = sum(self.send_counts)
        self.max_send = max(sum(int(matrix[r][q]) for r in range(world)) for q in range(world))
        self.send_rows = send_rows
        # one mapped buffer shape for every rank: its own rows followed by its halo rows
        self.buffer_rows = max(self.part.n_local(r) + sum(int(c) for c in matrix[r]) for r in range(world))

    # ---- per aggregation
    def feature_buffer(self, f, like=None):
        """Where a caller should write the rank's ``n_local`` feature rows of width ``f`` to save a copy
        per aggregation: the head of the buffer the aggregation reads (and, with the direct transport,
        the peers read).  Ask for it EVERY time before writing: with the direct transport the call
        also queues the wait for the readers of the previous exchange of this width."""
        if self.direct:
            self.transport.acquire(self, f)
            return self.transport.feature_buffer(self, f)[: self.n_local]
        if self.mode == "merged":
            return self._recv_buffer(f, like)[: self.n_local]
        return torch.empty((self.n_local, f), dtype=like.dtype, device=like.device)

    def half_buffer(self, f):
        """Direct transport with ``halo_half``: the fp16 buffer ``[>= n_local, f]`` the peers read.  Fill it
        together with :meth:`feature_buffer` (e.g. ``ops.linear_tf32(out=..., out_half=...)``) and call
        ``start`` / ``aggregate`` with ``half_ready=True``."""
        if not (self.direct and self.halo_half):
            raise RuntimeError("half_buffer: needs the direct transport with halo_half set")
        return self.transport.half_buffer(self, f)

    def _recv_buffer(self, f, like):
        buf = self._recv.get(f)
        if buf is None:
            rows = self.n_halo + (self.n_local if self.mode == "merged" else 0)
            buf = torch.empty((max(rows, 1), f), dtype=like.dtype, device=like.device)
            self._recv[f] = buf
        return buf

    def aggregate(self, x, bias=None, relu=False, half_ready=False):
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
            return self.finish(self.start(x, half_ready), bias, relu)
        else:
            return self.finish(self.start(x, half_ready))
        if bias is not None:
            y = y + bias
        return torch.relu(y) if relu else y

    def _aggregate(self, x, bias=None, relu=False):
        return self.finish(self.start(x), bias, relu)

    # ---- block-wise exchange (direct transport): rows produced and fetched block after block
    def part_tables(self, parts):
        """For every block ``c`` of ``parts``: the halo slots ``[begin[q], end[q])`` whose rows lie in block
        ``c`` of owner ``q`` (``needed`` is ascending, so a block of an owner is one run of it)."""
        cache = self.__dict__.setdefault("_part_tables", {})
        tables = cache.get(parts)
        if tables is None:
            world = self.part.world
            marks = [[self.part.bounds[q] + r for r in part_rows(self.part.n_local(q), parts)] for q in range(world)]
            flat = torch.tensor([m for row in marks for m in row], dtype=self.needed.dtype, device=self.needed.device)
            pos = torch.searchsorted(self.needed.contiguous(), flat).reshape(world, parts + 1).tolist() if self.n_halo else \
                [[0] * (parts + 1) for _ in range(world)]
            tables = [((ctypes.c_int64 * world)(*[int(pos[q][c]) for q in range(world)]),
                       (ctypes.c_int64 * world)(*[int(pos[q][c + 1]) for q in range(world)])) for c in range(parts)]
            cache[parts] = tables
        return tables

    def start_part(self, f, c, parts, half_ready=False, ctas=None):
        """Block ``c`` of ``parts`` (:func:`part_rows`) of the rank's rows has been written into
        ``feature_buffer(f)`` (and ``half_buffer(f)`` when ``half_ready``): offers it to the peers and starts
        fetching the halo rows of the same block of every owner.  Call for ``c = 0 .. parts - 1`` in order, then
        :meth:`finish_parts` with the handles.  Direct transport, merged schedule, forward only."""
        if not (self.direct and self.mode == "merged"):
            raise RuntimeError("start_part: needs the direct transport and the merged schedule")
        if c == 0:
            if f in self._inflight:
                raise RuntimeError(f"an aggregation of width {f} is already in flight on this graph")
            self._inflight.add(f)
        return self.transport.begin_part(self, f, c, parts, half_ready, ctas)

    def finish_parts(self, f, handles, bias=None, relu=False):
        """Waits for every block's halo rows and aggregates (the second half of :meth:`start_part`)."""
        for h in handles:
            h.wait()
        buf = self.transport.feature_buffer(self, f)
        extra = {"reserve_ctas": self.transport.pull_ctas} if len(self._inflight) > 1 and self.transport.pull_ctas > 0 else {}
        y = self.backend.aggregate(buf, self.merged[0], self.merged[1], self.merged[2], self.n_local, self.merged_plan,
                                   bias=bias, relu=relu, **extra)
        self._inflight.discard(f)
        return y

    def aggregate_rows(self, pending, first, last, bias=None, relu=False, reserve_ctas=0):
        """The rows ``[first, last)`` of an aggregation whose exchange was started with :meth:`start` (wait for it
        with ``pending[2].wait()`` once, then call this for every row range; :meth:`done` ends it).  The rows of a
        range can feed the next layer's transform and exchange while the next range is aggregated."""
        if self.mode != "merged":
            raise RuntimeError("aggregate_rows: merged schedule only")
        buf = pending[1]
        idx, off, w = self.merged
        plans = self.__dict__.setdefault("_range_plans", {})
        plan = plans.get((first, last))
        if plan is None:
            plan = plans[(first, last)] = self.backend.plan(off[first: last + 1], idx.numel())
        return self.backend.aggregate(buf, idx, off[first: last + 1], w, last - first, plan, bias=bias, relu=relu,
                                      reserve_ctas=reserve_ctas)

    def done(self, pending):
        """Ends an aggregation that was consumed through :meth:`aggregate_rows`."""
        pending[2].release()
        self._inflight.discard(pending[0].shape[1])

    def start(self, x, half_ready=False):
        """First half of an aggregation: starts the exchange of the halo rows.  Aggregations of
        DIFFERENT widths may be started before the first is finished; their exchanges then run
        underneath the aggregation kernels of the earlier ones.  A second ``start`` of a width whose
        aggregation has not been finished raises: the two would share one buffer.  Forward only."""
        if x.shape[0] < self.n_local:
            raise RuntimeError(f"x has {x.shape[0]} rows, the rank owns {self.n_local}")
        f = x.shape[1]
        if f in self._inflight:
            raise RuntimeError(f"an aggregation of width {f} is already in flight on this graph: finish() it first "
                               "(aggregations of one width share their exchange buffers)")
        if self.direct:
            buf = self.transport.feature_buffer(self, f)
            if x.data_ptr() != buf.data_ptr():
                self.transport.acquire(self, f)
                buf[: self.n_local].copy_(x[: self.n_local])
            handle = self.transport.begin(self, f, half_ready)
            self._inflight.add(f)
            return (buf[: self.n_local], buf if self.mode == "merged" else buf[self.n_local:], handle)
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
        self._inflight.add(f)
        return (x, buf, handle)

    def finish(self, pending, bias=None, relu=False):
        """Second half: waits for the halo rows of ``pending`` (from :meth:`start`) and aggregates."""
        x, buf, handle = pending
        f = x.shape[1]
        # other exchanges still travelling: leave their pull kernels room beside this aggregation
        extra = {}
        if self.direct and len(self._inflight) > 1:
            extra = {"reserve_ctas": self.transport.pull_ctas}
        if self.mode == "merged":
            handle.wait()
            if bias is not None or relu:
                y = self.backend.aggregate(buf, self.merged[0], self.merged[1], self.merged[2], self.n_local,
                                           self.merged_plan, bias=bias, relu=relu, **extra)
            else:
                y = self.backend.aggregate(buf, self.merged[0], self.merged[1], self.merged[2], self.n_local,
                                           self.merged_plan, **extra)
            handle.release()
            self._inflight.discard(f)
            return y
        # the rank's own rows while the halo rows travel
        y = self.backend.aggregate(x, self.interior[0], self.interior[1], self.interior[2], self.n_local,
                                   self.interior_plan, **extra)
        handle.wait()
        if self.halo[0].numel():
            self.backend.aggregate(buf, self.halo[0], self.halo[1], self.halo[2], self.n_local, self.halo_plan,
                                   out=y, accumulate=True)
        handle.release()
        self._inflight.discard(f)
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
    the single-GPU example has and the graph-parallel one omits.  ``tf32=False`` keeps the transform
    in fp32 (comparisons at 1e-5)."""

    def __init__(self, in_channels, hidden_channels, out_channels, layers=2, manager=None, relu=False,
                 device=None, seed=0, tf32=True):
        super().__init__()
        widths = [in_channels] + [hidden_channels] * (layers - 1) + [out_channels]
        gen = torch.Generator().manual_seed(seed)
        self.weights = torch.nn.ParameterList()
        for a, b in zip(widths[:-1], widths[1:]):
            bound = (6.0 / (a + b)) ** 0.5                      # nn/inits.py:19-22
            w = (torch.rand((a, b), generator=gen) * 2 - 1) * bound
            self.weights.append(torch.nn.Parameter(w.to(device) if device is not None else w))
        self.relu = relu
        self.tf32 = tf32
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
            z = graph.aggregate(h)
            act = self.relu and i != last
            if z.is_cuda:                    # the library's own transforms: tcgen05 TF32, or fp32 on the CUDA cores
                h = ops.linear_tf32_autograd(z, w, relu=act) if self.tf32 else ops.linear_f32_autograd(z, w, relu=act)
            else:                            # CPU ranks of the tests
                h = z @ w
                if act:
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
