"""Multi-GPU leg of ``bench.py`` and the partitioned GCN forward (every N, N = 1 included).

SpMM sweep (N > 1): the scale-21 graph split into one contiguous destination-row shard per rank
(strong scaling); every rank generates and converts ONLY its own rows, halo rows are pulled out of
peer memory over NVLink (``dist.DirectTransport``), and after the timed region the rank's result is
compared with the reference's CPU aggregation on a sample of its rows.

``gcn_forward`` (``--gcn-scale``, default 26): the 2-layer GCN forward 128 -> 128 -> 64 of the
reference's graph-parallel example (examples/dist_gcn/dist_gcn.py:73-88) on the R-MAT graph of that
scale, on 1, 2, 4 or 8 GPUs, reported as a sub-record of the same JSON line.
Launched by torchrun, one process per GPU; ``bench.py`` calls :func:`gcn_forward_record` directly at N = 1."""
import json
import os
import time

import torch
import torch.distributed as dist

from jittorgeometric_b200 import dist as jd
from jittorgeometric_b200 import synth


def feature_seed(base, rank, f):
    return base + 17 * rank + 1000 * f


def build_shard(scale, pairs_per_node, seed, part, rank, world, dev):
    """This rank's rows of the gcn-normalised symmetric R-MAT graph, generated on the device without
    building the whole graph: ``(idx [global source ids], off, w, global nnz)``."""
    lo, hi = part.range(rank)
    idx, off, deg = synth.rmat_shard_csc(scale, pairs_per_node, seed, lo, hi, device=dev)
    if world > 1:
        pad = part.pad
        mine = torch.zeros(pad, dtype=torch.int32, device=dev)
        mine[: hi - lo] = deg
        every = torch.empty(pad * world, dtype=torch.int32, device=dev)
        dist.all_gather_into_tensor(every, mine)
        deg_global = torch.cat([every[q * pad: q * pad + part.n_local(q)] for q in range(world)])
        total = torch.tensor([idx.numel()], dtype=torch.int64, device=dev)
        dist.all_reduce(total)
        nnz = int(total.item())
    else:
        deg_global, nnz = deg, idx.numel()
    w = synth.gcn_weights(idx, off, deg_global, lo)
    return idx, off, w, nnz


def parity_sample(idx, off, w, y, x_of, part, world, f, rows=2048):
    """Compares the first ``rows`` result rows of this rank with the reference's CPU aggregation
    (compiled reference body when present, else its C restatement) over the same entries; the
    source rows come from ``x_of(q)``, which regenerates rank q's feature rows of width ``f``."""
    import numpy as np
    import oracle as O
    rows = min(rows, off.numel() - 1)
    e = int(off[rows])
    sub_idx = idx[:e].long()
    uniq, inv = torch.unique(sub_idx, return_inverse=True)
    owner = torch.bucketize(uniq, torch.tensor(part.bounds[1:], device=uniq.device), right=True)
    xs = torch.empty((uniq.numel(), f), device=uniq.device)
    for q in range(world):
        sel = owner == q
        if bool(sel.any()):
            xs[sel] = x_of(q)[uniq[sel] - part.bounds[q]]
    want = O.aggregate(xs.cpu().numpy(), inv.to(torch.int32).cpu().numpy(), off[: rows + 1].cpu().numpy(), w[:e].cpu().numpy(),
                       n_out=rows)
    _, scale = O.aggregate_f64(xs.cpu().numpy(), inv.to(torch.int32).cpu().numpy(), off[: rows + 1].cpu().numpy(),
                               w[:e].cpu().numpy(), n_out=rows)
    got = y[:rows].cpu().numpy()
    err = float((np.abs(got - want) / (scale + 1e-30)).max()) if rows else 0.0
    same = int((got == want).all(axis=1).sum()) if rows else 0
    return {"width": f, "rows": rows, "entries": e, "max_rel_err": err, "bit_identical_rows": same,
            "checker": "reference CPU aggregation on the same entries"}


def gcn_forward_record(args, dev, rank, world, sampler_cls=None):
    """2-layer GCN forward 128 -> 128 -> 64 (TF32 transform on tcgen05, fp32 aggregation with the
    bias/ReLU epilogue fused) on the R-MAT graph of ``args.gcn_scale`` (8 undirected pairs per node,
    mirrored, self-loops, gcn_norm): the whole graph on one GPU, or one destination-row shard per rank
    with the halo rows of every layer pulled out of peer memory.  Returns the sub-record (rank 0) or None."""
    import jittorgeometric_b200 as jg
    scale = args.gcn_scale
    seed = 20261125 + 5
    n = 1 << scale
    part = jd.RowPartition(n, world)
    t_build = time.perf_counter()
    idx, off, w, nnz = build_shard(scale, 8, seed, part, rank, world, dev)
    torch.cuda.synchronize()
    t_build = time.perf_counter() - t_build
    n_local = part.n_local(rank)
    W1, W2 = synth.glorot((128, 128), 1, dev), synth.glorot((128, 64), 2, dev)
    W1t, W2t = W1.t().contiguous(), W2.t().contiguous()
    b1 = torch.linspace(-0.1, 0.1, 128, device=dev)
    b2 = torch.linspace(-0.1, 0.1, 64, device=dev)
    x = torch.randn((n_local, 128), device=dev, generator=torch.Generator(device=dev).manual_seed(feature_seed(seed, rank, 128)))
    halo_rows, halo_half = 0, False
    if world > 1:
        g = jd.ShardedGraph(part, rank, idx, off, w, exchange=args.exchange, mode="merged")
        if g.direct:
            g.transport.pull_ctas = 0            # nothing runs beside a layer's exchange: the pull may take every SM
            g.halo_half = halo_half = args.gcn_halo == "fp16"
        halo_rows = g.n_halo
        del idx, w

        fused_half = g.direct and halo_half       # the transform's epilogue also writes the fp16 rows the peers read

        def transform(src, W, Wt, f):
            h = g.feature_buffer(f, x)
            jg.linear_tf32(src, W, weight_t=Wt, out=h, out_half=g.half_buffer(f) if fused_half else None)
            return h

        def forward_serial():
            z1 = g.aggregate(transform(x, W1, W1t, 128), bias=b1, relu=True, half_ready=fused_half)
            return g.aggregate(transform(z1, W2, W2t, 64), bias=b2, half_ready=fused_half)

        # Block-wise second layer: the first layer's aggregation runs over `parts` row ranges; as soon as a range
        # is done its rows go through the second transform and are offered to the peers, whose pulls (and this
        # rank's) run beside the aggregation of the next range.  Only the last block's exchange is exposed.
        parts = max(1, int(os.environ.get("JG_GCN_PARTS", "2"))) if g.direct else 1
        beside = int(os.environ.get("JG_GCN_BESIDE_CTAS", "16"))     # CTA slots a pull gets beside an aggregation
        rows = jd.part_rows(n_local, parts)

        def forward_blocks():
            pending = g.start(transform(x, W1, W1t, 128), fused_half)
            h2 = g.feature_buffer(64, x)                          # also waits for the readers of the last forward
            half2 = g.half_buffer(64) if fused_half else None
            pending[2].wait()
            handles = []
            for c in range(parts):
                a, b = rows[c], rows[c + 1]
                last = c == parts - 1
                z = g.aggregate_rows(pending, a, b, bias=b1, relu=True, reserve_ctas=beside if c > 0 else 0)
                jg.linear_tf32(z, W2, weight_t=W2t, out=h2[a:b], out_half=half2[a:b] if fused_half else None)
                handles.append(g.start_part(64, c, parts, half_ready=fused_half, ctas=0 if last else beside))
            g.done(pending)
            return g.finish_parts(64, handles, bias=b2)

        forward = forward_blocks if parts > 1 else forward_serial
    else:
        plan = jg.SpmmPlan(off, nnz)
        h1 = torch.empty((n, 128), device=dev)
        h2 = torch.empty((n, 64), device=dev)

        def forward():
            jg.linear_tf32(x, W1, weight_t=W1t, out=h1)
            z1 = jg.segment_aggregate(h1, idx, off, w, plan=plan, bias=b1, relu=True)
            jg.linear_tf32(z1, W2, weight_t=W2t, out=h2)
            del z1
            return jg.segment_aggregate(h2, idx, off, w, plan=plan, bias=b2)

    sampler = sampler_cls(dev.index) if (sampler_cls is not None and rank == 0) else None
    if sampler:
        sampler.start()
    for _ in range(args.gcn_warmup):
        forward()
    torch.cuda.synchronize()
    if sampler:
        sampler.mark()
    if world > 1:
        dist.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(args.gcn_steps)]
    a.record()
    for k in range(args.gcn_steps):
        out = forward()
        marks[k].record()
    b.record()
    torch.cuda.synchronize()
    clocks = sampler.stop() if sampler else None
    ms = torch.tensor([a.elapsed_time(b) / args.gcn_steps], device=dev)
    each = sorted(([a] + marks)[k].elapsed_time(marks[k]) for k in range(args.gcn_steps))   # this rank's forwards, one by one
    # one more forward with a synchronisation after every phase: where the time goes (not part of `ms`)
    phases = {}
    schedule, serial_ms, blocks_vs_serial = None, None, None
    if world > 1:
        dist.barrier()
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        schedule = "serial: transform, exchange, aggregation per layer"
        if parts > 1:
            schedule = (f"layer-1 aggregation in {parts} row ranges; each range's layer-2 transform and halo exchange "
                        f"run beside the aggregation of the next range (block-wise pulls, {beside} CTA slots)")
            # the serial schedule beside it, and the two results against each other
            ref = forward_serial()
            diff = torch.tensor([float((out - ref).abs().max() / ref.abs().max().clamp_min(1e-30))], device=dev)
            dist.all_reduce(diff, op=dist.ReduceOp.MAX)
            blocks_vs_serial = float(diff.item())
            del ref
            torch.cuda.synchronize(); dist.barrier(); torch.cuda.synchronize()
            a.record()
            for _ in range(args.gcn_steps):
                ref = forward_serial()
            b.record()
            torch.cuda.synchronize()
            del ref
            sm = torch.tensor([a.elapsed_time(b) / args.gcn_steps], device=dev)
            dist.all_reduce(sm, op=dist.ReduceOp.MAX)
            serial_ms = float(sm.item())

        def timed(name, fn):
            torch.cuda.synchronize(); t0 = time.perf_counter()
            r = fn()
            torch.cuda.synchronize()
            phases[name] = phases.get(name, 0.0) + (time.perf_counter() - t0) * 1e3
            return r
        h1 = timed("transform_ms", lambda: transform(x, W1, W1t, 128))
        p = timed("exchange_ms", lambda: (lambda q: (q[2].wait(), q)[1])(g.start(h1, fused_half)))
        z1 = timed("aggregate_ms", lambda: g.finish(p, b1, True))
        h2 = timed("transform_ms", lambda: transform(z1, W2, W2t, 64))
        p = timed("exchange_ms", lambda: (lambda q: (q[2].wait(), q)[1])(g.start(h2, fused_half)))
        out = timed("aggregate_ms", lambda: g.finish(p, b2))
        if g.direct:
            g.transport.check()
        worst = torch.tensor([phases["transform_ms"], phases["exchange_ms"], phases["aggregate_ms"]], device=dev)
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        phases = dict(zip(("transform_ms", "exchange_ms", "aggregate_ms"), [float(v) for v in worst.tolist()]))
    finite = bool(torch.isfinite(out).all())
    peak_mem = torch.cuda.max_memory_allocated(dev) / 1e9
    ms = float(ms.item())
    if rank != 0:
        return None
    alg = sum(nnz * (8 + 4 * f) + 4 * (n + 1) + 4 * n * f for f in (128, 64)) + 4 * n * (128 + 128) + 4 * n * (128 + 64)
    import bench
    peak, kind = bench.measured_peaks()
    rec = {"metric": "gcn_forward_edge_feat_per_s", "value": nnz * (128 + 64) / (ms * 1e-3), "unit": "edge*feat/s",
           "ms": ms, "ms_median_forward_rank0": each[len(each) // 2], "ms_slowest_forward_rank0": each[-1],
           "steps": args.gcn_steps, "warmup": args.gcn_warmup, "n_gpus": world,
           "workload": f"2-layer GCN forward 128->128->64 (TF32 transform on tcgen05, fp32 aggregation, bias+ReLU fused): R-MAT "
                       f"scale {scale}, {n} nodes, {nnz} directed edges incl. self-loops, gcn_norm weights; {world} contiguous "
                       f"destination-row shard(s), each generated and converted by its own rank",
           "alg_gbs_per_gpu": alg / world / ms / 1e6, "frac_of_hbm_peak_per_gpu": alg / world / ms / 1e6 / peak, "peak_kind": kind,
           "halo_payload": None if world == 1 else ("fp16 (rows widened to fp32 on arrival; own rows fp32)" if halo_half else "fp32"),
           "halo_rows_rank0": halo_rows, "halo_bytes_per_forward_rank0": halo_rows * (128 + 64) * (2 if halo_half else 4),
           "remote_rows_rank0": n - n_local, "schedule": schedule, "serial_schedule_ms": serial_ms,
           "max_rel_diff_to_serial_schedule": blocks_vs_serial, "phases_ms_max_over_ranks": phases or None,
           "output_finite": finite, "peak_device_memory_gb": peak_mem, "graph_build_s": t_build, "clocks": clocks}
    return rec


def pick_exchange(args, dev):
    """``direct`` needs symmetric memory between the GPUs; probed collectively so every rank takes the same branch."""
    if args.exchange != "direct":
        return args.exchange
    ok = torch.ones(1, device=dev)
    try:
        import torch.distributed._symmetric_memory as symm
        probe = symm.empty((16,), dtype=torch.float32, device=dev)
        symm.rendezvous(probe, dist.group.WORLD.group_name)
    except Exception:
        ok.zero_()
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    return "direct" if float(ok.item()) == 1.0 else "nccl"


def run(args):
    """N > 1: the SpMM sweep (headline metric, strong scaling on the scale-21 graph) plus the
    ``gcn_forward`` sub-record; one JSON line from rank 0."""
    import bench
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    dist.init_process_group("nccl", device_id=dev)
    widths = tuple(getattr(args, "width_list", bench.WIDTHS))
    bench.WIDTHS = widths
    args.exchange = pick_exchange(args, dev)
    n = 1 << args.scale
    part = jd.RowPartition(n, world)
    idx, off, w, nnz = build_shard(args.scale, args.edge_factor, bench.SEED, part, rank, world, dev)
    g = jd.ShardedGraph(part, rank, idx, off, w, exchange=args.exchange, mode=os.environ.get("JG_DIST_MODE", "merged"))
    if g.direct and "JG_PULL_CTAS" in os.environ:
        g.transport.pull_ctas = int(os.environ["JG_PULL_CTAS"])
    local_nnz = idx.numel()
    halo_rows, remote_rows = g.n_halo, n - g.n_local

    def x_of(q, f):
        gen = torch.Generator(device=dev); gen.manual_seed(feature_seed(bench.SEED, q, f))
        return torch.randn((part.n_local(q), f), generator=gen, device=dev)

    xs = {}
    for f in widths:                                   # the head of the buffer the aggregation (and the peers) read
        x = g.feature_buffer(f, torch.empty(0, device=dev))
        x.copy_(x_of(rank, f))
        xs[f] = x

    ahead = max(1, int(os.environ.get("JG_SWEEP_AHEAD", str(len(widths)))))

    def step():
        # the aggregations of a step are independent: every exchange is started first, so the halo rows of
        # the next width travel beside the current aggregation kernel
        # (a start queued after an aggregation waits for it in stream order, so by default all starts come first;
        # JG_SWEEP_AHEAD = k keeps only k exchanges ahead of the aggregation being queued)
        if ahead >= len(widths):
            pending = [g.start(xs[f]) for f in widths]
            return [g.finish(p) for p in pending]
        pending, ys = [g.start(xs[f]) for f in widths[:ahead]], []
        for f in widths[ahead:]:
            ys.append(g.finish(pending.pop(0)))
            pending.append(g.start(xs[f]))
        ys.extend(g.finish(p) for p in pending)
        return ys

    sampler = bench.ClockSampler(dev.index)
    if rank == 0:
        sampler.start()
    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize(); dist.barrier()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    if rank == 0:
        sampler.mark()
    torch.cuda.synchronize(); dist.barrier(); torch.cuda.synchronize()
    t0.record()
    for k in range(args.steps):
        ys = step()
        marks[k].record()
    t1.record()
    torch.cuda.synchronize(); dist.barrier()
    clocks = sampler.stop() if rank == 0 else None
    if g.direct:
        g.transport.check()
    ms = torch.tensor([t0.elapsed_time(t1) / args.steps], device=dev)
    mine = ms.clone()
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_step = float(ms.item())
    every = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(every, mine)
    timeline = {"mean_step_ms_by_rank": [float(v.item()) for v in every],
                "steps_ms_rank0": [([t0] + marks)[k].elapsed_time(marks[k]) for k in range(args.steps)]}

    # where the time of a step goes (one extra, untimed step; events around every aggregation)
    breakdown = None
    if g.direct:
        g.transport.profile = True
        ev = {f: (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for f in widths}
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        handles = {}
        torch.cuda.synchronize(); dist.barrier(); torch.cuda.synchronize()
        e0.record()

        def fin(f, p):
            p[2].wait()
            ev[f][0].record()
            g.finish(p)
            ev[f][1].record()
        pending = [(f, g.start(xs[f])) for f in widths]
        for f, p in pending:
            handles[f] = p[2]
            fin(f, p)
        e1.record()
        torch.cuda.synchronize()
        g.transport.profile = False
        breakdown = {"step_ms": e0.elapsed_time(e1),
                     "aggregate_ms": {str(f): ev[f][0].elapsed_time(ev[f][1]) for f in widths},
                     "aggregate_starts_at_ms": {str(f): e0.elapsed_time(ev[f][0]) for f in widths},
                     "pull_ms": {str(f): h.begun.elapsed_time(h.landed) for f, h in handles.items() if h is not None},
                     "pull_starts_at_ms": {str(f): e0.elapsed_time(h.begun) for f, h in handles.items() if h is not None}}

    # parity after the timed region: this rank's rows against the reference's CPU aggregation
    pf = 128 if 128 in widths else widths[-1]
    par = parity_sample(idx, off, w, ys[widths.index(pf)], lambda q: x_of(q, pf), part, world, pf)
    ok = torch.tensor([1.0 if par["max_rel_err"] <= 1e-5 else 0.0, par["max_rel_err"]], device=dev)
    okmin, errmax = ok.clone(), ok.clone()
    dist.all_reduce(okmin, op=dist.ReduceOp.MIN); dist.all_reduce(errmax, op=dist.ReduceOp.MAX)
    par["max_rel_err_over_ranks"] = float(errmax[1]); par["rows"] = par["rows"] * world
    del ys

    # end to end: the rank's feature rows from pinned host memory, its output rows back to the host
    e2e_ms, e2e_steps = float("nan"), max(1, min(args.steps, 5))
    if not args.skip_e2e:
        hx = {f: torch.empty((max(g.n_local, 1), f)).pin_memory() for f in widths}
        hy = {f: torch.empty((g.n_local, f)).pin_memory() for f in widths}
        for f in widths:
            hx[f].copy_(xs[f])
        s_in, s_out, cur = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.current_stream()
        ev_in = {f: torch.cuda.Event() for f in widths}
        ev_done = {f: torch.cuda.Event() for f in widths}
        for f in widths:
            ev_done[f].record(cur)

        def e2e_step():
            pending = {}
            for f in widths:
                with torch.cuda.stream(s_in):
                    s_in.wait_event(ev_done[f])                 # last step's kernels have read xs[f]
                    if g.direct:
                        g.transport.acquire(g, f)               # ... and so have the peers
                    xs[f].copy_(hx[f], non_blocking=True)
                    ev_in[f].record(s_in)
                cur.wait_event(ev_in[f])
                pending[f] = g.start(xs[f])
            for f in widths:
                y = g.finish(pending[f])
                ev_done[f].record(cur)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_done[f])
                    hy[f].copy_(y, non_blocking=True)
                y.record_stream(s_out)

        def e2e_join():
            cur.wait_stream(s_in); cur.wait_stream(s_out)

        e2e_step(); e2e_join(); torch.cuda.synchronize(); dist.barrier()
        t0.record()
        for _ in range(e2e_steps):
            e2e_step()
        e2e_join()
        t1.record(); torch.cuda.synchronize(); dist.barrier()
        e = torch.tensor([t0.elapsed_time(t1) / e2e_steps], device=dev)
        dist.all_reduce(e, op=dist.ReduceOp.MAX)
        e2e_ms = float(e.item())
        del hx, hy
    imb = torch.tensor([float(local_nnz)], device=dev)
    dist.all_reduce(imb, op=dist.ReduceOp.MAX)
    exchange_text = ("pulled straight out of the owners' feature buffers over NVLink (bulk asynchronous copies, epoch words, "
                     "no pack step); the pull of the next width runs beside the current aggregation kernel"
                     if g.direct else "packed by their owners and exchanged with one NCCL all-to-all per aggregation")
    if g.mode == "overlap":
        exchange_text += "; entries with owned sources are aggregated while the halo rows travel"
    launches = args.steps * len(widths) * (4 if g.direct else 5)

    # free the sweep's graph before the GCN workload is built
    del g, xs, idx, off, w
    torch.cuda.empty_cache()
    gcn = None
    if args.gcn_scale > 0:
        gcn = gcn_forward_record(args, dev, rank, world, bench.ClockSampler)

    if rank == 0:
        peak, peak_kind = bench.measured_peaks()
        total_bytes = sum(bench.alg_bytes(nnz, n, f) for f in widths)
        io_bytes = sum(n * f * 4 for f in widths)
        line = {
            "metric": "spmm_edge_feat_per_s", "value": nnz * sum(widths) / (ms_step * 1e-3), "unit": "edge*feat/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": bench.workload_config(args.scale, args.edge_factor, n, nnz, world),
            "gflops": 2.0 * nnz * sum(widths) / (ms_step * 1e-3) / 1e9,
            "roofline": {"bound": "hbm", "achieved": None, "peak": peak, "unit": "GB/s", "frac": None, "traffic": None,
                         "peak_kind": peak_kind, "kernel": "aggregate_rows_kernel",
                         "model_gbs_per_gpu": total_bytes / world / ms_step / 1e6,
                         "model_frac": total_bytes / world / ms_step / 1e6 / peak,
                         "note": "no DRAM counter record for the partitioned run: frac is null; model_* = per-GPU bytes of the "
                                 "no-reuse gather model (index + weight + one source row per nonzero) over the whole step, "
                                 "exchange included, which counts L2 hits as DRAM bytes"},
            "cpu_baseline": None,
            "e2e": {"value": nnz * sum(widths) / (e2e_ms * 1e-3), "unit": "edge*feat/s", "ms_per_step": e2e_ms,
                    "steps": e2e_steps, "h2d_bytes_per_step": io_bytes, "d2h_bytes_per_step": io_bytes},
            "gpu_launches": launches,
            "max_shard_nnz_over_mean": float(imb.item()) * world / nnz,
            "halo": {"rows_rank0": halo_rows, "remote_rows_rank0": remote_rows,
                     "bytes_per_step_rank0": halo_rows * 4 * sum(widths)},
            "exchange": "referenced remote rows only (%.0f %% of the remote rows on rank 0), " % (
                100.0 * halo_rows / max(remote_rows, 1)) + exchange_text,
            "breakdown_rank0": breakdown,
            "timeline": timeline,
            "parity": par, "parity_ok": bool(float(okmin[0]) == 1.0),
            "gcn_forward": gcn,
            "clocks": clocks,
        }
        print(json.dumps(line))
    dist.barrier()
    dist.destroy_process_group()
