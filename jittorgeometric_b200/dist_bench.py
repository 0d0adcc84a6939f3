"""Multi-GPU leg of ``bench.py``: the SpMM sweep on the same graph, split into one contiguous
destination-row shard per rank (strong scaling).  Launched by torchrun, one process per GPU."""
import json
import os

import torch
import torch.distributed as dist

from . import dist as jd


def run(args):
    import bench  # the repository's bench.py (graph builder, clock sampler, workload description)
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    widths = tuple(getattr(args, "width_list", bench.WIDTHS))
    bench.WIDTHS = widths
    # every rank generates the same graph from the seed and keeps its own rows
    csc, n = bench.build_graph(dev, args.scale, args.edge_factor)
    nnz = csc.row_indices.numel()
    part = jd.RowPartition(n, world)
    exchange = os.environ.get("JG_EXCHANGE", "peer")
    mode = os.environ.get("JG_DIST_MODE", "merged")
    shard = jd.shard_rows(csc.row_indices, csc.column_offset, csc.edge_weight, part, rank)
    if exchange == "peer":
        # symmetric memory is probed collectively, so every rank takes the same branch
        ok = torch.ones(1, device=dev)
        try:
            import torch.distributed._symmetric_memory as symm
            probe = symm.empty((16,), dtype=torch.float32, device=dev)
            symm.rendezvous(probe, dist.group.WORLD.group_name)
        except Exception:
            ok.zero_()
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if float(ok.item()) == 0.0:
            exchange = "nccl"
    g = jd.ShardedGraph(part, rank, *shard, exchange=exchange, mode=mode)
    local_nnz = int(g.merged[0].numel()) if g.mode == "merged" else g.interior[0].numel() + g.halo[0].numel()
    halo_rows, remote_rows = g.n_halo, n - g.n_local
    del csc
    torch.cuda.empty_cache()
    gen = torch.Generator(device=dev); gen.manual_seed(bench.SEED + 17 * rank)
    xs = {}
    for f in widths:
        x = g.feature_buffer(f, torch.empty(0, device=dev))     # the head of the buffer the aggregation reads
        x[: g.n_local] = torch.randn((g.n_local, f), generator=gen, device=dev)
        xs[f] = x

    def step():
        # the four aggregations are independent: every exchange is started first (pack + pulls on the
        # copy engines), so the halo rows of the next width travel underneath the current kernel
        pending = [g.start(xs[f]) for f in widths]
        for p in pending:
            g.finish(p)

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize(); dist.barrier()
    sampler = bench.ClockSampler(dev.index)
    if rank == 0:
        sampler.start()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(); dist.barrier(); torch.cuda.synchronize()
    t0.record()
    for _ in range(args.steps):
        step()
    t1.record()
    torch.cuda.synchronize(); dist.barrier()
    clocks = sampler.stop() if rank == 0 else None
    ms = torch.tensor([t0.elapsed_time(t1) / args.steps], device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_step = float(ms.item())

    # end to end: the rank's feature rows from pinned host memory, its output rows back to the host
    hx = {f: torch.empty((max(g.n_local, 1), f)).pin_memory() for f in widths}
    hy = {f: torch.empty((g.n_local, f)).pin_memory() for f in widths}
    for f in widths:
        hx[f].copy_(xs[f])
    e2e_ms = float("nan")
    if not args.skip_e2e:
        # uploads, exchanges + kernels and downloads on three event-chained streams, as in the 1-GPU leg
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

        e2e_steps = max(1, min(args.steps, 5))
        e2e_step(); e2e_join(); torch.cuda.synchronize(); dist.barrier()
        t0.record()
        for _ in range(e2e_steps):
            e2e_step()
        e2e_join()
        t1.record(); torch.cuda.synchronize(); dist.barrier()
        e = torch.tensor([t0.elapsed_time(t1) / e2e_steps], device=dev)
        dist.all_reduce(e, op=dist.ReduceOp.MAX)
        e2e_ms = float(e.item())
    imb = torch.tensor([float(local_nnz)], device=dev)
    dist.all_reduce(imb, op=dist.ReduceOp.MAX)

    if rank == 0:
        peak, peak_kind = bench.measured_peaks()
        total_bytes = sum(bench.alg_bytes(nnz, n, f) for f in widths)
        achieved = total_bytes / world / ms_step / 1e6
        io_bytes = sum(n * f * 4 for f in widths)
        line = {
            "metric": "spmm_edge_feat_per_s", "value": nnz * sum(widths) / (ms_step * 1e-3), "unit": "edge*feat/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": bench.workload_config(args.scale, args.edge_factor, n, nnz, world),
            "gflops": 2.0 * nnz * sum(widths) / (ms_step * 1e-3) / 1e9,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": None, "peak_kind": peak_kind, "kernel": "aggregate_rows_kernel",
                         "note": "per-GPU algorithmic bytes (no-reuse gather model / world size) over the whole step, "
                                 "shard exchange included"},
            "cpu_baseline": None,
            "e2e": {"value": nnz * sum(widths) / (e2e_ms * 1e-3), "unit": "edge*feat/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": io_bytes, "d2h_bytes_per_step": io_bytes},
            "gpu_launches": args.steps * len(widths) * 5,
            "max_shard_nnz_over_mean": float(imb.item()) * world / nnz,
            "exchange": ("referenced remote rows only (%.0f %% of the remote rows on rank 0), packed by their owners and "
                         % (100.0 * halo_rows / max(remote_rows, 1)) +
                         ("pulled from peer memory over NVLink by the copy engines, overlapped with interior rows"
                          if exchange == "peer" else "exchanged with one NCCL all-to-all per aggregation")),
            "clocks": clocks,
        }
        print(json.dumps(line))
    dist.destroy_process_group()
