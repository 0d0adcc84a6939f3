#!/usr/bin/env python
"""Benchmark of the message-passing hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

N = 1: the standalone SpMM workload (R-MAT scale 21, edge factor 32, symmetrised,
gcn_norm weights, feature width swept over 32/64/128/256).  One step = one
aggregation at every width of the sweep.  N > 1 (under torchrun): the same graph
split into N contiguous destination-row shards, halo feature rows exchanged over
NCCL, strong scaling.  Prints ONE JSON line (rank 0).
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WIDTHS = (32, 64, 128, 256)
SEED = 20261125 + 1


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines, self.first = index, None, [], 0

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(self.index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def mark(self, wait_s=4.0):
        """Call where the timed region starts (the sampler was started before the warm-up: nvidia-smi takes
        up to a few seconds to deliver its first line on a box with several GPUs).  Waits for that first line,
        then remembers how many lines came before the timed region."""
        t0 = time.time()
        while self.proc is not None and not self.lines and time.time() - t0 < wait_s:
            time.sleep(0.02)
        self.first = len(self.lines)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        t0 = time.time()
        while not self.lines and time.time() - t0 < 3.0:      # a slow start of nvidia-smi: wait for its first line
            time.sleep(0.05)
        self.proc.terminate()
        self.t.join(timeout=2)
        sm, mx, reasons = [], [], set()
        window = self.lines[self.first:]
        if not window:                      # timed region shorter than one sampling period: the nearest samples
            window = self.lines[-3:]
        for ln in window:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 8:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def build_graph(device, scale=21, edge_factor=32):
    """CSC of the gcn-normalised symmetric R-MAT graph (setup, outside every timed region).
    On a GPU the library's own fused gcn_norm + conversion builds it; the CPU-only reference arm
    (no CUDA device) builds the same layout with torch tensor operations."""
    from jittorgeometric_b200 import synth
    import jittorgeometric_b200 as jg
    ei, n = synth.rmat_graph(scale, edge_factor, SEED, device=device)
    if torch.device(device).type == "cuda":
        csc, _ = jg.gcn_norm_csc_csr(ei, None, n, want_csr=False)
        return jg.CSC(csc.row_indices.clone(), csc.column_offset, csc.edge_weight.clone()), n
    loops = torch.arange(n, dtype=torch.int32, device=device)
    src = torch.cat([ei[0], loops]); dst = torch.cat([ei[1], loops])
    deg = torch.bincount(dst.long(), minlength=n).to(torch.float32)
    dis = (1.0 / deg.double().sqrt()).float()
    order = torch.sort(dst.long(), stable=True)[1]
    src, dst = src[order], dst[order]
    w = (dis[src.long()] * 1.0) * dis[dst.long()]
    off = torch.zeros(n + 1, dtype=torch.int32, device=device)
    off[1:] = torch.cumsum(deg.to(torch.int64), 0).to(torch.int32)
    return jg.CSC(src.contiguous(), off, w.contiguous()), n


def measured_traffic(nnz, widths):
    """DRAM bytes (read + write) per aggregation launch at each width, from the committed table of ncu
    counters (``dram__bytes_read.sum + dram__bytes_write.sum``, one capture at full size).  The record is
    used only for the workload it was taken on (same nonzero count) and only while the kernel source
    it was taken with is unchanged; otherwise there is no traffic figure (``None``)."""
    import hashlib
    table = os.path.join(ROOT, "profiles", "dram_traffic.json")
    src = os.path.join(ROOT, "jittorgeometric_b200", "csrc", "spmm.cu")
    try:
        rec = json.load(open(table))["aggregate_rows_kernel"]["spmm_sweep"]
        sha = hashlib.sha256(open(src, "rb").read()).hexdigest()
    except (OSError, KeyError, ValueError):
        return None
    if rec.get("nnz") != nnz or rec.get("source_sha256") != sha:
        return None
    out = {}
    for f in widths:
        b = rec.get("bytes", {}).get(str(f))
        if b is None:
            return None
        out[f] = int(b)
    return out


def alg_bytes(nnz, n, f):
    """No-reuse gather model: per nonzero its index, weight and one f-wide source row;
    offsets read once; every output row written once."""
    return nnz * (4 + 4 + 4 * f) + 4 * (n + 1) + 4 * n * f


def min_bytes(nnz, n, f):
    """Compulsory bytes: every index and weight once, X read once, Y written once."""
    return 8 * nnz + 4 * (n + 1) + 8 * n * f


def cpu_reference_sample(csc, n, widths, budget_s, xs=None, ys=None):
    """Times the reference's own CPU aggregation (compiled reference body when present,
    else the C restatement) on the first rows of the same CSC: a bounded sample."""
    import numpy as np
    import oracle as O
    impl = "ref" if O.have_ref() else "port"
    off = csc.column_offset.cpu().numpy()
    idx_all = csc.row_indices.cpu().numpy()
    w_all = csc.edge_weight.cpu().numpy()
    rng = np.random.default_rng(SEED)
    per_width = budget_s / len(widths)
    done_ef, done_t, rows_used = 0.0, 0.0, []
    parity = {}
    for f in widths:
        # the GPU run's own X when there is one, so that the two results can be compared
        x = rng.standard_normal((n, f), dtype=np.float32) if xs is None else xs[f].cpu().numpy()
        # calibrate on 20k rows, then size the sample for the per-width budget
        r0 = min(n, 20000)
        t0 = time.perf_counter()
        _sample_aggregate(O, impl, x, idx_all, off, w_all, r0)
        dt = time.perf_counter() - t0
        rate = max(int(off[r0]), 1) / max(dt, 1e-6)
        target = int(rate * per_width)
        r = int(np.searchsorted(off, min(target, int(off[-1])), side="left"))
        r = max(min(r, n), r0)
        t0 = time.perf_counter()
        want = _sample_aggregate(O, impl, x, idx_all, off, w_all, r)
        dt = time.perf_counter() - t0
        done_ef += float(off[r]) * f
        done_t += dt
        rows_used.append(r)
        if ys is not None:
            # full-size parity: the GPU's rows [0, r) of this width against the CPU result on the same X;
            # error scale = sum |w x| per element (float64 on the GPU, sampled rows only)
            got = ys[f][:r].cpu().numpy()
            e = int(off[r])
            dev = ys[f].device
            seg = torch.repeat_interleave(torch.arange(r, device=dev), (csc.column_offset[1:r + 1] - csc.column_offset[:r]).long())
            scale = torch.zeros((r, f), dtype=torch.float64, device=dev)
            step = (1 << 27) // f
            for a in range(0, e, step):
                b = min(e, a + step)
                term = (xs[f][csc.row_indices[a:b].long()].double() * csc.edge_weight[a:b].double().unsqueeze(1)).abs()
                scale.index_add_(0, seg[a:b], term)
            err = np.abs(got - want) / (scale.cpu().numpy() + 1e-30)
            parity[str(f)] = {"rows": r, "max_rel_err": float(err.max()),
                              "bit_identical_rows": int((got == want).all(axis=1).sum())}
            del scale, seg
    return {"value": done_ef / done_t, "unit": "edge*feat/s", "cores": 1, "parity": parity or None,
            "kind": "reference" if impl == "ref" else "port",
            "sample": f"first {rows_used} destination rows of the same CSC at widths {list(widths)}; "
                      f"{done_t:.1f} s of single-thread CPU work (the reference loop is single-threaded)",
            "seconds": done_t}


def _sample_aggregate(O, impl, x, idx, off, w, rows):
    """Aggregates destination rows [0, rows) with the CPU checker."""
    import ctypes
    import numpy as np
    sub_off = np.ascontiguousarray(off[: rows + 1])
    out = np.zeros((rows, x.shape[1]), np.float32)
    if impl == "ref":
        # the reference body takes its row count from x: hand it a view with `rows` rows whose
        # base pointer is x itself, so gathered source rows beyond `rows` are still addressable
        L = O.ref_lib()
        L.ref_aggregate(out.ctypes.data_as(O.oracle.c_f32p), x.ctypes.data_as(O.oracle.c_f32p),
                        idx.ctypes.data_as(O.oracle.c_i32p), sub_off.ctypes.data_as(O.oracle.c_i32p),
                        w.ctypes.data_as(O.oracle.c_f32p), ctypes.c_long(rows), ctypes.c_long(x.shape[1]),
                        ctypes.c_long(int(sub_off[-1])))
    else:
        O.port_lib().orc_aggregate(out.ctypes.data_as(O.oracle.c_f32p), x.ctypes.data_as(O.oracle.c_f32p),
                                   idx.ctypes.data_as(O.oracle.c_i32p), sub_off.ctypes.data_as(O.oracle.c_i32p),
                                   w.ctypes.data_as(O.oracle.c_f32p), ctypes.c_int64(rows), ctypes.c_int64(x.shape[1]))
    return out


def run_reference(args):
    """Reference arm: the reference's CPU aggregation on this box's host cores, rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    device = "cuda" if torch.cuda.is_available() else "cpu"
    scale = args.scale if device == "cuda" else min(args.scale, 16)
    csc, n = build_graph(device, scale, args.edge_factor)
    nnz = csc.row_indices.numel()
    per_step = []
    res = None
    for _ in range(args.warmup + args.steps):
        res = cpu_reference_sample(csc, n, WIDTHS, budget_s=max(2.0, 60.0 / (args.warmup + args.steps)))
        per_step.append(res)
    timed = per_step[args.warmup:]
    value = sum(r["value"] for r in timed) / len(timed)
    res = dict(timed[-1]); res["value"] = value
    line = {
        "impl": "reference", "metric": "spmm_edge_feat_per_s", "value": value, "unit": "edge*feat/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * sum(r["seconds"] for r in timed) / len(timed),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(scale, args.edge_factor, n, nnz, args.gpus),
        "cpu_baseline": res,
        "e2e": {"value": value, "unit": "edge*feat/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def workload_config(scale, ef, n, nnz, gpus):
    return {"workload": f"standalone SpMM Y=A*X: R-MAT(0.57,0.19,0.19,0.05) scale {scale}, edge factor {ef}, "
                        "symmetrised, deduplicated, vertex ids relabelled, self-loops + gcn_norm fp32 weights, "
                        "int32 indices; X fp32 N(0,1); one step = widths 32,64,128,256",
            "nodes": n, "nnz": nnz, "widths": list(WIDTHS),
            "l2": "inputs larger than L2 (indices+weights %.0f MB, X %.0f-%.0f MB)" % (
                nnz * 8 / 1e6, n * 32 * 4 / 1e6, n * 256 * 4 / 1e6),
            "partition": "none" if gpus == 1 else f"{gpus} contiguous destination-row shards, compact-halo exchange over NVLink"}


def run_single(args):
    import jittorgeometric_b200 as jg
    from jittorgeometric_b200 import ops
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    csc, n = build_graph(dev, args.scale, args.edge_factor)
    nnz = csc.row_indices.numel()
    plan = ops.SpmmPlan(csc.column_offset, nnz)
    g = torch.Generator(device=dev); g.manual_seed(SEED)
    xs = {f: torch.randn((n, f), generator=g, device=dev) for f in WIDTHS}
    ys = {f: torch.empty((n, f), device=dev) for f in WIDTHS}

    def step(events=None):
        for f in WIDTHS:
            if events is not None:
                events[f][0].record()
            ops.segment_aggregate(xs[f], csc.row_indices, csc.column_offset, csc.edge_weight, plan=plan, out=ys[f])
            if events is not None:
                events[f][1].record()

    sampler = ClockSampler(dev.index); sampler.start()
    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    evs = [{f: (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for f in WIDTHS}
           for _ in range(args.steps)]
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    sampler.mark()
    t0.record()
    for k in range(args.steps):
        step(evs[k])
    t1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms_step = t0.elapsed_time(t1) / args.steps
    per_f = {f: sum(e[f][0].elapsed_time(e[f][1]) for e in evs) / args.steps for f in WIDTHS}

    peak, peak_kind = measured_peaks()
    traffic = measured_traffic(nnz, WIDTHS)
    sweep = {}
    for f in WIDTHS:
        b, bm = alg_bytes(nnz, n, f), min_bytes(nnz, n, f)
        t = per_f[f]
        sweep[str(f)] = {"ms": t, "gflops": 2.0 * nnz * f / t / 1e6,
                         "dram_gbs": traffic[f] / t / 1e6 if traffic else None,
                         "frac": traffic[f] / t / 1e6 / peak if traffic else None,
                         "traffic": traffic[f] if traffic else None,
                         "traffic_over_compulsory": traffic[f] / bm if traffic else None,
                         "model_gbs": b / t / 1e6, "model_frac": b / t / 1e6 / peak,
                         "min_gbs": bm / t / 1e6, "min_frac": bm / t / 1e6 / peak}
    total_bytes = sum(alg_bytes(nnz, n, f) for f in WIDTHS)
    total_min = sum(min_bytes(nnz, n, f) for f in WIDTHS)
    total_traffic = sum(traffic.values()) if traffic else None
    kernel_ms = sum(per_f.values())
    achieved = total_traffic / kernel_ms / 1e6 if traffic else None
    value = nnz * sum(WIDTHS) / (ms_step * 1e-3)

    # end to end through the public API with host buffers: X from pinned host memory, Y back to pinned host memory
    hx = {f: torch.empty((n, f), dtype=torch.float32).pin_memory() for f in WIDTHS}
    for f in WIDTHS:
        hx[f].copy_(xs[f])
    hy = {f: torch.empty((n, f), dtype=torch.float32).pin_memory() for f in WIDTHS}
    dx = {f: torch.empty((n, f), device=dev) for f in WIDTHS}

    # Every step copies every X from pinned host memory and every Y back.  Uploads, aggregations and
    # downloads run on three streams chained by events, so the two PCIe directions and the kernels
    # overlap across the widths of a step (what a caller feeding host buffers would do); the timed
    # region ends when the last download has finished.
    cur = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    ev_in = {f: torch.cuda.Event() for f in WIDTHS}
    ev_done = {f: torch.cuda.Event() for f in WIDTHS}
    ev_out = {f: torch.cuda.Event() for f in WIDTHS}
    for f in WIDTHS:
        ev_done[f].record(cur); ev_out[f].record(cur)

    def e2e_step():
        for f in WIDTHS:
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_done[f])                     # last step's aggregation has read dx[f]
                dx[f].copy_(hx[f], non_blocking=True)
                ev_in[f].record(s_in)
            cur.wait_event(ev_in[f])
            cur.wait_event(ev_out[f])                           # last step's download has read ys[f]
            y = ops.segment_aggregate(dx[f], csc.row_indices, csc.column_offset, csc.edge_weight, plan=plan, out=ys[f])
            ev_done[f].record(cur)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_done[f])
                hy[f].copy_(y, non_blocking=True)
                ev_out[f].record(s_out)

    def e2e_join():
        cur.wait_stream(s_in); cur.wait_stream(s_out)

    e2e_steps = max(1, min(args.steps, 5))
    e2e_ms = float("nan")
    if not args.skip_e2e:
        e2e_step(); e2e_join(); torch.cuda.synchronize()
        t0.record()
        for _ in range(e2e_steps):
            e2e_step()
        e2e_join()
        t1.record(); torch.cuda.synchronize()
        e2e_ms = t0.elapsed_time(t1) / e2e_steps
    io_bytes = sum(n * f * 4 for f in WIDTHS)

    cpu = cpu_reference_sample(csc, n, WIDTHS, budget_s=args.cpu_budget, xs=xs, ys=ys) if args.cpu_budget > 0 else None
    parity = cpu.pop("parity") if cpu else None
    line = {
        "metric": "spmm_edge_feat_per_s", "value": value, "unit": "edge*feat/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.scale, args.edge_factor, n, nnz, 1),
        "gflops": 2.0 * value / 1e9,
        "sweep": sweep,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak if achieved else None, "traffic": total_traffic, "peak_kind": peak_kind,
                     "kernel": "aggregate_rows_kernel",
                     "model_gbs": total_bytes / kernel_ms / 1e6, "model_frac": total_bytes / kernel_ms / 1e6 / peak,
                     "min_gbs": total_min / kernel_ms / 1e6, "min_frac": total_min / kernel_ms / 1e6 / peak,
                     "note": "achieved / frac = DRAM bytes the four aggregation launches really move (ncu dram__bytes read + "
                             "write, one capture at full size, kept as a table beside the ncu summaries and dropped when the "
                             "kernel source changes) / CUDA-event time of the same launches, summed over the widths; model_* = "
                             "no-reuse gather model (index + weight + one source row per nonzero, output written once), which "
                             "counts L2 hits as DRAM bytes and can exceed the peak; min_* = compulsory bytes"},
        "cpu_baseline": cpu,
        "parity": parity,
        "parity_ok": bool(parity) and all(v["max_rel_err"] <= 1e-5 for v in parity.values()),
        "e2e": {"value": nnz * sum(WIDTHS) / (e2e_ms * 1e-3), "unit": "edge*feat/s", "ms_per_step": e2e_ms, "steps": e2e_steps,
                "h2d_bytes_per_step": io_bytes, "d2h_bytes_per_step": io_bytes},
        "gpu_launches": args.steps * len(WIDTHS) * 2,
        "clocks": clocks,
    }
    # free the sweep before the other workloads are built
    del xs, ys, dx, hx, hy, csc, plan
    torch.cuda.empty_cache()
    if not args.skip_secondary:
        import bench_extra
        line["secondary"] = bench_extra.secondary(args)
    if args.gcn_scale > 0:
        import bench_dist
        torch.cuda.empty_cache()
        line["gcn_forward"] = bench_dist.gcn_forward_record(args, dev, 0, 1, ClockSampler)
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--scale", type=int, default=21)
    ap.add_argument("--edge-factor", type=int, default=32)
    ap.add_argument("--cpu-budget", type=float, default=16.0, help="seconds of CPU-baseline work (0 = skip)")
    ap.add_argument("--workload", default="spmm", choices=["spmm", "convert", "gat", "gcn", "gemm", "sample", "citation", "edgeops", "exchange"],
                    help="spmm (default, the headline) or one of the other hot-path workloads (1 GPU; gcn also N > 1)")
    ap.add_argument("--widths", default=None, help="comma-separated subset of the sweep (profiling runs)")
    ap.add_argument("--skip-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--skip-secondary", action="store_true", help="skip the secondary workloads of the default line")
    ap.add_argument("--exchange", default="direct", choices=["direct", "nccl"],
                    help="N > 1: halo rows pulled out of peer memory (default) or packed + one NCCL all-to-all")
    ap.add_argument("--gcn-scale", type=int, default=26, help="R-MAT scale of the gcn_forward sub-record (0 = skip)")
    ap.add_argument("--gcn-halo", default="fp16", choices=["fp16", "fp32"],
                    help="N > 1, gcn_forward: payload of the halo rows (fp16 stays within 5e-4, inside the 2e-3 of the TF32 transform)")
    ap.add_argument("--gcn-steps", type=int, default=10)
    ap.add_argument("--gcn-warmup", type=int, default=3)
    args = ap.parse_args()
    global WIDTHS
    if args.widths:
        WIDTHS = tuple(int(v) for v in args.widths.split(","))
    args.width_list = WIDTHS
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        return run_reference(args)
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path)")
    if args.workload != "spmm":
        import bench_extra
        return bench_extra.run(args)
    if args.gpus == 1:
        return run_single(args)
    import bench_dist
    return bench_dist.run(args)


if __name__ == "__main__":
    main()
