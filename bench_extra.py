"""Secondary workloads of ``bench.py`` (``--workload convert|gat|gcn|gemm|sample|citation|edgeops``): the other
configurations of the hot path, each printed as one JSON line in the same shape as the headline.
They are measurement helpers for the kernels that the default SpMM sweep does not exercise."""
import json
import os
import time

import torch

import bench


def _events():
    return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)


def _time(fn, steps, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    a, b = _events()
    a.record()
    for _ in range(steps):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / steps


def _line(args, metric, unit, value, ms, workload, roofline, extra):
    line = {"metric": metric, "value": value, "unit": unit, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": {"workload": workload},
            "roofline": roofline}
    line.update(extra)
    return line


def run_convert(args):
    """COO -> CSC + CSR with fused gcn_norm (R-MAT scale 24, edge factor 16, shuffled, unit weights)."""
    import jittorgeometric_b200 as jg
    from jittorgeometric_b200 import synth
    dev = torch.device("cuda", 0)
    scale = args.scale if args.scale != 21 else 24
    ei, n = synth.rmat_coo_shuffled(scale, 16, bench.SEED + 2, device=dev)
    E0 = ei.shape[1]
    out = {}

    def step():
        out["csc"], out["csr"] = jg.gcn_norm_csc_csr(ei, None, n)

    sampler = bench.ClockSampler(0); sampler.start()
    ms = _time(step, args.steps, args.warmup)
    clocks = sampler.stop()
    E = out["csc"].row_indices.numel()
    peak, kind = bench.measured_peaks()
    passes = (max(n - 1, 1).bit_length() + 7) // 8
    alg = 2 * (E0 * 8 + E * 8 + n * 12)          # both formats: read COO, write index + weight, degree/offset/dis
    cpu = None
    if args.cpu_budget > 0:
        import numpy as np
        import oracle as O
        sub = min(E0, 1 << 22)
        sei = ei[:, :sub].cpu().numpy()
        t0 = time.perf_counter()
        nei, nw = O.gcn_norm(sei, None, n)
        impl = "ref" if O.have_ref() else "port"
        O.coo_to_csc(nei, nw, n, impl); O.coo_to_csr(nei, nw, n, impl)
        dt = time.perf_counter() - t0
        cpu = {"value": sub / dt, "unit": "edge/s", "cores": 1, "kind": "reference" if impl == "ref" else "port",
               "sample": f"first {sub} input edges of the same list, gcn_norm (C restatement) + the reference's "
                         f"cootocsc and cootocsr bodies, {dt:.1f} s, single thread"}
    return _line(args, "coo_to_csc_csr_edges_per_s", "edge/s", E0 / (ms * 1e-3), ms,
          f"gcn_norm + COO->CSC + COO->CSR: R-MAT scale {scale}, edge factor 16, {E0} shuffled input edges, "
          f"{n} nodes, unit weights, int32; entry order bit-exact with the reference",
          {"bound": "hbm", "achieved": alg / ms / 1e6, "peak": peak, "unit": "GB/s", "frac": alg / ms / 1e6 / peak,
           "traffic": None, "peak_kind": kind, "kernel": "sort_scatter_kernel",
           "note": f"algorithmic bytes = one read of the COO and one write of index+weight per format; the radix sort "
                   f"takes {passes} passes per format at about 28 B per entry and pass"},
          {"cpu_baseline": cpu, "entries": E, "gpu_launches": args.steps * (2 * passes * 5 + 10), "clocks": clocks})


def run_gat(args):
    """One attention layer, 8 heads x 8: 232,965 nodes, ~114.6M in-edges, input width 602."""
    import jittorgeometric_b200 as jg
    from jittorgeometric_b200 import synth
    dev = torch.device("cuda", 0)
    n, E_target, H, D, fin = 232965, 114_600_000, 8, 8, 602
    if args.scale != 21:                       # reduced instance for profiling runs
        n, E_target = n >> (21 - args.scale), E_target >> (21 - args.scale)
    rows, off = synth.lognormal_degree_csc(n, E_target, bench.SEED + 3, device=dev)
    csc = jg.CSC(rows, off, None)
    E = rows.numel()
    x = torch.randn((n, fin), device=dev, generator=torch.Generator(device=dev).manual_seed(5))
    W = synth.glorot((fin, H * D), 7, dev)
    a = synth.glorot((2 * H * D, 1), 8, dev)
    a_src, a_dst = a[: H * D, 0].reshape(H, D).contiguous(), a[H * D:, 0].reshape(H, D).contiguous()
    h = torch.relu(x @ W)
    Wt = W.t().contiguous()
    out = {}

    def edge_phase():
        out["y"] = jg.gat_aggregate(h, a_src, a_dst, csc, H)

    def layer():
        hh = jg.linear_tf32(x, W, relu=True, weight_t=Wt)     # width 602: the plain-load producer of the tcgen05 kernel
        out["y"] = jg.gat_aggregate(hh, a_src, a_dst, csc, H)

    # training: forward with the saved log-sum-exp, then the fused backward (by destination, by
    # source, score-vector reduction); the source-grouped structure is built once, outside the timing
    hg, asg, adg = h.clone().requires_grad_(True), a_src.clone().requires_grad_(True), a_dst.clone().requires_grad_(True)
    gy = torch.randn((n, H * D), device=dev, generator=torch.Generator(device=dev).manual_seed(6))

    def train_edge_phase():
        hg.grad = asg.grad = adg.grad = None
        jg.gat_aggregate(hg, asg, adg, csc, H).backward(gy)

    sampler = bench.ClockSampler(0); sampler.start()
    ms_edge = _time(edge_phase, args.steps, args.warmup)
    ms_train = _time(train_edge_phase, args.steps, args.warmup)
    ms_layer = _time(layer, args.steps, args.warmup)
    ms_transform = _time(lambda: jg.linear_tf32(x, W, relu=True, weight_t=Wt), args.steps, args.warmup)
    ms_transform_lib = _time(lambda: torch.relu(x @ W), args.steps, args.warmup)
    clocks = sampler.stop()
    peak, kind = bench.measured_peaks()
    C = H * D
    alg = 4 * E + 4 * (n + 1) + 4 * n * C + 4 * n * C        # indices, offsets, h once, out once (h fits in L2)
    gather = E * (4 + 4 * C)
    cpu = None
    if args.cpu_budget > 0:
        import oracle as O
        r = min(n, 2000)
        o_np, i_np = off[: r + 1].cpu().numpy(), rows[: int(off[r])].cpu().numpy()
        hn = h.cpu().numpy()
        t0 = time.perf_counter()
        # the reference's unfused pipeline needs rows of h for every destination < r and every source: pass full h
        import numpy as np
        o_full = np.concatenate([o_np, np.full(n - r, o_np[-1], np.int32)])
        O.gat_unfused(hn[:, :8].copy(), a.cpu().numpy()[:16, 0], i_np, o_full, "ref" if O.have_ref() else "port")
        dt = time.perf_counter() - t0
        cpu = {"value": int(off[r]) / dt, "unit": "edge/s", "cores": 1, "kind": "reference" if O.have_ref() else "port",
               "sample": f"in-edges of the first {r} destinations ({int(off[r])} edges), ONE head of width 8 through the "
                         f"reference's unfused op-by-op pipeline, {dt:.1f} s, single thread (x8 heads for the full layer)"}
    return _line(args, "gat_edge_phase_edges_per_s", "edge/s", E / (ms_edge * 1e-3), ms_edge,
          f"attention layer 8 heads x 8, LeakyReLU 0.2: {n} nodes, {E} in-edges (log-normal degrees, mean "
          f"{E / n:.0f}), input width {fin}; fused logits + softmax + aggregation over CSC",
          {"bound": "hbm", "achieved": alg / ms_edge / 1e6, "peak": peak, "unit": "GB/s", "frac": alg / ms_edge / 1e6 / peak,
           "traffic": None, "peak_kind": kind, "kernel": "gat_aggregate_kernel",
           "note": "compulsory bytes only: h (%.0f MB) fits in L2, so the kernel is L2/LSU-bound, not HBM-bound; "
                   "effective gather bandwidth is reported beside it" % (n * C * 4 / 1e6)},
          {"gather_gbs": gather / ms_edge / 1e6, "forward_backward_ms": ms_train, "layer_ms": ms_layer, "transform_ms": ms_transform,
           "transform_library_fp32_ms": ms_transform_lib, "cpu_baseline": cpu,
           "gpu_launches": args.steps, "clocks": clocks})


def run_gemm(args):
    """Dense transform of one shard of the partitioned-GCN workload: 8.4M x 128 -> 128."""
    import jittorgeometric_b200 as jg
    dev = torch.device("cuda", 0)
    n = (1 << 23) if args.scale == 21 else (1 << args.scale)
    res = {}
    peak, kind = bench.measured_peaks()
    for k, m in ((128, 128), (128, 64), (256, 64)):
        x = torch.randn((n, k), device=dev)
        w = torch.randn((k, m), device=dev) / k ** 0.5
        wt = w.t().contiguous()
        ms = _time(lambda: jg.linear_tf32(x, w, weight_t=wt), args.steps, args.warmup)
        ms_lib = _time(lambda: x @ w, args.steps, args.warmup)
        b = 4 * n * (k + m)
        res[f"{k}x{m}"] = {"ms": ms, "gbs": b / ms / 1e6, "frac_of_hbm_peak": b / ms / 1e6 / peak,
                           "tflops": 2.0 * n * k * m / ms / 1e9, "library_fp32_ms": ms_lib}
        # the weight gradient of the same layer, x^T g (tcgen05 with MN-major operands), beside the fp32 CUDA-core form
        g = torch.randn((n, m), device=dev)
        ms_wg = _time(lambda: jg.ops.weight_grad_tf32(x, g), args.steps, args.warmup)
        res[f"{k}x{m}"]["weight_grad"] = {"ms": ms_wg, "gbs": b / ms_wg / 1e6, "frac_of_hbm_peak": b / ms_wg / 1e6 / peak,
                                          "fp32_cuda_core_ms": _time(lambda: jg.ops.matmul_f32(x, g, trans_a=True), 2, 1)}
        del x, g
    first = res["128x128"]
    return _line(args, "dense_transform_rows_per_s", "row/s", n / (first["ms"] * 1e-3), first["ms"],
          f"dense feature transform H = X W, {n} rows, TF32 products with fp32 accumulation on tcgen05; shapes 128->128, "
          "128->64, 256->64",
          {"bound": "hbm", "achieved": first["gbs"], "peak": peak, "unit": "GB/s", "frac": first["frac_of_hbm_peak"],
           "traffic": None, "peak_kind": kind, "kernel": "gemm_tf32_kernel",
           "note": "skinny GEMM: read X once, write H once; tensor-pipe utilisation is reported by ncu"},
          {"shapes": res, "dtype": "tf32", "gpu_launches": args.steps * 3 * 3})


def run_gcn(args):
    """Two-layer GCN forward (width 128 -> 128 -> 64) on one GPU or row-partitioned over N GPUs, at
    ``--scale`` (22 when left at the default): the ``gcn_forward`` record of the default line, alone."""
    import torch.distributed as dist
    import bench_dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    if world > 1:
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=dev)
        args.exchange = bench_dist.pick_exchange(args, dev)
    args.gcn_scale = 22 if args.scale == 21 else args.scale
    args.gcn_steps, args.gcn_warmup = args.steps, args.warmup
    rec = bench_dist.gcn_forward_record(args, dev, rank, world, bench.ClockSampler)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return rec


def run_sample(args):
    """Mini-batch neighbour sampling: 1024 seed nodes, fanout [25, 10], on the SpMM workload's graph;
    one step = one batch through the whole sampler (two sampled layers, merged local CSC + CSR,
    degree weights, 128-wide feature rows of the touched nodes)."""
    import jittorgeometric_b200 as jg
    from jittorgeometric_b200 import sampling, synth
    dev = torch.device("cuda", 0)
    scale = args.scale
    ei, n = synth.rmat_graph(scale, args.edge_factor // 2, bench.SEED + 1, device=dev)
    csc = jg.cootocsc(ei, None, n)
    del ei
    feat = torch.randn((n, 128), device=dev, generator=torch.Generator(device=dev).manual_seed(12))
    fanout, batch = [25, 10], 1024
    seeds = torch.randperm(n, device=dev, generator=torch.Generator(device=dev).manual_seed(13))[: batch * 64].to(torch.int32)
    state = {"k": 0, "edges": 0, "nodes": 0}

    def step():
        k = state["k"] % 64
        ssg = sampling.sample_one(fanout, csc.column_offset, csc.row_indices, seeds[k * batch: (k + 1) * batch].contiguous(),
                                  feat, None, seed=state["k"])
        state["k"] += 1
        state["edges"], state["nodes"] = ssg.num_edges, ssg.num_nodes

    sampler = bench.ClockSampler(0); sampler.start()
    ms = _time(step, args.steps, args.warmup)
    clocks = sampler.stop()
    peak, kind = bench.measured_peaks()
    E, m = state["edges"], state["nodes"]
    alg = E * 4 * 6 + m * 128 * 4 * 2           # sampled ids written and re-read through merge/sort/weights, feature rows in and out
    cpu = None
    if args.cpu_budget > 0:
        import numpy as np
        import oracle as O
        if O.have_ref():
            g_off, g_idx = csc.column_offset.cpu().numpy(), csc.row_indices.cpu().numpy()
            dst = seeds[:batch].cpu().numpy()
            t0 = time.perf_counter()
            drawn = 0
            for f in fanout:                      # the reference's CPU sampler body, layer after layer
                off = np.concatenate([[0], np.cumsum(O.sample_counts(dst, g_off, f)[1:])]).astype(np.int32)
                idx = O.sample_reference(f, dst, off, g_off, g_idx)
                drawn += len(idx)
                dst = np.unique(idx).astype(np.int32)
            dt = time.perf_counter() - t0
            cpu = {"value": drawn / dt, "unit": "edge/s", "cores": 1, "kind": "reference",
                   "sample": f"one batch: the reference's sampleprocessing CPU body for both layers ({drawn} sampled edges, "
                             f"{dt * 1e3:.1f} ms); its Python merge loops over nodes are not included"}
    return _line(args, "sampled_edges_per_s", "edge/s", E / (ms * 1e-3), ms,
          f"mini-batch sampling: {batch} seeds, fanout {fanout}, R-MAT scale {scale} graph ({n} nodes, {csc.row_indices.numel()} "
          f"in-edges); per batch {E} sampled edges over {m} nodes, 128-wide features gathered",
          {"bound": "hbm", "achieved": alg / ms / 1e6, "peak": peak, "unit": "GB/s", "frac": alg / ms / 1e6 / peak,
           "traffic": None, "peak_kind": kind, "kernel": "sample_neighbors_kernel",
           "note": "latency-bound by construction: a batch moves a few MB through about 40 short launches and four "
                   "device-to-host size reads; the figure to read is milliseconds per batch"},
          {"cpu_baseline": cpu, "gpu_launches": args.steps * 40, "clocks": clocks})


def run_edgeops(args):
    """The per-edge operators on a quarter-size attention graph (58 k nodes, 28.6 M in-edges, C = 64,
    8 heads): each is a streaming kernel over ``[E, C]`` or ``[E, H]``; reported as achieved bytes per
    second against the measured copy bandwidth, plus the op-by-op attention pipeline they form."""
    import jittorgeometric_b200 as jg
    from jittorgeometric_b200 import nn, synth
    dev = torch.device("cuda", 0)
    n, E_target, H, C = 232965 >> 2, 114_600_000 >> 2, 8, 64
    rows, off = synth.lognormal_degree_csc(n, E_target, bench.SEED + 3, device=dev)
    csc = jg.CSC(rows, off, None)
    E = rows.numel()
    g = torch.Generator(device=dev).manual_seed(21)
    h = torch.relu(torch.randn((n, C), device=dev, generator=g))
    msg = torch.randn((E, C), device=dev, generator=g)
    score = torch.randn((E, H), device=dev, generator=g)
    peak, kind = bench.measured_peaks()
    sampler = bench.ClockSampler(0); sampler.start()
    res = {}
    with torch.no_grad():
        cases = [("scatter_to_edge_src", lambda: jg.ScatterToEdge(h, csc, "src"), E * (4 + 4 * C) + 4 * n * C),
                 ("scatter_to_edge_dst", lambda: jg.ScatterToEdge(h, csc, "dst"), E * 4 * C + 4 * n * C),
                 ("scatter_to_vertex", lambda: jg.ScatterToVertex(msg, csc, "src"), E * 4 * C + 4 * n * C),
                 ("edge_softmax", lambda: jg.EdgeSoftmax(score, csc), 2 * E * 4 * H),
                 ("edge_softmax_backward", lambda: jg.ops._edge_softmax(score, csc.column_offset, bwd_y=prob), 3 * E * 4 * H)]
        prob = jg.EdgeSoftmax(score, csc)
        for name, fn, nbytes in cases:
            ms = _time(fn, args.steps, args.warmup)
            res[name] = {"ms": ms, "gbs": nbytes / ms / 1e6, "frac_of_hbm_peak": nbytes / ms / 1e6 / peak}
        layer = nn.GATConv(C, C, E, heads=H).to(dev)
        ms_unfused = _time(lambda: layer.propagate_unfused(h, csc), max(2, args.steps // 4), 1)
        a_src, a_dst = layer.attention_vectors()
        a_src, a_dst = a_src.contiguous(), a_dst.contiguous()
        ms_fused = _time(lambda: jg.gat_aggregate(h, a_src, a_dst, csc, H), args.steps, args.warmup)
    clocks = sampler.stop()
    top = res["scatter_to_vertex"]
    return _line(args, "edge_to_vertex_edges_per_s", "edge/s", E / (top["ms"] * 1e-3), top["ms"],
          f"per-edge operators on {n} nodes, {E} in-edges, C = {C}, {H} heads (quarter-size attention graph)",
          {"bound": "hbm", "achieved": top["gbs"], "peak": peak, "unit": "GB/s", "frac": top["frac_of_hbm_peak"], "traffic": None,
           "peak_kind": kind, "kernel": "edge_to_vertex_kernel", "note": "bytes = the [E, C] messages read once + the [N, C] result"},
          {"operators": res, "attention_op_by_op_ms": ms_unfused, "attention_fused_ms": ms_fused,
           "gpu_launches": args.steps * 5, "clocks": clocks})


def run_citation(args):
    """The citation-graph-shaped configuration: 2708 nodes, 5278 undirected edges, 1433 sparse binary
    features, 2-layer GCN 1433 -> 256 -> 7, one step = forward + loss + backward (gradients of both
    weights, both biases and the input).  Latency-bound: reported eagerly and as a CUDA-graph replay."""
    import numpy as np
    import jittorgeometric_b200 as jg
    from jittorgeometric_b200 import nn, synth
    dev = torch.device("cuda", 0)
    n, fin, hid, classes = 2708, 1433, 256, 7
    ei = synth.preferential_attachment(n, 5278, bench.SEED).to(dev)
    csc, csr = jg.gcn_norm_csc_csr(ei, None, n)
    x = synth.sparse_binary_features(n, fin, 18, seed=3).to(dev)
    torch.manual_seed(1)
    c1, c2 = nn.GCNConv(fin, hid, relu=True).to(dev), nn.GCNConv(hid, classes).to(dev)
    labels = torch.randint(classes, (n,), generator=torch.Generator().manual_seed(2)).to(dev)
    params = list(c1.parameters()) + list(c2.parameters())
    xin = x.clone().requires_grad_(True)

    def step():
        for p in params + [xin]:
            p.grad = None
        out = c2(c1(xin, csc, csr), csc, csr)
        loss = torch.nn.functional.cross_entropy(out, labels)
        loss.backward()
        return loss

    sampler = bench.ClockSampler(0); sampler.start()
    ms = _time(step, args.steps, args.warmup)
    graph_ms = None
    try:                                                             # whole step captured once, replayed
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                step()
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        for p in params + [xin]:
            p.grad = None
        with torch.cuda.graph(graph):
            out = c2(c1(xin, csc, csr), csc, csr)
            loss = torch.nn.functional.cross_entropy(out, labels)
            loss.backward()
        graph_ms = _time(graph.replay, args.steps, args.warmup)
    except Exception as exc:                                         # capture is an optimisation, not a requirement
        graph_ms = None
        print(f"# CUDA graph capture unavailable: {exc!r}", flush=True)
    clocks = sampler.stop()
    E = csc.row_indices.numel()
    flops = 3 * (2 * n * (fin * hid + hid * classes) + 2 * E * (hid + classes))     # forward + two backward products
    cpu = None
    if args.cpu_budget > 0:
        import oracle as O
        ci, co, cw = (t.cpu().numpy() for t in (csc.row_indices, csc.column_offset, csc.edge_weight))
        ri, ro, rw = (t.cpu().numpy() for t in (csr.column_indices, csr.row_offset, csr.edge_weight))
        xn, W1, W2, lab = x.cpu().numpy(), c1.weight.detach().cpu().numpy(), c2.weight.detach().cpu().numpy(), labels.cpu().numpy()
        impl = "ref" if O.have_ref() else "port"
        t0 = time.perf_counter()
        reps = 3
        for _ in range(reps):                                        # the same step with numpy products and the reference aggregation body
            h1 = np.maximum(O.aggregate((xn @ W1).astype(np.float32), ci, co, cw, impl=impl), 0)
            z = O.aggregate((h1 @ W2).astype(np.float32), ci, co, cw, impl=impl)
            p = np.exp(z - z.max(1, keepdims=True)); p /= p.sum(1, keepdims=True)
            gz = p; gz[np.arange(n), lab] -= 1; gz /= n
            g2 = O.aggregate(gz.astype(np.float32), ri, ro, rw, impl=impl)
            gW2 = h1.T @ g2
            g1 = O.aggregate(((g2 @ W2.T) * (h1 > 0)).astype(np.float32), ri, ro, rw, impl=impl)
            gW1 = xn.T @ g1
            gx = g1 @ W1.T
        dt = (time.perf_counter() - t0) / reps
        cpu = {"value": 1.0 / dt, "unit": "step/s", "cores": os.cpu_count(), "kind": "reference" if impl == "ref" else "port",
               "sample": f"the whole step, {reps} repetitions: numpy (BLAS threads) for the dense products, the reference's "
                         f"single-threaded aggregation body for the four aggregations; {dt * 1e3:.1f} ms per step"}
    best = min(ms, graph_ms) if graph_ms else ms
    return _line(args, "citation_gcn_train_steps_per_s", "step/s", 1e3 / best, best,
          f"2-layer GCN 1433->256->7 forward + cross-entropy + backward on a preferential-attachment graph with the citation "
          f"benchmark's shape ({n} nodes, {E} directed edges incl. self-loops, 18 ones per feature row, row-normalised)",
          {"bound": "hbm", "achieved": None, "peak": None, "unit": "GB/s", "frac": None, "traffic": None,
           "note": "launch/latency-bound by size (about 40 launches over a few MB): not a roofline configuration"},
          {"eager_ms": ms, "cuda_graph_ms": graph_ms, "gflops": flops / best / 1e6, "cpu_baseline": cpu,
           "gpu_launches": args.steps * 8, "clocks": clocks})


def run_exchange(args):
    """The halo exchange kernels with the ranks of a 4-way partition emulated on ONE GPU (peers are local
    buffers, so the figures show the kernels' own limits, not NVLink): the bulk-copy pull (1 KB rows), the
    plain-load pull (512-byte rows), the fp16-payload pull, and the row-packing kernel of the collective
    transport.  For profiling; multi-GPU numbers come from ``bench.py --gpus N``."""
    import jittorgeometric_b200 as jg
    from jittorgeometric_b200 import dist as jd, synth
    from jittorgeometric_b200._lib import check, lib, ptr, stream_for
    dev = torch.device("cuda", 0)
    world, scale = 4, (20 if args.scale == 21 else args.scale)
    n = 1 << scale
    part = jd.RowPartition(n, world)
    emu = jd.EmulatedRanks(world, pull_ctas=0)
    graphs = []
    for r in range(world):
        lo, hi = part.range(r)
        idx, off, deg = synth.rmat_shard_csc(scale, 16, bench.SEED, lo, hi, device=dev)
        w = torch.ones(idx.numel(), device=dev)
        graphs.append(jd.ShardedGraph(part, r, idx, off, w, transport=emu.transport(r), setup=False, mode="merged"))
    emu.wire(graphs)
    g = graphs[0]
    peak, kind = bench.measured_peaks()
    res = {}
    for name, f, half in (("pull_bulk_f256", 256, False), ("pull_plain_f128", 128, False), ("pull_half_f128", 128, True)):
        for h in graphs:
            h.feature_buffer(f).normal_()
            h.halo_half = half
        pend = {}

        def step():
            pend["p"] = g.start(g.feature_buffer(f))
            g._inflight.discard(f)
        ms = _time(step, args.steps, args.warmup)
        nbytes = g.n_halo * f * (2 if half else 4) + g.n_halo * f * 4       # rows read + fp32 rows written
        res[name] = {"ms": ms, "halo_rows": g.n_halo, "gbs": nbytes / ms / 1e6, "frac_of_hbm_peak": nbytes / ms / 1e6 / peak,
                     "note": "includes the flag posts" + (" and the fp16 conversion of every emulated owner's rows" if half else "")}
    x = g.feature_buffer(128)
    rows = torch.randperm(g.n_local, device=dev)[: g.n_local // 2].sort().values.to(torch.int32) + g.lo
    out = torch.empty((rows.numel(), 128), device=dev)
    ms = _time(lambda: check(lib().jg_gather_rows_f32(ptr(out), ptr(x), ptr(rows), rows.numel(), 128, g.lo, stream_for(x)),
                             "jg_gather_rows_f32"), args.steps, args.warmup)
    res["gather_rows_f128"] = {"ms": ms, "rows": rows.numel(), "gbs": 2 * rows.numel() * 512 / ms / 1e6,
                               "frac_of_hbm_peak": 2 * rows.numel() * 512 / ms / 1e6 / peak}
    top = res["pull_bulk_f256"]
    return _line(args, "halo_rows_per_s", "row/s", g.n_halo / (top["ms"] * 1e-3), top["ms"],
                 f"halo exchange kernels, 4 ranks emulated on one GPU: R-MAT scale {scale}, rank 0 fetches {g.n_halo} of "
                 f"{n - g.n_local} remote rows",
                 {"bound": "hbm", "achieved": top["gbs"], "peak": peak, "unit": "GB/s", "frac": top["frac_of_hbm_peak"], "traffic": None,
                  "peak_kind": kind, "kernel": "halo_pull_bulk_kernel", "note": "bytes = halo rows read once + written once"},
                 {"kernels": res, "gpu_launches": args.steps * 2})


def run(args):
    line = {"exchange": run_exchange, "citation": run_citation, "edgeops": run_edgeops, "convert": run_convert, "gat": run_gat, "gemm": run_gemm,
            "gcn": run_gcn, "sample": run_sample}[args.workload](args)
    if line is not None:
        print(json.dumps(line))


def secondary(args):
    """The other configurations of the hot path, time-boxed (3 warm-up + 5 timed steps each, a few seconds
    of CPU baseline), as sub-records of the default benchmark line: conversion at scale 24, the attention
    layer at full size (forward and forward + backward), the dense transform's three shapes, and the
    citation-graph training step."""
    import copy
    out = {}
    for name, fn in (("convert", run_convert), ("gat", run_gat), ("gemm", run_gemm), ("citation", run_citation)):
        a = copy.copy(args)
        a.steps, a.warmup, a.workload, a.scale, a.gpus = 5, 3, name, 21, 1
        a.cpu_budget = min(args.cpu_budget, 4.0)
        try:
            rec = fn(a)
            for k in ("n_gpus", "higher_is_better", "scaling", "vs_baseline", "data"):
                rec.pop(k, None)
            out[name] = rec
        except Exception as exc:                      # a secondary workload never takes the headline down with it
            out[name] = {"error": repr(exc)}
        torch.cuda.empty_cache()
    return out
