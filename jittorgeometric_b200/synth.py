"""Seeded synthetic graphs with the shapes of the benchmark workloads.

Nothing is downloaded: every graph comes from a ``torch.Generator`` seeded by the
caller and is generated on whatever device is asked for (CPU for small parity
cases, CUDA for the full-size workloads).  All edge lists are ``[2, E]`` int32
(row 0 = source, row 1 = destination), as the reference operators expect
(ops/cpp/cootocsr_op.cc:46-47).
"""
import math

import torch


def _gen(seed, device):
    g = torch.Generator(device=device)
    g.manual_seed(int(seed))
    return g


def rmat_edge_batches(scale, n_edges, seed, device="cpu", a=0.57, b=0.19, c=0.19, batch=1 << 24):
    """R-MAT edge list in batches: each edge picks one quadrant per bit level with
    probabilities (a, b, c, d); bit k of (src, dst) is the (row, column) half
    chosen at level k.  No noise.  Yields int64 ``(src, dst)`` pairs of tensors; the stream depends
    only on (seed, device type, batch), so every rank of a job can regenerate it."""
    g = _gen(seed, device)
    ab, abc = a + b, a + b + c
    for start in range(0, n_edges, batch):
        m = min(batch, n_edges - start)
        src = torch.zeros(m, dtype=torch.int64, device=device)
        dst = torch.zeros(m, dtype=torch.int64, device=device)
        for level in range(scale):
            r = torch.rand(m, generator=g, device=device)
            row_bit = (r >= ab).to(torch.int64)                        # quadrants c, d
            col_bit = ((r >= a) & (r < ab) | (r >= abc)).to(torch.int64)  # quadrants b, d
            src |= row_bit << level
            dst |= col_bit << level
        yield src, dst


def rmat_edges(scale, n_edges, seed, device="cpu", a=0.57, b=0.19, c=0.19, batch=1 << 24):
    """All batches of :func:`rmat_edge_batches` as one int64 ``src, dst`` pair of length n_edges."""
    srcs, dsts = zip(*rmat_edge_batches(scale, n_edges, seed, device, a, b, c, batch))
    return torch.cat(srcs), torch.cat(dsts)


def rmat_shard_csc(scale, edge_factor, seed, lo, hi, device="cpu", relabel=True, degrees=None):
    """Destination rows ``[lo, hi)`` of the gcn-normalised graph of :func:`rmat_graph` (symmetrised,
    deduplicated, relabelled, one self-loop per node), built WITHOUT materialising the whole graph:
    the edge stream is regenerated batch by batch and only the entries whose destination lies in
    the range are kept.  Returns ``(row_indices int32 [global source ids], column_offset int32,
    in_degree int32 [hi - lo])`` in the layout ``gcn_norm`` + ``cootocsc`` give for those rows
    (sources ascending within a column, the loop last); weights follow from the degrees of both
    endpoints (:func:`gcn_weights`), the remote ones gathered from their owners."""
    n = 1 << scale
    perm = torch.randperm(n, generator=_gen(seed + 1, device), device=device) if relabel else None
    keys = []
    held = 0
    for src, dst in rmat_edge_batches(scale, edge_factor * n, seed, device):
        if perm is not None:
            src, dst = perm[src], perm[dst]
        keep = src != dst
        src, dst = src[keep], dst[keep]
        for a, b in ((src, dst), (dst, src)):                    # the edge and its mirror image
            m = (b >= lo) & (b < hi)
            keys.append((b[m] - lo) * n + a[m])                  # (destination, source): CSC order when sorted
            held += int(keys[-1].numel())
        if held > (1 << 28):                                     # bound the working set: merge what has been collected
            keys = [torch.unique(torch.cat(keys))]
            held = int(keys[0].numel())
    key = torch.unique(torch.cat(keys)) if keys else torch.empty(0, dtype=torch.int64, device=device)
    del keys
    col = key // n
    src = (key - col * n).to(torch.int32)
    counts = torch.bincount(col, minlength=hi - lo)
    del key
    deg = (counts + 1).to(torch.int32)                           # in-edges + the loop
    off = torch.zeros(hi - lo + 1, dtype=torch.int64, device=device)
    off[1:] = torch.cumsum(counts + 1, 0)
    # entries shift right by one place per earlier column (its loop); the loop closes each column
    idx = torch.empty(int(off[-1]), dtype=torch.int32, device=device)
    pos = torch.arange(src.numel(), device=device, dtype=torch.int64) + col
    idx[pos] = src
    idx[off[1:] - 1] = torch.arange(lo, hi, device=device, dtype=torch.int32)
    assert int(off[-1]) < 2**31
    return idx, off.to(torch.int32), deg


def gcn_weights(idx, off, deg_global, lo):
    """``gcn_norm`` weights of a CSC shard with unit input weights: ``(dis[src] * 1) * dis[dst]``,
    ``dis = deg^-1/2`` rounded to fp32 from double (nn/conv/gcn_conv.py:35-37), bit for bit what the
    fused conversion kernel writes."""
    dis = (1.0 / deg_global.double().sqrt()).float()
    n_rows = off.numel() - 1
    col = torch.repeat_interleave(torch.arange(lo, lo + n_rows, device=idx.device), (off[1:] - off[:-1]).long())
    return dis[idx.long()] * dis[col]


def symmetrise_dedupe(src, dst, n, relabel_seed=None):
    """Mirror every edge, drop self-loops and duplicate (src, dst) pairs, sort by
    (src, dst); optionally relabel vertices by a seeded random permutation first.
    Returns ``edge_index [2, E] int32``."""
    device = src.device
    if relabel_seed is not None:
        perm = torch.randperm(n, generator=_gen(relabel_seed, device), device=device)
        src, dst = perm[src], perm[dst]
    keep = src != dst
    src, dst = src[keep], dst[keep]
    key = torch.cat([src * n + dst, dst * n + src])
    del src, dst
    key = torch.unique(key)  # sorted
    return torch.stack([(key // n).to(torch.int32), (key % n).to(torch.int32)])


def rmat_graph(scale, edge_factor, seed, device="cpu", symmetric=True, relabel=True):
    """Graph of the SpMM and partitioned-GCN workloads: R-MAT(0.57, 0.19, 0.19,
    0.05), 2**scale nodes, edge_factor * 2**scale generated edges; symmetrised and
    deduplicated (self-loops removed), vertex ids randomly relabelled."""
    n = 1 << scale
    src, dst = rmat_edges(scale, edge_factor * n, seed, device)
    if not symmetric:
        return torch.stack([src.to(torch.int32), dst.to(torch.int32)]), n
    return symmetrise_dedupe(src, dst, n, relabel_seed=seed + 1 if relabel else None), n


def rmat_coo_shuffled(scale, edge_factor, seed, device="cpu"):
    """Edge list of the conversion workload: raw R-MAT edges (duplicates and
    self-loops kept) in a seeded random order."""
    n = 1 << scale
    src, dst = rmat_edges(scale, edge_factor * n, seed, device)
    perm = torch.randperm(src.numel(), generator=_gen(seed + 2, device), device=device)
    return torch.stack([src[perm].to(torch.int32), dst[perm].to(torch.int32)]), n


def preferential_attachment(n, n_undirected, seed):
    """Citation-graph-shaped workload: grow a preferential-attachment graph to
    exactly ``n`` nodes and ``n_undirected`` undirected edges (each new node links
    to one or two earlier nodes picked proportionally to degree), then mirror.
    Returns ``edge_index [2, 2*n_undirected] int32`` on the CPU."""
    g = _gen(seed, "cpu")
    assert n >= 3 and n - 1 <= n_undirected <= 2 * (n - 2) + 1
    extra = n_undirected - (n - 1)             # nodes (among 2..n-1) that get a second link
    two = torch.zeros(n, dtype=torch.bool)
    two[2 + torch.randperm(n - 2, generator=g)[:extra]] = True
    ends = [0, 1]                              # every edge endpoint, for degree-proportional picks
    src, dst = [0], [1]
    for v in range(2, n):
        t1 = ends[int(torch.randint(len(ends), (1,), generator=g))]
        targets = [t1]
        if two[v]:
            t2 = t1
            while t2 == t1:
                t2 = ends[int(torch.randint(len(ends), (1,), generator=g))]
            targets.append(t2)
        for t in targets:
            src.append(v)
            dst.append(t)
            ends += [v, t]
    s = torch.tensor(src, dtype=torch.int32)
    d = torch.tensor(dst, dtype=torch.int32)
    return torch.stack([torch.cat([s, d]), torch.cat([d, s])])


def sparse_binary_features(n, f, ones_per_row, seed, device="cpu"):
    """Bag-of-words-shaped features: about ``ones_per_row`` ones per row at uniform
    random columns, then each row divided by its sum
    (transforms/normalize_features.py:5)."""
    g = _gen(seed, device)
    x = torch.zeros((n, f), dtype=torch.float32, device=device)
    cols = torch.randint(f, (n, ones_per_row), generator=g, device=device)
    x.scatter_(1, cols, 1.0)
    return x / x.sum(1, keepdim=True).clamp(min=1.0)


def glorot(shape, seed, device="cpu"):
    """U(-s, s) with s = sqrt(6 / (fan_in + fan_out)) (nn/inits.py:19-22)."""
    s = math.sqrt(6.0 / (shape[-2] + shape[-1]))
    return (torch.rand(shape, generator=_gen(seed, device), device=device) * 2 - 1) * s


def lognormal_degree_csc(n, n_edges, seed, device="cpu", sigma=1.1, zipf=0.8):
    """Graph of the attention workload, built directly as CSC: in-degrees drawn
    log-normal and rescaled to sum to ``n_edges - n``, sources drawn from a
    power-law weight over nodes, one self-loop appended to every column.
    Returns ``(row_indices int32, column_offset int32)``."""
    g = _gen(seed, device)
    z = torch.randn(n, generator=g, device=device, dtype=torch.float64) * sigma
    d = torch.exp(z)
    d = d * ((n_edges - n) / d.sum())
    deg = d.round().clamp(min=1, max=n - 1).to(torch.int64) + 1  # + self-loop
    off = torch.zeros(n + 1, dtype=torch.int64, device=device)
    off[1:] = torch.cumsum(deg, 0)
    E = int(off[-1])
    assert E < 2**31
    wts = (torch.arange(1, n + 1, device=device, dtype=torch.float64)) ** (-zipf)
    wts = wts[torch.randperm(n, generator=g, device=device)]
    cdf = torch.cumsum(wts, 0)
    cdf = cdf / cdf[-1]
    rows = torch.empty(E, dtype=torch.int32, device=device)
    step = 1 << 25
    for s in range(0, E, step):
        m = min(step, E - s)
        r = torch.rand(m, generator=g, device=device, dtype=torch.float64)
        rows[s:s + m] = torch.searchsorted(cdf, r).clamp(max=n - 1).to(torch.int32)
    # the last entry of every column is its self-loop (gcn_norm-style layout, utils/loop.py:124-126)
    rows[(off[1:] - 1)] = torch.arange(n, device=device, dtype=torch.int32)
    return rows, off.to(torch.int32)
