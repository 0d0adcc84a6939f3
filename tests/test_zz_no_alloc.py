"""The allocation-free aggregation entry point (jg_aggregate_f32_static).

It serves callers that must not allocate device memory while they run (a server whose
memory pool is fixed at start-up, a plugin inside a process that owns the allocator): its
scratch is a fixed array inside the library instead of a caller-provided workspace.  The
test drives it through the C ABI exactly as such a caller would - preallocated inputs and
outputs, no workspace - and checks it against the workspace-taking entry point on the same
inputs, twice in a row (the second call reuses the array with the first call's leftovers in
it).  This file sorts last so that a run stopping at the first failure has already run
every other test.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def hub_graph(rng, n_out, n_in, E, hubs, hub_deg):
    dst = np.concatenate([rng.integers(0, n_out, size=E), np.repeat(rng.integers(0, n_out, size=hubs), hub_deg)])
    src = rng.integers(0, n_in, size=len(dst))
    order = np.argsort(dst, kind="stable")
    off = np.concatenate([[0], np.cumsum(np.bincount(dst, minlength=n_out))]).astype(np.int32)
    w = rng.standard_normal(len(dst)).astype(np.float32)
    return src[order].astype(np.int32), off, w


@pytest.mark.parametrize("f", [7, 64, 128])
def test_static_scratch_matches_workspace_entry_point_twice(cuda, oracle, f):
    from jittorgeometric_b200 import _lib
    L = _lib.lib()
    rng = np.random.default_rng(77 + f)
    n_out, n_in = 3000, 2500
    idx, off, w = hub_graph(rng, n_out, n_in, 40000, hubs=3, hub_deg=6000)   # hubs longer than one piece
    nnz = len(idx)
    t = lambda a: torch.from_numpy(a).cuda()
    idx_t, off_t, w_t = t(idx), t(off), t(w)
    stream = _lib.stream_for(idx_t)
    for call in range(2):
        x = rng.standard_normal((n_in, f)).astype(np.float32)
        x_t = t(x)
        want = cuda.ops.segment_aggregate(x_t, idx_t, off_t, w_t, n_out=n_out, plan=cuda.ops.SpmmPlan(off_t, nnz, 1024))
        got = torch.full((n_out, f), float("nan"), device="cuda")
        _lib.check(L.jg_aggregate_f32_static(_lib.ptr(got), _lib.ptr(x_t), _lib.ptr(idx_t), _lib.ptr(off_t),
                                             _lib.ptr(w_t), n_out, n_in, f, nnz, stream), "jg_aggregate_f32_static")
        torch.cuda.synchronize()
        got, want = got.cpu().numpy(), want.cpu().numpy()
        _, scale = oracle.aggregate_f64(x, idx, off, w, n_out=n_out)
        assert float((np.abs(got - want) / (scale + 1e-30)).max()) <= 1e-5, f"call {call}"
        # and against the CPU checker itself (the reference's sequential loop), not only the sibling entry point
        ref = oracle.aggregate(x, idx, off, w, n_out=n_out)
        assert float((np.abs(got - ref) / (scale + 1e-30)).max()) <= 1e-5, f"call {call} vs the CPU checker"
        short = np.diff(off) <= 1024                      # unsplit rows: identical summation order
        if f >= 128 or f % 4:
            assert np.array_equal(got[short], want[short]), f"call {call}"
            assert np.array_equal(got[short], ref[short]), f"call {call} vs the CPU checker"


def test_static_scratch_rejects_sizes_beyond_its_capacity(cuda):
    from jittorgeometric_b200 import _lib
    L = _lib.lib()
    assert L.jg_aggregate_static_capacity_bytes() == 32 << 20
    z = torch.zeros(8, device="cuda")
    zi = torch.zeros(8, dtype=torch.int32, device="cuda")
    # sizes only: 2e9 nonzeros at width 4096 cannot fit 32 MiB of partial rows; nothing is launched
    st = L.jg_aggregate_f32_static(_lib.ptr(z), _lib.ptr(z), _lib.ptr(zi), _lib.ptr(zi), _lib.ptr(z),
                                   1000, 1000, 4096, 2_000_000_000, _lib.stream_for(z))
    assert st == -3 and b"built-in scratch" in L.jg_last_error()
