"""GPU parity of the segment aggregation kernel (through the C ABI) against the CPU
checker: golden vectors, seeded random graphs, hubs, odd widths, empty inputs."""
import hashlib
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
G = os.path.join(os.path.dirname(__file__), "golden")


def load(name):
    return dict(np.load(os.path.join(G, name + ".npz")))


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def run(jg, x, idx, off, w, chunk=None, n_out=None):
    off_t = dev(off)
    plan = jg.ops.SpmmPlan(off_t, len(idx), chunk) if chunk else None
    y = jg.ops.segment_aggregate(dev(x), dev(idx), off_t, dev(w), n_out=n_out, plan=plan)
    torch.cuda.synchronize()
    return y.cpu().numpy()


def rel_err(y, truth, scale):
    """max |y - truth| / sum_j |w_j x_j| : the error scale of an fp32 sum of those terms."""
    return float((np.abs(y - truth) / (scale + 1e-30)).max()) if y.size else 0.0


def test_reference_smoke_inputs(cuda, oracle):
    d = load("ref_test_mp_spmm")
    assert np.array_equal(run(cuda, d["x"], d["row_indices"], d["column_offset"], d["csc_weight"]), d["out_csc"])
    assert np.array_equal(run(cuda, d["x"], d["column_indices"], d["row_offset"], d["csr_weight"]), d["out_csr"])
    d = load("ref_test_aggregate")
    assert np.array_equal(run(cuda, d["x"], d["row_indices"], d["column_offset"], d["csc_weight"]), d["out_fwd"])
    assert np.array_equal(run(cuda, d["x"], d["column_indices"], d["row_offset"], d["csr_weight"]), d["out_bwd"])


def test_citation_graph_bit_exact(cuda, oracle):
    d = load("citation_2708")
    y7 = run(cuda, d["x7"], d["row_indices"], d["column_offset"], d["csc_weight"])
    assert np.array_equal(y7, d["y7"])
    x256 = np.random.default_rng(int(d["x256_seed"]))
    _ = x256.standard_normal((2708, 7))
    x = x256.standard_normal((2708, 256)).astype(np.float32)
    y = run(cuda, x, d["row_indices"], d["column_offset"], d["csc_weight"], chunk=1024)
    assert np.array_equal(y[::97], d["y256_rows"])
    assert hashlib.sha256(y.tobytes()).digest() == d["y256_sha256"].tobytes()


def random_graph(rng, n_out, n_in, E, hubs=0, hub_deg=0):
    dst = rng.integers(0, n_out, size=E)
    if hubs:
        dst = np.concatenate([dst, np.repeat(rng.integers(0, n_out, size=hubs), hub_deg)])
    src = rng.integers(0, n_in, size=len(dst))
    order = np.argsort(dst, kind="stable")
    off = np.zeros(n_out + 1, np.int32)
    np.add.at(off, dst + 1, 1)
    off = np.cumsum(off).astype(np.int32)
    w = rng.standard_normal(len(dst)).astype(np.float32)
    return src[order].astype(np.int32), off, w


@pytest.mark.parametrize("f", [1, 3, 4, 7, 10, 16, 17, 31, 32, 33, 40, 47, 64, 65, 100, 128, 200, 256, 260, 512, 516])
def test_widths_against_oracle(cuda, oracle, f):
    rng = np.random.default_rng(100 + f)
    idx, off, w = random_graph(rng, 700, 500, 9000, hubs=2, hub_deg=300)
    x = rng.standard_normal((500, f)).astype(np.float32)
    want = oracle.aggregate(x, idx, off, w, n_out=700)
    truth, scale = oracle.aggregate_f64(x, idx, off, w, n_out=700)
    for chunk in (None, 64):
        y = run(cuda, x, idx, off, w, chunk=chunk, n_out=700)
        assert rel_err(y, truth, scale) <= 1e-5
        assert rel_err(y, want, scale) <= 1e-5
        if f < 32 or f > 64:    # one lane group walks the row alone: the reference's summation order
            deg = np.diff(off)
            rows = deg <= (chunk or 1 << 30)
            assert np.array_equal(y[rows], want[rows])


@pytest.mark.parametrize("chunk", [1, 5, 32, 1000])
def test_hub_rows_split_into_pieces(cuda, oracle, chunk):
    rng = np.random.default_rng(chunk)
    idx, off, w = random_graph(rng, 50, 400, 300, hubs=3, hub_deg=5000)
    x = rng.standard_normal((400, 128)).astype(np.float32)
    truth, scale = oracle.aggregate_f64(x, idx, off, w, n_out=50)
    y1 = run(cuda, x, idx, off, w, chunk=chunk, n_out=50)
    y2 = run(cuda, x, idx, off, w, chunk=chunk, n_out=50)
    assert rel_err(y1, truth, scale) <= 1e-5
    assert np.array_equal(y1, y2)  # no atomics on data: run-to-run identical


def test_empty_rows_and_empty_graph(cuda, oracle):
    x = np.ones((4, 128), np.float32)
    off = np.zeros(6, np.int32)
    y = run(cuda, x, np.zeros(0, np.int32), off, np.zeros(0, np.float32), n_out=5)
    assert y.shape == (5, 128) and not y.any()
    off = np.array([0, 0, 2, 2, 2, 3], np.int32)
    idx = np.array([3, 0, 1], np.int32)
    w = np.array([2, 3, 4], np.float32)
    for chunk in (None, 1):
        y = run(cuda, x, idx, off, w, chunk=chunk, n_out=5)
        assert y[:, 0].tolist() == [0, 5, 0, 0, 4]
    y = cuda.ops.segment_aggregate(torch.zeros((3, 0), device="cuda"), dev(idx), dev(off), dev(w), n_out=5)
    assert tuple(y.shape) == (5, 0)


def test_int64_indices_are_narrowed(cuda, oracle):
    d = load("ref_test_spmm")
    # transposed structure of the reference's int64 CSR smoke input (tests/test_spmmcsr.py:13-17)
    src = np.repeat(np.arange(3), np.diff(d["row_offset"]))
    order = np.argsort(d["column_indices"], kind="stable")
    toff = np.concatenate([[0], np.cumsum(np.bincount(d["column_indices"], minlength=3))])
    y = cuda.ops.segment_aggregate(dev(d["csr_x"]), dev(src[order].astype(np.int64)), dev(toff.astype(np.int64)),
                                   dev(d["csr_weight"][order]))
    assert np.array_equal(y.cpu().numpy(), d["csr_out"])


def test_bad_arguments_raise(cuda):
    x = torch.zeros((4, 8), device="cuda")
    off = torch.tensor([0, 1, 2], dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError):
        cuda.ops.segment_aggregate(x, torch.zeros(2, dtype=torch.int32, device="cuda"), off, torch.zeros(3, device="cuda"))
    with pytest.raises(RuntimeError):
        cuda.ops.segment_aggregate(x.double(), torch.zeros(2, dtype=torch.int32, device="cuda"), off, torch.zeros(2, device="cuda"))
    from jittorgeometric_b200 import _lib
    L = _lib.lib()
    st = L.jg_aggregate_f32(_lib.ptr(x), _lib.ptr(x), _lib.ptr(off), _lib.ptr(off), _lib.ptr(x), 2, 4, 8, 2, None, 0, None, 0, None)
    assert st == -3 and b"workspace" in L.jg_last_error()
    st = L.jg_aggregate_f32(None, _lib.ptr(x), _lib.ptr(off), _lib.ptr(off), _lib.ptr(x), 2, 4, 8, 2, None, 0, None, 0, None)
    assert st == -1


def test_autograd_pairing(cuda, oracle):
    d = load("citation_2708")
    csc = cuda.CSC(dev(d["row_indices"]), dev(d["column_offset"]), dev(d["csc_weight"]))
    csr = cuda.CSR(dev(d["column_indices"]), dev(d["row_offset"]), dev(d["csr_weight"]))
    x = dev(d["x7"]).requires_grad_(True)
    y = cuda.aggregateWithWeight(x, csc, csr)
    g = torch.from_numpy(np.random.default_rng(5).standard_normal((2708, 7)).astype(np.float32)).cuda()
    y.backward(g)
    want = oracle.aggregate(g.cpu().numpy(), d["column_indices"], d["row_offset"], d["csr_weight"])
    got = x.grad.cpu().numpy()
    # rows no longer than a hub piece are summed in the reference's order: bit-identical; the few
    # longer rows of this small graph are cut into pieces (short ones, so that no warp walks a long
    # row alone) and agree to rounding
    whole = np.diff(d["row_offset"]) <= cuda.ops.default_chunk(len(d["column_indices"]))
    assert whole.sum() > 2600 and not whole.all()
    assert np.array_equal(got[whole], want[whole])
    _, scale = oracle.aggregate_f64(g.cpu().numpy(), d["column_indices"], d["row_offset"], d["csr_weight"])
    assert rel_err(got, want, scale) <= 1e-5


def test_structure_validation(cuda):
    t = lambda a, dt: torch.tensor(a, dtype=dt, device="cuda")
    good_idx, good_off = t([0, 2, 1], torch.int32), t([0, 1, 1, 3], torch.int32)
    cuda.ops.validate_structure(good_idx, good_off, 3)
    for idx, off in (([0, 3, 1], [0, 1, 1, 3]),        # index out of range
                     ([0, -1, 1], [0, 1, 1, 3]),       # negative index
                     ([0, 2, 1], [0, 2, 1, 3]),        # decreasing offsets
                     ([0, 2, 1], [1, 1, 1, 3]),        # does not start at 0
                     ([0, 2, 1], [0, 1, 1, 2])):       # does not end at the entry count
        with pytest.raises(RuntimeError, match="bad structure"):
            cuda.ops.validate_structure(t(idx, torch.int32), t(off, torch.int32), 3)
    cuda.ops.validate_structure(t([], torch.int32), t([0, 0], torch.int32), 5)   # empty graph is fine


def test_cuda_graph_replay(cuda, oracle):
    """The aggregation is a fixed launch sequence with caller-owned buffers: captured once in a CUDA
    graph it can be replayed on new feature values (launch-bound small graphs)."""
    d = load("citation_2708")
    idx, off, w = dev(d["row_indices"]), dev(d["column_offset"]), dev(d["csc_weight"])
    plan = cuda.ops.SpmmPlan(off, idx.numel())
    x = torch.zeros((2708, 64), device="cuda")
    y = torch.empty_like(x)
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        cuda.ops.segment_aggregate(x, idx, off, w, plan=plan, out=y)      # warm-up outside capture
    torch.cuda.current_stream().wait_stream(s)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        cuda.ops.segment_aggregate(x, idx, off, w, plan=plan, out=y)
    rng = np.random.default_rng(3)
    for _ in range(2):
        xv = rng.standard_normal((2708, 64)).astype(np.float32)
        x.copy_(torch.from_numpy(xv))
        g.replay()
        torch.cuda.synchronize()
        got = y.cpu().numpy()
        eager = cuda.ops.segment_aggregate(x, idx, off, w, plan=plan).cpu().numpy()
        assert np.array_equal(got, eager)
        want = oracle.aggregate(xv, d["row_indices"], d["column_offset"], d["csc_weight"])
        truth, scale = oracle.aggregate_f64(xv, d["row_indices"], d["column_offset"], d["csc_weight"])
        assert rel_err(got, want, scale) <= 1e-5


@pytest.mark.parametrize("f", [7, 32, 64, 100, 128, 256, 512])
def test_fused_bias_and_relu_epilogue(cuda, f):
    """act(sum + bias) written by the aggregation kernel equals the aggregation followed by the two
    elementwise passes, bit for bit; rows split into pieces (hubs) and empty rows included."""
    rng = np.random.default_rng(40 + f)
    n = 900
    idx, off, w = random_graph(rng, n, n, 12000, hubs=2, hub_deg=3000)
    off[-1] = off[-2]                                            # make sure the last row is empty
    idx, w = idx[: off[-1]], w[: off[-1]]
    x = rng.standard_normal((n, f)).astype(np.float32)
    bias = rng.standard_normal(f).astype(np.float32)
    off_t = dev(off)
    plan = cuda.ops.SpmmPlan(off_t, len(idx), 1024)
    for pl in (plan, None):
        plain = cuda.ops.segment_aggregate(dev(x), dev(idx), off_t, dev(w), plan=pl)
        for b, relu in ((dev(bias), True), (dev(bias), False), (None, True)):
            got = cuda.ops.segment_aggregate(dev(x), dev(idx), off_t, dev(w), plan=pl, bias=b, relu=relu)
            want = plain if b is None else plain + b
            want = torch.relu(want) if relu else want
            assert torch.equal(got, want)
    assert torch.equal(got[-1], torch.zeros(f, device="cuda"))   # empty row: relu(0) with no bias
    with pytest.raises(RuntimeError):
        cuda.ops.segment_aggregate(dev(x), dev(idx), off_t, dev(w), out=plain, accumulate=True, relu=True)


def test_fused_epilogue_autograd(cuda):
    """aggregate_bias_act against the unfused composition: outputs equal, gradients of x and bias
    equal (the backward masks with the saved output and aggregates over the CSR)."""
    rng = np.random.default_rng(50)
    n, f = 600, 64
    ei = np.unique(rng.integers(0, n, size=(7000, 2)), axis=0).T.astype(np.int32)
    w = rng.random(ei.shape[1]).astype(np.float32)
    csc, csr = cuda.cootocsc(dev(ei), dev(w), n), cuda.cootocsr(dev(ei), dev(w), n)
    x0 = rng.standard_normal((n, f)).astype(np.float32)
    b0 = rng.standard_normal(f).astype(np.float32)
    g0 = dev(rng.standard_normal((n, f)).astype(np.float32))
    res = []
    for fused in (True, False):
        x, b = dev(x0).requires_grad_(True), dev(b0).requires_grad_(True)
        y = cuda.ops.aggregate_bias_act(x, csc, csr, b, relu=True) if fused else torch.relu(cuda.aggregateWithWeight(x, csc, csr) + b)
        y.backward(g0)
        res.append((y.detach(), x.grad, b.grad))
    assert torch.equal(res[0][0], res[1][0]) and torch.equal(res[0][1], res[1][1])
    assert (res[0][2] - res[1][2]).abs().max().item() <= 1e-4 * res[1][2].abs().max().item()
