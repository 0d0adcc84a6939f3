"""GPU parity of the tcgen05 dense transform against a float64 matmul (TF32 tolerance 2e-3)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def run(cuda, n, k, m, bias, relu, seed=0):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((n, k)).astype(np.float32)
    w = (rng.standard_normal((k, m)) / np.sqrt(k)).astype(np.float32)
    b = rng.standard_normal(m).astype(np.float32) if bias else None
    got = cuda.ops.linear_tf32(torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda(),
                               None if b is None else torch.from_numpy(b).cuda(), relu=relu, check_status=True)
    want = x.astype(np.float64) @ w.astype(np.float64)
    if b is not None:
        want = want + b
    if relu:
        want = np.maximum(want, 0)
    scale = np.abs(x).astype(np.float64) @ np.abs(w).astype(np.float64) + (np.abs(b) if b is not None else 0)
    return got.cpu().numpy(), want, scale


@pytest.mark.parametrize("n,k,m", [(128, 32, 16), (1000, 128, 128), (5000, 256, 64), (3000, 128, 7), (777, 64, 256),
                                   (20000, 128, 64), (129, 36, 24), (40000, 604, 64),
                                   (5000, 602, 64), (2708, 1433, 256), (300, 7, 5), (1000, 33, 16)])
def test_against_float64(cuda, n, k, m):
    assert cuda.ops.linear_tf32_supported(n, k, m)
    got, want, scale = run(cuda, n, k, m, bias=False, relu=False, seed=n + k + m)
    assert np.isfinite(got).all()
    assert (np.abs(got - want) / scale).max() <= 2e-3


def test_bias_and_relu_epilogue(cuda):
    got, want, scale = run(cuda, 3000, 128, 128, bias=True, relu=True, seed=3)
    assert (np.abs(got - want) / scale).max() <= 2e-3
    assert (got >= 0).all() and (got == 0).any()


def test_runs_are_identical_and_large(cuda):
    x = torch.randn((300000, 128), device="cuda")
    w = torch.randn((128, 128), device="cuda") / 11.3
    a = cuda.ops.linear_tf32(x, w, check_status=True)
    b = cuda.ops.linear_tf32(x, w, check_status=True)
    assert torch.equal(a, b)
    ref = (x.double() @ w.double())
    assert ((a.double() - ref).abs() / (x.double().abs() @ w.double().abs())).max().item() <= 2e-3


def test_unsupported_shapes_are_refused(cuda):
    assert cuda.ops.linear_tf32_supported(100, 602, 64)          # row pitch not a multiple of 16 bytes: plain-load producer
    assert not cuda.ops.linear_tf32_supported(100, 128, 257)
    with pytest.raises(RuntimeError):
        cuda.ops.linear_tf32(torch.zeros((10, 128), device="cuda"), torch.zeros((128, 300), device="cuda"))
