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
                                   (5000, 602, 64), (2708, 1433, 256), (300, 7, 5), (1000, 33, 16),
                                   (3000, 128, 300), (2000, 64, 512), (1500, 1433, 600), (900, 602, 1030), (233000, 602, 64)])
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
    assert cuda.ops.linear_tf32_supported(100, 128, 257)          # wider than one accumulator: 256-column tiles
    assert not cuda.ops.linear_tf32_supported(100, 128, 5000)
    with pytest.raises(RuntimeError):
        cuda.ops.linear_tf32(torch.zeros((10, 128), device="cuda"), torch.zeros((128, 5000), device="cuda"))


@pytest.mark.parametrize("n,k,m,relu", [(5000, 128, 64, True), (3001, 602, 64, True), (2048, 64, 128, False), (1000, 300, 16, False)])
def test_trainable_transform(cuda, n, k, m, relu):
    """Forward and both gradients of the TF32 transform against float64 autograd, at the TF32 bar
    (2e-3 of the sum of absolute products); k = 300 exceeds the kernel's output width for the
    input gradient and takes the library matmul there."""
    g = torch.Generator(device="cuda").manual_seed(n + k)
    x0 = torch.randn((n, k), device="cuda", generator=g)
    w0 = torch.randn((k, m), device="cuda", generator=g) * 0.1
    go = torch.randn((n, m), device="cuda", generator=g)
    x, w = x0.clone().requires_grad_(True), w0.clone().requires_grad_(True)
    y = cuda.ops.linear_tf32_autograd(x, w, relu=relu)
    y.backward(go)
    xd, wd = x0.double(), w0.double()
    yd = xd @ wd
    yd = torch.relu(yd) if relu else yd
    # ReLU decisions differ where the pre-activation is within TF32 rounding of zero; the gradients are
    # checked for the decisions the kernel took
    same = ((y > 0) == (yd > 0)) if relu else torch.ones_like(y, dtype=torch.bool)
    assert same.float().mean().item() > 0.999
    scale_y = x0.abs().double() @ w0.abs().double()
    assert (((y.double() - yd).abs() / (scale_y + 1e-30))[same]).max().item() <= 2e-3
    gm = go.double() * ((y > 0) if relu else 1.0)
    want_gx, want_gw = gm @ wd.t(), xd.t() @ gm
    scale_x = gm.abs() @ w0.abs().double().t()
    assert ((x.grad.double() - want_gx).abs() / (scale_x + 1e-30)).max().item() <= 2e-3
    scale_w = x0.abs().double().t() @ gm.abs()
    assert ((w.grad.double() - want_gw).abs() / (scale_w + 1e-30)).max().item() <= 2e-3


def test_gcn_layer_trains_in_tf32(cuda):
    from jittorgeometric_b200 import nn
    torch.manual_seed(0)
    n = 3000
    ei = torch.randint(0, n, (2, 40000), device="cuda", dtype=torch.int32)
    csc, csr = cuda.gcn_norm_csc_csr(ei, None, n)
    x = torch.randn(n, 128, device="cuda")
    a, b = nn.GCNConv(128, 64, tf32=True, relu=True).cuda(), nn.GCNConv(128, 64, tf32=False, relu=True).cuda()
    with torch.no_grad():
        b.weight.copy_(a.weight)
    outs = []
    for layer in (a, b):
        layer(x, csc, csr).square().mean().backward()
        outs.append(layer.weight.grad.clone())
    assert (outs[0] - outs[1]).abs().max().item() <= 5e-3 * outs[1].abs().max().item()


@pytest.mark.parametrize("n,k,m", [(5000, 128, 128), (3001, 128, 64), (777, 96, 8), (2000, 64, 512)])
def test_second_output_in_fp16(cuda, n, k, m):
    """The fp16 copy written from the same epilogue is the round-to-nearest fp16 of the fp32 result."""
    g = torch.Generator(device="cuda").manual_seed(n + m)
    x = torch.randn((n, k), device="cuda", generator=g)
    w = torch.randn((k, m), device="cuda", generator=g) / k ** 0.5
    b = torch.randn(m, device="cuda", generator=g)
    out = torch.empty((n, m), device="cuda")
    half = torch.full((n + 3, m), float("nan"), dtype=torch.float16, device="cuda")
    y = cuda.ops.linear_tf32(x, w, b, relu=True, out=out, out_half=half, check_status=True)
    assert y.data_ptr() == out.data_ptr()
    assert torch.equal(half[:n], out.to(torch.float16))
    assert torch.isnan(half[n:]).all()                       # rows beyond n are not touched
    assert torch.equal(out, cuda.ops.linear_tf32(x, w, b, relu=True))


def test_status_word_is_polled_without_a_synchronisation(cuda):
    """The transform reports a bounded wait that ran out through a pinned host word.  After normal runs it is
    zero; once set (here by hand: nothing on the device is made to fail) the next call refuses to carry on
    and clears it."""
    from jittorgeometric_b200 import ops
    x = torch.randn((4096, 128), device="cuda")
    w = torch.randn((128, 64), device="cuda")
    for _ in range(3):
        ops.linear_tf32(x, w)
    ops.check_transform_status(x.device, synchronize=True)          # nothing to report
    word = ops._tf32_status_word(x.device)
    assert int(word[0]) == 0
    word[0] = 1
    with pytest.raises(RuntimeError, match="JG_ETIMEOUT"):
        ops.linear_tf32(x, w)
    assert int(word[0]) == 0
    ops.linear_tf32(x, w, check_status=True)                         # and the path works again


def test_bounded_wait_runs_out_and_the_kernel_returns(cuda):
    """Failure path of the transform without any fault: the self-test entry runs the same kernel with one
    ring fill left out per CTA and a short wait limit.  The consumer's wait runs out, the CTAs free their
    TMEM and return, the status call reports JG_ETIMEOUT; the very next transform on the device (which needs
    its TMEM) runs and is correct."""
    import ctypes
    from jittorgeometric_b200 import ops
    from jittorgeometric_b200._lib import lib, ptr, stream_for
    n, k, m = 40000, 256, 64                       # 313 row tiles: every CTA of the persistent grid has work
    x = torch.randn((n, k), device="cuda")
    w = torch.randn((k, m), device="cuda")
    wt = w.t().contiguous()
    out = torch.zeros((n, m), device="cuda")
    ws = torch.zeros(lib().jg_gemm_tf32_workspace_bytes(), dtype=torch.uint8, device="cuda")
    rc = lib().jg_gemm_tf32_timeout_selftest(ptr(out), ptr(x), ptr(wt), n, k, m, 1, 1 << 12, ptr(ws), ws.numel(), stream_for(x))
    assert rc == 0
    status = lib().jg_gemm_tf32_status(ptr(ws), stream_for(x))
    assert status == -5                            # JG_ETIMEOUT
    torch.cuda.synchronize()                       # the context is intact
    rc = lib().jg_gemm_tf32(ptr(out), ptr(x), ptr(wt), None, n, k, m, 0, ptr(ws), ws.numel(), stream_for(x))
    assert rc == 0 and lib().jg_gemm_tf32_status(ptr(ws), stream_for(x)) == 0
    want = x.double() @ w.double()
    scale = x.abs().double() @ w.abs().double()
    assert ((out.double() - want).abs() / scale).max().item() <= 2e-3
    assert torch.equal(out, ops.linear_tf32(x, w))


@pytest.mark.parametrize("M,N,K,ta,tb", [(300, 70, 45, False, False), (64, 64, 16, False, False), (2708, 256, 1433, False, False),
                                        (1433, 256, 2708, True, False), (5000, 1433, 256, False, True), (128, 64, 300000, True, False),
                                        (7, 5, 100000, True, False), (1, 1, 1, False, False)])
def test_fp32_product_on_the_cuda_cores(cuda, M, N, K, ta, tb):
    """``matmul_f32`` (x @ W, g @ W^T, x^T @ g by strides; long reductions sliced) against float64 at the
    fp32 bar, and run-to-run identical."""
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    a = torch.randn((K, M) if ta else (M, K), device="cuda", generator=g)
    b = torch.randn((N, K) if tb else (K, N), device="cuda", generator=g)
    bias = torch.randn(N, device="cuda", generator=g)
    got = cuda.ops.matmul_f32(a, b, trans_a=ta, trans_b=tb, bias=bias, relu=True)
    A, B = (a.t() if ta else a).double(), (b.t() if tb else b).double()
    want = torch.relu(A @ B + bias.double())
    scale = A.abs() @ B.abs() + bias.abs().double()
    assert ((got.double() - want).abs() / scale).max().item() <= 1e-5
    assert torch.equal(got, cuda.ops.matmul_f32(a, b, trans_a=ta, trans_b=tb, bias=bias, relu=True))


def test_no_vendor_gemm_in_the_layers(cuda):
    """GCNConv in both precisions trains without any library matmul: forward and all gradients agree with
    float64 autograd at the bar of the precision chosen."""
    from jittorgeometric_b200 import nn
    torch.manual_seed(0)
    n = 2000
    ei = torch.randint(0, n, (2, 30000), device="cuda", dtype=torch.int32)
    csc, csr = cuda.gcn_norm_csc_csr(ei, None, n)
    x0 = torch.randn(n, 96, device="cuda")
    A = torch.zeros((n, n), dtype=torch.float64, device="cuda")
    seg = torch.repeat_interleave(torch.arange(n, device="cuda"), (csc.column_offset[1:] - csc.column_offset[:-1]).long())
    A.index_put_((seg, csc.row_indices.long()), csc.edge_weight.double(), accumulate=True)
    for tf32, bar in ((False, 1e-5), (True, 2e-3)):
        layer = nn.GCNConv(96, 40, tf32=tf32, relu=True).cuda()
        x = x0.clone().requires_grad_(True)
        y = layer(x, csc, csr)
        y.square().sum().backward()
        xd = x0.double().requires_grad_(True)
        wd = layer.weight.detach().double().requires_grad_(True)
        bd = layer.bias.detach().double().requires_grad_(True)
        yd = torch.relu(A @ (xd @ wd) + bd)
        yd.square().sum().backward()
        for have, want in ((y, yd), (x.grad, xd.grad), (layer.weight.grad, wd.grad), (layer.bias.grad, bd.grad)):
            assert (have.double() - want).abs().max().item() <= 20 * bar * want.abs().max().item()


@pytest.mark.parametrize("n,k,m", [(64, 128, 128), (5000, 128, 64), (300000, 128, 128), (4097, 256, 64), (1000, 64, 16),
                                   (20000, 132, 36), (777, 4, 4), (50000, 512, 256), (63, 32, 32)])
def test_weight_gradient_on_the_tensor_cores(cuda, n, k, m):
    """``x^T g`` with MN-major tcgen05 operands against float64 at the TF32 bar, identical run to run."""
    assert cuda.ops.lib().jg_gemm_tn_tf32_supported(n, k, m)
    gen = torch.Generator(device="cuda").manual_seed(n + k + m)
    x = torch.randn((n, k), device="cuda", generator=gen)
    g = torch.randn((n, m), device="cuda", generator=gen)
    got = cuda.ops.weight_grad_tf32(x, g)
    cuda.ops.check_transform_status(x.device, synchronize=True)
    want = x.double().t() @ g.double()
    scale = x.abs().double().t() @ g.abs().double()
    assert got.shape == (k, m) and torch.isfinite(got).all()
    assert ((got.double() - want).abs() / scale).max().item() <= 2e-3
    assert torch.equal(got, cuda.ops.weight_grad_tf32(x, g))
