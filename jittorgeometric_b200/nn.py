"""Layer shims with the reference's constructor and call signatures, built on the operators of
:mod:`jittorgeometric_b200.ops`: ``gcn_norm``, ``GCNConv``, ``SGConv``, ``APPNP``, ``GATConv``
(jittor_geometric/nn/conv/{gcn_conv,sg_conv,appnp_conv,gat_conv}.py)."""
import math

import torch

from . import ops
from .data import CSC, CSR  # noqa: F401  (re-exported: layers take these containers)


def glorot_(t):
    """In-place U(-s, s), s = sqrt(6 / (fan_in + fan_out)) (nn/inits.py:19-22)."""
    s = math.sqrt(6.0 / (t.shape[-2] + t.shape[-1]))
    with torch.no_grad():
        t.uniform_(-s, s)
    return t


def gcn_norm(edge_index, edge_weight=None, num_nodes=None, improved=False, add_self_loops=True, dtype=None):
    """Self-loops + symmetric normalisation as a COO list (nn/conv/gcn_conv.py:18-37).  Returned
    in the reference's order (kept entries, then one loop per node); ``ops.gcn_norm_csc_csr`` gives
    the CSC/CSR directly without materialising this list."""
    if num_nodes is None:
        num_nodes = int(edge_index.max()) + 1 if edge_index.numel() else 0
    return ops.gcn_norm_coo(edge_index, edge_weight, num_nodes, improved=improved, add_self_loops=add_self_loops)


def _transform(x, weight, tf32, relu=False):
    """``x @ weight`` (optionally ReLU): the tcgen05 TF32 kernel (2e-3 tolerance; in training its input
    gradient runs in TF32 as well), or with ``tf32=False`` the library's fp32 CUDA-core kernel.  Neither
    path calls a vendor GEMM."""
    needs_grad = torch.is_grad_enabled() and (x.requires_grad or weight.requires_grad)
    if tf32 and ops.linear_tf32_supported(x.shape[0], x.shape[1], weight.shape[1]):
        if needs_grad:
            return ops.linear_tf32_autograd(x, weight, relu=relu)
        return ops.linear_tf32(x, weight, relu=relu)
    if needs_grad:
        return ops.linear_f32_autograd(x, weight, relu=relu)
    return ops.matmul_f32(x, weight, relu=relu)


class GCNConv(torch.nn.Module):
    """``out = A_hat (x W) + b`` (nn/conv/gcn_conv.py:70-112).  ``spmm`` is accepted for signature
    compatibility; there is one backend.  The bias (and, with ``relu=True``, the activation the
    reference's models apply right after the layer) is added inside the aggregation kernel.  The
    transform runs on the tcgen05 kernel with TF32 products (results within 2e-3 of fp32);
    ``tf32=False`` keeps it in fp32 for comparisons at 1e-5."""

    def __init__(self, in_channels, out_channels, bias=True, spmm=True, tf32=True, relu=False, **kwargs):
        super().__init__()
        self.in_channels, self.out_channels, self.spmm, self.tf32 = in_channels, out_channels, spmm, tf32
        self.relu = relu
        self.weight = torch.nn.Parameter(torch.empty(in_channels, out_channels))
        self.bias = torch.nn.Parameter(torch.zeros(out_channels)) if bias else None
        self.reset_parameters()

    def reset_parameters(self):
        glorot_(self.weight)
        if self.bias is not None:
            with torch.no_grad():
                self.bias.zero_()

    def forward(self, x, csc, csr):
        x = _transform(x, self.weight, self.tf32)
        return ops.aggregate_bias_act(x, csc, csr, self.bias, self.relu)

    def __repr__(self):
        return f"{self.__class__.__name__}({self.in_channels}, {self.out_channels})"


class Linear(torch.nn.Module):
    """``x W^T + b`` with ``weight`` stored ``[out, in]`` like the reference's ``Linear`` (nn/dense/linear.py),
    on the library's own kernels (TF32 tensor-core transform, or fp32 with ``tf32=False``)."""

    def __init__(self, in_channels, out_channels, bias=True, tf32=True):
        super().__init__()
        self.tf32 = tf32
        self.weight = torch.nn.Parameter(torch.empty(out_channels, in_channels))
        self.bias = torch.nn.Parameter(torch.zeros(out_channels)) if bias else None
        glorot_(self.weight)

    def forward(self, x):
        return ops.linear_nt(x, self.weight, self.bias, tf32=self.tf32)


class SGConv(torch.nn.Module):
    """``lin(A_hat^K x)`` (nn/conv/sg_conv.py:43-70)."""

    def __init__(self, in_channels, out_channels, K=1, bias=True, spmm=True, tf32=True, **kwargs):
        super().__init__()
        self.K = K
        self.lin = Linear(in_channels, out_channels, bias=bias, tf32=tf32)

    def forward(self, x, csc, csr):
        for _ in range(self.K):
            x = ops.aggregateWithWeight(x, csc, csr)
        return self.lin(x)


class APPNP(torch.nn.Module):
    """``x <- (1 - alpha) A_hat x + alpha h`` repeated K times (nn/conv/appnp_conv.py:27-52)."""

    def __init__(self, K, alpha, spmm=True, **kwargs):
        super().__init__()
        self.K, self.alpha = K, alpha

    def forward(self, x, csc, csr):
        ah = self.alpha * x                      # alpha * h, formed once
        for _ in range(self.K):
            x = torch.add(ah, ops.aggregateWithWeight(x, csc, csr), alpha=1 - self.alpha)
        return x


class GATConv(torch.nn.Module):
    """Attention layer (nn/conv/gat_conv.py:20-88) with the reference's constructor,
    ``GATConv(in_channels, out_channels, e_num, improved=False, cached=False, add_self_loops=True,
    normalize=True, bias=True)``: ``e_num`` (the edge count the reference asks for) and the four flags
    are accepted and, as in the reference's ``execute``, unused.  ``h = relu(x W)``, edge logits
    ``leaky_relu([h_src, h_dst] a, 0.2)``, softmax over each destination's in-edges, weighted sum.
    Keyword-only extensions: ``heads`` > 1 splits the channels into independent heads (the reference
    layer is single-head); ``tf32=False`` runs the transform in fp32; ``fused=False`` keeps the
    reference's op-by-op pipeline on the per-edge operators, which also serves the shapes the fused
    kernels (forward and backward) do not take."""

    def __init__(self, in_channels, out_channels, e_num, improved=False, cached=False, add_self_loops=True,
                 normalize=True, bias=True, *, heads=1, tf32=True, fused=True, **kwargs):
        super().__init__()
        if out_channels % heads:
            raise ValueError(f"out_channels ({out_channels}) must be a multiple of heads ({heads})")
        self.in_channels, self.out_channels, self.heads, self.tf32 = in_channels, out_channels, heads, tf32
        self.e_num, self.improved, self.cached = e_num, improved, cached
        self.add_self_loops, self.normalize = add_self_loops, normalize
        self.fused = fused
        self.weight = torch.nn.Parameter(torch.empty(in_channels, out_channels))
        self.edge_weight = torch.nn.Parameter(torch.empty(2 * out_channels, 1))
        self.reset_parameters()

    def reset_parameters(self):
        glorot_(self.weight)
        glorot_(self.edge_weight)

    def attention_vectors(self):
        c = self.out_channels
        return self.edge_weight[:c, 0].reshape(self.heads, -1), self.edge_weight[c:, 0].reshape(self.heads, -1)

    def forward(self, x, csc):
        h = _transform(x, self.weight, self.tf32, relu=True)
        dim = self.out_channels // self.heads
        if self.fused and ops.gat_aggregate_supported(self.heads, dim):
            a_src, a_dst = self.attention_vectors()
            return ops.gat_aggregate(h, a_src, a_dst, csc, self.heads)      # fused forward and backward
        return self.propagate_unfused(h, csc)

    def propagate_unfused(self, h, csc):
        e_s = ops.ScatterToEdge(h, csc, "src")
        e_d = ops.ScatterToEdge(h, csc, "dst")
        a_src, a_dst = self.attention_vectors()
        E, H = e_s.shape[0], self.heads
        m = (e_s.reshape(E, H, -1) * a_src).sum(-1) + (e_d.reshape(E, H, -1) * a_dst).sum(-1)
        m = torch.nn.functional.leaky_relu(m, 0.2)
        alpha = ops.EdgeSoftmax(m, csc)
        msg = (e_s.reshape(E, H, -1) * alpha.unsqueeze(-1)).reshape(E, -1)
        return ops.ScatterToVertex(msg, csc, "src")

    def __repr__(self):
        return f"{self.__class__.__name__}({self.in_channels}, {self.out_channels})"
