// Dense products in full fp32 on the CUDA cores (sm_100a): C[M,N] = op(A) * op(B) (+ bias, ReLU).
//
// The reference's layers hand `x @ self.weight` and its two gradient products to the runtime, which
// calls cuBLAS (nn/conv/gcn_conv.py:95, nn/conv/gat_conv.py:86).  The tensor-core kernel
// (gemm.cu, TF32 products) is the transform of the hot path; this kernel serves what it does not:
// the fp32 opt-out of the layers (comparisons at 1e-5 need fp32 products), the weight gradient
// x^T * g (a reduction over the rows, the one operand layout the row-tiled kernel does not take) and
// shapes the tensor-core kernel refuses.  With it no product of the path goes to a library.
//
// Operands are addressed by two strides each, A(i,l) = a[i*sa0 + l*sa1], B(l,j) = b[l*sb0 + j*sb1],
// so x @ W, g @ W^T and x^T @ g are the same kernel.  64x64 output tile per CTA, 16-deep slices
// through shared memory, 4x4 register block per thread, fp32 FMA.  A long reduction (x^T g over
// millions of rows) is cut into slices across CTAs whose partial tiles are added in a fixed order by a
// second kernel: no atomics, identical results run to run.
#include "common.cuh"

namespace jg {

constexpr int kBM = 64, kBN = 64, kBK = 16;

struct SgemmArgs {
    float* c;             // output [M, ldc] (single slice) or partial tiles [slices][M][N]
    const float* a;
    const float* b;
    const float* bias;    // [N] or null (single slice only; else applied by the reduction)
    int64_t M, N, K;
    int64_t sa0, sa1, sb0, sb1, ldc;
    int64_t k_slice;      // reduction length per slice (a multiple of kBK)
    int relu;
    int slices;
};

__global__ void __launch_bounds__(256) sgemm_kernel(SgemmArgs g) {
    __shared__ float As[kBK][kBM + 4];
    __shared__ float Bs[kBK][kBN + 4];
    const int tid = threadIdx.x, tx = tid % 16, ty = tid / 16;
    const int64_t i0 = (int64_t)blockIdx.x * kBM, j0 = (int64_t)blockIdx.y * kBN;
    const int64_t l_begin = (int64_t)blockIdx.z * g.k_slice;
    const int64_t l_end = l_begin + g.k_slice < g.K ? l_begin + g.k_slice : g.K;
    float acc[4][4];
#pragma unroll
    for (int r = 0; r < 4; r++)
#pragma unroll
        for (int c = 0; c < 4; c++) acc[r][c] = 0.f;
    const bool a_rows_contig = g.sa0 == 1;     // consecutive i adjacent in memory (A given transposed)
    const bool b_cols_contig = g.sb1 == 1;     // consecutive j adjacent in memory
    for (int64_t l0 = l_begin; l0 < l_end; l0 += kBK) {
#pragma unroll
        for (int e = tid; e < kBM * kBK; e += 256) {
            const int ii = a_rows_contig ? e % kBM : e / kBK;
            const int ll = a_rows_contig ? e / kBM : e % kBK;
            const int64_t i = i0 + ii, l = l0 + ll;
            As[ll][ii] = (i < g.M && l < l_end) ? __ldg(g.a + i * g.sa0 + l * g.sa1) : 0.f;
        }
#pragma unroll
        for (int e = tid; e < kBN * kBK; e += 256) {
            const int jj = b_cols_contig ? e % kBN : e / kBK;
            const int ll = b_cols_contig ? e / kBN : e % kBK;
            const int64_t j = j0 + jj, l = l0 + ll;
            Bs[ll][jj] = (j < g.N && l < l_end) ? __ldg(g.b + l * g.sb0 + j * g.sb1) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int l = 0; l < kBK; l++) {
            const float4 av = *reinterpret_cast<const float4*>(&As[l][ty * 4]);
            const float4 bv = *reinterpret_cast<const float4*>(&Bs[l][tx * 4]);
            const float a4[4] = {av.x, av.y, av.z, av.w}, b4[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
            for (int r = 0; r < 4; r++)
#pragma unroll
                for (int c = 0; c < 4; c++) acc[r][c] = fmaf(a4[r], b4[c], acc[r][c]);
        }
        __syncthreads();
    }
    const bool single = g.slices == 1;
    float* out = single ? g.c : g.c + (size_t)blockIdx.z * (size_t)g.M * (size_t)g.N;
    const int64_t ld = single ? g.ldc : g.N;
#pragma unroll
    for (int r = 0; r < 4; r++) {
        const int64_t i = i0 + ty * 4 + r;
        if (i >= g.M) continue;
#pragma unroll
        for (int c = 0; c < 4; c++) {
            const int64_t j = j0 + tx * 4 + c;
            if (j >= g.N) continue;
            float v = acc[r][c];
            if (single) {
                if (g.bias) v += __ldg(g.bias + j);
                if (g.relu) v = fmaxf(v, 0.f);
            }
            out[i * ld + j] = v;
        }
    }
}

// C = sum of the slices' partial tiles in slice order (+ bias, ReLU).
__global__ void __launch_bounds__(256) sgemm_reduce_kernel(float* __restrict__ c, const float* __restrict__ partial, int64_t M,
                                                           int64_t N, int64_t ldc, int slices, const float* __restrict__ bias, int relu) {
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < M * N; t += (int64_t)gridDim.x * blockDim.x) {
        float v = partial[t];
        for (int s = 1; s < slices; s++) v = __fadd_rn(v, partial[(size_t)s * (size_t)(M * N) + t]);
        const int64_t i = t / N, j = t - i * N;
        if (bias) v += __ldg(bias + j);
        if (relu) v = fmaxf(v, 0.f);
        c[i * ldc + j] = v;
    }
}

// Used by the tensor-core weight gradient as well: c[M, N] = sum of `slices` partial results, in order.
int reduce_slices(float* c, const float* partial, int64_t M, int64_t N, int slices, cudaStream_t st) {
    int64_t blocks = (M * N + 255) / 256;
    if (blocks > (int64_t)sm_count() * 8) blocks = (int64_t)sm_count() * 8;
    if (blocks < 1) blocks = 1;
    sgemm_reduce_kernel<<<(unsigned)blocks, 256, 0, st>>>(c, partial, M, N, N, slices, nullptr, 0);
    JG_LAUNCH_CHECK();
    return JG_OK;
}

static int sgemm_slices(int64_t M, int64_t N, int64_t K) {
    const int64_t tiles = ((M + kBM - 1) / kBM) * ((N + kBN - 1) / kBN);
    int64_t want = (2 * (int64_t)sm_count() + tiles - 1) / tiles;      // enough CTAs to fill the device twice
    const int64_t most = (K + 4 * kBK - 1) / (4 * kBK);                  // at least four slices' worth of work each
    if (want > most) want = most;
    if (want > 1024) want = 1024;
    return want < 1 ? 1 : (int)want;
}

}  // namespace jg

using namespace jg;

extern "C" {

size_t jg_gemm_f32_workspace_bytes(int64_t M, int64_t N, int64_t K) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    const int s = sgemm_slices(M, N, K);
    return s > 1 ? align_up((size_t)s * (size_t)M * (size_t)N * sizeof(float), 256) : 0;
}

int jg_gemm_f32(float* c, const float* a, const float* b, const float* bias, int64_t M, int64_t N, int64_t K, int64_t sa0,
                int64_t sa1, int64_t sb0, int64_t sb1, int64_t ldc, int relu, void* workspace, size_t workspace_bytes,
                jg_stream_t stream) {
    JG_CHECK_ARG(M >= 0 && N >= 0 && K >= 0 && ldc >= N, JG_EINVAL, "gemm_f32: bad size");
    if (M == 0 || N == 0) return JG_OK;
    JG_CHECK_ARG(c && (K == 0 || (a && b)), JG_EINVAL, "gemm_f32: null pointer");
    JG_CHECK_ARG((N + kBN - 1) / kBN < 65536 && (M + kBM - 1) / kBM < 2147483647, JG_ESHAPE, "gemm_f32: output too large");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    SgemmArgs g = {};
    g.a = a; g.b = b; g.bias = bias; g.M = M; g.N = N; g.K = K;
    g.sa0 = sa0; g.sa1 = sa1; g.sb0 = sb0; g.sb1 = sb1; g.ldc = ldc; g.relu = relu;
    g.slices = K > 0 ? sgemm_slices(M, N, K) : 1;
    g.k_slice = ((K + g.slices - 1) / g.slices + kBK - 1) / kBK * kBK;
    if (g.k_slice < kBK) g.k_slice = kBK;
    g.slices = (int)((K + g.k_slice - 1) / g.k_slice);
    if (g.slices < 1) g.slices = 1;
    if (g.slices > 1) {
        const size_t need = (size_t)g.slices * (size_t)M * (size_t)N * sizeof(float);
        JG_CHECK_ARG(workspace && workspace_bytes >= need, JG_EWORKSPACE, "gemm_f32: workspace %zu < %zu", workspace_bytes, need);
        g.c = static_cast<float*>(workspace);
    } else {
        g.c = c;
    }
    dim3 grid((unsigned)((M + kBM - 1) / kBM), (unsigned)((N + kBN - 1) / kBN), (unsigned)g.slices);
    sgemm_kernel<<<grid, 256, 0, st>>>(g);
    JG_LAUNCH_CHECK();
    if (g.slices > 1) {
        int64_t blocks = (M * N + 255) / 256;
        if (blocks > (int64_t)sm_count() * 8) blocks = (int64_t)sm_count() * 8;
        sgemm_reduce_kernel<<<(unsigned)blocks, 256, 0, st>>>(c, static_cast<const float*>(workspace), M, N, ldc, g.slices, bias, relu);
        JG_LAUNCH_CHECK();
    }
    return JG_OK;
}

}  // extern "C"
