// Decode-path matrix-vector kernel: y[m][n] = sum_k W[n][k] x[m][k] for M <= 32 rows against one
// read of the bf16 weights.  Memory-bound by design:
//   * a persistent grid (a multiple of the SM count) strides over (row group, column split) items,
//     so every SM streams the same share of the matrix and there is no partial last wave;
//   * 16-byte streaming loads that bypass L1, four in flight per lane;
//   * launched with programmatic dependent launch: before it waits for its predecessor it asks
//     the L2 to prefetch the weight rows of its first items (weights are never written), so HBM
//     keeps streaming across the kernel boundary;
//   * fp32 accumulation in a fixed order, so a row's result does not depend on how many other rows
//     share the step.
// (Role of the reference's src/kernels/gemv.hip:8-42.)
#include "gemv.cuh"
#include "sgemv.cuh"

namespace qw {

template <int MT>
__global__ void __launch_bounds__(256) gemv_bf16_kernel(GemvArgs a) {
    __shared__ float part[8][MT];
    gemv_body<MT>(a, part);
}

template <int NT, bool FUSED>
__global__ void __launch_bounds__(SG_THREADS, 1) sgemv_kernel(SGemvArgs a) {
    extern __shared__ __align__(128) unsigned char sg_smem[];
    sgemv_body<NT, FUSED>(a, sg_smem);
}

template <int NT>
static cudaError_t launch_sgemv_nt(SGemvArgs &a, size_t smem, int grid, cudaStream_t s) {
    static bool configured = false;
    if (!configured) {
        cudaFuncSetAttribute(sgemv_kernel<NT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SG_SMEM_MAX);
        cudaFuncSetAttribute(sgemv_kernel<NT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SG_SMEM_MAX);
        configured = true;
    }
    if (a.fi.active || a.fo.mode) return launch_pdl(sgemv_kernel<NT, true>, dim3(grid), dim3(SG_THREADS), smem, s, a);
    return launch_pdl(sgemv_kernel<NT, false>, dim3(grid), dim3(SG_THREADS), smem, s, a);
}

// Up to 8 activation rows per pass, or 16 when they fit in shared memory next to the weight stages.
static cudaError_t launch_sgemv(SGemvArgs &a, cudaStream_t s) {
    int grid;
    if (a.M > 8) {
        const size_t smem2 = sgemv_plan(a, 2, grid);
        if (smem2) return launch_sgemv_nt<2>(a, smem2, grid, s);
    }
    const size_t smem1 = sgemv_plan(a, 1, grid);
    if (!smem1) return cudaErrorInvalidValue;
    return launch_sgemv_nt<1>(a, smem1, grid, s);
}

}  // namespace qw

using namespace qw;

// Launches the bf16 GEMV.  K must be a multiple of 8 and all row starts 16-byte aligned.
// nsplit > 1 runs `nsplit` independent column splits (offsets in elements).
QW_API int qwk_gemv_bf16(const void *W, const void *x, float *y, void *y_bf16, int N, int K, int M, int ldw, int ldx,
                         int ldy, int accumulate, int nsplit, long long w_split, long long x_split, long long y_split,
                         cudaStream_t s) {
    if (N <= 0 || M <= 0) return 0;
    if ((K & 7) || (ldw & 7) || (ldx & 7)) return -1;
    if (nsplit <= 1 && (K & 15) == 0 && (size_t)K * 2 <= 16384) {
        // the streaming kernel: bulk-async weight pipeline, one block per SM
        SGemvArgs g;
        g.W = (const bf16 *)W; g.x = (const bf16 *)x; g.y = y; g.y_bf16 = (bf16 *)y_bf16;
        g.N = N; g.K = K; g.M = M; g.ldw = ldw; g.ldx = ldx; g.ldy = ldy; g.accumulate = accumulate; g.nsplit = 1; g.w_split = 0; g.err = g_err_ptr; g.pf = take_pf();
        g.fi = take_fi(); g.fo = take_fo();
        const cudaError_t e = launch_sgemv(g, s);
        return e == cudaSuccess ? 0 : -2;
    }
    if (g_fi.active || g_fo.mode) return -1;          // only the streaming kernel carries fused collectives
    GemvArgs a;
    a.W = (const bf16 *)W; a.x = (const bf16 *)x; a.y = y; a.y_bf16 = (bf16 *)y_bf16;
    a.N = N; a.K = K; a.M = M; a.ldw = ldw; a.ldx = ldx; a.ldy = ldy;
    a.accumulate = accumulate;
    a.nsplit = nsplit < 1 ? 1 : nsplit;
    a.w_split = w_split; a.x_split = x_split; a.y_split = y_split;
    const int grid = gemv_plan(a);
    cudaError_t e;
    if (M == 1) e = launch_pdl(gemv_bf16_kernel<1>, dim3(grid), dim3(256), 0, s, a);
    else if (M == 2) e = launch_pdl(gemv_bf16_kernel<2>, dim3(grid), dim3(256), 0, s, a);
    else if (M <= 4) e = launch_pdl(gemv_bf16_kernel<4>, dim3(grid), dim3(256), 0, s, a);
    else e = launch_pdl(gemv_bf16_kernel<8>, dim3(grid), dim3(256), 0, s, a);
    return e == cudaSuccess ? 0 : -2;
}
