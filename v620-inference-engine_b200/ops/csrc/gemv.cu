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

template <int MT>
__global__ void __launch_bounds__(256, 1) sgemv_kernel(SGemvArgs a) {
    extern __shared__ __align__(128) unsigned char sg_smem[];
    sgemv_body<MT>(a, sg_smem);
}

template <int MT>
static cudaError_t launch_sgemv(SGemvArgs &a, cudaStream_t s) {
    int grid;
    const size_t smem = sgemv_plan(a, MT, grid);
    static size_t configured = 0;
    if (smem > configured) {
        cudaFuncSetAttribute(sgemv_kernel<MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        configured = 200 * 1024;
    }
    return launch_pdl(sgemv_kernel<MT>, dim3(grid), dim3(256), smem, s, a);
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
    if (nsplit <= 1 && (size_t)K * 2 <= 16384) {
        // the streaming kernel: bulk-async weight pipeline, one block per SM
        SGemvArgs g;
        g.W = (const bf16 *)W; g.x = (const bf16 *)x; g.y = y; g.y_bf16 = (bf16 *)y_bf16;
        g.N = N; g.K = K; g.M = M; g.ldw = ldw; g.ldx = ldx; g.ldy = ldy; g.accumulate = accumulate; g.err = g_err_ptr;
        cudaError_t e;
        if (M == 1) e = launch_sgemv<1>(g, s);
        else if (M == 2) e = launch_sgemv<2>(g, s);
        else if (M <= 4) e = launch_sgemv<4>(g, s);
        else e = launch_sgemv<8>(g, s);
        return e == cudaSuccess ? 0 : -2;
    }
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
