// Decode-path matrix-vector kernels: y[m][n] = sum_k W[n][k] x[m][k] for M <= 32 rows against
// one read of the weights.  bf16 weights (dense layers) and q4 weights (routed experts, per
// (row, expert) pair).  Memory-bound by design: 16-byte streaming loads, several in flight per
// lane, fp32 accumulation in a fixed order so a row's result does not depend on how many other
// rows share the step (the role of the reference's src/kernels/gemv.hip:8-42 and
// src/kernels/moe_experts.hip:189-246).
#include "common.cuh"

namespace qw {

// ------------------------------------------------------------------------------------------
// bf16 GEMV.  Block = 8 warps.  `wpr` warps cooperate on one output row (K split between them,
// partials summed in warp order), so a block covers 8/wpr rows.  blockIdx.y selects a column
// split (used by the hyper-connection down projection, which needs per-stream partial sums).
// ------------------------------------------------------------------------------------------
struct GemvArgs {
    const bf16 *W;      // [N][ldw]
    const bf16 *x;      // [M][ldx]
    float *y;           // [M][ldy]
    int N, K, M;
    int ldw, ldx, ldy;
    int wpr;            // warps per row: 1, 2, 4 or 8
    int accumulate;     // y += instead of y =
    // column splits (gridDim.y): element offsets added per split
    long long w_split, x_split, y_split;
    bf16 *y_bf16;       // optional second output in bf16 (same indexing as y), may be null
};

template <int MT>
__global__ void __launch_bounds__(256) gemv_bf16_kernel(GemvArgs a) {
    __shared__ float part[8][MT];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int wpr = a.wpr;
    const int rpb = 8 / wpr;
    const int row = blockIdx.x * rpb + warp / wpr;
    const int kw = warp % wpr;
    const bf16 *W = a.W + (long long)blockIdx.y * a.w_split;
    const bf16 *x = a.x + (long long)blockIdx.y * a.x_split;
    float *y = a.y + (long long)blockIdx.y * a.y_split;
    const int nchunk = a.K >> 3;
    const int stride = wpr * 32;
    for (int m0 = 0; m0 < a.M; m0 += MT) {
        float acc[MT];
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[m] = 0.f;
        if (row < a.N) {
            const uint4 *wp = reinterpret_cast<const uint4 *>(W + (long long)row * a.ldw);
            for (int c = kw * 32 + lane; c < nchunk; c += 4 * stride) {
                uint4 w[4];
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    if (c + u * stride < nchunk) w[u] = ld_stream(wp + c + u * stride);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    if (c + u * stride < nchunk) {
#pragma unroll
                        for (int m = 0; m < MT; ++m) {
                            if (m0 + m < a.M) {
                                const uint4 xv = __ldg(reinterpret_cast<const uint4 *>(x + (long long)(m0 + m) * a.ldx) + c + u * stride);
                                acc[m] = dot8(w[u], xv, acc[m]);
                            }
                        }
                    }
                }
            }
        }
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[m] = warp_sum(acc[m]);
        if (wpr > 1) {
            __syncthreads();
            if (lane == 0) {
#pragma unroll
                for (int m = 0; m < MT; ++m) part[warp][m] = acc[m];
            }
            __syncthreads();
            if (kw == 0) {
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    float s = 0.f;
                    for (int j = 0; j < wpr; ++j) s += part[warp + j][m];
                    acc[m] = s;
                }
            }
        }
        if (kw == 0 && lane == 0 && row < a.N) {
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                if (m0 + m < a.M) {
                    const long long o = (long long)(m0 + m) * a.ldy + row;
                    float v = acc[m];
                    if (a.accumulate) v += y[o];
                    y[o] = v;
                    if (a.y_bf16) (a.y_bf16 + (long long)blockIdx.y * a.y_split)[o] = __float2bfloat16(v);
                }
            }
        }
    }
}

static inline int pick_wpr(int N, int nsplit) {
    // aim for >= ~4 blocks per SM without shrinking a warp's K share below one pass
    long long rows = (long long)N * nsplit;
    if (rows >= 148 * 4 * 8) return 1;
    if (rows >= 148 * 4 * 4) return 2;
    if (rows >= 148 * 4 * 2) return 4;
    return 8;
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
    GemvArgs a;
    a.W = (const bf16 *)W; a.x = (const bf16 *)x; a.y = y; a.y_bf16 = (bf16 *)y_bf16;
    a.N = N; a.K = K; a.M = M; a.ldw = ldw; a.ldx = ldx; a.ldy = ldy;
    a.accumulate = accumulate;
    a.w_split = w_split; a.x_split = x_split; a.y_split = y_split;
    if (nsplit < 1) nsplit = 1;
    a.wpr = pick_wpr(N, nsplit);
    const int rpb = 8 / a.wpr;
    dim3 grid((N + rpb - 1) / rpb, nsplit);
    if (M == 1) gemv_bf16_kernel<1><<<grid, 256, 0, s>>>(a);
    else if (M == 2) gemv_bf16_kernel<2><<<grid, 256, 0, s>>>(a);
    else if (M <= 4) gemv_bf16_kernel<4><<<grid, 256, 0, s>>>(a);
    else gemv_bf16_kernel<8><<<grid, 256, 0, s>>>(a);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
