// Hyper-connection kernels for row batches (decode rows and prefill rows alike).
//
// The residual X has `hc` streams; a rank owns SH = H/ranks columns of each, X[m][s][c] fp32.
// A mixer is computed as
//   pre : X += pend * 2*sigmoid(inj/hc) (deferred combine of the previous block), y = bf16(X*(1+w)),
//         ssq[s] = sum_c X^2                                          (hc_pre)
//   down: part[s][j] = sum_c Wd[j][s,c] * y[s][c]                     (bf16 GEMV with column splits)
//   --- all-reduce of [ssq | part] over ranks ---
//   up  : r_s = rsqrt(ssq_s/H + eps); d_j = sum_s r_s part[s][j]; inj = d[rank..rank+hc);
//         u = silu(d/hc); g[s][c] = Wu[c][s] . u; block_in[c] = mean_s sigmoid(g) * y[s][c] * r_s   (hc_up_mix)
// which uses that the down projection is linear in the un-normalised y (the algebra of the
// reference's src/kernels/hc.hip:98-166 and src/engine/decode.hip:53-61).
#include "common.cuh"

namespace qw {

// X[m][s][:] = embedding row of tokens[m] (this rank's columns) for every stream.
__global__ void embed_rows_kernel(const int *tokens, const bf16 *table, int ld_table, int col0, int SH, int hc,
                                  int vocab, float *X) {
    const int m = blockIdx.x;
    int t = tokens[m];
    if (t < 0 || t >= vocab) t = 0;
    const bf16 *row = table + (long long)t * ld_table + col0;
    for (int c = threadIdx.x; c < SH; c += blockDim.x) {
        const float v = __bfloat162float(row[c]);
        for (int s = 0; s < hc; ++s) X[((long long)m * hc + s) * SH + c] = v;
    }
}

// grid (M, hc).  pend may be null (no deferred combine).  y and ssq may be null (combine only).
__global__ void __launch_bounds__(256) hc_pre_kernel(float *X, const float *pend, int ld_pend, const float *inj, int ld_inj,
                                                     const float *w1 /* (1+w) [hc][SH] */, int SH, int hc, bf16 *y,
                                                     float *ssq, int ld_ssq) {
    __shared__ float scratch[32];
    const int m = blockIdx.x, s = blockIdx.y;
    float *x = X + ((long long)m * hc + s) * SH;
    float coef = 0.f;
    if (pend) coef = 2.f * sigmoidf_(inj[(long long)m * ld_inj + s] / float(hc));
    float acc = 0.f;
    for (int c = threadIdx.x; c < SH; c += 256) {
        float v = x[c];
        if (pend) {
            v = fmaf(pend[(long long)m * ld_pend + c], coef, v);
            x[c] = v;
        }
        if (y) y[((long long)m * hc + s) * SH + c] = __float2bfloat16(v * w1[s * SH + c]);
        acc = fmaf(v, v, acc);
    }
    if (ssq) {
        acc = block_sum<256>(acc, scratch);
        if (threadIdx.x == 0) ssq[(long long)m * ld_ssq + s] = acc;
    }
}

constexpr int UP_ROWS = 4;     // rows per block of hc_up_mix

// grid (ceil(SH/8), ceil(M/UP_ROWS)), 256 threads.  hc must be 4 (one 8-lane group per stream).
__global__ void __launch_bounds__(256) hc_up_mix_kernel(const float *red, int ld_red, const bf16 *Wu /* [SH][hc][R] */,
                                                        const bf16 *y, int SH, int hc, int R, int hc_down, float inv_H,
                                                        float eps, int M, float *inj, int ld_inj, bf16 *bin, int ld_bin,
                                                        int bin_col0) {
    extern __shared__ float sm[];
    float *u = sm;                         // [UP_ROWS][R]
    float *rs = sm + UP_ROWS * R;          // [UP_ROWS][hc]
    const int m0 = blockIdx.y * UP_ROWS;
    const int nrow = min(UP_ROWS, M - m0);
    for (int i = threadIdx.x; i < nrow * hc; i += 256) {
        const int mm = i / hc, s = i % hc;
        rs[mm * hc + s] = rsqrtf(red[(long long)(m0 + mm) * ld_red + s] * inv_H + eps);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < nrow * hc_down; i += 256) {
        const int mm = i / hc_down, j = i % hc_down;
        const float *p = red + (long long)(m0 + mm) * ld_red + hc + j;
        float d = 0.f;
        for (int s = 0; s < hc; ++s) d = fmaf(rs[mm * hc + s], p[s * hc_down], d);
        if (j < R) u[mm * R + j] = siluf_(d / float(hc));
        else if (inj && blockIdx.x == 0) inj[(long long)(m0 + mm) * ld_inj + (j - R)] = d;
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int c = blockIdx.x * 8 + warp;
    if (c >= SH) return;
    const int s = lane >> 3, li = lane & 7;
    const uint4 *wp = reinterpret_cast<const uint4 *>(Wu + ((long long)c * hc + s) * R);
    const int nch = R >> 3;
    float acc[UP_ROWS];
#pragma unroll
    for (int mm = 0; mm < UP_ROWS; ++mm) acc[mm] = 0.f;
    for (int ch = li; ch < nch; ch += 8) {
        const uint4 w = ld_stream(wp + ch);
        const float wf[8] = {bf16_lo(w.x), bf16_hi(w.x), bf16_lo(w.y), bf16_hi(w.y),
                             bf16_lo(w.z), bf16_hi(w.z), bf16_lo(w.w), bf16_hi(w.w)};
#pragma unroll
        for (int mm = 0; mm < UP_ROWS; ++mm) {
            if (mm < nrow) {
                const float *uu = u + mm * R + ch * 8;
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[mm] = fmaf(wf[i], uu[i], acc[mm]);
            }
        }
    }
#pragma unroll
    for (int mm = 0; mm < UP_ROWS; ++mm) {
        float g = acc[mm];
        g += __shfl_xor_sync(0xffffffffu, g, 1);
        g += __shfl_xor_sync(0xffffffffu, g, 2);
        g += __shfl_xor_sync(0xffffffffu, g, 4);
        float v = 0.f;
        if (mm < nrow) {
            const float yv = __bfloat162float(y[((long long)(m0 + mm) * hc + s) * SH + c]);
            v = sigmoidf_(g) * yv * rs[mm * hc + s];
        }
        v += __shfl_xor_sync(0xffffffffu, v, 8);
        v += __shfl_xor_sync(0xffffffffu, v, 16);
        if (lane == 0 && mm < nrow) bin[(long long)(m0 + mm) * ld_bin + bin_col0 + c] = __float2bfloat16(v / float(hc));
    }
}

}  // namespace qw

using namespace qw;

QW_API int qwk_embed_rows(const int *tokens, const void *table, int ld_table, int col0, int SH, int hc, int vocab,
                          float *X, int M, cudaStream_t s) {
    embed_rows_kernel<<<M, 256, 0, s>>>(tokens, (const bf16 *)table, ld_table, col0, SH, hc, vocab, X);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

QW_API int qwk_hc_pre(float *X, const float *pend, int ld_pend, const float *inj, int ld_inj, const float *w1, int SH,
                      int hc, void *y, float *ssq, int ld_ssq, int M, cudaStream_t s) {
    dim3 grid(M, hc);
    hc_pre_kernel<<<grid, 256, 0, s>>>(X, pend, ld_pend, inj, ld_inj, w1, SH, hc, (bf16 *)y, ssq, ld_ssq);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

QW_API int qwk_hc_up_mix(const float *red, int ld_red, const void *Wu, const void *y, int SH, int hc, int R, int n_inj,
                         int H, float eps, int M, float *inj, int ld_inj, void *bin, int ld_bin, int bin_col0,
                         cudaStream_t s) {
    if (hc != 4 || (R & 7)) return -1;
    dim3 grid((SH + 7) / 8, (M + UP_ROWS - 1) / UP_ROWS);
    const size_t smem = sizeof(float) * (UP_ROWS * R + UP_ROWS * hc);
    hc_up_mix_kernel<<<grid, 256, smem, s>>>(red, ld_red, (const bf16 *)Wu, (const bf16 *)y, SH, hc, R, R + n_inj,
                                             1.f / float(H), eps, M, inj, ld_inj, (bf16 *)bin, ld_bin, bin_col0);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
