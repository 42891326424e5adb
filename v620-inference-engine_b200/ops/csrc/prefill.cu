// Token-major (prefill) glue kernels around the tcgen05 GEMMs: hyper-connection norm / mid / mix,
// q4 -> bf16 expert dequantisation, swiglu on expert-sorted rows and the weighted combine back to
// token order (roles of the reference's src/kernels/hc.hip:8-94, src/kernels/moe_route.hip:168-224
// and the dequant stage of src/kernels/moe_experts.hip:46-150).
#include "common.cuh"

namespace qw {

// grid (T, hc), 256 threads.  X[t][s][:] (+= pend[t][:] * 2*sigmoid(inj[t][s]/hc)); xn = bf16(X * w1 * rsqrt(mean X^2 + eps)).
__global__ void __launch_bounds__(256) hc_prenorm_T_kernel(float *X, const float *pend, int ld_pend, const float *inj,
                                                           const float *w1, int SH, int hc, float eps, bf16 *xn) {
    __shared__ float scratch[32];
    const int t = blockIdx.x, s = blockIdx.y;
    float *x = X + ((long long)t * hc + s) * SH;
    float coef = 0.f;
    if (pend) coef = 2.f * sigmoidf_(inj[(long long)t * hc + s] / float(hc));
    float v[16];            // SH <= 4096
    float ss = 0.f;
    int n = 0;
    for (int c = threadIdx.x; c < SH; c += 256, ++n) {
        float a = x[c];
        if (pend) {
            a = fmaf(pend[(long long)t * ld_pend + c], coef, a);
            x[c] = a;
        }
        v[n] = a;
        ss = fmaf(a, a, ss);
    }
    ss = block_sum<256>(ss, scratch);
    const float r = rsqrtf(ss / float(SH) + eps);
    n = 0;
    for (int c = threadIdx.x; c < SH; c += 256, ++n)
        xn[((long long)t * hc + s) * SH + c] = __float2bfloat16(v[n] * w1[s * SH + c] * r);
}

// d [T][ld_d] fp32 (R + n_inj columns) -> u bf16 [T][R] = silu(d/hc), inj fp32 [T][n_inj].
__global__ void hc_mid_T_kernel(const float *d, int ld_d, int R, int n_inj, int hc, bf16 *u, float *inj, long long total) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int w = R + n_inj;
    const long long t = i / w;
    const int j = (int)(i - t * w);
    const float v = d[t * ld_d + j];
    if (j < R) u[t * R + j] = __float2bfloat16(siluf_(v / float(hc)));
    else inj[t * n_inj + (j - R)] = v;
}

// g [T][SH*hc] fp32 with columns ordered (c, s); bin[t][c] = mean_s sigmoid(g[t][c][s]) * xn[t][s][c].  hc == 4.
__global__ void hc_mix_T_kernel(const float *g, const bf16 *xn, int SH, bf16 *bin, int ld_bin, long long total) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long t = i / SH;
    const int c = (int)(i - t * SH);
    const float4 gg = *reinterpret_cast<const float4 *>(g + (t * SH + c) * 4);
    const bf16 *x = xn + t * 4 * SH + c;
    const float v = sigmoidf_(gg.x) * __bfloat162float(x[0]) + sigmoidf_(gg.y) * __bfloat162float(x[SH]) +
                    sigmoidf_(gg.z) * __bfloat162float(x[2 * SH]) + sigmoidf_(gg.w) * __bfloat162float(x[3 * SH]);
    bin[t * ld_bin + c] = __float2bfloat16(v * 0.25f);
}

// q4 (engine order) rows -> bf16 rows.  One thread per word (8 values).
__global__ void q4_dequant_kernel(const uint32_t *w, const bf16 *scale, int K, bf16 *out, long long words) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= words) return;
    const int wpr = K >> 3;
    const long long row = i / wpr;
    const int c = (int)(i - row * wpr);
    const float sc = __bfloat162float(scale[row * (K >> 7) + (c >> 4)]);
    const uint32_t word = w[i];
    uint4 o;
    float e0, e1;
    q4_pair(word, 0, e0, e1); o.x = pack_bf16(e0 * sc, e1 * sc);
    q4_pair(word, 1, e0, e1); o.y = pack_bf16(e0 * sc, e1 * sc);
    q4_pair(word, 2, e0, e1); o.z = pack_bf16(e0 * sc, e1 * sc);
    q4_pair(word, 3, e0, e1); o.w = pack_bf16(e0 * sc, e1 * sc);
    *reinterpret_cast<uint4 *>(out + i * 8) = o;
}

// h13 [P][2F] bf16 (gate | up) -> h [P][F] = silu(gate) * up.
__global__ void swiglu_T_kernel(const bf16 *h13, int F, bf16 *h, long long total) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long p = i / F;
    const int f = (int)(i - p * F);
    const float g = __bfloat162float(h13[p * 2 * F + f]), u = __bfloat162float(h13[p * 2 * F + F + f]);
    h[i] = __float2bfloat16(siluf_(g) * u);
}

// out[t][c] = sum_j w[t][j] * y[inv[t*top_k + j]][c] + shared[t][c].  inv maps a pair to its expert-sorted row (-1: none).
__global__ void moe_combine_T_kernel(const float *y, int ld_y, const int *inv, const float *pair_w, int top_k, const float *shared,
                                     int H, float *out, long long total) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long t = i / H;
    const int c = (int)(i - t * H);
    float acc = 0.f;
    for (int j = 0; j < top_k; ++j) {
        const int r = inv[t * top_k + j];
        if (r >= 0) acc = fmaf(pair_w[t * top_k + j], y[(long long)r * ld_y + c], acc);
    }
    if (shared) acc += shared[i];
    out[i] = acc;
}

}  // namespace qw

using namespace qw;

static inline unsigned blocks_for(long long n, int per) { return (unsigned)((n + per - 1) / per); }

QW_API int qwk_hc_prenorm_T(float *X, const float *pend, int ld_pend, const float *inj, const float *w1, int SH, int hc,
                            float eps, void *xn, int T, cudaStream_t s) {
    if (SH > 4096) return -1;
    hc_prenorm_T_kernel<<<dim3(T, hc), 256, 0, s>>>(X, pend, ld_pend, inj, w1, SH, hc, eps, (bf16 *)xn);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
QW_API int qwk_hc_mid_T(const float *d, int ld_d, int R, int n_inj, int hc, void *u, float *inj, int T, cudaStream_t s) {
    const long long total = (long long)T * (R + n_inj);
    hc_mid_T_kernel<<<blocks_for(total, 256), 256, 0, s>>>(d, ld_d, R, n_inj, hc, (bf16 *)u, inj, total);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
QW_API int qwk_hc_mix_T(const float *g, const void *xn, int SH, void *bin, int ld_bin, int T, cudaStream_t s) {
    const long long total = (long long)T * SH;
    hc_mix_T_kernel<<<blocks_for(total, 256), 256, 0, s>>>(g, (const bf16 *)xn, SH, (bf16 *)bin, ld_bin, total);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
QW_API int qwk_q4_dequant(const void *w, const void *scale, long long rows, int K, void *out, cudaStream_t s) {
    if (K & 127) return -1;
    const long long words = rows * (K >> 3);
    q4_dequant_kernel<<<blocks_for(words, 256), 256, 0, s>>>((const uint32_t *)w, (const bf16 *)scale, K, (bf16 *)out, words);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
QW_API int qwk_swiglu_T(const void *h13, int F, void *h, long long P, cudaStream_t s) {
    const long long total = P * F;
    swiglu_T_kernel<<<blocks_for(total, 256), 256, 0, s>>>((const bf16 *)h13, F, (bf16 *)h, total);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
QW_API int qwk_moe_combine_T(const float *y, int ld_y, const int *inv, const float *pair_w, int top_k, const float *shared,
                             int H, float *out, int T, cudaStream_t s) {
    const long long total = (long long)T * H;
    moe_combine_T_kernel<<<blocks_for(total, 256), 256, 0, s>>>(y, ld_y, inv, pair_w, top_k, shared, H, out, total);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
