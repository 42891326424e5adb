// Token-major (prefill) glue kernels around the tcgen05 GEMMs: hyper-connection norm / mid / mix,
// q4 -> bf16 expert dequantisation, swiglu on expert-sorted rows and the weighted combine back to
// token order (roles of the reference's src/kernels/hc.hip:8-94, src/kernels/moe_route.hip:168-224
// and the dequant stage of src/kernels/moe_experts.hip:46-150).
#include "common.cuh"

namespace qw {

// grid (T, hc), 256 threads.  X[t][s][:] (+= pend[t][:] * 2*sigmoid(inj[t][s]/hc)); xn = bf16(X * w1 * rsqrt(mean X^2 + eps)).
// SH % 4 == 0, SH <= 4096: a thread keeps its (up to four) float4 pieces of the row in registers between the two passes.
__global__ void __launch_bounds__(256) hc_prenorm_T_kernel(float *X, const float *pend, int ld_pend, const float *inj,
                                                           const float *w1, int SH, int hc, float eps, bf16 *xn) {
    __shared__ float scratch[32];
    const int t = blockIdx.x, s = blockIdx.y;
    float4 *x = reinterpret_cast<float4 *>(X + ((long long)t * hc + s) * SH);
    const float4 *pe = reinterpret_cast<const float4 *>(pend + (pend ? (long long)t * ld_pend : 0));
    const int n4 = SH >> 2;
    float4 v[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int c = threadIdx.x + i * 256;
        v[i] = c < n4 ? x[c] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float ss = 0.f;
    if (pend) {
        const float coef = 2.f * sigmoidf_(inj[(long long)t * hc + s] / float(hc));
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int c = threadIdx.x + i * 256;
            if (c < n4) {
                const float4 p = pe[c];
                v[i].x = fmaf(p.x, coef, v[i].x); v[i].y = fmaf(p.y, coef, v[i].y);
                v[i].z = fmaf(p.z, coef, v[i].z); v[i].w = fmaf(p.w, coef, v[i].w);
                x[c] = v[i];
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
    ss = block_sum<256>(ss, scratch);
    const float r = rsqrtf(ss / float(SH) + eps);
    const float4 *w4 = reinterpret_cast<const float4 *>(w1 + (long long)s * SH);
    uint2 *o = reinterpret_cast<uint2 *>(xn + ((long long)t * hc + s) * SH);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int c = threadIdx.x + i * 256;
        if (c < n4) {
            const float4 w = w4[c];
            o[c] = make_uint2(pack_bf16(v[i].x * w.x * r, v[i].y * w.y * r), pack_bf16(v[i].z * w.z * r, v[i].w * w.w * r));
        }
    }
}

// d [nsplit][T][ld_d] fp32 (R + n_inj columns; the split-K partial sums of the down projection, added here in order)
// -> u bf16 [T][R] = silu(d/hc), inj fp32 [T][n_inj].
__global__ void hc_mid_T_kernel(const float *d, int ld_d, int R, int n_inj, int hc, bf16 *u, float *inj, long long total,
                                int nsplit, long long split_stride) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int w = R + n_inj;
    const long long t = i / w;
    const int j = (int)(i - t * w);
    float v = d[t * ld_d + j];
    for (int s = 1; s < nsplit; ++s) v += d[s * split_stride + t * ld_d + j];
    if (j < R) u[t * R + j] = __float2bfloat16(siluf_(v / float(hc)));
    else inj[t * n_inj + (j - R)] = v;
}

// g [T][SH*hc] fp32 with columns ordered (c, s); bin[t][c] = mean_s sigmoid(g[t][c][s]) * xn[t][s][c].  hc == 4, SH even,
// ld_bin even.  One thread per two neighbouring columns.
__global__ void hc_mix_T_kernel(const float *g, const bf16 *xn, int SH, bf16 *bin, int ld_bin, long long total2) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total2) return;
    const int h2 = SH >> 1;
    const long long t = i / h2;
    const int c = (int)(i - t * h2) * 2;
    const float4 g0 = *reinterpret_cast<const float4 *>(g + (t * SH + c) * 4);
    const float4 g1 = *reinterpret_cast<const float4 *>(g + (t * SH + c + 1) * 4);
    const bf16 *x = xn + t * 4 * SH + c;
    const float2 x0 = __bfloat1622float2(*reinterpret_cast<const bf162 *>(x));
    const float2 x1 = __bfloat1622float2(*reinterpret_cast<const bf162 *>(x + SH));
    const float2 x2 = __bfloat1622float2(*reinterpret_cast<const bf162 *>(x + 2 * SH));
    const float2 x3 = __bfloat1622float2(*reinterpret_cast<const bf162 *>(x + 3 * SH));
    const float v0 = sigmoidf_(g0.x) * x0.x + sigmoidf_(g0.y) * x1.x + sigmoidf_(g0.z) * x2.x + sigmoidf_(g0.w) * x3.x;
    const float v1 = sigmoidf_(g1.x) * x0.y + sigmoidf_(g1.y) * x1.y + sigmoidf_(g1.z) * x2.y + sigmoidf_(g1.w) * x3.y;
    *reinterpret_cast<bf162 *>(bin + t * ld_bin + c) = __floats2bfloat162_rn(v0 * 0.25f, v1 * 0.25f);
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

// Expert sort of a chunk's (token, choice) pairs in one block: rows of one expert become consecutive.
// pair_expert [P] (local expert id, or < 0 / >= E: not on this rank) -> inv [P] (pair -> sorted row, -1 = none),
// src_token [P] (sorted row -> token), and the two tile tables of the grouped GEMMs ({first row, valid rows, first W row of
// the expert, 0} per 128-row tile; unused entries zero).  The order of an expert's rows among themselves follows the
// atomics and may differ between runs; every row's result is independent of where it sits, so outputs do not.
// One block of 1024 threads; E <= 1024.
__global__ void __launch_bounds__(1024) moe_sort_kernel(const int *pair_expert, int P, int top_k, int E, int Nw13, int Nw2,
                                                        int max_tiles, int *inv, int *src_token, int4 *t13, int4 *t2) {
    __shared__ int cnt[1024], off[1024], tb[1024], cur[1024];
    __shared__ int warp_tot[2][32];
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    cnt[tid] = 0;
    cur[tid] = 0;
    for (int i = tid; i < max_tiles; i += 1024) t13[i] = t2[i] = make_int4(0, 0, 0, 0);
    __syncthreads();
    for (int i = tid; i < P; i += 1024) {
        const int e = pair_expert[i];
        if (e >= 0 && e < E) atomicAdd(&cnt[e], 1);
    }
    __syncthreads();
    // exclusive scans of the counts (row offsets) and of the tile counts (tile-table offsets)
    const int c = tid < E ? cnt[tid] : 0, nt = (c + 127) >> 7;
    int sc = c, st = nt;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int a = __shfl_up_sync(0xffffffffu, sc, o), b = __shfl_up_sync(0xffffffffu, st, o);
        if (lane >= o) { sc += a; st += b; }
    }
    if (lane == 31) { warp_tot[0][wid] = sc; warp_tot[1][wid] = st; }
    __syncthreads();
    if (wid == 0) {
        int a = warp_tot[0][lane], b = warp_tot[1][lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int x = __shfl_up_sync(0xffffffffu, a, o), y = __shfl_up_sync(0xffffffffu, b, o);
            if (lane >= o) { a += x; b += y; }
        }
        warp_tot[0][lane] = a;
        warp_tot[1][lane] = b;
    }
    __syncthreads();
    const int row0 = sc - c + (wid ? warp_tot[0][wid - 1] : 0), tile0 = st - nt + (wid ? warp_tot[1][wid - 1] : 0);
    off[tid] = row0;
    tb[tid] = tile0;
    if (tid < E)
        for (int j = 0; j < nt && tile0 + j < max_tiles; ++j) {
            const int valid = min(128, c - j * 128);
            t13[tile0 + j] = make_int4(row0 + j * 128, valid, tid * Nw13, 0);
            t2[tile0 + j] = make_int4(row0 + j * 128, valid, tid * Nw2, 0);
        }
    __syncthreads();
    for (int i = tid; i < P; i += 1024) {
        const int e = pair_expert[i];
        int r = -1;
        if (e >= 0 && e < E) {
            r = off[e] + atomicAdd(&cur[e], 1);
            src_token[r] = i / top_k;
        }
        inv[i] = r;
    }
}

// xperm[r][:] = x[src_token[r]][:] for the first n_rows sorted rows (bf16 rows of H elements, H % 8 == 0).  grid n_rows.
__global__ void moe_gather_rows_kernel(const bf16 *x, int ldx, const int *src_token, int H, bf16 *xperm) {
    const int r = blockIdx.x;
    const uint4 *src = reinterpret_cast<const uint4 *>(x + (long long)src_token[r] * ldx);
    uint4 *dst = reinterpret_cast<uint4 *>(xperm + (long long)r * H);
    for (int i = threadIdx.x; i < H / 8; i += blockDim.x) dst[i] = src[i];
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
    if (SH > 4096 || (SH & 3) || (ld_pend & 3)) return -1;
    hc_prenorm_T_kernel<<<dim3(T, hc), 256, 0, s>>>(X, pend, ld_pend, inj, w1, SH, hc, eps, (bf16 *)xn);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
QW_API int qwk_hc_mid_T(const float *d, int ld_d, int R, int n_inj, int hc, void *u, float *inj, int T, int nsplit,
                        long long split_stride, cudaStream_t s) {
    const long long total = (long long)T * (R + n_inj);
    hc_mid_T_kernel<<<blocks_for(total, 256), 256, 0, s>>>(d, ld_d, R, n_inj, hc, (bf16 *)u, inj, total, nsplit < 1 ? 1 : nsplit,
                                                           split_stride);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
QW_API int qwk_hc_mix_T(const float *g, const void *xn, int SH, void *bin, int ld_bin, int T, cudaStream_t s) {
    if ((SH & 1) || (ld_bin & 1)) return -1;
    const long long total = (long long)T * (SH >> 1);
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

// Expert sort + row gather of a prefill chunk (see moe_sort_kernel).  pair_expert [T*top_k]; x bf16 [T][ldx];
// outputs inv [T*top_k], src_token [T*top_k] (scratch), t13 / t2 [max_tiles] int4, xperm bf16 [T*top_k][H].  With all pairs
// local, xperm holds T*top_k rows; rows past the last local pair are left as they were.
QW_API int qwk_moe_sort_T(const int *pair_expert, int T, int top_k, int E, int Nw13, int Nw2, int max_tiles, int *inv,
                          int *src_token, void *t13, void *t2, const void *x, int ldx, int H, void *xperm, cudaStream_t s) {
    if (E > 1024 || (H & 7) || (ldx & 7)) return -1;
    const int P = T * top_k;
    cudaMemsetAsync(src_token, 0, sizeof(int) * (size_t)P, s);
    moe_sort_kernel<<<1, 1024, 0, s>>>(pair_expert, P, top_k, E, Nw13, Nw2, max_tiles, inv, src_token, (int4 *)t13, (int4 *)t2);
    moe_gather_rows_kernel<<<P, 256, 0, s>>>((const bf16 *)x, ldx, src_token, H, (bf16 *)xperm);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
