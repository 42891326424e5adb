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
#include "fuse.cuh"

namespace qw {

// X[m][s][:] = embedding row of tokens[m] (this rank's columns) for every stream.
__global__ void embed_rows_kernel(const int *tokens, const bf16 *table, int ld_table, int col0, int SH, int hc,
                                  int vocab, float *X) {
    const int m = blockIdx.x;
    int t = tokens[m];
    QW_DCHECK(t >= 0 && t < vocab, 0x01000000u | (unsigned)(m & 0xffffff));          // token id outside the vocabulary (row m)
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

constexpr int UP_ROWS = 4;     // rows per block of hc_up_mix (8 in steps of more than four rows: the weights are read once per block)
constexpr int UP_MAXI = 5;     // 16-byte weight pieces per lane: covers mixer ranks up to 320

// grid (ceil(SH/8), ceil(M/UPR)), 256 threads.  hc must be 4 (one 8-lane group per stream).
// y[s][c] = bf16(X[s][c] * w1[s][c]) is recomputed here exactly as hc_down_kernel computed it.
template <bool FUSED, int UPR>
__global__ void __launch_bounds__(256, 3) hc_up_mix_kernel(const float *red, int ld_red, const bf16 *Wu /* [SH][hc][R] */,
                                                        const float *X, const float *w1, int SH, int hc, int R, int hc_down,
                                                        float inv_H, float eps, int M, float *inj, int ld_inj, bf16 *bin,
                                                        int ld_bin, int bin_col0, PfArgs pf, FuseIn fi, FuseOut fo) {
    extern __shared__ float sm[];
    float *u = sm;                         // [UPR][R]
    float *rs = sm + UPR * R;          // [UPR][hc]
    const int m0 = blockIdx.y * UPR;
    const int nrow = min(UPR, M - m0);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int c = blockIdx.x * 8 + warp;
    const int s = lane >> 3, li = lane & 7;
    const int nch = R >> 3;
    // weights first: they do not depend on the predecessor
    uint4 w[UP_MAXI];
    if (c < SH) {
        const uint4 *wp = reinterpret_cast<const uint4 *>(Wu + ((long long)c * hc + s) * R);
#pragma unroll
        for (int i = 0; i < UP_MAXI; ++i)
            if (li + 8 * i < nch) w[i] = ld_stream(wp + li + 8 * i);
    }
    pf_issue(pf);
    pdl_wait();
    pdl_trigger();
    // this lane's residual values times the norm weight: needed only at the very end, fetched now so that their L2
    // round trip overlaps the staging of the reduced vector
    float xw[UPR];
    {
        const float w1v = c < SH ? w1[s * SH + c] : 0.f;
#pragma unroll
        for (int mm = 0; mm < UPR; ++mm)
            xw[mm] = (c < SH && mm < nrow) ? __ldcg(X + ((long long)(m0 + mm) * hc + s) * SH + c) * w1v : 0.f;
    }
    // element i of the reduced vector: the local buffer, or (fused all-reduce) the ranks' words added in rank
    // order - staged once per block into shared memory, with every thread's loads in flight together
    float *reds = rs + UPR * hc;       // [UPR][ld_red]
    if constexpr (FUSED) {
        const unsigned int seq_in = fuse_seq(fi);
        // what this mixer's down projection wrote of each row (an even count), as pairs of words; a thread has
        // the loads of two pairs from four ranks in flight at once
        const int npair = (hc + hc * hc_down) >> 1, total = nrow * npair;
        for (int p0 = threadIdx.x; p0 < total; p0 += 512) {
            const int p1 = p0 + 256;
            const bool two = p1 < total;
            const int mm0 = p0 / npair, j0 = (p0 - mm0 * npair) * 2;
            const int mm1 = two ? p1 / npair : mm0, j1 = two ? (p1 - mm1 * npair) * 2 : j0;
            float2 a, b;
            fuse_sum2x2(fi, seq_in, (long long)(m0 + mm0) * ld_red + j0, (long long)(m0 + mm1) * ld_red + j1, a, b);
            reds[mm0 * ld_red + j0] = a.x;
            reds[mm0 * ld_red + j0 + 1] = a.y;
            if (two) {
                reds[mm1 * ld_red + j1] = b.x;
                reds[mm1 * ld_red + j1 + 1] = b.y;
            }
        }
        __syncthreads();
    }
    if constexpr (!FUSED) {
        // the same staging from the local buffer: every thread's loads in flight together (one L2 round trip per batch)
        const int used = hc + hc * hc_down, total = nrow * used;
        for (int i0 = threadIdx.x; i0 < total; i0 += 2048) {
            float v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int i = i0 + u * 256;
                const int mm = i / used, j = i - mm * used;
                v[u] = i < total ? __ldcg(red + (long long)(m0 + mm) * ld_red + j) : 0.f;
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int i = i0 + u * 256;
                const int mm = i / used, j = i - mm * used;
                if (i < total) reds[mm * ld_red + j] = v[u];
            }
        }
        __syncthreads();
    }
    auto red_at = [&](long long i) -> float { return reds[i - (long long)m0 * ld_red]; };
    for (int i = threadIdx.x; i < nrow * hc; i += 256) {
        const int mm = i / hc, ss = i % hc;
        rs[mm * hc + ss] = rsqrtf(red_at((long long)(m0 + mm) * ld_red + ss) * inv_H + eps);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < nrow * hc_down; i += 256) {
        const int mm = i / hc_down, j = i % hc_down;
        const long long p = (long long)(m0 + mm) * ld_red + hc + j;
        float d = 0.f;
        for (int ss = 0; ss < hc; ++ss) d = fmaf(rs[mm * hc + ss], red_at(p + ss * hc_down), d);
        if (j < R) u[mm * R + j] = siluf_(d / float(hc));
        else if (inj && blockIdx.x == 0) inj[(long long)(m0 + mm) * ld_inj + (j - R)] = d;
    }
    __syncthreads();
    if (c >= SH) return;
    const unsigned int seq_out = FUSED ? fuse_seq(fo) : 0u;
    float acc[UPR];
#pragma unroll
    for (int mm = 0; mm < UPR; ++mm) acc[mm] = 0.f;
#pragma unroll
    for (int i = 0; i < UP_MAXI; ++i) {
        const int ch = li + 8 * i;
        if (ch < nch) {
            const float wf[8] = {bf16_lo(w[i].x), bf16_hi(w[i].x), bf16_lo(w[i].y), bf16_hi(w[i].y),
                                 bf16_lo(w[i].z), bf16_hi(w[i].z), bf16_lo(w[i].w), bf16_hi(w[i].w)};
#pragma unroll
            for (int mm = 0; mm < UPR; ++mm) {
                if (mm < nrow) {
                    const float *uu = u + mm * R + ch * 8;
#pragma unroll
                    for (int k = 0; k < 8; ++k) acc[mm] = fmaf(wf[k], uu[k], acc[mm]);
                }
            }
        }
    }
#pragma unroll
    for (int mm = 0; mm < UPR; ++mm) {
        float g = acc[mm];
        g += __shfl_xor_sync(0xffffffffu, g, 1);
        g += __shfl_xor_sync(0xffffffffu, g, 2);
        g += __shfl_xor_sync(0xffffffffu, g, 4);
        float v = 0.f;
        if (mm < nrow) {
            const float yv = __bfloat162float(__float2bfloat16(xw[mm]));
            v = sigmoidf_(g) * yv * rs[mm * hc + s];
        }
        v += __shfl_xor_sync(0xffffffffu, v, 8);
        v += __shfl_xor_sync(0xffffffffu, v, 16);
        if (lane == 0 && mm < nrow) {
            const bf16 o = __float2bfloat16(v / float(hc));
            if (FUSED) fuse_put_all(fo, seq_out, m0 + mm, c, (unsigned int)__bfloat16_as_ushort(o));      // fused all-gather
            else bin[(long long)(m0 + mm) * ld_bin + bin_col0 + c] = o;
        }
    }
}

// ------------------------------------------------------------------------------------------
// Fused mixer front end: deferred combine + per-stream sum of squares + down projection.
//   Xout[m][s][:] = Xin[m][s][:] + pend[m][:] * 2*sigmoid(inj_prev[m][s]/hc)     (when pend != null)
//   send[m][s]               = sum_c X^2
//   send[m][hc + s*down + j] = sum_c Wd[j][s][c] * bf16(X[s][c] * w1[s][c])
// Every block rebuilds the bf16 row slice it needs in shared memory (the residual is tiny and
// sits in L2); blocks with blockIdx.x == 0 also store X and the sums of squares.  X is written
// to a second buffer because other blocks still read the old one.
// grid (ceil(down/rpb), hc, ceil(M/8)), 256 threads, dynamic smem 8*SH bf16.
// ------------------------------------------------------------------------------------------
constexpr int DN_PF = 5;      // 16-byte weight pieces per lane fetched before the dependency wait (2560 columns / 2 warps / 32 lanes / 8)
constexpr int DN_CP = 3;      // column pieces of 1024 handled per pass of hc_down's row builder (SH <= 3072 in one pass)

struct HcDownArgs {
    const float *Xin;
    float *Xout;            // null: no combine, X stays where it is
    const float *pend;      // [M][ld_pend] or null
    int ld_pend;
    const float *inj_prev;  // [M][hc]
    const float *w1;        // [hc][SH]
    const bf16 *Wd;         // [down][hc][SH]
    float *send;            // [M][ld_send]
    int ld_send, SH, hc, down, M, wpr;
    PfArgs pf;
    FuseIn fi;              // fused reduce-scatter: `pend` is the sum of the ranks' slots
    FuseOut fo;             // fused all-reduce of `send`
};

template <bool FUSED>
__global__ void __launch_bounds__(256, 3) hc_down_kernel(HcDownArgs a) {
    extern __shared__ __align__(16) unsigned char smraw[];
    bf16 *ybuf = reinterpret_cast<bf16 *>(smraw);          // [8][SH]
    __shared__ float part[8][8];
    __shared__ float scratch[32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int s = blockIdx.y, m0 = blockIdx.z * 8;
    const int nrow = min(8, a.M - m0);
    const int wpr = a.wpr, rpb = 8 / wpr;
    const int j = blockIdx.x * rpb + warp / wpr, kw = warp % wpr;
    const int nchunk = a.SH >> 3;
    const bf16 *wrow = a.Wd + ((long long)j * a.hc + s) * a.SH;
    // weights first: prefetch this warp's share of its row into registers / L2
    uint4 w0[DN_PF];          // this warp's share of its weight row: all of it for the model's shapes, so no load is issued late
    const int stride = wpr * 32;
    if (j < a.down) {
#pragma unroll
        for (int u = 0; u < DN_PF; ++u) {
            const int c = kw * 32 + lane + u * stride;
            if (c < nchunk) w0[u] = ld_stream(reinterpret_cast<const uint4 *>(wrow) + c);
        }
    }
    pf_issue(a.pf);
    pdl_wait();
    pdl_trigger();
    const unsigned int seq_in = FUSED && a.fi.active ? fuse_seq(a.fi) : 0u;
    const unsigned int seq_out = FUSED ? fuse_seq(a.fo) : 0u;
    for (int r = 0; r < nrow; ++r) {           // the whole block builds each row slice: short dependent chains
        const int m = m0 + r;
        const float *xin = a.Xin + ((long long)m * a.hc + s) * a.SH;
        float coef = 0.f;
        if (a.pend) coef = 2.f * sigmoidf_(a.inj_prev[(long long)m * a.hc + s] / float(a.hc));
        float ss = 0.f;
        // up to DN_CP pieces of 1024 columns per pass, every load of the pass issued before the first use (the residual,
        // the pending block output and the norm weight all come from L2: one round trip per pass instead of one per piece)
        constexpr int CP = FUSED ? 1 : DN_CP;          // the fused form keeps the ranks' words in flight instead (SH is a shard there)
        for (int c0 = threadIdx.x * 4; c0 < a.SH; c0 += 1024 * CP) {
            float4 xv[CP], pv[CP], wv[CP];
#pragma unroll
            for (int q = 0; q < CP; ++q) {
                const int c = c0 + q * 1024;
                if (c < a.SH) {
                    xv[q] = __ldcg(reinterpret_cast<const float4 *>(xin + c));
                    wv[q] = __ldg(reinterpret_cast<const float4 *>(a.w1 + s * a.SH + c));
                    if (a.pend && !(FUSED && a.fi.active)) pv[q] = __ldcg(reinterpret_cast<const float4 *>(a.pend + (long long)m * a.ld_pend + c));
                }
            }
#pragma unroll
            for (int q = 0; q < CP; ++q) {
                const int c = c0 + q * 1024;
                if (c < a.SH) {
                    float4 v = xv[q];
                    if (a.pend) {
                        // fused reduce-scatter: the ranks' parts of the block output, added in rank order
                        const float4 p = (FUSED && a.fi.active) ? fuse_sum4(a.fi, seq_in, (long long)m * a.ld_pend + c) : pv[q];
                        v.x = fmaf(p.x, coef, v.x); v.y = fmaf(p.y, coef, v.y);
                        v.z = fmaf(p.z, coef, v.z); v.w = fmaf(p.w, coef, v.w);
                        if (blockIdx.x == 0) *reinterpret_cast<float4 *>(a.Xout + ((long long)m * a.hc + s) * a.SH + c) = v;
                    }
                    ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
                    uint2 pk;
                    pk.x = pack_bf16(v.x * wv[q].x, v.y * wv[q].y);
                    pk.y = pack_bf16(v.z * wv[q].z, v.w * wv[q].w);
                    *reinterpret_cast<uint2 *>(ybuf + r * a.SH + c) = pk;
                }
            }
        }
        if (blockIdx.x == 0) {                 // block-uniform: only these blocks need the sum of squares
            ss = block_sum<256>(ss, scratch);
            if (threadIdx.x == 0) {
                if (FUSED) fuse_put_all(a.fo, seq_out, m, s, __float_as_uint(ss));      // fused all-reduce
                else a.send[(long long)m * a.ld_send + s] = ss;
            }
        }
    }
    __syncthreads();
    float acc[8];
#pragma unroll
    for (int m = 0; m < 8; ++m) acc[m] = 0.f;
    if (j < a.down) {
        for (int c0 = kw * 32 + lane, first = 1; c0 < nchunk; c0 += DN_PF * stride, first = 0) {
            uint4 w[DN_PF];
#pragma unroll
            for (int u = 0; u < DN_PF; ++u) {
                const int c = c0 + u * stride;
                if (c < nchunk) w[u] = first ? w0[u] : ld_stream(reinterpret_cast<const uint4 *>(wrow) + c);
            }
#pragma unroll
            for (int u = 0; u < DN_PF; ++u) {
                const int c = c0 + u * stride;
                if (c < nchunk) {
#pragma unroll
                    for (int m = 0; m < 8; ++m)
                        if (m < nrow) acc[m] = dot8(w[u], *reinterpret_cast<const uint4 *>(ybuf + m * a.SH + c * 8), acc[m]);
                }
            }
        }
    }
#pragma unroll
    for (int m = 0; m < 8; ++m) acc[m] = warp_sum(acc[m]);
    if (wpr > 1) {
        if (lane == 0) {
#pragma unroll
            for (int m = 0; m < 8; ++m) part[warp][m] = acc[m];
        }
        __syncthreads();
        if (kw == 0) {
#pragma unroll
            for (int m = 0; m < 8; ++m) {
                float t = 0.f;
                for (int q = 0; q < wpr; ++q) t += part[warp + q][m];
                acc[m] = t;
            }
        }
    }
    if (kw == 0 && lane == 0 && j < a.down) {
#pragma unroll
        for (int m = 0; m < 8; ++m)
            if (m < nrow) {
                if (FUSED) fuse_put_all(a.fo, seq_out, m0 + m, a.hc + s * a.down + j, __float_as_uint(acc[m]));
                else a.send[(long long)(m0 + m) * a.ld_send + a.hc + s * a.down + j] = acc[m];
            }
    }
}

}  // namespace qw

using namespace qw;

QW_DCHECK_TU(hc)

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

QW_API int qwk_hc_up_mix(const float *red, int ld_red, const void *Wu, const float *X, const float *w1, int SH, int hc,
                         int R, int n_inj, int H, float eps, int M, float *inj, int ld_inj, void *bin, int ld_bin,
                         int bin_col0, cudaStream_t s) {
    if (hc != 4 || (R & 7) || R > 8 * 8 * UP_MAXI) return -1;
    const int upr = UP_ROWS;          // eight rows per block (weights read once for up to eight rows) measured slower at 6 and 8 rows
    dim3 grid((SH + 7) / 8, (M + upr - 1) / upr);
    const FuseIn fi = take_fi();
    const size_t smem = sizeof(float) * ((size_t)upr * R + upr * hc + (size_t)upr * ld_red);
    if (smem > 96 * 1024) return -1;
    {
        static bool attr[64] = {};
        int dev = 0;
        cudaGetDevice(&dev);
        if (dev < 0 || dev >= 64) dev = 0;
        if (!attr[dev]) {
            cudaFuncSetAttribute(hc_up_mix_kernel<true, 2 * UP_ROWS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
            cudaFuncSetAttribute(hc_up_mix_kernel<false, 2 * UP_ROWS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
            attr[dev] = true;
        }
    }
    if (upr == UP_ROWS && smem > 48 * 1024) return -1;
    const FuseOut fo = take_fo();
    if ((fi.active != 0) != (fo.mode != 0)) return -1;          // the fused mixer both receives and sends
    cudaError_t e;
#define QW_UPMIX(F_, R_)                                                                                                        \
    launch_pdl(hc_up_mix_kernel<F_, R_>, grid, dim3(256), smem, s, red, ld_red, (const bf16 *)Wu, X, w1, SH, hc, R, R + n_inj, \
               1.f / float(H), eps, M, inj, ld_inj, (bf16 *)bin, ld_bin, bin_col0, take_pf(), fi, fo)
    if (fi.active) e = upr == UP_ROWS ? QW_UPMIX(true, UP_ROWS) : QW_UPMIX(true, 2 * UP_ROWS);
    else e = upr == UP_ROWS ? QW_UPMIX(false, UP_ROWS) : QW_UPMIX(false, 2 * UP_ROWS);
#undef QW_UPMIX
    return e == cudaSuccess ? 0 : -2;
}

// Fused combine + sum of squares + down projection (see hc_down_kernel).  Xout == null keeps X in place.
QW_API int qwk_hc_down(const float *Xin, float *Xout, const float *pend, int ld_pend, const float *inj_prev,
                       const float *w1, const void *Wd, float *send, int ld_send, int SH, int hc, int down, int M,
                       cudaStream_t s) {
    if ((SH & 7) || (pend && !Xout)) return -1;
    HcDownArgs a;
    a.Xin = Xin; a.Xout = Xout; a.pend = pend; a.ld_pend = ld_pend; a.inj_prev = inj_prev; a.w1 = w1;
    a.Wd = (const bf16 *)Wd; a.send = send; a.ld_send = ld_send; a.SH = SH; a.hc = hc; a.down = down; a.M = M; a.pf = take_pf();
    a.fi = take_fi(); a.fo = take_fo();
    const long long rows = (long long)down * hc;
    a.wpr = rows >= NUM_SMS * 8 * 2 ? 1 : (rows >= NUM_SMS * 4 * 2 ? 2 : (rows >= NUM_SMS * 2 * 2 ? 4 : 8));
    if ((SH >> 3) < a.wpr * 32) {          // short rows: do not spread a row over more warps than it has pieces
        while (a.wpr > 1 && (SH >> 3) < a.wpr * 32) a.wpr >>= 1;
    }
    const int rpb = 8 / a.wpr;
    dim3 grid((down + rpb - 1) / rpb, hc, (M + 7) / 8);
    const size_t smem = (size_t)8 * SH * sizeof(bf16);
    static bool attr_set = false;
    if (!attr_set && smem > 48 * 1024) {
        cudaFuncSetAttribute(hc_down_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
        cudaFuncSetAttribute(hc_down_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
        attr_set = true;
    }
    if (a.fi.active && !a.fo.mode) return -1;          // a fused down projection always sends its all-reduce
    cudaError_t e = a.fo.mode ? launch_pdl(hc_down_kernel<true>, grid, dim3(256), smem, s, a)
                              : launch_pdl(hc_down_kernel<false>, grid, dim3(256), smem, s, a);
    return e == cudaSuccess ? 0 : -2;
}
