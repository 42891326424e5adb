// Token-major prefill on several ranks: the glue kernels of a mixer and of the MoE combine in the form
// that carries the collectives (tp.cuh), plus stand-alone large-payload collectives over the same
// channel (push + reduce) for the few sites without a producer kernel of their own and as the unfused
// comparison.  The residual stream is sharded along the hidden dimension (SH = H / ranks columns of
// every stream per rank), so a mixer is
//     prenorm (X += reduce-scatter parts of the pending block output; sum of squares -> all ranks)
//  -> norm    (sums of squares of all ranks -> xn)
//  -> down projection GEMM, epilogue sends the partial products to all ranks
//  -> mid     (partial products of all ranks added in rank order -> u, injection logits)
//  -> up projection GEMM -> mix (block input columns of this rank -> all ranks)
// (reference: src/engine/prefill.hip:208-224 and the kernels of src/kernels/hc.hip:8-72).
#include "kernels.h"
#include "tp.cuh"

namespace qw {

struct Peers {
    char *p[TP_MAX_RANKS];
};

// Kernels of this file that wait for or publish a collective run as a few fat CTAs (TP_CTAS_PER_SM per SM) that walk
// their share of the rows: the wait (an acquire poll) and the publication (a system-wide fence and a ticket) are paid
// once per CTA, not once per row - with one CTA per row a 4,096-token chunk paid 16,384 fences per launch, which cost
// more than the kernel's work.
constexpr int TP_CTAS_PER_SM = 8;
constexpr int TP_PRENORM_ITEMS = 64;          // (row, stream) items per CTA of hc_prenorm_tp, at most

// grid: CTAs that each own a contiguous range of `per` (row, stream) items, 256 threads = 8 warps, one item per warp at a
// time (an item is SH floats: a warp has all of its loads in flight at once, and eight items are in flight per CTA; one
// CTA per item spent its time in the chain load -> reduce -> store).  X[t][s][:] += coef(t, s) * sum_r part_r[t][:]
// (parts added in rank order), then the items' sums of squares go to every rank in one coalesced store per CTA.
// SH % 4 == 0, per <= TP_PRENORM_ITEMS.
__global__ void __launch_bounds__(256) hc_prenorm_tp_kernel(float *X, const float *pend, int nparts, long long part_stride,
                                                            int ld_pend, const float *inj, int SH, int hc, long long items, int per,
                                                            TpWait wait, Peers ssq_dst, int ranks, TpSignal sig) {
    __shared__ float s_ssq[TP_PRENORM_ITEMS];
    const long long first = (long long)blockIdx.x * per;
    const int mine = (int)min((long long)per, items - first);
    const int n4 = SH >> 2, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool ok = pend ? tp_wait(wait) : true;
    for (int k = warp; k < mine; k += 8) {
        const long long it = first + k;
        const long long t = it / hc;
        float4 *x = reinterpret_cast<float4 *>(X + it * SH);
        const float coef = (pend && ok) ? 2.f * sigmoidf_(inj[it] / float(hc)) : 0.f;
        float ss = 0.f;
#pragma unroll 4
        for (int c = lane; c < n4; c += 32) {
            float4 v = x[c];
            if (pend && ok) {
                float4 p = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int r = 0; r < nparts; ++r) {
                    const float4 q = __ldcg(reinterpret_cast<const float4 *>(pend + r * part_stride + t * ld_pend) + c);
                    p.x += q.x; p.y += q.y; p.z += q.z; p.w += q.w;
                }
                v.x = fmaf(p.x, coef, v.x); v.y = fmaf(p.y, coef, v.y);
                v.z = fmaf(p.z, coef, v.z); v.w = fmaf(p.w, coef, v.w);
                x[c] = v;
            }
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (lane == 0) s_ssq[k] = ss;
    }
    __syncthreads();
    if (ok && (int)threadIdx.x < mine) {
#pragma unroll
        for (int d = 0; d < TP_MAX_RANKS; ++d)
            if (d < ranks) reinterpret_cast<float *>(ssq_dst.p[d])[first + threadIdx.x] = s_ssq[threadIdx.x];
    }
    tp_signal(sig);
}

// grid: CTAs of 8 warps that stride over the (row, stream) items, one item per warp at a time.
// xn[t][s][:] = bf16(X * w1 * rsqrt(sum_r ssq_r[t][s] / H + eps)).
__global__ void __launch_bounds__(256) hc_norm_tp_kernel(const float *X, const float *ssq_parts, int nparts, long long part_stride,
                                                         const float *w1, int SH, int hc, int H, float eps, bf16 *xn, long long items,
                                                         TpWait wait) {
    if (!tp_wait(wait)) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n4 = SH >> 2;
    for (long long it = (long long)blockIdx.x * 8 + warp; it < items; it += (long long)gridDim.x * 8) {
        const int s = (int)(it % hc);
        float tot = 0.f;
        for (int r = 0; r < nparts; ++r) tot += __ldcg(ssq_parts + r * part_stride + it);
        const float rn = rsqrtf(tot / float(H) + eps);
        const float4 *x = reinterpret_cast<const float4 *>(X + it * SH);
        const float4 *w4 = reinterpret_cast<const float4 *>(w1 + (long long)s * SH);
        uint2 *o = reinterpret_cast<uint2 *>(xn + it * SH);
#pragma unroll 4
        for (int c = lane; c < n4; c += 32) {
            const float4 v = x[c], w = w4[c];
            o[c] = make_uint2(pack_bf16(v.x * w.x * rn, v.y * w.y * rn), pack_bf16(v.z * w.z * rn, v.w * w.w * rn));
        }
    }
}

// The partial down projections of all ranks ([T][ld_d] fp32 each) added in rank order -> u bf16 [T][R] = silu(d / hc),
// inj fp32 [T][n_inj].
__global__ void __launch_bounds__(256) hc_mid_tp_kernel(const float *parts, int nparts, long long part_stride, int ld_d, int R,
                                                        int n_inj, int hc, bf16 *u, float *inj, long long total, TpWait wait) {
    if (!tp_wait(wait)) return;
    const int w = R + n_inj;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / w;
        const int j = (int)(i - t * w);
        float v = 0.f;
        for (int r = 0; r < nparts; ++r) v += __ldcg(parts + r * part_stride + t * ld_d + j);
        if (j < R) u[t * R + j] = __float2bfloat16(siluf_(v / float(hc)));
        else inj[t * n_inj + (j - R)] = v;
    }
}

// g [T][SH*4] fp32 with columns ordered (c, s); this rank's block-input columns bin[t][col0 + c] = mean_s sigmoid(g) * xn
// go to every rank's block-input matrix.  One thread per eight columns (a 16-byte store per destination); a form with one
// thread per two columns and the stores gathered by shuffles measured slower (5.4 -> 7.7 ms per chunk on 2 GPUs).
// SH % 8 == 0, col0 % 8 == 0, ld_bin % 8 == 0.
__global__ void __launch_bounds__(256) hc_mix_tp_kernel(const float *g, const bf16 *xn, int SH, Peers bin_dst, int ranks,
                                                        int ld_bin, int col0, long long total8, TpSignal sig) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total8; i += (long long)gridDim.x * blockDim.x) {
        const int h8 = SH >> 3;
        const long long t = i / h8;
        const int c = (int)(i - t * h8) * 8;
        const float4 *gp = reinterpret_cast<const float4 *>(g + (t * SH + c) * 4);
        const bf16 *x = xn + t * 4 * SH + c;
        float xs[4][8];
#pragma unroll
        for (int s = 0; s < 4; ++s) {
            const uint4 q = *reinterpret_cast<const uint4 *>(x + (long long)s * SH);
            xs[s][0] = bf16_lo(q.x); xs[s][1] = bf16_hi(q.x); xs[s][2] = bf16_lo(q.y); xs[s][3] = bf16_hi(q.y);
            xs[s][4] = bf16_lo(q.z); xs[s][5] = bf16_hi(q.z); xs[s][6] = bf16_lo(q.w); xs[s][7] = bf16_hi(q.w);
        }
        float o[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const float4 gg = gp[k];
            o[k] = 0.25f * (sigmoidf_(gg.x) * xs[0][k] + sigmoidf_(gg.y) * xs[1][k] + sigmoidf_(gg.z) * xs[2][k] + sigmoidf_(gg.w) * xs[3][k]);
        }
        const uint4 pk = make_uint4(pack_bf16(o[0], o[1]), pack_bf16(o[2], o[3]), pack_bf16(o[4], o[5]), pack_bf16(o[6], o[7]));
        const long long off = (t * ld_bin + col0 + c) * 2;
#pragma unroll
        for (int d = 0; d < TP_MAX_RANKS; ++d)
            if (d < ranks) *reinterpret_cast<uint4 *>(bin_dst.p[d] + off) = pk;
    }
    tp_signal(sig);
}

// out[t][c] = sum_j w[t][j] * y[inv[t*top_k + j]][c] + shared[t][c], four columns per thread, sent to the rank that owns
// the columns (reduce-scatter part of this rank: rows of SH floats).  H % 4 == 0, SH % 4 == 0.
__global__ void __launch_bounds__(256) moe_combine_tp_kernel(const float *y, int ld_y, const int *inv, const float *pair_w,
                                                             int top_k, const float *shared, int H, int SH, Peers rs_dst,
                                                             long long total4, TpSignal sig) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total4; i += (long long)gridDim.x * blockDim.x) {
        const int h4 = H >> 2;
        const long long t = i / h4;
        const int c = (int)(i - t * h4) * 4;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int j = 0; j < top_k; ++j) {
            const int r = inv[t * top_k + j];
            if (r >= 0) {
                const float w = pair_w[t * top_k + j];
                const float4 q = *reinterpret_cast<const float4 *>(y + (long long)r * ld_y + c);
                acc.x = fmaf(w, q.x, acc.x); acc.y = fmaf(w, q.y, acc.y); acc.z = fmaf(w, q.z, acc.z); acc.w = fmaf(w, q.w, acc.w);
            }
        }
        if (shared) {
            const float4 q = *reinterpret_cast<const float4 *>(shared + t * H + c);
            acc.x += q.x; acc.y += q.y; acc.z += q.z; acc.w += q.w;
        }
        const int d = c / SH;
        char *dst = rs_dst.p[0];
#pragma unroll
        for (int r = 1; r < TP_MAX_RANKS; ++r)
            if (r == d) dst = rs_dst.p[r];
        *reinterpret_cast<float4 *>(dst + (t * SH + (c - d * SH)) * 4) = acc;
    }
    tp_signal(sig);
}

// ---- stand-alone collectives over the channel ------------------------------------------------------------------
// Push: rows of row_bytes bytes (a multiple of 16) from src (row stride src_stride bytes) to dst_d (row stride
// dst_stride) on every rank d; with scatter, rank d gets bytes [d * row_bytes, (d + 1) * row_bytes) of each source row.
__global__ void __launch_bounds__(256) tp_push_kernel(const char *src, long long src_stride, int rows, int row_bytes, Peers dst,
                                                      long long dst_stride, int ranks, int scatter, TpSignal sig) {
    const int per_row = row_bytes >> 4;
    const long long total = (long long)rows * per_row;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long m = i / per_row;
        const int c = (int)(i - m * per_row) * 16;
#pragma unroll
        for (int d = 0; d < TP_MAX_RANKS; ++d) {
            if (d >= ranks) continue;
            const uint4 v = *reinterpret_cast<const uint4 *>(src + m * src_stride + (scatter ? (long long)d * row_bytes : 0) + c);
            *reinterpret_cast<uint4 *>(dst.p[d] + m * dst_stride + c) = v;
        }
    }
    tp_signal(sig);
}

// Reduce: dst[i] = sum_r part_r[i] (fp32, rank order) once the collective has arrived.
__global__ void __launch_bounds__(256) tp_reduce_kernel(const float *parts, int nparts, long long part_stride, float *dst,
                                                        long long n, TpWait wait) {
    if (!tp_wait(wait)) return;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        float v = 0.f;
        for (int r = 0; r < nparts; ++r) v += __ldcg(parts + r * part_stride + i);
        dst[i] = v;
    }
}

// Waits for a collective whose payload later kernels of the stream read in place.
__global__ void tp_wait_kernel(TpWait wait) { tp_wait(wait); }

// rows [M][ld_src] fp32 (strided) -> dense [M][n] (staging of a strided source for tp_push).
__global__ void copy_rows_kernel(const float *src, long long ld_src, float *dst, int n, long long total) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long m = i / n;
    dst[i] = src[m * ld_src + (i - m * n)];
}


// X[rows_i[j]][s][:] = emb[j][col0 .. col0 + SH) for every stream s: rows whose embedding comes from the vision tower.
__global__ void embed_override_kernel(float *X, const int *rows_i, const float *emb, int ld_emb, int col0, int SH, int hc, long long total) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int c = (int)(i % SH);
    const long long js = i / SH;
    const int s = (int)(js % hc);
    const long long j = js / hc;
    X[((long long)rows_i[j] * hc + s) * SH + c] = emb[j * ld_emb + col0 + c];
}

// grid M, 256 threads: ssq[m] = sum over this rank's hc * SH values of row m.
__global__ void __launch_bounds__(256) mtp_ssq_kernel(const float *hidden, int n, float *ssq) {
    __shared__ float scratch[32];
    const float *x = hidden + (long long)blockIdx.x * n;
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += 256) ss = fmaf(x[i], x[i], ss);
    ss = block_sum<256>(ss, scratch);
    if (threadIdx.x == 0) ssq[blockIdx.x] = ss;
}

// grid M, 256 threads.  This rank's columns of the normalised hidden streams, hn[(m*hc + s)][col0 + c] =
// hidden[m][s][c] * rsqrt(ssq[m] / (hc*H) + eps) * nh1[s*H + col0 + c], go to every rank's [M*hc][H] bf16 matrix;
// en[m][:] = gemma_norm(embed[token m]) (whole rows, local).  SH % 8 == 0.
__global__ void __launch_bounds__(256) mtp_norm_tp_kernel(const float *hidden, const float *ssq, const int *tokens, const bf16 *embed,
                                                          int vocab, const float *nh1, const float *ne1, int H, int SH, int hc,
                                                          int col0, float eps, Peers hn_dst, int ranks, bf16 *en, TpSignal sig) {
    __shared__ float scratch[32];
    const int m = blockIdx.x;
    const float r = rsqrtf(ssq[m] / float(hc * H) + eps);
    const float *x = hidden + (long long)m * hc * SH;
    const int per = SH >> 3;
    for (int i = threadIdx.x; i < hc * per; i += 256) {
        const int s = i / per, c = (i - s * per) * 8;
        const float4 a = *reinterpret_cast<const float4 *>(x + s * SH + c), b = *reinterpret_cast<const float4 *>(x + s * SH + c + 4);
        const float *w = nh1 + (long long)s * H + col0 + c;
        const uint4 pk = make_uint4(pack_bf16(a.x * r * w[0], a.y * r * w[1]), pack_bf16(a.z * r * w[2], a.w * r * w[3]),
                                    pack_bf16(b.x * r * w[4], b.y * r * w[5]), pack_bf16(b.z * r * w[6], b.w * r * w[7]));
        const long long off = (((long long)m * hc + s) * H + col0 + c) * 2;
#pragma unroll
        for (int d = 0; d < TP_MAX_RANKS; ++d)
            if (d < ranks) *reinterpret_cast<uint4 *>(hn_dst.p[d] + off) = pk;
    }
    int t = tokens[m];
    if (t < 0 || t >= vocab) t = 0;
    const bf16 *e = embed + (long long)t * H;
    float es = 0.f;
    for (int i = threadIdx.x; i < H; i += 256) {
        const float v = __bfloat162float(e[i]);
        es = fmaf(v, v, es);
    }
    es = block_sum<256>(es, scratch);
    const float re = rsqrtf(es / float(H) + eps);
    for (int i = threadIdx.x; i < H; i += 256) en[(long long)m * H + i] = __float2bfloat16(__bfloat162float(e[i]) * re * ne1[i]);
    tp_signal(sig);
}

// Vocabulary-parallel argmax over the channel: every rank contributes {value, index, 0, 0} per row.
__global__ void amax_pack16_kernel(const float *val, const int *idx, float4 *out, int M) {
    const int m = blockIdx.x * blockDim.x + threadIdx.x;
    if (m < M) out[m] = make_float4(val[m], __int_as_float(idx[m]), 0.f, 0.f);
}
__global__ void amax_merge16_kernel(const float4 *gathered, int M, int ranks, int *out_idx, float *out_val, TpWait wait) {
    if (!tp_wait(wait)) return;
    const int m = blockIdx.x * blockDim.x + threadIdx.x;
    if (m >= M) return;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int r = 0; r < ranks; ++r) {
        const float4 p = __ldcg(gathered + (long long)m * ranks + r);
        const int i = __float_as_int(p.y);
        if (p.x > bv || (p.x == bv && i < bi)) { bv = p.x; bi = i; }
    }
    out_idx[m] = bi;
    if (out_val) out_val[m] = bv;
}

}  // namespace qw

using namespace qw;

static inline unsigned blocks_for(long long n, int per) { return (unsigned)((n + per - 1) / per); }
// A grid of at most TP_CTAS_PER_SM CTAs per SM for `n` work items of `per` per CTA pass.
static inline unsigned fat_grid(long long n, int per) {
    const long long want = (n + per - 1) / per, cap = (long long)TP_CTAS_PER_SM * NUM_SMS;
    return (unsigned)(want < 1 ? 1 : want < cap ? want : cap);
}
static bool tp_ok(const QwTp *tp) { return tp && tp->ranks >= 1 && tp->ranks <= TP_MAX_RANKS && tp->rank >= 0 && tp->rank < tp->ranks; }

// Mixer step 1.  pend: null, a local [T][ld_pend] matrix (pend_kind < 0), or the reduce-scatter parts of kind pend_kind
// (rows of SH floats) in this rank's receive buffer.  Sends the rows' sums of squares (kind 0) to every rank.
QW_API int qwk_hc_prenorm_tp(void *tp_, float *X, const float *pend_local, int ld_pend, int pend_kind, const float *inj, int SH,
                             int hc, int T, cudaStream_t s) {
    QwTp *tp = (QwTp *)tp_;
    if (!tp_ok(tp) || SH > 4096 || (SH & 3) || (ld_pend & 3)) return -1;
    if ((long long)T * hc * 4 > tp->part_bytes[0]) return -1;
    const float *pend = pend_local;
    int nparts = pend_local ? 1 : 0;
    long long stride = 0;
    TpWait w{};
    if (pend_kind >= 0) {
        pend = (const float *)tp_parts(tp, pend_kind);
        nparts = tp->ranks;
        stride = tp->part_bytes[pend_kind] >> 2;
        ld_pend = SH;
        w = tp_make_wait(tp, pend_kind);
    }
    Peers dst{};
    for (int d = 0; d < tp->ranks; ++d) dst.p[d] = tp_part_on(tp, 0, d);
    const long long items = (long long)T * hc;
    int per = (int)((items + (long long)TP_CTAS_PER_SM * NUM_SMS - 1) / ((long long)TP_CTAS_PER_SM * NUM_SMS));
    if (per < 1) per = 1;
    if (per > TP_PRENORM_ITEMS) per = TP_PRENORM_ITEMS;          // more rows than that: more CTAs, each still with one fence
    const unsigned grid = blocks_for(items, per);
    const TpSignal sig = tp_make_signal(tp, 0, grid);
    hc_prenorm_tp_kernel<<<grid, 256, 0, s>>>(X, pend, nparts, stride, ld_pend, inj, SH, hc, items, per, w, dst, tp->ranks, sig);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// Mixer step 2: xn from X and the sums of squares of all ranks (kind 0).
QW_API int qwk_hc_norm_tp(void *tp_, const float *X, const float *w1, int SH, int hc, int H, float eps, void *xn, int T,
                          cudaStream_t s) {
    QwTp *tp = (QwTp *)tp_;
    if (!tp_ok(tp) || (SH & 3)) return -1;
    const long long items = (long long)T * hc;
    hc_norm_tp_kernel<<<fat_grid(items, 8), 256, 0, s>>>(X, (const float *)tp_parts(tp, 0), tp->ranks, tp->part_bytes[0] >> 2, w1, SH, hc,
                                                         H, eps, (bf16 *)xn, items, tp_make_wait(tp, 0));
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// Mixer step 4: the ranks' partial down projections (kind 1, rows of ld_d floats) -> u, inj.
QW_API int qwk_hc_mid_tp(void *tp_, int ld_d, int R, int n_inj, int hc, void *u, float *inj, int T, cudaStream_t s) {
    QwTp *tp = (QwTp *)tp_;
    if (!tp_ok(tp)) return -1;
    const long long total = (long long)T * (R + n_inj);
    hc_mid_tp_kernel<<<fat_grid(total, 256), 256, 0, s>>>((const float *)tp_parts(tp, 1), tp->ranks, tp->part_bytes[1] >> 2, ld_d, R,
                                                            n_inj, hc, (bf16 *)u, inj, total, tp_make_wait(tp, 1));
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// Mixer step 6: this rank's columns of the block input -> the block-input matrix (kind 2, [T][ld_bin] bf16) of every rank.
QW_API int qwk_hc_mix_tp(void *tp_, const float *g, const void *xn, int SH, int ld_bin, int T, cudaStream_t s) {
    QwTp *tp = (QwTp *)tp_;
    if (!tp_ok(tp) || (SH & 7) || (ld_bin & 7)) return -1;
    if ((long long)T * ld_bin * 2 > tp->part_bytes[2]) return -1;
    Peers dst{};
    for (int d = 0; d < tp->ranks; ++d) dst.p[d] = (char *)tp->peer[d] + tp->off_buf[2];
    const long long total8 = (long long)T * (SH >> 3);
    const unsigned grid = fat_grid(total8, 256);
    const TpSignal sig = tp_make_signal(tp, 2, grid);
    hc_mix_tp_kernel<<<grid, 256, 0, s>>>(g, (const bf16 *)xn, SH, dst, tp->ranks, ld_bin, tp->rank * SH, total8, sig);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// MoE combine whose output goes to the owners of its columns (reduce-scatter, kind 3).
QW_API int qwk_moe_combine_tp(void *tp_, const float *y, int ld_y, const int *inv, const float *pair_w, int top_k,
                              const float *shared, int H, int T, cudaStream_t s) {
    QwTp *tp = (QwTp *)tp_;
    if (!tp_ok(tp) || (H & 3) || H % tp->ranks) return -1;
    const int SH = H / tp->ranks;
    if ((SH & 3) || (long long)T * SH * 4 > tp->part_bytes[3]) return -1;
    Peers dst{};
    for (int d = 0; d < tp->ranks; ++d) dst.p[d] = tp_part_on(tp, 3, d);
    const long long total4 = (long long)T * (H >> 2);
    const unsigned grid = fat_grid(total4, 256);
    const TpSignal sig = tp_make_signal(tp, 3, grid);
    moe_combine_tp_kernel<<<grid, 256, 0, s>>>(y, ld_y, inv, pair_w, top_k, shared, H, SH, dst, total4, sig);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

static unsigned push_grid(long long rows, int row_bytes) {
    const long long pieces = rows * (row_bytes >> 4);
    long long g = (pieces + 1023) / 1024;          // four pieces per thread
    if (g < 1) g = 1;
    if (g > 4 * NUM_SMS) g = 4 * NUM_SMS;
    return (unsigned)g;
}

// The sending half of a stand-alone collective: rows of row_bytes bytes (a multiple of 16; source row stride src_stride).
//   mode 0: the rows become this rank's part on every rank (all-reduce / all-gather by parts);
//   mode 1: source rows hold ranks * row_bytes bytes and rank d gets bytes [d * row_bytes, (d + 1) * row_bytes) as this
//           rank's part (reduce-scatter);
//   mode 2: the rows land at byte column rank * row_bytes of the matrix [rows][ranks * row_bytes] at the start of every
//           rank's buffer (all-gather into one matrix).
// The receiving half is qwk_tp_reduce, qwk_tp_wait or any kernel that waits for the kind.
QW_API int qwk_tp_push(void *tp_, int kind, const void *src, long long src_stride, int rows, int row_bytes, int mode,
                       cudaStream_t s) {
    QwTp *tp = (QwTp *)tp_;
    if (!tp_ok(tp) || kind < 0 || kind >= TP_KINDS || mode < 0 || mode > 2) return -1;
    if ((row_bytes & 15) || (src_stride & 15) || ((uintptr_t)src & 15) || rows < 1) return -1;
    const bool whole = kind == 2 || kind == 5;          // kinds whose buffer is one matrix, not one part per source
    Peers p{};
    long long dst_stride = row_bytes;
    if (mode == 2) {
        dst_stride = (long long)tp->ranks * row_bytes;
        if (rows * dst_stride > tp->part_bytes[kind] * (whole ? 1 : tp->ranks)) return -1;
        for (int d = 0; d < tp->ranks; ++d) p.p[d] = (char *)tp->peer[d] + tp->off_buf[kind] + (long long)tp->rank * row_bytes;
    } else {
        if (whole || (long long)rows * row_bytes > tp->part_bytes[kind]) return -1;
        for (int d = 0; d < tp->ranks; ++d) p.p[d] = tp_part_on(tp, kind, d);
    }
    const unsigned grid = push_grid(rows, row_bytes);
    const TpSignal sig = tp_make_signal(tp, kind, grid);
    tp_push_kernel<<<grid, 256, 0, s>>>((const char *)src, src_stride, rows, row_bytes, p, dst_stride, tp->ranks, mode == 1, sig);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// Stand-alone all-reduce (fp32, sum in rank order): src [rows][n] -> dst [rows][n] on every rank.  n % 4 == 0.
QW_API int qwk_tp_allreduce(void *tp_, int kind, const float *src, float *dst, int rows, int n, cudaStream_t s) {
    const int rc = qwk_tp_push(tp_, kind, src, (long long)n * 4, rows, n * 4, 0, s);
    return rc ? rc : qwk_tp_reduce(tp_, kind, dst, (long long)rows * n, s);
}

// Stand-alone reduce-scatter: src [rows][ranks * n] fp32 -> dst [rows][n] = sum over ranks of their columns [rank*n, rank*n+n).
QW_API int qwk_tp_reduce_scatter(void *tp_, int kind, const float *src, float *dst, int rows, int n, cudaStream_t s) {
    QwTp *tp = (QwTp *)tp_;
    if (!tp_ok(tp)) return -1;
    const int rc = qwk_tp_push(tp_, kind, src, (long long)tp->ranks * n * 4, rows, n * 4, 1, s);
    return rc ? rc : qwk_tp_reduce(tp_, kind, dst, (long long)rows * n, s);
}

// Stand-alone all-gather into the matrix [rows][ranks * row_bytes] at the start of every rank's buffer of `kind`; with
// wait != 0 a one-block kernel then waits for all ranks, so later kernels of the stream may read the matrix.
QW_API int qwk_tp_allgather(void *tp_, int kind, const void *src, long long src_stride, int rows, int row_bytes, int wait,
                            cudaStream_t s) {
    const int rc = qwk_tp_push(tp_, kind, src, src_stride, rows, row_bytes, 2, s);
    if (rc || !wait) return rc;
    return qwk_tp_wait(tp_, kind, s);
}

// One-block kernel that waits for the latest collective of `kind` (test vehicle for the bounded wait, too).
QW_API int qwk_tp_wait(void *tp_, int kind, cudaStream_t s) {
    QwTp *tp = (QwTp *)tp_;
    if (!tp_ok(tp) || kind < 0 || kind >= TP_KINDS) return -1;
    tp_wait_kernel<<<1, 32, 0, s>>>(tp_make_wait(tp, kind));
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// Reduces the latest collective of `kind` (parts of n floats) into dst.
QW_API int qwk_tp_reduce(void *tp_, int kind, float *dst, long long n, cudaStream_t s) {
    QwTp *tp = (QwTp *)tp_;
    if (!tp_ok(tp) || kind < 0 || kind >= TP_KINDS || n * 4 > tp->part_bytes[kind]) return -1;
    unsigned rg = blocks_for(n, 1024);
    if (rg > 4 * NUM_SMS) rg = 4 * NUM_SMS;
    tp_reduce_kernel<<<rg, 256, 0, s>>>((const float *)tp_parts(tp, kind), tp->ranks, tp->part_bytes[kind] >> 2, dst, n,
                                        tp_make_wait(tp, kind));
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

QW_API int qwk_copy_rows(const float *src, long long ld_src, float *dst, int n, int M, cudaStream_t s) {
    const long long total = (long long)M * n;
    copy_rows_kernel<<<blocks_for(total, 256), 256, 0, s>>>(src, ld_src, dst, n, total);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

QW_API int qwk_embed_override(float *X, const int *rows_i, const float *emb, int ld_emb, int col0, int SH, int hc, int n,
                              cudaStream_t s) {
    if (n <= 0) return 0;
    const long long total = (long long)n * hc * SH;
    embed_override_kernel<<<blocks_for(total, 256), 256, 0, s>>>(X, rows_i, emb, ld_emb, col0, SH, hc, total);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

QW_API int qwk_mtp_ssq(const float *hidden, int n, float *ssq, int M, cudaStream_t s) {
    mtp_ssq_kernel<<<M, 256, 0, s>>>(hidden, n, ssq);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// MTP input norm on several ranks: hidden [M][hc][SH] (this rank's columns), ssq [M] summed over all ranks.  The
// normalised streams are gathered into the [M*hc][H] bf16 matrix at the start of every rank's kind-5 buffer.
QW_API int qwk_mtp_norm_tp(void *tp_, const float *hidden, const float *ssq, const int *tokens, const void *embed, int vocab,
                           const float *nh1, const float *ne1, int H, int hc, float eps, void *en, int M, cudaStream_t s) {
    QwTp *tp = (QwTp *)tp_;
    if (!tp_ok(tp) || H % tp->ranks) return -1;
    const int SH = H / tp->ranks;
    if ((SH & 7) || (long long)M * hc * H * 2 > tp->part_bytes[5]) return -1;
    Peers dst{};
    for (int d = 0; d < tp->ranks; ++d) dst.p[d] = (char *)tp->peer[d] + tp->off_buf[5];
    const TpSignal sig = tp_make_signal(tp, 5, (unsigned)M);
    mtp_norm_tp_kernel<<<M, 256, 0, s>>>(hidden, ssq, tokens, (const bf16 *)embed, vocab, nh1, ne1, H, SH, hc, tp->rank * SH, eps, dst,
                                         tp->ranks, (bf16 *)en, sig);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// Argmax over the vocabulary shards of all ranks (ties to the lowest index), in two halves over the kind-4 buffer:
// send packs this rank's val / idx [M] into scratch16 ([M] float4 of local scratch) and gathers the packs on every rank;
// merge waits for all ranks' packs and picks.
QW_API int qwk_tp_argmax_send(void *tp_, const float *val, const int *idx, void *scratch16, int M, cudaStream_t s) {
    QwTp *tp = (QwTp *)tp_;
    if (!tp_ok(tp)) return -1;
    amax_pack16_kernel<<<blocks_for(M, 64), 64, 0, s>>>(val, idx, (float4 *)scratch16, M);
    return qwk_tp_push(tp_, 4, scratch16, 16, M, 16, 2, s);
}
QW_API int qwk_tp_argmax_merge(void *tp_, int M, int *out_idx, float *out_val, cudaStream_t s) {
    QwTp *tp = (QwTp *)tp_;
    if (!tp_ok(tp) || M > 256) return -1;
    amax_merge16_kernel<<<1, 256, 0, s>>>((const float4 *)tp_parts(tp, 4), M, tp->ranks, out_idx, out_val, tp_make_wait(tp, 4));
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
