// PLE (per-layer n-gram embedding) kernels for row batches: device-side n-gram hashing and the
// 16-row gather straight out of the host-resident table (pinned, mapped memory), the gate
// statistics, the gated value / normalised conv input, the dilated causal conv and its ring
// (roles of the reference's src/core/ple.cpp:86-125,184-211 on the host and
// src/kernels/ple.hip:8-215 on the device; math in docs/MODEL.md:185-219).
#include "common.cuh"

namespace qw {

constexpr int MAX_NGRAM_HEADS = 32;

struct NgramConst {
    unsigned long long mult[4];
    unsigned long long sizes[MAX_NGRAM_HEADS];
    long long offsets[MAX_NGRAM_HEADS];
    int ngram, heads, eos;
};
__constant__ NgramConst c_ng;
__constant__ float c_f8_lut[256];

enum PleLayout { PLE_F8 = 0, PLE_BF16 = 1, PLE_INT8 = 2, PLE_INT4 = 3 };

struct PleGatherArgs {
    const int *ctx;              // [M][3]: token at the row's position, the one before, two before (-1 = none)
    const void *const *shards;   // per shard: value rows
    const void *const *scales;   // per shard: fp16 scales (int8 / int4 layouts)
    long long rows_per_shard, rows;
    int layout, width;
    bf16 *e;                     // [M][heads*width]
    long long *ids_out;          // optional [M][heads]
};

// grid (M, heads), 64 threads.
__global__ void ple_gather_kernel(PleGatherArgs a) {
    const int m = blockIdx.x, h = blockIdx.y;
    const int eos = c_ng.eos;
    const int t0 = a.ctx[m * 3], c1 = a.ctx[m * 3 + 1], c2 = a.ctx[m * 3 + 2];
    const unsigned long long tok0 = (unsigned long long)t0;
    const int t1 = c1 >= 0 ? c1 : eos;
    const int t2 = (c2 >= 0 && t1 != eos) ? c2 : eos;
    const int per = c_ng.heads / (c_ng.ngram - 1);
    const int order = 2 + h / per;
    unsigned long long mixed = tok0 * c_ng.mult[0] ^ (unsigned long long)t1 * c_ng.mult[1];
    if (order >= 3) mixed ^= (unsigned long long)t2 * c_ng.mult[2];
    long long id = (long long)(mixed % c_ng.sizes[h]) + c_ng.offsets[h];
    id %= a.rows;                                   // scaled-down synthetic tables wrap
    if (a.ids_out && threadIdx.x == 0) a.ids_out[m * c_ng.heads + h] = id;
    const long long sh = id / a.rows_per_shard, r = id % a.rows_per_shard;
    bf16 *out = a.e + ((long long)m * c_ng.heads + h) * a.width;
    const int W = a.width;
    if (a.layout == PLE_F8) {
        const unsigned char *row = (const unsigned char *)a.shards[sh] + r * W;
        for (int j = threadIdx.x; j < W; j += blockDim.x) out[j] = __float2bfloat16(c_f8_lut[row[j]]);
    } else if (a.layout == PLE_BF16) {
        const bf16 *row = (const bf16 *)a.shards[sh] + r * W;
        for (int j = threadIdx.x; j < W; j += blockDim.x) out[j] = row[j];
    } else if (a.layout == PLE_INT8) {
        const signed char *row = (const signed char *)a.shards[sh] + r * W;
        const __half *sc = (const __half *)a.scales[sh] + r * (W / 16);
        for (int j = threadIdx.x; j < W; j += blockDim.x) out[j] = __float2bfloat16(float(row[j]) * __half2float(sc[j / 16]));
    } else {
        const unsigned char *row = (const unsigned char *)a.shards[sh] + r * (W / 2);
        const __half *sc = (const __half *)a.scales[sh] + r * (W / 16);
        for (int j = threadIdx.x; j < W; j += blockDim.x) {
            const unsigned char b = row[j >> 1];
            const int q = (j & 1) ? (b >> 4) : (b & 0xf);
            out[j] = __float2bfloat16(float(q - 8) * __half2float(sc[j / 16]));
        }
    }
}

// grid (M, hc), 256 threads.  kv[m] = [ key (hc x SH) | value (SH) ] fp32.
// send[m][3s..3s+2] = sum k^2, sum x^2, sum k(1+wk) x(1+wq); send[m][3*hc] = sum v^2.
__global__ void __launch_bounds__(256) ple_stats_kernel(const float *kv, int ld_kv, const float *X, const float *nk1,
                                                        const float *nq1, int SH, int hc, float *send, int ld_send) {
    __shared__ float scratch[32];
    const int m = blockIdx.x, s = blockIdx.y;
    const float *k = kv + (long long)m * ld_kv + s * SH;
    const float *x = X + ((long long)m * hc + s) * SH;
    float kk = 0.f, xx = 0.f, kx = 0.f, vv = 0.f;
    for (int c = threadIdx.x; c < SH; c += 256) {
        const float kc = k[c], xc = x[c];
        kk = fmaf(kc, kc, kk);
        xx = fmaf(xc, xc, xx);
        kx = fmaf(kc * nk1[s * SH + c], xc * nq1[s * SH + c], kx);
        if (s == 0) {
            const float v = kv[(long long)m * ld_kv + hc * SH + c];
            vv = fmaf(v, v, vv);
        }
    }
    kk = block_sum<256>(kk, scratch);
    xx = block_sum<256>(xx, scratch);
    kx = block_sum<256>(kx, scratch);
    if (s == 0) vv = block_sum<256>(vv, scratch);
    if (threadIdx.x == 0) {
        float *o = send + (long long)m * ld_send;
        o[3 * s] = kk; o[3 * s + 1] = xx; o[3 * s + 2] = kx;
        if (s == 0) o[3 * hc] = vv;
    }
}

// grid (M, hc): gate, gated value gv and normalised conv input nc for the batch rows.
__global__ void __launch_bounds__(256) ple_nc_kernel(const float *kv, int ld_kv, const float *red, int ld_red,
                                                     const float *nc1, int SH, int hc, int H, float eps, float *gv,
                                                     float *nc) {
    const int m = blockIdx.x, s = blockIdx.y;
    const float *r = red + (long long)m * ld_red;
    const float rk = rsqrtf(r[3 * s] / float(H) + eps), rq = rsqrtf(r[3 * s + 1] / float(H) + eps);
    const float gs = r[3 * s + 2] * rk * rq * rsqrtf(float(H));
    const float mag = sqrtf(fmaxf(fabsf(gs), 1e-6f));
    const float gate = sigmoidf_(gs < 0.f ? -mag : (gs > 0.f ? mag : 0.f));
    const float rn = rsqrtf(gate * gate * r[3 * hc] / float(H) + eps);
    const float *v = kv + (long long)m * ld_kv + hc * SH;
    for (int c = threadIdx.x; c < SH; c += 256) {
        const float g = gate * v[c];
        const long long o = ((long long)m * hc + s) * SH + c;
        gv[o] = g;
        nc[o] = g * rn * nc1[s * SH + c];
    }
}

// grid (M, hc): X += gv + silu(dilated conv of nc); taps at p-9, p-6, p-3, p from the batch or the ring.
__global__ void __launch_bounds__(256) ple_conv_kernel(const float *gv, const float *nc, const float *ring, const float *cw,
                                                       int SH, int hc, int taps, int dil, Rows rows, float *X) {
    const int m = blockIdx.x, s = blockIdx.y;
    const int slot = rows.slot[m], pos = rows.pos[m], rs = rows.run_start[m];
    const int xw = hc * SH;
    const float *rg = ring + (long long)slot * PLE_RING * xw;
    for (int c = threadIdx.x; c < SH; c += 256) {
        const int col = s * SH + c;
        float acc = 0.f;
        for (int k = 0; k < taps; ++k) {
            const int back = (taps - 1 - k) * dil;
            const int q = pos - back;
            float v;
            if (m - back >= rs) v = nc[(long long)(m - back) * xw + col];
            else if (q >= 0) v = rg[(q % PLE_RING) * xw + col];
            else v = 0.f;
            acc = fmaf(cw[col * taps + k], v, acc);
        }
        X[(long long)m * xw + col] += gv[(long long)m * xw + col] + siluf_(acc);
    }
}

// grid (M, ceil(xw/256)): store the batch's nc rows in the ring (after ple_conv has read it).
__global__ void ple_ring_kernel(const float *nc, float *ring, int xw, Rows rows) {
    const int m = blockIdx.x, col = blockIdx.y * 256 + threadIdx.x;
    if (col >= xw) return;
    const int rs = rows.run_start[m], len = rows.run_len[rs];
    if ((m - rs) < len - PLE_RING) return;
    ring[((long long)rows.slot[m] * PLE_RING + (rows.pos[m] % PLE_RING)) * xw + col] = nc[(long long)m * xw + col];
}

}  // namespace qw

using namespace qw;

QW_API int qwk_ple_init(const unsigned long long *mult, int ngram, const unsigned long long *sizes,
                        const long long *offsets, int heads, int eos, const float *f8_lut) {
    if (heads > MAX_NGRAM_HEADS || ngram > 4 || ngram < 2) return -1;
    NgramConst c;
    for (int i = 0; i < ngram; ++i) c.mult[i] = mult[i];
    for (int i = 0; i < heads; ++i) { c.sizes[i] = sizes[i]; c.offsets[i] = offsets[i]; }
    c.ngram = ngram; c.heads = heads; c.eos = eos;
    if (cudaMemcpyToSymbol(c_ng, &c, sizeof(c)) != cudaSuccess) return -2;
    if (f8_lut && cudaMemcpyToSymbol(c_f8_lut, f8_lut, 256 * sizeof(float)) != cudaSuccess) return -2;
    return 0;
}

QW_API int qwk_ple_gather(const int *ctx, const void *const *shards, const void *const *scales, long long rows_per_shard,
                          long long rows, int layout, int width, int heads, void *e, long long *ids_out, int M,
                          cudaStream_t s) {
    PleGatherArgs a;
    a.ctx = ctx; a.shards = shards; a.scales = scales; a.rows_per_shard = rows_per_shard; a.rows = rows;
    a.layout = layout; a.width = width; a.e = (bf16 *)e; a.ids_out = ids_out;
    dim3 grid(M, heads);
    ple_gather_kernel<<<grid, 64, 0, s>>>(a);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

QW_API int qwk_ple_stats(const float *kv, int ld_kv, const float *X, const float *nk1, const float *nq1, int SH, int hc,
                         float *send, int ld_send, int M, cudaStream_t s) {
    dim3 grid(M, hc);
    ple_stats_kernel<<<grid, 256, 0, s>>>(kv, ld_kv, X, nk1, nq1, SH, hc, send, ld_send);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

QW_API int qwk_ple_apply(const float *kv, int ld_kv, const float *red, int ld_red, const float *nc1, const float *cw,
                         int SH, int hc, int H, float eps, int taps, int dil, float *gv, float *nc, float *ring,
                         float *X, int M, const int *slot, const int *pos, const int *run_start, const int *run_len,
                         cudaStream_t s) {
    dim3 grid(M, hc);
    Rows rows{M, slot, pos, run_start, run_len};
    ple_nc_kernel<<<grid, 256, 0, s>>>(kv, ld_kv, red, ld_red, nc1, SH, hc, H, eps, gv, nc);
    ple_conv_kernel<<<grid, 256, 0, s>>>(gv, nc, ring, cw, SH, hc, taps, dil, rows, X);
    dim3 g2(M, (hc * SH + 255) / 256);
    ple_ring_kernel<<<g2, 256, 0, s>>>(nc, ring, hc * SH, rows);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
