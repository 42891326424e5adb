// Persistent, L2-prefetching bf16 matrix-vector body shared by gemv.cu and moe.cu (see gemv.cu).
#pragma once
#include "common.cuh"

namespace qw {

struct GemvArgs {
    const bf16 *W;      // [N][ldw]
    const bf16 *x;      // [M][ldx]
    float *y;           // [M][ldy]
    int N, K, M;
    int ldw, ldx, ldy;
    int wpr;            // warps per row: 1, 2, 4 or 8
    int accumulate;     // y += instead of y =
    int nsplit;         // column splits: element offsets added per split
    long long w_split, x_split, y_split;
    bf16 *y_bf16;       // optional second output in bf16 (same indexing as y), may be null
    int prefetch_items; // items per block to prefetch into L2 before waiting for the predecessor
};

// L2 prefetch of `bytes` (multiple of 16) starting at a 16-byte aligned address.
__device__ __forceinline__ void l2_prefetch(const void *p, unsigned bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

// The whole GEMV as a device function, so kernels with an epilogue (router + top-k) can reuse it.
// `part` is an [8][MT] shared array.
template <int MT>
__device__ __forceinline__ void gemv_body(const GemvArgs &a, float (*part)[MT]) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int wpr = a.wpr;
    const int rpb = 8 / wpr;
    const int groups = (a.N + rpb - 1) / rpb;
    const int items = groups * a.nsplit;
    const int kw = warp % wpr;
    const int nchunk = a.K >> 3;
    const int stride = wpr * 32;
    // ---- before the predecessor has finished: warm the L2 with this block's first weight rows
    if (lane == 0) {
        const unsigned seg = (unsigned)(((nchunk + wpr - 1) / wpr) * 16);     // this warp's share of a row
        int it = blockIdx.x;
        for (int i = 0; i < a.prefetch_items && it < items; ++i, it += gridDim.x) {
            const int split = it / groups, row = (it % groups) * rpb + warp / wpr;
            if (row < a.N) {
                const char *base = reinterpret_cast<const char *>(a.W + split * a.w_split + (long long)row * a.ldw);
                const unsigned off = (unsigned)kw * seg;
                const unsigned total = (unsigned)nchunk * 16;
                if (off < total) l2_prefetch(base + off, min(seg, total - off));
            }
        }
    }
    pdl_wait();
    pdl_trigger();
    for (int it = blockIdx.x; it < items; it += gridDim.x) {
        const int split = it / groups;
        const int row = (it % groups) * rpb + warp / wpr;
        const bf16 *W = a.W + split * a.w_split;
        const bf16 *x = a.x + split * a.x_split;
        float *y = a.y + split * a.y_split;
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
                        if (a.y_bf16) (a.y_bf16 + split * a.y_split)[o] = __float2bfloat16(v);
                    }
                }
            }
        }
    }
}

static inline int pick_wpr(int N, int nsplit) {
    // enough (row, split) items to give every SM several blocks' worth of rows
    long long rows = (long long)N * nsplit;
    if (rows >= NUM_SMS * 4 * 8) return 1;
    if (rows >= NUM_SMS * 4 * 4) return 2;
    if (rows >= NUM_SMS * 4 * 2) return 4;
    return 8;
}

// Fills the launch-dependent fields of `a` (wpr, prefetch depth) and returns the grid size.
static inline int gemv_plan(GemvArgs &a) {
    a.wpr = pick_wpr(a.N, a.nsplit);
    const int rpb = 8 / a.wpr;
    const int items = ((a.N + rpb - 1) / rpb) * a.nsplit;
    const int grid = items < NUM_SMS * 4 ? items : NUM_SMS * 4;
    const long long item_bytes = (long long)rpb * a.K * 2;
    long long pf = (40ll << 20) / (item_bytes * grid);      // at most ~40 MB warmed ahead of the predecessor's end
    const int per_block = (items + grid - 1) / grid;
    a.prefetch_items = (int)(pf < 1 ? 1 : (pf > per_block ? per_block : pf));
    return grid;
}

}  // namespace qw
