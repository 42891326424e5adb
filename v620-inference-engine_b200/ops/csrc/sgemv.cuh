// Streaming bf16 matrix-vector product: y[m][n] = sum_k W[n][k] x[m][k], M <= 32 rows.
//
// One persistent block per SM.  Weight rows travel global -> shared memory as bulk-async copies
// (8 rows, or 4 long rows, per stage; 2-6 stages in flight) that one thread issues; the first
// stages are issued before the kernel waits for its predecessor (programmatic dependent launch),
// so they overlap the predecessor's tail.  The x rows are staged in shared memory once per tile of
// 8 rows.  Each warp owns one weight row of a stage (two warps share a long row), reads it and x
// with conflict-free 16-byte loads and accumulates in fp32 in a fixed order, so a row's result does
// not depend on how many other rows share the step.
#pragma once
#include "stream.cuh"

namespace qw {

struct SGemvArgs {
    const bf16 *W;      // [N][ldw]
    const bf16 *x;      // [M][ldx]
    float *y;           // [M][ldy]
    bf16 *y_bf16;       // optional bf16 copy of y
    int N, K, M;
    int ldw, ldx, ldy;
    int accumulate;
    int wpr;            // warps per weight row: 1 or 2
    int nstage;
    ErrorWord *err;
};

constexpr int SG_HDR = 512;     // mbarriers + partial sums

template <int MT>
__device__ __forceinline__ void sgemv_body(const SGemvArgs &a, unsigned char *smem) {
    uint64_t *bar = reinterpret_cast<uint64_t *>(smem);
    float(*part)[8] = reinterpret_cast<float(*)[8]>(smem + 128);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int srows = 8 / a.wpr;                           // weight rows per stage
    const unsigned Kb = (unsigned)a.K * 2u;
    const unsigned stage_bytes = (unsigned)srows * Kb;
    unsigned char *stages = smem + SG_HDR;
    unsigned char *xs = stages + (size_t)a.nstage * stage_bytes;
    const int nitems = (a.N + srows - 1) / srows;
    const int cnt = blockIdx.x < nitems ? (nitems - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
    const int mtiles = (a.M + MT - 1) / MT;
    const int total = cnt * mtiles;
    if (tid == 0) {
        for (int s = 0; s < a.nstage; ++s) mbar_init(bar + s, 1);
        mbar_fence_init();
    }
    __syncthreads();
    auto issue = [&](int qi) {
        const int i = qi % cnt;
        const int row0 = ((int)blockIdx.x + i * (int)gridDim.x) * srows;
        const int rows = min(srows, a.N - row0);
        const int s = qi % a.nstage;
        unsigned char *dst = stages + (size_t)s * stage_bytes;
        mbar_expect_tx(bar + s, (unsigned)rows * Kb);
        if (a.ldw == a.K) {
            bulk_g2s(dst, a.W + (long long)row0 * a.ldw, (unsigned)rows * Kb, bar + s);
        } else {
            for (int r = 0; r < rows; ++r) bulk_g2s(dst + (size_t)r * Kb, a.W + (long long)(row0 + r) * a.ldw, Kb, bar + s);
        }
    };
    if (tid == 0)
        for (int qi = 0; qi < a.nstage && qi < total; ++qi) issue(qi);
    pdl_wait();
    pdl_trigger();
    const int nchunk = a.K >> 3;
    const int half = a.wpr == 2 ? (warp & 1) : 0;
    const int c_begin = a.wpr == 2 ? half * ((nchunk + 1) / 2) : 0;
    const int c_end = a.wpr == 2 ? (half ? nchunk : (nchunk + 1) / 2) : nchunk;
    const int srow = a.wpr == 2 ? (warp >> 1) : warp;
    bool ok = true;
    for (int tile = 0; tile < mtiles && ok; ++tile) {
        const int m0 = tile * MT;
        const int nm = min(MT, a.M - m0);
        for (int i = tid; i < nm * nchunk; i += 256) {
            const int m = i / nchunk, c = i - m * nchunk;
            reinterpret_cast<uint4 *>(xs + (size_t)m * Kb)[c] =
                __ldg(reinterpret_cast<const uint4 *>(a.x + (long long)(m0 + m) * a.ldx) + c);
        }
        __syncthreads();
        for (int i = 0; i < cnt; ++i) {
            const int qi = tile * cnt + i;
            const int s = qi % a.nstage;
            ok = mbar_wait(bar + s, (unsigned)(qi / a.nstage) & 1u, a.err);
            if (!ok) break;
            const int row = ((int)blockIdx.x + i * (int)gridDim.x) * srows + srow;
            float acc[MT];
#pragma unroll
            for (int m = 0; m < MT; ++m) acc[m] = 0.f;
            if (row < a.N) {
                const uint4 *wp = reinterpret_cast<const uint4 *>(stages + (size_t)s * stage_bytes + (size_t)srow * Kb);
#pragma unroll 2
                for (int c = c_begin + lane; c < c_end; c += 32) {
                    const uint4 w = wp[c];
#pragma unroll
                    for (int m = 0; m < MT; ++m)
                        if (m < nm) acc[m] = dot8(w, reinterpret_cast<const uint4 *>(xs + (size_t)m * Kb)[c], acc[m]);
                }
            }
#pragma unroll
            for (int m = 0; m < MT; ++m) acc[m] = warp_sum(acc[m]);
            if (a.wpr == 2 && half == 1 && lane == 0) {
#pragma unroll
                for (int m = 0; m < MT; ++m) part[warp][m] = acc[m];
            }
            __syncthreads();                 // stage consumed (and partial sums visible)
            if (tid == 0 && qi + a.nstage < total) issue(qi + a.nstage);
            if (half == 0 && lane == 0 && row < a.N) {
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    if (m < nm) {
                        float v = acc[m];
                        if (a.wpr == 2) v += part[warp + 1][m];
                        const long long o = (long long)(m0 + m) * a.ldy + row;
                        if (a.accumulate) v += a.y[o];
                        a.y[o] = v;
                        if (a.y_bf16) a.y_bf16[o] = __float2bfloat16(v);
                    }
                }
            }
            if (a.wpr == 2) __syncthreads();  // partial sums read before the next stage overwrites them
        }
    }
    if (!ok && tid == 0) {
        // give copies still in flight a last bounded chance to land before the block exits
        for (int s = 0; s < a.nstage; ++s) mbar_wait(bar + s, 0, nullptr, 1u << 12), mbar_wait(bar + s, 1, nullptr, 1u << 12);
    }
}

// Picks warps-per-row and the pipeline depth; returns the dynamic shared memory size.
static inline size_t sgemv_plan(SGemvArgs &a, int MT, int &grid) {
    const size_t Kb = (size_t)a.K * 2;
    a.wpr = Kb > 8192 ? 2 : 1;
    const size_t stage = (size_t)(8 / a.wpr) * Kb;
    const size_t xbytes = (size_t)MT * Kb;
    const size_t budget = 100 * 1024;                 // leaves room for the successor's block on the same SM
    long long ns = ((long long)budget - SG_HDR - (long long)xbytes) / (long long)stage;
    if (ns < 2) ns = 2;
    if (ns > 6) ns = 6;
    a.nstage = (int)ns;
    const int nitems = (a.N + 8 / a.wpr - 1) / (8 / a.wpr);
    grid = nitems < NUM_SMS ? nitems : NUM_SMS;
    return SG_HDR + (size_t)a.nstage * stage + xbytes;
}

}  // namespace qw
