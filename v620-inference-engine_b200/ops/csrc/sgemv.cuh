// Streaming bf16 matrix-vector product: y[m][n] = sum_k W[n][k] x[m][k], M <= 32 rows.
//
// One persistent block per SM.  Weight rows travel global -> shared memory as bulk-async copies
// (16 rows x up to 2.5 KB per stage, three stages in flight) that one thread issues; the first
// stages are issued before the kernel waits for its predecessor (programmatic dependent launch),
// so they overlap the predecessor's tail.  The 8 warps split a stage's k range and feed the tensor
// core (ldmatrix + m16n8k16, fp32 accumulate) with the activation rows as the narrow operand, so up
// to 16 activation rows cost the same instructions as one; partial sums of the warps are added in
// warp order, so a row's result does not depend on how many other rows share the step.
#pragma once
#include "mma.cuh"

namespace qw {

struct SGemvArgs {
    const bf16 *W;      // [N][ldw]
    const bf16 *x;      // [M][ldx]
    float *y;           // [M][ldy]
    bf16 *y_bf16;       // optional bf16 copy of y
    int N, K, M;
    int ldw, ldx, ldy;
    int accumulate;
    int P;              // k parts per row tile
    int TR;             // weight rows per tile: 16, or 8 for short matrices (finer tiles balance the SMs better)
    int nstage;
    ErrorWord *err;
    PfArgs pf;          // weights of later kernels to pull into L2
};

constexpr int SG_HDR = 128;              // mbarriers: full[8], empty[8]
constexpr int SG_THREADS = 288;          // 8 consumer warps + 1 producer warp
constexpr int SG_TILE = 16;              // weight rows per tile

// NT = activation-row tiles of 8 handled per pass (1 or 2).
template <int NT>
__device__ __forceinline__ void sgemv_body(const SGemvArgs &a, unsigned char *smem) {
    uint64_t *bar = reinterpret_cast<uint64_t *>(smem);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int Kc = a.K / a.P;
    const unsigned KcB = (unsigned)Kc * 2u, srow = KcB + ROW_PAD;          // stage row stride
    const int TR = a.TR;
    const unsigned stage_bytes = (unsigned)TR * srow;
    const unsigned xrow = (unsigned)a.K * 2u + ROW_PAD;
    unsigned char *stages = smem + SG_HDR;
    float *part = reinterpret_cast<float *>(stages + (size_t)a.nstage * stage_bytes);     // [2][8][NT][128]
    unsigned char *xs = reinterpret_cast<unsigned char *>(part + 2 * 8 * NT * 128);      // [(8*NT)+1][xrow]
    const int ntiles = (a.N + TR - 1) / TR;
    const int cnt = (int)blockIdx.x < ntiles ? (ntiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
    const int MT = 8 * NT;
    const int mtiles = (a.M + MT - 1) / MT;
    const int total = cnt * a.P * mtiles;
    uint64_t *full = bar, *empty = bar + 8;
    if (tid == 0) {
        for (int s = 0; s < a.nstage; ++s) {
            mbar_init(full + s, 1);
            mbar_init(empty + s, 8);          // one arrival per consumer warp
        }
        mbar_fence_init();
    }
    __syncthreads();
    if (warp == 8) {
        // ---- producer warp: lane r copies row r of each stage; runs ahead of the consumers, and does not
        // wait for the predecessor kernel because weights do not depend on it
        for (int q = 0; q < total; ++q) {
            const int s = q % a.nstage;
            if (q >= a.nstage && !mbar_wait(empty + s, (unsigned)(q / a.nstage - 1) & 1u, a.err)) break;
            const int kp = q % a.P, i = (q / a.P) % cnt;
            const int row0 = ((int)blockIdx.x + i * (int)gridDim.x) * TR;
            const int rows = min(TR, a.N - row0);
            unsigned char *dst = stages + (size_t)s * stage_bytes;
            if (lane == 0) mbar_expect_tx(full + s, (unsigned)rows * KcB);
            __syncwarp();
            if (lane < rows)
                bulk_g2s(dst + (size_t)lane * srow, a.W + (long long)(row0 + lane) * a.ldw + (long long)kp * Kc, KcB, full + s);
        }
        return;
    }
    pf_issue(a.pf);
    pdl_wait();
    pdl_trigger();
    const uint32_t xs_base = smem_u32(xs), st_base = smem_u32(stages);
    const int steps = Kc >> 4;
    bool ok = true;
    int q = 0;
    for (int tile = 0; tile < mtiles && ok; ++tile) {
        const int m0 = tile * MT;
        const int nm = min(MT, a.M - m0);
        const int nchunk = a.K >> 3;
        for (int i = tid; i < (nm + 1) * nchunk; i += 256) {      // activation rows + one zero row
            const int m = i / nchunk, c = i - m * nchunk;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (m < nm) v = __ldg(reinterpret_cast<const uint4 *>(a.x + (long long)(m0 + m) * a.ldx) + c);
            *reinterpret_cast<uint4 *>(xs + (size_t)m * xrow + (size_t)c * 16) = v;
        }
        consumer_sync(256);
        for (int i = 0; i < cnt && ok; ++i) {
            float c[NT][4];
#pragma unroll
            for (int t = 0; t < NT; ++t) c[t][0] = c[t][1] = c[t][2] = c[t][3] = 0.f;
            for (int kp = 0; kp < a.P; ++kp, ++q) {
                const int s = q % a.nstage;
                ok = mbar_wait(full + s, (unsigned)(q / a.nstage) & 1u, a.err);
                if (!ok) break;
                const uint32_t tb = st_base + (unsigned)s * stage_bytes;
                for (int st = warp; st < steps; st += 8) {
                    uint32_t a0, a1 = 0u, a2, a3 = 0u;
                    if (TR == 16) ldmatrix_x4(a0, a1, a2, a3, a_tile_addr(tb, srow, st << 4, lane));
                    else ldmatrix_x2(a0, a2, tb + (unsigned)(lane & 7) * srow + (unsigned)((st << 4) + (((lane >> 3) & 1) << 3)) * 2u);
#pragma unroll
                    for (int t = 0; t < NT; ++t) {
                        uint32_t b0, b1;
                        ldmatrix_x2(b0, b1, b_tile_addr(xs_base, xrow, t * 8, nm, nm, kp * Kc + (st << 4), lane));
                        mma_bf16(c[t], a0, a1, a2, a3, b0, b1);
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(empty + s);      // this warp is done with the stage
            }
            if (!ok) break;
            float *pp = part + ((size_t)(i & 1) * 8 + warp) * NT * 128;
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                const int r = lane >> 2, n = (lane & 3) * 2;
                pp[t * 128 + r * 8 + n] = c[t][0];
                pp[t * 128 + r * 8 + n + 1] = c[t][1];
                pp[t * 128 + (r + 8) * 8 + n] = c[t][2];
                pp[t * 128 + (r + 8) * 8 + n + 1] = c[t][3];
            }
            consumer_sync(256);                  // partial sums of all warps visible
            // sum the 8 warps' partials in warp order and store
            const int row0 = ((int)blockIdx.x + i * (int)gridDim.x) * TR;
            for (int e = tid; e < NT * 128; e += 256) {
                const int t = e >> 7, r = (e >> 3) & 15, n = e & 7;
                const int m = t * 8 + n;
                if (m < nm && r < TR && row0 + r < a.N) {
                    const float *ps = part + (size_t)(i & 1) * 8 * NT * 128 + e;
                    float v = 0.f;
#pragma unroll
                    for (int w = 0; w < 8; ++w) v += ps[(size_t)w * NT * 128];
                    const long long o = (long long)(m0 + m) * a.ldy + row0 + r;
                    if (a.accumulate) v += a.y[o];
                    a.y[o] = v;
                    if (a.y_bf16) a.y_bf16[o] = __float2bfloat16(v);
                }
            }
        }
        consumer_sync(256);          // xs is rewritten by the next activation tile
    }
}

// Picks the k partition and the pipeline depth; returns the dynamic shared memory size.
static inline size_t sgemv_plan(SGemvArgs &a, int NT, int &grid) {
    // shared memory holds only the activation rows that exist (plus the zero row)
    const size_t Kb = (size_t)a.K * 2;
    int P = (int)((Kb + 2559) / 2560);
    while (a.K % (16 * P)) ++P;
    a.P = P;
    a.TR = (a.N + 15) / 16 < 3 * NUM_SMS ? 8 : 16;
    const size_t stage = (size_t)a.TR * (Kb / P + ROW_PAD);
    const int xrows = (a.M < 8 * NT ? a.M : 8 * NT) + 1;
    const size_t xbytes = (size_t)xrows * (Kb + ROW_PAD);
    const size_t partb = (size_t)2 * 8 * NT * 128 * 4;
    long long ns = ((long long)(224 * 1024) - SG_HDR - (long long)partb - (long long)xbytes) / (long long)stage;
    a.nstage = (int)(ns > 6 ? 6 : (ns < 2 ? 2 : ns));
    const int ntiles = (a.N + a.TR - 1) / a.TR;
    grid = ntiles < NUM_SMS ? ntiles : NUM_SMS;
    return SG_HDR + (size_t)a.nstage * stage + partb + xbytes;
}

}  // namespace qw
