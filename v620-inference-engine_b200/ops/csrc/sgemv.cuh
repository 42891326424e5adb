// Streaming skinny matrix product core: D[n][m] = sum_k W[n][k] x[m][k] for bf16 weights and up to
// 16 activation rows per pass, with caller-supplied functors that build the activation rows in
// shared memory and consume each finished 16-row tile.
//
// One persistent block per SM, 8 consumer warps + 1 producer warp.  The producer warp copies weight
// rows global -> shared memory with bulk-async copies (16 rows x up to 2.5 KB per stage, up to six
// stages in flight), runs ahead of the consumers through full/empty mbarriers, and never waits for
// the predecessor kernel because weights do not depend on it (programmatic dependent launch lets it
// start during the predecessor's tail).  The consumer warps split a stage's k range and feed the
// tensor core (ldmatrix + m16n8k16, fp32 accumulate) with the activation rows as the narrow operand,
// so 16 activation rows cost the same instructions as one; the warps' partial sums are added in warp
// order, so a row's result does not depend on how many other rows share the step.
//
// Used by: the bf16 GEMV (projections, lm_head, PLE), the MoE router (+ routing epilogue), the
// hyper-connection down projection (column splits, fused combine/norm prologue) and up projection
// (fused gate/mean epilogue).
#pragma once
#include "mma.cuh"
#include "fuse.cuh"

namespace qw {

struct SGemvArgs {
    const bf16 *W;      // [N][ldw] (+ split * w_split)
    const bf16 *x;      // [M][ldx]           (default activation fill)
    float *y;           // [M][ldy]           (default store)
    bf16 *y_bf16;       // optional bf16 copy of y
    int N, K, M;
    int ldw, ldx, ldy;
    int accumulate;
    int nsplit;         // independent column splits of W (each with its own activation rows)
    long long w_split;  // element offset of a split inside a weight row
    int P;              // k parts per row tile
    int nstage;
    ErrorWord *err;
    PfArgs pf;          // weights of later kernels to pull into L2
    FuseIn fi = {};     // fused all-gather: the activation rows are built from the ranks' words
    FuseOut fo = {};    // fused reduce-scatter: y goes to the ranks that own its columns instead of memory
};

constexpr int SG_HDR = 128;              // mbarriers: full[8], empty[8]
constexpr int SG_THREADS = 288;          // 8 consumer warps + 1 producer warp
constexpr int SG_TILE = 16;              // weight rows per tile
constexpr size_t SG_SMEM_MAX = 224 * 1024;

struct SGemvSmem {
    unsigned char *stages;
    float *part;        // [2][8][NT][128] per-warp partial tiles (double buffered by tile parity)
    float *sum;         // [NT][16][8] summed tile handed to the epilogue
    unsigned char *xs;  // [(rows)+1][xrow] activation rows + one zero row
    unsigned xrow;      // bytes between activation rows
    unsigned char *extra;   // caller's scratch behind the activation rows
};

// Default activation fill: rows m0.. of a.x, converted as they are (bf16), plus the zero row.
struct XFillCopy {
    const SGemvArgs &a;
    __device__ __forceinline__ void operator()(int /*split*/, int /*row0*/, int m0, int nm, const SGemvSmem &sm, int tid) const {
        const int nchunk = a.K >> 3, total = (nm + 1) * nchunk;
        // four loads per thread in flight: the fill is on the kernel's critical path (one L2 round trip per batch)
        for (int i0 = tid; i0 < total; i0 += 1024) {
            uint4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = i0 + u * 256;
                const int m = i / nchunk, c = i - m * nchunk;
                v[u] = make_uint4(0u, 0u, 0u, 0u);
                if (i < total && m < nm) v[u] = __ldcg(reinterpret_cast<const uint4 *>(a.x + (long long)(m0 + m) * a.ldx) + c);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = i0 + u * 256;
                const int m = i / nchunk, c = i - m * nchunk;
                if (i < total) *reinterpret_cast<uint4 *>(sm.xs + (size_t)m * sm.xrow + (size_t)c * 16) = v[u];
            }
        }
    }
};

// Activation fill from a fused all-gather: column r * n + w of row m is word w of row m in rank r's slot (one bf16
// per word).  Block 0 also leaves the dense rows in a.x for later kernels that read them from memory.
struct XFillGather {
    const SGemvArgs &a;
    __device__ __forceinline__ void operator()(int /*split*/, int /*row0*/, int m0, int nm, const SGemvSmem &sm, int tid) const {
        const unsigned int seq = fuse_seq(a.fi);
        const int n = a.fi.n;                              // columns per rank (a multiple of 8)
        const int nchunk = a.K >> 3;
        for (int i = tid; i < nm * nchunk; i += 256) {
            const int m = i / nchunk, c = (i - m * nchunk) * 8;
            const int r = c / n, w = c - r * n;
            const uint4 v = fuse_get8_u16(a.fi, seq, r, (long long)(m0 + m) * n + w);
            *reinterpret_cast<uint4 *>(sm.xs + (size_t)m * sm.xrow + (size_t)c * 2) = v;
            if (blockIdx.x == 0) *reinterpret_cast<uint4 *>(const_cast<bf16 *>(a.x) + (long long)(m0 + m) * a.ldx + c) = v;
        }
        for (int c = tid; c < (a.K >> 3); c += 256)
            *reinterpret_cast<uint4 *>(sm.xs + (size_t)nm * sm.xrow + (size_t)c * 16) = make_uint4(0u, 0u, 0u, 0u);
    }
};

// Default epilogue: y[m][row] (+)= D.
template <int NT, bool FUSED = false>
struct EpiStore {
    const SGemvArgs &a;
    __device__ __forceinline__ void operator()(int /*split*/, int row0, int m0, int nm, const SGemvSmem &sm, int tid) const {
        const unsigned int seq = FUSED && a.fo.mode ? fuse_seq(a.fo) : 0u;
        for (int e = tid; e < NT * 128; e += 256) {
            const int t = e >> 7, r = (e >> 3) & 15, n = e & 7;
            const int m = t * 8 + n;
            if (m < nm && row0 + r < a.N) {
                float v = sm.sum[e];
                if (FUSED && a.fo.mode) {          // fused reduce-scatter: straight to the owner of the column
                    fuse_put_col(a.fo, seq, m0 + m, row0 + r, __float_as_uint(v));
                    continue;
                }
                const long long o = (long long)(m0 + m) * a.ldy + row0 + r;
                if (a.accumulate) v += a.y[o];
                a.y[o] = v;
                if (a.y_bf16) a.y_bf16[o] = __float2bfloat16(v);
            }
        }
    }
};

// NT = activation-row tiles of 8 handled per pass (1 or 2).
template <int NT, class XFill, class Epi>
__device__ __forceinline__ void sgemv_core(const SGemvArgs &a, unsigned char *smem, const XFill &xfill, const Epi &epi) {
    uint64_t *full = reinterpret_cast<uint64_t *>(smem), *empty = full + 8;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int Kc = a.K / a.P;
    const unsigned KcB = (unsigned)Kc * 2u, srow = KcB + ROW_PAD;          // stage row stride
    const unsigned stage_bytes = SG_TILE * srow;
    const int MT = 8 * NT;
    SGemvSmem sm;
    sm.stages = smem + SG_HDR;
    sm.part = reinterpret_cast<float *>(sm.stages + (size_t)a.nstage * stage_bytes);
    sm.sum = sm.part + 2 * 8 * NT * 128;
    sm.xs = reinterpret_cast<unsigned char *>(sm.sum + NT * 128);
    sm.xrow = (unsigned)a.K * 2u + ROW_PAD;
    sm.extra = sm.xs + (size_t)((a.M < MT ? a.M : MT) + 1) * sm.xrow;
    const int tps = (a.N + SG_TILE - 1) / SG_TILE;          // tiles per split
    const int nitems = tps * a.nsplit;
    const int cnt = (int)blockIdx.x < nitems ? (nitems - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
    const int mtiles = (a.M + MT - 1) / MT;
    const int total = cnt * a.P * mtiles;
    if (tid == 0) {
        for (int s = 0; s < a.nstage; ++s) {
            mbar_init(full + s, 1);
            mbar_init(empty + s, 8);          // one arrival per consumer warp
        }
        mbar_fence_init();
    }
    __syncthreads();
    if (warp == 8) {
        // ---- producer warp: lane r copies row r of each stage
        for (int q = 0; q < total; ++q) {
            const int s = q % a.nstage;
            if (q >= a.nstage && !mbar_wait(empty + s, (unsigned)(q / a.nstage - 1) & 1u, a.err)) break;
            const int kp = q % a.P, i = (q / a.P) % cnt;
            const int it = (int)blockIdx.x + i * (int)gridDim.x;
            const int split = it / tps, row0 = (it - split * tps) * SG_TILE;
            const int rows = min(SG_TILE, a.N - row0);
            unsigned char *dst = sm.stages + (size_t)s * stage_bytes;
            if (lane == 0) mbar_expect_tx(full + s, (unsigned)rows * KcB);
            __syncwarp();
            if (lane < rows)
                bulk_g2s(dst + (size_t)lane * srow,
                         a.W + (long long)(row0 + lane) * a.ldw + split * a.w_split + (long long)kp * Kc, KcB, full + s);
        }
        return;
    }
    pf_issue(a.pf);
    pdl_wait();
    pdl_trigger();
    const uint32_t xs_base = smem_u32(sm.xs), st_base = smem_u32(sm.stages);
    const int steps = Kc >> 4;
    bool ok = true;
    int q = 0;
    for (int tile = 0; tile < mtiles && ok; ++tile) {
        const int m0 = tile * MT;
        const int nm = min(MT, a.M - m0);
        int cur_split = -1;
        for (int i = 0; i < cnt && ok; ++i) {
            const int it = (int)blockIdx.x + i * (int)gridDim.x;
            const int split = it / tps, row0 = (it - split * tps) * SG_TILE;
            if (split != cur_split) {
                if (cur_split >= 0) consumer_sync(256);          // everyone is done reading the old rows
                xfill(split, row0, m0, nm, sm, tid);
                cur_split = split;
                consumer_sync(256);
            }
            float c[NT][4];
#pragma unroll
            for (int t = 0; t < NT; ++t) c[t][0] = c[t][1] = c[t][2] = c[t][3] = 0.f;
            for (int kp = 0; kp < a.P; ++kp, ++q) {
                const int s = q % a.nstage;
                ok = mbar_wait(full + s, (unsigned)(q / a.nstage) & 1u, a.err);
                if (!ok) break;
                const uint32_t tb = st_base + (unsigned)s * stage_bytes;
                for (int st = warp; st < steps; st += 8) {
                    uint32_t a0, a1, a2, a3;
                    ldmatrix_x4(a0, a1, a2, a3, a_tile_addr(tb, srow, st << 4, lane));
#pragma unroll
                    for (int t = 0; t < NT; ++t) {
                        uint32_t b0, b1;
                        ldmatrix_x2(b0, b1, b_tile_addr(xs_base, sm.xrow, t * 8, nm, nm, kp * Kc + (st << 4), lane));
                        mma_bf16(c[t], a0, a1, a2, a3, b0, b1);
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(empty + s);      // this warp is done with the stage
            }
            if (!ok) break;
            float *pp = sm.part + ((size_t)(i & 1) * 8 + warp) * NT * 128;
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                const int r = lane >> 2, n = (lane & 3) * 2;
                pp[t * 128 + r * 8 + n] = c[t][0];
                pp[t * 128 + r * 8 + n + 1] = c[t][1];
                pp[t * 128 + (r + 8) * 8 + n] = c[t][2];
                pp[t * 128 + (r + 8) * 8 + n + 1] = c[t][3];
            }
            consumer_sync(256);                  // partial sums of all warps visible (and the previous epilogue is over)
            for (int e = tid; e < NT * 128; e += 256) {
                const float *ps = sm.part + (size_t)(i & 1) * 8 * NT * 128 + e;
                float v = 0.f;
#pragma unroll
                for (int w = 0; w < 8; ++w) v += ps[(size_t)w * NT * 128];      // warp order: fixed
                sm.sum[e] = v;
            }
            consumer_sync(256);
            epi(split, row0, m0, nm, sm, tid);
        }
        consumer_sync(256);          // activation rows are rewritten by the next tile of rows
    }
}

// Picks the k partition and the pipeline depth with `extra` bytes of caller scratch behind the
// activation rows; returns the dynamic shared memory size (0 = does not fit).
static inline size_t sgemv_plan(SGemvArgs &a, int NT, int &grid, size_t extra = 0) {
    const size_t Kb = (size_t)a.K * 2;
    int P = (int)((Kb + 2559) / 2560);
    while (a.K % (16 * P)) ++P;
    a.P = P;
    if (a.nsplit < 1) a.nsplit = 1;
    const size_t stage = (size_t)SG_TILE * (Kb / P + ROW_PAD);
    const int xrows = (a.M < 8 * NT ? a.M : 8 * NT) + 1;
    const size_t xbytes = (size_t)xrows * (Kb + ROW_PAD);
    const size_t fixed = SG_HDR + (size_t)(2 * 8 + 1) * NT * 128 * 4 + xbytes + extra;
    if (fixed + 2 * stage > SG_SMEM_MAX) return 0;
    long long ns = ((long long)SG_SMEM_MAX - (long long)fixed) / (long long)stage;
    a.nstage = (int)(ns > 6 ? 6 : ns);
    const int nitems = ((a.N + SG_TILE - 1) / SG_TILE) * a.nsplit;
    grid = nitems < NUM_SMS ? nitems : NUM_SMS;
    return fixed + (size_t)a.nstage * stage;
}

// The plain GEMV body: default fill and store.
template <int NT, bool FUSED = false>
__device__ __forceinline__ void sgemv_body(const SGemvArgs &a, unsigned char *smem) {
    if constexpr (FUSED) {
        if (a.fi.active) sgemv_core<NT>(a, smem, XFillGather{a}, EpiStore<NT, true>{a});
        else sgemv_core<NT>(a, smem, XFillCopy{a}, EpiStore<NT, true>{a});
    } else {
        sgemv_core<NT>(a, smem, XFillCopy{a}, EpiStore<NT>{a});
    }
}

}  // namespace qw
