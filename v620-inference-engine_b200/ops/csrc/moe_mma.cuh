// Routed-expert products of the decode path on the tensor cores.
//
// The q4 expert matrices are read once per chosen expert; with one token per pair the products are
// matrix-vector shaped, and in scalar code the unpack + multiply-add of every 4-bit weight made both
// kernels instruction-issue bound (63 % issue utilisation at 10 % of DRAM bandwidth).  Here a warp owns a
// tile of 16 weight rows and feeds mma.sync.m16n8k16 (bf16 x bf16 -> fp32) with the unpacked weights as the
// 16 x 16 operand and the activation vector as column 0 of the 16 x 8 operand: about 1.5 instructions per
// weight instead of ~16.
//
// Operand trick.  A dot product does not care in which order k is walked, as long as both operands agree.
// Lane (r = lane / 4, q = lane % 4) loads whole 32-bit words (8 weights, k = 8 w .. 8 w + 7) of rows r and
// r + 8 at word index w = w0 + q; nibble pair j of such a word ((word >> 4 j) & 0x000F000F, biased into bf16
// and re-centred) is exactly one operand register: two consecutive k of one row.  Pairs 0 / 1 feed one MMA
// (k slots 2q, 2q+1 and 2q+8, 2q+9), pairs 2 / 3 the next.  The matching activation registers of that lane are
// then the four 32-bit words of x[8 w .. 8 w + 7] - one 16-byte shared-memory load in natural order.
// Every byte a lane loads is used, a quad reads 32 contiguous bytes of a row, and nothing is shuffled.
// bf16 rows (the shared expert) use the same scheme with 16-byte loads as the operand registers directly.
//
// Scales: one per 128 k; a group is 8 MMAs into a fresh accumulator, then acc += scale * group.
// (Role of the reference's src/kernels/moe.hip pair kernels; the scheme is this engine's own.)
#pragma once
#include "fuse.cuh"
#include "mma.cuh"

namespace qw {

// bf16 pair (exact integers -8..7) of nibble pair j of a q4 word in engine order
__device__ __forceinline__ uint32_t q4_frag(uint32_t w, int j) {
    uint32_t p = ((w >> (4 * j)) & 0x000F000Fu) | 0x43004300u;
    bf162 v = *reinterpret_cast<bf162 *>(&p);
    const bf162 off = __floats2bfloat162_rn(136.f, 136.f);
    v = __hsub2(v, off);
    return *reinterpret_cast<uint32_t *>(&v);
}

// Two MMAs for one word of rows r (wr) and r + 8 (wr8) against the activation words xv of the same 8 k.
__device__ __forceinline__ void mma_q4_word(float (&c)[4], uint32_t wr, uint32_t wr8, const uint4 &xv) {
    mma_bf16(c, q4_frag(wr, 0), q4_frag(wr8, 0), q4_frag(wr, 1), q4_frag(wr8, 1), xv.x, xv.y);
    mma_bf16(c, q4_frag(wr, 2), q4_frag(wr8, 2), q4_frag(wr, 3), q4_frag(wr8, 3), xv.z, xv.w);
}
// The same for 8 bf16 weights of rows r and r + 8 (16-byte loads).
__device__ __forceinline__ void mma_bf16_chunk(float (&c)[4], const uint4 &wr, const uint4 &wr8, const uint4 &xv) {
    mma_bf16(c, wr.x, wr8.x, wr.y, wr8.y, xv.x, xv.y);
    mma_bf16(c, wr.z, wr8.z, wr.w, wr8.w, xv.z, xv.w);
}

// Shared expert's activation of row m: sh_h[m][f] = bf16(silu(gate_f) * up_f * sigmoid(shared gate logit)), by one block.
__device__ __forceinline__ void shared_act_row(const SharedAct &sa, int m) {
    const float *l = sa.rs + (long long)m * sa.ld_rs + sa.E;
    const float sg = sigmoidf_(__ldcg(l));
    bf16 *o = reinterpret_cast<bf16 *>(sa.sh_h) + (long long)m * sa.SF;
    for (int f0 = threadIdx.x; f0 < sa.SF; f0 += 4 * blockDim.x) {          // four independent loads of each kind in flight
        float g[4], u[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int f = f0 + k * blockDim.x;
            g[k] = f < sa.SF ? __ldcg(l + 1 + f) : 0.f;
            u[k] = f < sa.SF ? __ldcg(l + 1 + sa.SF + f) : 0.f;
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int f = f0 + k * blockDim.x;
            if (f < sa.SF) o[f] = __float2bfloat16(siluf_(g[k]) * u[k] * sg);
        }
    }
}

constexpr int MM_WARPS = 4;          // warps per block (128 threads: three blocks per SM stay resident, so 400 tiles are one wave)
constexpr int GU_NG = 5;             // k groups of 128 per warp in the gate/up kernel: K <= 4 * 5 * 128
constexpr int DN_NI = 13;            // (expert, k group) items per warp in the down kernel: top_k * F / 128 <= 52
constexpr int DN_NS = 5;             // quad-steps of the shared expert per warp: SF <= 4 * 5 * 32

// h[p][f] = silu(gate_e[f] . x_m) * (up_e[f] . x_m) for pair p = (m, j).  grid (F / 16, pairs), 128 threads.
// Warp w takes the k groups g = w, w + 4, ...; every weight load of the block is issued before the first
// one is used, and the four partial tiles are added in warp order.
__global__ void __launch_bounds__(128) moe_gate_up_mma_kernel(const uint32_t *w13, const bf16 *s13, const bf16 *x, int ldx,
                                                              const int *pair_expert, int top_k, int F, int K, bf16 *h, PfArgs pf,
                                                              SharedAct sa, int npairs) {
    extern __shared__ __align__(16) unsigned char mm_smem[];
    uint4 *xs = reinterpret_cast<uint4 *>(mm_smem);                       // [K / 8] activation words
    float *red = reinterpret_cast<float *>(mm_smem + (size_t)K * 2);     // [4 warps][2][16]
    pf_issue(pf);
    pdl_wait();
    pdl_trigger();
    if ((int)blockIdx.y >= npairs) {          // the extra rows of the grid: the shared expert's activation
        if (blockIdx.x == 0) shared_act_row(sa, blockIdx.y - npairs);
        return;
    }
    const int p = blockIdx.y;
    const int e = pair_expert[p];
    if (e < 0) return;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int r = lane >> 2, q = lane & 3;
    const int f0 = blockIdx.x * 16;
    const int m = p / top_k;
    const int wpr = K >> 3, ks = K >> 7;                                   // words and scale groups per row
    const long long row_g = (long long)e * 2 * F + f0 + r, row_u = row_g + F;
    const uint32_t *pg = w13 + row_g * wpr, *pg8 = pg + 8LL * wpr, *pu = w13 + row_u * wpr, *pu8 = pu + 8LL * wpr;
    uint2 wg[GU_NG][2], wg8[GU_NG][2], wu[GU_NG][2], wu8[GU_NG][2];
    float sg[GU_NG], sg8[GU_NG], su[GU_NG], su8[GU_NG];
#pragma unroll
    for (int i = 0; i < GU_NG; ++i) {
        const int g = warp + MM_WARPS * i;
        if (g < ks) {
#pragma unroll
            for (int ds = 0; ds < 2; ++ds) {
                const int wi = g * 16 + ds * 8 + 2 * q;
                wg[i][ds] = ld_stream8(pg + wi);
                wg8[i][ds] = ld_stream8(pg8 + wi);
                wu[i][ds] = ld_stream8(pu + wi);
                wu8[i][ds] = ld_stream8(pu8 + wi);
            }
            sg[i] = __bfloat162float(s13[row_g * ks + g]);
            sg8[i] = __bfloat162float(s13[(row_g + 8) * ks + g]);
            su[i] = __bfloat162float(s13[row_u * ks + g]);
            su8[i] = __bfloat162float(s13[(row_u + 8) * ks + g]);
        }
    }
    const uint4 *xr = reinterpret_cast<const uint4 *>(x + (long long)m * ldx);
    for (int i = tid; i < wpr; i += 128) xs[i] = __ldcg(xr + i);
    __syncthreads();
    float ag = 0.f, ag8 = 0.f, au = 0.f, au8 = 0.f;
#pragma unroll
    for (int i = 0; i < GU_NG; ++i) {
        const int g = warp + MM_WARPS * i;
        if (g < ks) {
            float cg[4] = {0.f, 0.f, 0.f, 0.f}, cu[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int ds = 0; ds < 2; ++ds) {
                const int wi = g * 16 + ds * 8 + 2 * q;
                uint4 x0 = make_uint4(0u, 0u, 0u, 0u), x1 = x0;
                if (r == 0) {                                               // column 0 of the narrow operand is the token
                    x0 = xs[wi];
                    x1 = xs[wi + 1];
                }
                mma_q4_word(cg, wg[i][ds].x, wg8[i][ds].x, x0);
                mma_q4_word(cg, wg[i][ds].y, wg8[i][ds].y, x1);
                mma_q4_word(cu, wu[i][ds].x, wu8[i][ds].x, x0);
                mma_q4_word(cu, wu[i][ds].y, wu8[i][ds].y, x1);
            }
            // column 0 of the result sits in the lanes with q == 0: c[0] is row r, c[2] row r + 8
            ag = fmaf(sg[i], cg[0], ag); ag8 = fmaf(sg8[i], cg[2], ag8);
            au = fmaf(su[i], cu[0], au); au8 = fmaf(su8[i], cu[2], au8);
        }
    }
    if (q == 0) {
        red[(warp * 2 + 0) * 16 + r] = ag; red[(warp * 2 + 0) * 16 + r + 8] = ag8;
        red[(warp * 2 + 1) * 16 + r] = au; red[(warp * 2 + 1) * 16 + r + 8] = au8;
    }
    __syncthreads();
    if (tid < 16) {
        float gs = 0.f, us = 0.f;
#pragma unroll
        for (int w = 0; w < MM_WARPS; ++w) { gs += red[(w * 2) * 16 + tid]; us += red[(w * 2 + 1) * 16 + tid]; }
        h[(long long)p * F + f0 + tid] = __float2bfloat16(siluf_(gs) * us);
    }
}

// out[m][c] = sum_j w_j * (down_{e_j}[c] . h[p_j]) + shared_down[c] . sh_h[m].  grid (H / 16, M), 128 threads.
// The (expert, k group) items and the shared expert's k are dealt round-robin to the four warps; every weight
// load of the block is issued before the first one is used.
template <bool FUSED>
__global__ void __launch_bounds__(128) moe_down_mma_kernel(const uint32_t *w2, const bf16 *s2, const bf16 *h, const int *pair_expert,
                                                           const float *pair_w, int top_k, int F, int H, const bf16 *shared_down,
                                                           int ld_sd, const bf16 *sh_h, int SF, float *out, int ldo, PfArgs pf, FuseOut fo) {
    extern __shared__ __align__(16) unsigned char mm_smem[];
    uint4 *hs = reinterpret_cast<uint4 *>(mm_smem);                                       // [top_k][F / 8]
    uint4 *ss = hs + (size_t)top_k * (F >> 3);                                            // [SF / 8]
    float *red = reinterpret_cast<float *>(ss + (SF >> 3));                               // [4][16]
    pf_issue(pf);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int r = lane >> 2, q = lane & 3;
    const int m = blockIdx.y, c0 = blockIdx.x * 16;
    // the shared expert's rows do not depend on the routing: fetch them before waiting for the router
    const int sch = SF >> 3;                                   // 16-byte pieces per shared row
    const bf16 *sr = shared_down ? shared_down + (long long)(c0 + r) * ld_sd : nullptr;
    uint4 sw[DN_NS], sw8[DN_NS];
#pragma unroll
    for (int i = 0; i < DN_NS; ++i) {
        const int pc = (warp + MM_WARPS * i) * 4 + q;
        sw[i] = sw8[i] = make_uint4(0u, 0u, 0u, 0u);
        if (shared_down && pc < sch) {
            sw[i] = ld_stream(reinterpret_cast<const uint4 *>(sr) + pc);
            sw8[i] = ld_stream(reinterpret_cast<const uint4 *>(sr + 8LL * ld_sd) + pc);
        }
    }
    pdl_wait();
    pdl_trigger();
    const int wpr = F >> 3, ks = F >> 7;
    const int nitems = top_k * ks;
    uint2 wv[DN_NI][2], wv8[DN_NI][2];
    float sc[DN_NI], sc8[DN_NI];
#pragma unroll
    for (int i = 0; i < DN_NI; ++i) {
        const int it = warp + MM_WARPS * i;
        sc[i] = sc8[i] = 0.f;
        if (it < nitems) {
            const int j = it / ks, g = it - j * ks;
            const int p = m * top_k + j;
            const int e = pair_expert[p];
            if (e >= 0) {
                const float pw = pair_w[p];
                const long long row = (long long)e * H + c0 + r;
                const uint32_t *pr = w2 + row * wpr;
#pragma unroll
                for (int ds = 0; ds < 2; ++ds) {
                    const int wi = g * 16 + ds * 8 + 2 * q;
                    wv[i][ds] = ld_stream8(pr + wi);
                    wv8[i][ds] = ld_stream8(pr + 8LL * wpr + wi);
                }
                sc[i] = __bfloat162float(s2[row * ks + g]) * pw;
                sc8[i] = __bfloat162float(s2[(row + 8) * ks + g]) * pw;
            } else {
#pragma unroll
                for (int ds = 0; ds < 2; ++ds) wv[i][ds] = wv8[i][ds] = make_uint2(0x88888888u, 0x88888888u);      // zeros in q4
            }
        }
    }
    for (int i = tid; i < top_k * wpr; i += 128) hs[i] = __ldcg(reinterpret_cast<const uint4 *>(h + (long long)m * top_k * F) + i);
    if (shared_down)
        for (int i = tid; i < sch; i += 128) ss[i] = __ldcg(reinterpret_cast<const uint4 *>(sh_h + (long long)m * SF) + i);
    __syncthreads();
    float a0 = 0.f, a8 = 0.f;
#pragma unroll
    for (int i = 0; i < DN_NI; ++i) {
        const int it = warp + MM_WARPS * i;
        if (it < nitems) {
            const int j = it / ks, g = it - j * ks;
            const uint4 *xj = hs + (size_t)j * wpr;
            float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int ds = 0; ds < 2; ++ds) {
                const int wi = g * 16 + ds * 8 + 2 * q;
                uint4 x0 = make_uint4(0u, 0u, 0u, 0u), x1 = x0;
                if (r == 0) {
                    x0 = xj[wi];
                    x1 = xj[wi + 1];
                }
                mma_q4_word(c, wv[i][ds].x, wv8[i][ds].x, x0);
                mma_q4_word(c, wv[i][ds].y, wv8[i][ds].y, x1);
            }
            a0 = fmaf(sc[i], c[0], a0);
            a8 = fmaf(sc8[i], c[2], a8);
        }
    }
    if (shared_down) {
        float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < DN_NS; ++i) {
            const int pc = (warp + MM_WARPS * i) * 4 + q;
            if ((warp + MM_WARPS * i) * 4 < sch) {          // warp-uniform: the MMA needs every lane
                const uint4 xv = (r == 0 && pc < sch) ? ss[pc] : make_uint4(0u, 0u, 0u, 0u);
                mma_bf16_chunk(c, sw[i], sw8[i], xv);
            }
        }
        a0 += c[0];
        a8 += c[2];
    }
    if (q == 0) {
        red[warp * 16 + r] = a0;
        red[warp * 16 + r + 8] = a8;
    }
    __syncthreads();
    if (tid < 16) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < MM_WARPS; ++w) v += red[w * 16 + tid];
        if (FUSED) fuse_put_col(fo, fuse_seq(fo), m, c0 + tid, __float_as_uint(v));      // fused reduce-scatter: to the column's owner
        else out[(long long)m * ldo + c0 + tid] = v;
    }
}

// ---------------------------------------------------------------------------------------------------------------
// The same two products with the weights brought in by bulk-async (TMA, untiled) row copies into padded shared memory.
// Direct 8-byte loads from sixteen rows at once touch one 32-byte sector per row per request, which HBM serves badly
// (measured: 16 us for 17 MB); one bulk copy per weight row is fully coalesced, needs no registers while in flight, and
// the operand words are then read from shared memory exactly as before (row stride padded by 32 bytes: the eight rows
// of a request fall into disjoint bank groups).  One block per tile, every copy of the block issued at once, one
// mbarrier; enough blocks are resident for the whole launch to be one wave.
// ---------------------------------------------------------------------------------------------------------------
constexpr int TM_PAD = 32;                 // bytes added to a weight row in shared memory

// grid (F / 16, pairs [+ M extra rows for the shared activation]), 512 threads.
__global__ void __launch_bounds__(512) moe_gate_up_tma_kernel(const uint32_t *w13, const bf16 *s13, const bf16 *x, int ldx,
                                                              const int *pair_expert, int top_k, int F, int K, bf16 *h, ErrorWord *err,
                                                              SharedAct sa, int npairs) {
    extern __shared__ __align__(128) unsigned char tm_smem[];
    const int rowb = K >> 1, srow = rowb + TM_PAD, ks = K >> 7, wpr = K >> 3;
    uint64_t *bar = reinterpret_cast<uint64_t *>(tm_smem);
    unsigned char *wg = tm_smem + 128, *wu = wg + 16 * srow;
    bf16 *sg = reinterpret_cast<bf16 *>(wu + 16 * srow), *su = sg + 16 * ks;
    uint4 *xs = reinterpret_cast<uint4 *>(reinterpret_cast<unsigned char *>(su + 16 * ks) + ((-(16 * ks * 4)) & 15));
    float *red = reinterpret_cast<float *>(xs + wpr);          // [16 warps][2][16]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        mbar_init(bar, 1);
        mbar_fence_init();
    }
    pdl_wait();
    pdl_trigger();
    if ((int)blockIdx.y >= npairs) {          // the extra rows of the grid: the shared expert's activation
        if (blockIdx.x == 0) shared_act_row(sa, blockIdx.y - npairs);
        return;
    }
    const int p = blockIdx.y;
    const int e = pair_expert[p];
    if (e < 0) return;
    const int f0 = blockIdx.x * 16, m = p / top_k;
    const long long row_g = (long long)e * 2 * F + f0, row_u = row_g + F;
    __syncthreads();                          // the barrier is initialised
    if (warp == 0) {
        if (lane == 0) mbar_expect_tx(bar, (unsigned)(32 * rowb + 2 * 16 * ks * 2));
        __syncwarp();
        if (lane < 16) bulk_g2s(wg + lane * srow, w13 + (row_g + lane) * wpr, (unsigned)rowb, bar);
        else bulk_g2s(wu + (lane - 16) * srow, w13 + (row_u + lane - 16) * wpr, (unsigned)rowb, bar);
        if (lane == 0) bulk_g2s(sg, s13 + row_g * ks, (unsigned)(16 * ks * 2), bar);
        if (lane == 1) bulk_g2s(su, s13 + row_u * ks, (unsigned)(16 * ks * 2), bar);
    }
    const uint4 *xr = reinterpret_cast<const uint4 *>(x + (long long)m * ldx);
    for (int i = tid; i < wpr; i += 512) xs[i] = __ldcg(xr + i);
    __syncthreads();
    const bool ok = mbar_wait(bar, 0u, err);
    const int r = lane >> 2, q = lane & 3;
    float ag = 0.f, ag8 = 0.f, au = 0.f, au8 = 0.f;
    if (ok) {
        for (int g = warp; g < ks; g += 16) {
            float cg[4] = {0.f, 0.f, 0.f, 0.f}, cu[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int ds = 0; ds < 2; ++ds) {
                const int wi = g * 16 + ds * 8 + 2 * q;
                const uint2 a0 = *reinterpret_cast<const uint2 *>(wg + r * srow + wi * 4), a8 = *reinterpret_cast<const uint2 *>(wg + (r + 8) * srow + wi * 4);
                const uint2 b0 = *reinterpret_cast<const uint2 *>(wu + r * srow + wi * 4), b8 = *reinterpret_cast<const uint2 *>(wu + (r + 8) * srow + wi * 4);
                uint4 x0 = make_uint4(0u, 0u, 0u, 0u), x1 = x0;
                if (r == 0) {                                               // column 0 of the narrow operand is the token
                    x0 = xs[wi];
                    x1 = xs[wi + 1];
                }
                mma_q4_word(cg, a0.x, a8.x, x0);
                mma_q4_word(cg, a0.y, a8.y, x1);
                mma_q4_word(cu, b0.x, b8.x, x0);
                mma_q4_word(cu, b0.y, b8.y, x1);
            }
            if (q == 0) {
                ag = fmaf(__bfloat162float(sg[r * ks + g]), cg[0], ag);
                ag8 = fmaf(__bfloat162float(sg[(r + 8) * ks + g]), cg[2], ag8);
                au = fmaf(__bfloat162float(su[r * ks + g]), cu[0], au);
                au8 = fmaf(__bfloat162float(su[(r + 8) * ks + g]), cu[2], au8);
            }
        }
    }
    if (q == 0) {
        red[(warp * 2 + 0) * 16 + r] = ag; red[(warp * 2 + 0) * 16 + r + 8] = ag8;
        red[(warp * 2 + 1) * 16 + r] = au; red[(warp * 2 + 1) * 16 + r + 8] = au8;
    }
    __syncthreads();
    if (tid < 16) {
        float gs = 0.f, us = 0.f;
#pragma unroll
        for (int w = 0; w < 16; ++w) { gs += red[(w * 2) * 16 + tid]; us += red[(w * 2 + 1) * 16 + tid]; }
        h[(long long)p * F + f0 + tid] = __float2bfloat16(siluf_(gs) * us);
    }
}

// grid (H / 16, M), 512 threads.  Shared memory: barrier(s) | top_k expert tiles [16][F/2 + pad] | shared tile
// [16][SF*2 + pad] | scales [top_k][16][F/128] | h vectors | shared activation | reduction scratch.
template <bool FUSED>
__global__ void __launch_bounds__(512) moe_down_tma_kernel(const uint32_t *w2, const bf16 *s2, const bf16 *h, const int *pair_expert,
                                                           const float *pair_w, int top_k, int F, int H, const bf16 *shared_down,
                                                           int ld_sd, const bf16 *sh_h, int SF, float *out, int ldo, ErrorWord *err,
                                                           FuseOut fo) {
    extern __shared__ __align__(128) unsigned char tm_smem[];
    const int rowb = F >> 1, srow = rowb + TM_PAD, ks = F >> 7, wpr = F >> 3;
    const int srowb = SF * 2, ssrow = srowb + TM_PAD, sch = SF >> 3;
    uint64_t *bar = reinterpret_cast<uint64_t *>(tm_smem);              // [0] routed experts, [1] shared expert
    unsigned char *we = tm_smem + 128;                                   // [top_k][16][srow]
    unsigned char *wsd = we + (size_t)top_k * 16 * srow;                 // [16][ssrow]
    bf16 *sc = reinterpret_cast<bf16 *>(wsd + (shared_down ? 16 * ssrow : 0));      // [top_k][16 * ks] (+ pad to 16 bytes per expert)
    const int scb = ((16 * ks * 2) + 15) & ~15;                          // bytes of one expert's scales in shared memory
    uint4 *hs = reinterpret_cast<uint4 *>(reinterpret_cast<unsigned char *>(sc) + (size_t)top_k * scb);      // [top_k][wpr]
    uint4 *ss = hs + (size_t)top_k * wpr;                                // [sch]
    float *red = reinterpret_cast<float *>(ss + sch);                    // [16 warps][16]
    int *s_e = reinterpret_cast<int *>(red + 16 * 16);                   // [top_k]
    float *s_w = reinterpret_cast<float *>(s_e + 32);                    // [top_k]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int m = blockIdx.y, c0 = blockIdx.x * 16;
    if (tid == 0) {
        mbar_init(bar, 1);
        mbar_init(bar + 1, 1);
        mbar_fence_init();
    }
    __syncthreads();
    // the shared expert's rows do not depend on the routing: their copies start before the wait for the router
    if (shared_down && warp == 0) {
        if (lane == 0) mbar_expect_tx(bar + 1, (unsigned)(16 * srowb));
        __syncwarp();
        if (lane < 16) bulk_g2s(wsd + lane * ssrow, shared_down + (long long)(c0 + lane) * ld_sd, (unsigned)srowb, bar + 1);
    }
    pdl_wait();
    pdl_trigger();
    if (tid < top_k) {
        const int p = m * top_k + tid;
        s_e[tid] = pair_expert[p];
        s_w[tid] = pair_w[p];
    }
    __syncthreads();
    // every warp issues the copies of its experts (one warp issuing all 170 of them took microseconds); the expected byte
    // count is posted once by thread 0 - copies that complete earlier are accounted against it
    if (tid == 0) {
        int nloc = 0;
        for (int j = 0; j < top_k; ++j) nloc += s_e[j] >= 0;
        mbar_expect_tx(bar, (unsigned)(nloc * (16 * rowb + 16 * ks * 2)));
    }
    for (int j = warp; j < top_k; j += 16) {
        const int e = s_e[j];
        if (e < 0) continue;
        const long long row = (long long)e * H + c0;
        if (lane < 16) bulk_g2s(we + ((size_t)j * 16 + lane) * srow, w2 + (row + lane) * wpr, (unsigned)rowb, bar);
        if (lane == 16) bulk_g2s(reinterpret_cast<unsigned char *>(sc) + (size_t)j * scb, s2 + row * ks, (unsigned)(16 * ks * 2), bar);
    }
    {
        // the activations: both loops' loads in flight together
        const uint4 *hg = reinterpret_cast<const uint4 *>(h + (long long)m * top_k * F);
        const int nh = top_k * wpr;
        uint4 v0 = make_uint4(0u, 0u, 0u, 0u), v1 = v0, v2 = v0;
        if (tid < nh) v0 = __ldcg(hg + tid);
        if (tid + 512 < nh) v1 = __ldcg(hg + tid + 512);
        if (shared_down && tid < sch) v2 = __ldcg(reinterpret_cast<const uint4 *>(sh_h + (long long)m * SF) + tid);
        if (tid < nh) hs[tid] = v0;
        if (tid + 512 < nh) hs[tid + 512] = v1;
        for (int i = tid + 1024; i < nh; i += 512) hs[i] = __ldcg(hg + i);
        if (shared_down) {
            if (tid < sch) ss[tid] = v2;
            for (int i = tid + 512; i < sch; i += 512) ss[i] = __ldcg(reinterpret_cast<const uint4 *>(sh_h + (long long)m * SF) + i);
        }
    }
    __syncthreads();
    const int r = lane >> 2, q = lane & 3;
    float a0 = 0.f, a8 = 0.f;
    bool ok = mbar_wait(bar, 0u, err);
    if (ok) {
        const int nitems = top_k * ks;
        for (int it = warp; it < nitems; it += 16) {
            const int j = it / ks, g = it - j * ks;
            if (s_e[j] < 0) continue;                       // warp-uniform
            const unsigned char *wj = we + (size_t)j * 16 * srow;
            const uint4 *xj = hs + (size_t)j * wpr;
            float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int ds = 0; ds < 2; ++ds) {
                const int wi = g * 16 + ds * 8 + 2 * q;
                const uint2 v0 = *reinterpret_cast<const uint2 *>(wj + r * srow + wi * 4), v8 = *reinterpret_cast<const uint2 *>(wj + (r + 8) * srow + wi * 4);
                uint4 x0 = make_uint4(0u, 0u, 0u, 0u), x1 = x0;
                if (r == 0) {
                    x0 = xj[wi];
                    x1 = xj[wi + 1];
                }
                mma_q4_word(c, v0.x, v8.x, x0);
                mma_q4_word(c, v0.y, v8.y, x1);
            }
            if (q == 0) {
                const bf16 *sj = reinterpret_cast<const bf16 *>(reinterpret_cast<const unsigned char *>(sc) + (size_t)j * scb);
                a0 = fmaf(__bfloat162float(sj[r * ks + g]) * s_w[j], c[0], a0);
                a8 = fmaf(__bfloat162float(sj[(r + 8) * ks + g]) * s_w[j], c[2], a8);
            }
        }
    }
    if (shared_down && mbar_wait(bar + 1, 0u, err)) {
        float c[4] = {0.f, 0.f, 0.f, 0.f};
        for (int st = warp; st * 4 < sch; st += 16) {         // quad-steps of four 16-byte pieces
            const int pc = st * 4 + q;
            uint4 w0 = make_uint4(0u, 0u, 0u, 0u), w8 = w0, xv = w0;
            if (pc < sch) {
                w0 = *reinterpret_cast<const uint4 *>(wsd + r * ssrow + pc * 16);
                w8 = *reinterpret_cast<const uint4 *>(wsd + (r + 8) * ssrow + pc * 16);
                if (r == 0) xv = ss[pc];
            }
            mma_bf16_chunk(c, w0, w8, xv);
        }
        a0 += c[0];
        a8 += c[2];
    }
    if (q == 0) {
        red[warp * 16 + r] = a0;
        red[warp * 16 + r + 8] = a8;
    }
    __syncthreads();
    if (tid < 16) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < 16; ++w) v += red[w * 16 + tid];
        if (FUSED) fuse_put_col(fo, fuse_seq(fo), m, c0 + tid, __float_as_uint(v));      // fused reduce-scatter: to the column's owner
        else out[(long long)m * ldo + c0 + tid] = v;
    }
}

}  // namespace qw
