// Decode-path MoE kernels.
//   moe_router : one kernel = the router / shared-gate / shared gate-up matrix-vector product, and,
//                in the block that finishes last, the routing itself (softmax, top-k by repeated
//                argmax with ties to the lowest index, renormalisation, expert-parallel filter) and
//                the shared expert's gated activation.
//   moe_gate_up_pair / moe_down_combine : q4 matrix-vector products per (row, expert) pair, 32
//                weights (16 bytes) per lane and load, all loads of a warp independent, with the
//                weighted combine and the shared expert's down projection fused into the second.
// (Roles of the reference's src/kernels/moe_route.hip:65-224 and src/kernels/moe_experts.hip:189-246.)
#include <cstdlib>
#include <cstring>

#include "sgemv.cuh"
#include "moe_mma.cuh"

namespace qw {

// Routing of row m from rs[m] = [ router logits (E) | shared gate logit | shared gate rows (F) | shared up rows (F) ].
// One warp per row.
__device__ __forceinline__ void route_row(const float *l, int E, int top_k, int e_first, int e_local, int *pair_expert,
                                          float *pair_w, int lane, int *stats) {
    // The ranking is done on the logits (the softmax is monotonic); only the chosen ones are exponentiated:
    // w_j = exp(l_j - l_top) / sum over the chosen.  Every lane keeps the best of its own elements cached, so a round
    // is one warp arg-max (5 shuffle steps) plus a rescan by the one lane that lost its best.
    float v[32];     // E <= 1024
    const int ni = (E + 31) >> 5;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        const int e = lane + 32 * i;
        v[i] = (i < ni && e < E) ? __ldcg(l + e) : -INFINITY;
    }
    float bv = -INFINITY;
    int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < 32; ++i)          // ascending index: strict > keeps the lowest index
        if (v[i] > bv) { bv = v[i]; bi = lane + 32 * i; }
    float topsum = 0.f, mine_w = 0.f, top0 = 0.f;
    int mine_e = -1;
    for (int j = 0; j < top_k; ++j) {
        float wv = bv;
        int wi = bi;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, wv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, wi, o);
            if (ov > wv || (ov == wv && oi < wi)) { wv = ov; wi = oi; }
        }
        if (j == 0) top0 = wv;
        const float p = __expf(wv - top0);
        topsum += p;
        if (lane == j) { mine_e = wi; mine_w = p; }
        if ((wi & 31) == lane) {          // the winner's lane drops it and looks for its next best
            bv = -INFINITY;
            bi = 0x7fffffff;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                if (i == (wi >> 5)) v[i] = -INFINITY;
                if (v[i] > bv) { bv = v[i]; bi = lane + 32 * i; }
            }
        }
    }
    if (lane < top_k) {
        const int loc = mine_e - e_first;
        const bool local = loc >= 0 && loc < e_local;
        pair_expert[lane] = local ? loc : -1;
        if (stats && local) atomicAdd(stats, 1);          // balance counter: pairs this rank computes in this layer
        pair_w[lane] = mine_w / topsum;
    }
}

struct RouteArgs {
    int E, top_k, F, e_first, e_local;
    int *pair_expert;     // [M][top_k]
    float *pair_w;
    bf16 *sh_h;           // [M][F] or null
    unsigned int *ticket; // zero before the launch; the last block resets it
    // expert weights, so the block that routes can pull the chosen experts into L2 right away
    const char *w13, *w2;
    unsigned long long w13_bytes, w2_bytes;     // per expert
    int prefetch_rows;                           // rows (from 0) whose experts are prefetched
    int *stats;                                  // optional counter of local pairs (MoE balance statistics)
};

// `scratch`: 1056 floats of shared memory the caller does not need any more.
__device__ __forceinline__ void route_all(const float *rs, int ld_rs, int M, const RouteArgs &r, float *scratch) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    float *s_log = scratch, *s_top = scratch + 1024;
    for (int m = warp; m < M; m += nw)
        route_row(rs + (long long)m * ld_rs, r.E, r.top_k, r.e_first, r.e_local, r.pair_expert + m * r.top_k,
                  r.pair_w + m * r.top_k, lane, r.stats);
    (void)s_log; (void)s_top;
    if (r.sh_h) {
        for (int i = threadIdx.x; i < M * r.F; i += blockDim.x) {
            const int m = i / r.F, f = i % r.F;
            const float *l = rs + (long long)m * ld_rs;
            const float sg = sigmoidf_(__ldcg(l + r.E));
            r.sh_h[i] = __float2bfloat16(siluf_(__ldcg(l + r.E + 1 + f)) * __ldcg(l + r.E + 1 + r.F + f) * sg);
        }
    }
}

// Router GEMV (streaming kernel) with the routing done by the block that finishes last.
template <int NT, bool FUSED>
__global__ void __launch_bounds__(SG_THREADS, 1) moe_router_kernel(SGemvArgs a, RouteArgs r) {
    extern __shared__ __align__(128) unsigned char sg_smem[];
    __shared__ unsigned int s_last;
    sgemv_body<NT, FUSED>(a, sg_smem);
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = atomicAdd(r.ticket, 1u) == gridDim.x - 1 ? 1u : 0u;
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    if (r.prefetch_rows < 0) {          // timing diagnostic (QW_SKIP=route_tail): leave the routing tables as they are
        if (threadIdx.x == 0) *r.ticket = 0u;
        return;
    }
    route_all(a.y, a.ldy, a.M, r, reinterpret_cast<float *>(sg_smem + SG_HDR));      // the weight stages are free now
    if (threadIdx.x == 0) *r.ticket = 0u;
}

template <int NT>
static void configure_router_nt() {          // once per device: the kernels' dynamic shared memory opt-in
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (!configured[dev]) {
        cudaFuncSetAttribute(moe_router_kernel<NT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024);
        cudaFuncSetAttribute(moe_router_kernel<NT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024);
        configured[dev] = true;
    }
}
template <int NT>
static cudaError_t launch_router_nt(SGemvArgs &a, const RouteArgs &r, size_t smem, int grid, cudaStream_t s) {
    configure_router_nt<NT>();
    if (a.fi.active) return launch_pdl(moe_router_kernel<NT, true>, dim3(grid), dim3(SG_THREADS), smem, s, a, r);
    return launch_pdl(moe_router_kernel<NT, false>, dim3(grid), dim3(SG_THREADS), smem, s, a, r);
}

static cudaError_t launch_router(SGemvArgs &a, const RouteArgs &r, cudaStream_t s) {
    int grid;
    if (a.M > 8) {
        const size_t smem2 = sgemv_plan(a, 2, grid);
        if (smem2) return launch_router_nt<2>(a, r, smem2, grid, s);
    }
    const size_t smem1 = sgemv_plan(a, 1, grid);
    return launch_router_nt<1>(a, r, smem1, grid, s);
}

// Stand-alone routing (tests, and callers that computed the logits elsewhere).  One block.
// Each block routes 8 rows (a warp per row) and applies the shared activation to them.
__global__ void __launch_bounds__(256) moe_route_kernel(const float *rs, int ld_rs, int M, RouteArgs r) {
    pdl_wait();
    pdl_trigger();
    const int m0 = blockIdx.x * 8;
    const int nm = min(8, M - m0);
    RouteArgs q = r;
    q.pair_expert += m0 * r.top_k;
    q.pair_w += m0 * r.top_k;
    if (q.sh_h) q.sh_h += (long long)m0 * r.F;
    __shared__ float s_route[1056];
    route_all(rs + (long long)m0 * ld_rs, ld_rs, nm, q, s_route);
}

// 32 q4 values (one 16-byte load, engine order) dot 32 bf16 activations.
__device__ __forceinline__ float dot_q4x32(const uint4 w, const uint4 *x) {
    float a = 0.f, e0, e1;
    const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const uint4 xv = x[q];
        q4_pair(ww[q], 0, e0, e1); a = fmaf(e0, bf16_lo(xv.x), a); a = fmaf(e1, bf16_hi(xv.x), a);
        q4_pair(ww[q], 1, e0, e1); a = fmaf(e0, bf16_lo(xv.y), a); a = fmaf(e1, bf16_hi(xv.y), a);
        q4_pair(ww[q], 2, e0, e1); a = fmaf(e0, bf16_lo(xv.z), a); a = fmaf(e1, bf16_hi(xv.z), a);
        q4_pair(ww[q], 3, e0, e1); a = fmaf(e0, bf16_lo(xv.w), a); a = fmaf(e1, bf16_hi(xv.w), a);
    }
    return a;
}

constexpr int GU_T = 5;      // 16-byte pieces per lane over the gate+up row pair: K <= 2560
constexpr int DN_T = 8;      // pieces per lane over top_k down rows: top_k * F/32 <= 256

// h[p][f] = silu(gate_e[f] . x_m) * (up_e[f] . x_m) for pair p = (m, j).  grid (ceil(F/8), pairs).
__global__ void __launch_bounds__(256) moe_gate_up_pair_kernel(const uint32_t *w13, const bf16 *s13, const bf16 *x, int ldx,
                                                               const int *pair_expert, int top_k, int F, int K, bf16 *h, PfArgs pf,
                                                               SharedAct sa, int npairs) {
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
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int f = blockIdx.x * 8 + warp;
    if (f >= F) return;
    const int m = p / top_k;
    const int cpr = K >> 5;                    // 16-byte pieces per row
    const int ks = K >> 7;
    const long long rg = (long long)e * 2 * F + f;
    const uint4 *xr = reinterpret_cast<const uint4 *>(x + (long long)m * ldx);
    uint4 w[GU_T];
    float sc[GU_T];
#pragma unroll
    for (int t = 0; t < GU_T; ++t) {
        const int i = lane + 32 * t;
        if (i < 2 * cpr) {
            const int up = i >= cpr, ch = up ? i - cpr : i;
            const long long row = rg + (up ? F : 0);
            w[t] = ld_stream(reinterpret_cast<const uint4 *>(w13 + row * (K >> 3)) + ch);
            sc[t] = __bfloat162float(s13[row * ks + (ch >> 2)]);
        }
    }
    float g = 0.f, u = 0.f;
#pragma unroll
    for (int t = 0; t < GU_T; ++t) {
        const int i = lane + 32 * t;
        if (i < 2 * cpr) {
            const int up = i >= cpr, ch = up ? i - cpr : i;
            uint4 xv[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) xv[q] = __ldg(xr + ch * 4 + q);
            const float d = sc[t] * dot_q4x32(w[t], xv);
            if (up) u += d; else g += d;
        }
    }
    g = warp_sum(g);
    u = warp_sum(u);
    if (lane == 0) h[(long long)p * F + f] = __float2bfloat16(siluf_(g) * u);
}

// out[m][c] = sum_j w_j * (down_{e_j}[c] . h[p_j]) + shared_down[c] . sh_h[m].  grid (ceil(H/8), M).
template <bool FUSED>
__global__ void __launch_bounds__(256) moe_down_combine_kernel(const uint32_t *w2, const bf16 *s2, const bf16 *h,
                                                               const int *pair_expert, const float *pair_w, int top_k,
                                                               int F, int H, const bf16 *shared_down, int ld_sd,
                                                               const bf16 *sh_h, int SF, float *out, int ldo, PfArgs pf,
                                                               FuseOut fo) {
    pf_issue(pf);
    const int m = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int c = blockIdx.x * 8 + warp;
    // the shared expert's row does not depend on the routing: fetch it before waiting
    uint4 sw[3];
    const int sch = SF >> 3;
    if (shared_down && c < H) {
#pragma unroll
        for (int t = 0; t < 3; ++t)
            if (lane + 32 * t < sch) sw[t] = ld_stream(reinterpret_cast<const uint4 *>(shared_down + (long long)c * ld_sd) + lane + 32 * t);
    }
    pdl_wait();
    pdl_trigger();
    if (c >= H) return;
    const int cpr = F >> 5, ks = F >> 7;
    const int total = top_k * cpr;
    uint4 w[DN_T];
    float sc[DN_T];
#pragma unroll
    for (int t = 0; t < DN_T; ++t) {
        const int i = lane + 32 * t;
        sc[t] = 0.f;
        if (i < total) {
            const int j = i / cpr, ch = i - j * cpr;
            const int p = m * top_k + j;
            const int e = pair_expert[p];
            if (e >= 0) {
                const long long r = (long long)e * H + c;
                w[t] = ld_stream(reinterpret_cast<const uint4 *>(w2 + r * (F >> 3)) + ch);
                sc[t] = __bfloat162float(s2[r * ks + (ch >> 2)]) * pair_w[p];
            } else {
                w[t] = make_uint4(0x88888888u, 0x88888888u, 0x88888888u, 0x88888888u);   // all zeros in q4
            }
        }
    }
    float acc = 0.f;
#pragma unroll
    for (int t = 0; t < DN_T; ++t) {
        const int i = lane + 32 * t;
        if (i < total) {
            const int j = i / cpr, ch = i - j * cpr;
            const uint4 *hp = reinterpret_cast<const uint4 *>(h + (long long)(m * top_k + j) * F) + ch * 4;
            uint4 xv[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) xv[q] = __ldg(hp + q);
            acc = fmaf(sc[t], dot_q4x32(w[t], xv), acc);
        }
    }
    if (shared_down) {
        const uint4 *xp = reinterpret_cast<const uint4 *>(sh_h + (long long)m * SF);
        float a = 0.f;
#pragma unroll
        for (int t = 0; t < 3; ++t)
            if (lane + 32 * t < sch) a = dot8(sw[t], __ldg(xp + lane + 32 * t), a);
        acc += a;
    }
    acc = warp_sum(acc);
    if (lane == 0) {
        if (FUSED) fuse_put_col(fo, fuse_seq(fo), m, c, __float_as_uint(acc));      // fused reduce-scatter: to the column's owner
        else out[(long long)m * ldo + c] = acc;
    }
}

}  // namespace qw

using namespace qw;

// Which form of the routed-expert kernels runs: bit 0 / 1 = gate-up / down on the tensor cores with direct loads,
// bit 2 / 3 = gate-up / down on the tensor cores fed by bulk-async row copies (wins over bits 0 / 1), 0 = scalar kernels.
// Default 12, measured inside the decode graph on the full model: scalar 5.37 ms per step, direct-load tensor-core forms
// 5.37 / 5.7, bulk-copy-fed forms 4.85.  QW_MOE_MMA overrides at start-up, qwk_set_moe_mma at run time.
static int g_moe_mma = -1;
static int moe_mma_mask() {
    if (g_moe_mma < 0) {
        const char *e = getenv("QW_MOE_MMA");
        g_moe_mma = e ? atoi(e) & 15 : 12;
    }
    return g_moe_mma;
}
QW_API int qwk_set_moe_mma(int mask) {
    g_moe_mma = mask & 15;
    return 0;
}

static RouteArgs make_route(int E, int top_k, int F, int e_first, int e_local, int *pair_expert, float *pair_w,
                            void *sh_h, unsigned int *ticket) {
    RouteArgs r;
    r.E = E; r.top_k = top_k; r.F = F; r.e_first = e_first; r.e_local = e_local;
    r.pair_expert = pair_expert; r.pair_w = pair_w; r.sh_h = (bf16 *)sh_h; r.ticket = ticket;
    r.w13 = r.w2 = nullptr; r.w13_bytes = r.w2_bytes = 0; r.prefetch_rows = 0;
    r.stats = qw::g_moe_stats;
    qw::g_moe_stats = nullptr;
    return r;
}

// rs = Wrs . x, then routing + shared activation in the same launch.  `ticket` is one zeroed word.
QW_API int qwk_moe_router(const void *Wrs, const void *x, float *rs, int nrs, int K, int M, int ldx, int E, int top_k,
                          int F, int e_first, int e_local, int *pair_expert, float *pair_w, void *sh_h,
                          unsigned int *ticket, const void *w13, const void *w2, long long w13_bytes, long long w2_bytes,
                          cudaStream_t s) {
    if (E > 1024 || top_k > 32 || (K & 15) || (ldx & 7)) return -1;
    SGemvArgs a;
    a.W = (const bf16 *)Wrs; a.x = (const bf16 *)x; a.y = rs; a.y_bf16 = nullptr;
    a.N = nrs; a.K = K; a.M = M; a.ldw = K; a.ldx = ldx; a.ldy = nrs; a.accumulate = 0; a.nsplit = 1; a.w_split = 0; a.err = g_err_ptr; a.pf = take_pf();
    a.fi = take_fi();
    RouteArgs r = make_route(E, top_k, F, e_first, e_local, pair_expert, pair_w, sh_h, ticket);
    r.w13 = (const char *)w13; r.w2 = (const char *)w2; r.w13_bytes = w13_bytes; r.w2_bytes = w2_bytes;
    r.prefetch_rows = 0;
#ifdef QW_DIAG
    {          // timing instrument: QW_SKIP=route_tail leaves the routing tables as they are
        static int skip_tail = -1;
        if (skip_tail < 0) { const char *e = getenv("QW_SKIP"); skip_tail = e && strstr(e, "route_tail") ? 1 : 0; }
        if (skip_tail) r.prefetch_rows = -1;
    }
#endif
    const cudaError_t e = launch_router(a, r, s);
    return e == cudaSuccess ? 0 : -2;
}

QW_API int qwk_moe_route(const float *rs, int ld_rs, int M, int E, int top_k, int F, int e_first, int e_local,
                         int *pair_expert, float *pair_w, void *sh_h, cudaStream_t s) {
    if (E > 1024 || top_k > 32) return -1;
    RouteArgs r = make_route(E, top_k, F, e_first, e_local, pair_expert, pair_w, sh_h, nullptr);
    cudaError_t e = launch_pdl(moe_route_kernel, dim3((M + 7) / 8), dim3(256), 0, s, rs, ld_rs, M, r);
    return e == cudaSuccess ? 0 : -2;
}

QW_API int qwk_moe_gate_up_pair(const void *w13, const void *s13, const void *x, int ldx, const int *pair_expert, int M,
                                int top_k, int F, int K, void *h, cudaStream_t s) {
    if ((K & 127) || (ldx & 7)) return -1;
    const SharedAct sa = take_shared_act();
    const int extra = sa.rs ? M : 0;          // one extra grid row per token for the shared expert's activation
    if ((moe_mma_mask() & 4) && (F & 15) == 0 && (K & 127) == 0) {
        // bulk-copy-fed tensor-core form
        const int ks = K >> 7;
        const size_t smem = 128 + 2 * 16 * ((size_t)(K >> 1) + TM_PAD) + 2 * 16 * ks * 2 + 16 + (size_t)(K >> 3) * 16 + 16 * 2 * 16 * sizeof(float);
        static bool attr[64] = {};
        int dev = 0;
        cudaGetDevice(&dev);
        if (dev < 0 || dev >= 64) dev = 0;
        if (!attr[dev]) {
            cudaFuncSetAttribute(moe_gate_up_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
            attr[dev] = true;
        }
        if (smem <= 100 * 1024) {
            cudaError_t e = launch_pdl(moe_gate_up_tma_kernel, dim3(F / 16, M * top_k + extra), dim3(512), smem, s, (const uint32_t *)w13,
                                       (const bf16 *)s13, (const bf16 *)x, ldx, pair_expert, top_k, F, K, (bf16 *)h, g_err_ptr, sa, M * top_k);
            return e == cudaSuccess ? 0 : -2;
        }
    }
    if ((moe_mma_mask() & 1) && (F & 15) == 0 && (K >> 7) <= MM_WARPS * GU_NG) {
        // tensor-core form: 16 rows of gate and of up per block
        const size_t smem = (size_t)K * 2 + MM_WARPS * 2 * 16 * sizeof(float);
        cudaError_t e = launch_pdl(moe_gate_up_mma_kernel, dim3(F / 16, M * top_k + extra), dim3(128), smem, s, (const uint32_t *)w13,
                                   (const bf16 *)s13, (const bf16 *)x, ldx, pair_expert, top_k, F, K, (bf16 *)h, take_pf(), sa, M * top_k);
        return e == cudaSuccess ? 0 : -2;
    }
    if (2 * (K >> 5) > 32 * GU_T) return -1;
    dim3 grid((F + 7) / 8, M * top_k + extra);
    cudaError_t e = launch_pdl(moe_gate_up_pair_kernel, grid, dim3(256), 0, s, (const uint32_t *)w13, (const bf16 *)s13,
                               (const bf16 *)x, ldx, pair_expert, top_k, F, K, (bf16 *)h, take_pf(), sa, M * top_k);
    return e == cudaSuccess ? 0 : -2;
}

QW_API int qwk_moe_down_combine(const void *w2, const void *s2, const void *h, const int *pair_expert,
                                const float *pair_w, int M, int top_k, int F, int H, const void *shared_down, int ld_sd,
                                const void *sh_h, int SF, float *out, int ldo, cudaStream_t s) {
    if ((F & 127) || (SF & 7)) return -1;
    const FuseOut fo = take_fo();
    if ((moe_mma_mask() & 8) && (H & 15) == 0 && (F & 127) == 0 && (SF & 7) == 0 && (ld_sd & 7) == 0 && top_k <= 32) {
        // bulk-copy-fed tensor-core form
        const int ks = F >> 7;
        const size_t smem = 128 + (size_t)top_k * 16 * ((F >> 1) + TM_PAD) + (shared_down ? 16 * ((size_t)SF * 2 + TM_PAD) : 0) +
                            (size_t)top_k * (((16 * ks * 2) + 15) & ~15) + ((size_t)top_k * (F >> 3) + (SF >> 3)) * 16 + 16 * 16 * 4 + 32 * 4 + 32 * 4;
        static bool attr = false;
        if (!attr) {
            cudaFuncSetAttribute(moe_down_tma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 110 * 1024);
            cudaFuncSetAttribute(moe_down_tma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 110 * 1024);
            attr = true;
        }
        if (smem <= 110 * 1024) {
            const dim3 g2(H / 16, M);
            cudaError_t e = fo.mode ? launch_pdl(moe_down_tma_kernel<true>, g2, dim3(512), smem, s, (const uint32_t *)w2, (const bf16 *)s2,
                                                 (const bf16 *)h, pair_expert, pair_w, top_k, F, H, (const bf16 *)shared_down, ld_sd,
                                                 (const bf16 *)sh_h, SF, out, ldo, g_err_ptr, fo)
                                    : launch_pdl(moe_down_tma_kernel<false>, g2, dim3(512), smem, s, (const uint32_t *)w2, (const bf16 *)s2,
                                                 (const bf16 *)h, pair_expert, pair_w, top_k, F, H, (const bf16 *)shared_down, ld_sd,
                                                 (const bf16 *)sh_h, SF, out, ldo, g_err_ptr, fo);
            return e == cudaSuccess ? 0 : -2;
        }
    }
    if ((moe_mma_mask() & 2) && (H & 15) == 0 && top_k * (F >> 7) <= MM_WARPS * DN_NI && (SF >> 5) <= MM_WARPS * DN_NS && (ld_sd & 7) == 0) {
        // tensor-core form: 16 output columns per block
        const size_t smem = ((size_t)top_k * (F >> 3) + (SF >> 3)) * 16 + MM_WARPS * 16 * sizeof(float);
        if (smem <= 48 * 1024) {
            const dim3 g2(H / 16, M);
            cudaError_t e = fo.mode ? launch_pdl(moe_down_mma_kernel<true>, g2, dim3(128), smem, s, (const uint32_t *)w2, (const bf16 *)s2,
                                                 (const bf16 *)h, pair_expert, pair_w, top_k, F, H, (const bf16 *)shared_down, ld_sd,
                                                 (const bf16 *)sh_h, SF, out, ldo, take_pf(), fo)
                                    : launch_pdl(moe_down_mma_kernel<false>, g2, dim3(128), smem, s, (const uint32_t *)w2, (const bf16 *)s2,
                                                 (const bf16 *)h, pair_expert, pair_w, top_k, F, H, (const bf16 *)shared_down, ld_sd,
                                                 (const bf16 *)sh_h, SF, out, ldo, take_pf(), fo);
            return e == cudaSuccess ? 0 : -2;
        }
    }
    if (top_k * (F >> 5) > 32 * DN_T || (SF >> 3) > 96) return -1;
    dim3 grid((H + 7) / 8, M);
    cudaError_t e = fo.mode ? launch_pdl(moe_down_combine_kernel<true>, grid, dim3(256), 0, s, (const uint32_t *)w2, (const bf16 *)s2,
                                         (const bf16 *)h, pair_expert, pair_w, top_k, F, H, (const bf16 *)shared_down, ld_sd,
                                         (const bf16 *)sh_h, SF, out, ldo, take_pf(), fo)
                            : launch_pdl(moe_down_combine_kernel<false>, grid, dim3(256), 0, s, (const uint32_t *)w2, (const bf16 *)s2,
                                         (const bf16 *)h, pair_expert, pair_w, top_k, F, H, (const bf16 *)shared_down, ld_sd,
                                         (const bf16 *)sh_h, SF, out, ldo, take_pf(), fo);
    return e == cudaSuccess ? 0 : -2;
}

// ---------------------------------------------------------------------------------------------------
// qwk_moe_router_static: the router launch for callers that may not allocate device memory.
// Declared and documented in no_alloc.h.  The scratch (router outputs + the block ticket) lives in this
// file-scope array, whose address is looked up once per device.
// ---------------------------------------------------------------------------------------------------
#include "no_alloc.h"

static __device__ __align__(256) unsigned char g_router_static_scratch[QWK_ROUTER_STATIC_SCRATCH_BYTES];
static unsigned char *g_router_static_ptr[QWK_ROUTER_STATIC_MAX_DEVICES];     // per device, null until set up

extern "C" __attribute__((visibility("default"))) int qwk_moe_router_static_setup(void) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= QWK_ROUTER_STATIC_MAX_DEVICES) return -3;
    if (g_router_static_ptr[dev]) return 0;
    unsigned char *p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress((void **)&p, g_router_static_scratch);
    if (e != cudaSuccess || p == nullptr) return -3;
    g_router_static_ptr[dev] = p;
    configure_router_nt<1>();          // the kernels' attributes too, so that a first call inside a capture has nothing left to set up
    configure_router_nt<2>();
    return 0;
}

extern "C" __attribute__((visibility("default"))) int qwk_moe_router_static(const void *Wrs, const void *x, int nrs, int K, int M, int ldx, int E, int top_k, int F,
                                 int e_first, int e_local, int *pair_expert, float *pair_w, void *sh_h, cudaStream_t s) {
    if (E > 1024 || top_k > 32 || (K & 15) || (ldx & 7)) return -1;
    if (M < 1 || M > QWK_ROUTER_STATIC_MAX_ROWS || nrs < 1 || nrs > QWK_ROUTER_STATIC_MAX_OUTPUTS) return -4;
    // the routing reads E logits of a row and, for the shared activation, the gate logit and 2 F more outputs behind them
    if (nrs < E + (sh_h ? 1 + 2 * F : 0)) return -1;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= QWK_ROUTER_STATIC_MAX_DEVICES) return -3;
    if (!g_router_static_ptr[dev] && qwk_moe_router_static_setup() != 0) return -3;
    unsigned char *base = g_router_static_ptr[dev];
    unsigned int *ticket = (unsigned int *)base;                       // first 256 bytes: the ticket word
    float *rs = (float *)(base + 256);                                 // then [M][nrs] router outputs
    // The ticket has to be zero when the kernel starts.  A finished launch leaves it at zero; the clear is
    // for the launch that did not finish (an earlier error on the stream).
    if (cudaMemsetAsync(ticket, 0, sizeof(unsigned int), s) != cudaSuccess) return -2;
    SGemvArgs a;
    a.W = (const bf16 *)Wrs; a.x = (const bf16 *)x; a.y = rs; a.y_bf16 = nullptr;
    a.N = nrs; a.K = K; a.M = M; a.ldw = K; a.ldx = ldx; a.ldy = nrs; a.accumulate = 0; a.nsplit = 1; a.w_split = 0; a.err = g_err_ptr; a.pf = take_pf();
    RouteArgs r = make_route(E, top_k, F, e_first, e_local, pair_expert, pair_w, sh_h, ticket);
    r.w13 = nullptr; r.w2 = nullptr; r.w13_bytes = 0; r.w2_bytes = 0; r.prefetch_rows = 0;
    const cudaError_t e = launch_router(a, r, s);
    return e == cudaSuccess ? 0 : -2;
}
