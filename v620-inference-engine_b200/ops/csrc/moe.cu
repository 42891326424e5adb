// Decode-path MoE kernels: router (softmax, top-k by repeated argmax with ties to the lowest
// index, renormalisation, expert-parallel filter), the shared expert's gated activation, and
// the per-(row, expert) q4 matrix-vector products with the weighted combine fused into the down
// projection (roles of the reference's src/kernels/moe_route.hip:65-224 and
// src/kernels/moe_experts.hip:189-246).
#include "common.cuh"

namespace qw {

constexpr int MAX_TOPK = 16;

// One block per row.  Warp 0 routes; all threads then apply the shared expert's activation.
// rs[m] = [ router logits (E) | shared gate logit (1) | shared gate rows (F) | shared up rows (F) ].
__global__ void __launch_bounds__(256) moe_route_kernel(const float *rs, int ld_rs, int E, int top_k, int F, int e_first,
                                                        int e_local, int *pair_expert, float *pair_w, bf16 *sh_h) {
    const int m = blockIdx.x;
    const float *l = rs + (long long)m * ld_rs;
    const int lane = threadIdx.x & 31;
    if (threadIdx.x < 32) {
        float v[32];     // E <= 1024
        float mx = -INFINITY;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            const int e = lane + 32 * i;
            v[i] = e < E ? l[e] : -INFINITY;
            mx = fmaxf(mx, v[i]);
        }
        mx = warp_max(mx);
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = (lane + 32 * i) < E ? expf(v[i] - mx) : -1.f;
        float topsum = 0.f, mine_w = 0.f;
        int mine_e = -1;
        for (int j = 0; j < top_k; ++j) {
            float bv = -1.f;
            int bi = 0x7fffffff;
#pragma unroll
            for (int i = 0; i < 32; ++i) {      // ascending index: strict > keeps the lowest index
                if (v[i] > bv) { bv = v[i]; bi = lane + 32 * i; }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
            }
            topsum += bv;
            if (lane == j) { mine_e = bi; mine_w = bv; }
            if ((bi & 31) == lane) {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    if (i == (bi >> 5)) v[i] = -1.f;
            }
        }
        if (lane < top_k) {
            const int loc = mine_e - e_first;
            const bool local = loc >= 0 && loc < e_local;
            pair_expert[m * top_k + lane] = local ? loc : -1;
            pair_w[m * top_k + lane] = mine_w / topsum;
        }
    }
    if (sh_h) {
        const float sg = sigmoidf_(l[E]);
        for (int f = threadIdx.x; f < F; f += blockDim.x)
            sh_h[(long long)m * F + f] = __float2bfloat16(siluf_(l[E + 1 + f]) * l[E + 1 + F + f] * sg);
    }
}

// integer dot of 16 q4 values (2 words) with 16 bf16 activations
__device__ __forceinline__ float dot_q4x16(const uint2 w, const uint4 x0, const uint4 x1) {
    float a = 0.f, e0, e1;
    q4_pair(w.x, 0, e0, e1); a = fmaf(e0, bf16_lo(x0.x), a); a = fmaf(e1, bf16_hi(x0.x), a);
    q4_pair(w.x, 1, e0, e1); a = fmaf(e0, bf16_lo(x0.y), a); a = fmaf(e1, bf16_hi(x0.y), a);
    q4_pair(w.x, 2, e0, e1); a = fmaf(e0, bf16_lo(x0.z), a); a = fmaf(e1, bf16_hi(x0.z), a);
    q4_pair(w.x, 3, e0, e1); a = fmaf(e0, bf16_lo(x0.w), a); a = fmaf(e1, bf16_hi(x0.w), a);
    q4_pair(w.y, 0, e0, e1); a = fmaf(e0, bf16_lo(x1.x), a); a = fmaf(e1, bf16_hi(x1.x), a);
    q4_pair(w.y, 1, e0, e1); a = fmaf(e0, bf16_lo(x1.y), a); a = fmaf(e1, bf16_hi(x1.y), a);
    q4_pair(w.y, 2, e0, e1); a = fmaf(e0, bf16_lo(x1.z), a); a = fmaf(e1, bf16_hi(x1.z), a);
    q4_pair(w.y, 3, e0, e1); a = fmaf(e0, bf16_lo(x1.w), a); a = fmaf(e1, bf16_hi(x1.w), a);
    return a;
}

// q4 row (K values) dot bf16 activation row; lanes stride over 16-element pieces.
__device__ __forceinline__ float q4_row_dot(const uint32_t *wrow, const bf16 *srow, const bf16 *x, int K, int lane) {
    float acc = 0.f;
    const int pieces = K >> 4;
    for (int i = lane; i < pieces; i += 32) {
        const uint2 w = ld_stream8(wrow + 2 * i);
        const float sc = __bfloat162float(srow[i >> 3]);
        const uint4 x0 = __ldg(reinterpret_cast<const uint4 *>(x) + 2 * i);
        const uint4 x1 = __ldg(reinterpret_cast<const uint4 *>(x) + 2 * i + 1);
        acc = fmaf(sc, dot_q4x16(w, x0, x1), acc);
    }
    return acc;
}

// h[p][f] = silu(gate_e[f] . x_m) * (up_e[f] . x_m) for pair p = (m, j).  grid (ceil(F/8), pairs).
__global__ void __launch_bounds__(256) moe_gate_up_pair_kernel(const uint32_t *w13, const bf16 *s13, const bf16 *x, int ldx,
                                                               const int *pair_expert, int top_k, int F, int K, bf16 *h) {
    const int p = blockIdx.y;
    const int e = pair_expert[p];
    if (e < 0) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int f = blockIdx.x * 8 + warp;
    if (f >= F) return;
    const int m = p / top_k;
    const long long rg = (long long)e * 2 * F + f, ru = rg + F;
    const int kw = K >> 3, ks = K >> 7;
    const bf16 *xr = x + (long long)m * ldx;
    float g = q4_row_dot(w13 + rg * kw, s13 + rg * ks, xr, K, lane);
    float u = q4_row_dot(w13 + ru * kw, s13 + ru * ks, xr, K, lane);
    g = warp_sum(g);
    u = warp_sum(u);
    if (lane == 0) h[(long long)p * F + f] = __float2bfloat16(siluf_(g) * u);
}

// out[m][c] = sum_j w_j * (down_{e_j}[c] . h[p_j]) + shared_down[c] . sh_h[m].  grid (ceil(H/8), M).
__global__ void __launch_bounds__(256) moe_down_combine_kernel(const uint32_t *w2, const bf16 *s2, const bf16 *h,
                                                               const int *pair_expert, const float *pair_w, int top_k,
                                                               int F, int H, const bf16 *shared_down, int ld_sd,
                                                               const bf16 *sh_h, int SF, float *out, int ldo) {
    const int m = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int c = blockIdx.x * 8 + warp;
    if (c >= H) return;
    const int kw = F >> 3, ks = F >> 7;
    float acc = 0.f;
    for (int j = 0; j < top_k; ++j) {
        const int p = m * top_k + j;
        const int e = pair_expert[p];
        if (e < 0) continue;
        const long long r = (long long)e * H + c;
        const float d = q4_row_dot(w2 + r * kw, s2 + r * ks, h + (long long)p * F, F, lane);
        acc = fmaf(pair_w[p], d, acc);
    }
    if (shared_down) {
        const uint4 *wp = reinterpret_cast<const uint4 *>(shared_down + (long long)c * ld_sd);
        const uint4 *xp = reinterpret_cast<const uint4 *>(sh_h + (long long)m * SF);
        float a = 0.f;
        for (int i = lane; i < (SF >> 3); i += 32) a = dot8(ld_stream(wp + i), __ldg(xp + i), a);
        acc += a;
    }
    acc = warp_sum(acc);
    if (lane == 0) out[(long long)m * ldo + c] = acc;
}

}  // namespace qw

using namespace qw;

QW_API int qwk_moe_route(const float *rs, int ld_rs, int M, int E, int top_k, int F, int e_first, int e_local,
                         int *pair_expert, float *pair_w, void *sh_h, cudaStream_t s) {
    if (E > 1024 || top_k > 32 || top_k > MAX_TOPK) return -1;
    moe_route_kernel<<<M, 256, 0, s>>>(rs, ld_rs, E, top_k, F, e_first, e_local, pair_expert, pair_w, (bf16 *)sh_h);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

QW_API int qwk_moe_gate_up_pair(const void *w13, const void *s13, const void *x, int ldx, const int *pair_expert, int M,
                                int top_k, int F, int K, void *h, cudaStream_t s) {
    if ((K & 127) || (ldx & 7)) return -1;
    dim3 grid((F + 7) / 8, M * top_k);
    moe_gate_up_pair_kernel<<<grid, 256, 0, s>>>((const uint32_t *)w13, (const bf16 *)s13, (const bf16 *)x, ldx,
                                                 pair_expert, top_k, F, K, (bf16 *)h);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

QW_API int qwk_moe_down_combine(const void *w2, const void *s2, const void *h, const int *pair_expert,
                                const float *pair_w, int M, int top_k, int F, int H, const void *shared_down, int ld_sd,
                                const void *sh_h, int SF, float *out, int ldo, cudaStream_t s) {
    if ((F & 127) || (SF & 7)) return -1;
    dim3 grid((H + 7) / 8, M);
    moe_down_combine_kernel<<<grid, 256, 0, s>>>((const uint32_t *)w2, (const bf16 *)s2, (const bf16 *)h, pair_expert,
                                                 pair_w, top_k, F, H, (const bf16 *)shared_down, ld_sd,
                                                 (const bf16 *)sh_h, SF, out, ldo);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
