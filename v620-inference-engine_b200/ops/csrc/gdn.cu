// Gated delta net kernels for row batches: causal depthwise conv + gating + per-head L2 norm,
// and the recurrent delta-rule update with the gated output norm fused in
// (roles of the reference's src/kernels/gdn.hip:174-309; math in docs/MODEL.md:108-133).
//
// Per-rank layout of the projection output row (fp32): [ q (KL heads) | k (KL heads) | v (VL heads) |
// z (VL heads x 128) | b (VL) | a (VL) ], head dim 128.
#include "common.cuh"

namespace qw {

constexpr int GD = 128;      // GDN head dim

struct GdnConvArgs {
    const float *proj;       // [M][ld_proj]
    int ld_proj;
    float *ring;             // [slots][GDN_RING][qkv_l] pre-conv rows of this layer
    const float *cw;         // [qkv_l][4] conv taps (oldest first)
    const float *A_log, *dt_bias;   // [VL]
    int KL, VL;
    Rows rows;
    float *qkv;              // [M][qkv_l] conv output: q (normed, scaled) | k (normed) | v
    float *decay, *beta;     // [M][VL]
    float eps;
};

// Pre-conv value of channel c at `back` rows before row m: from this batch while that row belongs to m's run, else from
// the slot's ring (positions before the run), else zero (before the sequence's start).
__device__ __forceinline__ float gdn_preconv(const GdnConvArgs &a, const float *ring, int qkv_l, int m, int rs, int pos,
                                             int back, int c) {
    if (m - back >= rs) return a.proj[(long long)(m - back) * a.ld_proj + c];
    const int q = pos - back;
    return q >= 0 ? ring[(q % GDN_RING) * qkv_l + c] : 0.f;
}

constexpr int CONV_ROWS = 8;     // rows of the batch per block

// grid (ceil(M / 8), 2*KL+VL), 128 threads: one head and eight consecutive rows per block.  The four-tap window slides
// down the rows in registers (one new load per row while the rows stay in one run).
__global__ void __launch_bounds__(128) gdn_conv_kernel(GdnConvArgs a) {
    __shared__ float scratch[32];
    const int m_first = blockIdx.x * CONV_ROWS, head = blockIdx.y, d = threadIdx.x;
    const int qkv_l = (2 * a.KL + a.VL) * GD;
    const int c = head * GD + d;
    float tap[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) tap[k] = a.cw[c * 4 + k];
    float w0 = 0.f, w1 = 0.f, w2 = 0.f;      // values 3, 2, 1 rows back
    int prev_rs = -1;
    for (int i = 0; i < CONV_ROWS; ++i) {
        const int m = m_first + i;
        if (m >= a.rows.M) break;                // uniform for the block
        const int slot = a.rows.slot[m], pos = a.rows.pos[m], rs = a.rows.run_start[m];
        const float *ring = a.ring + (long long)slot * GDN_RING * qkv_l;
        if (i == 0 || rs != prev_rs || m == rs) {
            w0 = gdn_preconv(a, ring, qkv_l, m, rs, pos, 3, c);
            w1 = gdn_preconv(a, ring, qkv_l, m, rs, pos, 2, c);
            w2 = gdn_preconv(a, ring, qkv_l, m, rs, pos, 1, c);
        }
        prev_rs = rs;
        const float cur = a.proj[(long long)m * a.ld_proj + c];
        const float acc = fmaf(tap[3], cur, fmaf(tap[2], w2, fmaf(tap[1], w1, tap[0] * w0)));
        w0 = w1; w1 = w2; w2 = cur;
        float v = siluf_(acc);
        if (head < 2 * a.KL) {
            const float ss = block_sum<128>(v * v, scratch);
            v = v / sqrtf(ss + a.eps);
            if (head < a.KL) v *= 0.08838834764831845f;    // 1/sqrt(128)
        }
        a.qkv[(long long)m * qkv_l + c] = v;
        if (head == 0 && d < a.VL) {
            const float *row = a.proj + (long long)m * a.ld_proj + qkv_l + a.VL * GD;
            const float bb = row[d], aa = row[a.VL + d];
            const float g = -__expf(a.A_log[d]) * softplusf_(aa + a.dt_bias[d]);
            a.decay[m * a.VL + d] = __expf(g);
            a.beta[m * a.VL + d] = sigmoidf_(bb);
        }
    }
}

// Stores the batch's pre-conv rows into the ring (after gdn_conv has read the old entries).
// grid (M, ceil(qkv_l/256)).
__global__ void gdn_ring_kernel(const float *proj, int ld_proj, float *ring, int qkv_l, Rows rows, int m_first) {
    const int m = m_first + blockIdx.x;
    const int c = blockIdx.y * 256 + threadIdx.x;
    if (c >= qkv_l) return;
    const int slot = rows.slot[m], pos = rows.pos[m];
    // a run longer than the ring keeps only its last GDN_RING rows
    const int rs = rows.run_start[m], len = rows.run_len[rs];
    if (m - rs < len - GDN_RING) return;
    ring[((long long)slot * GDN_RING + (pos % GDN_RING)) * qkv_l + c] = proj[(long long)m * ld_proj + c];
}

struct GdnScanArgs {
    const float *qkv;        // [M][qkv_l]
    const float *decay, *beta;   // [M][VL]
    const float *proj;       // for z: proj[m][qkv_l + h*128 + d]
    int ld_proj;
    float *S;                // [slots][VL][128 k][128 v] state of this layer
    float *save;             // optional [M][VL][128][128]: state after each row (speculative rollback)
    const float *norm_w;     // [128]
    int KL, VL;
    Rows rows;
    bf16 *o;                 // [M][VL*128] gated, normed output
    float eps;
};

// grid (M, VL), 512 threads.  Only the first row of a run does work; it walks the run's rows.
// Thread (kg = tid/128, c = tid%128) holds S[kg*32 .. +32][c].
__global__ void __launch_bounds__(512) gdn_scan_kernel(GdnScanArgs a) {
    __shared__ float kq[2][GD];        // k and q of the row
    __shared__ float red[4][GD];
    __shared__ float scratch[32];
    const int m0 = blockIdx.x, h = blockIdx.y;
    if (a.rows.run_start[m0] != m0) return;
    const int len = a.rows.run_len[m0], slot = a.rows.slot[m0];
    const int tid = threadIdx.x, c = tid & 127, kg = tid >> 7;
    const int qkv_l = (2 * a.KL + a.VL) * GD;
    const int kh = h / (a.VL / a.KL);
    float *Sg = a.S + ((long long)slot * a.VL + h) * GD * GD;
    float S[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) S[i] = Sg[(kg * 32 + i) * GD + c];
    for (int r = 0; r < len; ++r) {
        const int m = m0 + r;
        const float *row = a.qkv + (long long)m * qkv_l;
        __syncthreads();
        if (tid < GD) kq[0][tid] = row[(a.KL + kh) * GD + tid];
        else if (tid < 2 * GD) kq[1][tid - GD] = row[kh * GD + (tid - GD)];
        __syncthreads();
        const float dec = a.decay[m * a.VL + h], be = a.beta[m * a.VL + h];
        float p = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            S[i] *= dec;
            p = fmaf(S[i], kq[0][kg * 32 + i], p);
        }
        red[kg][c] = p;
        __syncthreads();
        const float stk = red[0][c] + red[1][c] + red[2][c] + red[3][c];
        const float u = (row[2 * a.KL * GD + h * GD + c] - stk) * be;
        float oq = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            S[i] = fmaf(kq[0][kg * 32 + i], u, S[i]);
            oq = fmaf(S[i], kq[1][kg * 32 + i], oq);
        }
        __syncthreads();
        red[kg][c] = oq;
        __syncthreads();
        if (a.save) {
            float *sv = a.save + ((long long)m * a.VL + h) * GD * GD;
#pragma unroll
            for (int i = 0; i < 32; ++i) sv[(kg * 32 + i) * GD + c] = S[i];
        }
        // gated rms norm over the head's 128 outputs
        float ov = 0.f;
        if (kg == 0) ov = red[0][c] + red[1][c] + red[2][c] + red[3][c];
        const float ss = block_sum<512>(ov * ov, scratch);
        if (kg == 0) {
            const float z = a.proj[(long long)m * a.ld_proj + qkv_l + h * GD + c];
            const float y = ov * rsqrtf(ss / float(GD) + a.eps) * a.norm_w[c] * sigmoidf_(z);
            a.o[(long long)m * a.VL * GD + h * GD + c] = __float2bfloat16(y);
        }
    }
#pragma unroll
    for (int i = 0; i < 32; ++i) Sg[(kg * 32 + i) * GD + c] = S[i];
}

// ------------------------------------------------------------------------------------------
// Fused decode step for short runs (M <= GDN_RING - 4): conv + gating + L2 norm + delta-rule update +
// gated norm in one kernel, and the ring store.  grid (M, VL), 512 threads; the block of (run start,
// head h) walks the run.  q/k of the head's key head are recomputed by each of the value heads that
// share it.  Ring entries written here (positions of the run) never alias the entries read
// (positions before the run) because the run is shorter than the ring minus the conv window.
// ------------------------------------------------------------------------------------------
struct GdnFusedArgs {
    const float *proj;
    int ld_proj;
    float *ring;
    const float *cw, *A_log, *dt_bias, *norm_w;
    int KL, VL;
    Rows rows;
    float *S, *save;
    bf16 *o;
    float eps;
    PfArgs pf;
};

__global__ void __launch_bounds__(512) gdn_fused_kernel(GdnFusedArgs a) {
    __shared__ float kq[2][GD];
    __shared__ float vv[GD];
    __shared__ float red[4][GD];
    __shared__ float scratch[32];
    __shared__ float s_gate[2];
    const int m0 = blockIdx.x, h = blockIdx.y;
    const int tid = threadIdx.x, c = tid & 127, kg = tid >> 7;
    const int qkv_l = (2 * a.KL + a.VL) * GD;
    const int rep = a.VL / a.KL, kh = h / rep;
    // conv taps of this thread's channel (weights: independent of the predecessor)
    int ch = -1;
    if (kg == 0) ch = kh * GD + c;                       // q
    else if (kg == 1) ch = (a.KL + kh) * GD + c;         // k
    else if (kg == 2) ch = (2 * a.KL + h) * GD + c;      // v
    float tap[4] = {0.f, 0.f, 0.f, 0.f};
    if (ch >= 0) {
#pragma unroll
        for (int k = 0; k < 4; ++k) tap[k] = a.cw[ch * 4 + k];
    }
    pf_issue(a.pf);
    // The row table was written before the step began and the recurrent state only by this kernel in the previous step:
    // neither depends on the predecessor, so the state (64 KB per head, from HBM) is fetched before waiting for it.
    if (a.rows.run_start[m0] != m0) return;
    const int len = a.rows.run_len[m0], slot = a.rows.slot[m0];
    float *ring = a.ring + (long long)slot * GDN_RING * qkv_l;
    float *Sg = a.S + ((long long)slot * a.VL + h) * GD * GD;
    float S[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) S[i] = Sg[(kg * 32 + i) * GD + c];
    pdl_wait();
    pdl_trigger();
    for (int r = 0; r < len; ++r) {
        const int m = m0 + r, pos = a.rows.pos[m];
        // conv + silu for q / k / v channels
        float val = 0.f;
        if (ch >= 0) {
            float acc = 0.f;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int back = 3 - k, q = pos - back;
                float x;
                if (r - back >= 0) x = a.proj[(long long)(m - back) * a.ld_proj + ch];
                else if (q >= 0) x = ring[(q % GDN_RING) * qkv_l + ch];
                else x = 0.f;
                acc = fmaf(tap[k], x, acc);
            }
            val = siluf_(acc);
        }
        // L2 norms of q (warps 0-3) and k (warps 4-7)
        const float ssw = warp_sum(kg < 2 ? val * val : 0.f);
        __syncthreads();
        if ((tid & 31) == 0) scratch[tid >> 5] = ssw;
        if (tid == 0) {
            const float *row = a.proj + (long long)m * a.ld_proj + qkv_l + a.VL * GD;
            const float g = -__expf(a.A_log[h]) * softplusf_(row[a.VL + h] + a.dt_bias[h]);
            s_gate[0] = __expf(g);
            s_gate[1] = sigmoidf_(row[h]);
        }
        __syncthreads();
        if (kg == 0) {
            const float ss = scratch[0] + scratch[1] + scratch[2] + scratch[3];
            kq[1][c] = val / sqrtf(ss + a.eps) * 0.08838834764831845f;
        } else if (kg == 1) {
            const float ss = scratch[4] + scratch[5] + scratch[6] + scratch[7];
            kq[0][c] = val / sqrtf(ss + a.eps);
        } else if (kg == 2) {
            vv[c] = val;
        }
        __syncthreads();
        const float dec = s_gate[0], be = s_gate[1];
        float p = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            S[i] *= dec;
            p = fmaf(S[i], kq[0][kg * 32 + i], p);
        }
        red[kg][c] = p;
        __syncthreads();
        const float stk = red[0][c] + red[1][c] + red[2][c] + red[3][c];
        const float u = (vv[c] - stk) * be;
        float oq = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            S[i] = fmaf(kq[0][kg * 32 + i], u, S[i]);
            oq = fmaf(S[i], kq[1][kg * 32 + i], oq);
        }
        __syncthreads();
        red[kg][c] = oq;
        __syncthreads();
        if (a.save) {
            float *sv = a.save + ((long long)m * a.VL + h) * GD * GD;
#pragma unroll
            for (int i = 0; i < 32; ++i) sv[(kg * 32 + i) * GD + c] = S[i];
        }
        float ov = 0.f;
        if (kg == 0) ov = red[0][c] + red[1][c] + red[2][c] + red[3][c];
        const float ss = block_sum<512>(ov * ov, scratch);
        if (kg == 0) {
            const float z = a.proj[(long long)m * a.ld_proj + qkv_l + h * GD + c];
            const float y = ov * rsqrtf(ss / float(GD) + a.eps) * a.norm_w[c] * sigmoidf_(z);
            a.o[(long long)m * a.VL * GD + h * GD + c] = __float2bfloat16(y);
        }
        // ring store of this row's pre-conv values: v channels by every head, q/k by the first head of the group
        if (ch >= 0 && (kg == 2 || h % rep == 0))
            ring[(pos % GDN_RING) * qkv_l + ch] = a.proj[(long long)m * a.ld_proj + ch];
    }
#pragma unroll
    for (int i = 0; i < 32; ++i) Sg[(kg * 32 + i) * GD + c] = S[i];
}


// Speculative acceptance: for every (slot, row) pair and every GDN layer, the state saved after `row` of the last
// verification step becomes the slot's state.  grid (blocks, pairs, layers); S_ptrs[layer] = [slots][state] fp32,
// save = [layers][max_rows][state].  state % 4 == 0.
__global__ void __launch_bounds__(256) gdn_accept_kernel(float *const *S_ptrs, const float *save, int max_rows, long long state,
                                                         const int *pairs) {
    const int layer = blockIdx.z, slot = pairs[2 * blockIdx.y], row = pairs[2 * blockIdx.y + 1];
    if (row < 0) return;
    const float4 *src = reinterpret_cast<const float4 *>(save + ((long long)layer * max_rows + row) * state);
    float4 *dst = reinterpret_cast<float4 *>(S_ptrs[layer] + (long long)slot * state);
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < (state >> 2); i += (long long)gridDim.x * blockDim.x) dst[i] = src[i];
}

}  // namespace qw

using namespace qw;

QW_API int qwk_gdn_conv(const float *proj, int ld_proj, float *ring, const float *cw, const float *A_log,
                        const float *dt_bias, int KL, int VL, int M, const int *slot, const int *pos,
                        const int *run_start, const int *run_len, float *qkv, float *decay, float *beta, float eps,
                        cudaStream_t s) {
    GdnConvArgs a;
    a.proj = proj; a.ld_proj = ld_proj; a.ring = ring; a.cw = cw; a.A_log = A_log; a.dt_bias = dt_bias;
    a.KL = KL; a.VL = VL; a.rows = Rows{M, slot, pos, run_start, run_len};
    a.qkv = qkv; a.decay = decay; a.beta = beta; a.eps = eps;
    if (VL > 128) return -1;
    dim3 grid((M + CONV_ROWS - 1) / CONV_ROWS, 2 * KL + VL);
    gdn_conv_kernel<<<grid, 128, 0, s>>>(a);
    const int qkv_l = (2 * KL + VL) * GD;
    // A batch of more than MAX_ROWS rows is one run of one slot (a prefill chunk): only its last GDN_RING rows stay in the ring.
    const int m_first = M > MAX_ROWS ? M - GDN_RING : 0;
    dim3 g2(M - m_first, (qkv_l + 255) / 256);
    gdn_ring_kernel<<<g2, 256, 0, s>>>(proj, ld_proj, ring, qkv_l, a.rows, m_first);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

QW_API int qwk_gdn_scan(const float *qkv, const float *decay, const float *beta, const float *proj, int ld_proj, float *S,
                        float *save, const float *norm_w, int KL, int VL, int M, const int *slot, const int *pos,
                        const int *run_start, const int *run_len, void *o, float eps, cudaStream_t s) {
    GdnScanArgs a;
    a.qkv = qkv; a.decay = decay; a.beta = beta; a.proj = proj; a.ld_proj = ld_proj; a.S = S; a.save = save;
    a.norm_w = norm_w; a.KL = KL; a.VL = VL; a.rows = Rows{M, slot, pos, run_start, run_len};
    a.o = (bf16 *)o; a.eps = eps;
    dim3 grid(M, VL);
    gdn_scan_kernel<<<grid, 512, 0, s>>>(a);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// One GDN step for M rows: the fused kernel for short batches, else conv + ring + scan.
QW_API int qwk_gdn_step(const float *proj, int ld_proj, float *ring, const float *cw, const float *A_log,
                        const float *dt_bias, const float *norm_w, int KL, int VL, int M, const int *slot, const int *pos,
                        const int *run_start, const int *run_len, float *S, float *save, float *qkv, float *decay,
                        float *beta, void *o, float eps, cudaStream_t s) {
    if (M <= GDN_RING - 4) {
        GdnFusedArgs a;
        a.proj = proj; a.ld_proj = ld_proj; a.ring = ring; a.cw = cw; a.A_log = A_log; a.dt_bias = dt_bias;
        a.norm_w = norm_w; a.KL = KL; a.VL = VL; a.rows = Rows{M, slot, pos, run_start, run_len};
        a.S = S; a.save = save; a.o = (bf16 *)o; a.eps = eps; a.pf = take_pf();
        cudaError_t e = launch_pdl(gdn_fused_kernel, dim3(M, VL), dim3(512), 0, s, a);
        return e == cudaSuccess ? 0 : -2;
    }
    int rc = qwk_gdn_conv(proj, ld_proj, ring, cw, A_log, dt_bias, KL, VL, M, slot, pos, run_start, run_len, qkv, decay,
                          beta, eps, s);
    if (rc) return rc;
    return qwk_gdn_scan(qkv, decay, beta, proj, ld_proj, S, save, norm_w, KL, VL, M, slot, pos, run_start, run_len, o,
                        eps, s);
}


// S_ptrs: device array of n_layers state pointers; pairs: device [n_pairs][2] = {slot, saved row (-1: keep)}.
QW_API int qwk_gdn_accept(const void *S_ptrs, const float *save, int n_layers, int max_rows, long long state, const int *pairs,
                          int n_pairs, cudaStream_t s) {
    if (n_pairs <= 0 || n_layers <= 0) return 0;
    if (state & 3) return -1;
    gdn_accept_kernel<<<dim3(8, n_pairs, n_layers), 256, 0, s>>>((float *const *)S_ptrs, save, max_rows, state, pairs);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
