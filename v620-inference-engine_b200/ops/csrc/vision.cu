// Vision tower (Qwen3-VL ViT) kernels: everything between the tower's GEMMs (which run on the tcgen05 GEMM of
// gemm_tc.cu).  Residual stream fp32, GEMM operands bf16.
//
//   vit_embed          x = patch_gemm + bias + bilinear interpolation of the learned 48x48 position table
//   vit_layernorm      bf16(LayerNorm(x) * w + b)
//   vit_bias_rope      qkv += bias, then 2-D rotary on q and k (pairs (t, t+36); first 18 frequencies by row,
//                      last 18 by column)
//   vit_attention      non-causal attention over one image / video slice, head dim 72, flash style on the tensor
//                      cores (mma.sync m16n8k16 bf16, fp32 softmax state), 64 queries per block
//   vit_bias_gelu      y = gelu(y + bias), tanh or erf form
//   vit_residual_add   x += y + bias        vit_bias_out   out = y + bias
// (Role of the reference's src/kernels/vision.hip:33-217.)
#include "mma.cuh"

namespace qw {

constexpr int VHD = 72;          // head dim
constexpr int VHALF = 36;
constexpr int VNF = 18;

__global__ void __launch_bounds__(256) vit_embed_kernel(float *x, const float *y, const float *bias, const float *table,
                                                        const int *idx, const float *wts, int D) {
    const int n = blockIdx.x;
    const int i0 = idx[n * 4], i1 = idx[n * 4 + 1], i2 = idx[n * 4 + 2], i3 = idx[n * 4 + 3];
    const float w0 = wts[n * 4], w1 = wts[n * 4 + 1], w2 = wts[n * 4 + 2], w3 = wts[n * 4 + 3];
    for (int c = threadIdx.x; c < D; c += 256) {
        const float p = w0 * table[(long long)i0 * D + c] + w1 * table[(long long)i1 * D + c] +
                        w2 * table[(long long)i2 * D + c] + w3 * table[(long long)i3 * D + c];
        x[(long long)n * D + c] = y[(long long)n * D + c] + bias[c] + p;
    }
}

__global__ void __launch_bounds__(256) vit_layernorm_kernel(const float *x, const float *w, const float *b, int D, float eps,
                                                            bf16 *out) {
    __shared__ float scratch[32];
    const int n = blockIdx.x;
    const float *row = x + (long long)n * D;
    float s = 0.f;
    for (int c = threadIdx.x; c < D; c += 256) s += row[c];
    const float mean = block_sum<256>(s, scratch) / float(D);
    float v = 0.f;
    for (int c = threadIdx.x; c < D; c += 256) {
        const float d = row[c] - mean;
        v = fmaf(d, d, v);
    }
    const float rstd = rsqrtf(block_sum<256>(v, scratch) / float(D) + eps);
    for (int c = threadIdx.x; c < D; c += 256) out[(long long)n * D + c] = __float2bfloat16((row[c] - mean) * rstd * w[c] + b[c]);
}

// one block per patch: bias on the whole row, rotary on q and k
__global__ void __launch_bounds__(256) vit_bias_rope_kernel(bf16 *qkv, const float *bias, const int *pos_hw, int heads) {
    const int n = blockIdx.x;
    const int D = heads * VHD;
    bf16 *row = qkv + (long long)n * 3 * D;
    for (int c = 2 * D + threadIdx.x; c < 3 * D; c += 256) row[c] = __float2bfloat16(__bfloat162float(row[c]) + bias[c]);
    const float pr = float(pos_hw[n * 2]), pc = float(pos_hw[n * 2 + 1]);
    for (int i = threadIdx.x; i < 2 * heads * VHALF; i += 256) {
        const int t = i % VHALF, hh = i / VHALF;          // hh over q heads then k heads
        const int f = t % VNF;
        const float inv = exp2f(-2.f * float(f) / float(VHALF) * 13.287712379549449f);      // 10000^(-2f/36)
        float sn, cs;
        sincosf((t < VNF ? pr : pc) * inv, &sn, &cs);
        const int base = hh * VHD;
        const float a = __bfloat162float(row[base + t]) + bias[base + t];
        const float b = __bfloat162float(row[base + t + VHALF]) + bias[base + t + VHALF];
        row[base + t] = __float2bfloat16(a * cs - b * sn);
        row[base + t + VHALF] = __float2bfloat16(b * cs + a * sn);
    }
}

__global__ void vit_bias_gelu_kernel(bf16 *y, const float *bias, long long total, int D, int tanh_form) {
    const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (i >= total) return;
    const float v = __bfloat162float(y[i]) + bias[i % D];
    const float g = tanh_form ? 0.5f * v * (1.f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)))
                              : 0.5f * v * (1.f + erff(v * 0.7071067811865476f));
    y[i] = __float2bfloat16(g);
}

__global__ void vit_residual_add_kernel(float *x, const float *y, const float *bias, long long total, int D, int assign) {
    const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (i >= total) return;
    const float v = y[i] + bias[i % D];
    x[i] = assign ? v : x[i] + v;
}

// ---- attention -----------------------------------------------------------------------------------------------
constexpr int VA_Q = 64, VA_K = 64;            // queries per block, keys per tile
constexpr int VA_QS = 88, VA_VS = 80;          // shared-memory row strides (elements): q/k rows padded to 80 dims + 8, v rows 72 + 8

__device__ __forceinline__ void ldmatrix_x2_trans(uint32_t &r0, uint32_t &r1, uint32_t saddr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(saddr));
}
__device__ __forceinline__ uint32_t pack2(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&h);
}

__global__ void __launch_bounds__(128) vit_attention_kernel(const bf16 *qkv, int L, int heads, bf16 *out) {
    __shared__ __align__(16) bf16 sq[VA_Q * VA_QS];
    __shared__ __align__(16) bf16 sk[VA_K * VA_QS];
    __shared__ __align__(16) bf16 sv[VA_K * VA_VS];
    const int h = blockIdx.y, q0 = blockIdx.x * VA_Q;
    const int D = heads * VHD, ld = 3 * D;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // queries of this block (rows past L and dims 72..79 are zero)
    for (int i = tid; i < VA_Q * 10; i += 128) {
        const int r = i / 10, c = i - r * 10;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (c < 9 && q0 + r < L) v = *reinterpret_cast<const uint4 *>(qkv + (long long)(q0 + r) * ld + h * VHD + c * 8);
        *reinterpret_cast<uint4 *>(sq + r * VA_QS + c * 8) = v;
    }
    __syncthreads();
    uint32_t qa[5][4];
    const uint32_t sq_base = smem_u32(sq) + (unsigned)(warp * 16) * VA_QS * 2;
#pragma unroll
    for (int ks = 0; ks < 5; ++ks) ldmatrix_x4(qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], a_tile_addr(sq_base, VA_QS * 2, ks * 16, lane));
    float o[9][4];
#pragma unroll
    for (int j = 0; j < 9; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    float mx0 = -1e30f, mx1 = -1e30f, sum0 = 0.f, sum1 = 0.f;          // rows lane/4 and lane/4 + 8
    const float scale = 1.4426950408889634f * rsqrtf(float(VHD));      // scores in log2 units
    const uint32_t sk_base = smem_u32(sk), sv_base = smem_u32(sv);
    for (int k0 = 0; k0 < L; k0 += VA_K) {
        __syncthreads();                                                // the previous tile is consumed
        for (int i = tid; i < VA_K * 10; i += 128) {
            const int r = i / 10, c = i - r * 10;
            uint4 kv = make_uint4(0u, 0u, 0u, 0u), vv = kv;
            if (c < 9 && k0 + r < L) {
                const bf16 *p = qkv + (long long)(k0 + r) * ld + h * VHD + c * 8;
                kv = *reinterpret_cast<const uint4 *>(p + D);
                vv = *reinterpret_cast<const uint4 *>(p + 2 * D);
            }
            *reinterpret_cast<uint4 *>(sk + r * VA_QS + c * 8) = kv;
            if (c < 9) *reinterpret_cast<uint4 *>(sv + r * VA_VS + c * 8) = vv;
        }
        __syncthreads();
        // S = Q K^T for 16 queries x 64 keys
        float s[8][4];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
            for (int ks = 0; ks < 5; ++ks) {
                uint32_t b0, b1;
                ldmatrix_x2(b0, b1, sk_base + (unsigned)(j * 8 + (lane & 7)) * VA_QS * 2 + (unsigned)(ks * 16 + (((lane >> 3) & 1) << 3)) * 2u);
                mma_bf16(s[j], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b0, b1);
            }
        }
        // scale, mask keys past L, running max / sum per row
        float t0 = -1e30f, t1 = -1e30f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int kc = k0 + j * 8 + (lane & 3) * 2;
            s[j][0] = kc < L ? s[j][0] * scale : -1e30f;
            s[j][1] = kc + 1 < L ? s[j][1] * scale : -1e30f;
            s[j][2] = kc < L ? s[j][2] * scale : -1e30f;
            s[j][3] = kc + 1 < L ? s[j][3] * scale : -1e30f;
            t0 = fmaxf(t0, fmaxf(s[j][0], s[j][1]));
            t1 = fmaxf(t1, fmaxf(s[j][2], s[j][3]));
        }
        t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, 1)); t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, 2));
        t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, 1)); t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, 2));
        const float n0 = fmaxf(mx0, t0), n1 = fmaxf(mx1, t1);
        const float c0 = exp2f(mx0 - n0), c1 = exp2f(mx1 - n1);
        mx0 = n0; mx1 = n1;
        float p0 = 0.f, p1 = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            s[j][0] = exp2f(s[j][0] - n0); s[j][1] = exp2f(s[j][1] - n0);
            s[j][2] = exp2f(s[j][2] - n1); s[j][3] = exp2f(s[j][3] - n1);
            p0 += s[j][0] + s[j][1];
            p1 += s[j][2] + s[j][3];
        }
        sum0 = sum0 * c0 + p0;
        sum1 = sum1 * c1 + p1;
#pragma unroll
        for (int j = 0; j < 9; ++j) { o[j][0] *= c0; o[j][1] *= c0; o[j][2] *= c1; o[j][3] *= c1; }
        // O += P V : P from the score fragments (two key tiles of 8 make one k step of 16), V transposed on load
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
            const uint32_t a0 = pack2(s[2 * kk][0], s[2 * kk][1]), a1 = pack2(s[2 * kk][2], s[2 * kk][3]);
            const uint32_t a2 = pack2(s[2 * kk + 1][0], s[2 * kk + 1][1]), a3 = pack2(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int j = 0; j < 9; ++j) {
                uint32_t b0, b1;
                ldmatrix_x2_trans(b0, b1, sv_base + (unsigned)(kk * 16 + (lane & 15)) * VA_VS * 2 + (unsigned)(j * 8) * 2u);
                mma_bf16(o[j], a0, a1, a2, a3, b0, b1);
            }
        }
    }
    sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1); sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
    sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1); sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
    const float r0 = 1.f / sum0, r1 = 1.f / sum1;
    const int row0 = q0 + warp * 16 + (lane >> 2), row1 = row0 + 8;
#pragma unroll
    for (int j = 0; j < 9; ++j) {
        const int c = h * VHD + j * 8 + (lane & 3) * 2;
        if (row0 < L) *reinterpret_cast<uint32_t *>(out + (long long)row0 * D + c) = pack2(o[j][0] * r0, o[j][1] * r0);
        if (row1 < L) *reinterpret_cast<uint32_t *>(out + (long long)row1 * D + c) = pack2(o[j][2] * r1, o[j][3] * r1);
    }
}

}  // namespace qw

using namespace qw;

static inline unsigned blocks_for(long long n) { return (unsigned)((n + 255) / 256); }

QW_API int qwk_vit_embed(float *x, const float *y, const float *bias, const float *table, const int *idx, const float *wts,
                         int L, int D, cudaStream_t s) {
    vit_embed_kernel<<<L, 256, 0, s>>>(x, y, bias, table, idx, wts, D);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

QW_API int qwk_vit_layernorm(const float *x, const float *w, const float *b, int L, int D, float eps, void *out,
                             cudaStream_t s) {
    vit_layernorm_kernel<<<L, 256, 0, s>>>(x, w, b, D, eps, (bf16 *)out);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

QW_API int qwk_vit_bias_rope(void *qkv, const float *bias, const int *pos_hw, int L, int heads, cudaStream_t s) {
    vit_bias_rope_kernel<<<L, 256, 0, s>>>((bf16 *)qkv, bias, pos_hw, heads);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// qkv [L][3 * heads * 72] bf16 (bias and rotary applied) -> out [L][heads * 72] bf16.  Row starts must be 16-byte aligned.
QW_API int qwk_vit_attention(const void *qkv, int L, int heads, void *out, cudaStream_t s) {
    if (L <= 0) return 0;
    dim3 grid((L + VA_Q - 1) / VA_Q, heads);
    vit_attention_kernel<<<grid, 128, 0, s>>>((const bf16 *)qkv, L, heads, (bf16 *)out);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

QW_API int qwk_vit_bias_gelu(void *y, const float *bias, int L, int D, int tanh_form, cudaStream_t s) {
    const long long total = (long long)L * D;
    vit_bias_gelu_kernel<<<blocks_for(total), 256, 0, s>>>((bf16 *)y, bias, total, D, tanh_form);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// assign = 0: x += y + bias; assign = 1: x = y + bias.
QW_API int qwk_vit_residual_add(float *x, const float *y, const float *bias, int L, int D, int assign, cudaStream_t s) {
    const long long total = (long long)L * D;
    vit_residual_add_kernel<<<blocks_for(total), 256, 0, s>>>(x, y, bias, total, D, assign);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
