// MTP head plumbing kernels: the input of the MTP layer is, per stream, fc_hidden(norm(hidden stream)) +
// fc_embedding(gemma_norm(embedding of the next token)), where `norm` is ONE RMS norm over all hc*H values
// of the backbone's pre-final-mixer state (roles of the reference's src/kernels/mtp.hip:7-54;
// math in docs/MODEL.md:221-231).
#include "common.cuh"

namespace qw {

// grid M, 256 threads.  hidden [M][hc][H] fp32 -> hn bf16 [(m*hc + s)][H] = hidden * rsqrt(mean over all) * nh1;
// en bf16 [m][H] = gemma_norm(embed[token m]) with ne1 = 1 + w.
__global__ void __launch_bounds__(256) mtp_norm_kernel(const float *hidden, const int *tokens, const bf16 *embed, int vocab,
                                                       const float *nh1, const float *ne1, int H, int hc, float eps, bf16 *hn,
                                                       bf16 *en) {
    __shared__ float scratch[32];
    pdl_wait();
    pdl_trigger();
    const int m = blockIdx.x;
    const float *x = hidden + (long long)m * hc * H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < hc * H; i += 256) ss = fmaf(x[i], x[i], ss);
    ss = block_sum<256>(ss, scratch);
    const float r = rsqrtf(ss / float(hc * H) + eps);
    for (int i = threadIdx.x; i < hc * H; i += 256) hn[(long long)m * hc * H + i] = __float2bfloat16(x[i] * r * nh1[i]);
    int t = tokens[m];
    if (t < 0 || t >= vocab) t = 0;
    const bf16 *e = embed + (long long)t * H;
    float es = 0.f;
    for (int i = threadIdx.x; i < H; i += 256) {
        const float v = __bfloat162float(e[i]);
        es = fmaf(v, v, es);
    }
    es = block_sum<256>(es, scratch);
    const float re = rsqrtf(es / float(H) + eps);
    for (int i = threadIdx.x; i < H; i += 256) en[(long long)m * H + i] = __float2bfloat16(__bfloat162float(e[i]) * re * ne1[i]);
}

// X[m][s][c] = fh[(m*hc + s)][c] + fe[m][c]
__global__ void mtp_add_kernel(const float *fh, const float *fe, int H, int hc, float *X, long long total) {
    pdl_wait();
    pdl_trigger();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long m = i / ((long long)hc * H);
    const int c = (int)(i % H);
    X[i] = fh[i] + fe[m * H + c];
}

}  // namespace qw

using namespace qw;

QW_API int qwk_mtp_norm(const float *hidden, const int *tokens, const void *embed, int vocab, const float *nh1, const float *ne1,
                        int H, int hc, float eps, void *hn, void *en, int M, cudaStream_t s) {
    return launch_pdl(mtp_norm_kernel, dim3(M), dim3(256), 0, s, hidden, tokens, (const bf16 *)embed, vocab, nh1, ne1, H, hc, eps,
                      (bf16 *)hn, (bf16 *)en) == cudaSuccess ? 0 : -2;
}
QW_API int qwk_mtp_add(const float *fh, const float *fe, int H, int hc, float *X, int M, cudaStream_t s) {
    const long long total = (long long)M * hc * H;
    return launch_pdl(mtp_add_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, s, fh, fe, H, hc, X, total) == cudaSuccess ? 0 : -2;
}
