// Reductions over a vocabulary shard of logits: (max, argmax with ties to the lowest index) and
// (max, sum exp) per row (roles of the reference's src/kernels/logits.hip:7-70).  Results of the
// shards are merged by merge_argmax / on the host.
#include "common.cuh"

namespace qw {

// grid M, 1024 threads.  out_val[m], out_idx[m] (index offset by idx0); lse parts: out_max[m], out_sum[m].
__global__ void __launch_bounds__(1024) row_reduce_kernel(const float *logits, int ld, int V, int idx0, float *out_val,
                                                          int *out_idx, float *out_max, float *out_sum) {
    __shared__ float sv[32];
    __shared__ int si[32];
    __shared__ float scratch[32];
    const int m = blockIdx.x;
    const float *l = logits + (long long)m * ld;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += 1024) {
        const float v = l[i];
        if (v > bv) { bv = v; bi = i; }       // ascending i: keeps the lowest index among equals
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) { sv[w] = bv; si[w] = bi; }
    __syncthreads();
    if (w == 0) {
        bv = sv[lane]; bi = si[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) { sv[0] = bv; si[0] = bi; }
    }
    __syncthreads();
    const float mx = sv[0];
    if (threadIdx.x == 0) {
        if (out_val) out_val[m] = mx;
        if (out_idx) out_idx[m] = si[0] + idx0;
    }
    if (out_sum) {
        float z = 0.f;
        for (int i = threadIdx.x; i < V; i += 1024) z += __expf(l[i] - mx);
        z = block_sum<1024>(z, scratch);
        if (threadIdx.x == 0) { out_max[m] = mx; out_sum[m] = z; }
    }
}

// Merge per-rank (value, index) pairs: parts[r][m]; ties to the lowest index.  One thread per row.
__global__ void merge_argmax_kernel(const float *vals, const int *idx, int ranks, int M, int stride, int *out_idx,
                                    float *out_val) {
    const int m = blockIdx.x * blockDim.x + threadIdx.x;
    if (m >= M) return;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int r = 0; r < ranks; ++r) {
        const float v = vals[r * stride + m];
        const int i = idx[r * stride + m];
        if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
    }
    out_idx[m] = bi;
    if (out_val) out_val[m] = bv;
}

// Chained decoding: the sampled token of each row becomes the row's next input, its position
// advances and the n-gram context shifts, all on the device, so consecutive steps need no host
// round trip (the reference chains its draft steps the same way, src/engine/decode.hip:293-334).
__global__ void advance_rows_kernel(int *tokens, int *pos, int *ctx3, const int *next, int M) {
    const int m = blockIdx.x * blockDim.x + threadIdx.x;
    if (m >= M) return;
    const int t = next[m];
    ctx3[3 * m + 2] = ctx3[3 * m + 1];
    ctx3[3 * m + 1] = ctx3[3 * m];
    ctx3[3 * m] = t;
    tokens[m] = t;
    pos[m] += 1;
}

// Vocabulary-parallel argmax: every rank packs its (value, index) per row into its column pair of the
// gathered matrix; after the all-gather every rank picks the best pair (ties to the lowest index).
__global__ void amax_pack_kernel(const float *val, const int *idx, float *pairs, int M, int rank, int ranks) {
    pdl_wait();
    pdl_trigger();
    const int m = blockIdx.x * blockDim.x + threadIdx.x;
    if (m >= M) return;
    pairs[(long long)m * ranks * 2 + rank * 2] = val[m];
    pairs[(long long)m * ranks * 2 + rank * 2 + 1] = __int_as_float(idx[m]);
}
__global__ void amax_merge_kernel(const float *pairs, int M, int ranks, int *out_idx, float *out_val) {
    pdl_wait();
    pdl_trigger();
    const int m = blockIdx.x * blockDim.x + threadIdx.x;
    if (m >= M) return;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int r = 0; r < ranks; ++r) {
        const float v = __ldcg(pairs + (long long)m * ranks * 2 + r * 2);
        const int i = __float_as_int(__ldcg(pairs + (long long)m * ranks * 2 + r * 2 + 1));
        if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
    }
    out_idx[m] = bi;
    if (out_val) out_val[m] = bv;
}

}  // namespace qw

using namespace qw;

QW_API int qwk_amax_pack(const float *val, const int *idx, float *pairs, int M, int rank, int ranks, cudaStream_t s) {
    return launch_pdl(amax_pack_kernel, dim3((M + 63) / 64), dim3(64), 0, s, val, idx, pairs, M, rank, ranks) == cudaSuccess ? 0 : -2;
}
QW_API int qwk_amax_merge(const float *pairs, int M, int ranks, int *out_idx, float *out_val, cudaStream_t s) {
    return launch_pdl(amax_merge_kernel, dim3((M + 63) / 64), dim3(64), 0, s, pairs, M, ranks, out_idx, out_val) == cudaSuccess ? 0 : -2;
}


QW_API int qwk_advance_rows(int *tokens, int *pos, int *ctx3, const int *next, int M, cudaStream_t s) {
    advance_rows_kernel<<<(M + 63) / 64, 64, 0, s>>>(tokens, pos, ctx3, next, M);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

QW_API int qwk_row_reduce(const float *logits, int ld, int V, int idx0, int M, float *out_val, int *out_idx,
                          float *out_max, float *out_sum, cudaStream_t s) {
    row_reduce_kernel<<<M, 1024, 0, s>>>(logits, ld, V, idx0, out_val, out_idx, out_max, out_sum);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

QW_API int qwk_merge_argmax(const float *vals, const int *idx, int ranks, int M, int stride, int *out_idx,
                            float *out_val, cudaStream_t s) {
    merge_argmax_kernel<<<(M + 63) / 64, 64, 0, s>>>(vals, idx, ranks, M, stride, out_idx, out_val);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
