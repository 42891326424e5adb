// GPU sampler: penalties from per-slot count tables, then per row either the argmax or an exact draw
// from the temperature / top-k / top-p / min-p truncated distribution, with the log-probability of the
// chosen token under the raw distribution (role of the reference's src/kernels/sampling.hip:17-246).
//
// One block of 1024 threads per row.  The 256 most likely tokens (by penalised logit, ties to the lower
// index) are found with a 4-pass radix select, sorted in shared memory and truncated exactly like the
// host sampler does; the draw is an inverse-CDF walk over them with a counter-based uniform
// (splitmix64 of seed and position), so the same seed and position always give the same token.  When the
// nucleus does not fit into the 256 candidates the row reports fallback = 1 and the caller samples that
// row on the host from the full logits.
#include "common.cuh"

namespace qw {

constexpr int CAND = 256;

struct SampleParams {
    float temperature, top_p;
    int top_k;
    float min_p, presence, frequency, repetition;
    unsigned long long seed;
    int slot;            // count-table row (-1: no penalties)
    int position;        // tokens in the sequence so far (RNG counter)
};

struct SampleOut {
    int token;
    float logprob;
    int fallback;
    float lse;
};

__device__ __forceinline__ unsigned int order_key(float f) {      // monotone float -> uint
    const unsigned int u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ unsigned long long splitmix64(unsigned long long v) {
    v += 0x9E3779B97F4A7C15ull;
    v = (v ^ (v >> 30)) * 0xBF58476D1CE4E5B9ull;
    v = (v ^ (v >> 27)) * 0x94D049BB133111EBull;
    return v ^ (v >> 31);
}

__device__ __forceinline__ float penalised(const float *l, int i, const SampleParams &p, const unsigned short *gen,
                                           const unsigned char *seen) {
    float v = l[i];
    if (p.slot >= 0) {
        if (p.repetition != 1.f && seen[i]) v = v > 0.f ? v / p.repetition : v * p.repetition;
        const int c = gen[i];
        if (c) v -= p.presence + p.frequency * float(c);
    }
    return v;
}

// counts: gen [slots][V] uint16 (occurrences among generated tokens), seen [slots][V] uint8 (anywhere in the sequence)
__global__ void __launch_bounds__(1024) sample_kernel(const float *logits, int ld, int V, const SampleParams *params,
                                                      const unsigned short *gen, const unsigned char *seen, SampleOut *out) {
    __shared__ int hist[256];
    __shared__ float s_red[32];
    __shared__ int s_redi[32];
    __shared__ unsigned int s_prefix;
    __shared__ int s_need, s_count, s_ties;
    __shared__ float c_val[CAND];
    __shared__ int c_idx[CAND];
    __shared__ float scratch[32];
    const int m = blockIdx.x, tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    const SampleParams p = params[m];
    const float *l = logits + (long long)m * ld;
    const unsigned short *g = p.slot >= 0 ? gen + (long long)p.slot * V : nullptr;
    const unsigned char *sn = p.slot >= 0 ? seen + (long long)p.slot * V : nullptr;
    // ---- raw max / lse and penalised max / argmax
    float rmax = -INFINITY, bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = tid; i < V; i += 1024) {
        rmax = fmaxf(rmax, l[i]);
        const float v = penalised(l, i, p, g, sn);
        if (v > bv) { bv = v; bi = i; }
    }
    rmax = warp_max(rmax);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) { s_red[w] = bv; s_redi[w] = bi; scratch[w] = rmax; }
    __syncthreads();
    if (w == 0) {
        bv = s_red[lane]; bi = s_redi[lane]; rmax = scratch[lane];
        rmax = warp_max(rmax);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) { s_red[0] = bv; s_redi[0] = bi; scratch[0] = rmax; }
    }
    __syncthreads();
    const float lmax = s_red[0], raw_max = scratch[0];
    const int best = s_redi[0];
    __syncthreads();
    float z = 0.f;
    for (int i = tid; i < V; i += 1024) z += __expf(l[i] - raw_max);
    z = block_sum<1024>(z, scratch);
    const float lse = raw_max + __logf(z);
    if (p.temperature <= 0.f) {
        if (tid == 0) out[m] = SampleOut{best, l[best] - lse, 0, lse};
        return;
    }
    const float inv_t = 1.f / p.temperature;
    // ---- normaliser of the untruncated distribution (tokens within 30 nats of the maximum)
    float za = 0.f;
    for (int i = tid; i < V; i += 1024) {
        const float zz = (penalised(l, i, p, g, sn) - lmax) * inv_t;
        if (zz >= -30.f) za += __expf(zz);
    }
    za = block_sum<1024>(za, scratch);
    // ---- no truncation: an exact draw from the whole vocabulary by the Gumbel-max trick, one pass, no sort
    if (p.top_k <= 0 && p.top_p >= 1.f && p.min_p <= 0.f) {
        const unsigned long long key = splitmix64(p.seed ^ ((unsigned long long)p.position * 0x9E3779B97F4A7C15ull));
        double gb = -INFINITY;
        int gi = 0x7fffffff;
        for (int i = tid; i < V; i += 1024) {
            const float zz = (penalised(l, i, p, g, sn) - lmax) * inv_t;
            if (zz < -30.f) continue;
            const unsigned long long bits = splitmix64(key ^ ((unsigned long long)(i + 1) * 0x9E3779B97F4A7C15ull));
            const double u = (double(bits >> 11) + 0.5) * (1.0 / 9007199254740992.0);
            const double v = double(zz) - log(-log(u));
            if (v > gb) { gb = v; gi = i; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const double ov = __shfl_xor_sync(0xffffffffu, gb, o);
            const int oi = __shfl_xor_sync(0xffffffffu, gi, o);
            if (ov > gb || (ov == gb && oi < gi)) { gb = ov; gi = oi; }
        }
        __shared__ double s_gd[32];
        if (lane == 0) { s_gd[w] = gb; s_redi[w] = gi; }
        __syncthreads();
        if (tid == 0) {
            for (int k = 1; k < 32; ++k)
                if (s_gd[k] > gb || (s_gd[k] == gb && s_redi[k] < gi)) { gb = s_gd[k]; gi = s_redi[k]; }
            out[m] = SampleOut{gi, l[gi] - lse, 0, lse};
        }
        return;
    }
    // ---- radix select of the CAND-th largest penalised logit
    const int want = min(CAND, V);
    if (tid == 0) { s_prefix = 0u; s_need = want; }
    for (int pass = 0; pass < 4; ++pass) {
        const int shift = 24 - 8 * pass;
        if (tid < 256) hist[tid] = 0;
        __syncthreads();
        const unsigned int prefix = s_prefix;
        const unsigned int mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
        for (int i = tid; i < V; i += 1024) {
            const unsigned int k = order_key(penalised(l, i, p, g, sn));
            if ((k & mask) == prefix) atomicAdd(&hist[(k >> shift) & 0xff], 1);
        }
        __syncthreads();
        if (tid == 0) {
            int need = s_need, b = 255;
            for (; b > 0; --b) {
                if (hist[b] >= need) break;
                need -= hist[b];
            }
            s_need = need;
            s_prefix = prefix | ((unsigned int)b << shift);
        }
        __syncthreads();
    }
    const unsigned int T = s_prefix;
    // ---- collect: everything above T, plus the lowest-index entries equal to T
    if (tid == 0) s_count = 0;
    __syncthreads();
    for (int i = tid; i < V; i += 1024) {
        const float v = penalised(l, i, p, g, sn);
        if (order_key(v) > T) {
            const int o = atomicAdd(&s_count, 1);
            if (o < CAND) { c_val[o] = v; c_idx[o] = i; }
        }
    }
    __syncthreads();
    const int above = min(s_count, CAND);
    __syncthreads();
    // ---- the entries equal to T (at least the want-th best itself): all threads look for them; if there are more than
    // are needed (equal floats straddling the cut: rare) one thread takes the lowest indices serially instead
    if (tid == 0) s_ties = 0;
    __syncthreads();
    for (int i = tid; i < V; i += 1024) {
        const float v = penalised(l, i, p, g, sn);
        if (order_key(v) == T) {
            const int o = above + atomicAdd(&s_ties, 1);
            if (o < CAND) { c_val[o] = v; c_idx[o] = i; }
        }
    }
    __syncthreads();
    if (tid == 0) {
        if (above + s_ties <= want) {
            s_count = above + s_ties;
        } else {
            int o = above;
            for (int i = 0; i < V && o < want; ++i) {
                const float v = penalised(l, i, p, g, sn);
                if (order_key(v) == T) { c_val[o] = v; c_idx[o] = i; ++o; }
            }
            s_count = o;
        }
    }
    __syncthreads();
    const int n = s_count;
    for (int i = n + tid; i < CAND; i += 1024) { c_val[i] = -INFINITY; c_idx[i] = 0x7fffffff; }
    __syncthreads();
    // ---- bitonic sort, descending by (value, -index)
    for (int k = 2; k <= CAND; k <<= 1)
        for (int j = k >> 1; j > 0; j >>= 1) {
            if (tid < CAND) {
                const int ixj = tid ^ j;
                if (ixj > tid) {
                    const bool up = (tid & k) == 0;
                    const float a = c_val[tid], b = c_val[ixj];
                    const int ia = c_idx[tid], ib = c_idx[ixj];
                    const bool a_first = a > b || (a == b && ia < ib);
                    if (up ? !a_first : a_first) { c_val[tid] = b; c_val[ixj] = a; c_idx[tid] = ib; c_idx[ixj] = ia; }
                }
            }
            __syncthreads();
        }
    // ---- truncation and draw (one thread: at most 256 candidates)
    if (tid == 0) {
        int K = n;
        if (p.top_k > 0 && p.top_k < K) K = p.top_k;
        int fallback = 0;
        if (p.top_k > CAND) fallback = 1;   // needs more than the candidates
        double zk = 0;
        for (int i = 0; i < K; ++i) zk += exp(double((c_val[i] - lmax) * inv_t));
        const double norm = p.top_k > 0 ? zk : double(za);
        int keep = K;
        if (p.top_p < 1.f) {
            double acc = 0;
            keep = -1;
            for (int i = 0; i < K; ++i) {
                acc += exp(double((c_val[i] - lmax) * inv_t)) / norm;
                if (acc >= p.top_p) { keep = i + 1; break; }
            }
            if (keep < 0) {
                if (p.top_k <= 0 && n < V) fallback = 1;          // nucleus wider than the candidates
                keep = K;
            }
        }
        if (p.min_p > 0.f) {
            const double thr = double(p.min_p);                  // relative to the best token (weight 1)
            int k2 = 0;
            while (k2 < keep && exp(double((c_val[k2] - lmax) * inv_t)) >= thr) ++k2;
            if (k2 == keep && keep == K && K == n && n < V && p.top_k <= 0) fallback = 1;      // the cut may lie beyond the candidates
            keep = k2 > 0 ? k2 : 1;
        }
        double tot = 0;
        for (int i = 0; i < keep; ++i) tot += exp(double((c_val[i] - lmax) * inv_t));
        const unsigned long long bits = splitmix64(p.seed ^ ((unsigned long long)p.position * 0x9E3779B97F4A7C15ull));
        double r = double(bits >> 11) * (1.0 / 9007199254740992.0) * tot;
        int pick = keep - 1;
        for (int i = 0; i < keep; ++i) {
            r -= exp(double((c_val[i] - lmax) * inv_t));
            if (r <= 0) { pick = i; break; }
        }
        const int tok = c_idx[pick];
        out[m] = SampleOut{tok, l[tok] - lse, fallback, lse};
    }
}

// counts update: the token joins the sequence of `slot` (generated tokens also count for presence / frequency)
__global__ void penalty_add_kernel(unsigned short *gen, unsigned char *seen, int V, const int *slots, const int *tokens,
                                   const int *generated, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int t = tokens[i];
    if (t < 0 || t >= V) return;
    seen[(long long)slots[i] * V + t] = 1;
    if (generated[i]) {
        unsigned short *c = gen + (long long)slots[i] * V + t;
        if (*c < 65535) *c += 1;          // rows of one call are distinct (slot, token) pairs or sequential appends by one thread each
    }
}

}  // namespace qw

using namespace qw;

// params: device array of M SampleParams (48 bytes each); out: device array of M SampleOut.
QW_API int qwk_sample(const float *logits, int ld, int V, int M, const void *params, const void *gen, const void *seen, void *out,
                      cudaStream_t s) {
    sample_kernel<<<M, 1024, 0, s>>>(logits, ld, V, (const SampleParams *)params, (const unsigned short *)gen,
                                     (const unsigned char *)seen, (SampleOut *)out);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

QW_API int qwk_penalty_add(void *gen, void *seen, int V, const int *slots, const int *tokens, const int *generated, int n,
                           cudaStream_t s) {
    penalty_add_kernel<<<(n + 127) / 128, 128, 0, s>>>((unsigned short *)gen, (unsigned char *)seen, V, slots, tokens, generated, n);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
