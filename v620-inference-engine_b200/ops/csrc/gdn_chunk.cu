// Chunked (WY) gated delta rule for token-major prefill: the recurrent scan of a run of M tokens done as
// dense 64-token chunk products on the tensor cores, with the state in fp32.
//
// The reference only has the token-by-token scan (gdn_scan_T, src/kernels/gdn.hip:229-309) and lists the
// chunked form as future work (its design document under docs/, line 512).  Math (per value head, state S [128 k][128 v], chunk of
// C = 64 rows, entry state S0, g_t = sum_{s<=t} log decay_s):
//
//     A[t,s] = beta_t exp(g_t - g_s) (k_t . k_s)       s <  t
//     (I + A) Wv = diag(beta) V      (I + A) Wk = diag(beta exp(g)) K
//     P[t,s] = exp(g_t - g_s) (q_t . k_s)              s <= t
//     U  = Wv - Wk S0
//     O  = diag(exp(g)) Q S0 + P U
//     S1 = exp(g_C) S0 + (diag(exp(g_C - g)) K)^T U
//
// Three launches per layer:
//   1. gdn_chunk_prep_kernel   grid (chunks, VL): everything that does not depend on the state (A, Wv, Wk, P, g),
//      all chunks in parallel.  K K^T and Q K^T on mma.sync tf32; the two triangular solves by forward
//      substitution in fp32, one column of [Wv | Wk] per thread.
//   2. gdn_chunk_apply_kernel  grid (2, VL): walks the chunks in order with the state of one head's 64 value
//      columns in shared memory; three tf32 products per chunk.  The value columns of a head are independent in
//      every state-dependent product, so a head is split over two blocks.
//   3. gdn_chunk_norm_kernel   grid (M, VL): gated RMS norm over the head's 128 outputs -> bf16.
//
// The run must be one slot's: rows 0..M-1 of the batch are consecutive positions of slot[0].  Rows past M in
// the last chunk are masked (beta = 0, decay = 1, q = k = 0), which leaves the state untouched.
#include "common.cuh"

namespace qw {

constexpr int CD = 128;          // head dim (keys and values)
constexpr int CC = 64;           // rows per chunk
constexpr int LDA = CD + 4;      // row stride of a [64][128] A-operand tile: 4 mod 32 words -> fragment loads hit 32 banks
constexpr int LDT = CD + 8;      // row stride of a [64][128] tile read transposed (8 mod 32)
constexpr int LDP = CC + 4;      // [64][64] A-operand tile
constexpr int LDS = 64 + 8;      // [.][64] B-operand tile (state half, U)

__device__ __forceinline__ uint32_t tf32(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ void mma_tf32(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// A fragment of a 16 x 8 tile at (r0, k0) of a row-major matrix: lane (g = lane / 4, t = lane % 4) holds
// (r0+g, k0+t), (r0+g+8, k0+t), (r0+g, k0+t+4), (r0+g+8, k0+t+4).
__device__ __forceinline__ void lda_frag(uint32_t (&a)[4], const float *m, int ld, int r0, int k0, int g, int t) {
    const float *p = m + (r0 + g) * ld + k0 + t;
    a[0] = tf32(p[0]);
    a[1] = tf32(p[8 * ld]);
    a[2] = tf32(p[4]);
    a[3] = tf32(p[8 * ld + 4]);
}

struct GdnChunkArgs {
    const float *qkv;            // [M][qkv_l]  q (KL heads) | k (KL heads) | v (VL heads), after conv / norm
    const float *decay, *beta;   // [M][VL]
    const float *proj;           // z gate: proj[m][qkv_l + h*128 + d]
    int ld_proj;
    float *S;                    // [slots][VL][128 k][128 v]
    const float *norm_w;         // [128]
    int KL, VL, M;
    const int *slot;             // slot[0] = the run's slot
    float *Wk, *Wv;              // scratch [chunks][VL][64][128]
    float *P;                    // scratch [chunks][VL][64][64]
    float *G;                    // scratch [chunks][VL][64]   cumulative log decay
    float *Oraw;                 // scratch [M][VL*128]
    bf16 *o;                     // [M][VL*128]
    float eps;
};

// Loads rows [m0, m0+64) x 128 floats at column offset col of the qkv rows into a shared tile of stride ld;
// rows >= M are zero.  256 threads.
__device__ __forceinline__ void load_tile(float *dst, int ld, const float *qkv, int qkv_l, int col, int m0, int M, int tid) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int idx = tid + i * 256;          // float4 index: 64 rows x 32
        const int r = idx >> 5, c4 = idx & 31;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (m0 + r < M) v = *reinterpret_cast<const float4 *>(qkv + (long long)(m0 + r) * qkv_l + col + c4 * 4);
        *reinterpret_cast<float4 *>(dst + r * ld + c4 * 4) = v;
    }
}

// ------------------------------------------------------------------------------------------------
// 1. state-independent part of every chunk
// ------------------------------------------------------------------------------------------------
constexpr int PREP_SMEM = (2 * CC * LDA + 2 * CC) * 4;      // 68 KB: three blocks per SM

__global__ void __launch_bounds__(256, 3) gdn_chunk_prep_kernel(GdnChunkArgs a) {
    extern __shared__ __align__(16) float sm[];
    float *Ks = sm;                      // [64][LDA]
    float *Qs = Ks + CC * LDA;           // [64][LDA]
    float *As = Qs;                      // [64][LDP]  takes Q's place once Q K^T is done
    float *gs = Qs + CC * LDA;           // [64] cumulative log decay
    float *bs = gs + CC;                 // [64] beta
    const int ch = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int qkv_l = (2 * a.KL + a.VL) * CD;
    const int kh = h / (a.VL / a.KL);
    const int m0 = ch * CC;
    load_tile(Ks, LDA, a.qkv, qkv_l, (a.KL + kh) * CD, m0, a.M, tid);
    load_tile(Qs, LDA, a.qkv, qkv_l, kh * CD, m0, a.M, tid);
    if (w == 0) {
        const int r0 = 2 * lane, r1 = r0 + 1;
        float x0 = 0.f, x1 = 0.f, b0 = 0.f, b1 = 0.f;
        if (m0 + r0 < a.M) {
            x0 = fmaxf(__logf(a.decay[(long long)(m0 + r0) * a.VL + h]), -87.f);
            b0 = a.beta[(long long)(m0 + r0) * a.VL + h];
        }
        if (m0 + r1 < a.M) {
            x1 = fmaxf(__logf(a.decay[(long long)(m0 + r1) * a.VL + h]), -87.f);
            b1 = a.beta[(long long)(m0 + r1) * a.VL + h];
        }
        float s = x0 + x1;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float n = __shfl_up_sync(0xffffffffu, s, o);
            if (lane >= o) s += n;
        }
        gs[r0] = s - x1;
        gs[r1] = s;
        bs[r0] = b0;
        bs[r1] = b1;
    }
    __syncthreads();
    // K K^T and Q K^T: warp tile 16 rows x 32 columns
    const int r0 = (w & 3) * 16, c0 = (w >> 2) * 32;
    float akk[4][4], aqk[4][4];
#pragma unroll
    for (int n = 0; n < 4; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) akk[n][i] = aqk[n][i] = 0.f;
#pragma unroll 4
    for (int k0 = 0; k0 < CD; k0 += 8) {
        uint32_t fk[4], fq[4];
        lda_frag(fk, Ks, LDA, r0, k0, g, t);
        lda_frag(fq, Qs, LDA, r0, k0, g, t);
#pragma unroll
        for (int n = 0; n < 4; ++n) {
            const float *p = Ks + (c0 + n * 8 + g) * LDA + k0 + t;      // B[k][n] = K[n][k]
            const uint32_t b0 = tf32(p[0]), b1 = tf32(p[4]);
            mma_tf32(akk[n], fk, b0, b1);
            mma_tf32(aqk[n], fq, b0, b1);
        }
    }
    __syncthreads();                     // every warp is done reading Q before A overwrites it
    float *Pg = a.P + ((long long)ch * a.VL + h) * CC * CC;
#pragma unroll
    for (int n = 0; n < 4; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int r = r0 + g + (i >> 1) * 8, c = c0 + n * 8 + 2 * t + (i & 1);
            const float d = __expf(gs[r] - gs[c]);
            As[r * LDP + c] = c < r ? bs[r] * d * akk[n][i] : 0.f;
            Pg[r * CC + c] = c <= r ? d * aqk[n][i] : 0.f;
        }
    if (tid < CC) a.G[((long long)ch * a.VL + h) * CC + tid] = gs[tid];
    __syncthreads();
    // forward substitution: thread j owns column j of [Wv | Wk]
    const int j = tid & 127;
    const bool isk = tid >= 128;
    float wcol[CC];
#pragma unroll
    for (int r = 0; r < CC; ++r) {
        float b;
        if (isk) b = bs[r] * __expf(gs[r]) * Ks[r * LDA + j];
        else b = (m0 + r < a.M) ? bs[r] * a.qkv[(long long)(m0 + r) * qkv_l + (2 * a.KL + h) * CD + j] : 0.f;
        wcol[r] = b;
    }
#pragma unroll
    for (int r = 1; r < CC; ++r) {
        float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f, acc3 = 0.f;      // four independent chains: a row's sum is r / 4 dependent FMAs deep
#pragma unroll
        for (int s4 = 0; s4 < r; s4 += 4) {
            const float4 av = *reinterpret_cast<const float4 *>(As + r * LDP + s4);     // zero at s >= r
            acc0 = fmaf(av.x, wcol[s4], acc0);
            if (s4 + 1 < r) acc1 = fmaf(av.y, wcol[s4 + 1], acc1);
            if (s4 + 2 < r) acc2 = fmaf(av.z, wcol[s4 + 2], acc2);
            if (s4 + 3 < r) acc3 = fmaf(av.w, wcol[s4 + 3], acc3);
        }
        wcol[r] -= (acc0 + acc1) + (acc2 + acc3);
    }
    float *Wg = (isk ? a.Wk : a.Wv) + ((long long)ch * a.VL + h) * CC * CD;
#pragma unroll
    for (int r = 0; r < CC; ++r) Wg[r * CD + j] = wcol[r];
}

// ------------------------------------------------------------------------------------------------
// 2. state-dependent part: one block per (half of the value columns, head) walks the chunks
// ------------------------------------------------------------------------------------------------
// NC = value columns of the state per block (64, 32 or 16): the value columns of a head are independent in every
// state-dependent product, so a head is split over 128 / NC blocks; with few heads per rank (tensor parallel) a finer
// split keeps the number of blocks up.  Every output element's sum runs over k in the same order whatever NC is.
template <int NC>
constexpr int apply_smem() {
    return (CD * (NC + 8) + 2 * CC * LDA + CC * LDT + 2 * CC * LDP + CC * (NC + 8) + 2 * CC) * 4;
}

// 16-byte asynchronous copy global -> shared; `ok` false: the destination is zero-filled (rows past the run's end).
__device__ __forceinline__ void cp_async16(float *dst, const float *src, bool ok) {
    const unsigned int d = (unsigned int)__cvta_generic_to_shared(dst);
    const int n = ok ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Rows [m0, m0+64) x 128 floats at column offset col of the qkv rows -> shared tile of stride ld, asynchronously; rows
// >= M become zero.  256 threads.
__device__ __forceinline__ void load_tile_async(float *dst, int ld, const float *qkv, int qkv_l, int col, int m0, int M, int tid) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int idx = tid + i * 256;          // float4 index: 64 rows x 32
        const int r = idx >> 5, c4 = idx & 31;
        const bool ok = m0 + r < M;
        cp_async16(dst + r * ld + c4 * 4, qkv + (long long)(ok ? m0 + r : 0) * qkv_l + col + c4 * 4, ok);
    }
}

// The kernel walks the chunks in order; what a chunk needs from global memory is in shared memory before its products
// start: Wk, Q, P and the cumulative log decays of chunk c + 1 are fetched (cp.async) into the tiles that chunk c's first
// product has finished with, under chunk c's second and third products; K of chunk c, needed only by the third
// product, is fetched under the first two.  The chain of 64 chunk steps of a 4,096-token run is what bounds the
// kernel (it does not shorten with fewer heads per rank), so nothing on it waits for a global load.
template <int NC>
__global__ void __launch_bounds__(256) gdn_chunk_apply_kernel(GdnChunkArgs a) {
    constexpr int LDS = NC + 8;          // [.][NC] B-operand tile (state slice, U)
    constexpr int NT = NC / 16;          // 8-column tiles of a warp in the row-tiled products
    constexpr int NS = NC / 8;           // 8-column tiles of a warp in the state update
    extern __shared__ __align__(16) float sm[];
    float *Ss = sm;                      // [128 k][LDS]   state, this block's NC value columns
    float *Wks = Ss + CD * LDS;          // [64][LDA]
    float *Qs = Wks + CC * LDA;          // [64][LDA]
    float *Ks = Qs + CC * LDA;           // [64][LDT]      read transposed in the state update
    float *Ps = Ks + CC * LDT;           // [2][64][LDP]   chunk c in buffer c & 1
    float *Us = Ps + 2 * CC * LDP;       // [64][LDS]
    float *gb = Us + CC * LDS;           // [2][64]        cumulative log decay g_t of the chunk
    const int vh = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int qkv_l = (2 * a.KL + a.VL) * CD;
    const int kh = h / (a.VL / a.KL);
    const int slot = a.slot[0];
    float *Sg = a.S + ((long long)slot * a.VL + h) * CD * CD + vh * NC;
    const int nch = (a.M + CC - 1) / CC;
    // what chunk `ch` needs before its first product: Q, Wk, P, g
    auto fetch_front = [&](int ch) {
        const long long cb = (long long)ch * a.VL + h;
        load_tile_async(Qs, LDA, a.qkv, qkv_l, kh * CD, ch * CC, a.M, tid);
        load_tile_async(Wks, LDA, a.Wk + cb * CC * CD, CD, 0, 0, CC, tid);
        const float *Pg = a.P + cb * CC * CC;
        float *Pd = Ps + (ch & 1) * CC * LDP;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = tid + i * 256;      // float4 index: 64 rows x 16
            const int r = idx >> 4, c4 = idx & 15;
            cp_async16(Pd + r * LDP + c4 * 4, Pg + r * CC + c4 * 4, true);
        }
        if (tid < CC / 4) cp_async16(gb + (ch & 1) * CC + tid * 4, a.G + cb * CC + tid * 4, true);
    };
    fetch_front(0);
    cp_async_commit();
    for (int idx = tid; idx < CD * (NC / 4); idx += 256) {      // float4 index: 128 rows x NC / 4
        const int r = idx / (NC / 4), c4 = idx % (NC / 4);
        *reinterpret_cast<float4 *>(Ss + r * LDS + c4 * 4) = *reinterpret_cast<const float4 *>(Sg + r * CD + c4 * 4);
    }
    const int r0 = (w & 3) * 16, c0 = (w >> 2) * (NC / 2);
    for (int ch = 0; ch < nch; ++ch) {
        const int m0 = ch * CC;
        const long long cb = (long long)ch * a.VL + h;
        const float *Pc = Ps + (ch & 1) * CC * LDP, *gc = gb + (ch & 1) * CC;
        load_tile_async(Ks, LDT, a.qkv, qkv_l, (a.KL + kh) * CD, m0, a.M, tid);      // for the third product
        cp_async_commit();
        cp_async_wait<1>();              // everything but K: this chunk's Q, Wk, P, g are in
        __syncthreads();
        // Wv of this thread's U elements: issued now, used after the first product
        const float *Wvg = a.Wv + cb * CC * CD + vh * NC;
        float2 wv0[NT], wv1[NT];
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            const int c = c0 + n * 8 + 2 * t;
            wv0[n] = *reinterpret_cast<const float2 *>(Wvg + (r0 + g) * CD + c);
            wv1[n] = *reinterpret_cast<const float2 *>(Wvg + (r0 + g + 8) * CD + c);
        }
        // U = Wv - Wk S0 and Q S0: warp tile 16 rows x NC / 2 value columns
        float accW[NT][4], accO[NT][4];
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) accW[n][i] = accO[n][i] = 0.f;
#pragma unroll 4
        for (int k0 = 0; k0 < CD; k0 += 8) {
            uint32_t fw[4], fq[4];
            lda_frag(fw, Wks, LDA, r0, k0, g, t);
            lda_frag(fq, Qs, LDA, r0, k0, g, t);
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                const float *p = Ss + (k0 + t) * LDS + c0 + n * 8 + g;
                const uint32_t b0 = tf32(p[0]), b1 = tf32(p[4 * LDS]);
                mma_tf32(accW[n], fw, b0, b1);
                mma_tf32(accO[n], fq, b0, b1);
            }
        }
        {
            const float e0 = __expf(gc[r0 + g]), e1 = __expf(gc[r0 + g + 8]);
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                const int c = c0 + n * 8 + 2 * t;
                *reinterpret_cast<float2 *>(Us + (r0 + g) * LDS + c) = make_float2(wv0[n].x - accW[n][0], wv0[n].y - accW[n][1]);
                *reinterpret_cast<float2 *>(Us + (r0 + g + 8) * LDS + c) = make_float2(wv1[n].x - accW[n][2], wv1[n].y - accW[n][3]);
                accO[n][0] *= e0; accO[n][1] *= e0;
                accO[n][2] *= e1; accO[n][3] *= e1;
            }
        }
        __syncthreads();                 // U is complete; the Q and Wk tiles are free
        const bool more = ch + 1 < nch;
        if (more) {
            fetch_front(ch + 1);
            cp_async_commit();
        }
        // O += P U (P is zero above the diagonal: k tiles past the warp's rows are skipped)
        for (int k0 = 0; k0 < r0 + 16; k0 += 8) {
            uint32_t fp[4];
            lda_frag(fp, Pc, LDP, r0, k0, g, t);
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                const float *p = Us + (k0 + t) * LDS + c0 + n * 8 + g;
                mma_tf32(accO[n], fp, tf32(p[0]), tf32(p[4 * LDS]));
            }
        }
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            const int c = h * CD + vh * NC + c0 + n * 8 + 2 * t;
            const int ra = m0 + r0 + g, rb = ra + 8;
            if (ra < a.M) *reinterpret_cast<float2 *>(a.Oraw + (long long)ra * a.VL * CD + c) = make_float2(accO[n][0], accO[n][1]);
            if (rb < a.M) *reinterpret_cast<float2 *>(a.Oraw + (long long)rb * a.VL * CD + c) = make_float2(accO[n][2], accO[n][3]);
        }
        if (more) cp_async_wait<1>();    // K of this chunk (the next chunk's front tiles may still be on their way)
        else cp_async_wait<0>();
        __syncthreads();
        // S1 = exp(g_C) S0 + (diag(ek) K)^T U: warp w owns state rows 16w .. 16w+15, all NC columns
        {
            const int i0 = w * 16;
            const float gC = gc[CC - 1];
            const float eC = __expf(gC);
            float accS[NS][4];
#pragma unroll
            for (int n = 0; n < NS; ++n) {
                const float2 s0 = *reinterpret_cast<const float2 *>(Ss + (i0 + g) * LDS + n * 8 + 2 * t);
                const float2 s1 = *reinterpret_cast<const float2 *>(Ss + (i0 + g + 8) * LDS + n * 8 + 2 * t);
                accS[n][0] = s0.x * eC; accS[n][1] = s0.y * eC;
                accS[n][2] = s1.x * eC; accS[n][3] = s1.y * eC;
            }
#pragma unroll 2
            for (int k0 = 0; k0 < CC; k0 += 8) {
                const float ea = __expf(gC - gc[k0 + t]), eb = __expf(gC - gc[k0 + t + 4]);
                const float *p = Ks + (k0 + t) * LDT + i0 + g;      // A[i][s] = K[s][i] ek[s]
                uint32_t fa[4];
                fa[0] = tf32(p[0] * ea);
                fa[1] = tf32(p[8] * ea);
                fa[2] = tf32(p[4 * LDT] * eb);
                fa[3] = tf32(p[4 * LDT + 8] * eb);
#pragma unroll
                for (int n = 0; n < NS; ++n) {
                    const float *q = Us + (k0 + t) * LDS + n * 8 + g;
                    mma_tf32(accS[n], fa, tf32(q[0]), tf32(q[4 * LDS]));
                }
            }
#pragma unroll
            for (int n = 0; n < NS; ++n) {
                *reinterpret_cast<float2 *>(Ss + (i0 + g) * LDS + n * 8 + 2 * t) = make_float2(accS[n][0], accS[n][1]);
                *reinterpret_cast<float2 *>(Ss + (i0 + g + 8) * LDS + n * 8 + 2 * t) = make_float2(accS[n][2], accS[n][3]);
            }
        }
        __syncthreads();
    }
    for (int idx = tid; idx < CD * (NC / 4); idx += 256) {
        const int r = idx / (NC / 4), c4 = idx % (NC / 4);
        *reinterpret_cast<float4 *>(Sg + r * CD + c4 * 4) = *reinterpret_cast<const float4 *>(Ss + r * LDS + c4 * 4);
    }
}

// ------------------------------------------------------------------------------------------------
// 3. gated RMS norm over each head's 128 outputs
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) gdn_chunk_norm_kernel(GdnChunkArgs a) {
    __shared__ float scratch[32];
    const int m = blockIdx.x, h = blockIdx.y, c = threadIdx.x;
    const int qkv_l = (2 * a.KL + a.VL) * CD;
    const long long oi = (long long)m * a.VL * CD + h * CD + c;
    const float ov = a.Oraw[oi];
    const float ss = block_sum<128>(ov * ov, scratch);
    const float z = a.proj[(long long)m * a.ld_proj + qkv_l + h * CD + c];
    a.o[oi] = __float2bfloat16(ov * rsqrtf(ss / float(CD) + a.eps) * a.norm_w[c] * sigmoidf_(z));
}

}  // namespace qw

using namespace qw;

// The scan of one slot's run of M rows (rows 0..M-1 consecutive positions of slot[0]): same inputs and outputs
// as qwk_gdn_scan without the per-row state saves.  `scratch` holds
// 4 * (ceil(M / 64) * VL * (2 * 64 * 128 + 64 * 64 + 64) + M * VL * 128) bytes.
QW_API int qwk_gdn_scan_chunked(const float *qkv, const float *decay, const float *beta, const float *proj, int ld_proj,
                                float *S, const float *norm_w, int KL, int VL, int M, const int *slot, float *scratch,
                                void *o, float eps, cudaStream_t s) {
    if (M < 1 || KL < 1 || VL % KL != 0) return -1;
    static bool attr_done[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (!attr_done[dev]) {
        if (cudaFuncSetAttribute(gdn_chunk_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PREP_SMEM) != cudaSuccess ||
            cudaFuncSetAttribute(gdn_chunk_apply_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, apply_smem<64>()) != cudaSuccess ||
            cudaFuncSetAttribute(gdn_chunk_apply_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, apply_smem<32>()) != cudaSuccess ||
            cudaFuncSetAttribute(gdn_chunk_apply_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, apply_smem<16>()) != cudaSuccess)
            return -3;
        attr_done[dev] = true;
    }
    const long long nch = (M + CC - 1) / CC;
    GdnChunkArgs a;
    a.qkv = qkv; a.decay = decay; a.beta = beta; a.proj = proj; a.ld_proj = ld_proj; a.S = S; a.norm_w = norm_w;
    a.KL = KL; a.VL = VL; a.M = M; a.slot = slot; a.eps = eps; a.o = (bf16 *)o;
    a.Wk = scratch;
    a.Wv = a.Wk + nch * VL * CC * CD;
    a.P = a.Wv + nch * VL * CC * CD;
    a.G = a.P + nch * VL * CC * CC;
    a.Oraw = a.G + nch * VL * CC;
    gdn_chunk_prep_kernel<<<dim3((unsigned)nch, VL), 256, PREP_SMEM, s>>>(a);
    // blocks of the sequential walk: 128 / NC per head, NC chosen so that about a hundred blocks run
    if (VL >= 32) gdn_chunk_apply_kernel<64><<<dim3(2, VL), 256, apply_smem<64>(), s>>>(a);
    else if (VL >= 16) gdn_chunk_apply_kernel<32><<<dim3(4, VL), 256, apply_smem<32>(), s>>>(a);
    else gdn_chunk_apply_kernel<16><<<dim3(8, VL), 256, apply_smem<16>(), s>>>(a);
    gdn_chunk_norm_kernel<<<dim3(M, VL), 128, 0, s>>>(a);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
