// QSA (sparse attention with a learned indexer) kernels for row batches over a paged KV cache:
// prep (norms, RoPE, KV/raw-key/compressed-key writes), indexer scores, top-k group selection by
// radix select with ties to the lowest index, flash-decode over the selected tokens and the merge
// of its partials with the output gate (roles of the reference's src/kernels/qsa.hip:136-243 and
// src/kernels/model_common.cuh:92-303; math in docs/MODEL.md:135-174).
//
// Projection row layout per rank (fp32): [ per q head: q(256) gate(256) | k (KVL x 256) | v (KVL x 256) |
// indexer q (IH x 128) | raw indexer key (128) ].
//
// KV pages: a page holds KV_PAGE tokens of one layer, row = KVL*256 bf16.  page ids < n_dev_pages
// live in the device pool, the rest in the host pool (pinned, mapped: the kernels read host RAM
// directly).  page_table[slot][i] is the page of tokens i*KV_PAGE ...
#include "common.cuh"
#include "mma.cuh"

namespace qw {

constexpr int HD = 256;      // attention head dim
constexpr int ID = 128;      // indexer head dim
constexpr int MAX_HALF = 64; // rope_dim/2 upper bound

__constant__ double c_inv_freq[MAX_HALF];
__constant__ int c_rope_half;

struct KvPool {
    bf16 *k_dev, *v_dev;
    bf16 *k_host, *v_host;
    int n_dev_pages;
    const int *page_table;   // [slots][max_pages]
    int max_pages;
    int row;                 // elements per token row (KVL*256)
};

__device__ __forceinline__ long long kv_off(const KvPool &kv, int slot, int pos, bool &host) {
    const int page = kv.page_table[(long long)slot * kv.max_pages + pos / KV_PAGE];
    host = page >= kv.n_dev_pages;
    const long long p = host ? page - kv.n_dev_pages : page;
    return (p * KV_PAGE + (pos % KV_PAGE)) * kv.row;
}
__device__ __forceinline__ bf16 *k_row(const KvPool &kv, int slot, int pos) {
    bool host;
    const long long o = kv_off(kv, slot, pos, host);
    return (host ? kv.k_host : kv.k_dev) + o;
}
__device__ __forceinline__ bf16 *v_row(const KvPool &kv, int slot, int pos) {
    bool host;
    const long long o = kv_off(kv, slot, pos, host);
    return (host ? kv.v_host : kv.v_dev) + o;
}

// Device-memory cache in front of the host KV pages: direct mapped, one entry = the K row and the V row of one
// token of one layer, tagged with the host address of the K row.  The attention kernel looks a host row up, reads the
// cached copy on a hit and the host row itself on a miss (then also lists the row); the fill kernel that runs right
// after the attention kernels copies the listed rows in.  A kernel that writes a host row drops its entry.
// (Role of the reference's SpillCache, src/kernels/types.hpp:48-70, and spill_cache_fill, src/kernels/qsa.hip:247-273.)
struct SpillCache {
    unsigned long long *tags;    // [mask + 1]: host address of the cached K row; 0 = empty, 1 = being filled
    bf16 *rows;                  // [mask + 1][2][row]
    unsigned long long *miss;    // [miss_cap] K-row addresses that missed since the last fill
    unsigned *ctl;               // [0] number of misses listed (may run past miss_cap), [1] fill ticket
    unsigned long long *stats;   // [0] hits, [1] misses; nullptr = not counted
    unsigned mask;
    int miss_cap;
};
__device__ __forceinline__ unsigned spill_index(unsigned long long key, unsigned mask) {
    return (unsigned)(((key >> 9) * 0x9E3779B97F4A7C15ull) >> 40) & mask;
}

// K and V row of (slot, pos) for reading.  `record`: this thread lists a miss (one thread per token).
__device__ __forceinline__ void kv_rows_read(const KvPool &kv, const SpillCache &sc, int slot, int pos, bool record,
                                             const bf16 *&kp, const bf16 *&vp) {
    bool host;
    const long long o = kv_off(kv, slot, pos, host);
    if (!host) {
        kp = kv.k_dev + o;
        vp = kv.v_dev + o;
        return;
    }
    kp = kv.k_host + o;
    vp = kv.v_host + o;
    if (sc.tags == nullptr) return;
    const unsigned long long key = reinterpret_cast<unsigned long long>(kp);
    const unsigned idx = spill_index(key, sc.mask);
    const bool hit = __ldcg(sc.tags + idx) == key;
    if (hit) {
        kp = sc.rows + (long long)idx * 2 * kv.row;
        vp = kp + kv.row;
    } else if (record) {
        const unsigned n = atomicAdd(sc.ctl, 1u);
        if (n < (unsigned)sc.miss_cap) sc.miss[n] = key;
    }
    if (record && sc.stats) atomicAdd(sc.stats + (hit ? 0 : 1), 1ull);
}
// A host row is about to be rewritten: its cached copy is dropped.
__device__ __forceinline__ void spill_drop(const KvPool &kv, const SpillCache &sc, int slot, int pos) {
    if (sc.tags == nullptr) return;
    bool host;
    const long long o = kv_off(kv, slot, pos, host);
    if (!host) return;
    const unsigned long long key = reinterpret_cast<unsigned long long>(kv.k_host + o);
    const unsigned idx = spill_index(key, sc.mask);
    if (__ldcg(sc.tags + idx) == key) sc.tags[idx] = 0ull;
}

// One warp per listed miss.  The entry is claimed by exchanging its tag with 1: a warp that finds 1 there leaves the
// entry to the warp that is filling it, a warp that finds its own key puts it back.  The last block resets the list.
__global__ void __launch_bounds__(256) spill_cache_fill_kernel(SpillCache sc, const bf16 *k_host, const bf16 *v_host, int row) {
    const int lane = threadIdx.x & 31;
    const unsigned n = min(__ldcg(sc.ctl), (unsigned)sc.miss_cap);
    const unsigned nw = gridDim.x * (blockDim.x >> 5);
    for (unsigned i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); i < n; i += nw) {
        const unsigned long long key = __ldcg(sc.miss + i);
        const unsigned idx = spill_index(key, sc.mask);
        unsigned long long prev = 0ull;
        if (lane == 0) prev = atomicExch(sc.tags + idx, 1ull);
        prev = __shfl_sync(0xffffffffu, prev, 0);
        if (prev == 1ull) continue;
        if (prev != key) {
            const uint4 *ks = reinterpret_cast<const uint4 *>(key);
            const uint4 *vs = reinterpret_cast<const uint4 *>(v_host + (reinterpret_cast<const bf16 *>(key) - k_host));
            uint4 *dst = reinterpret_cast<uint4 *>(sc.rows + (long long)idx * 2 * row);
            const int n16 = row >> 3;
            for (int j = lane; j < n16; j += 32) {
                dst[j] = ks[j];
                dst[n16 + j] = vs[j];
            }
            __threadfence();
        }
        __syncwarp();
        if (lane == 0) atomicExch(sc.tags + idx, key);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(sc.ctl + 1, 1u) == gridDim.x - 1) {
            sc.ctl[0] = 0u;
            sc.ctl[1] = 0u;
        }
    }
}

struct QsaPrepArgs {
    SpillCache sc;
    const float *proj;
    int ld_proj;
    int QL, KVL, IH;
    const float *qn1, *kn1, *iqn1, *ikn1;   // (1+w) norm weights: [256],[256],[128],[128]
    Rows rows;
    KvPool kv;
    float *q;            // [M][QL][256] normed + rotated queries
    float *iq;           // [M][IH][128]
    float *raw_ring;     // [slots][RAW_RING][128]
    bf16 *ck;            // [slots][ck_cap][128]
    int ck_cap;
    int ratio;           // tokens per compressed group
    float eps;
    int ring_inline;     // 1: the raw-key block also stores its row in the ring (safe for runs <= RAW_RING - ratio)
};

// Normalise (gemma: * (1+w)), rotate the first 2*half dims NeoX style.  v lives in sm[0..D).
template <int D>
__device__ __forceinline__ float norm_rope(float v, float *sm, float *scratch, const float *cs, const float *w1, float eps,
                                           int d) {
    const float ss = block_sum<256>(d < D ? v * v : 0.f, scratch);
    const float r = rsqrtf(ss / float(D) + eps);
    if (d < D) sm[d] = v * r * w1[d];
    __syncthreads();
    float out = 0.f;
    if (d < D) {
        const int half = c_rope_half;
        if (d < half) out = sm[d] * cs[d] - sm[d + half] * cs[MAX_HALF + d];
        else if (d < 2 * half) out = sm[d] * cs[d - half] + sm[d - half] * cs[MAX_HALF + d - half];
        else out = sm[d];
    }
    __syncthreads();
    return out;
}

__device__ __forceinline__ void fill_cs(float *cs, int pos) {
    if (threadIdx.x < c_rope_half) {
        double sd, cd;
        sincos(double(pos) * c_inv_freq[threadIdx.x], &sd, &cd);
        cs[threadIdx.x] = float(cd);
        cs[MAX_HALF + threadIdx.x] = float(sd);
    }
    __syncthreads();
}

// grid (M, QL + 2*KVL + IH + 1), 256 threads.
__global__ void __launch_bounds__(256) qsa_prep_kernel(QsaPrepArgs a) {
    pdl_wait();          // launched with programmatic dependent launch: the predecessor's results are needed from here on
    pdl_trigger();
    __shared__ float sm[HD];
    __shared__ float scratch[32];
    __shared__ float cs[2 * MAX_HALF];
    const int m = blockIdx.x, hb = blockIdx.y, d = threadIdx.x;
    const int slot = a.rows.slot[m], pos = a.rows.pos[m];
    // a position beyond the slot's page table, or a page entry that is not a page (row m)
    QW_DCHECK(slot >= 0 && pos >= 0 && pos / KV_PAGE < a.kv.max_pages, 0x02000000u | (unsigned)(m & 0xffffff));
    QW_DCHECK(a.kv.page_table[(long long)slot * a.kv.max_pages + pos / KV_PAGE] >= 0, 0x03000000u | (unsigned)(m & 0xffffff));
    const float *row = a.proj + (long long)m * a.ld_proj;
    const int off_k = a.QL * 2 * HD, off_v = off_k + a.KVL * HD, off_iq = off_v + a.KVL * HD, off_raw = off_iq + a.IH * ID;
    if (hb < a.QL) {                                   // query head
        fill_cs(cs, pos);
        const float v = norm_rope<HD>(row[hb * 2 * HD + d], sm, scratch, cs, a.qn1, a.eps, d);
        a.q[((long long)m * a.QL + hb) * HD + d] = v;
    } else if (hb < a.QL + a.KVL) {                    // key head
        const int j = hb - a.QL;
        fill_cs(cs, pos);
        const float v = norm_rope<HD>(row[off_k + j * HD + d], sm, scratch, cs, a.kn1, a.eps, d);
        if (j == 0 && d == 0) spill_drop(a.kv, a.sc, slot, pos);
        k_row(a.kv, slot, pos)[j * HD + d] = __float2bfloat16(v);
    } else if (hb < a.QL + 2 * a.KVL) {                // value head
        const int j = hb - a.QL - a.KVL;
        v_row(a.kv, slot, pos)[j * HD + d] = __float2bfloat16(row[off_v + j * HD + d]);
    } else if (hb < a.QL + 2 * a.KVL + a.IH) {         // indexer query head
        const int j = hb - a.QL - 2 * a.KVL;
        fill_cs(cs, pos);
        const float v = norm_rope<ID>(d < ID ? row[off_iq + j * ID + d] : 0.f, sm, scratch, cs, a.iqn1, a.eps, d);
        if (d < ID) a.iq[((long long)m * a.IH + j) * ID + d] = v;
    } else {                                           // raw key: ring write + compressed key when a group completes
        const int rs = a.rows.run_start[m];
        float *ring = a.raw_ring + (long long)slot * RAW_RING * ID;
        const int len = a.rows.run_len[rs];
        // The ring entry of position p is shared with p +- RAW_RING: with long runs another row's block
        // could overwrite an entry this block still reads, so long batches store the ring in a second kernel.
        if (a.ring_inline && d < ID && (m - rs) >= len - RAW_RING) ring[(pos % RAW_RING) * ID + d] = row[off_raw + d];
        if ((pos + 1) % a.ratio != 0) return;
        float mean = 0.f;
        if (d < ID) {
            for (int r = 0; r < a.ratio; ++r) {        // positions pos-ratio+1 .. pos, oldest first
                const int back = a.ratio - 1 - r;
                if (m - back >= rs) mean += a.proj[(long long)(m - back) * a.ld_proj + off_raw + d];
                else mean += ring[((pos - back) % RAW_RING) * ID + d];
            }
            mean /= float(a.ratio);
        }
        const int gpos = pos + 1 - a.ratio;
        fill_cs(cs, gpos);
        const float v = norm_rope<ID>(mean, sm, scratch, cs, a.ikn1, a.eps, d);
        const int g = pos / a.ratio;
        if (d < ID && g < a.ck_cap) a.ck[((long long)slot * a.ck_cap + g) * ID + d] = __float2bfloat16(v);
    }
}

// grid M, 128 threads: raw-key ring store for long batches (runs after qsa_prep_kernel).
__global__ void qsa_raw_ring_kernel(const float *proj, int ld_proj, int off_raw, float *raw_ring, Rows rows) {
    pdl_wait();          // launched with programmatic dependent launch: the predecessor's results are needed from here on
    pdl_trigger();
    const int m = blockIdx.x, d = threadIdx.x;
    const int rs = rows.run_start[m], len = rows.run_len[rs];
    if ((m - rs) < len - RAW_RING) return;
    raw_ring[((long long)rows.slot[m] * RAW_RING + (rows.pos[m] % RAW_RING)) * ID + d] = proj[(long long)m * ld_proj + off_raw + d];
}

// ------------------------------------------------------------------------------------------
// Indexer scores: score[m][c] = sum_h relu(iq[m][h] . ck[c]) / sqrt(128), c < nb(m); only for
// rows whose visible groups exceed the budget.  grid (ceil(cap/64), M), 256 threads.
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) qsa_scores_kernel(const float *iq, int IH, const bf16 *ck, int ck_cap, Rows rows,
                                                         int ratio, int topk_blocks, float *scores, int ld_scores) {
    pdl_wait();          // launched with programmatic dependent launch: the predecessor's results are needed from here on
    pdl_trigger();
    __shared__ float q[8 * ID];          // IH <= 8
    const int m = blockIdx.y;
    const int slot = rows.slot[m], pos = rows.pos[m];
    const int nb = (pos + 1) / ratio;
    if (nb <= topk_blocks) return;
    const int g0 = blockIdx.x * 64;
    if (g0 >= nb) return;
    for (int i = threadIdx.x; i < IH * ID; i += 256) q[i] = iq[(long long)m * IH * ID + i];
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, half = lane >> 4, l16 = lane & 15;
    const bf16 *base = ck + (long long)slot * ck_cap * ID;
#pragma unroll
    for (int it = 0; it < 4; ++it) {
        const int g = g0 + warp * 8 + it * 2 + half;
        const int gc = g < nb ? g : nb - 1;      // clamp so every lane runs the same shuffles
        float s = 0.f;
        const uint4 kv = __ldg(reinterpret_cast<const uint4 *>(base + (long long)gc * ID) + l16);
        const float kf[8] = {bf16_lo(kv.x), bf16_hi(kv.x), bf16_lo(kv.y), bf16_hi(kv.y),
                             bf16_lo(kv.z), bf16_hi(kv.z), bf16_lo(kv.w), bf16_hi(kv.w)};
        for (int h = 0; h < IH; ++h) {
            float p = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) p = fmaf(kf[i], q[h * ID + l16 * 8 + i], p);
            p += __shfl_xor_sync(0xffffffffu, p, 1);
            p += __shfl_xor_sync(0xffffffffu, p, 2);
            p += __shfl_xor_sync(0xffffffffu, p, 4);
            p += __shfl_xor_sync(0xffffffffu, p, 8);
            s += fmaxf(p, 0.f);
        }
        if (g < nb && l16 == 0) scores[(long long)m * ld_scores + g] = s * 0.08838834764831845f;
    }
}

// ------------------------------------------------------------------------------------------
// Selection.  One block of 1024 threads per row.  sel_n[m] = -1: every visible token is attended
// (dense); else sel[m][0..topk) = the chosen groups in ascending order.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ int block_exscan_1024(int v, int *wsum, int &total) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    int x = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int y = __shfl_up_sync(0xffffffffu, x, o);
        if (lane >= o) x += y;
    }
    __syncthreads();
    if (lane == 31) wsum[w] = x;
    __syncthreads();
    if (w == 0) {
        int s = wsum[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int y = __shfl_up_sync(0xffffffffu, s, o);
            if (lane >= o) s += y;
        }
        wsum[lane] = s;
    }
    __syncthreads();
    total = wsum[31];
    return x - v + (w ? wsum[w - 1] : 0);
}

__global__ void __launch_bounds__(1024) qsa_select_kernel(const float *scores, int ld_scores, Rows rows, int ratio,
                                                          int topk, int *sel, int *sel_n) {
    pdl_wait();          // launched with programmatic dependent launch: the predecessor's results are needed from here on
    pdl_trigger();
    __shared__ int hist[256];
    __shared__ int wsum[32];
    __shared__ unsigned int s_prefix;
    __shared__ int s_need;
    const int m = blockIdx.x;
    const int pos = rows.pos[m];
    const int nb = (pos + 1) / ratio;
    if (nb <= topk) {
        if (threadIdx.x == 0) sel_n[m] = -1;
        return;
    }
    const unsigned int *key = reinterpret_cast<const unsigned int *>(scores + (long long)m * ld_scores);
    if (threadIdx.x == 0) { s_prefix = 0u; s_need = topk; }
    for (int pass = 0; pass < 4; ++pass) {
        const int shift = 24 - 8 * pass;
        if (threadIdx.x < 256) hist[threadIdx.x] = 0;
        __syncthreads();
        const unsigned int prefix = s_prefix;
        const unsigned int mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
        for (int i = threadIdx.x; i < nb; i += 1024) {
            const unsigned int k = key[i];
            if ((k & mask) == prefix) atomicAdd(&hist[(k >> shift) & 0xff], 1);
        }
        __syncthreads();
        if (threadIdx.x < 32) {
            // the highest bin b whose count from the top reaches `need` (0 if none does), found by one warp: lane l owns
            // bins 8 l .. 8 l + 7, a suffix sum over the lanes locates the lane, a scan of its 8 bins the bin
            const int lane = threadIdx.x, need = s_need;
            int loc[8], own = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) { loc[j] = hist[8 * lane + j]; own += loc[j]; }
            int suf = own;                                   // bins of this lane and of all higher lanes
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const int t = __shfl_down_sync(0xffffffffu, suf, off);
                if (lane + off < 32) suf += t;
            }
            const int above = suf - own;
            const bool mine = above < need && need <= suf;
            const unsigned int who = __ballot_sync(0xffffffffu, mine);
            if (who == 0u) {                                 // fewer than `need` entries in all bins above 0: bin 0 takes the rest
                const int tot = __shfl_sync(0xffffffffu, suf, 0);
                if (lane == 0) { s_need = need - (tot - loc[0]); s_prefix = prefix; }
            } else if (mine) {
                int rem = need - above, b = 7;
                for (; b > 0; --b) {
                    if (loc[b] >= rem) break;
                    rem -= loc[b];
                }
                s_need = rem;
                s_prefix = prefix | ((unsigned int)(8 * lane + b) << shift);
            }
        }
        __syncthreads();
    }
    const unsigned int T = s_prefix;
    const int need_eq = s_need;          // entries equal to T to take, lowest indices first
    int base_out = 0, base_eq = 0;
    for (int i0 = 0; i0 < nb; i0 += 1024) {
        const int i = i0 + threadIdx.x;
        const unsigned int k = i < nb ? key[i] : 0u;
        const int gt = (i < nb && k > T) ? 1 : 0;
        const int eq = (i < nb && k == T) ? 1 : 0;
        int tot_eq, tot_out;
        const int eq_rank = base_eq + block_exscan_1024(eq, wsum, tot_eq);
        const int take = gt | (eq && eq_rank < need_eq ? 1 : 0);
        const int o = base_out + block_exscan_1024(take, wsum, tot_out);
        if (take && o < topk) sel[(long long)m * topk + o] = i;
        base_eq += tot_eq;
        base_out += tot_out;
        __syncthreads();
    }
    if (threadIdx.x == 0) sel_n[m] = topk;
}

// ------------------------------------------------------------------------------------------
// Flash-decode over the token list.  grid (NSPLIT, M, QL/HT), 256 threads; each block covers 64
// list entries for HT query heads that share one KV head.
// ------------------------------------------------------------------------------------------
struct QsaAttendArgs {
    SpillCache sc;
    const float *q;          // [M][QL][256]
    int QL, KVL;
    Rows rows;
    KvPool kv;
    const int *sel, *sel_n;  // [M][topk], [M]
    int topk, ratio;
    int nsplit;
    float *pm, *pl;          // [M][QL][nsplit]
    float *pacc;             // [M][QL][nsplit][256]
};

__device__ __forceinline__ int list_token(int t, int dense, const int *sel, int ratio, int topk, int nb) {
    if (dense) return t;
    if (t < topk * ratio) return sel[t / ratio] * ratio + t % ratio;
    return nb * ratio + (t - topk * ratio);
}

template <int HT>
__global__ void __launch_bounds__(256) qsa_attend_kernel(QsaAttendArgs a) {
    pdl_wait();          // launched with programmatic dependent launch: the predecessor's results are needed from here on
    pdl_trigger();
    __shared__ float s_acc[8][HT][HD];
    __shared__ float s_m[8][HT], s_l[8][HT];
    const int sp = blockIdx.x, m = blockIdx.y, h0 = blockIdx.z * HT;
    const int slot = a.rows.slot[m], pos = a.rows.pos[m];
    const int nb = (pos + 1) / a.ratio;
    const int dense = a.sel_n[m] < 0;
    const int count = dense ? pos + 1 : a.topk * a.ratio + (pos + 1 - nb * a.ratio);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kvh = (h0 * a.KVL) / a.QL;      // local KV head of this head tile
    const int *sel = a.sel + (long long)m * a.topk;
    float qv[HT][8], acc[HT][8], mx[HT], l[HT];
#pragma unroll
    for (int j = 0; j < HT; ++j) {
        const float4 *qp = reinterpret_cast<const float4 *>(a.q + ((long long)m * a.QL + h0 + j) * HD + lane * 8);
        const float4 q0 = qp[0], q1 = qp[1];
        qv[j][0] = q0.x; qv[j][1] = q0.y; qv[j][2] = q0.z; qv[j][3] = q0.w;
        qv[j][4] = q1.x; qv[j][5] = q1.y; qv[j][6] = q1.z; qv[j][7] = q1.w;
        mx[j] = -INFINITY;
        l[j] = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[j][i] = 0.f;
    }
    for (int it = 0; it < 8; ++it) {
        const int t = sp * 64 + it * 8 + warp;
        if (t >= count) break;                 // warp-uniform
        const int tok = list_token(t, dense, sel, a.ratio, a.topk, nb);
        const bf16 *kp, *vp;
        kv_rows_read(a.kv, a.sc, slot, tok, blockIdx.z == 0 && lane == 0, kp, vp);
        const uint4 kk = *(reinterpret_cast<const uint4 *>(kp + kvh * HD) + lane);
        const uint4 vv = *(reinterpret_cast<const uint4 *>(vp + kvh * HD) + lane);
        const float kf[8] = {bf16_lo(kk.x), bf16_hi(kk.x), bf16_lo(kk.y), bf16_hi(kk.y),
                             bf16_lo(kk.z), bf16_hi(kk.z), bf16_lo(kk.w), bf16_hi(kk.w)};
        const float vf[8] = {bf16_lo(vv.x), bf16_hi(vv.x), bf16_lo(vv.y), bf16_hi(vv.y),
                             bf16_lo(vv.z), bf16_hi(vv.z), bf16_lo(vv.w), bf16_hi(vv.w)};
#pragma unroll
        for (int j = 0; j < HT; ++j) {
            float p = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) p = fmaf(qv[j][i], kf[i], p);
            p = warp_sum(p) * 0.0625f;          // 1/sqrt(256)
            const float nm = fmaxf(mx[j], p);
            const float sc = __expf(mx[j] - nm), w = __expf(p - nm);
            l[j] = l[j] * sc + w;
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[j][i] = fmaf(acc[j][i], sc, w * vf[i]);
            mx[j] = nm;
        }
    }
#pragma unroll
    for (int j = 0; j < HT; ++j) {
        if (lane == 0) { s_m[warp][j] = mx[j]; s_l[warp][j] = l[j]; }
#pragma unroll
        for (int i = 0; i < 8; ++i) s_acc[warp][j][lane * 8 + i] = acc[j][i];
    }
    __syncthreads();
    // merge the 8 warps: thread d handles dim d of every head in the tile
    const int d = threadIdx.x;
#pragma unroll
    for (int j = 0; j < HT; ++j) {
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 8; ++w) M = fmaxf(M, s_m[w][j]);
        float L = 0.f, A = 0.f;
        if (M > -INFINITY) {
#pragma unroll
            for (int w = 0; w < 8; ++w) {
                const float sc = s_m[w][j] > -INFINITY ? __expf(s_m[w][j] - M) : 0.f;
                L = fmaf(s_l[w][j], sc, L);
                A = fmaf(s_acc[w][j][d], sc, A);
            }
        }
        const long long o = ((long long)m * a.QL + h0 + j) * a.nsplit + sp;
        a.pacc[o * HD + d] = A;
        if (d == 0) { a.pm[o] = M; a.pl[o] = L; }
    }
}

// grid (M, QL), 256 threads: merge the splits, apply sigmoid(gate), write bf16.
__global__ void __launch_bounds__(256) qsa_combine_kernel(const float *pm, const float *pl, const float *pacc, int nsplit,
                                                          const float *proj, int ld_proj, int QL, bf16 *o) {
    pdl_wait();          // launched with programmatic dependent launch: the predecessor's results are needed from here on
    pdl_trigger();
    const int m = blockIdx.x, h = blockIdx.y, d = threadIdx.x;
    const long long b = ((long long)m * QL + h) * nsplit;
    float M = -INFINITY;
    for (int s = 0; s < nsplit; ++s) M = fmaxf(M, pm[b + s]);
    float L = 0.f, A = 0.f;
    for (int s = 0; s < nsplit; ++s) {
        const float ms = pm[b + s];
        if (ms == -INFINITY) continue;
        const float sc = __expf(ms - M);
        L = fmaf(pl[b + s], sc, L);
        A = fmaf(pacc[(b + s) * HD + d], sc, A);
    }
    const float gate = proj[(long long)m * ld_proj + h * 2 * HD + HD + d];
    o[((long long)m * QL + h) * HD + d] = __float2bfloat16(A / L * sigmoidf_(gate));
}

#include "qsa_mma.cuh"

}  // namespace qw

using namespace qw;

QW_DCHECK_TU(qsa)

QW_API int qwk_rope_init(double theta, int rope_dim) {
    double inv[MAX_HALF];
    const int half = rope_dim / 2;
    if (half > MAX_HALF) return -1;
    for (int i = 0; i < half; ++i) inv[i] = pow(theta, -2.0 * double(i) / double(rope_dim));
    if (cudaMemcpyToSymbol(c_inv_freq, inv, sizeof(double) * half) != cudaSuccess) return -2;
    if (cudaMemcpyToSymbol(c_rope_half, &half, sizeof(int)) != cudaSuccess) return -2;
    return 0;
}

static SpillCache g_spill{};          // process-wide; all-null = no cache

static KvPool make_pool(void *k_dev, void *v_dev, void *k_host, void *v_host, int n_dev_pages, const int *page_table,
                        int max_pages, int row) {
    KvPool p;
    p.k_dev = (bf16 *)k_dev; p.v_dev = (bf16 *)v_dev; p.k_host = (bf16 *)k_host; p.v_host = (bf16 *)v_host;
    p.n_dev_pages = n_dev_pages; p.page_table = page_table; p.max_pages = max_pages; p.row = row;
    return p;
}

QW_API int qwk_qsa_prep(const float *proj, int ld_proj, int QL, int KVL, int IH, const float *qn1, const float *kn1,
                        const float *iqn1, const float *ikn1, int M, const int *slot, const int *pos,
                        const int *run_start, const int *run_len, void *k_dev, void *v_dev, void *k_host, void *v_host,
                        int n_dev_pages, const int *page_table, int max_pages, float *q, float *iq, float *raw_ring,
                        void *ck, int ck_cap, int ratio, float eps, cudaStream_t s) {
    if (IH > 8) return -1;
    QsaPrepArgs a;
    a.proj = proj; a.ld_proj = ld_proj; a.QL = QL; a.KVL = KVL; a.IH = IH;
    a.qn1 = qn1; a.kn1 = kn1; a.iqn1 = iqn1; a.ikn1 = ikn1;
    a.rows = Rows{M, slot, pos, run_start, run_len};
    a.kv = make_pool(k_dev, v_dev, k_host, v_host, n_dev_pages, page_table, max_pages, KVL * HD);
    a.sc = k_host ? g_spill : SpillCache{};
    a.q = q; a.iq = iq; a.raw_ring = raw_ring; a.ck = (bf16 *)ck; a.ck_cap = ck_cap; a.ratio = ratio; a.eps = eps;
    a.ring_inline = M <= RAW_RING - ratio ? 1 : 0;
    dim3 grid(M, QL + 2 * KVL + IH + 1);
    launch_pdl(qsa_prep_kernel, grid, dim3(256), 0, s, a);
    if (!a.ring_inline)
        launch_pdl(qsa_raw_ring_kernel, dim3(M), dim3(ID), 0, s, proj, ld_proj, QL * 2 * HD + 2 * KVL * HD + IH * ID, raw_ring, a.rows);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

QW_API int qwk_qsa_scores(const float *iq, int IH, const void *ck, int ck_cap, int M, const int *slot, const int *pos,
                          int ratio, int topk_blocks, float *scores, int ld_scores, int max_groups, cudaStream_t s) {
    if (max_groups <= topk_blocks) return 0;
    if (M > MAX_ROWS && IH == 4) {
        // a batch of more than MAX_ROWS rows is one run of one slot (a prefill chunk): tensor-core form
        qsa_scores_mma_kernel<<<dim3((M + 15) / 16, SC_SPLIT), 128, 0, s>>>(iq, (const bf16 *)ck, ck_cap,
                                                                            Rows{M, slot, pos, nullptr, nullptr}, ratio, topk_blocks,
                                                                            scores, ld_scores);
        return cudaGetLastError() == cudaSuccess ? 0 : -2;
    }
    dim3 grid((max_groups + 63) / 64, M);
    launch_pdl(qsa_scores_kernel, grid, dim3(256), 0, s, iq, IH, (const bf16 *)ck, ck_cap, Rows{M, slot, pos, nullptr, nullptr}, ratio,
               topk_blocks, scores, ld_scores);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

QW_API int qwk_qsa_select(const float *scores, int ld_scores, int M, const int *pos, int ratio, int topk, int *sel,
                          int *sel_n, cudaStream_t s) {
    launch_pdl(qsa_select_kernel, dim3(M), dim3(1024), 0, s, scores, ld_scores, Rows{M, nullptr, pos, nullptr, nullptr}, ratio, topk, sel,
               sel_n);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

QW_API int qwk_qsa_attend(const float *q, int QL, int KVL, int M, const int *slot, const int *pos, void *k_dev,
                          void *v_dev, void *k_host, void *v_host, int n_dev_pages, const int *page_table,
                          int max_pages, const int *sel, const int *sel_n, int topk, int ratio, int nsplit, float *pm,
                          float *pl, float *pacc, const float *proj, int ld_proj, void *o, cudaStream_t s) {
    QsaAttendArgs a;
    a.q = q; a.QL = QL; a.KVL = KVL; a.rows = Rows{M, slot, pos, nullptr, nullptr};
    a.kv = make_pool(k_dev, v_dev, k_host, v_host, n_dev_pages, page_table, max_pages, KVL * HD);
    a.sc = k_host ? g_spill : SpillCache{};
    a.sel = sel; a.sel_n = sel_n; a.topk = topk; a.ratio = ratio; a.nsplit = nsplit;
    a.pm = pm; a.pl = pl; a.pacc = pacc;
    const int per_kv = QL / KVL;
    int ht = per_kv % 4 == 0 ? 4 : (per_kv % 3 == 0 ? 3 : (per_kv % 2 == 0 ? 2 : 1));
    dim3 grid(nsplit, M, QL / ht);
    if (ht == 4) launch_pdl(qsa_attend_kernel<4>, grid, dim3(256), 0, s, a);
    else if (ht == 3) launch_pdl(qsa_attend_kernel<3>, grid, dim3(256), 0, s, a);
    else if (ht == 2) launch_pdl(qsa_attend_kernel<2>, grid, dim3(256), 0, s, a);
    else launch_pdl(qsa_attend_kernel<1>, grid, dim3(256), 0, s, a);
    dim3 g2(M, QL);
    launch_pdl(qsa_combine_kernel, g2, dim3(256), 0, s, (const float *)pm, (const float *)pl, (const float *)pacc, nsplit, proj, ld_proj, QL, (bf16 *)o);
    // plain launch: it starts when both kernels above have finished, so nothing reads the cache while entries change
    if (a.sc.tags) spill_cache_fill_kernel<<<64, 256, 0, s>>>(a.sc, (const bf16 *)k_host, (const bf16 *)v_host, KVL * HD);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// The same attention for the rows of a token-major prefill chunk, on the tensor cores: one launch for all M rows, no
// partial buffers.  Needs QL / KVL <= 16 query heads per KV head.
QW_API int qwk_qsa_attend_mma(const float *q, int QL, int KVL, int M, const int *slot, const int *pos, void *k_dev,
                              void *v_dev, void *k_host, void *v_host, int n_dev_pages, const int *page_table,
                              int max_pages, const int *sel, const int *sel_n, int topk, int ratio, const float *proj,
                              int ld_proj, void *o, cudaStream_t s) {
    if (KVL < 1 || QL % KVL != 0 || QL / KVL > 16 || M < 1 || M > 65535) return -1;
    static bool attr_done = false;
    if (!attr_done) {
        if (cudaFuncSetAttribute(qsa_attend_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ATT_SMEM) != cudaSuccess)
            return -3;
        attr_done = true;
    }
    QsaAttendArgs a;
    a.q = q; a.QL = QL; a.KVL = KVL; a.rows = Rows{M, slot, pos, nullptr, nullptr};
    a.kv = make_pool(k_dev, v_dev, k_host, v_host, n_dev_pages, page_table, max_pages, KVL * HD);
    a.sc = k_host ? g_spill : SpillCache{};
    a.sel = sel; a.sel_n = sel_n; a.topk = topk; a.ratio = ratio; a.nsplit = 0;
    a.pm = nullptr; a.pl = nullptr; a.pacc = nullptr;
    qsa_attend_mma_kernel<<<dim3(KVL, M), 128, ATT_SMEM, s>>>(a, proj, ld_proj, (bf16 *)o, g_err_ptr);
    if (a.sc.tags) spill_cache_fill_kernel<<<64, 256, 0, s>>>(a.sc, (const bf16 *)k_host, (const bf16 *)v_host, KVL * HD);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// Installs (entries > 0, a power of two) or removes (entries == 0) the cache of host KV rows.  tags: entries x u64,
// zeroed; rows: entries x 2 x row bf16; miss: miss_cap x u64; ctl: 2 x u32, zeroed; stats: 2 x u64 or null.
QW_API int qwk_set_spill_cache(void *tags, void *rows, void *miss, void *ctl, void *stats, int entries, int miss_cap) {
    if (entries == 0) {
        g_spill = SpillCache{};
        return 0;
    }
    if (entries < 0 || (entries & (entries - 1)) || !tags || !rows || !miss || !ctl || miss_cap <= 0) return -1;
    g_spill.tags = (unsigned long long *)tags; g_spill.rows = (bf16 *)rows; g_spill.miss = (unsigned long long *)miss;
    g_spill.ctl = (unsigned *)ctl; g_spill.stats = (unsigned long long *)stats; g_spill.mask = (unsigned)entries - 1u;
    g_spill.miss_cap = miss_cap;
    return 0;
}
// 1 when launches that get host pages also launch the fill kernel (launch accounting).
QW_API int qwk_spill_cache_active(int unused) { return (void)unused, g_spill.tags ? 1 : 0; }
