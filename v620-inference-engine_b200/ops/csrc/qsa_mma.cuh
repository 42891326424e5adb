// Tensor-core QSA attention for token-major prefill (included by qsa.cu inside namespace qw).
//
// One block per (query row, local KV head): the query heads that share the KV head (<= 16; 12 in the full model at
// one rank) are the 16 rows of the MMA tile, so the gathered K and V rows of a token are fetched once for all of
// them.  The row's token list (every visible token below the budget, else the selected groups plus the open tail) is
// walked in tiles of 64 tokens: rows gathered into padded shared memory by one 512-byte bulk-async copy per row
// straight from the paged pool (device pages or the spill cache; rows that live in host pages are copied by their
// thread with plain loads), completing on an mbarrier per tile, S = Q K^T and O += P V on mma.sync m16n8k16 bf16 with
// fp32 accumulation, online softmax in fp32 with one running maximum per query head shared by the four warps.
// The copies of the next tile's K overlap P V of this tile and the copies of its V overlap the next S.  Every wait on
// a tile's mbarrier is bounded.
// Output: o = softmax(..) V * sigmoid(gate) in bf16, with no partial buffers and no merge kernel
// (role of the reference's qsa_attend_T + combine, src/kernels/qsa.hip:136-243).
#pragma once

constexpr int AT = 64;               // tokens per tile
constexpr int KV_LD = HD + 8;        // shared row stride (bf16): 528 bytes keeps the 8 rows of an ldmatrix in distinct banks
constexpr int P_LD = AT + 8;
constexpr int ATT_SMEM = (2 * AT * KV_LD + 16 * P_LD) * 2 + (4 * 16 * 2) * 4 + 16;

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3, uint32_t saddr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(saddr));
}

// Starts the copies of one tile of K rows (which = 0) or V rows (which = 1): thread r < 64 owns token r of the tile
// and arrives once on `bar` (64 arrivals complete a tile).  Device rows: one bulk-async copy of the head's 512 bytes.
// Rows in host pages: copied here with plain loads.  Tokens past the list's end: zero-filled.
__device__ __forceinline__ void att_issue(const QsaAttendArgs &a, bf16 *dst_tile, uint64_t *bar, int which, int tile,
                                          int count, int dense, const int *sel, int nb, int slot, int kvh, bool record) {
    const int r = threadIdx.x;
    if (r >= AT) return;
    bf16 *dst = dst_tile + r * KV_LD;
    const int t = tile * AT + r;
    if (t < count) {
        const int tok = list_token(t, dense, sel, a.ratio, a.topk, nb);
        bool host;
        const long long off = kv_off(a.kv, slot, tok, host);
        const bf16 *kp = a.kv.k_dev + off, *vp = a.kv.v_dev + off;
        bool from_host = false;
        if (host) {
            kv_rows_read(a.kv, a.sc, slot, tok, record && which == 0, kp, vp);
            from_host = kp == a.kv.k_host + off;           // not in the spill cache
        }
        const bf16 *src = (which ? vp : kp) + kvh * HD;
        if (!from_host) {
            mbar_expect_tx(bar, HD * 2);
            bulk_g2s(dst, src, HD * 2, bar);
            return;
        }
        const uint4 *s4 = reinterpret_cast<const uint4 *>(src);
        uint4 *d4 = reinterpret_cast<uint4 *>(dst);
#pragma unroll 8
        for (int i = 0; i < HD * 2 / 16; ++i) d4[i] = s4[i];
    } else {
        uint4 *d4 = reinterpret_cast<uint4 *>(dst);
#pragma unroll 8
        for (int i = 0; i < HD * 2 / 16; ++i) d4[i] = make_uint4(0u, 0u, 0u, 0u);
    }
    mbar_arrive(bar);
}

// grid (KVL, M), 128 threads.
__global__ void __launch_bounds__(128, 3) qsa_attend_mma_kernel(QsaAttendArgs a, const float *proj, int ld_proj, bf16 *o,
                                                                ErrorWord *g_err) {
    extern __shared__ __align__(16) unsigned char att_sm[];
    bf16 *Ks = reinterpret_cast<bf16 *>(att_sm);             // [64][KV_LD]   (first: the 16 query rows, staged once)
    bf16 *Vs = Ks + AT * KV_LD;                              // [64][KV_LD]
    bf16 *Ps = Vs + AT * KV_LD;                              // [16][P_LD]
    float *s_max = reinterpret_cast<float *>(Ps + 16 * P_LD);    // [4][16]
    float *s_l = s_max + 64;                                 // [4][16]
    uint64_t *kbar = reinterpret_cast<uint64_t *>(s_l + 64), *vbar = kbar + 1;     // one phase per tile
    const int kvh = blockIdx.x, m = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5, g = lane >> 2, t4 = lane & 3;
    const int per_kv = a.QL / a.KVL, h0 = kvh * per_kv;
    const int slot = a.rows.slot[m], pos = a.rows.pos[m];
    const int nb = (pos + 1) / a.ratio;
    const int dense = a.sel_n[m] < 0;
    const int count = dense ? pos + 1 : a.topk * a.ratio + (pos + 1 - nb * a.ratio);
    const int ntiles = (count + AT - 1) / AT;
    const int *sel = a.sel + (long long)m * a.topk;
    const uint32_t ks_base = (uint32_t)__cvta_generic_to_shared(Ks), vs_base = (uint32_t)__cvta_generic_to_shared(Vs);
    if (tid == 0) {
        mbar_init(kbar, AT);
        mbar_init(vbar, AT);
        mbar_fence_init();
    }
    const uint32_t ps_base = (uint32_t)__cvta_generic_to_shared(Ps);
    // ---- the query rows -> bf16 in shared memory -> A fragments held in registers for the whole walk
    for (int i = tid; i < 16 * (HD / 2); i += 128) {
        const int r = i / (HD / 2), c = (i % (HD / 2)) * 2;
        float2 v = make_float2(0.f, 0.f);
        if (r < per_kv) v = *reinterpret_cast<const float2 *>(a.q + ((long long)m * a.QL + h0 + r) * HD + c);
        *reinterpret_cast<bf162 *>(Ks + r * KV_LD + c) = __floats2bfloat162_rn(v.x, v.y);
    }
    __syncthreads();
    uint32_t qf[16][4];
#pragma unroll
    for (int ks = 0; ks < 16; ++ks)
        ldmatrix_x4(qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], a_tile_addr(ks_base, KV_LD * 2, ks * 16, lane));
    __syncthreads();
    att_issue(a, Ks, kbar, 0, 0, count, dense, sel, nb, slot, kvh, kvh == 0);
    att_issue(a, Vs, vbar, 1, 0, count, dense, sel, nb, slot, kvh, false);
    float acc[8][4];
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[n][i] = 0.f;
    float mx0 = -INFINITY, mx1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    for (int tile = 0; tile < ntiles; ++tile) {
        mbar_wait(kbar, (unsigned)tile & 1u, g_err);        // this tile's K rows have landed (bounded; a time-out is recorded)
        // ---- S = Q K^T for this warp's 16 tokens
        float s[2][4];
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) s[n][i] = 0.f;
        {
            const int mid = lane >> 3;
            const uint32_t brow = ks_base + (uint32_t)((w * 16 + (mid >> 1) * 8 + (lane & 7)) * KV_LD * 2 + (mid & 1) * 16);
#pragma unroll
            for (int ks = 0; ks < 16; ++ks) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4(b0, b1, b2, b3, brow + ks * 32);
                mma_bf16(s[0], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b0, b1);
                mma_bf16(s[1], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b2, b3);
            }
        }
        float tm0 = -INFINITY, tm1 = -INFINITY;
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int t = tile * AT + w * 16 + n * 8 + 2 * t4 + (i & 1);
                const float v = t < count ? s[n][i] * 0.0625f : -INFINITY;       // 1/sqrt(256)
                s[n][i] = v;
                if (i < 2) tm0 = fmaxf(tm0, v); else tm1 = fmaxf(tm1, v);
            }
        tm0 = fmaxf(tm0, __shfl_xor_sync(0xffffffffu, tm0, 1));
        tm0 = fmaxf(tm0, __shfl_xor_sync(0xffffffffu, tm0, 2));
        tm1 = fmaxf(tm1, __shfl_xor_sync(0xffffffffu, tm1, 1));
        tm1 = fmaxf(tm1, __shfl_xor_sync(0xffffffffu, tm1, 2));
        if (t4 == 0) { s_max[w * 16 + g] = tm0; s_max[w * 16 + g + 8] = tm1; }
        __syncthreads();         // every warp is past its reads of the K tile, too
        if (tile + 1 < ntiles) att_issue(a, Ks, kbar, 0, tile + 1, count, dense, sel, nb, slot, kvh, kvh == 0);
        const float n0 = fmaxf(fmaxf(fmaxf(s_max[g], s_max[16 + g]), fmaxf(s_max[32 + g], s_max[48 + g])), mx0);
        const float n1 = fmaxf(fmaxf(fmaxf(s_max[g + 8], s_max[24 + g]), fmaxf(s_max[40 + g], s_max[56 + g])), mx1);
        // the first tile always holds a visible token, so n0 / n1 are finite
        const float c0 = __expf(mx0 - n0), c1 = __expf(mx1 - n1);
        mx0 = n0; mx1 = n1;
        l0 *= c0; l1 *= c1;
#pragma unroll
        for (int n = 0; n < 2; ++n) {
            const float p0 = __expf(s[n][0] - n0), p1 = __expf(s[n][1] - n0);
            const float p2 = __expf(s[n][2] - n1), p3 = __expf(s[n][3] - n1);
            l0 += p0 + p1;
            l1 += p2 + p3;
            const int c = w * 16 + n * 8 + 2 * t4;
            *reinterpret_cast<bf162 *>(Ps + g * P_LD + c) = __floats2bfloat162_rn(p0, p1);
            *reinterpret_cast<bf162 *>(Ps + (g + 8) * P_LD + c) = __floats2bfloat162_rn(p2, p3);
        }
#pragma unroll
        for (int n = 0; n < 8; ++n) {
            acc[n][0] *= c0; acc[n][1] *= c0;
            acc[n][2] *= c1; acc[n][3] *= c1;
        }
        __syncthreads();         // P visible
        mbar_wait(vbar, (unsigned)tile & 1u, g_err);        // this tile's V rows have landed
        // ---- O += P V for this warp's 64 output dims
        {
            const int mid = lane >> 3;
            const uint32_t vrow = vs_base + (uint32_t)((((mid & 1) * 8 + (lane & 7)) * KV_LD + w * 64 + (mid >> 1) * 8) * 2);
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                uint32_t p0, p1, p2, p3;
                ldmatrix_x4(p0, p1, p2, p3, a_tile_addr(ps_base, P_LD * 2, ks * 16, lane));
#pragma unroll
                for (int n2 = 0; n2 < 4; ++n2) {
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4_trans(b0, b1, b2, b3, vrow + (uint32_t)(ks * 16 * KV_LD * 2 + n2 * 32));
                    mma_bf16(acc[2 * n2], p0, p1, p2, p3, b0, b1);
                    mma_bf16(acc[2 * n2 + 1], p0, p1, p2, p3, b2, b3);
                }
            }
        }
        __syncthreads();         // V, P and the maxima are free again
        if (tile + 1 < ntiles) att_issue(a, Vs, vbar, 1, tile + 1, count, dense, sel, nb, slot, kvh, false);
    }
    // ---- normalise, gate, store
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    if (t4 == 0) { s_l[w * 16 + g] = l0; s_l[w * 16 + g + 8] = l1; }
    __syncthreads();
    const float L0 = s_l[g] + s_l[16 + g] + s_l[32 + g] + s_l[48 + g];
    const float L1 = s_l[g + 8] + s_l[24 + g] + s_l[40 + g] + s_l[56 + g];
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        const int r = g + hh * 8;
        if (r >= per_kv) continue;
        const float inv = 1.f / (hh ? L1 : L0);
        const float *gate = proj + (long long)m * ld_proj + (long long)(h0 + r) * 2 * HD + HD;
        bf16 *orow = o + ((long long)m * a.QL + h0 + r) * HD;
#pragma unroll
        for (int n = 0; n < 8; ++n) {
            const int d = w * 64 + n * 8 + 2 * t4;
            const float2 gt = *reinterpret_cast<const float2 *>(gate + d);
            const float y0 = acc[n][2 * hh] * inv * sigmoidf_(gt.x), y1 = acc[n][2 * hh + 1] * inv * sigmoidf_(gt.y);
            *reinterpret_cast<bf162 *>(orow + d) = __floats2bfloat162_rn(y0, y1);
        }
    }
}

// ------------------------------------------------------------------------------------------------------------------
// Indexer scores of a prefill chunk on the tensor cores: score[m][c] = sum_h relu(iq[m][h] . ck[c]) / sqrt(128) for the
// groups c visible to row m, for rows whose visible groups exceed the budget (the others attend densely).
// A block takes 16 consecutive rows of the chunk (one slot, ascending positions): the MMA rows of a warp are its 4
// query rows x 4 indexer heads, the fp32 queries split into a bf16 high and low part (two MMAs per step) so that the
// ranking keeps fp32-like resolution against the bf16 keys; key tiles of 64 groups go through shared memory and are
// shared by the four warps.  The sum over the heads is two lane shuffles on the accumulator fragment.
// grid (ceil(M / 16), SC_SPLIT), 128 threads; block y takes key tiles y, y + SC_SPLIT, ...   IH == 4.
// (Role of the reference's score GEMM + score_reduce, src/kernels/qsa.hip and docs/MODEL.md:150-160.)
// ------------------------------------------------------------------------------------------------------------------
constexpr int SC_SPLIT = 4;
constexpr int SC_LD = ID + 8;        // shared row stride of a key tile (bf16)

__global__ void __launch_bounds__(128) qsa_scores_mma_kernel(const float *iq, const bf16 *ck, int ck_cap, Rows rows, int ratio,
                                                             int topk_blocks, float *scores, int ld_scores) {
    __shared__ __align__(16) bf16 tile[64 * SC_LD];
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5, g = lane >> 2, t4 = lane & 3;
    const int m0 = blockIdx.x * 16;
    const int m_last = min(m0 + 15, rows.M - 1);
    const int nb_max = (rows.pos[m_last] + 1) / ratio;
    if (nb_max <= topk_blocks) return;                       // every row of the block attends densely (uniform)
    const int slot = rows.slot[m0];
    const bf16 *keys = ck + (long long)slot * ck_cap * ID;
    // ---- A fragments: MMA row i = 4 * (query row within the warp) + head; rows g and g + 8 of this lane
    uint32_t ahi[8][4], alo[8][4];
    int nb_row[2];
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        const int i = g + hh * 8, m = m0 + w * 4 + (i >> 2), h = i & 3;
        const bool ok = m < rows.M;
        nb_row[hh] = ok ? (rows.pos[m] + 1) / ratio : 0;
        const float *q = iq + ((long long)(ok ? m : m0) * 4 + h) * ID;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                float2 v = *reinterpret_cast<const float2 *>(q + ks * 16 + half * 8 + 2 * t4);
                if (!ok) v = make_float2(0.f, 0.f);
                const bf162 hi = __floats2bfloat162_rn(v.x, v.y);
                const float2 hf = __bfloat1622float2(hi);
                const bf162 lo = __floats2bfloat162_rn(v.x - hf.x, v.y - hf.y);
                ahi[ks][hh + 2 * half] = *reinterpret_cast<const uint32_t *>(&hi);
                alo[ks][hh + 2 * half] = *reinterpret_cast<const uint32_t *>(&lo);
            }
    }
    const uint32_t tile_base = (uint32_t)__cvta_generic_to_shared(tile);
    const int ntiles = (nb_max + 63) / 64;
    for (int kt = blockIdx.y; kt < ntiles; kt += SC_SPLIT) {
        const int c0 = kt * 64;
        __syncthreads();                                     // the previous tile has been read
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int idx = tid + i * 128;                   // 16-byte piece: 64 groups x 16
            const int r = idx >> 4, p = idx & 15;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (c0 + r < nb_max) v = __ldg(reinterpret_cast<const uint4 *>(keys + (long long)(c0 + r) * ID) + p);
            *reinterpret_cast<uint4 *>(tile + r * SC_LD + p * 8) = v;
        }
        __syncthreads();
        float acc[8][4];
#pragma unroll
        for (int n = 0; n < 8; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[n][i] = 0.f;
        const int mid = lane >> 3;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
#pragma unroll
            for (int n2 = 0; n2 < 4; ++n2) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4(b0, b1, b2, b3, tile_base + (uint32_t)(((n2 * 16 + (mid >> 1) * 8 + (lane & 7)) * SC_LD + ks * 16 + (mid & 1) * 8) * 2));
                mma_bf16(acc[2 * n2], ahi[ks][0], ahi[ks][1], ahi[ks][2], ahi[ks][3], b0, b1);
                mma_bf16(acc[2 * n2], alo[ks][0], alo[ks][1], alo[ks][2], alo[ks][3], b0, b1);
                mma_bf16(acc[2 * n2 + 1], ahi[ks][0], ahi[ks][1], ahi[ks][2], ahi[ks][3], b2, b3);
                mma_bf16(acc[2 * n2 + 1], alo[ks][0], alo[ks][1], alo[ks][2], alo[ks][3], b2, b3);
            }
        // relu, sum over the 4 heads (lanes that differ in the low two bits of g), store
#pragma unroll
        for (int n = 0; n < 8; ++n) {
            float s[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float v = fmaxf(acc[n][i], 0.f);
                v += __shfl_xor_sync(0xffffffffu, v, 4);
                v += __shfl_xor_sync(0xffffffffu, v, 8);
                s[i] = v * 0.08838834764831845f;
            }
            if ((g & 3) == 0) {
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    const int m = m0 + w * 4 + ((g + hh * 8) >> 2);
                    const int nb = nb_row[hh];
                    if (m < rows.M && nb > topk_blocks) {
#pragma unroll
                        for (int j = 0; j < 2; ++j) {
                            const int c = c0 + n * 8 + 2 * t4 + j;
                            if (c < nb) scores[(long long)m * ld_scores + c] = s[hh * 2 + j];
                        }
                    }
                }
            }
        }
    }
}
