// Dense bf16 GEMM on the 5th-generation tensor cores: C[T][N] = A[T][K] . W[N][K]^T, fp32 accumulate in
// tensor memory, fp32 or bf16 output (prefill path: projections, mixers, router with fp32 output,
// lm_head; role of the reference's rocBLAS call sites, src/kernels/gemm.hip:10-18).
//
// Persistent CTAs (two per SM) walk the 128 x 128 output tiles round-robin.  Warp roles:
//   warp 0   : TMA producer - one thread issues cp.async.bulk.tensor loads (no multicast) of the
//              128 x 64 A tile and the 128 x 64 W tile of each k block into a 3-stage ring of
//              128B-swizzled shared-memory tiles, completing on the stage's "full" mbarrier;
//   warp 1   : allocates 256 TMEM columns (two accumulators), and one thread issues tcgen05.mma (M=128, N=128, K=16,
//              four per k block) reading both operands straight from shared memory through matrix descriptors;
//              tcgen05.commit releases a stage ("empty" mbarrier) and, after a tile's last k block, signals that
//              tile's accumulator ("done" mbarrier of the buffer);
//   warps 2-9: epilogue - tcgen05.ld the accumulator (each warp its 32 TMEM lanes = 32 output rows; warps 2-5 the
//              first 64 columns, warps 6-9 the other 64), convert and store, then hand the buffer back
//              ("acc_empty" mbarrier, one arrival per warp).
// The ring and the barriers' phases run on across tiles, so the loads and MMAs of the next tile start while the
// epilogue of this one drains the other accumulator; barrier set-up, the TMEM allocation and the tensor-map fetch are
// paid once per CTA, not once per tile (what weighed on the products with 5-10 k blocks per tile).  Two CTAs share
// an SM: 3 stages x 32 KB and 256 of the 512 TMEM columns each.
// Every mbarrier wait is bounded; a wait that runs out records an error, the roles leave their loops and the
// TMEM allocation is released before the kernel returns.
#include <cuda.h>

#include "stream.cuh"
#include "tp.cuh"

namespace qw {

constexpr int TC_BM = 128, TC_BN = 128, TC_BK = 64, TC_STAGES = 3;
constexpr int TC_A_BYTES = TC_BM * TC_BK * 2, TC_B_BYTES = TC_BN * TC_BK * 2;     // 16 KB each
constexpr int TC_STAGE_BYTES = TC_A_BYTES + TC_B_BYTES;
constexpr int TC_SMEM = TC_STAGES * TC_STAGE_BYTES + 1024 /*alignment*/ + 256 /*barriers*/;
constexpr int TC_TMEM_COLS = 2 * TC_BN;          // two accumulators
// The wide form of the dense kernel: 128 x 256 tiles (the widest MMA: per k block 48 KB of operands feed twice the
// math of a 128 x 128 tile's 32 KB), four stages, one CTA per SM holding all 512 TMEM columns for its two accumulators.
constexpr int TC_WIDE_BN = 256, TC_WIDE_STAGES = 4;
template <int BN>
constexpr int tc_stage_bytes() { return TC_A_BYTES + BN * TC_BK * 2; }
// Staged epilogue (the tensor-parallel forms): 4 KB per epilogue warp behind the barriers, where a 32 x 32 fp32 piece is
// turned from "a thread owns a row" into "eight lanes own 128 contiguous bytes of a row" before it leaves for a peer.
constexpr int TC_EPI_WARPS = 8, TC_STG_BYTES = 4096;
constexpr int TC_STG_STAGES = 5;                 // k-block ring of the staged 128-wide form (one CTA per SM)
template <int BN, int ST, bool STG = false>
constexpr int tc_smem_bytes() {
    return ST * tc_stage_bytes<BN>() + 1024 /*alignment*/ + 256 /*barriers*/ + (STG ? TC_EPI_WARPS * TC_STG_BYTES : 0);
}

__device__ __forceinline__ uint64_t make_sw128_desc(uint32_t saddr) {
    // K-major operand tile, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFF) >> 4);          // start address
    d |= (uint64_t)1 << 16;                           // leading byte offset (unused with swizzle)
    d |= (uint64_t)(1024 >> 4) << 32;                 // stride byte offset
    d |= (uint64_t)1 << 46;                           // descriptor version (sm_100)
    d |= (uint64_t)2 << 61;                           // SWIZZLE_128B
    return d;
}

__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, int c0, int c1, uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(c0), "r"(c1), "r"(smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_c, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_c), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

struct GemmTcArgs {
    float *C32;          // one of the two outputs
    bf16 *C16;
    int T, N, K, ldc;
    ErrorWord *err;
    // grouped mode (expert-sorted rows): tiles[entry] = {first A row, valid rows, first W row of the group, -}
    const int4 *tiles;
    int total, tiles_t, tiles_n;     // linear tile ids 0..total-1; plain: id = (split * tiles_n + n) * tiles_t + t; grouped: id = entry * tiles_n + n
    // split-K (plain mode, fp32 output): split s covers k blocks [s * kb_per, (s + 1) * kb_per) and writes its partial sums
    // to C + s * c_split (the consumer adds the splits in order); ksplit == 1: the whole K, c_split unused
    int ksplit, kb_per;
    long long c_split;
    // tensor-parallel prefill (tp.cuh): the producer thread waits for a gathered A operand before its first load; the
    // epilogue sends fp32 tiles to other ranks' receive buffers instead of (mode != 0) storing them to C
    TpWait wait;
    TpEpilogue epi;
};

struct TileAt {
    int t0, rows_valid, n0, w0;
    int kb0, kbn;                    // first k block and number of k blocks of this tile's share of K
    long long c_off;                 // element offset of its output within C
};
// Tile `id` of the launch; false for an unused entry of the tile table (every role skips it alike).
template <int BN = TC_BN>
__device__ __forceinline__ bool tile_at(const GemmTcArgs &a, int id, TileAt &t) {
    const int kblocks = (a.K + TC_BK - 1) / TC_BK;
    t.kb0 = 0;
    t.kbn = kblocks;
    t.c_off = 0;
    if (a.tiles) {
        const int4 tl = __ldg(a.tiles + id / a.tiles_n);
        t.n0 = (id % a.tiles_n) * BN;
        t.t0 = tl.x;
        t.rows_valid = tl.y;
        t.w0 = tl.z + t.n0;
        return tl.y > 0;
    }
    // plain: the row tiles of one column panel are neighbours, so the CTAs in flight share a W panel and the (smaller)
    // activation matrix stays in L2 while W streams through once
    if (a.ksplit > 1) {
        const int per = a.tiles_t * a.tiles_n, sp = id / per;
        id -= sp * per;
        t.kb0 = sp * a.kb_per;
        t.kbn = min(a.kb_per, kblocks - t.kb0);
        t.c_off = sp * a.c_split;
    }
    t.n0 = (id / a.tiles_t) * BN;
    t.t0 = (id % a.tiles_t) * TC_BM;
    t.rows_valid = TC_BM;
    t.w0 = t.n0;
    return true;
}

// One 32-column piece of an accumulator row -> C.
__device__ __forceinline__ void store_piece(const GemmTcArgs &a, long long c_off, int row, int col0, const uint32_t (&v)[32]) {
    const int nmax = a.N - col0;
    if (a.epi.mode) {
        // fp32 pieces to the receive buffers: every rank's (parts of an all-reduce) or the column owner's (reduce-scatter)
        const int owner = a.epi.mode == 2 ? col0 / a.epi.cols_per_rank : 0;
        const long long off = (long long)row * a.epi.ld + (col0 - owner * a.epi.cols_per_rank * (a.epi.mode == 2));
        const bool vec = nmax >= 32 && ((a.epi.ld | col0) & 3) == 0;
#pragma unroll
        for (int d = 0; d < TP_MAX_RANKS; ++d) {
            if (d >= a.epi.ranks || (a.epi.mode == 2 && d != owner)) continue;
            float *o = a.epi.dst[d] + off;
            if (vec) {
#pragma unroll
                for (int j = 0; j < 32; j += 4)
                    *reinterpret_cast<float4 *>(o + j) = make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]),
                                                                     __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
            } else {
                for (int j = 0; j < 32 && j < nmax; ++j) o[j] = __uint_as_float(v[j]);
            }
        }
        return;
    }
    if (a.C32) {
        float *o = a.C32 + c_off + (long long)row * a.ldc + col0;
        if (nmax >= 32 && ((a.ldc | col0) & 3) == 0) {
#pragma unroll
            for (int j = 0; j < 32; j += 4)
                *reinterpret_cast<float4 *>(o + j) = make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]),
                                                                 __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
        } else {
            for (int j = 0; j < 32 && j < nmax; ++j) o[j] = __uint_as_float(v[j]);
        }
    } else {
        bf16 *o = a.C16 + (long long)row * a.ldc + col0;
        if (nmax >= 32 && ((a.ldc | col0) & 7) == 0) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
                uint4 pk;
                pk.x = pack_bf16(__uint_as_float(v[j]), __uint_as_float(v[j + 1]));
                pk.y = pack_bf16(__uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
                pk.z = pack_bf16(__uint_as_float(v[j + 4]), __uint_as_float(v[j + 5]));
                pk.w = pack_bf16(__uint_as_float(v[j + 6]), __uint_as_float(v[j + 7]));
                *reinterpret_cast<uint4 *>(o + j) = pk;
            }
        } else {
            for (int j = 0; j < 32 && j < nmax; ++j) o[j] = __float2bfloat16(__uint_as_float(v[j]));
        }
    }
}

// The same piece on its way to other ranks, through the warp's staging buffer: lane r writes its row as eight 16-byte
// chunks (chunk k at position k ^ (r & 7): no bank conflicts either way), then lanes 8i..8i+7 read row 4j + i back and
// store its 128 bytes as one contiguous line - a peer store of whole 128-byte lines instead of 32 scattered 16-byte ones,
// which is what NVLink carries at full rate.  `row0` is the output row of lane 0, `rows_ok` how many of the 32 rows exist.
template <bool LOCAL = false>
__device__ __forceinline__ void send_piece(const GemmTcArgs &a, float *stg, int lane, int row0, int rows_ok, int col0,
                                           const uint32_t (&v)[32], long long c_off = 0) {
    float4 *s4 = reinterpret_cast<float4 *>(stg);
#pragma unroll
    for (int k = 0; k < 8; ++k)
        s4[lane * 8 + (k ^ (lane & 7))] = make_float4(__uint_as_float(v[4 * k]), __uint_as_float(v[4 * k + 1]),
                                                      __uint_as_float(v[4 * k + 2]), __uint_as_float(v[4 * k + 3]));
    __syncwarp();
    const int ch = lane & 7, rsub = lane >> 3;
    const int col = col0 + ch * 4;                                   // first of this lane's four columns
    if constexpr (LOCAL) {
        // the same transposition for this GPU's own fp32 output: whole lines instead of 16-byte pieces of 32 rows
        const bool vec = ((a.ldc | col0) & 3) == 0 && col + 4 <= a.N;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int r = 4 * i + rsub;
            const float4 val = s4[r * 8 + (ch ^ (r & 7))];
            if (r >= rows_ok || col >= a.N) continue;
            float *o = a.C32 + c_off + (long long)(row0 + r) * a.ldc + col;
            if (vec) {
                *reinterpret_cast<float4 *>(o) = val;
            } else {
                const float e[4] = {val.x, val.y, val.z, val.w};
                for (int j = 0; j < 4 && col + j < a.N; ++j) o[j] = e[j];
            }
        }
        __syncwarp();
        return;
    }
    // the lane's eight float4 (rows rsub, rsub + 4, ...) come out of shared memory once; the destination is chosen once
    // per piece (reduce-scatter: the owner of these columns) or per rank (all-reduce), not once per store
    float4 val[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int r = 4 * i + rsub;
        val[i] = s4[r * 8 + (ch ^ (r & 7))];
    }
    __syncwarp();
    if (col >= a.N) return;
    const bool rs = a.epi.mode == 2;
    const int owner = rs ? col0 / a.epi.cols_per_rank : 0;
    const int ccol = col - (rs ? owner * a.epi.cols_per_rank : 0);
    const bool vec = ((a.epi.ld | col0) & 3) == 0 && col + 4 <= a.N;
    const long long off0 = (long long)(row0 + rsub) * a.epi.ld + ccol, step = 4ll * a.epi.ld;
    const int d0 = rs ? owner : 0, d1 = rs ? owner + 1 : a.epi.ranks;
    for (int d = d0; d < d1; ++d) {
        float *o = tp_pick(a.epi.dst, d) + off0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (4 * i + rsub >= rows_ok) break;
            if (vec) {
                *reinterpret_cast<float4 *>(o + i * step) = val[i];
            } else {
                const float e[4] = {val[i].x, val[i].y, val[i].z, val[i].w};
                for (int j = 0; j < 4 && col + j < a.N; ++j) o[i * step + j] = e[j];
            }
        }
    }
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// The epilogue role of both kernels: warps `first_warp` .. `first_warp + n_warps - 1` (n_warps = 4: all 128 columns per warp;
// 8: half of them), for every tile of this CTA in order.
template <int BN = TC_BN, bool STG = false>
__device__ __forceinline__ void epilogue_role(const GemmTcArgs &a, uint32_t tmem, uint64_t *done, uint64_t *acc_empty,
                                              int warp, int lane, int first_warp, int n_warps, float *stg = nullptr) {
    const int q = warp & 3;
    const int cbeg = (n_warps == 8 && warp >= first_warp + 4) ? BN / 2 : 0;
    const int cend = n_warps == 8 ? cbeg + BN / 2 : BN;
    int j = 0;
    for (int id = blockIdx.x; id < a.total; id += gridDim.x) {
        TileAt t;
        if (!tile_at<BN>(a, id, t)) continue;
        const int b = j & 1;
        if (!mbar_wait(done + b, (unsigned)(j >> 1) & 1u, a.err)) return;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int row = t.t0 + q * 32 + lane;
        const bool row_ok = row < a.T && q * 32 + lane < t.rows_valid;
#pragma unroll 1
        for (int c0 = cbeg; c0 < cend; c0 += 32) {
            uint32_t v[32];
            tmem_ld32(tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(b * BN + c0), v);
            if constexpr (STG) {
                const int r0 = t.t0 + q * 32, rows_ok = min(32, min(a.T - r0, t.rows_valid - q * 32));
                if (a.epi.mode) {
                    send_piece(a, stg, lane, r0, rows_ok, t.n0 + c0, v);
                    continue;
                }
                if (a.C32) {
                    send_piece<true>(a, stg, lane, r0, rows_ok, t.n0 + c0, v, t.c_off);
                    continue;
                }
            }
            if (row_ok) store_piece(a, t.c_off, row, t.n0 + c0, v);
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(acc_empty + b);
        ++j;
    }
}

// The MMA role of both kernels (one thread).
template <int BN = TC_BN, int ST = TC_STAGES>
__device__ __forceinline__ void mma_role(const GemmTcArgs &a, unsigned char *smem, uint32_t tmem, uint64_t *full, uint64_t *empty,
                                         uint64_t *done, uint64_t *acc_empty, int kblocks) {
    // instruction descriptor: D fp32, A/B bf16, both K-major, N and M of the tile
    const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
    int j = 0;
    unsigned it = 0;
    for (int id = blockIdx.x; id < a.total; id += gridDim.x) {
        TileAt t;
        if (!tile_at<BN>(a, id, t)) continue;
        const int b = j & 1;
        if (j >= 2 && !mbar_wait(acc_empty + b, (unsigned)((j >> 1) - 1) & 1u, a.err)) return;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        for (int kb = 0; kb < t.kbn; ++kb, ++it) {
            const unsigned s = it % ST;
            if (!mbar_wait(full + s, (it / ST) & 1u, a.err)) return;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t sa = smem_u32(smem + s * tc_stage_bytes<BN>()), sb = sa + TC_A_BYTES;
#pragma unroll
            for (int k = 0; k < TC_BK / 16; ++k) {
                const uint64_t da = make_sw128_desc(sa + k * 32), db = make_sw128_desc(sb + k * 32);
                umma_bf16(tmem + (uint32_t)(b * BN), da, db, idesc, (kb | k) ? 1u : 0u);
            }
            umma_commit(empty + s);          // the stage is free once these MMAs have read it
        }
        umma_commit(done + b);               // this tile's accumulator is complete
        ++j;
    }
}

// Shared set-up of both kernels: barriers, TMEM allocation (warp 1), and the pointers into shared memory.
struct TcShared {
    unsigned char *smem;
    uint64_t *full, *empty, *done, *acc_empty;
    uint32_t tmem;
};
template <int BN = TC_BN, int ST = TC_STAGES>
__device__ __forceinline__ TcShared tc_setup(unsigned char *raw, int warp, unsigned full_count, unsigned acc_empty_count) {
    TcShared t;
    t.smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~(uintptr_t)1023);
    t.full = reinterpret_cast<uint64_t *>(t.smem + ST * tc_stage_bytes<BN>());
    t.empty = t.full + ST;
    t.done = t.empty + ST;
    t.acc_empty = t.done + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(t.acc_empty + 2);
    if (threadIdx.x == 0) {
        for (int s = 0; s < ST; ++s) {
            mbar_init(t.full + s, full_count);
            mbar_init(t.empty + s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(t.done + b, 1);
            mbar_init(t.acc_empty + b, acc_empty_count);
        }
        mbar_fence_init();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(2 * BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    t.tmem = *tmem_slot;
    return t;
}
template <int BN = TC_BN>
__device__ __forceinline__ void tc_teardown(const TcShared &t, int warp) {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(t.tmem), "r"(2 * BN) : "memory");
    }
}

// grid: min(tiles, CTAs per SM x SMs) CTAs of 320 threads (two per SM with 128-wide tiles, one with 256-wide tiles).
template <int BN, int ST, bool STG = false>
__global__ void __launch_bounds__(320, (BN == TC_BN && !STG) ? 2 : 1) gemm_tc_kernel(const __grid_constant__ CUtensorMap mapA,
                                                         const __grid_constant__ CUtensorMap mapW, GemmTcArgs a) {
    extern __shared__ unsigned char raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const TcShared sh = tc_setup<BN, ST>(raw, warp, 1, 8);
    const int kblocks = (a.K + TC_BK - 1) / TC_BK;
    if (warp == 0) {
        if (lane == 0) {
            unsigned it = 0;
            bool ok = tp_wait_thread(a.wait);
            for (int id = blockIdx.x; id < a.total && ok; id += gridDim.x) {
                TileAt t;
                if (!tile_at<BN>(a, id, t)) continue;
                for (int kb = 0; kb < t.kbn; ++kb, ++it) {
                    const unsigned s = it % ST;
                    if (it >= ST && !mbar_wait(sh.empty + s, (it / ST - 1) & 1u, a.err)) { ok = false; break; }
                    mbar_expect_tx(sh.full + s, tc_stage_bytes<BN>());
                    unsigned char *st = sh.smem + s * tc_stage_bytes<BN>();
                    tma_load_2d(st, &mapA, (t.kb0 + kb) * TC_BK, t.t0, sh.full + s);
                    tma_load_2d(st + TC_A_BYTES, &mapW, (t.kb0 + kb) * TC_BK, t.w0, sh.full + s);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) mma_role<BN, ST>(a, sh.smem, sh.tmem, sh.full, sh.empty, sh.done, sh.acc_empty, kblocks);
    } else {
        float *stg = nullptr;
        if constexpr (STG)
            stg = reinterpret_cast<float *>(sh.smem + ST * tc_stage_bytes<BN>() + 256 + (warp - 2) * TC_STG_BYTES);
        epilogue_role<BN, STG>(a, sh.tmem, sh.done, sh.acc_empty, warp, lane, 2, TC_EPI_WARPS, stg);
    }
    tc_teardown<BN>(sh, warp);
    tp_signal(a.epi.sig);
}

// ------------------------------------------------------------------------------------------------------------------
// The pair form of the dense kernel: two CTAs of a cluster (two neighbouring SMs) compute one 256 x 256 output tile with
// tcgen05.mma.cta_group::2.  Each CTA loads its own 128 rows of A and ONE HALF of the tile's W rows (128 of 256) per k
// block - 32 KB for 128 x 256 x 64 multiply-adds per SM, where the single-CTA forms need 48 KB (128 x 256 tile) or 64 KB
// (two 128 x 128 tiles) for the same math: those stop at what an SM can pull out of L2 (~64 bytes per cycle), this one
// does not.  The tensor cores of both SMs read both CTAs' shared memory; each SM accumulates its 128 rows x 256 columns
// in its own tensor memory (two accumulators = all 512 columns).
//   producer (warp 0, one thread, both CTAs): waits for its own "empty" barrier of the stage, loads its A tile and its W
//       half with cp.async.bulk.tensor.cta_group::2 (no multicast), both completing on the LEADER's "full" barrier, on
//       which the leader's producer has announced the 64 KB of the pair;
//   MMA (warp 1, one thread, leader CTA only): four cta_group::2 MMAs per k block; tcgen05.commit (to both CTAs of the
//       pair) frees the stage in both CTAs and, after a tile's last k block, publishes the accumulator to both CTAs'
//       epilogue warps;
//   epilogue (warps 2-9, both CTAs): as in the single-CTA kernel, on the CTA's own 128 rows; hands the accumulator back
//       by arriving on the leader's "acc_empty" barrier (16 arrivals: 8 warps of 2 CTAs).
// Barriers are initialised before a cluster-wide barrier and nobody leaves before another one, so no signal is ever
// sent to a CTA that is not there; every wait is bounded as elsewhere.
// ------------------------------------------------------------------------------------------------------------------
constexpr int TC_PAIR_BN = 256, TC_PAIR_BM = 256, TC_PAIR_STAGES = 6, TC_PAIR_STG_STAGES = 5;
constexpr int TC_PAIR_STAGE_BYTES = TC_A_BYTES + TC_B_BYTES;          // per CTA: 128 x 64 of A and 128 x 64 of W
template <int ST, bool STG>
constexpr int tc_pair_smem_bytes() { return ST * TC_PAIR_STAGE_BYTES + 1024 + 256 + (STG ? TC_EPI_WARPS * TC_STG_BYTES : 0); }

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank) {          // the same offset in CTA `rank` of the cluster
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(void *dst, const CUtensorMap *map, int c0, int c1, uint32_t bar_cluster_addr) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(c0), "r"(c1), "r"(bar_cluster_addr)
                 : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_c, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_c), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrives (once the MMAs issued so far have completed) on the barrier at this offset in both CTAs of the pair.
__device__ __forceinline__ void umma_commit_pair(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"((unsigned short)3)
                 : "memory");
}

struct PairTile {
    int t0, n0, w0, rows_valid;          // this CTA's first A row / the tile's first column / this CTA's first W row
};
__device__ __forceinline__ PairTile pair_tile_at(const GemmTcArgs &a, int id, uint32_t rank) {
    PairTile t;
    // the row tiles of one column panel are neighbours (W streams once, A stays in L2)
    t.n0 = (id / a.tiles_t) * TC_PAIR_BN;
    t.t0 = (id % a.tiles_t) * TC_PAIR_BM + (int)rank * TC_BM;
    t.w0 = t.n0 + (int)rank * (TC_PAIR_BN / 2);
    t.rows_valid = TC_BM;
    return t;
}

// grid: 2 x min(pair tiles, SMs / 2) CTAs of 320 threads in clusters of two.  a.tiles_t / a.total count 256 x 256 tiles.
template <int ST, bool STG>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(320, 1) gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap mapA,
                                                                                        const __grid_constant__ CUtensorMap mapW,
                                                                                        GemmTcArgs a) {
    extern __shared__ unsigned char raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~(uintptr_t)1023);
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + ST * TC_PAIR_STAGE_BYTES);
    uint64_t *empty = full + ST, *done = empty + ST, *acc_empty = done + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_empty + 2);
    if (threadIdx.x == 0) {
        for (int s = 0; s < ST; ++s) {
            mbar_init(full + s, 1);          // the leader's: one arrival (its producer's expect_tx) + the pair's bytes
            mbar_init(empty + s, 1);         // one commit arrival
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(done + b, 1);
            mbar_init(acc_empty + b, 2 * TC_EPI_WARPS);          // the leader's: the epilogue warps of both CTAs
        }
        mbar_fence_init();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all();                      // both CTAs' barriers exist before anything is sent to them
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;
    const int kblocks = (a.K + TC_BK - 1) / TC_BK;
    if (warp == 0) {
        if (lane == 0) {
            unsigned it = 0;
            bool ok = tp_wait_thread(a.wait);
            for (int id = cluster_id; id < a.total && ok; id += n_clusters) {
                const PairTile t = pair_tile_at(a, id, rank);
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const unsigned s = it % ST;
                    if (it >= ST && !mbar_wait(empty + s, (it / ST - 1) & 1u, a.err)) { ok = false; break; }
                    if (rank == 0) mbar_expect_tx(full + s, 2 * TC_PAIR_STAGE_BYTES);
                    const uint32_t bar = map_to_cta(smem_u32(full + s), 0);
                    unsigned char *st = smem + s * TC_PAIR_STAGE_BYTES;
                    tma_load_2d_pair(st, &mapA, kb * TC_BK, t.t0, bar);
                    tma_load_2d_pair(st + TC_A_BYTES, &mapW, kb * TC_BK, t.w0, bar);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            // instruction descriptor: D fp32, A/B bf16, both K-major, N = 256, M = 256 (the pair's rows)
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TC_PAIR_BN >> 3) << 17) | ((uint32_t)(TC_PAIR_BM >> 4) << 24);
            int j = 0;
            unsigned it = 0;
            bool ok = true;
            for (int id = cluster_id; id < a.total && ok; id += n_clusters) {
                const int b = j & 1;
                if (j >= 2 && !mbar_wait(acc_empty + b, (unsigned)((j >> 1) - 1) & 1u, a.err)) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const unsigned s = it % ST;
                    if (!mbar_wait(full + s, (it / ST) & 1u, a.err)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t sa = smem_u32(smem + s * TC_PAIR_STAGE_BYTES), sb = sa + TC_A_BYTES;
#pragma unroll
                    for (int k = 0; k < TC_BK / 16; ++k)
                        umma_bf16_pair(tmem + (uint32_t)(b * TC_PAIR_BN), make_sw128_desc(sa + k * 32), make_sw128_desc(sb + k * 32), idesc,
                                       (kb | k) ? 1u : 0u);
                    umma_commit_pair(empty + s);
                }
                if (ok) umma_commit_pair(done + b);
                ++j;
            }
        }
    } else {
        float *stg = nullptr;
        if constexpr (STG) stg = reinterpret_cast<float *>(smem + ST * TC_PAIR_STAGE_BYTES + 256 + (warp - 2) * TC_STG_BYTES);
        const int q = warp & 3;
        const int cbeg = warp >= 6 ? TC_PAIR_BN / 2 : 0, cend = cbeg + TC_PAIR_BN / 2;
        const uint32_t acc_bar = map_to_cta(smem_u32(acc_empty), 0);
        int j = 0;
        for (int id = cluster_id; id < a.total; id += n_clusters) {
            const PairTile t = pair_tile_at(a, id, rank);
            const int b = j & 1;
            if (!mbar_wait(done + b, (unsigned)(j >> 1) & 1u, a.err)) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int row = t.t0 + q * 32 + lane;
            const bool row_ok = row < a.T;
#pragma unroll 1
            for (int c0 = cbeg; c0 < cend; c0 += 32) {
                uint32_t v[32];
                tmem_ld32(tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(b * TC_PAIR_BN + c0), v);
                if (t.n0 + c0 >= a.N) continue;
                if constexpr (STG) {
                    const int r0 = t.t0 + q * 32;
                    if (a.epi.mode) {
                        send_piece(a, stg, lane, r0, min(32, a.T - r0), t.n0 + c0, v);
                        continue;
                    }
                    if (a.C32) {
                        send_piece<true>(a, stg, lane, r0, min(32, a.T - r0), t.n0 + c0, v);
                        continue;
                    }
                }
                if (row_ok) store_piece(a, 0, row, t.n0 + c0, v);
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(acc_bar + (uint32_t)(b * 8));
            ++j;
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all();                      // nothing is in flight towards either CTA any more
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
    }
    tp_signal(a.epi.sig);
}

// ------------------------------------------------------------------------------------------------------------------
// Grouped GEMM with the weights in q4 (group 128, bf16 scales): the expert products of token-major prefill without a
// bf16 copy of the layer's experts.  Same tile, pipeline and epilogue as gemm_tc_kernel; the W operand of a stage is
// not loaded by TMA but produced by eight extra warps: two threads own row r of the 128 x 64 W tile, each fetches 4 q4
// words (16 bytes) and the block's scale four k blocks ahead, converts them to four 16-byte bf16 chunks of the row with
// packed bf16 arithmetic (the same values as the stand-alone dequantisation) and stores them where the 128-byte
// swizzle puts them (chunk c of row r at chunk c ^ (r & 7)); a proxy fence makes the stores visible to the tensor
// core's reads, and the thread arrives on the stage's "full" barrier (1 TMA arrival + 256 producer arrivals).  What
// bounds the kernel is how fast the producer warps turn words into tiles (~150 instructions per thread and k block),
// hence eight of them and two-wide arithmetic.
// (Role of the reference's moe_gate_up_T / moe_down_T, src/kernels/moe_experts.hip:17-27.)
// ------------------------------------------------------------------------------------------------------------------
constexpr int Q4_AHEAD = 4;

// grid: min(tiles, 2 x SMs) CTAs of 448 threads: warp 0 TMA (A), warp 1 MMA, warps 2-5 epilogue, warps 6-13 W producers.
__global__ void __launch_bounds__(448, 2) gemm_tc_q4_kernel(const __grid_constant__ CUtensorMap mapA, GemmTcArgs a,
                                                            const uint32_t *Wq, const bf16 *scale, long long w_rows) {
    extern __shared__ unsigned char raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const TcShared sh = tc_setup(raw, warp, 1 + 256, 4);
    const int kblocks = (a.K + TC_BK - 1) / TC_BK;
    if (warp == 0) {
        if (lane == 0) {
            unsigned it = 0;
            bool ok = true;
            for (int id = blockIdx.x; id < a.total && ok; id += gridDim.x) {
                TileAt t;
                if (!tile_at(a, id, t)) continue;
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const unsigned s = it % TC_STAGES;
                    if (it >= TC_STAGES && !mbar_wait(sh.empty + s, (it / TC_STAGES - 1) & 1u, a.err)) { ok = false; break; }
                    mbar_expect_tx(sh.full + s, TC_A_BYTES);
                    tma_load_2d(sh.smem + s * TC_STAGE_BYTES, &mapA, kb * TC_BK, t.t0, sh.full + s);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) mma_role(a, sh.smem, sh.tmem, sh.full, sh.empty, sh.done, sh.acc_empty, kblocks);
    } else if (warp >= 6) {
        // W producers: two threads per row of the tile, 32 k values (4 words, 4 chunks) each
        const int p = threadIdx.x - 192, r = p >> 1, hf = p & 1;
        const int wpr = a.K >> 3, spr = a.K >> 7;
        const bf162 off2 = __floats2bfloat162_rn(136.f, 136.f);
        unsigned it0 = 0;                        // k blocks of the tiles before this one
        bool ok = true;
        for (int id = blockIdx.x; id < a.total && ok; id += gridDim.x) {
            TileAt t;
            if (!tile_at(a, id, t)) continue;
            const long long wrow = (long long)t.w0 + r;
            const bool row_ok = t.n0 + r < a.N && wrow < w_rows;
            const uint4 *src = reinterpret_cast<const uint4 *>(Wq + (row_ok ? wrow : 0) * wpr) + hf;
            const unsigned short *sc_bits = reinterpret_cast<const unsigned short *>(scale + (row_ok ? wrow : 0) * spr);
            uint4 ring[Q4_AHEAD];
            unsigned short sring[Q4_AHEAD];      // the k block's scale travels with its words: no dependent load in the loop
#pragma unroll
            for (int i = 0; i < Q4_AHEAD; ++i) {
                ring[i] = make_uint4(0u, 0u, 0u, 0u);
                sring[i] = 0;
                if (row_ok && i < kblocks) {
                    ring[i] = __ldg(src + 2 * i);
                    sring[i] = __ldg(sc_bits + (i >> 1));
                }
            }
            for (int kb0 = 0; kb0 < kblocks && ok; kb0 += Q4_AHEAD) {
#pragma unroll
                for (int i = 0; i < Q4_AHEAD; ++i) {
                    const int kb = kb0 + i;
                    if (kb >= kblocks) break;
                    const unsigned it = it0 + (unsigned)kb, s = it % TC_STAGES;
                    const uint4 q = ring[i];
                    // scale as a bf16 pair; (nibble - 8) is exact in bf16 and its product with a bf16 scale, rounded once to
                    // bf16, equals the fp32 product rounded to bf16: the stand-alone conversion's values bit for bit
                    const uint32_t sb = (uint32_t)sring[i] | ((uint32_t)sring[i] << 16);
                    const bf162 sc2 = *reinterpret_cast<const bf162 *>(&sb);
                    if (row_ok && kb + Q4_AHEAD < kblocks) {
                        ring[i] = __ldg(src + 2 * (kb + Q4_AHEAD));
                        sring[i] = __ldg(sc_bits + ((kb + Q4_AHEAD) >> 1));
                    }
                    if (it >= TC_STAGES && !mbar_wait(sh.empty + s, (it / TC_STAGES - 1) & 1u, a.err)) { ok = false; break; }
                    unsigned char *dst = sh.smem + s * TC_STAGE_BYTES + TC_A_BYTES + r * 128;
                    const uint32_t words[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        uint32_t o[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            uint32_t bits = ((words[c] >> (4 * j)) & 0x000F000Fu) | 0x43004300u;
                            const bf162 v = __hmul2(__hsub2(*reinterpret_cast<bf162 *>(&bits), off2), sc2);
                            o[j] = *reinterpret_cast<const uint32_t *>(&v);
                        }
                        *reinterpret_cast<uint4 *>(dst + (((hf * 4 + c) ^ (r & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    mbar_arrive(sh.full + s);
                }
            }
            it0 += (unsigned)kblocks;
        }
    } else {
        epilogue_role(a, sh.tmem, sh.done, sh.acc_empty, warp, lane, 2, 4);
    }
    tc_teardown(sh, warp);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess) fn = (EncodeTiledFn)p;
    }
    return fn;
}

// 2-D bf16 row-major matrix [rows][cols] (row stride ld elements), box = 64 columns x box_rows rows, 128B swizzle.
// A chunk issues ~800 of these for a few dozen distinct (address, shape) pairs - weights and the engine's fixed buffers -
// so encoded maps are kept in a small direct-mapped table (per thread: the launchers run on the caller's thread) and an
// encode is paid only on a miss.  A map depends on nothing but the key: the same address with the same shape encodes to
// the same map whatever the memory holds.
struct MapKey {
    const void *base;
    long long rows, cols, ld;
    int box_rows, dev;
    bool operator==(const MapKey &o) const {
        return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows && dev == o.dev;
    }
};
struct MapSlot {
    MapKey key;
    CUtensorMap map;
    bool used;
};
constexpr int MAP_SLOTS = 256;

static bool make_map(CUtensorMap *m, const void *base, long long rows, long long cols, long long ld, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    static thread_local MapSlot table[MAP_SLOTS] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    const MapKey key{base, rows, cols, ld, box_rows, dev};
    unsigned long long h = (unsigned long long)(uintptr_t)base * 0x9E3779B97F4A7C15ull;
    h ^= (unsigned long long)rows * 0xC2B2AE3D27D4EB4Full + (unsigned long long)cols * 0x165667B19E3779F9ull + (unsigned long long)ld * 31 + box_rows;
    MapSlot &slot = table[(h >> 40) % MAP_SLOTS];
    if (slot.used && slot.key == key) {
        *m = slot.map;
        return true;
    }
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)TC_BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    if (fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    slot.key = key;
    slot.map = *m;
    slot.used = true;
    return true;
}

// `per_sm` persistent CTAs per SM of the current device, or one CTA per tile when there are fewer tiles.
static unsigned persistent_grid(int total, int per_sm = 2) {
    static int sms[64] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (!sms[dev]) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        sms[dev] = n;
    }
    const int cap = per_sm * sms[dev];
    return (unsigned)(total < cap ? total : cap);
}

}  // namespace qw

using namespace qw;

// One-time (per device) opt-in to the kernels' dynamic shared memory.
static bool configure_once(int which) {          // 0 dense 128-wide, 1 q4 grouped, 2 dense 256-wide, 3 / 4 the two with a staged epilogue, 5 / 6 the pair form
    static bool done[7][64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (!done[which][dev]) {
        cudaError_t e;
        if (which == 0) e = cudaFuncSetAttribute(gemm_tc_kernel<TC_BN, TC_STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM);
        else if (which == 1) e = cudaFuncSetAttribute(gemm_tc_q4_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM);
        else if (which == 2) e = cudaFuncSetAttribute(gemm_tc_kernel<TC_WIDE_BN, TC_WIDE_STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                      tc_smem_bytes<TC_WIDE_BN, TC_WIDE_STAGES>());
        else if (which == 3) e = cudaFuncSetAttribute(gemm_tc_kernel<TC_BN, TC_STG_STAGES, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                      tc_smem_bytes<TC_BN, TC_STG_STAGES, true>());
        else if (which == 4) e = cudaFuncSetAttribute(gemm_tc_kernel<TC_WIDE_BN, TC_WIDE_STAGES, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                      tc_smem_bytes<TC_WIDE_BN, TC_WIDE_STAGES, true>());
        else if (which == 5) e = cudaFuncSetAttribute(gemm_tc_pair_kernel<TC_PAIR_STAGES, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                      tc_pair_smem_bytes<TC_PAIR_STAGES, false>());
        else e = cudaFuncSetAttribute(gemm_tc_pair_kernel<TC_PAIR_STG_STAGES, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      tc_pair_smem_bytes<TC_PAIR_STG_STAGES, true>());
        if (e != cudaSuccess) return false;
        done[which][dev] = true;
    }
    return true;
}

static int g_wide_min_n = 1024;          // products at least this wide use the 128 x 256 tile form (0: never)
static int g_pair_min_n = 1024;          // products at least this wide (and 256 rows tall) use CTA pairs (0: never)
static int g_stage_local = 1;            // 1: fp32 output of the wide and pair forms also leaves through the staging buffers

static int gemm_plain(GemmTcArgs &a, const void *A, const void *W, void *C, int T, int N, int K, int lda, int ldw, int ldc,
                      int out_bf16, cudaStream_t s) {
    if ((K & 7) || (lda & 7) || (ldw & 7) || ((uintptr_t)A & 15) || ((uintptr_t)W & 15)) return -1;
    // wide tiles pay when there are enough of them to fill the SMs and the last column tile is not mostly padding
    const int tiles_t = (T + TC_BM - 1) / TC_BM;
    const bool wide = g_wide_min_n > 0 && N >= g_wide_min_n && (N % TC_WIDE_BN == 0 || N % TC_WIDE_BN > TC_BN) &&
                      tiles_t * ((N + TC_WIDE_BN - 1) / TC_WIDE_BN) >= NUM_SMS / 2;
    // pairs pay when the padding of the 256 x 256 tiles stays under ~6 % of the work and there are tiles for every pair of SMs
    const long long pad_t = (long long)((T + TC_PAIR_BM - 1) / TC_PAIR_BM) * TC_PAIR_BM, pad_n = (long long)((N + TC_PAIR_BN - 1) / TC_PAIR_BN) * TC_PAIR_BN;
    const bool pair = g_pair_min_n > 0 && N >= g_pair_min_n && T >= TC_PAIR_BM && pad_t * pad_n * 100 <= (long long)T * N * 106 &&
                      (pad_t / TC_PAIR_BM) * (pad_n / TC_PAIR_BN) >= NUM_SMS / 4;
    if (pair) {
        CUtensorMap mA, mW;
        if (!make_map(&mA, A, T, K, lda, TC_BM) || !make_map(&mW, W, N, K, ldw, TC_PAIR_BN / 2)) return -3;
        a.C32 = out_bf16 ? nullptr : (float *)C;
        a.C16 = out_bf16 ? (bf16 *)C : nullptr;
        a.T = T; a.N = N; a.K = K; a.ldc = ldc; a.err = g_err_ptr; a.tiles = nullptr;
        a.tiles_t = (T + TC_PAIR_BM - 1) / TC_PAIR_BM; a.tiles_n = (N + TC_PAIR_BN - 1) / TC_PAIR_BN; a.total = a.tiles_t * a.tiles_n;
        a.ksplit = 1; a.kb_per = 0; a.c_split = 0;
        const bool staged = a.epi.mode != 0 || (g_stage_local && !out_bf16);
        if (!configure_once(staged ? 6 : 5)) return -3;
        const unsigned sm_pairs = persistent_grid(1 << 30, 1) / 2;          // SMs / 2
        const unsigned clusters = (unsigned)a.total < sm_pairs ? (unsigned)a.total : sm_pairs;
        const unsigned ctas = 2 * clusters;
        if (a.epi.sig.ticket) a.epi.sig.nblocks = ctas;
        if (staged) gemm_tc_pair_kernel<TC_PAIR_STG_STAGES, true><<<ctas, 320, tc_pair_smem_bytes<TC_PAIR_STG_STAGES, true>(), s>>>(mA, mW, a);
        else gemm_tc_pair_kernel<TC_PAIR_STAGES, false><<<ctas, 320, tc_pair_smem_bytes<TC_PAIR_STAGES, false>(), s>>>(mA, mW, a);
        return cudaGetLastError() == cudaSuccess ? 0 : -2;
    }
    const int BN = wide ? TC_WIDE_BN : TC_BN;
    CUtensorMap mA, mW;
    if (!make_map(&mA, A, T, K, lda, TC_BM) || !make_map(&mW, W, N, K, ldw, BN)) return -3;
    a.C32 = out_bf16 ? nullptr : (float *)C;
    a.C16 = out_bf16 ? (bf16 *)C : nullptr;
    a.T = T; a.N = N; a.K = K; a.ldc = ldc; a.err = g_err_ptr; a.tiles = nullptr;
    a.tiles_t = tiles_t; a.tiles_n = (N + BN - 1) / BN; a.total = a.tiles_t * a.tiles_n;
    a.ksplit = 1; a.kb_per = 0; a.c_split = 0;
    // tiles that leave for other ranks go out as whole 128-byte lines (optionally this GPU's own fp32 tiles of the wide form too)
    const bool staged = a.epi.mode != 0 || (g_stage_local && wide && !out_bf16);
    if (!configure_once(staged ? (wide ? 4 : 3) : (wide ? 2 : 0))) return -3;
    const unsigned grid = persistent_grid(a.total, (wide || staged) ? 1 : 2);
    if (a.epi.sig.ticket) a.epi.sig.nblocks = grid;
    if (staged && wide)
        gemm_tc_kernel<TC_WIDE_BN, TC_WIDE_STAGES, true><<<grid, 320, tc_smem_bytes<TC_WIDE_BN, TC_WIDE_STAGES, true>(), s>>>(mA, mW, a);
    else if (staged)
        gemm_tc_kernel<TC_BN, TC_STG_STAGES, true><<<grid, 320, tc_smem_bytes<TC_BN, TC_STG_STAGES, true>(), s>>>(mA, mW, a);
    else if (wide) gemm_tc_kernel<TC_WIDE_BN, TC_WIDE_STAGES><<<grid, 320, tc_smem_bytes<TC_WIDE_BN, TC_WIDE_STAGES>(), s>>>(mA, mW, a);
    else gemm_tc_kernel<TC_BN, TC_STAGES><<<grid, 320, TC_SMEM, s>>>(mA, mW, a);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// Products at least `min_n` columns wide use the 128 x 256 tile form (0 switches it off; measurements and tests).
QW_API int qwk_gemm_tc_wide_min_n(int min_n) {
    const int old = g_wide_min_n;
    g_wide_min_n = min_n;
    return old;
}

// 1: the wide and pair forms write fp32 output through the staging buffers as well (whole lines per store instruction).
QW_API int qwk_gemm_tc_stage_local(int on) {
    const int old = g_stage_local;
    g_stage_local = on;
    return old;
}

// Products at least `min_n` columns wide (and 256 rows tall) use the CTA-pair form (0 switches it off).
QW_API int qwk_gemm_tc_pair_min_n(int min_n) {
    const int old = g_pair_min_n;
    g_pair_min_n = min_n;
    return old;
}

// C = A . W^T.  A bf16 [T][lda], W bf16 [N][ldw], C fp32 (out_bf16 = 0) or bf16 [T][ldc].
// Base addresses 16-byte aligned, lda/ldw multiples of 8 elements, K a multiple of 8.
QW_API int qwk_gemm_bf16_tc(const void *A, const void *W, void *C, int T, int N, int K, int lda, int ldw, int ldc,
                            int out_bf16, cudaStream_t s) {
    if (T <= 0 || N <= 0) return 0;
    GemmTcArgs a{};
    return gemm_plain(a, A, W, C, T, N, K, lda, ldw, ldc, out_bf16, s);
}

// Tensor-parallel forms of the same product (tp.cuh); `tp` is the rank's QwTp channel.
//   wait_kind >= 0 : A lies in the receive buffer of that all-gather kind; the kernel waits for the kind's latest
//                    collective before its first load of A.
//   epi_mode 0     : C as above.
//   epi_mode 1     : the fp32 result goes to every rank's receive buffer of kind `epi_kind` as this rank's part of an
//                    all-reduce (rows of ld_epi floats); C is not written.
//   epi_mode 2     : N = ranks * cols_per_rank; columns go to the rank that owns them, as this rank's part of a
//                    reduce-scatter (rows of cols_per_rank floats, cols_per_rank a multiple of 32); C is not written.
// In modes 1 and 2 the kernel publishes the collective when its last CTA has stored its tiles.
QW_API int qwk_gemm_bf16_tc_tp(void *tp_, const void *A, const void *W, void *C, int T, int N, int K, int lda, int ldw, int ldc,
                               int out_bf16, int wait_kind, int epi_mode, int epi_kind, int ld_epi, cudaStream_t s) {
    if (T <= 0 || N <= 0) return 0;
    QwTp *tp = (QwTp *)tp_;
    GemmTcArgs a{};
    if (!tp || tp->ranks < 1 || tp->ranks > TP_MAX_RANKS) return -1;
    if (wait_kind >= 0) {
        if (wait_kind >= TP_KINDS) return -1;
        a.wait = tp_make_wait(tp, wait_kind);
    }
    if (epi_mode) {
        if (epi_kind < 0 || epi_kind >= TP_KINDS || out_bf16) return -1;
        a.epi.mode = epi_mode;
        a.epi.ranks = tp->ranks;
        if (epi_mode == 2) {
            if (N % tp->ranks) return -1;
            a.epi.cols_per_rank = N / tp->ranks;
            if (a.epi.cols_per_rank & 31) return -1;
            a.epi.ld = a.epi.cols_per_rank;
        } else {
            a.epi.cols_per_rank = 0;
            a.epi.ld = ld_epi;
            if (ld_epi < N) return -1;
        }
        if ((long long)T * a.epi.ld * 4 > tp->part_bytes[epi_kind]) return -1;
        for (int d = 0; d < tp->ranks; ++d) a.epi.dst[d] = (float *)tp_part_on(tp, epi_kind, d);
        a.epi.sig = tp_make_signal(tp, epi_kind, 1);
    }
    return gemm_plain(a, A, W, C, T, N, K, lda, ldw, ldc, out_bf16, s);
}

// Grouped form for expert-sorted rows: A bf16 [rows][lda] holds the rows of group after group, W bf16
// [w_rows][ldw] the groups' weight matrices one after another (Nw rows each), tiles (device, int4 x max_tiles)
// lists {first A row, valid rows (0 = unused entry), first W row of the group, 0} per 128-row tile.
// C[row][0..Nw) = A[row] . W_group^T.
QW_API int qwk_gemm_bf16_tc_grouped(const void *A, const void *W, void *C, const void *tiles, int max_tiles, int rows,
                                    long long w_rows, int Nw, int K, int lda, int ldw, int ldc, int out_bf16,
                                    cudaStream_t s) {
    if (rows <= 0 || max_tiles <= 0) return 0;
    if ((K & 7) || (lda & 7) || (ldw & 7) || ((uintptr_t)A & 15) || ((uintptr_t)W & 15)) return -1;
    CUtensorMap mA, mW;
    if (!make_map(&mA, A, rows, K, lda, TC_BM) || !make_map(&mW, W, w_rows, K, ldw, TC_BN)) return -3;
    GemmTcArgs a{};
    a.C32 = out_bf16 ? nullptr : (float *)C;
    a.C16 = out_bf16 ? (bf16 *)C : nullptr;
    a.T = rows; a.N = Nw; a.K = K; a.ldc = ldc; a.err = g_err_ptr; a.tiles = (const int4 *)tiles;
    a.tiles_t = max_tiles; a.tiles_n = (Nw + TC_BN - 1) / TC_BN; a.total = a.tiles_t * a.tiles_n;
    a.ksplit = 1; a.kb_per = 0; a.c_split = 0;
    if (!configure_once(0)) return -3;
    gemm_tc_kernel<TC_BN, TC_STAGES><<<persistent_grid(a.total), 320, TC_SMEM, s>>>(mA, mW, a);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// Grouped form with q4 weights: Wq uint32 [w_rows][K/8] (engine nibble order), scale bf16 [w_rows][K/128]; otherwise
// as qwk_gemm_bf16_tc_grouped.  K a multiple of 128.
QW_API int qwk_gemm_q4_tc_grouped(const void *A, const void *Wq, const void *scale, void *C, const void *tiles, int max_tiles,
                                  int rows, long long w_rows, int Nw, int K, int lda, int ldc, int out_bf16, cudaStream_t s) {
    if (rows <= 0 || max_tiles <= 0) return 0;
    if ((K & 127) || (lda & 7) || ((uintptr_t)A & 15) || ((uintptr_t)Wq & 15)) return -1;
    CUtensorMap mA;
    if (!make_map(&mA, A, rows, K, lda, TC_BM)) return -3;
    GemmTcArgs a{};
    a.C32 = out_bf16 ? nullptr : (float *)C;
    a.C16 = out_bf16 ? (bf16 *)C : nullptr;
    a.T = rows; a.N = Nw; a.K = K; a.ldc = ldc; a.err = g_err_ptr; a.tiles = (const int4 *)tiles;
    a.tiles_t = max_tiles; a.tiles_n = (Nw + TC_BN - 1) / TC_BN; a.total = a.tiles_t * a.tiles_n;
    a.ksplit = 1; a.kb_per = 0; a.c_split = 0;
    if (!configure_once(1)) return -3;
    gemm_tc_q4_kernel<<<persistent_grid(a.total), 448, TC_SMEM, s>>>(mA, a, (const uint32_t *)Wq, (const bf16 *)scale, w_rows);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// Split-K form for products with few output tiles and a long K (the mixers' down projection): C_s = A[:, K_s] . W[:, K_s]^T
// for ksplit shares of K, partial s written as fp32 to C + s * c_split (elements); the consumer adds the partials in
// order, so the sum does not depend on timing.  ksplit <= number of k blocks.
QW_API int qwk_gemm_bf16_tc_splitk(const void *A, const void *W, float *C, int T, int N, int K, int lda, int ldw, int ldc,
                                   int ksplit, long long c_split, cudaStream_t s) {
    if (T <= 0 || N <= 0) return 0;
    const int kblocks = (K + TC_BK - 1) / TC_BK;
    if ((K & 7) || (lda & 7) || (ldw & 7) || ((uintptr_t)A & 15) || ((uintptr_t)W & 15) || ksplit < 1 || ksplit > kblocks) return -1;
    CUtensorMap mA, mW;
    if (!make_map(&mA, A, T, K, lda, TC_BM) || !make_map(&mW, W, N, K, ldw, TC_BN)) return -3;
    GemmTcArgs a{};
    a.C32 = C; a.C16 = nullptr;
    a.T = T; a.N = N; a.K = K; a.ldc = ldc; a.err = g_err_ptr; a.tiles = nullptr;
    a.tiles_t = (T + TC_BM - 1) / TC_BM; a.tiles_n = (N + TC_BN - 1) / TC_BN;
    a.kb_per = (kblocks + ksplit - 1) / ksplit;
    a.ksplit = (kblocks + a.kb_per - 1) / a.kb_per;          // every share holds at least one k block
    if (a.ksplit != ksplit) return -1;
    a.c_split = c_split;
    a.total = a.tiles_t * a.tiles_n * a.ksplit;
    if (!configure_once(0)) return -3;
    gemm_tc_kernel<TC_BN, TC_STAGES><<<persistent_grid(a.total), 320, TC_SMEM, s>>>(mA, mW, a);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
