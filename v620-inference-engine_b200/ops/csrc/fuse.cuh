// Collectives fused into the kernels around them (tensor / expert parallel decode), low-latency protocol.
//
// Every value that has to cross NVLink travels as one 8-byte word {payload, sequence number}, written
// with a single 8-byte store straight from the thread that computed it into the receive slot of every
// rank that needs it.  A consumer polls the word itself until it carries the sequence number of the
// collective it is waiting for - bounded - so there are no flags, no fences and no "last block": the
// transfer starts while the producer kernel is still running and costs one NVLink crossing.
// Reductions are done by the consumer, adding the ranks' words in rank order, so every rank computes
// bit-identical sums.  No kernel sits between producer and consumer.
//
//   all-reduce      hc_down  -> [every rank]        -> hc_up_mix adds the ranks' partial sums
//   all-gather      hc_up_mix -> [every rank]       -> the block's first matrix product builds its rows
//   reduce-scatter  out-projection / expert down    -> [owner of the column] -> hc_down adds the ranks' parts
//
// Sequence numbers are `*base + k` (a device counter bumped once per step + the collective's static
// index in the step), slots are double buffered by the parity of k; both as in p2p.cu, whose
// stand-alone collectives can be mixed with fused ones inside a step.
// (Role of the reference's src/comm/comm.hip:43-202, where collectives are separate launches.)
#pragma once
#include "common.cuh"
#include "stream.cuh"

namespace qw {

constexpr int FUSE_MAX_RANKS = 8;
constexpr unsigned FUSE_SPIN_LIMIT = 1u << 26;      // polls of one word before a wait gives up (~15 s: a rank whose host launches its step a second late is not a failure)

struct FuseOut {
    int mode;                    // 0 off | 1 every word to every rank (all-reduce, all-gather) | 2 column c of a row to rank c / n (reduce-scatter)
    int ranks, rank;
    char *slot[FUSE_MAX_RANKS];  // on rank r: this rank's receive slot for collective k ([rows][n] words)
    const unsigned int *base;    // local: sequence base of this step
    unsigned int k;              // static index of this collective in the step
    int n;                       // words per row in a slot
};

struct FuseIn {
    int active, ranks;
    const char *slots;           // local: slot of rank r at slots + r * slot_bytes
    long long slot_bytes;
    const unsigned int *base;
    unsigned int k;
    int n;                       // words per row in a slot
    ErrorWord *err;
};

// host side: what the next launcher should fuse (cleared when taken), and their builders (p2p.cu)
extern FuseOut g_fo;
extern FuseIn g_fi;
inline FuseOut take_fo() { FuseOut r = g_fo; g_fo = FuseOut{}; return r; }
inline FuseIn take_fi() { FuseIn r = g_fi; g_fi = FuseIn{}; return r; }
FuseOut make_fuse_out(const void *p2p, int kind, unsigned k, int mode, int n);
FuseIn make_fuse_in(const void *p2p, int kind, unsigned k, int n);

__device__ __forceinline__ void st_release_sys(unsigned int *p, unsigned int v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int *p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_word(char *p, unsigned int payload, unsigned int seq) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(payload), "r"(seq) : "memory");
}
__device__ __forceinline__ uint2 ld_word(const char *p) {
    uint2 v;
    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ unsigned int fuse_seq(const FuseOut &o) { return __ldcg(o.base) + o.k; }
__device__ __forceinline__ unsigned int fuse_seq(const FuseIn &in) { return __ldcg(in.base) + in.k; }

// Producer: word `w` of row `m` goes to every rank.  (Static indices only: a dynamically indexed kernel-parameter
// array would be copied to local memory by every thread.)
__device__ __forceinline__ void fuse_put_all(const FuseOut &o, unsigned int seq, int m, int w, unsigned int payload) {
    const long long off = ((long long)m * o.n + w) * 8;
#pragma unroll
    for (int d = 0; d < FUSE_MAX_RANKS; ++d)
        if (d < o.ranks) st_word(o.slot[d] + off, payload, seq);
}
// Producer: column `c` of row `m` of a [rows][ranks * n] matrix goes to the rank that owns the column.
__device__ __forceinline__ void fuse_put_col(const FuseOut &o, unsigned int seq, int m, int c, unsigned int payload) {
    const int d = c / o.n, w = c - d * o.n;
    char *p = o.slot[0];
#pragma unroll
    for (int r = 1; r < FUSE_MAX_RANKS; ++r)
        if (r == d) p = o.slot[r];
    st_word(p + ((long long)m * o.n + w) * 8, payload, seq);
}

// Consumer: the payload of word `w` of row `m` in rank r's slot, once it carries `seq`.
__device__ __forceinline__ unsigned int fuse_get(const FuseIn &in, unsigned int seq, int r, long long word) {
    const char *p = in.slots + r * in.slot_bytes + word * 8;
    uint2 v = ld_word(p);
    unsigned int i = 0;
    while (v.y != seq) {
        if (++i > FUSE_SPIN_LIMIT) {
            report(in.err, ERR_WAIT_TIMEOUT, 0x40000000u | ((unsigned)r << 24) | (in.k & 0xffffffu));
            return 0u;
        }
        if (in.err && (i & 4095u) == 0 && in.err->code) return 0u;     // someone already gave up
        v = ld_word(p);
    }
    return v.x;
}
__device__ __forceinline__ uint4 ld_word2(const char *p) {          // two adjacent words, 16-byte aligned
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

// Element `i` (row-major over [rows][n]) of a reduced result: the ranks' words added in rank order.  The loads of
// four ranks are issued before the first one is looked at; a word that has not arrived yet is then polled.
__device__ __forceinline__ float fuse_sum(const FuseIn &in, unsigned int seq, long long i) {
    float v = 0.f;
    for (int r0 = 0; r0 < in.ranks; r0 += 4) {
        uint2 w[4];
#pragma unroll
        for (int r = 0; r < 4; ++r)
            if (r0 + r < in.ranks) w[r] = ld_word(in.slots + (r0 + r) * in.slot_bytes + i * 8);
#pragma unroll
        for (int r = 0; r < 4; ++r)
            if (r0 + r < in.ranks) v += __uint_as_float(w[r].y == seq ? w[r].x : fuse_get(in, seq, r0 + r, i));
    }
    return v;
}

// Two consecutive elements starting at `i` (i even), for two positions at once.
__device__ __forceinline__ void fuse_sum2x2(const FuseIn &in, unsigned int seq, long long i0, long long i1, float2 &s0, float2 &s1) {
    s0 = make_float2(0.f, 0.f);
    s1 = make_float2(0.f, 0.f);
    for (int r0 = 0; r0 < in.ranks; r0 += 4) {
        uint4 a[4], b[4];
#pragma unroll
        for (int r = 0; r < 4; ++r)
            if (r0 + r < in.ranks) {
                a[r] = ld_word2(in.slots + (r0 + r) * in.slot_bytes + i0 * 8);
                b[r] = ld_word2(in.slots + (r0 + r) * in.slot_bytes + i1 * 8);
            }
#pragma unroll
        for (int r = 0; r < 4; ++r)
            if (r0 + r < in.ranks) {
                s0.x += __uint_as_float(a[r].y == seq ? a[r].x : fuse_get(in, seq, r0 + r, i0));
                s0.y += __uint_as_float(a[r].w == seq ? a[r].z : fuse_get(in, seq, r0 + r, i0 + 1));
                s1.x += __uint_as_float(b[r].y == seq ? b[r].x : fuse_get(in, seq, r0 + r, i1));
                s1.y += __uint_as_float(b[r].w == seq ? b[r].z : fuse_get(in, seq, r0 + r, i1 + 1));
            }
    }
}

// Four consecutive elements starting at `i` (i even).
__device__ __forceinline__ float4 fuse_sum4(const FuseIn &in, unsigned int seq, long long i) {
    float2 lo, hi;
    fuse_sum2x2(in, seq, i, i + 2, lo, hi);
    return make_float4(lo.x, lo.y, hi.x, hi.y);
}

// Eight consecutive 16-bit payloads (all-gather of bf16) of rank r starting at word `i` (a multiple of 2), packed.
__device__ __forceinline__ uint4 fuse_get8_u16(const FuseIn &in, unsigned int seq, int r, long long i) {
    const char *p = in.slots + r * in.slot_bytes + i * 8;
    uint4 q[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) q[j] = ld_word2(p + 16 * j);
    unsigned int h[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        h[2 * j] = q[j].y == seq ? q[j].x : fuse_get(in, seq, r, i + 2 * j);
        h[2 * j + 1] = q[j].w == seq ? q[j].z : fuse_get(in, seq, r, i + 2 * j + 1);
    }
    return make_uint4((h[0] & 0xffffu) | (h[1] << 16), (h[2] & 0xffffu) | (h[3] << 16), (h[4] & 0xffffu) | (h[5] << 16),
                      (h[6] & 0xffffu) | (h[7] << 16));
}

}  // namespace qw
