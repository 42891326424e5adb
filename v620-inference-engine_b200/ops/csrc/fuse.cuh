// Collectives fused into the kernels around them (tensor / expert parallel decode).
//
// A producer kernel (one that computes what a collective sends) ends with fuse_publish: the block that
// finishes last copies the kernel's result straight into every peer's receive slot over NVLink with
// plain peer stores and then raises this rank's sequence flag on every peer with a release store.
// A consumer kernel (one that needs the collective's result) starts, after its weight prefetch, with
// fuse_wait: it polls - bounded - the flags the peers raise in its own memory, and then reads the
// result, summing the ranks' slots in rank order where the collective is a reduction, so every rank
// computes bit-identical sums.  No kernel sits between the two: the transfer overlaps the consumer's
// launch and weight prefetch, and a step has no collective launches at all.
//
// Flags, slots, sequence numbers (`*base + k`, parity double buffering) are those of the stand-alone
// collectives in p2p.cu, so fused and stand-alone sites can be mixed inside a step.
// (Role of the reference's src/comm/comm.hip:43-202, where collectives are separate launches.)
#pragma once
#include "common.cuh"
#include "stream.cuh"

namespace qw {

constexpr int FUSE_MAX_RANKS = 8;
constexpr unsigned FUSE_SPIN_LIMIT = 1u << 24;      // polls before a wait gives up (about a second)

struct FuseOut {
    int mode;                    // 0 off | 1 whole rows to every rank's slot (all-reduce) | 2 column block d to rank d's
                                 // slot (reduce-scatter) | 3 rows into place in every peer's matrix (all-gather)
    int ranks, rank;
    char *peer[FUSE_MAX_RANKS];  // base of every rank's symmetric region
    const unsigned int *base;    // local: sequence base of this step
    unsigned int k;              // static index of this collective in the step
    long long off_flags, off_recv, slot_bytes, off_gather;
    const char *src;             // local result of this kernel
    int ld_src;                  // row stride of src in elements
    int rows, n, elem;           // rows x n elements of `elem` bytes per destination
    unsigned int *ticket;        // zero before the launch; the last block resets it
    ErrorWord *err;
};

struct FuseIn {
    int active, ranks;
    const unsigned int *flags;   // local: flag of rank r at flags[r * 16]
    const unsigned int *base;
    unsigned int k;
    const float *slots;          // reductions: slot of rank r at slots + r * sstride
    long long sstride;           // floats
    ErrorWord *err;
};

// host side: what the next launcher should fuse (cleared when taken), and their builders (p2p.cu)
extern FuseOut g_fo;
extern FuseIn g_fi;
inline FuseOut take_fo() { FuseOut r = g_fo; g_fo = FuseOut{}; return r; }
inline FuseIn take_fi() { FuseIn r = g_fi; g_fi = FuseIn{}; return r; }
FuseOut make_fuse_out(const void *p2p, int kind, unsigned k, int mode, const void *src, int ld_src, int rows, int n,
                      int elem, long long off_gather, unsigned int *ticket);
FuseIn make_fuse_in(const void *p2p, int kind, unsigned k, bool reduce);

__device__ __forceinline__ void st_release_sys(unsigned int *p, unsigned int v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int *p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Every thread of every block calls this as the kernel's last statement.
__device__ __forceinline__ void fuse_publish(const FuseOut &o) {
    if (o.mode == 0) return;
    __shared__ unsigned int s_fuse_last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int total = gridDim.x * gridDim.y * gridDim.z;
        s_fuse_last = atomicAdd(o.ticket, 1u) == total - 1 ? 1u : 0u;
    }
    __syncthreads();
    if (!s_fuse_last) return;
    __threadfence();
    const unsigned int seq = __ldcg(o.base) + o.k;
    const int parity = o.k & 1;
    const long long row_bytes = (long long)o.n * o.elem, ld_bytes = (long long)o.ld_src * o.elem;
    const bool wide = ((row_bytes | ld_bytes | (long long)(size_t)o.src | o.slot_bytes | o.off_recv | o.off_gather) & 15) == 0;
    for (int dd = 0; dd < o.ranks; ++dd) {
        const int d = (o.rank + dd) % o.ranks;
        if (o.mode == 3 && d == o.rank) continue;            // a gather's own rows are already in place
        char *dbase;
        long long drow, scol = 0;
        if (o.mode == 3) {
            dbase = o.peer[d] + o.off_gather + (long long)o.rank * row_bytes;
            drow = (long long)o.ranks * row_bytes;
        } else {
            dbase = o.peer[d] + o.off_recv + ((long long)parity * o.ranks + o.rank) * o.slot_bytes;
            drow = row_bytes;
            if (o.mode == 2) scol = (long long)d * row_bytes;
        }
        if (wide) {
            const int chunks = (int)(row_bytes >> 4);
            for (int i = threadIdx.x; i < o.rows * chunks; i += blockDim.x) {
                const int m = i / chunks, c = i - m * chunks;
                const uint4 v = __ldcg(reinterpret_cast<const uint4 *>(o.src + m * ld_bytes + scol) + c);
                *reinterpret_cast<uint4 *>(dbase + m * drow + (long long)c * 16) = v;
            }
        } else {
            const int chunks = (int)(row_bytes >> 2);
            for (int i = threadIdx.x; i < o.rows * chunks; i += blockDim.x) {
                const int m = i / chunks, c = i - m * chunks;
                const unsigned int v = __ldcg(reinterpret_cast<const unsigned int *>(o.src + m * ld_bytes + scol) + c);
                *reinterpret_cast<unsigned int *>(dbase + m * drow + (long long)c * 4) = v;
            }
        }
    }
    __threadfence_system();
    __syncthreads();
    if ((int)threadIdx.x < o.ranks) {
        unsigned int *f = reinterpret_cast<unsigned int *>(o.peer[threadIdx.x] + o.off_flags) + (parity * o.ranks + o.rank) * 16;
        st_release_sys(f, seq);
    }
    if (threadIdx.x == 0) *o.ticket = 0u;
}

// Threads 0..ranks-1 of the calling group poll; `named` = the group is the 256 consumer threads of the
// streaming core (named barrier 1), otherwise the whole block.  Returns false after a timeout (the error
// word holds where); the caller carries on so that the kernel ends.
__device__ __forceinline__ bool fuse_wait(const FuseIn &in, bool named) {
    if (!in.active) return true;
    __shared__ int s_fuse_ok;
    if (threadIdx.x == 0) s_fuse_ok = 1;
    if (named) consumer_sync(256); else __syncthreads();
    if ((int)threadIdx.x < in.ranks) {
        const unsigned int want = __ldcg(in.base) + in.k;
        const unsigned int *f = in.flags + threadIdx.x * 16;
        unsigned int i = 0;
        while ((int)(ld_acquire_sys(f) - want) < 0) {
            if (++i > FUSE_SPIN_LIMIT) {
                report(in.err, ERR_WAIT_TIMEOUT, 0x40000000u | (threadIdx.x << 24) | (in.k & 0xffffffu));
                s_fuse_ok = 0;
                break;
            }
            if (in.err && (i & 1023u) == 0 && in.err->code) { s_fuse_ok = 0; break; }     // someone already gave up
        }
    }
    if (named) consumer_sync(256); else __syncthreads();
    return s_fuse_ok != 0;
}

// Element i of a reduced result: the ranks' slots added in rank order.
__device__ __forceinline__ float fuse_sum(const FuseIn &in, long long i) {
    float v = 0.f;
    for (int r = 0; r < in.ranks; ++r) v += __ldcg(in.slots + r * in.sstride + i);
    return v;
}
__device__ __forceinline__ float4 fuse_sum4(const FuseIn &in, long long i) {
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < in.ranks; ++r) {
        const float4 t = __ldcg(reinterpret_cast<const float4 *>(in.slots + r * in.sstride + i));
        v.x += t.x; v.y += t.y; v.z += t.z; v.w += t.w;
    }
    return v;
}

}  // namespace qw
