// Tensor-parallel token-major prefill: collectives carried by the kernels that produce and consume
// their payload, for payloads of megabytes (a 4,096-token chunk moves 20-40 MB per sublayer).
//
// Transport: every rank owns a region of the same layout that all ranks have mapped (NVLink peer
// memory).  A producer kernel stores its results straight into the receive buffers of the ranks that
// need them - the reduce-scatter of a block output from the epilogue of the out-projection GEMM, the
// all-gather of the block input from the mixer's last kernel, the mixers' two all-reduces from the
// kernels that form the partial sums - so the transfer runs tile by tile under the producer's math.
// When a CTA has stored everything it will store, it fences system-wide and takes a ticket; the CTA
// that takes the last ticket publishes the collective's sequence number to every destination with a
// release store.  A consumer kernel polls (bounded) the flags of all source ranks in its own memory,
// then reads its receive buffer past L1 and adds the ranks' parts in rank order, so sums do not
// depend on timing.  Tensor maps only ever cover the rank's own memory.
//
// One collective kind has one flag per source rank and one receive buffer; reuse of a buffer by the
// next collective of the same kind is safe because every rank passes through an all-reduce (which needs
// every rank's kernels up to that point) between two uses.  Sequence numbers count the collectives of
// a kind since the channel was made and are handed to the kernels by value (prefill is not graph
// captured).
// (Role of the reference's src/comm/comm.hip:276-335 large-payload paths and of the collective sites
// of src/engine/prefill.hip:208-224,318,340.)
#pragma once
#include "fuse.cuh"

namespace qw {

constexpr int TP_MAX_RANKS = 8;
constexpr int TP_KINDS = 6;          // 0 ssq all-reduce | 1 mixer-down all-reduce | 2 block-input all-gather | 3 reduce-scatter | 4 small all-reduce / gather | 5 wide all-gather (MTP)

// What a producer CTA does when its stores are done.
struct TpSignal {
    unsigned int *ticket;                 // local, zero between launches
    unsigned int nblocks;                 // CTAs of the launch that will call tp_signal
    unsigned int *flag[TP_MAX_RANKS];     // on rank d: the flag of (kind, this rank)
    int ranks;
    unsigned int seq;
};
// What a consumer waits for.
struct TpWait {
    const unsigned int *flags;            // local: flags of the kind, one per source rank, 64 bytes apart
    int ranks;
    unsigned int seq;
    unsigned int limit;                   // polls before the wait gives up
    ErrorWord *err;
};

// All threads of the CTA call this after their last store of the collective.
__device__ __forceinline__ void tp_signal(const TpSignal &s) {
    if (!s.ticket) return;
    __syncthreads();
    if (threadIdx.x == 0 && threadIdx.y == 0 && threadIdx.z == 0) {
        __threadfence_system();
        const unsigned int old = atomicAdd(s.ticket, 1u);
        if (old == s.nblocks - 1u) {
            atomicExch(s.ticket, 0u);
            __threadfence_system();
#pragma unroll
            for (int d = 0; d < TP_MAX_RANKS; ++d)
                if (d < s.ranks) st_release_sys(s.flag[d], s.seq);
        }
    }
}

// One thread's bounded wait for the flag of source rank r.
__device__ __forceinline__ bool tp_wait_one(const TpWait &w, int r) {
    const unsigned int *f = w.flags + r * 16;
    unsigned int i = 0;
    while ((int)(ld_acquire_sys(f) - w.seq) < 0) {
        if (w.err && (i & 1023u) == 0u && *reinterpret_cast<volatile unsigned int *>(&w.err->code)) return false;       // someone already gave up
        if (++i > w.limit) {
            report(w.err, ERR_WAIT_TIMEOUT, 0x20000000u | ((unsigned)r << 24) | (w.seq & 0xffffffu));
            return false;
        }
    }
    return true;
}

// All threads of the CTA call this before the first read of the receive buffer; false = gave up (skip the work).
__device__ __forceinline__ bool tp_wait(const TpWait &w) {
    if (!w.flags) return true;
    __shared__ int s_tp_ok;
    const int tid = threadIdx.x + blockDim.x * (threadIdx.y + blockDim.y * threadIdx.z);
    if (tid == 0) s_tp_ok = 1;
    __syncthreads();
    if (tid < w.ranks && !tp_wait_one(w, tid)) s_tp_ok = 0;
    __syncthreads();
    return s_tp_ok != 0;
}

// A single thread waits for every source rank (GEMM producer thread before its first load of a gathered operand).
__device__ __forceinline__ bool tp_wait_thread(const TpWait &w) {
    if (!w.flags) return true;
    for (int r = 0; r < w.ranks; ++r)
        if (!tp_wait_one(w, r)) return false;
    asm volatile("fence.proxy.async;" ::: "memory");      // the loads that follow go through the async proxy
    return true;
}

// Where the epilogue of a GEMM sends its output tile.
struct TpEpilogue {
    int mode;                        // 0 local store only | 1 every rank gets the tile (all-reduce parts) | 2 the owner of the columns gets it (reduce-scatter)
    int ranks;
    int cols_per_rank;               // mode 2: columns [d * cols_per_rank, (d + 1) * cols_per_rank) belong to rank d
    int ld;                          // row stride (elements) of the destination buffers
    float *dst[TP_MAX_RANKS];        // on rank d: this rank's part ([rows][ld] fp32)
    TpSignal sig;
};

__device__ __forceinline__ float *tp_pick(float *const (&p)[TP_MAX_RANKS], int d) {
    float *r = p[0];
#pragma unroll
    for (int i = 1; i < TP_MAX_RANKS; ++i)
        if (i == d) r = p[i];
    return r;
}

}  // namespace qw

// ---- the channel as the host sees it (filled by Python through a ctypes mirror of the same layout) ----
extern "C" {
typedef struct QwTp {
    void *peer[8];                 // base of every rank's region (peer[rank] is this rank's own)
    int ranks, rank;
    long long off_flags;           // [TP_KINDS][8] words, 64 bytes apart, zero at start
    long long off_buf[6];          // receive buffer of each kind inside a region
    long long part_bytes[6];       // bytes between the parts of two source ranks (kinds that keep one part per source)
    unsigned int *ticket;          // local device memory: TP_KINDS zeroed words
    unsigned int seq[6];           // collectives of each kind issued so far (host counter)
    unsigned int spin_limit;       // polls before a wait gives up
    int pad_;
} QwTp;
}

namespace qw {

// The next collective of `kind` as its producer sees it (advances the kind's sequence number).
inline TpSignal tp_make_signal(QwTp *tp, int kind, unsigned nblocks) {
    TpSignal s{};
    s.ticket = tp->ticket + kind;
    s.nblocks = nblocks;
    s.ranks = tp->ranks;
    s.seq = ++tp->seq[kind];
    for (int d = 0; d < tp->ranks && d < TP_MAX_RANKS; ++d)
        s.flag[d] = reinterpret_cast<unsigned int *>((char *)tp->peer[d] + tp->off_flags) + (kind * 8 + tp->rank) * 16;
    return s;
}
// The latest collective of `kind` as its consumer sees it.
inline TpWait tp_make_wait(const QwTp *tp, int kind) {
    TpWait w{};
    w.flags = reinterpret_cast<const unsigned int *>((const char *)tp->peer[tp->rank] + tp->off_flags) + kind * 8 * 16;
    w.ranks = tp->ranks;
    w.seq = tp->seq[kind];
    // default: ~2^25 polls, tens of seconds.  A peer whose host stalls in the middle of enqueueing a chunk (a page-locking call in
    // another thread, a collection pause) is late by a second or more; a peer that is gone is found by the host long before
    w.limit = tp->spin_limit ? tp->spin_limit : (1u << 25);
    w.err = g_err_ptr;
    return w;
}
// This rank's part inside rank d's receive buffer of `kind`.
inline char *tp_part_on(const QwTp *tp, int kind, int d) {
    return (char *)tp->peer[d] + tp->off_buf[kind] + (long long)tp->rank * tp->part_bytes[kind];
}
// The parts of all source ranks in this rank's own receive buffer of `kind` (part r at + r * part_bytes).
inline const char *tp_parts(const QwTp *tp, int kind) { return (const char *)tp->peer[tp->rank] + tp->off_buf[kind]; }

}  // namespace qw
