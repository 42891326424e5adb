// Kernel-initiated collectives over NVLink peer memory (no NCCL): all-reduce, reduce-scatter and
// all-gather for the decode path's small payloads, each as ONE kernel that pushes this rank's data
// into every peer's receive slot with plain peer stores, publishes a sequence number with a
// release store, waits (bounded) for the peers' sequence numbers in its own memory and reduces the
// slots in rank order, so every rank computes bit-identical sums.
//
// Sequence numbers are `*base + k` with `base` a device-resident counter bumped once per step and k
// the collective's static index inside the step, so a captured CUDA graph replays correctly.  Slots
// and flags are double-buffered by the parity of k: a rank can be at most one collective ahead of
// any other, because each collective needs every rank's contribution.
// (Role of the reference's src/comm/comm.hip:43-202; the transport there is PCIe P2P.)
#include "fuse.cuh"

namespace qw {

constexpr int P2P_MAX_RANKS = 8;
constexpr unsigned SPIN_LIMIT = 1u << 28;      // polls before a wait gives up (~15 s)

struct P2PArgs {
    char *peer[P2P_MAX_RANKS];   // base of every rank's symmetric region (peer[rank] is local)
    int ranks, rank;
    const unsigned int *base;    // local: sequence base of this step
    unsigned int k;              // static index of this collective in the step
    long long off_flags;         // [2][ranks] uint32 per kind, 64 B apart
    long long off_recv;          // [2][ranks][slot_bytes]
    long long slot_bytes;
    int rows, n;                 // payload: rows x n elements per destination
    int elem;                    // bytes per element (4 fp32, 2 bf16)
    const char *src;             // local source
    int ld_src;                  // source row stride in elements
    int scatter;                 // 1: destination d gets columns [d*n, (d+1)*n) of each source row
    char *dst;                   // local result ([rows][ld_dst] elements); gather: [rows][ranks*n] in the symmetric region
    int ld_dst;
    long long off_gather;        // all-gather: offset of the destination matrix inside every region
    ErrorWord *err;
};

__device__ __forceinline__ bool wait_flags(const P2PArgs &a, unsigned int want, int parity) {
    __shared__ int s_ok;
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
    if ((int)threadIdx.x < a.ranks) {
        const unsigned int *f = reinterpret_cast<const unsigned int *>(a.peer[a.rank] + a.off_flags) + (parity * a.ranks + threadIdx.x) * 16;
        unsigned i = 0;
        while ((int)(ld_acquire_sys(f) - want) < 0) {
            if (++i > SPIN_LIMIT) {
                report(a.err, ERR_WAIT_TIMEOUT, 0x80000000u | (a.rank << 28) | (threadIdx.x << 24) | (a.k & 0xffffff));
                s_ok = 0;
                break;
            }
            if (a.err && (i & 1023) == 0 && a.err->code) { s_ok = 0; break; }     // someone already gave up
        }
    }
    __syncthreads();
    return s_ok != 0;
}

// grid = ranks + 1 blocks.  Blocks 0..ranks-1 push to peer (rank + b) % ranks; the last block waits and reduces.
// mode 0: all-reduce / reduce-scatter (fp32 sum in rank order), mode 1: all-gather (bytes land in place).
__global__ void __launch_bounds__(256) p2p_exchange_kernel(P2PArgs a, int mode) {
    pdl_wait();
    pdl_trigger();
    const unsigned int seq = *a.base + a.k;
    const int parity = a.k & 1;
    if ((int)blockIdx.x < a.ranks) {
        const int d = (a.rank + blockIdx.x) % a.ranks;
        const int row_bytes = a.n * a.elem;
        char *dbase;
        long long drow;
        if (mode == 0) {
            dbase = a.peer[d] + a.off_recv + ((long long)parity * a.ranks + a.rank) * a.slot_bytes;
            drow = row_bytes;
        } else {
            dbase = a.peer[d] + a.off_gather + (long long)a.rank * row_bytes;
            drow = (long long)a.ranks * row_bytes;
        }
        const int chunks = row_bytes >> 2;                      // 4-byte pieces per row
        const long long scol = a.scatter ? (long long)d * row_bytes : 0;
        if (!(mode == 1 && d == a.rank)) {                       // a gather's own slice is already in place
            for (int i = threadIdx.x; i < a.rows * chunks; i += blockDim.x) {
                const int m = i / chunks, c = i - m * chunks;
                const unsigned int v = *reinterpret_cast<const unsigned int *>(a.src + (long long)m * a.ld_src * a.elem + scol + c * 4);
                *reinterpret_cast<unsigned int *>(dbase + m * drow + c * 4) = v;
            }
        }
        __threadfence_system();
        __syncthreads();
        if (threadIdx.x == 0) {
            unsigned int *f = reinterpret_cast<unsigned int *>(a.peer[d] + a.off_flags) + (parity * a.ranks + a.rank) * 16;
            st_release_sys(f, seq);
        }
        return;
    }
    if (!wait_flags(a, seq, parity)) return;
    if (mode == 1) return;
    const float *slots = reinterpret_cast<const float *>(a.peer[a.rank] + a.off_recv + (long long)parity * a.ranks * a.slot_bytes);
    const long long sstride = a.slot_bytes >> 2;
    float *out = reinterpret_cast<float *>(a.dst);
    for (int i = threadIdx.x; i < a.rows * a.n; i += blockDim.x) {
        const int m = i / a.n, c = i - m * a.n;
        float v = 0.f;
        for (int r = 0; r < a.ranks; ++r) v += __ldcg(slots + r * sstride + i);     // rank order: identical on every rank
        out[(long long)m * a.ld_dst + c] = v;
    }
}

__global__ void bump_base_kernel(unsigned int *base, unsigned int by) {
    pdl_wait();
    pdl_trigger();
    if (threadIdx.x == 0) *base += by;
}

}  // namespace qw

using namespace qw;

extern "C" {
typedef struct QwP2P {
    void *peer[8];             // symmetric region base on every rank
    int ranks, rank;
    unsigned int *base;        // local sequence counter
    long long off_flags[4];    // per kind: 0 all-reduce, 1 all-gather, 2 reduce-scatter, 3 small gather
    long long off_recv[4];
    long long slot_bytes[4];
    long long off_bin;         // block-input matrix [rows][H] bf16 inside the region (gather target)
    long long off_amax;        // [rows][ranks*2] fp32 gather target
} QwP2P;
}

static void fill(P2PArgs &a, const QwP2P *p, int kind, unsigned k) {
    for (int i = 0; i < 8; ++i) a.peer[i] = (char *)p->peer[i];
    a.ranks = p->ranks; a.rank = p->rank; a.base = p->base; a.k = k;
    a.off_flags = p->off_flags[kind]; a.off_recv = p->off_recv[kind]; a.slot_bytes = p->slot_bytes[kind];
    a.err = g_err_ptr; a.scatter = 0; a.off_gather = 0; a.dst = nullptr; a.ld_dst = 0;
}

namespace qw {
// Where a producer kernel's words for collective k of `kind` go: this rank's slot on every rank.
FuseOut make_fuse_out(const void *p2p, int kind, unsigned k, int mode, int n) {
    const QwP2P *p = (const QwP2P *)p2p;
    FuseOut o{};
    const int parity = k & 1;
    o.mode = mode; o.ranks = p->ranks; o.rank = p->rank;
    for (int i = 0; i < p->ranks && i < FUSE_MAX_RANKS; ++i)
        o.slot[i] = (char *)p->peer[i] + p->off_recv[kind] + ((long long)parity * p->ranks + p->rank) * p->slot_bytes[kind];
    o.base = p->base; o.k = k; o.n = n;
    return o;
}

// Where a consumer kernel finds the ranks' words of collective k of `kind`.
FuseIn make_fuse_in(const void *p2p, int kind, unsigned k, int n) {
    const QwP2P *p = (const QwP2P *)p2p;
    FuseIn in{};
    const int parity = k & 1;
    in.active = 1; in.ranks = p->ranks;
    in.slots = (const char *)p->peer[p->rank] + p->off_recv[kind] + (long long)parity * p->ranks * p->slot_bytes[kind];
    in.slot_bytes = p->slot_bytes[kind];
    in.base = p->base; in.k = k; in.n = n;
    in.err = g_err_ptr;
    return in;
}
}  // namespace qw

// kind 0: dst[rows][n] = sum over ranks of src[rows][n] (fp32).
QW_API int qwk_p2p_allreduce(const void *p2p, unsigned int k, const float *src, float *dst, int rows, int n, cudaStream_t s) {
    const QwP2P *p = (const QwP2P *)p2p;
    P2PArgs a;
    fill(a, p, 0, k);
    if ((long long)rows * n * 4 > a.slot_bytes) return -1;
    a.rows = rows; a.n = n; a.elem = 4; a.src = (const char *)src; a.ld_src = n; a.dst = (char *)dst; a.ld_dst = n;
    return launch_pdl(p2p_exchange_kernel, dim3(p->ranks + 1), dim3(256), 0, s, a, 0) == cudaSuccess ? 0 : -2;
}

// kind 2: dst[rows][n] = sum over ranks of their src[rows][rank*n .. rank*n+n) (fp32).
QW_API int qwk_p2p_reduce_scatter(const void *p2p, unsigned int k, const float *src, float *dst, int rows, int n,
                                  cudaStream_t s) {
    const QwP2P *p = (const QwP2P *)p2p;
    P2PArgs a;
    fill(a, p, 2, k);
    if ((long long)rows * n * 4 > a.slot_bytes) return -1;
    a.rows = rows; a.n = n; a.elem = 4; a.src = (const char *)src; a.ld_src = p->ranks * n; a.scatter = 1;
    a.dst = (char *)dst; a.ld_dst = n;
    return launch_pdl(p2p_exchange_kernel, dim3(p->ranks + 1), dim3(256), 0, s, a, 0) == cudaSuccess ? 0 : -2;
}

// kind 1 / 3: every rank's slice [rows][n] (already at column rank*n of its own matrix at `off` inside the
// region) lands at the same place in every peer's matrix.  elem = bytes per element.
QW_API int qwk_p2p_allgather(const void *p2p, unsigned int k, int kind, long long off, int rows, int n, int elem,
                             cudaStream_t s) {
    const QwP2P *p = (const QwP2P *)p2p;
    P2PArgs a;
    fill(a, p, kind, k);
    if ((n * elem) & 3) return -1;
    a.rows = rows; a.n = n; a.elem = elem; a.off_gather = off;
    a.src = (const char *)p->peer[p->rank] + off + (long long)p->rank * n * elem;
    a.ld_src = p->ranks * n;
    return launch_pdl(p2p_exchange_kernel, dim3(p->ranks + 1), dim3(256), 0, s, a, 1) == cudaSuccess ? 0 : -2;
}

QW_API int qwk_p2p_bump_base(const void *p2p, unsigned int by, cudaStream_t s) {
    const QwP2P *p = (const QwP2P *)p2p;
    return launch_pdl(bump_base_kernel, dim3(1), dim3(32), 0, s, p->base, by) == cudaSuccess ? 0 : -2;
}
