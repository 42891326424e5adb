// Shared device helpers for the sm_100a kernels: warp/block reductions, bf16 packing, the
// exact q4 -> bf16 pair conversion, activation functions, bounded waits and the row tables
// that batched-decode kernels take.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define QW_API extern "C" __attribute__((visibility("default")))

namespace qw {

typedef __nv_bfloat16 bf16;
typedef __nv_bfloat162 bf162;

constexpr int MAX_ROWS = 32;       // rows of one batched decode step
constexpr int KV_PAGE = 256;       // tokens per KV page (also the prefix-cache block size)
constexpr int RAW_RING = 16;       // raw indexer keys kept per slot and layer
constexpr int GDN_RING = 16;       // pre-conv rows kept per slot and layer
constexpr int PLE_RING = 32;       // normalised conv inputs kept per slot
constexpr int LIST_CAP = 2048 + 8; // attended tokens per query: 512 groups x 4 + open tail

// Error word shared by every kernel that can give up (bounded waits, bounds checks).  Kernels
// never trap: they record a code here (first writer wins) and return.
struct ErrorWord {
    unsigned int code;      // 0 = ok
    unsigned int detail;
};
enum ErrCode : unsigned int {
    ERR_NONE = 0,
    ERR_WAIT_TIMEOUT = 1,   // a flag / mbarrier wait ran out
    ERR_BOUNDS = 2,         // a data-derived index was out of range (checked builds)
    ERR_CAPACITY = 3,       // a table or list was too small
};
__device__ __forceinline__ void report(ErrorWord *e, unsigned int code, unsigned int detail) {
    if (e && atomicCAS(&e->code, 0u, code) == 0u) e->detail = detail;
}
// Checked builds (-DQW_DEVICE_CHECKS, the library libqw_kernels_checked.so): indices that come from data - token ids,
// positions, page numbers - are validated where they are used.  A violation records ERR_BOUNDS with `detail` in the
// error word and the kernel skips the access and returns; nothing traps, so the context stays usable and the host reads
// the word like any other kernel failure.  Without the flag the checks compile to nothing.  A translation unit that uses
// QW_DCHECK registers itself with QW_DCHECK_TU(name); qwk_set_error_word then hands the word's address to every one of
// them (each unit keeps its own copy: the library is built without relocatable device code).
// (Role of the reference's QW_DCHECK, src/kernels/common.cuh:13-24, which traps instead.)
#ifdef QW_DEVICE_CHECKS
static __device__ __attribute__((unused)) ErrorWord *s_dcheck_word = nullptr;
#define QW_DCHECK(cond, detail)                                             \
    do {                                                                    \
        if (!(cond)) {                                                      \
            report(s_dcheck_word, ERR_BOUNDS, (unsigned int)(detail));      \
            return;                                                         \
        }                                                                   \
    } while (0)
#define QW_DCHECK_TU(name)                                                                                  \
    extern "C" __attribute__((visibility("default"))) int qw_dcheck_set_##name(void *p) {                   \
        return cudaMemcpyToSymbol(qw::s_dcheck_word, &p, sizeof(p)) == cudaSuccess ? 0 : -2;                \
    }
#else
#define QW_DCHECK(cond, detail) \
    do {                        \
    } while (0)
#define QW_DCHECK_TU(name)
#endif

// Device address of the error word every launcher hands to its kernel (set once by the host through
// qwk_set_error_word; null until then, in which case kernels only give up silently).
extern ErrorWord *g_err_ptr;
// host side: asks the next expert gate/up launch to also form the shared expert's activation from the router's outputs
// (a few extra blocks of that launch, in parallel with the routed experts) instead of the router's last block doing it
// in its serial tail.  rs == null: nothing extra.
struct SharedAct {
    const float *rs;     // [M][ld_rs]: router logits (E) | shared gate logit | shared gate rows (SF) | shared up rows (SF)
    int ld_rs, E, SF;
    void *sh_h;          // out: [M][SF] bf16
};
extern SharedAct g_shared_act;
inline SharedAct take_shared_act() {
    SharedAct r = g_shared_act;
    g_shared_act = SharedAct{nullptr, 0, 0, 0, nullptr};
    return r;
}
extern int *g_moe_stats;     // host side: where the next routing launch adds its count of local pairs (null = nowhere)

// Row tables of a batched step.  Row i appends one token to slot[i] at position pos[i]; rows of
// one slot are consecutive and run_start[i] is the first row of that slot's run.
struct Rows {
    int M;
    const int *slot;        // [M]
    const int *pos;         // [M]
    const int *run_start;   // [M]
    const int *run_len;     // [M] (valid at the first row of a run)
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of NT threads (NT a multiple of 32, <= 1024); every thread gets the result.
// Fixed order: lanes by xor-shuffle, then warps 0..n-1 serially.
template <int NT>
__device__ __forceinline__ float block_sum(float v, float *scratch /* >= 32 floats */) {
    v = warp_sum(v);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    __syncthreads();
    if (l == 0) scratch[w] = v;
    __syncthreads();
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < NT / 32; ++i) s += scratch[i];
    return s;
}

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }
__device__ __forceinline__ float siluf_(float x) { return x * sigmoidf_(x); }
__device__ __forceinline__ float softplusf_(float x) { return x > 20.f ? x : log1pf(__expf(x)); }

__device__ __forceinline__ float bf16_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
    bf162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&h);
}

// Streaming 16-byte load that does not allocate in L1 (weights are read once).
__device__ __forceinline__ uint4 ld_stream(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ld_stream8(const void *p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}

// q4 engine order: elements 2j and 2j+1 of a word sit at bits 4j and 16+4j.  (w >> 4j) & 0x000F000F
// OR 0x43004300 is the bf16 pair (128+n_even, 128+n_odd); subtracting 136 gives the exact values.
__device__ __forceinline__ void q4_pair(uint32_t w, int j, float &e0, float &e1) {
    uint32_t p = ((w >> (4 * j)) & 0x000F000Fu) | 0x43004300u;
    e0 = bf16_lo(p) - 136.f;
    e1 = bf16_hi(p) - 136.f;
}
// Same as a packed bf16 pair (exact: the integers -8..7 are representable).
__device__ __forceinline__ uint32_t q4_pair_bf16(uint32_t w, int j) {
    uint32_t p = ((w >> (4 * j)) & 0x000F000Fu) | 0x43004300u;
    bf162 v = *reinterpret_cast<bf162 *>(&p);
    bf162 off = __floats2bfloat162_rn(136.f, 136.f);
    bf162 r = __hsub2(v, off);
    return *reinterpret_cast<uint32_t *>(&r);
}

// dot of 8 bf16 weights (uint4) with 8 bf16 activations (uint4), fp32 accumulate, fixed order
__device__ __forceinline__ float dot8(const uint4 &w, const uint4 &x, float acc) {
    acc = fmaf(bf16_lo(w.x), bf16_lo(x.x), acc);
    acc = fmaf(bf16_hi(w.x), bf16_hi(x.x), acc);
    acc = fmaf(bf16_lo(w.y), bf16_lo(x.y), acc);
    acc = fmaf(bf16_hi(w.y), bf16_hi(x.y), acc);
    acc = fmaf(bf16_lo(w.z), bf16_lo(x.z), acc);
    acc = fmaf(bf16_hi(w.z), bf16_hi(x.z), acc);
    acc = fmaf(bf16_lo(w.w), bf16_lo(x.w), acc);
    acc = fmaf(bf16_hi(w.w), bf16_hi(x.w), acc);
    return acc;
}

// ---- programmatic dependent launch (PDL) -------------------------------------------------
// Every kernel of the decode step is launched with the programmatic-stream-serialization
// attribute.  A kernel first lets its successor start (pdl_trigger), prefetches weights — which
// no kernel writes — and only then waits for its predecessor to finish and flush (pdl_wait)
// before it touches activations.  Every block must reach pdl_wait before it exits: a grid that
// completes without waiting would let its successor run ahead of the grid before it.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

constexpr int NUM_SMS = 148;

// ---- L2 prefetch plan ----------------------------------------------------------------------
// Weights never depend on activations, so every kernel of the decode step starts by asking the L2
// to fetch the weights of the kernels a few tens of MB *ahead* of it in launch order.  HBM then
// streams continuously, decoupled from the chain of short dependent kernels, which find their
// weights in L2.  The runtime computes the ranges (up to three per kernel) and hands them to the
// next launcher through g_pf; a launcher copies g_pf into its kernel's arguments and clears it.
struct PfArgs {
    const char *p[3];
    unsigned long long n[3];
};
extern PfArgs g_pf;          // host side: ranges for the next launch (all zero = none)
inline PfArgs take_pf() {
    PfArgs r = g_pf;
    g_pf = PfArgs{};
    return r;
}

__device__ __forceinline__ void l2_prefetch_bulk(const void *p, unsigned bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

// Every warp of the grid takes 8 KB pieces of the ranges round-robin; lane 0 issues the prefetch.
__device__ __forceinline__ void pf_issue(const PfArgs &pf) {
    if ((threadIdx.x & 31) != 0) return;
    const unsigned CH = 8192;
    const unsigned wpb = (blockDim.x * blockDim.y * blockDim.z) >> 5;
    const unsigned long long bid = blockIdx.x + (unsigned long long)gridDim.x * (blockIdx.y + (unsigned long long)gridDim.y * blockIdx.z);
    const unsigned long long gw = bid * wpb + ((threadIdx.x + blockDim.x * (threadIdx.y + blockDim.y * threadIdx.z)) >> 5);
    const unsigned long long nw = (unsigned long long)gridDim.x * gridDim.y * gridDim.z * wpb;
#pragma unroll
    for (int r = 0; r < 3; ++r) {
        const unsigned long long n = pf.n[r];
        if (!n) continue;
        const unsigned long long nch = (n + CH - 1) / CH;
        for (unsigned long long i = gw; i < nch; i += nw) {
            unsigned long long len = n - i * CH;
            if (len > CH) len = CH;
            len &= ~15ull;
            if (len) l2_prefetch_bulk(pf.p[r] + i * CH, (unsigned)len);
        }
    }
}

// NeoX rotation angle tables: cos/sin for (pos, i) computed in double like the oracle.
__device__ __forceinline__ void rope_cs(int pos, int i, int rope_dim, double theta, float &c, float &s) {
    double inv = pow(theta, -2.0 * double(i) / double(rope_dim));
    double a = double(pos) * inv;
    double sd, cd;
    sincos(a, &sd, &cd);
    c = float(cd);
    s = float(sd);
}

}  // namespace qw
