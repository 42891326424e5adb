// An entry point for callers that cannot allocate device memory.
//
// This function has no counterpart in the reference engine; it was added on request.
//
// Who needs it: a host that hands the library fully laid-out device buffers and must not see the library
// (or anything it calls) reserve or release device memory while it runs - for example a process whose
// whole device heap is owned by another allocator, or a real-time loop that cannot tolerate the implicit
// synchronisation of an allocation.  qwk_moe_router (kernels.h) already allocates nothing itself, but it
// needs two caller-provided scratch buffers: the router outputs `rs` [M][nrs] fp32 and one zeroed
// `ticket` word.  A caller with no allocator has nowhere to take those from.  qwk_moe_router_static
// does the same launch with both held in a fixed array compiled into the library's device image.
//
// What it computes: exactly what qwk_moe_router computes with the expert-prefetch arguments null -
// rs = Wrs . x for every row, then the top_k expert choice with normalised weights for each row
// (pair_expert, pair_w; experts outside [e_first, e_first + e_local) are reported as -1) and, when sh_h
// is not null, the gated shared-expert activation [M][F] in bf16.  Same kernel, same results bit for bit.
//
// Limits: M <= QWK_ROUTER_STATIC_MAX_ROWS rows and nrs <= QWK_ROUTER_STATIC_MAX_OUTPUTS outputs per row
// (the scratch is 256 + 32 * 4096 * 4 bytes = 524,544 bytes per device).  Larger shapes are refused with
// -4 and nothing is launched; use qwk_moe_router with your own buffers for those.
//
// Set-up: the array's device address is looked up once per device with cudaGetSymbolAddress, with that
// device current.  qwk_moe_router_static_setup() does it explicitly; otherwise the first call of
// qwk_moe_router_static on a device does it.  Do the set-up (or that first call) before any stream capture
// begins on the device.  Neither function calls cudaMalloc, cudaFree or any other allocating routine.
//
// Sharing: all calls on one device use the same array.  Calls enqueued on one stream are ordered and
// safe.  Calls whose launches can overlap (different streams without a dependency, or different host
// threads on different streams) race on the scratch and on the ticket and give wrong results: serialise
// them.  Only the ticket word must be zero when the kernel starts; each call clears it on the stream
// before the launch and the kernel leaves it at zero, the rest of the scratch is written before it is
// read.  The results are in the caller's own buffers, so they stay valid after the next call.
//
// Like qwk_moe_router, a call takes the library's one-shot launch options that a caller of the step runtime may
// have armed for "the next launch" (weight prefetch ranges, balance counters); callers of this entry point alone
// never arm any.
//
// Return values: 0 enqueued; -1 unsupported shape (as qwk_moe_router; also nrs < E, or < E + 1 + 2 F with sh_h); -2 launch error; -3 set-up failed
// (no current device, device index >= QWK_ROUTER_STATIC_MAX_DEVICES, or the symbol lookup failed);
// -4 M or nrs beyond the limits above.
#pragma once
#include <cuda_runtime.h>

#define QWK_ROUTER_STATIC_MAX_ROWS 32
#define QWK_ROUTER_STATIC_MAX_OUTPUTS 4096
#define QWK_ROUTER_STATIC_MAX_DEVICES 64
#define QWK_ROUTER_STATIC_SCRATCH_BYTES (256 + QWK_ROUTER_STATIC_MAX_ROWS * QWK_ROUTER_STATIC_MAX_OUTPUTS * 4)

#ifdef __cplusplus
extern "C" {
#endif

int qwk_moe_router_static_setup(void);

int qwk_moe_router_static(const void *Wrs, const void *x, int nrs, int K, int M, int ldx, int E, int top_k, int F,
                          int e_first, int e_local, int *pair_expert, float *pair_w, void *sh_h, cudaStream_t s);

#ifdef __cplusplus
}
#endif
