// Copy helpers of the host tier (prefix-cache blocks, snapshots, slot copies): a block's payload is many
// separate pieces of slot state - per layer a K page, a V page and the compressed keys of the page - that
// have to become one contiguous buffer (export) or be filled from one (import).  One launch moves all
// pieces; the contiguous side is a staging buffer on the device that a single asynchronous copy then
// moves to or from a pinned unit of host memory, or mapped host memory that the kernel addresses itself.
// (Role of the reference's src/engine/host_tier.hip:56-119: export_kv / import_kv into pinned units.)
#include "common.cuh"

namespace qw {

// grid (blocks, segments), 256 threads.  Segment i: bytes[i] bytes (a multiple of 16) from src[i] to dst[i].
__global__ void __launch_bounds__(256) segments_copy_kernel(const void *const *src, void *const *dst, const long long *bytes) {
    const int i = blockIdx.y;
    const uint4 *s = reinterpret_cast<const uint4 *>(src[i]);
    uint4 *d = reinterpret_cast<uint4 *>(dst[i]);
    const long long n = bytes[i] >> 4;
    for (long long j = (long long)blockIdx.x * blockDim.x + threadIdx.x; j < n; j += (long long)gridDim.x * blockDim.x) d[j] = s[j];
}

}  // namespace qw

using namespace qw;

// src / dst / bytes: device arrays of n entries (addresses 16-byte aligned, sizes multiples of 16).
QW_API int qwk_segments_copy(const void *src, const void *dst, const long long *bytes, int n, cudaStream_t s) {
    if (n <= 0) return 0;
    segments_copy_kernel<<<dim3(16, n), 256, 0, s>>>((const void *const *)src, (void *const *)dst, bytes);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// One asynchronous copy (kind: 1 host -> device, 2 device -> host, 3 device -> device); host memory should be pinned.
QW_API int qwk_memcpy_async(void *dst, const void *src, long long bytes, int kind, cudaStream_t s) {
    const cudaMemcpyKind k = kind == 1 ? cudaMemcpyHostToDevice : kind == 2 ? cudaMemcpyDeviceToHost : cudaMemcpyDeviceToDevice;
    return cudaMemcpyAsync(dst, src, (size_t)bytes, k, s) == cudaSuccess ? 0 : -2;
}
