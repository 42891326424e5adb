// Micro-benchmarks of launch mechanics (role of the reference's bench/graph_launch_bench.hip):
// a chain of dependent, nearly empty kernels, launched plainly or with programmatic dependent
// launch, to measure the cost of one kernel boundary inside a CUDA graph on this machine.
#include "common.cuh"

namespace qw {

__global__ void bench_touch_kernel(float *p, int pdl) {
    if (pdl) {
        pdl_wait();
        pdl_trigger();
    }
    if (threadIdx.x == 0) p[blockIdx.x] += 1.f;
}

}  // namespace qw

using namespace qw;

// Enqueues n dependent launches of a tiny kernel (grid blocks x 128 threads) on s.
QW_API int qwk_bench_chain(float *p, int n, int blocks, int pdl, cudaStream_t s) {
    for (int i = 0; i < n; ++i) {
        if (pdl) {
            if (launch_pdl(bench_touch_kernel, dim3(blocks), dim3(128), 0, s, p, 1) != cudaSuccess) return -2;
        } else {
            bench_touch_kernel<<<blocks, 128, 0, s>>>(p, 0);
        }
    }
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
