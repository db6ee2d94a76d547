// Test helper (not part of the library): the bounded mbarrier wait of csrc/tcgen05.cuh, built with a small
// time limit (2^22 SM clocks, ~2 ms), on a barrier that nobody ever arrives at.  The wait must give up, raise the CTA's abort flag and
// let the kernel end normally - the path the tensor-core kernels take when a device-side wait times out.
// Nothing here faults, traps or spins without bound.
#define XL_TC_WAIT_CLOCKS (1ll << 22)
#include "tcgen05.cuh"

namespace {

__global__ void timeout_probe_kernel(int *out) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        xl::tc::mbar_init(&bar, 1);
        xl::tc::mbar_fence_init();
    }
    __syncthreads();
    const bool ok = xl::tc::mbar_wait(&bar, 0, &abort_flag);      // no arrival will ever come
    const bool ok2 = xl::tc::mbar_wait(&bar, 0, &abort_flag);     // a second role sees the abort flag and leaves too
    __syncthreads();
    if (threadIdx.x == 0) {
        out[0] = ok ? 1 : 0;
        out[1] = ok2 ? 1 : 0;
        out[2] = abort_flag;
    }
}

}  // namespace

// returns 0 and fills host_out[3] = {first wait succeeded, second wait succeeded, abort flag}; -1 on a CUDA error
extern "C" int timeout_probe_run(int *host_out) {
    int *d = nullptr;
    if (cudaMalloc(&d, 3 * sizeof(int)) != cudaSuccess) return -1;
    timeout_probe_kernel<<<1, 64>>>(d);
    int rc = 0;
    if (cudaGetLastError() != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess ||
        cudaMemcpy(host_out, d, 3 * sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess)
        rc = -1;
    cudaFree(d);
    return rc;
}
