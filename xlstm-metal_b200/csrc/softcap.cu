// Soft-cap y = cap * tanh(x / cap): one HBM-bound pass, 128-bit accesses.
#include "common.cuh"

namespace xl {

template <typename T, int VEC>
__global__ void __launch_bounds__(256) softcap_kernel(const T *__restrict__ x, T *__restrict__ y, int64_t n,
                                                      float cap, float inv_cap) {
    // 16-byte vectors: VEC = 4 (fp32) or 8 (bf16); grid-stride over vectors, scalar tail.
    const int64_t nvec = n / VEC;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
        float4 a = ld4(x + i * VEC);
        a.x = cap * tanhf(a.x * inv_cap); a.y = cap * tanhf(a.y * inv_cap);
        a.z = cap * tanhf(a.z * inv_cap); a.w = cap * tanhf(a.w * inv_cap);
        if (VEC == 8) {
            float4 b = ld4(x + i * VEC + 4);
            b.x = cap * tanhf(b.x * inv_cap); b.y = cap * tanhf(b.y * inv_cap);
            b.z = cap * tanhf(b.z * inv_cap); b.w = cap * tanhf(b.w * inv_cap);
            st4(y + i * VEC + 4, b);
        }
        st4(y + i * VEC, a);
    }
    for (int64_t i = nvec * VEC + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        Elem<T>::st(y + i, cap * tanhf(Elem<T>::ld(x + i) * inv_cap));
}

template <typename T>
__global__ void softcap_scalar_kernel(const T *__restrict__ x, T *__restrict__ y, int64_t n, float cap, float inv_cap) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        Elem<T>::st(y + i, cap * tanhf(Elem<T>::ld(x + i) * inv_cap));
}

template <typename T, int VEC>
static int softcap_launch(const void *x, void *y, int64_t n, float cap, cudaStream_t st) {
    const T *xp = static_cast<const T *>(x);
    T *yp = static_cast<T *>(y);
    // 148 SMs x 8 resident CTAs of 256 threads; fewer when the tensor is small
    int64_t want = (n / VEC + 255) / 256;
    int grid = (int)(want < 1 ? 1 : (want > 148 * 8 ? 148 * 8 : want));
    const bool aligned = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15u) == 0;
    if (aligned)
        softcap_kernel<T, VEC><<<grid, 256, 0, st>>>(xp, yp, n, cap, 1.0f / cap);
    else
        softcap_scalar_kernel<T><<<grid, 256, 0, st>>>(xp, yp, n, cap, 1.0f / cap);
    return launch_status();
}

}  // namespace xl

extern "C" int xlstm_softcap(const void *x, void *y, int64_t n, float cap, int dtype, void *stream) {
    if (n < 0 || (n > 0 && (!x || !y))) return XLSTM_ERR_INVALID;
    if (dtype != XLSTM_F32 && dtype != XLSTM_BF16) return XLSTM_ERR_UNSUPPORTED;
    if (n == 0) return XLSTM_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (!(cap > 0.0f)) {  // identity, as the reference cell does for cap <= 0
        if (x != y) {
            size_t bytes = (size_t)n * (dtype == XLSTM_F32 ? 4 : 2);
            if (cudaMemcpyAsync(y, x, bytes, cudaMemcpyDeviceToDevice, st) != cudaSuccess) return XLSTM_ERR_CUDA;
        }
        return XLSTM_OK;
    }
    return dtype == XLSTM_F32 ? xl::softcap_launch<float, 4>(x, y, n, cap, st)
                              : xl::softcap_launch<__nv_bfloat16, 8>(x, y, n, cap, st);
}
