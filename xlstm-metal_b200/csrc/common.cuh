// Shared device/host helpers for the xLSTM kernels (sm_100a).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "xlstm_cuda.h"

namespace xl {

// ---- element types ------------------------------------------------------
template <typename T> struct Elem;
template <> struct Elem<float> {
    static __device__ __forceinline__ float ld(const float *p) { return *p; }
    static __device__ __forceinline__ void st(float *p, float v) { *p = v; }
};
template <> struct Elem<__nv_bfloat16> {
    static __device__ __forceinline__ float ld(const __nv_bfloat16 *p) { return __bfloat162float(*p); }
    static __device__ __forceinline__ void st(__nv_bfloat16 *p, float v) { *p = __float2bfloat16_rn(v); }
};

// four consecutive elements <-> float4 (pointer must be aligned to 4 elements)
__device__ __forceinline__ float4 ld4(const float *p) { return *reinterpret_cast<const float4 *>(p); }
__device__ __forceinline__ float4 ld4(const __nv_bfloat16 *p) {
    uint2 u = *reinterpret_cast<const uint2 *>(p);
    __nv_bfloat162 a = *reinterpret_cast<__nv_bfloat162 *>(&u.x);
    __nv_bfloat162 b = *reinterpret_cast<__nv_bfloat162 *>(&u.y);
    float2 fa = __bfloat1622float2(a), fb = __bfloat1622float2(b);
    return make_float4(fa.x, fa.y, fb.x, fb.y);
}
__device__ __forceinline__ void st4(float *p, float4 v) { *reinterpret_cast<float4 *>(p) = v; }
__device__ __forceinline__ void st4(__nv_bfloat16 *p, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y);
    __nv_bfloat162 b = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<uint32_t *>(&a);
    u.y = *reinterpret_cast<uint32_t *>(&b);
    *reinterpret_cast<uint2 *>(p) = u;
}

// ---- math -----------------------------------------------------------------
// log(sigmoid(x)) in the branch-free stable form; equal to -log(1+exp(-x)) to
// fp32 rounding on the soft-capped range |x| <= 15 and finite everywhere.
__device__ __forceinline__ float logsigmoid(float x) { return fminf(x, 0.0f) - log1pf(expf(-fabsf(x))); }
__device__ __forceinline__ float sigmoidf(float x) { return 1.0f / (1.0f + expf(-x)); }
// sigmoid of an output-gate pre-activation: bf16 outputs take it from ONE special-function op (tanh.approx, relative
// error 2^-11, below the bf16 rounding), fp32 outputs the exact form
template <typename T> __device__ __forceinline__ float gate_sigmoid(float x) {
    if (sizeof(T) == 2) {
        float t;
        asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * x));
        return fmaf(0.5f, t, 0.5f);
    }
    return 1.0f / (1.0f + expf(-x));
}
// gate soft-cap folded into the kernels that consume the gates: cap <= 0 leaves x as it is
__device__ __forceinline__ float gate_softcap(float x, float cap) { return cap > 0.0f ? cap * tanhf(x / cap) : x; }

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

// streaming (evict-first) 128-bit global accesses for data touched once
__device__ __forceinline__ float4 ldg_stream(const float *p) {
    float4 v;
    asm volatile("ld.global.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void stg_stream(float *p, float4 v) {
    asm volatile("st.global.L1::no_allocate.v4.f32 [%0], {%1,%2,%3,%4};"
                 :: "l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

inline int launch_status() { return cudaGetLastError() == cudaSuccess ? XLSTM_OK : XLSTM_ERR_CUDA; }

// ---- programmatic dependent launch ---------------------------------------------------
// A kernel launched with launch_overlapped() may become resident while the kernel before it in the stream is
// still draining.  Inside such a kernel everything BEFORE grid_dependency_wait() may only read memory that the
// preceding kernel does not write (weights, a state written by an earlier launch); the wait returns once that
// kernel has completed and its writes are visible.  allow_dependents() is issued right AFTER the wait, so the
// pre-wait part of launch k+1 can only ever overlap launch k, never anything older.  Both instructions do
// nothing in a kernel launched the ordinary way, or after a stream operation that is not such a kernel.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void allow_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline int launch_overlapped(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...) == cudaSuccess ? launch_status() : XLSTM_ERR_CUDA;
}

}  // namespace xl
