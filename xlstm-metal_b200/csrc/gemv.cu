// Single-token projections: y[m] = epilogue(W . norm(x[m]) + bias) for M <= 4 rows of x, bf16 weights.
// At one token per sequence a Linear layer is a weight-streaming pass (2 bytes of W per multiply-add), so
// it is written as one: a warp per output row reads the row with 16-byte loads (512 contiguous bytes per
// warp and trip, four trips in flight), x sits in shared memory, fp32 accumulation, one warp reduction
// per row.  What a separate kernel would do before or after is folded in:
//   prologue  RMSNorm of x (every CTA recomputes the 1/rms of the few rows: 8 KB from L2),
//   epilogue  + bias, + residual (the block's residual stream), or silu(gate) * up when W holds the two
//             FFN up projections (gate rows first): the SwiGLU gate without the [M, 2F] intermediate.
// The weights are the one operand the kernel before this one cannot have written, so every warp asks L2 for the
// head of its first weight row BEFORE it waits for that kernel (programmatic dependent launch): in a decode loop
// the weight stream of layer i+1 starts under the tail of layer i and the norm prologue, at no cost in registers.
#include "common.cuh"

namespace xl {
namespace {

constexpr int GV_THREADS = 256;
constexpr int GV_MAXM = 4;

__device__ __forceinline__ void unpack8(const uint4 &u, float *f) {
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

// dot products of one weight row with the M rows of x held in shared memory (bf16, [M][K])
template <int M>
__device__ __forceinline__ void row_dot(const __nv_bfloat16 *__restrict__ wrow, const __nv_bfloat16 *sx, int K, int lane,
                                        float (&acc)[M]) {
#pragma unroll
    for (int m = 0; m < M; ++m) acc[m] = 0.f;
    const int nvec = K >> 3;
    const uint4 *wv = reinterpret_cast<const uint4 *>(wrow);
    int v = lane;
    for (; v + 224 < nvec; v += 256) {         // eight 16-byte loads of the row in flight
        uint4 w8[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) w8[u] = wv[v + 32 * u];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            float wf[8];
            unpack8(w8[u], wf);
#pragma unroll
            for (int m = 0; m < M; ++m) {
                float xf[8];
                unpack8(*reinterpret_cast<const uint4 *>(sx + (size_t)m * K + (size_t)(v + 32 * u) * 8), xf);
#pragma unroll
                for (int e = 0; e < 8; ++e) acc[m] = fmaf(wf[e], xf[e], acc[m]);
            }
        }
    }
    for (; v + 96 < nvec; v += 128) {          // four 16-byte loads of the row in flight
        uint4 w4[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) w4[u] = wv[v + 32 * u];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            float wf[8];
            unpack8(w4[u], wf);
#pragma unroll
            for (int m = 0; m < M; ++m) {
                float xf[8];
                unpack8(*reinterpret_cast<const uint4 *>(sx + (size_t)m * K + (size_t)(v + 32 * u) * 8), xf);
#pragma unroll
                for (int e = 0; e < 8; ++e) acc[m] = fmaf(wf[e], xf[e], acc[m]);
            }
        }
    }
    for (; v < nvec; v += 32) {
        float wf[8];
        unpack8(wv[v], wf);
#pragma unroll
        for (int m = 0; m < M; ++m) {
            float xf[8];
            unpack8(*reinterpret_cast<const uint4 *>(sx + (size_t)m * K + (size_t)v * 8), xf);
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[m] = fmaf(wf[e], xf[e], acc[m]);
        }
    }
#pragma unroll
    for (int m = 0; m < M; ++m) acc[m] = warp_sum(acc[m]);
}

// EPI: 0 = bias only, 1 = + residual, 2 = SwiGLU pair (W has 2 N rows: gate rows, then up rows)
template <int M, int EPI>
__global__ void __launch_bounds__(GV_THREADS) gemv_kernel(const __nv_bfloat16 *__restrict__ W,
                                                          const __nv_bfloat16 *__restrict__ x,
                                                          const __nv_bfloat16 *__restrict__ bias,
                                                          const __nv_bfloat16 *__restrict__ norm_w, float norm_eps,
                                                          const __nv_bfloat16 *__restrict__ residual,
                                                          __nv_bfloat16 *__restrict__ y, int N, int K) {
    extern __shared__ __align__(16) unsigned char gv_smem[];
    const __nv_bfloat16 *sx = reinterpret_cast<const __nv_bfloat16 *>(gv_smem);   // [M][K] normalised rows
    __shared__ float s_part[M][GV_THREADS / 32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nvec = K >> 3;
    const int total_warps = gridDim.x * (GV_THREADS / 32);
    const int n_first = blockIdx.x * (GV_THREADS / 32) + warp;

    // ---- L2 prefetch of the head of this warp's first weight row (4 KB: what the first loads will ask for; more
    //      would only push the running kernel's lines out of L2), then the wait for the preceding kernel
    if (n_first < N) {
        const char *row = reinterpret_cast<const char *>(W + (size_t)n_first * K);
        const int head = K * 2 < 4096 ? K * 2 : 4096;
        if (lane * 128 < head) asm volatile("prefetch.global.L2 [%0];" ::"l"(row + lane * 128));
    }
    grid_dependency_wait();
    allow_dependents();

    // ---- x into shared memory, normalised on the way when a norm weight is given
    if (norm_w) {
        float ss[M];
#pragma unroll
        for (int m = 0; m < M; ++m) ss[m] = 0.f;
        for (int v = tid; v < nvec; v += GV_THREADS)
#pragma unroll
            for (int m = 0; m < M; ++m) {
                float xf[8];
                unpack8(*reinterpret_cast<const uint4 *>(x + (size_t)m * K + (size_t)v * 8), xf);
#pragma unroll
                for (int e = 0; e < 8; ++e) ss[m] = fmaf(xf[e], xf[e], ss[m]);
            }
#pragma unroll
        for (int m = 0; m < M; ++m) {
            ss[m] = warp_sum(ss[m]);
            if (lane == 0) s_part[m][warp] = ss[m];
        }
        __syncthreads();
        float inv[M];
#pragma unroll
        for (int m = 0; m < M; ++m) {
            float tot = 0.f;
#pragma unroll
            for (int i = 0; i < GV_THREADS / 32; ++i) tot += s_part[m][i];
            inv[m] = rsqrtf(tot / (float)K + norm_eps);
        }
        for (int v = tid; v < nvec; v += GV_THREADS) {
            float wf[8];
            unpack8(*reinterpret_cast<const uint4 *>(norm_w + (size_t)v * 8), wf);
#pragma unroll
            for (int m = 0; m < M; ++m) {
                float xf[8];
                unpack8(*reinterpret_cast<const uint4 *>(x + (size_t)m * K + (size_t)v * 8), xf);
                uint32_t o[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {   // rounded to bf16, as the stand-alone norm kernel hands it to the GEMM
                    __nv_bfloat162 pk = __floats2bfloat162_rn(xf[2 * e] * inv[m] * wf[2 * e], xf[2 * e + 1] * inv[m] * wf[2 * e + 1]);
                    o[e] = *reinterpret_cast<uint32_t *>(&pk);
                }
                *reinterpret_cast<uint4 *>(gv_smem + ((size_t)m * K + (size_t)v * 8) * 2) = make_uint4(o[0], o[1], o[2], o[3]);
            }
        }
        __syncthreads();
    } else {
        sx = const_cast<__nv_bfloat16 *>(x);   // nothing to prepare: the rows are read through L1 as they are
    }

    // ---- one warp per output row (per gate/up pair for the SwiGLU epilogue), rows by grid stride
    for (int n = n_first; n < N; n += total_warps) {
        float acc[M];
        row_dot<M>(W + (size_t)n * K, sx, K, lane, acc);
        if (EPI == 2) {
            float up[M];
            row_dot<M>(W + (size_t)(n + N) * K, sx, K, lane, up);
            if (lane == 0) {
                const float bg = bias ? __bfloat162float(bias[n]) : 0.f, bu = bias ? __bfloat162float(bias[n + N]) : 0.f;
#pragma unroll
                for (int m = 0; m < M; ++m) {
                    // the two projections are rounded to bf16 before the gate, as separate GEMM outputs would be
                    const float g = __bfloat162float(__float2bfloat16_rn(acc[m] + bg));
                    const float u = __bfloat162float(__float2bfloat16_rn(up[m] + bu));
                    y[(size_t)m * N + n] = __float2bfloat16_rn(g / (1.0f + expf(-g)) * u);
                }
            }
        } else if (lane == 0) {
            const float b = bias ? __bfloat162float(bias[n]) : 0.f;
#pragma unroll
            for (int m = 0; m < M; ++m) {
                float v = acc[m] + b;
                if (EPI == 1) v = __bfloat162float(__float2bfloat16_rn(v)) + __bfloat162float(residual[(size_t)m * N + n]);
                y[(size_t)m * N + n] = __float2bfloat16_rn(v);
            }
        }
    }
}

template <int M, int EPI>
int gemv_launch(const void *W, const void *x, const void *bias, const void *norm_w, float eps, const void *residual, void *y,
                int N, int K, cudaStream_t st) {
    auto kern = gemv_kernel<M, EPI>;
    const size_t smem = (size_t)M * K * sizeof(__nv_bfloat16);
    if (smem > 200 * 1024) return XLSTM_ERR_UNSUPPORTED;
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return XLSTM_ERR_CUDA;
    // rows are spread over all SMs: enough CTAs of 8 warps for one row per warp, at most 8 CTAs per SM
    const int want = (N + GV_THREADS / 32 - 1) / (GV_THREADS / 32);
    const int grid = want < 148 * 8 ? want : 148 * 8;
    return launch_overlapped(kern, dim3(grid), dim3(GV_THREADS), smem, st, static_cast<const __nv_bfloat16 *>(W),
                             static_cast<const __nv_bfloat16 *>(x), static_cast<const __nv_bfloat16 *>(bias),
                             static_cast<const __nv_bfloat16 *>(norm_w), eps, static_cast<const __nv_bfloat16 *>(residual),
                             static_cast<__nv_bfloat16 *>(y), N, K);
}

template <int M>
int gemv_epi(int epi, const void *W, const void *x, const void *bias, const void *norm_w, float eps, const void *residual,
             void *y, int N, int K, cudaStream_t st) {
    switch (epi) {
        case 0: return gemv_launch<M, 0>(W, x, bias, norm_w, eps, residual, y, N, K, st);
        case 1: return gemv_launch<M, 1>(W, x, bias, norm_w, eps, residual, y, N, K, st);
        case 2: return gemv_launch<M, 2>(W, x, bias, norm_w, eps, residual, y, N, K, st);
        default: return XLSTM_ERR_INVALID;
    }
}

}  // namespace
}  // namespace xl

extern "C" int xlstm_linear_token(const void *W, const void *x, const void *bias, const void *norm_w, float norm_eps,
                                  const void *residual, void *y, int M, int N, int K, int epilogue, int dtype,
                                  void *stream) {
    if (M <= 0 || N <= 0 || K <= 0 || !W || !x || !y) return XLSTM_ERR_INVALID;
    if (epilogue < 0 || epilogue > 2 || (epilogue == 1 && !residual)) return XLSTM_ERR_INVALID;
    if (dtype != XLSTM_BF16 || M > xl::GV_MAXM || K % 8) return XLSTM_ERR_UNSUPPORTED;
    const uintptr_t al = reinterpret_cast<uintptr_t>(W) | reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(norm_w);
    if (al & 15u) return XLSTM_ERR_UNSUPPORTED;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (M) {
        case 1: return xl::gemv_epi<1>(epilogue, W, x, bias, norm_w, norm_eps, residual, y, N, K, st);
        case 2: return xl::gemv_epi<2>(epilogue, W, x, bias, norm_w, norm_eps, residual, y, N, K, st);
        case 3: return xl::gemv_epi<3>(epilogue, W, x, bias, norm_w, norm_eps, residual, y, N, K, st);
        default: return xl::gemv_epi<4>(epilogue, W, x, bias, norm_w, norm_eps, residual, y, N, K, st);
    }
}
