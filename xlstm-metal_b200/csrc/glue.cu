// The elementwise / row-reduction kernels on either side of the recurrent cells: RMSNorm, the mLSTM
// output epilogue (per-head RMS norm x weight x sigmoid(output gate)), the SwiGLU gate and the causal
// depthwise convolution of the sLSTM projection.  All are single-pass and HBM-bound: every input is
// read once with 16-byte accesses, reductions and math in fp32, one rounding on the way out.
// Two forms each: register-resident kernels for few rows (decode), and for many rows (prefill) STREAMED
// kernels - one CTA of 16 warps per SM, inputs arriving through per-lane rings of 16-byte cp.async slots in
// shared memory a fixed distance ahead, so the bytes in flight do not depend on the register allocation.
#include "common.cuh"

namespace xl {

template <typename T> struct Vec16 { static constexpr int N = 16 / sizeof(T); };

template <typename T> __device__ __forceinline__ void ld16(const T *p, float *f);
template <> __device__ __forceinline__ void ld16<float>(const float *p, float *f) {
    const float4 a = *reinterpret_cast<const float4 *>(p);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
}
template <> __device__ __forceinline__ void ld16<__nv_bfloat16>(const __nv_bfloat16 *p, float *f) {
    const uint4 u = *reinterpret_cast<const uint4 *>(p);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}
template <typename T> __device__ __forceinline__ void st16(T *p, const float *f);
template <> __device__ __forceinline__ void st16<float>(float *p, const float *f) {
    *reinterpret_cast<float4 *>(p) = make_float4(f[0], f[1], f[2], f[3]);
}
template <> __device__ __forceinline__ void st16<__nv_bfloat16>(__nv_bfloat16 *p, const float *f) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        __nv_bfloat162 v = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
        w[i] = *reinterpret_cast<uint32_t *>(&v);
    }
    *reinterpret_cast<uint4 *>(p) = make_uint4(w[0], w[1], w[2], w[3]);
}

// 16 raw bytes already in registers -> VN floats
template <typename T> __device__ __forceinline__ void unpack16(const uint4 &u, float *f);
template <> __device__ __forceinline__ void unpack16<float>(const uint4 &u, float *f) {
    f[0] = __uint_as_float(u.x); f[1] = __uint_as_float(u.y); f[2] = __uint_as_float(u.z); f[3] = __uint_as_float(u.w);
}
template <> __device__ __forceinline__ void unpack16<__nv_bfloat16>(const uint4 &u, float *f) {
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

// sigmoid / SiLU: exact division and expf for fp32 outputs; for bf16 outputs (8 elements per 16 bytes,
// where these kernels would otherwise be bound by instruction issue, not by HBM) the approximate
// exp / reciprocal, whose ~2 ulp fp32 error disappears in the bf16 rounding
template <typename T> __device__ __forceinline__ float sigmoid_t(float x) {
    if (sizeof(T) == 2) return __fdividef(1.0f, 1.0f + __expf(-x));
    return 1.0f / (1.0f + expf(-x));
}
template <typename T> __device__ __forceinline__ float silu_t(float x) {
    if (sizeof(T) == 2) return __fdividef(x, 1.0f + __expf(-x));
    return x / (1.0f + expf(-x));
}

// 16-byte asynchronous copies global -> shared memory; a thread that only ever reads back the slots it filled
// itself needs no barrier, only the wait on its own copy groups
__device__ __forceinline__ void cp_async16(void *smem_dst, const void *gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;"
                 :: "r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" :: "n"(N) : "memory"); }

// ---------------------------------------------------------------------------
// RMSNorm: one CTA per row, the row cached in registers (NV 16-byte vectors per thread)
// ---------------------------------------------------------------------------
constexpr int RN_THREADS = 128;

// With a residual r: s = x + r is rounded to the activation type, written to `sum` (the new residual
// stream) and the norm is taken of that rounded value, exactly as two separate ops would.
template <typename T, int NV>
__global__ void __launch_bounds__(RN_THREADS) rms_norm_kernel(const T *__restrict__ x, const T *__restrict__ r,
                                                              const T *__restrict__ w, T *__restrict__ sum,
                                                              T *__restrict__ y, int64_t rows, int cols, float eps) {
    constexpr int VN = Vec16<T>::N;
    __shared__ float s_part[2][RN_THREADS / 32];
    const int nvec = cols / VN;
    int par = 0;
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x, par ^= 1) {
    const T *xr = x + (size_t)row * cols;
    T *yr = y + (size_t)row * cols;
    float v[NV][VN];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int iv = threadIdx.x + i * RN_THREADS;
        if (iv < nvec) {
            ld16<T>(xr + (size_t)iv * VN, v[i]);
            if (r) {
                float rv[VN];
                ld16<T>(r + (size_t)row * cols + (size_t)iv * VN, rv);
#pragma unroll
                for (int e = 0; e < VN; ++e) v[i][e] += rv[e];
                st16<T>(sum + (size_t)row * cols + (size_t)iv * VN, v[i]);
                if (sizeof(T) == 2) {
#pragma unroll
                    for (int e = 0; e < VN; ++e) v[i][e] = __bfloat162float(__float2bfloat16_rn(v[i][e]));
                }
            }
#pragma unroll
            for (int e = 0; e < VN; ++e) ss += v[i][e] * v[i][e];
        }
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) s_part[par][threadIdx.x >> 5] = ss;   // two buffers: one barrier per row
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < RN_THREADS / 32; ++i) tot += s_part[par][i];
    const float inv = rsqrtf(tot / (float)cols + eps);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int iv = threadIdx.x + i * RN_THREADS;
        if (iv < nvec) {
            float wv[VN];
            if (w) ld16<T>(w + (size_t)iv * VN, wv);
#pragma unroll
            for (int e = 0; e < VN; ++e) v[i][e] = v[i][e] * inv * (w ? wv[e] : 1.0f);
            st16<T>(yr + (size_t)iv * VN, v[i]);
        }
    }
    }
}

// any width / alignment: two passes over the row (the second one hits L1/L2)
template <typename T>
__global__ void __launch_bounds__(RN_THREADS) rms_norm_generic_kernel(const T *__restrict__ x, const T *__restrict__ r,
                                                                      const T *__restrict__ w, T *__restrict__ sum,
                                                                      T *__restrict__ y, int cols, float eps) {
    __shared__ float s_part[RN_THREADS / 32];
    const T *xr = x + (size_t)blockIdx.x * cols;
    T *yr = y + (size_t)blockIdx.x * cols;
    float ss = 0.f;
    if (r) {   // first pass also forms the new residual stream; later passes read it back
        T *sr = sum + (size_t)blockIdx.x * cols;
        for (int i = threadIdx.x; i < cols; i += RN_THREADS)
            Elem<T>::st(sr + i, Elem<T>::ld(xr + i) + Elem<T>::ld(r + (size_t)blockIdx.x * cols + i));
        __syncthreads();
        xr = sr;
    }
    for (int i = threadIdx.x; i < cols; i += RN_THREADS) { const float a = Elem<T>::ld(xr + i); ss += a * a; }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
    for (int i = 0; i < RN_THREADS / 32; ++i) tot += s_part[i];
    const float inv = rsqrtf(tot / (float)cols + eps);
    for (int i = threadIdx.x; i < cols; i += RN_THREADS)
        Elem<T>::st(yr + i, Elem<T>::ld(xr + i) * inv * (w ? Elem<T>::ld(w + i) : 1.0f));
}

// Many rows: one WARP per row, the row kept as packed 16-byte vectors in registers (NV per lane), no
// CTA barrier, rows by grid stride.  All NV loads of a row are in flight at once.
constexpr int RW_WARPS = 8;

template <typename T, int NV>
__global__ void __launch_bounds__(RW_WARPS * 32) rms_norm_warp_kernel(const T *__restrict__ x, const T *__restrict__ r,
                                                                     const T *__restrict__ w, T *__restrict__ sum,
                                                                     T *__restrict__ y, int64_t rows, int cols, float eps) {
    constexpr int VN = Vec16<T>::N;
    const int lane = threadIdx.x & 31;
    const int nvec = cols / VN;
    for (int64_t row = (int64_t)blockIdx.x * RW_WARPS + (threadIdx.x >> 5); row < rows; row += (int64_t)gridDim.x * RW_WARPS) {
        const uint4 *xr = reinterpret_cast<const uint4 *>(x + (size_t)row * cols);
        uint4 raw[NV];
#pragma unroll
        for (int i = 0; i < NV; ++i)
            if (lane + 32 * i < nvec) raw[i] = xr[lane + 32 * i];
        if (r) {   // residual add: s = x + r rounded to the activation type, written as the new residual stream
            const uint4 *rr = reinterpret_cast<const uint4 *>(r + (size_t)row * cols);
            uint4 *sr = reinterpret_cast<uint4 *>(sum + (size_t)row * cols);
#pragma unroll
            for (int i = 0; i < NV; ++i)
                if (lane + 32 * i < nvec) {
                    float a[VN], b[VN];
                    unpack16<T>(raw[i], a);
                    unpack16<T>(rr[lane + 32 * i], b);
#pragma unroll
                    for (int e = 0; e < VN; ++e) a[e] += b[e];
                    st16<T>(reinterpret_cast<T *>(&raw[i]), a);
                    sr[lane + 32 * i] = raw[i];
                }
        }
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i)
            if (lane + 32 * i < nvec) {
                float a[VN];
                unpack16<T>(raw[i], a);
#pragma unroll
                for (int e = 0; e < VN; ++e) ss = fmaf(a[e], a[e], ss);
            }
        ss = warp_sum(ss);
        const float inv = rsqrtf(ss / (float)cols + eps);
        uint4 *yr = reinterpret_cast<uint4 *>(y + (size_t)row * cols);
#pragma unroll
        for (int i = 0; i < NV; ++i)
            if (lane + 32 * i < nvec) {
                float a[VN], wv[VN];
                unpack16<T>(raw[i], a);
                if (w) ld16<T>(w + (size_t)(lane + 32 * i) * VN, wv);
#pragma unroll
                for (int e = 0; e < VN; ++e) a[e] = a[e] * inv * (w ? wv[e] : 1.0f);
                uint4 o;
                st16<T>(reinterpret_cast<T *>(&o), a);
                yr[lane + 32 * i] = o;
            }
    }
}

// Residual add + RMSNorm over many rows, as a stream: one warp per row, 16 warps per CTA, one CTA per SM (with 8
// warps the kernel was bound by instruction issue: two warps per scheduler cannot hide their own dependent
// instructions).  The two input rows (x and the residual) arrive through a ring of RS_RING chunks per warp in
// shared memory, a chunk being one 16-byte vector of x and one of r per lane (1 KB per warp), filled by cp.async
// RS_RING chunks ahead - across row boundaries - so 192 KB per SM are in flight whatever the registers do.  The sum s = x + r is rounded to the
// activation type, stored as the new residual stream and kept packed in registers for the second pass.
constexpr int RS_WARPS = 16, RS_RING = 12;

template <typename T, int NV>
__global__ void __launch_bounds__(RS_WARPS * 32, 1) add_rms_norm_stream_kernel(const T *__restrict__ x, const T *__restrict__ r,
                                                                              const T *__restrict__ w, T *__restrict__ sum,
                                                                              T *__restrict__ y, int64_t rows, int cols,
                                                                              float eps) {
    constexpr int VN = Vec16<T>::N;
    constexpr int NT = RS_WARPS * 32;
    extern __shared__ __align__(16) unsigned char rs_smem[];
    uint4 *ring = reinterpret_cast<uint4 *>(rs_smem);          // [RS_RING][2][NT]
    const int tid = threadIdx.x, lane = tid & 31;
    const int nvec = cols / VN;
    const int64_t row0 = (int64_t)blockIdx.x * RS_WARPS + (tid >> 5), rstride = (int64_t)gridDim.x * RS_WARPS;
    if (row0 >= rows) return;                                   // no CTA barrier below
    const int my_rows = (int)((rows - row0 + rstride - 1) / rstride);
    // the copy stream runs RS_RING chunks ahead of the compute loop: (a_row, a_i) is the chunk it issues next
    int a_k = 0, a_i = 0;
    size_t a_off = (size_t)row0 * cols;
    auto issue = [&](int slot) {
        if (a_k < my_rows) {
            const int iv = lane + 32 * a_i;
            if (iv < nvec) {
                cp_async16(ring + (size_t)(slot * 2 + 0) * NT + tid, x + a_off + (size_t)iv * VN);
                cp_async16(ring + (size_t)(slot * 2 + 1) * NT + tid, r + a_off + (size_t)iv * VN);
            }
            if (++a_i == NV) {
                a_i = 0;
                ++a_k;
                a_off += (size_t)rstride * cols;
            }
        }
        cp_async_commit();
    };
#pragma unroll 1
    for (int c = 0; c < RS_RING; ++c) issue(c);
    int slot = 0;
    for (int k = 0; k < my_rows; ++k) {
        const size_t off = ((size_t)row0 + (size_t)k * rstride) * cols;
        uint4 keep[NV];
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            cp_async_wait<RS_RING - 1>();                       // the oldest chunk in flight has landed
            const int iv = lane + 32 * i;
            if (iv < nvec) {
                float a[VN], b[VN];
                unpack16<T>(ring[(size_t)(slot * 2 + 0) * NT + tid], a);
                unpack16<T>(ring[(size_t)(slot * 2 + 1) * NT + tid], b);
#pragma unroll
                for (int e = 0; e < VN; ++e) a[e] += b[e];
                st16<T>(reinterpret_cast<T *>(&keep[i]), a);
                *reinterpret_cast<uint4 *>(sum + off + (size_t)iv * VN) = keep[i];
                unpack16<T>(keep[i], a);                        // the norm is taken of the rounded sum
#pragma unroll
                for (int e = 0; e < VN; ++e) ss = fmaf(a[e], a[e], ss);
            }
            issue(slot);                                        // refill the slot just consumed
            slot = slot + 1 == RS_RING ? 0 : slot + 1;
        }
        ss = warp_sum(ss);
        const float inv = rsqrtf(ss / (float)cols + eps);
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int iv = lane + 32 * i;
            if (iv < nvec) {
                float a[VN], wv[VN];
                unpack16<T>(keep[i], a);
                if (w) ld16<T>(w + (size_t)iv * VN, wv);
#pragma unroll
                for (int e = 0; e < VN; ++e) a[e] = a[e] * inv * (w ? wv[e] : 1.0f);
                st16<T>(y + off + (size_t)iv * VN, a);
            }
        }
    }
    cp_async_wait<0>();
}

template <typename T, int NV>
static int add_rms_norm_stream_launch(const T *xp, const T *rp, const T *wp, T *sp, T *yp, int64_t rows, int cols, float eps,
                                      cudaStream_t st) {
    auto kern = add_rms_norm_stream_kernel<T, NV>;
    const size_t smem = (size_t)RS_RING * 2 * RS_WARPS * 32 * sizeof(uint4);
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return XLSTM_ERR_CUDA;
    const int64_t want = (rows + RS_WARPS - 1) / RS_WARPS;
    kern<<<(unsigned)(want < 148 ? want : 148), RS_WARPS * 32, smem, st>>>(xp, rp, wp, sp, yp, rows, cols, eps);
    return launch_status();
}

template <typename T>
static int rms_norm_launch(const void *x, const void *r, const void *w, void *sum, void *y, int64_t rows, int cols,
                           float eps, cudaStream_t st) {
    constexpr int VN = Vec16<T>::N;
    const T *xp = static_cast<const T *>(x), *rp = static_cast<const T *>(r), *wp = static_cast<const T *>(w);
    T *sp = static_cast<T *>(sum), *yp = static_cast<T *>(y);
    const bool aligned = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(w) |
                           reinterpret_cast<uintptr_t>(r) | reinterpret_cast<uintptr_t>(sum)) & 15u) == 0 &&
                         cols % VN == 0;
    const int nvec = cols / VN;
    const dim3 grid((unsigned)rows);
    if (aligned && r && rows >= 8 * 148 && nvec <= 32 * 16) {    // two input streams, many rows: the streamed kernel
        if (nvec <= 32 * 4) return add_rms_norm_stream_launch<T, 4>(xp, rp, wp, sp, yp, rows, cols, eps, st);
        if (nvec <= 32 * 8) return add_rms_norm_stream_launch<T, 8>(xp, rp, wp, sp, yp, rows, cols, eps, st);
        return add_rms_norm_stream_launch<T, 16>(xp, rp, wp, sp, yp, rows, cols, eps, st);
    }
    if (aligned && !r && rows >= 4 * 148 && nvec <= 32 * 16) {   // enough rows to give every SM several warps' worth
        const int64_t want = (rows + RW_WARPS - 1) / RW_WARPS;
        const unsigned wg = (unsigned)(want < 148 * 8 ? want : 148 * 8);
        if (nvec <= 32 * 4) rms_norm_warp_kernel<T, 4><<<wg, RW_WARPS * 32, 0, st>>>(xp, rp, wp, sp, yp, rows, cols, eps);
        else if (nvec <= 32 * 8) rms_norm_warp_kernel<T, 8><<<wg, RW_WARPS * 32, 0, st>>>(xp, rp, wp, sp, yp, rows, cols, eps);
        else rms_norm_warp_kernel<T, 16><<<wg, RW_WARPS * 32, 0, st>>>(xp, rp, wp, sp, yp, rows, cols, eps);
        return launch_status();
    }
    if (aligned && nvec <= RN_THREADS * 1) rms_norm_kernel<T, 1><<<grid, RN_THREADS, 0, st>>>(xp, rp, wp, sp, yp, rows, cols, eps);
    else if (aligned && nvec <= RN_THREADS * 2) rms_norm_kernel<T, 2><<<grid, RN_THREADS, 0, st>>>(xp, rp, wp, sp, yp, rows, cols, eps);
    else if (aligned && nvec <= RN_THREADS * 4) rms_norm_kernel<T, 4><<<grid, RN_THREADS, 0, st>>>(xp, rp, wp, sp, yp, rows, cols, eps);
    else if (aligned && nvec <= RN_THREADS * 8) rms_norm_kernel<T, 8><<<grid, RN_THREADS, 0, st>>>(xp, rp, wp, sp, yp, rows, cols, eps);
    else rms_norm_generic_kernel<T><<<grid, RN_THREADS, 0, st>>>(xp, rp, wp, sp, yp, cols, eps);
    return launch_status();
}

// ---------------------------------------------------------------------------
// mLSTM output epilogue: one warp per (batch, token, head) row of dv values
// ---------------------------------------------------------------------------
constexpr int OG_WARPS = 8;

__device__ __forceinline__ uint4 ldg16_raw(const void *p) { return *reinterpret_cast<const uint4 *>(p); }

template <typename T> __device__ __forceinline__ float og_sigmoid(float x) { return gate_sigmoid<T>(x); }

// The warps of the grid walk the rows; a warp holds its row (h and the gate pre-activations) as packed 16-byte
// vectors and has the NEXT row's loads in flight while it reduces, scales and stores the current one.  The row
// stride of the grid is a multiple of NH (the launcher sees to it), so a warp stays on one head and its
// (batch, token) position advances by additions: no division in the loop.
template <typename T, int NV>
__global__ void __launch_bounds__(OG_WARPS * 32) mlstm_output_gate_kernel(
    const T *__restrict__ h, const T *__restrict__ og, const T *__restrict__ w, T *__restrict__ y, int64_t rows, int NH,
    int S, int dv, int64_t hsb, int64_t hsh, int64_t hss, int64_t ldo, float eps) {
    constexpr int VN = Vec16<T>::N;
    const int lane = threadIdx.x & 31;
    const int nvec = dv / VN;
    const int64_t stride = (int64_t)gridDim.x * OG_WARPS;      // rows between two rows of a warp: k * NH
    int64_t row = (int64_t)blockIdx.x * OG_WARPS + (threadIdx.x >> 5);
    grid_dependency_wait();   // h and the gate pre-activations come from the kernels before this one
    allow_dependents();
    if (row >= rows) return;
    // row = (b * S + s) * NH + head
    const int head = (int)(row % NH);
    int64_t bs = row / NH;                                     // b * S + s
    const int64_t bs_step = stride / NH;
    int64_t b = bs / S;
    int s = (int)(bs % S);
    const int64_t b_step = bs_step / S;
    const int s_step = (int)(bs_step % S);
    const T *hbase = h + head * hsh;
    const T *ogbase = og + (size_t)head * dv;

    auto load_row = [&](int64_t b_, int s_, int64_t bs_, uint4 (&hv)[NV], uint4 (&ov)[NV]) {
        const T *hr = hbase + b_ * hsb + s_ * hss;
        const T *ogr = ogbase + bs_ * ldo;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int iv = lane + i * 32;
            if (iv < nvec) {
                hv[i] = ldg16_raw(hr + (size_t)iv * VN);
                ov[i] = ldg16_raw(ogr + (size_t)iv * VN);
            }
        }
    };
    // the norm weight of the head, unpacked once
    float wf[NV][VN];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int iv = lane + i * 32;
        if (w && iv < nvec) unpack16<T>(ldg16_raw(w + (size_t)head * dv + (size_t)iv * VN), wf[i]);
        else
#pragma unroll
            for (int e = 0; e < VN; ++e) wf[i][e] = 1.0f;
    }

    uint4 hv[NV], ov[NV];
    load_row(b, s, bs, hv, ov);
    for (; row < rows; row += stride) {
        // position of this warp's next row
        int64_t bn = b + b_step, bsn = bs + bs_step;
        int sn = s + s_step;
        if (sn >= S) {
            sn -= S;
            ++bn;
        }
        uint4 hn[NV], on[NV];
        if (row + stride < rows) load_row(bn, sn, bsn, hn, on);
        float v[NV][VN];
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i)
            if (lane + i * 32 < nvec) {
                unpack16<T>(hv[i], v[i]);
#pragma unroll
                for (int e = 0; e < VN; ++e) ss = fmaf(v[i][e], v[i][e], ss);
            }
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / (float)dv + eps);
        T *yr = y + row * dv;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int iv = lane + i * 32;
            if (iv < nvec) {
                float o[VN];
                unpack16<T>(ov[i], o);
#pragma unroll
                for (int e = 0; e < VN; ++e) v[i][e] = v[i][e] * inv * wf[i][e] * og_sigmoid<T>(o[e]);
                st16<T>(yr + (size_t)iv * VN, v[i]);
            }
        }
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            hv[i] = hn[i];
            ov[i] = on[i];
        }
        b = bn;
        s = sn;
        bs = bsn;
    }
}

// The same epilogue over MANY rows, as a stream (the form of add_rms_norm_stream_kernel): 16 warps per CTA, one
// CTA per SM, a warp per row; the h row and the gate row arrive through a ring of OGS_RING chunks per warp in
// shared memory (a chunk = one 16-byte vector of h and one of the gate per lane), filled by cp.async OGS_RING
// chunks ahead across row boundaries, so the bytes in flight do not depend on the register allocation.  With
// rows in registers the kernel sat at 16 resident warps per SM and 64 KB in flight: 0.73 of the copy peak.
constexpr int OGS_WARPS = 16, OGS_RING = 12;

template <typename T, int NV>
__global__ void __launch_bounds__(OGS_WARPS * 32, 1) mlstm_output_gate_stream_kernel(
    const T *__restrict__ h, const T *__restrict__ og, const T *__restrict__ w, T *__restrict__ y, int64_t rows, int NH,
    int S, int dv, int64_t hsb, int64_t hsh, int64_t hss, int64_t ldo, float eps) {
    constexpr int VN = Vec16<T>::N;
    constexpr int NT = OGS_WARPS * 32;
    extern __shared__ __align__(16) unsigned char ogs_smem[];
    uint4 *ring = reinterpret_cast<uint4 *>(ogs_smem);         // [OGS_RING][2][NT]
    const int tid = threadIdx.x, lane = tid & 31;
    const int nvec = dv / VN;
    const int64_t stride = (int64_t)gridDim.x * OGS_WARPS;     // a multiple of NH: the warp stays on one head
    const int64_t row0 = (int64_t)blockIdx.x * OGS_WARPS + (tid >> 5);
    if (row0 >= rows) return;                                   // no CTA barrier below
    const int my_rows = (int)((rows - row0 + stride - 1) / stride);
    const int head = (int)(row0 % NH);
    const int64_t bs_step = stride / NH, b_step = bs_step / S;
    const int s_step = (int)(bs_step % S);
    const T *hbase = h + head * hsh;
    const T *ogbase = og + (size_t)head * dv;
    // the copy stream: position (a_b, a_s, a_bs) of the row it is in, a_i the chunk of that row it issues next
    int a_k = 0, a_i = 0;
    int64_t a_bs = row0 / NH, a_b = a_bs / S;
    int a_s = (int)(a_bs % S);
    auto issue = [&](int slot) {
        if (a_k < my_rows) {
            const int iv = lane + 32 * a_i;
            if (iv < nvec) {
                cp_async16(ring + (size_t)(slot * 2 + 0) * NT + tid, hbase + a_b * hsb + a_s * hss + (size_t)iv * VN);
                cp_async16(ring + (size_t)(slot * 2 + 1) * NT + tid, ogbase + a_bs * ldo + (size_t)iv * VN);
            }
            if (++a_i == NV) {
                a_i = 0;
                ++a_k;
                a_bs += bs_step;
                a_b += b_step;
                a_s += s_step;
                if (a_s >= S) {
                    a_s -= S;
                    ++a_b;
                }
            }
        }
        cp_async_commit();
    };
#pragma unroll 1
    for (int c = 0; c < OGS_RING; ++c) issue(c);
    // the norm weight of the head, packed
    uint4 wv[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i)
        if (w && lane + 32 * i < nvec) wv[i] = ldg16_raw(w + (size_t)head * dv + (size_t)(lane + 32 * i) * VN);
    int slot = 0;
    for (int k = 0; k < my_rows; ++k) {
        T *yr = y + (row0 + (int64_t)k * stride) * dv;
        uint4 hv[NV], ov[NV];
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            cp_async_wait<OGS_RING - 1>();                      // the oldest chunk in flight has landed
            if (lane + 32 * i < nvec) {
                hv[i] = ring[(size_t)(slot * 2 + 0) * NT + tid];
                ov[i] = ring[(size_t)(slot * 2 + 1) * NT + tid];
                float v[VN];
                unpack16<T>(hv[i], v);
#pragma unroll
                for (int e = 0; e < VN; ++e) ss = fmaf(v[e], v[e], ss);
            }
            issue(slot);                                        // refill the slot just consumed
            slot = slot + 1 == OGS_RING ? 0 : slot + 1;
        }
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / (float)dv + eps);
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int iv = lane + 32 * i;
            if (iv < nvec) {
                float v[VN], o[VN], wf[VN];
                unpack16<T>(hv[i], v);
                unpack16<T>(ov[i], o);
                if (w) unpack16<T>(wv[i], wf);
#pragma unroll
                for (int e = 0; e < VN; ++e) v[e] = v[e] * inv * (w ? wf[e] : 1.0f) * og_sigmoid<T>(o[e]);
                st16<T>(yr + (size_t)iv * VN, v);
            }
        }
    }
    cp_async_wait<0>();
}

template <typename T, int NV>
static int output_gate_stream_launch(const T *hp, const T *op, const T *wp, T *yp, int64_t rows, int NH, int S, int dv,
                                     const int64_t *hs, int64_t ldo, float eps, cudaStream_t st) {
    auto kern = mlstm_output_gate_stream_kernel<T, NV>;
    const size_t smem = (size_t)OGS_RING * 2 * OGS_WARPS * 32 * sizeof(uint4);
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return XLSTM_ERR_CUDA;
    int grid = 148;
    while ((grid * OGS_WARPS) % NH) ++grid;                     // row stride of the grid: a multiple of NH
    kern<<<grid, OGS_WARPS * 32, smem, st>>>(hp, op, wp, yp, rows, NH, S, dv, hs[0], hs[1], hs[2], ldo, eps);
    return launch_status();
}

template <typename T>
static int output_gate_launch(const void *h, const void *og, const void *w, void *y, int B, int NH, int S, int dv,
                              const int64_t *hs, int64_t ldo, float eps, cudaStream_t st) {
    constexpr int VN = Vec16<T>::N;
    const int nvec = dv / VN;
    const int64_t rows = (int64_t)B * S * NH;
    // enough CTAs to fill the GPU, rounded up so that the grid's row stride (grid * OG_WARPS) is a multiple of NH:
    // a warp then stays on one head
    const int64_t want = (rows + OG_WARPS - 1) / OG_WARPS;
    int64_t cap = 148 * 8;
    while ((cap * OG_WARPS) % NH) ++cap;
    const unsigned grid = (unsigned)(want < cap ? want : cap);
    const T *hp = static_cast<const T *>(h), *op = static_cast<const T *>(og), *wp = static_cast<const T *>(w);
    T *yp = static_cast<T *>(y);
    // many rows (prefill): the streamed kernel; 16-byte copies need 16-byte aligned rows
    const bool aligned16 = ((reinterpret_cast<uintptr_t>(h) | reinterpret_cast<uintptr_t>(og)) & 15u) == 0 &&
                           (hs[0] * sizeof(T)) % 16 == 0 && (hs[1] * sizeof(T)) % 16 == 0 && (hs[2] * sizeof(T)) % 16 == 0 &&
                           (ldo * sizeof(T)) % 16 == 0 && dv % VN == 0;
    if (aligned16 && rows >= 4 * 148 * OGS_WARPS && NH <= 64) {
        if (nvec <= 32) return output_gate_stream_launch<T, 1>(hp, op, wp, yp, rows, NH, S, dv, hs, ldo, eps, st);
        if (nvec <= 64) return output_gate_stream_launch<T, 2>(hp, op, wp, yp, rows, NH, S, dv, hs, ldo, eps, st);
        if (nvec <= 128) return output_gate_stream_launch<T, 4>(hp, op, wp, yp, rows, NH, S, dv, hs, ldo, eps, st);
    }
    const dim3 g(grid), blk(OG_WARPS * 32);
    if (nvec <= 32) return launch_overlapped(mlstm_output_gate_kernel<T, 1>, g, blk, 0, st, hp, op, wp, yp, rows, NH, S, dv, hs[0], hs[1], hs[2], ldo, eps);
    if (nvec <= 64) return launch_overlapped(mlstm_output_gate_kernel<T, 2>, g, blk, 0, st, hp, op, wp, yp, rows, NH, S, dv, hs[0], hs[1], hs[2], ldo, eps);
    if (nvec <= 128) return launch_overlapped(mlstm_output_gate_kernel<T, 4>, g, blk, 0, st, hp, op, wp, yp, rows, NH, S, dv, hs[0], hs[1], hs[2], ldo, eps);
    if (nvec <= 256) return launch_overlapped(mlstm_output_gate_kernel<T, 8>, g, blk, 0, st, hp, op, wp, yp, rows, NH, S, dv, hs[0], hs[1], hs[2], ldo, eps);
    return XLSTM_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------------------
// SwiGLU gate: y[r, c] = silu(g[r, c]) * u[r, c]; g and u may be column blocks of one GEMM output
// ---------------------------------------------------------------------------
// One CTA per row at a time (rows by grid stride); the threads walk the row's 16-byte vectors, two per
// thread per trip so that four loads are in flight.
template <typename T>
__global__ void __launch_bounds__(256) swiglu_kernel(const T *__restrict__ g, const T *__restrict__ u, T *__restrict__ y,
                                                     int64_t rows, int cols, int64_t ldg, int64_t ldu) {
    constexpr int VN = Vec16<T>::N;
    const int nvec = cols / VN;
    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        const T *gr = g + r * ldg, *ur = u + r * ldu;
        T *yr = y + r * cols;
        for (int v = threadIdx.x; v < nvec; v += 512) {
            const int v2 = v + 256;
            float a0[VN], b0[VN], a1[VN], b1[VN];
            ld16<T>(gr + (size_t)v * VN, a0);
            ld16<T>(ur + (size_t)v * VN, b0);
            if (v2 < nvec) {
                ld16<T>(gr + (size_t)v2 * VN, a1);
                ld16<T>(ur + (size_t)v2 * VN, b1);
            }
#pragma unroll
            for (int e = 0; e < VN; ++e) a0[e] = silu_t<T>(a0[e]) * b0[e];
            st16<T>(yr + (size_t)v * VN, a0);
            if (v2 < nvec) {
#pragma unroll
                for (int e = 0; e < VN; ++e) a1[e] = silu_t<T>(a1[e]) * b1[e];
                st16<T>(yr + (size_t)v2 * VN, a1);
            }
        }
    }
}

// Many rows: the same gate as a stream.  The 512-byte chunks (one 16-byte vector of g and of u per lane) of all rows
// form one sequence, dealt to the warps of the grid round-robin (neighbouring warps read neighbouring chunks);
// a warp's chunks arrive through its ring in shared memory, SGS_RING chunks ahead, by cp.async.
constexpr int SGS_WARPS = 16, SGS_RING = 12;

template <typename T> __device__ __forceinline__ float silu_stream(float x) {
    if (sizeof(T) == 2) {   // bf16 result: the sigmoid from one tanh.approx (relative error 2^-11)
        float t;
        const float hx = 0.5f * x;
        asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(hx));
        return fmaf(hx, t, hx);
    }
    return x / (1.0f + expf(-x));
}

template <typename T>
__global__ void __launch_bounds__(SGS_WARPS * 32, 1) swiglu_stream_kernel(const T *__restrict__ g, const T *__restrict__ u,
                                                                         T *__restrict__ y, int rows, int cols, int64_t ldg,
                                                                         int64_t ldu) {
    constexpr int VN = Vec16<T>::N;
    constexpr int NT = SGS_WARPS * 32;
    extern __shared__ __align__(16) unsigned char sgs_smem[];
    uint4 *ring = reinterpret_cast<uint4 *>(sgs_smem);         // [SGS_RING][2][NT]
    const int tid = threadIdx.x, lane = tid & 31;
    const int nvec = cols / VN, cpr = (nvec + 31) >> 5;          // chunks per row
    const int gw = blockIdx.x * SGS_WARPS + (tid >> 5), GW = gridDim.x * SGS_WARPS;
    const int step_row = GW / cpr, step_i = GW % cpr;            // a warp's next chunk: GW chunks further on
    // position of the chunk the copy stream issues next, and of the chunk the compute loop consumes next
    int a_row = gw / cpr, a_i = gw % cpr, c_row = a_row, c_i = a_i;
    auto advance = [&](int &row, int &i) {
        row += step_row;
        i += step_i;
        if (i >= cpr) {
            i -= cpr;
            ++row;
        }
    };
    auto issue = [&](int slot) {
        if (a_row < rows) {
            const int iv = lane + 32 * a_i;
            if (iv < nvec) {
                cp_async16(ring + (size_t)(slot * 2 + 0) * NT + tid, g + (size_t)a_row * ldg + (size_t)iv * VN);
                cp_async16(ring + (size_t)(slot * 2 + 1) * NT + tid, u + (size_t)a_row * ldu + (size_t)iv * VN);
            }
            advance(a_row, a_i);
        }
        cp_async_commit();
    };
#pragma unroll 1
    for (int c = 0; c < SGS_RING; ++c) issue(c);
    int slot = 0;
    while (c_row < rows) {
        cp_async_wait<SGS_RING - 1>();                          // the oldest chunk in flight has landed
        const int iv = lane + 32 * c_i;
        if (iv < nvec) {
            float a[VN], b[VN];
            unpack16<T>(ring[(size_t)(slot * 2 + 0) * NT + tid], a);
            unpack16<T>(ring[(size_t)(slot * 2 + 1) * NT + tid], b);
#pragma unroll
            for (int e = 0; e < VN; ++e) a[e] = silu_stream<T>(a[e]) * b[e];
            st16<T>(y + (size_t)c_row * cols + (size_t)iv * VN, a);
        }
        advance(c_row, c_i);
        issue(slot);                                            // refill the slot just consumed
        slot = slot + 1 == SGS_RING ? 0 : slot + 1;
    }
    cp_async_wait<0>();
}

template <typename T>
__global__ void swiglu_scalar_kernel(const T *__restrict__ g, const T *__restrict__ u, T *__restrict__ y, int64_t rows,
                                     int cols, int64_t ldg, int64_t ldu) {
    const int64_t total = rows * cols;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int64_t r = i / cols;
        const int c = (int)(i % cols);
        Elem<T>::st(y + i, silu_t<T>(Elem<T>::ld(g + r * ldg + c)) * Elem<T>::ld(u + r * ldu + c));
    }
}

template <typename T>
static int swiglu_launch(const void *g, const void *u, void *y, int64_t rows, int cols, int64_t ldg, int64_t ldu,
                         cudaStream_t st) {
    constexpr int VN = Vec16<T>::N;
    const bool aligned = ((reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(u) | reinterpret_cast<uintptr_t>(y)) & 15u) == 0 &&
                         cols % VN == 0 && ldg % VN == 0 && ldu % VN == 0;
    const T *gp = static_cast<const T *>(g), *up = static_cast<const T *>(u);
    if (aligned && rows * (int64_t)((cols / VN + 31) / 32) >= 64 * 148 * SGS_WARPS && rows < (1 << 24) && cols < (1 << 24)) {
        auto kern = swiglu_stream_kernel<T>;
        const size_t smem = (size_t)SGS_RING * 2 * SGS_WARPS * 32 * sizeof(uint4);
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return XLSTM_ERR_CUDA;
        kern<<<148, SGS_WARPS * 32, smem, st>>>(gp, up, static_cast<T *>(y), (int)rows, cols, ldg, ldu);
    } else if (aligned) {
        const unsigned grid = (unsigned)(rows < 148 * 8 ? rows : 148 * 8);   // 8 resident CTAs per SM
        swiglu_kernel<T><<<grid, 256, 0, st>>>(gp, up, static_cast<T *>(y), rows, cols, ldg, ldu);
    } else {
        int64_t want = (rows * cols + 255) / 256;
        const int grid = (int)(want < 1 ? 1 : (want > 148 * 8 ? 148 * 8 : want));
        swiglu_scalar_kernel<T><<<grid, 256, 0, st>>>(gp, up, static_cast<T *>(y), rows, cols, ldg, ldu);
    }
    return launch_status();
}

// ---------------------------------------------------------------------------
// causal depthwise conv1d (+ SiLU), channels-last.  A thread owns VN adjacent channels and a run of consecutive
// tokens.  Its input rows arrive through a private ring of CONV_RING 16-byte slots in shared memory filled by
// cp.async, so CONV_RING rows per thread are in flight without costing registers, and the window of the last
// K - 1 inputs is carried in registers, so only the first token of a run re-reads its K - 1 halo rows.  A warp
// covers 32*VN adjacent channels (one 512-byte piece of a row), the four warps of a CTA four consecutive runs.
// Every slot is written and read by the same thread: no barrier in the loop.
// ---------------------------------------------------------------------------
constexpr int CONV_RING = 16;       // input rows in flight per thread
constexpr int CONV_MIN_RUN = 8;     // tokens per thread: at least / at most
constexpr int CONV_MAX_RUN = 128;
constexpr int CONV_ALIAS_MAX = 16;  // longest call whose new state may overwrite the old one in place (one CTA per batch row)
constexpr int CONV_KMAX = 8;


// SiLU for the convolution output: bf16 results take the sigmoid from one tanh.approx
template <typename T> __device__ __forceinline__ float conv_silu(float x) {
    if (sizeof(T) == 2) {
        float t;
        const float hx = 0.5f * x;
        asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(hx));
        return fmaf(hx, t, hx);
    }
    return x / (1.0f + expf(-x));
}

template <typename T, int K>
__global__ void __launch_bounds__(128, (K * (16 / sizeof(T)) <= 40) ? 4 : 2) causal_conv1d_kernel(const T *__restrict__ x, const T *__restrict__ w,
                                                               const T *__restrict__ bias, const T *__restrict__ state_in,
                                                               T *__restrict__ state_out, T *__restrict__ y, int S, int C,
                                                               int act_silu, int run) {
    constexpr int VN = Vec16<T>::N;
    constexpr int H = K - 1;                               // history length
    __shared__ uint4 ring[CONV_RING][128];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int cv = blockIdx.x * 32 + lane;                 // channel vector
    const bool ch_ok = cv * VN < C;
    const int c0 = ch_ok ? cv * VN : 0;
    const int b = blockIdx.z;
    const int cta_tokens = 4 * run;
    const int s_begin = blockIdx.y * cta_tokens + warp * run;
    const int n_tok = ch_ok ? min(run, S - s_begin) : 0;   // tokens of this thread (<= 0: none)
    const T *xb = x + (size_t)b * S * C + c0;
    T *yb = y + (size_t)b * S * C + c0;
    const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
    // the first CONV_RING rows of the run go out at once (one group per row, empty groups past the end)
#pragma unroll
    for (int r = 0; r < CONV_RING; ++r) {
        if (r < n_tok) cp_async16(&ring[r][tid], xb + (size_t)(s_begin + r) * C);
        cp_async_commit();
    }
    // rows before token 0 come from the state (or are zero)
    auto load_old = [&](int t) -> uint4 {
        if (t >= 0) return *reinterpret_cast<const uint4 *>(xb + (size_t)t * C);
        if (state_in) return *reinterpret_cast<const uint4 *>(state_in + ((size_t)b * H + (H + t)) * C + c0);
        return zero4;
    };
    if (n_tok > 0) {
        uint4 hist[H > 0 ? H : 1];
#pragma unroll
        for (int j = 0; j < H; ++j) hist[j] = load_old(s_begin - H + j);
        // the VN x K taps of this thread's channels are VN*K contiguous elements = K 16-byte vectors
        float wflat[VN * K];
#pragma unroll
        for (int j = 0; j < K; ++j) ld16<T>(w + (size_t)c0 * K + j * VN, wflat + j * VN);
        float wk[K][VN];                                   // wk[j][e]: tap j of channel c0 + e
#pragma unroll
        for (int e = 0; e < VN; ++e)
#pragma unroll
            for (int j = 0; j < K; ++j) wk[j][e] = wflat[e * K + j];
        float bv[VN];
        if (bias) ld16<T>(bias + c0, bv);
        else
#pragma unroll
            for (int e = 0; e < VN; ++e) bv[e] = 0.f;
        // window of the last K rows, unpacked once each, as a ring of K register rows: at step u of an unrolled
        // block of K steps the newest row sits in slot u and tap j reads slot (u + 1 + j) % K
        float win[K][VN];
#pragma unroll
        for (int j = 0; j < H; ++j) unpack16<T>(hist[j], win[j + 1]);
        for (int i0 = 0; i0 < n_tok; i0 += K) {
#pragma unroll
            for (int u = 0; u < K; ++u) {
                const int i = i0 + u;
                if (i < n_tok) {
                    cp_async_wait<CONV_RING - 1>();            // the group of row i has landed
                    const uint4 raw = ring[i % CONV_RING][tid];
                    unpack16<T>(raw, win[u]);
                    float acc[VN];
#pragma unroll
                    for (int e = 0; e < VN; ++e) acc[e] = bv[e];
#pragma unroll
                    for (int j = 0; j < K; ++j)
#pragma unroll
                        for (int e = 0; e < VN; ++e) acc[e] = fmaf(wk[j][e], win[(u + 1 + j) % K][e], acc[e]);
                    if (act_silu)
#pragma unroll
                        for (int e = 0; e < VN; ++e) acc[e] = conv_silu<T>(acc[e]);
                    st16<T>(yb + (size_t)(s_begin + i) * C, acc);
                    // refill the slot just consumed with the row CONV_RING ahead (after its value has been used)
                    if (i + CONV_RING < n_tok) cp_async16(&ring[i % CONV_RING][tid], xb + (size_t)(s_begin + i + CONV_RING) * C);
                    cp_async_commit();
                }
            }
        }
    }
    cp_async_wait<0>();
    // the new state = last K-1 inputs of [state ; x]: written by the CTA that owns the last token, after
    // every warp of it has read what it needs from the old state (in-place update)
    if (state_out != nullptr) {          // uniform over the CTA
        __syncthreads();
        if ((int)blockIdx.y == (S - 1) / cta_tokens && warp == 0 && ch_ok) {
            uint4 st_new[H > 0 ? H : 1];
#pragma unroll
            for (int j = 0; j < H; ++j) st_new[j] = load_old(S - H + j);
#pragma unroll
            for (int j = 0; j < H; ++j) *reinterpret_cast<uint4 *>(state_out + ((size_t)b * H + j) * C + c0) = st_new[j];
        }
    }
}

}  // namespace xl

using namespace xl;

static inline bool dtype_ok(int dtype) { return dtype == XLSTM_F32 || dtype == XLSTM_BF16; }

extern "C" int xlstm_rms_norm(const void *x, const void *w, void *y, int64_t rows, int cols, float eps, int dtype,
                              void *stream) {
    if (rows < 0 || cols <= 0 || (rows > 0 && (!x || !y))) return XLSTM_ERR_INVALID;
    if (!dtype_ok(dtype)) return XLSTM_ERR_UNSUPPORTED;
    if (rows == 0) return XLSTM_OK;
    if (rows > 0x7fffffffLL) return XLSTM_ERR_UNSUPPORTED;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return dtype == XLSTM_F32 ? rms_norm_launch<float>(x, nullptr, w, nullptr, y, rows, cols, eps, st)
                              : rms_norm_launch<__nv_bfloat16>(x, nullptr, w, nullptr, y, rows, cols, eps, st);
}

extern "C" int xlstm_add_rms_norm(const void *x, const void *r, const void *w, void *sum, void *y, int64_t rows,
                                  int cols, float eps, int dtype, void *stream) {
    if (rows < 0 || cols <= 0 || (rows > 0 && (!x || !r || !sum || !y))) return XLSTM_ERR_INVALID;
    if (!dtype_ok(dtype)) return XLSTM_ERR_UNSUPPORTED;
    if (rows == 0) return XLSTM_OK;
    if (rows > 0x7fffffffLL) return XLSTM_ERR_UNSUPPORTED;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return dtype == XLSTM_F32 ? rms_norm_launch<float>(x, r, w, sum, y, rows, cols, eps, st)
                              : rms_norm_launch<__nv_bfloat16>(x, r, w, sum, y, rows, cols, eps, st);
}

extern "C" int xlstm_mlstm_output_gate(const void *h, const void *ogate, const void *w, void *y, int B, int NH, int S,
                                       int dv, const int64_t *h_strides, int64_t ogate_ld, float eps, int dtype,
                                       void *stream) {
    if (B < 0 || NH <= 0 || S < 0 || dv <= 0) return XLSTM_ERR_INVALID;
    if (!dtype_ok(dtype)) return XLSTM_ERR_UNSUPPORTED;
    if (B == 0 || S == 0) return XLSTM_OK;
    if (!h || !ogate || !y) return XLSTM_ERR_INVALID;
    const int vn = dtype == XLSTM_F32 ? 4 : 8;
    int64_t hs[3] = {(int64_t)NH * S * dv, (int64_t)S * dv, (int64_t)dv};   // dense [B,NH,S,dv]
    if (h_strides) { hs[0] = h_strides[0]; hs[1] = h_strides[1]; hs[2] = h_strides[2]; }
    const uintptr_t al = reinterpret_cast<uintptr_t>(h) | reinterpret_cast<uintptr_t>(ogate) | reinterpret_cast<uintptr_t>(y) |
                         reinterpret_cast<uintptr_t>(w);
    const int64_t ldo = ogate_ld > 0 ? ogate_ld : (int64_t)NH * dv;
    if (ldo < (int64_t)NH * dv) return XLSTM_ERR_INVALID;
    if (dv % vn || hs[0] % vn || hs[1] % vn || hs[2] % vn || ldo % vn || (al & 15u)) return XLSTM_ERR_UNSUPPORTED;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return dtype == XLSTM_F32 ? output_gate_launch<float>(h, ogate, w, y, B, NH, S, dv, hs, ldo, eps, st)
                              : output_gate_launch<__nv_bfloat16>(h, ogate, w, y, B, NH, S, dv, hs, ldo, eps, st);
}

extern "C" int xlstm_swiglu(const void *g, const void *u, void *y, int64_t rows, int cols, int64_t ldg, int64_t ldu,
                            int dtype, void *stream) {
    if (rows < 0 || cols <= 0 || ldg < cols || ldu < cols) return XLSTM_ERR_INVALID;
    if (!dtype_ok(dtype)) return XLSTM_ERR_UNSUPPORTED;
    if (rows == 0) return XLSTM_OK;
    if (!g || !u || !y) return XLSTM_ERR_INVALID;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return dtype == XLSTM_F32 ? swiglu_launch<float>(g, u, y, rows, cols, ldg, ldu, st)
                              : swiglu_launch<__nv_bfloat16>(g, u, y, rows, cols, ldg, ldu, st);
}

extern "C" int xlstm_causal_conv1d(const void *x, const void *w, const void *bias, const void *state_in, void *state_out,
                                   void *y, int B, int S, int C, int K, int act_silu, int dtype, void *stream) {
    if (B < 0 || S < 0 || C <= 0 || K <= 0) return XLSTM_ERR_INVALID;
    if (!dtype_ok(dtype) || K > CONV_KMAX) return XLSTM_ERR_UNSUPPORTED;
    if (B == 0 || S == 0) return XLSTM_OK;
    if (!x || !w || !y) return XLSTM_ERR_INVALID;
    // the in-place state update is only safe while one token block reads the old state and writes the new one
    if (state_out && state_out == state_in && S > CONV_ALIAS_MAX) return XLSTM_ERR_INVALID;
    const int vn = dtype == XLSTM_F32 ? 4 : 8;
    const uintptr_t al = reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(bias) |
                         reinterpret_cast<uintptr_t>(state_in) | reinterpret_cast<uintptr_t>(state_out) |
                         reinterpret_cast<uintptr_t>(w);
    if (C % vn || (al & 15u) || B > 65535) return XLSTM_ERR_UNSUPPORTED;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int cvec = C / vn;
    // tokens per thread: the longest run (fewest halo re-reads) that still gives every SM four CTAs
    int run = CONV_MAX_RUN;
    while (run > CONV_MIN_RUN && (int64_t)((cvec + 31) / 32) * ((S + 4 * run - 1) / (4 * run)) * B < 148 * 4) run >>= 1;
    const int cta_tokens = 4 * run;
    if ((S + cta_tokens - 1) / cta_tokens > 65535) return XLSTM_ERR_UNSUPPORTED;
    const dim3 grid((cvec + 31) / 32, (S + cta_tokens - 1) / cta_tokens, B);
#define XL_CONV_CASE(KK)                                                                                              \
    case KK:                                                                                                          \
        if (dtype == XLSTM_F32)                                                                                       \
            causal_conv1d_kernel<float, KK><<<grid, 128, 0, st>>>(                                                    \
                static_cast<const float *>(x), static_cast<const float *>(w), static_cast<const float *>(bias),      \
                static_cast<const float *>(state_in), static_cast<float *>(state_out), static_cast<float *>(y), S, C, \
                act_silu, run);                                                                                       \
        else                                                                                                          \
            causal_conv1d_kernel<__nv_bfloat16, KK><<<grid, 128, 0, st>>>(                                            \
                static_cast<const __nv_bfloat16 *>(x), static_cast<const __nv_bfloat16 *>(w),                         \
                static_cast<const __nv_bfloat16 *>(bias), static_cast<const __nv_bfloat16 *>(state_in),               \
                static_cast<__nv_bfloat16 *>(state_out), static_cast<__nv_bfloat16 *>(y), S, C, act_silu, run);       \
        break;
    switch (K) {
        XL_CONV_CASE(1) XL_CONV_CASE(2) XL_CONV_CASE(3) XL_CONV_CASE(4)
        XL_CONV_CASE(5) XL_CONV_CASE(6) XL_CONV_CASE(7) XL_CONV_CASE(8)
        default: return XLSTM_ERR_UNSUPPORTED;
    }
#undef XL_CONV_CASE
    return launch_status();
}
