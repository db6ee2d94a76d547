// Single-token mLSTM decode step: a streaming read-modify-write of the
// dqk x dv fp32 matrix memory of every (batch, head), fused with the output
// read-out.  HBM-bound: ~2*dqk*dv*4 bytes per head against ~5*dqk*dv flops.
//
// Work split: one CTA owns DVT columns of one head's C for all dqk rows, so
// the h = q~ . C' reduction never leaves the CTA; the 1 KB normaliser vector is
// recomputed by every CTA of the head (cheaper than a second pass).  Rows are
// walked in batches of UNROLL independent 128-bit streaming loads per thread,
// the first batch issued before the gate prologue and each next batch before
// the current one is consumed, to keep enough bytes in flight for HBM3e.
// The kernel is launched so that its CTAs may become resident under the tail of the kernel before it; when the
// caller promises that the state it reads was written by an earlier launch than that one (decode over a stack
// of layers: the kernel before a layer's step is that layer's projection), the first batch of state loads goes
// out before the wait on that kernel, so the HBM stream does not stop at the kernel boundary.
#include "common.cuh"

namespace xl {

// tile shape (the measured best on B200): dv columns per CTA, threads, rows in flight per thread, CTAs per SM
constexpr int STEP_DVT = 64, STEP_THREADS = 256, STEP_UNROLL = 4, STEP_MIN_CTAS = 4;

template <typename T, int DVT, int THREADS, int UNROLL>
__global__ void __launch_bounds__(THREADS, STEP_MIN_CTAS)
mlstm_step_kernel(const T *__restrict__ q, const T *__restrict__ k, const T *__restrict__ v,
                  const T *__restrict__ ig, const T *__restrict__ fg,
                  const float *C0, const float *__restrict__ n0, const float *__restrict__ m0,
                  T *__restrict__ h, float *C1, float *__restrict__ n1, float *__restrict__ m1,
                  int dqk, int dv, float eps, float qscale, float gate_cap, int state_settled) {
    constexpr int CV = DVT / 4;       // 128-bit column vectors per row of the tile
    constexpr int RG = THREADS / CV;  // row groups walking the rows in parallel
    extern __shared__ float smem[];
    float *s_q = smem;                // [dqk]  q * dqk^-1/2
    float *s_kw = s_q + dqk;          // [dqk]  e^{i-m'} * k
    float *s_red = s_kw + dqk;        // [RG][DVT] partial h
    __shared__ float s_warp[THREADS / 32];
    __shared__ float s_den;

    const int bh = blockIdx.x;
    const int tile = blockIdx.y;
    const int tid = threadIdx.x;
    const bool has_state = (C0 != nullptr);
    const int cv = tid % CV, rg = tid / CV;
    const int col = tile * DVT + cv * 4;
    const bool active = col < dv;
    const float *Cin = C0 + (size_t)bh * dqk * dv + col;
    float *Cout = C1 + (size_t)bh * dqk * dv + col;
    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);

    // first batch of state rows: in flight while the prologue below runs (and, for a settled state, while the
    // preceding kernel drains)
    float4 c[UNROLL];
    if (state_settled) {
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int j = rg + u * RG;
            c[u] = (active && has_state && j < dqk) ? ldg_stream(Cin + (size_t)j * dv) : zero4;
        }
    }
    grid_dependency_wait();
    allow_dependents();
    if (!state_settled) {
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int j = rg + u * RG;
            c[u] = (active && has_state && j < dqk) ? ldg_stream(Cin + (size_t)j * dv) : zero4;
        }
    }

    // stabilised gates (every thread: two exps and a log1p are cheaper than a broadcast)
    const float it = gate_softcap(Elem<T>::ld(ig + bh), gate_cap);
    const float flog = logsigmoid(gate_softcap(Elem<T>::ld(fg + bh), gate_cap));
    const float mold = has_state ? m0[bh] : 0.0f;
    const float mnew = fmaxf(flog + mold, it);
    const float fgate = expf(flog + mold - mnew);
    const float igate = expf(it - mnew);

    // q~, gated k, normaliser update and q~ . n'
    float qn = 0.0f;
    for (int j = tid; j < dqk; j += THREADS) {
        const float qj = Elem<T>::ld(q + (size_t)bh * dqk + j) * qscale;
        const float kj = Elem<T>::ld(k + (size_t)bh * dqk + j);
        const float nj = fgate * (has_state ? n0[(size_t)bh * dqk + j] : 0.0f) + igate * kj;
        s_q[j] = qj;
        s_kw[j] = igate * kj;
        qn += nj * qj;
        if (tile == 0) n1[(size_t)bh * dqk + j] = nj;
    }
    qn = warp_sum(qn);
    if ((tid & 31) == 0) s_warp[tid >> 5] = qn;
    __syncthreads();
    if (tid == 0) {
        float t = 0.0f;
#pragma unroll
        for (int w = 0; w < THREADS / 32; ++w) t += s_warp[w];
        s_den = fmaxf(fabsf(t), expf(-mnew)) + eps;
        if (tile == 0) m1[bh] = mnew;
    }

    float4 acc = zero4;
    if (active) {
        const float4 v4 = ld4(v + (size_t)bh * dv + col);
        for (int j0 = rg; j0 < dqk; j0 += RG * UNROLL) {
            // next batch goes out before this one is consumed
            float4 nx[UNROLL];
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                const int j = j0 + (UNROLL + u) * RG;
                nx[u] = (has_state && j < dqk) ? ldg_stream(Cin + (size_t)j * dv) : zero4;
            }
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                const int j = j0 + u * RG;
                if (j < dqk) {
                    const float kw = s_kw[j], qj = s_q[j];
                    float4 o;
                    o.x = fmaf(fgate, c[u].x, kw * v4.x);
                    o.y = fmaf(fgate, c[u].y, kw * v4.y);
                    o.z = fmaf(fgate, c[u].z, kw * v4.z);
                    o.w = fmaf(fgate, c[u].w, kw * v4.w);
                    stg_stream(Cout + (size_t)j * dv, o);
                    acc.x = fmaf(o.x, qj, acc.x);
                    acc.y = fmaf(o.y, qj, acc.y);
                    acc.z = fmaf(o.z, qj, acc.z);
                    acc.w = fmaf(o.w, qj, acc.w);
                }
            }
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) c[u] = nx[u];
        }
    }
    st4(s_red + rg * DVT + cv * 4, acc);
    __syncthreads();
    if (tid < DVT && tile * DVT + tid < dv) {
        float t = 0.0f;
#pragma unroll
        for (int r = 0; r < RG; ++r) t += s_red[r * DVT + tid];
        Elem<T>::st(h + (size_t)bh * dv + tile * DVT + tid, t / s_den);
    }
}

template <typename T>
static int mlstm_step_launch(const void *q, const void *k, const void *v, const void *ig, const void *fg,
                             const float *C0, const float *n0, const float *m0, void *h, float *C1, float *n1,
                             float *m1, int BH, int dqk, int dv, float eps, float gate_cap, int state_settled,
                             cudaStream_t st) {
    constexpr int DVT = STEP_DVT, THREADS = STEP_THREADS, UNROLL = STEP_UNROLL;
    dim3 grid(BH, (dv + DVT - 1) / DVT);
    size_t smem = sizeof(float) * (2 * (size_t)dqk + (THREADS / (DVT / 4)) * DVT);
    auto kern = mlstm_step_kernel<T, DVT, THREADS, UNROLL>;
    if (smem > 48 * 1024) {
        if (smem > 200 * 1024) return XLSTM_ERR_UNSUPPORTED;
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return XLSTM_ERR_CUDA;
    }
    return launch_overlapped(kern, grid, dim3(THREADS), smem, st, static_cast<const T *>(q), static_cast<const T *>(k),
                             static_cast<const T *>(v), static_cast<const T *>(ig), static_cast<const T *>(fg), C0, n0, m0,
                             static_cast<T *>(h), C1, n1, m1, dqk, dv, eps, 1.0f / sqrtf((float)dqk), gate_cap,
                             state_settled);
}

}  // namespace xl

static int mlstm_step_checked(const void *q, const void *k, const void *v, const void *ig, const void *fg,
                              const float *C0, const float *n0, const float *m0, void *h, float *C1, float *n1,
                              float *m1, int B, int NH, int dqk, int dv, float eps, float gate_cap, int flags,
                              int dtype, void *stream) {
    if (!q || !k || !v || !ig || !fg || !h || !C1 || !n1 || !m1) return XLSTM_ERR_INVALID;
    if (B <= 0 || NH <= 0 || dqk <= 0 || dv <= 0) return XLSTM_ERR_INVALID;
    if (C0 && (!n0 || !m0)) return XLSTM_ERR_INVALID;
    if (C0 && (n1 == n0 || m1 == m0)) return XLSTM_ERR_INVALID;  // other CTAs of the head still read n0/m0
    if (dv % 4 != 0) return XLSTM_ERR_UNSUPPORTED;
    if (dtype != XLSTM_F32 && dtype != XLSTM_BF16) return XLSTM_ERR_UNSUPPORTED;
    if ((int64_t)B * NH > 2147483647LL || (dv + xl::STEP_DVT - 1) / xl::STEP_DVT > 65535) return XLSTM_ERR_UNSUPPORTED;
    if (flags & ~XLSTM_STEP_STATE_SETTLED) return XLSTM_ERR_INVALID;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int settled = (flags & XLSTM_STEP_STATE_SETTLED) ? 1 : 0;
    if (dtype == XLSTM_F32)
        return xl::mlstm_step_launch<float>(q, k, v, ig, fg, C0, n0, m0, h, C1, n1, m1, B * NH, dqk, dv, eps, gate_cap,
                                            settled, st);
    return xl::mlstm_step_launch<__nv_bfloat16>(q, k, v, ig, fg, C0, n0, m0, h, C1, n1, m1, B * NH, dqk, dv, eps, gate_cap,
                                                settled, st);
}

extern "C" int xlstm_mlstm_step(const void *q, const void *k, const void *v, const void *ig, const void *fg,
                                const float *C0, const float *n0, const float *m0, void *h, float *C1, float *n1,
                                float *m1, int B, int NH, int dqk, int dv, float eps, int dtype, void *stream) {
    return mlstm_step_checked(q, k, v, ig, fg, C0, n0, m0, h, C1, n1, m1, B, NH, dqk, dv, eps, 0.0f, 0, dtype, stream);
}

extern "C" int xlstm_mlstm_step_gatecap(const void *q, const void *k, const void *v, const void *ig, const void *fg,
                                        const float *C0, const float *n0, const float *m0, void *h, float *C1,
                                        float *n1, float *m1, int B, int NH, int dqk, int dv, float eps, float gate_cap,
                                        int dtype, void *stream) {
    return mlstm_step_checked(q, k, v, ig, fg, C0, n0, m0, h, C1, n1, m1, B, NH, dqk, dv, eps, gate_cap, 0, dtype, stream);
}

extern "C" int xlstm_mlstm_step_ex(const void *q, const void *k, const void *v, const void *ig, const void *fg,
                                   const float *C0, const float *n0, const float *m0, void *h, float *C1, float *n1,
                                   float *m1, int B, int NH, int dqk, int dv, float eps, float gate_cap, int flags,
                                   int dtype, void *stream) {
    return mlstm_step_checked(q, k, v, ig, fg, C0, n0, m0, h, C1, n1, m1, B, NH, dqk, dv, eps, gate_cap, flags, dtype, stream);
}
