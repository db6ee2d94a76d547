// sLSTM kernels.
//
// (1) slstm_scan: the packaged cell (scalar gates per head, no recurrent
//     weights) has no dependence on h_{t-1}, so the whole sequence is one
//     first-order scan per (batch, head): a single launch walks S timesteps,
//     the per-step gate scalars are computed once per head (not once per
//     unit) and the unit state lives in registers.  HBM-bound on z and h.
//
// (2) slstm_recurrent: the block-diagonal variant is truly sequential through
//     h_{t-1}.  A thread-block cluster owns one (head, batch group); every CTA
//     keeps its slice of the four recurrent matrices resident in shared memory
//     for all timesteps and the CTAs exchange their slice of h_t through
//     distributed shared memory once per step.  Latency-bound.
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace xl {

// ---------------------------------------------------------------------------
// (1) scan over S timesteps, packaged cell
// ---------------------------------------------------------------------------
constexpr int SCAN_TT = 32;  // timesteps per gate tile (one warp lane each)
constexpr int SCAN_HPT = 4;  // units per thread at most

template <typename T>
__global__ void __launch_bounds__(256)
slstm_scan_kernel(const T *__restrict__ z, const T *__restrict__ ig, const T *__restrict__ fg,
                  const T *__restrict__ og, const float *c0, const float *n0, const float *__restrict__ m0,
                  T *__restrict__ h, float *c1, float *n1, float *__restrict__ m1, int S, int NH, int H, float eps) {
    __shared__ float s_f[SCAN_TT], s_i[SCAN_TT], s_o[SCAN_TT];
    __shared__ float s_m;
    const int bh = blockIdx.x, b = bh / NH, hd = bh % NH;
    const int tid = threadIdx.x;
    float c[SCAN_HPT], n[SCAN_HPT];
#pragma unroll
    for (int u = 0; u < SCAN_HPT; ++u) {
        const int j = tid + u * blockDim.x;
        c[u] = (c0 && j < H) ? c0[(size_t)bh * H + j] : 0.f;
        n[u] = (c0 && j < H) ? n0[(size_t)bh * H + j] : 0.f;
    }
    if (tid == 0) s_m = c0 ? m0[bh] : 0.f;
    __syncthreads();

    for (int t0 = 0; t0 < S; t0 += SCAN_TT) {
        const int nt = min(SCAN_TT, S - t0);
        if (tid < 32) {
            // lane = timestep: transcendental work in parallel, then the exact
            // sequential stabiliser recurrence m_t = max(m_{t-1} + logsig f_t, i_t)
            const size_t g = ((size_t)b * S + t0 + tid) * NH + hd;
            const bool valid = tid < nt;
            const float lf = valid ? logsigmoid(Elem<T>::ld(fg + g)) : 0.f;
            const float it = valid ? Elem<T>::ld(ig + g) : 0.f;
            const float ot = valid ? sigmoidf(Elem<T>::ld(og + g)) : 0.f;
            float m = s_m, m_prev_mine = 0.f, m_mine = 0.f;
            for (int s = 0; s < nt; ++s) {
                const float lfs = __shfl_sync(0xffffffffu, lf, s);
                const float is = __shfl_sync(0xffffffffu, it, s);
                const float mn = fmaxf(m + lfs, is);
                if (s == tid) { m_prev_mine = m; m_mine = mn; }
                m = mn;
            }
            if (valid) {
                s_f[tid] = expf(m_prev_mine + lf - m_mine);
                s_i[tid] = expf(it - m_mine);
                s_o[tid] = ot;
            }
            if (tid == 0) s_m = m;
        }
        __syncthreads();
#pragma unroll
        for (int u = 0; u < SCAN_HPT; ++u) {
            const int j = tid + u * blockDim.x;
            if (j < H) {
                const T *zp = z + (((size_t)b * S + t0) * NH + hd) * H + j;
                T *hp = h + (((size_t)b * S + t0) * NH + hd) * H + j;
                const size_t tstride = (size_t)NH * H;
                float cc = c[u], nn = n[u];
                for (int s0 = 0; s0 < nt; s0 += 8) {
                    float zz[8];
#pragma unroll
                    for (int s = 0; s < 8; ++s) zz[s] = (s0 + s < nt) ? Elem<T>::ld(zp + (s0 + s) * tstride) : 0.f;
#pragma unroll
                    for (int s = 0; s < 8; ++s) {
                        if (s0 + s < nt) {
                            cc = fmaf(s_f[s0 + s], cc, s_i[s0 + s] * tanhf(zz[s]));
                            nn = fmaf(s_f[s0 + s], nn, s_i[s0 + s]);
                            Elem<T>::st(hp + (s0 + s) * tstride, s_o[s0 + s] * cc / (fabsf(nn) + eps));
                        }
                    }
                }
                c[u] = cc; n[u] = nn;
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int u = 0; u < SCAN_HPT; ++u) {
        const int j = tid + u * blockDim.x;
        if (j < H) { c1[(size_t)bh * H + j] = c[u]; n1[(size_t)bh * H + j] = n[u]; }
    }
    if (tid == 0) m1[bh] = s_m;
}

// ---------------------------------------------------------------------------
// (2) block-diagonal recurrent sLSTM, recurrent weights resident in shared memory
// ---------------------------------------------------------------------------
constexpr int REC_THREADS = 256;
#ifndef XL_REC_BG
#define XL_REC_BG 4
#endif
constexpr int REC_BG = XL_REC_BG;  // batch rows per cluster

template <typename T> struct RStore;     // how R sits in shared memory
template <> struct RStore<float> {
    using type = float;                  // sR[k][col]
    static constexpr int KPACK = 1;
};
template <> struct RStore<__nv_bfloat16> {
    using type = __nv_bfloat162;         // sR[k/2][col] = (R[k], R[k+1])
    static constexpr int KPACK = 2;
};

template <typename T>
__global__ void __launch_bounds__(REC_THREADS, 1)
slstm_recurrent_kernel(const T *__restrict__ gx, const T *__restrict__ R, const float *__restrict__ rb,
                       const float *__restrict__ c0, const float *__restrict__ n0, const float *__restrict__ h0,
                       const float *__restrict__ m0, T *__restrict__ hs, float *__restrict__ c1,
                       float *__restrict__ n1, float *__restrict__ h1, float *__restrict__ m1, int B, int S, int NH,
                       int dh, int U, float cap) {
    using RT = typename RStore<T>::type;
    constexpr int KPACK = RStore<T>::KPACK;
    cg::cluster_group cluster = cg::this_cluster();
    const int CL = (int)cluster.num_blocks();
    const int rank = (int)cluster.block_rank();
    const int hd = blockIdx.y, b0 = blockIdx.z * REC_BG;
    const int D = NH * dh, NCOL = 4 * U, u0 = rank * U;
    const int tid = threadIdx.x;

    extern __shared__ __align__(16) unsigned char smem_raw[];
    RT *sR = reinterpret_cast<RT *>(smem_raw);                                    // [dh/KPACK][NCOL]
    float *sH = reinterpret_cast<float *>(smem_raw + (size_t)(dh / KPACK) * NCOL * sizeof(RT));  // [2][BG][dh]
    float *sPre = sH + 2 * REC_BG * dh;                                            // [BG][NCOL]

    // resident slice of the recurrent weights: column = gate*U + unit
    for (int e = tid; e < (dh / KPACK) * NCOL; e += REC_THREADS) {
        const int kk = e / NCOL, col = e % NCOL, g = col / U, u = col % U;
        const T *row = R + (((size_t)g * NH + hd) * dh + u0 + u) * dh;
        if constexpr (KPACK == 1) {
            sR[e] = row[kk];
        } else {
            sR[e] = __halves2bfloat162(row[2 * kk], row[2 * kk + 1]);
        }
    }
    // h_{-1} for the whole head, own copy in every CTA
    for (int e = tid; e < REC_BG * dh; e += REC_THREADS) {
        const int bb = e / dh, kx = e % dh;
        sH[e] = (h0 && b0 + bb < B) ? h0[(size_t)(b0 + bb) * D + hd * dh + kx] : 0.f;
    }
    // unit state of the (batch row, unit) pairs this thread owns
    constexpr int PPT = (REC_BG * 64 + REC_THREADS - 1) / REC_THREADS;
    float sc[PPT], sn[PPT], sm[PPT], sh_last[PPT];
#pragma unroll
    for (int pi = 0; pi < PPT; ++pi) {
        const int pr = tid + pi * REC_THREADS, bb = pr / U, u = pr % U;
        const bool ok = pr < REC_BG * U && b0 + bb < B;
        const size_t so = ok ? (size_t)(b0 + bb) * D + hd * dh + u0 + u : 0;
        sc[pi] = (ok && c0) ? c0[so] : 0.f;
        sn[pi] = (ok && c0) ? n0[so] : 1.f;
        sm[pi] = (ok && c0) ? m0[so] : 0.f;
        sh_last[pi] = (ok && c0) ? h0[so] : 0.f;
    }
    const int col = tid, g_of_col = col < NCOL ? col / U : 0, u_of_col = col < NCOL ? col % U : 0;
    const float bias = col < NCOL ? rb[(size_t)g_of_col * D + hd * dh + u0 + u_of_col] : 0.f;
    cluster.sync();

    int cur = 0;
    for (int t = 0; t < S; ++t) {
        // input-side pre-activations for this step (independent of the recurrence)
        float gxv[REC_BG];
#pragma unroll
        for (int bb = 0; bb < REC_BG; ++bb)
            gxv[bb] = (col < NCOL && b0 + bb < B)
                          ? Elem<T>::ld(gx + (((size_t)(b0 + bb) * S + t) * 4 + g_of_col) * D + hd * dh + u0 + u_of_col)
                          : 0.f;
        // recurrent mat-vec: acc[b] = sum_k R[col][k] h[b][k]
        if (col < NCOL) {
            float acc[REC_BG];
#pragma unroll
            for (int bb = 0; bb < REC_BG; ++bb) acc[bb] = 0.f;
            const float *hcur = sH + cur * REC_BG * dh;
            for (int k4 = 0; k4 < dh; k4 += 4) {
                float r[4];
                if constexpr (KPACK == 1) {
#pragma unroll
                    for (int x = 0; x < 4; ++x) r[x] = sR[(k4 + x) * NCOL + col];
                } else {
                    const float2 r01 = __bfloat1622float2(sR[(k4 / 2) * NCOL + col]);
                    const float2 r23 = __bfloat1622float2(sR[(k4 / 2 + 1) * NCOL + col]);
                    r[0] = r01.x; r[1] = r01.y; r[2] = r23.x; r[3] = r23.y;
                }
#pragma unroll
                for (int bb = 0; bb < REC_BG; ++bb) {
                    const float4 hv = *reinterpret_cast<const float4 *>(hcur + bb * dh + k4);
                    acc[bb] = fmaf(r[0], hv.x, acc[bb]);
                    acc[bb] = fmaf(r[1], hv.y, acc[bb]);
                    acc[bb] = fmaf(r[2], hv.z, acc[bb]);
                    acc[bb] = fmaf(r[3], hv.w, acc[bb]);
                }
            }
#pragma unroll
            for (int bb = 0; bb < REC_BG; ++bb) sPre[bb * NCOL + col] = gxv[bb] + (acc[bb] + bias);
        }
        __syncthreads();
        // pointwise gating for the owned (batch row, unit) pairs; publish h_t to every CTA of the cluster
        float *hnext_local = sH + (cur ^ 1) * REC_BG * dh;
#pragma unroll
        for (int pi = 0; pi < PPT; ++pi) {
            const int pr = tid + pi * REC_THREADS;
            if (pr < REC_BG * U) {
                const int bb = pr / U, u = pr % U;
                float it = sPre[bb * NCOL + 0 * U + u], ft = sPre[bb * NCOL + 1 * U + u];
                if (cap > 0.f) { it = cap * tanhf(it / cap); ft = cap * tanhf(ft / cap); }
                const float zt = tanhf(sPre[bb * NCOL + 2 * U + u]);
                const float ot = sigmoidf(sPre[bb * NCOL + 3 * U + u]);
                const float mt = fmaxf(ft + sm[pi], it);
                const float ie = expf(it - mt), fe = expf(ft - mt + sm[pi]);
                sc[pi] = fmaf(fe, sc[pi], ie * zt);
                sn[pi] = fmaf(fe, sn[pi], ie);
                sm[pi] = mt;
                const float hv = ot * (sc[pi] / fmaxf(sn[pi], 1.0f));
                sh_last[pi] = hv;
                if (b0 + bb < B) Elem<T>::st(hs + ((size_t)(b0 + bb) * S + t) * D + hd * dh + u0 + u, hv);
                for (int r = 0; r < CL; ++r) cluster.map_shared_rank(hnext_local, r)[bb * dh + u0 + u] = hv;
            }
        }
        cluster.sync();  // every CTA holds the complete h_t; sPre may be overwritten
        cur ^= 1;
    }
#pragma unroll
    for (int pi = 0; pi < PPT; ++pi) {
        const int pr = tid + pi * REC_THREADS, bb = pr / U, u = pr % U;
        if (pr < REC_BG * U && b0 + bb < B) {
            const size_t so = (size_t)(b0 + bb) * D + hd * dh + u0 + u;
            c1[so] = sc[pi]; n1[so] = sn[pi]; m1[so] = sm[pi]; h1[so] = sh_last[pi];
        }
    }
}

template <typename T>
static int slstm_recurrent_launch(const void *gx, const void *R, const float *rb, const float *c0, const float *n0,
                                  const float *h0, const float *m0, void *hs, float *c1, float *n1, float *h1,
                                  float *m1, int B, int S, int NH, int dh, float cap, cudaStream_t st) {
    // units per CTA: at most 64, and the resident weight slice must fit in shared memory
    int CL = 1;
    auto slice_bytes = [&](int cl) { return (size_t)dh * 4 * (dh / cl) * sizeof(T); };
    while (CL <= 8 && (dh / CL > 64 || slice_bytes(CL) > 160 * 1024 || dh % CL)) CL *= 2;
    if (CL > 8 || dh % 4) return XLSTM_ERR_UNSUPPORTED;
    const int U = dh / CL;
    const size_t smem = slice_bytes(CL) + sizeof(float) * (2 * REC_BG * dh + REC_BG * 4 * U);
    auto kern = slstm_recurrent_kernel<T>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return XLSTM_ERR_CUDA;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(CL, NH, (B + REC_BG - 1) / REC_BG);
    cfg.blockDim = dim3(REC_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CL;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, static_cast<const T *>(gx), static_cast<const T *>(R), rb, c0, n0,
                                       h0, m0, static_cast<T *>(hs), c1, n1, h1, m1, B, S, NH, dh, U, cap);
    return e == cudaSuccess ? launch_status() : XLSTM_ERR_CUDA;
}

}  // namespace xl

namespace xl {
// tensor-core version (slstm_tc.cu): bf16, head dimension 256
bool slstm_recurrent_tc_supported(int dtype, int dh, const void *R, const void *gx, const void *hs);
int slstm_recurrent_tc_status(cudaStream_t st);
int slstm_recurrent_tc(const void *gx, const void *R, const float *rb, const float *c0, const float *n0, const float *h0,
                       const float *m0, void *hs, float *c1, float *n1, float *h1, float *m1, int B, int S, int NH,
                       float cap, cudaStream_t st);
}  // namespace xl

extern "C" int xlstm_slstm_scan(const void *z, const void *ig, const void *fg, const void *og, const float *c0,
                                const float *n0, const float *m0, void *h, float *c1, float *n1, float *m1, int B,
                                int S, int NH, int H, float eps, int dtype, void *stream) {
    if (!z || !ig || !fg || !og || !h || !c1 || !n1 || !m1) return XLSTM_ERR_INVALID;
    if (B <= 0 || S <= 0 || NH <= 0 || H <= 0) return XLSTM_ERR_INVALID;
    if (c0 && (!n0 || !m0)) return XLSTM_ERR_INVALID;
    if (dtype != XLSTM_F32 && dtype != XLSTM_BF16) return XLSTM_ERR_UNSUPPORTED;
    int threads = H >= 256 ? 256 : ((H + 31) / 32) * 32;
    if (H > threads * xl::SCAN_HPT) return XLSTM_ERR_UNSUPPORTED;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == XLSTM_F32)
        xl::slstm_scan_kernel<float><<<B * NH, threads, 0, st>>>(
            static_cast<const float *>(z), static_cast<const float *>(ig), static_cast<const float *>(fg),
            static_cast<const float *>(og), c0, n0, m0, static_cast<float *>(h), c1, n1, m1, S, NH, H, eps);
    else
        xl::slstm_scan_kernel<__nv_bfloat16><<<B * NH, threads, 0, st>>>(
            static_cast<const __nv_bfloat16 *>(z), static_cast<const __nv_bfloat16 *>(ig),
            static_cast<const __nv_bfloat16 *>(fg), static_cast<const __nv_bfloat16 *>(og), c0, n0, m0,
            static_cast<__nv_bfloat16 *>(h), c1, n1, m1, S, NH, H, eps);
    return xl::launch_status();
}

extern "C" int xlstm_slstm_recurrent(const void *gx, const void *R, const float *rb, const float *c0, const float *n0,
                                     const float *h0, const float *m0, void *hs, float *c1, float *n1, float *h1,
                                     float *m1, int B, int S, int NH, int dh, float cap, int dtype, void *stream) {
    if (!gx || !R || !rb || !hs || !c1 || !n1 || !h1 || !m1) return XLSTM_ERR_INVALID;
    if (B <= 0 || S <= 0 || NH <= 0 || dh <= 0) return XLSTM_ERR_INVALID;
    if (c0 && (!n0 || !h0 || !m0)) return XLSTM_ERR_INVALID;
    if (c0 && (c1 == c0 || n1 == n0 || h1 == h0 || m1 == m0)) return XLSTM_ERR_INVALID;
    if (dtype != XLSTM_F32 && dtype != XLSTM_BF16) return XLSTM_ERR_UNSUPPORTED;
    if (NH > 65535 || (B + xl::REC_BG - 1) / xl::REC_BG > 65535) return XLSTM_ERR_UNSUPPORTED;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (xl::slstm_recurrent_tc_supported(dtype, dh, R, gx, hs))
        return xl::slstm_recurrent_tc(gx, R, rb, c0, n0, h0, m0, hs, c1, n1, h1, m1, B, S, NH, cap, st);
    if (dtype == XLSTM_F32)
        return xl::slstm_recurrent_launch<float>(gx, R, rb, c0, n0, h0, m0, hs, c1, n1, h1, m1, B, S, NH, dh, cap, st);
    return xl::slstm_recurrent_launch<__nv_bfloat16>(gx, R, rb, c0, n0, h0, m0, hs, c1, n1, h1, m1, B, S, NH, dh, cap, st);
}

extern "C" int xlstm_slstm_recurrent_status(void *stream) {
    return xl::slstm_recurrent_tc_status(static_cast<cudaStream_t>(stream));
}
