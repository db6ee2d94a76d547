// Chunkwise mLSTM forward on CUDA cores, all arithmetic in fp32.
//
// This is the exact path: fp32 inputs keep 1e-6-class agreement with the
// step-by-step recurrence, and it accepts any shape (partial last chunk,
// dqk/dv that are not tile multiples).  The bf16 tensor-core path covers the
// production shapes; both implement the same per-chunk algebra:
//
//   b_t = cumsum logsig(f),  m_t = b_t + max(m, max_{s<=t}(i_s - b_s)),  m' = m_{L-1}
//   h_t = [e^{b_t+m-m_t} q~ C + sum_{s<=t} e^{b_t-b_s+i_s-m_t} (q~.k_s) v_s] / (max(|den_t|, e^{-m_t}) + eps)
//   C'  = e^{b_{L-1}+m-m'} C + sum_t e^{b_{L-1}-b_t+i_t-m'} k_t (x) v_t      (n' likewise)
//
// One CTA owns a 64-column slice of one head's C (kept in shared memory for the
// whole sequence) and walks the chunks in order.  Q and K stream through shared
// memory in 64-wide pieces of dqk; per piece the CTA accumulates Q K^T, reads
// the old C rows out (q~ C), then updates those rows in place.
#include "mlstm_chunkwise.cuh"

namespace xl {

namespace {

constexpr int LT = 64;    // chunk tile (tokens)
constexpr int DVT = 64;   // dv columns per CTA
constexpr int KP = 64;    // dqk piece
constexpr int LDP = KP + 4;  // padded row of the Q/K/P tiles (keeps float4 alignment, spreads banks)
constexpr int THREADS = 256;

template <typename T>
__device__ __forceinline__ void load_tile(float *dst, int ld, const T *src, int64_t row_stride, int rows_valid,
                                          int col0, int cols_valid_total, int tile_cols) {
    // dst[r][c] = src[r*row_stride + col0 + c] for r < rows_valid, col0 + c < cols_valid_total, else 0
    const int vec_per_row = tile_cols / 4;
    for (int e = threadIdx.x; e < LT * vec_per_row; e += THREADS) {
        const int r = e / vec_per_row, c = (e % vec_per_row) * 4;
        float4 val = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r < rows_valid && col0 + c < cols_valid_total) val = ld4(src + (int64_t)r * row_stride + col0 + c);
        *reinterpret_cast<float4 *>(dst + r * ld + c) = val;
    }
}

template <typename T>
__global__ void __launch_bounds__(THREADS, 1) mlstm_chunkwise_simt_kernel(ChunkwiseParams p, int dqkp) {
    extern __shared__ __align__(16) float smem[];
    float *sC = smem;                    // [dqkp][DVT]
    float *sN = sC + dqkp * DVT;         // [dqkp]
    float *sQ = sN + dqkp;               // [LT][LDP]
    float *sK = sQ + LT * LDP;           // [LT][LDP]
    float *sP = sK + LT * LDP;           // [LT][LDP]
    float *sV = sP + LT * LDP;           // [LT][DVT]
    float *sVw = sV + LT * DVT;          // [LT][DVT]  rows scaled by the state-update weights
    float *sFl = sVw + LT * DVT;         // [LT] logsig(f)
    float *sI = sFl + LT;                // [LT] i
    float *sM = sI + LT;                 // [LT] m_t
    float *sWin = sM + LT;               // [LT] e^{b_t+m-m_t}
    float *sW = sWin + LT;               // [LT] e^{a_t-m'}
    float *sQn = sW + LT;                // [LT] q~ . n
    float *sRow = sQn + LT;              // [LT] row sums of P
    __shared__ float s_m;                // carried stabiliser
    __shared__ double sBd[LT], sUd[LT], sXd[LT];  // cumsum b, u = i - b, running max x

    const int tid = threadIdx.x, tx = tid % 16, ty = tid / 16;
    const int bh = blockIdx.x, b = bh / p.NH, hd = bh % p.NH;
    const int col0 = blockIdx.y * DVT;
    const int dqk = p.dqk, dv = p.dv, L = p.L;
    const bool has_state = p.C0 != nullptr;

    const T *qb = static_cast<const T *>(p.q) + b * p.sq[0] + hd * p.sq[1];
    const T *kb = static_cast<const T *>(p.k) + b * p.sk[0] + hd * p.sk[1];
    const T *vb = static_cast<const T *>(p.v) + b * p.sv[0] + hd * p.sv[1];
    T *hb = static_cast<T *>(p.h) + b * p.sh[0] + hd * p.sh[1];
    const T *ib = static_cast<const T *>(p.ig) + b * p.sg[0] + hd * p.sg[1];
    const T *fb = static_cast<const T *>(p.fg) + b * p.sg[0] + hd * p.sg[1];

    // initial state
    for (int e = tid; e < dqkp * (DVT / 4); e += THREADS) {
        const int j = e / (DVT / 4), c = (e % (DVT / 4)) * 4;
        float4 val = make_float4(0.f, 0.f, 0.f, 0.f);
        if (has_state && j < dqk && col0 + c < dv) val = ld4(p.C0 + ((size_t)bh * dqk + j) * dv + col0 + c);
        *reinterpret_cast<float4 *>(sC + j * DVT + c) = val;
    }
    for (int j = tid; j < dqkp; j += THREADS) sN[j] = (has_state && j < dqk) ? p.n0[(size_t)bh * dqk + j] : 0.f;
    if (tid == 0) s_m = has_state ? p.m0[bh] : 0.f;
    __syncthreads();

    const int NC = (p.S + L - 1) / L;
    for (int ch = 0; ch < NC; ++ch) {
        const int t0 = ch * L;
        const int Lc = min(L, p.S - t0);
        const float m_old = s_m;

        // ---- gates ------------------------------------------------------
        // With u_s = i_s - b_s and x_t = max(m, max_{s<=t} u_s):  m_t = b_t + x_t, and every
        // exponent of the chunk is a difference u_s - x_t (or m - x_t).  b can reach
        // ~1e3 in a chunk of strongly negative forget gates, so u and x are kept
        // in double: the differences stay exact to fp32 rounding of the result.
        if (tid < LT) {
            const bool valid = tid < Lc;
            sFl[tid] = valid ? logsigmoid(gate_softcap(Elem<T>::ld(fb + (int64_t)(t0 + tid) * p.sg[2]), p.gate_cap)) : 0.f;
            sI[tid] = valid ? gate_softcap(Elem<T>::ld(ib + (int64_t)(t0 + tid) * p.sg[2]), p.gate_cap) : -INFINITY;
        }
        __syncthreads();
        if (tid < LT) {
            double acc = 0.0;
            for (int s = 0; s <= tid; ++s) acc += (double)sFl[s];
            sBd[tid] = acc;
            sUd[tid] = (double)sI[tid] - acc;
        }
        __syncthreads();
        if (tid < LT) {
            double mx = (double)m_old;
            for (int s = 0; s <= tid; ++s) mx = fmax(mx, sUd[s]);
            sXd[tid] = mx;
            sM[tid] = (float)(sBd[tid] + mx);
            sWin[tid] = expf((float)((double)m_old - mx));  // e^{b_t + m - m_t}
            sQn[tid] = 0.f;
        }
        __syncthreads();
        const double x_last = sXd[LT - 1];
        const float m_new = sM[LT - 1];
        const float decay = expf((float)((double)m_old - x_last));          // e^{G + m - m'}
        if (tid < LT) sW[tid] = expf((float)(sUd[tid] - x_last));           // e^{a_t - m'}; 0 for masked tokens

        // ---- V tile -----------------------------------------------------
        load_tile<T>(sV, DVT, vb + (int64_t)t0 * p.sv[2], p.sv[2], Lc, col0, dv, DVT);
        __syncthreads();
        for (int e = tid; e < LT * DVT; e += THREADS) sVw[e] = sW[e / DVT] * sV[e];

        float sacc[4][4], hacc[4][4];
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int c = 0; c < 4; ++c) { sacc[a][c] = 0.f; hacc[a][c] = 0.f; }

        for (int j0 = 0; j0 < dqkp; j0 += KP) {
            __syncthreads();  // previous piece fully consumed
            load_tile<T>(sQ, LDP, qb + (int64_t)t0 * p.sq[2], p.sq[2], Lc, j0, dqk, KP);
            load_tile<T>(sK, LDP, kb + (int64_t)t0 * p.sk[2], p.sk[2], Lc, j0, dqk, KP);
            __syncthreads();

            // phase 1: S[t][s] += Q[t][.] . K[s][.]   t = ty+16a, s = tx+16c
#pragma unroll 4
            for (int jj = 0; jj < KP; jj += 4) {
                float4 qa[4], kc[4];
#pragma unroll
                for (int a = 0; a < 4; ++a) qa[a] = *reinterpret_cast<const float4 *>(sQ + (ty + 16 * a) * LDP + jj);
#pragma unroll
                for (int c = 0; c < 4; ++c) kc[c] = *reinterpret_cast<const float4 *>(sK + (tx + 16 * c) * LDP + jj);
#pragma unroll
                for (int a = 0; a < 4; ++a)
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        sacc[a][c] = fmaf(qa[a].x, kc[c].x, sacc[a][c]);
                        sacc[a][c] = fmaf(qa[a].y, kc[c].y, sacc[a][c]);
                        sacc[a][c] = fmaf(qa[a].z, kc[c].z, sacc[a][c]);
                        sacc[a][c] = fmaf(qa[a].w, kc[c].w, sacc[a][c]);
                    }
            }
            // phase 2: H[t][c] += Q[t][j] C_old[j][c]   t = ty+16a, c = 4tx..4tx+3
#pragma unroll 2
            for (int jj = 0; jj < KP; jj += 4) {
                float4 qa[4], cr[4];
#pragma unroll
                for (int a = 0; a < 4; ++a) qa[a] = *reinterpret_cast<const float4 *>(sQ + (ty + 16 * a) * LDP + jj);
#pragma unroll
                for (int r = 0; r < 4; ++r) cr[r] = *reinterpret_cast<const float4 *>(sC + (j0 + jj + r) * DVT + 4 * tx);
#pragma unroll
                for (int a = 0; a < 4; ++a) {
                    const float qv[4] = {qa[a].x, qa[a].y, qa[a].z, qa[a].w};
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        hacc[a][0] = fmaf(qv[r], cr[r].x, hacc[a][0]);
                        hacc[a][1] = fmaf(qv[r], cr[r].y, hacc[a][1]);
                        hacc[a][2] = fmaf(qv[r], cr[r].z, hacc[a][2]);
                        hacc[a][3] = fmaf(qv[r], cr[r].w, hacc[a][3]);
                    }
                }
            }
            // q . n_old for this piece (threads 64..127, one token each)
            if (tid >= 64 && tid < 64 + LT) {
                const int t = tid - 64;
                float acc = 0.f;
                for (int jj = 0; jj < KP; ++jj) acc = fmaf(sQ[t * LDP + jj], sN[j0 + jj], acc);
                sQn[t] += acc;
            }
            __syncthreads();

            // phase 3: C[j][c] = decay*C[j][c] + sum_t K[t][j] Vw[t][c]   j = j0+4ty..+3, c = 4tx..+3
            {
                float cacc[4][4];
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const float4 c4 = *reinterpret_cast<const float4 *>(sC + (j0 + 4 * ty + r) * DVT + 4 * tx);
                    cacc[r][0] = decay * c4.x; cacc[r][1] = decay * c4.y;
                    cacc[r][2] = decay * c4.z; cacc[r][3] = decay * c4.w;
                }
#pragma unroll 4
                for (int t = 0; t < LT; ++t) {
                    const float4 k4 = *reinterpret_cast<const float4 *>(sK + t * LDP + 4 * ty);
                    const float4 v4 = *reinterpret_cast<const float4 *>(sVw + t * DVT + 4 * tx);
                    const float kv[4] = {k4.x, k4.y, k4.z, k4.w};
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        cacc[r][0] = fmaf(kv[r], v4.x, cacc[r][0]);
                        cacc[r][1] = fmaf(kv[r], v4.y, cacc[r][1]);
                        cacc[r][2] = fmaf(kv[r], v4.z, cacc[r][2]);
                        cacc[r][3] = fmaf(kv[r], v4.w, cacc[r][3]);
                    }
                }
#pragma unroll
                for (int r = 0; r < 4; ++r)
                    *reinterpret_cast<float4 *>(sC + (j0 + 4 * ty + r) * DVT + 4 * tx) =
                        make_float4(cacc[r][0], cacc[r][1], cacc[r][2], cacc[r][3]);
            }
            // n[j] = decay*n[j] + sum_t w_t K[t][j]   (threads 0..63, one row each)
            if (tid < KP) {
                float acc = decay * sN[j0 + tid];
                for (int t = 0; t < LT; ++t) acc = fmaf(sW[t], sK[t * LDP + tid], acc);
                sN[j0 + tid] = acc;
            }
        }

        // ---- gate matrix, P = S * D, row sums -----------------------------
#pragma unroll
        for (int a = 0; a < 4; ++a) {
            const int t = ty + 16 * a;
            const double xt = sXd[t];
            float rs = 0.f;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int s = tx + 16 * c;
                float pv = 0.f;
                if (s <= t) pv = sacc[a][c] * p.qscale * expf((float)(sUd[s] - xt));
                sP[t * LDP + s] = pv;
                rs += pv;
            }
            rs += __shfl_xor_sync(0xffffffffu, rs, 8);
            rs += __shfl_xor_sync(0xffffffffu, rs, 4);
            rs += __shfl_xor_sync(0xffffffffu, rs, 2);
            rs += __shfl_xor_sync(0xffffffffu, rs, 1);
            if (tx == 0) sRow[t] = rs;
        }
        __syncthreads();

        // ---- intra-chunk read-out, combine, normalise -----------------------
#pragma unroll
        for (int a = 0; a < 4; ++a) {
            const float w = sWin[ty + 16 * a] * p.qscale;
#pragma unroll
            for (int c = 0; c < 4; ++c) hacc[a][c] *= w;
        }
#pragma unroll 2
        for (int s = 0; s < LT; s += 4) {
            float4 pa[4], vr[4];
#pragma unroll
            for (int a = 0; a < 4; ++a) pa[a] = *reinterpret_cast<const float4 *>(sP + (ty + 16 * a) * LDP + s);
#pragma unroll
            for (int r = 0; r < 4; ++r) vr[r] = *reinterpret_cast<const float4 *>(sV + (s + r) * DVT + 4 * tx);
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                const float pv[4] = {pa[a].x, pa[a].y, pa[a].z, pa[a].w};
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    hacc[a][0] = fmaf(pv[r], vr[r].x, hacc[a][0]);
                    hacc[a][1] = fmaf(pv[r], vr[r].y, hacc[a][1]);
                    hacc[a][2] = fmaf(pv[r], vr[r].z, hacc[a][2]);
                    hacc[a][3] = fmaf(pv[r], vr[r].w, hacc[a][3]);
                }
            }
        }
#pragma unroll
        for (int a = 0; a < 4; ++a) {
            const int t = ty + 16 * a;
            if (t < Lc && col0 + 4 * tx < dv) {
                const float den = sWin[t] * p.qscale * sQn[t] + sRow[t];
                const float inv = 1.0f / (fmaxf(fabsf(den), expf(-sM[t])) + p.eps);
                st4(hb + (int64_t)(t0 + t) * p.sh[2] + col0 + 4 * tx,
                    make_float4(hacc[a][0] * inv, hacc[a][1] * inv, hacc[a][2] * inv, hacc[a][3] * inv));
            }
        }
        __syncthreads();
        if (tid == 0) s_m = m_new;
        __syncthreads();
    }

    // ---- final state --------------------------------------------------------
    for (int e = tid; e < dqk * (DVT / 4); e += THREADS) {
        const int j = e / (DVT / 4), c = (e % (DVT / 4)) * 4;
        if (col0 + c < dv)
            *reinterpret_cast<float4 *>(p.C1 + ((size_t)bh * dqk + j) * dv + col0 + c) =
                *reinterpret_cast<const float4 *>(sC + j * DVT + c);
    }
    if (blockIdx.y == 0) {
        for (int j = tid; j < dqk; j += THREADS) p.n1[(size_t)bh * dqk + j] = sN[j];
        if (tid == 0) p.m1[bh] = s_m;
    }
}

}  // namespace

int mlstm_chunkwise_simt(const ChunkwiseParams &p_in, int dtype, cudaStream_t st) {
    if (p_in.L < 1) return XLSTM_ERR_UNSUPPORTED;
    // The chunkwise form is a re-association of the recurrence: any internal tile gives the same result, so a
    // chunk size beyond the kernel's tile is walked in tiles of LT tokens instead of being refused.
    ChunkwiseParams p = p_in;
    if (p.L > LT) p.L = LT;
    if (p.dqk % 4 || p.dv % 4) return XLSTM_ERR_UNSUPPORTED;
    for (int d = 0; d < 3; ++d)
        if (p.sq[d] % 4 || p.sk[d] % 4 || p.sv[d] % 4 || p.sh[d] % 4) return XLSTM_ERR_UNSUPPORTED;
    const size_t esz = dtype == XLSTM_F32 ? 4 : 2;
    const uintptr_t mask = 4 * esz - 1;
    if ((reinterpret_cast<uintptr_t>(p.q) | reinterpret_cast<uintptr_t>(p.k) | reinterpret_cast<uintptr_t>(p.v) |
         reinterpret_cast<uintptr_t>(p.h)) & mask)
        return XLSTM_ERR_UNSUPPORTED;
    const int dqkp = (p.dqk + KP - 1) / KP * KP;
    const size_t smem = sizeof(float) * ((size_t)dqkp * DVT + dqkp + 3 * LT * LDP + 2 * LT * DVT + 7 * LT);
    if (smem > 227 * 1024) return XLSTM_ERR_UNSUPPORTED;
    dim3 grid(p.B * p.NH, (p.dv + DVT - 1) / DVT);
    if (dtype == XLSTM_F32) {
        auto kern = mlstm_chunkwise_simt_kernel<float>;
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return XLSTM_ERR_CUDA;
        kern<<<grid, THREADS, smem, st>>>(p, dqkp);
    } else {
        auto kern = mlstm_chunkwise_simt_kernel<__nv_bfloat16>;
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return XLSTM_ERR_CUDA;
        kern<<<grid, THREADS, smem, st>>>(p, dqkp);
    }
    return launch_status();
}

}  // namespace xl
