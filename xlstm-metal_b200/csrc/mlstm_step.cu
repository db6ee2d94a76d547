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
#include <cooperative_groups.h>

#include "common.cuh"

namespace xl {

// tile shape (the measured best on B200): dv columns per CTA, threads, rows in flight per thread, CTAs per SM
constexpr int STEP_DVT = 64, STEP_THREADS = 256, STEP_UNROLL = 4, STEP_MIN_CTAS = 4;

// GATED: the output epilogue of the layer (per-head RMS norm x weight x sigmoid(output gate)) is applied before
// the result leaves the chip.  The CTAs of one head (its dv / DVT column tiles) are then launched as ONE CLUSTER
// and exchange their partial sums of squares through distributed shared memory: h is never written, `h` receives
// y[b, head*dv + j] = hn_j * w_j * sigmoid(og_j) in the [B, NH*dv] layout the out-projection reads.
struct StepGate {
    const void *ogate;      // [B rows, pitch ogate_ld elements], this head's columns at head*dv
    const void *norm_w;     // [NH*dv] or nullptr
    long long ogate_ld;
    float norm_eps;
    int NH;
};

template <typename T, int DVT, int THREADS, int UNROLL, bool GATED>
__global__ void __launch_bounds__(THREADS, STEP_MIN_CTAS)
mlstm_step_kernel(const T *__restrict__ q, const T *__restrict__ k, const T *__restrict__ v,
                  const T *__restrict__ ig, const T *__restrict__ fg,
                  const float *C0, const float *__restrict__ n0, const float *__restrict__ m0,
                  T *__restrict__ h, float *C1, float *__restrict__ n1, float *__restrict__ m1,
                  int dqk, int dv, float eps, float qscale, float gate_cap, int state_settled, StepGate gate) {
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
    if (!GATED) {
        if (tid < DVT && tile * DVT + tid < dv) {
            float t = 0.0f;
#pragma unroll
            for (int r = 0; r < RG; ++r) t += s_red[r * DVT + tid];
            Elem<T>::st(h + (size_t)bh * dv + tile * DVT + tid, t / s_den);
        }
    } else {
        namespace cg = cooperative_groups;
        static_assert(!GATED || DVT <= THREADS, "one thread per column of the tile");
        __shared__ float s_ss[2];          // [0..1]: the two warps' partial sums of squares; [0] then the CTA's
        cg::cluster_group cluster = cg::this_cluster();
        const bool col_ok = tid < DVT && tile * DVT + tid < dv;
        float hv = 0.0f;
        if (tid < DVT) {
            if (col_ok) {
                float t = 0.0f;
#pragma unroll
                for (int r = 0; r < RG; ++r) t += s_red[r * DVT + tid];
                // rounded to the activation type, as the separate epilogue kernel would read it back
                hv = sizeof(T) == 2 ? __bfloat162float(__float2bfloat16_rn(t / s_den)) : t / s_den;
            }
            const float ss = warp_sum(hv * hv);
            if ((tid & 31) == 0) s_ss[tid >> 5] = ss;
        }
        __syncthreads();
        if (tid == 0) s_ss[0] = s_ss[0] + (DVT > 32 ? s_ss[1] : 0.0f);
        cluster.sync();                    // every CTA of the head has its partial in s_ss[0]
        if (col_ok) {
            float tot = 0.0f;
            const unsigned nc = cluster.num_blocks();
            for (unsigned p = 0; p < nc; ++p) tot += cluster.map_shared_rank(s_ss, p)[0];
            const float inv = 1.0f / sqrtf(tot / (float)dv + gate.norm_eps);
            const int b = bh / gate.NH, head = bh % gate.NH;
            const int c = tile * DVT + tid;
            const float w = gate.norm_w ? Elem<T>::ld(static_cast<const T *>(gate.norm_w) + (size_t)head * dv + c) : 1.0f;
            const float og = Elem<T>::ld(static_cast<const T *>(gate.ogate) + (size_t)b * gate.ogate_ld + (size_t)head * dv + c);
            Elem<T>::st(h + (size_t)bh * dv + c, hv * inv * w * gate_sigmoid<T>(og));
        }
        cluster.sync();                    // nobody leaves while a peer still reads its shared memory
    }
}

template <typename T>
static int mlstm_step_launch(const void *q, const void *k, const void *v, const void *ig, const void *fg,
                             const float *C0, const float *n0, const float *m0, void *h, float *C1, float *n1,
                             float *m1, int BH, int dqk, int dv, float eps, float gate_cap, int state_settled,
                             const StepGate *gate, cudaStream_t st) {
    constexpr int DVT = STEP_DVT, THREADS = STEP_THREADS, UNROLL = STEP_UNROLL;
    dim3 grid(BH, (dv + DVT - 1) / DVT);
    size_t smem = sizeof(float) * (2 * (size_t)dqk + (THREADS / (DVT / 4)) * DVT);
    if (smem > 200 * 1024) return XLSTM_ERR_UNSUPPORTED;
    const float qscale = 1.0f / sqrtf((float)dqk);
    if (!gate) {
        auto kern = mlstm_step_kernel<T, DVT, THREADS, UNROLL, false>;
        if (smem > 48 * 1024 &&
            cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return XLSTM_ERR_CUDA;
        return launch_overlapped(kern, grid, dim3(THREADS), smem, st, static_cast<const T *>(q), static_cast<const T *>(k),
                                 static_cast<const T *>(v), static_cast<const T *>(ig), static_cast<const T *>(fg), C0, n0,
                                 m0, static_cast<T *>(h), C1, n1, m1, dqk, dv, eps, qscale, gate_cap, state_settled,
                                 StepGate{});
    }
    // fused output epilogue: the column tiles of a head form one cluster (portable size: at most 8)
    if (grid.y > 8) return XLSTM_ERR_UNSUPPORTED;
    auto kern = mlstm_step_kernel<T, DVT, THREADS, UNROLL, true>;
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return XLSTM_ERR_CUDA;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = 1;
    attr[1].val.clusterDim.y = grid.y;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    if (cudaLaunchKernelEx(&cfg, kern, static_cast<const T *>(q), static_cast<const T *>(k), static_cast<const T *>(v),
                           static_cast<const T *>(ig), static_cast<const T *>(fg), C0, n0, m0, static_cast<T *>(h), C1, n1, m1,
                           dqk, dv, eps, qscale, gate_cap, state_settled, *gate) != cudaSuccess)
        return XLSTM_ERR_CUDA;
    return launch_status();
}

}  // namespace xl

static int mlstm_step_checked(const void *q, const void *k, const void *v, const void *ig, const void *fg,
                              const float *C0, const float *n0, const float *m0, void *h, float *C1, float *n1,
                              float *m1, int B, int NH, int dqk, int dv, float eps, float gate_cap, int flags,
                              const xl::StepGate *gate, int dtype, void *stream) {
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
                                            settled, gate, st);
    return xl::mlstm_step_launch<__nv_bfloat16>(q, k, v, ig, fg, C0, n0, m0, h, C1, n1, m1, B * NH, dqk, dv, eps, gate_cap,
                                                settled, gate, st);
}

extern "C" int xlstm_mlstm_step(const void *q, const void *k, const void *v, const void *ig, const void *fg,
                                const float *C0, const float *n0, const float *m0, void *h, float *C1, float *n1,
                                float *m1, int B, int NH, int dqk, int dv, float eps, int dtype, void *stream) {
    return mlstm_step_checked(q, k, v, ig, fg, C0, n0, m0, h, C1, n1, m1, B, NH, dqk, dv, eps, 0.0f, 0, nullptr, dtype, stream);
}

extern "C" int xlstm_mlstm_step_gatecap(const void *q, const void *k, const void *v, const void *ig, const void *fg,
                                        const float *C0, const float *n0, const float *m0, void *h, float *C1,
                                        float *n1, float *m1, int B, int NH, int dqk, int dv, float eps, float gate_cap,
                                        int dtype, void *stream) {
    return mlstm_step_checked(q, k, v, ig, fg, C0, n0, m0, h, C1, n1, m1, B, NH, dqk, dv, eps, gate_cap, 0, nullptr, dtype, stream);
}

extern "C" int xlstm_mlstm_step_ex(const void *q, const void *k, const void *v, const void *ig, const void *fg,
                                   const float *C0, const float *n0, const float *m0, void *h, float *C1, float *n1,
                                   float *m1, int B, int NH, int dqk, int dv, float eps, float gate_cap, int flags,
                                   int dtype, void *stream) {
    return mlstm_step_checked(q, k, v, ig, fg, C0, n0, m0, h, C1, n1, m1, B, NH, dqk, dv, eps, gate_cap, flags, nullptr, dtype, stream);
}

extern "C" int xlstm_mlstm_step_gated(const void *q, const void *k, const void *v, const void *ig, const void *fg,
                                      const float *C0, const float *n0, const float *m0, const void *ogate,
                                      int64_t ogate_ld, const void *norm_w, float norm_eps, void *y, float *C1, float *n1,
                                      float *m1, int B, int NH, int dqk, int dv, float eps, float gate_cap, int flags,
                                      int dtype, void *stream) {
    if (!ogate || ogate_ld < (int64_t)NH * dv) return XLSTM_ERR_INVALID;
    xl::StepGate g;
    g.ogate = ogate;
    g.norm_w = norm_w;
    g.ogate_ld = ogate_ld;
    g.norm_eps = norm_eps;
    g.NH = NH;
    return mlstm_step_checked(q, k, v, ig, fg, C0, n0, m0, y, C1, n1, m1, B, NH, dqk, dv, eps, gate_cap, flags, &g, dtype,
                              stream);
}
