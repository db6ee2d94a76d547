// State-only scan for the segment-parallel prefill: the end state (C, n) of every segment from an EMPTY state.
//
// The first pass of the segment-parallel mode needs no outputs, only the local end states that the combine step
// turns into the true start state of every segment.  Of the four MMA groups of the forward kernel that leaves
// the state update C~ += K^T V~ alone: no Q, no S / P, no read-out, no bf16 copy of C, no epilogue.  With Q and
// Cb gone, K and V fit twice into shared memory, so the loads of tile k+1 run under the MMAs of tile k and the
// tile period is the update itself.  Same factorisation as the bounded-spread forward kernel (a_s = e^{u_s - m - rho}
// on the V rows, C~ = C e^{-rho}, one multiplication of C~ when -rho passes the threshold), same gate scratch,
// same grid (one CTA per (batch, head, segment) and 128 dv columns); segments whose gates need the general
// kernel are left to it (path flag).
//
// Roles (640 threads): warp 0 TMA producer (two stages of K and V), warp 1 MMA issuer (+TMEM alloc), warps 4-7
// V~ = diag(a) V in place, warps 8-11 n~ += K^T a, warps 12-15 / 16-19 the rows [0,128) / [128,256) of C~:
// the occasional rescale in TMEM and, after the last tile, the fp32 state to global memory.
// Every mbarrier wait is bounded; a time-out sets the status word, releases all roles and frees TMEM.
#include "mlstm_chunkwise_tc.cuh"

namespace xl {

namespace {

using namespace tc;
using namespace tcw;

enum { S_KFULL0 = 0, S_KFULL1, S_VFULL0, S_VFULL1, S_VSCALED0, S_VSCALED1, S_UPD0, S_UPD1, S_NREAD0, S_NREAD1, S_CFREE,
       S_NBARS };

template <int DQK> struct ScanSmem {
    static constexpr int NBOX = DQK / 64;
    static constexpr uint32_t BOX = LT * 128;
    static constexpr uint32_t KSTAGE = NBOX * BOX, VSTAGE = 2 * BOX;
    static constexpr uint32_t K = 0;                       // two stages
    static constexpr uint32_t V = K + 2 * KSTAGE;          // two stages
    static constexpr uint32_t N_VEC = V + 2 * VSTAGE;      // float[DQK]
    static constexpr uint32_t BARS = N_VEC + DQK * 4;
    static constexpr uint32_t MISC = BARS + 16 * 8;
    static constexpr uint32_t TOTAL = MISC + 16;
};

template <int DQK>
__global__ void __launch_bounds__(THREADS, 1) mlstm_chunkwise_tc_scan_kernel(const __grid_constant__ TcParams p) {
    using SM = ScanSmem<DQK>;
    constexpr int NBOX = SM::NBOX;
    constexpr int NHALF = DQK / 128;
    extern __shared__ __align__(1024) unsigned char smem[];
    const int bh = blockIdx.x;     // (batch, head, segment)
    if (p.path[bh] != 1) return;   // this segment's gates need the general kernel

    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + SM::BARS);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + SM::MISC);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + SM::MISC + 4);
    float *s_n = reinterpret_cast<float *>(smem + SM::N_VEC);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int bhr = bh / p.P, tile0 = (bh % p.P) * p.seg_tiles;
    const int b = bhr / p.NH, hd = bhr % p.NH;
    const int col0 = blockIdx.y * DVS;
    const int NCH = min(p.seg_tiles, p.NCH - tile0);
    const float *gbase = p.gates + ((size_t)bhr * p.NCH + tile0) * GW;

    if (tid == 0) {
        *abort_flag = (smem_u32(smem) & 1023u) ? 1 : 0;
        for (int s = 0; s < 2; ++s) {
            mbar_init(&bars[S_KFULL0 + s], 1);     mbar_init(&bars[S_VFULL0 + s], 1);
            mbar_init(&bars[S_VSCALED0 + s], 128); mbar_init(&bars[S_UPD0 + s], 1);
            mbar_init(&bars[S_NREAD0 + s], 128);
        }
        mbar_init(&bars[S_CFREE], 128 * NHALF);
        mbar_fence_init();
        tma_prefetch_desc(&p.tk); tma_prefetch_desc(&p.tv);
    }
    if (warp == 1) tmem_alloc(tmem_slot, 256);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t T_C = *tmem_slot;

    if (warp == 0) {
        // ================= TMA producer: stage k & 1 is free once the update and the n pass of tile k-2 are done =================
        if (lane == 0) {
            for (int k = 0; k < NCH; ++k) {
                const int s = k & 1, t0 = (tile0 + k) * LT;
                const uint32_t pp = ((k >> 1) - 1) & 1;   // parity of the stage's previous use
                if (k >= 2 && !(mbar_wait(&bars[S_UPD0 + s], pp, abort_flag) && mbar_wait(&bars[S_NREAD0 + s], pp, abort_flag))) break;
                mbar_expect_tx(&bars[S_KFULL0 + s], NBOX * SM::BOX);
                for (int q = 0; q < NBOX; ++q)
                    tma_load_4d(smem + SM::K + s * SM::KSTAGE + q * SM::BOX, &p.tk, &bars[S_KFULL0 + s], q * 64, t0, hd, b);
                mbar_expect_tx(&bars[S_VFULL0 + s], 2 * SM::BOX);
                for (int q = 0; q < 2; ++q)
                    tma_load_4d(smem + SM::V + s * SM::VSTAGE + q * SM::BOX, &p.tv, &bars[S_VFULL0 + s], col0 + q * 64, t0, hd, b);
            }
        }
    } else if (warp == 1) {
        // ================= MMA issuer: C~ += K^T V~ (the first tile overwrites: the segment starts from an empty state) =================
        if (lane == 0) {
            constexpr uint32_t ID_MM = idesc_bf16(128, 128, true, true);
            for (int k = 0; k < NCH; ++k) {
                const int s = k & 1;
                const uint32_t ph = (k >> 1) & 1;
                const uint64_t dKm = smem_desc_sw128(smem_u32(smem + SM::K + s * SM::KSTAGE), SM::BOX, 1024);
                const uint64_t dV = smem_desc_sw128(smem_u32(smem + SM::V + s * SM::VSTAGE), SM::BOX, 1024);
                if (!(mbar_wait(&bars[S_KFULL0 + s], ph, abort_flag) && mbar_wait(&bars[S_VSCALED0 + s], ph, abort_flag))) break;
                if (k > 0 && !mbar_wait(&bars[S_CFREE], (k - 1) & 1, abort_flag)) break;   // rescale of C~ (if any) has finished
                tc_fence_after_sync();
#pragma unroll
                for (int hf = 0; hf < NHALF; ++hf)
#pragma unroll
                    for (int kk = 0; kk < LT / 16; ++kk)
                        mma_ss(T_C + hf * 128, dKm + ((hf * 2 * SM::BOX + kk * 2048) >> 4), dV + kk * (2048 >> 4), ID_MM,
                               k > 0 || kk > 0);
                mma_commit(&bars[S_UPD0 + s]);
            }
        }
    } else if (warp >= 4 && warp < 8) {
        // ================= V~ = diag(a) V in place =================
        const int t = tid - 128;
        for (int k = 0; k < NCH; ++k) {
            const int s = k & 1;
            const float a = gbase[(size_t)k * GW + G_W + t];
            if (!mbar_wait(&bars[S_VFULL0 + s], (k >> 1) & 1, abort_flag)) break;
            scale_tile_rows<2>(smem + SM::V + s * SM::VSTAGE, SM::BOX, t, a);
            fence_proxy_async_smem();
            mbar_arrive(&bars[S_VSCALED0 + s]);
        }
    } else if (warp >= 8 && warp < 12) {
        // ================= n~ = (n~ + K^T a) * mul =================
        const int r = tid - 256;
        const int q = r >> 5, cp = r & 31;   // warp -> 64-column box of K, lane -> column pair
        for (int j = r; j < DQK; j += 128) s_n[j] = 0.f;
        for (int k = 0; k < NCH; ++k) {
            const int s = k & 1;
            const float *g = gbase + (size_t)k * GW;
            const bool last = (k == NCH - 1);
            const float mul = g[G_SCAL + 0], frame = g[G_SCAL + 2];
            const float *ga = g + G_W;   // a_s straight from the gate scratch (same address in every lane: one L1 line per load)
            if (!mbar_wait(&bars[S_KFULL0 + s], (k >> 1) & 1, abort_flag)) break;
            if (q < NBOX) {
                const unsigned char *box = smem + SM::K + s * SM::KSTAGE + q * SM::BOX + ((cp & 3) << 2);
                float a0[4] = {0.f, 0.f, 0.f, 0.f}, a1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 8
                for (int tt = 0; tt < LT; tt += 4) {
                    const float4 av = *reinterpret_cast<const float4 *>(ga + tt);
                    const float aw[4] = {av.x, av.y, av.z, av.w};
#pragma unroll
                    for (int x = 0; x < 4; ++x) {
                        const uint32_t off = (tt + x) * 128 + ((((cp >> 2) ^ ((tt + x) & 7))) << 4);
                        const float2 f = unpack_bf16(*reinterpret_cast<const uint32_t *>(box + off));
                        a0[x] = fmaf(f.x, aw[x], a0[x]); a1[x] = fmaf(f.y, aw[x], a1[x]);
                    }
                }
                const int j = q * 64 + cp * 2;
                const float n0v = s_n[j] + (a0[0] + a0[1]) + (a0[2] + a0[3]);
                const float n1v = s_n[j + 1] + (a1[0] + a1[1]) + (a1[2] + a1[3]);
                s_n[j] = n0v * mul;
                s_n[j + 1] = n1v * mul;
                if (last && blockIdx.y == 0) {
                    p.n1[(size_t)bh * DQK + j] = n0v * frame; p.n1[(size_t)bh * DQK + j + 1] = n1v * frame;
                }
            }
            mbar_arrive(&bars[S_NREAD0 + s]);
        }
    } else if (warp >= 12 && warp - 12 < 4 * NHALF) {
        // ================= rows of C~: rescale when the frame calls for it; after the last tile the state goes out =================
        const int hf = (warp - 12) >> 2;
        const int r = (tid - 384) & 127;
        const uint32_t t_half = T_C + hf * 128 + ((uint32_t)(r & ~31) << 16);
        float *dst = p.C1 + ((size_t)bh * DQK + hf * 128 + r) * p.dv + col0;
        for (int k = 0; k < NCH; ++k) {
            const float *g = gbase + (size_t)k * GW;
            const bool last = (k == NCH - 1);
            const float mul = g[G_SCAL + 0], frame = g[G_SCAL + 2];
            if (!mbar_wait(&bars[S_UPD0 + (k & 1)], (k >> 1) & 1, abort_flag)) break;
            tc_fence_after_sync();
            if (last || mul != 1.0f) {
#pragma unroll 1
                for (int c0 = 0; c0 < DVS; c0 += 32) {
                    uint32_t va[32];
                    tmem_ld32(t_half + c0, va);
                    tmem_wait_ld();
                    if (last) {
#pragma unroll
                        for (int x = 0; x < 32; x += 4)
                            *reinterpret_cast<float4 *>(dst + c0 + x) =
                                make_float4(__uint_as_float(va[x]) * frame, __uint_as_float(va[x + 1]) * frame,
                                            __uint_as_float(va[x + 2]) * frame, __uint_as_float(va[x + 3]) * frame);
                    } else {
#pragma unroll
                        for (int x = 0; x < 32; ++x) va[x] = __float_as_uint(__uint_as_float(va[x]) * mul);
                        tmem_st32(t_half + c0, va);
                    }
                }
                tmem_wait_st();
            }
            tc_fence_before_sync();
            if (!last) mbar_arrive(&bars[S_CFREE]);
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(T_C, 256);
    if (tid == 0 && *abort_flag) atomicExch(p.status, 1);
}

}  // namespace

int mlstm_chunkwise_tc_scan_launch(const tcw::TcParams &tp, dim3 grid, int dqk, cudaStream_t st) {
    if (dqk == 256) {
        auto kern = mlstm_chunkwise_tc_scan_kernel<256>;
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ScanSmem<256>::TOTAL) != cudaSuccess)
            return XLSTM_ERR_CUDA;
        kern<<<grid, THREADS, ScanSmem<256>::TOTAL, st>>>(tp);
    } else {
        auto kern = mlstm_chunkwise_tc_scan_kernel<128>;
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ScanSmem<128>::TOTAL) != cudaSuccess)
            return XLSTM_ERR_CUDA;
        kern<<<grid, THREADS, ScanSmem<128>::TOTAL, st>>>(tp);
    }
    return cudaGetLastError() == cudaSuccess ? XLSTM_OK : XLSTM_ERR_CUDA;
}

}  // namespace xl
