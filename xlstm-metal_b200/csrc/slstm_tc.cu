// Block-diagonal recurrent sLSTM on the tensor cores (bf16, head dim 256): the sequential loop over t
// with the four recurrent matrices resident in TENSOR MEMORY for the whole sequence.
//
// One cluster of 4 CTAs per (head, 32 batch rows); CTA `rank` owns 64 of the head's 256 units, i.e. 256
// gate-output rows (4 gates x 64 units) of R_g.  Per step the CTA needs pre[m][b] = sum_k R[m][k] h_{t-1}[b][k]
// for its 256 rows m and 32 batch rows b: two groups of 16 tcgen05.mma (M=128, N=32, K=16) with
//   A = the CTA's slice of R, bf16, written once into TMEM (2 x 128 columns),
//   B = h_{t-1} [32 x 256] bf16 in shared memory (128-byte swizzle, K-major, 16 KB, double-buffered),
//   D = fp32 in TMEM (2 x 32 columns).
// The accumulators go through shared memory to the threads that own (unit, batch row) cells, which add
// the input-side pre-activations, run the gating, write h_t to global memory and, as bf16, into the
// B buffer of the next step in all four CTAs (distributed shared memory); one cluster barrier per
// step.  Only the MMA's smem traffic is the 1 KB of h per instruction: R is never re-read from
// shared memory (the CUDA-core version reads its 128 KB slice every step).
#include <cooperative_groups.h>

#include "common.cuh"
#include "tcgen05.cuh"

namespace cg = cooperative_groups;

namespace xl {
namespace {
using namespace tc;

constexpr int TCR_THREADS = 256;
constexpr int TCR_NB = 32;     // batch rows per cluster = N of the MMA
constexpr int TCR_U = 64;      // units per CTA
constexpr int TCR_DH = 256;    // head dimension = K of the MMA
constexpr int TCR_CL = 4;      // CTAs per cluster
constexpr int TCR_PAD = 33;    // row pitch of the accumulator staging (floats): conflict-free both ways
constexpr uint32_t TCR_BBOX = TCR_NB * 128;              // one 64-column box of h: 32 rows x 128 B
constexpr uint32_t TCR_BBUF = (TCR_DH / 64) * TCR_BBOX;  // 16 KB
constexpr uint32_t TCR_OFF_PRE = 2 * TCR_BBUF;
constexpr uint32_t TCR_OFF_BAR = TCR_OFF_PRE + 4 * TCR_U * TCR_PAD * 4;
constexpr uint32_t TCR_SMEM = TCR_OFF_BAR + 32;

__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

__global__ void __launch_bounds__(TCR_THREADS, 1)
slstm_recurrent_tc_kernel(const __nv_bfloat16 *__restrict__ gx, const __nv_bfloat16 *__restrict__ R,
                          const float *__restrict__ rb, const float *__restrict__ c0, const float *__restrict__ n0,
                          const float *__restrict__ h0, const float *__restrict__ m0, __nv_bfloat16 *__restrict__ hs,
                          float *__restrict__ c1, float *__restrict__ n1, float *__restrict__ h1, float *__restrict__ m1,
                          int B, int S, int NH, float cap) {
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = (int)cluster.block_rank();
    const int hd = blockIdx.y, b0 = blockIdx.z * TCR_NB;
    const int D = NH * TCR_DH, u0 = rank * TCR_U;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    extern __shared__ __align__(1024) unsigned char smem[];
    float *sPre = reinterpret_cast<float *>(smem + TCR_OFF_PRE);       // [4*64 rows m][TCR_PAD]
    uint64_t *bar = reinterpret_cast<uint64_t *>(smem + TCR_OFF_BAR);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + TCR_OFF_BAR + 8);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + TCR_OFF_BAR + 12);

    if (tid == 0) {
        *abort_flag = (smem_u32(smem) & 1023u) ? 1 : 0;
        mbar_init(bar, 1);
        mbar_fence_init();
    }
    if (warp == 0) tmem_alloc(tmem_slot, 512);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    const uint32_t T_A = tmem, T_D = tmem + 256;
    const int hf = warp >> 2;                                 // which 128-row half this warp addresses in TMEM
    const int row = 32 * (warp & 3) + lane;                   // TMEM lane = row within the half
    const uint32_t lane_off = (uint32_t)(32 * (warp & 3)) << 16;
    const int m_row = hf * 128 + row;                         // gate-output row: gate = m_row / 64, unit = m_row % 64

    // ---- the CTA's slice of R into TMEM: row m_row, 256 bf16 = 128 columns of packed pairs
    {
        const int g = m_row >> 6, u = m_row & 63;
        const uint4 *src = reinterpret_cast<const uint4 *>(R + (((size_t)g * NH + hd) * TCR_DH + u0 + u) * TCR_DH);
#pragma unroll 1
        for (int c = 0; c < 128; c += 32) {
            uint32_t v[32];
#pragma unroll
            for (int x = 0; x < 8; ++x) {
                const uint4 q = src[(c >> 2) + x];
                v[4 * x] = q.x; v[4 * x + 1] = q.y; v[4 * x + 2] = q.z; v[4 * x + 3] = q.w;
            }
            tmem_st32(T_A + hf * 128 + lane_off + c, v);
        }
        tmem_wait_st();
    }
    // ---- h_{-1} of the whole head into B[0] (every CTA keeps its own copy)
    for (int e = tid; e < TCR_NB * TCR_DH; e += TCR_THREADS) {
        const int bb = e >> 8, kx = e & 255;
        const float hv = (h0 && b0 + bb < B) ? h0[(size_t)(b0 + bb) * D + hd * TCR_DH + kx] : 0.f;
        *reinterpret_cast<__nv_bfloat16 *>(smem + (kx >> 6) * TCR_BBOX + sw128_off(bb, kx & 63)) = __float2bfloat16_rn(hv);
    }
    // ---- cells owned by this thread: unit u, batch rows bq + 4 j
    const int u = tid & 63, bq = tid >> 6;
    float sc[8], sn[8], sm[8], shl[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int bb = bq + 4 * j;
        const bool ok = c0 != nullptr && b0 + bb < B;
        const size_t so = ok ? (size_t)(b0 + bb) * D + hd * TCR_DH + u0 + u : 0;
        sc[j] = ok ? c0[so] : 0.f;
        sn[j] = ok ? n0[so] : 1.f;
        sm[j] = ok ? m0[so] : 0.f;
        shl[j] = ok ? h0[so] : 0.f;
    }
    float bias[4];
#pragma unroll
    for (int g = 0; g < 4; ++g) bias[g] = rb[(size_t)g * D + hd * TCR_DH + u0 + u];
    fence_proxy_async_all();
    tc_fence_before_sync();
    cluster.sync();

    constexpr uint32_t IDESC = idesc_bf16(128, TCR_NB, false, false);
    const uint64_t dB0 = smem_desc_sw128(smem_u32(smem), 0, 1024);
    const __nv_bfloat16 *gxb = gx + (size_t)hd * TCR_DH + u0 + u;

    for (int t = 0; t < S; ++t) {
        const int p = t & 1;
        // recurrent pre-activations: pre[m][b] = sum_k R[m][k] h_{t-1}[b][k]
        if (tid == 0 && !*abort_flag) {
            tc_fence_after_sync();
            fence_proxy_async_all();
            const uint64_t dB = dB0 + ((p * TCR_BBUF) >> 4);
#pragma unroll
            for (int h2 = 0; h2 < 2; ++h2)
#pragma unroll
                for (int kk = 0; kk < TCR_DH / 16; ++kk)
                    mma_ts(T_D + h2 * TCR_NB, T_A + h2 * 128 + kk * 8, dB + (((kk >> 2) * TCR_BBOX + (kk & 3) * 32) >> 4),
                           IDESC, kk > 0);
            mma_commit(bar);
        }
        // input-side pre-activations of this step for the owned cells (independent of the recurrence)
        float gxv[8][4];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int bb = bq + 4 * j;
            const bool ok = b0 + bb < B;
#pragma unroll
            for (int g = 0; g < 4; ++g)
                gxv[j][g] = ok ? __bfloat162float(gxb[(((size_t)(b0 + bb) * S + t) * 4 + g) * D]) : 0.f;
        }
        mbar_wait(bar, (uint32_t)(t & 1), abort_flag);   // bounded; a time-out sets the flag and poisons the state below
        tc_fence_after_sync();
        {
            uint32_t v[32];
            tmem_ld32(T_D + hf * TCR_NB + lane_off, v);
            tmem_wait_ld();
#pragma unroll
            for (int bb = 0; bb < TCR_NB; ++bb) sPre[m_row * TCR_PAD + bb] = __uint_as_float(v[bb]);
        }
        tc_fence_before_sync();
        __syncthreads();
        // gating of the owned cells; h_t to global memory and (bf16) to the next B buffer of all four CTAs
        unsigned char *bnext = smem + (p ^ 1) * TCR_BBUF + rank * TCR_BBOX;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int bb = bq + 4 * j;
            float it = sPre[(0 * 64 + u) * TCR_PAD + bb] + gxv[j][0] + bias[0];
            float ft = sPre[(1 * 64 + u) * TCR_PAD + bb] + gxv[j][1] + bias[1];
            if (cap > 0.f) { it = cap * tanhf(it / cap); ft = cap * tanhf(ft / cap); }
            const float zt = tanhf(sPre[(2 * 64 + u) * TCR_PAD + bb] + gxv[j][2] + bias[2]);
            const float ot = sigmoidf(sPre[(3 * 64 + u) * TCR_PAD + bb] + gxv[j][3] + bias[3]);
            const float mt = fmaxf(ft + sm[j], it);
            const float ie = expf(it - mt), fe = expf(ft - mt + sm[j]);
            sc[j] = fmaf(fe, sc[j], ie * zt);
            sn[j] = fmaf(fe, sn[j], ie);
            sm[j] = mt;
            const float hv = ot * (sc[j] / fmaxf(sn[j], 1.0f));
            shl[j] = hv;
            const __nv_bfloat16 hb = __float2bfloat16_rn(hv);
            if (b0 + bb < B) hs[((size_t)(b0 + bb) * S + t) * D + hd * TCR_DH + u0 + u] = hb;
            __nv_bfloat16 *dst = reinterpret_cast<__nv_bfloat16 *>(bnext + sw128_off(bb, u));
#pragma unroll
            for (int r = 0; r < TCR_CL; ++r) *cluster.map_shared_rank(dst, r) = hb;
        }
        fence_proxy_async_all();
        cluster.sync();   // every CTA holds the complete h_t; D and the staging buffer may be overwritten
    }
    const bool failed = *abort_flag != 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int bb = bq + 4 * j;
        if (b0 + bb < B) {
            const size_t so = (size_t)(b0 + bb) * D + hd * TCR_DH + u0 + u;
            c1[so] = sc[j]; n1[so] = sn[j]; h1[so] = shl[j];
            m1[so] = failed ? __int_as_float(0x7fc00000) : sm[j];   // a device-side time-out shows as NaN state
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 512);
}

}  // namespace

bool slstm_recurrent_tc_supported(int dtype, int dh, const void *R, const void *gx) {
    return dtype == XLSTM_BF16 && dh == TCR_DH && ((reinterpret_cast<uintptr_t>(R) | reinterpret_cast<uintptr_t>(gx)) & 15u) == 0;
}

int slstm_recurrent_tc(const void *gx, const void *R, const float *rb, const float *c0, const float *n0, const float *h0,
                       const float *m0, void *hs, float *c1, float *n1, float *h1, float *m1, int B, int S, int NH,
                       float cap, cudaStream_t st) {
    auto kern = slstm_recurrent_tc_kernel;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TCR_SMEM) != cudaSuccess)
        return XLSTM_ERR_CUDA;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(TCR_CL, NH, (B + TCR_NB - 1) / TCR_NB);
    cfg.blockDim = dim3(TCR_THREADS);
    cfg.dynamicSmemBytes = TCR_SMEM;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = TCR_CL;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, static_cast<const __nv_bfloat16 *>(gx),
                                       static_cast<const __nv_bfloat16 *>(R), rb, c0, n0, h0, m0,
                                       static_cast<__nv_bfloat16 *>(hs), c1, n1, h1, m1, B, S, NH, cap);
    return e == cudaSuccess ? launch_status() : XLSTM_ERR_CUDA;
}

}  // namespace xl
