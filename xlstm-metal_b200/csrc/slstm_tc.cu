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

constexpr int TCR_THREADS = 512;
constexpr int TCR_NB = 32;     // batch rows per cluster = N of the MMA
constexpr int TCR_U = 64;      // units per CTA
constexpr int TCR_DH = 256;    // head dimension = K of the MMA
constexpr int TCR_CL = 4;      // CTAs per cluster
constexpr int TCR_PAD = 33;    // row pitch of the accumulator staging (floats): conflict-free both ways
constexpr uint32_t TCR_BBOX = TCR_NB * 128;              // one 64-column box of h: 32 rows x 128 B
constexpr uint32_t TCR_BBUF = (TCR_DH / 64) * TCR_BBOX;  // 16 KB
constexpr uint32_t TCR_OFF_PRE = 2 * TCR_BBUF;
constexpr uint32_t TCR_OFF_BAR = TCR_OFF_PRE + 4 * TCR_U * TCR_PAD * 4;
constexpr uint32_t TCR_SMEM = TCR_OFF_BAR + 64;

#ifdef XL_TCR_TRACE
__device__ long long g_tcr_trace[64 * 16];
#define TCR_TRACE(id) do { if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && tid == 0 && t < 64) g_tcr_trace[t * 16 + (id)] = clock64(); } while (0)
#else
#define TCR_TRACE(id) do { } while (0)
#endif

// gating math on the approximate exp / reciprocal units: absolute error ~1e-6, far below the bf16
// rounding of the h that is fed back
__device__ __forceinline__ float rcp_fast(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float tanh_fast(float x) { return 1.0f - 2.0f * rcp_fast(1.0f + __expf(2.0f * x)); }
__device__ __forceinline__ float sigmoid_fast(float x) { return rcp_fast(1.0f + __expf(-x)); }

// shared::cta address of this CTA -> shared::cluster address of the same offset in CTA `rank`
__device__ __forceinline__ uint32_t mapa_u32(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
// bulk copy from this CTA's shared memory into a peer's, completing bytes on the PEER's mbarrier
__device__ __forceinline__ void bulk_copy_to_peer(uint32_t dst_cluster, uint32_t src_cta, uint32_t bytes, uint32_t bar_cluster) {
    asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst_cluster), "r"(src_cta), "r"(bytes), "r"(bar_cluster) : "memory");
}

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
    uint64_t *bar = reinterpret_cast<uint64_t *>(smem + TCR_OFF_BAR);   // MMAs of the step done
    uint64_t *hbar = bar + 1;                                           // [2]: the peers' parts of h have landed in B[q]
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + TCR_OFF_BAR + 32);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + TCR_OFF_BAR + 36);

    if (tid == 0) {
        *abort_flag = (smem_u32(smem) & 1023u) ? 1 : 0;
        mbar_init(bar, 1);
        mbar_init(&hbar[0], 1);
        mbar_init(&hbar[1], 1);
        mbar_fence_init();
    }
    if (warp == 0) tmem_alloc(tmem_slot, 512);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    const uint32_t T_A = tmem, T_D = tmem + 256;
    // warps 0-7 move data between TMEM and the CUDA cores: warp w addresses lanes 32 (w % 4) .. + 31 of half w / 4
    const int hf = (warp >> 2) & 1;
    const int row = 32 * (warp & 3) + lane;                   // TMEM lane = row within the half
    const uint32_t lane_off = (uint32_t)(32 * (warp & 3)) << 16;
    const int m_row = hf * 128 + row;                         // gate-output row: gate = m_row / 64, unit = m_row % 64

    // ---- the CTA's slice of R into TMEM: row m_row, 256 bf16 = 128 columns of packed pairs
    if (warp < 8) {
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
    // ---- h_{-1} of the whole head into B[0] (every CTA loads its own copy: no exchange for step 0)
    for (int e = tid; e < TCR_NB * TCR_DH; e += TCR_THREADS) {
        const int b2 = e >> 8, kx = e & 255;
        const float hv = (h0 && b0 + b2 < B) ? h0[(size_t)(b0 + b2) * D + hd * TCR_DH + kx] : 0.f;
        *reinterpret_cast<__nv_bfloat16 *>(smem + (kx >> 6) * TCR_BBOX + sw128_off(b2, kx & 63)) = __float2bfloat16_rn(hv);
    }
    // ---- cells owned by this thread: batch row bb = lane, the 4 adjacent units uq .. uq + 3 (warp = chunk):
    //      8-byte accesses for the gate inputs, the h output and this CTA's part of the next B buffer
    const int bb = lane, uq = warp * 4;
    const bool row_ok = b0 + bb < B;
    const size_t so = row_ok ? (size_t)(b0 + bb) * D + hd * TCR_DH + u0 + uq : 0;
    float sc[4], sn[4], sm[4], shl[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const bool ok = c0 != nullptr && row_ok;
        sc[e] = ok ? c0[so + e] : 0.f;
        sn[e] = ok ? n0[so + e] : 1.f;
        sm[e] = ok ? m0[so + e] : 0.f;
        shl[e] = ok ? h0[so + e] : 0.f;
    }
    float bias[4][4];
#pragma unroll
    for (int g = 0; g < 4; ++g)
#pragma unroll
        for (int e = 0; e < 4; ++e) bias[g][e] = rb[(size_t)g * D + hd * TCR_DH + u0 + uq + e];
    fence_proxy_async_smem();
    tc_fence_before_sync();
    cluster.sync();   // barriers initialised, R in TMEM and B[0] complete in every CTA before any peer copy can land

    constexpr uint32_t IDESC = idesc_bf16(128, TCR_NB, false, false);
    const float inv_cap = cap > 0.f ? 1.0f / cap : 0.f;
    const uint64_t dB0 = smem_desc_sw128(smem_u32(smem), 0, 1024);
    const __nv_bfloat16 *gxb = gx + (size_t)hd * TCR_DH + u0 + uq;
    // input-side pre-activations of the owned cells, fetched one step ahead of their use
    uint2 gnext[4];
#pragma unroll
    for (int g = 0; g < 4; ++g)
        gnext[g] = row_ok ? *reinterpret_cast<const uint2 *>(gxb + (((size_t)(b0 + bb) * S + 0) * 4 + g) * D) : make_uint2(0u, 0u);

    for (int t = 0; t < S; ++t) {
        const int p = t & 1;
        TCR_TRACE(0);
        // recurrent pre-activations: pre[m][b] = sum_k R[m][k] h_{t-1}[b][k]
        if (tid == 0 && !*abort_flag) {
            // h_{t-1}: this CTA's own 64 columns were written and fenced last step, so their MMAs go first;
            // the peers' parts arrive by bulk copies that complete hbar[p]
            tc_fence_after_sync();
            const uint64_t dB = dB0 + ((p * TCR_BBUF) >> 4);
#pragma unroll
            for (int h2 = 0; h2 < 2; ++h2)
#pragma unroll
                for (int k4 = 0; k4 < 4; ++k4)
                    mma_ts(T_D + h2 * TCR_NB, T_A + h2 * 128 + (rank * 4 + k4) * 8,
                           dB + ((rank * TCR_BBOX + k4 * 32) >> 4), IDESC, k4 > 0);
            const uint32_t k_done = p ? (uint32_t)((t - 1) >> 1) : (uint32_t)((t >> 1) - 1);
            if (t == 0 || mbar_wait(&hbar[p], k_done & 1u, abort_flag)) {
#pragma unroll
                for (int h2 = 0; h2 < 2; ++h2)
#pragma unroll
                    for (int kb = 1; kb < TCR_CL; ++kb) {
                        const int kbx = (rank + kb) % TCR_CL;
#pragma unroll
                        for (int k4 = 0; k4 < 4; ++k4)
                            mma_ts(T_D + h2 * TCR_NB, T_A + h2 * 128 + (kbx * 4 + k4) * 8,
                                   dB + ((kbx * TCR_BBOX + k4 * 32) >> 4), IDESC, true);
                    }
                mma_commit(bar);
            }
        }
        TCR_TRACE(1);
        uint2 graw[4];
#pragma unroll
        for (int g = 0; g < 4; ++g) graw[g] = gnext[g];
        if (t + 1 < S && row_ok) {
#pragma unroll
            for (int g = 0; g < 4; ++g)
                gnext[g] = *reinterpret_cast<const uint2 *>(gxb + (((size_t)(b0 + bb) * S + t + 1) * 4 + g) * D);
        }
        TCR_TRACE(2);
        if (warp < 8) {
            mbar_wait(bar, (uint32_t)(t & 1), abort_flag);   // bounded; a time-out sets the flag and poisons the state below
            tc_fence_after_sync();
            TCR_TRACE(3);
            uint32_t v[32];
            tmem_ld32(T_D + hf * TCR_NB + lane_off, v);
            tmem_wait_ld();
#pragma unroll
            for (int b2 = 0; b2 < TCR_NB; ++b2) sPre[m_row * TCR_PAD + b2] = __uint_as_float(v[b2]);
            tc_fence_before_sync();
        }
        TCR_TRACE(4);
        __syncthreads();
        TCR_TRACE(5);
        // gating of the owned cells; h_t to global memory and (bf16) into this CTA's box of the next B buffer
        uint32_t hpk[2];
#pragma unroll
        for (int e2 = 0; e2 < 2; ++e2) {
            float hv2[2];
#pragma unroll
            for (int x = 0; x < 2; ++x) {
                const int e = 2 * e2 + x;
                const uint32_t wi = e2 ? graw[0].y : graw[0].x, wf = e2 ? graw[1].y : graw[1].x;
                const uint32_t wz = e2 ? graw[2].y : graw[2].x, wo = e2 ? graw[3].y : graw[3].x;
                const float gi = x ? __uint_as_float(wi & 0xffff0000u) : __uint_as_float(wi << 16);
                const float gf = x ? __uint_as_float(wf & 0xffff0000u) : __uint_as_float(wf << 16);
                const float gz = x ? __uint_as_float(wz & 0xffff0000u) : __uint_as_float(wz << 16);
                const float go = x ? __uint_as_float(wo & 0xffff0000u) : __uint_as_float(wo << 16);
                float it = sPre[(0 * 64 + uq + e) * TCR_PAD + bb] + gi + bias[0][e];
                float ft = sPre[(1 * 64 + uq + e) * TCR_PAD + bb] + gf + bias[1][e];
                if (cap > 0.f) { it = cap * tanh_fast(it * inv_cap); ft = cap * tanh_fast(ft * inv_cap); }
                const float zt = tanh_fast(sPre[(2 * 64 + uq + e) * TCR_PAD + bb] + gz + bias[2][e]);
                const float ot = sigmoid_fast(sPre[(3 * 64 + uq + e) * TCR_PAD + bb] + go + bias[3][e]);
                const float mt = fmaxf(ft + sm[e], it);
                const float ie = __expf(it - mt), fe = __expf(ft - mt + sm[e]);
                sc[e] = fmaf(fe, sc[e], ie * zt);
                sn[e] = fmaf(fe, sn[e], ie);
                sm[e] = mt;
                const float hv = ot * sc[e] * rcp_fast(fmaxf(sn[e], 1.0f));
                shl[e] = hv;
                hv2[x] = hv;
            }
            const __nv_bfloat162 pk = __floats2bfloat162_rn(hv2[0], hv2[1]);
            hpk[e2] = *reinterpret_cast<const uint32_t *>(&pk);
        }
        TCR_TRACE(8);
        const uint2 hvec = make_uint2(hpk[0], hpk[1]);
        if (row_ok) *reinterpret_cast<uint2 *>(hs + ((size_t)(b0 + bb) * S + t) * D + hd * TCR_DH + u0 + uq) = hvec;
        if (t + 1 < S) {
            unsigned char *mybox = smem + (p ^ 1) * TCR_BBUF + rank * TCR_BBOX;
            *reinterpret_cast<uint2 *>(mybox + sw128_off(bb, uq)) = hvec;
            fence_proxy_async_smem();     // generic-proxy writes -> visible to the bulk copies and the MMAs (async proxy)
            TCR_TRACE(6);
            __syncthreads();
            TCR_TRACE(7);
            if (tid == 0) {
                // this CTA's 4 KB box of h_t goes to the same place in the three peers; each copy completes its
                // bytes on the RECEIVER's barrier.  Own barrier: one arrival + the 3 x 4 KB it will receive.
                mbar_expect_tx(&hbar[p ^ 1], 3 * TCR_BBOX);
                const uint32_t src = smem_u32(mybox), barl = smem_u32(&hbar[p ^ 1]);
#pragma unroll
                for (int r = 1; r < TCR_CL; ++r) {
                    const uint32_t peer = (uint32_t)((rank + r) % TCR_CL);
                    bulk_copy_to_peer(mapa_u32(src, peer), src, TCR_BBOX, mapa_u32(barl, peer));
                }
            }
        }
    }
    const bool failed = *abort_flag != 0;
    if (row_ok) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            c1[so + e] = sc[e]; n1[so + e] = sn[e]; h1[so + e] = shl[e];
            m1[so + e] = failed ? __int_as_float(0x7fc00000) : sm[e];   // a device-side time-out shows as NaN state
        }
    }
    tc_fence_before_sync();
    cluster.sync();   // no CTA leaves while a peer's copy may still read or write its shared memory
    if (warp == 0) tmem_dealloc(tmem, 512);
}

}  // namespace

bool slstm_recurrent_tc_supported(int dtype, int dh, const void *R, const void *gx, const void *hs) {
    return dtype == XLSTM_BF16 && dh == TCR_DH &&
           ((reinterpret_cast<uintptr_t>(R) | reinterpret_cast<uintptr_t>(gx) | reinterpret_cast<uintptr_t>(hs)) & 15u) == 0;
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

#ifdef XL_TCR_TRACE
extern "C" int xlstm_debug_trace_slstm(long long *host_out) {
    return (int)cudaMemcpyFromSymbol(host_out, xl::g_tcr_trace, sizeof(long long) * 64 * 16);
}
#endif
