// Chunkwise mLSTM forward on the Blackwell tensor cores (bf16 in, fp32 accumulate).
//
// One persistent CTA owns a 128-column slice of one head's matrix memory C and
// walks the sequence in tiles of 128 tokens.  C (dqk x 128, fp32) never leaves
// the SM: it is the TMEM accumulator of the state-update MMA for the whole
// sequence, so the inter-chunk carry and the intra-chunk read-out are ONE kernel
// and no per-chunk state is materialised in HBM.  Per tile (tcgen05.mma, M = 128):
//
//   S  = Q K^T                       [128 x 128]   A: Q  K-major (TMA)   B: K  K-major (TMA)
//   H  = Q~ Cb                       [128 x 128]   A: Q~ K-major         B: Cb MN-major (bf16 copy of C)
//   H += P V     P = S * D (causal)  [128 x 128]   A: P  bf16 in TMEM    B: V  MN-major (TMA)
//   C += K~^T V  (two halves of dqk) [128 x 128]   A: K~ MN-major        B: V  MN-major
//
// with Q~ = Q * e^{m-x_t} * dqk^-1/2 and K~ = K * e^{u_t-x_last} scaled in place in
// shared memory after S has consumed the raw tiles.  All exponents are
// differences that are <= 0 (u_s = i_s - b_s, x_t = max(m, max_{s<=t} u_s)), so
// nothing can overflow whatever the gates are.  The gate scalars come from a
// small pre-pass kernel (one warp per head, sequential over tiles) that writes
// them to caller-provided scratch.
//
// Roles (640 threads): warp 0 TMA producer, warp 1 MMA issuer (+TMEM alloc), warp 2 TMA stores of h,
// warps 4-7 gate matrix P, then q~.n, then the C pass for rows [128,256) of C;
// warps 8-11 Q~ scaling; warps 12-15 K~ scaling, then the C pass for rows [0,128) (refresh Cb);
// warps 16-19 normaliser update (column sums of K~) and the H epilogue.
// MMA issue order per tile: S, state update, P V, read-out (the update only needs the short K~
// pass and frees K for the next tile's load while the longer Q~ pass still runs).
// C is held in TMEM as C~ = C e^{-rho}: rho absorbs the per-tile decay, so the accumulator is not
// rescaled every tile (TMEM load/store bandwidth, ~64 B/clk/SM, is the scarce resource); it is
// multiplied once whenever -rho would pass 30.
// TMEM columns: C [0,256)  S/P [256,384)  H [384,512).
// Every mbarrier wait is bounded; a time-out sets the status word in the
// scratch buffer, releases all roles and frees TMEM before the CTA returns.
#include <atomic>

#include "mlstm_chunkwise_tc.cuh"

namespace xl {

namespace {

using namespace tc;
using namespace tcw;

// ---------------------------------------------------------------------------
// gate pre-pass.  Only the stabiliser m couples the tiles, and only through two numbers per tile
// (G = sum of log-sigmoid f, U = max of u = i - b), so it runs as three small launches:
//   mlstm_gate_stats_kernel   one warp per (head, tile): G_c, U_c                      -> scratch
//   mlstm_gate_chain_kernel   one warp per head: m_{c+1} = G_c + max(m_c, U_c), the frame rho of the
//                             lazily rescaled accumulator, the head's path flag        -> scratch
//   mlstm_gate_write_kernel   one warp per (head, tile): the per-token scalars          -> scratch
// Sums and maxima are kept in double so that differences of large cumulative sums stay exact.
// ---------------------------------------------------------------------------
constexpr int GP_THREADS = 256;        // 8 warps = 8 tiles per CTA
constexpr int GC = 6;                  // doubles of chain scratch per (head, tile): G, U, m_in, rho_in, rho_out, mul
constexpr double RESCALE_AT = 30.0;    // general kernel: rescale C~ when the frame exponent would exceed e^30
// A head takes the bounded-spread kernel when no tile raises the running maximum by more than SPREAD_LIMIT (in
// natural-log units): its per-token factors a_s = e^{u_s - m - rho} then stay below e^{SPREAD_LIMIT + RESCALE_AT_B}
// = e^65, which leaves the fp32 accumulators (sums of a few thousand products of a_s with O(10) values) a
// margin of e^10 below overflow.
constexpr double SPREAD_LIMIT = 45.0;
constexpr double RESCALE_AT_B = 20.0;

template <typename T>
__device__ __forceinline__ void gate_tile_scan(const T *ip, const T *fp, int64_t sg_s, float cap, int c, int lane,
                                               double (&bcum)[4], double (&u)[4], double (&pmax)[4], double &excl_max,
                                               double &G, double &U) {
    const int t0 = c * LT + lane * 4;
    float iv[4];
    double run = 0.0;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        iv[e] = gate_softcap(Elem<T>::ld(ip + (int64_t)(t0 + e) * sg_s), cap);
        run += (double)logsigmoid(gate_softcap(Elem<T>::ld(fp + (int64_t)(t0 + e) * sg_s), cap));
        bcum[e] = run;
    }
    double incl = run;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const double v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
    }
    const double off = incl - run;
    double pm = -INFINITY;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        bcum[e] += off;
        u[e] = (double)iv[e] - bcum[e];
        pm = fmax(pm, u[e]);
        pmax[e] = pm;
    }
    double mincl = pm;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const double v = __shfl_up_sync(0xffffffffu, mincl, o);
        if (lane >= o) mincl = fmax(mincl, v);
    }
    excl_max = __shfl_up_sync(0xffffffffu, mincl, 1);
    if (lane == 0) excl_max = -INFINITY;
    U = __shfl_sync(0xffffffffu, mincl, 31);
    G = __shfl_sync(0xffffffffu, bcum[3], 31);
}

template <typename T>
__global__ void __launch_bounds__(GP_THREADS)
mlstm_gate_stats_kernel(const T *__restrict__ ig, const T *__restrict__ fg, int64_t sg_b, int64_t sg_h, int64_t sg_s,
                        double *__restrict__ chain, int NH, int NCH, float cap) {
    const int bh = blockIdx.y, b = bh / NH, hd = bh % NH;
    const int lane = threadIdx.x & 31, c = blockIdx.x * (GP_THREADS / 32) + (threadIdx.x >> 5);
    if (c >= NCH) return;
    double bcum[4], u[4], pmax[4], excl, G, U;
    gate_tile_scan<T>(ig + b * sg_b + hd * sg_h, fg + b * sg_b + hd * sg_h, sg_s, cap, c, lane, bcum, u, pmax, excl, G, U);
    if (lane == 0) {
        double *o = chain + ((size_t)bh * NCH + c) * GC;
        o[0] = G; o[1] = U;
    }
}

// One warp per (head, segment).  The chain is sequential but tiny; the warp loads 32 tiles' (G, U) at once and
// every lane walks them through shuffles, keeping the results of "its" tile for a coalesced write.
// m0_auto: the segment starts from an EMPTY state (C = n = 0): any stabiliser below the first maximum gives the
// same end state, so the chain starts at the first tile's U (spread 0) instead of -inf.
__global__ void __launch_bounds__(32)
mlstm_gate_chain_kernel(const float *__restrict__ m0, double *__restrict__ chain, float *__restrict__ m_out,
                        int *__restrict__ path, int NCH, int P, int seg_tiles, int general_only, int m0_auto) {
    const int bhv = blockIdx.x, lane = threadIdx.x;
    const int tile0 = (bhv % P) * seg_tiles, n = min(seg_tiles, NCH - tile0);
    double *ch = chain + ((size_t)(bhv / P) * NCH + tile0) * GC;
    // pass 1: the stabiliser chain, and whether every tile's spread x_last - m is bounded
    double m = m0_auto ? ch[1] : (m0 ? (double)m0[bhv] : 0.0);
    bool bounded = !general_only;
    for (int c0 = 0; c0 < n; c0 += 32) {
        const int c = c0 + lane;
        const double Gl = c < n ? ch[(size_t)c * GC + 0] : 0.0, Ul = c < n ? ch[(size_t)c * GC + 1] : 0.0;
        double m_mine = 0.0;
        const int nb = min(32, n - c0);
        for (int j = 0; j < nb; ++j) {
            const double Gj = __shfl_sync(0xffffffffu, Gl, j), Uj = __shfl_sync(0xffffffffu, Ul, j);
            const double x_last = fmax(m, Uj);
            if (x_last - m > SPREAD_LIMIT) bounded = false;
            if (j == lane) m_mine = m;
            m = Gj + x_last;
        }
        if (c < n) ch[(size_t)c * GC + 2] = m_mine;    // stabiliser carried INTO tile c
    }
    if (lane == 0) { m_out[bhv] = (float)m; path[bhv] = bounded ? 1 : 0; }
    // pass 2: C is kept in TMEM as C~ = C e^{-rho}: rho absorbs the per-tile decay so that the accumulator is
    // NOT rescaled every tile; only when -rho would exceed the threshold is C~ multiplied once (mul).
    // General kernel: the multiplication happens BEFORE tile c's update (mul also carries the decay of that
    // tile); bounded-spread kernel: AFTER tile c's update, so that update and read-out of a tile share one
    // frame.  rho_in = frame the read-out of tile c sees, rho_out = frame after tile c's update.
    double rho = 0.0;
    for (int c0 = 0; c0 < n; c0 += 32) {
        const int c = c0 + lane;
        double ld = 0.0;
        if (c < n) ld = ch[(size_t)c * GC + 2] - fmax(ch[(size_t)c * GC + 2], ch[(size_t)c * GC + 1]);   // m - x_last <= 0
        double rin = 0.0, rout = 0.0, mul = 1.0;
        const int nb = min(32, n - c0);
        for (int j = 0; j < nb; ++j) {
            const double logdec = __shfl_sync(0xffffffffu, ld, j);
            const double r_in = rho;
            double r_out, mu = 1.0;
            if (bounded) {
                rho += logdec;
                r_out = rho;
                if (rho < -RESCALE_AT_B) { mu = exp(rho); rho = 0.0; }
            } else {
                if (rho + logdec < -RESCALE_AT) { mu = exp(rho + logdec); rho = 0.0; }
                else rho += logdec;
                r_out = rho;
            }
            if (j == lane) { rin = r_in; rout = r_out; mul = mu; }
        }
        if (c < n) {
            ch[(size_t)c * GC + 3] = rin; ch[(size_t)c * GC + 4] = rout; ch[(size_t)c * GC + 5] = mul;
        }
    }
}

// Segment-parallel prefill: the end state of segment j from an EMPTY state (Cl, nl, ml) and the total log-decay
// G_j of the segment combine associatively with the state before it,
//   m' = max(G_j + m, ml);  C' = e^{G_j + m - m'} C + e^{ml - m'} Cl;  n' likewise,
// so one cheap pass over the P local states yields the true state at the start of every segment (Cs, ns, ms)
// and the final state.  One CTA per (head, slab of elements); the scalar chain is recomputed per CTA.
constexpr int COMB_THREADS = 256;
constexpr int COMB_VEC = 4;        // elements per thread (one 16-byte vector)
__global__ void __launch_bounds__(COMB_THREADS)
mlstm_segment_combine_kernel(const float *__restrict__ C0, const float *__restrict__ n0, const float *__restrict__ m0,
                             const float *__restrict__ Cl, const float *__restrict__ nl, const float *__restrict__ ml,
                             const double *__restrict__ chain, float *__restrict__ Cs, float *__restrict__ ns,
                             float *__restrict__ ms, float *__restrict__ C1, float *__restrict__ n1, float *__restrict__ m1,
                             int NCH, int P, int seg_tiles, int dqk, int dv) {
    __shared__ float s_wc[64], s_wl[64];   // weights of the carried and of the local state per segment (P <= 64)
    __shared__ double s_G[64];             // summed log forget gates per segment
    const int bh = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // per-segment sums by the warps (lanes stride over the segment's tiles), then one thread chains the P segments
    for (int j = warp; j < P; j += COMB_THREADS / 32) {
        const int tile0 = j * seg_tiles, n = min(seg_tiles, NCH - tile0);
        double G = 0.0;
        for (int c = lane; c < n; c += 32) G += chain[((size_t)bh * NCH + tile0 + c) * GC + 0];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) G += __shfl_xor_sync(0xffffffffu, G, o);
        if (lane == 0) s_G[j] = G;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        double m = C0 ? (double)m0[bh] : 0.0;
        for (int j = 0; j < P; ++j) {
            const double mloc = (double)ml[(size_t)bh * P + j];
            const double mn = fmax(s_G[j] + m, mloc);
            if (blockIdx.y == 0) ms[(size_t)bh * P + j] = (float)m;
            s_wc[j] = (float)exp(s_G[j] + m - mn);
            s_wl[j] = (float)exp(mloc - mn);
            m = mn;
        }
        if (blockIdx.y == 0) m1[bh] = (float)m;
    }
    __syncthreads();
    // elements of C, then of n, as 16-byte vectors (dqk * dv and dqk are multiples of 4); a thread owns one vector
    // of every segment: its P loads are independent of the chain and are issued ahead of it, 8 at a time
    const size_t CE = (size_t)dqk * dv, total_vec = (CE + dqk) / COMB_VEC;
    for (size_t e4 = (size_t)blockIdx.y * COMB_THREADS + threadIdx.x; e4 < total_vec; e4 += (size_t)gridDim.y * COMB_THREADS) {
        const size_t e = e4 * COMB_VEC;
        const bool isC = e < CE;
        const size_t off = isC ? e : e - CE, per = isC ? CE : (size_t)dqk;
        const float *src0 = isC ? C0 : n0, *loc = isC ? Cl : nl;
        float *st = isC ? Cs : ns, *fin = isC ? C1 : n1;
        float4 v = C0 ? *reinterpret_cast<const float4 *>(src0 + (size_t)bh * per + off) : make_float4(0.f, 0.f, 0.f, 0.f);
        for (int j0 = 0; j0 < P; j0 += 8) {
            float4 l[8];
#pragma unroll
            for (int u = 0; u < 8; ++u)
                if (j0 + u < P) l[u] = ldg_stream(loc + ((size_t)bh * P + j0 + u) * per + off);
#pragma unroll
            for (int u = 0; u < 8; ++u)
                if (j0 + u < P) {
                    const int j = j0 + u;
                    stg_stream(st + ((size_t)bh * P + j) * per + off, v);
                    const float wc = s_wc[j], wl = s_wl[j];
                    v.x = wc * v.x + wl * l[u].x;
                    v.y = wc * v.y + wl * l[u].y;
                    v.z = wc * v.z + wl * l[u].z;
                    v.w = wc * v.w + wl * l[u].w;
                }
        }
        *reinterpret_cast<float4 *>(fin + (size_t)bh * per + off) = v;
    }
}

template <typename T>
__global__ void __launch_bounds__(GP_THREADS)
mlstm_gate_write_kernel(const T *__restrict__ ig, const T *__restrict__ fg, int64_t sg_b, int64_t sg_h, int64_t sg_s,
                        const double *__restrict__ chain, const int *__restrict__ path, float *__restrict__ gates,
                        int NH, int NCH, int P, int seg_tiles, float qscale, float cap) {
    const int bh = blockIdx.y, b = bh / NH, hd = bh % NH;
    const int lane = threadIdx.x & 31, c = blockIdx.x * (GP_THREADS / 32) + (threadIdx.x >> 5);
    if (c >= NCH) return;
    const bool bounded = path[(size_t)bh * P + c / seg_tiles] != 0;
    double bcum[4], u[4], pmax[4], excl, G, U;
    gate_tile_scan<T>(ig + b * sg_b + hd * sg_h, fg + b * sg_b + hd * sg_h, sg_s, cap, c, lane, bcum, u, pmax, excl, G, U);
    const double *ch = chain + ((size_t)bh * NCH + c) * GC;
    const double m = ch[2], rho_in = ch[3], rho_out = ch[4];
    const double x_last = fmax(U, m);
    const double carry = fmax(excl, m);
    float *g = gates + ((size_t)bh * NCH + c) * GW;
    float4 o_u2, o_x2, o_wq, o_w, o_em;
    float *pu = &o_u2.x, *px = &o_x2.x, *pq = &o_wq.x, *pw = &o_w.x, *pe = &o_em.x;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const double xt = fmax(pmax[e], carry);
        pu[e] = (float)(u[e] * (double)LOG2E);
        px[e] = (float)(xt * (double)LOG2E);
        pq[e] = expf((float)(m - xt + rho_in)) * qscale;   // read-out sees C~ = C e^{-rho_in}
        // weight of token s in the update: general kernel e^{u_s - x_last - rho_out} (<= e^{RESCALE_AT});
        // bounded-spread kernel a_s = e^{u_s - m - rho_in} (the same number except on rescale tiles)
        pw[e] = bounded ? expf((float)(u[e] - m - rho_in)) : expf((float)(u[e] - x_last - rho_out));
        pe[e] = expf(-(float)(bcum[e] + xt));
    }
    *reinterpret_cast<float4 *>(g + G_U2 + lane * 4) = o_u2;
    *reinterpret_cast<float4 *>(g + G_X2 + lane * 4) = o_x2;
    *reinterpret_cast<float4 *>(g + G_WINQ + lane * 4) = o_wq;
    *reinterpret_cast<float4 *>(g + G_W + lane * 4) = o_w;
    *reinterpret_cast<float4 *>(g + G_EMT + lane * 4) = o_em;
    if (lane == 0) {
        g[G_SCAL + 0] = (float)ch[5];               // multiplier for C~ and n~: before this tile (general) / after its update (bounded)
        g[G_SCAL + 1] = (float)(G + x_last);        // stabiliser after this tile
        g[G_SCAL + 2] = expf((float)rho_out);       // C = C~ * this after the tile's update (used for the final state)
    }
}

// ---------------------------------------------------------------------------
// main kernel (general gates)
// ---------------------------------------------------------------------------
enum { B_QFULL = 0, B_KFULL, B_VFULL, B_SDONE, B_H1DONE, B_UPDDONE, B_H2DONE, B_QSCALED, B_KSCALED, B_CBREADY,
       B_PREADY, B_HFREE, B_NDONE, B_KREAD, B_HSTAGED, B_VFREE, B_QNDONE, B_NBARS };

// C pass for one 128-row half after the state update: TMEM -> Cb (bf16) and back to TMEM scaled by
// the next tile's decay; after the last tile the fp32 rows go to `dst` instead.
template <int DQK>
__device__ __forceinline__ void c_pass_half(unsigned char *smem, uint32_t t_half, int j, bool last, float decay_next,
                                            float *dst) {
    using SM = Smem<DQK>;
#pragma unroll 1
    for (int c0 = 0; c0 < DVS; c0 += 64) {
        uint32_t va[32], vb[32];
        tmem_ld32(t_half + c0, va);
        tmem_ld32(t_half + c0 + 32, vb);
        tmem_wait_ld();
        if (last) {   // decay_next carries the frame factor e^{rho}: C = C~ e^{rho}
#pragma unroll
            for (int x = 0; x < 32; x += 4) {
                *reinterpret_cast<float4 *>(dst + c0 + x) =
                    make_float4(__uint_as_float(va[x]) * decay_next, __uint_as_float(va[x + 1]) * decay_next,
                                __uint_as_float(va[x + 2]) * decay_next, __uint_as_float(va[x + 3]) * decay_next);
                *reinterpret_cast<float4 *>(dst + c0 + 32 + x) =
                    make_float4(__uint_as_float(vb[x]) * decay_next, __uint_as_float(vb[x + 1]) * decay_next,
                                __uint_as_float(vb[x + 2]) * decay_next, __uint_as_float(vb[x + 3]) * decay_next);
            }
        } else {
#pragma unroll
            for (int x = 0; x < 32; x += 8) {
                uint4 o;
                o.x = pack_bf16(__uint_as_float(va[x]), __uint_as_float(va[x + 1]));
                o.y = pack_bf16(__uint_as_float(va[x + 2]), __uint_as_float(va[x + 3]));
                o.z = pack_bf16(__uint_as_float(va[x + 4]), __uint_as_float(va[x + 5]));
                o.w = pack_bf16(__uint_as_float(va[x + 6]), __uint_as_float(va[x + 7]));
                int c = c0 + x;
                *reinterpret_cast<uint4 *>(smem + SM::CB + (c >> 6) * SM::CB_BLOCK + sw128_off(j, c & 63)) = o;
                o.x = pack_bf16(__uint_as_float(vb[x]), __uint_as_float(vb[x + 1]));
                o.y = pack_bf16(__uint_as_float(vb[x + 2]), __uint_as_float(vb[x + 3]));
                o.z = pack_bf16(__uint_as_float(vb[x + 4]), __uint_as_float(vb[x + 5]));
                o.w = pack_bf16(__uint_as_float(vb[x + 6]), __uint_as_float(vb[x + 7]));
                c += 32;
                *reinterpret_cast<uint4 *>(smem + SM::CB + (c >> 6) * SM::CB_BLOCK + sw128_off(j, c & 63)) = o;
            }
            if (decay_next != 1.0f) {   // CTA-uniform: a rescale tile (rare); otherwise C~ stays as it is
#pragma unroll
                for (int x = 0; x < 32; ++x) {
                    va[x] = __float_as_uint(__uint_as_float(va[x]) * decay_next);
                    vb[x] = __float_as_uint(__uint_as_float(vb[x]) * decay_next);
                }
                tmem_st32(t_half + c0, va);
                tmem_st32(t_half + c0 + 32, vb);
            }
        }
    }
}

template <int DQK>
__global__ void __launch_bounds__(THREADS, 1) mlstm_chunkwise_tc_kernel(const __grid_constant__ TcParams p) {
    using SM = Smem<DQK>;
    constexpr int NBOX = SM::NBOX;
    constexpr int NHALF = DQK / 128;
    extern __shared__ __align__(1024) unsigned char smem[];
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + SM::BARS);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + SM::MISC);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + SM::MISC + 4);
    float *s_n = reinterpret_cast<float *>(smem + SM::N_VEC);
    float *s_qn = reinterpret_cast<float *>(smem + SM::QN);
    float *s_rs = reinterpret_cast<float *>(smem + SM::INV);   // row sums of P, by tile parity

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int bh = blockIdx.x;     // (batch, head, segment): index of the states and of the path flag
    if (p.path[bh] != 0) return;   // this segment runs in the bounded-spread kernel (CTA-uniform, before any set-up)
    const int bhr = bh / p.P, tile0 = (bh % p.P) * p.seg_tiles;   // (batch, head) and first tile of this segment
    const int b = bhr / p.NH, hd = bhr % p.NH;
    const int col0 = blockIdx.y * DVS;
    const int NCH = min(p.seg_tiles, p.NCH - tile0);
    const float *gbase = p.gates + ((size_t)bhr * p.NCH + tile0) * GW;

    if (tid == 0) {
        *abort_flag = (smem_u32(smem) & 1023u) ? 1 : 0;  // swizzled tiles need a 1024-byte aligned base
        mbar_init(&bars[B_QFULL], 1);   mbar_init(&bars[B_KFULL], 1);   mbar_init(&bars[B_VFULL], 1);
        mbar_init(&bars[B_SDONE], 1);   mbar_init(&bars[B_H1DONE], 1);  mbar_init(&bars[B_UPDDONE], 1);
        mbar_init(&bars[B_H2DONE], 1);
        mbar_init(&bars[B_QSCALED], 128); mbar_init(&bars[B_KSCALED], 128); mbar_init(&bars[B_CBREADY], 128 * NHALF);
        mbar_init(&bars[B_PREADY], 128);  mbar_init(&bars[B_HFREE], 128);   mbar_init(&bars[B_NDONE], 128);  mbar_init(&bars[B_KREAD], 128);
        mbar_init(&bars[B_HSTAGED], 128); mbar_init(&bars[B_VFREE], 1); mbar_init(&bars[B_QNDONE], 128);
        mbar_fence_init();
        tma_prefetch_desc(&p.tq); tma_prefetch_desc(&p.tk); tma_prefetch_desc(&p.tv);
    }
    if (warp == 1) tmem_alloc(tmem_slot, 512);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    const uint32_t T_C = tmem, T_S = tmem + 256, T_H = tmem + 384;

    if (warp == 0) {
        // ================= TMA producer =================
        // Q is free once the read-out MMA of the previous tile has run (and the scaling warps are
        // done with it: they finish before that MMA is issued); K once the state update has run
        // and the normaliser sums are taken; V once both its consumers (update, P V) have run AND the
        // h tile that the epilogue stages in the V buffer has been read by its TMA stores.
        if (lane == 0) {
            for (int k = 0; k < NCH; ++k) {
                const int t0 = (tile0 + k) * LT;
                if (k > 0 && !(mbar_wait(&bars[B_UPDDONE], (k - 1) & 1, abort_flag) &&
                               mbar_wait(&bars[B_KREAD], (k - 1) & 1, abort_flag))) break;
                mbar_expect_tx(&bars[B_KFULL], NBOX * SM::BOX);
                for (int q = 0; q < NBOX; ++q) tma_load_4d(smem + SM::K + q * SM::BOX, &p.tk, &bars[B_KFULL], q * 64, t0, hd, b);
                if (k > 0 && !(mbar_wait(&bars[B_H1DONE], (k - 1) & 1, abort_flag) &&
                               mbar_wait(&bars[B_QNDONE], (k - 1) & 1, abort_flag))) break;
                mbar_expect_tx(&bars[B_QFULL], NBOX * SM::BOX);
                for (int q = 0; q < NBOX; ++q) tma_load_4d(smem + SM::Q + q * SM::BOX, &p.tq, &bars[B_QFULL], q * 64, t0, hd, b);
                if (k > 0 && !mbar_wait(&bars[B_VFREE], (k - 1) & 1, abort_flag)) break;   // h tile staged in V has been stored
                mbar_expect_tx(&bars[B_VFULL], 2 * SM::BOX);
                for (int q = 0; q < 2; ++q) tma_load_4d(smem + SM::V + q * SM::BOX, &p.tv, &bars[B_VFULL], col0 + q * 64, t0, hd, b);
            }
        }
    } else if (warp == 1) {
        // ================= MMA issuer =================
        if (lane == 0) {
            constexpr uint32_t ID_KK = idesc_bf16(128, 128, false, false);  // S
            constexpr uint32_t ID_KM = idesc_bf16(128, 128, false, true);   // inter read-out, P V
            constexpr uint32_t ID_MM = idesc_bf16(128, 128, true, true);    // state update
            // descriptors differ only in the start address (low word, units of 16 bytes)
            const uint64_t dQ = smem_desc_sw128(smem_u32(smem + SM::Q), 0, 1024);
            const uint64_t dK = smem_desc_sw128(smem_u32(smem + SM::K), 0, 1024);
            const uint64_t dCb = smem_desc_sw128(smem_u32(smem + SM::CB), SM::CB_BLOCK, 1024);
            const uint64_t dKm = smem_desc_sw128(smem_u32(smem + SM::K), SM::BOX, 1024);
            const uint64_t dV = smem_desc_sw128(smem_u32(smem + SM::V), SM::BOX, 1024);
            for (int k = 0; k < NCH; ++k) {
                const uint32_t ph = k & 1;
                // S = Q K^T  (the previous tile's P V, issued earlier, finishes first: in-order pipe)
                if (!(mbar_wait(&bars[B_QFULL], ph, abort_flag) && mbar_wait(&bars[B_KFULL], ph, abort_flag))) break;
                tc_fence_after_sync();
#pragma unroll
                for (int kk = 0; kk < DQK / 16; ++kk) {
                    const uint32_t o = ((kk >> 2) * SM::BOX + (kk & 3) * 32) >> 4;
                    mma_ss(T_S, dQ + o, dK + o, ID_KK, kk > 0);
                }
                mma_commit(&bars[B_SDONE]);
                // C += K~^T V first: it only needs K~ (a short pass) and frees K for the next tile's load,
                // which then overlaps the longer Q~ pass.  C was pre-scaled by the previous C pass.
                if (!(mbar_wait(&bars[B_KSCALED], ph, abort_flag) && mbar_wait(&bars[B_VFULL], ph, abort_flag) &&
                      mbar_wait(&bars[B_CBREADY], ph, abort_flag))) break;
                tc_fence_after_sync();
#pragma unroll
                for (int hf = 0; hf < NHALF; ++hf)
#pragma unroll
                    for (int kk = 0; kk < LT / 16; ++kk)
                        mma_ss(T_C + hf * 128, dKm + ((hf * 2 * SM::BOX + kk * 2048) >> 4), dV + kk * (2048 >> 4), ID_MM, true);
                mma_commit(&bars[B_UPDDONE]);
                // H = P V  (first write of H for this tile: the previous epilogue must have drained it)
                if (!mbar_wait(&bars[B_PREADY], ph, abort_flag)) break;
                if (k > 0 && !mbar_wait(&bars[B_HFREE], (k - 1) & 1, abort_flag)) break;
                tc_fence_after_sync();
#pragma unroll
                for (int kk = 0; kk < LT / 16; ++kk) mma_ts(T_H, T_S + kk * 8, dV + kk * (2048 >> 4), ID_KM, kk > 0);
                mma_commit(&bars[B_H2DONE]);
                // H += Q~ Cb   (Q~ scaled in place; Cb from the previous C pass)
                if (!mbar_wait(&bars[B_QSCALED], ph, abort_flag)) break;
                tc_fence_after_sync();
#pragma unroll
                for (int kk = 0; kk < DQK / 16; ++kk) {
                    const uint32_t o = ((kk >> 2) * SM::BOX + (kk & 3) * 32) >> 4;
                    mma_ss(T_H, dQ + o, dCb + kk * (2048 >> 4), ID_KM, true);
                }
                mma_commit(&bars[B_H1DONE]);
            }
        }
    }
    else if (warp == 2) {
        // ================= h store: TMA from the staged tile to this GPU's h and to the peers =================
        if (lane == 0) {
            for (int k = 0; k < NCH; ++k) {
                if (!mbar_wait(&bars[B_HSTAGED], k & 1, abort_flag)) break;
                const int tk = (tile0 + k) * LT;
                if (p.tok_per_rank > 0 && p.n_h > 0) {   // token-sharded: only the rank that owns these tokens gets the tile
                    const int d = tk / p.tok_per_rank;
                    for (int bx = 0; bx < 2; ++bx)
                        tma_store_4d(&p.th[d], smem + SM::V + bx * SM::BOX, col0 + bx * 64, tk - d * p.tok_per_rank, hd, b);
                } else {
                    for (int d = 0; d < p.n_h; ++d)
                        for (int bx = 0; bx < 2; ++bx)
                            tma_store_4d(&p.th[d], smem + SM::V + bx * SM::BOX, col0 + bx * 64, tk, hd, b);
                }
                tma_store_commit();
                tma_store_wait_read();            // staging tile consumed: V may be reloaded
                mbar_arrive(&bars[B_VFREE]);
            }
            tma_store_wait_all();                 // all h writes performed before the CTA exits
        }
    }
    else if (warp >= 4 && warp < 8) {
        // ================= gate matrix P = S * D and the denominators =================
        const int t = tid - 128;                       // token row = TMEM lane
        const int t0w = t & ~31;                       // first row of this warp
        const uint32_t lane_off = (uint32_t)t0w << 16;
        if (NHALF == 2) {  // rows [128,256) of the initial state
            c_init_half<DQK>(smem, T_C + 128 + lane_off, p.C0 ? p.C0 + ((size_t)bh * DQK + 128 + t) * p.dv + col0 : nullptr,
                             128 + t, gbase[G_SCAL + 0]);
            tmem_wait_st();
            fence_proxy_async_smem();
            tc_fence_before_sync();
            mbar_arrive(&bars[B_CBREADY]);
        }
        for (int k = 0; k < NCH; ++k) {
            const uint32_t ph = k & 1;
            const float *g = gbase + (size_t)k * GW;
            const float x2 = g[G_X2 + t] - p.log2_qscale;  // dqk^-1/2 folded into the exponent
            float u2v[4];                                  // lane holds u2 of column s0 + lane
#pragma unroll
            for (int pc = 0; pc < 4; ++pc) u2v[pc] = g[G_U2 + pc * 32 + lane];
            if (!mbar_wait(&bars[B_SDONE], ph, abort_flag)) break;
            tc_fence_after_sync();
            float rowsum = 0.f;
#pragma unroll
            for (int pc = 0; pc < 4; ++pc) {
                const int s0 = pc * 32;
                uint32_t packed[16];
                if (s0 <= t0w) {  // warp-uniform; columns beyond the warp's rows are all masked
                    uint32_t r[32];
                    tmem_ld32(T_S + lane_off + s0, r);
                    tmem_wait_ld();
                    const bool diag = (s0 == t0w);
#pragma unroll
                    for (int j = 0; j < 32; j += 2) {
                        const float ua = __shfl_sync(0xffffffffu, u2v[pc], j);
                        const float ub = __shfl_sync(0xffffffffu, u2v[pc], j + 1);
                        float p0 = __uint_as_float(r[j]) * ex2_approx(ua - x2);
                        float p1 = __uint_as_float(r[j + 1]) * ex2_approx(ub - x2);
                        if (diag) {
                            if (j > lane) p0 = 0.f;
                            if (j + 1 > lane) p1 = 0.f;
                        }
                        rowsum += p0 + p1;   // fp32, before rounding: keeps the normaliser well conditioned
                        packed[j >> 1] = pack_bf16(p0, p1);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) packed[j] = 0u;
                }
                tmem_st16(T_S + lane_off + (s0 >> 1), packed);
            }
            tmem_wait_st();
            s_rs[ph * LT + t] = rowsum;   // read by the epilogue warps after PREADY
            tc_fence_before_sync();
            mbar_arrive(&bars[B_PREADY]);
            if (NHALF == 2) {  // C pass for rows [128,256) of C (the K~ warps take rows [0,128))
                const bool last = (k == NCH - 1);
                if (!(mbar_wait(&bars[B_UPDDONE], ph, abort_flag) && mbar_wait(&bars[B_H1DONE], ph, abort_flag))) break;
                tc_fence_after_sync();
                c_pass_half<DQK>(smem, T_C + 128 + lane_off, 128 + t, last, last ? g[G_SCAL + 2] : g[GW + G_SCAL + 0],
                                 p.C1 + ((size_t)bh * DQK + 128 + t) * p.dv + col0);
                if (!last) {
                    tmem_wait_st();
                    fence_proxy_async_smem();
                    tc_fence_before_sync();
                    mbar_arrive(&bars[B_CBREADY]);
                }
            }
        }
    } else if (warp >= 8 && warp < 12) {
        // ================= Q~ = Q * e^{m-x_t+rho} dqk^-1/2 in place =================
        const int t = tid - 256;
        for (int k = 0; k < NCH; ++k) {
            const uint32_t ph = k & 1;
            const float winq = gbase[(size_t)k * GW + G_WINQ + t];
            if (!(mbar_wait(&bars[B_QFULL], ph, abort_flag) && mbar_wait(&bars[B_SDONE], ph, abort_flag))) break;
            // q . n from the raw tile first (Q~ is only needed by the last MMA group of the tile, so this is
            // off the critical path): needs n of the previous tile final and the previous epilogue done with s_qn
            if (!(k == 0 ? mbar_wait(&bars[B_CBREADY], 0, abort_flag) : mbar_wait(&bars[B_NDONE], (k - 1) & 1, abort_flag))) break;
            if (k > 0 && !mbar_wait(&bars[B_HFREE], (k - 1) & 1, abort_flag)) break;
            qn_pass<DQK>(smem, s_n, s_qn, gbase + (size_t)k * GW + G_WINQ, warp - 8, lane);
            mbar_arrive(&bars[B_QNDONE]);
            scale_rows<DQK>(smem + SM::Q, t, winq);
            fence_proxy_async_smem();   // generic-proxy writes -> visible to the tensor-core (async) proxy
            mbar_arrive(&bars[B_QSCALED]);
        }
    } else if (warp >= 12 && warp < 16) {
        // ================= K~ = K * e^{u_t-x_last} in place; C pass =================
        const int r = tid - 384;                         // K row / row within a 128-row half of C = TMEM lane
        const uint32_t lane_off = (uint32_t)(r & ~31) << 16;
        const bool has_state = p.C0 != nullptr;
        // ---- prologue: rows [0,128) of the initial state (rows [128,256) by the P warps), and n
        {
            c_init_half<DQK>(smem, T_C + lane_off, has_state ? p.C0 + ((size_t)bh * DQK + r) * p.dv + col0 : nullptr, r,
                             gbase[G_SCAL + 0]);
            for (int j = r; j < DQK; j += 128) s_n[j] = has_state ? p.n0[(size_t)bh * DQK + j] : 0.f;
            tmem_wait_st();
            fence_proxy_async_smem();
            tc_fence_before_sync();
            mbar_arrive(&bars[B_CBREADY]);
        }
        for (int k = 0; k < NCH; ++k) {
            const uint32_t ph = k & 1;
            const float *g = gbase + (size_t)k * GW;
            const float w = g[G_W + r];
            const bool last = (k == NCH - 1);
            const float decay_next = last ? g[G_SCAL + 2] : g[GW + G_SCAL + 0];
            if (!(mbar_wait(&bars[B_KFULL], ph, abort_flag) && mbar_wait(&bars[B_SDONE], ph, abort_flag))) break;
            scale_rows<DQK>(smem + SM::K, r, w);
            fence_proxy_async_smem();
            mbar_arrive(&bars[B_KSCALED]);
            // C pass after the state update: refresh Cb (needs the read-out of this tile finished with the
            // old Cb), pre-scale C for the next tile; after the last tile write C out instead.
            if (!(mbar_wait(&bars[B_UPDDONE], ph, abort_flag) && mbar_wait(&bars[B_H1DONE], ph, abort_flag))) break;
            tc_fence_after_sync();
            c_pass_half<DQK>(smem, T_C + lane_off, r, last, decay_next, p.C1 + ((size_t)bh * DQK + r) * p.dv + col0);
            if (!last) {
                tmem_wait_st();
                fence_proxy_async_smem();
                tc_fence_before_sync();
                mbar_arrive(&bars[B_CBREADY]);
            }
        }
    } else if (warp >= 16) {
        // ===== normaliser update n' = decay n + colsum(K~); H epilogue =====
        const int r = tid - 512;                         // token row of H = TMEM lane
        const uint32_t lane_off = (uint32_t)(r & ~31) << 16;
        for (int k = 0; k < NCH; ++k) {
            const uint32_t ph = k & 1;
            const float *g = gbase + (size_t)k * GW;
            const float decay = g[G_SCAL + 0];
            const bool last = (k == NCH - 1);
            // column sums of K~
            if (!mbar_wait(&bars[B_KSCALED], ph, abort_flag)) break;
            const int q = r >> 5, cp = r & 31;   // warp -> 64-column box, lane -> column pair
            float s0 = 0.f, s1 = 0.f;
            if (q < NBOX) {
                const unsigned char *box = smem + SM::K + q * SM::BOX + ((cp & 3) << 2);
                float a0[4] = {0.f, 0.f, 0.f, 0.f}, a1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 8
                for (int tt = 0; tt < LT; tt += 4) {
#pragma unroll
                    for (int x = 0; x < 4; ++x) {
                        const uint32_t off = (tt + x) * 128 + ((((cp >> 2) ^ ((tt + x) & 7))) << 4);
                        const float2 f = unpack_bf16(*reinterpret_cast<const uint32_t *>(box + off));
                        a0[x] += f.x; a1[x] += f.y;
                    }
                }
                s0 = (a0[0] + a0[1]) + (a0[2] + a0[3]);
                s1 = (a1[0] + a1[1]) + (a1[2] + a1[3]);
            }
            mbar_arrive(&bars[B_KREAD]);   // K~ no longer read by the CUDA cores: the tile may be reloaded
            // n is rewritten only after q~ . n of this tile has been taken
            if (!mbar_wait(&bars[B_QNDONE], ph, abort_flag)) break;
            if (q < NBOX) {
                const int j = q * 64 + cp * 2;
                const float n0v = decay * s_n[j] + s0, n1v = decay * s_n[j + 1] + s1;
                s_n[j] = n0v;
                s_n[j + 1] = n1v;
                if (last && blockIdx.y == 0) {
                    const float fr = g[G_SCAL + 2];   // n = n~ e^{rho}
                    p.n1[(size_t)bh * DQK + j] = n0v * fr; p.n1[(size_t)bh * DQK + j + 1] = n1v * fr;
                }
            }
            mbar_arrive(&bars[B_NDONE]);
            // epilogue: h = H / (max(|den|, e^{-m_t}) + eps)
            if (!(mbar_wait(&bars[B_PREADY], ph, abort_flag) && mbar_wait(&bars[B_H2DONE], ph, abort_flag) &&
                  mbar_wait(&bars[B_H1DONE], ph, abort_flag))) break;
            tc_fence_after_sync();
            const float den = s_qn[r] + s_rs[ph * LT + r];   // q~ . n already carries the row scale
            const float inv = 1.0f / (fmaxf(fabsf(den), g[G_EMT + r]) + p.eps);
            // H -> bf16 h tile staged in the (now idle) V buffer, in the swizzled box layout of the h
            // tensor maps; one thread then issues TMA stores to this GPU's h and to every peer's buffer
            unsigned char *stage = smem + SM::V + r * 128;
#pragma unroll 1
            for (int c0 = 0; c0 < DVS; c0 += 64) {
                uint32_t va[32], vb[32];
                tmem_ld32(T_H + lane_off + c0, va);
                tmem_ld32(T_H + lane_off + c0 + 32, vb);
                tmem_wait_ld();
                unsigned char *box = stage + (c0 >> 6) * SM::BOX;
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                    uint4 o;
                    o.x = pack_bf16(__uint_as_float(va[j]) * inv, __uint_as_float(va[j + 1]) * inv);
                    o.y = pack_bf16(__uint_as_float(va[j + 2]) * inv, __uint_as_float(va[j + 3]) * inv);
                    o.z = pack_bf16(__uint_as_float(va[j + 4]) * inv, __uint_as_float(va[j + 5]) * inv);
                    o.w = pack_bf16(__uint_as_float(va[j + 6]) * inv, __uint_as_float(va[j + 7]) * inv);
                    *reinterpret_cast<uint4 *>(box + ((((j >> 3)) ^ (r & 7)) << 4)) = o;
                    o.x = pack_bf16(__uint_as_float(vb[j]) * inv, __uint_as_float(vb[j + 1]) * inv);
                    o.y = pack_bf16(__uint_as_float(vb[j + 2]) * inv, __uint_as_float(vb[j + 3]) * inv);
                    o.z = pack_bf16(__uint_as_float(vb[j + 4]) * inv, __uint_as_float(vb[j + 5]) * inv);
                    o.w = pack_bf16(__uint_as_float(vb[j + 6]) * inv, __uint_as_float(vb[j + 7]) * inv);
                    *reinterpret_cast<uint4 *>(box + ((((j >> 3) + 4) ^ (r & 7)) << 4)) = o;
                }
            }
            tc_fence_before_sync();
            mbar_arrive(&bars[B_HFREE]);          // H in TMEM has been read
            fence_proxy_async_smem();
            mbar_arrive(&bars[B_HSTAGED]);
        }
    }

    // ---- teardown (every thread gets here, also after an abort) ----------------
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, 512);
    if (tid == 0 && *abort_flag) atomicExch(p.status, 1);
}

}  // namespace

bool mlstm_chunkwise_tc_shape_ok(const ChunkwiseParams &p, int dtype) {
    if (dtype != XLSTM_BF16) return false;
    if (p.dqk != 256 && p.dqk != 128) return false;
    if (p.dv % DVS) return false;
    if (p.S < LT || p.S / LT > 65535 * (GP_THREADS / 32)) return false;   // grid of the gate pre-pass
    for (int d = 0; d < 3; ++d)
        if (p.sq[d] % 8 || p.sk[d] % 8 || p.sv[d] % 8 || p.sh[d] % 8) return false;  // 16-byte TMA / store alignment
    if ((reinterpret_cast<uintptr_t>(p.q) | reinterpret_cast<uintptr_t>(p.k) | reinterpret_cast<uintptr_t>(p.v) |
         reinterpret_cast<uintptr_t>(p.h)) & 15u)   // (h is NULL in the token-sharded mode)
        return false;
    if (p.dv / DVS > 65535) return false;
    return true;
}

bool mlstm_chunkwise_tc_driver_ok() { return get_encode_tiled() != nullptr; }

bool mlstm_chunkwise_tc_supported(const ChunkwiseParams &p, int dtype) {
    return mlstm_chunkwise_tc_shape_ok(p, dtype) && mlstm_chunkwise_tc_driver_ok();
}

namespace {

// Layout of the caller-provided scratch.  P > 1 adds the per-segment states of the segment-parallel mode.
struct WsLayout {
    size_t gates, tail_n, tail_m, path, chain, seg_C[2], seg_n[2], seg_m[2], total;
    int P, seg_tiles;
};

constexpr int SM_COUNT = 148;          // B200
constexpr int MIN_SEG_TILES = 16;      // a shorter segment is dominated by its prologue (state in) and epilogue (state out)

// Number of segments every sequence is cut into: while the grid of persistent CTAs (one per head and 128 dv
// columns) fills at most half of the SMs, cutting the sequence buys parallelism at the price of the state-only
// first pass (about a quarter of a full pass) and of the states going through HBM once.
int plan_segments(int BH, int dv, int nch) {
    const int ctas = BH * (dv / DVS);
    int P = SM_COUNT / ctas;
    if (P > nch / MIN_SEG_TILES) P = nch / MIN_SEG_TILES;
    if (P > 64) P = 64;
    if (P < 2) return 1;
    for (int d = P; 4 * d >= 3 * P; --d)      // segments of equal length, if a count close to P divides the tiles
        if (nch % d == 0) return d;
    return P;
}

WsLayout ws_layout(int B, int NH, int S, int dqk, int dv, int P) {
    WsLayout w{};
    const size_t BH = (size_t)B * NH, nch = (size_t)(S / LT);
    w.P = P;
    w.seg_tiles = (int)((nch + P - 1) / P);
    w.P = (int)((nch + w.seg_tiles - 1) / w.seg_tiles);          // no empty segment
    auto up = [](size_t x) { return (x + 255) & ~(size_t)255; };
    size_t o = WS_HEADER;                                        // status word
    w.gates = o;  o = up(o + BH * nch * GW * sizeof(float));     // per-token gate scalars
    w.tail_n = o; o = up(o + BH * dqk * sizeof(float));          // hand-over state for a tail on the exact path
    w.tail_m = o; o = up(o + BH * sizeof(float));
    w.path = o;   o = up(o + BH * w.P * sizeof(int));            // path flag per (head, segment)
    w.chain = o;  o = up(o + BH * nch * GC * sizeof(double));    // chain scratch of the gate pre-pass
    if (w.P > 1) {                                               // local / end states and start states of the segments
        const size_t VH = BH * w.P;
        for (int set = 0; set < 2; ++set) {
            w.seg_C[set] = o; o = up(o + VH * dqk * dv * sizeof(float));
            w.seg_n[set] = o; o = up(o + VH * dqk * sizeof(float));
            w.seg_m[set] = o; o = up(o + VH * sizeof(float));
        }
    }
    w.total = o + 256;
    return w;
}

std::atomic<int> g_general_only{0};
std::atomic<int> g_segments{-1};       // -1: planned from the grid size; >= 1: forced (tests)

}  // namespace

size_t mlstm_chunkwise_tc_workspace(int B, int NH, int S, int dqk, int dv, int L) {
    (void)L;
    const int nch = S / LT;
    const int forced = g_segments.load();
    const int P = forced >= 1 ? (forced > nch ? (nch > 0 ? nch : 1) : forced) : plan_segments(B * NH, dv, nch);
    return ws_layout(B, NH, S, dqk, dv, P).total;
}

size_t mlstm_chunkwise_tc_workspace_min(int B, int NH, int S, int dqk, int dv) {
    return ws_layout(B, NH, S, dqk, dv, 1).total;
}

void mlstm_chunkwise_tc_set_general_only(int on) { g_general_only.store(on ? 1 : 0); }
void mlstm_chunkwise_tc_set_segments(int segments) { g_segments.store(segments >= 1 ? segments : -1); }

int mlstm_chunkwise_tc(const ChunkwiseParams &p, void *workspace, size_t workspace_bytes, cudaStream_t st) {
    const int s_full = (p.S / LT) * LT;
    const int nch = s_full / LT;
    const int BH = p.B * p.NH;
    if (!workspace) return XLSTM_ERR_WORKSPACE;
    // the segment-parallel mode if the scratch holds its states, else the plain single pass
    const int forced = g_segments.load();
    int P = forced >= 1 ? (forced > nch ? nch : forced) : plan_segments(BH, p.dv, nch);
    WsLayout w = ws_layout(p.B, p.NH, s_full, p.dqk, p.dv, P);
    if (workspace_bytes < w.total) {
        w = ws_layout(p.B, p.NH, s_full, p.dqk, p.dv, 1);
        if (workspace_bytes < w.total) return XLSTM_ERR_WORKSPACE;
    }
    P = w.P;
    const int seg_tiles = w.seg_tiles;
    unsigned char *ws = static_cast<unsigned char *>(workspace);
    int *status = reinterpret_cast<int *>(ws);
    float *gates = reinterpret_cast<float *>(ws + w.gates);
    float *tail_n = reinterpret_cast<float *>(ws + w.tail_n);
    float *tail_m = reinterpret_cast<float *>(ws + w.tail_m);
    int *path = reinterpret_cast<int *>(ws + w.path);
    double *chain = reinterpret_cast<double *>(ws + w.chain);
    const size_t CE = (size_t)p.dqk * p.dv;                         // elements of one C
    // set A: pass 1 local end states (pass 2: end states, unused); set B: the true start state of every segment
    float *segA_C = reinterpret_cast<float *>(ws + w.seg_C[0]), *segA_n = reinterpret_cast<float *>(ws + w.seg_n[0]);
    float *segA_m = reinterpret_cast<float *>(ws + w.seg_m[0]);
    float *segB_C = reinterpret_cast<float *>(ws + w.seg_C[1]), *segB_n = reinterpret_cast<float *>(ws + w.seg_n[1]);
    float *segB_m = reinterpret_cast<float *>(ws + w.seg_m[1]);
    const bool tail = s_full < p.S;
    if (tail && p.n_peer) return XLSTM_ERR_UNSUPPORTED;   // the exact tail path writes the local h only
    if (p.tok_per_rank > 0 && (p.tok_per_rank % LT || (long long)p.tok_per_rank * p.n_peer != s_full)) return XLSTM_ERR_INVALID;
    if (cudaMemsetAsync(status, 0, sizeof(int), st) != cudaSuccess) return XLSTM_ERR_CUDA;

    const __nv_bfloat16 *ig = static_cast<const __nv_bfloat16 *>(p.ig), *fg = static_cast<const __nv_bfloat16 *>(p.fg);
    const dim3 tg((nch + GP_THREADS / 32 - 1) / (GP_THREADS / 32), BH);
    mlstm_gate_stats_kernel<__nv_bfloat16><<<tg, GP_THREADS, 0, st>>>(ig, fg, p.sg[0], p.sg[1], p.sg[2], chain, p.NH, nch,
                                                                      p.gate_cap);
    if (cudaGetLastError() != cudaSuccess) return XLSTM_ERR_CUDA;

    TcParams tp{};
    if (!make_tmap_bf16_4d(&tp.tq, p.q, p.dqk, s_full, p.NH, p.B, p.sq[2], p.sq[1], p.sq[0], LT) ||
        !make_tmap_bf16_4d(&tp.tk, p.k, p.dqk, s_full, p.NH, p.B, p.sk[2], p.sk[1], p.sk[0], LT) ||
        !make_tmap_bf16_4d(&tp.tv, p.v, p.dv, s_full, p.NH, p.B, p.sv[2], p.sv[1], p.sv[0], LT))
        return XLSTM_ERR_UNSUPPORTED;
    const int n_dest = p.tok_per_rank > 0 ? p.n_peer : 1 + p.n_peer;
    for (int i = 0; i < n_dest; ++i) {
        void *dst = p.tok_per_rank > 0 ? p.h_peer[i] : (i == 0 ? p.h : p.h_peer[i - 1]);
        if (!make_tmap_bf16_4d(&tp.th[i], dst, p.dv, p.tok_per_rank > 0 ? p.tok_per_rank : s_full, p.NH, p.B, p.sh[2], p.sh[1],
                               p.sh[0], LT))
            return XLSTM_ERR_UNSUPPORTED;
    }
    tp.tok_per_rank = p.tok_per_rank;
    tp.gates = gates;
    tp.NH = p.NH; tp.dv = p.dv; tp.NCH = nch; tp.eps = p.eps; tp.log2_qscale = log2f(p.qscale); tp.status = status;
    tp.path = path; tp.h = p.h; tp.P = P; tp.seg_tiles = seg_tiles;
    for (int d = 0; d < 3; ++d) tp.sh[d] = p.sh[d];
    const dim3 grid(BH * P, p.dv / DVS);

    // one forward over all (head, segment) pairs: chain + per-token scalars of the gate pre-pass, then the two
    // tensor-core kernels.  Two launches over the same grid: every CTA looks at its path flag (written by the
    // pre-pass) and returns at once if it belongs to the other kernel, so the choice needs no host round trip.
    auto forward = [&](const float *m0v, int m0_auto, float *m_out, bool state_only) -> int {
        mlstm_gate_chain_kernel<<<BH * P, 32, 0, st>>>(m0v, chain, m_out, path, nch, P, seg_tiles, g_general_only.load(),
                                                       m0_auto);
        mlstm_gate_write_kernel<__nv_bfloat16><<<tg, GP_THREADS, 0, st>>>(ig, fg, p.sg[0], p.sg[1], p.sg[2], chain, path, gates,
                                                                          p.NH, nch, P, seg_tiles, p.qscale, p.gate_cap);
        if (cudaGetLastError() != cudaSuccess) return XLSTM_ERR_CUDA;
        const int rc = state_only ? mlstm_chunkwise_tc_scan_launch(tp, grid, p.dqk, st) : mlstm_chunkwise_tc_fast_launch(tp, grid, p.dqk, st);
        if (rc != XLSTM_OK) return rc;
        if (p.dqk == 256) {
            auto kern = mlstm_chunkwise_tc_kernel<256>;
            if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Smem<256>::TOTAL) != cudaSuccess)
                return XLSTM_ERR_CUDA;
            kern<<<grid, THREADS, Smem<256>::TOTAL, st>>>(tp);
        } else {
            auto kern = mlstm_chunkwise_tc_kernel<128>;
            if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Smem<128>::TOTAL) != cudaSuccess)
                return XLSTM_ERR_CUDA;
            kern<<<grid, THREADS, Smem<128>::TOTAL, st>>>(tp);
        }
        return cudaGetLastError() == cudaSuccess ? XLSTM_OK : XLSTM_ERR_CUDA;
    };

    float *n_final = tail ? tail_n : p.n1, *m_final = tail ? tail_m : p.m1;
    if (P == 1) {
        tp.C0 = p.C0; tp.n0 = p.n0; tp.C1 = p.C1; tp.n1 = n_final; tp.n_h = n_dest;
        const int rc = forward(p.C0 ? p.m0 : nullptr, 0, m_final, false);
        if (rc != XLSTM_OK) return rc;
    } else {
        // pass 1: every segment from an empty state -> its local end state: the state-only scan kernel (segments whose
        // gates need the general kernel run that one in full, with nothing stored)
        tp.C0 = nullptr; tp.n0 = nullptr; tp.C1 = segA_C; tp.n1 = segA_n; tp.n_h = 0;
        int rc = forward(nullptr, 1, segA_m, true);
        if (rc != XLSTM_OK) return rc;
        // the true state at the start of every segment, and the final state
        const int slabs = (int)(((CE + p.dqk) / COMB_VEC + COMB_THREADS - 1) / COMB_THREADS);   // one vector per thread
        mlstm_segment_combine_kernel<<<dim3(BH, slabs), COMB_THREADS, 0, st>>>(
            p.C0, p.n0, p.C0 ? p.m0 : nullptr, segA_C, segA_n, segA_m, chain, segB_C, segB_n, segB_m, p.C1, n_final,
            m_final, nch, P, seg_tiles, p.dqk, p.dv);
        if (cudaGetLastError() != cudaSuccess) return XLSTM_ERR_CUDA;
        // pass 2: every segment from its true start state
        tp.C0 = segB_C; tp.n0 = segB_n; tp.C1 = segA_C; tp.n1 = segA_n; tp.n_h = n_dest;
        rc = forward(segB_m, 0, segA_m, false);
        if (rc != XLSTM_OK) return rc;
    }
    if (!tail) return XLSTM_OK;

    // S mod 128 tail on the exact path, continuing from (C1, tail_n, tail_m).  C is handed over in
    // place: every CTA of that kernel reads only the columns it later writes.
    ChunkwiseParams t = p;
    const size_t esz = 2;
    t.q = static_cast<const unsigned char *>(p.q) + (size_t)s_full * p.sq[2] * esz;
    t.k = static_cast<const unsigned char *>(p.k) + (size_t)s_full * p.sk[2] * esz;
    t.v = static_cast<const unsigned char *>(p.v) + (size_t)s_full * p.sv[2] * esz;
    t.h = static_cast<unsigned char *>(p.h) + (size_t)s_full * p.sh[2] * esz;
    t.ig = static_cast<const unsigned char *>(p.ig) + (size_t)s_full * p.sg[2] * esz;
    t.fg = static_cast<const unsigned char *>(p.fg) + (size_t)s_full * p.sg[2] * esz;
    t.S = p.S - s_full;
    t.L = 64;
    t.C0 = p.C1; t.n0 = tail_n; t.m0 = tail_m;
    return mlstm_chunkwise_simt(t, XLSTM_BF16, st);
}

}  // namespace xl
