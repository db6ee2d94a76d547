// Chunkwise mLSTM forward on the Blackwell tensor cores for gates of bounded in-tile spread.
//
// Same decomposition as the general kernel (one persistent CTA per 128 dv columns of a head, C resident in
// TMEM for the whole sequence, 128-token tiles), but with every gate factor moved off the 64 KB Q and K
// tiles.  With u_s = i_s - b_s, m the stabiliser carried into the tile, x_t = max(m, max_{s<=t} u_s) and
// the accumulator kept as C~ = C e^{-rho}:
//
//   a_s    = e^{u_s - m - rho}                 one factor per token, applied to its V row:  V~ = diag(a) V
//   C~    += K^T V~                            raw K; no decay of C~ (rho absorbs it: rho' = rho + m - x_last)
//   H'     = Q C~b + tril(Q K^T) V~            raw Q; tril(S) only masked and rounded, no exponentials
//   h_t    = winq_t H'_t / (max(|winq_t (q_t . n~ + sum_{s<=t} S_ts a_s)|, e^{-m_t}) + eps),
//   winq_t = e^{m - x_t + rho} dqk^-1/2
//
// which equals the stabilised recurrence because e^{u_s - x_t} = winq_t a_s dqk^1/2.  The factorisation
// needs a_s inside the fp32 / bf16 exponent range, i.e. max_s u_s - m bounded for every tile of the head;
// the gate pre-pass checks that (path flag per head) and heads that fail it run the general kernel, whose
// exponents are all differences <= 0.  When -rho' passes the rescale threshold C~ and n~ are multiplied
// by e^{rho'} once, after that tile's update, and rho restarts at 0.
//
// What this removes from the tile: the in-place scaling passes over Q and K (256 KB of shared-memory
// traffic, both on the serial chain between the S MMAs and the update) and the per-element exponentials
// of the gate matrix; what is left on the CUDA cores is one pass over the 32 KB V tile.
// MMA issue order per tile: read-out (Q, Cb of the previous tile), S (Q, K), update (K, V~), P V~ (V~) - every
// operand buffer is used by two ADJACENT groups and is free for about half a tile, so the reload of the
// next tile's Q, K, V hides under the other groups although each is single-buffered; the update is issued
// per 128-row half of C so that the bf16 refresh of Cb for one half runs under the MMAs of the other.
//
// Roles (640 threads): warp 0 TMA producer, warp 1 MMA issuer (+TMEM alloc), warp 2 TMA stores of the staged h
// tile (to this GPU and, in head-sharded runs, to every peer); warps 4-7 V~ scaling, gate matrix P and the C pass for rows
// [128,256); warps 8-11 q . n~ from the raw Q tile; warps 12-15 normaliser update and the C pass for rows
// [0,128); warps 16-19 the upper pieces of the gate matrix, then the epilogue (h tile staged in the V buffer
// once P V~ has read it).
// Every mbarrier wait is bounded; a time-out sets the status word in the scratch buffer, releases all roles
// and frees TMEM before the CTA returns.
#include "mlstm_chunkwise_tc.cuh"

namespace xl {

namespace {

using namespace tc;
using namespace tcw;

enum { F_QFULL = 0, F_KFULL, F_VFULL, F_SDONE, F_UPDA, F_UPDB, F_PVDONE, F_VSCALED, F_PREADY, F_CBA, F_CBB,
       F_HFREE, F_QNDONE, F_NDONE, F_HSTAGED, F_VFREE, F_SAREADY, F_NBARS };
static_assert(F_NBARS <= 24, "barrier slots");

// C pass for one 128-row half after the state update: optional rescale of C~ in TMEM, then the bf16 copy
// Cb (in the frame the next tile reads it in); after the last tile the fp32 rows go to `dst` instead.
template <int DQK>
__device__ __forceinline__ void c_pass_fast(unsigned char *smem, uint32_t t_half, int j, bool last, float mul,
                                            float frame, float *dst) {
    using SM = Smem<DQK>;
#pragma unroll 1
    for (int c0 = 0; c0 < DVS; c0 += 64) {
        uint32_t va[32], vb[32];
        tmem_ld32(t_half + c0, va);
        tmem_ld32(t_half + c0 + 32, vb);
        tmem_wait_ld();
        if (last) {
#pragma unroll
            for (int x = 0; x < 32; x += 4) {
                *reinterpret_cast<float4 *>(dst + c0 + x) =
                    make_float4(__uint_as_float(va[x]) * frame, __uint_as_float(va[x + 1]) * frame,
                                __uint_as_float(va[x + 2]) * frame, __uint_as_float(va[x + 3]) * frame);
                *reinterpret_cast<float4 *>(dst + c0 + 32 + x) =
                    make_float4(__uint_as_float(vb[x]) * frame, __uint_as_float(vb[x + 1]) * frame,
                                __uint_as_float(vb[x + 2]) * frame, __uint_as_float(vb[x + 3]) * frame);
            }
        } else {
            if (mul != 1.0f) {   // CTA-uniform: a rescale tile (rare)
#pragma unroll
                for (int x = 0; x < 32; ++x) {
                    va[x] = __float_as_uint(__uint_as_float(va[x]) * mul);
                    vb[x] = __float_as_uint(__uint_as_float(vb[x]) * mul);
                }
                tmem_st32(t_half + c0, va);
                tmem_st32(t_half + c0 + 32, vb);
            }
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
        }
    }
}

// One 32 x 32 piece of the gate matrix: S values in `r` -> causal mask on the diagonal piece, row-sum
// contribution sum_s S_ts a_s (fp32, before rounding; four independent partial sums) and the bf16 pairs of P.
// P piece pc is written over the FIRST 16 columns of S piece pc (columns [32 pc, 32 pc + 16)), so a piece
// never lands on S values that another warp has still to read; the P V~ MMAs address the pieces accordingly.
__device__ __forceinline__ float p_piece(const uint32_t (&r)[32], uint32_t t_rows, int pc, bool diag, int lane, const float4 *a4) {
    uint32_t packed[16];
    float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
        const float4 a = a4[(pc * 32 + j) >> 2];
        float p0 = __uint_as_float(r[j]), p1 = __uint_as_float(r[j + 1]);
        float p2 = __uint_as_float(r[j + 2]), p3 = __uint_as_float(r[j + 3]);
        if (diag) {
            if (j > lane) p0 = 0.f;
            if (j + 1 > lane) p1 = 0.f;
            if (j + 2 > lane) p2 = 0.f;
            if (j + 3 > lane) p3 = 0.f;
        }
        s0 = fmaf(p0, a.x, s0); s1 = fmaf(p1, a.y, s1);
        s2 = fmaf(p2, a.z, s2); s3 = fmaf(p3, a.w, s3);
        packed[j >> 1] = pack_bf16(p0, p1);
        packed[(j >> 1) + 1] = pack_bf16(p2, p3);
    }
    tmem_st16(t_rows + pc * 32, packed);
    return (s0 + s1) + (s2 + s3);
}

// The gate-matrix pass is shared by TWO warps per block of 32 rows (the triangle gives row block q the pieces
// 0..q, so one warp per block would leave the last block with four pieces and the first with one): the "lower"
// warp takes the pieces [0, nl), the "upper" warp [nl, q] and zero-fills the pieces above the diagonal, with
// nl = (q + 2) / 2: at most two pieces per warp.  This function does the pieces [first, last) and zero-fills
// [zfirst, 4); it returns the warp's part of the row sums of tril(S) diag(a).
__device__ __forceinline__ float p_pass_part(uint32_t t_rows, int q, int lane, const float4 *a4, int first, int last,
                                             int zfirst) {
    float rowsum = 0.f;
    uint32_t r[32];
    for (int pc = first; pc < last; ++pc) {
        tmem_ld32(t_rows + pc * 32, r);
        tmem_wait_ld();
        rowsum += p_piece(r, t_rows, pc, pc == q, lane, a4);
    }
#pragma unroll
    for (int j = 0; j < 32; ++j) r[j] = 0u;
    for (int pc = zfirst; pc < 4; ++pc) tmem_st16(t_rows + pc * 32, reinterpret_cast<const uint32_t (&)[16]>(r));
    tmem_wait_st();
    return rowsum;
}

template <int DQK>
__global__ void __launch_bounds__(THREADS, 1) mlstm_chunkwise_tc_fast_kernel(const __grid_constant__ TcParams p) {
    using SM = Smem<DQK>;
    constexpr int NBOX = SM::NBOX;
    constexpr int NHALF = DQK / 128;
    constexpr int F_UPDLAST = (NHALF == 2) ? F_UPDB : F_UPDA;
    extern __shared__ __align__(1024) unsigned char smem[];
    const int bh = blockIdx.x;     // (batch, head, segment): index of the states and of the path flag
    if (p.path[bh] != 1) return;   // these gates need the general kernel (CTA-uniform, before any set-up)

    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + SM::BARS);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + SM::MISC);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + SM::MISC + 4);
    float *s_n = reinterpret_cast<float *>(smem + SM::N_VEC);
    float *s_qn = reinterpret_cast<float *>(smem + SM::QN);
    float *s_rs = reinterpret_cast<float *>(smem + SM::INV);        // row sums of tril(S) diag(a)
    float *s_a = s_rs + LT;                                          // a_s of the current tile

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int bhr = bh / p.P, tile0 = (bh % p.P) * p.seg_tiles;   // (batch, head) and first tile of this segment
    const int b = bhr / p.NH, hd = bhr % p.NH;
    const int col0 = blockIdx.y * DVS;
    const int NCH = min(p.seg_tiles, p.NCH - tile0);
    const float *gbase = p.gates + ((size_t)bhr * p.NCH + tile0) * GW;

    if (tid == 0) {
        *abort_flag = (smem_u32(smem) & 1023u) ? 1 : 0;  // swizzled tiles need a 1024-byte aligned base
        mbar_init(&bars[F_QFULL], 1);    mbar_init(&bars[F_KFULL], 1);    mbar_init(&bars[F_VFULL], 1);
        mbar_init(&bars[F_SDONE], 1);    mbar_init(&bars[F_UPDA], 1);     mbar_init(&bars[F_UPDB], 1);
        mbar_init(&bars[F_PVDONE], 1);
        mbar_init(&bars[F_VSCALED], 128); mbar_init(&bars[F_PREADY], 256); mbar_init(&bars[F_CBA], 128);
        mbar_init(&bars[F_CBB], 128);     mbar_init(&bars[F_HFREE], 128);  mbar_init(&bars[F_QNDONE], 128);
        mbar_init(&bars[F_NDONE], 128);   mbar_init(&bars[F_HSTAGED], 128); mbar_init(&bars[F_VFREE], 1);
        mbar_init(&bars[F_SAREADY], 128);
        mbar_fence_init();
        tma_prefetch_desc(&p.tq); tma_prefetch_desc(&p.tk); tma_prefetch_desc(&p.tv);
    }
    if (warp == 1) tmem_alloc(tmem_slot, 512);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    // S/P and H swap their two 128-column regions every tile: the read-out of tile k+1 accumulates where S/P of
    // tile k lived (free as soon as P V~ of tile k has run, in issue order) instead of waiting for the epilogue to
    // drain H of tile k; only S of tile k+1, issued a group later, needs the drained region.
    const uint32_t T_C = tmem;
    auto t_s = [tmem](int k) -> uint32_t { return tmem + 256 + 128 * (k & 1); };
    auto t_h = [tmem](int k) -> uint32_t { return tmem + 384 - 128 * (k & 1); };

    if (warp == 0) {
        // ================= TMA producer =================
        // Each buffer is reloaded as soon as its two consumers of the previous tile are done: Q after S (which
        // follows the read-out) and the q . n pass, K after the update and the normaliser sums, V after P V.
        if (lane == 0) {
            for (int k = 0; k < NCH; ++k) {
                const int t0 = (tile0 + k) * LT;
                const uint32_t pp = (k - 1) & 1;
                if (k > 0 && !(mbar_wait(&bars[F_SDONE], pp, abort_flag) && mbar_wait(&bars[F_QNDONE], pp, abort_flag))) break;
                mbar_expect_tx(&bars[F_QFULL], NBOX * SM::BOX);
                for (int q = 0; q < NBOX; ++q) tma_load_4d(smem + SM::Q + q * SM::BOX, &p.tq, &bars[F_QFULL], q * 64, t0, hd, b);
                // the normaliser update of tile k-1 is completion k of its barrier (completion 0 = initial n)
                if (k > 0 && !(mbar_wait(&bars[F_UPDLAST], pp, abort_flag) && mbar_wait(&bars[F_NDONE], k & 1, abort_flag))) break;
                mbar_expect_tx(&bars[F_KFULL], NBOX * SM::BOX);
                for (int q = 0; q < NBOX; ++q) tma_load_4d(smem + SM::K + q * SM::BOX, &p.tk, &bars[F_KFULL], q * 64, t0, hd, b);
                if (k > 0 && !mbar_wait(&bars[F_VFREE], pp, abort_flag)) break;   // P V~ done and the h tile staged in V stored
                mbar_expect_tx(&bars[F_VFULL], 2 * SM::BOX);
                for (int q = 0; q < 2; ++q) tma_load_4d(smem + SM::V + q * SM::BOX, &p.tv, &bars[F_VFULL], col0 + q * 64, t0, hd, b);
            }
        }
    } else if (warp == 1) {
        // ================= MMA issuer =================
        if (lane == 0) {
            constexpr uint32_t ID_KK = idesc_bf16(128, 128, false, false);  // S
            constexpr uint32_t ID_KM = idesc_bf16(128, 128, false, true);   // read-out, P V~
            constexpr uint32_t ID_MM = idesc_bf16(128, 128, true, true);    // state update
            const uint64_t dQ = smem_desc_sw128(smem_u32(smem + SM::Q), 0, 1024);
            const uint64_t dK = smem_desc_sw128(smem_u32(smem + SM::K), 0, 1024);
            const uint64_t dCb = smem_desc_sw128(smem_u32(smem + SM::CB), SM::CB_BLOCK, 1024);
            const uint64_t dKm = smem_desc_sw128(smem_u32(smem + SM::K), SM::BOX, 1024);
            const uint64_t dV = smem_desc_sw128(smem_u32(smem + SM::V), SM::BOX, 1024);
            for (int k = 0; k < NCH; ++k) {
                const uint32_t ph = k & 1;
                // H = Q Cb, one 128-row half of Cb at a time (the C pass of the other half may still run)
                // (H goes where S/P of the previous tile was: free, since that tile's P V~ was issued before)
                const uint32_t T_S = t_s(k), T_H = t_h(k);
                if (!(mbar_wait(&bars[F_QFULL], ph, abort_flag) && mbar_wait(&bars[F_CBA], ph, abort_flag))) break;
                tc_fence_after_sync();
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
                    const uint32_t o = ((kk >> 2) * SM::BOX + (kk & 3) * 32) >> 4;
                    mma_ss(T_H, dQ + o, dCb + kk * (2048 >> 4), ID_KM, kk > 0);
                }
                if (NHALF == 2) {
                    if (!mbar_wait(&bars[F_CBB], ph, abort_flag)) break;
                    tc_fence_after_sync();
#pragma unroll
                    for (int kk = 8; kk < 16; ++kk) {
                        const uint32_t o = ((kk >> 2) * SM::BOX + (kk & 3) * 32) >> 4;
                        mma_ss(T_H, dQ + o, dCb + kk * (2048 >> 4), ID_KM, true);
                    }
                }
                // S = Q K^T (the previous tile's P V~ was issued earlier and finishes first: in-order pipe)
                if (!mbar_wait(&bars[F_KFULL], ph, abort_flag)) break;
                if (k > 0 && !mbar_wait(&bars[F_HFREE], (k - 1) & 1, abort_flag)) break;   // S lands where H of the previous tile was
                tc_fence_after_sync();
#pragma unroll
                for (int kk = 0; kk < DQK / 16; ++kk) {
                    const uint32_t o = ((kk >> 2) * SM::BOX + (kk & 3) * 32) >> 4;
                    mma_ss(T_S, dQ + o, dK + o, ID_KK, kk > 0);
                }
                mma_commit(&bars[F_SDONE]);
                // C~ += K^T V~, per 128-row half (the C passes of the previous tile were waited for above)
                if (!mbar_wait(&bars[F_VSCALED], ph, abort_flag)) break;
                tc_fence_after_sync();
#pragma unroll
                for (int hf = 0; hf < NHALF; ++hf) {
#pragma unroll
                    for (int kk = 0; kk < LT / 16; ++kk)
                        mma_ss(T_C + hf * 128, dKm + ((hf * 2 * SM::BOX + kk * 2048) >> 4), dV + kk * (2048 >> 4), ID_MM, true);
                    mma_commit(&bars[hf == 0 ? F_UPDA : F_UPDB]);
                }
                // H += P V~
                if (!mbar_wait(&bars[F_PREADY], ph, abort_flag)) break;
                tc_fence_after_sync();
#pragma unroll
                for (int kk = 0; kk < LT / 16; ++kk)   // P piece kk / 2 sits in the first 16 columns of S piece kk / 2
                    mma_ts(T_H, T_S + (kk >> 1) * 32 + (kk & 1) * 8, dV + kk * (2048 >> 4), ID_KM, true);
                mma_commit(&bars[F_PVDONE]);
            }
        }
    } else if (warp == 2) {
        // ================= TMA stores of the staged h tile to this GPU's h and, in head-sharded runs, to the peers =================
        if (lane == 0) {
            for (int k = 0; k < NCH; ++k) {
                if (!mbar_wait(&bars[F_HSTAGED], k & 1, abort_flag)) break;
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
                mbar_arrive(&bars[F_VFREE]);
            }
            tma_store_wait_all();                 // all h writes performed before the CTA exits
        }
    } else if (warp >= 4 && warp < 8) {
        // ================= P = bf16(tril(S)) in place, row sums of tril(S) diag(a); C pass rows [128,256) =================
        const int t = tid - 128;                       // token row = TMEM lane
        const int t0w = t & ~31;                       // first row of this warp
        const uint32_t lane_off = (uint32_t)t0w << 16;
        if (NHALF == 2) {
            c_init_half<DQK>(smem, T_C + 128 + lane_off, p.C0 ? p.C0 + ((size_t)bh * DQK + 128 + t) * p.dv + col0 : nullptr,
                             128 + t, 1.0f);
            tmem_wait_st();
            fence_proxy_async_smem();
            tc_fence_before_sync();
            mbar_arrive(&bars[F_CBB]);
        }
        const float4 *a4 = reinterpret_cast<const float4 *>(s_a);
        for (int k = 0; k < NCH; ++k) {
            const uint32_t ph = k & 1;
            const float *g = gbase + (size_t)k * GW;
            // V~ = diag(a) V in place (these warps are idle until S completes; V arrives early in the tile)
            if (!mbar_wait(&bars[F_VFULL], ph, abort_flag)) break;
            scale_tile_rows<2>(smem + SM::V, SM::BOX, t, g[G_W + t]);
            fence_proxy_async_smem();   // generic-proxy writes -> visible to the tensor-core (async) proxy
            mbar_arrive(&bars[F_VSCALED]);
            if (!(mbar_wait(&bars[F_SAREADY], ph, abort_flag) && mbar_wait(&bars[F_SDONE], ph, abort_flag))) break;
            tc_fence_after_sync();
            // the lower pieces of this row block; the epilogue warp of the same rows takes the rest
            const float rowsum = p_pass_part(t_s(k) + lane_off, warp & 3, lane, a4, 0, ((warp & 3) + 2) >> 1, 4);
            s_rs[t] = rowsum;   // read by the epilogue warps after PREADY
            tc_fence_before_sync();
            mbar_arrive(&bars[F_PREADY]);
            if (NHALF == 2) {
                const bool last = (k == NCH - 1);
                if (!mbar_wait(&bars[F_UPDB], ph, abort_flag)) break;
                tc_fence_after_sync();
                c_pass_fast<DQK>(smem, T_C + 128 + lane_off, 128 + t, last, g[G_SCAL + 0], g[G_SCAL + 2],
                                 p.C1 + ((size_t)bh * DQK + 128 + t) * p.dv + col0);
                if (!last) {
                    tmem_wait_st();
                    fence_proxy_async_smem();
                    tc_fence_before_sync();
                    mbar_arrive(&bars[F_CBB]);
                }
            }
        }
    } else if (warp >= 8 && warp < 12) {
        // ================= a_s to shared memory, q . n~ from the raw Q tile =================
        const int t = tid - 256;
        for (int k = 0; k < NCH; ++k) {
            const uint32_t ph = k & 1;
            const float a = gbase[(size_t)k * GW + G_W + t];
            // the previous epilogue has read s_qn and the previous P pass / normaliser update have read s_a
            if (k > 0 && !mbar_wait(&bars[F_HFREE], (k - 1) & 1, abort_flag)) break;
            if (!mbar_wait(&bars[F_NDONE], ph, abort_flag)) break;    // n~ before this tile is final
            s_a[t] = a;
            mbar_arrive(&bars[F_SAREADY]);   // the gate-matrix warps need a_s, not q . n~
            if (!mbar_wait(&bars[F_QFULL], ph, abort_flag)) break;
            qn_pass<DQK>(smem, s_n, s_qn, nullptr, warp - 8, lane);
            mbar_arrive(&bars[F_QNDONE]);
        }
    } else if (warp >= 12 && warp < 16) {
        // ================= n~ += K^T a; C pass rows [0,128) =================
        const int r = tid - 384;
        const uint32_t lane_off = (uint32_t)(r & ~31) << 16;
        const bool has_state = p.C0 != nullptr;
        {
            c_init_half<DQK>(smem, T_C + lane_off, has_state ? p.C0 + ((size_t)bh * DQK + r) * p.dv + col0 : nullptr, r, 1.0f);
            for (int j = r; j < DQK; j += 128) s_n[j] = has_state ? p.n0[(size_t)bh * DQK + j] : 0.f;
            tmem_wait_st();
            fence_proxy_async_smem();
            tc_fence_before_sync();
            mbar_arrive(&bars[F_CBA]);
            mbar_arrive(&bars[F_NDONE]);      // completion 0: the initial n~
        }
        const int q = r >> 5, cp = r & 31;   // warp -> 64-column box of K, lane -> column pair
        for (int k = 0; k < NCH; ++k) {
            const uint32_t ph = k & 1;
            const float *g = gbase + (size_t)k * GW;
            const bool last = (k == NCH - 1);
            const float mul = g[G_SCAL + 0], frame = g[G_SCAL + 2];
            if (!(mbar_wait(&bars[F_KFULL], ph, abort_flag) && mbar_wait(&bars[F_QNDONE], ph, abort_flag))) break;
            if (q < NBOX) {
                const unsigned char *box = smem + SM::K + q * SM::BOX + ((cp & 3) << 2);
                float a0[4] = {0.f, 0.f, 0.f, 0.f}, a1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 8
                for (int tt = 0; tt < LT; tt += 4) {
                    const float4 av = *reinterpret_cast<const float4 *>(s_a + tt);
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
                if (last && blockIdx.y == 0) {   // n = n~ e^{rho'}
                    p.n1[(size_t)bh * DQK + j] = n0v * frame; p.n1[(size_t)bh * DQK + j + 1] = n1v * frame;
                }
            }
            mbar_arrive(&bars[F_NDONE]);   // K no longer read by the CUDA cores; n~ after this tile is final
            if (!mbar_wait(&bars[F_UPDA], ph, abort_flag)) break;
            tc_fence_after_sync();
            c_pass_fast<DQK>(smem, T_C + lane_off, r, last, mul, frame, p.C1 + ((size_t)bh * DQK + r) * p.dv + col0);
            if (!last) {
                tmem_wait_st();
                fence_proxy_async_smem();
                tc_fence_before_sync();
                mbar_arrive(&bars[F_CBA]);
            }
        }
    } else if (warp >= 16) {
        // ================= upper pieces of the gate matrix; epilogue: h = winq H' / (max(|den|, e^{-m_t}) + eps) =================
        const int r = tid - 512;                         // token row of S and H = TMEM lane
        const uint32_t lane_off = (uint32_t)(r & ~31) << 16;
        const float4 *a4 = reinterpret_cast<const float4 *>(s_a);
        const int q = warp & 3;
        for (int k = 0; k < NCH; ++k) {
            const uint32_t ph = k & 1;
            const float *g = gbase + (size_t)k * GW;
            const float winq = g[G_WINQ + r], emt = g[G_EMT + r];
            if (!(mbar_wait(&bars[F_SAREADY], ph, abort_flag) && mbar_wait(&bars[F_SDONE], ph, abort_flag))) break;
            tc_fence_after_sync();
            const float rs_upper = p_pass_part(t_s(k) + lane_off, q, lane, a4, (q + 2) >> 1, q + 1, q + 1);
            tc_fence_before_sync();
            mbar_arrive(&bars[F_PREADY]);
            if (!(mbar_wait(&bars[F_QNDONE], ph, abort_flag) && mbar_wait(&bars[F_PREADY], ph, abort_flag) &&
                  mbar_wait(&bars[F_PVDONE], ph, abort_flag))) break;
            tc_fence_after_sync();
            const float den = winq * (s_qn[r] + s_rs[r] + rs_upper);
            const float inv = winq / (fmaxf(fabsf(den), emt) + p.eps);
            // H -> bf16 h tile staged in the V buffer (idle: update and P V~ of this tile have completed), in the
            // swizzled box layout of the h tensor maps.  (Direct 16-byte stores from registers to global memory
            // were measured slower: 32 rows per instruction keep the load/store unit busy for ~2.5 k clocks per
            // tile and stall every other warp's shared-memory accesses.)
            unsigned char *stage = smem + SM::V + r * 128;
#pragma unroll 1
            for (int c0 = 0; c0 < DVS; c0 += 64) {
                uint32_t va[32], vb[32];
                tmem_ld32(t_h(k) + lane_off + c0, va);
                tmem_ld32(t_h(k) + lane_off + c0 + 32, vb);
                tmem_wait_ld();
                if (c0 == DVS - 64) {                 // H (and s_qn, s_rs) have been read: the next tile may proceed
                    tc_fence_before_sync();
                    mbar_arrive(&bars[F_HFREE]);
                }
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
            fence_proxy_async_smem();
            mbar_arrive(&bars[F_HSTAGED]);
        }
    }

    // ---- teardown (every thread gets here, also after an abort) ----------------
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, 512);
    if (tid == 0 && *abort_flag) atomicExch(p.status, 1);
}

}  // namespace

int mlstm_chunkwise_tc_fast_launch(const tcw::TcParams &tp, dim3 grid, int dqk, cudaStream_t st) {
    if (dqk == 256) {
        auto kern = mlstm_chunkwise_tc_fast_kernel<256>;
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Smem<256>::TOTAL) != cudaSuccess)
            return XLSTM_ERR_CUDA;
        kern<<<grid, THREADS, Smem<256>::TOTAL, st>>>(tp);
    } else {
        auto kern = mlstm_chunkwise_tc_fast_kernel<128>;
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Smem<128>::TOTAL) != cudaSuccess)
            return XLSTM_ERR_CUDA;
        kern<<<grid, THREADS, Smem<128>::TOTAL, st>>>(tp);
    }
    return cudaGetLastError() == cudaSuccess ? XLSTM_OK : XLSTM_ERR_CUDA;
}

}  // namespace xl
