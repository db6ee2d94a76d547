// Pieces shared by the two tensor-core kernels of the chunkwise mLSTM forward (the general one and the
// one for gate patterns whose in-tile spread is bounded): tile constants, the layout of the gate
// scratch, the kernel parameter block, the shared-memory map and the CUDA-core helpers.
#pragma once
#include "mlstm_chunkwise.cuh"
#include "tcgen05.cuh"

namespace xl {
namespace tcw {

using namespace tc;

constexpr int LT = 128;        // tokens per tile
constexpr int DVS = 128;       // dv columns per CTA
constexpr int THREADS = 640;
constexpr int GW = 6 * LT;     // floats of gate scratch per (head, tile)
constexpr int G_U2 = 0, G_X2 = LT, G_WINQ = 2 * LT, G_W = 3 * LT, G_EMT = 4 * LT, G_SCAL = 5 * LT;
constexpr float LOG2E = 1.4426950408889634f;
constexpr size_t WS_HEADER = 256;  // status word lives in the first bytes of the scratch

struct TcParams {
    CUtensorMap tq, tk, tv;
    const float *gates;            // [B*NH][NCH][GW]
    const float *C0, *n0;
    CUtensorMap th[8];             // h of this GPU, then the same head slot of up to 7 peer GPUs' buffers
    int n_h;                       // number of destinations (1 + peers); 0: h is not stored at all
    int tok_per_rank;              // > 0: th[r] is rank r's token-sharded buffer; a tile goes to the owner of its tokens only
    float *C1, *n1;
    int NH, dv, NCH;
    float eps, log2_qscale;
    int *status;
    const int *path;               // [B*NH*P] 1: this (head, segment) fits the bounded-spread kernel, 0: general kernel
    int P, seg_tiles;              // the sequence of every head is cut into P segments of seg_tiles tiles (P = 1: no cut);
                                   // blockIdx.x = (batch * NH + head) * P + segment; C0, n0, C1, n1 and path are per segment
    void *h;                       // h of this GPU as a plain pointer with its element strides (batch, head, token)
    int64_t sh[3];
};

template <int DQK> struct Smem {
    static constexpr int NBOX = DQK / 64;                  // 64-column TMA boxes of a Q / K tile
    static constexpr uint32_t BOX = LT * 128;              // bytes of one box: 128 rows x 128 B
    static constexpr uint32_t Q = 0;
    static constexpr uint32_t K = Q + NBOX * BOX;
    static constexpr uint32_t V = K + NBOX * BOX;          // 2 boxes (128 dv columns)
    static constexpr uint32_t CB = V + 2 * BOX;            // 2 N-blocks of [DQK rows x 128 B]
    static constexpr uint32_t CB_BLOCK = DQK * 128;
    static constexpr uint32_t SMALL = CB + 2 * CB_BLOCK;
    static constexpr uint32_t N_VEC = SMALL;               // float[DQK]   normaliser n
    static constexpr uint32_t QN = N_VEC + DQK * 4;        // float[LT]    q . n of the current tile
    static constexpr uint32_t INV = QN + LT * 4;           // float[2][LT] row sums of P, by tile parity
    static constexpr uint32_t BARS = INV + 2 * LT * 4;     // uint64[24]
    static constexpr uint32_t MISC = BARS + 24 * 8;        // tmem base, abort flag
    static constexpr uint32_t TOTAL = MISC + 16;
};

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&v);
}
// x * w for a packed pair of bf16, w = whi + wlo given as two packed bf16 pairs: rn(x*whi + rn(x*wlo)).
// Within 2^-16 of the correctly rounded product with the fp32 factor, at 2 instructions per pair.
__device__ __forceinline__ uint32_t scale_bf16x2(uint32_t x, uint32_t whi2, uint32_t wlo2) {
    const __nv_bfloat162 xv = *reinterpret_cast<const __nv_bfloat162 *>(&x);
    const __nv_bfloat162 r = __hfma2(xv, *reinterpret_cast<const __nv_bfloat162 *>(&whi2),
                                     __hmul2(xv, *reinterpret_cast<const __nv_bfloat162 *>(&wlo2)));
    return *reinterpret_cast<const uint32_t *>(&r);
}
__device__ __forceinline__ void split_scale(float w, uint32_t &whi2, uint32_t &wlo2) {
    const float hi = __bfloat162float(__float2bfloat16_rn(w));
    whi2 = pack_bf16(hi, hi);
    wlo2 = pack_bf16(w - hi, w - hi);
}
__device__ __forceinline__ float2 unpack_bf16(uint32_t u) {
    return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xffff0000u));
}

// q~ . n for all rows from the RAW Q tile (before it is scaled in place): the dot product q . n is taken
// in fp32 from the exact bf16 inputs and multiplied by the row scale afterwards, so the state part of the
// normaliser carries no bf16 rounding of Q~ (it matters where q . n cancels).  Lane mapping: lane = (g, c) with
// c the physical 16-byte chunk and g a row group; a warp owns the rows with (row & 7) in {2w, 2w+1}, so
// for a fixed residue rho every lane always meets the same LOGICAL chunk c ^ rho: its 8 values of n are
// loaded once per (rho, box) and the tile loads are 4 x 128 contiguous bytes per instruction.
template <int DQK>
__device__ __forceinline__ void qn_pass(const unsigned char *smem, const float *s_n, float *s_qn, const float *row_scale,
                                        int wl, int lane) {
    using SM = Smem<DQK>;
    constexpr int NBOX = SM::NBOX;
    const int c = lane & 7, g = lane >> 3;
    float part[2][4];
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        const int rho = 2 * wl + rr;
        const int row0 = rho + 8 * g;                 // rows row0 + 32 i
#pragma unroll
        for (int i = 0; i < 4; ++i) part[rr][i] = 0.f;
#pragma unroll
        for (int q = 0; q < NBOX; ++q) {
            // the lane's 8 values of n: two 16-byte loads, issued in an order that puts the 8 lanes of a
            // quarter-warp on 8 different 16-byte bank groups (lanes with logical chunk >= 4 take the upper half first)
            const int cx = c ^ rho, sw = (cx >> 2) & 1;
            const float *np = s_n + q * 64 + (cx << 3);
            const float4 x0 = *reinterpret_cast<const float4 *>(np + 4 * sw);
            const float4 x1 = *reinterpret_cast<const float4 *>(np + 4 * (1 - sw));
            const float4 na = sw ? x1 : x0, nb = sw ? x0 : x1;
            const unsigned char *base = smem + SM::Q + q * SM::BOX + row0 * 128 + (c << 4);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint4 v = *reinterpret_cast<const uint4 *>(base + i * 32 * 128);
                const float2 f0 = unpack_bf16(v.x), f1 = unpack_bf16(v.y), f2 = unpack_bf16(v.z), f3 = unpack_bf16(v.w);
                part[rr][i] += (f0.x * na.x + f0.y * na.y + f1.x * na.z + f1.y * na.w) +
                               (f2.x * nb.x + f2.y * nb.y + f3.x * nb.z + f3.y * nb.w);
            }
        }
    }
#pragma unroll
    for (int rr = 0; rr < 2; ++rr)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float v = part[rr][i];
            v += __shfl_xor_sync(0xffffffffu, v, 1);
            v += __shfl_xor_sync(0xffffffffu, v, 2);
            v += __shfl_xor_sync(0xffffffffu, v, 4);
            if (c == 0) {
                const int row = (2 * wl + rr) + 8 * g + 32 * i;
                s_qn[row] = row_scale ? v * row_scale[row] : v;
            }
        }
}

// In-place row scaling of a [128 x NB*64] bf16 tile (NB boxes of 64 columns, `box_bytes` apart, 128-byte
// swizzle): thread = row, 16-byte chunks visited in a rotated order so that the 8 lanes of a quarter-warp
// hit 8 different banks.
template <int NB>
__device__ __forceinline__ void scale_tile_rows(unsigned char *tile, uint32_t box_bytes, int row, float w) {
    uint32_t whi, wlo;
    split_scale(w, whi, wlo);
#pragma unroll 2
    for (int q = 0; q < NB; ++q) {
        unsigned char *rowp = tile + q * box_bytes + row * 128;
        uint4 v[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) v[c] = *reinterpret_cast<const uint4 *>(rowp + (((c + row) & 7) << 4));
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            v[c].x = scale_bf16x2(v[c].x, whi, wlo); v[c].y = scale_bf16x2(v[c].y, whi, wlo);
            v[c].z = scale_bf16x2(v[c].z, whi, wlo); v[c].w = scale_bf16x2(v[c].w, whi, wlo);
        }
#pragma unroll
        for (int c = 0; c < 8; ++c) *reinterpret_cast<uint4 *>(rowp + (((c + row) & 7) << 4)) = v[c];
    }
}
template <int DQK>
__device__ __forceinline__ void scale_rows(unsigned char *tile, int row, float w) {
    scale_tile_rows<Smem<DQK>::NBOX>(tile, Smem<DQK>::BOX, row, w);
}

// One 128-row half of the initial state: global fp32 -> Cb (bf16, swizzled MN-major) and TMEM
// (pre-scaled by the first tile's decay).  `src` is this thread's row (NULL = zero state).
template <int DQK>
__device__ __forceinline__ void c_init_half(unsigned char *smem, uint32_t t_half, const float *src, int j, float decay0) {
    using SM = Smem<DQK>;
#pragma unroll 1
    for (int c0 = 0; c0 < DVS; c0 += 32) {
        uint32_t v[32];
#pragma unroll
        for (int x = 0; x < 32; x += 4) {
            float4 f = src ? *reinterpret_cast<const float4 *>(src + c0 + x) : make_float4(0.f, 0.f, 0.f, 0.f);
            v[x] = __float_as_uint(f.x); v[x + 1] = __float_as_uint(f.y);
            v[x + 2] = __float_as_uint(f.z); v[x + 3] = __float_as_uint(f.w);
        }
#pragma unroll
        for (int x = 0; x < 32; x += 8) {
            uint4 o;
            o.x = pack_bf16(__uint_as_float(v[x]), __uint_as_float(v[x + 1]));
            o.y = pack_bf16(__uint_as_float(v[x + 2]), __uint_as_float(v[x + 3]));
            o.z = pack_bf16(__uint_as_float(v[x + 4]), __uint_as_float(v[x + 5]));
            o.w = pack_bf16(__uint_as_float(v[x + 6]), __uint_as_float(v[x + 7]));
            const int c = c0 + x;
            *reinterpret_cast<uint4 *>(smem + SM::CB + (c >> 6) * SM::CB_BLOCK + sw128_off(j, c & 63)) = o;
        }
#pragma unroll
        for (int x = 0; x < 32; ++x) v[x] = __float_as_uint(__uint_as_float(v[x]) * decay0);
        tmem_st32(t_half + c0, v);
    }
}

}  // namespace tcw

// the kernel for gates of bounded in-tile spread (mlstm_chunkwise_tc_fast.cu); CTAs of other heads return at once
int mlstm_chunkwise_tc_fast_launch(const tcw::TcParams &tp, dim3 grid, int dqk, cudaStream_t st);
// state-only scan of every segment from an empty state (mlstm_chunkwise_tc_scan.cu): C1, n1 only, no h
int mlstm_chunkwise_tc_scan_launch(const tcw::TcParams &tp, dim3 grid, int dqk, cudaStream_t st);

}  // namespace xl
