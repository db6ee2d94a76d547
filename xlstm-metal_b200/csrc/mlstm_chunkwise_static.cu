// Chunkwise mLSTM forward for callers that cannot hand the library any scratch memory.
//
// Some hosts of this library have no way to obtain device memory at the moment they need
// the prefill: an inference server that has already carved all of HBM into its own
// fixed pools (weights, state cache, activations) and forbids further cudaMalloc calls,
// a plugin that only receives input and output pointers from its runtime, or a process
// that runs under a memory budget enforced by an allocator it does not control.  The
// regular entry point asks such a caller for a scratch buffer it does not have.  This
// variant brings its own: a fixed, modest block that is part of the library image.
//
// The block is a file-scope __device__ array, so every GPU that loads the library
// carries XLSTM_STATIC_SCRATCH_BYTES of it until the process exits.  Its device address
// is looked up once per device (cudaGetSymbolAddress with that device current) the first
// time the entry point runs there; that first call should therefore come before any
// stream capture.  All calls on a device share the block and it keeps whatever the last
// call left in it: the status word is cleared at the start of every call, everything
// else is overwritten before it is read.  Two calls that overlap on the GPU (different
// streams) would race on the block; serialise them.
#include <mutex>

#include "mlstm_chunkwise.cuh"

#define XLSTM_STATIC_SCRATCH_BYTES (8u << 20)

static __device__ __align__(256) unsigned char g_static_scratch[XLSTM_STATIC_SCRATCH_BYTES];

namespace {

constexpr int kMaxDevices = 64;
std::mutex g_mu;
void *g_scratch_ptr[kMaxDevices] = {};

// Device address of g_static_scratch on the current device (host code must not use the
// symbol itself as a pointer: on the host it is only a stand-in for the device array).
int scratch_for_current_device(void **out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return XLSTM_ERR_CUDA;
    std::lock_guard<std::mutex> lock(g_mu);
    if (!g_scratch_ptr[dev]) {
        void *p = nullptr;
        if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || !p) return XLSTM_ERR_CUDA;
        g_scratch_ptr[dev] = p;
    }
    *out = g_scratch_ptr[dev];
    return XLSTM_OK;
}

}  // namespace

namespace xl {
// device address of the built-in scratch block on the current device (for the status query)
int mlstm_chunkwise_static_scratch(void **out) { return scratch_for_current_device(out); }
}  // namespace xl

extern "C" int xlstm_mlstm_chunkwise_fwd_static(const void *q, const void *k, const void *v, const void *ig,
                                                const void *fg, const float *C0, const float *n0, const float *m0,
                                                void *h, float *C1, float *n1, float *m1, int B, int NH, int S,
                                                int dqk, int dv, int L, float eps, int dtype, const int64_t *strides,
                                                void *stream) {
    if (!q || !k || !v || !ig || !fg || !h || !C1 || !n1 || !m1) return XLSTM_ERR_INVALID;
    if (B <= 0 || NH <= 0 || S <= 0 || dqk <= 0 || dv <= 0 || L <= 0) return XLSTM_ERR_INVALID;
    if (C0 && (!n0 || !m0)) return XLSTM_ERR_INVALID;
    if (C0 && (C1 == C0 || n1 == n0 || m1 == m0)) return XLSTM_ERR_INVALID;
    if (dtype != XLSTM_F32 && dtype != XLSTM_BF16) return XLSTM_ERR_UNSUPPORTED;
    if ((int64_t)B * NH > 2147483647LL) return XLSTM_ERR_UNSUPPORTED;
    cudaStream_t st = static_cast<cudaStream_t>(stream);

    xl::ChunkwiseParams p{};
    p.q = q; p.k = k; p.v = v; p.ig = ig; p.fg = fg;
    p.C0 = C0; p.n0 = n0; p.m0 = m0;
    p.h = h; p.C1 = C1; p.n1 = n1; p.m1 = m1;
    p.B = B; p.NH = NH; p.S = S; p.dqk = dqk; p.dv = dv; p.L = L;
    p.eps = eps; p.qscale = 1.0f / sqrtf((float)dqk);
    if (strides) {
        for (int d = 0; d < 3; ++d) {
            p.sq[d] = strides[d]; p.sk[d] = strides[3 + d]; p.sv[d] = strides[6 + d];
            p.sh[d] = strides[9 + d]; p.sg[d] = strides[12 + d];
        }
    } else {
        const int64_t s = S, nh = NH;
        p.sq[0] = nh * s * dqk; p.sq[1] = s * dqk; p.sq[2] = dqk;
        p.sk[0] = p.sq[0]; p.sk[1] = p.sq[1]; p.sk[2] = p.sq[2];
        p.sv[0] = nh * s * dv; p.sv[1] = s * dv; p.sv[2] = dv;
        p.sh[0] = p.sv[0]; p.sh[1] = p.sv[1]; p.sh[2] = p.sv[2];
        p.sg[0] = nh * s; p.sg[1] = s; p.sg[2] = 1;
    }
    // the exact CUDA-core path needs no scratch at all
    if (!xl::mlstm_chunkwise_tc_shape_ok(p, dtype)) return xl::mlstm_chunkwise_simt(p, dtype, st);

    // size check before anything else can launch: a problem beyond the block is an error, never a fallback
    const size_t need = xl::mlstm_chunkwise_tc_workspace_min(B, NH, S, dqk, dv);   // the block is used by the single-pass mode
    if (need > XLSTM_STATIC_SCRATCH_BYTES) return XLSTM_ERR_STATIC_SCRATCH;
    if (!xl::mlstm_chunkwise_tc_driver_ok()) return XLSTM_ERR_CUDA;
    void *scratch = nullptr;
    const int rc = scratch_for_current_device(&scratch);
    if (rc != XLSTM_OK) return rc;
    return xl::mlstm_chunkwise_tc(p, scratch, XLSTM_STATIC_SCRATCH_BYTES, st);
}
