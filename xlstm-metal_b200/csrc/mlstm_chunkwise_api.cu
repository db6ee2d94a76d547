// C entry point of the chunkwise mLSTM forward: argument checks and dispatch
// between the tensor-core path (bf16, production shapes) and the exact
// CUDA-core path (everything else, and the partial last chunk).
#include "mlstm_chunkwise.cuh"

namespace {

void dense_strides(xl::ChunkwiseParams &p) {
    const int64_t S = p.S, NH = p.NH;
    p.sq[0] = NH * S * p.dqk; p.sq[1] = S * p.dqk; p.sq[2] = p.dqk;
    p.sk[0] = p.sq[0]; p.sk[1] = p.sq[1]; p.sk[2] = p.sq[2];
    p.sv[0] = NH * S * p.dv; p.sv[1] = S * p.dv; p.sv[2] = p.dv;
    p.sh[0] = p.sv[0]; p.sh[1] = p.sv[1]; p.sh[2] = p.sv[2];
    p.sg[0] = NH * S; p.sg[1] = S; p.sg[2] = 1;
}

}  // namespace

extern "C" int xlstm_mlstm_chunkwise_set_general_only(int on) {
    xl::mlstm_chunkwise_tc_set_general_only(on);
    return XLSTM_OK;
}

extern "C" int xlstm_mlstm_chunkwise_set_segments(int segments) {
    xl::mlstm_chunkwise_tc_set_segments(segments);
    return XLSTM_OK;
}

extern "C" int xlstm_mlstm_chunkwise_status(const void *workspace, void *stream) {
    const void *ws = workspace;
    if (!ws) {
        void *blk = nullptr;
        const int rc = xl::mlstm_chunkwise_static_scratch(&blk);
        if (rc != XLSTM_OK) return rc;
        ws = blk;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int word = 0;   // the status word is the first int of the scratch
    if (cudaMemcpyAsync(&word, ws, sizeof(int), cudaMemcpyDeviceToHost, st) != cudaSuccess ||
        cudaStreamSynchronize(st) != cudaSuccess)
        return XLSTM_ERR_CUDA;
    return word ? XLSTM_ERR_TIMEOUT : XLSTM_OK;
}

extern "C" size_t xlstm_mlstm_chunkwise_workspace_bytes(int B, int NH, int S, int dqk, int dv, int L, int dtype) {
    if (dtype != XLSTM_BF16) return 0;
    return xl::mlstm_chunkwise_tc_workspace(B, NH, S, dqk, dv, L);
}

static int chunkwise_dispatch(const void *q, const void *k, const void *v, const void *ig, const void *fg,
                              const float *C0, const float *n0, const float *m0, void *h, float *C1,
                              float *n1, float *m1, int B, int NH, int S, int dqk, int dv, int L,
                              float eps, int dtype, const int64_t *strides, void *workspace,
                              size_t workspace_bytes, void *stream, void *const *h_peers, int n_peers,
                              float gate_cap = 0.0f, int tok_per_rank = 0) {
    if (!q || !k || !v || !ig || !fg || (!h && tok_per_rank <= 0) || !C1 || !n1 || !m1) return XLSTM_ERR_INVALID;
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
    p.gate_cap = gate_cap;
    if (strides) {
        for (int d = 0; d < 3; ++d) {
            p.sq[d] = strides[d]; p.sk[d] = strides[3 + d]; p.sv[d] = strides[6 + d];
            p.sh[d] = strides[9 + d]; p.sg[d] = strides[12 + d];
        }
    } else {
        dense_strides(p);
    }

    if (n_peers < 0 || n_peers > (tok_per_rank > 0 ? 8 : 7) || (n_peers > 0 && !h_peers)) return XLSTM_ERR_INVALID;
    if (tok_per_rank > 0 && n_peers < 1) return XLSTM_ERR_INVALID;
    p.n_peer = n_peers;
    p.tok_per_rank = tok_per_rank > 0 ? tok_per_rank : 0;
    for (int i = 0; i < n_peers; ++i) {
        if (!h_peers[i] || (reinterpret_cast<uintptr_t>(h_peers[i]) & 15u)) return XLSTM_ERR_INVALID;
        p.h_peer[i] = h_peers[i];
    }
    if (!xl::mlstm_chunkwise_tc_supported(p, dtype)) {
        if (n_peers) return XLSTM_ERR_UNSUPPORTED;   // peer stores exist in the tensor-core kernel only
        return xl::mlstm_chunkwise_simt(p, dtype, st);
    }

    // Whole 128-token tiles on the tensor cores, then the remaining tokens (with the carried
    // state) on the exact path: the split the reference neuron makes between its chunkwise and
    // recurrent cells (mlx_jit/.../mlstm_neuron.py:222-257).  The tile size is internal: the
    // chunkwise form is a re-association of the recurrence and its result does not depend on L.
    const size_t need = xl::mlstm_chunkwise_tc_workspace_min(B, NH, S, dqk, dv);
    if (!workspace || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255u))
        return XLSTM_ERR_WORKSPACE;
    return xl::mlstm_chunkwise_tc(p, workspace, workspace_bytes, st);
}

extern "C" int xlstm_mlstm_chunkwise_fwd(const void *q, const void *k, const void *v, const void *ig, const void *fg,
                                         const float *C0, const float *n0, const float *m0, void *h, float *C1,
                                         float *n1, float *m1, int B, int NH, int S, int dqk, int dv, int L,
                                         float eps, int dtype, const int64_t *strides, void *workspace,
                                         size_t workspace_bytes, void *stream) {
    return chunkwise_dispatch(q, k, v, ig, fg, C0, n0, m0, h, C1, n1, m1, B, NH, S, dqk, dv, L, eps, dtype, strides,
                              workspace, workspace_bytes, stream, nullptr, 0);
}

extern "C" int xlstm_mlstm_chunkwise_fwd_gather(const void *q, const void *k, const void *v, const void *ig,
                                                const void *fg, const float *C0, const float *n0, const float *m0,
                                                void *h, float *C1, float *n1, float *m1, int B, int NH, int S,
                                                int dqk, int dv, int L, float eps, int dtype, const int64_t *strides,
                                                void *workspace, size_t workspace_bytes, void *const *h_peers,
                                                int n_peers, void *stream) {
    return chunkwise_dispatch(q, k, v, ig, fg, C0, n0, m0, h, C1, n1, m1, B, NH, S, dqk, dv, L, eps, dtype, strides,
                              workspace, workspace_bytes, stream, h_peers, n_peers);
}

extern "C" int xlstm_mlstm_chunkwise_fwd_scatter(const void *q, const void *k, const void *v, const void *ig,
                                                 const void *fg, const float *C0, const float *n0, const float *m0,
                                                 float *C1, float *n1, float *m1, int B, int NH, int S, int dqk, int dv,
                                                 int L, float eps, int dtype, const int64_t *strides, void *workspace,
                                                 size_t workspace_bytes, void *const *h_ranks, int world,
                                                 int tokens_per_rank, void *stream) {
    if (tokens_per_rank <= 0) return XLSTM_ERR_INVALID;
    return chunkwise_dispatch(q, k, v, ig, fg, C0, n0, m0, nullptr, C1, n1, m1, B, NH, S, dqk, dv, L, eps, dtype, strides,
                              workspace, workspace_bytes, stream, h_ranks, world, 0.0f, tokens_per_rank);
}

extern "C" int xlstm_mlstm_chunkwise_fwd_gatecap(const void *q, const void *k, const void *v, const void *ig,
                                                 const void *fg, const float *C0, const float *n0, const float *m0,
                                                 void *h, float *C1, float *n1, float *m1, int B, int NH, int S,
                                                 int dqk, int dv, int L, float eps, float gate_cap, int dtype,
                                                 const int64_t *strides, void *workspace, size_t workspace_bytes,
                                                 void *stream) {
    return chunkwise_dispatch(q, k, v, ig, fg, C0, n0, m0, h, C1, n1, m1, B, NH, S, dqk, dv, L, eps, dtype, strides,
                              workspace, workspace_bytes, stream, nullptr, 0, gate_cap);
}
