// Shared between the chunkwise mLSTM translation units.
#pragma once
#include "common.cuh"

namespace xl {

struct ChunkwiseParams {
    const void *q, *k, *v, *ig, *fg;
    const float *C0, *n0, *m0;
    void *h;
    float *C1, *n1, *m1;
    int B, NH, S, dqk, dv, L;
    float eps, qscale;
    float gate_cap;   // > 0: i and f are soft-capped (cap * tanh(x / cap)) as they are read
    // element strides (batch, head, token); innermost dimension contiguous
    int64_t sq[3], sk[3], sv[3], sh[3], sg[3];
    // optional extra destinations of h (same strides and offsets as `h`): buffers of peer GPUs
    void *h_peer[8];
    int n_peer;
    // > 0: token-sharded destinations instead of replicas - h_peer[r] (r = 0 .. n_peer-1, this rank included, `h` unused)
    // is rank r's [B, tok_per_rank, NH_total, dv] buffer and a tile of tokens goes ONLY to the rank that owns them
    int tok_per_rank;
};

// exact-fp32 CUDA-core path: any dqk <= 512, dv, S, L <= 64
int mlstm_chunkwise_simt(const ChunkwiseParams &p, int dtype, cudaStream_t st);

// tcgen05 / TMEM / TMA path: bf16, L == 64, dqk == 256 (or 128/64), dv % 128 == 0, whole chunks
// shape_ok: the shape, strides and alignment fit the tensor-core kernel; driver_ok: the driver entry point
// that encodes TMA descriptors could be resolved; supported = both
bool mlstm_chunkwise_tc_shape_ok(const ChunkwiseParams &p, int dtype);
bool mlstm_chunkwise_tc_driver_ok();
bool mlstm_chunkwise_tc_supported(const ChunkwiseParams &p, int dtype);
size_t mlstm_chunkwise_tc_workspace(int B, int NH, int S, int dqk, int dv, int L);
// scratch of the single-pass mode (no segment states): what the forward needs at least
size_t mlstm_chunkwise_tc_workspace_min(int B, int NH, int S, int dqk, int dv);
int mlstm_chunkwise_tc(const ChunkwiseParams &p, void *workspace, size_t workspace_bytes, cudaStream_t st);
// 1: every head takes the general tensor-core kernel whatever its gates are; 0: per-head choice (default)
void mlstm_chunkwise_tc_set_general_only(int on);
// segments >= 1: cut every sequence into that many segments (segment-parallel two-pass mode); < 1: planned from
// the grid size (default)
void mlstm_chunkwise_tc_set_segments(int segments);

int mlstm_chunkwise_static_scratch(void **out);

}  // namespace xl
