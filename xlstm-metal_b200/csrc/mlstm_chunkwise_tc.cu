// tcgen05 / TMEM / TMA chunkwise mLSTM forward (bf16).  Placeholder until the
// tensor-core kernel lands: reports "not supported" so every call takes the
// exact CUDA-core path.
#include "mlstm_chunkwise.cuh"

namespace xl {
bool mlstm_chunkwise_tc_supported(const ChunkwiseParams &, int) { return false; }
size_t mlstm_chunkwise_tc_workspace(int, int, int, int, int, int) { return 0; }
int mlstm_chunkwise_tc(const ChunkwiseParams &, void *, size_t, cudaStream_t) { return XLSTM_ERR_UNSUPPORTED; }
}  // namespace xl
