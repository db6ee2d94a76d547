/*
 * libxlstm_cuda -- hand-written sm_100a kernels for the xLSTM inference hot
 * path, behind a plain C ABI.
 *
 * Conventions for every entry point
 *   - all tensor arguments are DEVICE pointers (tensor.data_ptr()); the library
 *     never allocates or frees memory: scratch is passed in by the caller;
 *   - `dtype` selects the element type of the activations (q, k, v, gates, h,
 *     z ...): XLSTM_F32 or XLSTM_BF16.  Recurrent state is always fp32;
 *   - `stream` is a cudaStream_t (NULL = default stream).  Calls are
 *     asynchronous on that stream and never synchronise;
 *   - the return value is 0 or a negative xlstm_status; nothing throws,
 *     aborts or traps.  xlstm_strerror() names a status.
 *
 * The reference project has no C ABI of its own: its native kernels are Metal
 * shaders reached through pybind11 modules built at first use
 * (torch.utils.cpp_extension.load, e.g.
 * xlstm_metal/torch_native/blocks/mlstm/mlstm_chunkwise/forward/mlstm_chunkwise_recurrent_fw_C.py:29-35).
 * Each function below names the reference interface it stands in for.
 */
#ifndef XLSTM_CUDA_H
#define XLSTM_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum { XLSTM_F32 = 0, XLSTM_BF16 = 1 } xlstm_dtype;

typedef enum {
    XLSTM_OK = 0,
    XLSTM_ERR_INVALID = -1,      /* null pointer, bad size, aliasing that is not allowed */
    XLSTM_ERR_UNSUPPORTED = -2,  /* shape or dtype outside what the kernels cover */
    XLSTM_ERR_CUDA = -3,         /* a CUDA runtime call or launch failed */
    XLSTM_ERR_WORKSPACE = -4,    /* caller-provided scratch is too small or misaligned */
    XLSTM_ERR_TIMEOUT = -5,      /* a bounded device-side wait gave up (status word set) */
    XLSTM_ERR_STATIC_SCRATCH = -6 /* problem needs more scratch than the library's built-in block holds */
} xlstm_status;

int xlstm_version(void);
const char *xlstm_strerror(int status);

/*
 * y = cap * tanh(x / cap), elementwise over n elements; cap <= 0 copies x to y.
 * y may alias x.
 * Replaces soft_cap_forward(x, cap) -> Tensor
 * (xlstm_metal/torch_native/blocks/soft_cap/soft_cap_extension.mm:60-99,
 *  kernel soft_cap_kernel.metal:4-15; Python entry softcap.py:14-36).
 */
int xlstm_softcap(const void *x, void *y, int64_t n, float cap, int dtype, void *stream);

/*
 * One mLSTM decode step for every (batch, head):
 *   m' = max(logsigmoid(f) + m, i);  C' = e^{logsig(f)+m-m'} C + e^{i-m'} k (x) v;  n' likewise;
 *   h  = (q~ . C') / (max(|q~ . n'|, e^{-m'}) + eps),  q~ = q * dqk^-1/2.
 * q,k: [B*NH, dqk]  v,h: [B*NH, dv]  ig,fg: [B*NH]  (dense, `dtype`)
 * C0,C1: [B*NH, dqk, dv]  n0,n1: [B*NH, dqk]  m0,m1: [B*NH]  (fp32).
 * C0 == NULL means the zero state (n0, m0 ignored).  C1 may alias C0 (in-place
 * update); n1/m1 must not alias n0/m0.
 * Replaces mLSTMRecurrentKernelCell.forward at S == 1
 * (xlstm_metal/torch_native/blocks/mlstm/mlstm_chunkwise/mlstm_recurrent_kernel_cell.py:53-161)
 * and the draft Metal step kernel
 * (kernel_development/xlstm/pytorch_mm/mlstm_kernels.metal:37-107).
 */
int xlstm_mlstm_step(const void *q, const void *k, const void *v, const void *ig, const void *fg,
                     const float *C0, const float *n0, const float *m0,
                     void *h, float *C1, float *n1, float *m1,
                     int B, int NH, int dqk, int dv, float eps, int dtype, void *stream);

/*
 * Chunkwise mLSTM forward over S tokens (any S >= 1; the last chunk may be
 * partial), equal in exact arithmetic to S decode steps.
 * q,k: [B,NH,S,dqk]  v,h: [B,NH,S,dv]  ig,fg: [B,NH,S]  (`dtype`).
 * `strides` (host pointer, may be NULL for dense tensors) holds 15 element
 * strides: q(b,h,s) k(b,h,s) v(b,h,s) h(b,h,s) gates(b,h,s); the innermost
 * dimension is always contiguous.  This lets the caller pass the [B,S,NH,d]
 * projection output without a transposed copy.
 * State as in xlstm_mlstm_step; C1/n1/m1 must not alias C0/n0/m0.
 * `workspace` must hold xlstm_mlstm_chunkwise_workspace_bytes(...) bytes,
 * 256-byte aligned (may be NULL when that size is 0).
 * Replaces mLSTMParallelKernelCell.__call__
 * (xlstm_metal/mlx_jit/blocks/mlstm/mlstm_chunkwise/mlstm_parallel_kernel_cell.py:132-249)
 * and the two native kernels under it: mlstm_recurrent_fw_C_forward(...)
 * (xlstm_metal/torch_native/blocks/mlstm/mlstm_chunkwise/forward/mlstm_chunkwise_recurrent_fw_C_extension.mm:62-175)
 * and mlstm_chunkwise_parallel_fw_Hintra_metal
 * (xlstm_metal/mlx_jit/blocks/mlstm/mlstm_chunkwise/forward/mlstm_chunkwise_parallel_fw_Hintra.py:430-506);
 * also mLSTMRecurrentKernelCell.forward at S > 1.
 */
int xlstm_mlstm_chunkwise_fwd(const void *q, const void *k, const void *v, const void *ig, const void *fg,
                              const float *C0, const float *n0, const float *m0,
                              void *h, float *C1, float *n1, float *m1,
                              int B, int NH, int S, int dqk, int dv, int L, float eps, int dtype,
                              const int64_t *strides, void *workspace, size_t workspace_bytes, void *stream);

size_t xlstm_mlstm_chunkwise_workspace_bytes(int B, int NH, int S, int dqk, int dv, int L, int dtype);

/*
 * The bf16 tensor-core forward has two kernels and picks one per (batch, head) on the device: one for gates
 * whose running maximum rises by at most e^30 within any 128-token tile (every gate factor is then applied
 * to the V rows and to the output rows, none to the Q and K tiles), and a general one whose exponents are all
 * differences <= 0 and which therefore takes any gate pattern.  Both compute the same function.
 * on != 0 sends every head to the general kernel (process-wide; meant for tests and comparisons),
 * on == 0 restores the per-head choice.  No counterpart in the reference.
 */
int xlstm_mlstm_chunkwise_set_general_only(int on);

/*
 * Segment-parallel prefill.  One persistent CTA per (batch, head, 128 dv columns) walks the whole sequence, so
 * a call with few heads (a head-sharded rank, a single prompt) leaves most SMs idle.  The carry (decay, m, C, n)
 * of the recurrence is associative: the forward then cuts every sequence into P segments, runs all segments
 * from an empty state to get their local end states, combines those into the true state at the start of every
 * segment, and runs all segments again from there - two passes over 1/P of the sequence per CTA.  P is chosen
 * from the grid size (1 when the grid already fills the GPU); xlstm_mlstm_chunkwise_workspace_bytes() includes
 * the segment states, and a forward whose scratch only holds the single-pass amount runs the single pass.
 * segments >= 1 forces P (process-wide; tests and comparisons), < 1 restores the automatic choice.
 * No counterpart in the reference (its chunk loop is sequential: .../mlstm_chunkwise_recurrent_fw_C_kernel.metal:156-299).
 */
int xlstm_mlstm_chunkwise_set_segments(int segments);

/*
 * xlstm_mlstm_chunkwise_fwd fused with the all-gather of h for head-sharded execution: the
 * epilogue stores every h tile to `h` AND, with the same strides and offsets, to `n_peers` (<= 7)
 * further base pointers - the same head slot of the peer GPUs' [B,S,NH_total,dv] buffers, mapped
 * into this process (symmetric memory / IPC).  Each staged h tile goes to every destination by a TMA tile store
 * (cp.async.bulk.tensor shared -> global over NVLink; no multicast and no load from peer memory)
 * and overlaps the tensor-core work tile by tile; after the kernels of all ranks have finished (one
 * cross-rank barrier) every rank holds the complete h and can run the out-projection on it.
 * `h_peers` is a HOST array of device pointers.  bf16, tensor-core shapes, S a multiple of 128.
 * The reference has no multi-device path (its docs say "Single-device only", docs/COMPONENTS.md:4334-4339); this stands in for the
 * all-gather that precedes mLSTMOutputCell.out_proj
 * (xlstm_metal/torch_native/blocks/mlstm/mlstm_chunkwise/mlstm_output_cell.py:84-99) when heads are sharded.
 */
int xlstm_mlstm_chunkwise_fwd_gather(const void *q, const void *k, const void *v, const void *ig, const void *fg,
                                     const float *C0, const float *n0, const float *m0,
                                     void *h, float *C1, float *n1, float *m1,
                                     int B, int NH, int S, int dqk, int dv, int L, float eps, int dtype,
                                     const int64_t *strides, void *workspace, size_t workspace_bytes,
                                     void *const *h_peers, int n_peers, void *stream);

/*
 * The token-sharded counterpart of xlstm_mlstm_chunkwise_fwd_gather.  With the gather every rank ends up with
 * ALL tokens of all heads and repeats the whole out-projection; here a tile of h goes ONLY to the rank that
 * owns its tokens: `h_ranks[r]` (r = 0 .. world-1, this rank's own buffer at its own index; a HOST array of
 * device pointers) is the slot of THIS rank's heads inside rank r's [B, tokens_per_rank, NH_total, dv] buffer,
 * tokens [r * tokens_per_rank, (r+1) * tokens_per_rank) of the sequence.  After one cross-rank barrier every
 * rank holds all heads for S / world tokens and runs 1 / world of the out-projection; each rank sends
 * (world-1) / world of its h over NVLink instead of world-1 copies of it.  The element strides of h in
 * `strides` describe those buffers; tokens_per_rank is a multiple of 128 and world * tokens_per_rank == S.
 * No local copy of h is written.  TMA tile stores, no multicast, no load from peer memory.
 * Same role in the reference as xlstm_mlstm_chunkwise_fwd_gather (none: single-device).
 */
int xlstm_mlstm_chunkwise_fwd_scatter(const void *q, const void *k, const void *v, const void *ig, const void *fg,
                                      const float *C0, const float *n0, const float *m0,
                                      float *C1, float *n1, float *m1,
                                      int B, int NH, int S, int dqk, int dv, int L, float eps, int dtype,
                                      const int64_t *strides, void *workspace, size_t workspace_bytes,
                                      void *const *h_ranks, int world, int tokens_per_rank, void *stream);

/*
 * xlstm_mlstm_chunkwise_fwd for callers that cannot supply scratch memory (no counterpart in
 * the reference: its launchers allocate their outputs through the framework).  Same arguments
 * and results as xlstm_mlstm_chunkwise_fwd without `workspace`; the scratch is an 8 MiB block
 * built into the library image (present on every GPU that loads the library, until exit).
 * It covers B*NH*(S/128) <= ~2700 tiles, e.g. one 32k-token prompt at NH = 8; larger problems
 * return XLSTM_ERR_STATIC_SCRATCH.  Calls cudaMalloc / cudaFree never.  The first call on a
 * device resolves the block's address and should precede any stream capture.  All calls on a
 * device share the block: do not let two of them overlap on the GPU.
 */
int xlstm_mlstm_chunkwise_fwd_static(const void *q, const void *k, const void *v, const void *ig, const void *fg,
                                     const float *C0, const float *n0, const float *m0,
                                     void *h, float *C1, float *n1, float *m1,
                                     int B, int NH, int S, int dqk, int dv, int L, float eps, int dtype,
                                     const int64_t *strides, void *stream);

/*
 * Outcome of the device-side waits of the last chunkwise forward that used `workspace` (NULL = the built-in
 * block of xlstm_mlstm_chunkwise_fwd_static): the tensor-core kernels bound every wait on a barrier; a wait
 * that gives up sets a status word in the scratch, releases the other roles of its CTA and the kernel ends
 * normally with incomplete results.  This call copies that word back (it SYNCHRONISES `stream`) and returns
 * XLSTM_OK or XLSTM_ERR_TIMEOUT.  The forward calls themselves never synchronise, so a caller that wants the
 * check makes this call where it synchronises anyway.  No counterpart in the reference (its launchers block
 * on waitUntilCompleted and have no device-side waits).
 */
int xlstm_mlstm_chunkwise_status(const void *workspace, void *stream);

/*
 * Packaged sLSTM cell (scalar gates per head, state c,n,m) applied to S
 * timesteps in one launch:
 *   m' = max(m + logsigmoid(f), i); c' = e^{m+logsig(f)-m'} c + e^{i-m'} tanh(z);
 *   n' = ... + e^{i-m'};  h = sigmoid(o) c' / (|n'| + eps).
 * z,h: [B,S,NH,H]  ig,fg,og: [B,S,NH]  (`dtype`);  c,n: [B,NH,H]  m: [B,NH] (fp32).
 * c0 == NULL means the zero state.  c1/n1 may alias c0/n0; m1 must not alias m0.
 * Replaces sLSTMStepwiseKernelCell.forward
 * (xlstm_metal/torch_native/blocks/slstm/slstm_layers/stepwise/slstm_stepwise_kernel_cell.py:47-97)
 * and the per-timestep Python loop around it (slstm_neuron.py:132-143); Metal
 * twin xlstm_metal/mlx_jit/blocks/slstm/slstm_layers/stepwise/slstm_metal_kernel.py:60-123.
 */
int xlstm_slstm_scan(const void *z, const void *ig, const void *fg, const void *og,
                     const float *c0, const float *n0, const float *m0,
                     void *h, float *c1, float *n1, float *m1,
                     int B, int S, int NH, int H, float eps, int dtype, void *stream);

/*
 * sLSTM with block-diagonal recurrent weights (state c,n,h,m per unit), S
 * timesteps in one launch, recurrent weights resident on chip:
 *   pre_g = gx_g + R_g h_{t-1} + rb_g   (g = i,f,z,o; i and f soft-capped with `cap` when cap > 0)
 *   m' = max(f + m, i); c' = e^{f-m'+m} c + e^{i-m'} tanh(z); n' = e^{f-m'+m} n + e^{i-m'};
 *   h = sigmoid(o) c' / max(n', 1).
 * gx: [B,S,4,D] (`dtype`, gate order i,f,z,o, D = NH*dh)   R: [4,NH,dh,dh] (`dtype`, [out][in])
 * rb: [4,D] fp32   hs: [B,S,D] (`dtype`)   state c,n,h,m: [B,D] fp32.
 * c0 == NULL means the initial state c=h=m=0, n=1.  Final state must not alias the initial one.
 * Replaces sLSTMBlock.forward_step's recurrence
 * (kernel_development/xlstm/implementations/pytorch/xlstm_pytorch_enhanced.py:428-461,
 *  BlockLinear :207-229, init_hidden :407-413) and the loop over t (:463-488).
 */
int xlstm_slstm_recurrent(const void *gx, const void *R, const float *rb,
                          const float *c0, const float *n0, const float *h0, const float *m0,
                          void *hs, float *c1, float *n1, float *h1, float *m1,
                          int B, int S, int NH, int dh, float cap, int dtype, void *stream);

/*
 * The same for the tensor-core path of xlstm_slstm_recurrent (its CTAs wait, bounded, for their cluster
 * peers' slices of h_t): XLSTM_ERR_TIMEOUT if any launch on this device since the last query gave up a wait
 * (its final state m is then NaN as well); the word is cleared by the query.  Synchronises `stream`.
 */
int xlstm_slstm_recurrent_status(void *stream);

/*
 * Gate soft-cap folded into the consumers: the same two functions with the raw gate projections as
 * input; i and f pass through cap * tanh(x / cap) (in fp32) as they are read when gate_cap > 0.
 * Removes the separate soft-cap pass and its round trip of mLSTMProjectionCell.forward
 * (xlstm_metal/torch_native/blocks/mlstm/mlstm_chunkwise/mlstm_projection_cell.py:97-104); logsigmoid,
 * the in-chunk cumulative sums and the [B,S,NH] -> [B,NH,S] transpose (strides) were already inside
 * (mlx_jit/.../mlstm_parallel_kernel_cell.py:211-217).
 */
int xlstm_mlstm_step_gatecap(const void *q, const void *k, const void *v, const void *ig, const void *fg,
                             const float *C0, const float *n0, const float *m0,
                             void *h, float *C1, float *n1, float *m1,
                             int B, int NH, int dqk, int dv, float eps, float gate_cap, int dtype, void *stream);
/*
 * The decode step with launch flags.  All single-token kernels of this library (xlstm_mlstm_step*,
 * xlstm_linear_token, xlstm_mlstm_output_gate) are launched with programmatic stream serialisation: their
 * CTAs may become resident while the kernel before them in the stream is still draining, and they wait for
 * that kernel before they touch anything it could have written.  What a kernel may read BEFORE that wait is
 * what the preceding kernel cannot have written: the weight matrix in xlstm_linear_token, and here, with
 *   XLSTM_STEP_STATE_SETTLED   the caller promises that C0 was not written by the kernel launched
 *                              immediately before this call on the stream (true in a layer stack, where a
 *                              layer's step follows that layer's projection; NOT true when the same state
 *                              is stepped twice in a row with nothing in between),
 * the first rows of the state, so that the HBM stream does not stop at the kernel boundary.  Without the flag
 * (and through xlstm_mlstm_step / xlstm_mlstm_step_gatecap) nothing is read early.  gate_cap <= 0: no cap.
 * No counterpart in the reference (its recurrent cell is a sequence of torch ops).
 */
#define XLSTM_STEP_STATE_SETTLED 1
int xlstm_mlstm_step_ex(const void *q, const void *k, const void *v, const void *ig, const void *fg,
                        const float *C0, const float *n0, const float *m0,
                        void *h, float *C1, float *n1, float *m1,
                        int B, int NH, int dqk, int dv, float eps, float gate_cap, int flags, int dtype,
                        void *stream);
/*
 * Decode step WITH the layer's output epilogue applied before the result leaves the chip (single token):
 *   y[b, head*dv + j] = h_j / sqrt(mean_j(h^2) + norm_eps) * norm_w[head*dv + j] * sigmoid(ogate[b, head*dv + j])
 * where h is what xlstm_mlstm_step_ex would have written (rounded to the activation type first, as the separate
 * epilogue reads it back).  The CTAs that hold the dv / 64 column tiles of one head run as one thread-block
 * cluster and exchange their partial sums of squares through distributed shared memory, so h itself is never
 * stored.  ogate: rows of pitch ogate_ld elements (a column block of the fused projection output), norm_w:
 * [NH*dv] or NULL, y: [B, NH*dv] dense.  dv <= 512 (eight tiles: the portable cluster size), else
 * XLSTM_ERR_UNSUPPORTED.  flags, gate_cap as in xlstm_mlstm_step_ex.
 * Replaces mLSTMRecurrentKernelCell.forward at S = 1 followed by mLSTMOutputCell.forward's per-head norm,
 * sigmoid and product (mlstm_recurrent_kernel_cell.py:106-153, mlstm_output_cell.py:84-94,
 * multihead_norm.py:43-64).
 */
int xlstm_mlstm_step_gated(const void *q, const void *k, const void *v, const void *ig, const void *fg,
                           const float *C0, const float *n0, const float *m0,
                           const void *ogate, int64_t ogate_ld, const void *norm_w, float norm_eps,
                           void *y, float *C1, float *n1, float *m1,
                           int B, int NH, int dqk, int dv, float eps, float gate_cap, int flags, int dtype,
                           void *stream);
int xlstm_mlstm_chunkwise_fwd_gatecap(const void *q, const void *k, const void *v, const void *ig, const void *fg,
                                      const float *C0, const float *n0, const float *m0,
                                      void *h, float *C1, float *n1, float *m1,
                                      int B, int NH, int S, int dqk, int dv, int L, float eps, float gate_cap, int dtype,
                                      const int64_t *strides, void *workspace, size_t workspace_bytes, void *stream);

/*
 * ---- the callers either side of the cells: norm, output epilogue, FFN gate, causal convolution ----
 * One pass over HBM each, 16-byte accesses, fp32 math, one rounding to `dtype` on the way out.
 */

/*
 * RMSNorm over the last dimension of x [rows, cols]:
 *   y = x * rsqrt(mean(x^2) + eps) * w      (w: [cols] in `dtype`, or NULL for no weight).
 * y may alias x.
 * Replaces rms_norm_forward(x2d, weight, eps) -> Tensor
 * (xlstm_metal/torch_native/blocks/rms_norm/rms_norm_extension.mm:61-105, kernel
 *  rms_norm_kernel.metal:11-31; Python entry rmsnorm.py:30-40).
 */
int xlstm_rms_norm(const void *x, const void *w, void *y, int64_t rows, int cols, float eps, int dtype, void *stream);

/*
 * Residual add fused into the norm that follows it: sum = x + r (rounded to `dtype`, the new residual
 * stream), y = RMSNorm(sum) * w.  sum may alias x or r.  Replaces the pair
 * `x = x + mlstm_out; x_normed = self.norm_ffn(x)` of mLSTMBlock.forward
 * (xlstm_metal/torch_native/blocks/mlstm/mlstm_block.py:192-198) and of sLSTMBlock.forward
 * (.../slstm/slstm_block.py:101-131).
 */
int xlstm_add_rms_norm(const void *x, const void *r, const void *w, void *sum, void *y, int64_t rows, int cols,
                       float eps, int dtype, void *stream);

/*
 * mLSTM output epilogue in one pass:
 *   y[b,s,head*dv+j] = h[b,head,s,j] / sqrt(mean_j(h^2) + eps) * w[head*dv+j] * sigmoid(ogate[b,s,head*dv+j]).
 * h: [B,NH,S,dv] with element strides h_strides = (batch, head, token), innermost contiguous (NULL = dense);
 * ogate: [B*S rows, NH*dv] with leading dimension ogate_ld elements (0 = dense), so it may be a column block
 * of a fused projection output; y: [B,S,NH*dv] dense; w: [NH*dv] or NULL.  dv, the strides and ogate_ld
 * must be multiples of 16 bytes.
 * Replaces the per-head norm, sigmoid and product of mLSTMOutputCell.forward
 * (xlstm_metal/torch_native/blocks/mlstm/mlstm_chunkwise/mlstm_output_cell.py:84-94) with
 * MultiHeadRMSNorm.forward (.../multihead_norm/multihead_norm.py:43-64).
 */
int xlstm_mlstm_output_gate(const void *h, const void *ogate, const void *w, void *y, int B, int NH, int S, int dv,
                            const int64_t *h_strides, int64_t ogate_ld, float eps, int dtype, void *stream);

/*
 * SwiGLU gate: y[r,c] = silu(g[r,c]) * u[r,c] for r < rows, c < cols.  g and u have leading dimensions
 * ldg, ldu (elements), so they may be the two column blocks of one fused GEMM output; y is dense.
 * Replaces F.silu(gate) * up in mLSTMBlock.forward
 * (xlstm_metal/torch_native/blocks/mlstm/mlstm_block.py:198-204).
 */
int xlstm_swiglu(const void *g, const void *u, void *y, int64_t rows, int cols, int64_t ldg, int64_t ldu, int dtype,
                 void *stream);

/*
 * Linear layer for up to 4 token rows (single-token decode), bf16, as ONE weight-streaming pass with the
 * neighbouring ops folded in:
 *   xh[m] = norm_w ? RMSNorm(x[m]; norm_eps) * norm_w : x[m]          (norm_w: [K] or NULL)
 *   epilogue 0:  y[m,n] = W[n,:] . xh[m] + bias[n]
 *   epilogue 1:  y[m,n] = residual[m,n] + (W[n,:] . xh[m] + bias[n])   (the block's residual stream)
 *   epilogue 2:  y[m,n] = silu(W[n,:] . xh[m] + bias[n]) * (W[N+n,:] . xh[m] + bias[N+n])   (W: [2N,K], gate rows first)
 * W: [N,K] (or [2N,K]) row-major, the layout of nn.Linear.weight; x: [M,K]; y: [M,N]; bias: [N] / [2N] or NULL.
 * Intermediate results are rounded to bf16 where the separate kernels would round them.
 * Replaces, for one token, the nn.Linear calls of mLSTMProjectionCell.forward / mLSTMOutputCell.forward
 * (xlstm_metal/torch_native/blocks/mlstm/mlstm_chunkwise/mlstm_projection_cell.py:85-106,
 * mlstm_output_cell.py:84-99) and of the FFN (mlstm_block.py:192-206) together with the RMSNorm before
 * them (rmsnorm.py:30-40), the residual adds and the SwiGLU gate around them.
 */
int xlstm_linear_token(const void *W, const void *x, const void *bias, const void *norm_w, float norm_eps,
                       const void *residual, void *y, int M, int N, int K, int epilogue, int dtype, void *stream);

/*
 * Causal depthwise convolution over tokens, channels last, optional SiLU:
 *   y[b,s,c] = act(bias[c] + sum_{j<K} w[c,j] * x[b, s-(K-1)+j, c]),   K <= 8.
 * x, y: [B,S,C]; w: [C,K] (the [C,1,K] weight of a depthwise nn.Conv1d); bias: [C] or NULL.
 * Tokens before the first one are taken from state_in [B,K-1,C] (oldest first; NULL = zeros, which is
 * what the reference does on every call); state_out (or NULL) receives the last K-1 inputs and may
 * alias state_in when S <= 16 (single-token decode).
 * Replaces causal_conv1d_depthwise(x_seq, weight, bias) -> Tensor
 * (xlstm_metal/torch_native/blocks/slstm/slstm_layers/causal_conv1d/causal_conv_extension.mm:114-164,
 *  depthwise_kernel.metal:12-44) in the tap order of the nn.Conv1d path (causal_conv1d.py:61-67), and
 * the SiLU that follows it (slstm_projection_cell.py:110-117).
 */
int xlstm_causal_conv1d(const void *x, const void *w, const void *bias, const void *state_in, void *state_out,
                        void *y, int B, int S, int C, int K, int act_silu, int dtype, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* XLSTM_CUDA_H */
