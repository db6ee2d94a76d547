"""mLSTM cells, neuron and block with the reference's call signatures, backed by the CUDA kernels.

Each class keeps the constructor arguments, attribute names (they are addressed by the
safetensors key map) and ``forward`` contract of its reference twin:

``mLSTMProjectionCell``      xlstm_metal/torch_native/blocks/mlstm/mlstm_chunkwise/mlstm_projection_cell.py:19-106
``mLSTMRecurrentKernelCell`` .../mlstm_recurrent_kernel_cell.py:19-161
``mLSTMParallelKernelCell``  xlstm_metal/mlx_jit/blocks/mlstm/mlstm_chunkwise/mlstm_parallel_kernel_cell.py:110-249
``mLSTMOutputCell``          .../mlstm_output_cell.py:22-99
``mLSTMNeuron``              .../mlstm_neuron.py:21-176 (dispatch rule: mlx_jit/.../mlstm_neuron.py:222-264)
``mLSTMBlock``               xlstm_metal/torch_native/blocks/mlstm/mlstm_block.py:69-283

The GEMMs are torch (cuBLAS) calls; the recurrence, the decode step, the gate soft-cap, the RMS
norms, the output epilogue (per-head norm x sigmoid(output gate)) and the SwiGLU gate are the
hand-written kernels.  q, k, v travel to the chunkwise kernel as strided views of the
[B,S,NH,d] projection output: no transposed copy.
"""
from __future__ import annotations

from typing import Any, Dict, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..utils import resolve_dtype
from .rms_norm import MultiHeadRMSNorm, RMSNormCell
from .soft_cap import SoftCap

State = Tuple[torch.Tensor, torch.Tensor, torch.Tensor]


class mLSTMProjectionCell(nn.Module):
    def __init__(self, input_size: int, num_heads: int, qk_dim_per_head: int, v_dim_per_head: int,
                 use_bias: bool = False, gate_soft_cap: Optional[float] = None):
        super().__init__()
        self.input_size = input_size
        self.num_heads = num_heads
        self.qk_dim_per_head = qk_dim_per_head
        self.v_dim_per_head = v_dim_per_head
        self.gate_soft_cap = gate_soft_cap
        self.soft_cap = SoftCap()
        self.q_proj = nn.Linear(input_size, num_heads * qk_dim_per_head, bias=use_bias)
        self.k_proj = nn.Linear(input_size, num_heads * qk_dim_per_head, bias=use_bias)
        self.v_proj = nn.Linear(input_size, num_heads * v_dim_per_head, bias=use_bias)
        self.igate_proj = nn.Linear(input_size, num_heads)  # gates always carry a bias
        self.fgate_proj = nn.Linear(input_size, num_heads)

    def forward(self, x: torch.Tensor):
        B, S, _ = x.shape
        NH = self.num_heads
        q = self.q_proj(x).view(B, S, NH, self.qk_dim_per_head).permute(0, 2, 1, 3)
        k = self.k_proj(x).view(B, S, NH, self.qk_dim_per_head).permute(0, 2, 1, 3)
        v = self.v_proj(x).view(B, S, NH, self.v_dim_per_head).permute(0, 2, 1, 3)
        i_preact = self.igate_proj(x)
        f_preact = self.fgate_proj(x)
        if self.gate_soft_cap is not None:
            i_preact = self.soft_cap(i_preact, self.gate_soft_cap)
            f_preact = self.soft_cap(f_preact, self.gate_soft_cap)
        return q, k, v, i_preact.permute(0, 2, 1), f_preact.permute(0, 2, 1)


class _KernelCellBase(nn.Module):
    def __init__(self, num_heads, qk_dim_per_head, v_dim_per_head, eps, compute_dtype, state_dtype):
        super().__init__()
        self.num_heads = num_heads
        self.qk_dim_per_head = qk_dim_per_head
        self.v_dim_per_head = v_dim_per_head
        self.eps = eps
        self.compute_dtype = compute_dtype
        self.state_dtype = state_dtype

    def _cast_in(self, q, k, v, i_preact, f_preact):
        cd = self.compute_dtype
        return tuple(t.to(dtype=cd) for t in (q, k, v, i_preact, f_preact))

    def _cast_state(self, st: State) -> State:
        if self.state_dtype == torch.float32:
            return st
        return tuple(s.to(self.state_dtype) for s in st)


class mLSTMRecurrentKernelCell(_KernelCellBase):
    """``cell(q,k,v,i,f,state) -> (h,(C,n,m))``.  One token: the decode-step kernel; several
    tokens: the chunkwise kernel, which is the same recurrence re-associated."""

    def __init__(self, num_heads: int, qk_dim_per_head: int, v_dim_per_head: int, eps: float = 1e-6,
                 compute_dtype: torch.dtype = torch.float32, state_dtype: torch.dtype = torch.float32):
        super().__init__(num_heads, qk_dim_per_head, v_dim_per_head, eps, compute_dtype, state_dtype)
        # True: a single-token step overwrites the caller's C instead of returning a new tensor (the
        # reference always returns new tensors; the runner switches this on for graph-captured decode)
        self.inplace_state = False

    def forward(self, q, k, v, i_preact, f_preact, state: Optional[State] = None, gate_cap: Optional[float] = None):
        """``gate_cap`` (not in the reference signature): the gates are raw projections and the kernel
        applies the soft-cap itself."""
        q, k, v, i_preact, f_preact = self._cast_in(q, k, v, i_preact, f_preact)
        if q.shape[2] == 1:
            h, st = ops.mlstm_step(q[:, :, 0], k[:, :, 0], v[:, :, 0], i_preact[:, :, 0], f_preact[:, :, 0],
                                   state, self.eps, inplace=self.inplace_state, gate_cap=gate_cap)
            return h.unsqueeze(2), self._cast_state(st)
        h, st = ops.mlstm_chunkwise(q, k, v, i_preact, f_preact, state, 64, self.eps, gate_cap=gate_cap)
        return h, self._cast_state(st)


class mLSTMParallelKernelCell(_KernelCellBase):
    """Chunkwise-parallel cell: same contract as the recurrent cell, ``chunk_size`` tokens at a time."""

    def __init__(self, num_heads: int, qk_dim_per_head: int, v_dim_per_head: int, chunk_size: int = 64,
                 eps: float = 1e-6, compute_dtype: torch.dtype = torch.float32,
                 state_dtype: torch.dtype = torch.float32):
        super().__init__(num_heads, qk_dim_per_head, v_dim_per_head, eps, compute_dtype, state_dtype)
        self.chunk_size = chunk_size

    def forward(self, q, k, v, i_preact, f_preact, state: Optional[State] = None, gate_cap: Optional[float] = None):
        q, k, v, i_preact, f_preact = self._cast_in(q, k, v, i_preact, f_preact)
        h, st = ops.mlstm_chunkwise(q, k, v, i_preact, f_preact, state, self.chunk_size, self.eps, gate_cap=gate_cap)
        return h, self._cast_state(st)


class mLSTMOutputCell(nn.Module):
    def __init__(self, input_size: int, num_heads: int, v_dim_per_head: int, use_bias: bool = False,
                 eps: float = 1e-6):
        super().__init__()
        self.input_size = input_size
        self.num_heads = num_heads
        self.v_dim_per_head = v_dim_per_head
        v_dim = num_heads * v_dim_per_head
        self.norm = MultiHeadRMSNorm(num_heads=num_heads, head_dim=v_dim_per_head, eps=eps)
        self.ogate_proj = nn.Linear(input_size, v_dim, bias=use_bias)
        self.out_proj = nn.Linear(v_dim, input_size, bias=use_bias)

    def forward(self, h: torch.Tensor, x_orig: torch.Tensor) -> torch.Tensor:
        return self.forward_gated(h, self.ogate_proj(x_orig))

    def gate(self, h: torch.Tensor, o_preact: torch.Tensor) -> torch.Tensor:
        """norm(h) * sigmoid(ogate) in one pass over h [B,NH,S,dv] -> [B,S,NH*dv]; no soft-cap on the output gate."""
        return ops.mlstm_output_gate(h, o_preact, self.norm.weight, self.norm.eps)

    def forward_gated(self, h: torch.Tensor, o_preact: torch.Tensor) -> torch.Tensor:
        """``o_preact`` = ``ogate_proj(x)`` computed by the caller (a column block of a fused GEMM)."""
        return self.out_proj(self.gate(h, o_preact))


class mLSTMNeuron(nn.Module):
    def __init__(self, input_size: int, num_heads: int, qk_dim_per_head: int, v_dim_per_head: int,
                 chunk_size: int = 64, kernel_mode: str = "parallel", use_bias: bool = False, eps: float = 1e-6,
                 gate_soft_cap: Optional[float] = None, compute_dtype: torch.dtype = torch.float32,
                 state_dtype: torch.dtype = torch.float32):
        super().__init__()
        valid_modes = {"parallel", "recurrent"}
        if kernel_mode not in valid_modes:
            raise ValueError(f"Invalid kernel_mode '{kernel_mode}'. Valid options: {sorted(valid_modes)}")
        self.input_size = input_size
        self.num_heads = num_heads
        self.qk_dim_per_head = qk_dim_per_head
        self.v_dim_per_head = v_dim_per_head
        self.chunk_size = chunk_size
        self.kernel_mode = kernel_mode
        self.eps = eps
        self.compute_dtype = compute_dtype
        self.state_dtype = state_dtype
        self.projection_cell = mLSTMProjectionCell(input_size, num_heads, qk_dim_per_head, v_dim_per_head,
                                                   use_bias=use_bias, gate_soft_cap=gate_soft_cap)
        self.parallel_kernel = mLSTMParallelKernelCell(num_heads, qk_dim_per_head, v_dim_per_head, chunk_size, eps,
                                                       compute_dtype, state_dtype)
        self.recurrent_kernel = mLSTMRecurrentKernelCell(num_heads, qk_dim_per_head, v_dim_per_head, eps,
                                                         compute_dtype, state_dtype)
        self.output_cell = mLSTMOutputCell(input_size, num_heads, v_dim_per_head, use_bias=use_bias, eps=eps)

    # ---- heads sharded over the ranks of a process group -------------------------------------------
    def shard_heads(self, rank: int, world: int, group=None) -> None:
        """Keep only this rank's heads ``[rank*NH/world, (rank+1)*NH/world)``: the row slices of the q, k, v,
        igate, fgate and ogate projections and of the per-head norm weight, and the heads' (C, n, m).  Heads
        never interact inside the cell and the norm is per head, so everything up to ``norm(h) * sigmoid(o)``
        is local; ``forward`` then all-gathers the gated ``[B, S, NH/world * dv]`` slices (one collective)
        and applies the replicated out-projection.  Call before loading weights: ``weight_row_slice`` tells
        the loader which rows of a full checkpoint tensor belong here."""
        from ..parallel import head_range
        if getattr(self, "_shard", None) is not None:
            raise RuntimeError("heads are already sharded")
        lo, hi = head_range(self.num_heads, world, rank)
        nh_total, dqk, dv = self.num_heads, self.qk_dim_per_head, self.v_dim_per_head
        pc, oc = self.projection_cell, self.output_cell

        def keep_rows(lin: nn.Linear, per_head: int) -> None:
            lin.weight = nn.Parameter(lin.weight.data[lo * per_head:hi * per_head].clone(), requires_grad=lin.weight.requires_grad)
            if lin.bias is not None:
                lin.bias = nn.Parameter(lin.bias.data[lo * per_head:hi * per_head].clone(), requires_grad=lin.bias.requires_grad)
            lin.out_features = (hi - lo) * per_head

        for lin, per in ((pc.q_proj, dqk), (pc.k_proj, dqk), (pc.v_proj, dv), (pc.igate_proj, 1), (pc.fgate_proj, 1),
                         (oc.ogate_proj, dv)):
            keep_rows(lin, per)
        if oc.norm.weight is not None:
            oc.norm.weight = nn.Parameter(oc.norm.weight.data[lo * dv:hi * dv].clone(), requires_grad=oc.norm.weight.requires_grad)
        for mod in (self, pc, oc, oc.norm, self.parallel_kernel, self.recurrent_kernel):
            mod.num_heads = hi - lo
        self._fused = None
        self._shard = (rank, world, group, nh_total, lo, hi)

    def weight_row_slice(self, path: str) -> Optional[slice]:
        """Rows of the FULL tensor that the (sharded) parameter ``path`` (relative to this neuron) holds."""
        shard = getattr(self, "_shard", None)
        if shard is None:
            return None
        lo, hi = shard[4], shard[5]
        per = {"projection_cell.q_proj": self.qk_dim_per_head, "projection_cell.k_proj": self.qk_dim_per_head,
               "projection_cell.v_proj": self.v_dim_per_head, "projection_cell.igate_proj": 1,
               "projection_cell.fgate_proj": 1, "output_cell.ogate_proj": self.v_dim_per_head,
               "output_cell.norm": self.v_dim_per_head}.get(path.rsplit(".", 1)[0])
        return None if per is None else slice(lo * per, hi * per)

    def _gather_gated(self, gated: torch.Tensor) -> torch.Tensor:
        shard = getattr(self, "_shard", None)
        if shard is None or shard[1] == 1:
            return gated
        from ..parallel import all_gather_features
        return all_gather_features(gated, shard[2])

    @property
    def state_size(self) -> Tuple[int, int, int]:
        return (self.num_heads * self.qk_dim_per_head * self.v_dim_per_head,
                self.num_heads * self.qk_dim_per_head, self.num_heads)

    @property
    def output_size(self) -> int:
        return self.input_size

    # ---- one GEMM for the six input-side projections ------------------------------------------------
    def fuse_projections(self) -> None:
        """Concatenate the q, k, v, igate, fgate and ogate weights into one ``[N, D]`` matrix, so that a
        block of tokens needs one GEMM instead of six.  The six parameters become views of that
        matrix (same storage): names, ``state_dict`` and later in-place loads are unchanged.  Moving
        the module afterwards (``.to``) detaches the views; ``forward`` notices and uses the
        separate projections until this is called again."""
        lins = self._fusable()
        W = torch.cat([l.weight.data for l in lins], dim=0)
        b = torch.cat([l.bias.data if l.bias is not None else W.new_zeros(l.out_features) for l in lins])
        off = 0
        for l in lins:
            n = l.out_features
            l.weight.data = W[off:off + n]
            if l.bias is not None:
                l.bias.data = b[off:off + n]
            off += n
        self._fused = (W, b)

    def _fusable(self):
        pc = self.projection_cell
        return [pc.q_proj, pc.k_proj, pc.v_proj, pc.igate_proj, pc.fgate_proj, self.output_cell.ogate_proj]

    def _fused_weights(self):
        fused = getattr(self, "_fused", None)
        if fused is None:
            return None
        W, b = fused
        off = 0
        for l in self._fusable():   # still views of the fused matrix?
            if l.weight.data_ptr() != W.data_ptr() + off * W.stride(0) * W.element_size() or l.weight.dtype != W.dtype:
                return None
            if l.bias is not None and l.bias.data_ptr() != b.data_ptr() + off * b.element_size():
                return None
            off += l.out_features
        return fused

    def _project(self, x: torch.Tensor):
        fused = self._fused_weights()
        if fused is None:
            q, k, v, i_preact, f_preact = self.projection_cell(x)
            return q, k, v, i_preact, f_preact, None
        B, S, _ = x.shape
        NH, dqk, dv = self.num_heads, self.qk_dim_per_head, self.v_dim_per_head
        y = F.linear(x, fused[0], fused[1])
        o_k, o_v, o_g, o_o = NH * dqk, 2 * NH * dqk, 2 * NH * dqk + NH * dv, 2 * NH * dqk + NH * dv + 2 * NH
        q = y[..., :o_k].view(B, S, NH, dqk).permute(0, 2, 1, 3)
        k = y[..., o_k:o_v].view(B, S, NH, dqk).permute(0, 2, 1, 3)
        v = y[..., o_v:o_g].view(B, S, NH, dv).permute(0, 2, 1, 3)
        # raw gate projections (strided views): the soft-cap is applied inside the kernels
        i_preact = y[..., o_g:o_g + NH].permute(0, 2, 1)
        f_preact = y[..., o_g + NH:o_o].permute(0, 2, 1)
        return q, k, v, i_preact, f_preact, y[..., o_o:]

    def forward(self, x: torch.Tensor, state: Optional[State] = None):
        q, k, v, i_preact, f_preact, o_preact = self._project(x)
        # fused projections hand over raw gates; the separate projection cell has already capped them
        cap = self.projection_cell.gate_soft_cap if o_preact is not None else None
        S = q.shape[2]
        use_parallel = self.kernel_mode == "parallel" and self.chunk_size > 0
        chunk_tokens = (S // self.chunk_size) * self.chunk_size if use_parallel else 0
        pieces, cur = [], state
        if chunk_tokens > 0:
            sl = slice(0, chunk_tokens)
            h_par, cur = self.parallel_kernel(q[:, :, sl], k[:, :, sl], v[:, :, sl], i_preact[:, :, sl],
                                              f_preact[:, :, sl], cur, gate_cap=cap)
            pieces.append(h_par)
        if S - chunk_tokens > 0:  # the S mod L tail and every decode token go through the recurrent cell
            sl = slice(chunk_tokens, S)
            h_seq, cur = self.recurrent_kernel(q[:, :, sl], k[:, :, sl], v[:, :, sl], i_preact[:, :, sl],
                                               f_preact[:, :, sl], cur, gate_cap=cap)
            pieces.append(h_seq)
        h = pieces[0] if len(pieces) == 1 else torch.cat(pieces, dim=2)
        oc = self.output_cell
        gated = oc.gate(h, oc.ogate_proj(x) if o_preact is None else o_preact)   # this rank's heads
        return oc.out_proj(self._gather_gated(gated)), cur

    def get_config(self) -> dict:
        return {"input_size": self.input_size, "num_heads": self.num_heads, "qk_dim_per_head": self.qk_dim_per_head,
                "v_dim_per_head": self.v_dim_per_head, "chunk_size": self.chunk_size, "kernel_mode": self.kernel_mode,
                "eps": self.eps}


def _round_up(value: int, multiple: int) -> int:
    return ((value + multiple - 1) // multiple) * multiple


class mLSTMBlock(nn.Module):
    """Pre-norm residual mLSTM followed by a pre-norm residual SwiGLU FFN (one xLSTM-7B block)."""

    def __init__(self, block_index: int, embedding_dim: int = 4096, num_heads: int = 8, qk_dim_factor: float = 0.5,
                 v_dim_factor: float = 1.0, gate_soft_cap: float = 15.0, ffn_proj_factor: float = 2.667,
                 ffn_round_up_to_multiple_of: int = 64, mlstm_round_up_to_multiple_of: int = 64, chunk_size: int = 64,
                 kernel_mode: str = "metal_chunkwise", norm_eps: float = 1e-6, use_bias: bool = False, eps: float = 1e-6,
                 sparsity_mask: Optional[torch.Tensor] = None, compute_dtype: torch.dtype = torch.float32,
                 state_dtype: torch.dtype = torch.float32, **_ignored) -> None:
        super().__init__()
        self.block_index = block_index
        self.embedding_dim = embedding_dim
        self.num_heads = num_heads
        self.eps = eps
        # per-head dims rounded up to the multiple, as the reference block does
        self.qk_dim_per_head = _round_up(int(embedding_dim * qk_dim_factor / num_heads), mlstm_round_up_to_multiple_of)
        self.v_dim_per_head = _round_up(int(embedding_dim * v_dim_factor / num_heads), mlstm_round_up_to_multiple_of)
        self.hidden_size = num_heads * self.v_dim_per_head
        self.ffn_hidden_dim = _round_up(int(embedding_dim * ffn_proj_factor), ffn_round_up_to_multiple_of)
        self.norm_mlstm = RMSNormCell(dims=embedding_dim, eps=norm_eps)
        # the reference torch block pins "recurrent" because it has no chunkwise kernel; here every
        # mode other than an explicit "recurrent" selects the chunkwise kernel
        mode = "recurrent" if kernel_mode == "recurrent" else "parallel"
        self.mlstm_cell = mLSTMNeuron(input_size=embedding_dim, num_heads=num_heads,
                                      qk_dim_per_head=self.qk_dim_per_head, v_dim_per_head=self.v_dim_per_head,
                                      chunk_size=chunk_size, use_bias=use_bias, eps=eps, gate_soft_cap=gate_soft_cap,
                                      kernel_mode=mode, compute_dtype=compute_dtype, state_dtype=state_dtype)
        self.norm_ffn = RMSNormCell(dims=embedding_dim, eps=norm_eps)
        self.ffn_proj_up = nn.Linear(embedding_dim, self.ffn_hidden_dim, bias=use_bias)
        self.ffn_proj_up_gate = nn.Linear(embedding_dim, self.ffn_hidden_dim, bias=use_bias)
        self.ffn_proj_down = nn.Linear(self.ffn_hidden_dim, embedding_dim, bias=use_bias)
        self.gate_soft_cap = gate_soft_cap
        self.compute_dtype = compute_dtype
        self.state_dtype = state_dtype

    def _token_step(self, x: torch.Tensor, state: Optional[State]):
        """Single-token path (at most 4 sequences, bf16, fused weights): every Linear is one
        weight-streaming kernel with its norm / bias / residual / SwiGLU folded in, so a block is five
        launches: projections, cell step with the output epilogue, out-projection, FFN up, FFN down."""
        cell = self.mlstm_cell
        W, b = cell._fused_weights()
        B = x.shape[0]
        NH, dqk, dv = cell.num_heads, cell.qk_dim_per_head, cell.v_dim_per_head
        x2 = x.reshape(B, -1)
        y = ops.linear_token(W, x2, bias=b, norm_weight=self.norm_mlstm.weight, norm_eps=self.norm_mlstm.eps)
        o_k, o_v, o_g, o_o = NH * dqk, 2 * NH * dqk, 2 * NH * dqk + NH * dv, 2 * NH * dqk + NH * dv + 2 * NH
        q, k, v = y[:, :o_k].view(B, NH, dqk), y[:, o_k:o_v].view(B, NH, dqk), y[:, o_v:o_g].view(B, NH, dv)
        rk = cell.recurrent_kernel
        oc = cell.output_cell
        if dv <= 512 and dv % 4 == 0:
            # cell step and output epilogue in one launch: the head's column-tile CTAs meet through their cluster
            gated, new_state = ops.mlstm_step_gated(
                q, k, v, y[:, o_g:o_g + NH], y[:, o_g + NH:o_o], y[:, o_o:], oc.norm.weight, state, rk.eps, oc.norm.eps,
                inplace=rk.inplace_state, gate_cap=cell.projection_cell.gate_soft_cap,
                state_settled=True)   # the launch before this one is the projection above
        else:
            h, new_state = ops.mlstm_step(q, k, v, y[:, o_g:o_g + NH], y[:, o_g + NH:o_o], state, rk.eps,
                                          inplace=rk.inplace_state, gate_cap=cell.projection_cell.gate_soft_cap,
                                          state_settled=True)
            gated = ops.mlstm_output_gate(h.unsqueeze(2), y[:, o_o:].unsqueeze(1), oc.norm.weight, oc.norm.eps)
        x1 = ops.linear_token(oc.out_proj.weight, gated.reshape(B, -1), bias=oc.out_proj.bias, residual=x2)
        act = ops.linear_token(self._fused_ffn(), x1, norm_weight=self.norm_ffn.weight, norm_eps=self.norm_ffn.eps,
                               swiglu_pair=True)
        x3 = ops.linear_token(self.ffn_proj_down.weight, act, bias=self.ffn_proj_down.bias, residual=x1)
        return x3.view_as(x), rk._cast_state(new_state)

    def shard_heads(self, rank: int, world: int, group=None) -> None:
        """Head-sharded mLSTM layer (see ``mLSTMNeuron.shard_heads``); norms and the FFN stay replicated."""
        self.mlstm_cell.shard_heads(rank, world, group)

    def weight_row_slice(self, path: str) -> Optional[slice]:
        prefix = "mlstm_cell."
        return self.mlstm_cell.weight_row_slice(path[len(prefix):]) if path.startswith(prefix) else None

    def _token_step_ok(self, x: torch.Tensor) -> bool:
        if getattr(self.mlstm_cell, "_shard", None) is not None:
            return False   # the single-token launch sequence has no gather step
        return (x.shape[1] == 1 and x.shape[0] <= ops.LINEAR_TOKEN_MAX_ROWS and x.dtype == torch.bfloat16 and
                self.mlstm_cell._fused_weights() is not None and self._fused_ffn() is not None and
                self.mlstm_cell.compute_dtype == torch.bfloat16)

    def forward(self, x: torch.Tensor, state: Optional[State] = None):
        if self._token_step_ok(x):
            return self._token_step(x, state)
        mlstm_out, new_state = self.mlstm_cell(self.norm_mlstm(x), state)
        x, xn = ops.add_rms_norm(x, mlstm_out, self.norm_ffn.weight, self.norm_ffn.eps)   # residual + pre-norm
        fused = self._fused_ffn()
        if fused is None:
            gated = ops.swiglu(self.ffn_proj_up_gate(xn), self.ffn_proj_up(xn))
        else:
            y = F.linear(xn, fused)
            gated = ops.swiglu(y[..., :self.ffn_hidden_dim], y[..., self.ffn_hidden_dim:])
        x = x + self.ffn_proj_down(gated)
        return x, new_state

    def fuse_projections(self) -> None:
        """One GEMM for the six input-side projections of the mLSTM layer and one for the two up
        projections of the FFN; the parameters become views of the fused matrices (see
        ``mLSTMNeuron.fuse_projections``)."""
        self.mlstm_cell.fuse_projections()
        if self.ffn_proj_up.bias is None and self.ffn_proj_up_gate.bias is None:
            W = torch.cat([self.ffn_proj_up_gate.weight.data, self.ffn_proj_up.weight.data], dim=0)
            self.ffn_proj_up_gate.weight.data = W[:self.ffn_hidden_dim]
            self.ffn_proj_up.weight.data = W[self.ffn_hidden_dim:]
            self._fused_ffn_w = W

    def _fused_ffn(self):
        W = getattr(self, "_fused_ffn_w", None)
        if W is None:
            return None
        row = W.stride(0) * W.element_size()
        if (self.ffn_proj_up_gate.weight.data_ptr() != W.data_ptr() or self.ffn_proj_up_gate.weight.dtype != W.dtype or
                self.ffn_proj_up.weight.data_ptr() != W.data_ptr() + self.ffn_hidden_dim * row):
            return None
        return W

    def get_weight_keys(self) -> Dict[str, str]:
        p = f"backbone.blocks.{self.block_index}"
        layer = {"q_proj.weight": "q.weight", "k_proj.weight": "k.weight", "v_proj.weight": "v.weight",
                 "igate_proj.weight": "igate_preact.weight", "igate_proj.bias": "igate_preact.bias",
                 "fgate_proj.weight": "fgate_preact.weight", "fgate_proj.bias": "fgate_preact.bias"}
        keys = {"norm_mlstm.weight": f"{p}.norm_mlstm.weight"}
        keys.update({f"mlstm_cell.projection_cell.{a}": f"{p}.mlstm_layer.{b}" for a, b in layer.items()})
        keys.update({
            "mlstm_cell.output_cell.ogate_proj.weight": f"{p}.mlstm_layer.ogate_preact.weight",
            "mlstm_cell.output_cell.norm.weight": f"{p}.mlstm_layer.multihead_norm.weight",
            "mlstm_cell.output_cell.out_proj.weight": f"{p}.mlstm_layer.out_proj.weight",
            "norm_ffn.weight": f"{p}.norm_ffn.weight",
            "ffn_proj_up.weight": f"{p}.ffn.proj_up.weight",
            "ffn_proj_up_gate.weight": f"{p}.ffn.proj_up_gate.weight",
            "ffn_proj_down.weight": f"{p}.ffn.proj_down.weight",
        })
        return keys

    @classmethod
    def from_config(cls, block_index: int, config: Dict[str, Any], sparsity_mask: Optional[torch.Tensor] = None,
                    **overrides) -> "mLSTMBlock":
        compute_dtype = overrides.get("compute_dtype", resolve_dtype(config.get("autocast_kernel_dtype", "float32")))
        state_dtype = overrides.get("state_dtype", resolve_dtype(config.get("inference_state_dtype", "float32")))
        return cls(block_index=block_index, embedding_dim=config["embedding_dim"], num_heads=config["num_heads"],
                   qk_dim_factor=config["qk_dim_factor"], v_dim_factor=config["v_dim_factor"],
                   gate_soft_cap=config["gate_soft_cap"], ffn_proj_factor=config.get("ffn_proj_factor", 2.667),
                   ffn_round_up_to_multiple_of=config.get("ffn_round_up_to_multiple_of", 64),
                   mlstm_round_up_to_multiple_of=config.get("mlstm_round_up_to_multiple_of", 64),
                   chunk_size=config.get("chunk_size", 64), kernel_mode=config.get("kernel_mode", "metal_chunkwise"),
                   norm_eps=config.get("norm_eps", 1e-6), use_bias=config.get("use_bias", False),
                   eps=config.get("eps", 1e-6), sparsity_mask=sparsity_mask, compute_dtype=compute_dtype,
                   state_dtype=state_dtype)

    def get_config(self) -> Dict[str, Any]:
        return {"block_index": self.block_index, "embedding_dim": self.embedding_dim, "num_heads": self.num_heads,
                "qk_dim_per_head": self.qk_dim_per_head, "v_dim_per_head": self.v_dim_per_head,
                "hidden_size": self.hidden_size, "ffn_hidden_dim": self.ffn_hidden_dim,
                "gate_soft_cap": self.gate_soft_cap, "eps": self.eps}


__all__ = ["mLSTMProjectionCell", "mLSTMRecurrentKernelCell", "mLSTMParallelKernelCell", "mLSTMOutputCell",
           "mLSTMNeuron", "mLSTMBlock"]
