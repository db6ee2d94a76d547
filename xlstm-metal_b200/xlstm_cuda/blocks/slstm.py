"""sLSTM cells, neuron and blocks with the reference's call signatures, backed by the CUDA kernels.

Two sLSTMs exist in the reference and both are served:

* the packaged one -- scalar gates per head computed from ``x`` only, state ``(c, n, m)``:
  ``sLSTMStepwiseKernelCell``  xlstm_metal/torch_native/blocks/slstm/slstm_layers/stepwise/slstm_stepwise_kernel_cell.py:18-97
  ``sLSTMProjectionCell``      .../slstm_layers/slstm_projection_cell.py:25-129
  ``sLSTMOutputCell``          .../slstm_layers/slstm_output_cell.py:20-88
  ``sLSTMNeuron``              .../slstm_layers/slstm_neuron.py:20-162
  ``sLSTMBlock``               xlstm_metal/torch_native/blocks/slstm/slstm_block.py:21-200
  The neuron's Python loop over timesteps (slstm_neuron.py:132-143) becomes one scan launch.

* the classic one with block-diagonal recurrent weights on ``h_{t-1}``, state ``(c, n, h, m)``:
  ``BlockLinear`` / ``sLSTMBlockDiag``  kernel_development/xlstm/implementations/pytorch/xlstm_pytorch_enhanced.py:207-229, 367-488
  (parameter names equal the reference class, so its ``state_dict`` loads unchanged).
"""
from __future__ import annotations

from typing import Any, Dict, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .rms_norm import RMSNormCell
from .soft_cap import soft_cap


class sLSTMStepwiseKernelCell(nn.Module):
    """``cell(z, i, f, o, state) -> (h, (c, n, m))`` for one timestep; ``scan`` for a sequence."""

    def __init__(self, num_heads: int, head_dim: int, eps: float = 1e-6):
        super().__init__()
        self.num_heads = num_heads
        self.head_dim = head_dim
        self.eps = eps

    def forward(self, z, i_preact, f_preact, o_preact, state=None):
        h, st = self.scan(z.unsqueeze(1), i_preact.unsqueeze(1), f_preact.unsqueeze(1), o_preact.unsqueeze(1), state)
        return h[:, 0], st

    def scan(self, z, i_preact, f_preact, o_preact, state=None):
        """z: [B,S,NH,H]; gates: [B,S,NH].  State dtype follows ``z`` as in the reference cell."""
        h, st = ops.slstm_scan(z, i_preact, f_preact, o_preact, state, self.eps)
        if z.dtype != torch.float32:
            st = tuple(s.to(z.dtype) for s in st)
        return h, st


class CausalConv1d(nn.Module):
    """Conv1d over [B, C, S] that only sees the past: left padding of ``kernel_size - 1``
    (xlstm_metal/torch_native/blocks/slstm/slstm_layers/causal_conv1d/causal_conv1d.py:14-67).
    No state is kept between calls, exactly as in the reference projection cell."""

    def __init__(self, in_channels: int, out_channels: int, kernel_size: int, groups: int = 1, bias: bool = True):
        super().__init__()
        self.conv = nn.Conv1d(in_channels, out_channels, kernel_size, groups=groups, bias=bias)
        self.padding = kernel_size - 1

    @property
    def depthwise(self) -> bool:
        return self.conv.groups == self.conv.in_channels == self.conv.out_channels

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.depthwise:   # [B,C,S] -> channels-last kernel -> [B,C,S]
            return ops.causal_conv1d(x.permute(0, 2, 1), self.conv.weight, self.conv.bias).permute(0, 2, 1)
        return self.conv(F.pad(x, (self.padding, 0)) if self.padding > 0 else x)

    def forward_tokens(self, x: torch.Tensor, silu: bool = False) -> torch.Tensor:
        """Depthwise path on ``[B,S,C]`` directly (no transposes), optional fused SiLU."""
        return ops.causal_conv1d(x, self.conv.weight, self.conv.bias, silu=silu)


class sLSTMProjectionCell(nn.Module):
    def __init__(self, input_size: int, num_heads: int, head_dim: int, conv1d_kernel_size: int = 4,
                 use_bias: bool = False, gate_soft_cap: float = 15.0):
        super().__init__()
        self.input_size, self.num_heads, self.head_dim = input_size, num_heads, head_dim
        self.conv1d_kernel_size = conv1d_kernel_size
        self.gate_soft_cap = gate_soft_cap
        # depthwise causal convolution (left padding k-1), then SiLU
        self.conv1d = (CausalConv1d(input_size, input_size, conv1d_kernel_size, groups=input_size)
                       if conv1d_kernel_size > 0 else None)
        self.igate_proj = nn.Linear(input_size, num_heads)
        self.fgate_proj = nn.Linear(input_size, num_heads)
        self.ogate_proj = nn.Linear(input_size, num_heads)
        self.z_proj = nn.Linear(input_size, num_heads * head_dim, bias=use_bias)

    def soft_cap(self, x: torch.Tensor) -> torch.Tensor:
        return x if self.gate_soft_cap is None else soft_cap(x, self.gate_soft_cap)

    def forward(self, x: torch.Tensor):
        B, S, _ = x.shape
        if self.conv1d is not None:
            x_conv = self.conv1d.forward_tokens(x, silu=True)   # causal depthwise conv + SiLU, one kernel
        else:
            x_conv = x
        i_preact = self.soft_cap(self.igate_proj(x_conv))
        f_preact = self.soft_cap(self.fgate_proj(x_conv))
        o_preact = self.soft_cap(self.ogate_proj(x))
        z = self.z_proj(x).view(B, S, self.num_heads, self.head_dim)
        return z, i_preact, f_preact, o_preact, x_conv


class sLSTMOutputCell(nn.Module):
    def __init__(self, input_size: int, num_heads: int, head_dim: int, use_bias: bool = False, eps: float = 1e-6):
        super().__init__()
        self.input_size, self.num_heads, self.head_dim = input_size, num_heads, head_dim
        hidden = num_heads * head_dim
        self.group_norm = nn.GroupNorm(num_groups=num_heads, num_channels=hidden, eps=eps)
        self.out_proj = nn.Linear(hidden, input_size, bias=use_bias)

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        B, S, NH, H = h.shape
        return self.out_proj(self.group_norm(h.reshape(B * S, NH * H)).view(B, S, NH * H))


class sLSTMNeuron(nn.Module):
    def __init__(self, input_size: int, num_heads: int, head_dim: int, conv1d_kernel_size: int = 4,
                 use_bias: bool = False, eps: float = 1e-6, gate_soft_cap: float = 15.0):
        super().__init__()
        self.input_size, self.num_heads, self.head_dim = input_size, num_heads, head_dim
        self.conv1d_kernel_size, self.eps, self.gate_soft_cap = conv1d_kernel_size, eps, gate_soft_cap
        self.projection_cell = sLSTMProjectionCell(input_size, num_heads, head_dim, conv1d_kernel_size, use_bias,
                                                   gate_soft_cap)
        self.kernel_cell = sLSTMStepwiseKernelCell(num_heads, head_dim, eps)
        self.output_cell = sLSTMOutputCell(input_size, num_heads, head_dim, use_bias, eps)

    @property
    def state_size(self) -> Tuple[int, int, int]:
        return (self.num_heads * self.head_dim, self.num_heads * self.head_dim, self.num_heads)

    @property
    def output_size(self) -> int:
        return self.input_size

    def forward(self, x: torch.Tensor, state=None):
        z, i_preact, f_preact, o_preact, _ = self.projection_cell(x)
        h, state = self.kernel_cell.scan(z, i_preact, f_preact, o_preact, state)  # all S steps, one launch
        return self.output_cell(h), state

    def get_config(self) -> dict:
        return {"input_size": self.input_size, "num_heads": self.num_heads, "head_dim": self.head_dim,
                "conv1d_kernel_size": self.conv1d_kernel_size, "eps": self.eps, "gate_soft_cap": self.gate_soft_cap}


class sLSTMBlock(nn.Module):
    """Pre-norm residual sLSTM followed by a pre-norm residual SwiGLU FFN."""

    def __init__(self, block_index: int, embedding_dim: int = 4096, num_heads: int = 4,
                 head_dim: Optional[int] = None, gate_soft_cap: float = 15.0, ffn_proj_factor: float = 2.667,
                 ffn_round_up_to_multiple_of: int = 64, norm_eps: float = 1e-6, use_bias: bool = False,
                 eps: float = 1e-6, **kwargs):
        super().__init__()
        self.block_index, self.embedding_dim, self.num_heads = block_index, embedding_dim, num_heads
        self.head_dim = head_dim if head_dim is not None else embedding_dim // num_heads
        self.hidden_size = num_heads * self.head_dim
        self.gate_soft_cap, self.eps = gate_soft_cap, eps
        raw = int(embedding_dim * ffn_proj_factor)
        m = ffn_round_up_to_multiple_of
        self.ffn_hidden_dim = (raw + m - 1) // m * m
        self.norm_slstm = RMSNormCell(dims=embedding_dim, eps=norm_eps)
        self.slstm_cell = sLSTMNeuron(embedding_dim, num_heads, self.head_dim,
                                      conv1d_kernel_size=kwargs.get("conv1d_kernel_size", 4), use_bias=use_bias,
                                      eps=eps, gate_soft_cap=gate_soft_cap)
        self.norm_ffn = RMSNormCell(dims=embedding_dim, eps=norm_eps)
        self.ffn_proj_up = nn.Linear(embedding_dim, self.ffn_hidden_dim, bias=False)
        self.ffn_proj_up_gate = nn.Linear(embedding_dim, self.ffn_hidden_dim, bias=False)
        self.ffn_proj_down = nn.Linear(self.ffn_hidden_dim, embedding_dim, bias=False)

    def forward(self, x: torch.Tensor, state=None):
        out, new_state = self.slstm_cell(self.norm_slstm(x), state)
        x = x + out
        xn = self.norm_ffn(x)
        x = x + self.ffn_proj_down(ops.swiglu(self.ffn_proj_up_gate(xn), self.ffn_proj_up(xn)))
        return x, new_state

    def get_weight_keys(self) -> Dict[str, str]:
        p = f"backbone.blocks.{self.block_index}"
        proj = "slstm_cell.projection_cell"
        return {
            "norm_slstm.weight": f"{p}.norm_slstm.weight",
            f"{proj}.z_proj.weight": f"{p}.slstm_layer.z.weight",
            f"{proj}.igate_proj.weight": f"{p}.slstm_layer.igate_preact.weight",
            f"{proj}.igate_proj.bias": f"{p}.slstm_layer.igate_preact.bias",
            f"{proj}.fgate_proj.weight": f"{p}.slstm_layer.fgate_preact.weight",
            f"{proj}.fgate_proj.bias": f"{p}.slstm_layer.fgate_preact.bias",
            f"{proj}.ogate_proj.weight": f"{p}.slstm_layer.ogate_preact.weight",
            "slstm_cell.output_cell.group_norm.weight": f"{p}.slstm_layer.group_norm.weight",
            "slstm_cell.output_cell.out_proj.weight": f"{p}.slstm_layer.out_proj.weight",
            "norm_ffn.weight": f"{p}.norm_ffn.weight",
            "ffn_proj_up.weight": f"{p}.ffn.proj_up.weight",
            "ffn_proj_up_gate.weight": f"{p}.ffn.proj_up_gate.weight",
            "ffn_proj_down.weight": f"{p}.ffn.proj_down.weight",
        }

    @classmethod
    def from_config(cls, block_index: int, config: Dict[str, Any], **kwargs) -> "sLSTMBlock":
        kwargs.pop("compute_dtype", None), kwargs.pop("state_dtype", None)
        kwargs.pop("norm_reduction_force_float32", None)
        return cls(block_index=block_index, embedding_dim=config["embedding_dim"],
                   num_heads=config.get("num_heads", 4), head_dim=config.get("head_dim", None),
                   gate_soft_cap=config.get("gate_soft_cap", 15.0), ffn_proj_factor=config.get("ffn_proj_factor", 2.667),
                   ffn_round_up_to_multiple_of=config.get("ffn_round_up_to_multiple_of", 64),
                   norm_eps=config.get("norm_eps", 1e-6), use_bias=config.get("use_bias", False),
                   eps=config.get("eps", 1e-6), **kwargs)

    def get_config(self) -> Dict[str, Any]:
        return {"block_index": self.block_index, "embedding_dim": self.embedding_dim, "num_heads": self.num_heads,
                "head_dim": self.head_dim, "hidden_size": self.hidden_size, "ffn_hidden_dim": self.ffn_hidden_dim,
                "gate_soft_cap": self.gate_soft_cap, "eps": self.eps}


# ---------------------------------------------------------------------------------------------
# block-diagonal recurrent variant
# ---------------------------------------------------------------------------------------------
class BlockLinear(nn.Module):
    """Block-diagonal linear layer: one ``nn.Linear`` per head on that head's slice."""

    def __init__(self, block_specs):
        super().__init__()
        self.blocks = nn.ModuleList(nn.Linear(i, o) for i, o in block_specs)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        size = x.shape[-1] // len(self.blocks)
        return torch.cat([blk(x[..., n * size:(n + 1) * size]) for n, blk in enumerate(self.blocks)], dim=-1)

    def stacked(self) -> Tuple[torch.Tensor, torch.Tensor]:
        """Weights as [NH, out, in] and biases as [NH*out] for the recurrent kernel."""
        return torch.stack([b.weight for b in self.blocks]), torch.cat([b.bias for b in self.blocks])


class _HiddenLayerNorm(nn.Module):
    """The reference block hands its hidden vector to ``MultiHeadLayerNorm`` as a 2-D ``[B, D]``
    tensor, which takes that module's plain branch: LayerNorm over all of ``D`` with a flat weight
    and bias, reductions in fp32 (xlstm_pytorch_enhanced.py:171-181, call site :455)."""

    def __init__(self, dim: int, eps: float):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))
        self.bias = nn.Parameter(torch.zeros(dim))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        # one fused pass (statistics in fp32 inside the op) instead of eight elementwise / reduction ops
        return F.layer_norm(x, (x.shape[-1],), self.weight.to(x.dtype), self.bias.to(x.dtype), self.eps)


class sLSTMBlockDiag(nn.Module):
    """sLSTM block with block-diagonal recurrent weights ``R_z, R_i, R_o, R_f``.

    ``config`` needs ``inp_dim, head_dim, head_num, p_factor, norm_eps, gate_soft_cap`` (the
    reference's ``xLSTMConfig`` works as is).  ``forward(x [B,S,D] or [B,D], hidden_state=None)``
    returns ``(out, (c, n, h, m))`` with state tensors ``[B, head_num*head_dim]``.  The input-side
    projections are batched GEMMs over the whole sequence; the recurrence over ``t`` is one
    kernel launch with the recurrent matrices resident in shared memory.
    """

    def __init__(self, config):
        super().__init__()
        self.config = config
        self.inp_dim, self.head_dim, self.head_num = config.inp_dim, config.head_dim, config.head_num
        self.hidden_dim = config.head_dim * config.head_num
        p_factor = config.p_factor[1]
        self.inp_norm = nn.LayerNorm(config.inp_dim, eps=config.norm_eps)
        self.hid_norm = _HiddenLayerNorm(self.hidden_dim, eps=config.norm_eps)
        self.W_z = nn.Linear(config.inp_dim, self.hidden_dim)
        self.W_i = nn.Linear(config.inp_dim, self.hidden_dim)
        self.W_o = nn.Linear(config.inp_dim, self.hidden_dim)
        self.W_f = nn.Linear(config.inp_dim, self.hidden_dim)
        spec = [(config.head_dim, config.head_dim)] * config.head_num
        self.R_z, self.R_i, self.R_o, self.R_f = (BlockLinear(spec) for _ in range(4))
        proj_dim = int(p_factor * self.hidden_dim)
        self.up_proj = nn.Linear(self.hidden_dim, 2 * proj_dim)
        self.down_proj = nn.Linear(proj_dim, config.inp_dim)

    @property
    def device(self):
        return next(self.parameters()).device

    def init_hidden(self, batch_size: int):
        z = torch.zeros(batch_size, self.hidden_dim, device=self.device)
        return z.clone(), torch.ones_like(z), z.clone(), z.clone()  # c, n, h, m

    def forward(self, x: torch.Tensor, hidden_state=None, use_conv: bool = False):
        if use_conv:
            raise NotImplementedError("the convolutional input path is outside the kernel-backed block")
        single = x.dim() == 2
        xs = x.unsqueeze(1) if single else x
        B, S, _ = xs.shape
        xn = self.inp_norm(xs)
        # gate order of the kernel: i, f, z, o.  One GEMM over the four stacked input projections writes
        # gx [B,S,4,D] directly (no stack copy of four [B,S,D] results)
        Wg = torch.cat([self.W_i.weight, self.W_f.weight, self.W_z.weight, self.W_o.weight], dim=0)
        bg = torch.cat([self.W_i.bias, self.W_f.bias, self.W_z.bias, self.W_o.bias], dim=0)
        gx = F.linear(xn, Wg, bg).view(B, S, 4, self.hidden_dim)
        Rs, rbs = zip(*(lin.stacked() for lin in (self.R_i, self.R_f, self.R_z, self.R_o)))
        R, rb = torch.stack(Rs), torch.stack(rbs)
        hs, state = ops.slstm_recurrent(gx, R, rb, hidden_state, self.head_num, self.config.gate_soft_cap)
        out = self.hid_norm(hs)
        Wu, bu, Wd, Pp = self._ffn_weights()
        y = F.linear(out, Wu, bu)
        out = F.linear(y[..., :Pp] * F.gelu(y[..., Pp:]), Wd, self.down_proj.bias) + xs
        return (out[:, 0] if single else out), state

    def _ffn_weights(self):
        """Gated-FFN weights with the projection width padded to a multiple of 8 (zero rows / columns):
        ``int(4/3 * hidden)`` is odd-sized (1365 at hidden 1024), which sends both GEMMs to unaligned
        legacy kernels several times slower; the padded product is identical.  Rebuilt when the
        parameters change."""
        up, down = self.up_proj, self.down_proj
        P = down.in_features
        Pp = (P + 7) // 8 * 8
        if Pp == P:
            return up.weight, up.bias, down.weight, P
        key = (up.weight._version, up.weight.data_ptr(), up.bias._version, down.weight._version, down.weight.data_ptr(),
               up.weight.dtype, up.weight.device)
        cache = getattr(self, "_ffn_cache", None)
        if cache is None or cache[0] != key:
            with torch.no_grad():
                Wu = up.weight.new_zeros(2 * Pp, up.in_features)
                Wu[:P], Wu[Pp:Pp + P] = up.weight[:P], up.weight[P:]
                bu = up.bias.new_zeros(2 * Pp)
                bu[:P], bu[Pp:Pp + P] = up.bias[:P], up.bias[P:]
                Wd = down.weight.new_zeros(down.out_features, Pp)
                Wd[:, :P] = down.weight
            self._ffn_cache = cache = (key, Wu, bu, Wd)
        return cache[1], cache[2], cache[3], Pp


__all__ = ["CausalConv1d", "sLSTMStepwiseKernelCell", "sLSTMProjectionCell", "sLSTMOutputCell", "sLSTMNeuron", "sLSTMBlock",
           "BlockLinear", "sLSTMBlockDiag"]
