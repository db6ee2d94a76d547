"""Normalisation cells around the hot path: RMS norms run the ``rms_norm`` kernel (fp32 math, one
rounding); like every kernel-backed cell they need CUDA tensors.

``RMSNormCell``        xlstm_metal/torch_native/blocks/rms_norm/rmsnorm.py:11-43 (math:
                       rms_norm_kernel.metal:20-30, tests/parity/canonical_reference.py:26-33)
``MultiHeadRMSNorm``   xlstm_metal/torch_native/blocks/mlstm/multihead_norm/multihead_norm.py:43-64
``MultiHeadLayerNorm`` same file :5-40
"""
from __future__ import annotations

import torch
import torch.nn as nn

from .. import ops


class RMSNormCell(nn.Module):
    def __init__(self, dims: int, eps: float = 1e-6, use_weight: bool = True,
                 force_float32_reductions: bool = True, param_dtype: torch.dtype = torch.float32) -> None:
        super().__init__()
        self.eps = eps
        self.force_float32 = force_float32_reductions
        if use_weight:
            self.weight = nn.Parameter(torch.ones(dims, dtype=param_dtype))
        else:
            self.register_parameter("weight", None)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.rms_norm(x, self.weight, self.eps)


class MultiHeadRMSNorm(nn.Module):
    """[B,S,NH,DH] -> per-head RMS normalisation -> [B,S,NH*DH] times a flat weight."""

    def __init__(self, num_heads: int, head_dim: int, eps: float = 1e-6, use_weight: bool = True):
        super().__init__()
        self.num_heads, self.head_dim, self.eps = num_heads, head_dim, eps
        if use_weight:
            self.weight = nn.Parameter(torch.ones(num_heads * head_dim))
        else:
            self.register_parameter("weight", None)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        B, S, NH, DH = x.shape
        if NH != self.num_heads or DH != self.head_dim:
            raise ValueError(f"Expected shape [B,S,{self.num_heads},{self.head_dim}], got {x.shape}")
        y = ops.rms_norm(x, None, self.eps).reshape(B, S, NH * DH)
        if self.weight is not None:
            y = y * self.weight.to(y.dtype)
        return y


class MultiHeadLayerNorm(nn.Module):
    """[B,S,NH,DH] -> per-head LayerNorm -> [B,S,NH*DH] with flat weight / bias."""

    def __init__(self, num_heads: int, head_dim: int, eps: float = 1e-6, use_weight: bool = True,
                 use_bias: bool = False):
        super().__init__()
        self.num_heads, self.head_dim, self.eps = num_heads, head_dim, eps
        self.weight = nn.Parameter(torch.ones(num_heads * head_dim)) if use_weight else None
        self.bias = nn.Parameter(torch.zeros(num_heads * head_dim)) if use_bias else None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        B, S, NH, DH = x.shape
        if NH != self.num_heads or DH != self.head_dim:
            raise ValueError(f"Expected shape [B,S,{self.num_heads},{self.head_dim}], got {x.shape}")
        mean = x.mean(dim=-1, keepdim=True)
        var = x.var(dim=-1, keepdim=True, unbiased=False)
        y = ((x - mean) / torch.sqrt(var + self.eps)).reshape(B, S, NH * DH)
        if self.weight is not None:
            y = y * self.weight
        if self.bias is not None:
            y = y + self.bias
        return y


__all__ = ["RMSNormCell", "MultiHeadRMSNorm", "MultiHeadLayerNorm"]
