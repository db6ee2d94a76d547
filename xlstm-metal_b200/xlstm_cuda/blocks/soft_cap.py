"""Soft-cap cell on the CUDA kernel.

Mirrors ``xlstm_metal/torch_native/blocks/soft_cap/softcap.py:14-36`` (``SoftCapCell`` and the
module-level ``soft_cap`` instance): ``cap <= 0`` or ``None`` is the identity, and a tensor that
is not on the accelerator raises ``RuntimeError`` (the reference insists on MPS the same way).
``SoftCap`` is the ``forward(x, cap)`` module the projection cell instantiates
(``.../mlstm_chunkwise/mlstm_projection_cell.py:16,53,101-104``).
"""
from __future__ import annotations

from typing import Optional, Union

import torch
import torch.nn as nn

from .. import ops


class SoftCapCell(nn.Module):
    def __init__(self, cap_value: Optional[float] = None) -> None:
        super().__init__()
        self._cap_value = float(cap_value) if cap_value is not None else 0.0

    def forward(self, x: torch.Tensor, cap_value: Optional[float] = None) -> torch.Tensor:
        cap = float(cap_value) if cap_value is not None else self._cap_value
        if cap <= 0.0:
            return x
        if not x.is_cuda:
            raise RuntimeError("SoftCapCell requires tensors on a CUDA device")
        return ops.softcap(x, cap)


class SoftCap(nn.Module):
    """``forward(x, cap)`` with ``cap`` a float or a 0-dim tensor."""

    def forward(self, x: torch.Tensor, cap: Union[float, torch.Tensor, None]) -> torch.Tensor:
        if cap is None:
            return x
        return soft_cap(x, float(cap))


soft_cap = SoftCapCell()

__all__ = ["SoftCapCell", "SoftCap", "soft_cap"]
