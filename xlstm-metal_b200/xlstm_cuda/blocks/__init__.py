"""Cells and blocks with the reference's names and call signatures."""
from .mlstm import (mLSTMBlock, mLSTMNeuron, mLSTMOutputCell, mLSTMParallelKernelCell, mLSTMProjectionCell,
                    mLSTMRecurrentKernelCell)
from .rms_norm import MultiHeadLayerNorm, MultiHeadRMSNorm, RMSNormCell
from .slstm import (BlockLinear, CausalConv1d, sLSTMBlock, sLSTMBlockDiag, sLSTMNeuron, sLSTMOutputCell,
                    sLSTMProjectionCell, sLSTMStepwiseKernelCell)
from .soft_cap import SoftCap, SoftCapCell, soft_cap

__all__ = [n for n in dir() if not n.startswith("_")]
