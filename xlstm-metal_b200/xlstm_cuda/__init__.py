"""xlstm_cuda: hand-written sm_100a kernels for the xLSTM inference hot path behind the
reference's ``torch_native`` call signatures.

``ops``       tensor-level entry points over the C ABI
``blocks``    drop-in cells, neurons and blocks (mLSTM, sLSTM, soft-cap, norms)
``models``    ``WiredxLSTM``;  ``generate``: ``xLSTMRunner``;  ``wiring`` / ``utils``: glue
``parallel``  head- and batch-sharding over several GPUs
"""
from . import _lib, ops  # noqa: F401

__all__ = ["_lib", "ops"]
