"""xlstm_cuda: hand-written sm_100a kernels for the xLSTM inference hot path behind the
reference's ``torch_native`` call signatures.  See ``ops`` for tensor-level entry points and
``blocks`` / ``models`` / ``generate`` for the drop-in cells, block stack and runner."""
from . import _lib, ops  # noqa: F401

__all__ = ["_lib", "ops"]
