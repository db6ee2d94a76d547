"""ctypes binding of ``libxlstm_cuda.so`` (the C ABI declared in ``include/xlstm_cuda.h``).

There is no fallback: if the shared library is missing or a kernel returns an
error status, the call raises.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_int64, c_size_t, c_void_p
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libxlstm_cuda.so"

F32, BF16 = 0, 1
STEP_STATE_SETTLED = 1

_SIGNATURES = {
    "xlstm_version": (c_int, []),
    "xlstm_strerror": (ctypes.c_char_p, [c_int]),
    "xlstm_softcap": (c_int, [c_void_p, c_void_p, c_int64, c_float, c_int, c_void_p]),
    "xlstm_mlstm_step": (c_int, [c_void_p] * 5 + [c_void_p] * 3 + [c_void_p] * 4 + [c_int] * 4 + [c_float, c_int, c_void_p]),
    "xlstm_mlstm_chunkwise_fwd": (c_int, [c_void_p] * 5 + [c_void_p] * 3 + [c_void_p] * 4 + [c_int] * 6
                                  + [c_float, c_int, ctypes.POINTER(c_int64), c_void_p, c_size_t, c_void_p]),
    "xlstm_mlstm_chunkwise_fwd_gather": (c_int, [c_void_p] * 5 + [c_void_p] * 3 + [c_void_p] * 4 + [c_int] * 6
                                         + [c_float, c_int, ctypes.POINTER(c_int64), c_void_p, c_size_t,
                                            ctypes.POINTER(c_void_p), c_int, c_void_p]),
    "xlstm_mlstm_chunkwise_fwd_scatter": (c_int, [c_void_p] * 5 + [c_void_p] * 3 + [c_void_p] * 3 + [c_int] * 6
                                          + [c_float, c_int, ctypes.POINTER(c_int64), c_void_p, c_size_t,
                                             ctypes.POINTER(c_void_p), c_int, c_int, c_void_p]),
    "xlstm_mlstm_chunkwise_workspace_bytes": (c_size_t, [c_int] * 7),
    "xlstm_mlstm_chunkwise_set_general_only": (c_int, [c_int]),
    "xlstm_mlstm_chunkwise_set_segments": (c_int, [c_int]),
    "xlstm_mlstm_chunkwise_status": (c_int, [c_void_p, c_void_p]),
    "xlstm_slstm_recurrent_status": (c_int, [c_void_p]),
    "xlstm_mlstm_chunkwise_fwd_static": (c_int, [c_void_p] * 5 + [c_void_p] * 3 + [c_void_p] * 4 + [c_int] * 6
                                         + [c_float, c_int, ctypes.POINTER(c_int64), c_void_p]),
    "xlstm_slstm_scan": (c_int, [c_void_p] * 4 + [c_void_p] * 3 + [c_void_p] * 4 + [c_int] * 4 + [c_float, c_int, c_void_p]),
    "xlstm_slstm_recurrent": (c_int, [c_void_p] * 3 + [c_void_p] * 4 + [c_void_p] * 5 + [c_int] * 4 + [c_float, c_int, c_void_p]),
    "xlstm_mlstm_step_gatecap": (c_int, [c_void_p] * 5 + [c_void_p] * 3 + [c_void_p] * 4 + [c_int] * 4
                                 + [c_float, c_float, c_int, c_void_p]),
    "xlstm_mlstm_step_ex": (c_int, [c_void_p] * 5 + [c_void_p] * 3 + [c_void_p] * 4 + [c_int] * 4
                            + [c_float, c_float, c_int, c_int, c_void_p]),
    "xlstm_mlstm_step_gated": (c_int, [c_void_p] * 5 + [c_void_p] * 3 + [c_void_p, c_int64, c_void_p, c_float]
                               + [c_void_p] * 4 + [c_int] * 4 + [c_float, c_float, c_int, c_int, c_void_p]),
    "xlstm_mlstm_chunkwise_fwd_gatecap": (c_int, [c_void_p] * 5 + [c_void_p] * 3 + [c_void_p] * 4 + [c_int] * 6
                                          + [c_float, c_float, c_int, ctypes.POINTER(c_int64), c_void_p, c_size_t, c_void_p]),
    "xlstm_rms_norm": (c_int, [c_void_p] * 3 + [c_int64, c_int, c_float, c_int, c_void_p]),
    "xlstm_add_rms_norm": (c_int, [c_void_p] * 5 + [c_int64, c_int, c_float, c_int, c_void_p]),
    "xlstm_mlstm_output_gate": (c_int, [c_void_p] * 4 + [c_int] * 4 + [ctypes.POINTER(c_int64), c_int64, c_float, c_int, c_void_p]),
    "xlstm_swiglu": (c_int, [c_void_p] * 3 + [c_int64, c_int, c_int64, c_int64, c_int, c_void_p]),
    "xlstm_linear_token": (c_int, [c_void_p] * 4 + [c_float, c_void_p, c_void_p] + [c_int] * 5 + [c_void_p]),
    "xlstm_causal_conv1d": (c_int, [c_void_p] * 6 + [c_int] * 6 + [c_void_p]),
}

_lib = None


class XlstmCudaError(RuntimeError):
    """A kernel entry point returned a negative status."""


def exported_symbols():
    return list(_SIGNATURES)


def load() -> ctypes.CDLL:
    """Load the shared library (once) and attach argument types."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m xlstm_cuda._build` "
                "(nvcc, sm_100a); xlstm_cuda has no fallback path")
        lib = ctypes.CDLL(str(LIB_PATH))
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(status: int, what: str) -> None:
    if status != 0:
        msg = load().xlstm_strerror(status).decode()
        raise XlstmCudaError(f"{what}: {msg} (status {status})")
