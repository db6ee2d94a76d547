"""ctypes front end of the CPU oracle (``xlstm_oracle.c``).  TEST INFRASTRUCTURE ONLY.

The oracle is the checker for the CUDA kernels: tests, the smoke check and the
cpu-baseline leg of the benchmark may import this module; the shipped package
must not.  Parity status: pinned against fixtures made by importing the
reference's own classes (``tests/golden/make_golden.py``).

Every function takes and returns numpy fp32 arrays in the reference's layouts
(``q,k,v: [B,NH,S,d]``, gates ``[B,NH,S]``, state ``C:[B,NH,dqk,dv] n:[B,NH,dqk]
m:[B,NH]``), see ``xlstm_oracle.c`` for the reference file:line of each one.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_SRC = _HERE / "xlstm_oracle.c"
_OUT = _HERE / "_build" / "libxlstm_oracle.so"

_f32p = ctypes.POINTER(ctypes.c_float)
_lib = None


def build(force: bool = False) -> Path:
    """Compile the C oracle with gcc (-O2, OpenMP) into ``oracle/_build``."""
    if _OUT.exists() and not force and _OUT.stat().st_mtime >= _SRC.stat().st_mtime:
        return _OUT
    _OUT.parent.mkdir(parents=True, exist_ok=True)
    cmd = ["gcc", "-O2", "-fopenmp", "-fno-fast-math", "-ffp-contract=off", "-shared", "-fPIC",
           str(_SRC), "-o", str(_OUT), "-lm"]
    subprocess.run(cmd, check=True)
    return _OUT


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(str(build()))
        _lib.xo_max_threads.restype = ctypes.c_int
    return _lib


def max_threads() -> int:
    return int(lib().xo_max_threads())


def set_threads(n: int) -> None:
    lib().xo_set_threads(ctypes.c_int(int(n)))


def _c(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a):
    return None if a is None else a.ctypes.data_as(_f32p)


def bf16_round(a: np.ndarray) -> np.ndarray:
    """Round fp32 values to the nearest bf16 (ties to even), kept as fp32."""
    u = _c(a).view(np.uint32).astype(np.uint64)
    lsb = (u >> 16) & 1
    u = ((u + 0x7FFF + lsb) & 0xFFFF0000).astype(np.uint32)
    return u.view(np.float32).reshape(np.shape(a))


def softcap(x, cap: float):
    x = _c(x)
    y = np.empty_like(x)
    lib().xo_softcap(_p(x), _p(y), ctypes.c_long(x.size), ctypes.c_float(cap if cap is not None else 0.0))
    return y


def rmsnorm(x, w, eps: float):
    x = _c(x)
    w = None if w is None else _c(w)
    y = np.empty_like(x)
    d = x.shape[-1]
    lib().xo_rmsnorm(_p(x), _p(w), _p(y), ctypes.c_long(x.size // d), ctypes.c_int(d), ctypes.c_float(eps))
    return y


def multihead_rmsnorm(x, w, eps: float):
    """x: [..., NH, DH] -> [..., NH*DH] (per-head RMS, flat weight)."""
    x = _c(x)
    w = None if w is None else _c(w)
    NH, DH = x.shape[-2:]
    y = np.empty_like(x)
    lib().xo_multihead_rmsnorm(_p(x), _p(w), _p(y), ctypes.c_long(x.size // (NH * DH)),
                               ctypes.c_int(NH), ctypes.c_int(DH), ctypes.c_float(eps))
    return y.reshape(*x.shape[:-2], NH * DH)


def mlstm_output_gate(h, og, w, eps: float):
    """h: [B,NH,S,dv]; og: [B,S,NH*dv]; w: [NH*dv] or None -> [B,S,NH*dv]."""
    h, og = _c(h), _c(og)
    w = None if w is None else _c(w)
    B, NH, S, dv = h.shape
    y = np.empty((B, S, NH * dv), dtype=np.float32)
    lib().xo_mlstm_output_gate(_p(h), _p(og), _p(w), _p(y), ctypes.c_int(B), ctypes.c_int(NH), ctypes.c_int(S),
                               ctypes.c_int(dv), ctypes.c_float(eps))
    return y


def linear(x, W, bias=None):
    """x: [..., K]; W: [N, K]; bias: [N] -> [..., N]."""
    x, W = _c(x), _c(W)
    bias = None if bias is None else _c(bias)
    K = x.shape[-1]
    N = W.shape[0]
    y = np.empty(x.shape[:-1] + (N,), dtype=np.float32)
    lib().xo_linear(_p(x), _p(W), _p(bias), _p(y), ctypes.c_long(x.size // K), ctypes.c_int(N), ctypes.c_int(K))
    return y


def swiglu(g, u):
    g, u = _c(g), _c(u)
    y = np.empty_like(g)
    lib().xo_swiglu(_p(g), _p(u), _p(y), ctypes.c_long(g.size))
    return y


def causal_conv1d(x, w, bias=None, state=None, silu: bool = False, return_state: bool = False):
    """x: [B,S,C]; w: [C,K]; bias: [C]; state: [B,K-1,C] (inputs before the first token)."""
    x, w = _c(x), _c(w)
    bias = None if bias is None else _c(bias)
    state = None if state is None else _c(state)
    B, S, C = x.shape
    K = w.shape[-1]
    y = np.empty_like(x)
    st = np.empty((B, K - 1, C), dtype=np.float32) if return_state else None
    lib().xo_causal_conv1d(_p(x), _p(w), _p(bias), _p(state), _p(st), _p(y), ctypes.c_int(B), ctypes.c_int(S),
                           ctypes.c_int(C), ctypes.c_int(K), ctypes.c_int(1 if silu else 0))
    return (y, st) if return_state else y


def _mlstm_common(fn, q, k, v, i, f, state, eps, *tail):
    q, k, v, i, f = map(_c, (q, k, v, i, f))
    B, NH, S, dqk = q.shape
    dv = v.shape[-1]
    if state is not None:
        C0, n0, m0 = (_c(s) for s in state)
        m0 = m0.reshape(B, NH)
    else:
        C0 = n0 = m0 = None
    h = np.empty((B, NH, S, dv), np.float32)
    C1 = np.empty((B, NH, dqk, dv), np.float32)
    n1 = np.empty((B, NH, dqk), np.float32)
    m1 = np.empty((B, NH), np.float32)
    fn(_p(q), _p(k), _p(v), _p(i), _p(f), _p(C0), _p(n0), _p(m0), _p(h), _p(C1), _p(n1), _p(m1),
       ctypes.c_int(B), ctypes.c_int(NH), ctypes.c_int(S), ctypes.c_int(dqk), ctypes.c_int(dv), *tail)
    return h, (C1, n1, m1)


def mlstm_recurrent(q, k, v, i, f, state=None, eps: float = 1e-6, emulate_bf16: bool = False):
    """Step-by-step mLSTM over S tokens: ``h, (C, n, m)``."""
    return _mlstm_common(lib().xo_mlstm_recurrent, q, k, v, i, f, state, eps,
                         ctypes.c_float(eps), ctypes.c_int(1 if emulate_bf16 else 0))


def mlstm_chunkwise(q, k, v, i, f, state=None, chunk_size: int = 64, eps: float = 1e-6):
    """Two-phase chunkwise mLSTM (S must be a multiple of ``chunk_size``)."""
    if np.shape(q)[2] % chunk_size:
        raise ValueError("S must be a multiple of chunk_size")
    return _mlstm_common(lib().xo_mlstm_chunkwise, q, k, v, i, f, state, eps,
                         ctypes.c_int(chunk_size), ctypes.c_float(eps))


def slstm_scan(z, i, f, o, state=None, eps: float = 1e-6):
    """Packaged sLSTM cell applied to every timestep.  z: [B,S,NH,H]; gates [B,S,NH]."""
    z, i, f, o = map(_c, (z, i, f, o))
    B, S, NH, H = z.shape
    if state is not None:
        c0, n0, m0 = (_c(s) for s in state)
    else:
        c0 = n0 = m0 = None
    h = np.empty_like(z)
    c1 = np.empty((B, NH, H), np.float32)
    n1 = np.empty((B, NH, H), np.float32)
    m1 = np.empty((B, NH), np.float32)
    lib().xo_slstm_scan(_p(z), _p(i), _p(f), _p(o), _p(c0), _p(n0), _p(m0), _p(h), _p(c1), _p(n1), _p(m1),
                        ctypes.c_int(B), ctypes.c_int(S), ctypes.c_int(NH), ctypes.c_int(H), ctypes.c_float(eps))
    return h, (c1, n1, m1)


def slstm_recurrent(gx, R, rb, state=None, num_heads: int = 4, cap: float = 15.0):
    """Block-diagonal-recurrent sLSTM.  gx: [B,S,4,D] (i,f,z,o); R: [4,NH,dh,dh]; rb: [4,D]."""
    gx, R, rb = map(_c, (gx, R, rb))
    B, S, _, D = gx.shape
    dh = D // num_heads
    if state is not None:
        c0, n0, h0, m0 = (_c(s) for s in state)
    else:
        c0 = n0 = h0 = m0 = None
    hs = np.empty((B, S, D), np.float32)
    outs = [np.empty((B, D), np.float32) for _ in range(4)]
    lib().xo_slstm_recurrent(_p(gx), _p(R), _p(rb), _p(c0), _p(n0), _p(h0), _p(m0), _p(hs),
                             *(_p(o) for o in outs), ctypes.c_int(B), ctypes.c_int(S),
                             ctypes.c_int(num_heads), ctypes.c_int(dh), ctypes.c_float(cap if cap else 0.0))
    return hs, tuple(outs)


if __name__ == "__main__":
    print(build(force=True), "threads:", max_threads(), "cpus:", os.cpu_count())
