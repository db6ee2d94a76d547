"""Tensor-level wrappers: torch CUDA tensors in, torch CUDA tensors out, kernels via the C ABI.

torch is used for device memory and the current stream only.  Every function
raises if its inputs are not on a CUDA device: there is no CPU path.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from . import _lib

_DT = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16}


def _dtype_code(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise TypeError(f"xlstm_cuda kernels take float32 or bfloat16 activations, got {t.dtype}") from None


def _need_cuda(*ts: torch.Tensor) -> None:
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("xlstm_cuda kernels need CUDA tensors (no CPU fallback exists)")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _state32(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.float32).contiguous()


def softcap(x: torch.Tensor, cap: Optional[float], out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``cap * tanh(x / cap)``; ``cap`` None or <= 0 returns ``x`` unchanged."""
    if cap is None or cap <= 0:
        return x
    _need_cuda(x)
    xc = x.contiguous()
    y = torch.empty_like(xc) if out is None else out
    _lib.check(_lib.load().xlstm_softcap(xc.data_ptr(), y.data_ptr(), xc.numel(), float(cap), _dtype_code(xc), _stream()),
               "xlstm_softcap")
    return y.view(x.shape)


def mlstm_step(q, k, v, i, f, state=None, eps: float = 1e-6, inplace: bool = False):
    """One decode step.  q,k: [B,NH,dqk]; v: [B,NH,dv]; i,f: [B,NH]; state (C,n,m) fp32 or None.

    Returns ``h [B,NH,dv]`` and the new state.  ``inplace=True`` overwrites the
    caller's ``C`` (the 2 x dqk x dv x 4 byte stream then hits one buffer).
    """
    _need_cuda(q, k, v, i, f)
    B, NH, dqk = q.shape
    dv = v.shape[-1]
    dt = _dtype_code(q)
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    i, f = i.to(q.dtype).contiguous(), f.to(q.dtype).contiguous()
    if state is not None:
        C0, n0, m0 = (_state32(s) for s in state)
        m0 = m0.reshape(B, NH)
    else:
        C0 = n0 = m0 = None
    dev = q.device
    h = torch.empty(B, NH, dv, dtype=q.dtype, device=dev)
    C1 = C0 if (inplace and C0 is not None) else torch.empty(B, NH, dqk, dv, dtype=torch.float32, device=dev)
    n1 = torch.empty(B, NH, dqk, dtype=torch.float32, device=dev)
    m1 = torch.empty(B, NH, dtype=torch.float32, device=dev)
    _lib.check(_lib.load().xlstm_mlstm_step(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), i.data_ptr(), f.data_ptr(), _ptr(C0), _ptr(n0), _ptr(m0),
        h.data_ptr(), C1.data_ptr(), n1.data_ptr(), m1.data_ptr(), B, NH, dqk, dv, float(eps), dt, _stream()),
        "xlstm_mlstm_step")
    return h, (C1, n1, m1)


def _strides3(t: torch.Tensor):
    # [B,NH,S,d] view with a contiguous last dimension -> (batch, head, token) element strides
    return [t.stride(0), t.stride(1), t.stride(2)]


def chunkwise_workspace_bytes(B, NH, S, dqk, dv, L, dtype: torch.dtype) -> int:
    return int(_lib.load().xlstm_mlstm_chunkwise_workspace_bytes(B, NH, S, dqk, dv, L, _DT[dtype]))


def mlstm_chunkwise(q, k, v, i, f, state=None, chunk_size: int = 64, eps: float = 1e-6,
                    workspace: Optional[torch.Tensor] = None, h_out: Optional[torch.Tensor] = None,
                    h_peer_ptrs=None):
    """Chunkwise forward.  q,k: [B,NH,S,dqk]; v: [B,NH,S,dv]; i,f: [B,NH,S] (any strides with a
    contiguous last dimension, e.g. the permuted [B,S,NH,d] projection output).

    ``h_out`` (optional) is a ``[B,NH,S,dv]`` view to write h into (e.g. a head slice of a
    ``[B,S,NH_total,dv]`` buffer); ``h_peer_ptrs`` (optional) are raw device pointers to the same
    slot in peer GPUs' buffers: the kernel stores every h tile there too (fused all-gather)."""
    _need_cuda(q, k, v, i, f)
    B, NH, S, dqk = q.shape
    dv = v.shape[-1]
    dt = _dtype_code(q)
    fix = lambda t: t if t.stride(-1) == 1 else t.contiguous()
    q, k, v = fix(q), fix(k.to(q.dtype)), fix(v.to(q.dtype))
    i, f = i.to(q.dtype), f.to(q.dtype)
    if i.stride() != f.stride():
        i, f = i.contiguous(), f.contiguous()
    if state is not None:
        C0, n0, m0 = (_state32(s) for s in state)
        m0 = m0.reshape(B, NH)
    else:
        C0 = n0 = m0 = None
    dev = q.device
    if h_out is not None:
        if tuple(h_out.shape) != (B, NH, S, dv) or h_out.dtype != q.dtype or h_out.stride(-1) != 1:
            raise ValueError("h_out must be a [B,NH,S,dv] view of the activation dtype with a contiguous last dimension")
        h = h_out
    else:
        h = torch.empty(B, NH, S, dv, dtype=q.dtype, device=dev)
    C1 = torch.empty(B, NH, dqk, dv, dtype=torch.float32, device=dev)
    n1 = torch.empty(B, NH, dqk, dtype=torch.float32, device=dev)
    m1 = torch.empty(B, NH, dtype=torch.float32, device=dev)
    strides = _strides3(q) + _strides3(k) + _strides3(v) + _strides3(h) + [i.stride(0), i.stride(1), i.stride(2)]
    sarr = (ctypes.c_int64 * 15)(*strides)
    need = chunkwise_workspace_bytes(B, NH, S, dqk, dv, chunk_size, q.dtype)
    if need and (workspace is None or workspace.numel() * workspace.element_size() < need):
        workspace = torch.empty(need, dtype=torch.uint8, device=dev)
    wbytes = 0 if workspace is None else workspace.numel() * workspace.element_size()
    if h_peer_ptrs:
        peers = (ctypes.c_void_p * len(h_peer_ptrs))(*[int(x) for x in h_peer_ptrs])
        _lib.check(_lib.load().xlstm_mlstm_chunkwise_fwd_gather(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), i.data_ptr(), f.data_ptr(), _ptr(C0), _ptr(n0), _ptr(m0),
            h.data_ptr(), C1.data_ptr(), n1.data_ptr(), m1.data_ptr(), B, NH, S, dqk, dv, int(chunk_size), float(eps),
            dt, sarr, _ptr(workspace), wbytes, peers, len(h_peer_ptrs), _stream()), "xlstm_mlstm_chunkwise_fwd_gather")
        return h, (C1, n1, m1)
    _lib.check(_lib.load().xlstm_mlstm_chunkwise_fwd(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), i.data_ptr(), f.data_ptr(), _ptr(C0), _ptr(n0), _ptr(m0),
        h.data_ptr(), C1.data_ptr(), n1.data_ptr(), m1.data_ptr(), B, NH, S, dqk, dv, int(chunk_size), float(eps), dt,
        sarr, _ptr(workspace), wbytes, _stream()), "xlstm_mlstm_chunkwise_fwd")
    return h, (C1, n1, m1)


def slstm_scan(z, i, f, o, state=None, eps: float = 1e-6):
    """Packaged sLSTM cell over S steps.  z: [B,S,NH,H]; i,f,o: [B,S,NH]; state (c,n,m) or None."""
    _need_cuda(z, i, f, o)
    B, S, NH, H = z.shape
    dt = _dtype_code(z)
    z = z.contiguous()
    i, f, o = (g.to(z.dtype).contiguous() for g in (i, f, o))
    if state is not None:
        c0, n0, m0 = (_state32(s) for s in state)
    else:
        c0 = n0 = m0 = None
    dev = z.device
    h = torch.empty_like(z)
    c1 = torch.empty(B, NH, H, dtype=torch.float32, device=dev)
    n1 = torch.empty(B, NH, H, dtype=torch.float32, device=dev)
    m1 = torch.empty(B, NH, dtype=torch.float32, device=dev)
    _lib.check(_lib.load().xlstm_slstm_scan(
        z.data_ptr(), i.data_ptr(), f.data_ptr(), o.data_ptr(), _ptr(c0), _ptr(n0), _ptr(m0),
        h.data_ptr(), c1.data_ptr(), n1.data_ptr(), m1.data_ptr(), B, S, NH, H, float(eps), dt, _stream()),
        "xlstm_slstm_scan")
    return h, (c1, n1, m1)


def slstm_recurrent(gx, R, rb, state=None, num_heads: int = 4, cap: Optional[float] = 15.0):
    """Block-diagonal recurrent sLSTM.  gx: [B,S,4,D] (i,f,z,o); R: [4,NH,dh,dh]; rb: [4,D] fp32;
    state (c,n,h,m) each [B,D] fp32 or None.  Returns ``hs [B,S,D]`` and the final state."""
    _need_cuda(gx, R, rb)
    B, S, four, D = gx.shape
    if four != 4 or D % num_heads:
        raise ValueError("gx must be [B,S,4,D] with D divisible by num_heads")
    dh = D // num_heads
    dt = _dtype_code(gx)
    gx = gx.contiguous()
    R = R.to(gx.dtype).contiguous()
    rb = rb.to(torch.float32).contiguous()
    if state is not None:
        c0, n0, h0, m0 = (_state32(s) for s in state)
    else:
        c0 = n0 = h0 = m0 = None
    dev = gx.device
    hs = torch.empty(B, S, D, dtype=gx.dtype, device=dev)
    outs = [torch.empty(B, D, dtype=torch.float32, device=dev) for _ in range(4)]
    _lib.check(_lib.load().xlstm_slstm_recurrent(
        gx.data_ptr(), R.data_ptr(), rb.data_ptr(), _ptr(c0), _ptr(n0), _ptr(h0), _ptr(m0), hs.data_ptr(),
        *(o.data_ptr() for o in outs), B, S, num_heads, dh, float(cap) if cap else 0.0, dt, _stream()),
        "xlstm_slstm_recurrent")
    return hs, tuple(outs)
