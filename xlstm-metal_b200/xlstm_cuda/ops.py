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


def mlstm_step(q, k, v, i, f, state=None, eps: float = 1e-6, inplace: bool = False,
               gate_cap: Optional[float] = None, state_settled: bool = False):
    """One decode step.  q,k: [B,NH,dqk]; v: [B,NH,dv]; i,f: [B,NH]; state (C,n,m) fp32 or None.

    Returns ``h [B,NH,dv]`` and the new state.  ``inplace=True`` overwrites the
    caller's ``C`` (the 2 x dqk x dv x 4 byte stream then hits one buffer).
    ``gate_cap`` > 0: ``i`` and ``f`` are the raw gate projections and are soft-capped inside the kernel.
    ``state_settled=True`` promises that ``state`` was not written by the kernel launched just before this call
    (a layer stack: the launch before a layer's step is its projection); the kernel then starts streaming the
    state while that kernel drains.
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
    flags = _lib.STEP_STATE_SETTLED if (state_settled and state is not None) else 0
    _lib.check(_lib.load().xlstm_mlstm_step_ex(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), i.data_ptr(), f.data_ptr(), _ptr(C0), _ptr(n0), _ptr(m0),
        h.data_ptr(), C1.data_ptr(), n1.data_ptr(), m1.data_ptr(), B, NH, dqk, dv, float(eps),
        float(gate_cap) if gate_cap is not None else 0.0, flags, dt, _stream()), "xlstm_mlstm_step_ex")
    return h, (C1, n1, m1)


def mlstm_step_gated(q, k, v, i, f, ogate, norm_weight, state=None, eps: float = 1e-6, norm_eps: float = 1e-6,
                     inplace: bool = False, gate_cap: Optional[float] = None, state_settled: bool = False):
    """Decode step with the output epilogue fused in: returns ``y [B, NH*dv] = MultiHeadRMSNorm(h) * weight *
    sigmoid(ogate)`` and the new state; ``h`` itself is never written.  ``ogate: [B, NH*dv]``, possibly a column
    block of a wider one-row-per-sequence tensor (row stride >= NH*dv).  ``dv`` must be at most 512."""
    _need_cuda(q, k, v, i, f, ogate, norm_weight)
    B, NH, dqk = q.shape
    dv = v.shape[-1]
    dt = _dtype_code(q)
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    i, f = i.to(q.dtype).contiguous(), f.to(q.dtype).contiguous()
    og = ogate.to(q.dtype)
    if og.dim() != 2 or og.stride(1) != 1 or og.shape[1] != NH * dv:
        og = og.reshape(B, NH * dv).contiguous()
    ld = og.stride(0) if B > 1 else NH * dv
    if ld < NH * dv:
        og, ld = og.contiguous(), NH * dv
    w = None if norm_weight is None else norm_weight.to(q.dtype).contiguous()
    if state is not None:
        C0, n0, m0 = (_state32(s) for s in state)
        m0 = m0.reshape(B, NH)
    else:
        C0 = n0 = m0 = None
    dev = q.device
    y = torch.empty(B, NH * dv, dtype=q.dtype, device=dev)
    C1 = C0 if (inplace and C0 is not None) else torch.empty(B, NH, dqk, dv, dtype=torch.float32, device=dev)
    n1 = torch.empty(B, NH, dqk, dtype=torch.float32, device=dev)
    m1 = torch.empty(B, NH, dtype=torch.float32, device=dev)
    flags = _lib.STEP_STATE_SETTLED if (state_settled and state is not None) else 0
    _lib.check(_lib.load().xlstm_mlstm_step_gated(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), i.data_ptr(), f.data_ptr(), _ptr(C0), _ptr(n0), _ptr(m0),
        og.data_ptr(), int(ld), _ptr(w), float(norm_eps), y.data_ptr(), C1.data_ptr(), n1.data_ptr(), m1.data_ptr(),
        B, NH, dqk, dv, float(eps), float(gate_cap) if gate_cap is not None else 0.0, flags, dt, _stream()),
        "xlstm_mlstm_step_gated")
    return y, (C1, n1, m1)


def _strides3(t: torch.Tensor):
    # [B,NH,S,d] view with a contiguous last dimension -> (batch, head, token) element strides
    return [t.stride(0), t.stride(1), t.stride(2)]


def chunkwise_general_only(on: bool) -> None:
    """Send every head of the bf16 chunkwise forward to the general tensor-core kernel (``True``) or let the
    device pick per head between it and the bounded-gate-spread kernel (``False``, the default)."""
    _lib.load().xlstm_mlstm_chunkwise_set_general_only(1 if on else 0)


def chunkwise_segments(segments: Optional[int]) -> None:
    """Force the number of segments of the segment-parallel prefill (``None`` or < 1: chosen from the grid size)."""
    _lib.load().xlstm_mlstm_chunkwise_set_segments(int(segments) if segments else -1)


def chunkwise_status(workspace: Optional[torch.Tensor] = None) -> None:
    """Raise ``XlstmCudaError`` if a bounded device-side wait of the last chunkwise forward that used
    ``workspace`` gave up (``None``: the library's built-in block).  Synchronises the current stream."""
    _lib.check(_lib.load().xlstm_mlstm_chunkwise_status(_ptr(workspace), _stream()), "xlstm_mlstm_chunkwise_status")


def slstm_recurrent_status() -> None:
    """The same for the tensor-core path of ``slstm_recurrent`` (all launches since the last query)."""
    _lib.check(_lib.load().xlstm_slstm_recurrent_status(_stream()), "xlstm_slstm_recurrent_status")


def chunkwise_workspace_bytes(B, NH, S, dqk, dv, L, dtype: torch.dtype) -> int:
    return int(_lib.load().xlstm_mlstm_chunkwise_workspace_bytes(B, NH, S, dqk, dv, L, _DT[dtype]))


def mlstm_chunkwise(q, k, v, i, f, state=None, chunk_size: int = 64, eps: float = 1e-6,
                    workspace: Optional[torch.Tensor] = None, h_out: Optional[torch.Tensor] = None,
                    h_peer_ptrs=None, gate_cap: Optional[float] = None):
    """Chunkwise forward.  q,k: [B,NH,S,dqk]; v: [B,NH,S,dv]; i,f: [B,NH,S] (any strides with a
    contiguous last dimension, e.g. the permuted [B,S,NH,d] projection output).

    ``h_out`` (optional) is a ``[B,NH,S,dv]`` view to write h into (e.g. a head slice of a
    ``[B,S,NH_total,dv]`` buffer); ``h_peer_ptrs`` (optional) are raw device pointers to the same
    slot in peer GPUs' buffers: the kernel stores every h tile there too (fused all-gather).
    ``gate_cap`` > 0: ``i`` and ``f`` are the raw gate projections, soft-capped inside the kernels."""
    _need_cuda(q, k, v, i, f)
    if gate_cap is not None and gate_cap > 0 and h_peer_ptrs:
        i, f, gate_cap = softcap(i, gate_cap), softcap(f, gate_cap), None   # the gather entry takes capped gates
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
    if gate_cap is not None and gate_cap > 0:
        _lib.check(_lib.load().xlstm_mlstm_chunkwise_fwd_gatecap(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), i.data_ptr(), f.data_ptr(), _ptr(C0), _ptr(n0), _ptr(m0),
            h.data_ptr(), C1.data_ptr(), n1.data_ptr(), m1.data_ptr(), B, NH, S, dqk, dv, int(chunk_size), float(eps),
            float(gate_cap), dt, sarr, _ptr(workspace), wbytes, _stream()), "xlstm_mlstm_chunkwise_fwd_gatecap")
        return h, (C1, n1, m1)
    _lib.check(_lib.load().xlstm_mlstm_chunkwise_fwd(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), i.data_ptr(), f.data_ptr(), _ptr(C0), _ptr(n0), _ptr(m0),
        h.data_ptr(), C1.data_ptr(), n1.data_ptr(), m1.data_ptr(), B, NH, S, dqk, dv, int(chunk_size), float(eps), dt,
        sarr, _ptr(workspace), wbytes, _stream()), "xlstm_mlstm_chunkwise_fwd")
    return h, (C1, n1, m1)


def mlstm_chunkwise_scatter(q, k, v, i, f, state, h_rank_ptrs, tokens_per_rank: int, h_strides, chunk_size: int = 64,
                            eps: float = 1e-6, workspace: Optional[torch.Tensor] = None):
    """Chunkwise forward whose h tiles go to the rank that owns their tokens (``h_rank_ptrs[r]`` = this rank's
    head slot in rank r's ``[B, tokens_per_rank, NH_total, dv]`` buffer, ``h_strides`` = its (batch, head, token)
    element strides).  Returns the final state only; h lives in the ranks' buffers."""
    _need_cuda(q, k, v, i, f)
    B, NH, S, dqk = q.shape
    dv = v.shape[-1]
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
    C1 = torch.empty(B, NH, dqk, dv, dtype=torch.float32, device=dev)
    n1 = torch.empty(B, NH, dqk, dtype=torch.float32, device=dev)
    m1 = torch.empty(B, NH, dtype=torch.float32, device=dev)
    strides = _strides3(q) + _strides3(k) + _strides3(v) + list(h_strides) + [i.stride(0), i.stride(1), i.stride(2)]
    sarr = (ctypes.c_int64 * 15)(*strides)
    need = chunkwise_workspace_bytes(B, NH, S, dqk, dv, chunk_size, q.dtype)
    if need and (workspace is None or workspace.numel() * workspace.element_size() < need):
        workspace = torch.empty(need, dtype=torch.uint8, device=dev)
    ranks = (ctypes.c_void_p * len(h_rank_ptrs))(*[int(x) for x in h_rank_ptrs])
    _lib.check(_lib.load().xlstm_mlstm_chunkwise_fwd_scatter(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), i.data_ptr(), f.data_ptr(), _ptr(C0), _ptr(n0), _ptr(m0),
        C1.data_ptr(), n1.data_ptr(), m1.data_ptr(), B, NH, S, dqk, dv, int(chunk_size), float(eps), _dtype_code(q), sarr,
        _ptr(workspace), workspace.numel() * workspace.element_size(), ranks, len(h_rank_ptrs), int(tokens_per_rank),
        _stream()), "xlstm_mlstm_chunkwise_fwd_scatter")
    return C1, n1, m1


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


def rms_norm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float = 1e-6) -> torch.Tensor:
    """RMSNorm over the last dimension; ``weight`` (or None) is cast to ``x.dtype``."""
    _need_cuda(x, weight)
    cols = x.shape[-1]
    xc = x.contiguous()
    w = None if weight is None else weight.to(xc.dtype).contiguous()
    y = torch.empty_like(xc)
    rows = xc.numel() // cols if cols else 0
    _lib.check(_lib.load().xlstm_rms_norm(xc.data_ptr(), _ptr(w), y.data_ptr(), rows, cols, float(eps), _dtype_code(xc),
                                          _stream()), "xlstm_rms_norm")
    return y


def add_rms_norm(x: torch.Tensor, residual: torch.Tensor, weight: Optional[torch.Tensor], eps: float = 1e-6):
    """``s = x + residual`` and ``RMSNorm(s) * weight`` in one pass; returns ``(s, normed)``."""
    _need_cuda(x, residual, weight)
    cols = x.shape[-1]
    xc, rc = x.contiguous(), residual.to(x.dtype).contiguous()
    w = None if weight is None else weight.to(xc.dtype).contiguous()
    s, y = torch.empty_like(xc), torch.empty_like(xc)
    rows = xc.numel() // cols if cols else 0
    _lib.check(_lib.load().xlstm_add_rms_norm(xc.data_ptr(), rc.data_ptr(), _ptr(w), s.data_ptr(), y.data_ptr(), rows, cols,
                                              float(eps), _dtype_code(xc), _stream()), "xlstm_add_rms_norm")
    return s, y


def mlstm_output_gate(h: torch.Tensor, ogate: torch.Tensor, weight: Optional[torch.Tensor], eps: float = 1e-6) -> torch.Tensor:
    """Per-head RMS norm of ``h [B,NH,S,dv]`` (any strides with a contiguous last dimension) times the
    flat ``weight [NH*dv]`` times ``sigmoid(ogate [B,S,NH*dv])`` -> ``[B,S,NH*dv]``.  ``ogate`` may be a
    column block of a wider ``[B,S,N]`` tensor (a fused projection output)."""
    _need_cuda(h, ogate, weight)
    B, NH, S, dv = h.shape
    if h.stride(3) != 1:
        h = h.contiguous()
    og = ogate.to(h.dtype)
    ok = og.dim() == 3 and og.stride(2) == 1
    ld = NH * dv
    if ok:   # rows (b, s) must sit at a constant pitch: row = b * S + s
        if S == 1:
            ld = og.stride(0) if B > 1 else NH * dv
        else:
            ld = og.stride(1)
            ok = B == 1 or og.stride(0) == S * ld
        # 16-byte accesses: the column block must start on and keep a 16-byte pitch
        ok = ok and ld >= NH * dv and og.data_ptr() % 16 == 0 and (ld * og.element_size()) % 16 == 0
    if not ok:
        og = og.contiguous()
        if og.data_ptr() % 16:      # a dense but misaligned view (column block of a one-row GEMM output)
            og = og.clone()
        ld = NH * dv
    w = None if weight is None else weight.to(h.dtype).contiguous()
    y = torch.empty(B, S, NH * dv, dtype=h.dtype, device=h.device)
    strides = (ctypes.c_int64 * 3)(h.stride(0), h.stride(1), h.stride(2))
    _lib.check(_lib.load().xlstm_mlstm_output_gate(h.data_ptr(), og.data_ptr(), _ptr(w), y.data_ptr(), B, NH, S, dv,
                                                   strides, ld, float(eps), _dtype_code(h), _stream()),
               "xlstm_mlstm_output_gate")
    return y


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` over ``[..., cols]``; the two may be column blocks of one wider tensor
    (row stride larger than ``cols``), the result is dense."""
    _need_cuda(gate, up)
    cols = gate.shape[-1]
    g2, u2 = gate.reshape(-1, cols), up.to(gate.dtype).reshape(-1, cols)
    if g2.stride(1) != 1:
        g2 = g2.contiguous()
    if u2.stride(1) != 1:
        u2 = u2.contiguous()
    rows = g2.shape[0]
    y = torch.empty(*gate.shape[:-1], cols, dtype=gate.dtype, device=gate.device)
    ldg = g2.stride(0) if rows > 1 else cols
    ldu = u2.stride(0) if rows > 1 else cols
    _lib.check(_lib.load().xlstm_swiglu(g2.data_ptr(), u2.data_ptr(), y.data_ptr(), rows, cols, ldg, ldu,
                                        _dtype_code(g2), _stream()), "xlstm_swiglu")
    return y


def causal_conv1d(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, silu: bool = False,
                  state: Optional[torch.Tensor] = None, return_state: bool = False):
    """Causal depthwise convolution over tokens of ``x [B,S,C]`` (channels last) with ``weight [C,K]``
    (or the ``[C,1,K]`` weight of a depthwise ``nn.Conv1d``), optional SiLU.  ``state [B,K-1,C]``
    holds the inputs before the first token (None = zeros); with ``return_state`` the last K-1
    inputs come back as the state for the next call."""
    _need_cuda(x, weight, bias, state)
    B, S, C = x.shape
    K = weight.shape[-1]
    xc = x.contiguous()
    w = weight.to(xc.dtype).reshape(C, K).contiguous()
    b = None if bias is None else bias.to(xc.dtype).contiguous()
    st_in = None if state is None else state.to(xc.dtype).contiguous()
    st_out = torch.empty(B, K - 1, C, dtype=xc.dtype, device=xc.device) if return_state else None
    y = torch.empty_like(xc)
    _lib.check(_lib.load().xlstm_causal_conv1d(xc.data_ptr(), w.data_ptr(), _ptr(b), _ptr(st_in), _ptr(st_out),
                                               y.data_ptr(), B, S, C, K, int(bool(silu)), _dtype_code(xc), _stream()),
               "xlstm_causal_conv1d")
    return (y, st_out) if return_state else y


LINEAR_TOKEN_MAX_ROWS = 4


def linear_token(weight: torch.Tensor, x: torch.Tensor, bias: Optional[torch.Tensor] = None,
                 norm_weight: Optional[torch.Tensor] = None, norm_eps: float = 1e-6,
                 residual: Optional[torch.Tensor] = None, swiglu_pair: bool = False) -> torch.Tensor:
    """``nn.Linear`` for up to 4 token rows as one weight-streaming pass (bf16).  ``x: [..., K]`` with at
    most 4 rows, ``weight: [N, K]``.  Optional RMSNorm of ``x`` first (``norm_weight``), optional
    ``residual + (...)``, or ``swiglu_pair``: ``weight`` holds gate rows then up rows (``[2F, K]``) and
    the result is ``silu(gate) * up`` of width ``F``."""
    _need_cuda(weight, x, bias, norm_weight, residual)
    if weight.dtype != torch.bfloat16:
        raise TypeError("linear_token is a bf16 kernel")
    K = x.shape[-1]
    x2 = x.reshape(-1, K).to(torch.bfloat16).contiguous()
    M = x2.shape[0]
    if M > LINEAR_TOKEN_MAX_ROWS:
        raise ValueError(f"linear_token takes at most {LINEAR_TOKEN_MAX_ROWS} rows, got {M}")
    w = weight if weight.is_contiguous() else weight.contiguous()
    rows = w.shape[0]
    N = rows // 2 if swiglu_pair else rows
    b = None if bias is None else bias.to(torch.bfloat16).contiguous()
    nw = None if norm_weight is None else norm_weight.to(torch.bfloat16).contiguous()
    r = None if residual is None else residual.reshape(-1, N).to(torch.bfloat16).contiguous()
    y = torch.empty(*x.shape[:-1], N, dtype=torch.bfloat16, device=x.device)
    epi = 2 if swiglu_pair else (1 if r is not None else 0)
    _lib.check(_lib.load().xlstm_linear_token(w.data_ptr(), x2.data_ptr(), _ptr(b), _ptr(nw), float(norm_eps), _ptr(r),
                                              y.data_ptr(), M, N, K, epi, _lib.BF16, _stream()), "xlstm_linear_token")
    return y
