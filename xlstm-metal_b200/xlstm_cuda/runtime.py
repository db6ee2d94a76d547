"""Host-fed decode: streams, pinned staging and events around the decode-step kernel.

``DecodePipeline`` is the call a serving loop makes when the per-token activations arrive in
host memory: it copies q,k,v,i,f host -> device as ONE packed transfer, runs the step kernel
through the C ABI, and copies h device -> host, on three streams with double-buffered staging so
the copies of neighbouring steps overlap the kernel.  State (C, n, m) stays resident on the GPU.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch

from . import _lib


class DecodePipeline:
    def __init__(self, B: int, NH: int, dqk: int, dv: int, device, eps: float = 1e-6, depth: int = 2):
        self.B, self.NH, self.dqk, self.dv, self.eps, self.depth = B, NH, dqk, dv, eps, depth
        self.device = torch.device(device)
        bf = torch.bfloat16
        self.n_in = B * NH * (2 * dqk + dv + 2)           # packed q | k | v | i | f, bf16 elements
        self.stage = [torch.empty(self.n_in, dtype=bf, device=self.device) for _ in range(depth)]
        self.h_dev = [torch.empty(B, NH, dv, dtype=bf, device=self.device) for _ in range(depth)]
        self.s_in, self.s_run, self.s_out = (torch.cuda.Stream(self.device) for _ in range(3))
        self.ev_in = [torch.cuda.Event() for _ in range(depth)]
        self.ev_run = [torch.cuda.Event() for _ in range(depth)]
        self.ev_out = [torch.cuda.Event() for _ in range(depth)]
        self.t = 0
        self.lib = _lib.load()
        o = 0
        self.off = []
        for nelem in (B * NH * dqk, B * NH * dqk, B * NH * dv, B * NH, B * NH):
            self.off.append(o * 2)  # byte offsets inside the packed buffer
            o += nelem

    def pack(self, q, k, v, i, f, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Pack host tensors into one pinned bf16 buffer (done once per step by the producer)."""
        buf = out if out is not None else torch.empty(self.n_in, dtype=torch.bfloat16).pin_memory()
        torch.cat([t.reshape(-1).to(torch.bfloat16) for t in (q, k, v, i, f)], out=buf)
        return buf

    def step(self, packed_host: torch.Tensor, state_in: Tuple[torch.Tensor, ...],
             state_out: Tuple[torch.Tensor, ...], h_host: torch.Tensor, state_settled: bool = False) -> None:
        """Enqueue one decode step.  ``packed_host`` and ``h_host`` are pinned host tensors;
        ``state_in`` / ``state_out`` are (C, n, m) fp32 device tensors (different buffers).
        ``state_settled``: ``state_in`` was not written by the step enqueued just before this one (a stack of
        layers), so the kernel may start streaming it while that step drains."""
        s = self.t % self.depth
        first_use = self.t < self.depth
        with torch.cuda.stream(self.s_in):
            if not first_use:
                self.s_in.wait_event(self.ev_run[s])      # staging slot free once its kernel ran
            self.stage[s].copy_(packed_host, non_blocking=True)
            self.ev_in[s].record(self.s_in)
        with torch.cuda.stream(self.s_run):
            self.s_run.wait_event(self.ev_in[s])
            if not first_use:
                self.s_run.wait_event(self.ev_out[s])     # h slot drained by its device -> host copy
            base = self.stage[s].data_ptr()
            st = self.lib.xlstm_mlstm_step_ex(
                base + self.off[0], base + self.off[1], base + self.off[2], base + self.off[3], base + self.off[4],
                state_in[0].data_ptr(), state_in[1].data_ptr(), state_in[2].data_ptr(), self.h_dev[s].data_ptr(),
                state_out[0].data_ptr(), state_out[1].data_ptr(), state_out[2].data_ptr(),
                self.B, self.NH, self.dqk, self.dv, self.eps, 0.0, _lib.STEP_STATE_SETTLED if state_settled else 0,
                _lib.BF16, self.s_run.cuda_stream)
            _lib.check(st, "xlstm_mlstm_step_ex")
            self.ev_run[s].record(self.s_run)
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(self.ev_run[s])
            h_host.copy_(self.h_dev[s], non_blocking=True)
            self.ev_out[s].record(self.s_out)
        self.t += 1

    def capture(self, steps) -> torch.cuda.CUDAGraph:
        """Record a sequence of ``step`` calls - each ``(packed_host, state_in, state_out, h_host)`` -
        into one CUDA graph: the copies and kernels keep their three-stream overlap as parallel
        branches of the graph, and a replay costs one launch instead of ~10 Python-side calls per
        step.  The producer refills the SAME pinned buffers between replays.  Replay on any stream
        with ``graph.replay()``."""
        graph = torch.cuda.CUDAGraph()
        self.t = 0
        with torch.cuda.graph(graph, stream=self.s_run, capture_error_mode="relaxed"):
            fork = torch.cuda.Event()
            fork.record(self.s_run)
            self.s_in.wait_event(fork)
            self.s_out.wait_event(fork)
            for item in steps:
                self.step(*item)   # (packed_host, state_in, state_out, h_host[, state_settled])
            for side in (self.s_in, self.s_out):
                join = torch.cuda.Event()
                join.record(side)
                self.s_run.wait_event(join)
        self.t = 0
        return graph

    def streams(self) -> List[torch.cuda.Stream]:
        return [self.s_in, self.s_run, self.s_out]

    def synchronize(self) -> None:
        for s in self.streams():
            s.synchronize()
