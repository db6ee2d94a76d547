"""Host-fed decode: streams, pinned staging and events around the decode-step kernel.

``DecodePipeline`` is the call a serving loop makes when the per-token activations arrive in
host memory: it copies q,k,v,i,f host -> device as ONE packed transfer, runs the step kernel
through the C ABI, and copies h device -> host, on three streams with double-buffered staging so
the copies of neighbouring steps overlap the kernel.  State (C, n, m) stays resident on the GPU.
With ``group`` > 1 the steps travel in groups: the input copies of a whole group are enqueued ahead of its
kernels and its result copies behind them (still one copy in and one copy out per step), so the kernels of a
group follow one another on their stream with no cross-stream dependency in between - on B200 such a
dependency costs about 3 us per kernel, more than a tenth of a decode step.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch

from . import _lib


class DecodePipeline:
    def __init__(self, B: int, NH: int, dqk: int, dv: int, device, eps: float = 1e-6, depth: int = 2, group: int = 1):
        self.B, self.NH, self.dqk, self.dv, self.eps, self.depth, self.group = B, NH, dqk, dv, eps, depth, group
        self.device = torch.device(device)
        bf = torch.bfloat16
        self.n_in = B * NH * (2 * dqk + dv + 2)           # packed q | k | v | i | f, bf16 elements
        self.stage = [torch.empty(self.n_in, dtype=bf, device=self.device) for _ in range(depth * group)]
        self.h_dev = [torch.empty(B, NH, dv, dtype=bf, device=self.device) for _ in range(depth * group)]
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
        self.step_group([(packed_host, state_in, state_out, h_host, state_settled)])

    def step_group(self, items) -> None:
        """Enqueue up to ``group`` decode steps - each ``(packed_host, state_in, state_out, h_host[, state_settled])`` -
        as one group: all their input copies, then their kernels back to back, then their result copies."""
        if not 1 <= len(items) <= self.group:
            raise ValueError(f"a group holds 1..{self.group} steps, got {len(items)}")
        g = self.t % self.depth
        first_use = self.t < self.depth
        base_slot = g * self.group
        with torch.cuda.stream(self.s_in):
            if not first_use:
                self.s_in.wait_event(self.ev_run[g])      # staging slots free once their kernels ran
            for j, item in enumerate(items):
                self.stage[base_slot + j].copy_(item[0], non_blocking=True)
            self.ev_in[g].record(self.s_in)
        with torch.cuda.stream(self.s_run):
            self.s_run.wait_event(self.ev_in[g])
            if not first_use:
                self.s_run.wait_event(self.ev_out[g])     # h slots drained by their device -> host copies
            for j, item in enumerate(items):
                state_in, state_out = item[1], item[2]
                settled = bool(item[4]) if len(item) > 4 else False
                base = self.stage[base_slot + j].data_ptr()
                st = self.lib.xlstm_mlstm_step_ex(
                    base + self.off[0], base + self.off[1], base + self.off[2], base + self.off[3], base + self.off[4],
                    state_in[0].data_ptr(), state_in[1].data_ptr(), state_in[2].data_ptr(),
                    self.h_dev[base_slot + j].data_ptr(),
                    state_out[0].data_ptr(), state_out[1].data_ptr(), state_out[2].data_ptr(),
                    self.B, self.NH, self.dqk, self.dv, self.eps, 0.0, _lib.STEP_STATE_SETTLED if settled else 0,
                    _lib.BF16, self.s_run.cuda_stream)
                _lib.check(st, "xlstm_mlstm_step_ex")
            self.ev_run[g].record(self.s_run)
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(self.ev_run[g])
            for j, item in enumerate(items):
                item[3].copy_(self.h_dev[base_slot + j], non_blocking=True)
            self.ev_out[g].record(self.s_out)
        self.t += 1

    def capture(self, steps) -> torch.cuda.CUDAGraph:
        """Record a sequence of steps - each ``(packed_host, state_in, state_out, h_host[, state_settled])``,
        taken ``group`` at a time - into one CUDA graph: the copies and kernels keep their three-stream overlap as parallel
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
            steps = list(steps)
            for lo in range(0, len(steps), self.group):
                self.step_group(steps[lo:lo + self.group])
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
