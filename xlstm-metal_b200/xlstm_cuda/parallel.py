"""Sharding of the hot path over the GPUs of one box (one process per GPU, torch.distributed).

mLSTM heads are independent (no cross-head term in the cell), so a layer shards by heads: rank r
owns heads ``[r*NH/G, (r+1)*NH/G)`` - its column slices of the q/k/v/gate projections and its
heads' (C, n, m) - and ONE all-gather of h precedes the replicated out-projection.  Decode batches
and the sLSTM stack shard by batch with no collective at all.  The backend is NCCL on GPUs and
gloo in the CPU tests.  No kernel ever LOADS from a peer's memory: remote data arrives either
through the collective or, in the fused head gather, by TMA tile stores that the prefill kernel of
the owning rank issues into every peer's buffer.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist


def head_range(num_heads: int, world: int, rank: int) -> Tuple[int, int]:
    """Heads owned by ``rank``; ``num_heads`` must divide evenly (NH = 8 gives G in 1, 2, 4, 8)."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank/world {rank}/{world}")
    if num_heads % world:
        raise ValueError(f"{num_heads} heads do not shard over {world} ranks")
    per = num_heads // world
    return rank * per, (rank + 1) * per


def batch_range(batch: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous batch rows owned by ``rank`` (sizes differ by at most one row)."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank/world {rank}/{world}")
    base, extra = divmod(batch, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard_heads(t: torch.Tensor, world: int, rank: int, dim: int = 1) -> torch.Tensor:
    """Slice of a ``[B, NH, ...]`` tensor (or a state tensor) holding this rank's heads."""
    lo, hi = head_range(t.shape[dim], world, rank)
    return t.narrow(dim, lo, hi - lo)


def all_gather_heads(h_local: torch.Tensor, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """``[B, NH/G, S, dv]`` on every rank -> ``[B, NH, S, dv]`` on every rank, one collective."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return h_local
    h_local = h_local.contiguous()
    B, nh, S, dv = h_local.shape
    gathered = torch.empty((world * B, nh, S, dv), dtype=h_local.dtype, device=h_local.device)  # rank-major
    dist.all_gather_into_tensor(gathered, h_local, group=group)
    return gathered.view(world, B, nh, S, dv).permute(1, 0, 2, 3, 4).reshape(B, world * nh, S, dv)


def all_gather_features(x_local: torch.Tensor, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """``[..., F/G]`` on every rank -> ``[..., F]`` on every rank (rank r's slice is block r of the last
    dimension): the gather of the gated per-head outputs before the replicated out-projection."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return x_local
    x_local = x_local.contiguous()
    shape = tuple(x_local.shape)
    gathered = torch.empty((world * shape[0],) + shape[1:], dtype=x_local.dtype, device=x_local.device)  # rank-major
    dist.all_gather_into_tensor(gathered, x_local, group=group)
    return torch.cat(list(gathered.view((world,) + shape).unbind(0)), dim=-1)


def head_sharded_prefill(cell: Callable, q, k, v, i, f, state=None, out_proj: Optional[torch.Tensor] = None,
                         group: Optional[dist.ProcessGroup] = None):
    """Run ``cell(q, k, v, i, f, state) -> (h, state)`` on this rank's heads, all-gather h, and apply
    the replicated out-projection ``[NH*dv, D]`` if given.  Inputs are the FULL tensors; each rank
    slices its heads.  Returns ``(y or h_full, local_state)``."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    sl = lambda t: shard_heads(t, world, rank)
    st = None if state is None else tuple(sl(s) for s in state)
    h_local, st_local = cell(sl(q), sl(k), sl(v), sl(i), sl(f), st)
    h = all_gather_heads(h_local, group)
    if out_proj is None:
        return h, st_local
    B, NH, S, dv = h.shape
    return h.permute(0, 2, 1, 3).reshape(B, S, NH * dv) @ out_proj, st_local


class FusedHeadGather:
    """Head-sharded chunkwise prefill whose all-gather is done by the kernel itself.

    Every rank owns a ``[B, S, NH, dv]`` buffer in symmetric memory (the layout the out-projection
    GEMM reads, so no permute is needed afterwards).  The chunkwise kernel of rank r writes each h
    tile of its heads into its own buffer AND, by TMA tile stores over NVLink, into the same slot of
    every peer's buffer while the tensor cores work on the next tile; one cross-rank barrier later
    every rank holds all heads.  No NCCL call and no extra pass over h.
    """

    def __init__(self, B: int, S: int, NH: int, dv: int, dtype: torch.dtype, device, group=None):
        self.B, self.S, self.NH, self.dv = B, S, NH, dv
        self.group = group if group is not None else (dist.group.WORLD if dist.is_initialized() else None)
        self.world = dist.get_world_size(self.group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(self.group) if dist.is_initialized() else 0
        self.lo, self.hi = head_range(NH, self.world, self.rank)
        self.handle = None
        if self.world > 1:
            import torch.distributed._symmetric_memory as symm_mem
            self.buf = symm_mem.empty(B, S, NH, dv, dtype=dtype, device=device)
            self.handle = symm_mem.rendezvous(self.buf, self.group)
            esz = self.buf.element_size()
            slot = self.lo * dv * esz   # byte offset of this rank's first head inside any rank's buffer
            self.peer_ptrs = [int(ptr) + slot for r, ptr in enumerate(self.handle.buffer_ptrs) if r != self.rank]
        else:
            self.buf = torch.empty(B, S, NH, dv, dtype=dtype, device=device)
            self.peer_ptrs = []
        self.h_view = self.buf[:, :, self.lo:self.hi, :].permute(0, 2, 1, 3)   # [B, NH/G, S, dv] strided

    def barrier(self) -> None:
        if self.handle is not None:
            self.handle.barrier()

    def run(self, q, k, v, i, f, state=None, out_proj: Optional[torch.Tensor] = None, workspace=None):
        """q, k, v, i, f hold THIS rank's heads (``[B, NH/G, S, d]``).  Returns ``(y or h_all, state)``
        where ``h_all`` is the ``[B, S, NH*dv]`` buffer complete on every rank."""
        from . import ops
        self.barrier()   # peers are done reading the previous contents of their buffers
        _, st = ops.mlstm_chunkwise(q, k, v, i, f, state, workspace=workspace, h_out=self.h_view,
                                    h_peer_ptrs=self.peer_ptrs)
        self.barrier()   # every rank's kernel has finished: all slots of all buffers are written
        h_all = self.buf.view(self.B, self.S, self.NH * self.dv)
        return (h_all if out_proj is None else h_all @ out_proj), st


class FusedHeadScatter:
    """Head-sharded chunkwise prefill with a TOKEN-sharded result: every rank ends up with all heads of
    ``S / world`` tokens and runs ``1 / world`` of the out-projection.

    Every rank owns a ``[B, S/world, NH, dv]`` buffer in symmetric memory.  The chunkwise kernel of rank r sends each
    h tile of its heads, by a TMA tile store, only to the rank that owns the tile's tokens (its own buffer for its
    own token range): ``(world-1)/world`` of h crosses NVLink once, where the all-gather layout of
    ``FusedHeadGather`` sends ``world-1`` copies and then repeats the full out-projection on every rank.  The
    output ``[B, S/world, D]`` is the token slice of this rank, which is what the per-token residual, norm and
    FFN that follow need.
    """

    def __init__(self, B: int, S: int, NH: int, dv: int, dtype: torch.dtype, device, group=None):
        self.group = group if group is not None else (dist.group.WORLD if dist.is_initialized() else None)
        self.world = dist.get_world_size(self.group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(self.group) if dist.is_initialized() else 0
        if S % (128 * self.world):
            raise ValueError("S must be a multiple of 128 * world for the token-sharded layout")
        self.B, self.S, self.NH, self.dv, self.tok = B, S, NH, dv, S // self.world
        self.lo, self.hi = head_range(NH, self.world, self.rank)
        self.handle = None
        if self.world > 1:
            import torch.distributed._symmetric_memory as symm_mem
            self.buf = symm_mem.empty(B, self.tok, NH, dv, dtype=dtype, device=device)
            self.handle = symm_mem.rendezvous(self.buf, self.group)
            ptrs = [int(x) for x in self.handle.buffer_ptrs]
        else:
            self.buf = torch.empty(B, self.tok, NH, dv, dtype=dtype, device=device)
            ptrs = [self.buf.data_ptr()]
        slot = self.lo * dv * self.buf.element_size()   # this rank's first head inside any rank's buffer
        self.rank_ptrs = [ptr + slot for ptr in ptrs]
        self.h_strides = [self.tok * NH * dv, dv, NH * dv]   # (batch, head, token) element strides of the buffers

    def barrier(self) -> None:
        if self.handle is not None:
            self.handle.barrier()

    def run(self, q, k, v, i, f, state=None, out_proj: Optional[torch.Tensor] = None, workspace=None):
        """q, k, v, i, f hold THIS rank's heads.  Returns ``(y or h, state)`` for this rank's tokens
        ``[rank*S/world, (rank+1)*S/world)``: ``[B, S/world, D]`` or ``[B, S/world, NH*dv]``."""
        from . import ops
        self.barrier()   # peers are done reading the previous contents of their buffers
        st = ops.mlstm_chunkwise_scatter(q, k, v, i, f, state, self.rank_ptrs, self.tok, self.h_strides, workspace=workspace)
        self.barrier()   # every rank's kernel has finished: all head slots of this rank's tokens are written
        h_tok = self.buf.view(self.B, self.tok, self.NH * self.dv)
        return (h_tok if out_proj is None else h_tok @ out_proj), st


__all__ = ["head_range", "batch_range", "shard_heads", "all_gather_heads", "all_gather_features", "head_sharded_prefill",
           "FusedHeadGather", "FusedHeadScatter"]
