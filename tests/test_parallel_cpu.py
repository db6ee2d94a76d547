"""Multi-rank host logic on CPU: two gloo ranks shard heads, all-gather h, apply the out-projection.

The cell here is the CPU oracle (this is a test of the sharding and the collective, not of a
kernel); the result must equal the single-rank computation exactly.
"""
import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _oracle_cell(q, k, v, i, f, state):
    from oracle import oracle as xo
    st = None if state is None else tuple(s.numpy() for s in state)
    h, new = xo.mlstm_chunkwise(q.numpy(), k.numpy(), v.numpy(), i.numpy(), f.numpy(), st, chunk_size=16)
    return torch.from_numpy(h), tuple(torch.from_numpy(s) for s in new)


def _worker(rank, world, port, tmp):
    for p in (ROOT, ROOT / "xlstm-metal_b200"):
        sys.path.insert(0, str(p))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from xlstm_cuda import parallel
    g = torch.Generator().manual_seed(0)
    B, NH, S, dqk, dv, D = 2, 4, 32, 16, 32, 24
    q, k = torch.randn(B, NH, S, dqk, generator=g), torch.randn(B, NH, S, dqk, generator=g)
    v = torch.randn(B, NH, S, dv, generator=g)
    i, f = torch.randn(B, NH, S, generator=g), torch.randn(B, NH, S, generator=g) + 3
    w = torch.randn(NH * dv, D, generator=g)
    state = (torch.randn(B, NH, dqk, dv, generator=g), torch.randn(B, NH, dqk, generator=g), torch.randn(B, NH, generator=g))
    y, st_local = parallel.head_sharded_prefill(_oracle_cell, q, k, v, i, f, state, out_proj=w)
    h_full, st_full = _oracle_cell(q, k, v, i, f, state)
    y_ref = h_full.permute(0, 2, 1, 3).reshape(B, S, NH * dv) @ w
    lo, hi = parallel.head_range(NH, world, rank)
    ok = torch.allclose(y, y_ref, rtol=1e-5, atol=1e-5) and torch.allclose(st_local[0], st_full[0][:, lo:hi], atol=1e-6)
    ok = ok and st_local[2].shape == (B, NH // world)
    # gather along the feature dimension (gated head outputs before the replicated out-projection)
    feats = torch.arange(B * S * NH * dv, dtype=torch.float32).reshape(B, S, NH * dv)
    per = NH * dv // world
    got = parallel.all_gather_features(feats[..., rank * per:(rank + 1) * per])
    ok = ok and torch.equal(got, feats)
    Path(tmp, f"ok{rank}").write_text("1" if ok else "0")
    dist.destroy_process_group()


def test_two_gloo_ranks_head_sharded_prefill(tmp_path):
    port = 29500 + os.getpid() % 2000
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert [Path(tmp_path, f"ok{r}").read_text() for r in range(2)] == ["1", "1"]


def test_ranges():
    from xlstm_cuda import parallel
    assert [parallel.head_range(8, 4, r) for r in range(4)] == [(0, 2), (2, 4), (4, 6), (6, 8)]
    assert [parallel.batch_range(10, 4, r) for r in range(4)] == [(0, 3), (3, 6), (6, 8), (8, 10)]
    assert parallel.batch_range(2, 4, 3) == (2, 2)
    with pytest.raises(ValueError):
        parallel.head_range(8, 3, 0)
    with pytest.raises(ValueError):
        parallel.batch_range(4, 2, 2)
    t = torch.arange(2 * 8 * 3).reshape(2, 8, 3)
    assert parallel.shard_heads(t, 2, 1).shape == (2, 4, 3) and parallel.shard_heads(t, 2, 1)[0, 0, 0] == 12
    assert parallel.all_gather_heads(t) is t  # no process group: single rank
