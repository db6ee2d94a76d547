"""Two-GPU test of the fused all-gather: the chunkwise kernel writes h into the peer's buffer itself.

Runs as two child processes (one per GPU, NCCL over 127.0.0.1); skipped on a single-GPU box.
The gathered h must equal, bit for bit, what each rank computes for its own heads, and the fused path
must equal the NCCL all-gather path.
"""
import os
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _worker(rank, world, port, tmp):
    for p in (ROOT, ROOT / "xlstm-metal_b200"):
        sys.path.insert(0, str(p))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from xlstm_cuda import ops, parallel
    B, NH, S, dqk, dv = 2, 4, 512, 256, 256
    g = torch.Generator().manual_seed(0)   # same full tensors on every rank
    bf = torch.bfloat16
    q = torch.randn(B, NH, S, dqk, generator=g).to(bf).to(dev)
    k = torch.randn(B, NH, S, dqk, generator=g).to(bf).to(dev)
    v = torch.randn(B, NH, S, dv, generator=g).to(bf).to(dev)
    i = torch.randn(B, NH, S, generator=g).to(bf).to(dev)
    f = (torch.randn(B, NH, S, generator=g) + 3).to(bf).to(dev)
    w = (torch.randn(NH * dv, 64, generator=g) * 0.05).to(bf).to(dev)
    sl = lambda t: parallel.shard_heads(t, world, rank).contiguous()
    fused = parallel.FusedHeadGather(B, S, NH, dv, bf, dev)
    ok = True
    for _ in range(2):   # twice: the second round overwrites buffers the peer has just read
        y, st = fused.run(sl(q), sl(k), sl(v), sl(i), sl(f), None, out_proj=w)
        h_all = fused.buf.clone()
        h_full, _ = ops.mlstm_chunkwise(q, k, v, i, f)           # all heads on this GPU
        ref = h_full.permute(0, 2, 1, 3).contiguous()            # [B,S,NH,dv]
        ok = ok and torch.equal(h_all, ref)
        y_ref, _ = parallel.head_sharded_prefill(lambda *a: ops.mlstm_chunkwise(*a), q, k, v, i, f, None, out_proj=w)
        ok = ok and torch.allclose(y.float(), y_ref.float(), rtol=1e-2, atol=1e-2)
    torch.cuda.synchronize()
    Path(tmp, f"ok{rank}").write_text("1" if ok else "0")
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_fused_head_gather_two_gpus(tmp_path):
    import torch.multiprocessing as mp
    port = 29600 + os.getpid() % 2000
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert [Path(tmp_path, f"ok{r}").read_text() for r in range(2)] == ["1", "1"]
