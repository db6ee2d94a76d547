"""Two-GPU test of the fused all-gather: the chunkwise kernel writes h into the peer's buffer itself.

Runs as two child processes (one per GPU, NCCL over 127.0.0.1); skipped on a single-GPU box.
The gathered h must equal, bit for bit, what each rank computes for its own heads, and the fused path
must equal the NCCL all-gather path.  The same ranks then run a whole model with head-sharded mLSTM layers
against the unsharded model.
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
    # token-sharded variant: every rank receives all heads of ITS token range only and projects those
    scatter = parallel.FusedHeadScatter(B, S, NH, dv, bf, dev)
    for _ in range(2):
        y_tok, _ = scatter.run(sl(q), sl(k), sl(v), sl(i), sl(f), None, out_proj=w)
        tok = S // world
        ok = ok and torch.equal(scatter.buf, ref[:, rank * tok:(rank + 1) * tok])
        ok = ok and torch.equal(y_tok, ref[:, rank * tok:(rank + 1) * tok].reshape(B, tok, NH * dv) @ w)
    # model level: every mLSTM layer head-sharded over the two ranks (sliced checkpoint load, local norm x gate,
    # all-gather of the gated heads, replicated out-projection) against the unsharded model on the same GPU
    sys.path.insert(0, str(ROOT / "tests" / "golden"))
    from make_golden_model import TINY
    from param_init import fill_parameters
    from xlstm_cuda.models import WiredxLSTM
    from xlstm_cuda.utils import write_model_dir
    d = write_model_dir(Path(tmp) / f"tiny{rank}", dict(TINY))
    full = WiredxLSTM.from_pretrained(d, load_weights=False, device=dev)
    fill_parameters(dict(full.named_parameters()), seed=21)
    ckpt = {"backbone.embeddings.weight": full.embedding.weight, "backbone.out_norm.weight": full.out_norm.weight,
            "lm_head.weight": full.lm_head.weight}
    for blk in full.blocks:
        params = dict(blk.named_parameters())
        ckpt.update({key: params[path] for path, key in blk.get_weight_keys().items()})
    sharded = WiredxLSTM.from_pretrained(d, load_weights=False, device=dev, head_shard=(rank, world))
    sharded._load_weights_from_dict({k_: v_.detach() for k_, v_ in ckpt.items()})
    ids = torch.randint(0, TINY["vocab_size"], (2, 70), generator=torch.Generator().manual_seed(5))
    with torch.inference_mode():
        want, st_full = full(ids, None, return_last_states=True)
        got, st_loc = sharded(ids, None, return_last_states=True)
        nxt, _ = sharded(ids[:, :1], st_loc, return_last_states=True)      # a decode step carrying the sharded state
        nxt_ref, _ = full(ids[:, :1], st_full, return_last_states=True)
    rel = lambda a, b: float((a.float() - b.float()).abs().max() / b.float().abs().max())
    lo, hi = parallel.head_range(TINY["num_heads"], world, rank)
    ok = ok and rel(got, want) < 1e-4 and rel(nxt, nxt_ref) < 1e-4
    ok = ok and all(rel(a[0], b[0][:, lo:hi]) < 1e-4 for a, b in zip(st_loc, st_full))
    torch.cuda.synchronize()
    Path(tmp, f"ok{rank}").write_text("1" if ok else "0")
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_fused_head_gather_two_gpus(tmp_path):
    import torch.multiprocessing as mp
    port = 29600 + os.getpid() % 2000
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert [Path(tmp_path, f"ok{r}").read_text() for r in range(2)] == ["1", "1"]
