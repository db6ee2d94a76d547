"""Checkpoint loading through the reference's key map: safetensors shards written here with the
NX-AI key names (mlstm_block.py:215-231, slstm_block.py:171) are read back by
``load_safetensor_shards`` / ``WiredxLSTM(load_weights=True)`` and land in the parameters the map
names, shard boundaries and dtype casts included.  CPU only: nothing is run forward."""
import json
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

sys.path.insert(0, str(Path(__file__).resolve().parent / "golden"))
from make_golden_model import TINY  # noqa: E402

safetensors_torch = pytest.importorskip("safetensors.torch")


def _checkpoint(tmp_path, block_types, dtype=torch.float32, seed=3):
    """A randomly filled model -> its tensors under checkpoint key names, split over two shards."""
    from xlstm_cuda.models import WiredxLSTM
    from xlstm_cuda.utils import write_model_dir
    cfg = dict(TINY, num_blocks=len(block_types))
    d = write_model_dir(tmp_path / "src", cfg, block_types=block_types)
    src = WiredxLSTM.from_pretrained(d, load_weights=False, device="cpu")
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for p in src.parameters():
            p.copy_(torch.randn(p.shape, generator=g))
    tensors = {"backbone.embeddings.weight": src.embedding.weight, "backbone.out_norm.weight": src.out_norm.weight,
               "lm_head.weight": src.lm_head.weight}
    for blk in src.blocks:
        params = dict(blk.named_parameters())
        for path, key in blk.get_weight_keys().items():
            assert path in params, f"key map names a parameter the block does not have: {path}"
            tensors[key] = params[path]
    tensors = {k: v.detach().to(dtype).contiguous().clone() for k, v in tensors.items()}
    out = tmp_path / "ckpt"
    out.mkdir()
    (out / "config.json").write_text(json.dumps(cfg))
    keys = sorted(tensors)
    half = len(keys) // 2
    shards = {"model-00001-of-00002.safetensors": keys[:half], "model-00002-of-00002.safetensors": keys[half:]}
    for name, ks in shards.items():
        safetensors_torch.save_file({k: tensors[k] for k in ks}, str(out / name))
    (out / "model.safetensors.index.json").write_text(
        json.dumps({"weight_map": {k: name for name, ks in shards.items() for k in ks}}))
    return src, tensors, out


@pytest.mark.parametrize("block_types", [["mlstm", "mlstm"], ["mlstm", "slstm", "mlstm"]])
def test_shards_land_in_the_named_parameters(tmp_path, block_types):
    from xlstm_cuda.models import WiredxLSTM
    from xlstm_cuda.utils import load_safetensor_shards
    src, tensors, ckpt = _checkpoint(tmp_path, block_types)
    loaded = load_safetensor_shards(str(ckpt))
    assert sorted(loaded) == sorted(tensors)
    model = WiredxLSTM.from_pretrained(ckpt, load_weights=True, device="cpu")
    assert [type(b).__name__ for b in model.blocks] == [type(b).__name__ for b in src.blocks]
    mapped = 0
    for (n1, p1), (n2, p2) in zip(src.named_parameters(), model.named_parameters()):
        assert n1 == n2
        if torch.equal(p1, p2):
            mapped += 1
    # every parameter the key map covers arrived bit for bit; what the map does not cover keeps its
    # own initialisation (sLSTM conv / gate biases the NX-AI checkpoint has no tensors for)
    covered = 3 + sum(len(b.get_weight_keys()) for b in src.blocks)
    assert mapped >= covered


def test_bf16_checkpoint_casts_to_the_compute_dtype_and_survives_fusion(tmp_path):
    from xlstm_cuda.models import WiredxLSTM
    src, tensors, ckpt = _checkpoint(tmp_path, ["mlstm", "mlstm"], dtype=torch.bfloat16)
    model = WiredxLSTM.from_pretrained(ckpt, load_weights=True, device="cpu")
    q = model.blocks[0].mlstm_cell.projection_cell.q_proj.weight
    assert q.dtype == torch.float32   # TINY runs fp32 kernels; the shard was bf16
    np.testing.assert_array_equal(q.detach().numpy(),
                                  tensors["backbone.blocks.0.mlstm_layer.q.weight"].float().numpy())
    # fusing the projections afterwards keeps names and values, and a second load still lands
    before = {k: v.clone() for k, v in model.state_dict().items()}
    assert model.fuse_projections() == 2
    after = model.state_dict()
    assert list(after) == list(before) and all(torch.equal(before[k], after[k]) for k in before)
    model.load_pretrained_weights()
    assert model.blocks[1].mlstm_cell._fused_weights() is not None
    assert all(torch.equal(before[k], v) for k, v in model.state_dict().items())


def test_missing_shards_raise(tmp_path):
    from xlstm_cuda.utils import load_safetensor_shards
    with pytest.raises(FileNotFoundError):
        load_safetensor_shards(str(tmp_path))


def test_infer_config_from_safetensors_reads_shapes_of_all_shards(tmp_path):
    """Follows xlstm_metal/torch_native/utils/infer_config_from_safetensors.py:30-103 on a two-shard checkpoint
    whose block-0 tensors sit in both shards; no config.json is consulted."""
    from xlstm_cuda.utils import infer_config_from_safetensors
    src, tensors, ckpt = _checkpoint(tmp_path, ["mlstm", "mlstm"])
    (ckpt / "config.json").unlink()
    cfg = infer_config_from_safetensors(str(ckpt))
    assert cfg["embedding_dim"] == TINY["embedding_dim"] and cfg["vocab_size"] == TINY["vocab_size"]
    assert cfg["num_blocks"] == 2 and cfg["num_heads"] == TINY["num_heads"]
    assert cfg["qk_dim_factor"] == pytest.approx(TINY["qk_dim_factor"]) and cfg["v_dim_factor"] == 1.0
    assert cfg["ffn_proj_factor"] * TINY["embedding_dim"] == src.blocks[0].ffn_hidden_dim
    assert cfg["gate_soft_cap"] == 15.0 and cfg["output_logit_soft_cap"] == 30.0 and cfg["chunk_size"] == 64
    assert cfg["use_bias"] is True and cfg["norm_eps"] == 1e-6
    with pytest.raises(FileNotFoundError):
        infer_config_from_safetensors(str(tmp_path))
    # a required tensor missing from the index -> ValueError, as in the reference
    idx = json.loads((ckpt / "model.safetensors.index.json").read_text())
    del idx["weight_map"]["lm_head.weight"]
    (ckpt / "model.safetensors.index.json").write_text(json.dumps(idx))
    with pytest.raises(ValueError):
        infer_config_from_safetensors(str(ckpt))


def test_head_sharded_model_loads_its_row_slices(tmp_path):
    """head_shard=(rank, world): every mLSTM layer keeps the rows of q/k/v/igate/fgate/ogate and of the per-head
    norm weight that belong to its heads (key map: xlstm_metal/torch_native/blocks/mlstm/mlstm_block.py:215-231);
    everything else, the out-projection included, is the full tensor."""
    from xlstm_cuda.models import WiredxLSTM
    src, tensors, ckpt = _checkpoint(tmp_path, ["mlstm", "slstm", "mlstm"])
    NH = TINY["num_heads"]
    full = dict(src.named_parameters())
    for rank in range(NH):
        m = WiredxLSTM.from_pretrained(ckpt, load_weights=True, device="cpu", head_shard=(rank, NH))
        cell = m.blocks[0].mlstm_cell
        dqk, dv = cell.qk_dim_per_head, cell.v_dim_per_head
        assert cell.num_heads == 1 and cell.projection_cell.q_proj.out_features == dqk
        rows = {"q_proj.weight": dqk, "k_proj.weight": dqk, "v_proj.weight": dv, "igate_proj.weight": 1, "igate_proj.bias": 1,
                "fgate_proj.weight": 1, "fgate_proj.bias": 1}
        for name, per in rows.items():
            want = full[f"blocks.0.mlstm_cell.projection_cell.{name}"][rank * per:(rank + 1) * per]
            assert torch.equal(dict(m.named_parameters())[f"blocks.0.mlstm_cell.projection_cell.{name}"], want), name
        mine = dict(m.named_parameters())
        for name in ("ogate_proj.weight", "norm.weight"):
            want = full[f"blocks.2.mlstm_cell.output_cell.{name}"][rank * dv:(rank + 1) * dv]
            assert torch.equal(mine[f"blocks.2.mlstm_cell.output_cell.{name}"], want), name
        for name in ("blocks.0.mlstm_cell.output_cell.out_proj.weight", "blocks.0.ffn_proj_down.weight", "lm_head.weight",
                     "blocks.0.norm_mlstm.weight"):
            assert torch.equal(mine[name], full[name]), name
        assert not m.blocks[0]._token_step_ok(torch.zeros(1, 1, TINY["embedding_dim"], dtype=torch.bfloat16))
    with pytest.raises(ValueError):
        WiredxLSTM.from_pretrained(ckpt, load_weights=False, device="cpu", head_shard=(0, 3))
