"""Host-side mirror of the reference interface: names, shapes, errors (CPU only, no kernel calls)."""
import json
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

sys.path.insert(0, str(Path(__file__).resolve().parent / "golden"))
from make_golden_model import TINY  # noqa: E402  (config dict only; the reference is not imported)


@pytest.fixture()
def tiny_dir(tmp_path):
    from xlstm_cuda.utils import write_model_dir
    return write_model_dir(tmp_path / "tiny", dict(TINY))


def test_config_and_wiring(tiny_dir):
    from xlstm_cuda.utils import load_config, resolve_dtype
    from xlstm_cuda.wiring import create_auto_wiring
    cfg = load_config(str(tiny_dir))
    assert (cfg["qk_dim"], cfg["v_dim"], cfg["qk_head_dim"], cfg["v_head_dim"]) == (128, 256, 64, 128)
    assert cfg["ffn_hidden_dim"] == 256 and cfg["chunk_size"] == 64
    assert resolve_dtype("bf16") is torch.bfloat16 and resolve_dtype(None) is torch.float32
    assert resolve_dtype("nonsense") is torch.float32
    w = create_auto_wiring(str(tiny_dir), cfg)
    assert w.structure["num_blocks"] == 2 and w.structure["has_lm_head"] and w.structure["has_out_norm"]
    assert [w.get_block_info(i)["type"] for i in range(2)] == ["mlstm", "mlstm"]
    with pytest.raises(FileNotFoundError):
        load_config(str(tiny_dir / "missing"))
    with pytest.raises(FileNotFoundError):
        create_auto_wiring(str(tiny_dir.parent), cfg)


def test_7b_dims_match_the_reference_rounding():
    from xlstm_cuda.blocks import mLSTMBlock
    with torch.device("meta"):
        blk = mLSTMBlock(0)
    assert (blk.qk_dim_per_head, blk.v_dim_per_head, blk.ffn_hidden_dim, blk.hidden_size) == (256, 512, 10944, 4096)


def test_parameter_names_equal_the_reference_modules(tiny_dir, golden):
    """Same module tree as the reference => its safetensors key map and state_dicts apply unchanged."""
    from xlstm_cuda.blocks import sLSTMBlock, sLSTMBlockDiag
    from xlstm_cuda.models import WiredxLSTM
    model = WiredxLSTM.from_pretrained(tiny_dir, load_weights=False, device="cpu")
    assert sorted(n for n, _ in model.named_parameters()) == list(golden("model_tiny_fp32")["param_names"])
    keys = model.blocks[1].get_weight_keys()
    assert keys["mlstm_cell.projection_cell.q_proj.weight"] == "backbone.blocks.1.mlstm_layer.q.weight"
    assert keys["mlstm_cell.output_cell.norm.weight"] == "backbone.blocks.1.mlstm_layer.multihead_norm.weight"
    params = dict(model.blocks[1].named_parameters())
    assert set(keys) == set(params)
    blk = sLSTMBlock(0, embedding_dim=64, num_heads=4, head_dim=16, ffn_proj_factor=1.0)
    assert sorted(n for n, _ in blk.named_parameters()) == list(golden("slstm_block_fp32")["param_names"])
    assert set(blk.get_weight_keys()) <= set(dict(blk.named_parameters()))

    class Cfg:
        inp_dim, head_dim, head_num, p_factor, norm_eps, gate_soft_cap = 64, 32, 4, (2.0, 4 / 3), 1e-6, 15.0
    bd = sLSTMBlockDiag(Cfg())
    assert sorted(n for n, _ in bd.named_parameters()) == list(golden("slstm_blockdiag_fp32")["param_names"])


def test_error_behaviour_matches_the_reference():
    from xlstm_cuda.blocks import SoftCapCell, mLSTMNeuron, soft_cap
    with pytest.raises(ValueError):
        mLSTMNeuron(64, 2, 32, 32, kernel_mode="quadratic")
    x = torch.ones(3)
    assert soft_cap(x, 0.0) is x and soft_cap(x, None) is x and SoftCapCell(-1.0)(x) is x
    with pytest.raises(RuntimeError):  # accelerator required, no CPU fallback
        soft_cap(x, 15.0)
    from xlstm_cuda.blocks import MultiHeadRMSNorm
    with pytest.raises(ValueError):
        MultiHeadRMSNorm(2, 8)(torch.zeros(1, 1, 3, 8))


def test_norm_cells_need_the_accelerator():
    """The norm cells run kernels; like every kernel-backed cell they refuse CPU tensors (the parity
    test against the reference's fixtures is in the GPU suite)."""
    from xlstm_cuda.blocks import MultiHeadRMSNorm, RMSNormCell
    with pytest.raises(RuntimeError):
        RMSNormCell(96)(torch.zeros(2, 96))
    with pytest.raises(RuntimeError):
        MultiHeadRMSNorm(4, 32)(torch.zeros(1, 2, 4, 32))


def test_runner_prompt_rules(tiny_dir):
    from xlstm_cuda.generate import xLSTMRunner
    cfg = json.loads((tiny_dir / "config.json").read_text())
    cfg["force_bos_token_insert"] = True
    (tiny_dir / "config.json").write_text(json.dumps(cfg))
    r = xLSTMRunner(str(tiny_dir), device="cpu")
    assert r._prepare_prompt([5, 6]) == [0, 5, 6] and r._prepare_prompt([0, 5]) == [0, 5]
    assert r._prepare_prompt(None) == [0] and r._prepare_prompt(torch.tensor([7])) == [0, 7]
    info = r.get_model_info()
    assert info["block_types"] == ["mlstm", "mlstm"] and info["qk_dim"] == 128 and info["total_blocks"] == 2
    with pytest.raises(ValueError):
        r.generate("text prompt needs a tokenizer")
    with pytest.raises(ValueError):
        xLSTMRunner.from_pretrained("no/such/model")
