"""Config, dtype and checkpoint helpers (plain dict configs, as in the reference torch backend).

``load_config``      xlstm_metal/torch_native/utils/config_loader.py:23-72 (derived dims, defaults)
``resolve_dtype``    xlstm_metal/torch_native/utils/dtype_utils.py:9-31
``load_safetensor_shards``  xlstm_metal/torch_native/utils/safetensors_torch_loader.py:11-45
``infer_config_from_safetensors``  xlstm_metal/torch_native/utils/infer_config_from_safetensors.py:30-103
``write_model_dir``  new: writes ``config.json`` plus a keys-only ``model.safetensors.index.json`` so a
                     random-init model can go through the unchanged wiring / ``from_pretrained`` API
                     (the wiring reads block types from that index: wiring/auto_wiring.py:37-70).
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Dict, Optional

import torch

_DTYPE_MAP = {
    "float32": torch.float32, "float": torch.float32, "fp32": torch.float32,
    "float16": torch.float16, "fp16": torch.float16, "half": torch.float16,
    "bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "int32": torch.int32, "int64": torch.int64,
}


def resolve_dtype(name: Optional[str], default: str = "float32") -> torch.dtype:
    key = (name or default).lower()
    return _DTYPE_MAP.get(key, _DTYPE_MAP[default])


def _round_up(value: int, multiple_of: int) -> int:
    return value if multiple_of <= 0 else ((value + multiple_of - 1) // multiple_of) * multiple_of


def load_config(model_path: str) -> Dict[str, Any]:
    path = Path(model_path)
    if path.is_dir():
        path = path / "config.json"
    if not path.exists():
        raise FileNotFoundError(f"Config file not found: {path}")
    config = json.loads(path.read_text())
    d = config["embedding_dim"]
    mult = config.get("mlstm_round_up_to_multiple_of", 64)
    config["qk_dim"] = _round_up(int(d * config["qk_dim_factor"]), mult)
    config["v_dim"] = _round_up(int(d * config["v_dim_factor"]), mult)
    config["ffn_hidden_dim"] = _round_up(int(d * config["ffn_proj_factor"]), config.get("ffn_round_up_to_multiple_of", 64))
    config["qk_head_dim"] = config["qk_dim"] // config["num_heads"]
    config["v_head_dim"] = config["v_dim"] // config["num_heads"]
    config.setdefault("chunk_size", 64)
    config.setdefault("mode", "inference")
    config.setdefault("return_last_states", True)
    config.setdefault("autocast_kernel_dtype", "bfloat16")
    config.setdefault("inference_state_dtype", "float32")
    config.setdefault("norm_reduction_force_float32", True)
    return config


def load_safetensor_shards(model_dir: str) -> Dict[str, torch.Tensor]:
    """Read every ``*.safetensors`` shard of a checkpoint directory into one dict (CPU tensors)."""
    from safetensors.torch import load_file
    out: Dict[str, torch.Tensor] = {}
    shards = sorted(Path(model_dir).glob("*.safetensors"))
    if not shards:
        raise FileNotFoundError(f"no .safetensors shards in {model_dir}")
    for shard in shards:
        out.update(load_file(str(shard)))
    return out


def infer_config_from_safetensors(model_dir: str) -> Dict[str, Any]:
    """Model configuration read off the tensor shapes of a checkpoint (no ``config.json`` needed).

    Same required tensors, consistency checks, error types and returned keys as the reference function.  Two
    differences, both additive: shapes are read from the shard headers of EVERY shard (the reference loads the
    tensors of the first shard only, so a block-0 tensor stored in a later shard is "not found"), and the head
    count comes from the input-gate bias (one entry per head) instead of the constant 8, which it falls back to."""
    from safetensors import safe_open
    root = Path(model_dir)
    index_path = root / "model.safetensors.index.json"
    if not index_path.exists():
        raise FileNotFoundError(f"Safetensors index not found: {index_path}")
    index = json.loads(index_path.read_text())
    weight_map = index["weight_map"]
    shapes: Dict[str, tuple] = {}
    for shard in sorted(set(weight_map.values())):
        if (root / shard).exists():
            with safe_open(str(root / shard), framework="pt", device="cpu") as f:
                for name in f.keys():
                    shapes[name] = tuple(f.get_slice(name).get_shape())

    def shape_of(name: str) -> tuple:
        if name in weight_map and name in shapes:
            return shapes[name]
        meta = index.get("metadata", {}).get(name, {}) if isinstance(index.get("metadata"), dict) else {}
        if isinstance(meta, dict) and meta.get("shape"):
            return tuple(meta["shape"])
        raise ValueError(f"Required tensor not found: {name}")

    vocab_size, d_model = shape_of("backbone.embeddings.weight")
    if shape_of("lm_head.weight") != (vocab_size, d_model):
        raise ValueError("LM head shape mismatch with embeddings")
    block_ids = {int(k.split(".")[2]) for k in weight_map if k.startswith("backbone.blocks.") and k.split(".")[2].isdigit()}
    if not block_ids:
        raise ValueError("No blocks found in checkpoint")
    b0 = "backbone.blocks.0"
    qk_dim = shape_of(f"{b0}.mlstm_layer.q.weight")[0]
    shape_of(f"{b0}.mlstm_layer.v.weight")
    ig_b = shape_of(f"{b0}.mlstm_layer.igate_preact.bias")
    fg_b = shape_of(f"{b0}.mlstm_layer.fgate_preact.bias")
    up, down = shape_of(f"{b0}.ffn.proj_up.weight"), shape_of(f"{b0}.ffn.proj_down.weight")
    if down[1] != up[0] or down[0] != d_model:
        raise ValueError("FFN shape inconsistency")
    if shape_of(f"{b0}.mlstm_layer.out_proj.weight") != (d_model, d_model):
        raise ValueError("Output projection shape mismatch")
    return {"embedding_dim": d_model, "vocab_size": vocab_size, "num_blocks": max(block_ids) + 1,
            "qk_dim_factor": float(qk_dim / d_model), "v_dim_factor": 1.0, "ffn_proj_factor": float(up[0] / d_model),
            "num_heads": int(ig_b[0]) if ig_b and ig_b[0] > 0 else 8, "gate_soft_cap": 15.0, "norm_eps": 1e-6,
            "use_bias": ig_b is not None and fg_b is not None, "output_logit_soft_cap": 30.0, "chunk_size": 64}


XLSTM_7B_CONFIG = {
    "embedding_dim": 4096, "num_heads": 8, "num_blocks": 32, "vocab_size": 50304, "qk_dim_factor": 0.5,
    "v_dim_factor": 1.0, "ffn_proj_factor": 2.667, "ffn_round_up_to_multiple_of": 64,
    "mlstm_round_up_to_multiple_of": 64, "gate_soft_cap": 15.0, "output_logit_soft_cap": 30.0, "chunk_size": 64,
    "norm_eps": 1e-6, "eps": 1e-6, "use_bias": False, "tie_word_embeddings": False, "bos_token_id": 0,
    "eos_token_id": 2, "pad_token_id": 1, "force_bos_token_insert": True,
    "autocast_kernel_dtype": "bfloat16", "inference_state_dtype": "float32",
}


def write_model_dir(path, config: Dict[str, Any], block_types=None) -> Path:
    """Write ``config.json`` and a keys-only safetensors index for ``config['num_blocks']`` blocks.

    ``block_types`` is an optional list of ``"mlstm"`` / ``"slstm"`` per block (default all mLSTM).
    """
    path = Path(path)
    path.mkdir(parents=True, exist_ok=True)
    nb = int(config["num_blocks"])
    types = list(block_types) if block_types is not None else ["mlstm"] * nb
    keys = ["backbone.embeddings.weight", "backbone.out_norm.weight", "lm_head.weight"]
    for i, t in enumerate(types):
        layer = "mlstm_layer" if t == "mlstm" else "slstm_layer"
        keys += [f"backbone.blocks.{i}.{layer}.out_proj.weight", f"backbone.blocks.{i}.norm_ffn.weight",
                 f"backbone.blocks.{i}.ffn.proj_up.weight"]
    (path / "config.json").write_text(json.dumps(config, indent=1))
    (path / "model.safetensors.index.json").write_text(
        json.dumps({"metadata": {}, "weight_map": {k: "model-00001-of-00001.safetensors" for k in keys}}))
    return path


__all__ = ["resolve_dtype", "load_config", "load_safetensor_shards", "infer_config_from_safetensors", "write_model_dir",
           "XLSTM_7B_CONFIG"]
