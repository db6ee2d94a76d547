"""Block discovery from the safetensors index and the per-block cell factory.

``analyze_safetensors_structure`` / ``detect_block_type`` / ``AutoWiring`` / ``create_auto_wiring``
follow xlstm_metal/torch_native/wiring/auto_wiring.py:20-205; the adjacency bookkeeping of the
base ``Wiring`` (wirings.py:12-117) is reduced to the sequential chain the models use.  Unlike
the reference torch backend (auto_wiring.py:186-187), ``slstm`` blocks are wired too.
"""
from __future__ import annotations

import json
from collections import defaultdict
from pathlib import Path
from typing import Any, Dict, List, Optional


def analyze_safetensors_structure(model_dir: str) -> Dict[str, Any]:
    index_path = Path(model_dir) / "model.safetensors.index.json"
    if not index_path.exists():
        raise FileNotFoundError(f"Safetensors index not found: {index_path}")
    keys = list(json.loads(index_path.read_text())["weight_map"].keys())
    comps: Dict[int, set] = defaultdict(set)
    for key in keys:
        parts = key.split(".")
        if key.startswith("backbone.blocks.") and len(parts) >= 4:
            comps[int(parts[2])].add(parts[3])
    return {
        "num_blocks": len(comps),
        "block_components": {i: sorted(c) for i, c in sorted(comps.items())},
        "has_embedding": any(k.startswith("backbone.embeddings") for k in keys),
        "has_lm_head": any(k.startswith("lm_head") for k in keys),
        "has_out_norm": any(k.startswith("backbone.out_norm") for k in keys),
    }


def detect_block_type(components: List[str]) -> str:
    c = set(components)
    if "mlstm_layer" in c:
        return "mlstm"
    if "slstm_layer" in c:
        return "slstm"
    if "attn_layer" in c or "attention" in c:
        return "attention"
    return "unknown"


class AutoWiring:
    def __init__(self, model_dir: str, config: Optional[Dict] = None):
        self.structure = analyze_safetensors_structure(model_dir)
        self.config = config or {}
        self.model_dir = Path(model_dir)
        self.block_types = {i: detect_block_type(c) for i, c in self.structure["block_components"].items()}
        nb = self.structure["num_blocks"]
        self.units = nb + sum([self.structure["has_embedding"], self.structure["has_out_norm"],
                               self.structure["has_lm_head"]])
        self.synapses = [(i, i + 1) for i in range(nb - 1)]  # blocks feed each other in order
        self.output_dim = 1

    def get_block_info(self, block_idx: int) -> Dict[str, Any]:
        return {"index": block_idx, "type": self.block_types.get(block_idx, "unknown"),
                "components": self.structure["block_components"].get(block_idx, [])}

    def create_block_cell(self, block_idx: int, **kwargs):
        t = self.get_block_info(block_idx)["type"]
        if t == "mlstm":
            from .blocks.mlstm import mLSTMBlock
            kwargs.pop("norm_reduction_force_float32", None)
            return mLSTMBlock.from_config(block_idx, self.config, **kwargs)
        if t == "slstm":
            from .blocks.slstm import sLSTMBlock
            return sLSTMBlock.from_config(block_idx, self.config, **kwargs)
        if t == "attention":
            raise NotImplementedError("Attention block not implemented")
        raise ValueError(f"Unknown block type: {t}")

    def get_config(self) -> Dict[str, Any]:
        return {"units": self.units, "num_blocks": self.structure["num_blocks"],
                "block_types": dict(self.block_types)}


def create_auto_wiring(model_dir: str, config: Optional[Dict] = None) -> AutoWiring:
    return AutoWiring(model_dir, config)


__all__ = ["analyze_safetensors_structure", "detect_block_type", "AutoWiring", "create_auto_wiring"]
