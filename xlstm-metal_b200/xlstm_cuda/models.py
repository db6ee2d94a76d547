"""``WiredxLSTM``: embedding -> blocks -> out_norm -> lm_head, threading one state tuple per block.

Constructor, ``forward(input_ids, state=None, return_last_states=False)`` and ``from_pretrained``
follow xlstm_metal/torch_native/models/wired_xlstm.py:17-302.  Differences, all additive: blocks
live in an ``nn.ModuleList`` (the reference keeps a plain list, so ``.to()`` and ``state_dict()``
miss them, wired_xlstm.py:98); sLSTM blocks are wired; the default device is CUDA.
"""
from __future__ import annotations

from pathlib import Path
from typing import Any, Dict, List, Optional, Tuple, Union

import torch
import torch.nn as nn

from .blocks.rms_norm import RMSNormCell
from .utils import load_config, load_safetensor_shards, resolve_dtype
from .wiring import AutoWiring, create_auto_wiring


class WiredxLSTM(nn.Module):
    def __init__(self, wiring: AutoWiring, load_weights: bool = False, model_dir: Optional[Union[str, Path]] = None,
                 compute_dtype: torch.dtype = torch.float32, state_dtype: torch.dtype = torch.float32,
                 norm_reduce_force_float32: bool = True, device: Optional[torch.device] = None,
                 head_shard: Optional[Tuple[int, int]] = None, head_shard_group=None):
        """``head_shard=(rank, world)`` (not in the reference, which is single-device): every mLSTM layer keeps only
        this rank's heads (column slices of q/k/v/igate/fgate/ogate, its heads' norm weights and states) and
        all-gathers the gated head outputs before its replicated out-projection; everything else is replicated."""
        super().__init__()
        self.head_shard, self.head_shard_group = head_shard, head_shard_group
        self.wiring = wiring
        self.config = wiring.config
        self.model_dir = Path(model_dir) if model_dir else wiring.model_dir
        self.compute_dtype = compute_dtype
        self.state_dtype = state_dtype
        self.norm_reduce_force_float32 = norm_reduce_force_float32
        self.device = torch.device(device) if device is not None else torch.device("cuda")
        for key in ("pad_token_id", "bos_token_id", "eos_token_id"):
            setattr(self, key, self.config.get(key))
        self.force_bos_token_insert = self.config.get("force_bos_token_insert", False)
        self.tie_word_embeddings = self.config.get("tie_word_embeddings", False)
        self._embeddings_tied = False
        self._build_model()
        if load_weights:
            self.load_pretrained_weights()
        if self.config.get("mode", "inference") == "inference":
            self.eval()

    def _build_model(self) -> None:
        st, cfg, dev, dt = self.wiring.structure, self.config, self.device, self.compute_dtype
        d, vocab = int(cfg["embedding_dim"]), int(cfg["vocab_size"])
        self.embedding = nn.Embedding(vocab, d, device=dev, dtype=dt) if st["has_embedding"] else None
        self.blocks = nn.ModuleList()
        for idx in range(st["num_blocks"]):
            with torch.device(dev):
                cell = self.wiring.create_block_cell(idx, compute_dtype=self.compute_dtype, state_dtype=self.state_dtype,
                                                     norm_reduction_force_float32=self.norm_reduce_force_float32)
            # every parameter, norm weights included, in the compute dtype: a stray fp32 weight would
            # promote the activations and break the next Linear
            if self.head_shard is not None and hasattr(cell, "shard_heads"):
                cell.shard_heads(self.head_shard[0], self.head_shard[1], self.head_shard_group)
            self.blocks.append(cell.to(device=dev, dtype=dt))
        self.out_norm = RMSNormCell(dims=d).to(device=dev, dtype=dt) if st["has_out_norm"] else None
        self.lm_head = nn.Linear(d, vocab, bias=False, device=dev, dtype=dt) if st["has_lm_head"] else None
        self._apply_weight_tying()

    def forward(self, input_ids: torch.Tensor, state: Optional[List[Tuple]] = None, return_last_states: bool = False,
                last_token_only: bool = False):
        """``last_token_only`` (not in the reference signature): logits of the last position only,
        ``[B, 1, vocab]`` -- what generation consumes after a prompt; skips the ``[B, S, vocab]`` head GEMM."""
        x = input_ids.to(self.device)
        if self.embedding is not None:
            x = self.embedding(x)
        if state is None:
            state = [None] * len(self.blocks)
        new_states = []
        for idx, block in enumerate(self.blocks):
            x, block_state = block(x, state[idx])
            new_states.append(block_state)
        if last_token_only:
            x = x[:, -1:]
        if self.out_norm is not None:
            x = self.out_norm(x)
        logits = self.lm_head(x) if self.lm_head is not None else x
        return (logits, new_states) if return_last_states else logits

    def fuse_projections(self) -> int:
        """Merge the per-block projection GEMMs (see ``mLSTMBlock.fuse_projections``); returns the
        number of blocks fused.  Parameter names and values are unchanged."""
        n = 0
        for block in self.blocks:
            if hasattr(block, "fuse_projections"):
                block.fuse_projections()
                n += 1
        return n

    def load_pretrained_weights(self) -> None:
        if self.model_dir is None:
            raise ValueError("model_dir must be provided to load weights")
        self._load_weights_from_dict(load_safetensor_shards(str(self.model_dir)))

    def _load_weights_from_dict(self, weights: Dict[str, torch.Tensor]) -> None:
        def assign(param: torch.Tensor, key: str, rows: Optional[slice] = None) -> None:
            if key in weights:
                w = weights[key] if rows is None else weights[key][rows]   # a head-sharded layer takes its row slice
                with torch.no_grad():
                    param.copy_(w.to(device=param.device, dtype=param.dtype))

        if self.embedding is not None:
            assign(self.embedding.weight, "backbone.embeddings.weight")
        for block in self.blocks:
            params = dict(block.named_parameters())
            for path, key in block.get_weight_keys().items():
                if path in params:
                    assign(params[path], key, block.weight_row_slice(path) if hasattr(block, "weight_row_slice") else None)
        if self.out_norm is not None:
            assign(self.out_norm.weight, "backbone.out_norm.weight")
        if self.lm_head is not None:
            assign(self.lm_head.weight, "lm_head.weight")
        self._apply_weight_tying()

    @classmethod
    def from_pretrained(cls, model_dir: Union[str, Path], load_weights: bool = True,
                        device: Optional[torch.device] = None, **kwargs) -> "WiredxLSTM":
        model_dir = Path(model_dir)
        config = load_config(str(model_dir))
        wiring = create_auto_wiring(str(model_dir), config)
        kwargs.setdefault("compute_dtype", resolve_dtype(config.get("autocast_kernel_dtype", "float32")))
        kwargs.setdefault("state_dtype", resolve_dtype(config.get("inference_state_dtype", "float32")))
        return cls(wiring=wiring, load_weights=load_weights, model_dir=model_dir, device=device, **kwargs)

    def get_config(self) -> Dict[str, Any]:
        st = self.wiring.structure
        return {"model_type": "wired_xlstm", "wiring_config": self.wiring.get_config(), "num_blocks": st["num_blocks"],
                "block_types": {i: self.wiring.get_block_info(i)["type"] for i in range(st["num_blocks"])},
                "embedding_dim": int(self.config["embedding_dim"]), "vocab_size": int(self.config["vocab_size"]),
                "has_embedding": st["has_embedding"], "has_out_norm": st["has_out_norm"],
                "has_lm_head": st["has_lm_head"], "pad_token_id": self.pad_token_id, "bos_token_id": self.bos_token_id,
                "eos_token_id": self.eos_token_id, "tie_word_embeddings": self.tie_word_embeddings,
                "device": str(self.device)}

    def _apply_weight_tying(self) -> None:
        tie = bool(self.tie_word_embeddings) and self.embedding is not None and self.lm_head is not None
        self._embeddings_tied = tie
        if tie:
            self.lm_head.weight = self.embedding.weight


__all__ = ["WiredxLSTM"]
