"""``xLSTMRunner``: config-driven inference runner with the reference's public methods.

``reset_state / forward / generate_next_token / generate / get_model_info`` follow
xlstm_metal/torch_native/generate.py:19-284.  Generation is stateful the way the MLX runner does
it (mlx_jit/generate.py:299-332): the prompt goes through the model once (chunkwise prefill), then
single tokens ``[1, 1]`` are fed with the carried state (decode-step kernel).  The torch reference
loop re-feeds the whole growing sequence while also carrying state
(torch_native/generate.py:214-218 with :130), which double-counts the prefix; that is not copied.
``generate`` accepts a list / tensor of token ids (returns a list of ids, as the MLX runner) or a
string when the model directory holds a ``tokenizer.json``.  Logits are soft-capped by the kernel.
"""
from __future__ import annotations

from pathlib import Path
from typing import List, Optional, Sequence, Union

import torch

from .blocks.soft_cap import soft_cap
from .models import WiredxLSTM
from .utils import load_config, resolve_dtype
from .wiring import create_auto_wiring


class xLSTMRunner:
    def __init__(self, model_path: str, show_wiring: bool = False, wiring_style: str = "unicode",
                 device: Optional[torch.device] = None, load_weights: Optional[bool] = None):
        self.model_path = Path(model_path)
        self.config = load_config(str(self.model_path))
        self.compute_dtype = resolve_dtype(self.config.get("autocast_kernel_dtype"))
        self.state_dtype = resolve_dtype(self.config.get("inference_state_dtype"))
        self.norm_reduce_force_float32 = self.config.get("norm_reduction_force_float32", True)
        self.embedding_dim = self.config["embedding_dim"]
        self.num_heads = self.config["num_heads"]
        self.num_blocks = self.config["num_blocks"]
        self.vocab_size = self.config["vocab_size"]
        self.output_logit_soft_cap = self.config.get("output_logit_soft_cap", 30.0)
        self.pad_token_id = self.config.get("pad_token_id", 0)
        self.bos_token_id = self.config.get("bos_token_id", 0)
        self.eos_token_id = self.config.get("eos_token_id", None)
        self.force_bos_token_insert = self.config.get("force_bos_token_insert", False)
        self.default_stop_tokens = [self.eos_token_id] if self.eos_token_id is not None else []
        self.wiring = create_auto_wiring(str(self.model_path), self.config)
        if show_wiring:
            print(self.wiring.get_config())
        if load_weights is None:  # random initialisation when the directory holds no weight shards
            load_weights = any(self.model_path.glob("*.safetensors"))
        self.model = WiredxLSTM(wiring=self.wiring, load_weights=load_weights, model_dir=self.model_path,
                                compute_dtype=self.compute_dtype, state_dtype=self.state_dtype,
                                norm_reduce_force_float32=self.norm_reduce_force_float32, device=device)
        self.model.eval()
        self.model.fuse_projections()   # one GEMM for q,k,v,i,f,o and one for the FFN up projections per block
        self.state = None
        self._graph = None          # captured single-token decode step (see _decode_step_graph)
        self.tokenizer = None
        if (self.model_path / "tokenizer.json").exists():
            from tokenizers import Tokenizer
            self.tokenizer = Tokenizer.from_file(str(self.model_path / "tokenizer.json"))

    @classmethod
    def from_pretrained(cls, model_id: str, **kwargs):
        if Path(model_id).exists():
            return cls(model_id, **kwargs)
        raise ValueError(f"Failed to load model {model_id}: not a local directory (no network access)")

    def reset_state(self) -> None:
        self.state = None

    # ---- graph-captured decode ------------------------------------------------------------------
    # A decode step of a 32-block model is ~700 small launches; replaying them as one CUDA graph removes
    # the per-launch host cost.  The graph works on static buffers: one token id, the per-block state
    # (C updated in place by the step kernel, n and m copied back) and the soft-capped logits.
    def _set_inplace(self, flag: bool) -> None:
        for blk in self.model.blocks:
            cell = getattr(getattr(blk, "mlstm_cell", None), "recurrent_kernel", None)
            if cell is not None:
                cell.inplace_state = flag

    def _eager_static_step(self) -> torch.Tensor:
        logits, new_state = self.model(self._g_ids, self._g_state, return_last_states=True)
        for old, new in zip(self._g_state, new_state):
            for o, n_ in zip(old, new):
                if n_ is not o:
                    o.copy_(n_)
        return soft_cap(logits, self.output_logit_soft_cap)

    def _build_decode_graph(self) -> None:
        dev = self.model.device
        self._g_ids = torch.zeros(1, 1, dtype=torch.long, device=dev)
        self._g_state = [tuple(t.detach().clone().contiguous() for t in st) for st in self.state]
        saved = [tuple(t.clone() for t in st) for st in self._g_state]
        self._set_inplace(True)
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side), torch.inference_mode():
            for _ in range(2):            # warm-up outside capture (allocator, cuBLAS handles)
                self._eager_static_step()
        torch.cuda.current_stream(dev).wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.inference_mode(), torch.cuda.graph(graph):
            self._g_logits = self._eager_static_step()
        self._set_inplace(False)
        for st, sv in zip(self._g_state, saved):   # the warm-up and capture steps advanced the state: restore it
            for t, v in zip(st, sv):
                t.copy_(v)
        self._graph = graph

    @torch.inference_mode()
    def _decode_step_graph(self, token: int) -> torch.Tensor:
        """Logits ``[vocab]`` for one more token, through the captured graph (state carried in place)."""
        if self._graph is None:
            self._build_decode_graph()
        elif self.state is not self._g_state:     # a new sequence: load its state into the static buffers
            for st, new in zip(self._g_state, self.state):
                for t, v in zip(st, new):
                    t.copy_(v)
        self.state = self._g_state
        self._g_ids.fill_(int(token))
        self._graph.replay()
        return self._g_logits[0, -1, :]

    @torch.inference_mode()
    def forward(self, input_ids: torch.Tensor) -> torch.Tensor:
        logits, self.state = self.model(input_ids, self.state, return_last_states=True)
        return soft_cap(logits, self.output_logit_soft_cap)

    @torch.inference_mode()
    def generate_next_token(self, input_ids: torch.Tensor, temperature: float = 1.0, top_k: Optional[int] = None,
                            top_p: Optional[float] = None) -> int:
        logits, self.state = self.model(input_ids, self.state, return_last_states=True, last_token_only=True)
        next_logits = soft_cap(logits, self.output_logit_soft_cap)[0, -1, :].float()
        if temperature == 0.0:  # greedy
            return int(torch.argmax(next_logits).item())
        if temperature != 1.0:
            next_logits = next_logits / temperature
        if top_k is not None and top_k > 0:
            kth = torch.topk(next_logits, k=min(top_k, next_logits.size(-1))).values[-1]
            next_logits = next_logits.masked_fill(next_logits < kth, -float("inf"))
        if top_p is not None and 0 < top_p < 1.0:
            sorted_logits, sorted_idx = torch.sort(next_logits, descending=True)
            keep = torch.cumsum(torch.softmax(sorted_logits, dim=-1), dim=-1) <= top_p
            keep[0] = True  # the most likely token always survives
            mask = torch.zeros_like(next_logits, dtype=torch.bool)
            mask[sorted_idx[keep]] = True
            next_logits = next_logits.masked_fill(~mask, -float("inf"))
        return int(torch.multinomial(torch.softmax(next_logits, dim=-1), num_samples=1).item())

    def generate(self, prompt: Union[str, Sequence[int], torch.Tensor], max_tokens: int = 50, temperature: float = 1.0,
                 top_k: Optional[int] = None, top_p: Optional[float] = None,
                 stop_tokens: Optional[List[int]] = None, use_cuda_graph: bool = False) -> Union[str, List[int]]:
        as_text = isinstance(prompt, str)
        if as_text:
            if self.tokenizer is None:
                raise ValueError("Tokenizer not available in model directory")
            prompt = self.tokenizer.encode(prompt).ids
        tokens = self._prepare_prompt(prompt)
        stop = stop_tokens if stop_tokens is not None else self.default_stop_tokens
        self.reset_state()
        generated = list(tokens)
        current = torch.tensor([tokens], dtype=torch.long)
        for step in range(max_tokens):
            if use_cuda_graph and step > 0 and temperature == 0.0:
                token = int(torch.argmax(self._decode_step_graph(generated[-1])).item())   # greedy, graph replay
            else:
                token = self.generate_next_token(current, temperature=temperature, top_k=top_k, top_p=top_p)
            generated.append(token)
            if stop and token in stop:
                break
            current = torch.tensor([[token]], dtype=torch.long)
        return self.tokenizer.decode(generated) if as_text else generated

    def get_model_info(self) -> dict:
        st = self.wiring.structure
        return {"model_path": str(self.model_path), "embedding_dim": self.embedding_dim, "num_heads": self.num_heads,
                "num_blocks": self.num_blocks, "vocab_size": self.vocab_size, "qk_dim": self.config["qk_dim"],
                "v_dim": self.config["v_dim"], "chunk_size": self.config.get("chunk_size", 64),
                "gate_soft_cap": self.config["gate_soft_cap"], "output_logit_soft_cap": self.output_logit_soft_cap,
                "total_blocks": len(self.model.blocks),
                "block_types": [self.wiring.get_block_info(i)["type"] for i in range(self.num_blocks)],
                "has_embedding": st["has_embedding"], "has_out_norm": st["has_out_norm"],
                "has_lm_head": st["has_lm_head"], "pad_token_id": self.pad_token_id, "bos_token_id": self.bos_token_id,
                "eos_token_id": self.eos_token_id, "force_bos_token_insert": self.force_bos_token_insert}

    def _prepare_prompt(self, prompt_ids) -> List[int]:
        if prompt_ids is None:
            tokens: List[int] = []
        elif hasattr(prompt_ids, "tolist"):
            tokens = prompt_ids.tolist()
        else:
            tokens = list(prompt_ids)
        tokens = [int(t) for t in tokens]
        bos = self.bos_token_id
        if not tokens and bos is not None:
            tokens = [int(bos)]
        elif tokens and self.force_bos_token_insert and bos is not None and tokens[0] != int(bos):
            tokens = [int(bos)] + tokens
        if not tokens:
            raise ValueError("Prompt is empty and no BOS token was available in config.json.")
        return tokens


__all__ = ["xLSTMRunner"]
