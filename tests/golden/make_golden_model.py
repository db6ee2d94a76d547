"""Model-level golden fixtures: the reference's OWN block / model classes run on CPU.

    python tests/golden/make_golden_model.py --reference /path/to/xLSTM-metal

Most of ``xlstm_metal.torch_native`` does not import off Apple hardware (a missing ``SoftCap``
class, a wrong ``MultiHeadRMSNorm`` import, Metal-only norm / soft-cap cells, an sLSTM package
``__init__`` that pulls in mlx).  Five monkey-patches, applied here in memory only, let the
reference's code paths execute unmodified otherwise:
  1. ``soft_cap.softcap.SoftCap``        := module computing cap*tanh(x/cap)   (mlstm_projection_cell.py:16)
  2. ``rms_norm.MultiHeadRMSNorm``       := the class in mlstm/multihead_norm/  (mlstm_output_cell.py:19)
  3. ``MultiHeadRMSNorm.forward``        := same math with reshape, not view    (multihead_norm.py:61)
  4. ``RMSNormCell.forward`` / ``SoftCapCell.forward`` := the CPU formula       (rmsnorm.py:31-32, softcap.py:29-30)
  5. a bare package for ``...blocks.slstm.slstm_layers`` so its ``__init__`` never runs
Each patched formula is the one pinned by tests/parity/canonical_reference.py.

Fixtures: ``model_tiny_fp32.npz`` (WiredxLSTM, 2 mLSTM blocks, D=256, NH=2 -> 64/128, vocab 96:
logits and per-block states for a 70-token pass and for a 50+20 split), ``slstm_block_fp32.npz``
(torch_native sLSTMBlock, D=64, NH=4), ``slstm_blockdiag_fp32.npz`` (block-diagonal sLSTMBlock).
Weights are NOT stored: both sides regenerate them with ``param_init.fill_parameters``.
"""
from __future__ import annotations

import argparse
import importlib
import importlib.util
import json
import sys
import tempfile
import types
from pathlib import Path

import numpy as np
import torch
import torch.nn as nn

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))
from param_init import fill_parameters  # noqa: E402

TINY = {"embedding_dim": 256, "num_heads": 2, "num_blocks": 2, "vocab_size": 96, "qk_dim_factor": 0.5,
        "v_dim_factor": 1.0, "ffn_proj_factor": 1.0, "ffn_round_up_to_multiple_of": 64,
        "mlstm_round_up_to_multiple_of": 64, "gate_soft_cap": 15.0, "output_logit_soft_cap": 30.0, "chunk_size": 64,
        "norm_eps": 1e-6, "eps": 1e-6, "use_bias": False, "tie_word_embeddings": False, "bos_token_id": 0,
        "autocast_kernel_dtype": "float32", "inference_state_dtype": "float32"}


def apply_shims(ref: Path):
    sys.path.insert(0, str(ref))
    sc = importlib.import_module("xlstm_metal.torch_native.blocks.soft_cap.softcap")

    class SoftCap(nn.Module):
        def forward(self, x, cap):
            return cap * torch.tanh(x / cap)

    sc.SoftCap = SoftCap
    sc.SoftCapCell.forward = lambda self, x, cap_value=None: (
        x if (cap_value if cap_value is not None else float(self._cap.item())) <= 0
        else float(cap_value if cap_value is not None else self._cap.item())
        * torch.tanh(x / float(cap_value if cap_value is not None else self._cap.item())))
    rn = importlib.import_module("xlstm_metal.torch_native.blocks.rms_norm")
    mh = importlib.import_module("xlstm_metal.torch_native.blocks.mlstm.multihead_norm.multihead_norm")

    def mh_forward(self, x):
        B, S, NH, DH = x.shape
        rms = torch.sqrt((x.float() ** 2).mean(dim=-1, keepdim=True) + self.eps)
        y = (x / rms).type_as(x).reshape(B, S, -1)
        return y * self.weight if self.weight is not None else y

    mh.MultiHeadRMSNorm.forward = mh_forward
    rn.MultiHeadRMSNorm = mh.MultiHeadRMSNorm

    def rms_forward(self, x):
        xf = x.to(torch.float32) if self.force_float32 else x
        y = xf / torch.sqrt((xf * xf).mean(dim=-1, keepdim=True) + self.eps)
        if self.weight is not None:
            y = y * self.weight.to(y.dtype)
        return y.to(x.dtype)

    rn.RMSNormCell.forward = rms_forward
    # sLSTM: keep the mlx-importing package __init__ from running
    pkg = "xlstm_metal.torch_native.blocks.slstm.slstm_layers"
    bare = types.ModuleType(pkg)
    bare.__path__ = [str(ref / "xlstm_metal/torch_native/blocks/slstm/slstm_layers")]
    sys.modules[pkg] = bare


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference project")
    ref = Path(ap.parse_args().reference)
    torch.set_grad_enabled(False)
    apply_shims(ref)
    from xlstm_metal.torch_native.models.wired_xlstm import WiredxLSTM
    from xlstm_metal.torch_native.utils import load_config
    from xlstm_metal.torch_native.wiring import create_auto_wiring

    # ---- tiny WiredxLSTM ------------------------------------------------------
    with tempfile.TemporaryDirectory() as tmp:
        tmp = Path(tmp)
        (tmp / "config.json").write_text(json.dumps(TINY))
        keys = ["backbone.embeddings.weight", "backbone.out_norm.weight", "lm_head.weight"]
        keys += [f"backbone.blocks.{i}.mlstm_layer.q.weight" for i in range(TINY["num_blocks"])]
        (tmp / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {k: "x" for k in keys}}))
        config = load_config(str(tmp))
        wiring = create_auto_wiring(str(tmp), config)
        model = WiredxLSTM(wiring, load_weights=False, device=torch.device("cpu"))
    named = {"embedding.weight": model.embedding.weight, "out_norm.weight": model.out_norm.weight,
             "lm_head.weight": model.lm_head.weight}
    for i, blk in enumerate(model.blocks):
        named.update({f"blocks.{i}.{n}": p for n, p in blk.named_parameters()})
    fill_parameters(named, seed=21)
    ids = np.random.default_rng(22).integers(0, TINY["vocab_size"], size=(2, 70))
    t_ids = torch.from_numpy(ids)
    logits, states = model(t_ids, None, return_last_states=True)
    l1, s1 = model(t_ids[:, :50], None, return_last_states=True)
    l2, s2 = model(t_ids[:, 50:], s1, return_last_states=True)
    print("split vs full:", float((torch.cat([l1, l2], 1) - logits).abs().max()))
    # block 0 alone, teacher-forced input
    x0 = model.embedding(t_ids)
    y0, st0 = model.blocks[0](x0, None)
    out = {"ids": ids, "logits": logits.numpy(), "logits_split": torch.cat([l1, l2], 1).numpy(),
           "block0_in": x0.numpy(), "block0_out": y0.numpy(), "param_names": np.array(sorted(named))}
    for i, (C, n, m) in enumerate(states):
        out[f"C{i}"], out[f"n{i}"], out[f"m{i}"] = C.numpy(), n.numpy(), m.numpy()
    np.savez_compressed(HERE / "model_tiny_fp32.npz", **out)

    # ---- torch_native sLSTMBlock (packaged sLSTM) -------------------------------------
    sb = importlib.import_module("xlstm_metal.torch_native.blocks.slstm.slstm_block")
    blk = sb.sLSTMBlock(0, embedding_dim=64, num_heads=4, head_dim=16, ffn_proj_factor=1.0).eval()
    named = dict(blk.named_parameters())
    fill_parameters(named, seed=31)
    x = torch.from_numpy(np.random.default_rng(32).standard_normal((3, 21, 64)).astype(np.float32))
    y, (c, n, m) = blk(x, None)
    np.savez_compressed(HERE / "slstm_block_fp32.npz", x=x.numpy(), y=y.numpy(), c=c.numpy(), n=n.numpy(), m=m.numpy(),
                        param_names=np.array(sorted(named)))

    # ---- block-diagonal sLSTM block -----------------------------------------------------
    spec = importlib.util.spec_from_file_location(
        "ref_enhanced", str(ref / "kernel_development/xlstm/implementations/pytorch/xlstm_pytorch_enhanced.py"))
    enh = importlib.util.module_from_spec(spec)
    sys.modules["ref_enhanced"] = enh
    spec.loader.exec_module(enh)
    cfg = enh.xLSTMConfig(inp_dim=64, head_dim=32, head_num=4, gate_soft_cap=15.0, dropout=0.0)
    blk = enh.sLSTMBlock(cfg).eval()
    named = {k: v for k, v in blk.named_parameters() if not k.startswith("causal_conv")}
    fill_parameters(named, seed=41)
    x = torch.from_numpy(np.random.default_rng(42).standard_normal((5, 12, 64)).astype(np.float32))
    y, st = blk(x)
    st = tuple(t.clone() for t in st)
    y2, st2 = blk(x[:, :7], tuple(t.clone() for t in st))
    np.savez_compressed(HERE / "slstm_blockdiag_fp32.npz", x=x.numpy(), y=y.numpy(), c=st[0].numpy(), n=st[1].numpy(),
                        h=st[2].numpy(), m=st[3].numpy(), y2=y2.numpy(), c2=st2[0].numpy(),
                        param_names=np.array(sorted(named)))
    print("model fixtures written to", HERE)


if __name__ == "__main__":
    main()
