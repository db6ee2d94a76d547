"""Golden fixtures for the kernels either side of the cells, from the reference's OWN modules on CPU.

    python tests/golden/make_golden_glue.py --reference /path/to/xLSTM-metal

``glue_fp32.npz``:
* output epilogue: the reference ``mLSTMOutputCell`` (mlstm_output_cell.py:84-94, behind the same
  in-memory shims as make_golden_model.py): its ``norm`` and ``ogate_proj`` sub-modules evaluated on
  a random h / x, stored as the output-gate pre-activation and the gated, normalised h;
* causal depthwise convolution: the reference ``CausalConv1d`` (CPU path, causal_conv1d.py:61-67)
  followed by SiLU as in slstm_projection_cell.py:110-117, whole sequence and split in two calls;
* SwiGLU gate: ``F.silu(gate) * up`` exactly as written in mlstm_block.py:198-204.
"""
from __future__ import annotations

import argparse
import importlib
import sys
from pathlib import Path

import numpy as np
import torch
import torch.nn.functional as F

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))
from make_golden_model import apply_shims  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference project")
    ref = Path(ap.parse_args().reference)
    torch.set_grad_enabled(False)
    apply_shims(ref)
    rng = np.random.default_rng(77)
    out = {}

    oc = importlib.import_module("xlstm_metal.torch_native.blocks.mlstm.mlstm_chunkwise.mlstm_output_cell")
    B, S, NH, dv, D = 2, 9, 4, 64, 96
    cell = oc.mLSTMOutputCell(input_size=D, num_heads=NH, v_dim_per_head=dv).eval()
    cell.norm.weight.data = torch.from_numpy(rng.uniform(0.5, 1.5, NH * dv).astype(np.float32))
    cell.ogate_proj.weight.data = torch.from_numpy((rng.standard_normal((NH * dv, D)) * 0.3).astype(np.float32))
    h = torch.from_numpy(rng.standard_normal((B, NH, S, dv)).astype(np.float32) * 2.0)
    x = torch.from_numpy(rng.standard_normal((B, S, D)).astype(np.float32))
    og = cell.ogate_proj(x)
    gated = cell.norm(h.permute(0, 2, 1, 3)) * torch.sigmoid(og)
    full = cell(h, x)
    assert float((cell.out_proj(gated) - full).abs().max()) < 1e-6
    out.update(og_h=h.numpy(), og_pre=og.numpy(), og_w=cell.norm.weight.numpy(), og_y=gated.numpy(),
               og_eps=np.float32(cell.norm.eps))

    cc = importlib.import_module("xlstm_metal.torch_native.blocks.slstm.slstm_layers.causal_conv1d.causal_conv1d")
    Bc, Sc, C, K = 3, 37, 48, 4
    conv = cc.CausalConv1d(C, C, K, groups=C).eval()
    conv.conv.weight.data = torch.from_numpy((rng.standard_normal((C, 1, K)) * 0.5).astype(np.float32))
    conv.conv.bias.data = torch.from_numpy((rng.standard_normal(C) * 0.1).astype(np.float32))
    xc = torch.from_numpy(rng.standard_normal((Bc, Sc, C)).astype(np.float32))
    yc = conv(xc.permute(0, 2, 1)).permute(0, 2, 1)
    out.update(conv_x=xc.numpy(), conv_w=conv.conv.weight.numpy().reshape(C, K), conv_b=conv.conv.bias.numpy(),
               conv_y=yc.numpy(), conv_y_silu=F.silu(yc).numpy())

    g = torch.from_numpy(rng.standard_normal((5, 7, 40)).astype(np.float32) * 3.0)
    u = torch.from_numpy(rng.standard_normal((5, 7, 40)).astype(np.float32))
    out.update(sw_g=g.numpy(), sw_u=u.numpy(), sw_y=(F.silu(g) * u).numpy())

    np.savez_compressed(HERE / "glue_fp32.npz", **out)
    print("wrote", HERE / "glue_fp32.npz", {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
