"""Golden fixtures at the FULL shapes of the benchmark configurations, from the reference's own classes on CPU.

    python tests/golden/make_golden_full.py --reference /path/to/xLSTM-metal

The same in-memory shims as ``make_golden_model.py`` let the reference's block classes run off Apple
hardware.  Weights and inputs are NOT stored: both sides regenerate them (``param_init.fill_parameters``
from a numpy PCG64 stream, inputs from seeded numpy generators), so a fixture holds only outputs, and
those subsampled where they are large.

Fixture                  produced by (path inside the reference project)
-----------------------  ----------------------------------------------------------------------------
block_7b_bf16            xlstm_metal/torch_native/blocks/mlstm/mlstm_block.py::mLSTMBlock at D=4096, NH=8
                         (256/512, FFN 10944), bf16 parameters and compute, fp32 state: 192 tokens in one
                         call, then 8 single-token calls carrying the state (teacher-forced input)
slstm_blockdiag_bf16_1024  kernel_development/xlstm/implementations/pytorch/xlstm_pytorch_enhanced.py::sLSTMBlock
                         at d=1024, 4 heads x 256, bf16, B=4, S=64
mlstm_extreme_bf16       xlstm_metal/torch_native/blocks/mlstm/mlstm_chunkwise/mlstm_recurrent_kernel_cell.py with
                         compute_dtype=bfloat16 on gates pinned at the soft-cap limits: per-token error of the
                         reference's own bf16 cell against a float64 evaluation of the recurrence
"""
from __future__ import annotations

import argparse
import importlib
import importlib.util
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))
from make_golden_model import apply_shims  # noqa: E402
from param_init import fill_parameters  # noqa: E402


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    """bf16 tensor -> uint16 bit patterns (numpy has no bfloat16)."""
    return t.to(torch.bfloat16).contiguous().view(torch.int16).numpy().view(np.uint16)


def block_7b_input(seed: int = 52, tokens: int = 200, dim: int = 4096) -> torch.Tensor:
    """The teacher-forced block input, regenerated identically by the test."""
    x = np.random.default_rng(seed).standard_normal((1, tokens, dim)).astype(np.float32)
    return torch.from_numpy(x).to(torch.bfloat16)


def fill_block_7b(blk, seed: int = 51) -> None:
    """Parameters of the 7B-shaped block: ``fill_parameters``, then the matrices brought to the N(0, 0.02) scale
    that BASELINE configs[2] names (``fill_parameters`` draws them at 0.06 for the small fixtures)."""
    named = dict(blk.named_parameters())
    fill_parameters(named, seed=seed)
    with torch.no_grad():
        for prm in named.values():
            if prm.dim() >= 2:
                prm.mul_(1.0 / 3.0)


def extreme_inputs():
    """Inputs of the extreme-gate case (gates held at -15 / 0 / +15 for stretches of 16 and 32 tokens)."""
    rng = np.random.default_rng(13)
    B, NH, S, dqk, dv = 1, 2, 768, 256, 256
    rnd = lambda a: torch.from_numpy(a).to(torch.bfloat16).float().numpy()
    q, k = (rnd(rng.standard_normal((B, NH, S, dqk)).astype(np.float32)) for _ in range(2))
    v = rnd(rng.standard_normal((B, NH, S, dv)).astype(np.float32))
    i = np.repeat(rng.choice([-15.0, 0.0, 15.0], size=(B, NH, S // 16)), 16, axis=-1).astype(np.float32)
    f = np.repeat(rng.choice([-15.0, 3.0, 15.0], size=(B, NH, S // 32), p=[0.1, 0.5, 0.4]), 32, axis=-1).astype(np.float32)
    return q, k, v, i, f


def recurrent_fp64(q, k, v, i, f, eps=1e-6):
    """The recurrence of mlstm_recurrent_kernel_cell.py:106-153 evaluated in float64."""
    q, k, v, i, f = (a.astype(np.float64) for a in (q, k, v, i, f))
    B, NH, S, dqk = q.shape
    C = np.zeros((B, NH, dqk, v.shape[-1])); n = np.zeros((B, NH, dqk)); m = np.zeros((B, NH)); hs = []
    for t in range(S):
        fl = -np.logaddexp(0, -f[:, :, t])
        mn = np.maximum(fl + m, i[:, :, t])
        fg, ig = np.exp(fl + m - mn), np.exp(i[:, :, t] - mn)
        C = fg[..., None, None] * C + ig[..., None, None] * k[:, :, t, :, None] * v[:, :, t, None, :]
        n = fg[..., None] * n + ig[..., None] * k[:, :, t]
        m = mn
        qs = q[:, :, t] / np.sqrt(dqk)
        den = np.maximum(np.abs(np.einsum("bhd,bhd->bh", qs, n)), np.exp(-m)) + eps
        hs.append(np.einsum("bhd,bhdv->bhv", qs, C) / den[..., None])
    return np.stack(hs, 2), (C, n, m)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference project")
    ref = Path(ap.parse_args().reference)
    torch.set_grad_enabled(False)
    apply_shims(ref)

    # ---- one mLSTM block at the 7B shape, bf16 --------------------------------------------
    mb = importlib.import_module("xlstm_metal.torch_native.blocks.mlstm.mlstm_block")
    blk = mb.mLSTMBlock(0, embedding_dim=4096, num_heads=8, compute_dtype=torch.bfloat16, state_dtype=torch.float32).eval()
    fill_block_7b(blk)
    blk = blk.to(torch.bfloat16)
    x = block_7b_input()
    P = 192

    def run(block, xin):
        y_pre, st = block(xin[:, :P], None)
        m_pre = block.mlstm_cell(block.norm_mlstm(xin[:, :P]), None)[0]    # the mLSTM branch alone (before the residual add)
        st_pre = tuple(t.clone().float() for t in st)
        ys = [y_pre]
        for t in range(P, xin.shape[1]):
            yt, st = block(xin[:, t:t + 1], st)
            ys.append(yt)
        return torch.cat(ys, 1).float(), m_pre.float(), st_pre, tuple(t.float() for t in st)

    y, m_pre, st_pre, st = run(blk, x)
    # the same block (bf16-rounded parameters and input) evaluated in fp32: how far the reference's own bf16
    # path is from exact arithmetic on this input - the yardstick for a second bf16 implementation
    blk32 = mb.mLSTMBlock(0, embedding_dim=4096, num_heads=8, compute_dtype=torch.float32, state_dtype=torch.float32).eval()
    blk32.load_state_dict({k_: v_.float() for k_, v_ in blk.state_dict().items()})
    y32, m32, st32_pre, st32 = run(blk32, x.float())
    rel = lambda a, b: float((a - b).abs().max() / b.abs().max())
    print("block_7b_bf16: reference bf16 vs its fp32 evaluation: y", rel(y, y32), "mlstm branch", rel(m_pre, m32),
          "C", rel(st_pre[0], st32_pre[0]), "n", rel(st_pre[1], st32_pre[1]), "C_end", rel(st[0], st32[0]))
    sub = lambda C: C[:, :, ::8, ::8].contiguous().float().numpy()
    np.savez_compressed(
        HERE / "block_7b_bf16.npz", y_cols=bf16_bits(y[:, :, ::8]), mlstm_cols=bf16_bits(m_pre[:, :, ::8]),
        y32_cols=bf16_bits(y32[:, :, ::8]), mlstm32_cols=bf16_bits(m32[:, :, ::8]),
        C_pre=sub(st_pre[0]), n_pre=st_pre[1].numpy(), m_pre=st_pre[2].numpy(),
        C_end=sub(st[0]), n_end=st[1].numpy(), m_end=st[2].numpy(),
        C32_pre=sub(st32_pre[0]), n32_pre=st32_pre[1].numpy(), m32_pre=st32_pre[2].numpy(),
        C32_end=sub(st32[0]), n32_end=st32[1].numpy(), m32_end=st32[2].numpy(),
        prefill_tokens=np.int64(P), seed_params=np.int64(51), seed_input=np.int64(52))
    print("block_7b_bf16: |y| max", float(y.abs().max()), "|mlstm branch| max", float(m_pre.abs().max()))

    # ---- block-diagonal sLSTM block at d=1024, bf16 ---------------------------------------
    spec = importlib.util.spec_from_file_location(
        "ref_enhanced", str(ref / "kernel_development/xlstm/implementations/pytorch/xlstm_pytorch_enhanced.py"))
    enh = importlib.util.module_from_spec(spec)
    sys.modules["ref_enhanced"] = enh
    spec.loader.exec_module(enh)
    cfg = enh.xLSTMConfig(inp_dim=1024, head_dim=256, head_num=4, gate_soft_cap=15.0, dropout=0.0)
    sblk = enh.sLSTMBlock(cfg).eval()
    named = {k: v for k, v in sblk.named_parameters() if not k.startswith("causal_conv")}
    fill_parameters(named, seed=61)
    with torch.no_grad():   # recurrent weights at the scale BASELINE configs[4] names
        for nme, prm in named.items():
            if ".R_" in nme or nme.startswith("R_"):
                prm.mul_(0.02 / 0.3)
    xs32 = torch.from_numpy(np.random.default_rng(62).standard_normal((4, 64, 1024)).astype(np.float32))
    # The class initialises its state in fp32 and mixes it with the parameters, so it does not run with bf16
    # parameters (checked when this fixture was made: "mat1 and mat2 must have the same dtype").  The fixture
    # is therefore its fp32 run on bf16-ROUNDED parameters and input: what a bf16 implementation approaches.
    sblk16 = sblk.to(torch.bfloat16)
    try:
        y16, st16 = sblk16(xs32.to(torch.bfloat16))
        ran_bf16 = True
    except RuntimeError as exc:
        print("bf16 run of the reference sLSTMBlock failed:", repr(exc))
        y16, st16, ran_bf16 = None, None, False
    y32b, st32b = sblk16.float()(xs32.to(torch.bfloat16).float())
    out = dict(y_fp32_of_bf16_params=y32b.numpy().astype(np.float32)[:, :, ::2],
               c=st32b[0].float().numpy(), n=st32b[1].float().numpy(), h=st32b[2].float().numpy(), m=st32b[3].float().numpy(),
               ran_bf16=np.bool_(ran_bf16), seed_params=np.int64(61), seed_input=np.int64(62))
    if ran_bf16:
        out["y_bf16"] = bf16_bits(y16[:, :, ::2])
        print("sLSTM block: bf16 vs fp32-of-bf16-params rel", float((y16.float() - y32b).abs().max() / y32b.abs().max()))
    np.savez_compressed(HERE / "slstm_blockdiag_bf16_1024.npz", **out)

    # ---- extreme gates: how far the reference's own bf16 cell is from float64 ------------------
    spec = importlib.util.spec_from_file_location(
        "ref_mlstm_cell", str(ref / "xlstm_metal/torch_native/blocks/mlstm/mlstm_chunkwise/mlstm_recurrent_kernel_cell.py"))
    cm = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(cm)
    q, k, v, i, f = extreme_inputs()
    h64, st64 = recurrent_fp64(q, k, v, i, f)
    cell = cm.mLSTMRecurrentKernelCell(2, 256, 256, compute_dtype=torch.bfloat16, state_dtype=torch.float32)
    hb, stb = cell(*(torch.from_numpy(a).to(torch.bfloat16) for a in (q, k, v, i, f)), None)
    err_tok = np.abs(hb.float().numpy() - h64).max(-1)            # [B, NH, S]
    mag_tok = np.abs(h64).max(-1)
    np.savez_compressed(HERE / "mlstm_extreme_bf16.npz", ref_err_tok=err_tok.astype(np.float32),
                        h64_mag_tok=mag_tok.astype(np.float32),
                        ref_C_rel=np.float32(np.abs(stb[0].float().numpy() - st64[0]).max() / np.abs(st64[0]).max()))
    big = mag_tok > 5.0
    print("extreme gates: tokens with |h| > 5:", float(big.mean()), " reference bf16 rel err there (median / 95%):",
          float(np.median(err_tok[big] / mag_tok[big])), float(np.quantile(err_tok[big] / mag_tok[big], 0.95)),
          " elsewhere:", float(np.median(err_tok[~big] / np.maximum(mag_tok[~big], 1e-9))))


if __name__ == "__main__":
    main()
