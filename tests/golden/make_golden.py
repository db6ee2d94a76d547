"""Generate the golden fixtures in this folder by running the REFERENCE's own code on CPU.

Run where a checkout of the reference project is available::

    python tests/golden/make_golden.py --reference /path/to/xLSTM-metal

Nothing here is needed at test time: the tests read the ``.npz`` files only.
The reference modules are loaded by file path (several package ``__init__``
files pull in Apple-only dependencies), never copied.

Fixture            produced by (path inside the reference project)
-----------------  ------------------------------------------------------------
mlstm_c1_fp32      xlstm_metal/torch_native/blocks/mlstm/mlstm_chunkwise/mlstm_recurrent_kernel_cell.py
                   (cross-checked against tests/parity/canonical_reference.py and the vendored
                   kernel_development/.../vendored/torch/native/fw.py::mlstm_chunkwise)
mlstm_ragged_fp32  same cell; non-zero initial state, S not a multiple of 64, dqk != dv
mlstm_step_bf16    same cell with compute_dtype=bfloat16 / state fp32, 8 carried single-token steps
mlstm_step_7b      same cell, one (batch, head) at 256/512, bf16 compute, 3 carried steps
slstm_a            .../slstm/slstm_layers/stepwise/slstm_stepwise_kernel_cell.py (shapes and seeds of
                   tests/test_slstm_metal_kernel.py: (2,4,8), (1,2,4), 5-step sequence, extreme gates)
slstm_b            kernel_development/xlstm/implementations/pytorch/xlstm_pytorch_enhanced.py::sLSTMBlock
kat                literal inputs of tests/test_mlx_torch_numerical_parity.py:10,22-24,51-54 and
                   tests/parity/test_numerical_parity.py:105-108, evaluated with torch as those tests do
norms              tests/parity/canonical_reference.py (rmsnorm, multihead rmsnorm) and
                   xlstm_metal/torch_native/blocks/mlstm/multihead_norm/multihead_norm.py
"""
from __future__ import annotations

import argparse
import importlib.util
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def load(path: Path, name: str):
    spec = importlib.util.spec_from_file_location(name, str(path))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def capped(x, cap=15.0):
    return cap * torch.tanh(x / cap)


def rel(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference project")
    args = ap.parse_args()
    ref = Path(args.reference)
    tn = ref / "xlstm_metal" / "torch_native" / "blocks"
    cellmod = load(tn / "mlstm/mlstm_chunkwise/mlstm_recurrent_kernel_cell.py", "ref_mlstm_cell")
    slstmmod = load(tn / "slstm/slstm_layers/stepwise/slstm_stepwise_kernel_cell.py", "ref_slstm_cell")
    canon = load(ref / "tests/parity/canonical_reference.py", "ref_canonical")
    mhn = load(tn / "mlstm/multihead_norm/multihead_norm.py", "ref_mhnorm")
    vend = load(ref / "kernel_development/xlstm/mlstm_block/mlstm_chunkwise/vendored/torch/native/fw.py", "ref_vendored_fw")
    enh = load(ref / "kernel_development/xlstm/implementations/pytorch/xlstm_pytorch_enhanced.py", "ref_enhanced")
    torch.set_grad_enabled(False)

    # ---- mlstm_c1_fp32: BASELINE config 1 ---------------------------------
    g = torch.Generator().manual_seed(0)
    B, NH, S, dqk, dv = 1, 4, 256, 64, 64
    q = torch.randn(B, NH, S, dqk, generator=g)
    k = torch.randn(B, NH, S, dqk, generator=g)
    v = torch.randn(B, NH, S, dv, generator=g)
    i = capped(torch.randn(B, NH, S, generator=g))
    f = capped(torch.randn(B, NH, S, generator=g) + 3.0)
    cell = cellmod.mLSTMRecurrentKernelCell(NH, dqk, dv)
    h, (C, n, m) = cell(q, k, v, i, f, None)
    hc, (Cc, nc, mc) = canon.canonical_mlstm_recurrent_sequence(q.numpy(), k.numpy(), v.numpy(), i.numpy(), f.numpy(), 1e-6)
    hv, (Cv, nv, mv) = vend.mlstm_chunkwise(q, k, v, i, f, return_last_states=True, chunk_size=64, eps=1e-6)
    print("c1: cell vs canonical", rel(hc, h), "| cell vs vendored chunkwise", rel(hv, h), rel(Cv, C))
    np.savez(HERE / "mlstm_c1_fp32.npz", q=q.numpy(), k=k.numpy(), v=v.numpy(), i=i.numpy(), f=f.numpy(),
             h=h.numpy(), C=C.numpy(), n=n.numpy(), m=m.numpy())

    # ---- mlstm_ragged_fp32 ---------------------------------------------------
    g = torch.Generator().manual_seed(11)
    B, NH, S, dqk, dv = 2, 2, 37, 32, 64
    q = torch.randn(B, NH, S, dqk, generator=g)
    k = torch.randn(B, NH, S, dqk, generator=g)
    v = torch.randn(B, NH, S, dv, generator=g)
    i = capped(torch.randn(B, NH, S, generator=g) * 2.0)
    f = capped(torch.randn(B, NH, S, generator=g) * 3.0 + 1.0)
    C0 = torch.randn(B, NH, dqk, dv, generator=g) * 0.5
    n0 = torch.randn(B, NH, dqk, generator=g) * 0.5
    m0 = torch.randn(B, NH, generator=g)
    cell = cellmod.mLSTMRecurrentKernelCell(NH, dqk, dv)
    h, (C, n, m) = cell(q, k, v, i, f, (C0, n0, m0))
    np.savez(HERE / "mlstm_ragged_fp32.npz", q=q.numpy(), k=k.numpy(), v=v.numpy(), i=i.numpy(), f=f.numpy(),
             C0=C0.numpy(), n0=n0.numpy(), m0=m0.numpy(), h=h.numpy(), C=C.numpy(), n=n.numpy(), m=m.numpy())

    # ---- mlstm_step_bf16: carried decode steps, bf16 compute / fp32 state ----
    def decode_fixture(name, B, NH, dqk, dv, steps, seed):
        g = torch.Generator().manual_seed(seed)
        cell = cellmod.mLSTMRecurrentKernelCell(NH, dqk, dv, compute_dtype=torch.bfloat16, state_dtype=torch.float32)
        cell32 = cellmod.mLSTMRecurrentKernelCell(NH, dqk, dv)
        C0 = torch.randn(B, NH, dqk, dv, generator=g) * 0.1
        n0 = torch.randn(B, NH, dqk, generator=g) * 0.1
        m0 = torch.zeros(B, NH)
        q = torch.randn(B, NH, steps, dqk, generator=g).bfloat16()
        k = torch.randn(B, NH, steps, dqk, generator=g).bfloat16()
        v = torch.randn(B, NH, steps, dv, generator=g).bfloat16()
        i = capped(torch.randn(B, NH, steps, generator=g)).bfloat16()
        f = capped(torch.randn(B, NH, steps, generator=g) + 3.0).bfloat16()
        st, st32 = (C0, n0, m0), (C0, n0, m0)
        hs, hs32 = [], []
        for t in range(steps):
            sl = slice(t, t + 1)
            ht, st = cell(q[:, :, sl], k[:, :, sl], v[:, :, sl], i[:, :, sl], f[:, :, sl], st)
            h32, st32 = cell32(q[:, :, sl].float(), k[:, :, sl].float(), v[:, :, sl].float(),
                               i[:, :, sl].float(), f[:, :, sl].float(), st32)
            hs.append(ht.float())
            hs32.append(h32)
        h = torch.cat(hs, 2)
        h32 = torch.cat(hs32, 2)
        print(name, "bf16-compute vs fp32-compute on same inputs:", rel(h, h32), rel(st[0], st32[0]))
        np.savez(HERE / f"{name}.npz", q=q.float().numpy(), k=k.float().numpy(), v=v.float().numpy(),
                 i=i.float().numpy(), f=f.float().numpy(), C0=C0.numpy(), n0=n0.numpy(), m0=m0.numpy(),
                 h_bf16=h.numpy(), C_bf16=st[0].numpy(), n_bf16=st[1].numpy(), m_bf16=st[2].numpy(),
                 h_fp32=h32.numpy(), C_fp32=st32[0].numpy(), n_fp32=st32[1].numpy(), m_fp32=st32[2].numpy())

    decode_fixture("mlstm_step_bf16", 2, 2, 64, 128, 8, 1)
    decode_fixture("mlstm_step_7b", 1, 1, 256, 512, 3, 5)

    # ---- slstm_a: packaged stepwise cell ------------------------------------
    out = {}
    cases = [("a", 42, (2, 4, 8), 1.0, 1.0), ("b", 123, (1, 2, 4), 1.0, 1.0), ("x", 456, (2, 4, 8), 10.0, 100.0)]
    for tag, seed, (B, NH, H), gscale, sscale in cases:
        g = torch.Generator().manual_seed(seed)
        S = 5
        z = torch.randn(B, S, NH, H, generator=g)
        ig = torch.randn(B, S, NH, generator=g) * gscale
        fg = torch.randn(B, S, NH, generator=g) * gscale
        og = torch.randn(B, S, NH, generator=g) * gscale
        c0 = torch.randn(B, NH, H, generator=g) * sscale
        n0 = torch.rand(B, NH, H, generator=g) * sscale
        m0 = torch.randn(B, NH, generator=g)
        cell = slstmmod.sLSTMStepwiseKernelCell(NH, H)
        st = (c0, n0, m0)
        hs = []
        for t in range(S):
            ht, st = cell(z[:, t], ig[:, t], fg[:, t], og[:, t], st)
            hs.append(ht)
        for nm, val in dict(z=z, i=ig, f=fg, o=og, c0=c0, n0=n0, m0=m0, h=torch.stack(hs, 1),
                            c=st[0], n=st[1], m=st[2]).items():
            out[f"{tag}_{nm}"] = val.numpy()
    # zero-state entry (state=None)
    g = torch.Generator().manual_seed(7)
    z = torch.randn(2, 3, 2, 16, generator=g)
    ig, fg, og = (torch.randn(2, 3, 2, generator=g) for _ in range(3))
    cell = slstmmod.sLSTMStepwiseKernelCell(2, 16)
    st, hs = None, []
    for t in range(3):
        ht, st = cell(z[:, t], ig[:, t], fg[:, t], og[:, t], st)
        hs.append(ht)
    for nm, val in dict(z=z, i=ig, f=fg, o=og, h=torch.stack(hs, 1), c=st[0], n=st[1], m=st[2]).items():
        out[f"z_{nm}"] = val.numpy()
    np.savez(HERE / "slstm_a.npz", **out)

    # ---- slstm_b: block-diagonal recurrent sLSTM block ----------------------
    torch.manual_seed(4)
    cfg = enh.xLSTMConfig(inp_dim=48, head_dim=16, head_num=4, gate_soft_cap=15.0, dropout=0.0)
    blk = enh.sLSTMBlock(cfg).eval()
    D = cfg.head_dim * cfg.head_num
    for lin in (blk.R_i, blk.R_f, blk.R_z, blk.R_o):
        for b in lin.blocks:
            b.weight.normal_(0.0, 0.3)  # strong enough that the recurrent path matters
    blk.W_f.bias.copy_(torch.linspace(3.0, 6.0, D))
    B, S = 3, 9
    x = torch.randn(B, S, cfg.inp_dim) * 2.0
    captured = []
    hook = blk.hid_norm.register_forward_hook(lambda mod, inp, outp: captured.append(inp[0].detach().clone()))
    y, (c, n, hfin, m) = blk(x)
    hook.remove()
    hs = torch.stack(captured, 1)  # [B,S,D]
    xn = blk.inp_norm(x)
    gx = torch.stack([blk.W_i(xn), blk.W_f(xn), blk.W_z(xn), blk.W_o(xn)], 2)  # [B,S,4,D]  (use_conv=False)
    R = torch.stack([torch.stack([b.weight for b in lin.blocks]) for lin in (blk.R_i, blk.R_f, blk.R_z, blk.R_o)])
    rb = torch.stack([torch.cat([b.bias for b in lin.blocks]) for lin in (blk.R_i, blk.R_f, blk.R_z, blk.R_o)])
    # a second call that continues from the returned state
    x2 = torch.randn(B, 4, cfg.inp_dim)
    captured.clear()
    hook = blk.hid_norm.register_forward_hook(lambda mod, inp, outp: captured.append(inp[0].detach().clone()))
    st_in = tuple(t.clone() for t in (c, n, hfin, m))
    y2, (c2, n2, h2, m2) = blk(x2, tuple(t.clone() for t in st_in))
    hook.remove()
    xn2 = blk.inp_norm(x2)
    gx2 = torch.stack([blk.W_i(xn2), blk.W_f(xn2), blk.W_z(xn2), blk.W_o(xn2)], 2)
    np.savez(HERE / "slstm_b.npz", gx=gx.numpy(), R=R.numpy(), rb=rb.numpy(), hs=hs.numpy(),
             c=st_in[0].numpy(), n=st_in[1].numpy(), h=st_in[2].numpy(), m=st_in[3].numpy(),
             gx2=gx2.numpy(), hs2=torch.stack(captured, 1).numpy(),
             c2=c2.numpy(), n2=n2.numpy(), h2=h2.numpy(), m2=m2.numpy(), num_heads=np.int32(cfg.head_num))

    # ---- kat: literal inputs of the reference's tests ------------------------
    x = torch.tensor([-50.0, -10.0, -1.0, 0.0, 1.0, 10.0, 50.0])
    ls = torch.nn.functional.logsigmoid(x)
    iv = torch.tensor([[-10.0], [0.0], [10.0]])
    fv = torch.tensor([[-10.0], [0.0], [10.0]])
    mv = torch.tensor([[0.0], [5.0], [-5.0]])
    fl = torch.nn.functional.logsigmoid(fv)
    mn = torch.max(fl + mv, iv)
    qs = torch.tensor([[[1e-8, 1e-8, 1e-8]]])
    ns = torch.tensor([[[1e-8, -1e-8, 0.0]]])
    ms = torch.tensor([[[10.0]]])
    den = torch.maximum((qs * ns).sum(-1, keepdim=True).abs(), torch.exp(-ms)) + 1e-6
    sc = {}
    for tag, vals, cap in [("small", [-0.5, 0.0, 0.5, 1.0], 15.0), ("large", [-50.0, -20.0, 20.0, 50.0], 15.0),
                           ("edge", [-100.0, 0.0, 100.0], 30.0)]:
        xv = torch.tensor(vals)
        sc[f"softcap_{tag}_x"] = xv.numpy()
        sc[f"softcap_{tag}_cap"] = np.float32(cap)
        sc[f"softcap_{tag}_y"] = (cap * torch.tanh(xv / cap)).numpy()
        assert np.allclose(canon.canonical_soft_cap(xv.numpy(), cap), sc[f"softcap_{tag}_y"], rtol=1e-6)
    np.savez(HERE / "kat.npz", logsig_x=x.numpy(), logsig_y=ls.numpy(), gate_i=iv.numpy(), gate_f=fv.numpy(),
             gate_m=mv.numpy(), gate_mnew=mn.numpy(), gate_fexp=torch.exp(fl + mv - mn).numpy(),
             gate_iexp=torch.exp(iv - mn).numpy(), den_q=qs.numpy(), den_n=ns.numpy(), den_m=ms.numpy(),
             den_out=den.numpy(), **sc)

    # ---- norms ---------------------------------------------------------------
    g = torch.Generator().manual_seed(9)
    xr = torch.randn(5, 96, generator=g) * 3.0
    wr = torch.rand(96, generator=g) + 0.5
    xm = torch.randn(2, 3, 4, 32, generator=g)
    norm = mhn.MultiHeadRMSNorm(4, 32, eps=1e-6)
    norm.weight.copy_(torch.rand(128, generator=g) + 0.5)
    # the reference's forward calls .view on a tensor that is contiguous here
    ym = norm(xm)
    np.savez(HERE / "norms.npz", rms_x=xr.numpy(), rms_w=wr.numpy(),
             rms_y=canon.canonical_rmsnorm(xr.numpy(), 1e-6, wr.numpy()),
             mh_x=xm.numpy(), mh_w=norm.weight.numpy(), mh_y=ym.numpy(),
             mh_y_canon=canon.canonical_multihead_rmsnorm(xm.numpy(), 1e-6, norm.weight.numpy()))
    print("fixtures written to", HERE)


if __name__ == "__main__":
    main()
