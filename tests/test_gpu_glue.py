"""GPU parity for the kernels either side of the cells (RMSNorm, output epilogue, SwiGLU gate, causal
depthwise convolution): through the C ABI against the CPU oracle and the fixtures made from the
reference's own modules.  fp32 1e-5 (elementwise math), bf16 2e-2 (max|a-b| / max|b|)."""
import numpy as np
import pytest
import torch

from conftest import relerr
from oracle import oracle as xo

pytestmark = pytest.mark.gpu

FP32_TOL = 1e-5
BF16_TOL = 2e-2


def dev(a, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a)).to("cuda", dtype)


def host(t):
    return t.detach().float().cpu().numpy()


def bf(a):
    return xo.bf16_round(np.asarray(a, np.float32))


@pytest.fixture(scope="module")
def ops():
    from xlstm_cuda import ops as _ops
    return _ops


# ---- RMSNorm ------------------------------------------------------------------------------
def test_rms_norm_golden(ops, golden):
    g = golden("norms")
    y = ops.rms_norm(dev(g["rms_x"]), dev(g["rms_w"]), 1e-6)
    np.testing.assert_allclose(host(y), g["rms_y"], rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("rows,cols", [(1, 4096), (5, 96), (3, 100), (7, 1023), (2, 8192), (2, 40000), (300, 4096)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rms_norm_shapes(ops, rows, cols, dtype):
    rng = np.random.default_rng(rows * 131 + cols)
    x = rng.standard_normal((rows, cols)).astype(np.float32) * 3.0
    w = rng.uniform(0.5, 1.5, cols).astype(np.float32)
    if dtype == torch.bfloat16:
        x, w = bf(x), bf(w)
    ref = xo.rmsnorm(x, w, 1e-6)
    y = ops.rms_norm(dev(x, dtype), dev(w, dtype), 1e-6)
    assert y.dtype == dtype and y.shape == (rows, cols)
    assert relerr(host(y), ref) <= (FP32_TOL if dtype == torch.float32 else BF16_TOL)
    y0 = ops.rms_norm(dev(x, dtype), None, 1e-6)
    assert relerr(host(y0), xo.rmsnorm(x, None, 1e-6)) <= (FP32_TOL if dtype == torch.float32 else BF16_TOL)


@pytest.mark.parametrize("rows,cols", [(3, 4096), (300, 4096), (2000, 4096), (1500, 1024), (1300, 2048), (1200, 96),
                                       (1187, 4104)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_add_rms_norm_shapes(ops, rows, cols, dtype):
    """Residual add + RMSNorm: few rows (CTA per row) and many rows (the streamed kernel, >= 1184 rows), widths that
    fill the warp's vectors exactly and ones that do not.  The sum is rounded to the activation type, stored as
    the new residual stream, and the norm is taken of the rounded value."""
    rng = np.random.default_rng(rows * 7 + cols)
    x = rng.standard_normal((rows, cols)).astype(np.float32) * 2.0
    r = rng.standard_normal((rows, cols)).astype(np.float32) * 2.0
    w = rng.uniform(0.5, 1.5, cols).astype(np.float32)
    if dtype == torch.bfloat16:
        x, r, w = bf(x), bf(r), bf(w)
    s_ref = x + r
    if dtype == torch.bfloat16:
        s_ref = bf(s_ref)
    y_ref = xo.rmsnorm(s_ref, w, 1e-6)
    s, y = ops.add_rms_norm(dev(x, dtype), dev(r, dtype), dev(w, dtype), 1e-6)
    np.testing.assert_array_equal(host(s), s_ref)                  # one rounding of an exact fp32 sum
    assert relerr(host(y), y_ref) <= (FP32_TOL if dtype == torch.float32 else BF16_TOL)
    s2, y2 = ops.add_rms_norm(dev(x, dtype), dev(r, dtype), None, 1e-6)
    assert torch.equal(s2, s)
    assert relerr(host(y2), xo.rmsnorm(s_ref, None, 1e-6)) <= (FP32_TOL if dtype == torch.float32 else BF16_TOL)


def test_rms_norm_empty_and_batched(ops):
    assert ops.rms_norm(torch.empty(0, 64, device="cuda"), None).shape == (0, 64)
    x = torch.randn(2, 3, 5, 64, device="cuda")
    y = ops.rms_norm(x, None, 1e-6)
    assert relerr(host(y), xo.rmsnorm(host(x), None, 1e-6)) <= FP32_TOL


def test_norm_cells_against_golden(golden):
    from xlstm_cuda.blocks import MultiHeadRMSNorm, RMSNormCell
    g = golden("norms")
    rn = RMSNormCell(96).cuda()
    rn.weight.data = dev(g["rms_w"])
    np.testing.assert_allclose(host(rn(dev(g["rms_x"]))), g["rms_y"], rtol=1e-5, atol=1e-6)
    mh = MultiHeadRMSNorm(4, 32).cuda()
    mh.weight.data = dev(g["mh_w"])
    np.testing.assert_allclose(host(mh(dev(g["mh_x"]))), g["mh_y"], rtol=1e-5, atol=1e-6)
    # permuted (non-contiguous) input, the layout the output cell hands over
    xp = dev(g["mh_x"]).permute(0, 2, 1, 3).contiguous().permute(0, 2, 1, 3)
    np.testing.assert_allclose(host(mh(xp)), g["mh_y"], rtol=1e-5, atol=1e-6)


# ---- output epilogue -------------------------------------------------------------------
def test_output_gate_golden(ops, golden):
    g = golden("glue_fp32")
    y = ops.mlstm_output_gate(dev(g["og_h"]), dev(g["og_pre"]), dev(g["og_w"]), float(g["og_eps"]))
    np.testing.assert_allclose(host(y), g["og_y"], rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("B,NH,S,dv", [(1, 8, 1, 512), (2, 4, 33, 64), (1, 2, 5, 1024), (3, 8, 130, 512), (2, 3, 7, 48),
                                       # more rows than warps in the grid: a warp walks several rows of its head
                                       (2, 8, 1500, 512), (2, 3, 2500, 48), (3, 5, 1111, 256)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_output_gate_shapes_and_strides(ops, B, NH, S, dv, dtype):
    rng = np.random.default_rng(B * 7 + NH * 11 + S * 13 + dv)
    h = rng.standard_normal((B, NH, S, dv)).astype(np.float32) * 2.0
    og = rng.standard_normal((B, S, NH * dv)).astype(np.float32) * 2.0
    w = rng.uniform(0.5, 1.5, NH * dv).astype(np.float32)
    if dtype == torch.bfloat16:
        h, og, w = bf(h), bf(og), bf(w)
    ref = xo.mlstm_output_gate(h, og, w, 1e-6)
    tol = FP32_TOL if dtype == torch.float32 else BF16_TOL
    y = ops.mlstm_output_gate(dev(h, dtype), dev(og, dtype), dev(w, dtype), 1e-6)
    assert y.shape == (B, S, NH * dv) and relerr(host(y), ref) <= tol
    # h as a permuted view of a [B,S,NH,dv] buffer (the layout the fused all-gather produces)
    hp = dev(h, dtype).permute(0, 2, 1, 3).contiguous().permute(0, 2, 1, 3)
    assert not hp.is_contiguous() or S == 1 or NH == 1
    y2 = ops.mlstm_output_gate(hp, dev(og, dtype), dev(w, dtype), 1e-6)
    assert torch.equal(y, y2)
    y3 = ops.mlstm_output_gate(dev(h, dtype), dev(og, dtype), None, 1e-6)
    assert relerr(host(y3), xo.mlstm_output_gate(h, og, None, 1e-6)) <= tol


# ---- SwiGLU gate ----------------------------------------------------------------------
def test_swiglu_golden(ops, golden):
    g = golden("glue_fp32")
    y = ops.swiglu(dev(g["sw_g"]), dev(g["sw_u"]))
    np.testing.assert_allclose(host(y), g["sw_y"], rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("rows,cols", [(1, 10944), (4, 64), (3, 41), (257, 2048),
                                       (4100, 10944), (40000, 1000)])   # the last two: the streamed kernel
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu_dense_and_column_blocks(ops, rows, cols, dtype):
    rng = np.random.default_rng(rows + cols)
    gu = rng.standard_normal((rows, 2 * cols)).astype(np.float32) * 3.0
    if dtype == torch.bfloat16:
        gu = bf(gu)
    ref = xo.swiglu(gu[:, :cols], gu[:, cols:])
    tol = FP32_TOL if dtype == torch.float32 else BF16_TOL
    t = dev(gu, dtype)
    y_blocks = ops.swiglu(t[:, :cols], t[:, cols:])              # the two halves of one GEMM output
    y_dense = ops.swiglu(t[:, :cols].contiguous(), t[:, cols:].contiguous())
    assert y_blocks.is_contiguous() and y_blocks.shape == (rows, cols)
    assert relerr(host(y_blocks), ref) <= tol and torch.equal(y_blocks, y_dense)


# ---- causal depthwise convolution -------------------------------------------------------
def test_causal_conv_golden(ops, golden):
    g = golden("glue_fp32")
    x, w, b = dev(g["conv_x"]), dev(g["conv_w"]), dev(g["conv_b"])
    np.testing.assert_allclose(host(ops.causal_conv1d(x, w, b)), g["conv_y"], rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(host(ops.causal_conv1d(x, w, b, silu=True)), g["conv_y_silu"], rtol=1e-5, atol=1e-6)
    # [C,1,K] weight of nn.Conv1d is accepted as is
    np.testing.assert_allclose(host(ops.causal_conv1d(x, w.view(-1, 1, 4), b)), g["conv_y"], rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("B,S,C,K", [(1, 1, 64, 4), (2, 2, 64, 4), (2, 16, 128, 4), (3, 17, 1024, 4), (2, 100, 40, 2),
                                     (1, 33, 256, 8), (2, 5, 64, 1),
                                     # long runs per thread: the shared-memory ring is refilled (32 / 64 / 128 tokens)
                                     (4, 4099, 1040, 4), (16, 4096, 1024, 4), (32, 4100, 1024, 3), (24, 2051, 512, 8)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_causal_conv_shapes_and_state(ops, B, S, C, K, dtype):
    rng = np.random.default_rng(B + 3 * S + 5 * C + 7 * K)
    x = rng.standard_normal((B, S, C)).astype(np.float32)
    w = (rng.standard_normal((C, K)) * 0.5).astype(np.float32)
    b = (rng.standard_normal(C) * 0.1).astype(np.float32)
    st = rng.standard_normal((B, K - 1, C)).astype(np.float32)
    if dtype == torch.bfloat16:
        x, w, b, st = bf(x), bf(w), bf(b), bf(st)
    tol = FP32_TOL if dtype == torch.float32 else BF16_TOL
    ref, ref_st = xo.causal_conv1d(x, w, b, state=st, silu=True, return_state=True)
    y, st1 = ops.causal_conv1d(dev(x, dtype), dev(w, dtype), dev(b, dtype), silu=True, state=dev(st, dtype),
                               return_state=True)
    assert relerr(host(y), ref) <= tol
    if K > 1:
        np.testing.assert_array_equal(host(st1), ref_st)          # the state is a copy of inputs: exact
    y0 = ops.causal_conv1d(dev(x, dtype), dev(w, dtype), None)    # no bias, zero history, no activation
    assert relerr(host(y0), xo.causal_conv1d(x, w, None)) <= tol


def test_causal_conv_token_by_token_equals_sequence(ops):
    rng = np.random.default_rng(5)
    B, S, C, K = 2, 40, 128, 4
    x = dev(rng.standard_normal((B, S, C)).astype(np.float32))
    w = dev((rng.standard_normal((C, K)) * 0.5).astype(np.float32))
    b = dev((rng.standard_normal(C) * 0.1).astype(np.float32))
    full = ops.causal_conv1d(x, w, b, silu=True)
    st, outs = None, []
    for t in range(S):
        y, st = ops.causal_conv1d(x[:, t:t + 1], w, b, silu=True, state=st, return_state=True)
        outs.append(y)
    assert torch.equal(torch.cat(outs, 1), full)
    y1, st = ops.causal_conv1d(x[:, :23], w, b, silu=True, return_state=True)
    y2 = ops.causal_conv1d(x[:, 23:], w, b, silu=True, state=st)
    assert torch.equal(torch.cat([y1, y2], 1), full)


def test_glue_rejects_cpu_tensors(ops):
    with pytest.raises(RuntimeError):
        ops.rms_norm(torch.zeros(2, 8), None)
    with pytest.raises(RuntimeError):
        ops.swiglu(torch.zeros(2, 8), torch.zeros(2, 8))


# ---- single-token Linear (weight-streaming pass with folded norm / residual / SwiGLU) ----------
@pytest.mark.parametrize("M,N,K", [(1, 4096, 4096), (1, 12304, 4096), (2, 4096, 10944), (4, 264, 520), (3, 33, 4096),
                                   (4, 300, 10944), (1, 500, 16), (2, 1000, 2056)])
def test_linear_token_plain_bias_residual(ops, M, N, K):
    rng = np.random.default_rng(M * 7 + N + K)
    x = bf(rng.standard_normal((M, K)).astype(np.float32))
    W = bf((rng.standard_normal((N, K)) * 0.05).astype(np.float32))
    b = bf((rng.standard_normal(N) * 0.1).astype(np.float32))
    r = bf(rng.standard_normal((M, N)).astype(np.float32))
    t = torch.bfloat16
    ref = xo.linear(x, W, b)
    y = ops.linear_token(dev(W, t), dev(x, t), bias=dev(b, t))
    assert y.shape == (M, N) and relerr(host(y), ref) <= BF16_TOL
    y0 = ops.linear_token(dev(W, t), dev(x, t))
    assert relerr(host(y0), xo.linear(x, W)) <= BF16_TOL
    yr = ops.linear_token(dev(W, t), dev(x, t), bias=dev(b, t), residual=dev(r, t))
    assert relerr(host(yr), bf(ref) + r) <= BF16_TOL


@pytest.mark.parametrize("M,F,K", [(1, 10944, 4096), (2, 320, 256), (4, 64, 4096)])
def test_linear_token_norm_and_swiglu(ops, M, F, K):
    rng = np.random.default_rng(M + F + K)
    x = bf(rng.standard_normal((M, K)).astype(np.float32) * 3.0)
    nw = bf(rng.uniform(0.5, 1.5, K).astype(np.float32))
    W = bf((rng.standard_normal((2 * F, K)) * 0.05).astype(np.float32))
    t = torch.bfloat16
    xn = bf(xo.rmsnorm(x, nw, 1e-6))
    # norm folded into the projection
    y = ops.linear_token(dev(W[:F], t), dev(x, t), norm_weight=dev(nw, t), norm_eps=1e-6)
    assert relerr(host(y), xo.linear(xn, W[:F])) <= BF16_TOL
    # ... and the SwiGLU gate on the two stacked up projections
    g, u = bf(xo.linear(xn, W[:F])), bf(xo.linear(xn, W[F:]))
    act = ops.linear_token(dev(W, t), dev(x, t), norm_weight=dev(nw, t), norm_eps=1e-6, swiglu_pair=True)
    assert act.shape == (M, F) and relerr(host(act), xo.swiglu(g, u)) <= BF16_TOL
    # equals the separate kernels up to bf16 rounding of the same intermediate values
    sep = ops.swiglu(*torch.nn.functional.linear(ops.rms_norm(dev(x, t), dev(nw, t), 1e-6), dev(W, t)).split(F, dim=-1))
    assert relerr(host(act), host(sep)) <= BF16_TOL


def test_linear_token_rejects_what_it_does_not_do(ops):
    t = torch.bfloat16
    with pytest.raises(ValueError):
        ops.linear_token(torch.zeros(8, 16, device="cuda", dtype=t), torch.zeros(5, 16, device="cuda", dtype=t))
    with pytest.raises(TypeError):
        ops.linear_token(torch.zeros(8, 16, device="cuda"), torch.zeros(1, 16, device="cuda"))
