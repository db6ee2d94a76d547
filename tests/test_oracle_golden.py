"""The CPU oracle against fixtures produced by the reference's own classes (CPU only)."""
import numpy as np
import pytest

from conftest import relerr
from oracle import oracle as xo

FP32 = 1e-5  # oracle vs reference on identical fp32 inputs (observed ~1e-6)


def test_mlstm_recurrent_config1(golden):
    g = golden("mlstm_c1_fp32")
    h, (C, n, m) = xo.mlstm_recurrent(g["q"], g["k"], g["v"], g["i"], g["f"])
    assert relerr(h, g["h"]) < FP32
    assert relerr(C, g["C"]) < FP32
    assert relerr(n, g["n"]) < FP32
    assert np.abs(m - g["m"]).max() < FP32


def test_mlstm_chunkwise_equals_reference_recurrent(golden):
    g = golden("mlstm_c1_fp32")
    for L in (16, 64, 128):
        h, (C, n, m) = xo.mlstm_chunkwise(g["q"], g["k"], g["v"], g["i"], g["f"], chunk_size=L)
        assert relerr(h, g["h"]) < FP32
        assert relerr(C, g["C"]) < FP32
        assert relerr(n, g["n"]) < FP32
        assert np.abs(m - g["m"]).max() < FP32


def test_mlstm_ragged_with_initial_state(golden):
    g = golden("mlstm_ragged_fp32")
    st = (g["C0"], g["n0"], g["m0"])
    h, (C, n, m) = xo.mlstm_recurrent(g["q"], g["k"], g["v"], g["i"], g["f"], st)
    assert relerr(h, g["h"]) < FP32 and relerr(C, g["C"]) < FP32 and relerr(n, g["n"]) < FP32
    assert np.abs(m - g["m"]).max() < FP32
    # 32 chunked tokens + 5 stepwise tail tokens, the dispatch rule of the reference neuron
    sl = lambda a, s: a[:, :, s]
    h1, st1 = xo.mlstm_chunkwise(*(sl(g[x], slice(0, 32)) for x in "qkvif"), state=st, chunk_size=16)
    h2, st2 = xo.mlstm_recurrent(*(sl(g[x], slice(32, 37)) for x in "qkvif"), state=st1)
    assert relerr(np.concatenate([h1, h2], 2), g["h"]) < FP32
    assert relerr(st2[0], g["C"]) < FP32


@pytest.mark.parametrize("name", ["mlstm_step_bf16", "mlstm_step_7b"])
def test_mlstm_decode_steps(golden, name):
    g = golden(name)
    st = (g["C0"], g["n0"], g["m0"])
    st_b = st
    hs, hs_b = [], []
    for t in range(g["q"].shape[2]):
        args = [g[x][:, :, t:t + 1] for x in "qkvif"]
        h, st = xo.mlstm_recurrent(*args, state=st)
        hb, st_b = xo.mlstm_recurrent(*args, state=st_b, emulate_bf16=True)
        hs.append(h)
        hs_b.append(hb)
    h, hb = np.concatenate(hs, 2), np.concatenate(hs_b, 2)
    assert relerr(h, g["h_fp32"]) < FP32 and relerr(st[0], g["C_fp32"]) < FP32
    assert relerr(st[1], g["n_fp32"]) < FP32 and np.abs(st[2] - g["m_fp32"]).max() < FP32
    # bf16 emulation: same cast points as the reference, so at most an ulp or two of bf16 apart
    assert relerr(hb, g["h_bf16"]) < 8e-3
    assert relerr(st_b[0], g["C_bf16"]) < 1e-5
    assert relerr(st_b[1], g["n_bf16"]) < 1e-5
    assert np.abs(st_b[2] - g["m_bf16"]).max() < 1e-5


@pytest.mark.parametrize("tag", ["a", "b", "x"])
def test_slstm_scan(golden, tag):
    g = golden("slstm_a")
    h, (c, n, m) = xo.slstm_scan(g[f"{tag}_z"], g[f"{tag}_i"], g[f"{tag}_f"], g[f"{tag}_o"],
                                 (g[f"{tag}_c0"], g[f"{tag}_n0"], g[f"{tag}_m0"]))
    tol = 1e-4 if tag == "x" else 1e-5  # tolerances of the reference's own sLSTM kernel test
    assert relerr(h, g[f"{tag}_h"]) < tol and relerr(c, g[f"{tag}_c"]) < tol
    assert relerr(n, g[f"{tag}_n"]) < tol and np.abs(m - g[f"{tag}_m"]).max() < tol


def test_slstm_scan_zero_state(golden):
    g = golden("slstm_a")
    h, (c, n, m) = xo.slstm_scan(g["z_z"], g["z_i"], g["z_f"], g["z_o"], None)
    assert relerr(h, g["z_h"]) < 1e-5 and relerr(c, g["z_c"]) < 1e-5 and relerr(n, g["z_n"]) < 1e-5


def test_slstm_recurrent_block_diagonal(golden):
    g = golden("slstm_b")
    nh = int(g["num_heads"])
    hs, (c, n, h, m) = xo.slstm_recurrent(g["gx"], g["R"], g["rb"], None, nh, 15.0)
    assert relerr(hs, g["hs"]) < FP32
    for got, key in ((c, "c"), (n, "n"), (h, "h"), (m, "m")):
        assert relerr(got, g[key]) < FP32
    hs2, st2 = xo.slstm_recurrent(g["gx2"], g["R"], g["rb"], (c, n, h, m), nh, 15.0)
    assert relerr(hs2, g["hs2"]) < FP32
    for got, key in zip(st2, ("c2", "n2", "h2", "m2")):
        assert relerr(got, g[key]) < FP32


def test_known_answer_inputs_of_the_reference_tests(golden):
    g = golden("kat")
    # soft-cap value lists
    for tag in ("small", "large", "edge"):
        y = xo.softcap(g[f"softcap_{tag}_x"], float(g[f"softcap_{tag}_cap"]))
        np.testing.assert_allclose(y, g[f"softcap_{tag}_y"], rtol=1e-6, atol=1e-6)
    # gate normalisation triples, driven through one mLSTM step with dqk=dv=1:
    # m1 = max(logsig(f)+m, i); C1 = fexp*C0 + iexp*k*v with C0=1,k=v=1 -> fexp + iexp
    for r in range(3):
        i, f, m0 = (g[k][r:r + 1].reshape(1, 1, 1) for k in ("gate_i", "gate_f", "gate_m"))
        one = np.ones((1, 1, 1, 1), np.float32)
        _, (C, n, m) = xo.mlstm_recurrent(one, one, one, i, f, (one, np.zeros((1, 1, 1), np.float32), m0.reshape(1, 1)))
        np.testing.assert_allclose(m.ravel(), g["gate_mnew"][r], rtol=1e-6, atol=1e-7)
        np.testing.assert_allclose(C.ravel(), g["gate_fexp"][r] + g["gate_iexp"][r], rtol=1e-6, atol=1e-7)
        np.testing.assert_allclose(n.ravel(), g["gate_iexp"][r], rtol=1e-6, atol=1e-7)
    # log-sigmoid points: f = x, i = -inf-ish so that m1 = logsig(x) + 0
    x = g["logsig_x"]
    for xv, yv in zip(x, g["logsig_y"]):
        one = np.ones((1, 1, 1, 1), np.float32)
        _, (_, _, m) = xo.mlstm_recurrent(one, one, one, np.full((1, 1, 1), -1e30, np.float32),
                                          np.full((1, 1, 1), xv, np.float32))
        np.testing.assert_allclose(m.ravel()[0], yv, rtol=1e-6, atol=1e-6)


def test_norm_glue(golden):
    g = golden("norms")
    np.testing.assert_allclose(xo.rmsnorm(g["rms_x"], g["rms_w"], 1e-6), g["rms_y"], rtol=1e-5, atol=1e-6)
    y = xo.multihead_rmsnorm(g["mh_x"], g["mh_w"], 1e-6)
    np.testing.assert_allclose(y, g["mh_y"], rtol=1e-5, atol=1e-6)


def test_output_gate_conv_swiglu_glue(golden):
    """The oracle's restatements of the kernels either side of the cells against the reference's own
    modules (tests/golden/make_golden_glue.py)."""
    g = golden("glue_fp32")
    y = xo.mlstm_output_gate(g["og_h"], g["og_pre"], g["og_w"], float(g["og_eps"]))
    np.testing.assert_allclose(y, g["og_y"], rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(xo.swiglu(g["sw_g"], g["sw_u"]), g["sw_y"], rtol=1e-5, atol=1e-6)
    x, w, b = g["conv_x"], g["conv_w"], g["conv_b"]
    np.testing.assert_allclose(xo.causal_conv1d(x, w, b), g["conv_y"], rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(xo.causal_conv1d(x, w, b, silu=True), g["conv_y_silu"], rtol=1e-5, atol=1e-6)
    # carried state: two calls give the one-call result (the reference keeps no state; this is the
    # property the stateful decode variant must have)
    y1, st = xo.causal_conv1d(x[:, :20], w, b, silu=True, return_state=True)
    y2, st2 = xo.causal_conv1d(x[:, 20:], w, b, state=st, silu=True, return_state=True)
    np.testing.assert_allclose(np.concatenate([y1, y2], 1), g["conv_y_silu"], rtol=1e-5, atol=1e-6)
    np.testing.assert_array_equal(st2, x[:, -3:])
    # single tokens shift the state
    st = None
    for t in range(5):
        yt, st = xo.causal_conv1d(x[:, t:t + 1], w, b, state=st, return_state=True)
        np.testing.assert_allclose(yt[:, 0], g["conv_y"][:, t], rtol=1e-5, atol=1e-6)
