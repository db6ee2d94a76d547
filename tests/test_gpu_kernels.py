"""GPU parity: every kernel through the C ABI against the CPU oracle and the golden fixtures.

Tolerances (max|a-b| / max|b|): fp32 1e-4 on h, C, n and 1e-4 absolute on m;
bf16 activations with fp32 state 2e-2.
"""
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from conftest import relerr
from oracle import oracle as xo

pytestmark = pytest.mark.gpu

FP32_TOL = 1e-4
BF16_TOL = 2e-2


def dev(a, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a)).to("cuda", dtype)


def host(t):
    return t.detach().float().cpu().numpy()


def gates(rng, shape, fmean=3.0):
    i = 15.0 * np.tanh(rng.standard_normal(shape).astype(np.float32) / 15.0)
    f = 15.0 * np.tanh((rng.standard_normal(shape).astype(np.float32) + fmean) / 15.0)
    return i, f


@pytest.fixture(scope="module")
def ops():
    from xlstm_cuda import ops as _ops
    return _ops


# ---- soft-cap ----------------------------------------------------------------
@pytest.mark.parametrize("n", [1, 7, 4096, 50304, 1 << 20 | 3])
@pytest.mark.parametrize("cap", [15.0, 30.0])
def test_softcap_fp32(ops, n, cap):
    rng = np.random.default_rng(n)
    x = (rng.standard_normal(n) * 20).astype(np.float32)
    y = host(ops.softcap(dev(x), cap))
    np.testing.assert_allclose(y, xo.softcap(x, cap), rtol=1e-5, atol=1e-5)


def test_softcap_bf16_and_unaligned_and_kat(ops, golden):
    rng = np.random.default_rng(0)
    x = xo.bf16_round((rng.standard_normal(10001) * 20).astype(np.float32))
    y = host(ops.softcap(dev(x, torch.bfloat16), 30.0))
    assert relerr(y, xo.softcap(x, 30.0)) < 4e-3
    base = dev(np.arange(1003, dtype=np.float32) / 10 - 50)
    view = base[1:]  # 4-byte aligned only
    np.testing.assert_allclose(host(ops.softcap(view, 15.0)), xo.softcap(host(view), 15.0), rtol=1e-5, atol=1e-5)
    g = golden("kat")
    for tag in ("small", "large", "edge"):
        y = host(ops.softcap(dev(g[f"softcap_{tag}_x"]), float(g[f"softcap_{tag}_cap"])))
        np.testing.assert_allclose(y, g[f"softcap_{tag}_y"], rtol=1e-6, atol=1e-6)
    x = dev(np.ones(5, np.float32))
    assert ops.softcap(x, None) is x and ops.softcap(x, 0.0) is x
    assert ops.softcap(torch.empty(0, device="cuda"), 15.0).numel() == 0


# ---- decode step ------------------------------------------------------------------
def run_steps(ops, g, dtype, inplace=False):
    st = (dev(g["C0"]), dev(g["n0"]), dev(g["m0"]))
    hs = []
    for t in range(g["q"].shape[2]):
        a = [dev(g[x][:, :, t], dtype) for x in "qkvif"]
        h, st = ops.mlstm_step(*a, state=st, inplace=inplace)
        hs.append(host(h))
    return np.stack(hs, 2), tuple(host(s) for s in st)


@pytest.mark.parametrize("name", ["mlstm_step_bf16", "mlstm_step_7b"])
def test_mlstm_step_against_reference_fixture(ops, golden, name):
    g = golden(name)
    # fp32 activations (bf16-representable values): 1e-4 against the reference's fp32 run
    h, (C, n, m) = run_steps(ops, g, torch.float32)
    assert relerr(h, g["h_fp32"]) < FP32_TOL and relerr(C, g["C_fp32"]) < FP32_TOL
    assert relerr(n, g["n_fp32"]) < FP32_TOL and np.abs(m - g["m_fp32"]).max() < FP32_TOL
    # bf16 activations, fp32 state: 2e-2 against the reference's bf16-compute run and its fp32 run
    h, (C, n, m) = run_steps(ops, g, torch.bfloat16, inplace=True)
    assert relerr(h, g["h_bf16"]) < BF16_TOL and relerr(h, g["h_fp32"]) < BF16_TOL
    assert relerr(C, g["C_bf16"]) < BF16_TOL and relerr(n, g["n_bf16"]) < BF16_TOL
    assert np.abs(m - g["m_bf16"]).max() < BF16_TOL


@pytest.mark.parametrize("B,NH,dqk,dv", [(16, 8, 256, 512), (3, 5, 64, 64), (2, 2, 100, 36), (1, 1, 512, 1024)])
def test_mlstm_step_against_oracle(ops, B, NH, dqk, dv):
    rng = np.random.default_rng(B * 1000 + dqk)
    q, k = (rng.standard_normal((B, NH, 1, dqk)).astype(np.float32) for _ in range(2))
    v = rng.standard_normal((B, NH, 1, dv)).astype(np.float32)
    i, f = gates(rng, (B, NH, 1))
    st = (rng.standard_normal((B, NH, dqk, dv)).astype(np.float32) * 0.1,
          rng.standard_normal((B, NH, dqk)).astype(np.float32) * 0.1, rng.standard_normal((B, NH)).astype(np.float32))
    for state in (st, None):
        h_ref, st_ref = xo.mlstm_recurrent(q, k, v, i, f, state)
        h, st_new = ops.mlstm_step(dev(q[:, :, 0]), dev(k[:, :, 0]), dev(v[:, :, 0]), dev(i[:, :, 0]), dev(f[:, :, 0]),
                                   None if state is None else tuple(dev(s) for s in state))
        assert relerr(host(h), h_ref[:, :, 0]) < FP32_TOL
        for got, want in zip(st_new, st_ref):
            assert relerr(host(got), want) < FP32_TOL


def test_mlstm_step_config2_256_steps_bf16(ops):
    """BASELINE config 2: B=16, NH=8, 256/512, bf16 activations, fp32 state, 256 carried steps."""
    B, NH, dqk, dv, T = 16, 8, 256, 512, 256
    g = torch.Generator().manual_seed(1)
    C = torch.randn(B, NH, dqk, dv, generator=g) * 0.1
    n = torch.randn(B, NH, dqk, generator=g) * 0.1
    m = torch.zeros(B, NH)
    q = torch.randn(B, NH, T, dqk, generator=g).bfloat16()
    k = torch.randn(B, NH, T, dqk, generator=g).bfloat16()
    v = torch.randn(B, NH, T, dv, generator=g).bfloat16()
    i = (15 * torch.tanh(torch.randn(B, NH, T, generator=g) / 15)).bfloat16()
    f = (15 * torch.tanh((torch.randn(B, NH, T, generator=g) + 3) / 15)).bfloat16()
    h_ref, st_ref = xo.mlstm_recurrent(q.float().numpy(), k.float().numpy(), v.float().numpy(), i.float().numpy(),
                                       f.float().numpy(), (C.numpy(), n.numpy(), m.numpy()))
    st = (C.cuda(), n.cuda(), m.cuda())
    qd, kd, vd, idv, fd = (t.cuda() for t in (q, k, v, i, f))
    hs = []
    for t in range(T):
        h, st = ops.mlstm_step(qd[:, :, t], kd[:, :, t], vd[:, :, t], idv[:, :, t], fd[:, :, t], st, inplace=True)
        hs.append(h)
    h = host(torch.stack(hs, 2))
    assert relerr(h, h_ref) < BF16_TOL
    assert relerr(host(st[0]), st_ref[0]) < FP32_TOL * 10 and relerr(host(st[1]), st_ref[1]) < FP32_TOL * 10
    assert np.abs(host(st[2]) - st_ref[2]).max() < 1e-3


def test_mlstm_step_layer_ring_overlapped_launches(ops):
    """A stack of layers stepped token by token with state_settled=True (each launch may start fetching its
    state while the launch before it - another layer - drains), eagerly and replayed as a CUDA graph, against
    the oracle stepping every layer on its own; and the same state stepped twice in a row WITHOUT the promise."""
    B, NH, dqk, dv, LAYERS, T = 2, 4, 128, 256, 3, 6
    rng = np.random.default_rng(77)
    q, k = (rng.standard_normal((LAYERS, B, NH, T, dqk)).astype(np.float32) for _ in range(2))
    v = rng.standard_normal((LAYERS, B, NH, T, dv)).astype(np.float32)
    i, f = gates(rng, (LAYERS, B, NH, T))
    st0 = [(rng.standard_normal((B, NH, dqk, dv)).astype(np.float32) * 0.1,
            rng.standard_normal((B, NH, dqk)).astype(np.float32) * 0.1, np.zeros((B, NH), np.float32)) for _ in range(LAYERS)]
    ref = [xo.mlstm_recurrent(q[l], k[l], v[l], i[l], f[l], st0[l]) for l in range(LAYERS)]
    qd, kd, vd, idv, fd = (dev(a) for a in (q, k, v, i, f))

    def run(states, hs):
        for t in range(T):
            for l in range(LAYERS):
                h, states[l] = ops.mlstm_step(qd[l, :, :, t], kd[l, :, :, t], vd[l, :, :, t], idv[l, :, :, t], fd[l, :, :, t],
                                              states[l], state_settled=True)
                hs[l][:, :, t] = h

    states = [tuple(dev(a) for a in st) for st in st0]
    hs = [torch.empty(B, NH, T, dv, device="cuda") for _ in range(LAYERS)]
    run(states, hs)
    for l in range(LAYERS):
        assert relerr(host(hs[l]), ref[l][0]) < FP32_TOL
        for got, want in zip(states[l], ref[l][1]):
            assert relerr(host(got), want) < FP32_TOL

    # the same launches as one CUDA graph (the decode loop's form): bit-identical to the eager run
    states_g = [tuple(dev(a) for a in st) for st in st0]
    hs_g = [torch.empty(B, NH, T, dv, device="cuda") for _ in range(LAYERS)]
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    final = []
    with torch.cuda.graph(graph, stream=side):
        work = list(states_g)
        run(work, hs_g)
        final = work
    torch.cuda.current_stream().wait_stream(side)
    graph.replay()
    torch.cuda.synchronize()
    for l in range(LAYERS):
        assert torch.equal(hs_g[l], hs[l])
        for got, want in zip(final[l], states[l]):
            assert torch.equal(got, want)

    # one state stepped T times back to back, no promise: every launch reads what the one before it wrote
    st = tuple(dev(a) for a in st0[0])
    out = []
    for t in range(T):
        h, st = ops.mlstm_step(qd[0, :, :, t], kd[0, :, :, t], vd[0, :, :, t], idv[0, :, :, t], fd[0, :, :, t], st, inplace=True)
        out.append(h)
    assert relerr(host(torch.stack(out, 2)), ref[0][0]) < FP32_TOL


@pytest.mark.parametrize("group", [1, 3])
def test_decode_pipeline_host_fed(ops, group):
    """runtime.DecodePipeline: pinned host q,k,v,i,f in, h out, every step; eager enqueue and the captured graph
    (steps travelling in groups) must both reproduce the plain decode step bit for bit, states included."""
    from xlstm_cuda.runtime import DecodePipeline
    B, NH, dqk, dv, LAYERS, T = 2, 4, 128, 256, 3, 4
    g = torch.Generator().manual_seed(5)
    steps = LAYERS * T
    q = torch.randn(steps, B, NH, dqk, generator=g).bfloat16()
    k = torch.randn(steps, B, NH, dqk, generator=g).bfloat16()
    v = torch.randn(steps, B, NH, dv, generator=g).bfloat16()
    i = torch.randn(steps, B, NH, generator=g).bfloat16()
    f = (torch.randn(steps, B, NH, generator=g) + 3).bfloat16()

    def fresh_states():
        gs = torch.Generator().manual_seed(6)
        return [[(torch.randn(B, NH, dqk, dv, generator=gs).cuda() * 0.1, torch.randn(B, NH, dqk, generator=gs).cuda() * 0.1,
                  torch.zeros(B, NH, device="cuda")),
                 tuple(torch.empty(s, device="cuda") for s in ((B, NH, dqk, dv), (B, NH, dqk), (B, NH)))] for _ in range(LAYERS)]

    # reference: the plain op, layer by layer
    st = [s[0] for s in fresh_states()]
    h_ref = []
    for t in range(steps):
        l = t % LAYERS
        h, st[l] = ops.mlstm_step(q[t].cuda(), k[t].cuda(), v[t].cuda(), i[t].cuda(), f[t].cuda(), st[l])
        h_ref.append(h)

    for captured in (False, True):
        pipe = DecodePipeline(B, NH, dqk, dv, "cuda", group=group)
        packed = [pipe.pack(q[t], k[t], v[t], i[t], f[t]) for t in range(steps)]
        h_host = [torch.empty(B, NH, dv, dtype=torch.bfloat16).pin_memory() for _ in range(steps)]
        states = fresh_states()
        side = [0] * LAYERS
        items = []
        for t in range(steps):
            l = t % LAYERS
            items.append((packed[t], states[l][side[l]], states[l][side[l] ^ 1], h_host[t], True))
            side[l] ^= 1
        if captured:
            graph = pipe.capture(items)
            graph.replay()
            torch.cuda.synchronize()
        else:
            for lo in range(0, steps, group):
                pipe.step_group(items[lo:lo + group])
            pipe.synchronize()
        for t in range(steps):
            assert torch.equal(h_host[t], h_ref[t].cpu()), (captured, t)
        for l in range(LAYERS):
            for got, want in zip(states[l][side[l]], st[l]):
                assert torch.equal(got, want)


@pytest.mark.parametrize("B,NH,dqk,dv", [(2, 4, 128, 256), (1, 8, 256, 512), (3, 2, 64, 96)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_mlstm_step_with_fused_output_epilogue(ops, B, NH, dqk, dv, dtype):
    """xlstm_mlstm_step_gated (norm x weight x sigmoid(output gate) applied inside the step kernel, the head's
    CTAs meeting through their cluster) against the two separate kernels and against the oracle; the output gate
    is handed over as a column block of a wider projection output, as the block does."""
    rng = np.random.default_rng(B * 100 + dv)
    rnd = (lambda a: xo.bf16_round(a)) if dtype == torch.bfloat16 else (lambda a: a)
    q, k = (rnd(rng.standard_normal((B, NH, dqk)).astype(np.float32)) for _ in range(2))
    v = rnd(rng.standard_normal((B, NH, dv)).astype(np.float32))
    i, f = (rnd(a[:, :, 0]) for a in gates(rng, (B, NH, 1)))
    wide = rnd(rng.standard_normal((B, NH * dv + 24)).astype(np.float32) * 2.0)
    og = wide[:, 16:16 + NH * dv]
    w = rnd(rng.uniform(0.5, 1.5, NH * dv).astype(np.float32))
    st = (rng.standard_normal((B, NH, dqk, dv)).astype(np.float32) * 0.1,
          rng.standard_normal((B, NH, dqk)).astype(np.float32) * 0.1, rng.standard_normal((B, NH)).astype(np.float32))
    d = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dtype).cuda()
    wide_d = d(wide)
    for state in (st, None):
        sd = None if state is None else tuple(dev(x) for x in state)
        h, st_ref = ops.mlstm_step(d(q), d(k), d(v), d(i), d(f), sd)
        y_ref = ops.mlstm_output_gate(h.unsqueeze(2), wide_d[:, 16:16 + NH * dv].unsqueeze(1), d(w), 1e-6)[:, 0]
        y, st_new = ops.mlstm_step_gated(d(q), d(k), d(v), d(i), d(f), wide_d[:, 16:16 + NH * dv], d(w), sd, norm_eps=1e-6)
        tol = FP32_TOL if dtype == torch.float32 else BF16_TOL
        assert y.shape == (B, NH * dv) and relerr(host(y), host(y_ref)) <= tol
        for got, want in zip(st_new, st_ref):
            assert torch.equal(got, want)
        # and against the oracle: recurrent step, then the epilogue restated on the host
        h_o, _ = xo.mlstm_recurrent(q[:, :, None], k[:, :, None], v[:, :, None], i[:, :, None], f[:, :, None], state)
        y_o = xo.mlstm_output_gate(rnd(h_o), og[:, None, :], w, 1e-6)[:, 0]
        assert relerr(host(y), y_o) <= tol * (1 if dtype == torch.float32 else 2)


# ---- chunkwise -------------------------------------------------------------------
def test_chunkwise_config1_fp32(ops, golden):
    g = golden("mlstm_c1_fp32")
    for L in (64, 32, 128):   # 128: beyond the exact kernel's tile, walked in tiles of 64
        h, st = ops.mlstm_chunkwise(*(dev(g[x]) for x in "qkvif"), state=None, chunk_size=L)
        assert relerr(host(h), g["h"]) < FP32_TOL
        assert relerr(host(st[0]), g["C"]) < FP32_TOL and relerr(host(st[1]), g["n"]) < FP32_TOL
        assert np.abs(host(st[2]) - g["m"]).max() < FP32_TOL


def test_chunkwise_ragged_with_state_fp32(ops, golden):
    g = golden("mlstm_ragged_fp32")
    st0 = tuple(dev(g[x]) for x in ("C0", "n0", "m0"))
    for L in (64, 16, 7):
        h, st = ops.mlstm_chunkwise(*(dev(g[x]) for x in "qkvif"), state=st0, chunk_size=L)
        assert relerr(host(h), g["h"]) < FP32_TOL
        assert relerr(host(st[0]), g["C"]) < FP32_TOL and relerr(host(st[1]), g["n"]) < FP32_TOL
        assert np.abs(host(st[2]) - g["m"]).max() < FP32_TOL


@pytest.mark.parametrize("B,NH,S,dqk,dv", [(1, 2, 128, 256, 512), (2, 1, 70, 128, 192), (1, 1, 1, 64, 64)])
def test_chunkwise_against_oracle_and_strided_inputs(ops, B, NH, S, dqk, dv):
    rng = np.random.default_rng(S)
    # projection-style layout [B,S,NH,d], handed over as a permuted view
    q, k = (rng.standard_normal((B, S, NH, dqk)).astype(np.float32) for _ in range(2))
    v = rng.standard_normal((B, S, NH, dv)).astype(np.float32)
    i, f = gates(rng, (B, S, NH))
    tr = lambda a: np.ascontiguousarray(np.moveaxis(a, 1, 2))
    h_ref, st_ref = xo.mlstm_recurrent(tr(q), tr(k), tr(v), tr(i), tr(f))
    h, st = ops.mlstm_chunkwise(dev(q).permute(0, 2, 1, 3), dev(k).permute(0, 2, 1, 3), dev(v).permute(0, 2, 1, 3),
                                dev(i).permute(0, 2, 1), dev(f).permute(0, 2, 1))
    assert relerr(host(h), h_ref) < FP32_TOL
    for got, want in zip(st, st_ref):
        assert relerr(host(got), want) < FP32_TOL
    # run twice: bitwise identical
    h2, _ = ops.mlstm_chunkwise(dev(q).permute(0, 2, 1, 3), dev(k).permute(0, 2, 1, 3), dev(v).permute(0, 2, 1, 3),
                                dev(i).permute(0, 2, 1), dev(f).permute(0, 2, 1))
    assert torch.equal(h, h2)


def test_chunkwise_equals_steps_and_split_sequence(ops):
    """chunkwise(S) == S decode steps == chunkwise(S1) then chunkwise(S2) with the carried state."""
    rng = np.random.default_rng(5)
    B, NH, S, dqk, dv = 2, 2, 96, 64, 128
    q, k = (dev(rng.standard_normal((B, NH, S, dqk)).astype(np.float32)) for _ in range(2))
    v = dev(rng.standard_normal((B, NH, S, dv)).astype(np.float32))
    i, f = (dev(a) for a in gates(rng, (B, NH, S)))
    h, st = ops.mlstm_chunkwise(q, k, v, i, f)
    h1, st1 = ops.mlstm_chunkwise(q[:, :, :50], k[:, :, :50], v[:, :, :50], i[:, :, :50], f[:, :, :50])
    h2, st2 = ops.mlstm_chunkwise(q[:, :, 50:], k[:, :, 50:], v[:, :, 50:], i[:, :, 50:], f[:, :, 50:], st1)
    assert relerr(host(torch.cat([h1, h2], 2)), host(h)) < FP32_TOL
    assert relerr(host(st2[0]), host(st[0])) < FP32_TOL
    s, hs = None, []
    for t in range(S):
        ht, s = ops.mlstm_step(q[:, :, t], k[:, :, t], v[:, :, t], i[:, :, t], f[:, :, t], s)
        hs.append(ht)
    assert relerr(host(torch.stack(hs, 2)), host(h)) < FP32_TOL
    assert relerr(host(s[0]), host(st[0])) < FP32_TOL and np.abs(host(s[2]) - host(st[2])).max() < FP32_TOL


def test_chunkwise_bf16_head_shape(ops):
    rng = np.random.default_rng(8)
    B, NH, S, dqk, dv = 1, 2, 256, 256, 512
    q, k = (xo.bf16_round(rng.standard_normal((B, NH, S, dqk)).astype(np.float32)) for _ in range(2))
    v = xo.bf16_round(rng.standard_normal((B, NH, S, dv)).astype(np.float32))
    i, f = (xo.bf16_round(a) for a in gates(rng, (B, NH, S)))
    h_ref, st_ref = xo.mlstm_recurrent(q, k, v, i, f)
    h, st = ops.mlstm_chunkwise(*(dev(a, torch.bfloat16) for a in (q, k, v, i, f)))
    assert relerr(host(h), h_ref) < BF16_TOL
    assert relerr(host(st[0]), st_ref[0]) < BF16_TOL and relerr(host(st[1]), st_ref[1]) < BF16_TOL
    assert np.abs(host(st[2]) - st_ref[2]).max() < BF16_TOL


def recurrent_fp64(q, k, v, i, f, eps=1e-6):
    """The recurrence in float64 (numpy), for inputs where fp32 itself is the limit."""
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


def test_extreme_gates_stay_finite(ops):
    """Gates at the soft-cap limits (+-15) over many chunks: no inf/nan.  Here the fp32 recurrence
    itself is 1.2e-4 away from exact arithmetic (sums near 1e3 inside exp), so the kernel is held to
    1e-4 against a float64 evaluation and to 5e-4 against the fp32 oracle."""
    rng = np.random.default_rng(3)
    B, NH, S, dqk, dv = 1, 2, 192, 64, 64
    q, k = (rng.standard_normal((B, NH, S, dqk)).astype(np.float32) for _ in range(2))
    v = rng.standard_normal((B, NH, S, dv)).astype(np.float32)
    i = rng.choice([-15.0, 0.0, 15.0], size=(B, NH, S)).astype(np.float32)
    f = rng.choice([-15.0, 0.0, 15.0], size=(B, NH, S)).astype(np.float32)
    h_ref, st_ref = xo.mlstm_recurrent(q, k, v, i, f)
    h64, st64 = recurrent_fp64(q, k, v, i, f)
    h, st = ops.mlstm_chunkwise(*(dev(a) for a in (q, k, v, i, f)))
    assert np.isfinite(host(h)).all()
    assert relerr(host(h), h64) < FP32_TOL and relerr(host(st[0]), st64[0]) < FP32_TOL
    assert relerr(host(h), h_ref) < 5e-4 and relerr(host(st[0]), st_ref[0]) < 5e-4
    assert np.abs(host(st[2]) - st_ref[2]).max() < 1e-3


def test_chunkwise_bf16_extreme_gates_tensor_core_path(ops):
    """bf16 tensor-core path with gates pinned at the soft-cap limits for long stretches: every exponent is a
    non-positive difference and the TMEM state is rescaled lazily, so nothing may overflow.  The final state
    must meet the bf16 tolerance against the float64 recurrence.  With such gates the normaliser q.n + sum(P)
    of many tokens is a near-cancellation (|h| reaches 1e4): there h = num/den amplifies the bf16 rounding of
    the weights by 1/|den| in ANY bf16 implementation, so h is compared on the well-conditioned tokens
    (|h| <= 5 in the float64 result, the usual range of h; 62 % of the tokens here) and only checked for finiteness elsewhere."""
    rng = np.random.default_rng(13)
    B, NH, S, dqk, dv = 1, 2, 768, 256, 256
    q, k = (xo.bf16_round(rng.standard_normal((B, NH, S, dqk)).astype(np.float32)) for _ in range(2))
    v = xo.bf16_round(rng.standard_normal((B, NH, S, dv)).astype(np.float32))
    i = np.repeat(rng.choice([-15.0, 0.0, 15.0], size=(B, NH, S // 16)), 16, axis=-1).astype(np.float32)
    f = np.repeat(rng.choice([-15.0, 3.0, 15.0], size=(B, NH, S // 32), p=[0.1, 0.5, 0.4]), 32, axis=-1).astype(np.float32)
    h64, st64 = recurrent_fp64(q, k, v, i, f)
    bf = torch.bfloat16
    assert ops.chunkwise_workspace_bytes(B, NH, S, dqk, dv, 64, bf) > 0  # really the tensor-core path
    h, st = ops.mlstm_chunkwise(*(dev(a, bf) for a in (q, k, v, i, f)))
    assert np.isfinite(host(h)).all() and np.isfinite(host(st[0])).all()
    ok = np.abs(h64).max(axis=-1, keepdims=True) <= 5.0
    assert ok.mean() > 0.5
    assert relerr(np.where(ok, host(h), 0.0), np.where(ok, h64, 0.0)) < BF16_TOL
    assert relerr(host(st[0]), st64[0]) < BF16_TOL and relerr(host(st[1]), st64[1]) < BF16_TOL
    assert np.abs(host(st[2]) - st64[2]).max() < 1e-3


def test_chunkwise_full_length_properties(ops):
    """BASELINE configs[3] length (S = 32768, 256/512, bf16): the oracle cannot run this in seconds, so check
    (a) the first 384 tokens against the oracle, (b) one pass == two half passes with the carried state,
    (c) run-to-run bitwise determinism."""
    B, NH, S, dqk, dv = 1, 4, 32768, 256, 512
    g = torch.Generator().manual_seed(3)
    bf = torch.bfloat16
    q = torch.randn(B, NH, S, dqk, generator=g).to(bf)
    k = torch.randn(B, NH, S, dqk, generator=g).to(bf)
    v = torch.randn(B, NH, S, dv, generator=g).to(bf)
    i = (15 * torch.tanh(torch.randn(B, NH, S, generator=g) / 15)).to(bf)
    f = (15 * torch.tanh((torch.randn(B, NH, S, generator=g) + 3) / 15)).to(bf)
    P = 384
    h_ref, _ = xo.mlstm_recurrent(*(t[:, :, :P].float().numpy() for t in (q, k, v, i, f)))
    qd, kd, vd, idv, fd = (t.cuda() for t in (q, k, v, i, f))
    h, st = ops.mlstm_chunkwise(qd, kd, vd, idv, fd)
    assert relerr(host(h[:, :, :P]), h_ref) < BF16_TOL
    H = S // 2
    h1, st1 = ops.mlstm_chunkwise(qd[:, :, :H], kd[:, :, :H], vd[:, :, :H], idv[:, :, :H], fd[:, :, :H])
    h2, st2 = ops.mlstm_chunkwise(qd[:, :, H:], kd[:, :, H:], vd[:, :, H:], idv[:, :, H:], fd[:, :, H:], st1)
    assert relerr(host(torch.cat([h1, h2], 2)), host(h)) < BF16_TOL
    assert relerr(host(st2[0]), host(st[0])) < BF16_TOL and np.abs(host(st2[2]) - host(st[2])).max() < 1e-3
    assert torch.isfinite(h.float()).all()
    h_again, _ = ops.mlstm_chunkwise(qd, kd, vd, idv, fd)
    assert torch.equal(h, h_again)


# ---- sLSTM ------------------------------------------------------------------------
@pytest.mark.parametrize("tag", ["a", "b", "x", "z"])
def test_slstm_scan_fixture(ops, golden, tag):
    g = golden("slstm_a")
    st = None if tag == "z" else tuple(dev(g[f"{tag}_{s}0"]) for s in "cnm")
    h, (c, n, m) = ops.slstm_scan(*(dev(g[f"{tag}_{x}"]) for x in "zifo"), state=st)
    tol = 1e-4 if tag == "x" else 1e-5
    assert relerr(host(h), g[f"{tag}_h"]) < tol and relerr(host(c), g[f"{tag}_c"]) < tol
    assert relerr(host(n), g[f"{tag}_n"]) < tol and np.abs(host(m) - g[f"{tag}_m"]).max() < tol


@pytest.mark.parametrize("B,S,NH,H,dtype", [(32, 100, 4, 256, torch.float32), (3, 33, 2, 40, torch.float32),
                                             (2, 64, 4, 1024, torch.float32), (4, 70, 4, 256, torch.bfloat16)])
def test_slstm_scan_oracle(ops, B, S, NH, H, dtype):
    rng = np.random.default_rng(H + S)
    rd = xo.bf16_round if dtype == torch.bfloat16 else (lambda a: a)
    z = rd(rng.standard_normal((B, S, NH, H)).astype(np.float32))
    i, f = (rd(a) for a in gates(rng, (B, S, NH)))
    o = rd(rng.standard_normal((B, S, NH)).astype(np.float32))
    h_ref, st_ref = xo.slstm_scan(z, i, f, o)
    h, st = ops.slstm_scan(*(dev(a, dtype) for a in (z, i, f, o)))
    tol = BF16_TOL if dtype == torch.bfloat16 else FP32_TOL
    assert relerr(host(h), h_ref) < tol
    for got, want in zip(st, st_ref):
        assert relerr(host(got), want) < FP32_TOL


def test_slstm_recurrent_fixture(ops, golden):
    g = golden("slstm_b")
    nh = int(g["num_heads"])
    hs, st = ops.slstm_recurrent(dev(g["gx"]), dev(g["R"]), dev(g["rb"]), None, nh, 15.0)
    assert relerr(host(hs), g["hs"]) < FP32_TOL
    for got, key in zip(st, "cnhm"):
        assert relerr(host(got), g[key]) < FP32_TOL
    hs2, st2 = ops.slstm_recurrent(dev(g["gx2"]), dev(g["R"]), dev(g["rb"]), st, nh, 15.0)
    assert relerr(host(hs2), g["hs2"]) < FP32_TOL
    for got, key in zip(st2, ("c2", "n2", "h2", "m2")):
        assert relerr(host(got), g[key]) < FP32_TOL


@pytest.mark.parametrize("B,S,NH,dh,dtype", [(5, 40, 4, 256, torch.float32), (9, 24, 2, 64, torch.float32),
                                              (8, 48, 4, 256, torch.bfloat16), (3, 17, 3, 128, torch.bfloat16)])
def test_slstm_recurrent_oracle(ops, B, S, NH, dh, dtype):
    rng = np.random.default_rng(dh + B)
    rd = xo.bf16_round if dtype == torch.bfloat16 else (lambda a: a)
    D = NH * dh
    gx = rd(rng.standard_normal((B, S, 4, D)).astype(np.float32))
    gx[:, :, 1] += np.linspace(3, 6, D, dtype=np.float32)
    gx = rd(gx)
    R = rd((rng.standard_normal((4, NH, dh, dh)) * 0.02).astype(np.float32))
    rb = (rng.standard_normal((4, D)) * 0.05).astype(np.float32)
    hs_ref, st_ref = xo.slstm_recurrent(gx, R, rb, None, NH, 15.0)
    hs, st = ops.slstm_recurrent(dev(gx, dtype), dev(R, dtype), dev(rb), None, NH, 15.0)
    tol = BF16_TOL if dtype == torch.bfloat16 else FP32_TOL
    assert relerr(host(hs), hs_ref) < tol
    for got, want in zip(st, st_ref):
        assert relerr(host(got), want) < (tol if dtype == torch.bfloat16 else FP32_TOL)


@pytest.mark.parametrize("B,S,NH", [(1, 5, 1), (33, 70, 2), (32, 600, 4)])
def test_slstm_recurrent_tensor_core_path(ops, B, S, NH):
    """bf16 with head dimension 256 runs the tcgen05 kernel (R resident in tensor memory, h fed back as
    bf16): ragged batch groups, a carried state, and a long sequence for drift."""
    dh, D = 256, NH * 256
    rng = np.random.default_rng(B * 1000 + S)
    gx = rng.standard_normal((B, S, 4, D)).astype(np.float32)
    gx[:, :, 1] += np.linspace(3, 6, D, dtype=np.float32)
    gx = xo.bf16_round(gx)
    R = xo.bf16_round((rng.standard_normal((4, NH, dh, dh)) * 0.02).astype(np.float32))
    rb = (rng.standard_normal((4, D)) * 0.05).astype(np.float32)
    bf = torch.bfloat16
    S1 = S // 2
    hs_ref, st_ref = xo.slstm_recurrent(gx, R, rb, None, NH, 15.0)
    hs1, st1 = ops.slstm_recurrent(dev(gx[:, :S1], bf), dev(R, bf), dev(rb), None, NH, 15.0)
    hs2, st2 = ops.slstm_recurrent(dev(gx[:, S1:], bf), dev(R, bf), dev(rb), st1, NH, 15.0)
    hs = torch.cat([hs1, hs2], 1)
    assert torch.isfinite(hs.float()).all()
    assert relerr(host(hs), hs_ref) < BF16_TOL
    for got, want in zip(st2, st_ref):
        assert relerr(host(got), want) < BF16_TOL


# ---- error behaviour of the C ABI --------------------------------------------------
def test_errors_are_statuses_not_crashes(ops):
    from xlstm_cuda import _lib
    lib = _lib.load()
    assert lib.xlstm_softcap(None, None, 8, 15.0, 0, None) == -1
    assert lib.xlstm_softcap(None, None, 0, 15.0, 0, None) == 0
    x = torch.zeros(16, device="cuda")
    assert lib.xlstm_softcap(x.data_ptr(), x.data_ptr(), 16, 15.0, 7, None) == -2
    assert lib.xlstm_mlstm_step(*([x.data_ptr()] * 5), None, None, None, *([x.data_ptr()] * 4), 1, 1, 2, 3, 1e-6, 0, None) == -2
    px = x.data_ptr()
    # flags the step does not know: invalid; output epilogue wider than eight 64-column tiles: unsupported (no launch)
    assert lib.xlstm_mlstm_step_ex(*([px] * 5), None, None, None, *([px] * 4), 1, 1, 8, 8, 1e-6, 0.0, 2, 0, None) == -1
    assert lib.xlstm_mlstm_step_gated(*([px] * 5), None, None, None, px, 1024, None, 1e-6, *([px] * 4), 1, 1, 8, 1024, 1e-6, 0.0,
                                      0, 0, None) == -2
    assert lib.xlstm_mlstm_step_gated(*([px] * 5), None, None, None, None, 8, None, 1e-6, *([px] * 4), 1, 1, 8, 8, 1e-6, 0.0,
                                      0, 0, None) == -1
    with pytest.raises(RuntimeError):
        ops.softcap(torch.zeros(4), 15.0)  # CPU tensor: no fallback
    with pytest.raises(TypeError):
        ops.softcap(torch.zeros(4, device="cuda", dtype=torch.float16), 15.0)


# ---- gate soft-cap folded into the kernels -------------------------------------------------
@pytest.mark.parametrize("dtype,shape", [(torch.float32, (2, 3, 200, 64, 64)), (torch.bfloat16, (2, 2, 300, 256, 256))])
def test_gate_cap_inside_the_kernels(ops, dtype, shape):
    """Raw gate projections + gate_cap give what pre-capped gates give: chunkwise (exact path in
    fp32, tensor-core path + exact tail in bf16) and the decode step."""
    B, NH, S, dqk, dv = shape
    rng = np.random.default_rng(S)
    q, k = (rng.standard_normal((B, NH, S, dqk)).astype(np.float32) for _ in range(2))
    v = rng.standard_normal((B, NH, S, dv)).astype(np.float32)
    i_raw = (rng.standard_normal((B, NH, S)) * 6.0).astype(np.float32)        # well into the tanh knee
    f_raw = (rng.standard_normal((B, NH, S)) * 6.0 + 8.0).astype(np.float32)
    if dtype == torch.bfloat16:
        q, k, v, i_raw, f_raw = (xo.bf16_round(a) for a in (q, k, v, i_raw, f_raw))
    cap = 15.0
    i_cap, f_cap = xo.softcap(i_raw, cap), xo.softcap(f_raw, cap)
    h_ref, (C_ref, n_ref, m_ref) = xo.mlstm_recurrent(q, k, v, i_cap, f_cap, None, 1e-6)
    tol = FP32_TOL if dtype == torch.float32 else BF16_TOL
    h, (C, n, m) = ops.mlstm_chunkwise(dev(q, dtype), dev(k, dtype), dev(v, dtype), dev(i_raw, dtype), dev(f_raw, dtype),
                                       None, 64, 1e-6, gate_cap=cap)
    assert relerr(host(h), h_ref) <= tol and relerr(host(C), C_ref) <= tol and relerr(host(n), n_ref) <= tol
    assert np.abs(host(m) - m_ref).max() <= (1e-4 if dtype == torch.float32 else 2e-2)
    # decode steps from that state, raw gates again
    st, st_ref = (C, n, m), (C_ref, n_ref, m_ref)
    for t in range(3):
        qs, ks, vs = q[:, :, t], k[:, :, t], v[:, :, t]
        hs, st = ops.mlstm_step(dev(qs, dtype), dev(ks, dtype), dev(vs, dtype), dev(i_raw[:, :, t], dtype),
                                dev(f_raw[:, :, t], dtype), st, 1e-6, gate_cap=cap)
        hr, st_ref = xo.mlstm_recurrent(qs[:, :, None], ks[:, :, None], vs[:, :, None], i_cap[:, :, t:t + 1],
                                        f_cap[:, :, t:t + 1], st_ref, 1e-6)
        assert relerr(host(hs), hr[:, :, 0]) <= tol
    # cap <= 0 / None: gates are taken as given
    h0, _ = ops.mlstm_chunkwise(dev(q, dtype), dev(k, dtype), dev(v, dtype), dev(i_cap, dtype), dev(f_cap, dtype), None, 64, 1e-6)
    h1, _ = ops.mlstm_chunkwise(dev(q, dtype), dev(k, dtype), dev(v, dtype), dev(i_cap, dtype), dev(f_cap, dtype), None, 64, 1e-6,
                                gate_cap=0.0)
    assert torch.equal(h0, h1)


@pytest.mark.parametrize("general", [False, True])
def test_chunkwise_segment_parallel_equals_single_pass(ops, general):
    """The segment-parallel two-pass mode (every segment from an empty state, states combined, every segment again
    from its true start state) against the single pass and against the oracle: bf16 tensor-core shapes, with a
    carried-in state and a sequence tail, for segment counts that divide the tiles evenly and unevenly."""
    rng = np.random.default_rng(21)
    B, NH, S, dqk, dv = 1, 2, 2048 + 70, 256, 256
    q, k = (xo.bf16_round(rng.standard_normal((B, NH, S, dqk)).astype(np.float32)) for _ in range(2))
    v = xo.bf16_round(rng.standard_normal((B, NH, S, dv)).astype(np.float32))
    i, f = (xo.bf16_round(a) for a in gates(rng, (B, NH, S)))
    st0 = ((rng.standard_normal((B, NH, dqk, dv)) * 0.1).astype(np.float32),
           (rng.standard_normal((B, NH, dqk)) * 0.1).astype(np.float32), rng.standard_normal((B, NH)).astype(np.float32))
    h_ref, st_ref = xo.mlstm_recurrent(q, k, v, i, f, st0)
    args = [dev(a, torch.bfloat16) for a in (q, k, v, i, f)]
    std = tuple(dev(a) for a in st0)
    try:
        ops.chunkwise_general_only(general)
        ops.chunkwise_segments(1)
        h1, s1 = ops.mlstm_chunkwise(*args, state=std)
        for P in (2, 3, 4, 16):
            ops.chunkwise_segments(P)
            h, s = ops.mlstm_chunkwise(*args, state=std)
            assert relerr(host(h), h_ref) < BF16_TOL and relerr(host(h), host(h1)) < BF16_TOL, P
            assert relerr(host(s[0]), st_ref[0]) < BF16_TOL and relerr(host(s[1]), st_ref[1]) < BF16_TOL, P
            assert np.abs(host(s[2]) - st_ref[2]).max() < 1e-3, P
            assert relerr(host(s[0]), host(s1[0])) < 5e-3, P
        ops.chunkwise_segments(None)     # planned from the grid size: 4 CTAs on 148 SMs -> segments
        h, s = ops.mlstm_chunkwise(*args, state=std)
        assert relerr(host(h), h_ref) < BF16_TOL and relerr(host(s[0]), st_ref[0]) < BF16_TOL
    finally:
        ops.chunkwise_segments(None)
        ops.chunkwise_general_only(False)


def test_bounded_wait_gives_up_and_status_queries_report_ok(ops):
    """Device-side time-outs without hanging anything: (a) the bounded mbarrier wait of the tensor-core kernels,
    built with a tiny poll limit in a test-only kernel, on a barrier nobody arrives at - it must return false,
    raise the abort flag (which releases every other role) and let the kernel end normally; (b) after real
    forwards the status queries of the C ABI report no time-out."""
    import ctypes
    sys_path = Path(__file__).resolve().parent / "helpers"
    sys.path.insert(0, str(sys_path))
    from build_helpers import build
    lib = ctypes.CDLL(str(build()))
    out = (ctypes.c_int * 3)()
    assert lib.timeout_probe_run(out) == 0
    assert list(out) == [0, 0, 1]
    rng = np.random.default_rng(2)
    B, NH, S, dqk, dv = 1, 1, 256, 128, 128
    q, k = (dev(rng.standard_normal((B, NH, S, dqk)).astype(np.float32), torch.bfloat16) for _ in range(2))
    v = dev(rng.standard_normal((B, NH, S, dv)).astype(np.float32), torch.bfloat16)
    i, f = (dev(a, torch.bfloat16) for a in gates(rng, (B, NH, S)))
    ws = torch.empty(ops.chunkwise_workspace_bytes(B, NH, S, dqk, dv, 64, torch.bfloat16), dtype=torch.uint8, device="cuda")
    ops.mlstm_chunkwise(q, k, v, i, f, workspace=ws)
    ops.chunkwise_status(ws)            # raises on XLSTM_ERR_TIMEOUT
    ops.slstm_recurrent_status()


def test_chunkwise_scatter_entry_point_single_rank(ops):
    """The token-sharded store mode with one rank: h lands in the [B, S, NH, dv] buffer exactly as the regular
    entry point writes it into a strided view of the same layout (the multi-rank routing is covered by the
    two-GPU test)."""
    from xlstm_cuda.parallel import FusedHeadScatter
    rng = np.random.default_rng(31)
    B, NH, S, dqk, dv = 2, 2, 512, 128, 256
    q, k = (dev(rng.standard_normal((B, NH, S, dqk)).astype(np.float32), torch.bfloat16) for _ in range(2))
    v = dev(rng.standard_normal((B, NH, S, dv)).astype(np.float32), torch.bfloat16)
    i, f = (dev(a, torch.bfloat16) for a in gates(rng, (B, NH, S)))
    w = dev((rng.standard_normal((NH * dv, 48)) * 0.05).astype(np.float32), torch.bfloat16)
    h, st = ops.mlstm_chunkwise(q, k, v, i, f)
    sc = FusedHeadScatter(B, S, NH, dv, torch.bfloat16, "cuda")
    y, st2 = sc.run(q, k, v, i, f, None, out_proj=w)
    assert torch.equal(sc.buf, h.permute(0, 2, 1, 3).contiguous())
    assert all(torch.equal(a, b) for a, b in zip(st, st2))
    assert torch.equal(y, h.permute(0, 2, 1, 3).reshape(B, S, NH * dv) @ w)
