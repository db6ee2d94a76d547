"""The scratch-free chunkwise entry point against the regular one (GPU, through the C ABI).

`xlstm_mlstm_chunkwise_fwd_static` exists for hosts that cannot give the library a scratch
buffer: a serving process that has already split all device memory into its own fixed pools
and forbids further allocation, or a plugin that only ever receives input and output pointers.
It keeps its scratch in a fixed block inside the library, shared by all calls, so this test
runs it twice in a row on different problems (the second sees the first one's leftovers) and
compares every output with the workspace-taking entry point.  Collected last on purpose.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _run_both(B, NH, S, dqk, dv, seed, with_state):
    from xlstm_cuda import _lib
    lib = _lib.load()
    g = torch.Generator().manual_seed(seed)
    bf = torch.bfloat16
    q = torch.randn(B, NH, S, dqk, generator=g).to(bf).cuda()
    k = torch.randn(B, NH, S, dqk, generator=g).to(bf).cuda()
    v = torch.randn(B, NH, S, dv, generator=g).to(bf).cuda()
    i = (15 * torch.tanh(torch.randn(B, NH, S, generator=g) / 15)).to(bf).cuda()
    f = (15 * torch.tanh((torch.randn(B, NH, S, generator=g) + 3) / 15)).to(bf).cuda()
    if with_state:
        st = [(torch.randn(B, NH, dqk, dv, generator=g) * 0.1).cuda(), (torch.randn(B, NH, dqk, generator=g) * 0.1).cuda(),
              torch.randn(B, NH, generator=g).cuda()]
        st_ptr = [t.data_ptr() for t in st]
    else:
        st_ptr = [None, None, None]
    stream = torch.cuda.current_stream().cuda_stream

    def outputs():
        return (torch.full((B, NH, S, dv), float("nan"), dtype=bf, device="cuda"),
                torch.full((B, NH, dqk, dv), float("nan"), device="cuda"),
                torch.full((B, NH, dqk), float("nan"), device="cuda"), torch.full((B, NH), float("nan"), device="cuda"))

    need = lib.xlstm_mlstm_chunkwise_workspace_bytes(B, NH, S, dqk, dv, 64, _lib.BF16)
    assert need > 0, "the test must exercise the scratch-using tensor-core path"
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    ref = outputs()
    rc = lib.xlstm_mlstm_chunkwise_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), i.data_ptr(), f.data_ptr(), *st_ptr,
                                       *(t.data_ptr() for t in ref), B, NH, S, dqk, dv, 64, 1e-6, _lib.BF16, None,
                                       ws.data_ptr(), need, stream)
    assert rc == 0, lib.xlstm_strerror(rc)
    got = outputs()
    rc = lib.xlstm_mlstm_chunkwise_fwd_static(q.data_ptr(), k.data_ptr(), v.data_ptr(), i.data_ptr(), f.data_ptr(),
                                              *st_ptr, *(t.data_ptr() for t in got), B, NH, S, dqk, dv, 64, 1e-6,
                                              _lib.BF16, None, stream)
    assert rc == 0, lib.xlstm_strerror(rc)
    torch.cuda.synchronize()
    # both entry points run the same kernels on the same inputs; only the address of the scratch differs,
    # so every output must agree bit for bit (a tolerance could hide a scratch-layout fault)
    for name, a, b in zip("hCnm", got, ref):
        assert torch.isfinite(a.float()).all(), name
        assert torch.equal(a, b), (name, float((a.float() - b.float()).abs().max()))


def test_static_scratch_entry_point_matches_workspace_entry_point_twice():
    _run_both(B=2, NH=2, S=512, dqk=256, dv=256, seed=1, with_state=False)
    # second call: other sizes, carried state, a sequence tail; the block still holds call one's data
    _run_both(B=1, NH=3, S=320, dqk=128, dv=128, seed=2, with_state=True)


def test_static_scratch_rejects_problems_beyond_its_block():
    """One long sequence whose gate scratch (3 KiB per 128-token tile) exceeds the 8 MiB block.  Every
    tensor has the size the arguments claim, so nothing could go out of bounds even if a kernel ran."""
    from xlstm_cuda import _lib
    lib = _lib.load()
    B, NH, S, dqk, dv = 1, 1, 128 * 2800, 128, 128
    bf = torch.bfloat16
    q = torch.zeros(B, NH, S, dqk, dtype=bf, device="cuda")
    v = torch.zeros(B, NH, S, dv, dtype=bf, device="cuda")
    g = torch.zeros(B, NH, S, dtype=bf, device="cuda")
    h = torch.empty_like(v)
    C1 = torch.empty(B, NH, dqk, dv, device="cuda")
    n1 = torch.empty(B, NH, dqk, device="cuda")
    m1 = torch.empty(B, NH, device="cuda")
    assert lib.xlstm_mlstm_chunkwise_workspace_bytes(B, NH, S, dqk, dv, 64, _lib.BF16) > (8 << 20)
    rc = lib.xlstm_mlstm_chunkwise_fwd_static(q.data_ptr(), q.data_ptr(), v.data_ptr(), g.data_ptr(), g.data_ptr(),
                                              None, None, None, h.data_ptr(), C1.data_ptr(), n1.data_ptr(),
                                              m1.data_ptr(), B, NH, S, dqk, dv, 64, 1e-6, _lib.BF16, None,
                                              torch.cuda.current_stream().cuda_stream)
    assert rc == -6 and b"static" in lib.xlstm_strerror(rc)
