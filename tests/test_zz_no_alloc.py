"""The allocation-free entry point, b200gmm_run_static, against b200gmm_run.

Some embedders cannot give the library device memory: everything free has gone
to their own pool, or they only ever see the input and output buffers.  For them
the library carries its scratch in a fixed device array; this test drives that
entry point through the C ABI with raw pointers, twice in a row on different
problems (the array is shared and keeps the previous call's contents), and checks
each result against the ordinary entry point within the tolerance the other GPU
tests use.  It is collected last on purpose, and passes on its own as well.
"""
import pytest
import torch

from grouped_gemm_b200 import _capi
from oracle import gmm_oracle

pytestmark = pytest.mark.gpu

RTOL = 1e-2
ATOL = 1e-2


def _run(entry, a, b, c, bs, trans_a, trans_b, status):
    lib = _capi.load()
    z = bs.shape[0]
    n = b.shape[1] if (trans_a or trans_b) else b.shape[2]
    stream = torch.cuda.current_stream().cuda_stream
    common = (a.data_ptr(), b.data_ptr(), c.data_ptr(), bs.data_ptr(), 1 if bs.is_cuda else 0, z,
              a.shape[0], a.shape[1], n, int(trans_a), int(trans_b))
    if entry == "static":
        return lib.b200gmm_run_static(*common, status.data_ptr(), stream)
    nbytes = _capi.workspace_bytes(z)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    return lib.b200gmm_run(*common, ws.data_ptr(), nbytes, status.data_ptr(), stream)


def _problem(seed, sizes, d1, n, mode):
    g = torch.Generator(device="cuda").manual_seed(seed)
    T, z = sum(sizes), len(sizes)
    a = torch.randn(T, d1, device="cuda", generator=g).bfloat16()
    if mode == "tn":
        b = torch.randn(T, n, device="cuda", generator=g).bfloat16()
        shape = (z, d1, n)
    elif mode == "nt":
        b = (torch.randn(z, n, d1, device="cuda", generator=g) * 0.1).bfloat16()
        shape = (T, n)
    else:
        b = (torch.randn(z, d1, n, device="cuda", generator=g) * 0.1).bfloat16()
        shape = (T, n)
    return a, b, shape


def test_static_entry_matches_workspace_entry_on_two_calls_in_a_row():
    assert torch.cuda.is_available()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    calls = [
        # wgrad first: it is the mode that edits tensor maps in the scratch
        (1, [300, 0, 77, 515, 64], 384, 520, "tn", True),
        (2, [129, 1000, 5, 0, 2000, 31], 512, 768, "nn", False),
        (3, [700, 45], 256, 264, "nt", True),
        # wgrad with batch_sizes in host memory: copies them into the scratch and
        # edits the tensor maps that live behind them
        (4, [5, 130, 0, 64], 256, 264, "tn", False),
    ]
    for seed, sizes, d1, n, mode, on_device in calls:
        a, b, shape = _problem(seed, sizes, d1, n, mode)
        bs = torch.tensor(sizes, dtype=torch.int64)
        if on_device:
            bs = bs.cuda()
        got = torch.full(shape, 3.0, dtype=torch.bfloat16, device="cuda")
        want = torch.full(shape, 5.0, dtype=torch.bfloat16, device="cuda")
        assert _run("static", a, b, got, bs, mode == "tn", mode == "nt", status) == 0
        assert _run("workspace", a, b, want, bs, mode == "tn", mode == "nt", status) == 0
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        assert torch.allclose(got.float(), want.float(), rtol=RTOL, atol=ATOL), mode
        # same kernel, same inputs: in fact bit-identical
        assert torch.equal(got, want), mode


def test_static_entry_rejects_too_many_experts():
    z = _capi.STATIC_MAX_EXPERTS + 1
    a = torch.zeros(z, 64, dtype=torch.bfloat16, device="cuda")
    b = torch.zeros(z, 64, 64, dtype=torch.bfloat16, device="cuda")
    c = torch.full((z, 64), 9.0, dtype=torch.bfloat16, device="cuda")
    bs = torch.ones(z, dtype=torch.int64, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = _run("static", a, b, c, bs, False, False, status)
    assert rc == -3 and "too many experts" in _capi.strerror(rc)
    torch.cuda.synchronize()
    assert bool((c == 9.0).all()), "a rejected call must not launch anything"
    # the ordinary entry point still takes this many experts
    assert _run("workspace", a, b, c, bs, False, False, status) == 0
    torch.cuda.synchronize()
    assert bool((c == 0).all())


@pytest.mark.parametrize("mode,on_device", [("nn", False), ("tn", True), ("tn", False)])
def test_static_entry_at_its_expert_limit_against_the_oracle(mode, on_device):
    """z = 256, the most the built-in scratch holds: the batch_sizes copy and the
    tensor-map copies sit back to back in it, so this is where their sizes would
    collide if either drifted.  Checked against the CPU oracle, not against the
    other entry point."""
    z = _capi.STATIC_MAX_EXPERTS
    g = torch.Generator().manual_seed(7)
    sizes = [int(v) for v in torch.randint(0, 40, (z,), generator=g)]
    sizes[3], sizes[100], sizes[255] = 0, 300, 129
    d1, n = 128, 264
    T = sum(sizes)
    a_cpu = torch.randn(T, d1, generator=g).bfloat16()
    bs_cpu = torch.tensor(sizes, dtype=torch.int64)
    if mode == "tn":
        b_cpu = torch.randn(T, n, generator=g).bfloat16()
        want = gmm_oracle.gmm(a_cpu, b_cpu, bs_cpu, trans_a=True)
        shape = (z, d1, n)
    else:
        b_cpu = (torch.randn(z, d1, n, generator=g) * 0.1).bfloat16()
        want = gmm_oracle.gmm(a_cpu, b_cpu, bs_cpu)
        shape = (T, n)
    a, b = a_cpu.cuda(), b_cpu.cuda()
    bs = bs_cpu.cuda() if on_device else bs_cpu
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    got = torch.full(shape, 3.0, dtype=torch.bfloat16, device="cuda")
    for _ in range(2):  # twice: the second call finds the first one's scratch
        assert _run("static", a, b, got, bs, mode == "tn", False, status) == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    err = (got.float().cpu() - want.float()).abs()
    assert bool((err <= ATOL + RTOL * want.float().abs()).all()), float(err.max())
