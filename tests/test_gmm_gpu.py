"""GPU parity tests (run with -m gpu on a B200).  Every product goes through the
C ABI (grouped_gemm_b200.backend -> b200gmm_run); the CPU oracle is the checker.

Tolerance for floating-point results: rtol 1e-2 / atol 1e-2 in bf16 against the
fp32-accumulated oracle.  Integer results (argument fill) are compared exactly.
The reference's own statistic (<= 2 % of elements outside isclose(rtol=1e-5),
grouped_gemm/ops_test.py:10-17) is checked as well on its test grid.
"""
import itertools

import numpy as np
import pytest
import torch

from oracle import gmm_oracle
from tests import util

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gg():
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    import grouped_gemm_b200
    return grouped_gemm_b200


@pytest.fixture(autouse=True, params=["1", "1-light", "2", "auto"],
                ids=["one-cta", "one-cta-transposed-tiles", "cta-pair", "auto"])
def _variant(request, monkeypatch, gg):
    """Every test runs on both kernel variants: tiles owned by one CTA (once more
    with experts of at most 64 rows as transposed tiles), and tiles owned by a
    pair of CTAs (tcgen05 cta_group::2), and once with the library's own choice of
    variant.  The library reads the variables on each call."""
    monkeypatch.delenv("B200GMM_LIGHT", raising=False)
    if request.param == "auto":
        monkeypatch.delenv("B200GMM_CTAS", raising=False)
    elif request.param == "1-light":
        monkeypatch.setenv("B200GMM_CTAS", "1")
        monkeypatch.setenv("B200GMM_LIGHT", "1")
    else:
        monkeypatch.setenv("B200GMM_CTAS", request.param)
    yield request.param
    assert gg.backend.device_status() == 0, "a kernel raised a status bit (timeout / bad sizes)"


def _check_fwd_bwd(gg, a_cpu, b_cpu, bs_cpu, trans_b, on_device, ref_stat=True):
    """Forward + out.sum().backward() as in ops_test.py:59-80, against the oracle."""
    a = a_cpu.cuda().requires_grad_(True)
    b = b_cpu.cuda().requires_grad_(True)
    bs = bs_cpu.cuda() if on_device else bs_cpu
    out = gg.ops.gmm(a, b, bs, trans_b)
    want = gmm_oracle.gmm(a_cpu, b_cpu, bs_cpu, trans_b=trans_b)
    rows = int(bs_cpu.sum())
    util.assert_close(out[:rows], want[:rows], what="forward")
    out.sum().backward()
    agrad, bgrad = gmm_oracle.gmm_backward(a_cpu, b_cpu, bs_cpu, torch.ones_like(want), trans_b=trans_b)
    util.assert_close(a.grad[:rows], agrad[:rows], what="a.grad")
    util.assert_close(b.grad, bgrad, what="b.grad")
    if ref_stat:
        assert gmm_oracle.reference_allclose_pct(out[:rows].cpu(), want[:rows]) <= 2.0
        assert gmm_oracle.reference_allclose_pct(a.grad[:rows].cpu(), agrad[:rows]) <= 2.0
        assert gmm_oracle.reference_allclose_pct(b.grad.cpu(), bgrad) <= 2.0


# ---- the reference's grid: ops_test.py:20-36 ---------------------------------
_PROBLEMS = [(1, 128, 128, 128), (8, 128, 128, 128), (16, 128, 128, 128),
             (1, 128, 256, 512), (8, 128, 256, 512), (16, 128, 256, 512)]
_GRID = [p + f for p, f in itertools.product(_PROBLEMS, itertools.product((False, True), (False, True)))]


@pytest.mark.parametrize("z,m,k,n,trans_b,on_device", _GRID)
def test_fixed_sizes(gg, z, m, k, n, trans_b, on_device):
    torch.manual_seed(0)
    a = util.reference_inputs(z, m, k).view(-1, k)
    b = util.reference_inputs(z, n, k) if trans_b else util.reference_inputs(z, k, n)
    _check_fwd_bwd(gg, a, b, torch.tensor([m] * z), trans_b, on_device)


@pytest.mark.parametrize("z,m,k,n,trans_b,on_device", _GRID)
def test_variable_sizes(gg, z, m, k, n, trans_b, on_device):
    torch.manual_seed(0)
    a = util.reference_inputs(z, m, k).view(-1, k)
    b = util.reference_inputs(z, n, k) if trans_b else util.reference_inputs(z, k, n)
    _check_fwd_bwd(gg, a, b, util.variable_batch_sizes(z, m), trans_b, on_device)


# ---- edge cases: ops_test.py:112-158 -------------------------------------------
@pytest.mark.parametrize("on_device", [False, True])
def test_zero_k_known_answer(gg, on_device):
    a = torch.ones(192, 128).cuda().to(torch.bfloat16)
    b = torch.ones(192, 128).cuda().to(torch.bfloat16)
    c = torch.ones(4, 128, 128).cuda().to(torch.bfloat16)
    bs = torch.tensor([0, 128, 0, 64]).to(torch.long)
    if on_device:
        bs = bs.cuda()
    got = gg.ops.backend.gmm(a, b, bs, trans_a=True, c=c)
    assert got is c
    for i, want in enumerate((0, 128, 0, 64)):
        assert bool((c[i] == want).all()), f"c[{i}] != {want}"


@pytest.mark.parametrize("on_device", [False, True])
def test_zero_size_expert_mixtral_shape(gg, on_device):
    """ops_test.py:115-141 at a quarter of its width to keep the CPU oracle to
    seconds; the full Mixtral shape is covered by test_full_size_* below."""
    torch.manual_seed(0)
    z, m, k, n = 8, 16384, 1024, 3584
    a = util.reference_inputs(z, m // z, k).view(-1, k)
    b = util.reference_inputs(z, k, n)
    bs = torch.tensor([219, 2246, 5, 8103, 1, 1117, 4693, 0]).to(torch.long)
    _check_fwd_bwd(gg, a, b, bs, False, on_device)


# ---- golden vectors made by the reference's own test functions --------------------
_DATA, _KEYS = util.golden_cases()


@pytest.mark.parametrize("key", _KEYS)
def test_against_reference_golden(gg, key):
    z, m, k, n, trans_b, variable = util.parse_key(key)
    torch.manual_seed(0)
    a_cpu = util.reference_inputs(z, m, k).view(-1, k)
    b_cpu = util.reference_inputs(z, n, k) if trans_b else util.reference_inputs(z, k, n)
    assert util.input_digest(a_cpu, b_cpu) == bytes(_DATA[key + "/input_sha256"]).decode()
    bs = torch.from_numpy(_DATA[key + "/batch_sizes"])
    a = a_cpu.cuda().requires_grad_(True)
    b = b_cpu.cuda().requires_grad_(True)
    out = gg.ops.gmm(a, b, bs.cuda(), trans_b)
    out.sum().backward()
    for got, name in ((out, "out"), (a.grad, "a_grad"), (b.grad, "b_grad")):
        gold, got = util.golden_pair(_DATA, key, name, got)
        assert gmm_oracle.reference_allclose_pct(got.cpu(), gold) <= 2.0, name
        util.assert_close(got, gold, rtol=1e-2, atol=1e-6, what=name)


# ---- benchmark configuration 1 -----------------------------------------------------------
@pytest.mark.parametrize("trans_b", [False, True])
@pytest.mark.parametrize("on_device", [False, True])
def test_config1_cpu_correctness_case(gg, trans_b, on_device):
    torch.manual_seed(0)
    a_cpu = torch.randn(512, 128).bfloat16()
    b_cpu = (torch.randn(4, 128, 128) * 0.02).bfloat16()
    bs = torch.tensor([128] * 4)
    _check_fwd_bwd(gg, a_cpu, b_cpu, bs, trans_b, on_device, ref_stat=False)
    # random upstream gradient as well
    grad_cpu = torch.randn(512, 128).bfloat16()
    a = a_cpu.cuda().requires_grad_(True)
    b = b_cpu.cuda().requires_grad_(True)
    gg.ops.gmm(a, b, bs.cuda() if on_device else bs, trans_b).backward(grad_cpu.cuda())
    agrad, bgrad = gmm_oracle.gmm_backward(a_cpu, b_cpu, bs, grad_cpu, trans_b=trans_b)
    util.assert_close(a.grad, agrad, what="a.grad")
    util.assert_close(b.grad, bgrad, what="b.grad")


# ---- ragged / odd shapes, all three layouts ------------------------------------------
_RAGGED = [
    ([5, 0, 300, 131], 512, 384),
    ([77, 129, 1], 200, 328),          # k, n not multiples of the tile
    ([0, 0, 0], 128, 256),             # nothing to do (wgrad still writes zeros)
    ([1], 8, 8),                       # smallest legal dims
    ([64, 64, 63, 65, 127, 129, 128, 0, 256, 257], 256, 520),
    ([33] * 40, 136, 264),
]


@pytest.mark.parametrize("sizes,d1,n", _RAGGED)
@pytest.mark.parametrize("mode", ["nn", "nt", "tn"])
@pytest.mark.parametrize("on_device", [False, True])
def test_ragged_all_layouts(gg, sizes, d1, n, mode, on_device):
    torch.manual_seed(1)
    z, T = len(sizes), sum(sizes)
    bs_cpu = torch.tensor(sizes, dtype=torch.int64)
    bs = bs_cpu.cuda() if on_device else bs_cpu
    pad = 3  # rows of a / c past sum(batch_sizes): must be ignored and left untouched
    a_cpu = torch.randn(T + pad, d1).bfloat16()
    if mode == "tn":
        b_cpu = torch.randn(T + pad, n).bfloat16()
        c = torch.full((z, d1, n), 7.0, dtype=torch.bfloat16, device="cuda")
        gg.backend.gmm(a_cpu.cuda(), b_cpu.cuda(), bs, trans_a=True, c=c)
        want = gmm_oracle.gmm(a_cpu, b_cpu, bs_cpu, trans_a=True)
        util.assert_close(c, want, rtol=1e-2, atol=1e-2 * max(1.0, float(want.abs().max())) / 8, what="wgrad")
        for i, s in enumerate(sizes):
            if s == 0:
                assert bool((c[i] == 0).all())
    else:
        trans_b = mode == "nt"
        b_cpu = (torch.randn(z, n, d1) if trans_b else torch.randn(z, d1, n)).bfloat16() * 0.25
        c = torch.full((T + pad, n), 7.0, dtype=torch.bfloat16, device="cuda")
        gg.backend.gmm(a_cpu.cuda(), b_cpu.cuda(), bs, trans_b=trans_b, c=c)
        want = gmm_oracle.gmm(a_cpu, b_cpu, bs_cpu, trans_b=trans_b)
        util.assert_close(c[:T], want[:T], rtol=1e-2, atol=2e-2, what="forward")
        assert bool((c[T:] == 7.0).all()), "rows past sum(batch_sizes) were written"


def test_output_rows_of_neighbour_expert_not_clobbered(gg):
    """A 1-row expert between two large ones: its tile computes 128 rows but may
    store one."""
    torch.manual_seed(2)
    sizes = [200, 1, 200]
    a_cpu = torch.randn(401, 64).bfloat16()
    b_cpu = torch.randn(3, 64, 256).bfloat16() * 0.25
    out = gg.backend.gmm(a_cpu.cuda(), b_cpu.cuda(), torch.tensor(sizes).cuda())
    util.assert_close(out, gmm_oracle.gmm(a_cpu, b_cpu, torch.tensor(sizes)), atol=2e-2, what="forward")


# ---- argument fill: bit-exact ---------------------------------------------------------
@pytest.mark.parametrize("trans_a,trans_b", [(False, False), (False, True), (True, False)])
@pytest.mark.parametrize("case", ["cfg1", "cfg2", "cfg4", "z1", "z1024", "empty-heavy"])
def test_fill_offsets_bit_exact(gg, case, trans_a, trans_b):
    import bench
    from grouped_gemm_b200 import _capi
    if case == "cfg1":
        sizes, d1, n = [128] * 4, 128, 128
    elif case == "cfg2":
        sizes, d1, n = bench.mixtral_batch_sizes(), 4096, 14336
    elif case == "cfg4":
        sizes, d1, n = bench.fine_grained_batch_sizes(), 7168, 2048  # offsets exceed 2^31
    elif case == "z1":
        sizes, d1, n = [12345], 4096, 14336
    elif case == "z1024":
        sizes, d1, n = list(np.random.default_rng(5).integers(0, 5000, size=1024)), 6144, 10752
    else:
        sizes, d1, n = [0, 0, 7, 0, 0, 0, 1, 0] * 9, 512, 1024
    bs = torch.tensor([int(s) for s in sizes], dtype=torch.int64, device="cuda")
    out = torch.full((len(sizes), 9), -1, dtype=torch.int64, device="cuda")
    rc = _capi.load().b200gmm_fill_offsets(bs.data_ptr(), len(sizes), d1, n, int(trans_a), int(trans_b),
                                           out.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    want = gmm_oracle.fill_offsets(np.asarray(sizes, dtype=np.int64), d1, n, trans_a, trans_b)
    assert np.array_equal(out.cpu().numpy(), want)


# ---- full benchmark sizes: size-independent properties ------------------------------------
def _mixtral(gg, trans_b=False):
    import bench
    torch.manual_seed(1)
    sizes = bench.mixtral_batch_sizes()
    g = torch.Generator(device="cuda").manual_seed(1)
    a = torch.randn(32768, 4096, device="cuda", generator=g).bfloat16()
    shape = (8, 14336, 4096) if trans_b else (8, 4096, 14336)
    b = (torch.randn(*shape, device="cuda", generator=g) * 0.02).bfloat16()
    return a, b, torch.tensor(sizes, dtype=torch.int64, device="cuda"), sizes


@pytest.mark.parametrize("trans_b", [False, True])
def test_full_size_forward_sampled_rows_and_linearity(gg, trans_b):
    a, b, bs, sizes = _mixtral(gg, trans_b)
    out = gg.backend.gmm(a, b, bs, trans_b=trans_b)
    # (1) oracle on a sample of rows of every expert (first, last, middle of each group)
    starts = np.concatenate([[0], np.cumsum(sizes)])
    for e in range(8):
        rows = sorted({int(starts[e]), int(starts[e + 1]) - 1, int((starts[e] + starts[e + 1]) // 2)})
        idx = torch.tensor(rows, device="cuda")
        want = gmm_oracle.gmm(a[idx].cpu(), b[e:e + 1].cpu(), torch.tensor([len(rows)]), trans_b=trans_b)
        util.assert_close(out[idx], want, what=f"expert {e} sampled rows")
    # (2) scaling a by 2 is exact in bf16 and fp32, so the result must double bit-for-bit
    out2 = gg.backend.gmm(a * 2, b, bs, trans_b=trans_b)
    assert torch.equal(out2, out * 2)
    # (3) same launch twice is deterministic
    assert torch.equal(gg.backend.gmm(a, b, bs, trans_b=trans_b), out)
    # (4) one call over all experts == per-expert calls
    e = 4
    solo = gg.backend.gmm(a[starts[e]:starts[e + 1]].contiguous(), b[e:e + 1].contiguous(),
                          torch.tensor([sizes[e]], device="cuda"), trans_b=trans_b)
    assert torch.equal(solo, out[starts[e]:starts[e + 1]])


def test_full_size_wgrad_properties(gg):
    a, _, bs, sizes = _mixtral(gg)
    g = torch.Generator(device="cuda").manual_seed(7)
    grad = torch.randn(32768, 14336, device="cuda", generator=g).bfloat16()
    w = gg.backend.gmm(a, grad, bs, trans_a=True)
    assert w.shape == (8, 4096, 14336)
    # oracle on a sampled block of each expert's output
    starts = np.concatenate([[0], np.cumsum(sizes)])
    for e in (0, 2, 4, 7):
        rows = slice(int(starts[e]), int(starts[e + 1]))
        want = (a[rows, 100:164].float().t() @ grad[rows, 5000:5064].float()).cpu()
        util.assert_close(w[e, 100:164, 5000:5064], want.bfloat16(), rtol=1e-2, atol=1.0, what=f"wgrad expert {e}")
    # doubling one operand doubles the result exactly; repeat run is bit-identical
    assert torch.equal(gg.backend.gmm(a * 2, grad, bs, trans_a=True), w * 2)
    assert torch.equal(gg.backend.gmm(a, grad, bs, trans_a=True), w)


def test_down_projection_config3_full_size(gg):
    """benchmark configuration 3's second projection, b [8, 14336, 4096]: forward, dgrad
    and wgrad at full size, sampled against the oracle, plus the exact doubling
    property."""
    import bench
    sizes = bench.mixtral_batch_sizes()
    starts = np.concatenate([[0], np.cumsum(sizes)])
    g = torch.Generator(device="cuda").manual_seed(3)
    a = torch.randn(32768, 14336, device="cuda", generator=g).bfloat16()
    b = (torch.randn(8, 14336, 4096, device="cuda", generator=g) * 0.02).bfloat16()
    grad = torch.randn(32768, 4096, device="cuda", generator=g).bfloat16()
    bs = torch.tensor(sizes, dtype=torch.int64, device="cuda")
    out = gg.backend.gmm(a, b, bs)
    dx = gg.backend.gmm(grad, b, bs, trans_b=True)
    dw = gg.backend.gmm(a, grad, bs, trans_a=True)
    assert out.shape == (32768, 4096) and dx.shape == (32768, 14336) and dw.shape == (8, 14336, 4096)
    for e in (1, 2, 4):
        rows = torch.tensor([int(starts[e]), int(starts[e + 1]) - 1], device="cuda")
        one = torch.tensor([2])
        util.assert_close(out[rows], gmm_oracle.gmm(a[rows].cpu(), b[e:e + 1].cpu(), one), what=f"fwd expert {e}")
        util.assert_close(dx[rows], gmm_oracle.gmm(grad[rows].cpu(), b[e:e + 1].cpu(), one, trans_b=True),
                          what=f"dgrad expert {e}")
        sl = slice(int(starts[e]), int(starts[e + 1]))
        want = (a[sl, 7000:7064].float().t() @ grad[sl, 1000:1064].float()).cpu()
        util.assert_close(dw[e, 7000:7064, 1000:1064], want.bfloat16(), rtol=1e-2, atol=1.0, what=f"wgrad expert {e}")
    assert torch.equal(gg.backend.gmm(a * 2, b, bs), out * 2)
    assert torch.equal(gg.backend.gmm(a, grad * 2, bs, trans_a=True), dw * 2)


def test_fine_grained_moe_config4_full_size(gg):
    """benchmark configuration 4 at full size (z=256, k=7168, n=2048, 65536 rows, 51 empty
    experts, offsets beyond 2^31): sampled rows of small, large and 1-row
    experts against the oracle; empty experts' wgrad blocks are exactly zero;
    doubling is exact; a second run is bit-identical."""
    import bench
    sizes = bench.fine_grained_batch_sizes()
    starts = np.concatenate([[0], np.cumsum(sizes)])
    g = torch.Generator(device="cuda").manual_seed(2)
    a = torch.randn(65536, 7168, device="cuda", generator=g).bfloat16()
    b = (torch.randn(256, 7168, 2048, device="cuda", generator=g) * 0.02).bfloat16()
    grad = torch.randn(65536, 2048, device="cuda", generator=g).bfloat16()
    bs = torch.tensor(sizes, dtype=torch.int64, device="cuda")
    out = gg.backend.gmm(a, b, bs)
    order = np.argsort(sizes)
    nonempty = [int(e) for e in order if sizes[e] > 0]
    picks = nonempty[:3] + nonempty[len(nonempty) // 2:len(nonempty) // 2 + 2] + nonempty[-2:] + [255 if sizes[255] else nonempty[-3]]
    one = torch.tensor([2])
    for e in picks:
        rows = torch.tensor([int(starts[e]), int(starts[e + 1]) - 1], device="cuda")
        util.assert_close(out[rows], gmm_oracle.gmm(a[rows].cpu(), b[e:e + 1].cpu(), one), what=f"fwd expert {e}")
    assert torch.equal(gg.backend.gmm(a * 2, b, bs), out * 2)
    dx = gg.backend.gmm(grad, b, bs, trans_b=True)
    for e in picks[:4]:
        rows = torch.tensor([int(starts[e]), int(starts[e + 1]) - 1], device="cuda")
        util.assert_close(dx[rows], gmm_oracle.gmm(grad[rows].cpu(), b[e:e + 1].cpu(), one, trans_b=True),
                          what=f"dgrad expert {e}")
    del out, dx
    dw = torch.full((256, 7168, 2048), 3.0, dtype=torch.bfloat16, device="cuda")
    gg.backend.gmm(a, grad, bs, trans_a=True, c=dw)
    for e in range(256):
        if sizes[e] == 0:
            assert bool((dw[e] == 0).all()), f"empty expert {e} not zeroed"
    for e in picks[:5]:
        sl = slice(int(starts[e]), int(starts[e + 1]))
        want = (a[sl, 3000:3064].float().t() @ grad[sl, 500:564].float()).cpu()
        util.assert_close(dw[e, 3000:3064, 500:564], want.bfloat16(), rtol=1e-2, atol=0.5, what=f"wgrad expert {e}")
    again = gg.backend.gmm(a, grad, bs, trans_a=True)
    assert torch.equal(again, dw)


def test_fine_grained_moe_config4_reduced_width(gg):
    """benchmark configuration 4's routing (256 experts, Zipf popularity, ~20 % empty,
    65536 rows) at reduced hidden sizes so the CPU oracle stays in seconds."""
    import bench
    sizes = bench.fine_grained_batch_sizes()
    assert sum(sizes) == 65536 and sum(1 for s in sizes if s == 0) >= 51
    torch.manual_seed(2)
    k, n = 256, 264
    a_cpu = torch.randn(65536, k).bfloat16()
    b_cpu = (torch.randn(256, k, n) * 0.02).bfloat16()
    bs_cpu = torch.tensor(sizes, dtype=torch.int64)
    _check_fwd_bwd(gg, a_cpu, b_cpu, bs_cpu, False, True, ref_stat=False)


def test_degenerate_shapes(gg):
    """Nothing to multiply: no rows, no experts' worth of work, k == 0."""
    dev = "cuda"
    bf = torch.bfloat16
    # no rows at all: forward returns an empty result, wgrad zeros
    a0 = torch.zeros(0, 64, device=dev, dtype=bf)
    b = torch.randn(3, 64, 128, device=dev).to(bf)
    bs0 = torch.zeros(3, dtype=torch.int64, device=dev)
    assert gg.backend.gmm(a0, b, bs0).shape == (0, 128)
    c = torch.full((3, 64, 128), 5.0, device=dev, dtype=bf)
    gg.backend.gmm(a0, torch.zeros(0, 128, device=dev, dtype=bf), bs0, trans_a=True, c=c)
    assert bool((c == 0).all())
    # rows exist but every expert is empty: c untouched, wgrad zeros
    a = torch.randn(10, 64, device=dev).to(bf)
    c = torch.full((10, 128), 5.0, device=dev, dtype=bf)
    gg.backend.gmm(a, b, bs0, c=c)
    assert bool((c == 5.0).all())
    c3 = torch.full((3, 64, 128), 5.0, device=dev, dtype=bf)
    gg.backend.gmm(a, torch.randn(10, 128, device=dev).to(bf), bs0, trans_a=True, c=c3)
    assert bool((c3 == 0).all())
    # k == 0: an empty sum per element
    c = torch.full((10, 128), 5.0, device=dev, dtype=bf)
    gg.backend.gmm(torch.zeros(10, 0, device=dev, dtype=bf), torch.zeros(3, 0, 128, device=dev, dtype=bf),
                   torch.tensor([4, 6, 0], device=dev), c=c)
    assert bool((c == 0).all())


def test_rejected_arguments_launch_nothing(gg):
    from grouped_gemm_b200 import _capi
    a = torch.randn(16, 60, device="cuda").bfloat16()          # 60 is not a multiple of 8
    b = torch.randn(1, 60, 64, device="cuda").bfloat16()
    before = _capi.launch_count()
    with pytest.raises(RuntimeError, match="multiples of 8"):
        gg.backend.gmm(a, b, torch.tensor([16], device="cuda"))
    with pytest.raises(RuntimeError, match="too many experts"):
        gg.backend.gmm(torch.zeros(8, 64, device="cuda", dtype=torch.bfloat16),
                       torch.zeros(1025, 64, 64, device="cuda", dtype=torch.bfloat16),
                       torch.zeros(1025, dtype=torch.int64, device="cuda"))
    assert _capi.launch_count() == before


def test_non_default_stream_and_second_device_guard(gg):
    """Work goes to the caller's current stream."""
    torch.manual_seed(9)
    a = torch.randn(300, 128, device="cuda").bfloat16()
    b = (torch.randn(2, 128, 256, device="cuda") * 0.1).bfloat16()
    bs = torch.tensor([100, 200], device="cuda")
    want = gg.backend.gmm(a, b, bs)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        got = gg.backend.gmm(a, b, bs)
    side.synchronize()
    assert torch.equal(got, want)


def test_call_from_thread_without_bound_context(gg):
    """A thread that has never made a CUDA call of its own (an autograd worker
    served entirely from the allocator cache looks like this) can run gmm: the
    library binds the device's context before it builds tensor maps."""
    import threading
    a = torch.randn(368, 512, device="cuda").bfloat16()
    b = (torch.randn(4, 256, 512, device="cuda") * 0.05).bfloat16()
    bs = torch.tensor([200, 0, 37, 131], device="cuda")
    want = gg.backend.gmm(a, b, bs, trans_b=True)
    c = torch.empty_like(want)
    torch.cuda.synchronize()
    errors = []

    def work():
        try:
            gg.backend.gmm(a, b, bs, trans_b=True, c=c)
        except Exception as e:  # noqa: BLE001
            errors.append(e)

    t = threading.Thread(target=work)
    t.start()
    t.join()
    torch.cuda.synchronize()
    assert not errors, errors
    assert torch.equal(c, want)


@pytest.mark.parametrize("trans_b", [False, True])
@pytest.mark.parametrize("on_device", [False, True])
def test_gmm_scatter_unsorts_in_the_epilogue(gg, trans_b, on_device):
    """gmm_scatter(a, b, bs, out, perm) == scatter of gmm(a, b, bs) by perm, bit for bit;
    rows no index names stay untouched."""
    torch.manual_seed(11)
    sizes = [300, 0, 5, 700, 129, 64]
    T, k, n = sum(sizes), 256, 328
    a = torch.randn(T, k, device="cuda").bfloat16()
    b = (torch.randn(len(sizes), n, k, device="cuda") if trans_b else torch.randn(len(sizes), k, n, device="cuda")).bfloat16() * 0.1
    bs = torch.tensor(sizes, dtype=torch.int64)
    if on_device:
        bs = bs.cuda()
    want_rows = gg.backend.gmm(a, b, bs, trans_b=trans_b)
    R = T + 7
    perm = torch.randperm(R, device="cuda")[:T]
    out = torch.full((R, n), 9.0, device="cuda", dtype=torch.bfloat16)
    got = gg.backend.gmm_scatter(a, b, bs, out, perm, trans_b=trans_b)
    assert got is out
    want = torch.full((R, n), 9.0, device="cuda", dtype=torch.bfloat16)
    want[perm] = want_rows
    assert torch.equal(out, want)
    util.assert_close(want_rows, gmm_oracle.gmm(a.cpu(), b.cpu(), bs.cpu(), trans_b=trans_b), atol=2e-2, what="rows")


@pytest.mark.parametrize("bulk", ["0", "1"], ids=["through-registers", "bulk-copies"])
@pytest.mark.parametrize("trans_b", [False, True])
@pytest.mark.parametrize("sizes,k,n,items,row_elems", [
    ([300, 0, 5, 700, 129, 64], 256, 328, 1500, 200),     # several tiles, rows of 400 bytes
    ([2048, 4096, 512, 1536], 1024, 2048, 9000, 2688),    # many tiles per CTA, rows of 5376 bytes
    ([3, 1, 0, 2], 64, 72, 4000, 8),                      # product far shorter than the transfer, 16-byte rows
    ([0, 0, 0], 64, 72, 300, 64),                         # empty product: the rows still move
])
def test_run_scatter_push_moves_rows_inside_the_launch(gg, monkeypatch, bulk, trans_b, sizes, k, n, items, row_elems):
    """b200gmm_run_scatter_push == b200gmm_run_scatter followed by b200gmm_push_rows,
    bit for bit, for the product and for the pushed rows (two destination buffers,
    gathered through a row index); rows nobody names stay untouched.  Both forms of
    the transfer: through registers by four warps, and as bulk copies by one thread."""
    from grouped_gemm_b200 import _capi
    monkeypatch.setenv("B200GMM_PUSH_TMA", bulk)
    lib = _capi.load()
    torch.manual_seed(31)
    z, T = len(sizes), sum(sizes)
    a = torch.randn(max(T, 1), k, device="cuda").bfloat16()[:T]
    b = (torch.randn(z, n, k, device="cuda") if trans_b else torch.randn(z, k, n, device="cuda")).bfloat16() * 0.1
    bs = torch.tensor(sizes, dtype=torch.int64, device="cuda")
    R = T + 5
    perm = torch.randperm(R, device="cuda")[:T]
    # the transfer: `items` rows of src, chosen through src_row, to rows of two buffers
    src = torch.randn(items + 11, row_elems, device="cuda").bfloat16()
    src_row = torch.randint(0, items + 11, (items,), device="cuda", dtype=torch.int32)
    dst_rank = torch.randint(0, 2, (items,), device="cuda", dtype=torch.int32)
    dst_row = torch.randperm(items, device="cuda").to(torch.int64)

    def run(fused):
        out = torch.full((R, n), 9.0, device="cuda", dtype=torch.bfloat16)
        bufs = [torch.full((items, row_elems), 5.0, device="cuda", dtype=torch.bfloat16) for _ in range(2)]
        table = torch.tensor([t.data_ptr() for t in bufs], dtype=torch.int64, device="cuda")
        dest = perm * (n * 2) + out.data_ptr()
        if T == 0:   # an empty tensor has no address; the table must still be a pointer
            dest = torch.zeros(1, dtype=torch.int64, device="cuda")
        ws_bytes = _capi.workspace_bytes(z)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
        status = gg.backend.backend.device_status(a.device).data_ptr()
        stream = torch.cuda.current_stream().cuda_stream
        head = (a.data_ptr(), b.data_ptr(), dest.data_ptr(), out.data_ptr(), out.numel() * 2, bs.data_ptr(), 1, z,
                T, k, n, 1 if trans_b else 0)
        push = (src.data_ptr(), row_elems * 2, items, src_row.data_ptr(), dst_rank.data_ptr(), dst_row.data_ptr(),
                table.data_ptr())
        if fused:
            rc = lib.b200gmm_run_scatter_push(*head, *push, ws.data_ptr(), ws_bytes, status, stream)
            assert rc == 0, rc
        else:
            rc = lib.b200gmm_run_scatter(*head, ws.data_ptr(), ws_bytes, status, stream)
            assert rc == 0, rc
            rc = lib.b200gmm_push_rows(*push, 0, stream)
            assert rc == 0, rc
        torch.cuda.synchronize()
        return out, bufs

    want_out, want_bufs = run(False)
    got_out, got_bufs = run(True)
    assert torch.equal(got_out, want_out)
    for g_, w_ in zip(got_bufs, want_bufs):
        assert torch.equal(g_, w_)
    # and the transfer is what it says: row dst_row[i] of buffer dst_rank[i] is row src_row[i] of src
    for r in range(2):
        sel = dst_rank == r
        assert torch.equal(got_bufs[r][dst_row[sel]], src[src_row[sel].long()])


@pytest.mark.parametrize("bulk", ["0", "1"], ids=["through-registers", "bulk-copies"])
def test_scatter_push_full_size_under_memory_pressure(gg, monkeypatch, bulk):
    """The product with 1.4 GB of rows moved by its push warps while it runs (the
    size at which a pair of thread blocks once lost the order of its tile
    hand-off: arrivals on a barrier of the other block have to release at cluster
    scope): three launches, each bit-identical to the plain product, the pushed
    rows exact, and no status bit (the hand-off checks itself)."""
    from grouped_gemm_b200 import _capi
    monkeypatch.setenv("B200GMM_PUSH_TMA", bulk)
    lib = _capi.load()
    z, rows, k, n = 16, 65536, 6144, 10752
    g = torch.Generator(device="cuda").manual_seed(1)
    sizes = torch.bincount(torch.randint(0, z, (rows,), generator=torch.Generator().manual_seed(3)), minlength=z)
    bs = sizes.cuda()
    a = torch.randn(rows, k, device="cuda", generator=g).bfloat16()
    w = (torch.randn(z, k, n, device="cuda", generator=g) * 0.02).bfloat16()
    want = gg.backend.gmm(a, w, bs)
    src = torch.randn(rows, n, device="cuda", generator=g).bfloat16()
    src_row = torch.randperm(rows, device="cuda").to(torch.int32)
    dst_row = torch.randperm(rows, device="cuda").to(torch.int64)
    dst_rank = torch.zeros(rows, dtype=torch.int32, device="cuda")
    perm = torch.randperm(rows, device="cuda")
    ws_bytes = _capi.workspace_bytes(z)
    status = gg.backend.backend.device_status(a.device).data_ptr()
    for _ in range(3):
        out = torch.full((rows, n), 9.0, device="cuda", dtype=torch.bfloat16)
        dst = torch.full((rows, n), 5.0, device="cuda", dtype=torch.bfloat16)
        table = torch.tensor([dst.data_ptr()], dtype=torch.int64, device="cuda")
        dest = perm * (n * 2) + out.data_ptr()
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
        rc = lib.b200gmm_run_scatter_push(
            a.data_ptr(), w.data_ptr(), dest.data_ptr(), out.data_ptr(), out.numel() * 2, bs.data_ptr(), 1, z,
            rows, k, n, 0, src.data_ptr(), n * 2, rows, src_row.data_ptr(), dst_rank.data_ptr(), dst_row.data_ptr(),
            table.data_ptr(), ws.data_ptr(), ws_bytes, status, torch.cuda.current_stream().cuda_stream)
        assert rc == 0, rc
        torch.cuda.synchronize()
        assert gg.backend.device_status() == 0
        assert torch.equal(out[perm], want)
        assert torch.equal(dst[dst_row], src[src_row.long()])


def test_randomised_shapes_against_oracle(gg):
    """Seeded random group sizes (tiny, tile-boundary, large, mostly empty), odd
    dimensions, all three layouts, batch sizes on either side: every case against
    the CPU oracle; rows past sum(batch_sizes) must stay untouched."""
    import random
    rng = random.Random(2024)
    torch.manual_seed(2024)
    edge = [0, 1, 7, 63, 64, 65, 127, 128, 129, 255, 256, 257, 300, 511, 513]
    for case in range(40):
        z = rng.choice([1, 2, 3, 5, 8, 17, 40])
        style = rng.choice(["tiny", "edge", "sparse"])
        if style == "tiny":
            sizes = [rng.randint(0, 40) for _ in range(z)]
        elif style == "edge":
            sizes = [rng.choice(edge) for _ in range(z)]
        else:
            sizes = [rng.choice([0, 0, 0, rng.randint(1, 400)]) for _ in range(z)]
        T, d1, n = sum(sizes), rng.choice([8, 16, 72, 128, 200, 264]), rng.choice([8, 24, 64, 136, 256, 328])
        mode, pad = rng.choice(["nn", "nt", "tn"]), rng.choice([0, 3])
        bs_cpu = torch.tensor(sizes, dtype=torch.int64)
        bs = bs_cpu.cuda() if rng.random() < 0.5 else bs_cpu
        a = torch.randn(T + pad, d1).bfloat16()
        what = f"case {case}: {mode} sizes={sizes[:8]} d1={d1} n={n}"
        if mode == "tn":
            b = torch.randn(T + pad, n).bfloat16()
            c = torch.full((z, d1, n), 3.0, dtype=torch.bfloat16, device="cuda")
            gg.backend.gmm(a.cuda(), b.cuda(), bs, trans_a=True, c=c)
            want = gmm_oracle.gmm(a, b, bs_cpu, trans_a=True)
            util.assert_close(c, want, rtol=1e-2, atol=max(1e-2, 2e-3 * float(want.abs().max())), what=what)
        else:
            b = ((torch.randn(z, n, d1) if mode == "nt" else torch.randn(z, d1, n)) * 0.2).bfloat16()
            c = torch.full((T + pad, n), 3.0, dtype=torch.bfloat16, device="cuda")
            gg.backend.gmm(a.cuda(), b.cuda(), bs, trans_b=(mode == "nt"), c=c)
            want = gmm_oracle.gmm(a, b, bs_cpu, trans_b=(mode == "nt"))
            util.assert_close(c[:T], want[:T], rtol=1e-2, atol=2e-2, what=what)
            assert bool((c[T:] == 3.0).all()), what + ": rows past sum(batch_sizes) written"


@pytest.mark.parametrize("trans_b", [False, True])
def test_gmm_gather_fuses_the_sort_by_expert(gg, trans_b):
    """gmm_gather(x, idx, ...) == gmm(x[idx], ...) bit for bit (same tiles, same
    arithmetic; only the way the rows reach shared memory differs), also with the
    un-sort fused on the way out."""
    torch.manual_seed(13)
    sizes = [300, 0, 5, 700, 129, 64, 1, 513]
    T, k, n, R = sum(sizes), 200, 328, 900
    x = torch.randn(R, k, device="cuda").bfloat16()
    idx = torch.randint(0, R, (T,), device="cuda")            # tokens may repeat (top-k routing)
    b = (torch.randn(len(sizes), n, k, device="cuda") if trans_b else torch.randn(len(sizes), k, n, device="cuda")).bfloat16() * 0.1
    bs = torch.tensor(sizes, dtype=torch.int64, device="cuda")
    want = gg.backend.gmm(x[idx].contiguous(), b, bs, trans_b=trans_b)
    got = gg.backend.gmm_gather(x, idx, b, bs, trans_b=trans_b)
    assert torch.equal(got, want)
    util.assert_close(want, gmm_oracle.gmm(x[idx].cpu(), b.cpu(), bs.cpu(), trans_b=trans_b), atol=2e-2, what="rows")
    perm = torch.randperm(T + 4, device="cuda")[:T]
    out = torch.full((T + 4, n), 9.0, device="cuda", dtype=torch.bfloat16)
    gg.backend.gmm_gather(x, idx, b, bs, trans_b=trans_b, out=out, out_index=perm)
    ref = torch.full((T + 4, n), 9.0, device="cuda", dtype=torch.bfloat16)
    ref[perm] = want
    assert torch.equal(out, ref)


@pytest.mark.parametrize("trans_b", [False, True])
def test_gmm_gather_deep_k(gg, trans_b):
    """Many k-blocks per tile (the row copies run several k-blocks ahead of the
    tensor core), a ragged last k-block, more tiles than CTAs."""
    torch.manual_seed(14)
    sizes = [1500, 0, 3000, 37, 4100, 900, 2, 1025]
    T, k, n, R = sum(sizes), 1000, 1536, 5000
    x = torch.randn(R, k, device="cuda").bfloat16()
    idx = torch.randint(0, R, (T,), device="cuda")
    b = (torch.randn(len(sizes), n, k, device="cuda") if trans_b else torch.randn(len(sizes), k, n, device="cuda")).bfloat16() * 0.05
    bs = torch.tensor(sizes, dtype=torch.int64, device="cuda")
    want = gg.backend.gmm(x[idx].contiguous(), b, bs, trans_b=trans_b)
    for _ in range(2):
        got = gg.backend.gmm_gather(x, idx, b, bs, trans_b=trans_b)
        assert torch.equal(got, want)
    assert gg.backend.device_status() == 0


def test_gmm_gather_row_index_out_of_range_reads_zeros(gg):
    """A row index outside x is never dereferenced: the row counts as zeros and
    the status word says so."""
    torch.manual_seed(15)
    sizes = [70, 130]
    T, k, n, R = sum(sizes), 128, 256, 50
    x = torch.randn(R, k, device="cuda").bfloat16()
    idx = torch.randint(0, R, (T,), device="cuda")
    bad = torch.tensor([3, 77, 199], device="cuda")
    idx_bad = idx.clone()
    idx_bad[bad] = torch.tensor([R, -1, 2**31 - 1], device="cuda")
    b = torch.randn(2, k, n, device="cuda").bfloat16() * 0.1
    bs = torch.tensor(sizes, dtype=torch.int64, device="cuda")
    word = gg.backend.backend.device_status("cuda")
    want = gg.backend.gmm_gather(x, idx, b, bs)
    assert gg.backend.device_status() == 0
    got = gg.backend.gmm_gather(x, idx_bad, b, bs)
    assert gg.backend.device_status() & 0x8
    word.zero_()
    want[bad] = 0
    assert torch.equal(got, want)


@pytest.mark.parametrize("trans_b", [False, True])
@pytest.mark.parametrize("sizes,k,n", [
    ([128, 128, 128, 128], 128, 128),            # whole tiles
    ([300, 0, 5, 700, 129, 64, 1, 513], 200, 328),  # ragged rows, k tail, n not a multiple of 128
    ([1000, 24], 512, 72),                        # a single narrow column tile
    ([0, 0, 3], 64, 1040),
])
def test_gmm_swiglu_matches_the_oracle(gg, trans_b, sizes, k, n):
    """silu(a @ b_gate) * (a @ b_up) from one kernel against the fp32 CPU
    composition, and against the two-launch composition on the GPU."""
    torch.manual_seed(16)
    T, z = sum(sizes), len(sizes)
    a = torch.randn(T, k, device="cuda").bfloat16()
    shape = (z, n, k) if trans_b else (z, k, n)
    bg = (torch.randn(*shape, device="cuda") * 0.1).bfloat16()
    bu = (torch.randn(*shape, device="cuda") * 0.1).bfloat16()
    bs = torch.tensor(sizes, dtype=torch.int64, device="cuda")
    got = gg.backend.gmm_swiglu(a, bg, bu, bs, trans_b=trans_b)
    want = gmm_oracle.gmm_swiglu(a.cpu(), bg.cpu(), bu.cpu(), bs.cpu(), trans_b=trans_b)
    util.assert_close(got, want, what="swiglu")
    two = torch.nn.functional.silu(gg.backend.gmm(a, bg, bs, trans_b=trans_b).float()) \
        * gg.backend.gmm(a, bu, bs, trans_b=trans_b).float()
    util.assert_close(got, two, rtol=2e-2, atol=2e-2, what="swiglu vs two launches")
    assert gg.backend.device_status() == 0


def test_gmm_swiglu_many_tiles(gg):
    """More tiles than CTAs, several k-blocks: both accumulator buffers in use."""
    torch.manual_seed(17)
    sizes = [1500, 0, 3000, 37, 4100, 900, 2, 1025]
    T, k, n = sum(sizes), 1024, 1536
    a = torch.randn(T, k, device="cuda").bfloat16()
    bg = (torch.randn(len(sizes), k, n, device="cuda") * 0.05).bfloat16()
    bu = (torch.randn(len(sizes), k, n, device="cuda") * 0.05).bfloat16()
    bs = torch.tensor(sizes, dtype=torch.int64, device="cuda")
    c = torch.full((T + 3, n), 7.0, device="cuda", dtype=torch.bfloat16)
    got = gg.backend.gmm_swiglu(a, bg, bu, bs, c=c[:T])
    want = gmm_oracle.gmm_swiglu(a.cpu(), bg.cpu(), bu.cpu(), bs.cpu())
    util.assert_close(got, want, what="swiglu")
    assert bool((c[T:] == 7.0).all())


@pytest.mark.parametrize("trans_b", [False, True])
def test_gmm_scatter_weighted_topk_combine(gg, trans_b):
    """Top-2 routing: every token has two rows (two experts); one call with
    row_weight and accumulate leaves sum_k w_k * (x @ b[e_k]) in the token's row."""
    torch.manual_seed(18)
    tokens, z, k, n, topk = 700, 6, 200, 328, 2
    x = torch.randn(tokens, k, device="cuda").bfloat16()
    b = (torch.randn(z, n, k, device="cuda") if trans_b else torch.randn(z, k, n, device="cuda")).bfloat16() * 0.1
    experts = torch.stack([torch.randperm(z, device="cuda")[:topk] for _ in range(tokens)])  # [tokens, 2] distinct
    weights = torch.rand(tokens, topk, device="cuda")
    flat_e = experts.reshape(-1)
    order = torch.argsort(flat_e, stable=True)
    token_of_row = (order // topk)
    a = x[token_of_row].contiguous()
    w = weights.reshape(-1)[order].contiguous()
    bs = torch.bincount(flat_e, minlength=z).to(torch.int64)
    out = torch.zeros(tokens + 2, n, device="cuda", dtype=torch.bfloat16)
    gg.backend.gmm_scatter(a, b, bs, out, token_of_row, trans_b=trans_b, row_weight=w, accumulate=True)
    rows = gmm_oracle.gmm(a.cpu().float(), b.cpu().float(), bs.cpu(), trans_b=trans_b)   # fp32 rows
    want = torch.zeros(tokens + 2, n)
    want.index_add_(0, token_of_row.cpu(), rows * w.cpu()[:, None])
    util.assert_close(out, want, rtol=2e-2, atol=2e-2, what="weighted top-k combine")
    assert bool((out[tokens:] == 0).all())
    # weights without accumulation: plain scatter of w * row (distinct destinations)
    out2 = torch.full((a.shape[0], n), 3.0, device="cuda", dtype=torch.bfloat16)
    perm = torch.randperm(a.shape[0], device="cuda")
    gg.backend.gmm_scatter(a, b, bs, out2, perm, trans_b=trans_b, row_weight=w)
    want2 = torch.empty(a.shape[0], n)
    want2[perm.cpu()] = rows * w.cpu()[:, None]
    util.assert_close(out2, want2, what="weighted scatter")
    assert gg.backend.device_status() == 0


@pytest.mark.parametrize("sizes,k,n", [
    ([300, 0, 5, 700, 129, 64, 1, 513], 200, 328),   # ragged k-blocks, empty expert, m and n tails
    ([64, 64, 64, 64], 128, 256),                     # whole k-blocks
    ([1500, 0, 3000, 37, 4100, 900, 2, 1025], 1000, 1536),  # many k-blocks per tile, many tiles
])
def test_gmm_gather_wgrad_matches_plain_wgrad(gg, sizes, k, n):
    """x[idx]^T @ grad per expert with the gather inside the kernel: bit-identical to
    the plain wgrad on the permuted copy (same tiles, same arithmetic)."""
    torch.manual_seed(19)
    T, R = sum(sizes), 2000
    x = torch.randn(R, k, device="cuda").bfloat16()
    idx = torch.randint(0, R, (T,), device="cuda")
    grad = torch.randn(T, n, device="cuda").bfloat16()
    bs = torch.tensor(sizes, dtype=torch.int64, device="cuda")
    want = gg.backend.gmm(x[idx].contiguous(), grad, bs, trans_a=True)
    for _ in range(2):
        got = gg.backend.gmm_gather_wgrad(x, idx, grad, bs)
        assert torch.equal(got, want)
    util.assert_close(want, gmm_oracle.gmm(x[idx].cpu(), grad.cpu(), bs.cpu(), trans_a=True), atol=3e-2, rtol=2e-2,
                      what="wgrad")
    assert gg.backend.device_status() == 0


@pytest.mark.parametrize("trans_b", [False, True])
def test_fused_gmm_gather_autograd(gg, trans_b):
    """fused.gmm_gather(x, idx, b) against ops.gmm(x[idx], b): same value, same
    gradients for x (summed over the rows that share a token) and b."""
    from grouped_gemm_b200 import fused
    torch.manual_seed(20)
    sizes = [300, 0, 5, 700, 129, 64]
    T, R, k, n = sum(sizes), 500, 200, 328
    x0 = torch.randn(R, k, device="cuda").bfloat16()
    b0 = (torch.randn(len(sizes), n, k, device="cuda") if trans_b else torch.randn(len(sizes), k, n, device="cuda")).bfloat16() * 0.1
    idx = torch.randint(0, R, (T,), device="cuda")
    bs = torch.tensor(sizes, dtype=torch.int64, device="cuda")
    dy = torch.randn(T, n, device="cuda").bfloat16()
    x1, b1 = x0.clone().requires_grad_(True), b0.clone().requires_grad_(True)
    y1 = fused.gmm_gather(x1, idx, b1, bs, trans_b)
    y1.backward(dy)
    x2, b2 = x0.clone().requires_grad_(True), b0.clone().requires_grad_(True)
    y2 = gg.ops.gmm(x2[idx], b2, bs, trans_b)
    y2.backward(dy)
    assert torch.equal(y1, y2)
    assert torch.equal(b1.grad, b2.grad)
    # x.grad: every token's row is the sum of the bf16 dgrad rows that name it.  The
    # fused path adds them in bf16 in memory (each addition rounds a partial sum that
    # is at most the sum of magnitudes), so the bound grows with the number of rows.
    rows = gg.backend.gmm(dy, b0, bs, trans_b=not trans_b).float()
    ref = torch.zeros(R, k, device="cuda").index_add_(0, idx, rows)
    mag = torch.zeros(R, k, device="cuda").index_add_(0, idx, rows.abs())
    count = torch.bincount(idx, minlength=R).float()[:, None]
    bound = 2.0 ** -8 * (count + 1) * mag + 1e-3
    err = (x1.grad.float() - ref).abs()
    assert bool((err <= bound).all()), f"x.grad: max excess {float((err - bound).max()):.4g}"
    err2 = (x2.grad.float() - ref).abs()   # torch's own bf16 index backward, same bound
    assert bool((err2 <= bound).all()), f"unfused x.grad: max excess {float((err2 - bound).max()):.4g}"


def test_status_flags_bad_batch_sizes(gg):
    """sum(batch_sizes) > rows of a: the kernel clamps, writes nothing out of
    bounds and raises the overflow status bit."""
    a = torch.randn(100, 64, device="cuda").bfloat16()
    b = torch.randn(2, 64, 128, device="cuda").bfloat16()
    c = torch.zeros(100 + 64, 128, device="cuda", dtype=torch.bfloat16)
    word = gg.backend.backend.device_status("cuda")
    gg.backend.gmm(a, b, torch.tensor([90, 90], device="cuda"), c=c[:100])
    assert gg.backend.device_status() & 0x4
    assert bool((c[100:] == 0).all())
    word.zero_()


@pytest.mark.parametrize("accumulate", [False, True])
@pytest.mark.parametrize("sizes", [[70, 130], [600, 40, 0, 9]])
def test_gmm_scatter_row_index_out_of_range_is_skipped_and_flagged(gg, sizes, accumulate):
    """A destination index outside ``out`` is never written through (neither by
    the store nor by the reduce-add form): the row is dropped, the words around
    ``out`` stay as they were and the status word says so.  The same index then
    reaches the kernel again through the backward of the gathered product."""
    torch.manual_seed(21)
    T, k, n, R = sum(sizes), 128, 264, 37
    a = torch.randn(T, k, device="cuda").bfloat16()
    b = torch.randn(len(sizes), k, n, device="cuda").bfloat16() * 0.1
    bs = torch.tensor(sizes, dtype=torch.int64, device="cuda")
    idx = torch.randperm(T, device="cuda") % R if accumulate else torch.randperm(max(T, R), device="cuda")[:T] % max(T, R)
    rows = R if accumulate else max(T, R)
    # ``out`` sits inside a larger buffer whose margins must survive
    margin = 16
    buf = torch.full((rows + 2 * margin, n), 7.0, device="cuda", dtype=torch.bfloat16)
    out = buf[margin:margin + rows]
    out.zero_()
    word = gg.backend.backend.device_status("cuda")
    good = torch.zeros_like(out)
    gg.backend.gmm_scatter(a, b, bs, good, idx, accumulate=accumulate)
    assert gg.backend.device_status() == 0
    bad_rows = torch.tensor([1, T // 2, T - 1], device="cuda")
    idx_bad = idx.clone()
    idx_bad[bad_rows] = torch.tensor([-1, rows, rows + 5], device="cuda")   # just below, just past, inside the margin
    gg.backend.gmm_scatter(a, b, bs, out, idx_bad, accumulate=accumulate)
    assert gg.backend.device_status() & 0x10
    word.zero_()
    assert bool((buf[:margin] == 7.0).all()) and bool((buf[margin + rows:] == 7.0).all()), "wrote outside out"
    if not accumulate:
        # every row but the three dropped ones arrived
        keep = torch.ones(T, dtype=torch.bool, device="cuda")
        keep[bad_rows] = False
        assert torch.equal(out[idx[keep]], good[idx[keep]])
        assert bool((out[idx[bad_rows]] == 0).all())


@pytest.mark.parametrize("trans_b", [False, True])
@pytest.mark.parametrize("sizes,k,n", [
    ([128, 128, 128, 128], 128, 128),
    ([300, 0, 5, 700, 129, 64, 1, 513], 200, 328),
    ([2000, 24], 512, 72),
])
def test_fused_gmm_swiglu_autograd(gg, trans_b, sizes, k, n):
    """fused.gmm_swiglu forward and backward against torch.autograd on the fp32
    composition of the oracle's per-expert loop (ops.py:14-29's contract, twice)."""
    from grouped_gemm_b200 import fused
    torch.manual_seed(31)
    T, z = sum(sizes), len(sizes)
    a_cpu = torch.randn(T, k).bfloat16()
    shape = (z, n, k) if trans_b else (z, k, n)
    wg_cpu = (torch.randn(*shape) * 0.1).bfloat16()
    wu_cpu = (torch.randn(*shape) * 0.1).bfloat16()
    dh_cpu = torch.randn(T, n).bfloat16()
    bs_cpu = torch.tensor(sizes, dtype=torch.int64)
    # fp32 reference with autograd
    a32, wg32, wu32 = (t.float().requires_grad_(True) for t in (a_cpu, wg_cpu, wu_cpu))
    outs, start = [], 0
    for i, size in enumerate(sizes):
        rows = a32[start:start + size]
        g = rows @ (wg32[i].t() if trans_b else wg32[i])
        u = rows @ (wu32[i].t() if trans_b else wu32[i])
        outs.append(torch.nn.functional.silu(g) * u)
        start += size
    ref = torch.cat(outs)
    ref.backward(dh_cpu.float())
    a = a_cpu.cuda().requires_grad_(True)
    wg = wg_cpu.cuda().requires_grad_(True)
    wu = wu_cpu.cuda().requires_grad_(True)
    out = fused.gmm_swiglu(a, wg, wu, bs_cpu.cuda(), trans_b)
    util.assert_close(out, ref.detach(), what="gated forward")
    out.backward(dh_cpu.cuda())
    # gradients are sums over up to 2000 rows / 328 columns of bf16-rounded terms:
    # tolerance relative to the size of the gradient tensor, as for the plain backward
    for got, want, name in ((a.grad, a32.grad, "a.grad"), (wg.grad, wg32.grad, "b_gate.grad"), (wu.grad, wu32.grad, "b_up.grad")):
        scale = float(want.abs().max()) + 1e-6
        err = (got.float().cpu() - want).abs()
        assert bool((err <= 2e-2 * scale + 1e-2 * want.abs()).all()), f"{name}: max err {float(err.max()):.4g} (scale {scale:.4g})"
    assert bool((wg.grad[[i for i, s_ in enumerate(sizes) if s_ == 0]] == 0).all())


@pytest.mark.parametrize("world", [1, 8])
def test_expert_parallel_per_rank_shape_config5(gg, world):
    """benchmark configuration 5 as one rank sees it: hidden 6144, ffn 10752, 64 / world
    local experts with that rank's share of the 262144 routed rows (uniform top-4
    routing, seed 3).  Forward, dgrad and wgrad at full per-rank size (world 8) or
    at a quarter of the rows per expert (world 1, to bound memory): sampled rows
    against the oracle, exact doubling, bit-identical repeat."""
    import bench
    counts = torch.bincount(bench.ep_routing().reshape(-1), minlength=64).tolist()
    per = 64 // world
    sizes = counts[:per] if world == 8 else [c // 4 for c in counts]
    z, k, n, T = len(sizes), 6144, 10752, sum(sizes)
    starts = np.concatenate([[0], np.cumsum(sizes)])
    g = torch.Generator(device="cuda").manual_seed(3)
    a = torch.randn(T, k, device="cuda", generator=g).bfloat16()
    b = (torch.randn(z, k, n, device="cuda", generator=g) * 0.02).bfloat16()
    grad = torch.randn(T, n, device="cuda", generator=g).bfloat16()
    bs = torch.tensor(sizes, dtype=torch.int64, device="cuda")
    out = gg.backend.gmm(a, b, bs)
    dx = gg.backend.gmm(grad, b, bs, trans_b=True)
    dw = gg.backend.gmm(a, grad, bs, trans_a=True)
    one = torch.tensor([2])
    for e in sorted({0, z // 2, z - 1}):
        rows = torch.tensor([int(starts[e]), int(starts[e + 1]) - 1], device="cuda")
        util.assert_close(out[rows], gmm_oracle.gmm(a[rows].cpu(), b[e:e + 1].cpu(), one), what=f"fwd expert {e}")
        util.assert_close(dx[rows], gmm_oracle.gmm(grad[rows].cpu(), b[e:e + 1].cpu(), one, trans_b=True),
                          what=f"dgrad expert {e}")
        sl = slice(int(starts[e]), int(starts[e + 1]))
        want = (a[sl, 3000:3064].float().t() @ grad[sl, 9000:9064].float()).cpu()
        util.assert_close(dw[e, 3000:3064, 9000:9064], want.bfloat16(), rtol=1e-2, atol=1.0, what=f"wgrad expert {e}")
    assert torch.equal(gg.backend.gmm(a * 2, b, bs), out * 2)
    assert torch.equal(gg.backend.gmm(a, grad, bs, trans_a=True), dw)
