"""CPU tests that pin the oracle: against golden vectors produced by the
reference's own test functions, against the reference's known-answer case, and
the numpy restatement of the argument fill against the C one."""
import numpy as np
import pytest
import torch

from oracle import gmm_oracle
from tests import util


def _inputs_for(key):
    z, m, k, n, trans_b, variable = util.parse_key(key)
    torch.manual_seed(0)
    a = util.reference_inputs(z, m, k).view(-1, k)
    b = util.reference_inputs(z, n, k) if trans_b else util.reference_inputs(z, k, n)
    return a, b, trans_b


_DATA, _KEYS = util.golden_cases()


@pytest.mark.parametrize("key", _KEYS)
def test_oracle_matches_reference_golden(key):
    a, b, trans_b = _inputs_for(key)
    digest = bytes(_DATA[key + "/input_sha256"]).decode()
    assert util.input_digest(a, b) == digest, "seeded inputs differ from the ones the golden was made with"
    bs = torch.from_numpy(_DATA[key + "/batch_sizes"])
    out = gmm_oracle.gmm(a, b, bs, trans_b=trans_b)
    gold, out_s = util.golden_pair(_DATA, key, "out", out)
    # The golden is the reference loop in bf16 on CPU; this oracle upcasts to
    # fp32 first.  Both accumulate in fp32 and round once, so they agree to the
    # last bit except where summation order flips a rounding.
    assert gmm_oracle.reference_allclose_pct(out_s, gold) <= 2.0
    util.assert_close(out_s, gold, rtol=1e-2, atol=1e-6, what="forward")
    # gradients of out.sum(): upstream gradient of ones (ops_test.py:77-80)
    grad = torch.ones_like(out)
    agrad, bgrad = gmm_oracle.gmm_backward(a, b, bs, grad, trans_b=trans_b)
    for got, name in ((agrad, "a_grad"), (bgrad, "b_grad")):
        gold, got_s = util.golden_pair(_DATA, key, name, got)
        util.assert_close(got_s, gold, rtol=1e-2, atol=1e-6, what=name)


def test_oracle_zero_k_known_answer():
    # grouped_gemm/ops_test.py:143-158: all-ones operands, sizes [0,128,0,64],
    # stale ones in c must become exact 0 / 128 / 0 / 64.
    a = torch.ones(192, 128, dtype=torch.bfloat16)
    b = torch.ones(192, 128, dtype=torch.bfloat16)
    c = torch.ones(4, 128, 128, dtype=torch.bfloat16)
    bs = torch.tensor([0, 128, 0, 64])
    gmm_oracle.gmm(a, b, bs, trans_a=True, c=c)
    for i, want in enumerate((0, 128, 0, 64)):
        assert bool((c[i] == want).all())


@pytest.mark.parametrize("trans_a,trans_b", [(False, False), (False, True), (True, False)])
@pytest.mark.parametrize("sizes", [[128] * 4, [219, 2246, 5, 8103, 1, 1117, 4693, 0], [0], [], [7] * 300])
def test_fill_numpy_equals_c(sizes, trans_a, trans_b):
    lib = util.load_c_oracle()
    bs = np.asarray(sizes, dtype=np.int64)
    got = gmm_oracle.fill_offsets(bs, 7168, 2048, trans_a, trans_b)
    want = np.zeros((len(sizes), 9), dtype=np.int64)
    if len(sizes):
        lib.oracle_fill_offsets(bs.ctypes.data, len(sizes), 7168, 2048, int(trans_a), int(trans_b),
                                want.ctypes.data)
    assert np.array_equal(got, want)


def test_fill_hand_checked_values():
    # NN, k=4, n=6, sizes [2,0,3]: starts 0,2,2.
    got = gmm_oracle.fill_offsets([2, 0, 3], 4, 6, False, False)
    assert got.tolist() == [
        [2, 6, 4, 4, 6, 6, 0, 0, 0],
        [0, 6, 4, 4, 6, 6, 8, 24, 12],
        [3, 6, 4, 4, 6, 6, 8, 48, 12],
    ]
    # NT differs only in ldb = k.
    assert gmm_oracle.fill_offsets([2, 0, 3], 4, 6, False, True)[:, 4].tolist() == [4, 4, 4]
    # TN, m=4, n=6: k_i = sizes, lda = m, a_off = m*start, b_off = start*n, c_off = e*m*n.
    got = gmm_oracle.fill_offsets([2, 0, 3], 4, 6, True, False)
    assert got.tolist() == [
        [4, 6, 2, 4, 6, 6, 0, 0, 0],
        [4, 6, 0, 4, 6, 6, 8, 12, 24],
        [4, 6, 3, 4, 6, 6, 8, 12, 48],
    ]


def test_fill_is_int64_beyond_int32():
    # The reference multiplies ints (csrc/fill_arguments.cuh:72-76); at
    # z=256, k=7168, n=2048 the last b offset is 255*7168*2048 > 2^31.
    got = gmm_oracle.fill_offsets([1] * 256, 7168, 2048, False, False)
    assert got[255, 7] == 255 * 7168 * 2048 > 2 ** 31


@pytest.mark.parametrize("trans_a,trans_b", [(False, False), (False, True), (True, False)])
def test_torch_oracle_equals_c_oracle_bitwise(trans_a, trans_b):
    """Two independent restatements (torch fp32 matmul vs scalar C loop) agree
    on a small ragged case up to fp32 summation order."""
    lib = util.load_c_oracle()
    torch.manual_seed(3)
    sizes = [5, 0, 19, 8]
    T, d1, n = sum(sizes), 24, 16
    a = torch.randn(T, d1).bfloat16()
    if trans_a:
        b = torch.randn(T, n).bfloat16()
        c = torch.zeros(len(sizes), d1, n, dtype=torch.bfloat16)
    else:
        b = (torch.randn(len(sizes), n, d1) if trans_b else torch.randn(len(sizes), d1, n)).bfloat16()
        c = torch.zeros(T, n, dtype=torch.bfloat16)
    bs = np.asarray(sizes, dtype=np.int64)
    lib.oracle_gmm_bf16(a.data_ptr(), b.data_ptr(), c.data_ptr(), bs.ctypes.data, len(sizes), d1, n,
                        int(trans_a), int(trans_b))
    want = gmm_oracle.gmm(a, b, torch.from_numpy(bs), trans_a=trans_a, trans_b=trans_b)
    util.assert_close(c, want, rtol=2 ** -7, atol=1e-3, what="C vs torch oracle")


def test_swiglu_composition():
    """gmm_swiglu = silu(gate product) * up product, per expert, fp32 inside."""
    torch.manual_seed(3)
    a = torch.randn(10, 16).bfloat16()
    bg, bu = torch.randn(2, 16, 8).bfloat16(), torch.randn(2, 16, 8).bfloat16()
    got = gmm_oracle.gmm_swiglu(a, bg, bu, torch.tensor([4, 6]))
    want = torch.empty(10, 8)
    for i, (s0, s1) in enumerate([(0, 4), (4, 10)]):
        gate = a[s0:s1].float() @ bg[i].float()
        want[s0:s1] = gate / (1 + torch.exp(-gate)) * (a[s0:s1].float() @ bu[i].float())
    assert torch.equal(got, want.bfloat16())
    got_t = gmm_oracle.gmm_swiglu(a, bg.transpose(1, 2).contiguous(), bu.transpose(1, 2).contiguous(),
                                  torch.tensor([4, 6]), trans_b=True)
    assert torch.equal(got_t, got)
