"""The schedule the GEMM kernels build for themselves, read back from the GPU, and
the kernels' bounded wait run to its limit.

``b200gmm_schedule_device`` runs the kernels' own prologue (prefix sums of
batch_sizes, expert order, tile prefix sums) and tile decoder in one CTA; the
result must equal the host replay (``b200gmm_schedule_host``) integer for
integer, which in turn is pinned to properties by the CPU tests.  This is the
scan the GEMM runs, not a sibling of it.
"""
import ctypes

import numpy as np
import pytest
import torch

from grouped_gemm_b200 import _capi

pytestmark = pytest.mark.gpu


def _host(sizes, tokens, d1, n, trans_a, trans_b, ctas):
    lib = _capi.load()
    bs = np.asarray(sizes, dtype=np.int64)
    count = ctypes.c_int64(0)
    assert lib.b200gmm_schedule_host(bs.ctypes.data, len(sizes), tokens, d1, n, trans_a, trans_b, ctas, None, 0,
                                     ctypes.byref(count)) == 0
    out = np.zeros((count.value, _capi.SCHEDULE_FIELDS), dtype=np.int64)
    assert lib.b200gmm_schedule_host(bs.ctypes.data, len(sizes), tokens, d1, n, trans_a, trans_b, ctas,
                                     out.ctypes.data, count.value, ctypes.byref(count)) == 0
    return out


def _device(sizes, tokens, d1, n, trans_a, trans_b, ctas, max_tiles):
    lib = _capi.load()
    bs = torch.tensor([int(s) for s in sizes], dtype=torch.int64, device="cuda")
    out = torch.full((max_tiles, _capi.SCHEDULE_FIELDS), -1, dtype=torch.int32, device="cuda")
    count = torch.zeros(1, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = lib.b200gmm_schedule_device(bs.data_ptr(), len(sizes), tokens, d1, n, trans_a, trans_b, ctas,
                                     out.data_ptr(), max_tiles, count.data_ptr(), status.data_ptr(),
                                     torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    return out.cpu().numpy().astype(np.int64), int(count.item()), int(status.item())


def _cases():
    import bench
    rng = np.random.default_rng(11)
    return {
        "cfg1": ([128] * 4, 128, 128),
        "mixtral": (bench.mixtral_batch_sizes(), 4096, 14336),
        "fine": (bench.fine_grained_batch_sizes(), 7168, 2048),
        "edge": ([219, 2246, 5, 8103, 1, 1117, 4693, 0], 1024, 3584),
        "remainders": ([64, 65, 192, 193, 16, 17, 0, 128, 127, 129], 512, 328),
        "z1024": ([int(v) for v in rng.integers(0, 300, size=1024)], 256, 512),
        "ties": ([64] * 37, 128, 256),
        "all-empty": ([0] * 5, 128, 256),
    }


@pytest.mark.parametrize("case", sorted(_cases()))
@pytest.mark.parametrize("mode", ["nn", "nt", "tn"])
@pytest.mark.parametrize("ctas,light", [(1, "0"), (1, "1"), (2, "0")])
def test_device_schedule_equals_host_replay(case, mode, ctas, light, monkeypatch):
    monkeypatch.setenv("B200GMM_LIGHT", light)
    sizes, d1, n = _cases()[case]
    tokens = sum(sizes)
    ta, tb = int(mode == "tn"), int(mode == "nt")
    want = _host(sizes, tokens, d1, n, ta, tb, ctas)
    got, count, status = _device(sizes, tokens, d1, n, ta, tb, ctas, max(len(want), 1))
    assert status == 0
    assert count == len(want)
    assert np.array_equal(got[:count], want)


def test_device_schedule_clamps_and_flags_bad_sizes():
    # sum(batch_sizes) beyond the rows of a, and a negative size: rows are clamped,
    # the status word says why, and host and device still agree
    sizes, tokens = [100, -5, 100, 100], 150
    want = _host(sizes, tokens, 128, 256, 0, 0, 1)
    got, count, status = _device(sizes, tokens, 128, 256, 0, 0, 1, 64)
    assert count == len(want) and np.array_equal(got[:count], want)
    assert status == (_capi.STATUS_NEGATIVE_SIZE | _capi.STATUS_ROWS_OVERFLOW)
    assert int((got[:count, 1] + got[:count, 3]).max()) <= tokens


def test_bounded_wait_runs_out_and_reports_timeout():
    """A wait that nothing ends returns after its limit with STATUS_TIMEOUT; the
    context stays usable and the next GEMM is correct."""
    lib = _capi.load()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    assert lib.b200gmm_selftest_wait_timeout(500_000, status.data_ptr(), stream) == 0   # 0.5 ms
    t1.record()
    torch.cuda.synchronize()
    assert int(status.item()) == _capi.STATUS_TIMEOUT
    assert 0.4 <= t0.elapsed_time(t1) < 50.0, "the wait must last its limit, not longer"
    # limits that would hold the GPU for no reason are refused on the host
    assert lib.b200gmm_selftest_wait_timeout(10 ** 9, status.data_ptr(), stream) == -1
    assert lib.b200gmm_selftest_wait_timeout(0, status.data_ptr(), stream) == -1
    # the context is intact: a product right after it is exact
    import grouped_gemm_b200 as gg
    a = torch.ones(192, 128, device="cuda", dtype=torch.bfloat16)
    b = torch.ones(3, 128, 64, device="cuda", dtype=torch.bfloat16)
    out = gg.backend.gmm(a, b, torch.tensor([64, 0, 128]))
    assert bool((out == 128).all())
    assert gg.backend.device_status() == 0
