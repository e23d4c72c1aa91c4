"""CPU-only checks of the C-ABI library: it loads, exports every symbol the
header declares, rejects bad arguments with the documented codes before touching
CUDA, and its host replay of the tile schedule covers every output exactly once."""
import ctypes
import os
import re

import numpy as np
import pytest

from grouped_gemm_b200 import _capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "b200gmm.h")


def _header_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200gmm_\w+)\s*\(", text)))


def test_header_symbols_all_exported():
    lib = ctypes.CDLL(_capi.LIB_PATH)
    names = _header_symbols()
    assert len(names) >= 7
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/b200gmm.h but not exported"
    assert set(names) == set(_capi.SIGNATURES), "ctypes prototypes out of step with the header"


def test_strerror_and_tile_shape():
    assert _capi.strerror(0) == "ok"
    assert "trans_a" in _capi.strerror(-1)
    assert _capi.tile_shape(1) == (128, 256, 64)
    assert _capi.tile_shape(2) == (256, 256, 64)


def test_workspace_bytes():
    maps = 256 * 8 * 2 * 128  # per-CTA tensor-map copies for wgrad
    assert _capi.workspace_bytes(0) == 128 + maps
    assert _capi.workspace_bytes(8) == 128 + maps
    assert _capi.workspace_bytes(100) == 896 + maps  # 800 + 16 rounded up to 128
    with pytest.raises(RuntimeError):
        _capi.workspace_bytes(_capi.MAX_EXPERTS + 1)


@pytest.mark.parametrize("kwargs,code", [
    (dict(trans_a=1, trans_b=1), -1),
    (dict(d1=100), -2),            # not a multiple of 8
    (dict(n=12), -2),
    (dict(z=2000), -3),
    (dict(tokens=-1), -1),
    (dict(tokens=2 ** 31), -3),
])
def test_run_rejects_bad_arguments_before_cuda(kwargs, code):
    args = dict(z=4, tokens=512, d1=128, n=128, trans_a=0, trans_b=0)
    args.update(kwargs)
    lib = _capi.load()
    rc = lib.b200gmm_run(None, None, None, None, 0, args["z"], args["tokens"], args["d1"], args["n"],
                         args["trans_a"], args["trans_b"], None, 0, None, None)
    assert rc == code


def test_run_with_no_work_is_ok_without_gpu():
    lib = _capi.load()
    # z == 0, and non-transposed with zero rows: nothing to do, no CUDA call made.
    assert lib.b200gmm_run(None, None, None, None, 0, 0, 0, 128, 128, 0, 0, None, 0, None, None) == 0
    bs = np.zeros(4, dtype=np.int64)
    assert lib.b200gmm_run(None, None, None, bs.ctypes.data, 0, 4, 0, 128, 128, 0, 0, None, 0, None, None) == 0


def test_fused_entry_points_reject_bad_arguments_before_cuda():
    """Argument checks of the scatter / combine / gather / swiglu entry points
    that return before any CUDA call (so they can run without a GPU)."""
    lib = _capi.load()
    bs = np.array([64, 64], dtype=np.int64)
    dummy = np.zeros(64, dtype=np.int64).ctypes.data  # any non-null, 16-byte aligned address
    # scatter and combine need a destination table
    assert lib.b200gmm_run_scatter(dummy, dummy, None, None, 0, bs.ctypes.data, 0, 2, 128, 64, 64, 0, None, 0, None, None) == -1
    assert lib.b200gmm_run_combine(dummy, dummy, None, None, 0, None, 1, bs.ctypes.data, 0, 2, 128, 64, 64, 0, None, 0, None, None) == -1
    # combine: weights must be 4-byte aligned; k == 0 overwrite has nothing to write through
    assert lib.b200gmm_run_combine(dummy, dummy, dummy, None, 0, dummy + 2, 1, bs.ctypes.data, 0, 2, 128, 64, 64, 0, None, 0, None, None) == -2
    assert lib.b200gmm_run_combine(dummy, dummy, dummy, None, 0, None, 0, bs.ctypes.data, 0, 2, 128, 0, 64, 0, None, 0, None, None) == -1
    assert lib.b200gmm_run_combine(dummy, dummy, dummy, None, 0, None, 1, bs.ctypes.data, 0, 2, 128, 0, 64, 0, None, 0, None, None) == 0
    # gather: row index table, a non-empty source below 2^31 rows, an output of some kind
    assert lib.b200gmm_run_gather(dummy, 100, None, dummy, dummy, None, None, 0, bs.ctypes.data, 0, 2, 128, 64, 64, 0, None, 0, None, None) == -1
    assert lib.b200gmm_run_gather(dummy, 0, dummy, dummy, dummy, None, None, 0, bs.ctypes.data, 0, 2, 128, 64, 64, 0, None, 0, None, None) == -1
    assert lib.b200gmm_run_gather(dummy, 2 ** 31, dummy, dummy, dummy, None, None, 0, bs.ctypes.data, 0, 2, 128, 64, 64, 0, None, 0, None, None) == -1
    assert lib.b200gmm_run_gather(dummy, 100, dummy, dummy, None, None, None, 0, bs.ctypes.data, 0, 2, 128, 64, 64, 0, None, 0, None, None) == -1
    # swiglu: both weight tensors, an output, column count a multiple of 8
    assert lib.b200gmm_run_swiglu(dummy, dummy, None, dummy, None, None, 0, bs.ctypes.data, 0, 2, 128, 64, 64, 0, None, 0, None, None) == -1
    assert lib.b200gmm_run_swiglu(dummy, dummy, dummy, None, None, None, 0, bs.ctypes.data, 0, 2, 128, 64, 64, 0, None, 0, None, None) == -1
    assert lib.b200gmm_run_swiglu(dummy, dummy, dummy, dummy, None, None, 0, bs.ctypes.data, 0, 2, 128, 64, 60, 0, None, 0, None, None) == -2
    assert lib.b200gmm_run_swiglu(dummy, dummy, dummy + 8, dummy, None, None, 0, bs.ctypes.data, 0, 2, 128, 64, 64, 0, None, 0, None, None) == -2
    # a destination window needs a destination table
    assert lib.b200gmm_run_gather(dummy, 100, dummy, dummy, dummy, None, dummy, 64, bs.ctypes.data, 0, 2, 128, 64, 64, 0, None, 0, None, None) == -1
    # the static-scratch entry point refuses more experts than its scratch holds
    assert lib.b200gmm_run_static(dummy, dummy, dummy, bs.ctypes.data, 0, 257, 128, 64, 64, 0, 0, None, None) == -3


def _schedule(sizes, tokens, d1, n, trans_a, trans_b, ctas=1):
    lib = _capi.load()
    bs = np.asarray(sizes, dtype=np.int64)
    count = ctypes.c_int64(0)
    ptr = bs.ctypes.data if len(sizes) else None
    rc = lib.b200gmm_schedule_host(ptr, len(sizes), tokens, d1, n, trans_a, trans_b, ctas, None, 0,
                                   ctypes.byref(count))
    assert rc == 0
    out = np.zeros((count.value, _capi.SCHEDULE_FIELDS), dtype=np.int64)
    rc = lib.b200gmm_schedule_host(ptr, len(sizes), tokens, d1, n, trans_a, trans_b, ctas,
                                   out.ctypes.data, count.value, ctypes.byref(count))
    assert rc == 0
    return out


SIZE_SETS = [
    [128] * 4,
    [219, 2246, 5, 8103, 1, 1117, 4693, 0],
    [0, 0, 0],
    [1],
    [3400, 1030, 17412, 1225, 363, 5908, 1691, 1739],
    [7, 0, 300, 129, 128, 127, 0, 1025],
    [64, 65, 192, 193, 16, 17],
]


@pytest.mark.parametrize("sizes", SIZE_SETS)
@pytest.mark.parametrize("trans_b", [0, 1])
@pytest.mark.parametrize("n", [128, 256, 328, 1536])
@pytest.mark.parametrize("ctas", [1, 2])
@pytest.mark.parametrize("light", ["0", "1"])
def test_schedule_covers_rows_and_columns_once(sizes, trans_b, n, ctas, light, monkeypatch):
    """Every output element belongs to exactly one tile: 128-column granularity,
    since the transposed tiles of the one-CTA variant (B200GMM_LIGHT=1) are 128
    columns wide."""
    monkeypatch.setenv("B200GMM_LIGHT", light)
    tokens = sum(sizes)
    tile_m = 128 * ctas
    tiles = _schedule(sizes, tokens, 512, n, 0, trans_b, ctas)
    cover = np.zeros((tokens, (n + 127) // 128), dtype=np.int32)
    starts = np.concatenate([[0], np.cumsum(sizes)])
    for e, row0, col0, valid, stages, kind in tiles:
        width = 128 if kind else 256
        assert col0 % width == 0 and col0 < n
        assert starts[e] <= row0 and row0 + valid <= starts[e + 1], "tile leaves its expert's rows"
        if kind:
            assert light == "1" and ctas == 1 and 0 < valid <= 64 and stages == 512 // 128
            assert row0 == starts[e] and row0 + valid == starts[e + 1], "a transposed tile holds a whole small expert"
        else:
            assert 0 < valid <= tile_m and stages == 512 // 64
            if ctas == 1 and light == "1":
                assert sizes[e] > 64, "experts of at most 64 rows go to transposed tiles"
        cover[row0:row0 + valid, col0 // 128:(col0 + width + 127) // 128] += 1
    assert (cover == 1).all()


@pytest.mark.parametrize("sizes", SIZE_SETS)
@pytest.mark.parametrize("ctas", [1, 2])
def test_schedule_wgrad_full_grid_for_every_expert(sizes, ctas):
    tokens, m, n = sum(sizes), 320, 520
    tile_m = 128 * ctas
    tiles = _schedule(sizes, tokens, m, n, 1, 0, ctas)
    per_expert = ((m + tile_m - 1) // tile_m) * ((n + 255) // 256)
    assert len(tiles) == per_expert * len(sizes)
    for e, size in enumerate(sizes):
        mine = tiles[tiles[:, 0] == e]
        cover = np.zeros(((m + tile_m - 1) // tile_m, (n + 255) // 256), dtype=np.int32)
        for _, row0, col0, valid, stages, kind in mine:
            assert kind == 0
            assert valid == min(tile_m, m - row0)
            assert stages == (size + 63) // 64  # 0 for an empty expert: zero-fill tile
            cover[row0 // tile_m, col0 // 256] += 1
        assert (cover == 1).all()


def test_schedule_order_largest_experts_first_for_wgrad():
    """wgrad launch order: experts sorted by rows, largest first (ties keep their
    index order), so that the launch ends on the shortest tiles."""
    sizes = [10, 500, 0, 70, 3000, 200]
    tiles = _schedule(sizes, sum(sizes), 128, 256, 1, 0, 1)     # one tile per expert
    assert tiles[:, 0].tolist() == [4, 1, 5, 3, 0, 2]
    tiles = _schedule([64, 64, 64, 64], 256, 128, 256, 1, 0, 1)
    assert tiles[:, 0].tolist() == [0, 1, 2, 3]
    # the forward layouts keep the experts in index order
    for ctas in (1, 2):
        tiles = _schedule([600, 100, 900], 1600, 128, 256, 0, 0, ctas)
        assert (np.diff(tiles[:, 0]) >= 0).all()


def test_schedule_clamps_rows_past_tokens():
    # sum(batch_sizes) > tokens must never schedule a row >= tokens
    for ctas in (1, 2):
        tiles = _schedule([100, 100, 100], 150, 128, 256, 0, 0, ctas)
        assert int((tiles[:, 1] + tiles[:, 3]).max()) <= 150


def test_variant_choice_depends_on_shapes_only(monkeypatch):
    """cluster_ctas=0 asks for the variant b200gmm_run would use: pairs for
    experts with many rows, single CTAs for fine-grained groups."""
    monkeypatch.setenv("B200GMM_LIGHT", "1")
    big = _schedule([4096] * 8, 32768, 512, 512, 0, 0, 0)
    small = _schedule([64] * 64, 4096, 512, 512, 0, 0, 0)
    assert int(big[:, 3].max()) == 256 and int(small[:, 3].max()) == 64
    assert (small[:, 5] == 1).all(), "64-row experts run as transposed tiles"
