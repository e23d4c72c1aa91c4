"""CPU-only checks of the Python mirror of the reference API: names, argument
checks and error types (no kernel runs; every case fails validation first)."""
import inspect

import pytest
import torch

import grouped_gemm_b200 as grouped_gemm
from grouped_gemm_b200 import backend, ops


def test_api_surface_matches_reference():
    # grouped_gemm/__init__.py:1-2, ops.py:32-33, backend.py:24
    assert grouped_gemm.ops is ops and grouped_gemm.backend is backend
    assert list(inspect.signature(ops.gmm).parameters) == ["a", "b", "batch_sizes", "trans_b"]
    assert list(inspect.signature(backend.gmm).parameters) == [
        "a", "b", "batch_sizes", "trans_a", "trans_b", "c"]
    assert issubclass(ops.GroupedGemm, torch.autograd.Function)
    # the test-suite of the reference reaches the backend through ops (ops_test.py:154)
    assert ops.backend.gmm is backend.gmm
    # the native binding is a compiled (pybind11) function: its signature is in its docstring
    doc = backend.backend.gmm.__doc__
    assert ("gmm(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor, batch_sizes: torch.Tensor, "
            "trans_a: bool, trans_b: bool) -> None") in doc
    assert type(backend.backend.gmm).__name__ == "builtin_function_or_method"


def _t(*shape, dtype=torch.bfloat16):
    return torch.zeros(*shape, dtype=dtype)


def test_allocate_output_shapes_and_asserts():
    bs = torch.tensor([4, 4])
    assert backend._allocate_output(_t(8, 16), _t(2, 16, 24), bs, False, False).shape == (8, 24)
    assert backend._allocate_output(_t(8, 16), _t(2, 24, 16), bs, False, True).shape == (8, 24)
    assert backend._allocate_output(_t(8, 16), _t(8, 24), bs, True, False).shape == (2, 16, 24)
    with pytest.raises(AssertionError):
        backend._allocate_output(_t(8, 16), _t(2, 16, 24), bs, True, True)
    with pytest.raises(AssertionError):
        backend._allocate_output(_t(8, 16), _t(2, 16, 24), bs.view(1, 2), False, False)
    with pytest.raises(AssertionError):
        backend._allocate_output(_t(2, 4, 16), _t(2, 16, 24), bs, False, False)
    with pytest.raises(AssertionError):
        backend._allocate_output(_t(8, 16), _t(16, 24), bs, False, False)


@pytest.mark.parametrize("kwargs,fragment", [
    (dict(trans_a=True, trans_b=True), "only one of"),
    (dict(batch_sizes=torch.tensor([4, 4], dtype=torch.int32)), "int64"),
    (dict(batch_sizes=torch.tensor([[4, 4]])), "1-D"),
    (dict(), "a must be a CUDA tensor"),
])
def test_native_binding_checks_raise_runtime_error(kwargs, fragment):
    args = dict(a=_t(8, 16), b=_t(2, 16, 24), c=_t(8, 24), batch_sizes=torch.tensor([4, 4]),
                trans_a=False, trans_b=False)
    args.update(kwargs)
    with pytest.raises(RuntimeError, match=fragment):
        backend.backend.gmm(args["a"], args["b"], args["c"], args["batch_sizes"], args["trans_a"],
                            args["trans_b"])


def test_no_cpu_fallback():
    """CPU tensors are refused, not computed some other way."""
    with pytest.raises(RuntimeError):
        ops.gmm(_t(8, 16), _t(2, 16, 24), torch.tensor([4, 4]))


def test_fused_entry_points_refuse_cpu_tensors():
    """gmm_scatter / gmm_gather / gmm_swiglu have no CPU path either."""
    a, b, bs = _t(8, 16), _t(2, 16, 24), torch.tensor([4, 4])
    with pytest.raises(RuntimeError):
        backend.gmm_swiglu(a, b, b.clone(), bs)
    with pytest.raises(RuntimeError):
        backend.gmm_gather(a, torch.arange(8), b, bs)
    with pytest.raises(RuntimeError):
        backend.gmm_scatter(a, b, bs, _t(8, 24), torch.arange(8))
    with pytest.raises(RuntimeError):
        backend.gmm_gather_wgrad(a, torch.arange(8), _t(8, 24), bs)
    from grouped_gemm_b200 import fused
    with pytest.raises(RuntimeError):
        fused.gmm_gather(a, torch.arange(8), b, bs)


@pytest.mark.parametrize("trans_b", [False, True])
def test_fused_gather_autograd_plumbing(monkeypatch, trans_b):
    """The operand choice of fused.GatheredGroupedGemm.backward, checked on CPU by
    standing the oracle in for the four kernels it calls: the gradients must equal
    those autograd derives for gmm(x[idx], b) written as a per-expert loop."""
    from grouped_gemm_b200 import fused
    from oracle import gmm_oracle

    def fake_gather(x, idx, b, bs, trans_b=False):
        return gmm_oracle.gmm(x[idx], b, bs, trans_b=trans_b)

    def fake_scatter(a, b, bs, out, row_index, trans_b=False, row_weight=None, accumulate=False):
        rows = gmm_oracle.gmm(a, b, bs, trans_b=trans_b)
        assert accumulate and row_weight is None
        return out.index_add_(0, row_index, rows)

    def fake_gather_wgrad(x, idx, grad, bs):
        return gmm_oracle.gmm(x[idx], grad, bs, trans_a=True)

    def fake_gmm(a, b, bs, trans_a=False, trans_b=False, c=None):
        return gmm_oracle.gmm(a, b, bs, trans_a=trans_a, trans_b=trans_b)

    monkeypatch.setattr(fused.backend, "gmm_gather", fake_gather)
    monkeypatch.setattr(fused.backend, "gmm_scatter", fake_scatter)
    monkeypatch.setattr(fused.backend, "gmm_gather_wgrad", fake_gather_wgrad)
    monkeypatch.setattr(fused.backend, "gmm", fake_gmm)

    torch.manual_seed(5)
    sizes, R, k, n = [5, 0, 9, 2], 12, 16, 24
    T = sum(sizes)
    bs = torch.tensor(sizes)
    idx = torch.randint(0, R, (T,))
    x0 = torch.randn(R, k, dtype=torch.float64)
    b0 = torch.randn(len(sizes), n, k, dtype=torch.float64) if trans_b else torch.randn(len(sizes), k, n, dtype=torch.float64)
    dy = torch.randn(T, n, dtype=torch.float64)

    x1, b1 = x0.clone().requires_grad_(True), b0.clone().requires_grad_(True)
    y1 = fused.gmm_gather(x1, idx, b1, bs, trans_b)
    y1.backward(dy)

    x2, b2 = x0.clone().requires_grad_(True), b0.clone().requires_grad_(True)
    a2, out, start = x2[idx], [], 0
    for i, size in enumerate(sizes):
        rhs = b2[i].t() if trans_b else b2[i]
        out.append(a2[start:start + size] @ rhs)
        start += size
    y2 = torch.cat(out)
    y2.backward(dy)
    # the oracle multiplies in fp32
    assert torch.allclose(y1, y2.detach(), rtol=1e-4, atol=1e-4)
    assert torch.allclose(x1.grad, x2.grad, rtol=1e-4, atol=1e-4)
    assert torch.allclose(b1.grad, b2.grad, rtol=1e-4, atol=1e-4)
