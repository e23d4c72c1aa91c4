"""Generate tests/golden/ops_test_golden.npz from the reference's own test code.

The reference's parity contract is its test file, grouped_gemm/ops_test.py: an
input generator (``randn``, :39-41) and a per-expert matmul oracle (``gmm``,
:44-53).  That file cannot be imported without the compiled CUDA extension, so
this script reads its source text from the reference checkout, extracts those two
function definitions with ``ast`` and executes them unchanged on CPU
(``Tensor.cuda`` is made a no-op for the duration).  Nothing from the reference is
written into this repository except the numbers its functions produce.

Run where a checkout of the reference exists:
    python tests/golden/make_golden.py /path/to/reference
(or set GROUPED_GEMM_REFERENCE).  Tests never run this; they read the committed .npz.

Cases follow the reference's grid (ops_test.py:29-36, :59-109, :143-158):
fixed and variable batch sizes, both trans_b settings, forward and the
``out.sum().backward()`` gradients, plus the all-ones zero-k known answer.
bf16 tensors are stored as their uint16 bit patterns.
"""
import ast
import hashlib
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "ops_test_golden.npz")

# (z, m, k, n, variable-size settings): the reference's whole grid
# (ops_test.py:29-36) with fixed and variable sizes, plus a smaller shape of the
# same family.  Results of more than MAX_ELEMS elements are stored as a regular
# sample (every sr-th row, every sc-th column of the tensor seen as 2-D), the steps
# beside them, so that the fixture stays around 1 MB.
CASES = [
    (1, 128, 128, 128, (False, True)),
    (8, 128, 128, 128, (False, True)),
    (16, 128, 128, 128, (False, True)),
    (1, 128, 256, 512, (False, True)),
    (8, 128, 256, 512, (False, True)),
    (16, 128, 256, 512, (False, True)),
    (4, 64, 128, 128, (False, True)),
]
MAX_ELEMS = 8192


def sample_steps(rows, cols):
    """Row and column steps that bring rows x cols down to about MAX_ELEMS; odd, so
    that the sample does not lock onto tile boundaries."""
    sr = sc = 1
    while (rows // sr + 1) * (cols // sc + 1) > MAX_ELEMS:
        if rows // sr >= cols // sc:
            sr += 2
        else:
            sc += 2
    return sr, sc


def sampled(t):
    t2 = t.detach().reshape(-1, t.shape[-1])
    sr, sc = sample_steps(t2.shape[0], t2.shape[1])
    return bits(t2[::sr, ::sc]), np.array([sr, sc], dtype=np.int64)


def load_reference_functions(ref_root):
    path = os.path.join(ref_root, "grouped_gemm", "ops_test.py")
    tree = ast.parse(open(path).read(), path)
    wanted = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name in ("randn", "gmm")]
    assert {n.name for n in wanted} == {"randn", "gmm"}
    ns = {"torch": torch, "np": np}
    exec(compile(ast.Module(body=wanted, type_ignores=[]), path, "exec"), ns)
    return ns["randn"], ns["gmm"]


def bits(t):
    return t.detach().contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def variable_sizes(z, m):
    # ops_test.py:87-92
    dist = torch.rand(z)
    dist /= dist.sum()
    batch_sizes = (dist * m).to(torch.long)
    batch_sizes[-1] += m * z - batch_sizes.sum()
    return batch_sizes


def main():
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("GROUPED_GEMM_REFERENCE", "reference")
    randn, ref_gmm = load_reference_functions(ref_root)
    real_cuda = torch.Tensor.cuda
    torch.Tensor.cuda = lambda self, *a, **k: self
    out = {}
    try:
        for (z, m, k, n, variants) in CASES:
            for trans_b in (False, True):
                for variable in variants:
                    torch.manual_seed(0)
                    a = randn(z, m, k).view(-1, k)
                    b = randn(z, n, k) if trans_b else randn(z, k, n)
                    bs = variable_sizes(z, m) if variable else torch.tensor([m] * z)
                    a.requires_grad_(True)
                    b.requires_grad_(True)
                    expected = ref_gmm(a, b, bs, trans_b)
                    expected.sum().backward()
                    key = f"z{z}_m{m}_k{k}_n{n}_tb{int(trans_b)}_var{int(variable)}"
                    out[key + "/batch_sizes"] = bs.numpy().astype(np.int64)
                    for name, t in (("out", expected), ("a_grad", a.grad), ("b_grad", b.grad)):
                        out[key + "/" + name], out[key + "/" + name + "_step"] = sampled(t)
                    # inputs are regenerated from the seed by the tests; the digest
                    # detects a generator that drifted
                    h = hashlib.sha256(bits(a).tobytes() + bits(b).tobytes()).hexdigest()
                    out[key + "/input_sha256"] = np.frombuffer(h.encode(), dtype=np.uint8)
    finally:
        torch.Tensor.cuda = real_cuda
    np.savez_compressed(OUT, **out)
    print(OUT, os.path.getsize(OUT), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main()
