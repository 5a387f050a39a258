"""Drop-in proof with the reference's own caller: its unmodified `kernel_attention/attention.py`
(Experiments/kernel_attention/attention.py:95-126, which does `from weighted_abs_sum import
weighted_abs_sum_full` and `from weighted_laplace_sum import weighted_laplace_sum` at :11-12) is imported
from the staged copy under baseline/_ref/ (oracle/ref_python.py) with this repository's two packages on
sys.path, so every efficient-path call of its `attention()` lands in this library. Skipped where the
staged copy is absent."""

import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
KERNELS = ("add_laplace", "add_riesz", "add_bump")


@pytest.fixture(scope="module")
def ref_attention():
    from oracle import ref_python
    mod = ref_python.load(stub_extensions=False)
    if mod is None:
        pytest.skip("the reference's attention.py is not staged (baseline/_ref/Experiments/kernel_attention)")
    import weighted_abs_sum
    import weighted_laplace_sum
    # the names the reference's module bound at import are this library's operators
    assert mod.weighted_abs_sum_full is weighted_abs_sum.weighted_abs_sum_full
    assert mod.weighted_laplace_sum is weighted_laplace_sum.weighted_laplace_sum
    return mod


@pytest.mark.parametrize("masked", [False, True])
@pytest.mark.parametrize("kernel", KERNELS)
def test_reference_caller_on_the_drop_in_packages_matches_its_golden_vectors(ref_attention, kernel, masked):
    """S = 48: below the reference's keops threshold, so its _abs_sum passes backend="keops" (attention.py:62-64)."""
    z = np.load(os.path.join(GOLD, "small_kernels.npz"))
    q, k, v = (torch.from_numpy(z[n]).cuda() for n in ("q", "k", "v"))
    keep = torch.from_numpy(z["keep"]).cuda() if masked else None
    with torch.no_grad():
        got = ref_attention.attention(q, k, v, kernel, float(z["tau"]), keep, impl="efficient")
    want = torch.from_numpy(z[f"att_{kernel}" + ("_masked" if masked else "")])
    assert got.shape == want.shape
    assert (got.cpu() - want).abs().max().item() < 2e-5 * max(1.0, want.abs().max().item())


@pytest.mark.parametrize("masked", [False, True])
@pytest.mark.parametrize("kernel", KERNELS)
def test_reference_caller_efficient_equals_its_own_naive_path(ref_attention, kernel, masked):
    """S = 700 (backend "cuda" in the reference's dispatch): `impl="efficient"` over this library against
    `impl="naive"`, the reference's full kernel matrix, both evaluated by the reference's own module on the GPU."""
    g = torch.Generator().manual_seed(21)
    B, H, S, D = 2, 3, 700, 16
    q, k, v = (torch.randn(B, H, S, D, generator=g).cuda() for _ in range(3))
    keep = (torch.rand(B, S, generator=g) > 0.2).cuda() if masked else None
    tau = ref_attention.KERNELS and {"add_laplace": 0.5, "add_riesz": 1.0, "add_bump": 1.5}[kernel]
    with torch.no_grad():
        fast = ref_attention.attention(q, k, v, kernel, tau, keep, impl="efficient")
        slow = ref_attention.attention(q, k, v, kernel, tau, keep, impl="naive")
    err = (fast - slow).abs().max().item() / slow.abs().max().item()
    assert err < 1e-4, err


def test_reference_caller_trains_through_the_abs_sum(ref_attention):
    """add_riesz with gradients: the reference's route differentiates its algebra around weighted_abs_sum_full
    (attention.py:75-81); the gradients must agree with autograd through its naive kernel matrix."""
    g = torch.Generator().manual_seed(22)
    B, H, S, D = 1, 2, 400, 8
    leaves = [torch.randn(B, H, S, D, generator=g).cuda().requires_grad_(True) for _ in range(3)]
    w = torch.randn(B, H, S, D, generator=g).cuda()
    (ref_attention.attention(*leaves, "add_riesz", 1.0, None, impl="efficient") * w).sum().backward()
    fast = [t.grad.clone() for t in leaves]
    for t in leaves:
        t.grad = None
    (ref_attention.attention(*leaves, "add_riesz", 1.0, None, impl="naive") * w).sum().backward()
    for a, b in zip(fast, (t.grad for t in leaves)):
        assert ((a - b).abs().max() / b.abs().max()).item() < 2e-3
