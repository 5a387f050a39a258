"""Parity with the reference's own CUDA extensions, compiled for sm_100 by oracle/build_ref.py
(binaries under oracle/_ref/; skipped when they are not there). Same seeded inputs, the bound of
the north star: max|a - b| / max|b| <= 1e-4."""

import pytest
import torch

from util import make_inputs, rel_err

pytestmark = pytest.mark.gpu
TOL = 1e-4


@pytest.fixture(scope="module")
def ref():
    from oracle import build_ref
    mods = build_ref.load_ref()
    if len(mods) < 2:
        pytest.skip("reference extensions not built (oracle/_ref)")
    return mods


SHAPES = [(2, 4, 300, 260, 16), (2, 8, 2000, 2500, 64), (1, 4, 5000, 5000, 33), (2, 2, 16384, 16384, 64)]


@pytest.mark.parametrize("shape", SHAPES)
def test_laplace_forward(ref, shape):
    from weighted_laplace_sum import weighted_laplace_sum
    P, D, N, M, C = shape
    q, k, v = make_inputs(P, D, N, M, C, seed=N + M, scale=2.0)
    rw, ru = ref["laplace"].weighted_laplace_sum_forward(q, k, v)
    ow, ou = weighted_laplace_sum(q, k, v)
    assert rel_err(ow, rw.double()) < TOL and rel_err(ou, ru.double()) < TOL


@pytest.mark.parametrize("shape", SHAPES)
def test_abs_forward_backward_sgn(ref, shape):
    import qlka_native
    P, D, N, M, C = shape
    q, k, v = make_inputs(P, D, N, M, C, seed=N + 3 * M, scale=0.5)
    g = torch.Generator().manual_seed(8)
    g_w, g_u = torch.randn(P, M, C, generator=g).cuda(), torch.randn(P, M, generator=g).cuda()
    rw, ru = ref["abs"].weighted_abs_sum_full_forward(q, k, v, -1)
    ow, ou = qlka_native.abs_forward(q, k, v, full=True)
    assert rel_err(ow, rw.double()) < TOL and rel_err(ou, ru.double()) < TOL
    for mine, theirs in zip(qlka_native.abs_backward(q, k, v, g_w, g_u), ref["abs"].weighted_abs_sum_full_backward(q, k, v, g_w, g_u)):
        assert rel_err(mine, theirs.double()) < TOL
    for mine, theirs in zip(qlka_native.abs_backward(q, k, v, g_w), ref["abs"].weighted_abs_sum_backward(q, k, v, g_w)):
        assert rel_err(mine, theirs.double()) < TOL
    assert rel_err(qlka_native.sgn_forward(q, k, v, g_w), ref["abs"].weighted_sgn_sum_forward(q, k, v, g_w).double()) < TOL
