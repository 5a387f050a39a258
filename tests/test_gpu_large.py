"""Segments longer than the shared-memory sort holds (max(N, M) > 16384): the global-memory
sort/rank path, through the same operators, against the C checker."""

import pytest
import torch

from oracle import sorted_scan
from util import make_inputs, rel_err

pytestmark = pytest.mark.gpu
TOL = 1e-4
# Laplace with tens of thousands of keys per unit length: every prefix state is a product of thousands of
# step decays that sit a few ulps below 1, and their fp32 rounding alone costs ~3e-5 at N = 65536 and
# ~3e-4 at N = 262144 (measured with a correctly rounded CPU emulation); the north-star bound against
# float64 is 1e-3
TOL_DENSE = 1e-3


@pytest.mark.parametrize("shape", [(1, 2, 20000, 17000, 8), (1, 2, 300, 40000, 4), (2, 1, 65536, 65536, 16), (1, 1, 262144, 131072, 4)])
def test_laplace_forward(shape):
    from weighted_laplace_sum import weighted_laplace_sum
    P, D, N, M, C = shape
    q, k, v = make_inputs(P, D, N, M, C, seed=N + M, scale=1.0)
    out_w, out_u = weighted_laplace_sum(q, k, v)
    ref_w, ref_u = sorted_scan.laplace_sum(q, k, v)
    tol = TOL_DENSE if N >= 65536 else TOL
    print("rel err", rel_err(out_w, ref_w), rel_err(out_u, ref_u))
    assert rel_err(out_w, ref_w) < tol, rel_err(out_w, ref_w)
    assert rel_err(out_u, ref_u) < tol, rel_err(out_u, ref_u)


@pytest.mark.parametrize("shape", [(1, 2, 20000, 17000, 8), (1, 1, 65536, 65536, 16)])
def test_abs_forward_backward_sgn(shape):
    import qlka_native
    from weighted_abs_sum import weighted_abs_sum_full, weighted_sgn_sum
    P, D, N, M, C = shape
    q, k, v = make_inputs(P, D, N, M, C, seed=N + 2 * M, scale=1.0)
    g = torch.Generator().manual_seed(5)
    g_w, g_u = torch.randn(P, M, C, generator=g).cuda(), torch.randn(P, M, generator=g).cuda()
    out_w, out_u = weighted_abs_sum_full(q, k, v)
    ref_w, ref_u = sorted_scan.abs_sum(q, k, v)
    assert rel_err(out_w, ref_w) < TOL and rel_err(out_u, ref_u) < TOL
    gq, gk, gv = qlka_native.abs_backward(q, k, v, g_w, g_u)
    rq, rk, rv = sorted_scan.abs_sum_backward(q, k, v, g_w, g_u)
    assert rel_err(gq, rq) < TOL and rel_err(gk, rk) < TOL and rel_err(gv, rv) < TOL
    assert rel_err(weighted_sgn_sum(q, k, v, g_w), sorted_scan.sgn_sum(q, k, v, g_w)) < TOL


def test_length_limit():
    from weighted_laplace_sum import weighted_laplace_sum
    q = torch.zeros(1, 1, 262145, device="cuda")
    with pytest.raises(RuntimeError, match="262144"):
        weighted_laplace_sum(q, q, torch.zeros(1, 262145, 1, device="cuda"))
