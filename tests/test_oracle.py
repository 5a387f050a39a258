"""The checkers themselves: fp64 direct evaluation and the C sorted-scan restatement
against the golden vectors produced by the reference's own Python code, and against
each other (CPU only)."""

import os

import numpy as np
import pytest
import torch

from oracle import chunked_ref, direct, sorted_scan

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def rel(a, b):
    a, b = torch.as_tensor(a, dtype=torch.float64), torch.as_tensor(b, dtype=torch.float64)
    return ((a - b).abs().max() / b.abs().max().clamp_min(1e-30)).item()


@pytest.fixture(scope="module")
def small():
    z = np.load(os.path.join(GOLD, "small_kernels.npz"))
    return {k: torch.from_numpy(z[k]) if z[k].ndim else float(z[k]) for k in z.files}


@pytest.mark.parametrize("kernel", ["add_laplace", "add_riesz", "add_bump"])
@pytest.mark.parametrize("masked", [False, True])
def test_kernel_matrix_and_attention_match_reference(small, kernel, masked):
    q, k, v, tau = small["q"], small["k"], small["v"], small["tau"]
    B, H, S, D = q.shape
    keep = small["keep"] if masked else None
    qp, kp = q.transpose(2, 3).reshape(B * H, D, S), k.transpose(2, 3).reshape(B * H, D, S)
    keep_p = None if keep is None else keep.repeat_interleave(H, dim=0)
    sfx = "_masked" if masked else ""
    A = direct.kernel_matrix(kernel, qp, kp, tau, keep_p)
    assert rel(A, small[f"A_{kernel}{sfx}"]) < 2e-6          # golden is fp32
    att = direct.attention(q, k, v, kernel, tau, keep)
    assert rel(att, small[f"att_{kernel}{sfx}"]) < 2e-5


def test_raw_sums_match_reference_kernel_matrices(small):
    """The operator-level sums are the kernel matrices contracted with [v, 1]."""
    q, k, v, tau = small["q"], small["k"], small["v"], small["tau"]
    B, H, S, D = q.shape
    P = B * H
    qp, kp, vp = (q / tau).transpose(2, 3).reshape(P, D, S), (k / tau).transpose(2, 3).reshape(P, D, S), v.reshape(P, S, D)
    A = small["A_add_laplace"].double()
    ow, ou = direct.laplace_sum(qp, kp, vp)
    assert rel(ow, A @ vp.double()) < 2e-6 and rel(ou, A.sum(2)) < 2e-6
    # add_riesz: A = |q|_1 + |k|_1 - |q-k|_1 + eps  ->  |q-k|_1 = |q|_1 + |k|_1 + eps - A
    Ar = small["A_add_riesz"].double()
    d1 = qp.double().abs().sum(1)[:, :, None] + kp.double().abs().sum(1)[:, None, :] + direct.EPS - Ar
    aw, au = direct.abs_sum(qp, kp, vp)
    assert rel(aw, d1 @ vp.double()) < 1e-5 and rel(au, d1.sum(2)) < 1e-5
    for fn in (sorted_scan.laplace_sum,):
        w2, u2 = fn(qp, kp, vp)
        assert rel(w2, ow) < 1e-12 and rel(u2, ou) < 1e-12
    w2, u2 = sorted_scan.abs_sum(qp, kp, vp)
    assert rel(w2, aw) < 1e-12 and rel(u2, au) < 1e-12


def test_config1_add_laplace_matches_reference():
    z = np.load(os.path.join(GOLD, "c1_add_laplace.npz"))
    q, k, v = (torch.from_numpy(z[n]) for n in ("q", "k", "v"))
    tau = float(z["tau"])
    B, H, S, D = q.shape
    P = B * H
    qp, kp, vp = (q / tau).transpose(2, 3).reshape(P, D, S), (k / tau).transpose(2, 3).reshape(P, D, S), v.reshape(P, S, D)
    ow, ou = sorted_scan.laplace_sum(qp, kp, vp)
    att = (ow / ou.clamp_min(direct.CLAMP)[:, :, None]).view(B, H, S, D)
    assert rel(att, z["naive"]) < 1e-5
    assert rel(att, z["chunked"]) < 1e-5
    mine = chunked_ref.add_laplace_attention_chunked(qp.contiguous(), kp.contiguous(), vp, tau).view(B, H, S, D)
    assert rel(mine, z["chunked"]) < 1e-5
    # one head through the O(N^2) fp64 definition as well
    dw, du = direct.laplace_sum(qp[:1], kp[:1], vp[:1])
    assert rel(ow[:1], dw) < 1e-12 and rel(ou[:1], du) < 1e-12


@pytest.mark.parametrize("shape", [(2, 3, 1, 1, 1), (1, 2, 33, 17, 5), (2, 4, 130, 257, 9)])
def test_sorted_scan_against_direct(shape):
    P, D, N, M, C = shape
    g = torch.Generator().manual_seed(N * 1000 + M)
    q, k, v = torch.randn(P, D, M, generator=g), torch.randn(P, D, N, generator=g), torch.randn(P, N, C, generator=g)
    gw, gu = torch.randn(P, M, C, generator=g), torch.randn(P, M, generator=g)
    n_tie = min(N, M, 4)
    k[0, 0, :n_tie] = q[0, 0, :n_tie]
    k[0, 1, :] = k[0, 1, 0]                                  # all keys equal in one dimension
    for a, b in zip(sorted_scan.laplace_sum(q, k, v), direct.laplace_sum(q, k, v)):
        assert rel(a, b) < 1e-12
    for a, b in zip(sorted_scan.abs_sum(q, k, v), direct.abs_sum(q, k, v)):
        assert rel(a, b) < 1e-12
    for a, b in zip(sorted_scan.abs_sum_backward(q, k, v, gw, gu), direct.abs_sum_backward(q, k, v, gw, gu)):
        assert rel(a, b) < 1e-12
    for a, b in zip(sorted_scan.abs_sum_backward(q, k, v, gw), direct.abs_sum_backward(q, k, v, gw)):
        assert rel(a, b) < 1e-12
    assert rel(sorted_scan.sgn_sum(q, k, v, gw), direct.sgn_sum(q, k, v, gw)) < 1e-12


def test_backward_is_the_autograd_gradient_away_from_ties():
    g = torch.Generator().manual_seed(7)
    P, D, N, M, C = 2, 3, 19, 23, 4
    q = torch.randn(P, D, M, generator=g, dtype=torch.float64, requires_grad=True)
    k = torch.randn(P, D, N, generator=g, dtype=torch.float64, requires_grad=True)
    v = torch.randn(P, N, C, generator=g, dtype=torch.float64, requires_grad=True)
    gw, gu = torch.randn(P, M, C, generator=g, dtype=torch.float64), torch.randn(P, M, generator=g, dtype=torch.float64)
    A = (k[:, :, None, :] - q[:, :, :, None]).abs().sum(1)
    ((A @ v) * gw).sum().add((A.sum(2) * gu).sum()).backward()
    # the checkers take fp32 inputs: compare on fp32-rounded copies
    q32, k32, v32 = q.detach().float(), k.detach().float(), v.detach().float()
    got = direct.abs_sum_backward(q32, k32, v32, gw.float(), gu.float())
    for a, b in zip(got, (q.grad, k.grad, v.grad)):
        assert rel(a, b) < 1e-5
