"""Gradients of weighted_laplace_sum on the GPU (through the C ABI) against float64 checkers.

The reference has no Laplace backward (training goes through its chunked PyTorch route,
Experiments/kernel_attention/attention.py:110-115), so the checkers are the direct float64
formula with the walk's tie rule and, away from ties, torch autograd through exp(-|k - q|).
"""

import pytest
import torch

from oracle import direct
from util import make_inputs, rel_err

pytestmark = pytest.mark.gpu
TOL = 1e-4          # max|a-b| / max|b| against float64

SHAPES = [
    (1, 1, 1, 1, 1), (2, 3, 7, 5, 4), (1, 2, 8, 9, 3), (2, 4, 100, 77, 32), (1, 3, 257, 300, 33),
    (1, 2, 64, 1000, 64), (1, 2, 1000, 3, 65), (2, 2, 600, 600, 64), (1, 2, 1024, 1024, 128),
    (1, 3, 2049, 1500, 16), (1, 2, 4096, 4096, 64), (2, 2, 5000, 7000, 8),
]


def _grads(P, M, C, seed, device="cuda"):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(P, M, C, generator=g).to(device), torch.randn(P, M, generator=g).to(device)


@pytest.mark.parametrize("full", [False, True])
@pytest.mark.parametrize("shape", SHAPES)
def test_backward_matches_direct(shape, full):
    from weighted_laplace_sum import weighted_laplace_sum_backward
    P, D, N, M, C = shape
    q, k, v = make_inputs(P, D, N, M, C, seed=3 * N + M + C, scale=2.0)
    g_w, g_u = _grads(P, M, C, seed=N + 7)
    if not full:
        g_u = None
    gq, gk, gv = weighted_laplace_sum_backward(q, k, v, g_w, g_u)
    torch.cuda.synchronize()
    rq, rk, rv = direct.laplace_sum_backward(q, k, v, g_w, g_u)
    assert gq.shape == (P, D, M) and gk.shape == (P, D, N) and gv.shape == (P, N, C)
    for name, a, b in (("grad_q", gq, rq), ("grad_k", gk, rk), ("grad_v", gv, rv)):
        assert rel_err(a, b) < TOL, f"{name} rel err {rel_err(a, b)}"


def test_autograd_matches_torch_away_from_ties():
    from weighted_laplace_sum import weighted_laplace_sum
    P, D, N, M, C = 2, 3, 300, 250, 20
    q, k, v = make_inputs(P, D, N, M, C, seed=11, scale=1.5, ties=False)
    g_w, g_u = _grads(P, M, C, seed=12)
    q.requires_grad_(True); k.requires_grad_(True); v.requires_grad_(True)
    out_w, out_u = weighted_laplace_sum(q, k, v)
    ((out_w * g_w).sum() + (out_u * g_u).sum()).backward()
    qd, kd, vd = (t.detach().double().cpu().requires_grad_(True) for t in (q, k, v))
    E = (-(kd[:, :, None, :] - qd[:, :, :, None]).abs()).exp().sum(1)        # (P, M, N)
    ((E @ vd * g_w.double().cpu()).sum() + (E.sum(2) * g_u.double().cpu()).sum()).backward()
    for name, a, b in (("grad_q", q.grad, qd.grad), ("grad_k", k.grad, kd.grad), ("grad_v", v.grad, vd.grad)):
        assert rel_err(a, b) < TOL, f"{name} rel err {rel_err(a, b)}"


def test_autograd_single_output_and_no_grad_route():
    from weighted_laplace_sum import weighted_laplace_sum
    P, D, N, M, C = 1, 2, 200, 220, 8
    q, k, v = make_inputs(P, D, N, M, C, seed=21, ties=False)
    g_w, g_u = _grads(P, M, C, seed=22)
    out = weighted_laplace_sum(q, k, v)
    assert not out[0].requires_grad and not out[1].requires_grad
    q.requires_grad_(True); v.requires_grad_(True)
    # only out_u used: g_w is None in the backward
    _, out_u = weighted_laplace_sum(q, k, v)
    (out_u * g_u).sum().backward()
    rq, _, rv = direct.laplace_sum_backward(q, k, v, torch.zeros_like(g_w), g_u)
    assert rel_err(q.grad, rq) < TOL
    assert v.grad.abs().max().item() == 0.0 and rv.abs().max().item() == 0.0
    # only out_w used
    q.grad = None; v.grad = None
    out_w, _ = weighted_laplace_sum(q, k, v)
    (out_w * g_w).sum().backward()
    rq, _, rv = direct.laplace_sum_backward(q, k, v, g_w)
    assert rel_err(q.grad, rq) < TOL and rel_err(v.grad, rv) < TOL


def test_backward_global_memory_sort():
    """Segments longer than the shared-memory sort holds."""
    from weighted_laplace_sum import weighted_laplace_sum_backward
    P, D, N, M, C = 1, 1, 20000, 17000, 8
    q, k, v = make_inputs(P, D, N, M, C, seed=31, scale=2.0)
    g_w, g_u = _grads(P, M, C, seed=32)
    gq, gk, gv = weighted_laplace_sum_backward(q, k, v, g_w, g_u)
    rq, rk, rv = direct.laplace_sum_backward(q, k, v, g_w, g_u)
    for name, a, b in (("grad_q", gq, rq), ("grad_k", gk, rk), ("grad_v", gv, rv)):
        assert rel_err(a, b) < 1e-3, f"{name} rel err {rel_err(a, b)}"


def test_attention_add_laplace_trains():
    """add_laplace attention with gradients: the sorted-walk backward against float64 autograd of the dense formula."""
    from kernel_attention import attention
    B, H, S, D = 1, 2, 192, 16
    g = torch.Generator().manual_seed(41)
    q, k, v = (torch.randn(B, H, S, D, generator=g).cuda().requires_grad_(True) for _ in range(3))
    up = torch.randn(B, H, S, D, generator=g)
    out = attention(q, k, v, "add_laplace", 0.5)
    (out * up.cuda()).sum().backward()
    qd, kd, vd = (t.detach().double().cpu().requires_grad_(True) for t in (q, k, v))
    A = (-((qd[:, :, :, None, :] - kd[:, :, None, :, :]) / 0.5).abs()).exp().sum(-1)      # (B, H, Sq, Sk)
    ref = A @ vd / A.sum(-1, keepdim=True).clamp_min(1e-6)
    (ref * up.double()).sum().backward()
    assert rel_err(out, ref) < TOL
    for name, a, b in (("q", q.grad, qd.grad), ("k", k.grad, kd.grad), ("v", v.grad, vd.grad)):
        assert rel_err(a, b) < 5e-4, f"grad {name} rel err {rel_err(a, b)}"
