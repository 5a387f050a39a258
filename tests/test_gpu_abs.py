"""weighted_abs_sum (forward, backward, autograd) and weighted_sgn_sum on the GPU, through
the C ABI, against the CPU checkers."""

import os

import numpy as np
import pytest
import torch

from oracle import direct, sorted_scan
from util import make_inputs, rel_err

pytestmark = pytest.mark.gpu
TOL = 1e-4
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

SHAPES = [
    (1, 1, 1, 1, 1), (2, 3, 7, 5, 4), (1, 2, 8, 9, 3), (2, 4, 100, 77, 32), (1, 3, 257, 300, 33),
    (1, 2, 64, 1000, 64), (1, 2, 1000, 3, 65), (4, 2, 600, 600, 64), (1, 2, 1024, 1024, 128),
    (2, 2, 4096, 4096, 64), (1, 2, 5000, 3000, 8), (1, 2, 16384, 16384, 64),
]


@pytest.mark.parametrize("shape", SHAPES)
def test_forward_full(shape):
    from weighted_abs_sum import weighted_abs_sum, weighted_abs_sum_full
    P, D, N, M, C = shape
    q, k, v = make_inputs(P, D, N, M, C, seed=N + 3 * M + C, scale=0.5)
    out_w, out_u = weighted_abs_sum_full(q, k, v)
    only_w = weighted_abs_sum(q, k, v)
    ref_w, ref_u = sorted_scan.abs_sum(q, k, v)
    assert rel_err(out_w, ref_w) < TOL, rel_err(out_w, ref_w)
    assert rel_err(out_u, ref_u) < TOL, rel_err(out_u, ref_u)
    assert rel_err(only_w, ref_w) < TOL


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("full", [False, True])
def test_backward(shape, full):
    import qlka_native
    P, D, N, M, C = shape
    q, k, v = make_inputs(P, D, N, M, C, seed=2 * N + M + C, scale=0.5)
    g = torch.Generator().manual_seed(11)
    g_w = torch.randn(P, M, C, generator=g).cuda()
    g_u = torch.randn(P, M, generator=g).cuda() if full else None
    gq, gk, gv = qlka_native.abs_backward(q, k, v, g_w, g_u)
    rq, rk, rv = sorted_scan.abs_sum_backward(q, k, v, g_w, g_u)
    assert rel_err(gq, rq) < TOL, ("grad_q", rel_err(gq, rq))
    assert rel_err(gk, rk) < TOL, ("grad_k", rel_err(gk, rk))
    assert rel_err(gv, rv) < TOL, ("grad_v", rel_err(gv, rv))


@pytest.mark.parametrize("shape", SHAPES[:9])
def test_sgn(shape):
    from weighted_abs_sum import weighted_sgn_sum
    P, D, N, M, C = shape
    q, k, v = make_inputs(P, D, N, M, C, seed=N + M, scale=0.5)
    g = torch.randn(P, M, C, generator=torch.Generator().manual_seed(3)).cuda()
    out = weighted_sgn_sum(q, k, v, g)
    assert out.shape == (P, D, M)
    assert rel_err(out, sorted_scan.sgn_sum(q, k, v, g)) < TOL


def test_autograd_through_the_ops():
    from weighted_abs_sum import weighted_abs_sum, weighted_abs_sum_full
    P, D, N, M, C = 2, 4, 300, 260, 16
    q, k, v = make_inputs(P, D, N, M, C, seed=21, scale=0.5, ties=False)
    g = torch.Generator().manual_seed(4)
    g_w, g_u = torch.randn(P, M, C, generator=g).cuda(), torch.randn(P, M, generator=g).cuda()
    for t in (q, k, v):
        t.requires_grad_(True)
    ow, ou = weighted_abs_sum_full(q, k, v)
    ((ow * g_w).sum() + (ou * g_u).sum()).backward()
    rq, rk, rv = direct.abs_sum_backward(q, k, v, g_w, g_u)
    assert rel_err(q.grad, rq) < TOL and rel_err(k.grad, rk) < TOL and rel_err(v.grad, rv) < TOL
    # only out_w used -> plain backward; only out_u used -> zero g_w
    for t in (q, k, v):
        t.grad = None
    ow, ou = weighted_abs_sum_full(q, k, v)
    (ow * g_w).sum().backward()
    rq, rk, rv = direct.abs_sum_backward(q, k, v, g_w)
    assert rel_err(q.grad, rq) < TOL and rel_err(k.grad, rk) < TOL and rel_err(v.grad, rv) < TOL
    for t in (q, k, v):
        t.grad = None
    ow, ou = weighted_abs_sum_full(q, k, v)
    (ou * g_u).sum().backward()
    rq, rk, rv = direct.abs_sum_backward(q, k, v, torch.zeros_like(g_w), g_u)
    assert rel_err(q.grad, rq) < TOL and rel_err(k.grad, rk) < TOL
    assert v.grad.abs().max().item() < 1e-3
    for t in (q, k, v):
        t.grad = None
    (weighted_abs_sum(q, k, v, backend="cuda-global") * g_w).sum().backward()
    rq, rk, rv = direct.abs_sum_backward(q, k, v, g_w)
    assert rel_err(q.grad, rq) < TOL and rel_err(k.grad, rk) < TOL and rel_err(v.grad, rv) < TOL


def test_training_step_config():
    """B=8,H=12,N=4096,D=Dv=64 forward + backward: a sampled head against the C restatement."""
    import qlka_native
    P, D, N, C = 96, 64, 4096, 64
    g = torch.Generator().manual_seed(0)
    q = (torch.randn(P, D, N, generator=g) * 0.5).cuda()
    k = (torch.randn(P, D, N, generator=g) * 0.5).cuda()
    v = torch.randn(P, N, C, generator=g).cuda()
    g_w = torch.randn(P, N, C, generator=g).cuda()
    ow, _ = qlka_native.abs_forward(q, k, v, full=False)
    gq, gk, gv = qlka_native.abs_backward(q, k, v, g_w)
    for p in (0, 95):
        s = slice(p, p + 1)
        rw, _ = sorted_scan.abs_sum(q[s], k[s], v[s])
        rq, rk, rv = sorted_scan.abs_sum_backward(q[s], k[s], v[s], g_w[s])
        assert rel_err(ow[s], rw) < TOL
        assert rel_err(gq[s], rq) < TOL and rel_err(gk[s], rk) < TOL and rel_err(gv[s], rv) < TOL


@pytest.mark.parametrize("kernel", ["add_laplace", "add_riesz", "add_bump"])
@pytest.mark.parametrize("masked", [False, True])
def test_attention_against_reference_golden(kernel, masked):
    from kernel_attention import attention
    z = np.load(os.path.join(GOLD, "small_kernels.npz"))
    q, k, v = (torch.from_numpy(z[n]).cuda() for n in ("q", "k", "v"))
    keep = torch.from_numpy(z["keep"]).cuda() if masked else None
    out = attention(q, k, v, kernel, float(z["tau"]), keep)
    want = torch.from_numpy(z[f"att_{kernel}{'_masked' if masked else ''}"])
    assert rel_err(out, want) < 2e-4, rel_err(out, want)


def test_latency_bound_bump_shape():
    """B=256,H=1,N=600,D=Dv=64, q,k ~ U(-3,3): add_bump attention on a slice against fp64."""
    from kernel_attention import attention
    g = torch.Generator().manual_seed(0)
    B, S, D = 256, 600, 64
    q = (torch.rand(B, 1, S, D, generator=g) * 6 - 3).cuda()
    k = (torch.rand(B, 1, S, D, generator=g) * 6 - 3).cuda()
    v = torch.randn(B, 1, S, D, generator=g).cuda()
    out = attention(q, k, v, "add_bump", 1.5)
    want = direct.attention(q[:3].cpu(), k[:3].cpu(), v[:3].cpu(), "add_bump", 1.5)
    assert rel_err(out[:3], want) < 1e-3, rel_err(out[:3], want)


def test_argument_errors():
    from weighted_abs_sum import weighted_abs_sum, weighted_sgn_sum
    q, k, v = make_inputs(1, 2, 5000, 5000, 4, seed=1)
    with pytest.raises(ValueError, match="backend must be one of"):
        weighted_abs_sum(q, k, v, backend="triton")
    with pytest.raises(RuntimeError, match="fused path pinned but unavailable"):
        weighted_abs_sum(q, k, v, backend="cuda-fused")
    with pytest.raises(ValueError, match="no fused path"):
        weighted_sgn_sum(q, k, v, torch.zeros(1, 5000, 4, device="cuda"), backend="cuda-fused")
    with pytest.raises(RuntimeError, match="CUDA tensors"):
        weighted_abs_sum(q.cpu(), k.cpu(), v.cpu())


@pytest.mark.parametrize("shape", [(2, 3, 50, 40, 4), (3, 4, 600, 600, 64), (1, 2, 3000, 5000, 33)])
def test_shifted_sum_equals_separate_sums(shape):
    """The folded entry point against three separate abs sums, and the fused add_bump against float64."""
    from weighted_abs_sum import weighted_abs_sum_full, weighted_abs_sum_shifted
    P, D, N, M, C = shape
    q, k, v = make_inputs(P, D, N, M, C, seed=N + M, scale=1.0)
    shifts, weights = (0.0, 1.0, -1.0), (-1.0, 0.5, 0.5)
    w, u = weighted_abs_sum_shifted(q, k, v, shifts, weights)
    rw = sum(wt * sorted_scan.abs_sum(q + sh, k, v)[0] for sh, wt in zip(shifts, weights))
    ru = sum(wt * sorted_scan.abs_sum(q + sh, k, v)[1] for sh, wt in zip(shifts, weights))
    assert rel_err(w, rw) < TOL, rel_err(w, rw)
    assert rel_err(u, ru) < TOL, rel_err(u, ru)
    w2, u2 = weighted_abs_sum_shifted(q, k, v, (0.25,), (2.0,))
    a, b = sorted_scan.abs_sum(q + 0.25, k, v)
    assert rel_err(w2, 2 * a) < TOL and rel_err(u2, 2 * b) < TOL


@pytest.mark.parametrize("masked", [False, True])
@pytest.mark.parametrize("kernel", ["add_riesz", "add_bump"])
@pytest.mark.parametrize("shape", [(1, 2, 50, 8, 8), (2, 3, 333, 16, 20), (1, 4, 1024, 32, 32), (2, 2, 700, 64, 33)])
def test_fused_attention_entry(shape, kernel, masked):
    """add_riesz / add_bump attention in one native call on (B, H, S, D) against the float64 dense formula and the op-by-op route."""
    import qlka_native
    from kernel_attention import TAU, attention
    from oracle import direct
    B, H, S, D, Dv = shape
    g = torch.Generator().manual_seed(S + D)
    q, k = (torch.randn(B, H, S, D, generator=g).cuda() for _ in range(2))
    v = torch.randn(B, H, S, Dv, generator=g).cuda()
    keep = None
    if masked:
        keep = (torch.rand(B, S, generator=g) > 0.3)
        keep[:, 0] = True
        keep = keep.cuda()
    tau = TAU[kernel]
    out = qlka_native.fused_attention(kernel, q, k, v, tau, keep)
    ref = direct.attention(q, k, v, kernel, tau, keep)
    assert out.shape == (B, H, S, Dv)
    assert rel_err(out, ref) < 2e-4, f"rel err {rel_err(out, ref)}"
    with torch.enable_grad():
        qg = q.clone().requires_grad_(True)
        slow = attention(qg, k, v, kernel, tau, keep)                      # op-by-op route
    assert rel_err(out, slow.double()) < 2e-4


def test_fused_bump_refuses_long_sequences():
    import qlka_native
    q = torch.zeros(1, 1, 6000, 4, device="cuda")
    with pytest.raises(RuntimeError):
        qlka_native.fused_attention("add_bump", q, q, q, 1.5)
