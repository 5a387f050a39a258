"""More than 65535 batch*head problems in one call: every kernel carries the head (or segment) index in the x extent of
its grid, whose limit is 2^31 - 1, never in y or z (limit 65535). Checked on the heads at both ends and around 65536
against the float64 definitions."""

import pytest
import torch

from oracle import direct
from util import rel_err

pytestmark = pytest.mark.gpu
P, D, N, M, C = 66000, 2, 24, 19, 4
HEADS = [0, 1, 65534, 65535, 65536, 65537, P - 1]


def _inputs():
    g = torch.Generator(device="cuda").manual_seed(11)
    q = torch.randn(P, D, M, device="cuda", generator=g)
    k = torch.randn(P, D, N, device="cuda", generator=g)
    v = torch.randn(P, N, C, device="cuda", generator=g)
    return q, k, v


def _pick(*ts):
    idx = torch.tensor(HEADS, device=ts[0].device)
    return tuple(t.index_select(0, idx).contiguous() for t in ts)


def test_laplace_forward_and_backward():
    from weighted_laplace_sum import weighted_laplace_sum, weighted_laplace_sum_backward
    q, k, v = _inputs()
    out_w, out_u = weighted_laplace_sum(q, k, v)
    g = torch.Generator(device="cuda").manual_seed(12)
    g_w = torch.randn(P, M, C, device="cuda", generator=g)
    g_u = torch.randn(P, M, device="cuda", generator=g)
    gq, gk, gv = weighted_laplace_sum_backward(q, k, v, g_w, g_u)
    torch.cuda.synchronize()
    qs, ks, vs, ws, us, gws, gus, gqs, gks, gvs = _pick(q, k, v, out_w, out_u, g_w, g_u, gq, gk, gv)
    ref_w, ref_u = direct.laplace_sum(qs, ks, vs)
    assert rel_err(ws, ref_w) < 1e-4 and rel_err(us, ref_u) < 1e-4
    rq, rk, rv = direct.laplace_sum_backward(qs, ks, vs, gws, gus)
    assert rel_err(gqs, rq) < 1e-4 and rel_err(gks, rk) < 1e-4 and rel_err(gvs, rv) < 1e-4


def test_abs_forward_backward_sgn():
    from weighted_abs_sum import weighted_abs_sum_full, weighted_sgn_sum
    q, k, v = _inputs()
    q.requires_grad_(True); k.requires_grad_(True); v.requires_grad_(True)
    out_w, out_u = weighted_abs_sum_full(q, k, v)
    g = torch.Generator(device="cuda").manual_seed(13)
    g_w = torch.randn(P, M, C, device="cuda", generator=g)
    g_u = torch.randn(P, M, device="cuda", generator=g)
    torch.autograd.backward((out_w, out_u), (g_w, g_u))
    sg = weighted_sgn_sum(q.detach(), k.detach(), v.detach(), g_w)
    torch.cuda.synchronize()
    qs, ks, vs, ws, us, gws, gus, gqs, gks, gvs, sgs = _pick(q.detach(), k.detach(), v.detach(), out_w.detach(), out_u.detach(),
                                                             g_w, g_u, q.grad, k.grad, v.grad, sg)
    ref_w, ref_u = direct.abs_sum(qs, ks, vs)
    assert rel_err(ws, ref_w) < 1e-4 and rel_err(us, ref_u) < 1e-4
    rq, rk, rv = direct.abs_sum_backward(qs, ks, vs, gws, gus)
    assert rel_err(gqs, rq) < 1e-4 and rel_err(gks, rk) < 1e-4 and rel_err(gvs, rv) < 1e-4
    assert rel_err(sgs, direct.sgn_sum(qs, ks, vs, gws)) < 1e-4


@pytest.mark.parametrize("kernel", ["add_laplace", "add_riesz"])
def test_attention_entry(kernel):
    import qlka_native
    B, H, S, Dq, Dv = 1100, 60, 12, 2, 4                       # B * H = 66000
    g = torch.Generator(device="cuda").manual_seed(14)
    q, k = (torch.randn(B, H, S, Dq, device="cuda", generator=g) for _ in range(2))
    v = torch.randn(B, H, S, Dv, device="cuda", generator=g)
    out = qlka_native.fused_attention(kernel, q, k, v, 0.7)
    torch.cuda.synchronize()
    for b in (0, B - 1):
        ref = direct.attention(q[b:b + 1], k[b:b + 1], v[b:b + 1], kernel, 0.7)
        assert rel_err(out[b:b + 1], ref) < 1e-4
