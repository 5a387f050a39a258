"""Normalised additive-kernel attention on (B, H, S, D) fp32 CUDA tensors for the three kernels whose
efficient evaluation goes through the sorted-walk operators: add_laplace, add_riesz, add_bump.

`attention(q, k, v, kernel, tau, keep=None)` answers the same call as the reference's
`attention(..., impl="efficient")` (Experiments/kernel_attention/attention.py:95-126) for those kernels;
the reference's own file also runs unchanged on top of the two operator packages of this library.

Two routes:
* no gradient needed - one native call per attention (`qlka_native.fused_attention`): layout change, tau,
  masking, the sums and the normalisation all happen inside the library;
* gradients needed - the sums are assembled here from the differentiable operators. Every kernel is described
  by two small functions: `sums` returns the unnormalised numerator sum_j A_ij v_j and row sum sum_j A_ij over
  ALL S keys, and `at_origin` returns A(q_i, 0), the weight a key placed at the origin has. Masked keys are moved
  to the origin with a zero value row, so they add nothing to the numerator and exactly `at_origin` each to the
  row sum, which is subtracted again.
"""

import torch

import qlka_native as _native
from weighted_abs_sum import weighted_abs_sum_full
from weighted_laplace_sum import weighted_laplace_sum

EPS = 1e-3        # offset of the Riesz kernel (Experiments/kernel_attention/kernels.py:9)
CLAMP = 1e-6      # floor of the row sum (Experiments/kernel_attention/attention.py:21)
TAU = {"add_laplace": 0.5, "add_riesz": 1.0, "add_bump": 1.5}   # default temperatures, kernels.py:13-25


# ---- add_laplace: A_ij = sum_d exp(-|q_id - k_jd|)
def _laplace_sums(q, k, v):
    return weighted_laplace_sum(q, k, v)


def _laplace_at_origin(q):
    return torch.exp(-q.abs()).sum(dim=1)


# ---- add_riesz: A_ij = |q_i|_1 + |k_j|_1 - |q_i - k_j|_1 + EPS; the two norms are rank-1 terms around the abs sum
def _riesz_sums(q, k, v):
    dist_v, dist_1 = weighted_abs_sum_full(q, k, v)
    q_norm = q.abs().sum(dim=1) + EPS                     # (P, S)   the offset rides with the query norm
    k_norm = k.abs().sum(dim=1)                           # (P, S)
    v_total = v.sum(dim=1)                                # (P, C)
    kv_total = torch.einsum("ps,psc->pc", k_norm, v)      # (P, C)
    num = q_norm.unsqueeze(2) * v_total.unsqueeze(1) + kv_total.unsqueeze(1) - dist_v
    row = q_norm * k.shape[2] + k_norm.sum(dim=1, keepdim=True) - dist_1
    return num, row


def _riesz_at_origin(q):
    return torch.full_like(q[:, 0, :], EPS)               # the norms cancel against |q - 0|_1


# ---- add_bump: A_ij = sum_d max(0, 1 - |x|), x = q_id - k_jd, and max(0, 1 - |x|) = (|x + 1| + |x - 1|) / 2 - |x|
_BUMP_TERMS = ((0.0, -1.0), (1.0, 0.5), (-1.0, 0.5))      # (query shift, weight) of the three abs sums


def _bump_sums(q, k, v):
    num = row = None
    for shift, weight in _BUMP_TERMS:
        dist_v, dist_1 = weighted_abs_sum_full(q + shift if shift else q, k, v)
        num = weight * dist_v if num is None else num + weight * dist_v
        row = weight * dist_1 if row is None else row + weight * dist_1
    return num, row


def _bump_at_origin(q):
    return (1.0 - q.abs()).clamp_min(0.0).sum(dim=1)


_ROUTES = {"add_laplace": (_laplace_sums, _laplace_at_origin),
           "add_riesz": (_riesz_sums, _riesz_at_origin),
           "add_bump": (_bump_sums, _bump_at_origin)}


def attention(q, k, v, kernel, tau, keep=None):
    """q, k (B, H, S, D), v (B, H, S, Dv) fp32 CUDA; keep (B, S) bool/float key-keep mask or None -> (B, H, S, Dv)."""
    assert q.dtype == k.dtype == v.dtype == torch.float32, "kernel attention runs in fp32 only"
    if kernel not in _ROUTES:
        raise ValueError(f"kernel must be one of {tuple(_ROUTES)}, got {kernel!r}")
    B, H, S, D = q.shape
    wants_grad = torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad)
    fused_fits = kernel != "add_bump" or 3 * S <= 16384      # the fused add_bump shares one shared-memory sort between its three shifts
    if not wants_grad and fused_fits:
        return _native.fused_attention(kernel, q, k, v, tau, keep)

    sums, at_origin = _ROUTES[kernel]
    heads = B * H
    qs = (q / tau).permute(0, 1, 3, 2).reshape(heads, D, S).contiguous()          # (P, D, S): one sorted axis per feature
    ks = (k / tau).permute(0, 1, 3, 2).reshape(heads, D, S)
    vs = v.reshape(heads, S, v.shape[3])
    if keep is not None:
        kept = keep.to(q.dtype).repeat_interleave(H, dim=0)                       # (P, S)
        ks, vs = ks * kept.unsqueeze(1), vs * kept.unsqueeze(2)
    num, row = sums(qs, ks.contiguous(), vs.contiguous())
    if keep is not None:
        row = row - (S - kept.sum(dim=1, keepdim=True)) * at_origin(qs)
    return (num / row.clamp_min(CLAMP).unsqueeze(2)).view(B, H, S, -1)
