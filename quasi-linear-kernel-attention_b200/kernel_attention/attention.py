"""The caller of the two operators: normalised additive-kernel attention on (B, H, S, D)
fp32 CUDA tensors, for the kernels whose efficient path goes through the sorted-scan
operators - add_laplace, add_riesz, add_bump.

Same call as the reference's `attention(q, k, v, kernel, tau, keep=None)`
(Experiments/kernel_attention/attention.py:95-126) restricted to those three kernels and
to its `impl="efficient"` route: layout change to (P, D, S), tau scaling, key-keep masking
by zeroing k and v with the n_pad correction, and the numerator / denominator algebra of
_add_laplace (:67-72), _add_riesz (:75-81) and _add_bump (:84-92). The other kernels of the
reference (dense matrix kernels) are not part of this library.
"""

import torch

import qlka_native as _native
from weighted_abs_sum import weighted_abs_sum_full, weighted_abs_sum_shifted
from weighted_laplace_sum import weighted_laplace_sum

EPS = 1e-3        # Riesz offset (Experiments/kernel_attention/kernels.py:9)
CLAMP = 1e-6      # denominator clamp (Experiments/kernel_attention/attention.py:21)
TAU = {"add_laplace": 0.5, "add_riesz": 1.0, "add_bump": 1.5}   # kernels.py:13-25


def _abs_sum(q, k, v):
    return weighted_abs_sum_full(q.contiguous(), k.contiguous(), v.contiguous())


def _add_laplace(q, k, v, n_pad):
    # a padded key (k=0, v=0) adds sum_d exp(-|q_d|) to the row sum
    out_w, out_u = weighted_laplace_sum(q.contiguous(), k.contiguous(), v.contiguous())
    den = out_u - n_pad * (-q.abs()).exp().sum(dim=1)
    return out_w / den.clamp_min(CLAMP)[:, :, None]


def _add_riesz(q, k, v, n_pad):
    # A[i,j] = |q_i|_1 + |k_j|_1 - |q_i - k_j|_1 + eps; a padded key adds only eps to the row sum
    out_w, out_u = _abs_sum(q, k, v)
    aq, ak, S = q.abs().sum(dim=1), k.abs().sum(dim=1), q.shape[2]
    num = (aq + EPS)[:, :, None] * v.sum(dim=1)[:, None, :] + (ak[:, :, None] * v).sum(dim=1)[:, None, :] - out_w
    den = (aq + EPS) * S + ak.sum(dim=1, keepdim=True) - out_u - EPS * n_pad
    return num / den.clamp_min(CLAMP)[:, :, None]


def _add_bump(q, k, v, n_pad):
    # max(0, 1 - |x|) = |x + 1| / 2 + |x - 1| / 2 - |x| with x = q_d - k_d
    grad = torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad)
    if not grad and k.shape[2] <= 16384 and 3 * q.shape[2] <= 16384:
        # inference: the three shifted abs sums share one sort of the keys and one walk
        num, den = weighted_abs_sum_shifted(q.contiguous(), k.contiguous(), v.contiguous(), (0.0, 1.0, -1.0), (-1.0, 0.5, 0.5))
        den = den - n_pad * (1 - q.abs()).clamp_min(0).sum(dim=1)
        return num / den.clamp_min(CLAMP)[:, :, None]
    w0, u0 = _abs_sum(q, k, v)
    wp, up = _abs_sum(q + 1, k, v)
    wm, um = _abs_sum(q - 1, k, v)
    num = (wp + wm) / 2 - w0
    den = (up + um) / 2 - u0 - n_pad * (1 - q.abs()).clamp_min(0).sum(dim=1)
    return num / den.clamp_min(CLAMP)[:, :, None]


_KERNELS = {"add_laplace": _add_laplace, "add_riesz": _add_riesz, "add_bump": _add_bump}


def attention(q, k, v, kernel, tau, keep=None):
    """q, k, v (B, H, S, D) fp32 CUDA; keep (B, S) bool/float key-keep mask or None."""
    assert q.dtype == k.dtype == v.dtype == torch.float32, "kernel attention runs in fp32 only"
    if kernel not in _KERNELS:
        raise ValueError(f"kernel must be one of {tuple(_KERNELS)}, got {kernel!r}")
    B, H, S, D = q.shape
    P = B * H
    needs_grad = torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad)
    if not needs_grad and (kernel != "add_bump" or 3 * S <= 16384):
        # inference: layout change, tau, masking, the sums and the normalisation in one native call
        return _native.fused_attention(kernel, q, k, v, tau, keep)
    q = q.transpose(2, 3).reshape(P, D, S)
    k = k.transpose(2, 3).reshape(P, D, S)
    v = v.reshape(P, S, v.shape[3])
    q, k, n_pad = q / tau, k / tau, 0
    if keep is not None:
        keep = keep.repeat_interleave(H, dim=0)
        k, v = k * keep[:, None, :], v * keep[:, :, None]
        n_pad = S - keep.sum(dim=1, keepdim=True)
    out = _KERNELS[kernel](q, k, v, n_pad)
    return out.view(B, H, S, -1)
