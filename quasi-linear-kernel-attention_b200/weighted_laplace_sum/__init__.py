"""Drop-in for the reference package `weighted_laplace_sum`
(Weighted_Laplace_Sum/weighted_laplace_sum/__init__.py:1-16): same name, same call.

The reference's operator is forward only. Here the same call is also differentiable (the
backward runs the same sort and walk kernels with the roles of queries and keys swapped);
under `torch.no_grad()` or with inputs that need no gradient it is exactly the reference's call.
"""

import torch

import qlka_native as _native


class _WeightedLaplaceSum(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v):
        ctx.set_materialize_grads(False)
        ctx.save_for_backward(q, k, v)
        return _native.laplace_forward(q, k, v)

    @staticmethod
    def backward(ctx, g_w, g_u):
        q, k, v = ctx.saved_tensors
        if g_w is None and g_u is None:
            return None, None, None
        if g_w is None:
            g_w = torch.zeros(q.shape[0], q.shape[2], v.shape[2], device=q.device, dtype=q.dtype)
        return _native.laplace_backward(q, k, v, g_w.contiguous(), None if g_u is None else g_u.contiguous())


def weighted_laplace_sum(q, k, v):
    """Exact O(N log N) weighted Laplace sum (fp32, CUDA).

    q: (P, D, M), k: (P, D, N), v: (P, N, C), float32 contiguous CUDA, C <= 128.
    Returns (out_w, out_u):
        out_w[p, m, c] = sum_{d, n} exp(-|k[p, d, n] - q[p, d, m]|) * v[p, n, c]    (P, M, C)
        out_u[p, m]    = sum_{d, n} exp(-|k[p, d, n] - q[p, d, m]|)                 (P, M)
    Differentiable in both outputs (where a key equals a query the one-sided derivative of the walk's
    tie side is taken). Padded keys: zero k and v there and subtract n_pad * sum_d exp(-|q_d|) from out_u.
    """
    if torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad):
        return _WeightedLaplaceSum.apply(q, k, v)
    return _native.laplace_forward(q, k, v)


def weighted_laplace_sum_backward(q, k, v, g_w, g_u=None):
    """(grad_q, grad_k, grad_v) of sum(out_w * g_w) + sum(out_u * g_u); not in the reference."""
    return _native.laplace_backward(q, k, v, g_w, g_u)


__all__ = ["weighted_laplace_sum", "weighted_laplace_sum_backward"]
