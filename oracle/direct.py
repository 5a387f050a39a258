"""TEST INFRASTRUCTURE ONLY - fp64 direct O(N^2) evaluation of the additive-kernel sums.

This module is the checker for the CUDA path: only tests, the smoke test and the
CPU-baseline leg of the benchmark may import it. Nothing in the product package does.

Every function restates a definition of the reference in float64, with the full
(D, m-chunk, N) difference tensor materialised chunk by chunk:

* Laplace sum     out_w[p,m,c] = sum_{d,n} exp(-|k[p,d,n]-q[p,d,m]|) v[p,n,c]
                  (Weighted_Laplace_Sum/weighted_laplace_sum/__init__.py:4-13,
                   Experiments/kernel_attention/kernels.py:80-84)
* abs sum         out_w[p,m,c] = sum_{d,n} |k[p,d,n]-q[p,d,m]| v[p,n,c]
                  (Weighted_Abs_Sum/weighted_abs_sum/ops.py:107-126)
* sgn sum         out[p,d,m] = sum_n sgn(k-q) <v[p,n,:], g[p,m,:]>, sgn(0) = +1
                  (Weighted_Abs_Sum/weighted_abs_sum/ops.py:129-139 and the tie rule
                   of Weighted_Abs_Sum/csrc/sgn_kernels.cu:157: a key equal to the
                   query is not yet in the prefix when the query is emitted)
* abs backward    the gradients of the abs sum with the same tie rule
                  (Weighted_Abs_Sum/csrc/binding.cpp:242-245)
* attention       add_laplace / add_riesz / add_bump normalised attention
                  (Experiments/kernel_attention/kernels.py:68-89,
                   Experiments/kernel_attention/attention.py:32-35)

Parity pin: tests/golden/ holds outputs of the reference's own Python code
(kernels.py + attention.py imported unchanged) and tests/test_oracle.py checks this
module against them.
"""

import torch

_BUDGET = 1 << 25   # elements of one (D, mc, N) float64 chunk


def _f64(*xs):
    return [x.detach().to(torch.float64).cpu() for x in xs]


def _chunks(D, N, M):
    mc = max(1, min(M, _BUDGET // max(1, D * N)))
    return range(0, M, mc), mc


def laplace_sum(q, k, v):
    """(out_w (P,M,C), out_u (P,M)) in float64."""
    q, k, v = _f64(q, k, v)
    P, D, M = q.shape
    N, C = k.shape[2], v.shape[2]
    out_w = torch.empty(P, M, C, dtype=torch.float64)
    out_u = torch.empty(P, M, dtype=torch.float64)
    starts, mc = _chunks(D, N, M)
    for p in range(P):
        for m0 in starts:
            qq = q[p, :, m0:m0 + mc]                                        # (D, mc)
            A = (-(k[p][:, None, :] - qq[:, :, None]).abs()).exp().sum(0)   # (mc, N)
            out_w[p, m0:m0 + mc] = A @ v[p]
            out_u[p, m0:m0 + mc] = A.sum(1)
    return out_w, out_u


def abs_sum(q, k, v):
    """(out_w (P,M,C), out_u (P,M)) in float64."""
    q, k, v = _f64(q, k, v)
    P, D, M = q.shape
    N, C = k.shape[2], v.shape[2]
    out_w = torch.empty(P, M, C, dtype=torch.float64)
    out_u = torch.empty(P, M, dtype=torch.float64)
    starts, mc = _chunks(D, N, M)
    for p in range(P):
        for m0 in starts:
            qq = q[p, :, m0:m0 + mc]
            A = (k[p][:, None, :] - qq[:, :, None]).abs().sum(0)           # (mc, N)
            out_w[p, m0:m0 + mc] = A @ v[p]
            out_u[p, m0:m0 + mc] = A.sum(1)
    return out_w, out_u


def _sign_ge(x):
    """+1 where x >= 0, -1 where x < 0 (the walk's tie rule)."""
    return torch.where(x >= 0, torch.ones_like(x), -torch.ones_like(x))


def sgn_sum(q, k, v, g):
    """out[p,d,m] = sum_n s(k-q) <v_n, g_m>, s(0) = +1; float64 (P,D,M)."""
    q, k, v, g = _f64(q, k, v, g)
    P, D, M = q.shape
    N = k.shape[2]
    out = torch.empty(P, D, M, dtype=torch.float64)
    starts, mc = _chunks(D, N, M)
    for p in range(P):
        for m0 in starts:
            qq = q[p, :, m0:m0 + mc]
            S = _sign_ge(k[p][:, None, :] - qq[:, :, None])                 # (D, mc, N)
            B = g[p, m0:m0 + mc] @ v[p].T                                   # (mc, N)
            out[p, :, m0:m0 + mc] = (S * B[None]).sum(2)
    return out


def abs_sum_backward(q, k, v, g_w, g_u=None):
    """Gradients (grad_q (P,D,M), grad_k (P,D,N), grad_v (P,N,C)) of
    sum(out_w * g_w) + sum(out_u * g_u), sub-gradient -1 at ties for q and k."""
    q, k, v, g_w = _f64(q, k, v, g_w)
    P, D, M = q.shape
    N, C = k.shape[2], v.shape[2]
    gu = None if g_u is None else _f64(g_u)[0]
    grad_q = torch.empty(P, D, M, dtype=torch.float64)
    grad_k = torch.zeros(P, D, N, dtype=torch.float64)
    grad_v = torch.zeros(P, N, C, dtype=torch.float64)
    starts, mc = _chunks(D, N, M)
    for p in range(P):
        for m0 in starts:
            qq = q[p, :, m0:m0 + mc]
            diff = k[p][:, None, :] - qq[:, :, None]                        # (D, mc, N) = k - q
            B = g_w[p, m0:m0 + mc] @ v[p].T                                 # (mc, N) <g_m, v_n>
            if gu is not None:
                B = B + gu[p, m0:m0 + mc, None]
            # d|k-q|/dq = +1 if k < q else -1 (tie -> -1); d|k-q|/dk = +1 if q < k else -1 (tie -> -1)
            sq = torch.where(diff < 0, torch.ones_like(diff), -torch.ones_like(diff))
            sk = torch.where(diff > 0, torch.ones_like(diff), -torch.ones_like(diff))
            grad_q[p, :, m0:m0 + mc] = (sq * B[None]).sum(2)
            grad_k[p] += (sk * B[None]).sum(1)
            grad_v[p] += diff.abs().sum(0).T @ g_w[p, m0:m0 + mc]
    return grad_q, grad_k, grad_v


def laplace_sum_backward(q, k, v, g_w, g_u=None):
    """Gradients (grad_q (P,D,M), grad_k (P,D,N), grad_v (P,N,C)) of sum(out_w * g_w) + sum(out_u * g_u)
    for the Laplace sum, float64. Where k == q the kernel exp(-|k - q|) has no derivative; the sorted walk
    counts a tied key on the upper side of the query, E = exp(-(k - q)), in both of its runs, so
    dE/dq = +1 and (roles swapped) dE/dk = +1 there. The reference has no Laplace backward; away from
    ties this is the autograd gradient of its chunked PyTorch route
    (Experiments/kernel_attention/attention.py:110-115)."""
    q, k, v, g_w = _f64(q, k, v, g_w)
    P, D, M = q.shape
    N, C = k.shape[2], v.shape[2]
    gu = None if g_u is None else _f64(g_u)[0]
    grad_q = torch.empty(P, D, M, dtype=torch.float64)
    grad_k = torch.zeros(P, D, N, dtype=torch.float64)
    grad_v = torch.zeros(P, N, C, dtype=torch.float64)
    starts, mc = _chunks(D, N, M)
    for p in range(P):
        for m0 in starts:
            qq = q[p, :, m0:m0 + mc]
            diff = k[p][:, None, :] - qq[:, :, None]                        # (D, mc, N) = k - q
            E = (-diff.abs()).exp()
            B = g_w[p, m0:m0 + mc] @ v[p].T                                 # (mc, N) <g_m, v_n>
            if gu is not None:
                B = B + gu[p, m0:m0 + mc, None]
            # dE/dq = +E if k >= q else -E;  dE/dk = +E if q >= k else -E
            sq = torch.where(diff >= 0, E, -E)
            sk = torch.where(diff <= 0, E, -E)
            grad_q[p, :, m0:m0 + mc] = (sq * B[None]).sum(2)
            grad_k[p] += (sk * B[None]).sum(1)
            grad_v[p] += E.sum(0).T @ g_w[p, m0:m0 + mc]
    return grad_q, grad_k, grad_v


# ---------------------------------------------------------------- attention algebra

EPS = 1e-3      # Riesz offset (Experiments/kernel_attention/kernels.py:9)
CLAMP = 1e-6    # denominator clamp (Experiments/kernel_attention/attention.py:21)


def kernel_matrix(kernel, q, k, tau=1.0, keep=None):
    """A (P, Sq, Sk) float64 for the three additive kernels; q, k (P, D, S)."""
    q, k = _f64(q, k)
    q, k = q / tau, k / tau
    x = q.unsqueeze(3) - k.unsqueeze(2)                                     # (P, D, Sq, Sk)
    if kernel == "add_laplace":
        A = (-x.abs()).exp().sum(1)
    elif kernel == "add_riesz":
        A = q.abs().sum(1)[:, :, None] + k.abs().sum(1)[:, None, :] - x.abs().sum(1) + EPS
    elif kernel == "add_bump":
        A = (1.0 - x.abs()).clamp(min=0.0).sum(1)
    else:
        raise ValueError(kernel)
    if keep is not None:
        A = A * keep.to(torch.float64).cpu()[:, None, :]
    return A


def attention(q, k, v, kernel, tau=1.0, keep=None):
    """Normalised attention on (B,H,S,D) inputs, float64 (B,H,S,Dv)."""
    B, H, S, D = q.shape
    P = B * H
    qq = q.transpose(2, 3).reshape(P, D, S)
    kk = k.transpose(2, 3).reshape(P, D, S)
    vv = _f64(v.reshape(P, S, v.shape[3]))[0]
    kp = None if keep is None else keep.repeat_interleave(H, dim=0)
    A = kernel_matrix(kernel, qq, kk, tau, kp)
    out = A @ vv / A.sum(2, keepdim=True).clamp_min(CLAMP)
    return out.view(B, H, S, -1)
