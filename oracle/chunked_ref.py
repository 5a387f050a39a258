"""TEST INFRASTRUCTURE ONLY - CPU restatement of the reference's chunked PyTorch path.

The reference evaluates add_laplace attention on a CPU (and on a GPU when gradients
are needed) by cutting the queries into chunks, building each chunk's full kernel
matrix A = sum_d exp(-|q_d - k_d|) and returning A @ v / A.sum
(Experiments/kernel_attention/attention.py:32-35 `_normalized`, :41-50 `_chunked`,
kernel matrix Experiments/kernel_attention/kernels.py:80-84). The chunk length there
is CHUNK // (P * S) query rows with CHUNK = 2**28 (attention.py:22,45).

This file restates that path in fp32 torch for the host cores: same chunk rule, same
arithmetic, but the D-sum is accumulated one feature dimension at a time instead of
through a (P, D, chunk, S) intermediate (the reference leaves that fusion to
torch.compile, which cannot be relied on here). It is used as the timed CPU baseline
and as a parity cross-check; the product never imports it.
"""

import torch

CHUNK = 2 ** 28
CLAMP = 1e-6


def laplace_kernel_rows(q, k):
    """A[p,i,j] = sum_d exp(-|q[p,d,i] - k[p,d,j]|); q (P,D,c), k (P,D,S) -> (P,c,S)."""
    P, D, c = q.shape
    A = torch.zeros(P, c, k.shape[2], dtype=q.dtype)
    for d in range(D):
        A += (-(q[:, d, :, None] - k[:, d, None, :]).abs()).exp()
    return A


def laplace_sum_chunked(q, k, v, chunk=CHUNK):
    """(out_w, out_u) of the weighted Laplace sum, fp32, query-chunked."""
    P, D, M = q.shape
    N = k.shape[2]
    c = max(1, chunk // (P * N))
    ws, us = [], []
    for i in range(0, M, c):
        A = laplace_kernel_rows(q[:, :, i:i + c], k)
        ws.append(A @ v)
        us.append(A.sum(2))
    return torch.cat(ws, 1), torch.cat(us, 1)


def add_laplace_attention_chunked(q, k, v, tau=1.0, keep=None, chunk=CHUNK):
    """Normalised add_laplace attention; q, k (P,D,S), v (P,S,Dv) -> (P,S,Dv)."""
    q, k = q / tau, k / tau
    P, D, S = q.shape
    c = max(1, chunk // (P * k.shape[2]))
    outs = []
    for i in range(0, S, c):
        A = laplace_kernel_rows(q[:, :, i:i + c], k)
        if keep is not None:
            A = A * keep[:, None, :]
        outs.append(A @ v / A.sum(2, keepdim=True).clamp_min(CLAMP))
    return torch.cat(outs, 1)
