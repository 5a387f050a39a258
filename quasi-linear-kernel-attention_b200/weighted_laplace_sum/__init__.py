"""Drop-in for the reference package `weighted_laplace_sum`
(Weighted_Laplace_Sum/weighted_laplace_sum/__init__.py:1-16): same name, same call."""

import qlka_native as _native


def weighted_laplace_sum(q, k, v):
    """Exact O(N log N) weighted Laplace sum (forward only, fp32, CUDA).

    q: (P, D, M), k: (P, D, N), v: (P, N, C), float32 contiguous CUDA, C <= 128.
    Returns (out_w, out_u):
        out_w[p, m, c] = sum_{d, n} exp(-|k[p, d, n] - q[p, d, m]|) * v[p, n, c]    (P, M, C)
        out_u[p, m]    = sum_{d, n} exp(-|k[p, d, n] - q[p, d, m]|)                 (P, M)
    No autograd. Padded keys: zero k and v there and subtract n_pad * sum_d exp(-|q_d|) from out_u.
    """
    return _native.laplace_forward(q, k, v)


__all__ = ["weighted_laplace_sum"]
