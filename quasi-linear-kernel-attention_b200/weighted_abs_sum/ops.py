"""Public abs-sum operators with the reference's signatures and backend names
(Weighted_Abs_Sum/weighted_abs_sum/ops.py:12-139).

The reference dispatches between a pykeops map-reduce for short sequences and its CUDA
extension (fused or global kernels). Here every backend name runs the same sm_100a
kernels, which cover short sequences as well; "keops" is accepted and means "the library".
`path` (-1 auto / 0 global / 1 fused) is still passed down so that pinning the fused path
beyond 4096 elements fails as it does in the reference.
"""

import torch

import qlka_native as _native

_BACKENDS = ("auto", "keops", "cuda", "cuda-fused", "cuda-global")
_PATH = {"auto": -1, "keops": -1, "cuda": -1, "cuda-fused": 1, "cuda-global": 0}

# kept for API compatibility: the reference switches to pykeops below this max(N, M)
KEOPS_CUTOFF = 512


def set_keops_cutoff(n):
    """Set the max(N,M) below which backend='auto' would use keops in the reference
    (stored and returned; it selects nothing here)."""
    global KEOPS_CUTOFF
    KEOPS_CUTOFF = int(n)
    return KEOPS_CUTOFF


def _resolve(backend):
    if backend not in _BACKENDS:
        raise ValueError(f"backend must be one of {_BACKENDS}, got {backend!r}")
    return _PATH[backend]


class _WeightedAbsSum(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, path):
        ctx.save_for_backward(q, k, v)
        ctx.set_materialize_grads(False)
        return _native.abs_forward(q, k, v, full=False, path=path)[0]

    @staticmethod
    def backward(ctx, g_w):
        q, k, v = ctx.saved_tensors
        if g_w is None:
            return None, None, None, None
        grad_q, grad_k, grad_v = _native.abs_backward(q, k, v, g_w.contiguous())
        return grad_q, grad_k, grad_v, None


class _WeightedAbsSumFull(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, path):
        ctx.save_for_backward(q, k, v)
        ctx.set_materialize_grads(False)
        return _native.abs_forward(q, k, v, full=True, path=path)

    @staticmethod
    def backward(ctx, g_w, g_u):
        q, k, v = ctx.saved_tensors
        if g_w is None and g_u is None:
            return None, None, None, None
        if g_u is None:     # nothing flowed back into the row sums: the native call skips their scalar terms
            grad_q, grad_k, grad_v = _native.abs_backward(q, k, v, g_w.contiguous())
        else:
            if g_w is None:
                g_w = torch.zeros(q.shape[0], q.shape[2], v.shape[2], device=q.device, dtype=q.dtype)
            grad_q, grad_k, grad_v = _native.abs_backward(q, k, v, g_w.contiguous(), g_u.contiguous())
        return grad_q, grad_k, grad_v, None


def weighted_abs_sum(q, k, v, backend="auto"):
    """out[p,m,c] = sum_{n,d} |k[p,d,n] - q[p,d,m]| * v[p,n,c]

    q: (P, D, M), k: (P, D, N), v: (P, N, C) -> (P, M, C). Differentiable.
    """
    return _WeightedAbsSum.apply(q, k, v, _resolve(backend))


def weighted_abs_sum_full(q, k, v, backend="auto"):
    """Returns (out_w, out_u): the weighted abs sum (P, M, C) and the unweighted abs sum
    out_u[p,m] = sum_{n,d} |k[p,d,n] - q[p,d,m]| (P, M). Differentiable in both outputs."""
    return _WeightedAbsSumFull.apply(q, k, v, _resolve(backend))


def weighted_abs_sum_shifted(q, k, v, shifts, weights):
    """(out_w, out_u) of sum_s weights[s] * weighted_abs_sum_full(q + shifts[s], k, v), evaluated with one
    sort of the keys (at most 4 shifts, N <= 16384, len(shifts) * M <= 16384). Not in the reference, whose
    add_bump calls the abs sum three times; forward only (no autograd)."""
    return _native.abs_shifted_forward(q, k, v, shifts, weights, full=True)


def weighted_sgn_sum(q, k, v, g, backend="auto"):
    """out[p,d,m] = sum_n sgn(k[p,d,n] - q[p,d,m]) * dot(v[p,n,:], g[p,m,:])   (P, D, M).

    sgn(0) = +1 (a key equal to the query counts as above it). Not differentiable.
    """
    _resolve(backend)
    if backend == "cuda-fused":
        raise ValueError("weighted_sgn_sum has no fused path; use 'cuda' or 'cuda-global'")
    return _native.sgn_forward(q, k, v, g.contiguous())
