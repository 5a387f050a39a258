"""Helpers shared by the GPU parity tests."""

import torch


def rel_err(a, b):
    """max|a - b| / max|b| with b the checker's float64 result."""
    a = a.detach().to(torch.float64).cpu()
    b = b.detach().to(torch.float64).cpu()
    return ((a - b).abs().max() / b.abs().max().clamp_min(1e-6)).item()


def err_stats(a, b, floor=1e-3):
    """(max|a - b| / max|b|, 99.9th percentile of the element-wise relative error), b the checker's result.

    The max-norm figure hides rows of small magnitude; the percentile figure looks at every element on its own,
    |a - b| / max(|b|, floor * max|b|) - the floor keeps elements where the sum cancels to nearly zero from
    dominating (their absolute error is what the max-norm already bounds)."""
    a = a.detach().to(torch.float64).cpu().reshape(-1)
    b = b.detach().to(torch.float64).cpu().reshape(-1)
    diff = (a - b).abs()
    top = b.abs().max().clamp_min(1e-6)
    elem = (diff / b.abs().clamp_min(floor * top)).numpy()
    kth = min(elem.size - 1, int(0.999 * elem.size))
    import numpy as np
    return (diff.max() / top).item(), float(np.partition(elem, kth)[kth])


def make_inputs_cuda(P, D, N, M, C, seed, scale=1.0):
    """Large cases: inputs drawn on the device (seeded CUDA generator), a few exact ties planted."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = torch.randn(P, D, M, generator=g, device="cuda") * scale
    k = torch.randn(P, D, N, generator=g, device="cuda") * scale
    v = torch.randn(P, N, C, generator=g, device="cuda")
    n = min(N, M, 5)
    k[0, 0, :n] = q[0, 0, :n]
    k[P - 1, D - 1, 1:3] = k[P - 1, D - 1, 0]
    return q, k, v


def make_inputs(P, D, N, M, C, seed, scale=1.0, ties=True, device="cuda"):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(P, D, M, generator=g) * scale
    k = torch.randn(P, D, N, generator=g) * scale
    v = torch.randn(P, N, C, generator=g)
    if ties and N * M > 1:            # (a lone key equal to the lone query makes the abs sum exactly 0)
        n = min(N, M, 5)
        k[0, 0, :n] = q[0, 0, :n]                 # keys equal to queries
        if N > 3:
            k[0, D - 1, 1:3] = k[0, D - 1, 0]     # duplicate keys
        if D > 1:
            k[P - 1, 1, :] = 0.25                 # one dimension with all keys equal
    return q.to(device), k.to(device), v.to(device)
