"""Helpers shared by the GPU parity tests."""

import torch


def rel_err(a, b):
    """max|a - b| / max|b| with b the checker's float64 result."""
    a = a.detach().to(torch.float64).cpu()
    b = b.detach().to(torch.float64).cpu()
    return ((a - b).abs().max() / b.abs().max().clamp_min(1e-6)).item()


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
