"""The end-to-end encoder harness (the 12-layer pre-LN encoder, shrunk): the add_laplace encoder output equals
the same network with its attention evaluated by the float64 O(N^2) checker."""

import pytest
import torch

from oracle import direct

pytestmark = pytest.mark.gpu


def test_encoder_matches_checker_attention():
    import importlib
    am = importlib.import_module("kernel_attention.attention")      # the module (the package also exports the function)
    from kernel_attention.encoder import Encoder
    torch.manual_seed(0)
    model = Encoder("add_laplace", layers=2, hidden=128, heads=2, mlp=256, vocab=1000).cuda().eval()
    ids = torch.randint(0, 1000, (2, 300), device="cuda")
    got = model(ids)
    real = am.attention
    try:
        am.attention = lambda q, k, v, kernel, tau, keep=None: direct.attention(q.cpu(), k.cpu(), v.cpu(), kernel, tau, keep).float().cuda()
        want = model(ids)
    finally:
        am.attention = real
    assert got.shape == (2, 300, 128)
    assert (got - want).abs().max().item() < 1e-3 * want.abs().max().item()


def test_measure_runs_small():
    from kernel_attention.encoder import measure
    ms, mib = measure("add_laplace", batch=1, seq=512, layers=2, reps=1)
    assert ms > 0 and mib > 0
