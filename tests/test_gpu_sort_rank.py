"""The sort/rank stage on its own, through the C ABI: every array of the walk records
against a numpy restatement (bit-exact for the integer parts)."""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

SHAPES = [(1, 1, 1, 1), (2, 3, 7, 5), (1, 2, 8, 9), (2, 2, 100, 77), (1, 3, 257, 300), (1, 2, 64, 1000),
          (1, 2, 1000, 3), (2, 2, 1024, 1024), (1, 2, 1025, 1500), (1, 2, 2049, 2048), (1, 2, 4096, 4000),
          (1, 2, 8191, 8192), (1, 2, 16384, 16384), (1, 1, 600, 16384)]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("mode", [0, 1])
def test_records(shape, mode):
    import qlka_native
    P, D, N, M = shape
    g = torch.Generator().manual_seed(N * 7 + M)
    x = torch.randn(P, D, N, generator=g) * 3
    y = torch.randn(P, D, M, generator=g) * 3
    n = min(N, M, 4)
    x[0, 0, :n] = y[0, 0, :n]
    if N > 10:
        x[0, D - 1, 3:9] = x[0, D - 1, 2]
        x[0, 0, N // 2] = -0.0
        x[0, 0, N // 2 + 1] = 0.0
    xperm, xval, yrec, mstart = (t.cpu().numpy() for t in qlka_native.sort_rank_records(x.cuda(), y.cuda(), mode))
    torch.cuda.synchronize()
    NBK = N // 8 + 1
    NP = NBK * 8
    xs_all, ys_all = x.numpy().reshape(P * D, N), y.numpy().reshape(P * D, M)
    for s in range(P * D):
        xs, ys = xs_all[s], ys_all[s]
        perm = xperm[s, :N].astype(np.int64)
        assert sorted(perm.tolist()) == list(range(N)), "xperm is not a permutation"
        sx = xs[perm]
        assert np.all(sx[1:] >= sx[:-1]), "keys not ascending"
        assert np.all(xperm[s, N:NP] == 0)
        if mode == 0:
            want = np.ones(NP + 8, np.float64)
            want[0] = 0.0
            want[1:N] = np.exp(-(sx[1:].astype(np.float64) - sx[:-1].astype(np.float64)))
            np.testing.assert_allclose(xval[s], want, rtol=2e-6, atol=1e-30)
        else:
            want = np.zeros(NP + 8, np.float32)
            want[:N] = sx
            assert np.array_equal(xval[s], want)
        assert yrec[s, M, 3] == -1, "sentinel record"
        rec = yrec[s, :M]
        rows = rec[:, 2].astype(np.int64)
        assert sorted(rows.tolist()) == list(range(M)), "query rows are not a permutation"
        sy = ys[rows]
        rank = rec[:, 3].astype(np.int64)
        assert np.all(rank[1:] >= rank[:-1]), "records not ordered by rank"       # equal ranks: any order
        assert np.array_equal(rank, np.searchsorted(sx, sy, side="left")), "rank != number of keys strictly below"
        e0, e1 = rec[:, 0].copy().view(np.float32), rec[:, 1].copy().view(np.float32)
        if mode == 0:
            w0 = np.where(rank > 0, np.exp(-(sy.astype(np.float64) - sx[np.maximum(rank - 1, 0)])), 0.0)
            w1 = np.where(rank < N, np.exp(-(sx[np.minimum(rank, N - 1)].astype(np.float64) - sy)), 0.0)
            # the query weights are taken with the hardware exponential: (2 + 1.2 gap) ulp
            g0 = np.where(rank > 0, sy.astype(np.float64) - sx[np.maximum(rank - 1, 0)], 0.0)
            g1 = np.where(rank < N, sx[np.minimum(rank, N - 1)].astype(np.float64) - sy, 0.0)
            assert np.all(np.abs(e0 - w0) <= (2e-6 + 1.5e-7 * g0) * w0 + 1e-37)
            assert np.all(np.abs(e1 - w1) <= (2e-6 + 1.5e-7 * g1) * w1 + 1e-37)
        else:
            assert np.array_equal(e0, 2.0 * sy)
        want_ms = np.concatenate([np.searchsorted(rank, np.arange(NBK) * 8, side="left"), [M]])
        assert np.array_equal(mstart[s, :NBK + 1].astype(np.int64), want_ms), "mstart"
