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
    check_records(x, y, mode)


# Key distributions that stress the sort and the rank search rather than the arithmetic: every key equal (one value bucket holds
# everything, and in the radix sort all lanes of a warp share every digit), two values, one far outlier (the bucket index of the rank search collapses to one bucket), keys already
# ascending / descending, values that differ only in their low mantissa bits, and infinities. Both the shared-memory kernel
# (N = 16384, 4096) and the long-sequence kernels (N = 20000).
KINDS = ["equal", "two_values", "outlier", "ascending", "descending", "low_bits", "infinities", "clump_40", "clump_200"]


@pytest.mark.parametrize("kind", KINDS)
@pytest.mark.parametrize("N", [4096, 16384, 20000])
def test_records_degenerate_keys(kind, N):
    P, D, M = 1, 2, N - 37
    g = torch.Generator().manual_seed(N + len(kind))
    y = torch.randn(P, D, M, generator=g)
    if kind == "equal":
        x = torch.full((P, D, N), 0.75)
        y[0, 0, :100] = 0.75
    elif kind == "two_values":
        x = torch.where(torch.rand(P, D, N, generator=g) < 0.5, torch.tensor(-1.5), torch.tensor(0.25))
        y[0, 1, :50] = 0.25
    elif kind == "outlier":
        x = torch.randn(P, D, N, generator=g) * 0.01
        x[:, :, 17] = 3.0e6
        y = y * 0.01
    elif kind == "ascending":
        x = torch.linspace(-2.0, 2.0, N).repeat(P, D, 1).contiguous()
    elif kind == "descending":
        x = torch.linspace(2.0, -2.0, N).repeat(P, D, 1).contiguous()
    elif kind == "low_bits":
        x = (1.0 + torch.randint(0, 4096, (P, D, N), generator=g).float() * 2.0 ** -23)
        y = 1.0 + torch.randint(0, 4096, (P, D, M), generator=g).float() * 2.0 ** -23
    elif kind.startswith("clump"):
        # a group of equal keys inside smooth ones: 40 stay under the bucket sort's limit of 64 keys per bucket (ties are then
        # ranked inside the bucket), 200 send the segment to the radix sort
        x = torch.randn(P, D, N, generator=g)
        n = int(kind.split("_")[1])
        x[:, :, 100:100 + n] = 0.123
        y[0, 0, :30] = 0.123
    else:
        x = torch.randn(P, D, N, generator=g)
        x[:, :, 5] = float("inf")
        x[:, :, 9] = float("-inf")
    check_records(x, y, 1)
    if kind not in ("infinities", "outlier"):       # (Laplace weights of infinite or 1e6-wide gaps are 0 or NaN by definition; the ranks are what is tested here)
        check_records(x, y, 0)


@pytest.mark.parametrize("shape", [(1, 2, 20000, 17000), (1, 1, 40000, 300), (1, 1, 16385, 16385), (1, 1, 70001, 65536)])
@pytest.mark.parametrize("mode", [0, 1])
def test_records_long_segments(shape, mode):
    P, D, N, M = shape
    g = torch.Generator().manual_seed(N * 3 + M)
    x = torch.randn(P, D, N, generator=g) * 2
    y = torch.randn(P, D, M, generator=g) * 2
    x[0, 0, 3:9] = x[0, 0, 2]
    x[0, 0, :4] = y[0, 0, :4]
    check_records(x, y, mode)


def check_records(x, y, mode):
    import qlka_native
    P, D, N = x.shape
    M = y.shape[2]
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
