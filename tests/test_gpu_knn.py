"""The simple-knn replacement on the GPU (`-m gpu`): exact neighbour distances against the brute-force oracle
(float32 arithmetic on the device: relative 1e-5), through the reference's import path."""
import numpy as np
import pytest
import torch

from oracle import oracle
from raygaussx_b200 import _lib

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dist():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device: there is no CPU path")
    _lib.lib()
    from simple_knn._C import distCUDA2          # classes/point_cloud.py:10
    return distCUDA2


def cloud(n, seed, kind):
    g = torch.Generator().manual_seed(seed)
    if kind == "uniform":
        return torch.rand(n, 3, generator=g) * 4 - 2
    if kind == "clustered":
        c = torch.randn(8, 3, generator=g) * 3
        return c[torch.randint(0, 8, (n,), generator=g)] + 0.02 * torch.randn(n, 3, generator=g)
    if kind == "plane":                       # degenerate extent along one axis
        p = torch.rand(n, 3, generator=g)
        p[:, 2] = 0.25
        return p
    raise ValueError(kind)


@pytest.mark.parametrize("n,kind", [(1, "uniform"), (2, "uniform"), (3, "uniform"), (4, "uniform"), (33, "uniform"),
                                    (1000, "uniform"), (1025, "clustered"), (3000, "plane"), (5000, "clustered")])
def test_matches_brute_force(dist, n, kind):
    pts = cloud(n, 10 + n, kind)
    got = dist(pts.cuda()).cpu().numpy().astype(np.float64)
    want = oracle.knn_mean_dist2(pts.numpy())
    assert got.shape == (n,)
    if n < 4:
        assert np.all(got > 1e37) and np.all(want > 1e37)
    else:
        assert np.abs(got - want).max() <= 1e-5 * want.max() + 1e-12
        assert (np.abs(got - want) / np.maximum(want, 1e-12)).max() < 1e-3


def test_duplicates_and_order_independence(dist):
    pts = cloud(2000, 3, "uniform")
    pts[100] = pts[7]                                  # a duplicate: distance zero counts
    got = dist(pts.cuda()).cpu()
    want = torch.from_numpy(oracle.knn_mean_dist2(pts.numpy())).float()
    assert torch.allclose(got, want, rtol=1e-4, atol=1e-9)
    perm = torch.randperm(2000, generator=torch.Generator().manual_seed(1))
    again = dist(pts[perm].cuda()).cpu()
    assert torch.equal(again, got[perm])               # the result does not depend on the order of the points


def test_large_cloud_properties(dist):
    n = 1_000_000
    pts = cloud(n, 5, "uniform").cuda()
    got = dist(pts)
    assert got.shape == (n,) and torch.isfinite(got).all() and (got > 0).all()
    # spot check 200 points against a dense distance computation on the device
    idx = torch.randint(0, n, (200,), generator=torch.Generator().manual_seed(2)).cuda()
    d = torch.cdist(pts[idx].double(), pts.double()) ** 2
    d[torch.arange(200), idx] = float("inf")
    want = d.topk(3, dim=1, largest=False).values.mean(dim=1)
    assert torch.allclose(got[idx].double(), want, rtol=1e-4)
    with pytest.raises(RuntimeError):
        dist(pts.cpu()[:10])
