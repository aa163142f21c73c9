"""The nearest-neighbour replacement pinned to the REFERENCE's own extension.

``tests/golden/knn.npz`` holds what ``SimpleKNN::knn`` (submodules/simple-knn/simple_knn.cu, compiled unmodified
into oracle/_ref/libref_knn.so and run on a B200 by tests/golden/make_knn_golden.py) returns for the seeded
clouds of tests/knn_clouds.py: uniform, clustered, planar, with coincident points, and with fewer than four
points.  Against it:

* the float64 brute-force oracle (``oracle.knn_mean_dist2``), on the CPU;
* ``rgx_knn_mean_dist2`` through the reference's import path ``simple_knn._C.distCUDA2``, on the GPU.

Tolerance 2e-6 relative: the reference sums three squared fp32 distances with fused multiply-adds, the
replacement without; infinities and the FLT_MAX / 3 of the three-point cloud must match exactly.
"""
import numpy as np
import pytest
import torch

from tests.helpers import load_golden
from tests.knn_clouds import CLOUDS, cloud

RTOL = 2e-6


def check(name, got, ref):
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape
    inf = np.isinf(ref)
    assert np.array_equal(np.isinf(got), inf), name
    if name == "three":
        assert np.array_equal(got.astype(np.float32), ref.astype(np.float32))       # FLT_MAX / 3 in fp32
        return
    fin = ~inf
    if fin.any():
        assert (np.abs(got[fin] - ref[fin]) <= RTOL * np.abs(ref[fin]) + 1e-30).all(), name


@pytest.mark.parametrize("name", [k for k, v in CLOUDS.items() if v[0] <= 5000])
def test_oracle_matches_the_reference_extension(name):
    n, seed, kind = CLOUDS[name]
    g = load_golden("knn")
    pts = cloud(n, seed, kind)
    assert pts.double().sum().item() == pytest.approx(float(g[name + "_sum"]), abs=1e-9)
    from oracle import oracle
    check(name, oracle.knn_mean_dist2(pts.numpy()), g[name])


@pytest.mark.gpu
@pytest.mark.parametrize("name", list(CLOUDS))
def test_cuda_replacement_matches_the_reference_extension(name):
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device: there is no CPU path")
    from simple_knn._C import distCUDA2          # the reference's import path (classes/point_cloud.py:10)
    n, seed, kind = CLOUDS[name]
    g = load_golden("knn")
    pts = cloud(n, seed, kind)
    assert pts.double().sum().item() == pytest.approx(float(g[name + "_sum"]), abs=1e-9)
    check(name, distCUDA2(pts.cuda()).cpu().numpy(), g[name])
