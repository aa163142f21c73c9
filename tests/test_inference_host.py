"""Host-side pieces of the forward-only entry points (no GPU): supersampling reduction, PSNR, 8-bit colour."""
import numpy as np
import torch

from oracle import oracle
from raygaussx_b200 import inference as inf


def test_reduce_supersampling_is_the_mean_over_each_pixels_rays():
    g = torch.Generator().manual_seed(3)
    w, h, fx, fy = 5, 4, 2, 3
    rays = torch.rand(w * fx * h * fy, 3, generator=g)
    got = inf.reduce_supersampling(w, h, rays, (fx, fy))
    assert got.shape == (h, w, 3)
    img = rays.reshape(h * fy, w * fx, 3)            # rays are row-major over the supersampled image
    for y in range(h):
        for x in range(w):
            want = img[y * fy:(y + 1) * fy, x * fx:(x + 1) * fx].reshape(-1, 3).mean(dim=0)
            assert torch.allclose(got[y, x], want, atol=1e-6)
    # the reference's way of writing it (utils/general_utils.py:489-502): strided sums, first along x, then along y
    s = rays[0::fx].clone()
    for i in range(1, fx):
        s += rays[i::fx]
    s = s.reshape(h * fy, w, 3)
    m = s[0::fy].clone()
    for i in range(1, fy):
        m += s[i::fy]
    assert torch.allclose(got, m / (fx * fy), atol=1e-6)
    assert torch.equal(inf.reduce_supersampling(w, h, rays[: w * h], (1, 1)), rays[: w * h].reshape(h, w, 3))


def test_psnr():
    a = np.full((4, 4, 3), 0.5)
    assert inf.PSNR(a, a) == 100
    assert abs(inf.PSNR(a, a + 0.1) - 20.0) < 1e-9
    assert abs(inf.PSNR(torch.tensor(a), torch.tensor(a) + 0.01) - 40.0) < 1e-6


def test_quantize_frame_known_answers():
    x = np.array([[-1.0, 0.0, 0.00390624], [0.00390625, 0.5, 0.999], [1.0, 2.0, 0.99609375]], dtype=np.float32)
    q = oracle.quantize_frame(x)
    assert q.dtype == np.uint8 and q.shape == (3, 4)
    assert q[:, :3].tolist() == [[0, 0, 0], [1, 128, 255], [255, 255, 255]]
    assert (q[:, 3] == 255).all()
