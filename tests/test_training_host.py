"""Host-side pieces of the training iteration (no GPU): losses against values of the reference's own
``utils/loss_utils.py`` (tests/golden/ssim.npz, made by tests/golden/make_ssim_golden.py), the isotropy
term, the accumulation schedule and the point cloud's statistics."""
import os
import random

import numpy as np
import pytest
import torch

from raygaussx_b200 import training as tr
from tests.golden.make_ssim_golden import CASES, images

GOLDEN = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ssim.npz"))


@pytest.mark.parametrize("seed,h,w", CASES)
def test_ssim_and_l1_match_the_reference(seed, h, w):
    a, b = images(seed, h, w)
    assert float(tr.ssim(a, b)) == pytest.approx(float(GOLDEN[f"ssim_{seed}"]), abs=2e-6)
    assert float(tr.ssim(a[None], b[None])) == pytest.approx(float(GOLDEN[f"ssim_batched_{seed}"]), abs=2e-6)
    assert float(tr.l1_loss(a, b)) == pytest.approx(float(GOLDEN[f"l1_{seed}"]), abs=1e-7)


def test_ssim_properties_and_direct_evaluation():
    a, b = images(11, 13, 17)
    assert float(tr.ssim(a, a)) == pytest.approx(1.0, abs=1e-6)
    assert float(tr.ssim(a, b)) == pytest.approx(float(tr.ssim(b, a)), abs=1e-7)
    # dense evaluation in float64, window by window
    k, sig = 11, 1.5
    x = torch.arange(k, dtype=torch.float64) - k // 2
    g = torch.exp(-x * x / (2 * sig * sig))
    g = g / g.sum()
    win = g[:, None] * g[None, :]
    A = torch.nn.functional.pad(a.double(), (k // 2,) * 4)
    B = torch.nn.functional.pad(b.double(), (k // 2,) * 4)
    tot = 0.0
    for c in range(3):
        for i in range(a.shape[1]):
            for j in range(a.shape[2]):
                pa, pb = A[c, i:i + k, j:j + k], B[c, i:i + k, j:j + k]
                m1, m2 = (win * pa).sum(), (win * pb).sum()
                s1, s2 = (win * pa * pa).sum() - m1 * m1, (win * pb * pb).sum() - m2 * m2
                s12 = (win * pa * pb).sum() - m1 * m2
                tot += ((2 * m1 * m2 + 1e-4) * (2 * s12 + 9e-4)) / ((m1 * m1 + m2 * m2 + 1e-4) * (s1 + s2 + 9e-4))
    assert float(tr.ssim(a, b)) == pytest.approx(float(tot) / a.numel(), abs=2e-6)
    a.requires_grad_(True)
    tr.ssim(a, b).backward()
    assert torch.isfinite(a.grad).all() and a.grad.abs().sum() > 0


def test_isotropy_term():
    s = torch.tensor([[1.0, 1.0, 1.0], [1.0, 1.0, 0.01], [2.0, 0.5, 0.1]], dtype=torch.float64)
    r = (2 / (3.14159265359 * 3 ** 0.5)) * (s ** 2).sum(1) ** 1.5 / s.prod(1)
    want = (r.clamp(min=10) - 10).mean()
    assert float(tr.isotropy_loss(s)) == pytest.approx(float(want), rel=1e-12)
    assert float(tr.isotropy_loss(torch.ones(5, 3))) == 0.0          # a sphere has r = 6 / pi < 10


def test_accumulation_schedule_and_camera_stack():
    sch = tr.AccumulationSchedule(accum_steps=20, accum_start=20000)
    assert not sch.use_accum(19999) and sch.use_accum(20000)
    assert not tr.AccumulationSchedule(accum_steps=1, accum_start=0).use_accum(5)
    random.seed(0)
    cams = list(range(7))
    stack, seen = [], []
    for _ in range(14):
        seen.append(tr.pick_camera(stack, lambda: cams.copy()))
    assert sorted(seen[:7]) == cams and sorted(seen[7:]) == cams      # without replacement, refilled when empty


def test_point_cloud_parameterisation_and_statistics():
    g = torch.Generator().manual_seed(5)
    n = 50
    pos = torch.randn(n, 3, generator=g)
    scales = torch.rand(n, 3, generator=g) * 0.1 + 0.01
    quats = torch.randn(n, 4, generator=g)
    dens = torch.rand(n, generator=g) * 5 + 0.2
    col = torch.randn(n, 3, 16, generator=g)
    sg = torch.randn(n, 3, 2, generator=g)
    sharp = torch.rand(n, 2, generator=g) * 3 + 0.1
    axis = torch.randn(n, 2, 3, generator=g)
    pc = tr.SimplePointCloud(pos, scales, quats, dens, col, sg, sharp, axis)
    p, s, q, d, c, f, b, a = pc.get_data()
    assert torch.allclose(s, scales, rtol=1e-6) and torch.equal(p, pos) and torch.equal(d, dens)
    assert torch.allclose(q.norm(dim=1), torch.ones(n), atol=1e-6) and torch.allclose(c, col)
    assert torch.allclose(b, sharp, rtol=1e-5) and torch.allclose(a.norm(dim=2), torch.ones(n, 2), atol=1e-6)
    assert torch.equal(pc.get_data(normalized_quaternion=False)[2], quats)
    cam = type("Cam", (), {"camera_center": torch.tensor([0.0, 0.0, 3.0])})()
    grad = torch.randn(n, 3, generator=g)
    grad[::3] = 0
    pc.accumulate_gradient(grad, cam)
    pc.accumulate_gradient(grad, cam)
    pc.accumulate_gradient_gaussians_not_visible(grad)
    dist = (pos - cam.camera_center).norm(dim=1).clamp(min=1.0)
    assert torch.allclose(pc.xyz_gradient_accum_norm, 2 * grad.norm(dim=1) * dist, rtol=1e-6)
    assert torch.equal(pc.num_accum, 2.0 * (grad.norm(dim=1) > 0)) and torch.equal(pc.num_accum_gnv, 1.0 * (grad.norm(dim=1) > 0))
    assert set(pc.optim_managers.get_lrs()) >= {"positions", "scales", "quaternions", "densities", "rgb"}
