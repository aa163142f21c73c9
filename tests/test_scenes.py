"""Seeded generators are deterministic and follow the stated recipes."""
import math

import torch

from raygaussx_b200 import scenes


def test_tiny_scene_is_deterministic_and_shaped():
    a, b = scenes.tiny_scene(), scenes.tiny_scene()
    for x, y in zip(a.tensors(), b.tensors()):
        assert torch.equal(x, y)
    assert a.positions.shape == (4096, 3) and a.color_features.shape == (4096, 3, 16)
    assert a.positions.abs().max() <= 1
    assert torch.allclose(a.quaternions.norm(dim=1), torch.ones(4096), atol=1e-6)
    cam = a.cameras[0]
    assert (cam.image_width, cam.image_height) == (64, 64)
    assert cam.camera_center.norm().item() == __import__("pytest").approx(4.0, abs=1e-5)
    assert a.march.dt_step == 0.0025 and not a.march.dynamic_sampling and a.march.max_prim_slice == 2048


def test_unbounded_scene_recipe_small():
    s = scenes.unbounded_scene(n=20000, n_cameras=4, width=32, height=20)
    r = s.positions.norm(dim=1)
    shell = r >= 4.99
    assert 0.15 < shell.float().mean() < 0.25
    ratio = s.scales[shell].max(dim=1).values / s.scales[shell].min(dim=1).values
    assert ratio.max() <= 10.0 + 1e-4
    assert s.march.dynamic_sampling and s.march.max_prim_slice == 512 and s.march.dt_step == 0.005
    c = s.cameras[1]
    assert c.camera_center[2].item() == __import__("pytest").approx(0.5, abs=1e-6)
    assert math.hypot(c.camera_center[0].item(), c.camera_center[1].item()) == __import__("pytest").approx(3.0, abs=1e-5)


def test_object_and_stress_recipes_small():
    o = scenes.object_scene(n=5000, n_cameras=3, width=16, height=16)
    assert o.positions.abs().max() <= 1.5 and o.march.white_background and not o.march.dynamic_sampling
    assert all(c.camera_center[2] >= 0 for c in o.cameras)
    t = scenes.stress_scene(n_uniform=3000, n_cluster=500, n_cameras=2, width=16, height=9)
    assert t.n == 3500 and t.march.transmittance_eps == 1e-4
    ratio = t.scales.max(dim=1).values / t.scales.min(dim=1).values
    assert ratio.max() <= 100.0 + 1e-3
