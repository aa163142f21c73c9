"""The training iteration on the GPU (`-m gpu`): the loss goes down, gradients of the whole loss agree with
finite differences of the rendered loss, accumulation steps the optimizers once per window."""
import random

import pytest
import torch

from raygaussx_b200 import _lib
from tests.helpers import make_scene

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def tr():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device: there is no CPU path")
    _lib.lib()
    from raygaussx_b200 import training
    return training


def setup(tr, perturb=0.15, seed=0):
    from raygaussx_b200 import render_optix as ro
    sc = make_scene("small_static")
    dev = torch.device("cuda")
    tens = [t.to(dev).contiguous() for t in sc.tensors()]
    cams = sc.cameras
    for c in cams:
        c.to(dev)
    m = sc.march
    cfg = tr.default_config(dt=m.dt_step, dynamic_sampling=m.dynamic_sampling, white_background=m.white_background,
                            max_prim_slice=m.max_prim_slice)
    # targets: the scene itself, rendered
    for c in cams:
        st = ro.RenderOptixSettings(None, False, None, None, None, None, None, m.dt_step, m.dynamic_sampling, c,
                                    m.max_prim_slice, 0, white_background=m.white_background)
        with torch.no_grad():
            img = ro.RenderOptixFunction.apply(*tens, st)
        c.original_image = img.reshape(c.image_height, c.image_width, 3).permute(2, 0, 1).contiguous()
    g = torch.Generator(device="cpu").manual_seed(seed)
    noisy = [t.clone() for t in tens]
    noisy[4] = noisy[4] + perturb * torch.randn(noisy[4].shape, generator=g).to(dev)          # colours
    noisy[3] = noisy[3] * (1 + perturb * torch.randn(noisy[3].shape, generator=g).to(dev)).clamp(0.5, 1.5)
    pc = tr.SimplePointCloud(*noisy[:5], lrs=dict(rgb=2e-2, spherical_harmonics=2e-3, densities=5e-2))
    return sc, cams, cfg, pc


def test_loss_decreases_and_statistics_fill(tr):
    random.seed(1)
    sc, cams, cfg, pc = setup(tr)
    sch = tr.AccumulationSchedule(accum_steps=20, accum_start=10 ** 9)      # no accumulation: a step per view
    stack, losses = [], []
    for it in range(60):
        cam = tr.pick_camera(stack, lambda: list(cams))
        loss, stepped = tr.training_iteration(pc, cam, cfg, it, sch)
        assert stepped and torch.isfinite(loss)
        losses.append(float(loss))
    first, last = sum(losses[:5]) / 5, sum(losses[-5:]) / 5
    assert last < 0.6 * first, (first, last)
    assert pc.num_accum.max() == 60 and (pc.num_accum > 0).float().mean() > 0.3
    assert torch.equal(pc.num_accum, pc.num_accum_gnv)
    assert (pc.xyz_gradient_accum_norm[pc.num_accum > 0] > 0).all()


def test_accumulation_steps_once_per_window(tr):
    random.seed(2)
    sc, cams, cfg, pc = setup(tr)
    sch = tr.AccumulationSchedule(accum_steps=4, accum_start=0)
    before = pc.rgb.detach().clone()
    stack = []
    flags = []
    for it in range(8):
        cam = tr.pick_camera(stack, lambda: list(cams))
        loss, stepped = tr.training_iteration(pc, cam, cfg, it, sch)
        flags.append(stepped)
        if it == 2:
            assert torch.equal(pc.rgb.detach(), before)        # nothing moved inside the window
            assert pc.rgb.grad is not None and pc.rgb.grad.abs().sum() > 0
    assert flags == [False, False, False, True, False, False, False, True]
    assert not torch.equal(pc.rgb.detach(), before)


def test_gradient_of_the_whole_loss_against_finite_differences(tr):
    sc, cams, cfg, pc = setup(tr, perturb=0.3)
    cfg.training.lambda_iso = 0.01
    cam = cams[0]
    sch = tr.AccumulationSchedule(accum_steps=2, accum_start=0)      # first view of a window: no step yet
    loss, stepped = tr.training_iteration(pc, cam, cfg, 0, sch)
    assert not stepped
    grad = pc.rgb.grad.clone()
    i = int(grad.abs().sum(dim=1).argmax())

    def loss_at(delta):
        with torch.no_grad():
            pc.rgb[i, 0] += delta
            data = pc.get_data()
            from raygaussx_b200 import render_optix as ro
            st = ro.RenderOptixSettings(None, False, None, None, None, None, None, cfg.scene.dt,
                                        cfg.scene.dynamic_sampling, cam, cfg.training.max_prim_slice, 0,
                                        white_background=cfg.scene.white_background)
            img = ro.RenderOptixFunction.apply(*data, st).reshape(cam.image_height, cam.image_width, 3).permute(2, 0, 1)
            val = ((1 - cfg.training.lambda_ssim) * tr.l1_loss(img, cam.original_image)
                   + cfg.training.lambda_ssim * (1 - tr.ssim(img, cam.original_image))
                   + cfg.training.lambda_iso * tr.isotropy_loss(data[1])) / 2.0
            pc.rgb[i, 0] -= delta
            return float(val.double())
    h = 2e-2
    fd = (loss_at(h) - loss_at(-h)) / (2 * h)
    assert fd == pytest.approx(float(grad[i, 0]), rel=0.05, abs=1e-6)
