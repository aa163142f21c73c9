"""The reference's own ``classes/point_cloud.py`` -- loaded UNCHANGED from a reference checkout -- trained through
this repository's renderer (B200, `-m gpu`).

What is shown: with this repository first and the reference checkout second on ``sys.path``, the reference's
``classes.point_cloud``, ``classes.optimizer``, ``utils.optim_utils``, ``utils.reordering_utils``,
``utils.sh_utils``, ``utils.graphics_utils``, ``utils.logger`` and ``scripts.ply`` import as they are; what they
import from the renderer's side resolves here: ``optix_raycasting.render_optix`` (the autograd entry point),
``simple_knn._C.distCUDA2`` (sizes the first Gaussians, classes/point_cloud.py:592) and ``utils.general_utils``
(the cupy-free stand-in).  A ``PointCloud`` made by ``init_random`` then runs the reference's training-loop body
(scripts/train.py:83-165, as ``training.training_iteration``), its densification, pruning and Z-order reordering
(classes/point_cloud.py:846-922,1017-1046), and trains on.

Needs the reference checkout: ``$RGX_REFERENCE_DIR`` or a directory ``reference`` beside this repository;
skipped where there is none.  matplotlib is not part of this image: ``classes/optimizer.py`` imports it for a
learning-rate plot that nothing here draws, so the test puts an empty module of that name in its place.
"""
import os
import random
import sys
import types
from types import SimpleNamespace

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def reference_dir():
    for cand in (os.environ.get("RGX_REFERENCE_DIR"), os.path.join(os.path.dirname(ROOT), "reference")):
        if cand and os.path.isfile(os.path.join(cand, "classes", "point_cloud.py")):
            return os.path.abspath(cand)
    return None


@pytest.fixture(scope="module")
def ref():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device: there is no CPU path")
    rd = reference_dir()
    if rd is None:
        pytest.skip("no reference checkout (RGX_REFERENCE_DIR): classes/point_cloud.py is loaded from there, unchanged")
    saved_path, saved_mods = list(sys.path), set(sys.modules)
    sys.path[:] = [ROOT, rd] + [p for p in sys.path if p not in (ROOT, rd)]
    try:
        import matplotlib.pyplot  # noqa: F401
    except ImportError:
        mpl = types.ModuleType("matplotlib")
        mpl.pyplot = types.ModuleType("matplotlib.pyplot")
        sys.modules["matplotlib"], sys.modules["matplotlib.pyplot"] = mpl, mpl.pyplot
    import classes.point_cloud as point_cloud
    import utils.general_utils as general_utils
    import utils.optim_utils as optim_utils
    # the modules came from where they should
    assert os.path.abspath(point_cloud.__file__).startswith(rd)
    assert os.path.abspath(optim_utils.__file__).startswith(rd)
    assert os.path.abspath(general_utils.__file__).startswith(ROOT)
    assert os.path.abspath(sys.modules["simple_knn._C"].__file__).startswith(ROOT)
    yield SimpleNamespace(point_cloud=point_cloud, optim_utils=optim_utils, dir=rd)
    sys.path[:] = saved_path
    for name in set(sys.modules) - saved_mods:
        if name.split(".")[0] in ("classes", "utils", "scripts", "matplotlib"):
            del sys.modules[name]


def optimizer_config():
    """The shape of configs/base.yml:83-150 (training.optimization), constant learning rates."""
    group = lambda lr: SimpleNamespace(scheduler=False, init_lr=lr, final_lr=lr, decay_step=0, delay_step=0, donotuse_steps=0)
    return SimpleNamespace(position=group(2e-4), rgb=group(2e-2), sh=group(1e-3), density=group(5e-2), scale=group(5e-3),
                           quaternion=group(1e-3), sph_gauss_features=group(1e-3), bandwidth_sharpness=group(1e-3),
                           lobe_axis=group(1e-3))


def attach_optimizers(ref, pc):
    m = ref.optim_utils.define_optimizer_manager(optimizer_config(), pc, [], [], [], [], [], [], [], [], [])
    names = ("xyz", "rgb", "sh", "density", "scales", "quaternions", "sph_gauss_features", "bandwidth_sharpness", "lobe_axis")
    pc.setup_optimizers(dict(zip(names, m)))                              # scripts/train.py:48-53


def test_reference_point_cloud_trains_densifies_and_reorders(ref):
    from raygaussx_b200 import scenes, training
    from raygaussx_b200 import render_optix as ro
    dev = torch.device("cuda")
    np.random.seed(0)
    random.seed(0)
    torch.manual_seed(0)
    pc = ref.point_cloud.PointCloud("float32", dev)
    pc.init_random(num_pts=6000, sh_nb=4, sg_nb=0, default_density=6.0)   # sizes the Gaussians with distCUDA2
    assert pc.positions.shape == (6000, 3) and torch.isfinite(pc.scales).all()
    attach_optimizers(ref, pc)
    cfg = training.default_config(dt=0.01, dynamic_sampling=False, white_background=False, max_prim_slice=1024,
                                  lambda_ssim=0.2, lambda_iso=0.0)
    # targets: a brighter, differently coloured version of the same cloud, rendered through the same operator
    cams = [scenes.SimpleCamera(eye, width=48, height=40, device=dev) for eye in
            ((3.5, 0.3, 0.8), (-0.5, 3.4, 1.0), (-3.2, -1.0, 1.4), (0.8, -3.3, -0.9))]
    with torch.no_grad():
        data = list(pc.get_data())
        g = torch.Generator().manual_seed(3)
        data[4] = data[4] + 0.25 * torch.rand(data[4].shape, generator=g).to(dev)
        for c in cams:
            st = ro.RenderOptixSettings(None, False, None, None, None, None, None, cfg.scene.dt, False, c, 1024, 0)
            img = ro.RenderOptixFunction.apply(*data, st)
            c.original_image = img.reshape(c.image_height, c.image_width, 3).permute(2, 0, 1).contiguous()
    sch = training.AccumulationSchedule(accum_steps=20, accum_start=10 ** 9)
    stack, losses = [], []
    for it in range(24):
        cam = training.pick_camera(stack, lambda: list(cams))
        loss, stepped = training.training_iteration(pc, cam, cfg, it, sch)
        assert stepped and torch.isfinite(loss)
        losses.append(float(loss))
    assert sum(losses[-4:]) < 0.8 * sum(losses[:4]), losses
    assert (pc.num_accum > 0).any() and pc.xyz_gradient_accum_norm.shape == (6000,)

    # densification, pruning and reordering of the reference change N and the order under the renderer's feet
    n0 = pc.positions.shape[0]
    grads = pc.xyz_gradient_accum_norm / pc.num_accum.clamp_min(1)
    threshold = float(grads[pc.num_accum > 0].quantile(0.9))
    with torch.no_grad():
        pc.densities[:50] = 0.001                                          # these fall to the density pruning
    pc.densify_and_prune(threshold, 0.01, 2.6, cams)
    n1 = pc.positions.shape[0]
    assert n1 != n0 and pc.scales.shape == (n1, 3) and pc.quaternions.shape == (n1, 4) and pc.num_accum.shape == (n1,)
    pc.reorder_zordercurve()
    assert pc.positions.shape == (n1, 3) and pc.positions.requires_grad
    pc.reset_gradient_accum()
    after = []
    for it in range(24, 36):
        cam = training.pick_camera(stack, lambda: list(cams))
        loss, _ = training.training_iteration(pc, cam, cfg, it, sch)
        assert torch.isfinite(loss)
        after.append(float(loss))
    for p in (pc.positions, pc.scales, pc.quaternions, pc.densities, pc.rgb, pc.spherical_harmonics):
        assert torch.isfinite(p).all()
    assert sum(after[-4:]) / 4 < sum(losses[:4]) / 4                        # still better than at the start
    # the renderer's workspace followed the new Gaussian count
    assert ro.get_renderer(dev)._n_built == n1
