"""Shared helpers of the test-suite."""
import os

import numpy as np
import torch

from raygaussx_b200 import scenes

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
GRAD_NAMES = ("positions", "scales", "quaternions", "densities", "color_features", "sph_gauss_features",
              "bandwidth_sharpness", "lobe_axis")
# kept in step with tests/golden/make_golden.py
CASES = {
    "config1": dict(),
    "small_static": dict(n=512, width=16, height=16, log_scale_mean=-2.5),
    "small_dynamic_white": dict(n=512, width=16, height=16, log_scale_mean=-2.5, dynamic_sampling=True,
                                white_background=True, dt_step=0.005),
    "small_lobes_deg2": dict(n=300, width=12, height=12, log_scale_mean=-2.3, sh_degree=2, lobes=3, seed=7),
    "small_deg0": dict(n=300, width=12, height=12, log_scale_mean=-2.3, sh_degree=0, seed=8),
    "small_deg1_cap": dict(n=400, width=12, height=12, log_scale_mean=-2.0, sh_degree=1, seed=9, max_prim_slice=4096),
}
SMALL_CASES = [k for k in CASES if k != "config1"]


def make_scene(name):
    return scenes.tiny_scene(**CASES[name])


def load_golden(name):
    return np.load(os.path.join(GOLDEN, name + ".npz"))


def input_checksum(sc):
    return float(sum(t.double().sum().item() for t in sc.tensors()))


def loss_gradient(rgb, n_rays):
    tgt = scenes.l1_target(n_rays).to(rgb.dtype)
    return torch.sign(rgb - tgt) / (3 * n_rays)


def rel_max(a, b):
    """max |a-b| over max |a| : the relative error used for gradients."""
    a = torch.as_tensor(a, dtype=torch.float64)
    b = torch.as_tensor(b, dtype=torch.float64)
    return ((a - b).abs().max() / a.abs().max().clamp_min(1e-300)).item()
