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


class FakePointCloud:
    """The accessors of the reference's classes/point_cloud.py that the forward-only entry points read,
    over a generated scene (scales are kept as logarithms, as the reference does)."""

    def __init__(self, sc, device="cpu"):
        t = [x.to(device) for x in sc.tensors()]
        self.positions, scales, self.quaternions, self.densities = t[0], t[1], t[2], t[3]
        self.scales = torch.log(scales)
        self._color = t[4]
        self.sph_gauss_features, self._sharp, self.lobe_axis = t[5], t[6], t[7]
        self.num_sph_gauss = t[5].shape[2]

    def get_scale(self):
        return torch.exp(self.scales)

    def get_normalized_quaternion(self):
        return self.quaternions / torch.norm(self.quaternions, dim=1)[:, None]

    def get_density(self):
        return self.densities

    def get_color_features(self):
        return self._color

    def get_bandwidth_sharpness(self):
        return self._sharp

    def get_normalized_lobe_axis(self):
        return self.lobe_axis

    def project_points(self, camera):
        return torch.matmul(self.positions, camera.world_view_transform[:3, :3]) + camera.world_view_transform[3, :3]

    def select_inside_mask(self, mask):
        return (self.positions[mask].contiguous(), self._color[mask].contiguous(), self.densities[mask].contiguous(),
                self.get_scale()[mask].contiguous(), self.get_normalized_quaternion()[mask].contiguous(),
                self.sph_gauss_features[mask].contiguous(), self._sharp[mask].contiguous(),
                self.lobe_axis[mask].contiguous())
