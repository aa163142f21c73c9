"""One training iteration around the ray-marching operator: the counterpart of the
loop body of the reference's ``scripts/train.py:83-165`` without its OptiX, cupy
and ``fused_ssim`` imports.

What an iteration does there, and here: pick a random training camera, render it
through ``RenderOptixFunction`` (``optix_raycasting/render_optix.py``), average the
supersampled rays, form the loss ``(1 - l) L1 + l (1 - SSIM) + l_iso * isotropy``,
divide it by the number of accumulated views once accumulation is on
(20 views per optimizer step from iteration 20,000), back-propagate, feed the
position gradients to the densification statistics
(``classes/point_cloud.py:468-479``) and step the optimizers when the window is
full.  The reference's OptiX context, pipelines and acceleration structure
(``scripts/train.py:95-115``) have no counterpart: the operator keeps its own
workspace.

``pointcloud`` is any object with the reference's interface: ``get_data(...)``,
``optim_managers`` (``zero_grad()``, ``step()``), ``positions``,
``accumulate_gradient(grad, cam)``, ``accumulate_gradient_gaussians_not_visible(grad)``
and ``num_sph_gauss``.  ``SimplePointCloud`` is a small one for tests and benchmarks.
"""
from __future__ import annotations

import math
import random
from types import SimpleNamespace
from typing import Callable, List, Optional

import torch
import torch.nn.functional as F

from . import render_optix as r_ox
from .inference import reduce_supersampling


# ----------------------------------------------------------------------------- losses
def l1_loss(image, target):
    return (image - target).abs().mean()


def _gaussian_taps(size: int, sigma: float, like: torch.Tensor) -> torch.Tensor:
    x = torch.arange(size, dtype=torch.float64) - size // 2
    g = torch.exp(-(x * x) / (2.0 * sigma * sigma))
    return (g / g.sum()).to(like.dtype).to(like.device)


def _blur(x: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """Separable Gaussian blur of ``[B, C, H, W]`` with zero padding, one pass per axis."""
    c = x.shape[1]
    k = taps.numel()
    kx = taps.view(1, 1, 1, k).expand(c, 1, 1, k)
    ky = taps.view(1, 1, k, 1).expand(c, 1, k, 1)
    x = F.conv2d(x, kx, padding=(0, k // 2), groups=c)
    return F.conv2d(x, ky, padding=(k // 2, 0), groups=c)


def ssim(img1: torch.Tensor, img2: torch.Tensor, window_size: int = 11, sigma: float = 1.5) -> torch.Tensor:
    """Mean structural similarity (Wang et al. 2004) of ``[B, 3, H, W]`` or ``[3, H, W]`` images in [0, 1] with
    the 11-tap, sigma 1.5 Gaussian window, zero padding and the constants (0.01^2, 0.03^2) that the reference's
    loss uses (``scripts/train.py:134`` through ``fused_ssim``; same definition as ``utils/loss_utils.py:37-62``)."""
    squeeze = img1.dim() == 3
    if squeeze:
        img1, img2 = img1.unsqueeze(0), img2.unsqueeze(0)
    taps = _gaussian_taps(window_size, sigma, img1)
    mu1, mu2 = _blur(img1, taps), _blur(img2, taps)
    mu1_sq, mu2_sq, mu12 = mu1 * mu1, mu2 * mu2, mu1 * mu2
    s1 = _blur(img1 * img1, taps) - mu1_sq
    s2 = _blur(img2 * img2, taps) - mu2_sq
    s12 = _blur(img1 * img2, taps) - mu12
    c1, c2 = 0.01 ** 2, 0.03 ** 2
    value = ((2 * mu12 + c1) * (2 * s12 + c2)) / ((mu1_sq + mu2_sq + c1) * (s1 + s2 + c2))
    return value.mean()


def isotropy_loss(scales: torch.Tensor) -> torch.Tensor:
    """``scripts/train.py:139-142``: mean over Gaussians of ``max(r, 10) - 10`` with
    ``r = 2 / (pi sqrt 3) * |s|^3 / (s_x s_y s_z)`` (the reference writes pi as 3.14159265359)."""
    r = (2 / (3.14159265359 * (3 ** 0.5))) * ((scales[:, 0] ** 2 + scales[:, 1] ** 2 + scales[:, 2] ** 2) ** (3 / 2)) / (
        scales[:, 0] * scales[:, 1] * scales[:, 2])
    return (torch.clamp(r, min=10) - 10).mean()


# ----------------------------------------------------------------------------- the iteration
class AccumulationSchedule:
    """Gradient accumulation of ``scripts/train.py:77-85,150-161``: from ``accum_start`` on, ``accum_steps``
    views share one optimizer step."""

    def __init__(self, accum_steps: int = 20, accum_start: int = 20000):
        self.accum_steps = accum_steps
        self.accum_start = accum_start
        self.counter = 0

    def use_accum(self, iteration: int) -> bool:
        return iteration >= self.accum_start and self.accum_steps > 1


def pick_camera(stack: List, cameras: Callable[[], List]):
    """``scripts/train.py:90-94``: cameras are drawn without replacement; the stack is refilled when empty."""
    if not stack:
        stack.extend(cameras())
    return stack.pop(random.randint(0, len(stack) - 1))


def training_iteration(pointcloud, viewpoint_cam, config, iteration: int, schedule: AccumulationSchedule,
                       hit_prim_idx=None):
    """The body of the reference's training loop for one camera (``scripts/train.py:86-165``).  ``config`` has the
    reference's fields: ``scene.dt``, ``scene.dynamic_sampling``, ``scene.white_background``,
    ``training.max_prim_slice``, ``training.jitter``, ``training.rnd_sample``, ``training.supersampling_x/_y``,
    ``training.lambda_ssim``, ``training.lambda_iso``, ``training.normalize_quaternion``,
    ``training.normalize_lobe_axis``.  Returns ``(loss, stepped)``: the detached loss as back-propagated and
    whether the optimizers stepped."""
    t = config.training
    use_accum = schedule.use_accum(iteration)
    if (not use_accum) or schedule.counter == 0:
        pointcloud.optim_managers.zero_grad()
    gt_image = viewpoint_cam.original_image.to(pointcloud.positions.device)
    supersampling = (t.supersampling_x, t.supersampling_y)
    settings = r_ox.RenderOptixSettings(None, False, None, None, None, None, None, config.scene.dt,
                                        config.scene.dynamic_sampling, viewpoint_cam, t.max_prim_slice,
                                        pointcloud.num_sph_gauss, iteration=iteration, jitter=t.jitter,
                                        rnd_sample=t.rnd_sample, supersampling=supersampling,
                                        white_background=config.scene.white_background, hit_prim_idx=hit_prim_idx)
    (positions, scales, quaternions, densities, color_features, sph_gauss_features, bandwidth_sharpness,
     lobe_axis) = pointcloud.get_data(normalized_quaternion=not t.normalize_quaternion,
                                      normalized_lobe_axis=not t.normalize_lobe_axis)
    image = r_ox.RenderOptixFunction.apply(positions, scales, quaternions, densities, color_features,
                                           sph_gauss_features, bandwidth_sharpness, lobe_axis, settings)
    image_mean = reduce_supersampling(viewpoint_cam.image_width, viewpoint_cam.image_height, image, supersampling)
    image_mean = image_mean.permute(2, 0, 1)
    loss = (1.0 - t.lambda_ssim) * l1_loss(image_mean, gt_image)
    if t.lambda_ssim != 0:
        loss = loss + t.lambda_ssim * (1.0 - ssim(image_mean, gt_image))
    loss = loss + t.lambda_iso * isotropy_loss(scales)
    if use_accum:
        loss = loss / float(schedule.accum_steps)
    loss.backward()
    if pointcloud.positions.grad is not None:
        pointcloud.accumulate_gradient(pointcloud.positions.grad, viewpoint_cam)
        pointcloud.accumulate_gradient_gaussians_not_visible(pointcloud.positions.grad)
    stepped = False
    if use_accum:
        schedule.counter += 1
        if schedule.counter >= schedule.accum_steps:
            pointcloud.optim_managers.step()
            pointcloud.optim_managers.zero_grad()
            schedule.counter = 0
            stepped = True
    else:
        pointcloud.optim_managers.step()
        pointcloud.optim_managers.zero_grad()
        stepped = True
    return loss.detach(), stepped


# ----------------------------------------------------------------------------- a small point cloud
class _Optimizers:
    """The part of the reference's optimizer manager the loop uses (``zero_grad``, ``step``, ``get_lrs``)."""

    def __init__(self, groups):
        self.optimizer = torch.optim.Adam(groups, eps=1e-15)

    def zero_grad(self):
        self.optimizer.zero_grad(set_to_none=True)

    def step(self):
        self.optimizer.step()

    def get_lrs(self):
        return {g["name"]: g["lr"] for g in self.optimizer.param_groups}


class SimplePointCloud:
    """Gaussians in the reference's parameterisation (``classes/point_cloud.py:509-559``): positions, logarithms
    of the scales, raw quaternions, densities, colour as DC term plus higher SH bands, lobe tensors -- with one
    Adam group per tensor and the densification statistics of ``classes/point_cloud.py:468-479``."""

    def __init__(self, positions, scales, quaternions, densities, color_features, sph_gauss_features=None,
                 bandwidth_sharpness=None, lobe_axis=None, lrs: Optional[dict] = None):
        dev = positions.device
        n = positions.shape[0]
        leaf = lambda x: x.detach().clone().contiguous().requires_grad_(True)
        self.positions = leaf(positions)
        self.scales = leaf(torch.log(scales))
        self.quaternions = leaf(quaternions)
        self.densities = leaf(densities)
        self.rgb = leaf(color_features[:, :, 0])
        self.spherical_harmonics = leaf(color_features[:, :, 1:])
        g = 0 if sph_gauss_features is None else sph_gauss_features.shape[2]
        self.num_sph_gauss = g
        self.sph_gauss_features = leaf(sph_gauss_features if g else torch.zeros(n, 3, 0, device=dev))
        # softplus is undone so that get_bandwidth_sharpness returns what was passed in
        sharp = bandwidth_sharpness if g else torch.zeros(n, 0, device=dev)
        self.bandwidth_sharpness = leaf(torch.where(sharp > 20, sharp, torch.log(torch.expm1(sharp.clamp_min(1e-6)))))
        self.lobe_axis = leaf(lobe_axis if g else torch.zeros(n, 0, 3, device=dev))
        lr = dict(positions=1.6e-4, scales=5e-3, quaternions=1e-3, densities=5e-2, rgb=2.5e-3,
                  spherical_harmonics=1.25e-4, sph_gauss_features=2.5e-3, bandwidth_sharpness=1e-3, lobe_axis=1e-3)
        lr.update(lrs or {})
        self.optim_managers = _Optimizers([dict(params=[getattr(self, k)], lr=v, name=k) for k, v in lr.items()
                                           if getattr(self, k).numel() > 0])
        self.reset_gradient_accum()

    # accessors of classes/point_cloud.py:509-559
    def get_color_features(self):
        return torch.cat([self.rgb[:, :, None], self.spherical_harmonics], dim=2)

    def get_scale(self):
        return torch.exp(self.scales)

    def get_normalized_quaternion(self):
        return self.quaternions / torch.norm(self.quaternions, dim=1)[:, None]

    def get_density(self):
        return self.densities

    def get_bandwidth_sharpness(self):
        return F.softplus(self.bandwidth_sharpness)

    def get_normalized_lobe_axis(self):
        if self.lobe_axis.numel() == 0:
            return self.lobe_axis
        return self.lobe_axis / torch.norm(self.lobe_axis, dim=2)[:, :, None]

    def get_data(self, normalized_quaternion=True, normalized_lobe_axis=True):
        q = self.get_normalized_quaternion() if normalized_quaternion else self.quaternions
        a = self.get_normalized_lobe_axis() if normalized_lobe_axis else self.lobe_axis
        return (self.positions, self.get_scale(), q, self.get_density(), self.get_color_features(),
                self.sph_gauss_features, self.get_bandwidth_sharpness(), a)

    # statistics of classes/point_cloud.py:468-485
    @torch.no_grad()
    def reset_gradient_accum(self):
        n, dev = self.positions.shape[0], self.positions.device
        self.xyz_gradient_accum_norm = torch.zeros(n, device=dev)
        self.num_accum = torch.zeros(n, device=dev)
        self.num_accum_gnv = torch.zeros(n, device=dev)

    @torch.no_grad()
    def accumulate_gradient(self, grad, camera):
        dist = torch.clamp(torch.norm(self.positions - camera.camera_center[None, :], dim=1), min=1.0)
        norm = torch.norm(grad, dim=1)
        self.xyz_gradient_accum_norm += norm * dist
        self.num_accum += torch.where(norm > 0, 1.0, 0.0)

    @torch.no_grad()
    def accumulate_gradient_gaussians_not_visible(self, grad):
        self.num_accum_gnv += torch.where(torch.norm(grad, dim=1) > 0, 1.0, 0.0)


def default_config(dt=0.01, dynamic_sampling=False, white_background=False, max_prim_slice=512, lambda_ssim=0.2,
                   lambda_iso=0.0) -> SimpleNamespace:
    """A configuration with the fields ``training_iteration`` reads, named as in the reference's YAML
    (``configs/base.yml``)."""
    return SimpleNamespace(
        scene=SimpleNamespace(dt=dt, dynamic_sampling=dynamic_sampling, white_background=white_background),
        training=SimpleNamespace(max_prim_slice=max_prim_slice, jitter=False, rnd_sample=0, supersampling_x=1,
                                 supersampling_y=1, lambda_ssim=lambda_ssim, lambda_iso=lambda_iso,
                                 normalize_quaternion=False, normalize_lobe_axis=False))
