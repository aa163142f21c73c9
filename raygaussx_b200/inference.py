"""Forward-only rendering of camera lists: the counterparts of ``inference`` and
``render`` in the reference's ``scripts/test.py:40-204``.

The reference's versions create an OptiX context, module, program groups and
pipeline, pack cupy arrays and call ``launch_pipeline_test``
(``optix_raycasting/optix_utils.py:503-640``), whose device code
(``cuda_test/gaussians_aabb.cu``) is the training forward verbatim.  Here the same
signatures and return values sit on ``rgx_build`` + ``rgx_forward``; nothing
OptiX- or cupy-related is touched.  ``frames`` adds what the reference's viewer
kernel writes (``cuda_gui/gaussians_aabb.cu:205-342``): 8-bit colour and expected
depth, into plain device buffers.

A ``pointcloud`` is anything with the accessors the reference's
``classes/point_cloud.py`` has: ``positions``, ``get_scale()``,
``get_normalized_quaternion()``, ``get_density()``, ``get_color_features()``,
``sph_gauss_features``, ``get_bandwidth_sharpness()``,
``get_normalized_lobe_axis()``, and for ``culling=True`` also
``project_points(cam)`` and ``select_inside_mask(mask)``.  Cameras need
``camera_center``, ``world_view_transform``, ``FoVx``, ``FoVy``, ``Px``, ``Py``,
``image_width``, ``image_height`` and, for ``inference``, ``original_image``.
"""
from __future__ import annotations

from math import log10, sqrt
from typing import List, Sequence, Tuple

import numpy as np
import torch

from . import render_optix as ro


def PSNR(original, compressed):
    """utils/metrics_utils.py:5-17: 100 for identical images, else 20 log10(1 / rmse)."""
    if torch.is_tensor(original):
        mse = torch.mean((original - compressed) ** 2)
    else:
        mse = np.mean((original - compressed) ** 2)
    if mse == 0:
        return 100
    return 20 * log10(1.0 / sqrt(mse))


def reduce_supersampling(target_width, target_height, ray_colors, factor):
    """utils/general_utils.py:489-502: mean over the ``factor_x x factor_y`` rays of a
    pixel; rays are row-major over the supersampled image.  Returns ``[H, W, 3]``."""
    fx, fy = factor
    img = ray_colors.reshape(target_height, fy, target_width, fx, 3)
    return img.sum(dim=(1, 3)) / float(fx * fy)


def _tensors(pointcloud):
    """The eight renderer inputs, as scripts/test.py:62-67 gathers them."""
    return [pointcloud.positions, pointcloud.get_scale(), pointcloud.get_normalized_quaternion(),
            pointcloud.get_density(), pointcloud.get_color_features(), pointcloud.sph_gauss_features,
            pointcloud.get_bandwidth_sharpness(), pointcloud.get_normalized_lobe_axis()]


def _culled(pointcloud, cam):
    """Frustum culling of scripts/test.py:80-96 (1.3 x the field of view, in front of the camera)."""
    p = pointcloud.project_points(cam)
    depth = p[:, 2] + 1e-6
    x = p[:, 0] / depth / torch.tan(torch.tensor(cam.FoVx / 2))
    y = p[:, 1] / depth / torch.tan(torch.tensor(cam.FoVy / 2))
    mask = (depth > 0) & (x >= -1.3) & (x <= 1.3) & (y >= -1.3) & (y <= 1.3)
    xyz, color, dens, scales, quats, sg, sharp, axis = pointcloud.select_inside_mask(mask)
    return [xyz, scales, quats, dens, color, sg, sharp, axis]


class _Settings:
    def __init__(self, cam, dt_step, dynamic_sampling, max_prim_slice, supersampling, white_background):
        self.viewpoint_cam = cam
        self.dt_step = dt_step
        self.dynamic_sampling = dynamic_sampling
        self.max_prim_slice = max_prim_slice
        self.supersampling = supersampling
        self.white_background = white_background
        self.transmittance_eps = ro.TRANSMITTANCE_EPSILON


def _render_list(tensors_of, cam_list, max_prim_slice, dt_step, supersampling, white_background, dynamic_sampling,
                 rebuild_each):
    """Renders every camera; yields (camera, rays [R,3] on the device, milliseconds)."""
    renderer = None
    tensors = None
    for cam in cam_list:
        if tensors is None or rebuild_each:
            tensors = [ro._as_input(t.detach(), "input") for t in tensors_of(cam)]
            renderer = ro.get_renderer(tensors[0].device)
            renderer.build(*tensors[:4])
        cs = ro.camera_struct(cam, supersampling)
        march = ro._settings_march(_Settings(cam, dt_step, dynamic_sampling, max_prim_slice, supersampling,
                                             white_background), cs)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        rays, _, _ = renderer.forward(*tensors, cs, march)
        end.record()
        torch.cuda.synchronize()
        yield cam, rays, start.elapsed_time(end)


def inference(hit_prim_idx, pointcloud, cam_list, max_prim_slice, dt_step, rnd_sample, supersampling,
              white_background, dynamic_sampling, culling=False):
    """scripts/test.py:40-141.  Returns ``(PSNR_list, gt_images_list, images_list, mean render time in ms)``;
    images are ``[H, W, 3]`` numpy arrays clipped to [0, 1].  ``hit_prim_idx`` and ``rnd_sample`` are accepted
    and unused (no hit buffer exists here; the reference's test-stage kernel ignores ``rnd_sample`` too)."""
    with torch.no_grad():
        psnr_list, gt_list, img_list, times = [], [], [], []
        tensors_of = (lambda cam: _culled(pointcloud, cam)) if culling else (lambda cam: _tensors(pointcloud))
        for cam, rays, ms in _render_list(tensors_of, cam_list, max_prim_slice, dt_step, supersampling,
                                          white_background, dynamic_sampling, rebuild_each=culling):
            times.append(ms)
            image = reduce_supersampling(cam.image_width, cam.image_height, rays, supersampling)
            image_np = image.detach().cpu().numpy().clip(0, 1)
            gt_np = cam.original_image.permute(1, 2, 0).detach().cpu().numpy().clip(0, 1)
            psnr_list.append(PSNR(image_np, gt_np))
            gt_list.append(gt_np)
            img_list.append(image_np)
        return psnr_list, gt_list, img_list, float(np.mean(times)) if times else 0.0


def render(pointcloud, cam_list, max_prim_slice, dt_step, rnd_sample, supersampling, white_background,
           dynamic_sampling):
    """scripts/test.py:143-203 (as used by main_render.py:85 and render_camera_path.py:143): the list of
    ``[H, W, 3]`` numpy images clipped to [0, 1]."""
    with torch.no_grad():
        images, times = [], []
        for cam, rays, ms in _render_list(lambda cam: _tensors(pointcloud), cam_list, max_prim_slice, dt_step,
                                          supersampling, white_background, dynamic_sampling, rebuild_each=False):
            times.append(ms)
            image = reduce_supersampling(cam.image_width, cam.image_height, rays, supersampling)
            images.append(image.detach().cpu().numpy().clip(0, 1))
        if times:
            print("Mean time", np.mean(times))
        return images


def frames(pointcloud, cam_list, max_prim_slice, dt_step, dynamic_sampling,
           transmittance_eps=None) -> List[Tuple[torch.Tensor, torch.Tensor]]:
    """What the reference's viewer shows for each camera (cuda_gui/gaussians_aabb.cu:205-342), without a
    window: ``(frame [H, W, 4] uint8, depth [H, W] float32)`` device tensors, black background."""
    with torch.no_grad():
        tensors = [ro._as_input(t.detach(), "input") for t in _tensors(pointcloud)]
        renderer = ro.get_renderer(tensors[0].device)
        renderer.build(*tensors[:4])
        out = []
        for cam in cam_list:
            cs = ro.camera_struct(cam)
            st = _Settings(cam, dt_step, dynamic_sampling, max_prim_slice, (1, 1), False)
            if transmittance_eps is not None:
                st.transmittance_eps = transmittance_eps
            out.append(renderer.forward_frame(*tensors, cs, ro._settings_march(st, cs)))
        return out
