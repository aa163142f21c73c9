"""Seeded synthetic scenes and cameras for tests and benchmarks.

The public datasets the reference trains on (NeRF-Synthetic, Mip-NeRF 360, ...)
are not reproduced here; these generators only take their *shapes*: Gaussian
counts, extents, size and density distributions, image sizes and camera
layouts.  Everything is drawn on the CPU from ``torch.Generator`` so that a
given seed yields the same scene on every machine.

Conventions follow the reference operator's inputs (classes/point_cloud.py:549-559):
``scales`` are already exponentiated, quaternions are unit ``(w, x, y, z)``,
``densities`` are raw (identity activation), ``color_features`` is ``[N, 3, K]``
channel-major with ``K = (degree + 1) ** 2``.  Cameras expose exactly the fields
the reference reads (optix_utils.py:258-266) and are built the way
classes/cameras.py:49-52 builds them (COLMAP axes: x right, y down, z forward).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional

import torch


@dataclass
class MarchParams:
    """Ray-marching parameters; defaults are the reference's shipped values
    (configs/base.yml:12-13,37; cuda_train/forward/gaussians_aabb.h:2-5)."""
    dt_step: float = 0.005
    dynamic_sampling: bool = True
    max_prim_slice: int = 512
    white_background: bool = False
    transmittance_eps: float = 1e-3
    sigma_threshold: float = 0.1


class SimpleCamera:
    """Duck-typed stand-in for classes/cameras.py:Camera (same field names)."""

    def __init__(self, eye, target=(0.0, 0.0, 0.0), up=(0.0, 0.0, 1.0), fovx=math.radians(40.0),
                 fovy=math.radians(40.0), width=64, height=64, px=0.5, py=0.5, device="cpu"):
        eye = torch.tensor(eye, dtype=torch.float64)
        target = torch.tensor(target, dtype=torch.float64)
        up = torch.tensor(up, dtype=torch.float64)
        fwd = target - eye
        fwd = fwd / fwd.norm()
        right = torch.linalg.cross(fwd, up)
        if right.norm() < 1e-6:  # looking along the up vector
            right = torch.linalg.cross(fwd, torch.tensor([0.0, 1.0, 0.0], dtype=torch.float64))
        right = right / right.norm()
        down = torch.linalg.cross(fwd, right)
        c2w_rot = torch.stack([right, down, fwd], dim=1)  # columns = camera x, y, z in world
        w2c = torch.eye(4, dtype=torch.float64)
        w2c[:3, :3] = c2w_rot.t()
        w2c[:3, 3] = -c2w_rot.t() @ eye
        self.world_view_transform = w2c.t().contiguous().to(torch.float32).to(device)
        self.camera_center = self.world_view_transform.inverse()[3, :3].contiguous()
        self.FoVx = float(fovx)
        self.FoVy = float(fovy)
        self.Px = float(px)
        self.Py = float(py)
        self.image_width = int(width)
        self.image_height = int(height)

    def to(self, device):
        self.world_view_transform = self.world_view_transform.to(device)
        self.camera_center = self.camera_center.to(device)
        return self


def crop_camera(cam, x0, y0, width, height):
    """A camera whose ``width`` x ``height`` image is the window of ``cam``'s image that starts at pixel
    ``(x0, y0)``: same eye and axes, the field of view narrowed and the principal point moved so that ray
    ``(x, y)`` of the crop is ray ``(x0 + x, y0 + y)`` of ``cam`` (the camera model of
    cuda_train/forward/gaussians_aabb.cu:95-110 expresses this exactly; the rays agree to fp32 rounding)."""
    import copy
    c = copy.copy(cam)
    w_full, h_full = cam.image_width, cam.image_height
    c.FoVx = 2.0 * math.atan(math.tan(cam.FoVx / 2) * width / w_full)
    c.FoVy = 2.0 * math.atan(math.tan(cam.FoVy / 2) * height / h_full)
    c.Px = (cam.Px * w_full - x0) / width
    c.Py = (cam.Py * h_full - y0) / height
    c.image_width, c.image_height = int(width), int(height)
    if hasattr(c, "_rgx_camera"):
        del c._rgx_camera
    return c


def lowres_camera(cam, width, height):
    """``cam`` with a coarser image: same eye, axes, field of view and principal point, ``width`` x ``height`` rays."""
    import copy
    c = copy.copy(cam)
    c.image_width, c.image_height = int(width), int(height)
    if hasattr(c, "_rgx_camera"):
        del c._rgx_camera
    return c


@dataclass
class Scene:
    positions: torch.Tensor
    scales: torch.Tensor
    quaternions: torch.Tensor
    densities: torch.Tensor
    color_features: torch.Tensor
    cameras: List[SimpleCamera]
    march: MarchParams
    name: str = ""
    sph_gauss_features: Optional[torch.Tensor] = None
    bandwidth_sharpness: Optional[torch.Tensor] = None
    lobe_axis: Optional[torch.Tensor] = None
    extras: dict = field(default_factory=dict)

    def __post_init__(self):
        n = self.positions.shape[0]
        if self.sph_gauss_features is None:
            self.sph_gauss_features = torch.zeros(n, 3, 0)
            self.bandwidth_sharpness = torch.zeros(n, 0)
            self.lobe_axis = torch.zeros(n, 0, 3)

    @property
    def n(self):
        return self.positions.shape[0]

    def tensors(self):
        return (self.positions, self.scales, self.quaternions, self.densities, self.color_features,
                self.sph_gauss_features, self.bandwidth_sharpness, self.lobe_axis)

    def to(self, device):
        for k in ("positions", "scales", "quaternions", "densities", "color_features", "sph_gauss_features",
                  "bandwidth_sharpness", "lobe_axis"):
            setattr(self, k, getattr(self, k).to(device).contiguous())
        for c in self.cameras:
            c.to(device)
        return self


def _softplus(x):
    return torch.nn.functional.softplus(x)


def _quats(n, g):
    q = torch.randn(n, 4, generator=g)
    return q / q.norm(dim=1, keepdim=True)


def _sh(n, g, degree=3):
    k = (degree + 1) ** 2
    sh = torch.randn(n, 3, k, generator=g) * 0.05
    sh[:, :, 0] = torch.randn(n, 3, generator=g) * 0.2 + 0.5
    return sh


def _sg(n, g, lobes):
    feats = torch.randn(n, 3, lobes, generator=g) * 0.1
    sharp = _softplus(torch.randn(n, lobes, generator=g)) * 4.0 + 0.5
    axis = torch.randn(n, lobes, 3, generator=g)
    axis = axis / axis.norm(dim=2, keepdim=True)
    return feats, sharp, axis


def tiny_scene(seed=0, n=4096, width=64, height=64, sh_degree=3, lobes=0, white_background=False,
               dynamic_sampling=False, dt_step=0.0025, max_prim_slice=2048, log_scale_mean=-3.5,
               density_scale=10.0) -> Scene:
    """The CPU-checkable scene: N Gaussians in [-1,1]^3, one pinhole camera at
    (2, -3, sqrt(3)) (radius 4) with 40 degree FoV.  With the defaults this is
    the 4,096-Gaussian 64x64 configuration."""
    g = torch.Generator().manual_seed(seed)
    pos = torch.rand(n, 3, generator=g) * 2 - 1
    scales = torch.exp(torch.randn(n, 3, generator=g) * 0.3 + log_scale_mean)
    quats = _quats(n, g)
    dens = density_scale * _softplus(torch.randn(n, generator=g))
    sh = _sh(n, g, sh_degree)
    cam = SimpleCamera((2.0, -3.0, math.sqrt(3.0)), width=width, height=height)
    sc = Scene(pos, scales, quats, dens, sh, [cam],
               MarchParams(dt_step, dynamic_sampling, max_prim_slice, white_background), name="tiny")
    if lobes:
        sc.sph_gauss_features, sc.bandwidth_sharpness, sc.lobe_axis = _sg(n, g, lobes)
    return sc


def object_scene(seed=1, n=300_000, n_cameras=100, width=800, height=800) -> Scene:
    """Object-centric scene of NeRF-Synthetic shape: a clipped normal blob seen
    from the upper hemisphere of radius 4, white background, static sampling."""
    g = torch.Generator().manual_seed(seed)
    pos = (torch.randn(n, 3, generator=g) * 0.5).clamp(-1.5, 1.5)
    scales = torch.exp(torch.randn(n, 3, generator=g) * 0.5 - 4.5)
    quats = _quats(n, g)
    dens = 20.0 * _softplus(torch.randn(n, generator=g))
    sh = _sh(n, g)
    u = torch.rand(n_cameras, generator=g)
    phi = torch.rand(n_cameras, generator=g) * 2 * math.pi
    cams = []
    for ui, pi in zip(u.tolist(), phi.tolist()):
        r = math.sqrt(max(0.0, 1 - ui * ui))
        cams.append(SimpleCamera((4 * r * math.cos(pi), 4 * r * math.sin(pi), 4 * ui), width=width, height=height))
    return Scene(pos, scales, quats, dens, sh, cams, MarchParams(0.0025, False, 2048, True), name="object")


def unbounded_scene(seed=2, n=3_000_000, n_cameras=200, width=1256, height=828) -> Scene:
    """Unbounded scene of Mip-NeRF-360 shape: 80 % of the Gaussians in a unit
    normal core, 20 % large anisotropic ones on a shell of radius 5..50; cameras
    on a ring of radius 3 at height 0.5; black background, dynamic sampling."""
    g = torch.Generator().manual_seed(seed)
    n_core = int(round(n * 0.8))
    n_shell = n - n_core
    pos_core = torch.randn(n_core, 3, generator=g)
    sc_core = torch.exp(torch.randn(n_core, 3, generator=g) * 0.6 - 4.0)
    dirs = torch.randn(n_shell, 3, generator=g)
    dirs = dirs / dirs.norm(dim=1, keepdim=True)
    rad = torch.rand(n_shell, 1, generator=g) * 45.0 + 5.0
    pos_shell = dirs * rad
    # the drawn log-scale is the longest axis; the other two are shorter by a log-uniform factor of up to 10
    base = torch.exp(torch.randn(n_shell, 1, generator=g) * 0.5 - 1.0)
    ratio = torch.exp(torch.rand(n_shell, 3, generator=g) * math.log(10.0))
    sc_shell = base * ratio.min(dim=1, keepdim=True).values / ratio
    pos = torch.cat([pos_core, pos_shell])
    scales = torch.cat([sc_core, sc_shell])
    perm = torch.randperm(n, generator=g)  # no spatial order in the input
    pos, scales = pos[perm].contiguous(), scales[perm].contiguous()
    quats = _quats(n, g)
    dens = 10.0 * _softplus(torch.randn(n, generator=g))
    sh = _sh(n, g)
    fovx = math.radians(60.0)
    fovy = 2 * math.atan(math.tan(fovx / 2) * height / width)
    cams = []
    for i in range(n_cameras):
        a = 2 * math.pi * i / n_cameras
        cams.append(SimpleCamera((3 * math.cos(a), 3 * math.sin(a), 0.5), fovx=fovx, fovy=fovy, width=width,
                                 height=height))
    return Scene(pos, scales, quats, dens, sh, cams, MarchParams(0.005, True, 512, False), name="unbounded")


def stress_scene(seed=4, n_uniform=6_000_000, n_cluster=1_000_000, n_cameras=60, width=1920, height=1080) -> Scene:
    """Forward-only stress scene: uniform fill of [-3,3]^3 plus 64 tight
    clusters, needle-like anisotropy up to 100:1, heavy overlap; transmittance
    threshold 1e-4."""
    g = torch.Generator().manual_seed(seed)
    n = n_uniform + n_cluster
    pos_u = torch.rand(n_uniform, 3, generator=g) * 6 - 3
    centres = torch.rand(64, 3, generator=g) * 6 - 3
    which = torch.randint(0, 64, (n_cluster,), generator=g)
    pos_c = centres[which] + torch.randn(n_cluster, 3, generator=g) * 0.05
    pos = torch.cat([pos_u, pos_c])
    smin = torch.exp(torch.randn(n, 1, generator=g) * 0.5 - 5.0)
    ratio = torch.exp(torch.rand(n, 3, generator=g) * math.log(100.0))
    scales = smin * ratio / ratio.min(dim=1, keepdim=True).values
    perm = torch.randperm(n, generator=g)
    pos, scales = pos[perm].contiguous(), scales[perm].contiguous()
    quats = _quats(n, g)
    dens = 30.0 * _softplus(torch.randn(n, generator=g) + 1.0)
    sh = _sh(n, g)
    fovx = math.radians(50.0)
    fovy = 2 * math.atan(math.tan(fovx / 2) * height / width)
    d = torch.randn(n_cameras, 3, generator=g)
    d = d / d.norm(dim=1, keepdim=True) * 6.0
    cams = [SimpleCamera(tuple(e), fovx=fovx, fovy=fovy, width=width, height=height) for e in d.tolist()]
    return Scene(pos, scales, quats, dens, sh, cams,
                 MarchParams(0.005, True, 512, False, transmittance_eps=1e-4), name="stress")


def l1_target(n_rays, seed=1234):
    """Seeded U[0,1] target image for the benchmark's L1 loss."""
    g = torch.Generator().manual_seed(seed)
    return torch.rand(n_rays, 3, generator=g)
