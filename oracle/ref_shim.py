"""TEST INFRASTRUCTURE ONLY -- never imported by the shipped package.

Python side of ``oracle/_ref``: runs the reference's own device sources
(compiled for the CPU by ``oracle/Makefile`` with an exhaustive-search stand-in
for OptiX traversal) through the same sequence of steps as the reference's
``RenderOptixFunction`` (optix_raycasting/render_optix.py:92-199).

What is the reference's code and what is restated here:

* device programs (ray generation, ellipsoid intersection, any-hit gather, slab
  march, compositing, backward, SH colour and its gradient): the reference's
  ``.cu`` files, compiled unmodified from where they lie;
* host-side array preparation, which the reference does with cupy expressions:
  restated below with the same expressions in numpy float32 --
  ``ellipsoids_bbox`` follows optix_utils.py:36-109, ``pack_prims`` follows
  optix_utils.py:268-304, ``reduce_replicas`` follows optix_utils.py:325-361;
* OptiX traversal: replaced (see optix_shim/optix.h).

All arithmetic is fp32, like the reference.
"""
from __future__ import annotations

import ctypes
import math
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_REF_DIR = os.path.join(_HERE, "_ref")
SIGMA_THRESHOLD = 0.1  # cuda_train/forward/gaussians_aabb.h:5
_libs = {}


def available() -> bool:
    return all(os.path.exists(os.path.join(_REF_DIR, f"libref_{s}.so")) for s in ("forward", "backward", "sh"))


def _lib(stage):
    if stage not in _libs:
        _libs[stage] = ctypes.CDLL(os.path.join(_REF_DIR, f"libref_{stage}.so"))
    return _libs[stage]


def _f32(a):
    return np.ascontiguousarray(np.asarray(a, dtype=np.float32))


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def ellipsoids_bbox(quaternions, centers, scales, densities):
    """optix_utils.py:36-109 (elementwise kernel + min/max reductions)."""
    q, c, s, d = _f32(quaternions), _f32(centers), _f32(scales), _f32(densities)
    f = np.float32
    with np.errstate(all="ignore"):
        t = d / f(SIGMA_THRESHOLD)
        dd = np.log(t * t)
        dd = np.where(dd > 0, dd, f(0)).astype(np.float32)
        dd = np.sqrt(dd)
        W, X, Y, Z = q[:, 0], q[:, 1], q[:, 2], q[:, 3]
        n = W * W + X * X + Y * Y + Z * Z
        invn = (f(1) / np.sqrt(n + f(1e-20))).astype(np.float32)
        W, X, Y, Z = W * invn, X * invn, Y * invn, Z * invn
        L1 = (f(1) - f(2) * (Y * Y + Z * Z), f(2) * (X * Y - W * Z), f(2) * (X * Z + W * Y))
        L2 = (f(2) * (X * Y + W * Z), f(1) - f(2) * (X * X + Z * Z), f(2) * (Y * Z - W * X))
        L3 = (f(2) * (X * Z - W * Y), f(2) * (Y * Z + W * X), f(1) - f(2) * (X * X + Y * Y))
        s0, s1, s2 = s[:, 0], s[:, 1], s[:, 2]
        h = [dd * np.sqrt((s0 * L[0]) ** 2 + (s1 * L[1]) ** 2 + (s2 * L[2]) ** 2) for L in (L1, L2, L3)]
    lo = np.stack([c[:, i] - h[i] for i in range(3)], axis=1).astype(np.float32)
    hi = np.stack([c[:, i] + h[i] for i in range(3)], axis=1).astype(np.float32)
    return np.concatenate([lo, hi], axis=1), lo.min(axis=0), hi.max(axis=0)


def pack_prims(camera_center, positions, scales, quaternions, densities, rgb):
    """optix_utils.py:268-304: the 64-byte PrimData records."""
    pos, s, q, d, rgb = _f32(positions), _f32(scales), _f32(quaternions), _f32(densities), _f32(rgb)
    cam = _f32(camera_center)
    n = pos.shape[0]
    prims = np.empty((n, 16), dtype=np.float32)
    with np.errstate(all="ignore"):
        prims[:, 0:3] = cam[None, :] - pos
        prims[:, 3] = 0
        k = np.sqrt(np.float32(2.0) * np.log(d / np.float32(SIGMA_THRESHOLD))).astype(np.float32)
        prims[:, 4:7] = (np.float32(1) / s) / k[:, None]
        prims[:, 7] = k
        prims[:, 8:12] = q
        prims[:, 12:15] = rgb * d[:, None]
        prims[:, 15] = d
    return prims


def reduce_replicas(a, n):
    """optix_utils.py:325-361: sum the 4 gradient replicas (index = prim*4 + replica)."""
    return a.reshape(n, 4, -1).sum(axis=1)


def _camera_args(camera, supersampling=(1, 1)):
    wvt = np.asarray(camera.world_view_transform.detach().cpu().numpy(), dtype=np.float32)
    eye = _f32(camera.camera_center.detach().cpu().numpy())
    u, v, w = _f32(wvt[:3, 0]), _f32(wvt[:3, 1]), _f32(wvt[:3, 2])
    intr = np.array([math.tan(camera.FoVx / 2), math.tan(camera.FoVy / 2), camera.Px, camera.Py], dtype=np.float32)
    return eye, u, v, w, intr, camera.image_width * supersampling[0], camera.image_height * supersampling[1]


def sh_forward(camera_center, positions, color_features, sg_features, sharpness, lobe_axis, sh_degree):
    """utils/sh_utils.cu:122-216 via render_optix.py:19-32."""
    pos, sh = _f32(positions), _f32(color_features).reshape(-1)
    n = pos.shape[0]
    g = int(np.asarray(sharpness).reshape(n, -1).shape[1]) if n else 0
    sgf, shp, ax = _f32(sg_features).reshape(-1), _f32(sharpness).reshape(-1), _f32(lobe_axis).reshape(-1)
    cam = _f32(camera_center)
    rgb = np.zeros((n, 3), dtype=np.float32)
    _lib("sh").ref_forward_sh(_p(cam), _p(pos), _p(sh), _p(sgf), _p(shp), _p(ax), g, int(sh_degree), n, _p(rgb))
    return rgb


def sh_backward(camera_center, positions, color_features, sg_features, sharpness, lobe_axis, sh_degree, dL_drgb):
    """utils/sh_utils.cu:218-412 via render_optix.py:34-52."""
    pos, sh = _f32(positions), _f32(color_features).reshape(-1)
    n = pos.shape[0]
    g = int(np.asarray(sharpness).reshape(n, -1).shape[1]) if n else 0
    sgf, shp, ax = _f32(sg_features).reshape(-1), _f32(sharpness).reshape(-1), _f32(lobe_axis).reshape(-1)
    cam, dl = _f32(camera_center), _f32(dL_drgb)
    ksh = (sh_degree + 1) ** 2
    d_sh = np.zeros(n * 3 * ksh, dtype=np.float32)
    d_pos = np.zeros((n, 3), dtype=np.float32)
    d_sg = np.zeros(n * g * 3 + 1, dtype=np.float32)
    d_shp = np.zeros(n * g + 1, dtype=np.float32)
    d_ax = np.zeros(n * g * 3 + 1, dtype=np.float32)
    _lib("sh").ref_backward_sh(_p(cam), _p(pos), _p(sh), _p(sgf), _p(shp), _p(ax), g, int(sh_degree), n, _p(dl),
                               _p(d_sh), _p(d_pos), _p(d_sg), _p(d_shp), _p(d_ax))
    return (d_sh.reshape(n, 3, ksh), d_pos, d_sg[:-1].reshape(n, 3, g), d_shp[:-1].reshape(n, g),
            d_ax[:-1].reshape(n, g, 3))


def _march_args(prims, n, bb_min, bb_max, march, cam_args):
    eye, u, v, w, intr, width, height = cam_args
    return [_p(prims), n, _p(bb_min), _p(bb_max), ctypes.c_float(march.dt_step), int(bool(march.dynamic_sampling)),
            int(width), int(height), _p(eye), _p(u), _p(v), _p(w), _p(intr), int(march.max_prim_slice)]


def render_forward(positions, scales, quaternions, densities, color_features, sg_features, sharpness, lobe_axis,
                   camera, march, supersampling=(1, 1), prefilter=True, n_threads=0):
    """The forward of render_optix.py:92-141.  Returns ``(ray_colors [R,3], rgb [N,3], ctx)``."""
    to_np = lambda t: t.detach().cpu().numpy() if hasattr(t, "detach") else np.asarray(t)
    pos, s, q, d = (_f32(to_np(x)) for x in (positions, scales, quaternions, densities))
    cf = _f32(to_np(color_features))
    n = pos.shape[0]
    _, bb_min, bb_max = ellipsoids_bbox(q, pos, s, d)
    degree = int(math.sqrt(cf.shape[2]) - 1)
    cam_args = _camera_args(camera, supersampling)
    rgb = sh_forward(cam_args[0], pos, cf, to_np(sg_features), to_np(sharpness), to_np(lobe_axis), degree)
    prims = pack_prims(cam_args[0], pos, s, q, d, rgb)
    width, height = cam_args[5], cam_args[6]
    r = width * height
    hit = np.zeros(r * march.max_prim_slice, dtype=np.int32)
    colors = np.zeros((r, 3), dtype=np.float32)
    stats = np.zeros(3, dtype=np.uint64)
    args = _march_args(prims, n, bb_min, bb_max, march, cam_args)
    _lib("forward").ref_forward(*args, int(bool(march.white_background)), _p(hit), _p(colors), int(prefilter),
                                int(n_threads), _p(stats))
    ctx = dict(pos=pos, s=s, q=q, d=d, cf=cf, sg=to_np(sg_features), shp=to_np(sharpness), ax=to_np(lobe_axis),
               degree=degree, rgb=rgb, prims=prims, bb_min=bb_min, bb_max=bb_max, cam_args=cam_args, hit=hit,
               colors=colors, march=march, stats=stats)
    return colors, rgb, ctx


def render_backward(ctx, dloss_dray_colors, prefilter=True, n_threads=0):
    """The backward of render_optix.py:144-199.  Returns the eight gradients in the
    order the reference returns them: positions, scales, quaternions, densities,
    color_features, sph_gauss_features, bandwidth_sharpness, lobe_axis (the last
    three ``None`` without lobes)."""
    n = ctx["pos"].shape[0]
    march = ctx["march"]
    dl = _f32(dloss_dray_colors.detach().cpu().numpy() if hasattr(dloss_dray_colors, "detach") else dloss_dray_colors)
    g_d = np.zeros(4 * n, dtype=np.float32)
    g_c = np.zeros((4 * n, 3), dtype=np.float32)
    g_p = np.zeros((4 * n, 3), dtype=np.float32)
    g_s = np.zeros((4 * n, 3), dtype=np.float32)
    g_q = np.zeros((4 * n, 4), dtype=np.float32)
    colors = ctx["colors"].copy()
    stats = np.zeros(3, dtype=np.uint64)
    args = _march_args(ctx["prims"], n, ctx["bb_min"], ctx["bb_max"], march, ctx["cam_args"])
    _lib("backward").ref_backward(*args, _p(ctx["hit"]), _p(colors), _p(dl), _p(g_d), _p(g_c), _p(g_p), _p(g_s),
                                  _p(g_q), int(prefilter), int(n_threads), _p(stats))
    d_dens = reduce_replicas(g_d, n)[:, 0]
    d_rgb = reduce_replicas(g_c, n)
    d_pos = reduce_replicas(g_p, n)
    d_scale = reduce_replicas(g_s, n)
    d_quat = reduce_replicas(g_q, n)
    d_sh, d_pos_dir, d_sg, d_shp, d_ax = sh_backward(ctx["cam_args"][0], ctx["pos"], ctx["cf"], ctx["sg"], ctx["shp"],
                                                     ctx["ax"], ctx["degree"], d_rgb)
    d_pos = d_pos + d_pos_dir
    if d_shp.shape[1] == 0:
        d_sg = d_shp = d_ax = None
    return d_pos, d_scale, d_quat, d_dens, d_sh, d_sg, d_shp, d_ax, dict(d_rgb=d_rgb, stats=stats)
