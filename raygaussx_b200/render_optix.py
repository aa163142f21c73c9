"""Drop-in replacement for the reference's ``optix_raycasting/render_optix.py``.

Same names, same argument order and meaning, same outputs:

* :class:`RenderOptixSettings` -- the settings record (render_optix.py:67-89).
  The OptiX handles it carries (context, acceleration structure, program groups,
  pipelines, ``hit_prim_idx`` scratch) are accepted and ignored: none of them
  exists here.
* :class:`RenderOptixFunction` -- the ``torch.autograd.Function``
  (render_optix.py:92-199): ``apply(positions, scales, normalized_quaternions,
  densities, color_features, sph_gauss_features, bandwidth_sharpness, lobe_axis,
  settings) -> ray_colors [R, 3]``; backward returns the eight gradients and
  ``None`` for the settings.

All device work goes through the C ABI of ``librgx.so`` (``include/rgx.h``) on the
current torch CUDA stream; nothing here computes on the CPU and nothing falls
back if the library is missing.

Additions beyond the reference's surface: :func:`render_full` (RGB, alpha and
expected depth, no gradient) and :class:`Renderer` (explicit control over when
the acceleration structure is rebuilt, row ranges for multi-GPU sharding,
gradient accumulation into caller-owned buffers, work counters).
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Optional, Tuple

import numpy as np
import torch

from . import _lib
from ._lib import Camera as _Camera, Counters, Grads as _Grads, March as _March, Scene as _Scene

# cuda_train/forward/gaussians_aabb.h:5; the reference re-exports it from optix_utils (optix_utils.py:14-33)
SIGMA_THRESHOLD = 0.1
TRANSMITTANCE_EPSILON = 0.001


class RenderOptixSettings:
    """Positional signature of render_optix.py:68-71.  ``transmittance_eps``, ``exact_sh_grad`` and ``rows`` are
    keyword-only additions with the reference's behaviour as default.  ``rows = (first, last + 1)`` restricts
    the render to those image rows (of the supersampled image): the other rays of the returned image are left
    unwritten and take no part in the backward -- how a view is shared between ranks.  ``next_viewpoint_cam``
    (with ``next_rows``) announces the view that will be rendered next with the same, unchanged Gaussians and
    ``reuse_acceleration_structure`` set (or the very same, untouched parameter tensors, which the forward
    recognises by itself): the backward of this view then prepares it beside its own kernels.
    ``accumulate_leaf_grads``: when every differentiable input is a leaf tensor, the backward adds its gradients
    straight into their ``.grad`` (allocated and zeroed on first use) and hands autograd nothing to accumulate --
    one pass over the 59 floats per Gaussian less per view.  Off by default, because hooks registered on those
    leaves (``register_hook``, ``register_post_accumulate_grad_hook``, DistributedDataParallel) do not see
    gradients that bypass autograd's accumulation."""

    def __init__(self, context, update, gas, program_grps_fwd, pipeline_fwd, program_grps_bwd, pipeline_bwd, dt_step,
                 dynamic_sampling, viewpoint_cam, max_prim_slice, num_sph_gauss, iteration=0, jitter=False,
                 rnd_sample=0, supersampling=(1, 1), white_background=False, hit_prim_idx=None, *,
                 transmittance_eps=TRANSMITTANCE_EPSILON, exact_sh_grad=False, rows=None,
                 next_viewpoint_cam=None, next_rows=None, reuse_acceleration_structure=False,
                 accumulate_leaf_grads=False):
        self.context = context
        self.update = update
        self.gas = gas
        self.program_grps_fwd = program_grps_fwd
        self.pipeline_fwd = pipeline_fwd
        self.program_grps_bwd = program_grps_bwd
        self.pipeline_bwd = pipeline_bwd
        self.dt_step = dt_step
        self.dynamic_sampling = dynamic_sampling
        self.viewpoint_cam = viewpoint_cam
        self.max_prim_slice = max_prim_slice
        self.num_sph_gauss = num_sph_gauss
        self.iteration = iteration          # plumbed but unused by the reference's kernels; unused here
        self.jitter = jitter                # likewise
        self.rnd_sample = rnd_sample        # likewise
        self.supersampling = supersampling
        self.white_background = white_background
        self.hit_prim_idx = hit_prim_idx
        self.transmittance_eps = transmittance_eps
        self.exact_sh_grad = exact_sh_grad
        self.rows = rows
        self.next_viewpoint_cam = next_viewpoint_cam
        self.next_rows = next_rows
        self.reuse_acceleration_structure = reuse_acceleration_structure   # the caller vouches: same geometry as the last build
        self.accumulate_leaf_grads = accumulate_leaf_grads


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None or t.numel() == 0 else t.data_ptr()


def _as_input(t: torch.Tensor, name: str) -> torch.Tensor:
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if t.dtype != torch.float32:
        raise ValueError(f"{name} must be float32, got {t.dtype}")
    t = t.detach().contiguous()
    if t.data_ptr() % 16:            # a row slice of a larger buffer: the kernels load 16 bytes at a time (rgx.h)
        t = t.clone()
    return t


def camera_struct(cam, supersampling=(1, 1)) -> _Camera:
    """Launch-parameter fill of optix_utils.py:258-266.  Reads two small tensors
    back from the device (as the reference's ``.get()`` calls do); the result is
    cached on the camera object until those tensors change."""
    key = (cam.world_view_transform._version, cam.camera_center._version, cam.world_view_transform.data_ptr(),
           tuple(supersampling), cam.image_width, cam.image_height, cam.FoVx, cam.FoVy, cam.Px, cam.Py)
    cached = getattr(cam, "_rgx_camera", None)
    if cached is not None and cached[0] == key:
        return cached[1]
    wvt = cam.world_view_transform.detach().to("cpu", torch.float32).numpy()
    eye = cam.camera_center.detach().to("cpu", torch.float32).numpy()
    c = _Camera()
    c.eye[:] = eye.tolist()
    c.u[:] = wvt[:3, 0].tolist()
    c.v[:] = wvt[:3, 1].tolist()
    c.w[:] = wvt[:3, 2].tolist()
    c.tan_half_fov[:] = [math.tan(cam.FoVx / 2), math.tan(cam.FoVy / 2)]
    c.pp[:] = [cam.Px, cam.Py]
    c.width = int(cam.image_width * supersampling[0])
    c.height = int(cam.image_height * supersampling[1])
    try:
        cam._rgx_camera = (key, c)
    except Exception:
        pass
    return c


class Renderer:
    """One rgx context on one CUDA device."""

    def __init__(self, device=None):
        if not torch.cuda.is_available():
            raise RuntimeError("raygaussx_b200 needs a CUDA device; there is no CPU path")
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self._lib = _lib.lib()
        h = C.c_void_p()
        rc = self._lib.rgx_create(self.device.index or 0, C.byref(h))
        if rc != 0:
            raise _lib.RgxError(rc, "rgx_create failed")
        self._ctx = h
        self._n_built = -1
        self._build_serial = 0       # counts the builds of this context
        self._built_from = None      # the four geometry tensors of the latest build, kept alive (see geometry_is_built)

    def __del__(self):
        try:
            if getattr(self, "_ctx", None):
                self._lib.rgx_destroy(self._ctx)
                self._ctx = None
        except Exception:
            pass

    # -- helpers
    def _stream(self):
        return C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    @staticmethod
    def _scene(positions, scales, quaternions, densities, color_features=None, sg_features=None, sharpness=None,
               lobe_axis=None) -> _Scene:
        s = _Scene()
        s.n = positions.shape[0]
        s.positions, s.scales, s.quaternions, s.densities = (_ptr(positions), _ptr(scales), _ptr(quaternions),
                                                             _ptr(densities))
        if color_features is not None:
            s.sh_coeffs = color_features.shape[2]
            s.color_features = _ptr(color_features)
            g = 0 if sharpness is None else (sharpness.shape[1] if sharpness.dim() == 2 else 0)
            s.num_lobes = g
            if g:
                s.sg_features, s.sharpness, s.lobe_axis = _ptr(sg_features), _ptr(sharpness), _ptr(lobe_axis)
        else:
            s.sh_coeffs = 1
        return s

    @staticmethod
    def _march(dt_step, dynamic_sampling, max_prim_slice, white_background, transmittance_eps, rows, height,
               flags) -> _March:
        m = _March()
        m.dt_step = float(dt_step)
        m.dynamic_sampling = 1 if dynamic_sampling else 0
        m.max_prim_slice = int(max_prim_slice)
        m.white_background = 1 if white_background else 0
        m.transmittance_eps = float(transmittance_eps)
        m.row_begin, m.row_end = (0, height) if rows is None else (int(rows[0]), int(rows[1]))
        m.flags = int(flags)
        return m

    # -- API
    def build(self, positions, scales, quaternions, densities, sigma_threshold=SIGMA_THRESHOLD, morton_bits=10,
              curve=_lib.CURVE_HILBERT):
        """Boxes, Morton sort and hierarchy refit for the current parameters
        (replaces ellipsoids_bbox_from_quat + create_acceleration_structure)."""
        positions, scales, quaternions, densities = (_as_input(positions, "positions"), _as_input(scales, "scales"),
                                                     _as_input(quaternions, "quaternions"),
                                                     _as_input(densities, "densities"))
        sc = self._scene(positions, scales, quaternions, densities)
        _lib.check(self._ctx, self._lib.rgx_build(self._ctx, C.byref(sc), float(sigma_threshold), int(morton_bits),
                                                  int(curve), self._stream()))
        self._n_built = positions.shape[0]
        self._build_serial += 1
        tensors = (positions, scales, quaternions, densities)
        self._built_from = (tensors, tuple((t.data_ptr(), t._version, tuple(t.shape)) for t in tensors))

    def geometry_is_built(self, positions, scales, quaternions, densities) -> bool:
        """True when the latest build was made from these very tensors and none of them has been written to
        since: same storage, same shape, same version counter.  The build keeps its tensors alive, so an equal
        address cannot belong to a new tensor that merely landed in recycled memory.  (Tensors recomputed from
        unchanged parameters -- ``exp`` of the log-scales, say -- are new tensors and count as changed; writes
        through ``tensor.data`` bypass the version counter here as they do for autograd.)"""
        if self._built_from is None:
            return False
        return self._built_from[1] == tuple((t.data_ptr(), t._version, tuple(t.shape))
                                            for t in (positions, scales, quaternions, densities))

    def forward(self, positions, scales, quaternions, densities, color_features, sg_features, sharpness, lobe_axis,
                cam: _Camera, march: _March, want_alpha=False, want_depth=False, out=None):
        """March rows ``[march.row_begin, march.row_end)``; returns ``(rgb, alpha, depth)``."""
        r = cam.width * cam.height
        rgb = out if out is not None else torch.empty(r, 3, device=self.device, dtype=torch.float32)
        alpha = torch.empty(r, device=self.device, dtype=torch.float32) if want_alpha else None
        depth = torch.empty(r, device=self.device, dtype=torch.float32) if want_depth else None
        sc = self._scene(positions, scales, quaternions, densities, color_features, sg_features, sharpness, lobe_axis)
        _lib.check(self._ctx, self._lib.rgx_forward(self._ctx, C.byref(sc), C.byref(cam), C.byref(march),
                                                    _ptr(rgb), _ptr(alpha), _ptr(depth), self._stream()))
        return rgb, alpha, depth

    def forward_frame(self, positions, scales, quaternions, densities, color_features, sg_features, sharpness,
                      lobe_axis, cam: _Camera, march: _March, want_depth=True):
        """The viewer's outputs (cuda_gui/gaussians_aabb.cu:205-342) into plain device
        buffers: ``(frame [H, W, 4] uint8, depth [H, W] float32 or None)``."""
        frame = torch.empty(cam.height, cam.width, 4, device=self.device, dtype=torch.uint8)
        depth = torch.empty(cam.height, cam.width, device=self.device, dtype=torch.float32) if want_depth else None
        sc = self._scene(positions, scales, quaternions, densities, color_features, sg_features, sharpness, lobe_axis)
        _lib.check(self._ctx, self._lib.rgx_forward_frame(self._ctx, C.byref(sc), C.byref(cam), C.byref(march),
                                                          _ptr(frame), _ptr(depth), self._stream()))
        return frame, depth

    def backward(self, positions, scales, quaternions, densities, color_features, sg_features, sharpness, lobe_axis,
                 cam: _Camera, march: _March, rgb, dl_drgb, grads: Tuple[torch.Tensor, ...]):
        """``grads`` = (positions, scales, quaternions, densities, color_features[, sg, sharpness, axis])
        gradient tensors to overwrite (or add to, with FLAG_ACCUMULATE in ``march.flags``)."""
        sc = self._scene(positions, scales, quaternions, densities, color_features, sg_features, sharpness, lobe_axis)
        g = _Grads()
        g.positions, g.scales, g.quaternions, g.densities, g.color_features = (_ptr(t) for t in grads[:5])
        if sc.num_lobes:
            g.sg_features, g.sharpness, g.lobe_axis = (_ptr(t) for t in grads[5:8])
        _lib.check(self._ctx, self._lib.rgx_backward(self._ctx, C.byref(sc), C.byref(cam), C.byref(march), _ptr(rgb),
                                                     _ptr(dl_drgb), C.byref(g), self._stream()))

    def hint_next_view(self, cam: Optional[_Camera], march: Optional[_March]):
        """Announce the view of the next forward: the next :meth:`backward` then makes its tile lists beside its own
        kernels.  ``None, None`` withdraws the announcement."""
        _lib.check(self._ctx, self._lib.rgx_hint_next_view(self._ctx, C.byref(cam) if cam is not None else None,
                                                           C.byref(march) if march is not None else None))

    def near_lists(self, budget_per_ray: int = -1, min_pairs: int = -1) -> dict:
        """Lists up to a horizon for recording forwards (``rgx_debug_near_lists``): sets the budget of pairs per ray
        (0 switches the feature off, negative leaves it) and the number of pairs below which a view gets complete
        lists anyway (negative leaves it), and returns the figures since the last call."""
        _lib.check(self._ctx, self._lib.rgx_debug_near_lists(self._ctx, int(budget_per_ray), int(min_pairs)))
        out = (C.c_longlong * 4)()
        _lib.check(self._ctx, self._lib.rgx_read_near_lists(self._ctx, out))
        return dict(views=out[0], pairs_estimated=out[1], pairs_kept=out[2], views_with_rays_beyond=out[3])

    def lists_made_ahead(self) -> int:
        return int(self._lib.rgx_lists_made_ahead(self._ctx))

    def gaussian_colors(self, positions, color_features, sg_features, sharpness, lobe_axis, eye):
        n = positions.shape[0]
        out = torch.empty(n, 3, device=self.device, dtype=torch.float32)
        sc = self._scene(positions, positions, positions, positions, color_features, sg_features, sharpness, lobe_axis)
        e = (C.c_float * 3)(*[float(v) for v in eye])
        _lib.check(self._ctx, self._lib.rgx_gaussian_colors(self._ctx, C.byref(sc), e, _ptr(out), self._stream()))
        return out

    def scene_box(self):
        lo, hi = (C.c_float * 3)(), (C.c_float * 3)()
        _lib.check(self._ctx, self._lib.rgx_scene_box(self._ctx, lo, hi, self._stream()))
        return np.array(lo[:], dtype=np.float32), np.array(hi[:], dtype=np.float32)

    def reset_counters(self):
        _lib.check(self._ctx, self._lib.rgx_reset_counters(self._ctx, self._stream()))

    def read_counters(self) -> dict:
        c = Counters()
        _lib.check(self._ctx, self._lib.rgx_read_counters(self._ctx, C.byref(c), self._stream()))
        return c.as_dict()

    def set_profiling(self, enable: bool):
        """Bracket every march kernel with CUDA events (see :meth:`read_kernel_times`)."""
        _lib.check(self._ctx, self._lib.rgx_set_profiling(self._ctx, 1 if enable else 0))

    def read_kernel_times(self) -> dict:
        """Summed march-kernel durations (ms) and launch counts since the last read."""
        f, b = C.c_float(), C.c_float()
        nf, nb = C.c_int(), C.c_int()
        _lib.check(self._ctx, self._lib.rgx_read_kernel_times(self._ctx, C.byref(f), C.byref(nf), C.byref(b),
                                                              C.byref(nb)))
        return dict(forward_ms=f.value, forward_launches=nf.value, backward_ms=b.value, backward_launches=nb.value)

    def read_binning(self) -> dict:
        """Tile-list construction: summed ms and runs since the last read (profiling on), pairs of the latest view."""
        ms, runs, pairs = C.c_float(), C.c_int(), C.c_longlong()
        _lib.check(self._ctx, self._lib.rgx_read_binning(self._ctx, C.byref(ms), C.byref(runs), C.byref(pairs)))
        return dict(ms=ms.value, runs=runs.value, pairs=pairs.value)

    def workspace_bytes(self) -> int:
        return int(self._lib.rgx_workspace_bytes(self._ctx))


_renderers = {}


def get_renderer(device=None) -> Renderer:
    """The process-wide renderer of a device (created on first use)."""
    idx = torch.cuda.current_device() if device is None else (torch.device(device).index or 0)
    if idx not in _renderers:
        _renderers[idx] = Renderer(torch.device("cuda", idx))
    return _renderers[idx]


def _settings_march(settings, cam: _Camera, flags=0, rows=None) -> _March:
    return Renderer._march(settings.dt_step, settings.dynamic_sampling, settings.max_prim_slice,
                           settings.white_background, getattr(settings, "transmittance_eps", TRANSMITTANCE_EPSILON),
                           rows, cam.height, flags)


class RenderOptixFunction(torch.autograd.Function):
    """The reference's autograd entry point (render_optix.py:92-199)."""

    @staticmethod
    def forward(ctx, positions, scales, normalized_quaternions, densities, color_features, sph_gauss_features,
                bandwidth_sharpness, lobe_axis, settings):
        tensors = [_as_input(t, n) for t, n in zip(
            (positions, scales, normalized_quaternions, densities, color_features, sph_gauss_features,
             bandwidth_sharpness, lobe_axis),
            ("positions", "scales", "normalized_quaternions", "densities", "color_features", "sph_gauss_features",
             "bandwidth_sharpness", "lobe_axis"))]
        r = get_renderer(positions.device)
        cam = camera_struct(settings.viewpoint_cam, settings.supersampling)
        # The reference rebuilds its acceleration structure in every forward
        # (scripts/train.py:117 passes update=False; update=True refits).  Same here,
        # unless the geometry tensors are the very ones of the latest build, untouched
        # since, or the caller vouches that their values are unchanged.
        vouched = getattr(settings, "reuse_acceleration_structure", False) and r._n_built == tensors[0].shape[0]
        if not (vouched or r.geometry_is_built(*tensors[:4])):
            r.build(*tensors[:4], sigma_threshold=SIGMA_THRESHOLD,
                    morton_bits=getattr(settings, "morton_bits", 10))
        # keep what the rays met, so that the backward of this view does not have to search again
        march = _settings_march(settings, cam, flags=_lib.FLAG_SAVE_HITS, rows=getattr(settings, "rows", None))
        rgb, _, _ = r.forward(*tensors, cam, march)
        ctx.settings = settings
        ctx.build_serial = r._build_serial
        ctx.leaves = None
        if getattr(settings, "accumulate_leaf_grads", False):
            given = (positions, scales, normalized_quaternions, densities, color_features, sph_gauss_features,
                     bandwidth_sharpness, lobe_axis)
            wanted = [g for g in given if g.requires_grad]
            if all(g.requires_grad for g in given[:5]) and all(
                    g.is_leaf and g.is_cuda and g.dtype == torch.float32 and g.is_contiguous()
                    and g.data_ptr() % 16 == 0 for g in wanted):
                ctx.leaves = given
        ctx.save_for_backward(*tensors, rgb)
        return rgb

    @staticmethod
    def backward(ctx, dloss_dray_colors):
        settings = ctx.settings
        *tensors, rgb = ctx.saved_tensors
        dl = dloss_dray_colors.contiguous().to(torch.float32)
        r = get_renderer(rgb.device)
        cam = camera_struct(settings.viewpoint_cam, settings.supersampling)
        flags = _lib.FLAG_EXACT_SH_GRAD if getattr(settings, "exact_sh_grad", False) else 0
        march = _settings_march(settings, cam, flags=flags, rows=getattr(settings, "rows", None))
        leaves = ctx.leaves
        if leaves is not None:
            targets = [t for t in leaves if t.requires_grad]       # the first five, and the lobe tensors that ask
            for t in targets:
                if t.grad is None:
                    t.grad = torch.zeros_like(t, memory_format=torch.contiguous_format)
            if not all(t.grad.is_contiguous() and t.grad.dtype == torch.float32 and t.grad.data_ptr() % 16 == 0
                       for t in targets):
                leaves = None
        if leaves is not None:
            # lobe tensors that ask for no gradient still need somewhere for it to go
            grads = [t.grad if t.requires_grad else torch.zeros_like(s) for t, s in zip(leaves, tensors)]
            flags |= _lib.FLAG_ACCUMULATE
            march = _settings_march(settings, cam, flags=flags, rows=getattr(settings, "rows", None))
        else:
            grads = [torch.empty_like(t) for t in tensors]
        if r._build_serial != ctx.build_serial:
            # another build came between this view's forward and its backward (a second model, an evaluation copy,
            # a finite-difference probe): the backward reads the geometry of the latest build, so build again from
            # the tensors this forward saw.  The forward's recording belonged to the old build: the rays are searched.
            r.build(*tensors[:4], sigma_threshold=SIGMA_THRESHOLD, morton_bits=getattr(settings, "morton_bits", 10))
        nxt = getattr(settings, "next_viewpoint_cam", None)      # same Gaussians, next view of an accumulation step
        if nxt is not None:
            ncam = camera_struct(nxt, settings.supersampling)
            r.hint_next_view(ncam, _settings_march(settings, ncam, flags=_lib.FLAG_SAVE_HITS,
                                                   rows=getattr(settings, "next_rows", None)))
        r.backward(*tensors, cam, march, rgb, dl, tuple(grads))
        if leaves is not None:            # already in the leaves' .grad: nothing for autograd to accumulate
            return (None,) * 9
        g_pos, g_scale, g_quat, g_dens, g_sh, g_sg, g_sharp, g_axis = grads
        if settings.num_sph_gauss == 0 or tensors[6].numel() == 0:       # render_optix.py:190-197
            g_sg = g_sharp = g_axis = None
        return g_pos, g_scale, g_quat, g_dens, g_sh, g_sg, g_sharp, g_axis, None


def render_full(positions, scales, normalized_quaternions, densities, color_features, sph_gauss_features,
                bandwidth_sharpness, lobe_axis, settings, rebuild=True):
    """Forward only: ``(rgb [R,3], alpha [R], depth [R])``.  alpha is one minus the
    final transmittance, depth the transmittance-weighted sample distance of the
    reference's viewer kernel (cuda_gui/gaussians_aabb.cu:189-202).  No gradients:
    the reference defines none for alpha or depth."""
    with torch.no_grad():
        tensors = [_as_input(t, "input") for t in (positions, scales, normalized_quaternions, densities,
                                                   color_features, sph_gauss_features, bandwidth_sharpness, lobe_axis)]
        r = get_renderer(positions.device)
        cam = camera_struct(settings.viewpoint_cam, settings.supersampling)
        if rebuild or r._n_built != tensors[0].shape[0]:
            r.build(*tensors[:4], sigma_threshold=SIGMA_THRESHOLD, morton_bits=getattr(settings, "morton_bits", 10))
        return r.forward(*tensors, cam, _settings_march(settings, cam), want_alpha=True, want_depth=True)
