"""TEST INFRASTRUCTURE ONLY -- the parity oracle.  Never imported by the shipped
package; only tests, the smoke check and the benchmark's CPU-baseline leg use it.

A float64 torch-CPU restatement of the reference's differentiable Gaussian
ray-marching operator (``optix_raycasting/render_optix.py:92-199``).  OptiX
traversal is restated as brute force: a trace over ``[tmin, tmax]`` visits every
Gaussian and keeps those whose intersection test passes.

Pinning: the reference ships no tests or golden vectors for this path.  The
oracle is pinned instead against the reference's own device sources compiled for
the CPU (``oracle/_ref``, see ``oracle/Makefile``; traversal replaced by an
exhaustive loop): ``tests/test_oracle.py`` compares the two live on seeded scenes wherever that build is
present, ``tests/golden/`` holds outputs of that build (small cases in full; a few hundred rays each of the
300 k, 3 M and 7 M scenes), and ``tests/golden/knn.npz`` holds the output of the reference's own
nearest-neighbour extension for :func:`knn_mean_dist2`.

Each function cites the reference lines it follows:

* ray generation           cuda_train/forward/gaussians_aabb.cu:95-110
* ray/ellipsoid interval   cuda_train/forward/gaussians_aabb.cu:36-92
* per-Gaussian AABB        optix_utils.py:36-109
* primitive records        optix_utils.py:268-304
* forward march            cuda_train/forward/gaussians_aabb.cu:112-340
* expected depth           cuda_gui/gaussians_aabb.cu:189-202
* backward march           cuda_train/backward/gaussians_aabb.cu:113-497
* SH / SG colour           utils/sh_utils.cu:122-216, gradient :218-412

Where the reference's forward and backward disagree (scene-box clip by
multiplication vs division, clamped vs unclamped slab interval, state after a
slab cut short) the forward's behaviour is used for both; in exact arithmetic
the two give the same hit sets because every ellipsoid lies inside the scene box.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional

import torch

F64 = torch.float64
BUFFER_SIZE = 32   # cuda_train/forward/gaussians_aabb.h:2
CHUNK_SIZE = 16    # :3

# utils/sh_utils.cu:6-23
C0 = 0.28209479177387814
C1 = 0.4886025119029199
C2 = (1.0925484305920792, -1.0925484305920792, 0.31539156525252005, -1.0925484305920792, 0.5462742152960396)
C3 = (-0.5900435899266435, 2.890611442640554, -0.4570457994644658, 0.3731763325901154, -0.4570457994644658,
      1.445305721320277, -0.5900435899266435)


# --------------------------------------------------------------------------- colour
def sh_basis(dirs: torch.Tensor, degree: int) -> torch.Tensor:
    """Real SH basis values ``[N, (degree+1)^2]`` with the reference's signs
    (utils/sh_utils.cu:157-209)."""
    x, y, z = dirs[:, 0], dirs[:, 1], dirs[:, 2]
    out = [torch.full_like(x, C0)]
    if degree > 0:
        out += [-C1 * y, C1 * z, -C1 * x]
    if degree > 1:
        xx, yy, zz, xy, yz, xz = x * x, y * y, z * z, x * y, y * z, x * z
        out += [C2[0] * xy, C2[1] * yz, C2[2] * (2.0 * zz - xx - yy), C2[3] * xz, C2[4] * (xx - yy)]
    if degree > 2:
        out += [C3[0] * y * (3.0 * xx - yy), C3[1] * xy * z, C3[2] * y * (4.0 * zz - xx - yy),
                C3[3] * z * (2.0 * zz - 3.0 * xx - 3.0 * yy), C3[4] * x * (4.0 * zz - xx - yy),
                C3[5] * z * (xx - yy), C3[6] * x * (xx - 3.0 * yy)]
    return torch.stack(out, dim=1)


def sh_basis_grad(dirs: torch.Tensor, degree: int, reference_quirk: bool) -> torch.Tensor:
    """d(basis_k)/d(dir) as ``[N, K, 3]`` (utils/sh_utils.cu:271-376).  With
    ``reference_quirk`` the y-derivative of basis 9 is ``C3[0]*(3x^2 - y^2)`` as
    coded at :367 instead of the exact ``3*C3[0]*(x^2 - y^2)``."""
    x, y, z = dirs[:, 0], dirs[:, 1], dirs[:, 2]
    o = torch.zeros_like(x)
    rows = [(o, o, o)]
    if degree > 0:
        c = torch.full_like(x, C1)
        rows += [(o, -c, o), (o, o, c), (-c, o, o)]
    if degree > 1:
        rows += [(C2[0] * y, C2[0] * x, o), (o, C2[1] * z, C2[1] * y),
                 (-2.0 * C2[2] * x, -2.0 * C2[2] * y, 4.0 * C2[2] * z), (C2[3] * z, o, C2[3] * x),
                 (2.0 * C2[4] * x, -2.0 * C2[4] * y, o)]
    if degree > 2:
        xx, yy, zz, xy, yz, xz = x * x, y * y, z * z, x * y, y * z, x * z
        d9y = C3[0] * (3.0 * xx - yy) if reference_quirk else 3.0 * C3[0] * (xx - yy)
        rows += [(6.0 * C3[0] * xy, d9y, o),
                 (C3[1] * yz, C3[1] * xz, C3[1] * xy),
                 (-2.0 * C3[2] * xy, C3[2] * (4.0 * zz - xx - 3.0 * yy), 8.0 * C3[2] * yz),
                 (-6.0 * C3[3] * xz, -6.0 * C3[3] * yz, 3.0 * C3[3] * (2.0 * zz - xx - yy)),
                 (C3[4] * (4.0 * zz - 3.0 * xx - yy), -2.0 * C3[4] * xy, 8.0 * C3[4] * xz),
                 (2.0 * C3[5] * xz, -2.0 * C3[5] * yz, C3[5] * (xx - yy)),
                 (3.0 * C3[6] * (xx - yy), -6.0 * C3[6] * xy, o)]
    return torch.stack([torch.stack(r, dim=1) for r in rows], dim=1)


def gaussian_rgb(cam_center, positions, color_features, sg_features, sharpness, lobe_axis):
    """Per-Gaussian view-dependent colour, ``0.5 + SH(dir) + lobes`` without
    clamping (utils/sh_utils.cu:122-216).  Differentiable torch."""
    v = positions - cam_center[None, :]
    dirs = v / v.norm(dim=1, keepdim=True)
    degree = int(round(math.sqrt(color_features.shape[2]))) - 1
    basis = sh_basis(dirs, degree)                                 # [N,K]
    rgb = (color_features * basis[:, None, :]).sum(dim=2) + 0.5
    if sharpness.shape[1] > 0:
        cosang = (dirs[:, None, :] * lobe_axis).sum(dim=2)         # [N,G]
        lobe = torch.exp(sharpness * (cosang - 1.0))
        rgb = rgb + (sg_features * lobe[:, None, :]).sum(dim=2)
    return rgb


def gaussian_rgb_backward(cam_center, positions, color_features, sg_features, sharpness, lobe_axis, dL_drgb,
                          reference_quirk=True):
    """Explicit gradient of :func:`gaussian_rgb` (utils/sh_utils.cu:218-412):
    returns ``dL/dSH [N,3,K]``, ``dL/dpos [N,3]`` (through the view direction),
    ``dL/dsg [N,3,G]``, ``dL/dsharpness [N,G]``, ``dL/daxis [N,G,3]``.  Rows whose
    ``dL/drgb`` is exactly zero stay zero (:226-228)."""
    v = positions - cam_center[None, :]
    r2 = (v * v).sum(dim=1, keepdim=True)
    dirs = v / r2.sqrt()
    degree = int(round(math.sqrt(color_features.shape[2]))) - 1
    basis = sh_basis(dirs, degree)
    d_sh = dL_drgb[:, :, None] * basis[:, None, :]
    dbasis = sh_basis_grad(dirs, degree, reference_quirk)          # [N,K,3]
    drgb_ddir = torch.einsum("nck,nkj->ncj", color_features, dbasis)
    dL_ddir = torch.einsum("nc,ncj->nj", dL_drgb, drgb_ddir)
    d_sg = torch.zeros_like(sg_features)
    d_sharp = torch.zeros_like(sharpness)
    d_axis = torch.zeros_like(lobe_axis)
    if sharpness.shape[1] > 0:
        cosm1 = (dirs[:, None, :] * lobe_axis).sum(dim=2) - 1.0
        lobe = torch.exp(sharpness * cosm1)
        d_sg = dL_drgb[:, :, None] * lobe[:, None, :]
        dl_dlobe = torch.einsum("nc,ncg->ng", dL_drgb, sg_features)
        d_axis = (dl_dlobe * sharpness * lobe)[:, :, None] * dirs[:, None, :]
        d_sharp = dl_dlobe * cosm1 * lobe
        dL_ddir = dL_ddir + ((dl_dlobe * sharpness * lobe)[:, :, None] * lobe_axis).sum(dim=1)
    # normalisation Jacobian (|v|^2 I - v v^T) / |v|^3   (:406-410)
    d_pos = (r2 * dL_ddir - v * (v * dL_ddir).sum(dim=1, keepdim=True)) / (r2 * r2.sqrt())
    zero = (dL_drgb == 0).all(dim=1)
    for t in (d_sh, d_pos, d_sg, d_sharp, d_axis):
        t[zero] = 0
    return d_sh, d_pos, d_sg, d_sharp, d_axis


# --------------------------------------------------------------------------- geometry
def quat_to_columns(q):
    """Columns (U, V, W) of the rotation from the un-normalised formula
    (cuda_train/forward/gaussians_aabb.cu:7-17); q = (r, i, j, k)."""
    r, i, j, k = q[:, 0], q[:, 1], q[:, 2], q[:, 3]
    U = torch.stack([1 - 2 * (j * j + k * k), 2 * (i * j + r * k), 2 * (i * k - r * j)], dim=1)
    V = torch.stack([2 * (i * j - r * k), 1 - 2 * (i * i + k * k), 2 * (j * k + r * i)], dim=1)
    W = torch.stack([2 * (i * k + r * j), 2 * (j * k - r * i), 1 - 2 * (i * i + j * j)], dim=1)
    return U, V, W


def quat_grad_from_columns(q, dU, dV, dW):
    """Gradient w.r.t. q of the same un-normalised formula, given gradients of the
    three columns (cuda_train/backward/gaussians_aabb.cu:469-481)."""
    r, i, j, k = q[:, 0], q[:, 1], q[:, 2], q[:, 3]
    gr = 2 * (k * dU[:, 1] - j * dU[:, 2] - k * dV[:, 0] + i * dV[:, 2] + j * dW[:, 0] - i * dW[:, 1])
    gi = 2 * (j * dU[:, 1] + k * dU[:, 2] + j * dV[:, 0] - 2 * i * dV[:, 1] + r * dV[:, 2]
              + k * dW[:, 0] - r * dW[:, 1] - 2 * i * dW[:, 2])
    gj = 2 * (-2 * j * dU[:, 0] + i * dU[:, 1] - r * dU[:, 2] + i * dV[:, 0] + k * dV[:, 2]
              + r * dW[:, 0] + k * dW[:, 1] - 2 * j * dW[:, 2])
    gk = 2 * (-2 * k * dU[:, 0] + r * dU[:, 1] + i * dU[:, 2] - r * dV[:, 0] - 2 * k * dV[:, 1] + j * dV[:, 2]
              + i * dW[:, 0] + j * dW[:, 1])
    return torch.stack([gr, gi, gj, gk], dim=1)


def ellipsoid_aabbs(positions, scales, quaternions, densities, sigma_threshold):
    """Per-Gaussian box of the sigma_threshold iso-ellipsoid and the scene box
    (optix_utils.py:36-109).  The quaternion is renormalised here, as there;
    Gaussians at or below the threshold give a zero-size box at the centre that
    still takes part in the scene box."""
    t = densities / sigma_threshold
    d = torch.log(t * t)
    d = torch.where(d > 0, d, torch.zeros_like(d)).sqrt()
    qn = quaternions / (quaternions * quaternions).sum(dim=1, keepdim=True).add(1e-20).sqrt()
    U, V, W = quat_to_columns(qn)
    # rows of R are (U_a, V_a, W_a); half extent along world axis a
    h = d[:, None] * ((scales[:, 0:1] * U) ** 2 + (scales[:, 1:2] * V) ** 2 + (scales[:, 2:3] * W) ** 2).sqrt()
    lo, hi = positions - h, positions + h
    if positions.shape[0] == 0:
        z = torch.zeros(3, dtype=positions.dtype)
        return lo, hi, z, z.clone()
    return lo, hi, lo.min(dim=0).values, hi.max(dim=0).values


@dataclass
class CameraParams:
    eye: torch.Tensor
    U: torch.Tensor
    V: torch.Tensor
    W: torch.Tensor
    tan_half_x: float
    tan_half_y: float
    px: float
    py: float
    width: int
    height: int

    @staticmethod
    def from_camera(cam, supersampling=(1, 1)):
        """Launch-parameter fill of optix_utils.py:258-266 (fp32 values, held in float64)."""
        wvt = cam.world_view_transform.detach().cpu().to(torch.float32)
        f32 = lambda v: float(torch.tensor(v, dtype=torch.float32))
        return CameraParams(eye=cam.camera_center.detach().cpu().to(torch.float32).to(F64),
                            U=wvt[:3, 0].to(F64), V=wvt[:3, 1].to(F64), W=wvt[:3, 2].to(F64),
                            tan_half_x=f32(math.tan(cam.FoVx / 2)), tan_half_y=f32(math.tan(cam.FoVy / 2)),
                            px=f32(cam.Px), py=f32(cam.Py), width=cam.image_width * supersampling[0],
                            height=cam.image_height * supersampling[1])


def generate_rays(cam: CameraParams, ray_ids: torch.Tensor):
    """cuda_train/forward/gaussians_aabb.cu:95-110; ray id = y * width + x."""
    x = (ray_ids % cam.width).to(F64)
    y = (ray_ids // cam.width).to(F64)
    a = 2.0 * ((x + 0.5) / cam.width - cam.px) * cam.tan_half_x
    b = 2.0 * ((y + 0.5) / cam.height - cam.py) * cam.tan_half_y
    d = a[:, None] * cam.U[None, :] + b[:, None] * cam.V[None, :] + cam.W[None, :]
    return d / d.norm(dim=1, keepdim=True)


# --------------------------------------------------------------------------- march
@dataclass
class MarchOutput:
    rgb: torch.Tensor
    alpha: torch.Tensor
    depth: torch.Tensor
    margin: torch.Tensor            # per ray: smallest relative distance of any evaluated predicate to flipping
    counters: dict = field(default_factory=dict)
    grads: Optional[dict] = None    # explicit backward: pos, scale, quat, density, rgb (per Gaussian)
    overflow: Optional[torch.Tensor] = None   # per ray: some slab had more hits than max_prim_slice (which hits
                                              # survive is then up to the traversal order: no parity defined)


def _trace_closest(valid, root1, root2, tmin, tmax):
    """Closest-hit trace: smallest max(tmin, root1) over the hit set, +inf on a miss."""
    lo = torch.maximum(tmin[:, None], root1)
    hi = torch.minimum(tmax[:, None], root2)
    hit = valid & (lo <= hi)
    t = torch.where(hit, lo, torch.full_like(lo, float("inf")))
    t = torch.cat([t, torch.full_like(tmin, float("inf"))[:, None]], dim=1)   # also covers "no Gaussians at all"
    return t.min(dim=1).values


def _march_chunk(o, d, P, S, Q, dens, rgb_g, bb_min, bb_max, mp, delta=None, c_final=None, diff=False):
    """Marches a chunk of rays ``d [B,3]`` from the common origin ``o`` against the
    Gaussians given (already restricted to those any ray of the chunk can hit).
    Returns per-ray outputs, counters, and -- when ``delta``/``c_final`` are
    given -- the explicit per-Gaussian gradients of
    cuda_train/backward/gaussians_aabb.cu:209-497."""
    B, M = d.shape[0], P.shape[0]
    dt0 = float(torch.tensor(mp.dt_step, dtype=torch.float32))
    eps = float(torch.tensor(mp.transmittance_eps, dtype=torch.float32))
    sig_t = float(torch.tensor(mp.sigma_threshold, dtype=torch.float32))
    inf = float("inf")
    want_grad = delta is not None

    U, V, W = quat_to_columns(Q)
    inv_s = 1.0 / S
    with torch.no_grad():
        k2 = 2.0 * torch.log(dens.detach() / sig_t)          # k^2, optix_utils.py:287
        prim_ok = (dens.detach() > sig_t) & torch.isfinite(k2) & (k2 > 0)
    k2 = torch.where(prim_ok, k2, torch.ones_like(k2))
    Mrows = torch.stack([U * inv_s[:, 0:1], V * inv_s[:, 1:2], W * inv_s[:, 2:3]], dim=1)   # [M,3,3]: y = Mrows @ x
    Ovec = o[None, :] - P                                                                  # pos4
    yO = torch.einsum("mkj,mj->mk", Mrows, Ovec)                                           # [M,3]
    yd = torch.einsum("mkj,bj->bmk", Mrows, d)                                             # [B,M,3]
    A0 = (yO * yO).sum(dim=1)[None, :].expand(B, M)
    A1 = (yO[None, :, :] * yd).sum(dim=2)
    A2 = (yd * yd).sum(dim=2)

    with torch.no_grad():
        # interval test, cuda_train/forward/gaussians_aabb.cu:57-91 (everything divided by k^2)
        a = A2.detach() / k2[None, :]
        b = -A1.detach() / k2[None, :]
        c = A0.detach() / k2[None, :] - 1.0
        p2 = (A0.detach() + 2 * (b / a) * A1.detach() + (b / a) ** 2 * A2.detach()) / k2[None, :]
        disc = 1.0 - p2
        ok = prim_ok[None, :] & (disc > 1e-7)
        sd = (disc.clamp_min(0) * a).sqrt()
        q = b + torch.copysign(sd, b)
        root1 = c / q
        root2 = q / a
        ok &= torch.isfinite(root1) & torch.isfinite(root2)

        # scene-box clip, :212-224
        inv_d = 1.0 / d
        t0 = (bb_min[None, :] - o[None, :]) * inv_d
        t1 = (bb_max[None, :] - o[None, :]) * inv_d
        tlo = torch.fmin(t0, t1)
        thi = torch.fmax(t0, t1)
        tenter = torch.fmax(torch.zeros(B, dtype=F64), torch.fmax(tlo[:, 0], torch.fmax(tlo[:, 1], tlo[:, 2])))
        texit = torch.fmin(thi[:, 0], torch.fmin(thi[:, 1], thi[:, 2]))

    bg = torch.ones(3, dtype=F64) if mp.white_background else torch.zeros(3, dtype=F64)
    T = torch.ones(B, dtype=F64)
    C = torch.zeros(B, 3, dtype=F64)
    depth = torch.zeros(B, dtype=F64)
    margin = torch.full((B,), inf, dtype=F64)
    ovf_ray = torch.zeros(B, dtype=torch.bool)
    cnt = dict(S=0, S_h=0, Q_c=0, P=0, E_in=0, OVF=0)

    with torch.no_grad():
        first = _trace_closest(ok, root1, root2, tenter, texit)                            # :233-257
        cnt["Q_c"] += B
        missed = ~torch.isfinite(first)
        tenter = torch.where(missed, tenter, first)
        running = ~missed & (tenter < texit)                                               # :260
        tbuf = tenter.clone()

    if want_grad:
        Dd = (delta * c_final).sum(dim=1)          # delta . (colour still to come, incl. background)
        g_pos = torch.zeros(M, 3, dtype=F64)
        g_scale = torch.zeros(M, 3, dtype=F64)
        g_dens = torch.zeros(M, dtype=F64)
        g_rgb = torch.zeros(M, 3, dtype=F64)
        g_U = torch.zeros(M, 3, dtype=F64)
        g_V = torch.zeros(M, 3, dtype=F64)
        g_W = torch.zeros(M, 3, dtype=F64)

    offs = (torch.arange(BUFFER_SIZE, dtype=F64) + 0.5)
    while True:
        with torch.no_grad():
            Td = T.detach()
            margin = torch.where(running, torch.minimum(margin, (Td - eps).abs() / eps), margin)
            running = running & (tbuf < texit) & (Td > eps)                                 # :266
            if not bool(running.any()):
                break
            idx = running.nonzero(as_tuple=True)[0]
            tb, Ta = tbuf[idx], Td[idx]
            if mp.dynamic_sampling:                                                         # :267-272
                dt = torch.minimum(torch.clamp_min(tb / 1024.0, dt0) * Ta.pow(-1.0 / 3.0),
                                   torch.full_like(tb, 4.0 * dt0))
            else:
                dt = torch.full_like(tb, dt0)
            slab = dt * BUFFER_SIZE
            smin = torch.maximum(tenter[idx], tb)                                           # :275-276
            smax = torch.minimum(texit[idx], tb + slab)
            traced = smax > tenter[idx]                                                     # :280
            lo = torch.maximum(smin[:, None], root1[idx])
            hi = torch.minimum(smax[:, None], root2[idx])
            hit = ok[idx] & (lo <= hi) & traced[:, None]
            p0 = hit.sum(dim=1)
            cnt["S"] += int(idx.numel())
            cnt["OVF"] += int((p0 > mp.max_prim_slice).sum())
            ovf_ray[idx[p0 > mp.max_prim_slice]] = True
            gap = torch.where(ok[idx], (hi - lo).abs() / slab[:, None], torch.full_like(lo, inf))
            gap = torch.cat([gap, torch.full_like(slab, inf)[:, None]], dim=1).min(dim=1).values
            margin[idx] = torch.minimum(margin[idx], gap)

            empty = traced & (p0 == 0)                                                      # :297-319
            if bool(empty.any()):
                e = idx[empty]
                nb = tb[empty] + slab[empty]
                nxt = _trace_closest(ok[e], root1[e], root2[e], nb, texit[e])
                cnt["Q_c"] += int(e.numel())
                gone = ~torch.isfinite(nxt)
                tbuf[e] = torch.where(gone, nb, nxt)
                running[e[gone]] = False
            skip = ~traced                                                                  # falls through to :324
            if bool(skip.any()):
                tbuf[idx[skip]] = tb[skip] + slab[skip]
            has = p0 > 0
            if not bool(has.any()):
                continue
            h = idx[has]
            tb, dt, slab, hit, p0 = tb[has], dt[has], slab[has], hit[has], p0[has]
            cnt["S_h"] += int(h.numel())
            cnt["P"] += int(p0.sum())
            ts = tb[:, None] + offs[None, :] * dt[:, None]                                  # [b,32] sample positions

        # power = |M(O + t d)|^2, :153-177 (evaluated directly instead of by second differences)
        tt = ts[:, None, :]
        power = A0[h][:, :, None] + 2.0 * A1[h][:, :, None] * tt + A2[h][:, :, None] * tt * tt       # [b,M,32]
        with torch.no_grad():
            inside = hit[:, :, None] & (power.detach() < k2[None, :, None])                 # :168
            rel = torch.where(hit[:, :, None], (power.detach() / k2[None, :, None] - 1.0).abs(),
                              torch.full_like(power, inf))
            margin[h] = torch.minimum(margin[h], rel.amin(dim=(1, 2)))
        gw = torch.where(inside, torch.exp(-0.5 * power), torch.zeros_like(power))
        sw = dens[None, :, None] * gw                                                        # sigma_i g
        sum_sigma = sw.sum(dim=1)                                                            # [b,32]
        sum_col = torch.einsum("bms,mc->bsc", sw, rgb_g)                                     # [b,32,3]

        # compositing, :190-201, with the chunk rule: the second 16 samples only if T > eps after the first
        Tl = T[h]
        Cl = C[h]
        Dl = depth[h]
        x = sum_sigma * dt[:, None]
        w = torch.exp(-x)
        sfac = dt[:, None] * (1.0 - w) / x.clamp_min(1e-6)
        alive = torch.ones_like(Tl, dtype=torch.bool)
        T_seq = []
        for s in range(BUFFER_SIZE):
            if s == CHUNK_SIZE:
                with torch.no_grad():
                    margin[h] = torch.minimum(margin[h], (Tl.detach() - eps).abs() / eps)
                    alive = Tl.detach() > eps
            T_seq.append(Tl)
            am = alive.to(F64)
            Cl = Cl + (am * Tl * sfac[:, s])[:, None] * sum_col[:, s, :]
            Dl = Dl + am * Tl * (1.0 - w[:, s]) * ts[:, s]
            Tl = torch.where(alive, Tl * w[:, s], Tl)
        with torch.no_grad():
            cnt["E_in"] += int((inside[:, :, :CHUNK_SIZE].sum()) + (inside[:, :, CHUNK_SIZE:].sum(dim=(1, 2))
                                                                     * alive).sum())

        if want_grad:
            with torch.no_grad():
                dl = delta[h]
                ci = dl @ rgb_g.t()                                                          # [b,M] delta . c_i
                dsum = (sw * ci[:, :, None]).sum(dim=1)                                      # [b,32] delta . sum_col
                pos_s = sum_sigma > 0
                chat = torch.where(pos_s, dsum / sum_sigma.clamp_min(1e-300), torch.zeros_like(dsum))
                inv_sig = torch.where(pos_s, 1.0 / sum_sigma.clamp_min(1e-300), torch.zeros_like(dsum))
                # running T_s and D_s over all 32 samples, backward .cu:330-352
                Ts = torch.empty_like(sum_sigma)
                Ds = torch.empty_like(sum_sigma)
                Tr, Dr = T[h].clone(), Dd[h].clone()
                for s in range(BUFFER_SIZE):
                    Ts[:, s], Ds[:, s] = Tr, Dr
                    Dr = Dr - Tr * (1.0 - w[:, s]) * chat[:, s]
                    Tr = Tr * w[:, s]
                live = torch.ones_like(sum_sigma, dtype=torch.bool)
                live[:, CHUNK_SIZE:] = (Ts[:, CHUNK_SIZE] > eps)[:, None]                   # backward .cu:398
                beta = Ts * (1.0 - w) * inv_sig
                alpha = (Ts * chat - Ds) * dt[:, None]
                m = inside & live[:, None, :]
                Aw = torch.where(m, gw * (alpha[:, None, :] + beta[:, None, :] * (ci[:, :, None] - chat[:, None, :])),
                                 torch.zeros_like(gw))                                       # g * dL/d(sigma g)
                g_rgb += torch.einsum("bms,bc->mc", torch.where(m, sw * beta[:, None, :], torch.zeros_like(sw)), dl)
                g_dens += Aw.sum(dim=(0, 2))
                om = Aw * dens[None, :, None]                                                # omega
                y = yO[None, :, None, :] + tt[..., None] * yd[h][:, :, None, :]             # [b,M,32,3]
                xs = Ovec[None, :, None, :] + tt[..., None] * d[h][:, None, None, :]        # x_s - p
                g_scale += torch.einsum("bms,bmsk->mk", om, y * y) * inv_s
                Sy = torch.einsum("bms,bmsk->mk", om, y)
                g_pos += torch.einsum("mkj,mk->mj", Mrows, Sy)
                oyx = torch.einsum("bms,bmsk,bmsj->mkj", om, y, xs)                         # sum omega y_k x_j
                g_U -= oyx[:, 0, :] * inv_s[:, 0:1]
                g_V -= oyx[:, 1, :] * inv_s[:, 1:2]
                g_W -= oyx[:, 2, :] * inv_s[:, 2:3]
                Dd[h] = Dr                                                                   # backward .cu:491-492
        T = T.clone()
        C = C.clone()
        depth = depth.clone()
        T[h], C[h], depth[h] = Tl, Cl, Dl
        with torch.no_grad():
            tbuf[h] = tb + slab                                                              # :324

    rgb = C + T[:, None] * bg[None, :]                                                       # :326-330
    out = MarchOutput(rgb=rgb, alpha=1.0 - T, depth=depth, margin=margin, counters=cnt, overflow=ovf_ray)
    if want_grad:
        out.grads = dict(pos=g_pos, scale=g_scale, quat=quat_grad_from_columns(Q, g_U, g_V, g_W), density=g_dens,
                         rgb=g_rgb)
    return out


def _bounding_radius(S, Q, dens, sig_t):
    """Radius of a sphere around each centre that contains the truncation
    ellipsoid {x : |S^-1 R^T x|^2 <= k^2}, valid for non-unit quaternions too."""
    with torch.no_grad():
        U, V, W = quat_to_columns(Q)
        inv_s = 1.0 / S
        Mrows = torch.stack([U * inv_s[:, 0:1], V * inv_s[:, 1:2], W * inv_s[:, 2:3]], dim=1)
        k = (2.0 * torch.log((dens / sig_t).clamp_min(1.0))).sqrt()
        inv = torch.linalg.inv(Mrows + 1e-300 * torch.eye(3, dtype=F64))
        return k * inv.flatten(1).norm(dim=1) * 1.0001 + 1e-12


def _prefilter(o, dirs, P, rad, dens, sig_t):
    """Conservative cull for a chunk: keep Gaussians whose bounding sphere touches
    a ray of the chunk.  Only saves memory and time: every Gaussian left out has
    an empty interval on every ray of the chunk."""
    with torch.no_grad():
        v = P - o[None, :]
        tproj = v @ dirs.t()                                      # [M,B]
        perp2 = (v * v).sum(dim=1, keepdim=True) - tproj * tproj
        near = (perp2 <= (rad * rad)[:, None] * 1.0001 + 1e-12) & (tproj + rad[:, None] >= 0)
        return near.any(dim=1) & (dens > sig_t)


def _pierced(o, dirs, P, S, Q, dens, sig_t):
    """Exact cull for a chunk: keep the Gaussians whose truncation ellipsoid the LINE of some ray of the chunk
    pierces (the discriminant test of cuda_train/forward/gaussians_aabb.cu:57-73 in float64, with a little slack).
    Bounding spheres say little about needles of 100:1; this leaves the few hundred Gaussians per ray that can
    appear in a hit set at all, so that the dense sample x Gaussian tensors stay small."""
    with torch.no_grad():
        U, V, W = quat_to_columns(Q)
        inv_s = 1.0 / S
        Mrows = torch.stack([U * inv_s[:, 0:1], V * inv_s[:, 1:2], W * inv_s[:, 2:3]], dim=1)
        k2 = 2.0 * torch.log((dens / sig_t).clamp_min(1e-300))
        yO = torch.einsum("mkj,mj->mk", Mrows, o[None, :] - P)
        keep = torch.zeros(P.shape[0], dtype=torch.bool)
        A0 = (yO * yO).sum(dim=1)
        for b in range(dirs.shape[0]):                      # ray by ray: [M, 3] temporaries only
            yd = torch.einsum("mkj,j->mk", Mrows, dirs[b])
            A1 = (yO * yd).sum(dim=1)
            A2 = (yd * yd).sum(dim=1)
            # |P|^2 / k^2 < 1 - 1e-7 is the reference's test; keep everything within a hair of it
            p2 = (A0 - A1 * A1 / A2) / k2
            keep |= (1.0 - p2) > 0.5e-7
        return keep & (dens > sig_t)


def _cone_cull(o, dirs, P, rad):
    """Conservative cull for a whole set of rays from one origin: keep the Gaussians whose bounding sphere
    reaches into the cone around the mean direction that contains every ray.  Like :func:`_prefilter` it only
    saves memory and time on large scenes (the per-chunk filter then works on what is left)."""
    with torch.no_grad():
        axis = dirs.mean(dim=0)
        axis = axis / axis.norm()
        half = torch.acos((dirs @ axis).min().clamp(-1.0, 1.0)) + 1e-6
        v = P - o[None, :]
        dist = v.norm(dim=1)
        inside = dist <= rad                                          # the origin lies in the sphere
        ang = torch.acos(((v @ axis) / dist.clamp_min(1e-300)).clamp(-1.0, 1.0))
        spread = torch.asin((rad / dist.clamp_min(1e-300)).clamp(max=1.0))
        return inside | (ang <= half + spread + 1e-9)


def march(positions, scales, quaternions, densities, rgb_g, cam: CameraParams, mp, ray_ids=None, delta=None,
          chunk=64, diff=False):
    """Forward (and, with ``delta = dL/dC [R,3]``, explicit backward) of the march
    for the rays ``ray_ids`` (default: the whole image).  Inputs are cast to
    float64.  With ``diff=True`` the inputs keep their autograd graph and the
    returned ``rgb`` is differentiable with the sample schedule and all
    predicates held fixed -- which is what the reference's backward
    differentiates."""
    cast = (lambda t: t.to(F64)) if diff else (lambda t: t.detach().to(F64))
    P, S, Q, dens, rgbg = (cast(t) for t in (positions, scales, quaternions, densities, rgb_g))
    R = cam.width * cam.height
    if ray_ids is None:
        ray_ids = torch.arange(R)
    n_r = ray_ids.numel()
    dirs = generate_rays(cam, ray_ids)
    o = cam.eye
    sig_t = float(torch.tensor(mp.sigma_threshold, dtype=torch.float32))
    with torch.no_grad():
        _, _, bb_min, bb_max = ellipsoid_aabbs(P.detach(), S.detach(), Q.detach(), dens.detach(), sig_t)
    N = P.shape[0]
    rad = _bounding_radius(S.detach(), Q.detach(), dens.detach(), sig_t)
    rgb = []
    alpha = torch.zeros(n_r, dtype=F64)
    depth = torch.zeros(n_r, dtype=F64)
    margin = torch.zeros(n_r, dtype=F64)
    overflow = torch.zeros(n_r, dtype=torch.bool)
    total = dict(S=0, S_h=0, Q_c=0, P=0, E_in=0, OVF=0)
    grads = None
    if delta is not None:
        delta = delta.detach().to(F64)
        # pass 1: final colours (the backward reads the forward's output, backward .cu:261-265)
        fwd = march(positions, scales, quaternions, densities, rgb_g, cam, mp, ray_ids=ray_ids, chunk=chunk)
        grads = dict(pos=torch.zeros(N, 3, dtype=F64), scale=torch.zeros(N, 3, dtype=F64),
                     quat=torch.zeros(N, 4, dtype=F64), density=torch.zeros(N, dtype=F64),
                     rgb=torch.zeros(N, 3, dtype=F64))
    cone = None
    if N > 100_000 and n_r > 0:
        cone = _cone_cull(o, dirs, P.detach(), rad).nonzero(as_tuple=True)[0]
    for s in range(0, n_r, chunk):
        sl = slice(s, min(n_r, s + chunk))
        dch = dirs[sl]
        if cone is None:
            keep = _prefilter(o, dch, P.detach(), rad, dens.detach(), sig_t)
            ids = keep.nonzero(as_tuple=True)[0]
        else:
            keep = _prefilter(o, dch, P.detach()[cone], rad[cone], dens.detach()[cone], sig_t)
            ids = cone[keep]
            ids = ids[_pierced(o, dch, P.detach()[ids], S.detach()[ids], Q.detach()[ids], dens.detach()[ids], sig_t)]
        out = _march_chunk(o, dch, P[ids], S[ids], Q[ids], dens[ids], rgbg[ids], bb_min, bb_max, mp,
                           delta=None if delta is None else delta[sl],
                           c_final=None if delta is None else fwd.rgb[sl], diff=diff)
        rgb.append(out.rgb)
        alpha[sl], depth[sl], margin[sl] = out.alpha.detach(), out.depth.detach(), out.margin
        overflow[sl] = out.overflow
        for kx in total:
            total[kx] += out.counters[kx]
        if grads is not None:
            for kx in grads:
                grads[kx].index_add_(0, ids, out.grads[kx])
    return MarchOutput(rgb=torch.cat(rgb, dim=0) if rgb else torch.zeros(0, 3, dtype=F64), alpha=alpha, depth=depth,
                       margin=margin, counters=total, grads=grads, overflow=overflow)


# --------------------------------------------------------------------------- operator
def knn_mean_dist2(points):
    """Mean of the squared distances from every point to its three nearest other points, by brute force in
    float64 (what SimpleKNN::knn computes, submodules/simple-knn/simple_knn.cu:146-185: a point is excluded by
    its index, so a duplicate counts with distance zero).  With fewer than four points the missing neighbours
    stay at FLT_MAX and the reference adds them up in fp32: one missing gives about FLT_MAX / 3, two or three
    overflow to +inf.  Pinned to the reference's own output by tests/golden/knn.npz."""
    import numpy as np
    p = np.asarray(points, dtype=np.float64)
    n = p.shape[0]
    out = np.empty(n, dtype=np.float64)
    flt_max = np.finfo(np.float32).max
    for i in range(n):
        d = ((p - p[i]) ** 2).sum(axis=1)
        d = np.delete(d, i)
        best = np.sort(d)[:3].tolist()
        if len(best) == 3:
            out[i] = (best[0] + best[1] + best[2]) / 3.0
        else:                                  # the reference's fp32 sum with FLT_MAX for what is missing
            with np.errstate(over="ignore"):
                total = np.float32(0.0)
                for b in [np.float32(x) for x in best] + [flt_max] * (3 - len(best)):
                    total = np.float32(total + b)
                out[i] = float(np.float32(total / np.float32(3.0)))
    return out


def quantize_frame(rgb):
    """8-bit colour of the reference's viewer (cuda_gui/helpers.h:45-58): clamp to [0, 1],
    times 256 in float32, truncated, at most 255; alpha byte 255.  ``rgb`` [..., 3] -> uint8 [..., 4]."""
    import numpy as np
    x = np.clip(np.asarray(rgb, dtype=np.float32), np.float32(0.0), np.float32(1.0))
    q = np.minimum((x * np.float32(256.0)).astype(np.uint32), 255).astype(np.uint8)
    return np.concatenate([q, np.full(q.shape[:-1] + (1,), 255, dtype=np.uint8)], axis=-1)


def render_forward(positions, scales, quaternions, densities, color_features, sg_features, sharpness, lobe_axis,
                   camera, mp, supersampling=(1, 1), ray_ids=None, chunk=64):
    """Forward of render_optix.py:92-141 in float64: returns the march output and
    the per-Gaussian colours."""
    cam = CameraParams.from_camera(camera, supersampling)
    to = lambda t: t.detach().cpu().to(F64)
    rgb_g = gaussian_rgb(cam.eye, to(positions), to(color_features), to(sg_features), to(sharpness), to(lobe_axis))
    out = march(to(positions), to(scales), to(quaternions), to(densities), rgb_g, cam, mp, ray_ids=ray_ids,
                chunk=chunk)
    return out, rgb_g


def render_backward(positions, scales, quaternions, densities, color_features, sg_features, sharpness, lobe_axis,
                    camera, mp, dloss_dray_colors, supersampling=(1, 1), ray_ids=None, chunk=64,
                    reference_quirk=True):
    """Explicit backward of render_optix.py:144-199 in float64.  Returns a dict
    with the eight gradients under the reference's argument names plus ``rgb``
    (dL/d per-Gaussian colour) and the forward ``out``."""
    cam = CameraParams.from_camera(camera, supersampling)
    to = lambda t: t.detach().cpu().to(F64)
    P, S, Q, D = to(positions), to(scales), to(quaternions), to(densities)
    cf, sg, shp, ax = to(color_features), to(sg_features), to(sharpness), to(lobe_axis)
    rgb_g = gaussian_rgb(cam.eye, P, cf, sg, shp, ax)
    out = march(P, S, Q, D, rgb_g, cam, mp, ray_ids=ray_ids, delta=to(dloss_dray_colors), chunk=chunk)
    g = out.grads
    d_sh, d_pos_dir, d_sg, d_shp, d_ax = gaussian_rgb_backward(cam.eye, P, cf, sg, shp, ax, g["rgb"],
                                                               reference_quirk=reference_quirk)
    return dict(positions=g["pos"] + d_pos_dir, scales=g["scale"], quaternions=g["quat"], densities=g["density"],
                color_features=d_sh, sph_gauss_features=d_sg, bandwidth_sharpness=d_shp, lobe_axis=d_ax,
                rgb=g["rgb"], out=out)


def render_autograd(positions, scales, quaternions, densities, color_features, sg_features, sharpness, lobe_axis,
                    camera, mp, dloss_dray_colors, supersampling=(1, 1), ray_ids=None, chunk=64):
    """The same gradients obtained by ``torch.autograd`` through the
    differentiable forward (schedule and predicates held fixed).  Used to check
    the explicit backward; always uses the exact SH derivative."""
    cam = CameraParams.from_camera(camera, supersampling)
    leaves = [t.detach().cpu().to(F64).clone().requires_grad_(True) for t in
              (positions, scales, quaternions, densities, color_features, sg_features, sharpness, lobe_axis)]
    P, S, Q, D, cf, sg, shp, ax = leaves
    rgb_g = gaussian_rgb(cam.eye, P, cf, sg, shp, ax)
    out = march(P, S, Q, D, rgb_g, cam, mp, ray_ids=ray_ids, chunk=chunk, diff=True)
    loss = (out.rgb * dloss_dray_colors.detach().cpu().to(F64)).sum()
    grads = torch.autograd.grad(loss, leaves, allow_unused=True)
    names = ("positions", "scales", "quaternions", "densities", "color_features", "sph_gauss_features",
             "bandwidth_sharpness", "lobe_axis")
    return {n: (torch.zeros_like(l) if g is None else g) for n, g, l in zip(names, grads, leaves)}, out
