"""Parity of the CUDA path with the reference on the CONTENT of the three large configurations: the 300 k
object scene, the 3 M unbounded scene and the 7 M stress scene (B200, `-m gpu`).

Every view of tests/scene_views.py is a few hundred rays against all Gaussians of its scene.  The CUDA path
(rgx_build + rgx_forward + rgx_backward through the C ABI) is compared with

* the float64 oracle's committed outputs (tests/golden/scene_*.npz, made by tests/golden/make_scene_golden.py):
  colours, alpha, depth, and the gradients at 1,024 sampled entries per tensor;
* the reference's own device code compiled for the CPU (oracle/_ref), run live on the host cores for the same
  view: colours and the complete gradient tensors.

Tolerances: 1e-4 on RGB and alpha for rays whose every discrete decision (truncation, termination, slab overlap)
keeps a relative margin above 3e-5 in float64; the other rays -- where fp32 may legitimately decide otherwise --
are held to a loose bound instead of being dropped, and their share is asserted per view.  Gradients: 1e-3 of
the tensor's largest entry everywhere, and element by element on the entries above a thousandth of the largest.
Rays with a slab that overflowed the hit cap are left out (which hits survive is the traversal's choice).
"""
import copy
import os

import numpy as np
import pytest
import torch

from raygaussx_b200 import _lib, scenes
from tests.helpers import GOLDEN, rel_max
from tests.scene_views import GRAD_NAMES, SCENES, input_checksum, view_camera

pytestmark = pytest.mark.gpu

RGB_TOL = 1e-4
GRAD_TOL = 1e-3
MARGIN = 3e-5
LOOSE_RGB_TOL = 1e-3        # rays with a marginal decision: one flipped truncation moves a pixel by up to sigma_t dt
# entry-by-entry relative error of the gradients on entries above a thousandth of the tensor's largest: an entirely
# wrong entry is off by 1.  The reference's own fp32 build differs from the float64 oracle by up to 1.2e-2 here
# (99th percentile 4.4e-3) -- flipped truncations on marginal rays and fp32 sums over thousands of rays
ELEM_MAX = 0.2
ELEM_P99 = 1e-2
# smallest share of rays that must be outside the margin, per view (dense views evaluate ~10^5 predicates per ray)
MIN_STEADY = {"object:whole": 0.80, "object:crop_centre": 0.55, "object:crop_rim": 0.75,
              "unbounded:whole": 0.60, "unbounded:crop_centre": 0.55, "unbounded:crop_sky": 0.55,
              "stress:whole": 0.70, "stress:crop_centre": 0.70}

VIEWS = [(s, v[0]) for s, (_, views) in SCENES.items() for v in views]
_cache = {}


def scene_on_gpu(name):
    """One scene at a time (the 7 M one is 1.6 GB on the host and on the device)."""
    if _cache.get("name") != name:
        _cache.clear()
        torch.cuda.empty_cache()
        from raygaussx_b200 import render_optix as ro
        sc = SCENES[name][0]()
        dev = torch.device("cuda")
        _cache.update(name=name, sc=sc, tens=[t.to(dev).contiguous() for t in sc.tensors()],
                      renderer=ro.Renderer(dev), csum=input_checksum(sc))
        _cache["renderer"].build(*_cache["tens"][:4])
    return _cache


def elementwise(ref, got, floor=1e-3):
    """Relative error entry by entry on the entries of ``ref`` above ``floor`` times its largest."""
    ref = np.asarray(ref, dtype=np.float64).reshape(-1)
    got = np.asarray(got, dtype=np.float64).reshape(-1)
    big = np.abs(ref) > floor * np.abs(ref).max()
    if not big.any():
        return 0.0, 0.0
    rel = np.abs(got[big] - ref[big]) / np.abs(ref[big])
    return float(rel.max()), float(np.quantile(rel, 0.99))


@pytest.mark.parametrize("scene_name,view_name", VIEWS)
def test_large_scene_view_matches_the_reference(scene_name, view_name):
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device: there is no CPU path")
    from raygaussx_b200 import render_optix as ro
    path = os.path.join(GOLDEN, f"scene_{scene_name}_{view_name}.npz")
    assert os.path.exists(path), "golden vectors missing: run tests/golden/make_scene_golden.py"
    g = np.load(path)
    c = scene_on_gpu(scene_name)
    sc, tens, r = c["sc"], c["tens"], c["renderer"]
    assert c["csum"] == pytest.approx(float(g["input_sum"]), rel=1e-12)
    _, cam_index, kind, geom = next(v for v in SCENES[scene_name][1] if v[0] == view_name)
    cam = view_camera(sc, kind, cam_index, geom)
    cam.to(torch.device("cuda"))
    cs = ro.camera_struct(cam)
    key = f"{scene_name}:{view_name}"
    report = []
    try:
        _compare(g, sc, tens, r, cam, cs, key, report)
    finally:
        print("\n".join(report))


def _compare(g, sc, tens, r, cam, cs, key, report):
    from raygaussx_b200 import render_optix as ro

    def march(eps, flags=0):
        m = sc.march
        return ro.Renderer._march(m.dt_step, m.dynamic_sampling, m.max_prim_slice, m.white_background, eps, None,
                                  cs.height, flags)

    # ---- forward at the configuration's own threshold against the float64 oracle
    eps_cfg = sc.march.transmittance_eps
    rgb, alpha, depth = r.forward(*tens, cs, march(eps_cfg, _lib.FLAG_SAVE_HITS), want_alpha=True, want_depth=True)
    plain, _, _ = r.forward(*tens, cs, march(eps_cfg))              # no recording: the two-depth path where it applies
    assert torch.equal(plain, rgb), "the forward-only path renders another image than the recording forward"
    ok = ~g["oracle_overflow"]
    steady = (g["oracle_margin"] > MARGIN) & ok
    loose = ~(g["oracle_margin"] > MARGIN) & ok
    err = np.abs(rgb.cpu().numpy().astype(np.float64) - g["oracle_rgb"]).max(axis=1)
    report.append(f"{key}: rays {err.size}, overflow {int((~ok).sum())}, steady {steady.mean():.3f}, "
                  f"max err steady {err[steady].max():.2e}" + (f", marginal {err[loose].max():.2e}" if loose.any() else ""))
    assert steady.mean() >= MIN_STEADY[key], report
    assert err[steady].max() <= RGB_TOL, report
    assert not loose.any() or err[loose].max() <= LOOSE_RGB_TOL, report
    assert np.abs(alpha.cpu().numpy() - g["oracle_alpha"])[steady].max() <= RGB_TOL
    rel_depth = np.abs(depth.cpu().numpy() - g["oracle_depth"]) / np.maximum(1.0, np.abs(g["oracle_depth"]))
    assert rel_depth[steady].max() <= 5e-4

    # ---- at the reference's fixed threshold (1e-3) against its own device code, run here on the host cores
    at_ref = abs(eps_cfg - 1e-3) < 1e-12
    if not at_ref:
        rgb, _, _ = r.forward(*tens, cs, march(1e-3, _lib.FLAG_SAVE_HITS))
        ok = ~g["oracle1e3_overflow"]
        steady = (g["oracle1e3_margin"] > MARGIN) & ok
        err3 = np.abs(rgb.cpu().numpy().astype(np.float64) - g["oracle1e3_rgb"]).max(axis=1)
        assert err3[steady].max() <= RGB_TOL
    err_ref = np.abs(rgb.cpu().numpy() - g["ref_rgb"]).max(axis=1)
    report.append(f"vs reference colours: steady {err_ref[steady].max():.2e}")
    assert err_ref[steady].max() <= RGB_TOL, report

    # ---- backward: replay of the recording, then by searching again
    dl = torch.from_numpy(g["dl"]).to(rgb.device, torch.float32).contiguous()
    grads = [torch.full_like(t, float("nan")) for t in tens]
    r.backward(*tens, cs, march(1e-3), rgb, dl, tuple(grads))
    torch.cuda.synchronize()
    for nm, gr in zip(GRAD_NAMES, grads):
        idx, val, mx = g["og_idx_" + nm], g["og_val_" + nm], float(g["og_max_" + nm])
        got = gr.reshape(-1)[torch.from_numpy(idx).to(gr.device)].cpu().numpy().astype(np.float64)
        assert np.isfinite(got).all(), nm
        at_max = np.abs(got - val).max() / mx
        emax, e99 = elementwise(val, got)
        report.append(f"{nm}: vs oracle max-normalised {at_max:.2e}, element-wise max {emax:.2e} p99 {e99:.2e}")
        assert at_max <= GRAD_TOL, report
        assert e99 <= ELEM_P99 and emax <= ELEM_MAX, report
    r.forward(*tens, cs, march(1e-3))                               # discards the recording
    searched = [torch.full_like(t, float("nan")) for t in tens]
    r.backward(*tens, cs, march(1e-3), rgb, dl, tuple(searched))
    torch.cuda.synchronize()
    for nm, a, b in zip(GRAD_NAMES, grads, searched):
        assert rel_max(a.cpu(), b.cpu()) <= 5e-4, (nm, report)

    # ---- the complete gradient tensors against the reference's backward, live
    from oracle import ref_shim
    if ref_shim.available():
        cpu = [t.cpu() for t in tens]
        m3 = copy.copy(sc.march)
        m3.transmittance_eps = 1e-3
        cam_cpu = copy.copy(cam)
        cam_cpu.to("cpu")
        col, _, rctx = ref_shim.render_forward(*cpu, cam_cpu, m3, n_threads=os.cpu_count() or 1)
        assert np.abs(col - g["ref_rgb"]).max() <= 1e-6            # the reference run here = the one in the golden file
        rg = ref_shim.render_backward(rctx, g["dl"].astype(np.float32), n_threads=os.cpu_count() or 1)
        for k, (nm, gr) in enumerate(zip(GRAD_NAMES, grads)):
            full = rel_max(rg[k], gr.cpu())
            emax, e99 = elementwise(rg[k], gr.cpu().numpy())
            report.append(f"{nm}: vs reference (all entries) max-normalised {full:.2e}, element-wise max {emax:.2e} p99 {e99:.2e}")
            assert full <= GRAD_TOL, report
            assert e99 <= ELEM_P99 and emax <= ELEM_MAX, report


def test_release_the_scene():
    _cache.clear()
    torch.cuda.empty_cache()
