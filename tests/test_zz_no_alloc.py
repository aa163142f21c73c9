"""The allocation-free forward entry point (B200, `-m gpu`; collected last on purpose).

Who needs it: hosts of the library that cannot allocate device memory when they want a
frame -- a viewer beside a trainer whose caching allocator already owns the memory, a
plug-in inside a process that forbids allocations after start-up, a latency path that
cannot take an allocation's implicit synchronisation.  `rgx_forward_static` serves them
from a fixed array inside the library image.

Checked here, through the C ABI: its image equals the image of the regular entry points
(`rgx_build` + `rgx_forward`) within the suite's RGB tolerance on two calls in a row (the shared array
keeps the previous call's contents, so the second call proves that stale state does not
leak), that device memory in use does not grow across the calls, and that sizes beyond
the stated maximum are refused.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from raygaussx_b200 import _lib, scenes
from tests.helpers import load_golden

pytestmark = pytest.mark.gpu

RGB_TOL = 1e-4
STATIC_MAX = 32768


def _call_static(ro, sc, cam_struct, march, tens, want_extra=True):
    dev = tens[0].device
    r = cam_struct.width * cam_struct.height
    rgb = torch.full((r, 3), -1.0, device=dev)
    alpha = torch.full((r,), -1.0, device=dev) if want_extra else None
    depth = torch.full((r,), -1.0, device=dev) if want_extra else None
    scene = ro.Renderer._scene(*tens)
    stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    rc = _lib.lib().rgx_forward_static(dev.index or 0, C.byref(scene), C.byref(cam_struct), C.byref(march),
                                       C.c_float(0.1), rgb.data_ptr(), None if alpha is None else alpha.data_ptr(),
                                       None if depth is None else depth.data_ptr(), stream)
    return rc, rgb, alpha, depth


def _march(ro, sc, cs):
    m = sc.march
    return ro.Renderer._march(m.dt_step, m.dynamic_sampling, m.max_prim_slice, m.white_background,
                              m.transmittance_eps, None, cs.height, 0)


def test_static_forward_matches_regular_forward_twice():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    from raygaussx_b200 import render_optix as ro
    dev = torch.device("cuda", torch.cuda.current_device())
    # two different scenes back to back: the second call must not see the first one's leftovers
    cases = [scenes.tiny_scene(n=4096, width=64, height=64),
             scenes.tiny_scene(n=700, width=24, height=20, log_scale_mean=-2.4, seed=41, dynamic_sampling=True,
                               dt_step=0.004, white_background=True, lobes=2, sh_degree=2)]
    expected = []
    r = ro.get_renderer(dev)
    prepared = []
    for sc in cases:
        tens = [t.to(dev).contiguous() for t in sc.tensors()]
        sc.cameras[0].to(dev)
        cs = ro.camera_struct(sc.cameras[0])
        r.build(*tens[:4])
        rgb, alpha, depth = r.forward(*tens, cs, _march(ro, sc, cs), want_alpha=True, want_depth=True)
        expected.append((rgb.clone(), alpha.clone(), depth.clone()))
        prepared.append((sc, tens, cs))
    torch.cuda.synchronize()
    _call_static(ro, *prepared[0][:1], prepared[0][2], _march(ro, prepared[0][0], prepared[0][2]), prepared[0][1])
    torch.cuda.synchronize()                      # first call: one-time set-up is over
    before = torch.cuda.mem_get_info(dev)[0]
    for (sc, tens, cs), (rgb_e, alpha_e, depth_e) in list(zip(prepared, expected)) * 2:
        rc, rgb, alpha, depth = _call_static(ro, sc, cs, _march(ro, sc, cs), tens)
        torch.cuda.synchronize()
        assert rc == _lib.RGX_OK
        assert (rgb - rgb_e).abs().max().item() <= RGB_TOL
        assert (alpha - alpha_e).abs().max().item() <= RGB_TOL
        assert (depth - depth_e).abs().max().item() <= 5e-4
        if sc is prepared[0][0]:
            # the first scene is the 4,096-Gaussian 64x64 configuration: also against the committed golden vectors
            # (float64 oracle and the reference's own device code), not only against this library's other path
            g = load_golden("config1")
            steady = g["oracle_margin"] > 3e-5
            got = rgb.cpu().numpy()
            assert np.abs(got.astype(np.float64) - g["oracle_rgb"]).max(axis=1)[steady].max() <= RGB_TOL
            assert np.abs(got - g["ref_rgb"]).max(axis=1)[steady].max() <= RGB_TOL
            assert np.abs(alpha.cpu().numpy() - g["oracle_alpha"])[steady].max() <= RGB_TOL
    after = torch.cuda.mem_get_info(dev)[0]
    # torch's own tensors of the loop are freed back to its cache; the driver-level free memory may only
    # shrink by what torch itself newly reserved (a few MiB), never by a workspace
    assert before - after < 64 * 2 ** 20


def test_static_forward_at_its_stated_maximum():
    """Exactly 32,768 Gaussians: the fixed carve-up of the array is at its tightest (every sub-array full, the
    hierarchy at its deepest for the limit).  Twice in a row against the regular entry points."""
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    from raygaussx_b200 import render_optix as ro
    dev = torch.device("cuda", torch.cuda.current_device())
    sc = scenes.tiny_scene(n=STATIC_MAX, width=32, height=24, log_scale_mean=-4.0, seed=77)
    tens = [t.to(dev).contiguous() for t in sc.tensors()]
    sc.cameras[0].to(dev)
    cs = ro.camera_struct(sc.cameras[0])
    r = ro.get_renderer(dev)
    r.build(*tens[:4])
    want, want_alpha, _ = r.forward(*tens, cs, _march(ro, sc, cs), want_alpha=True)
    assert want_alpha.max().item() > 0.5            # the view is not empty
    for _ in range(2):
        rc, rgb, alpha, _ = _call_static(ro, sc, cs, _march(ro, sc, cs), tens)
        torch.cuda.synchronize()
        assert rc == _lib.RGX_OK
        assert (rgb - want).abs().max().item() <= RGB_TOL
        assert (alpha - want_alpha).abs().max().item() <= RGB_TOL
    assert torch.cuda.current_device() == dev.index   # the caller's current device is left as it was


def test_static_forward_refuses_what_it_cannot_hold():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    from raygaussx_b200 import render_optix as ro
    dev = torch.device("cuda", torch.cuda.current_device())
    sc = scenes.tiny_scene(n=STATIC_MAX + 1, width=4, height=4)
    tens = [t.to(dev).contiguous() for t in sc.tensors()]
    sc.cameras[0].to(dev)
    cs = ro.camera_struct(sc.cameras[0])
    rc, rgb, _, _ = _call_static(ro, sc, cs, _march(ro, sc, cs), tens, want_extra=False)
    assert rc == _lib.RGX_E_TOO_LARGE
    assert (rgb == -1).all()                      # nothing was launched
    m = _march(ro, sc, cs)
    m.flags = _lib.FLAG_COUNT_WORK
    small = scenes.tiny_scene(n=16, width=4, height=4)
    t2 = [t.to(dev).contiguous() for t in small.tensors()]
    rc, _, _, _ = _call_static(ro, small, cs, m, t2, want_extra=False)
    assert rc == _lib.RGX_E_INVALID
    # an empty scene renders the background
    empty = scenes.tiny_scene(n=0, width=4, height=4, white_background=True)
    t3 = [t.to(dev).contiguous() for t in empty.tensors()]
    rc, rgb, alpha, _ = _call_static(ro, empty, cs, _march(ro, empty, cs), t3)
    torch.cuda.synchronize()
    assert rc == _lib.RGX_OK and (rgb == 1).all() and (alpha == 0).all()
