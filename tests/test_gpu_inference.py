"""Forward-only entry points on the GPU: inference(), render(), frames() (`-m gpu`).

Same tolerances as the training forward: 1e-4 on colours against the oracle's golden image, 5e-4 on depth;
the 8-bit frame is bit-exact against the quantisation of the float image and within one step of the oracle's.
"""
import numpy as np
import pytest
import torch

from oracle import oracle
from raygaussx_b200 import _lib
from tests.helpers import FakePointCloud, load_golden, make_scene

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mods():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device: there is no CPU path")
    _lib.lib()
    from raygaussx_b200 import inference, render_optix
    return inference, render_optix


def cloud_and_cam(name):
    sc = make_scene(name)
    dev = torch.device("cuda")
    cam = sc.cameras[0]
    cam.to(dev)
    return sc, FakePointCloud(sc, dev), cam


@pytest.mark.parametrize("name", ["small_static", "small_dynamic_white", "small_lobes_deg2"])
def test_inference_matches_the_oracle_image(mods, name):
    inf, _ = mods
    sc, pc, cam = cloud_and_cam(name)
    g = load_golden(name)
    m = sc.march
    h, w = cam.image_height, cam.image_width
    golden = np.clip(g["oracle_rgb"].reshape(h, w, 3), 0, 1)
    cam.original_image = torch.from_numpy(golden).permute(2, 0, 1).float()
    psnr, gts, imgs, ms = inf.inference(None, pc, [cam, cam], m.max_prim_slice, m.dt_step, 0, (1, 1),
                                        m.white_background, m.dynamic_sampling)
    assert len(psnr) == len(gts) == len(imgs) == 2 and ms > 0
    assert imgs[0].shape == (h, w, 3) and imgs[0].dtype == np.float32
    steady = (g["oracle_margin"] > 3e-5).reshape(h, w)
    assert np.abs(imgs[0] - golden).max(axis=2)[steady].max() <= 1e-4
    assert np.array_equal(imgs[0], imgs[1])
    assert psnr[0] > 60
    out = inf.render(pc, [cam], m.max_prim_slice, m.dt_step, 0, (1, 1), m.white_background, m.dynamic_sampling)
    assert len(out) == 1 and np.array_equal(out[0], imgs[0])


def test_supersampled_inference_is_the_mean_of_the_fine_image(mods):
    inf, ro = mods
    sc, pc, cam = cloud_and_cam("small_static")
    m = sc.march
    cam.original_image = torch.zeros(3, cam.image_height, cam.image_width)
    _, _, imgs, _ = inf.inference(None, pc, [cam], m.max_prim_slice, m.dt_step, 0, (2, 3), m.white_background,
                                  m.dynamic_sampling)
    # the same rays, rendered directly at the fine resolution
    tens = [t.contiguous() for t in (pc.positions, pc.get_scale(), pc.get_normalized_quaternion(), pc.get_density(),
                                     pc.get_color_features(), pc.sph_gauss_features, pc.get_bandwidth_sharpness(),
                                     pc.get_normalized_lobe_axis())]
    cs = ro.camera_struct(cam, (2, 3))
    assert (cs.width, cs.height) == (2 * cam.image_width, 3 * cam.image_height)
    r = ro.get_renderer()
    r.build(*tens[:4])
    st = ro.RenderOptixSettings(None, False, None, None, None, None, None, m.dt_step, m.dynamic_sampling, cam,
                                m.max_prim_slice, 0, supersampling=(2, 3), white_background=m.white_background)
    fine, _, _ = r.forward(*tens, cs, ro._settings_march(st, cs))
    fine = fine.reshape(cam.image_height, 3, cam.image_width, 2, 3).mean(dim=(1, 3)).cpu().numpy().clip(0, 1)
    assert np.abs(fine - imgs[0]).max() < 1e-6


def test_culling_keeps_the_image_when_everything_is_in_view(mods):
    inf, _ = mods
    sc, pc, cam = cloud_and_cam("small_static")
    m = sc.march
    cam.original_image = torch.zeros(3, cam.image_height, cam.image_width)
    args = (None, pc, [cam], m.max_prim_slice, m.dt_step, 0, (1, 1), m.white_background, m.dynamic_sampling)
    _, _, plain, _ = inf.inference(*args)
    _, _, culled, _ = inf.inference(*args, culling=True)
    # the scene of the small cases lies inside 1.3 x the field of view: same Gaussians, same order of sums
    # up to the permutation the selection applies
    assert np.abs(plain[0] - culled[0]).max() < 2e-6


@pytest.mark.parametrize("name", ["small_static", "config1"])
def test_frames_are_the_quantised_forward_and_its_depth(mods, name):
    inf, ro = mods
    sc, pc, cam = cloud_and_cam(name)
    g = load_golden(name)
    m = sc.march
    h, w = cam.image_height, cam.image_width
    (frame, depth), = inf.frames(pc, [cam], m.max_prim_slice, m.dt_step, m.dynamic_sampling,
                                 transmittance_eps=m.transmittance_eps)
    assert frame.shape == (h, w, 4) and frame.dtype == torch.uint8 and depth.shape == (h, w)
    tens = [t.contiguous() for t in (pc.positions, pc.get_scale(), pc.get_normalized_quaternion(), pc.get_density(),
                                     pc.get_color_features(), pc.sph_gauss_features, pc.get_bandwidth_sharpness(),
                                     pc.get_normalized_lobe_axis())]
    cs = ro.camera_struct(cam)
    r = ro.get_renderer()
    march = ro.Renderer._march(m.dt_step, m.dynamic_sampling, m.max_prim_slice, False, m.transmittance_eps, None,
                               cs.height, 0)
    rgb, _, dref = r.forward(*tens, cs, march, want_depth=True)
    want = oracle.quantize_frame(rgb.cpu().numpy().reshape(h, w, 3))
    assert np.array_equal(frame.cpu().numpy(), want)                       # bytes: bit-exact
    assert torch.equal(depth.reshape(-1), dref)
    if not m.white_background:                                             # the viewer composites over black
        steady = (g["oracle_margin"] > 3e-5).reshape(h, w)
        oq = oracle.quantize_frame(g["oracle_rgb"].reshape(h, w, 3))
        diff = np.abs(frame.cpu().numpy().astype(np.int32) - oq.astype(np.int32))
        assert diff[steady].max() <= 1                                     # a colour within 1e-4 of a step may cross it
        assert (diff[steady] > 0).mean() < 0.01
        assert np.abs(depth.cpu().numpy().reshape(-1) - g["oracle_depth"])[steady.reshape(-1)].max() <= 5e-4
