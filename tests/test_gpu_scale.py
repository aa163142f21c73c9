"""Full-size checks through size-independent properties (B200, `-m gpu`).

The oracle cannot run 3,000,000 Gaussians x 10^6 rays; at that size the CUDA path
is checked against itself through properties that hold exactly or to rounding:
determinism, equality of tiled and per-ray searches on a crop, row-sharded renders
equal to the whole, linearity in the background, alpha in [0,1], and a finite
gradient whose row-sharded accumulation equals the whole-image gradient.
"""
import pytest
import torch

from raygaussx_b200 import _lib, scenes

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def big():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    from raygaussx_b200 import render_optix as ro
    dev = torch.device("cuda")
    sc = scenes.unbounded_scene(n=3_000_000, n_cameras=2, width=1256, height=828)
    tens = [t.to(dev).contiguous() for t in sc.tensors()]
    cam = sc.cameras[1]
    cam.to(dev)
    r = ro.get_renderer()
    r.build(*tens[:4])
    return ro, r, sc, tens, ro.camera_struct(cam)


def march(ro, sc, cs, flags=0, rows=None, white=None):
    m = sc.march
    return ro.Renderer._march(m.dt_step, m.dynamic_sampling, m.max_prim_slice,
                              m.white_background if white is None else white, m.transmittance_eps, rows, cs.height, flags)


def test_full_size_forward_properties(big):
    ro, r, sc, tens, cs = big
    rgb, alpha, depth = r.forward(*tens, cs, march(ro, sc, cs), want_alpha=True, want_depth=True)
    again, _, _ = r.forward(*tens, cs, march(ro, sc, cs))
    assert torch.equal(rgb, again), "two identical launches must give identical images"
    assert torch.isfinite(rgb).all() and torch.isfinite(depth).all()
    assert alpha.min() >= 0 and alpha.max() <= 1 + 1e-6
    # white minus black background equals the final transmittance
    white, _, _ = r.forward(*tens, cs, march(ro, sc, cs, white=True))
    assert ((white - rgb) - (1 - alpha)[:, None]).abs().max() < 2e-6
    # a crop of rows: list march and per-ray search agree to rounding; sharded rows equal the whole
    rows = (400, 408)
    lo, hi = rows[0] * cs.width, rows[1] * cs.width
    a = torch.zeros_like(rgb)
    b = torch.zeros_like(rgb)
    r.forward(*tens, cs, march(ro, sc, cs, rows=rows), out=a)
    r.forward(*tens, cs, march(ro, sc, cs, rows=rows, flags=_lib.FLAG_PER_RAY_SEARCH), out=b)
    assert torch.equal(a[lo:hi], rgb[lo:hi])                       # a row shard equals the whole image bit for bit
    assert (a[lo:hi] - b[lo:hi]).abs().max().item() < 1e-5          # list march vs per-ray search: summation order only
    r.reset_counters()
    r.forward(*tens, cs, march(ro, sc, cs, flags=_lib.FLAG_COUNT_WORK))
    c = r.read_counters()
    assert c["rays"] == cs.width * cs.height and c["stack_overflows"] == 0


def test_full_size_backward_properties(big):
    ro, r, sc, tens, cs = big
    rgb, _, _ = r.forward(*tens, cs, march(ro, sc, cs))
    dl = torch.sign(rgb - 0.5) / (3 * rgb.shape[0])
    whole = [torch.zeros_like(t) for t in tens]
    r.backward(*tens, cs, march(ro, sc, cs), rgb, dl, tuple(whole))
    parts = [torch.zeros_like(t) for t in tens]
    for rows in ((0, 300), (300, 828)):
        r.backward(*tens, cs, march(ro, sc, cs, rows=rows, flags=_lib.FLAG_ACCUMULATE), rgb, dl, tuple(parts))
    torch.cuda.synchronize()
    # Which of the two is right?  A reference with far less rounding: the image in 46 bands of 18 rows, each band's
    # gradient accumulated on its own (a Gaussian then sums 46 times fewer fp32 terms per band) and the bands added
    # up in float64.  Only the order and grouping of additions differ between the three.
    ref64 = [torch.zeros_like(t, dtype=torch.float64) for t in tens[:5]]
    for lo in range(0, cs.height, 18):
        band = [torch.zeros_like(t) for t in tens]
        r.backward(*tens, cs, march(ro, sc, cs, rows=(lo, min(lo + 18, cs.height))), rgb, dl, tuple(band))
        for acc, g in zip(ref64, band[:5]):
            acc += g.double()
    torch.cuda.synchronize()
    report = []
    for nm, a, b, ref in zip(("positions", "scales", "quaternions", "densities", "color_features"), whole[:5], parts[:5], ref64):
        assert torch.isfinite(a).all()
        assert a.abs().sum() > 0
        scale = ref.abs().max()
        ea, eb = ((a.double() - ref).abs().max() / scale).item(), ((b.double() - ref).abs().max() / scale).item()
        ab = ((a - b).abs().max() / a.abs().max()).item()
        report.append(f"{nm}: whole vs banded-fp64 {ea:.2e}, two parts vs banded-fp64 {eb:.2e}, whole vs two parts {ab:.2e}")
    print("\n".join(report))
    for nm, a, b, ref in zip(("positions", "scales", "quaternions", "densities", "color_features"), whole[:5], parts[:5], ref64):
        scale = ref.abs().max()
        # Gaussians that cover much of the image sum ~10^5 contributions of both signs in fp32 atomics; measured
        # 3e-5 .. 7e-5 for all three comparisons, far inside the 1e-3 the gradients are held to
        assert ((a.double() - ref).abs().max() / scale).item() < 3e-4, report
        assert ((b.double() - ref).abs().max() / scale).item() < 3e-4, report
        assert ((a - b).abs().max() / a.abs().max()).item() < 3e-4, report


@pytest.mark.parametrize("cam_index", [0, 1, 2])
def test_tile_lists_find_every_hit_with_the_camera_inside_the_scene(cam_index):
    """The unbounded scene surrounds its cameras: Gaussians behind the eye, Gaussians that straddle the eye
    plane, Gaussians that fill the view.  The per-view tile lists must still hold every hit of every ray:
    same hit hash and counts as the per-ray search of the hierarchy."""
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device: there is no CPU path")
    from raygaussx_b200 import render_optix as ro
    dev = torch.device("cuda")
    sc = scenes.unbounded_scene(n=200_000, n_cameras=3, width=314, height=207)
    tens = [t.to(dev).contiguous() for t in sc.tensors()]
    cam = sc.cameras[cam_index]
    cam.to(dev)
    cs = ro.camera_struct(cam)
    r = ro.get_renderer()
    r.build(*tens[:4])
    got = {}
    for label, flags in (("lists", 0), ("per_ray", _lib.FLAG_PER_RAY_SEARCH)):
        r.reset_counters()
        rgb, _, _ = r.forward(*tens, cs, march(ro, sc, cs, flags=flags | _lib.FLAG_COUNT_WORK))
        got[label] = (rgb.clone(), r.read_counters())
    a, b = got["lists"][1], got["per_ray"][1]
    assert a["hits_hash"] == b["hits_hash"]
    for k in ("rays", "slabs", "slabs_hit", "closest_queries", "hits", "overflow_slabs"):
        assert a[k] == b[k], k
    # hits are met in a different order, sums differ in the last bit, and with them now and then the step size:
    # a sample at the very edge of an ellipsoid may fall on the other side
    assert abs(a["pairs_inside"] - b["pairs_inside"]) <= 1e-6 * b["pairs_inside"]
    assert a["hits"] > 50 * a["rays"]                      # the case is not trivial
    assert (got["lists"][0] - got["per_ray"][0]).abs().max().item() < 1e-5
    # a recorded forward and its replayed backward against a searched backward, at this size
    rgb, _, _ = r.forward(*tens, cs, march(ro, sc, cs, flags=_lib.FLAG_SAVE_HITS))
    dl = torch.sign(rgb - 0.5) / (3 * rgb.shape[0])
    replayed = [torch.zeros_like(t) for t in tens]
    r.backward(*tens, cs, march(ro, sc, cs), rgb, dl, tuple(replayed))
    r.forward(*tens, cs, march(ro, sc, cs, flags=_lib.FLAG_SAVE_HITS, rows=(0, 8)))      # overwrites the recording
    searched = [torch.zeros_like(t) for t in tens]
    r.backward(*tens, cs, march(ro, sc, cs), rgb, dl, tuple(searched))
    torch.cuda.synchronize()
    worst = max(((x - y).abs().max() / y.abs().max().clamp_min(1e-30)).item() for x, y in zip(replayed[:5], searched[:5]))
    print(f"camera {cam_index}: replayed vs searched gradients, worst max-normalised difference {worst:.2e}")
    assert worst < 1e-3


@pytest.mark.parametrize("cam_index", [0, 1])
def test_tile_lists_hold_every_hit_of_needle_like_gaussians(cam_index):
    """The stress recipe at reduced size: anisotropy up to 100:1 at random orientations, dense clusters, early
    termination at 1e-4.  Needles project to thin diagonal footprints, the hardest case for the tile
    rectangles and the per-(tile, Gaussian) ranges; the hit sets must still equal the per-ray search's."""
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device: there is no CPU path")
    from raygaussx_b200 import render_optix as ro
    dev = torch.device("cuda")
    sc = scenes.stress_scene(n_uniform=60_000, n_cluster=10_000, n_cameras=2, width=320, height=180)
    tens = [t.to(dev).contiguous() for t in sc.tensors()]
    cam = sc.cameras[cam_index]
    cam.to(dev)
    cs = ro.camera_struct(cam)
    r = ro.get_renderer()
    r.build(*tens[:4])
    got = {}
    for label, flags in (("lists", 0), ("per_ray", _lib.FLAG_PER_RAY_SEARCH)):
        r.reset_counters()
        rgb, alpha, depth = r.forward(*tens, cs, march(ro, sc, cs, flags=flags | _lib.FLAG_COUNT_WORK), want_alpha=True,
                                      want_depth=True)
        got[label] = (rgb.clone(), alpha.clone(), depth.clone(), r.read_counters())
    a, b = got["lists"][3], got["per_ray"][3]
    assert a["hits_hash"] == b["hits_hash"]
    for k in ("rays", "slabs", "slabs_hit", "closest_queries", "hits", "overflow_slabs"):
        assert a[k] == b[k], k
    assert a["hits"] > 10 * a["rays"]
    for x, y in zip(got["lists"][:3], got["per_ray"][:3]):
        assert (x - y).abs().max().item() < 2e-5
    # the viewer's frame of the same view: bytes of the float image
    frame, _ = r.forward_frame(*tens, cs, march(ro, sc, cs))
    want = (got["lists"][0].clamp(0, 1) * 256).to(torch.int32).clamp(max=255).reshape(cs.height, cs.width, 3)
    assert (frame[..., :3].to(torch.int32) - want).abs().max().item() <= 1      # one step where the two images round apart


def two_depth(r, min_pairs, budget):
    import ctypes as C
    _lib.check(r._ctx, r._lib.rgx_debug_two_depth(r._ctx, C.c_int(min_pairs), C.c_int(budget)))


def read_two_depth(r):
    import ctypes as C
    out = (C.c_longlong * 4)()
    _lib.check(r._ctx, r._lib.rgx_read_two_depth(r._ctx, out))
    return list(out)


@pytest.mark.parametrize("kind,budget", [("stress", 1), ("stress", 8), ("stress", 64), ("unbounded", 2), ("unbounded", 16),
                                         ("tiny", 1), ("tiny", 4)])
def test_two_depth_forward_is_bit_identical(kind, budget):
    """Lists made in two depths, march in two phases: the same slabs meet the same hits in the same order, so
    colour, alpha and depth equal the one-depth march bit for bit -- whatever share of the rays has to go on
    into the second depth."""
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device: there is no CPU path")
    from raygaussx_b200 import render_optix as ro
    dev = torch.device("cuda")
    if kind == "stress":
        sc = scenes.stress_scene(n_uniform=60_000, n_cluster=10_000, n_cameras=2, width=320, height=180)
    elif kind == "unbounded":
        sc = scenes.unbounded_scene(n=200_000, n_cameras=2, width=314, height=207)
    else:
        sc = scenes.tiny_scene(n=512, width=40, height=24, log_scale_mean=-2.5, dynamic_sampling=True, dt_step=0.005)
    tens = [t.to(dev).contiguous() for t in sc.tensors()]
    r = ro.Renderer(dev)
    r.build(*tens[:4])
    try:
        for cam in sc.cameras[:2]:
            cam.to(dev)
            cs = ro.camera_struct(cam)
            r.build(*tens[:4])
            two_depth(r, -1, 0)                                   # off
            want = r.forward(*tens, cs, march(ro, sc, cs), want_alpha=True, want_depth=True)
            assert read_two_depth(r) == [0, 0, 0, 0]
            r.build(*tens[:4])                                    # a new build: the next forward makes its lists anew
            two_depth(r, 0, budget)                               # forced, `budget` pairs per ray in the first depth
            got = r.forward(*tens, cs, march(ro, sc, cs), want_alpha=True, want_depth=True)
            emitted, first, stopped, second = read_two_depth(r)
            for a, b in zip(want, got):
                assert torch.equal(a, b)
            if emitted:                                           # (a budget that covers every pair falls back to one depth)
                assert 0 < first < emitted and second <= emitted
                assert (stopped == 0) == (second == 0)
            # a row range through the same path
            rows = (8, cs.height - 3)
            part = torch.zeros_like(want[0])
            r.forward(*tens, cs, march(ro, sc, cs, rows=rows), out=part)
            lo, hi = rows[0] * cs.width, rows[1] * cs.width
            assert torch.equal(part[lo:hi], want[0][lo:hi])
            read_two_depth(r)                                     # clears the figures of the row-range forward
    finally:
        two_depth(r, 48, 16)
        del r


@pytest.mark.parametrize("kind", ["tiny", "unbounded"])
def test_lists_made_ahead_change_nothing(kind):
    """Tile lists of an announced view, made on the context's own stream beside the backward of the view before:
    the announced forward gives the image it gives without the announcement bit for bit, the accumulated
    gradients agree to the order of the atomic additions, and a wrong announcement is harmless."""
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device: there is no CPU path")
    from raygaussx_b200 import dist as rdist
    from raygaussx_b200 import render_optix as ro
    dev = torch.device("cuda")
    if kind == "unbounded":
        sc = scenes.unbounded_scene(n=200_000, n_cameras=3, width=314, height=207)
    else:
        sc = scenes.tiny_scene(n=512, width=40, height=24, log_scale_mean=-2.5, dynamic_sampling=True, dt_step=0.005)
    tens = [t.to(dev).contiguous() for t in sc.tensors()]
    r = ro.Renderer(dev)
    cams = []
    for cam in sc.cameras[:3]:
        cam.to(dev)
        cams.append(ro.camera_struct(cam))
    if len(cams) == 1:                       # one camera: the blocks of a step are then row ranges of it
        views, world = [cams[0]] * 3, 2      # rank 0 of 2: views 0 and half of view 1
    else:
        views, world = cams, 1
    rays = views[0].width * views[0].height
    g = torch.Generator(device="cpu").manual_seed(5)
    targets = [torch.rand(rays, 3, generator=g).to(dev) for _ in views]
    march_of = lambda cam, rows, flags: march(ro, sc, cam, flags=flags, rows=rows)
    n = tens[0].shape[0]
    plain, ahead = rdist.GradBuffer(n, 16, dev), rdist.GradBuffer(n, 16, dev)
    blocks = rdist.shard_rows(len(views), views[0].height, 0, world)
    assert len(blocks) >= 2
    rdist.accumulation_step(r, tens, views, targets, march_of, plain, rank=0, world=world, lists_ahead=False)
    assert r.lists_made_ahead() == 0
    rdist.accumulation_step(r, tens, views, targets, march_of, ahead, rank=0, world=world, lists_ahead=True)
    torch.cuda.synchronize()
    assert r.lists_made_ahead() == len(blocks) - 1
    for name in rdist.GRAD_FIELDS:
        a, b = plain.views[name], ahead.views[name]
        assert torch.isfinite(b).all() and a.abs().sum() > 0
        assert ((a - b).abs().max() / a.abs().max()).item() < 1e-4, name

    # forward of the announced view: bit-identical; recording and replay as without the announcement
    first, second = blocks[0], blocks[1]
    c0, c1 = views[first.view], views[second.view]
    m0 = march_of(c0, (first.row_begin, first.row_end), _lib.FLAG_SAVE_HITS)
    m1 = march_of(c1, (second.row_begin, second.row_end), _lib.FLAG_SAVE_HITS)
    r.build(*tens[:4])
    want = torch.zeros(rays, 3, device=dev)
    r.forward(*tens, c1, m1, out=want)
    r.build(*tens[:4])
    rgb0 = torch.zeros(rays, 3, device=dev)
    r.forward(*tens, c0, m0, out=rgb0)
    dl = torch.sign(rgb0 - targets[0]) / (3 * rays)
    grads = [torch.zeros_like(t) for t in tens]
    made = r.lists_made_ahead()
    r.hint_next_view(c1, m1)
    r.backward(*tens, c0, m0, rgb0, dl, tuple(grads))
    assert r.lists_made_ahead() == made + 1
    got = torch.zeros(rays, 3, device=dev)
    r.forward(*tens, c1, m1, out=got)
    assert torch.equal(got, want)

    # an announcement that does not come true: the next forward makes its own lists
    r.hint_next_view(c1, m1)
    r.backward(*tens, c1, m1, got, dl, tuple(grads))      # (c1's lists are current: nothing to make)
    assert r.lists_made_ahead() == made + 1
    r.hint_next_view(c1, m1)
    r.forward(*tens, c0, m0, out=rgb0)
    r.backward(*tens, c0, m0, rgb0, dl, tuple(grads))      # makes c1's lists ...
    assert r.lists_made_ahead() == made + 2
    other = torch.zeros(rays, 3, device=dev)
    r.forward(*tens, c0, m0, out=other)                    # ... but c0 is rendered again
    assert torch.equal(other, rgb0)
    r.hint_next_view(None, None)


def test_lists_up_to_a_horizon_change_nothing(big):
    """A recording forward emits and sorts only the pairs that begin nearest to the eye; the image, the recording and
    the gradients must be those of the complete lists -- bit for bit while every ray ends before the horizon, and to
    summation rounding when the budget is so small that rays reach it and are finished by the per-ray search."""
    ro, r, sc, tens, cs = big
    r.build(*tens[:4])                              # other tests of this module built their own scenes meanwhile
    save = march(ro, sc, cs, flags=_lib.FLAG_SAVE_HITS)

    def run(budget):
        r.near_lists(budget)                        # also forgets the cached lists
        rgb, _, _ = r.forward(*tens, cs, save)
        rgb = rgb.clone()
        stats = r.near_lists()
        dl = torch.sign(rgb - 0.5) / (3 * rgb.shape[0])
        grads = [torch.zeros_like(t) for t in tens]
        r.backward(*tens, cs, march(ro, sc, cs), rgb, dl, tuple(grads))
        torch.cuda.synchronize()
        return rgb, grads, stats

    full_rgb, full_grads, st0 = run(0)
    assert st0["views"] == 0
    near_rgb, near_grads, st1 = run(5)
    assert st1["views"] == 1 and st1["views_with_rays_beyond"] == 0 and st1["pairs_kept"] * 2 < st1["pairs_estimated"]
    assert torch.equal(near_rgb, full_rgb)
    again_rgb, again_grads, st2 = run(1)            # one pair per ray: far too shallow
    assert st2["views"] == 1 and st2["views_with_rays_beyond"] == 1
    assert (again_rgb - full_rgb).abs().max().item() < 2e-5
    for a, b, c in zip(full_grads[:5], near_grads[:5], again_grads[:5]):
        scale = a.abs().max()
        assert ((a - b).abs().max() / scale).item() < 3e-4 and ((a - c).abs().max() / scale).item() < 3e-4
    # the budget was doubled after that view; put the default back for the tests that follow
    r.near_lists(5)
    # a forward without recording on the cached near lists, and a counting forward (which wants complete lists)
    r.forward(*tens, cs, save)
    plain, _, _ = r.forward(*tens, cs, march(ro, sc, cs))
    assert torch.equal(plain, full_rgb)
    r.reset_counters()
    counted, _, _ = r.forward(*tens, cs, march(ro, sc, cs, flags=_lib.FLAG_COUNT_WORK))
    assert torch.equal(counted, full_rgb) and r.read_counters()["rays"] == cs.width * cs.height


@pytest.mark.parametrize("kind,budget", [("stress", 2), ("stress", 4), ("unbounded", 2), ("unbounded", 12), ("tiny", 2),
                                         ("unbounded_mid", 3)])
def test_lists_up_to_a_horizon_on_small_and_awkward_views(kind, budget):
    """The culled emission on the views that are hardest for it -- the camera inside the scene (Gaussians that
    straddle the eye plane or fill the view), needles at random orientations, a view of 960 rays -- with the
    threshold on the view's size taken away: whatever the budget, whether the view has to be marched again or not,
    a recording forward gives the image of complete lists (bit for bit where no ray reaches the horizon, to summation
    rounding where some are finished by the per-ray search) and its backward the same gradients.  (Views of this size
    either get complete lists after all or have rays beyond the horizon; lists that stop at a horizon and suffice
    need the large scene of test_lists_up_to_a_horizon_change_nothing.)"""
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device: there is no CPU path")
    from raygaussx_b200 import render_optix as ro
    dev = torch.device("cuda")
    if kind == "stress":
        sc = scenes.stress_scene(n_uniform=60_000, n_cluster=10_000, n_cameras=2, width=320, height=180)
    elif kind == "unbounded":
        sc = scenes.unbounded_scene(n=200_000, n_cameras=3, width=314, height=207)
    elif kind == "unbounded_mid":
        sc = scenes.unbounded_scene(n=1_000_000, n_cameras=3, width=628, height=414)
    else:
        sc = scenes.tiny_scene(n=512, width=40, height=24, log_scale_mean=-2.5, dynamic_sampling=True, dt_step=0.005)
    tens = [t.to(dev).contiguous() for t in sc.tensors()]
    r = ro.Renderer(dev)
    r.build(*tens[:4])
    try:
        for cam in sc.cameras[:3]:
            cam.to(dev)
            cs = ro.camera_struct(cam)
            save = march(ro, sc, cs, flags=_lib.FLAG_SAVE_HITS)
            results = []
            for b in (0, budget):
                r.near_lists(b, 0)                            # also forgets the cached lists
                rgb, alpha, depth = r.forward(*tens, cs, save, want_alpha=True, want_depth=True)
                rgb, alpha, depth = rgb.clone(), alpha.clone(), depth.clone()
                st = r.near_lists()
                dl = torch.sign(rgb - 0.5) / (3 * rgb.shape[0])
                grads = [torch.zeros_like(t) for t in tens]
                r.backward(*tens, cs, march(ro, sc, cs), rgb, dl, tuple(grads))
                torch.cuda.synchronize()
                results.append((rgb, alpha, depth, grads, st))
            full, near = results
            assert full[4]["views"] == 0
            for a, b2, tol in zip(full[:3], near[:3], (2e-5, 2e-5, 2e-4)):
                if near[4]["views_with_rays_beyond"] == 0:
                    assert torch.equal(a, b2)
                else:
                    assert (a - b2).abs().max().item() < tol * max(1.0, a.abs().max().item())
            for a, b2 in zip(full[3][:5], near[3][:5]):
                scale = a.abs().max().clamp_min(1e-30)
                assert ((a - b2).abs().max() / scale).item() < 3e-4
            if near[4]["views"] == 1:
                assert near[4]["pairs_kept"] < near[4]["pairs_estimated"]
            print(f"{kind} budget {budget}: {near[4]}")
    finally:
        r.near_lists(5, 1 << 21)
        del r
