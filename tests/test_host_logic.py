"""Host-side logic: the reference-facing interface, row sharding, gradient buffer, gloo all-reduce."""
import inspect
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

from raygaussx_b200 import dist as rdist
from raygaussx_b200 import render_optix as ro
from raygaussx_b200 import scenes


def test_settings_signature_matches_the_reference():
    # positional order of optix_raycasting/render_optix.py:68-71
    expected = ["context", "update", "gas", "program_grps_fwd", "pipeline_fwd", "program_grps_bwd", "pipeline_bwd",
                "dt_step", "dynamic_sampling", "viewpoint_cam", "max_prim_slice", "num_sph_gauss", "iteration", "jitter",
                "rnd_sample", "supersampling", "white_background", "hit_prim_idx"]
    params = list(inspect.signature(ro.RenderOptixSettings.__init__).parameters)[1:]
    assert params[:len(expected)] == expected
    s = ro.RenderOptixSettings(1, False, 3, 4, 5, 6, 7, 0.01, True, "cam", 512, 0, 9, False, 0, (2, 1), True, "buf")
    assert (s.context, s.gas, s.dt_step, s.viewpoint_cam, s.supersampling, s.hit_prim_idx) == (1, 3, 0.01, "cam", (2, 1), "buf")
    assert s.white_background is True and s.max_prim_slice == 512


def test_reference_import_path_resolves():
    from optix_raycasting import optix_utils as u_ox
    from optix_raycasting import render_optix as r_ox
    assert r_ox.RenderOptixFunction is ro.RenderOptixFunction
    assert u_ox.SIGMA_THRESHOLD == 0.1


def test_function_rejects_cpu_tensors():
    sc = scenes.tiny_scene(n=8, width=2, height=2)
    st = ro.RenderOptixSettings(None, False, None, None, None, None, None, 0.01, False, sc.cameras[0], 16, 0)
    with pytest.raises((ValueError, RuntimeError)):
        ro.RenderOptixFunction.apply(*sc.tensors(), st)


def test_camera_struct_follows_the_launch_parameter_fill():
    cam = scenes.SimpleCamera((2.0, -3.0, 1.0), width=40, height=20)
    c = ro.camera_struct(cam, supersampling=(2, 3))
    assert (c.width, c.height) == (80, 60)
    wvt = cam.world_view_transform
    assert list(c.u) == pytest.approx(wvt[:3, 0].tolist())
    assert list(c.w) == pytest.approx(wvt[:3, 2].tolist())
    assert list(c.eye) == pytest.approx(cam.camera_center.tolist())
    # looking at the origin: forward axis points from the eye to the origin
    fwd = -cam.camera_center / cam.camera_center.norm()
    assert list(c.w) == pytest.approx(fwd.tolist(), abs=1e-6)


@pytest.mark.parametrize("views,height,world", [(20, 828, 1), (20, 828, 2), (20, 828, 8), (3, 5, 4), (1, 7, 3), (2, 1, 5)])
def test_shard_rows_partitions_every_row_once(views, height, world):
    seen = []
    sizes = []
    for rank in range(world):
        blocks = rdist.shard_rows(views, height, rank, world)
        sizes.append(sum(b.row_end - b.row_begin for b in blocks))
        for b in blocks:
            assert 0 <= b.row_begin < b.row_end <= height and 0 <= b.view < views
            seen += [(b.view, r) for r in range(b.row_begin, b.row_end)]
    assert sorted(seen) == [(v, r) for v in range(views) for r in range(height)]
    assert max(sizes) - min(sizes) <= 1


def test_shard_rows_eight_ranks_split_views_by_rows():
    blocks = rdist.shard_rows(20, 828, 0, 8)          # 2.5 views per rank
    assert [(b.view, b.row_begin, b.row_end) for b in blocks] == [(0, 0, 828), (1, 0, 828), (2, 0, 414)]


def test_grad_buffer_layout():
    gb = rdist.GradBuffer(10, 16, "cpu")
    assert gb.flat.numel() == 10 * 59
    p, s, q, d, c = gb.tensors()
    assert p.shape == (10, 3) and q.shape == (10, 4) and d.shape == (10,) and c.shape == (10, 3, 16)
    c[3, 1, 5] = 7.0
    assert gb.flat[10 * 11 + 3 * 48 + 16 + 5] == 7.0
    gb.zero_()
    assert gb.flat.abs().sum() == 0


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _gloo_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.distributed.init_process_group("gloo", rank=rank, world_size=world)
    gb = rdist.GradBuffer(5, 4, "cpu")
    # every rank contributes the rows it owns: stand-in for the per-rank backward
    for b in rdist.shard_rows(3, 4, rank, world):
        gb.views["positions"][b.view] += float(b.row_end - b.row_begin)
    gb.all_reduce()
    out[rank] = gb.views["positions"][:3, 0].tolist()
    torch.distributed.destroy_process_group()


def test_all_reduce_joins_the_ranks_gloo():
    world = 2
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_gloo_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    assert out[0] == out[1] == [4.0, 4.0, 4.0]      # every view's rows were covered exactly once


class _RecordingRenderer:
    """Stands in for the CUDA renderer: writes a colour that depends on (view, row), adds the loss gradient's sum
    per row range to the first gradient tensor, and keeps the order of calls."""

    def __init__(self):
        self.calls = []

    def build(self, *a):
        self.calls.append(("build",))

    def forward(self, *args):
        cam, march = args[-2], args[-1]
        self.calls.append(("forward", cam.view, march["rows"]))
        rgb = torch.zeros(cam.width * cam.height, 3)
        lo, hi = march["rows"]
        rgb[lo * cam.width:hi * cam.width] = 0.25 + cam.view
        return rgb, None, None

    def hint_next_view(self, cam, march):
        self.calls.append(("hint", cam.view, march["rows"]))

    def backward(self, *args):
        cam, march, rgb, dl, grads = args[-5:]
        self.calls.append(("backward", cam.view, march["rows"]))
        lo, hi = march["rows"]
        grads[0][cam.view, 0] += dl[lo * cam.width:hi * cam.width].sum()


class _Cam:
    def __init__(self, view, width, height):
        self.view, self.width, self.height = view, width, height


def _step_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.distributed.init_process_group("gloo", rank=rank, world_size=world)
    n_views, w, h = 3, 4, 6
    cams = [_Cam(v, w, h) for v in range(n_views)]
    targets = [torch.zeros(w * h, 3) for _ in cams]
    tensors = [torch.zeros(5, 3)] * 8
    march_of = lambda cam, rows, flags: {"rows": rows, "flags": flags}
    res = {}
    for ahead in (False, True):
        r = _RecordingRenderer()
        gb = rdist.GradBuffer(5, 4, "cpu")
        rdist.accumulation_step(r, tensors, cams, targets, march_of, gb, rank=rank, world=world, lists_ahead=ahead)
        res[ahead] = (r.calls, gb.views["positions"][:n_views, 0].tolist())
    out[rank] = res
    torch.distributed.destroy_process_group()


def test_accumulation_step_announces_each_next_block_gloo():
    world = 2
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_step_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    n_views, w, h = 3, 4, 6
    for rank in range(world):
        blocks = rdist.shard_rows(n_views, h, rank, world)
        plain, _ = out[rank][False]
        ahead, _ = out[rank][True]
        assert [c for c in plain if c[0] == "hint"] == []
        want = [("build",)]
        for i, b in enumerate(blocks):
            rows = (b.row_begin, b.row_end)
            want.append(("forward", b.view, rows))
            if i + 1 < len(blocks):       # the next block is announced before this one's backward
                nb = blocks[i + 1]
                want.append(("hint", nb.view, (nb.row_begin, nb.row_end)))
            want.append(("backward", b.view, rows))
        assert ahead == want
        assert [c for c in ahead if c[0] != "hint"] == plain
    # the all-reduced gradient is the whole step's, whichever way it was cut, with or without announcements:
    # sign(colour - 0) / (3 R n_views), three channels, all R rays of a view
    for ahead in (False, True):
        g0, g1 = out[0][ahead][1], out[1][ahead][1]
        assert g0 == g1
        assert g0 == pytest.approx([1.0 / n_views] * n_views, rel=1e-6)


@pytest.mark.parametrize("world", [1, 2, 3, 8])
def test_weighted_shards_cover_every_row_once_and_balance_the_cost(world):
    views, height = 20, 828
    costs = [22.0 + 0.6 * ((7 * v) % 5 - 2) for v in range(views)]          # views differ by a few per cent
    seen, share = [], []
    for rank in range(world):
        blocks = rdist.shard_rows_weighted(costs, height, rank, world)
        share.append(sum((b.row_end - b.row_begin) / height * costs[b.view] for b in blocks))
        for b in blocks:
            assert 0 <= b.row_begin < b.row_end <= height
            seen += [(b.view, r) for r in range(b.row_begin, b.row_end)]
    assert sorted(seen) == [(v, r) for v in range(views) for r in range(height)]
    assert max(share) - min(share) <= 2 * max(costs) / height + 1e-9        # equal up to a row
    # equal costs give the equal-count cuts; degenerate costs fall back to them
    for rank in range(world):
        assert rdist.shard_rows_weighted([1.0] * views, height, rank, world) == rdist.shard_rows(views, height, rank, world)
        assert rdist.shard_rows_weighted([0.0] * views, height, rank, world) == rdist.shard_rows(views, height, rank, world)


def test_view_costs_from_timed_blocks():
    B = rdist.RowBlock
    timed = [(B(0, 0, 10), 5.0), (B(1, 0, 4), 2.0), (B(1, 4, 10), 4.0)]     # view 2 was not timed
    costs = rdist.view_costs_from_blocks(3, 10, timed)
    assert costs[0] == pytest.approx(5.0) and costs[1] == pytest.approx(6.0) and costs[2] == pytest.approx(5.5)
    half = rdist.view_costs_from_blocks(1, 10, [(B(0, 0, 5), 3.0)])          # half a view timed: scaled to the whole
    assert half == [pytest.approx(6.0)]
