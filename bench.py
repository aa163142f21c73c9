#!/usr/bin/env python
"""Benchmark of the differentiable Gaussian ray-marching path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload ("unbounded-3M"): the seeded 3,000,000-Gaussian unbounded scene,
1256x828 pinhole cameras on a ring, SH degree 3, dynamic sampling, hit cap 512 --
synthetic, with the shape of a Mip-NeRF-360 scene.  One *step* is one training
step with gradient accumulation over 20 views: acceleration-structure build, then
per view colour evaluation, forward march, L1 loss gradient, backward march and
gradient finalise, accumulated into one flat gradient buffer.  With N GPUs the 20
views' image rows are split evenly over the ranks (every rank holds all Gaussians)
and one NCCL all-reduce of the gradient buffer ends the step, so total work is
fixed (strong scaling).

Printed JSON line (rank 0): ``value`` = forward+backward Mrays/s of the whole job
with all inputs resident in HBM; ``e2e`` = the same through the reference-facing
autograd entry point with the target images copied from pinned host memory and the
loss read back every step; ``roofline`` for the forward march kernel (the dominant one);
``cpu_baseline`` = the reference's own device code compiled for the host CPU
(oracle/_ref) on a bounded sample of the same workload.

``--impl reference`` times that CPU build alone, on all host threads.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N_VIEWS = 20
# DRAM bytes of one recording forward launch per byte it records, from ncu captures (profiles/): the recording is
# written once, the Gaussian records and the lists stream through once
TRAFFIC_PER_RECORDED_BYTE = 1.018
WORKLOAD = "unbounded-3M"
METRIC = "fwd+bwd Mrays/s (3M Gaussians, 1256x828)"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="rgx", choices=["rgx", "reference"])
    ap.add_argument("--gaussians", type=int, default=3_000_000, help="for quick runs only; the headline is 3,000,000")
    ap.add_argument("--width", type=int, default=1256)
    ap.add_argument("--height", type=int, default=828)
    ap.add_argument("--views", type=int, default=N_VIEWS)
    ap.add_argument("--cpu-sample", type=str, default="auto",
                    help="image size of the CPU sample, WxH (auto: 20x13 for the baseline leg; for --impl reference "
                         "sized so that the whole run takes about two minutes)")
    ap.add_argument("--no-secondary", action="store_true", help="skip the 300k-object and 7M-stress records")
    ap.add_argument("--weighted-cuts", action="store_true",
                    help="N > 1: cut the rows by the per-view cost measured in the second warm-up step instead of by count "
                         "(measured at N = 4: 110.5 ms per step against 110.0 with equal counts -- whole views per rank "
                         "beat balanced fractions of views, each of which pays its own colour pass and tile lists)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    return ap.parse_args()


# ----------------------------------------------------------------------------- clocks
class ClockSampler:
    """nvidia-smi clock/throttle samples during the timed region."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu)], stdout=open(self.path, "w"),
                                         stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1])); mx.append(float(f[2]))
                except ValueError:
                    continue
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            sm.sort()
            out.update(sm_mhz=sm[len(sm) // 2], sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))
        return out


# ----------------------------------------------------------------------------- CPU reference arm
def host_threads():
    """Threads for the CPU arm, stated explicitly: a launcher such as torchrun exports OMP_NUM_THREADS=1 to
    its workers, which the OpenMP runtime of oracle/_ref would otherwise obey."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except Exception:
        return max(1, os.cpu_count() or 1)


def sample_camera(scene, size):
    """View 0 of the scene at a coarse resolution: same eye, axes and field of view."""
    from raygaussx_b200 import scenes as S
    return S.lowres_camera(scene.cameras[0], size[0], size[1])


def cpu_reference_sample(scene, n_threads=0, size=(20, 13), repeats=1, keep=None):
    """Forward+backward of the reference's own device code (compiled for the CPU,
    OptiX traversal replaced by an exhaustive loop) on a low-resolution image of the
    same scene from the same camera.  Returns (rays, seconds per repeat); ``keep``
    (a dict) receives the colours of the last repeat."""
    import numpy as np
    from oracle import ref_shim
    from raygaussx_b200 import scenes as S
    n_threads = n_threads or host_threads()
    cam = sample_camera(scene, size)
    rays = size[0] * size[1]
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        col, _, ctx = ref_shim.render_forward(*scene.tensors(), cam, scene.march, n_threads=n_threads)
        tgt = S.l1_target(rays).numpy()
        dl = (np.sign(col - tgt) / (3 * rays)).astype(np.float32)
        ref_shim.render_backward(ctx, dl, n_threads=n_threads)
        times.append(time.perf_counter() - t0)
        if keep is not None:
            keep["rgb"] = col
    return rays, times


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import ref_shim
    from raygaussx_b200 import scenes as S
    if not ref_shim.available():
        print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref is not built (run `make -C oracle` where "
                                                              "the reference checkout is present)"}))
        return
    scene = S.unbounded_scene(n=args.gaussians, n_cameras=1, width=args.width, height=args.height)
    cores = host_threads()
    if args.cpu_sample == "auto":
        # a step is a bounded sample of the view, sized from a short calibration so that warm-up + steps take
        # about two minutes whatever K and W are and however many host cores the box has
        _, t_cal = cpu_reference_sample(scene, n_threads=cores, size=(8, 5))
        per_ray = max(t_cal[0] / 40.0, 1e-4)
        budget = 120.0 / max(1, args.steps + args.warmup)
        rays_wanted = int(min(20 * 13, max(6 * 4, budget / per_ray)))
        h = max(4, int(round((rays_wanted * args.height / args.width) ** 0.5)))
        w = max(6, rays_wanted // h)
    else:
        w, h = (int(x) for x in args.cpu_sample.split("x"))
    for _ in range(args.warmup):
        cpu_reference_sample(scene, n_threads=cores, size=(w, h))
    rays, times = cpu_reference_sample(scene, n_threads=cores, size=(w, h), repeats=max(1, args.steps))
    sec = sum(times) / len(times)
    val = rays / sec / 1e6
    sample = f"{w}x{h} rays of view 0 per step, forward+backward, all {args.gaussians} Gaussians, {cores} threads"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": "Mrays/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "gaussians": args.gaussians, "image": f"{args.width}x{args.height}",
                   "sample": sample},
        "cpu_baseline": {"value": val, "unit": "Mrays/s", "cores": cores, "kind": "reference", "sample": sample},
        "e2e": {"value": val, "unit": "Mrays/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


# ----------------------------------------------------------------------------- GPU arm
def main():
    args = parse()
    if args.impl == "reference":
        run_reference_arm(args)
        return

    import torch
    import torch.distributed as dist
    from raygaussx_b200 import _lib, scenes as S
    from raygaussx_b200 import render_optix as ro
    from raygaussx_b200.dist import (GradBuffer, accumulation_step, shard_rows, shard_rows_weighted,
                                     view_costs_from_blocks)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the ray-marching path has no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    # ---- inputs (identical on every rank: seeded CPU generators)
    scene = S.unbounded_scene(n=args.gaussians, n_cameras=200, width=args.width, height=args.height)
    cams_py = scene.cameras[:args.views]
    host_scene = scene
    R = args.width * args.height
    targets_host = [S.l1_target(R, seed=1000 + v).pin_memory() for v in range(args.views)]
    scene_dev_tensors = [t.to(dev).contiguous() for t in host_scene.tensors()]
    for c in cams_py:
        c.to(dev)
    cams = [ro.camera_struct(c) for c in cams_py]
    targets = [t.to(dev, non_blocking=True) for t in targets_host]
    mp = scene.march
    renderer = ro.get_renderer(dev)
    k_sh = scene_dev_tensors[4].shape[2]
    grads = GradBuffer(args.gaussians, k_sh, dev)

    def march_of(cam, rows, flags):
        return ro.Renderer._march(mp.dt_step, mp.dynamic_sampling, mp.max_prim_slice, mp.white_background,
                                  mp.transmittance_eps, rows, cam.height, flags)

    all_blocks = [shard_rows(args.views, args.height, r, world) for r in range(world)]

    def step(events=None):
        accumulation_step(renderer, scene_dev_tensors, cams, targets, march_of, grads, rank=rank, world=world,
                          blocks=all_blocks[rank], block_events=events)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing
    weigh_at = 1 if (world > 1 and args.warmup >= 3 and args.weighted_cuts) else -1
    for w in range(args.warmup):
        if w == weigh_at:
            # the second warm-up step (the first one pays for every first-use allocation), cut into equal row counts,
            # times every block; from then on the rows are cut so that every rank gets an equal share of the measured
            # cost (views differ by a few per cent)
            events = []
            step(events)
            torch.cuda.synchronize()
            mine = [(b, e0.elapsed_time(e1)) for b, e0, e1 in events]
            gathered = [None] * world
            dist.all_gather_object(gathered, mine)
            costs = view_costs_from_blocks(args.views, args.height, [x for g in gathered for x in g])
            all_blocks = [shard_rows_weighted(costs, args.height, r, world) for r in range(world)]
        else:
            step()
    barrier()
    renderer.set_profiling(True)
    renderer.read_kernel_times()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    launches0 = int(_lib.lib().rgx_kernel_launches())
    renderer.near_lists()                 # clears the figures of the warm-up
    ev0.record()
    for _ in range(args.steps):
        step()
    ev1.record()
    barrier()
    gpu_launches = int(_lib.lib().rgx_kernel_launches()) - launches0      # counted by the library at every launch
    near_lists = renderer.near_lists()    # views whose lists stopped at a horizon, and how many had to be marched twice
    ms = ev0.elapsed_time(ev1)
    clocks = sampler.stop() if rank == 0 else None
    ktimes = renderer.read_kernel_times()
    renderer.set_profiling(False)
    t_ms = torch.tensor([ms], device=dev)
    if world > 1:
        dist.all_reduce(t_ms, op=dist.ReduceOp.MAX)
    ms = float(t_ms.item())
    ms_per_step = ms / args.steps
    rays_per_step = args.views * R
    value = rays_per_step / (ms_per_step * 1e-3) / 1e6

    # ---- end to end through the reference-facing autograd entry point
    e2e = None
    if not args.no_e2e:
        params = [t.clone().requires_grad_(True) for t in scene_dev_tensors[:5]] + list(scene_dev_tensors[5:])
        my_blocks = all_blocks[rank]
        loss_host = torch.zeros(1).pin_memory()
        copy_stream = torch.cuda.Stream()

        def e2e_step(plain=False):
            """One accumulation step through RenderOptixFunction.  The parameter tensors are the same, untouched
            leaves for all views of the step, which the entry point recognises by itself (one build per step, as
            the device-resident loop does); each view announces the next one, and the gradients are added into
            the leaves' .grad in place.  plain=True: neither announcement nor in-place accumulation -- the
            reference's own call, nothing added."""
            for p in params[:5]:
                p.grad = None
            with torch.no_grad():
                params[0].add_(0.0)        # what an optimizer step does to the entry point: the parameters were written to,
                                           # so the first view of the step builds the acceleration structure again
            total = torch.zeros((), device=dev)
            # H2D of every block's target rows from pinned memory, on a copy stream beside the kernels (what a
            # data loader does); a block waits for its own copy only
            copy_stream.wait_stream(torch.cuda.current_stream())
            staged = []
            with torch.cuda.stream(copy_stream):
                for b in my_blocks:
                    lo, hi = b.row_begin * args.width, b.row_end * args.width
                    t = targets_host[b.view][lo:hi].to(dev, non_blocking=True)
                    ev = torch.cuda.Event()
                    ev.record(copy_stream)
                    staged.append((t, ev))
            for i, b in enumerate(my_blocks):                                    # this rank's rows of each of its views
                lo, hi = b.row_begin * args.width, b.row_end * args.width
                tgt, ev = staged[i]
                torch.cuda.current_stream().wait_event(ev)
                tgt.record_stream(torch.cuda.current_stream())
                extra = {}
                if not plain:
                    extra["accumulate_leaf_grads"] = True
                    if i + 1 < len(my_blocks):
                        nb = my_blocks[i + 1]
                        extra.update(next_viewpoint_cam=cams_py[nb.view], next_rows=(nb.row_begin, nb.row_end))
                st = ro.RenderOptixSettings(None, False, None, None, None, None, None, mp.dt_step, mp.dynamic_sampling,
                                            cams_py[b.view], mp.max_prim_slice, 0, white_background=mp.white_background,
                                            transmittance_eps=mp.transmittance_eps, rows=(b.row_begin, b.row_end),
                                            **extra)
                img = ro.RenderOptixFunction.apply(*params, st)
                loss = (img[lo:hi] - tgt).abs().sum() / float(3 * R * args.views)
                loss.backward()
                total = total + loss.detach()
            if world > 1:
                flat = torch.cat([p.grad.reshape(-1) for p in params[:5]])
                dist.all_reduce(flat)
            loss_host.copy_(total.reshape(1), non_blocking=True)                 # D2H of the step's loss
            torch.cuda.synchronize()
            return float(loss_host.item())

        def time_e2e(plain):
            for _ in range(2):
                e2e_step(plain)
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(n_e2e):
                e2e_step(plain)
            e1.record()
            barrier()
            t = torch.tensor([e0.elapsed_time(e1)], device=dev)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item()) / n_e2e

        n_e2e = max(1, args.steps)
        e_ms = time_e2e(False)
        p_ms = time_e2e(True)
        e2e = {"value": rays_per_step / (e_ms * 1e-3) / 1e6, "unit": "Mrays/s",
               "h2d_bytes_per_step": int(sum((b.row_end - b.row_begin) * args.width * 3 * 4 for b in my_blocks)),
               "d2h_bytes_per_step": 4, "ms_per_step": e_ms, "steps": n_e2e,
               "reference_call_only": {"value": rays_per_step / (p_ms * 1e-3) / 1e6, "ms_per_step": p_ms,
                                       "note": "the same loop with the reference's own arguments only: no next view "
                                               "announced, gradients returned to autograd (which adds them into .grad)"},
               "api": "RenderOptixFunction.apply + L1 loss + backward per view; the parameter tensors stay untouched "
                      "within the step, so the entry point builds its acceleration structure once per step by itself; "
                      "settings announce the next view (next_viewpoint_cam) and ask for in-place accumulation into "
                      ".grad (accumulate_leaf_grads); a view shared between ranks is rendered row range by row range"}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- roofline of the dominant kernel (the recording forward march), from live CUDA-event timings.
    # Bytes and operation counts are the compulsory ones: per Gaussian 300 B (forward) / 536 B (backward), per ray
    # 16 B / 28 B; per hit-list entry P, inside (sample, Gaussian) pair E_in and slab with hits S_h
    # F_fwd = 90 P + 12 E_in + 480 S_h, MUFU_fwd = E_in + 64 S_h, F_bwd = 290 P + 22 E_in + 640 S_h,
    # MUFU_bwd = 2 E_in + 96 S_h.  What the implementation moves on top (the recording) is traffic, not algorithm.
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    hbm_peak = float(peaks.get("hbm_gbs", 6650.0))
    peak_src = "measured" if "hbm_gbs" in peaks else "fallback"
    sm_max_mhz = float(peaks.get("sm_max_mhz", 1965.0))
    n_sm = torch.cuda.get_device_properties(dev).multi_processor_count
    bwd_ms = ktimes["backward_ms"] / max(1, ktimes["backward_launches"])
    fwd_ms = ktimes["forward_ms"] / max(1, ktimes["forward_launches"])
    blocks0 = all_blocks[0]
    rows_per_launch = sum(b.row_end - b.row_begin for b in blocks0) / max(1, len(blocks0))
    rays_per_launch = rows_per_launch * args.width
    # work counters of one view (outside the timed region)
    renderer.reset_counters()
    renderer.forward(*scene_dev_tensors, cams[0], march_of(cams[0], None, _lib.FLAG_COUNT_WORK))
    cn = renderer.read_counters()
    P, E, Sh = cn["hits"], cn["pairs_inside"], cn["slabs_hit"]
    frac_view = rays_per_launch / R
    alg_fwd = 300.0 * args.gaussians + 16.0 * rays_per_launch
    alg_bwd = 536.0 * args.gaussians + 28.0 * rays_per_launch
    # the forward's recording for the backward: per slab with hits a 528-byte head with the per-sample sums and
    # 4 bytes per hit; written once by the forward, read once by the backward
    tape_bytes = (528.0 * Sh + 4.0 * P) * frac_view
    # DRAM traffic of one forward launch = what it records + the Gaussian records and lists it streams once;
    # ratio taken from ncu captures of smaller cases on both sides of the L2 size (profiles/)
    traffic = TRAFFIC_PER_RECORDED_BYTE * tape_bytes
    f_fwd, mufu_fwd = (90.0 * P + 12.0 * E + 480.0 * Sh) * frac_view, (1.0 * E + 64.0 * Sh) * frac_view
    f_bwd, mufu_bwd = (290.0 * P + 22.0 * E + 640.0 * Sh) * frac_view, (2.0 * E + 96.0 * Sh) * frac_view
    fp32_peak = 2.0 * 128 * n_sm * sm_max_mhz * 1e6
    mufu_peak = 16.0 * n_sm * sm_max_mhz * 1e6
    # the same two ceilings measured on this device (register-chain kernels of the library, a few milliseconds)
    import ctypes as C
    fma_tf, ex2_g = C.c_float(), C.c_float()
    issue_src = "derived"
    if _lib.lib().rgx_measure_peaks(local, C.byref(fma_tf), C.byref(ex2_g)) == 0 and fma_tf.value > 0 and ex2_g.value > 0:
        fp32_peak, mufu_peak = fma_tf.value * 1e12, ex2_g.value * 1e9
        issue_src = "measured"
    achieved = alg_fwd / (fwd_ms * 1e-3) / 1e9
    # forward + backward of a launch's rays over everything the step spends on them (lists, colours, finalise included)
    view_ms = ms_per_step / max(1, len(blocks0))
    step_fp32 = (f_fwd + f_bwd) / (view_ms * 1e-3) / fp32_peak
    step_mufu = (mufu_fwd + mufu_bwd) / (view_ms * 1e-3) / mufu_peak
    roofline = {"kernel": "march_forward_lists_kernel<false,true,2> (forward march, recording for the backward, over lists that stop at a horizon)",
                "bound": "fp32-issue", "achieved": achieved, "peak": hbm_peak,
                "unit": "GB/s", "frac": achieved / hbm_peak, "peak_source": peak_src, "traffic": traffic,
                "traffic_note": "DRAM bytes of one launch: the recording (528 B per slab with hits + 4 B per hit) "
                                "times the ratio ncu measured on smaller cases; not part of the algorithmic bytes",
                "ms_per_launch": fwd_ms, "launches_timed": ktimes["forward_launches"],
                "algorithmic_bytes_per_launch": alg_fwd, "recorded_bytes_per_launch": tape_bytes,
                "fp32_frac": f_fwd / (fwd_ms * 1e-3) / fp32_peak, "mufu_frac": mufu_fwd / (fwd_ms * 1e-3) / mufu_peak,
                "achieved_step": max(step_fp32, step_mufu), "step_fp32_frac": step_fp32, "step_mufu_frac": step_mufu,
                "step_ms_per_launch_of_rays": view_ms,
                "backward": {"kernel": "march_backward_replay_kernel + march_backward_lists_kernel",
                             "ms_per_launch": bwd_ms, "launches_timed": ktimes["backward_launches"],
                             "algorithmic_bytes_per_launch": alg_bwd,
                             "achieved": alg_bwd / (bwd_ms * 1e-3) / 1e9,
                             "frac": alg_bwd / (bwd_ms * 1e-3) / 1e9 / hbm_peak,
                             "fp32_frac": f_bwd / (bwd_ms * 1e-3) / fp32_peak,
                             "mufu_frac": mufu_bwd / (bwd_ms * 1e-3) / mufu_peak},
                "fp32_peak_tflops": fp32_peak / 1e12, "ex2_peak_gops": mufu_peak / 1e9, "issue_peaks": issue_src,
                "note": "the march kernels are bound by instruction issue, not by HBM: frac is compulsory bytes over "
                        "time over the measured copy bandwidth, fp32_frac and mufu_frac are compulsory flops "
                        "(90 P + 12 E_in + 480 S_h) and ex2 (E_in + 64 S_h) per second over the fp32 FMA and ex2 rates "
                        "(measured by rgx_measure_peaks; derived 2*128*SMs*f and 16*SMs*f if that failed); "
                        "achieved_step = max(fp32, ex2) fraction of forward + backward over the whole per-view time; "
                        "the backward's time includes the next view's tile lists made beside it on a second stream",
                "counters_per_view": {k: cn[k] for k in ("rays", "slabs", "slabs_hit", "closest_queries", "hits",
                                                         "pairs_inside", "overflow_slabs", "prim_tests",
                                                         "ellipsoid_tests", "candidates")}}

    # ---- CPU baseline on a bounded sample (rank 0, N = 1 only): the reference's device code on the host cores,
    # and -- the same rays rendered by the CUDA path -- a parity check of every driver run at the full Gaussian count
    cpu_baseline = None
    if world == 1 and not args.no_cpu_baseline:
        try:
            from oracle import ref_shim
            if ref_shim.available():
                w, h = (20, 13) if args.cpu_sample == "auto" else tuple(int(x) for x in args.cpu_sample.split("x"))
                kept = {}
                cores = host_threads()
                cpu_scene = host_scene_cpu(scene)
                rays, times = cpu_reference_sample(cpu_scene, n_threads=cores, size=(w, h), keep=kept)
                cam_s = sample_camera(cpu_scene, (w, h))
                cam_s.to(dev)
                cs = ro.camera_struct(cam_s)
                got, _, _ = renderer.forward(*scene_dev_tensors, cs, march_of(cs, None, 0))
                diff = (got.cpu().numpy() - kept["rgb"]).__abs__().max(axis=1)
                diff.sort()
                cpu_baseline = {"value": rays / times[0] / 1e6, "unit": "Mrays/s", "cores": cores,
                                "kind": "reference",
                                "sample": f"{w}x{h} rays of view 0, forward+backward, all {args.gaussians} Gaussians "
                                          f"({times[0]:.1f} s)",
                                "parity": {"rays": int(rays), "max_abs_rgb_diff": float(diff[-1]),
                                           "p95_abs_rgb_diff": float(diff[int(0.95 * (len(diff) - 1))]),
                                           "note": "CUDA forward of the same rays against the reference's colours, "
                                                   "no ray left out (rays with a marginal discrete decision included)"}}
        except Exception as exc:  # the baseline is a report, never a reason to lose the bench line
            cpu_baseline = {"value": None, "unit": "Mrays/s", "cores": host_threads(), "kind": "reference",
                            "sample": f"failed: {exc}"}

    # ---- the two other full-size configurations, each with its own CUDA-event time (N = 1 only; after the headline)
    secondary = None
    if world == 1 and not args.no_secondary and args.gaussians == 3_000_000:
        del scene_dev_tensors, targets, grads
        torch.cuda.empty_cache()
        try:
            secondary = secondary_records(dev, hbm_peak)
        except Exception as exc:
            secondary = {"failed": str(exc)}

    out = {
        "metric": METRIC, "value": value, "unit": "Mrays/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "gaussians": args.gaussians, "image": f"{args.width}x{args.height}",
                   "views_per_step": args.views, "sh_degree": 3,
                   "sharding": f"rows/{world}" + (", cut by the per-view cost measured in the second warm-up step" if weigh_at >= 0 else ""),
                   "shell_scales": "the shell's drawn log-scale N(-1, 0.5) is the LONGEST axis, the two others "
                                   "shorter by log-uniform factors up to 10 (read as the shortest axis, every ray "
                                   "overflows the 512-hit cap in its first slab and parity is undefined)",
                   "l2": "inputs larger than L2 (Gaussian records 0.65 GB, gradient rows 0.8 GB, 3 GB recorded per view)"},
        "views_per_s": args.views / (ms_per_step * 1e-3),
        "clocks": clocks, "e2e": e2e, "gpu_launches": gpu_launches, "near_lists": near_lists,
        "roofline": roofline, "cpu_baseline": cpu_baseline, "secondary": secondary,
    }
    print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


def secondary_records(dev, hbm_peak):
    """Driver-run records of the two other full-size configurations.

    object-300k: 300,000 Gaussians, 800x800, static sampling, white background; forward + backward per view with the
    gradients of 20 views accumulated (one build per step), Mrays/s.
    stress-7M: 7,000,000 needle-like Gaussians, 1920x1080, transmittance threshold 1e-4, forward only into the 8-bit
    frame and depth buffers; frames/s, compulsory HBM bytes per second and the overflow count of one frame."""
    import torch
    from raygaussx_b200 import _lib, scenes as S
    from raygaussx_b200 import render_optix as ro
    from raygaussx_b200.dist import GradBuffer, accumulation_step
    out = {}
    # ---- object scene
    sc = S.object_scene(n_cameras=20)
    tens = [t.to(dev).contiguous() for t in sc.tensors()]
    for c in sc.cameras:
        c.to(dev)
    cams = [ro.camera_struct(c) for c in sc.cameras]
    R = cams[0].width * cams[0].height
    targets = [S.l1_target(R, seed=2000 + v).to(dev) for v in range(len(cams))]
    mp = sc.march
    r = ro.Renderer(dev)
    grads = GradBuffer(sc.n, tens[4].shape[2], dev)
    march_of = lambda cam, rows, flags: ro.Renderer._march(mp.dt_step, mp.dynamic_sampling, mp.max_prim_slice,
                                                           mp.white_background, mp.transmittance_eps, rows, cam.height, flags)
    for _ in range(3):
        accumulation_step(r, tens, cams, targets, march_of, grads)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n_steps = 3
    e0.record()
    for _ in range(n_steps):
        accumulation_step(r, tens, cams, targets, march_of, grads)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / n_steps
    r.reset_counters()
    r.forward(*tens, cams[0], march_of(cams[0], None, _lib.FLAG_COUNT_WORK))
    cn = r.read_counters()
    out["object-300k"] = {"metric": "fwd+bwd Mrays/s (300k Gaussians, 800x800, 20 views per step)",
                          "value": len(cams) * R / (ms * 1e-3) / 1e6, "unit": "Mrays/s", "ms_per_step": ms,
                          "steps": n_steps, "warmup": 3, "ms_per_view": ms / len(cams),
                          "counters_view0": {k: cn[k] for k in ("rays", "slabs", "slabs_hit", "hits", "pairs_inside",
                                                                "overflow_slabs")}}
    del r, tens, targets, grads
    torch.cuda.empty_cache()
    # ---- stress scene, forward only
    sc = S.stress_scene(n_cameras=12)
    tens = [t.to(dev).contiguous() for t in sc.tensors()]
    for c in sc.cameras:
        c.to(dev)
    cams = [ro.camera_struct(c) for c in sc.cameras]
    R = cams[0].width * cams[0].height
    mp = sc.march
    r = ro.Renderer(dev)
    r.build(*tens[:4])
    m_of = lambda cam, flags=0: ro.Renderer._march(mp.dt_step, mp.dynamic_sampling, mp.max_prim_slice, mp.white_background,
                                                   mp.transmittance_eps, None, cam.height, flags)
    for cam in cams[:3]:
        r.forward_frame(*tens, cam, m_of(cam))
    torch.cuda.synchronize()
    e0.record()
    for cam in cams[3:]:
        r.forward_frame(*tens, cam, m_of(cam))
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / len(cams[3:])
    r.reset_counters()
    r.forward(*tens, cams[3], m_of(cams[3], _lib.FLAG_COUNT_WORK))
    cn = r.read_counters()
    alg = 300.0 * sc.n + 16.0 * R
    out["stress-7M"] = {"metric": "forward frames/s (7M Gaussians, 1920x1080, T threshold 1e-4)",
                        "value": 1e3 / ms, "unit": "frames/s", "ms_per_frame": ms, "frames_timed": len(cams[3:]),
                        "warmup_frames": 3, "hbm_gbs": alg / (ms * 1e-3) / 1e9, "hbm_frac": alg / (ms * 1e-3) / 1e9 / hbm_peak,
                        "algorithmic_bytes_per_frame": alg, "overflow_slabs": cn["overflow_slabs"],
                        "workspace_gb": r.workspace_bytes() / 1e9,
                        "counters_frame3": {k: cn[k] for k in ("rays", "slabs", "slabs_hit", "hits", "pairs_inside",
                                                               "overflow_slabs")},
                        "note": "acceleration structure built once, as scripts/test.py does (one GAS per camera list); "
                                "every frame makes its own tile lists"}
    return out


def host_scene_cpu(scene):
    """A CPU copy of the scene for the host-side baseline."""
    import copy
    sc = copy.copy(scene)
    for k in ("positions", "scales", "quaternions", "densities", "color_features", "sph_gauss_features",
              "bandwidth_sharpness", "lobe_axis"):
        setattr(sc, k, getattr(scene, k).detach().cpu())
    sc.cameras = [c for c in scene.cameras]
    return sc


if __name__ == "__main__":
    main()
