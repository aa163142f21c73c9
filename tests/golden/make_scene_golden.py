"""Regenerates ``scene_<scene>_<view>.npz``: golden vectors on the content of the large configurations.

    make -C oracle && python tests/golden/make_scene_golden.py [scene[:view] ...]

For every view of tests/scene_views.py (a few hundred rays against all 300 k / 3 M / 7 M Gaussians) it stores

* ``oracle_*``  the float64 oracle's colours, alpha, depth, per-ray predicate margin, per-ray overflow flag
                and work counters;
* ``ref_rgb``   the colours of the reference's own device code (fp32, compiled for the CPU; its
                transmittance threshold is the constant 1e-3 of cuda_train/forward/gaussians_aabb.h:4, so for
                the 7 M scene, whose configuration asks for 1e-4, ``oracle1e3_*`` holds the oracle at 1e-3 too);
* ``dl``        the loss gradient dL/dC both backward passes were given (mean L1 against the seeded target);
* ``og_idx_<t>``, ``og_val_<t>``, ``og_max_<t>``  the float64 oracle's gradient of tensor ``t`` at the 256
                largest and 768 randomly drawn non-zero entries (flat indices), and its largest magnitude --
                the full tensors are 59 floats per Gaussian and are not stored;
* ``rg_val_<t>`` the reference's fp32 gradient at the same entries;
* ``input_sum`` a checksum of the generated scene.

Takes from half a minute (300 k Gaussians) to tens of minutes (7 M needles, the whole field of view) per view on
8 cores: the oracle first culls the Gaussians no ray of a chunk can pierce, then works densely on what is left.
"""
from __future__ import annotations

import os
import sys
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import oracle, ref_shim  # noqa: E402
from raygaussx_b200 import scenes  # noqa: E402
from tests.scene_views import GRAD_NAMES, SCENES, input_checksum, view_camera  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
CHUNK = 16


def pick_entries(g, seed):
    flat = g.reshape(-1)
    nz = flat.nonzero(as_tuple=True)[0]
    top = flat.abs().topk(min(256, flat.numel())).indices
    gen = torch.Generator().manual_seed(seed)
    rnd = nz[torch.randperm(nz.numel(), generator=gen)[:768]]
    return torch.unique(torch.cat([top, rnd]))


def generate(scene_name, only_view=None):
    make, views = SCENES[scene_name]
    sc = make()
    csum = input_checksum(sc)
    for vname, cam_index, kind, geom in views:
        if only_view and vname != only_view:
            continue
        t0 = time.time()
        cam = view_camera(sc, kind, cam_index, geom)
        out = {"input_sum": np.float64(csum)}
        col, _, ctx = ref_shim.render_forward(*sc.tensors(), cam, sc.march)
        fwd, _ = oracle.render_forward(*sc.tensors(), cam, sc.march, chunk=CHUNK)
        rays = col.shape[0]
        tgt = scenes.l1_target(rays).double()
        dl = torch.sign(fwd.rgb - tgt) / (3 * rays)
        out.update(ref_rgb=col, dl=dl.numpy(), oracle_rgb=fwd.rgb.numpy(), oracle_alpha=fwd.alpha.numpy(),
                   oracle_depth=fwd.depth.numpy(), oracle_margin=fwd.margin.numpy(),
                   oracle_overflow=fwd.overflow.numpy(),
                   oracle_counters=np.array([fwd.counters[k] for k in ("S", "S_h", "Q_c", "P", "E_in", "OVF")], dtype=np.int64))
        mp = sc.march
        if abs(mp.transmittance_eps - 1e-3) > 1e-12:      # the reference's constant: a second oracle run at 1e-3
            import copy
            mp3 = copy.copy(mp)
            mp3.transmittance_eps = 1e-3
            f3, _ = oracle.render_forward(*sc.tensors(), cam, mp3, chunk=CHUNK)
            out.update(oracle1e3_rgb=f3.rgb.numpy(), oracle1e3_margin=f3.margin.numpy(),
                       oracle1e3_overflow=f3.overflow.numpy())
            dl = torch.sign(f3.rgb - tgt) / (3 * rays)     # the backward is compared at the reference's threshold
            out["dl"] = dl.numpy()
            mp = mp3
        rg = ref_shim.render_backward(ctx, dl.float().numpy())
        og = oracle.render_backward(*sc.tensors(), cam, mp, dl, chunk=CHUNK)
        for k, nm in enumerate(GRAD_NAMES):
            g = og[nm]
            idx = pick_entries(g, seed=17 + k)
            out["og_idx_" + nm] = idx.numpy()
            out["og_val_" + nm] = g.reshape(-1)[idx].numpy()
            out["og_max_" + nm] = np.float64(g.abs().max().item())
            out["rg_val_" + nm] = np.asarray(rg[k]).reshape(-1)[idx.numpy()]
        np.savez_compressed(os.path.join(HERE, f"scene_{scene_name}_{vname}.npz"), **out)
        err = np.abs(out["oracle_rgb"] - col).max(axis=1)
        steady = out["oracle_margin"] > 3e-5
        print(f"{scene_name}:{vname}: {rays} rays, {time.time() - t0:.0f} s, counters {fwd.counters}, "
              f"ref-vs-oracle colour diff {err.max():.2e}, steady share {steady.mean():.2f}, "
              f"overflow rays {int(out['oracle_overflow'].sum())}", flush=True)


if __name__ == "__main__":
    if not ref_shim.available():
        sys.exit("oracle/_ref is not built: run `make -C oracle` where the reference checkout is available")
    for arg in (sys.argv[1:] or SCENES):
        name, _, view = arg.partition(":")
        generate(name, view or None)
