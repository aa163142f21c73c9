"""Regenerates the golden vectors of this directory.

    make -C oracle && python tests/golden/make_golden.py

Needs the reference checkout (oracle/Makefile compiles its device sources for the
CPU into oracle/_ref).  For every case below it stores, in ``<case>.npz``:

* ``ref_*``     outputs of the reference's own device code (fp32, OptiX traversal
                replaced by an exhaustive loop): ray colours, per-Gaussian colours
                and the eight gradients for an L1 loss against a seeded target;
* ``oracle_*``  the float64 oracle's outputs for the same inputs (stored as
                float64): colours, alpha, depth, per-ray predicate margin,
                gradients, work counters;
* ``input_sum`` a checksum of the generated inputs, so that a drift of the seeded
                scene generator is detected instead of silently comparing
                different scenes.

Inputs are not stored: ``raygaussx_b200.scenes`` regenerates them from the seed.
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import oracle, ref_shim  # noqa: E402
from raygaussx_b200 import scenes  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))

CASES = {
    # the 4,096-Gaussian 64x64 configuration, exactly as benchmarked
    "config1": dict(),
    # small cases covering the switches of the march and of the colour model
    "small_static": dict(n=512, width=16, height=16, log_scale_mean=-2.5),
    "small_dynamic_white": dict(n=512, width=16, height=16, log_scale_mean=-2.5, dynamic_sampling=True,
                                white_background=True, dt_step=0.005),
    "small_lobes_deg2": dict(n=300, width=12, height=12, log_scale_mean=-2.3, sh_degree=2, lobes=3, seed=7),
    "small_deg0": dict(n=300, width=12, height=12, log_scale_mean=-2.3, sh_degree=0, seed=8),
    "small_deg1_cap": dict(n=400, width=12, height=12, log_scale_mean=-2.0, sh_degree=1, seed=9, max_prim_slice=4096),
}

GRAD_NAMES = ("positions", "scales", "quaternions", "densities", "color_features", "sph_gauss_features",
              "bandwidth_sharpness", "lobe_axis")


def make_scene(name):
    return scenes.tiny_scene(**CASES[name])


def input_checksum(sc):
    return float(sum(t.double().sum().item() for t in sc.tensors()))


def loss_gradient(rgb, n_rays):
    """dL/dC of the mean L1 loss against the seeded uniform target."""
    tgt = scenes.l1_target(n_rays).to(rgb.dtype)
    return torch.sign(rgb - tgt) / (3 * n_rays)


def generate(name):
    sc = make_scene(name)
    cam = sc.cameras[0]
    out = {"input_sum": np.float64(input_checksum(sc))}
    col, rgb_g, ctx = ref_shim.render_forward(*sc.tensors(), cam, sc.march)
    o_fwd, o_rgb_g = oracle.render_forward(*sc.tensors(), cam, sc.march)
    dl = loss_gradient(o_fwd.rgb, col.shape[0])          # the same dL/dC for both implementations
    rg = ref_shim.render_backward(ctx, dl.float().numpy())
    og = oracle.render_backward(*sc.tensors(), cam, sc.march, dl)
    out["dl"] = dl.numpy()
    out["ref_rgb"], out["ref_gaussian_rgb"] = col, rgb_g
    for nm, g in zip(GRAD_NAMES, rg[:8]):
        if g is not None:
            out["ref_grad_" + nm] = g
    out["oracle_rgb"] = o_fwd.rgb.numpy()
    out["oracle_alpha"] = o_fwd.alpha.numpy()
    out["oracle_depth"] = o_fwd.depth.numpy()
    out["oracle_margin"] = o_fwd.margin.numpy()
    out["oracle_gaussian_rgb"] = o_rgb_g.numpy()
    out["oracle_counters"] = np.array([o_fwd.counters[k] for k in ("S", "S_h", "Q_c", "P", "E_in", "OVF")], dtype=np.int64)
    for nm in GRAD_NAMES:
        g = og[nm]
        if g is not None and g.numel():
            out["oracle_grad_" + nm] = g.numpy()
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
    err = np.abs(out["oracle_rgb"] - col).max()
    print(f"{name}: rays {col.shape[0]} ref-vs-oracle max colour diff {err:.2e} counters {o_fwd.counters}")


if __name__ == "__main__":
    if not ref_shim.available():
        sys.exit("oracle/_ref is not built: run `make -C oracle` where the reference checkout is available")
    for case in (sys.argv[1:] or CASES):
        generate(case)
