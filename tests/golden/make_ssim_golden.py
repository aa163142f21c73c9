"""Golden values for raygaussx_b200.training.ssim and isotropy_loss.

Run where the reference checkout is present:

    python tests/golden/make_ssim_golden.py /path/to/reference

Imports the reference's own ``utils/loss_utils.py`` (plain torch) and stores seeded inputs' results in
``tests/golden/ssim.npz``; the inputs are regenerated from the seeds by the test.
"""
import importlib.util
import os
import sys

import numpy as np
import torch


def images(seed, h, w):
    g = torch.Generator().manual_seed(seed)
    a = torch.rand(3, h, w, generator=g)
    b = (a + 0.1 * torch.randn(3, h, w, generator=g)).clamp(0, 1)
    return a, b


CASES = [(0, 16, 16), (1, 37, 23), (2, 64, 48), (3, 9, 30)]


def main(ref):
    spec = importlib.util.spec_from_file_location("ref_loss_utils", os.path.join(ref, "utils", "loss_utils.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    out = {}
    for seed, h, w in CASES:
        a, b = images(seed, h, w)
        out[f"ssim_{seed}"] = float(mod.ssim(a, b))
        out[f"ssim_batched_{seed}"] = float(mod.ssim(a.unsqueeze(0), b.unsqueeze(0)))
        out[f"l1_{seed}"] = float(mod.l1_loss(a, b))
    np.savez(os.path.join(os.path.dirname(os.path.abspath(__file__)), "ssim.npz"), **out)
    print(out)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_ssim_golden.py <path to the reference checkout>")
    main(sys.argv[1])
