"""Regenerates ``knn.npz``: outputs of the REFERENCE's own nearest-neighbour extension (submodules/simple-knn,
SimpleKNN::knn, compiled from where it lies into oracle/_ref/libref_knn.so by oracle/Makefile) on the seeded
clouds of tests/knn_clouds.py.  Device code: run it where a GPU is, e.g.

    python tests/golden/make_knn_golden.py <output.npz>      (default: tests/golden/knn.npz)

Stores per cloud the fp32 result array and a checksum of the generated points.
"""
import ctypes
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from tests.knn_clouds import CLOUDS, cloud  # noqa: E402


def main(out_path):
    lib = ctypes.CDLL(os.path.join(ROOT, "oracle", "_ref", "libref_knn.so"))
    lib.ref_knn_mean_dist2.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
    out = {}
    for name, (n, seed, kind) in CLOUDS.items():
        pts = cloud(n, seed, kind)
        dev = pts.cuda().contiguous()
        res = torch.zeros(n, device="cuda", dtype=torch.float32)      # spatial.cu fills with zeros first
        torch.cuda.synchronize()
        rc = lib.ref_knn_mean_dist2(n, dev.data_ptr(), res.data_ptr())
        assert rc == 0, rc
        out[name] = res.cpu().numpy()
        out[name + "_sum"] = np.float64(pts.double().sum().item())
        print(name, n, out[name][:3])
    np.savez_compressed(out_path, **out)


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "tests", "golden", "knn.npz"))
