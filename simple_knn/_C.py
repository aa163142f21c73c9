"""``distCUDA2`` of the reference's simple-knn extension (submodules/simple-knn/ext.cpp, simple_knn.cu), on
``rgx_knn_mean_dist2``: mean squared distance from every point to its three nearest other points."""
import ctypes as C

import torch

from raygaussx_b200 import _lib


def distCUDA2(points: torch.Tensor) -> torch.Tensor:
    if not points.is_cuda:
        raise RuntimeError("distCUDA2 needs a CUDA tensor: there is no CPU path")
    pts = points.detach().to(torch.float32).contiguous()
    if pts.dim() != 2 or pts.shape[1] != 3:
        raise ValueError("points must be [N, 3]")
    out = torch.empty(pts.shape[0], device=pts.device, dtype=torch.float32)
    with torch.cuda.device(pts.device):
        stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        rc = _lib.lib().rgx_knn_mean_dist2(pts.device.index or 0, C.c_void_p(pts.data_ptr()), pts.shape[0],
                                           C.c_void_p(out.data_ptr()), stream)
    if rc != 0:
        raise _lib.RgxError(rc, "rgx_knn_mean_dist2 failed")
    return out
