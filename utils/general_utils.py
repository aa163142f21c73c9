"""Stand-in for the reference's ``utils/general_utils.py`` on machines without cupy.

The reference's module imports cupy, imageio, matplotlib, scikit-image and ``turtle`` at module scope
(utils/general_utils.py:2-21), so nothing that imports it -- ``classes/point_cloud.py:12`` among them -- loads
without those packages, although the point cloud only wants two small torch functions from it.  This file
supplies what the hot path's callers use, with the reference's names and behaviour:

* ``inverse_sigmoid``, ``build_rotation``    (utils/general_utils.py:462-487; classes/point_cloud.py:12)
* ``reduce_supersampling``                   (utils/general_utils.py:489-502; scripts/train.py:129, scripts/test.py:129)
* ``torch2cupy`` / ``cupy2torch``            (utils/general_utils.py:453-460) raise: there is no cupy on this path

This directory deliberately has no ``__init__.py``: ``utils`` is a namespace package in the reference too, so
with this repository BEFORE the reference checkout on ``sys.path``, ``utils.general_utils`` resolves here and
every other ``utils.*`` module (``sh_utils``, ``optim_utils``, ``reordering_utils``, ...) to the reference's file.
"""
import torch

from raygaussx_b200.inference import reduce_supersampling  # noqa: F401  (same signature and result)


def inverse_sigmoid(x):
    """logit(x)."""
    return torch.log(x / (1 - x))


def build_rotation(r):
    """Rotation matrices ``[N, 3, 3]`` of the quaternions ``r [N, 4]`` (w, x, y, z), normalised first."""
    q = r / r.norm(dim=1, keepdim=True)
    w, x, y, z = q.unbind(dim=1)
    rows = (torch.stack([1 - 2 * (y * y + z * z), 2 * (x * y - w * z), 2 * (x * z + w * y)], dim=1),
            torch.stack([2 * (x * y + w * z), 1 - 2 * (x * x + z * z), 2 * (y * z - w * x)], dim=1),
            torch.stack([2 * (x * z - w * y), 2 * (y * z + w * x), 1 - 2 * (x * x + y * y)], dim=1))
    return torch.stack(rows, dim=1)


def torch2cupy(*args):
    raise RuntimeError("torch2cupy: this build has no cupy path; the renderer takes torch tensors directly "
                       "(optix_raycasting.render_optix.RenderOptixFunction)")


def cupy2torch(*args):
    raise RuntimeError("cupy2torch: this build has no cupy path")
