"""Data parallelism over rays for a gradient-accumulation step.

The reference is single-process; its training loop accumulates gradients over 20
views before an optimizer step (scripts/train.py:84-165).  Rays are independent
given the Gaussian set and gradients are sums over rays, so that step shards
cleanly: every rank holds all Gaussians, builds the same acceleration structure,
renders and back-propagates an equal share of the step's image rows (a view that
straddles two ranks is split by rows), and one all-reduce of the flat gradient
buffer joins the ranks.  Valid for per-pixel losses such as L1; a full-image loss
(SSIM) would need the image gathered first.

Nothing here launches a kernel of its own: device work goes through
:class:`raygaussx_b200.render_optix.Renderer`, the collective through
``torch.distributed`` (NCCL on GPUs, gloo in CPU tests of the host logic).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence, Tuple

import torch

GRAD_FIELDS = ("positions", "scales", "quaternions", "densities", "color_features")


@dataclass(frozen=True)
class RowBlock:
    view: int        # index into the step's list of views
    row_begin: int
    row_end: int


def shard_rows(n_views: int, height: int, rank: int, world: int) -> List[RowBlock]:
    """Rows of ``n_views`` images of ``height`` rows laid end to end and cut into
    ``world`` equal contiguous pieces (sizes differ by at most one row); returns
    the blocks of piece ``rank``."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError("rank must be in [0, world)")
    total = n_views * height
    lo = (total * rank) // world
    hi = (total * (rank + 1)) // world
    blocks = []
    v = lo // height if height else 0
    while lo < hi:
        end = min(hi, (v + 1) * height)
        blocks.append(RowBlock(v, lo - v * height, end - v * height))
        lo = end
        v += 1
    return blocks


def shard_rows_weighted(view_costs: Sequence[float], height: int, rank: int, world: int) -> List[RowBlock]:
    """Like :func:`shard_rows`, with the cuts placed by cost instead of by count: ``view_costs[v]`` is what view
    ``v`` costs as a whole (any unit -- the milliseconds the previous step spent on it, say), spread evenly over
    its rows, and every rank gets an equal share of the total.  Views differ by a few per cent in cost, and a
    step waits for its slowest rank.  Every rank must pass the same costs (all-gather them first)."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError("rank must be in [0, world)")
    n_views = len(view_costs)
    costs = [max(float(c), 0.0) for c in view_costs]
    total = sum(costs)
    if n_views == 0 or height <= 0 or not total > 0.0:
        return shard_rows(n_views, height, rank, world)
    # cumulative cost at every view boundary; cut k lies where the running cost reaches k / world of the total
    def cut(k):
        if k <= 0:
            return 0
        if k >= world:
            return n_views * height
        want, run = total * k / world, 0.0
        for v, c in enumerate(costs):
            if run + c >= want and c > 0.0:
                return v * height + min(height, max(0, int(round((want - run) / c * height))))
            run += c
        return n_views * height
    lo, hi = cut(rank), cut(rank + 1)
    blocks = []
    v = lo // height
    while lo < hi:
        end = min(hi, (v + 1) * height)
        blocks.append(RowBlock(v, lo - v * height, end - v * height))
        lo = end
        v += 1
    return blocks


def view_costs_from_blocks(n_views: int, height: int, timed_blocks) -> List[float]:
    """Per-view cost from ``(RowBlock, milliseconds)`` pairs of all ranks (a block's time is spread over its rows and
    scaled to the whole view; several blocks of a view add up)."""
    ms = [0.0] * n_views
    rows = [0] * n_views
    for blk, t in timed_blocks:
        ms[blk.view] += float(t)
        rows[blk.view] += blk.row_end - blk.row_begin
    known = [m / r * height for m, r in zip(ms, rows) if r > 0]
    mean = sum(known) / len(known) if known else 1.0
    return [m / r * height if r > 0 else mean for m, r in zip(ms, rows)]


def gradient_layout(n: int, sh_coeffs: int) -> List[Tuple[str, int, Tuple[int, ...]]]:
    """(name, offset, shape) of each gradient tensor inside the flat buffer:
    3 + 3 + 4 + 1 + 3*sh_coeffs floats per Gaussian, stored tensor after tensor."""
    shapes = {"positions": (n, 3), "scales": (n, 3), "quaternions": (n, 4), "densities": (n,),
              "color_features": (n, 3, sh_coeffs)}
    out, off = [], 0
    for name in GRAD_FIELDS:
        size = 1
        for d in shapes[name]:
            size *= d
        out.append((name, off, shapes[name]))
        off += size
    return out


class GradBuffer:
    """One contiguous fp32 buffer holding every per-Gaussian gradient, so that the
    step needs a single collective."""

    def __init__(self, n: int, sh_coeffs: int, device):
        self.layout = gradient_layout(n, sh_coeffs)
        name, off, shape = self.layout[-1]
        total = off + (shape[0] * shape[1] * shape[2])
        self.flat = torch.zeros(total, dtype=torch.float32, device=device)
        self.views = {}
        for name, off, shape in self.layout:
            size = 1
            for d in shape:
                size *= d
            self.views[name] = self.flat[off:off + size].view(*shape)

    def tensors(self):
        return tuple(self.views[k] for k in GRAD_FIELDS)

    def zero_(self):
        self.flat.zero_()

    def all_reduce(self, group=None):
        if torch.distributed.is_available() and torch.distributed.is_initialized() \
                and torch.distributed.get_world_size(group) > 1:
            torch.distributed.all_reduce(self.flat, op=torch.distributed.ReduceOp.SUM, group=group)


def l1_loss_gradient(rgb: torch.Tensor, target: torch.Tensor, n_rays_total: int, n_views: int) -> torch.Tensor:
    """dL/dC of ``mean(|C - target|)`` over an image of ``n_rays_total`` rays,
    divided by the number of accumulated views (scripts/train.py:145-146)."""
    return torch.sign(rgb - target) / float(3 * n_rays_total * n_views)


def accumulation_step(renderer, tensors: Sequence[torch.Tensor], cameras, targets, march_of, grads: GradBuffer,
                      rank: int = 0, world: int = 1, rebuild: bool = True, group=None, loss_out=None,
                      lists_ahead: bool = True, blocks=None, block_events=None):
    """One gradient-accumulation step over ``cameras`` (rgx camera structs) with
    per-view device targets ``targets[v]`` of shape ``[R, 3]``.

    ``march_of(cam, rows, flags)`` returns the march struct for a camera and row
    range.  On return ``grads`` holds the gradient of ``mean_v L1_v`` summed over
    all ranks.  Kernels launched: the acceleration-structure build (once), then per
    row block a forward, an elementwise loss gradient, and an accumulating backward
    (which, with ``lists_ahead``, also makes the next block's tile lists on a second stream).
    ``blocks``: this rank's row blocks (default: an equal share of the rows, :func:`shard_rows`).
    ``block_events``: a list that receives ``(block, start event, end event)`` per block, for cost-weighted cuts.
    """
    from . import _lib
    if rebuild:
        renderer.build(*tensors[:4])
    grads.zero_()
    n_views = len(cameras)
    blocks = list(shard_rows(n_views, cameras[0].height, rank, world)) if blocks is None else list(blocks)
    for i, blk in enumerate(blocks):
        cam = cameras[blk.view]
        if block_events is not None:
            ev0 = torch.cuda.Event(enable_timing=True)
            ev0.record()
        rows = (blk.row_begin, blk.row_end)
        r_total = cam.width * cam.height
        lo, hi = blk.row_begin * cam.width, blk.row_end * cam.width
        rgb, _, _ = renderer.forward(*tensors, cam, march_of(cam, rows, _lib.FLAG_SAVE_HITS))
        seg = rgb[lo:hi]
        dl = torch.empty_like(rgb)      # only rows [row_begin, row_end) are read by the backward
        dl[lo:hi] = l1_loss_gradient(seg, targets[blk.view][lo:hi], r_total, n_views)
        if loss_out is not None:
            loss_out += (seg - targets[blk.view][lo:hi]).abs().sum() / float(3 * r_total * n_views)
        if lists_ahead and i + 1 < len(blocks):
            nxt = blocks[i + 1]          # its tile lists are made beside this block's backward
            ncam = cameras[nxt.view]
            renderer.hint_next_view(ncam, march_of(ncam, (nxt.row_begin, nxt.row_end), _lib.FLAG_SAVE_HITS))
        renderer.backward(*tensors, cam, march_of(cam, rows, _lib.FLAG_ACCUMULATE), rgb, dl, grads.tensors())
        if block_events is not None:
            ev1 = torch.cuda.Event(enable_timing=True)
            ev1.record()
            block_events.append((blk, ev0, ev1))
    grads.all_reduce(group)
    return grads
