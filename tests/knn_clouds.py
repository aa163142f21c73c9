"""Seeded point clouds on which the nearest-neighbour replacement is pinned to the reference's simple-knn
(shared by tests/golden/make_knn_golden.py, which runs the reference's extension on a GPU, and by the tests)."""
import torch


def cloud(n, seed, kind):
    g = torch.Generator().manual_seed(seed)
    if kind == "uniform":
        return torch.rand(n, 3, generator=g) * 4 - 2
    if kind == "clustered":
        c = torch.randn(8, 3, generator=g) * 3
        return c[torch.randint(0, 8, (n,), generator=g)] + 0.02 * torch.randn(n, 3, generator=g)
    if kind == "plane":                       # degenerate extent along one axis
        p = torch.rand(n, 3, generator=g)
        p[:, 2] = 0.25
        return p
    if kind == "duplicates":                  # a pair and a triple of coincident points: distance zero counts
        p = torch.rand(n, 3, generator=g) * 4 - 2
        p[100] = p[7]
        p[300] = p[200]
        p[301] = p[200]
        return p
    raise ValueError(kind)


# name -> (n, seed, kind).  Fewer than four points: the missing neighbours stay at FLT_MAX in the reference's
# fp32 sum (simple_knn.cu: boxMeanDist), which overflows to +inf when two or more are missing.
CLOUDS = {
    "one": (1, 11, "uniform"), "two": (2, 12, "uniform"), "three": (3, 13, "uniform"), "four": (4, 14, "uniform"),
    "u33": (33, 43, "uniform"), "u1000": (1000, 1010, "uniform"), "c1025": (1025, 1035, "clustered"),
    "p3000": (3000, 3010, "plane"), "c5000": (5000, 5010, "clustered"), "d2000": (2000, 3, "duplicates"),
    "u20000": (20000, 5, "uniform"),
}
