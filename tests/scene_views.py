"""The views on which the CUDA path is compared with the reference on the content of the three large
configurations (300 k, 3 M and 7 M Gaussians).  Shared by the generator of the golden vectors
(tests/golden/make_scene_golden.py) and by the GPU test (tests/test_gpu_parity_scenes.py).

A full-size image cannot go through the float64 oracle or the CPU build of the reference, so every view is a
few hundred rays against ALL Gaussians of the scene: either the whole field of view at a coarse resolution
(``whole``: wide tiles, rays far apart) or a window of the full-resolution image (``crop``: the tile geometry
and ray spacing of the real workload; expressed through the reference's own camera model by narrowing the
field of view and moving the principal point).
"""
from raygaussx_b200 import scenes

SCENES = {
    # name: (generator, [(view name, camera index, kind, geometry)])
    "object": (lambda: scenes.object_scene(n_cameras=8),
               [("whole", 0, "whole", (16, 16)),                      # the blob from outside, white background
                ("crop_centre", 3, "crop", (392, 392, 16, 16)),       # through the dense middle
                ("crop_rim", 5, "crop", (250, 420, 16, 16))]),        # grazing the blob's edge: rays that miss, rays that skip
    "unbounded": (lambda: scenes.unbounded_scene(n_cameras=200),
                  [("whole", 0, "whole", (20, 13)),                   # camera inside the cloud, the whole 60 degree view
                   ("crop_centre", 50, "crop", (620, 406, 16, 16)),   # towards the core: hundreds of hits per ray
                   ("crop_sky", 100, "crop", (620, 60, 16, 16))]),    # above the core: long rays, shell Gaussians, step cap
    "stress": (lambda: scenes.stress_scene(n_cameras=8),
               [("whole", 0, "whole", (20, 12)),
                ("crop_centre", 5, "crop", (952, 532, 16, 16))]),     # 100:1 needles, heavy overlap
}


def view_camera(sc, kind, cam_index, geom):
    cam = sc.cameras[cam_index]
    if kind == "whole":
        return scenes.lowres_camera(cam, *geom)
    return scenes.crop_camera(cam, *geom)


def input_checksum(sc):
    return float(sum(t.double().sum().item() for t in sc.tensors()))


GRAD_NAMES = ("positions", "scales", "quaternions", "densities", "color_features")
