"""Writes tests/golden/loader_case: a tiny dataset in the reference's file format (two 16x12 RGBA images, a transforms.json that
uses file-level fields of view, scale, per-axis offset, an up vector, white_transparent and per-frame principal points) and,
where oracle/_ref/libref_testbed.so is present (built from a reference checkout, needs a GPU: the reference's loader keeps
its images in device memory), expected.npz: what ngp::load_nerf (src/nerf_loader.cu:197) returns for it -- cameras,
intrinsics, dataset scale / offset / up and every pixel byte.  tests/test_loader.py compares neus2_b200.loader with that file.

    python tests/golden/make_loader_golden.py            # dataset files (deterministic) and, if possible, expected.npz
"""
import json
import os
import subprocess
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
CASE = os.path.join(HERE, "loader_case")


def write_dataset():
    from PIL import Image
    rng = np.random.default_rng(20)
    os.makedirs(os.path.join(CASE, "images"), exist_ok=True)
    frames = []
    for i in range(2):
        img = rng.integers(0, 256, (12, 16, 4), dtype=np.uint8)
        img[0, 0] = (255, 255, 255, 255)
        img[0, 1] = (0, 0, 0, 0)        # transparent: white_transparent turns it white
        img[1, :4, 3] = 0
        Image.fromarray(img, "RGBA").save(os.path.join(CASE, "images", "%02d.png" % i))
        m = np.eye(4)
        m[:3, :3] = np.linalg.qr(rng.normal(size=(3, 3)))[0]
        m[:3, 3] = rng.normal(size=3)
        frames.append({"file_path": "images/%02d.png" % i, "transform_matrix": np.round(m, 6).tolist(), "w": 16, "h": 12,
                       "cx": 8.0 + 1.25 * i, "cy": 6.0 - 0.5 * i})
    js = {"camera_angle_x": 0.61, "camera_angle_y": 0.47, "scale": 0.41, "offset": [0.45, 0.5, 0.58], "up": [0.1, 0.2, 0.97], "aabb_scale": 1,
          "white_transparent": True, "frames": frames}
    with open(os.path.join(CASE, "transforms.json"), "w") as f:
        json.dump(js, f, indent=1)


def write_expected():
    lib = os.path.join(ROOT, "oracle", "_ref", "libref_testbed.so")
    if not os.path.exists(lib):
        print("oracle/_ref/libref_testbed.so is missing: expected.npz not written")
        return 1
    r = subprocess.run([sys.executable, os.path.join(ROOT, "oracle", "run_ref_testbed.py"), "--data", CASE, "--load-only", os.path.join(CASE, "expected.npz")])
    return r.returncode


if __name__ == "__main__":
    write_dataset()
    sys.exit(write_expected())
