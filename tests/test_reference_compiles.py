"""Drop-in check of the header surface: the reference's own, unmodified sources on the NeuS path compile (nvcc -c, sm_100a)
with this repository's include/ standing in for its un-vendored tiny-cuda-nn fork.  The reference is read where it lies
(a checkout next to this repository, or NEUS2_REFERENCE); nothing is copied.  Skipped where no checkout is present."""
import concurrent.futures
import os
import subprocess
import sys
import tempfile

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from neus2_b200 import build as B  # noqa: E402

# the training step, the trainer / optimizer / factory call sites, mesh extraction, the dataset loader, device helpers
SOURCES = ["src/testbed_nerf.cu", "src/testbed.cu", "src/marching_cubes.cu", "src/nerf_loader.cu", "src/common_device.cu",
           "src/camera_path.cu", "src/triangle_bvh.cu", "src/main.cu"]
# every member of the class template, instantiated explicitly
NERF_NETWORK_TU = """#include <neural-graphics-primitives/nerf_network.h>
using namespace tcnn;
template class ngp::NerfNetwork<__half>;
"""


def compile_one(src, flags, out_dir):
    obj = os.path.join(out_dir, os.path.basename(src) + ".o")
    cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "--extended-lambda", "--expt-relaxed-constexpr",
           "-O0", "-w", '-DNGP_VERSION="1.0dev"', "-DTCNN_MIN_GPU_ARCH=100"] + flags + ["-c", src, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    return src, r.returncode, (r.stdout + r.stderr)[-4000:]


def test_unmodified_reference_sources_compile_against_the_headers():
    ref = B.reference_root()
    flags = B.header_include_flags(with_reference=True)
    if ref is None or flags is None:
        pytest.skip("no reference checkout (or no nlohmann/json.hpp) on this machine")
    with tempfile.TemporaryDirectory() as tmp:
        tu = os.path.join(tmp, "nerf_network_tu.cu")
        with open(tu, "w") as f:
            f.write(NERF_NETWORK_TU)
        srcs = [tu] + [os.path.join(ref, s) for s in SOURCES]
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
            results = list(pool.map(lambda s: compile_one(s, flags, tmp), srcs))
    failed = [(s, log) for s, rc, log in results if rc != 0]
    assert not failed, "\n".join("%s:\n%s" % f for f in failed)
