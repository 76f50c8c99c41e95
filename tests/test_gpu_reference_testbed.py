"""The reference's own headless training loop -- Testbed(Nerf), load_training_data, the network from a json document, frame() per
step: its unmodified sources compiled over include/tiny-cuda-nn (oracle/_ref/libref_testbed.so, built where a reference checkout is
present) -- trains a synthetic scene on the GPU.  This is the drop-in claim end to end: the reference's host code, its ray marching,
loss and occupancy kernels, its NerfNetwork, Trainer and optimizer objects run unchanged; underneath them run this repository's
layered kernels.  Runs in a child process."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_training_loop_runs_over_the_headers():
    if not os.path.exists(os.path.join(ROOT, "oracle", "_ref", "libref_testbed.so")):
        pytest.skip("oracle/_ref/libref_testbed.so was not built: no reference checkout at build time")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "oracle", "run_ref_testbed.py"), "--views", "12", "--res", "128", "--batch", "16384",
                        "--warmup", "100", "--steps", "100"], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    line = [l for l in r.stdout.splitlines() if l.startswith("{")][-1]
    out = json.loads(line)
    assert out["rc"] == 0 and out["training_step"] == 200
    # the loss (an average of the last steps' Huber losses) falls by an order of magnitude within 200 steps on this scene
    assert out["loss_last"] < 0.2 * out["loss_first"] and out["loss_last"] < 1e-3
    assert out["measured_batch_size"] > 0 and out["rays_per_batch"] > 0
