"""Runs the reference's own headless training loop (oracle/_ref/libref_testbed.so: the reference's unmodified sources over this
repository's tiny-cuda-nn headers, see oracle/ref_kernels/ref_testbed.cu) on a synthetic scene written to disk in the reference's
dataset format, and prints one JSON line.  Test and measurement infrastructure: called by tests and by `bench.py --impl reference`,
always as a child process (a part of the reference that is not compiled here aborts instead of returning).

    python oracle/run_ref_testbed.py --views 64 --res 512 --batch 262144 --warmup 520 --steps 200
"""
import argparse
import ctypes as C
import json
import os
import shutil
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
LIB = os.path.join(HERE, "_ref", "libref_testbed.so")


def network_config(n_levels=16, per_level_scale=1.447, learning_rate=1e-2, ek_loss_weight=0.1):
    """BASELINE config 1 in the layout of the reference's configs/nerf/*.json."""
    return {
        "loss": {"otype": "Huber"},
        "optimizer": {"otype": "Ema", "decay": 0.95, "nested": {
            "otype": "ExponentialDecay", "decay_start": 20000, "decay_interval": 10000, "decay_base": 0.33, "nested": {
                "otype": "Adam", "learning_rate": learning_rate, "beta1": 0.9, "beta2": 0.99, "epsilon": 1e-15, "l2_reg": 1e-6}}},
        "encoding": {"otype": "HashGrid", "n_levels": n_levels, "n_features_per_level": 2, "log2_hashmap_size": 19, "base_resolution": 16,
                     "per_level_scale": per_level_scale},
        "network": {"otype": "FullyFusedMLP", "activation": "ReLU", "output_activation": "None", "n_neurons": 64, "n_hidden_layers": 1, "sdf_bias": -0.1},
        "dir_encoding": {"otype": "Composite", "nested": [{"n_dims_to_encode": 3, "otype": "SphericalHarmonics", "degree": 4},
                                                          {"otype": "Identity", "n_bins": 4, "degree": 4}]},
        "rgb_network": {"otype": "FullyFusedMLP", "activation": "ReLU", "output_activation": "None", "n_neurons": 64, "n_hidden_layers": 2},
        "hyperparams": {"linear_color": False, "first_frame_max_training_step": 10 ** 9, "next_frame_max_training_step": 10 ** 9,
                        "predict_global_movement": False, "mask_loss_weight": 0.0, "ek_loss_weight": ek_loss_weight, "anneal_end": 0}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--views", type=int, default=64)
    ap.add_argument("--res", type=int, default=512)
    ap.add_argument("--batch", type=int, default=1 << 18)
    ap.add_argument("--warmup", type=int, default=520)
    ap.add_argument("--steps", type=int, default=200)
    args = ap.parse_args()
    if not os.path.exists(LIB):
        print(json.dumps({"unavailable": "oracle/_ref/libref_testbed.so was not built (no reference checkout at build time)"}))
        return 0
    sys.path.insert(0, ROOT)
    import numpy as np
    from neus2_b200 import _lib as L
    from neus2_b200 import synthetic as S
    work = tempfile.mkdtemp(prefix="n2b_ref_")
    try:
        scene = S.render_sphere_views(args.views, args.res, args.res, fov_deg=40.0, radius=0.3, seed=0, device="cuda")
        transforms = S.write_transforms_dataset(scene, os.path.join(work, "data"))
        # the SDF network's initial weights, which the reference reads from utils/mlp_weights.txt in its working directory: the
        # sphere-like initialisation this repository's own runs start from
        os.makedirs(os.path.join(work, "utils"))
        init = S.init_params(L.grid_n_params(L.grid_desc()), seed=1337)
        np.savetxt(os.path.join(work, "utils", "mlp_weights.txt"), init[:4096].astype(np.float32), fmt="%.9g")
        lib = C.CDLL(LIB)
        n = args.warmup + args.steps
        losses, ms, stats = (C.c_float * n)(), C.c_float(0), (C.c_uint32 * 4)()
        sys.stdout.flush()
        rc = lib.ref_testbed_train(work.encode(), transforms.encode(), json.dumps(network_config()).encode(), C.c_uint32(args.batch),
                                   C.c_uint32(args.warmup), C.c_uint32(args.steps), losses, C.byref(ms), stats)
        ls = list(losses)
        print("\n" + json.dumps({"rc": rc, "ms_per_step": ms.value / max(args.steps, 1), "steps": args.steps, "warmup": args.warmup, "batch": args.batch,
                                 "views": args.views, "resolution": args.res, "loss_first": ls[0], "loss_after_warmup": ls[max(args.warmup - 1, 0)],
                                 "loss_last": ls[-1], "rays_per_batch": stats[0], "measured_batch_size": stats[1],
                                 "measured_batch_size_before_compaction": stats[2], "training_step": stats[3]}), flush=True)
        return 0 if rc == 0 else 1
    finally:
        shutil.rmtree(work, ignore_errors=True)


if __name__ == "__main__":
    sys.exit(main())
