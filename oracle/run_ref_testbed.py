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


def merged_config(extra=None):
    """network_config() with `extra` merged into its hyperparams; the entry "optimizer_leaf" goes into the innermost optimizer."""
    config = network_config()
    extra = dict(extra or {})
    leaf = config["optimizer"]
    while "nested" in leaf:
        leaf = leaf["nested"]
    leaf.update(extra.pop("optimizer_leaf", {}))
    config["hyperparams"].update(extra)
    return config


def load_only(transforms, out_path, max_images=256, pixel_capacity=1 << 28):
    """ngp::load_nerf on one transforms file; cameras and pixel bytes as the reference hands them to training."""
    import numpy as np
    lib = C.CDLL(LIB)
    header, floats = np.zeros(8, np.uint32), np.zeros(8, np.float32)
    xforms, focal, principal = np.zeros((max_images, 12), np.float32), np.zeros((max_images, 2), np.float32), np.zeros((max_images, 2), np.float32)
    pixels = np.zeros(pixel_capacity, np.uint8)
    ptr = lambda a: a.ctypes.data_as(C.c_void_p)
    rc = lib.ref_load_dataset(transforms.encode(), C.c_uint32(max_images), ptr(header), ptr(floats), ptr(xforms), ptr(focal), ptr(principal), ptr(pixels),
                              C.c_uint64(pixel_capacity))
    n = int(min(header[0], max_images))
    image_bytes = int(header[1]) * int(header[2]) * 4 * int(header[3])
    n_pix = min(n, pixel_capacity // max(image_bytes, 1))
    if rc == 0:
        np.savez(out_path, header=header, floats=floats, xforms=xforms[:n], focal=focal[:n], principal=principal[:n], pixels=pixels[:n_pix * image_bytes])
    print("\n" + json.dumps({"rc": rc, "n_images": n}), flush=True)
    return 0 if rc == 0 else 1


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--views", type=int, default=64)
    ap.add_argument("--res", type=int, default=512)
    ap.add_argument("--batch", type=int, default=1 << 18)
    ap.add_argument("--warmup", type=int, default=520)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--data", default=None, help="directory of an existing dataset (transforms.json); default: a synthetic scene is written")
    ap.add_argument("--params", default=None, help=".npy file of full-precision initial parameters that replace the drawn ones")
    ap.add_argument("--hyper", default=None, help="json object merged into the network configuration's hyperparams (and, under the key "
                    "\"optimizer_leaf\", into the innermost optimizer)")
    ap.add_argument("--snapshot-save", default=None, help="snapshot mode: build from --params, train --steps, save a snapshot here")
    ap.add_argument("--snapshot-load", default=None, help="snapshot mode: take everything from this snapshot instead")
    ap.add_argument("--mesh", default=None, help="snapshot mode: also run Testbed::compute_and_save_marching_cubes_mesh at --sdf-res into this file")
    ap.add_argument("--sdf-grid", default=None, help="with --params and --sdf-res: evaluate Testbed::get_density_on_grid without training and write it to this .npy file")
    ap.add_argument("--sdf-res", type=int, default=64)
    ap.add_argument("--load-only", default=None, help="only run the reference's dataset loader on --data and write what it returns to this .npz file")
    ap.add_argument("--trace", default=None, help="write per-step rays_per_batch / measured batch sizes / loss to this .npz file")
    ap.add_argument("--grid-after", type=int, default=0, help="with --trace: also store the occupancy grid's densities after this many steps")
    args = ap.parse_args()
    if not os.path.exists(LIB):
        print(json.dumps({"unavailable": "oracle/_ref/libref_testbed.so was not built (no reference checkout at build time)"}))
        return 0
    sys.path.insert(0, ROOT)
    import numpy as np
    from neus2_b200 import _lib as L
    from neus2_b200 import synthetic as S
    if args.load_only:
        return load_only(os.path.join(os.path.abspath(args.data), "transforms.json"), args.load_only)
    work = tempfile.mkdtemp(prefix="n2b_ref_")
    try:
        if args.data:  # a directory with transforms.json, or a directory of per-frame transforms files (a dynamic sequence)
            transforms = os.path.join(os.path.abspath(args.data), "transforms.json")
            if not os.path.exists(transforms):
                transforms = os.path.abspath(args.data)
        else:
            scene = S.render_sphere_views(args.views, args.res, args.res, fov_deg=40.0, radius=0.3, seed=0, device="cuda")
            transforms = S.write_transforms_dataset(scene, os.path.join(work, "data"))
        # the SDF network's initial weights, which the reference reads from utils/mlp_weights.txt in its working directory: the
        # sphere-like initialisation this repository's own runs start from
        os.makedirs(os.path.join(work, "utils"))
        init = S.init_params(L.grid_n_params(L.grid_desc()), seed=1337)
        np.savetxt(os.path.join(work, "utils", "mlp_weights.txt"), init[:4096].astype(np.float32), fmt="%.9g")
        lib = C.CDLL(LIB)
        if args.snapshot_save or args.snapshot_load or args.mesh:
            params = np.ascontiguousarray(np.load(args.params), np.float32) if args.params else np.zeros(1, np.float32)
            r = args.sdf_res
            out, info = np.zeros((r, r, r), np.float32), np.zeros(4, np.uint32)
            enc = lambda v: v.encode() if v else None
            rc = lib.ref_testbed_snapshot(work.encode(), transforms.encode(), json.dumps(merged_config(json.loads(args.hyper) if args.hyper else None)).encode(),
                                          params.ctypes.data_as(C.c_void_p), C.c_uint64(params.size), C.c_uint32(args.steps), enc(args.snapshot_load),
                                          enc(args.snapshot_save), C.c_uint32(r), out.ctypes.data_as(C.c_void_p), info.ctypes.data_as(C.c_void_p), enc(args.mesh))
            if args.sdf_grid:
                np.save(args.sdf_grid, out)
            print("\n" + json.dumps({"rc": rc, "training_step": int(info[0]), "rays_per_batch": int(info[1]), "measured_batch_size": int(info[2]),
                                     "occupied_cells": int(info[3])}), flush=True)
            return 0 if rc == 0 else 1
        if args.sdf_grid:
            params = np.ascontiguousarray(np.load(args.params), np.float32)
            r = args.sdf_res
            out = np.zeros((r, r, r), np.float32)
            rc = lib.ref_testbed_sdf_grid(work.encode(), transforms.encode(), json.dumps(merged_config(json.loads(args.hyper) if args.hyper else None)).encode(),
                                          params.ctypes.data_as(C.c_void_p), C.c_uint64(params.size), C.c_uint32(r), C.c_uint32(r), C.c_uint32(r),
                                          out.ctypes.data_as(C.c_void_p))
            np.save(args.sdf_grid, out)
            print("\n" + json.dumps({"rc": rc, "sdf_res": r}), flush=True)
            return 0 if rc == 0 else 1
        n = args.warmup + args.steps
        losses, ms, stats, step_stats = (C.c_float * n)(), C.c_float(0), (C.c_uint32 * 4)(), (C.c_uint32 * (3 * n))()
        params = np.ascontiguousarray(np.load(args.params), np.float32) if args.params else None
        grid = np.zeros(128 ** 3, np.float32) if args.grid_after else None  # cascade 0
        bits = np.zeros(8 * 128 ** 3 // 8, np.uint8) if args.grid_after else None  # all cascades
        step_frames, motion = np.zeros((n, 2), np.uint32), np.zeros(28, np.uint16)
        sys.stdout.flush()
        config = merged_config(json.loads(args.hyper) if args.hyper else None)
        rc = lib.ref_testbed_train(work.encode(), transforms.encode(), json.dumps(config).encode(), C.c_uint32(args.batch),
                                   C.c_uint32(args.warmup), C.c_uint32(args.steps), params.ctypes.data_as(C.c_void_p) if params is not None else None,
                                   C.c_uint64(params.size if params is not None else 0), losses, step_stats, C.byref(ms), stats,
                                   C.c_uint32(args.grid_after), grid.ctypes.data_as(C.c_void_p) if grid is not None else None, C.c_uint64(grid.size if grid is not None else 0),
                                   bits.ctypes.data_as(C.c_void_p) if bits is not None else None, C.c_uint64(bits.size if bits is not None else 0),
                                   step_frames.ctypes.data_as(C.c_void_p), motion.ctypes.data_as(C.c_void_p))
        ls = list(losses)
        if args.trace:
            np.savez(args.trace, loss=np.array(ls, np.float32), stats=np.array(list(step_stats), np.uint32).reshape(n, 3), frames=step_frames,
                     motion=motion.view(np.float16).astype(np.float32),
                     **({"density_grid": grid, "bitfield": bits} if grid is not None else {}))
        print("\n" + json.dumps({"rc": rc, "ms_per_step": ms.value / max(args.steps, 1), "steps": args.steps, "warmup": args.warmup, "batch": args.batch,
                                 "views": args.views, "resolution": args.res, "loss_first": ls[0], "loss_after_warmup": ls[max(args.warmup - 1, 0)],
                                 "loss_last": ls[-1], "rays_per_batch": stats[0], "measured_batch_size": stats[1],
                                 "measured_batch_size_before_compaction": stats[2], "training_step": stats[3]}), flush=True)
        return 0 if rc == 0 else 1
    finally:
        shutil.rmtree(work, ignore_errors=True)


if __name__ == "__main__":
    sys.exit(main())
