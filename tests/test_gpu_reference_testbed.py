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


def _run_ref(args, timeout=600):
    r = subprocess.run([sys.executable, os.path.join(ROOT, "oracle", "run_ref_testbed.py")] + args, capture_output=True, text=True, timeout=timeout, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])


def _need_ref():
    if not os.path.exists(os.path.join(ROOT, "oracle", "_ref", "libref_testbed.so")):
        pytest.skip("oracle/_ref/libref_testbed.so was not built: no reference checkout at build time")


VARIANTS = {
    # what the dataset writer produces: per-frame intrinsics, scale 1, offset 0
    "as_written": lambda js: None,
    # the defaults of the loader (scale 0.33, offset 0.5), file-level field of view, no per-frame intrinsics
    "defaults_and_camera_angle": lambda js: ([js.pop(k) for k in ("scale", "offset", "fl_x", "fl_y", "cx", "cy")],
                                             [[f.pop(k) for k in ("fl_x", "fl_y", "cx", "cy")] for f in js["frames"]],
                                             js.update(camera_angle_x=0.61, camera_angle_y=0.47)),
    # explicit scale and per-axis offset, an up vector, fewer frames than listed, per-frame principal points off centre
    "scale_offset_up_n_frames": lambda js: (js.update(scale=0.41, offset=[0.45, 0.5, 0.58], up=[0.1, 0.2, 0.97], n_frames=4),
                                            [f.update(cx=f["cx"] + 3.25, cy=f["cy"] - 1.5) for f in js["frames"]]),
    # an aabb that is fitted into the unit cube, transparent pixels turned white
    "aabb_fit_white_transparent": lambda js: js.update(aabb=[[-1.2, -0.9, -1.0], [1.1, 1.3, 0.8]], white_transparent=True),
}


@pytest.mark.parametrize("variant", sorted(VARIANTS))
def test_dataset_loader_equals_the_reference_loader(tmp_path, variant):
    """neus2_b200.loader against ngp::load_nerf (src/nerf_loader.cu:197) on the same files: cameras, intrinsics, dataset scale and
    offset, and every pixel byte as the reference hands them to training."""
    _need_ref()
    import numpy as np
    from neus2_b200 import loader
    from neus2_b200 import synthetic as S
    scene = S.render_sphere_views(6, 96, 64, fov_deg=40.0, radius=0.3, seed=0, device="cuda")
    tr = S.write_transforms_dataset(scene, str(tmp_path / "data"))
    with open(tr) as f:
        js = json.load(f)
    VARIANTS[variant](js)
    with open(tr, "w") as f:
        json.dump(js, f)
    out = _run_ref(["--data", str(tmp_path / "data"), "--load-only", str(tmp_path / "ld.npz")])
    assert out["rc"] == 0
    t = np.load(str(tmp_path / "ld.npz"))
    ds = loader.load_nerf_dataset(tr)
    n = int(t["header"][0])
    assert n == ds["n_images"] == (4 if variant == "scale_offset_up_n_frames" else 6)
    assert (int(t["header"][1]), int(t["header"][2]), int(t["header"][3])) == (96, 64, 1), "width, height, one byte per channel"
    assert int(t["header"][4]) == ds["aabb_scale"] and bool(t["header"][6]) == ds["from_na"] and bool(t["header"][7]) == ds["from_mitsuba"]
    assert np.float32(t["floats"][0]) == np.float32(ds["scale"]), "scale"
    assert np.array_equal(t["floats"][1:4], np.asarray(ds["offset"], np.float32)), "offset"
    assert np.array_equal(t["floats"][4:7], np.asarray(ds["up"], np.float32)), "up"
    mine = np.asarray(ds["xforms"], np.float32).reshape(-1, 4, 3).transpose(0, 2, 1).reshape(-1, 12)  # column major -> row major
    assert np.array_equal(mine.view(np.uint32), t["xforms"].view(np.uint32)), "camera matrices bit for bit"
    assert np.array_equal(np.asarray(ds["focal"], np.float32).view(np.uint32), t["focal"].view(np.uint32)), "focal lengths bit for bit"
    assert np.array_equal(np.asarray(ds["principal"], np.float32).view(np.uint32), t["principal"].view(np.uint32)), "principal points bit for bit"
    px = np.ascontiguousarray(ds["pixels"]).view(np.uint8).reshape(-1)
    assert px.size == t["pixels"].size and np.array_equal(px, t["pixels"]), "pixel bytes"


def _lockstep(mine_i, ref, mine_loss, ref_loss, restart_steps=()):
    """Compares per-step (rays per batch, compacted batch, samples before compaction) of the two loops; returns the number of
    steps for which they drew the same rays.  restart_steps: steps at which the ray count restarts (first step of a frame)."""
    in_step = 0
    for i in range(len(ref)):
        if i > 0 and i not in restart_steps and mine_i[i - 1, 0] != ref[i - 1, 0]:
            break  # the tuner moved apart one step earlier: different rays from here on
        assert abs(mine_i[i, 2] - ref[i, 2]) <= 2, "step %d: samples before compaction %d, reference %d" % (i, mine_i[i, 2], ref[i, 2])
        dropped = ref[i, 1] != ref[i, 2] or i == 0 or i in restart_steps  # (a frame's first step always has more samples than room)
        if not dropped:
            assert abs(mine_i[i, 1] - ref[i, 1]) <= 2, "step %d: compacted batch %d, reference %d" % (i, mine_i[i, 1], ref[i, 1])
            assert mine_i[i, 0] == ref[i, 0], "step %d: rays per batch %d, reference %d" % (i, mine_i[i, 0], ref[i, 0])
            # the reference reads its loss back on these steps; a ray's random background colour is drawn by its slot in the
            # batch, which is the arrival order there: the same rays, differently coloured, so the sums agree only roughly
            if i % 16 == 0 and i > 0 and ref_loss[i] > 0:
                assert abs(mine_loss[i] - ref_loss[i]) <= 0.2 * ref_loss[i], "step %d: loss %g, reference %g" % (i, mine_loss[i], ref_loss[i])
        else:
            assert abs(mine_i[i, 1] - ref[i, 1]) <= 0.01 * ref[i, 1], "step %d: compacted batch %d, reference %d" % (i, mine_i[i, 1], ref[i, 1])
        in_step = i + 1
    return in_step


def test_training_loop_follows_the_reference_loop(tmp_path):
    """This repository's training loop (neus2b_testbed_*) and the reference's own (Testbed::frame) on the same dataset files with the
    same seed and the same initial parameters: the batch tuner's ray count, the number of samples before compaction and the
    compacted batch size are compared step by step.

    Part one, all parameters zero: the network's outputs are then the same constants on both sides and stay so (no gradient
    reaches a weight through dead units; only the variance trains), which takes the arithmetic of the two network
    implementations out of the comparison and leaves the loop's machinery: the random streams and their seeding, the occupancy
    grid update and its bits, the sample generator, the loss pass's compaction, the room left by the previous step
    (max_inference), the tuner.  These must agree step for step.  Two things are not reproducible and are allowed for: the
    reference's build contracts multiplies and adds, which moves last bits of sample positions (a sample on a cell boundary now
    and then: counts may differ by one or two); and when a step has more samples than room, the reference drops the rays that
    arrive last in atomic order, this repository the last in ray order (the compacted size then differs by a ray or two, which
    can move the tuner by one granule of 128 rays -- from there on the two runs see different rays).

    Part two, the sphere initialisation: the first step (identical parameters) must give the same three numbers; from the second
    step on the two network implementations round differently, Adam turns that into +-learning-rate differences of individual
    weights, occupancy cells near the threshold fall differently, and the runs are compared by their averages and their loss."""
    _need_ref()
    import numpy as np
    from oracle import run_ref_testbed as R
    from neus2_b200 import _lib as L
    from neus2_b200 import synthetic as S
    from neus2_b200 import testbed as T
    from util import record
    n_steps, batch = 64, 1 << 17
    scene = S.render_sphere_views(12, 128, 128, fov_deg=40.0, radius=0.3, seed=0, device="cuda")
    tr = S.write_transforms_dataset(scene, str(tmp_path / "data"))

    def both(tag, params):
        tb = T.Testbed.from_network_config(R.network_config(), batch_size=batch)
        tb.load_training_data_from_json(tr)
        if params is not None:
            tb.set_params(params)
        np.save(str(tmp_path / (tag + ".npy")), tb.get_params())
        mine = []
        for _ in range(n_steps):
            s = tb.train(1)
            mine.append((s.rays_per_batch, s.measured_batch_size, s.measured_batch_size_before_compaction, s.loss))
        tb.close()
        out = _run_ref(["--data", str(tmp_path / "data"), "--batch", str(batch), "--warmup", "0", "--steps", str(n_steps), "--params",
                        str(tmp_path / (tag + ".npy")), "--trace", str(tmp_path / (tag + ".npz"))])
        assert out["rc"] == 0 and out["training_step"] == n_steps
        t = np.load(str(tmp_path / (tag + ".npz")))
        return np.array([m[:3] for m in mine], np.int64), np.array([m[3] for m in mine]), t["stats"].astype(np.int64), t["loss"]

    mine_i, mine_loss, ref, ref_loss = both("zero", None)
    assert not np.load(str(tmp_path / "zero.npy")).any()
    in_step = _lockstep(mine_i, ref, mine_loss, ref_loss)
    assert in_step >= 16, "the loops left each other after %d steps" % in_step
    assert abs(mine_i[8:, 0].mean() - ref[8:, 0].mean()) <= 0.03 * ref[8:, 0].mean()
    assert abs(mine_i[8:, 1].mean() - ref[8:, 1].mean()) <= 0.03 * ref[8:, 1].mean()
    record("loop_parity", steps_in_lockstep=in_step, steps=n_steps, exact_steps=int(((mine_i == ref).all(1)).sum()))

    ng = L.grid_n_params(L.grid_desc())
    live_i, live_loss, lref, lref_loss = both("sphere", S.init_params(ng, seed=1337))
    assert abs(live_i[0, 2] - lref[0, 2]) <= 2 and abs(live_i[0, 1] - lref[0, 1]) <= 0.01 * lref[0, 1] and live_i[0, 0] == lref[0, 0], (live_i[0], lref[0])
    assert abs(live_i[8:, 0].mean() - lref[8:, 0].mean()) <= 0.15 * lref[8:, 0].mean(), "rays per batch on average"
    assert abs(live_i[8:, 2].mean() - lref[8:, 2].mean()) <= 0.15 * lref[8:, 2].mean(), "samples before compaction on average"
    mine_end, ref_end = float(np.mean(live_loss[-16:])), float(np.mean(lref_loss[-16:]))
    assert mine_end < 0.3 * live_loss[0] and ref_end < 0.3 * lref_loss[0] and 0.4 * ref_end <= mine_end <= 2.5 * ref_end, (mine_end, ref_end)
    record("loop_parity_sphere_init", first_step=[int(v) for v in live_i[0]], reference_first_step=[int(v) for v in lref[0]],
           loss_last16=mine_end, reference_loss_last16=ref_end)


def test_dynamic_sequence_follows_the_reference_loop(tmp_path):
    """The same comparison across a frame switch of a dynamic sequence (a directory of per-frame transforms files; both loops
    move on by themselves when the frame's steps are done): 48 steps of the first frame, then the second frame with 16 steps of
    motion-only training (occupancy update every step, the running ray count restarted every step), the occupancy grid cleared
    when the canonical model joins, the tuner and the ray generator's stream restarted with the frame.  Zero parameters, as in
    part one above."""
    _need_ref()
    import numpy as np
    from oracle import run_ref_testbed as R
    from neus2_b200 import synthetic as S
    from neus2_b200 import testbed as T
    from util import record
    first, later, motion_only, batch = 48, 48, 16, 1 << 16
    hyper = {"first_frame_max_training_step": first, "next_frame_max_training_step": later, "predict_global_movement": True,
             "predict_global_movement_training_step": motion_only, "optimizer_leaf": {"after_learning_rate": 1e-3}}
    poses = S.sequence_poses(2, seed=4, bulge=0.0, max_rot_deg=12.0, max_shift=0.05)
    scenes = [S.render_sphere_views(12, 128, 128, fov_deg=40.0, device="cuda", seed=1, rotation=Rm, translation=t, radius=r) for Rm, t, r in poses]
    d = S.write_sequence_dataset(scenes, str(tmp_path / "seq"))
    tb = T.Testbed.from_network_config(R.merged_config(hyper), batch_size=batch)
    tb.load_training_data_from_json(d)
    np.save(str(tmp_path / "p0.npy"), tb.get_params())
    n = first + later
    mine, where = [], []
    for _ in range(n):
        tb.frame()
        s = tb.stats
        where.append((tb.movement()[0], s.training_step))
        mine.append((s.rays_per_batch, s.measured_batch_size, s.measured_batch_size_before_compaction, s.loss))
    tb.close()
    out = _run_ref(["--data", d, "--batch", str(batch), "--warmup", "0", "--steps", str(n), "--params", str(tmp_path / "p0.npy"), "--trace",
                    str(tmp_path / "trace.npz"), "--hyper", json.dumps(hyper)])
    assert out["rc"] == 0
    t = np.load(str(tmp_path / "trace.npz"))
    assert np.array_equal(np.array(where, np.int64), t["frames"].astype(np.int64)), "frame and step within the frame after every call"
    assert where[first - 1] == (0, first) and where[first] == (1, 1) and where[-1] == (1, later)
    mine_i = np.array([m[:3] for m in mine], np.int64)
    in_step = _lockstep(mine_i, t["stats"].astype(np.int64), [m[3] for m in mine], t["loss"], restart_steps=(first,))
    assert in_step >= first + motion_only + 8, "the loops left each other after %d steps" % in_step
    record("loop_parity_sequence", steps_in_lockstep=in_step, steps=n)


def test_sdf_lattice_equals_the_reference_testbed(tmp_path):
    """Testbed::get_density_on_grid of the reference (the lattice its marching cubes runs on: lattice positions, order, and the SDF
    through its NerfNetwork over the layered kernels) against neus2b_testbed_sdf_grid with the same parameters."""
    _need_ref()
    import numpy as np
    from oracle import run_ref_testbed as R
    from neus2_b200 import _lib as L
    from neus2_b200 import synthetic as S
    from neus2_b200 import testbed as T
    from util import record
    scene = S.render_sphere_views(4, 64, 64, fov_deg=40.0, radius=0.3, seed=0, device="cuda")
    tr = S.write_transforms_dataset(scene, str(tmp_path / "data"))
    tb = T.Testbed.from_network_config(R.network_config())
    tb.load_training_data_from_json(tr)
    ng = L.grid_n_params(tb.config.grid)
    p0 = S.init_params(ng, seed=1337)
    rng = np.random.default_rng(9)
    p0[12288:12288 + ng] = rng.uniform(-2e-2, 2e-2, ng)  # a table that matters
    p0[:3072].reshape(64, 48)[:, 3:35] = rng.normal(0, 0.05, (64, 32))
    tb.set_params(p0)
    np.save(str(tmp_path / "p0.npy"), tb.get_params())
    res = 48
    mine = tb.sdf_grid(res, use_ema=False).cpu().numpy()
    tb.close()
    out = _run_ref(["--data", str(tmp_path / "data"), "--params", str(tmp_path / "p0.npy"), "--sdf-grid", str(tmp_path / "sdf.npy"), "--sdf-res", str(res)])
    assert out["rc"] == 0
    ref = np.load(str(tmp_path / "sdf.npy"))
    assert mine.shape == ref.shape == (res, res, res)
    err = np.abs(mine - ref)
    record("ref_testbed_sdf_lattice", max_abs_err=float(err.max()), mean_abs_err=float(err.mean()), std=float(ref.std()))
    assert ref.std() > 0.05 and (ref < 0).any() and (ref > 0).any()
    assert err.max() <= 4e-3 * max(1.0, float(np.abs(ref).max())), err.max()
    assert (np.sign(mine) == np.sign(ref)).mean() > 0.999


def test_snapshots_load_across_the_two_testbeds(tmp_path):
    """Testbed::save_snapshot / load_snapshot of the reference (src/testbed.cu:3134-3244) against neus2_b200.snapshot, both ways:
    the reference trains 40 steps and saves, this repository loads the file (same SDF lattice, step and tuner state) and trains
    on; then this repository saves and the reference's load_snapshot takes the file (same lattice, step and tuner state)."""
    _need_ref()
    import ctypes as C
    import numpy as np
    import torch
    from oracle import run_ref_testbed as R
    from neus2_b200 import _lib as L
    from neus2_b200 import synthetic as S
    from neus2_b200 import testbed as T
    from util import record
    res, batch = 40, 1 << 16
    scene = S.render_sphere_views(8, 96, 96, fov_deg=40.0, radius=0.3, seed=0, device="cuda")
    S.write_transforms_dataset(scene, str(tmp_path / "data"))
    common = ["--data", str(tmp_path / "data"), "--batch", str(batch), "--sdf-res", str(res)]
    tb = T.Testbed.from_network_config(R.network_config(), batch_size=batch)
    tb.load_training_data_from_json(str(tmp_path / "data" / "transforms.json"))
    tb.set_params(S.init_params(L.grid_n_params(tb.config.grid), seed=1337))
    np.save(str(tmp_path / "p0.npy"), tb.get_params())

    def occupied(t):
        bits = torch.empty(128 ** 3 // 8, dtype=torch.uint8, device="cuda")
        torch.cuda.synchronize()
        C.CDLL("libcudart.so.12").cudaMemcpy(C.c_void_p(bits.data_ptr()), C.c_void_p(t.device_ptrs()["bitfield"]), C.c_size_t(bits.numel()), 3)
        return int(np.unpackbits(bits.cpu().numpy()).sum())

    saved = _run_ref(common + ["--params", str(tmp_path / "p0.npy"), "--steps", "40", "--snapshot-save", str(tmp_path / "ref.msgpack"), "--sdf-grid",
                               str(tmp_path / "ref_sdf.npy")])
    assert saved["rc"] == 0 and saved["training_step"] == 40
    tb.load_snapshot(str(tmp_path / "ref.msgpack"))
    ref_sdf = np.load(str(tmp_path / "ref_sdf.npy"))
    err_in = float(np.abs(tb.sdf_grid(res, use_ema=True).cpu().numpy() - ref_sdf).max())
    assert err_in <= 1e-3 and ref_sdf.std() > 0.02 and (ref_sdf < 0).any() and (ref_sdf > 0).any()
    assert tb.training_step == 40 and tb.stats.rays_per_batch == saved["rays_per_batch"]
    assert abs(occupied(tb) - saved["occupied_cells"]) <= 0.01 * saved["occupied_cells"]  # (the file holds the grid in fp16)
    st = tb.train(5)
    assert st.training_step == 45 and np.isfinite(st.loss)
    tb.save_snapshot(str(tmp_path / "mine.msgpack"))
    mine_sdf = tb.sdf_grid(res, use_ema=True).cpu().numpy()
    loaded = _run_ref(common + ["--snapshot-load", str(tmp_path / "mine.msgpack"), "--sdf-grid", str(tmp_path / "ref2_sdf.npy")])
    assert loaded["rc"] == 0 and loaded["training_step"] == 45 and loaded["rays_per_batch"] == st.rays_per_batch
    assert loaded["measured_batch_size"] == st.measured_batch_size
    err_out = float(np.abs(mine_sdf - np.load(str(tmp_path / "ref2_sdf.npy"))).max())
    assert err_out <= 1e-3
    assert abs(occupied(tb) - loaded["occupied_cells"]) <= 0.01 * loaded["occupied_cells"]
    record("snapshot_cross_load", sdf_err_reference_to_this=err_in, sdf_err_this_to_reference=err_out)
    tb.close()


def test_mesh_export_equals_the_reference_testbed(tmp_path):
    """Testbed::compute_and_save_marching_cubes_mesh of the reference (lattice, marching cubes, 1-ring normals, vertex colours from
    the network, writer) against Testbed.compute_and_save_marching_cubes_mesh here, from the same parameters after a short training
    of the reference's loop handed over as a snapshot.  The reference numbers vertices in the arrival order of its atomics:
    the OBJ files are compared as sets -- vertices matched by position, then positions, colours and normals as printed, and the
    faces through the matching."""
    _need_ref()
    import numpy as np
    from scipy.spatial import cKDTree
    from oracle import run_ref_testbed as R
    from neus2_b200 import _lib as L
    from neus2_b200 import synthetic as S
    from neus2_b200 import testbed as T
    from oracle import extract_mc_table as X
    from util import record
    table = X.load()
    if table is None:
        pytest.skip("the reference's case table was not extracted on this machine (oracle/_ref/mc_tri_table.npy is missing)")
    res, batch = 64, 1 << 16
    scene = S.render_sphere_views(8, 96, 96, fov_deg=40.0, radius=0.3, seed=0, device="cuda")
    S.write_transforms_dataset(scene, str(tmp_path / "data"))
    tb = T.Testbed.from_network_config(R.network_config(), batch_size=batch)
    tb.load_training_data_from_json(str(tmp_path / "data" / "transforms.json"))
    tb.set_params(S.init_params(L.grid_n_params(tb.config.grid), seed=1337))
    np.save(str(tmp_path / "p0.npy"), tb.get_params())
    out = _run_ref(["--data", str(tmp_path / "data"), "--batch", str(batch), "--sdf-res", str(res), "--params", str(tmp_path / "p0.npy"), "--steps", "60",
                    "--snapshot-save", str(tmp_path / "ref.msgpack"), "--mesh", str(tmp_path / "ref.obj")])
    assert out["rc"] == 0
    tb.load_snapshot(str(tmp_path / "ref.msgpack"))
    import torch
    tb.compute_and_save_marching_cubes_mesh(str(tmp_path / "mine.obj"), resolution=res, tri_table=torch.from_numpy(table))
    tb.close()

    def read(path):
        v, vn, f = [], [], []
        for line in open(path):
            p = line.split()
            if not p:
                continue
            if p[0] == "v":
                v.append([float(x) for x in p[1:7]])
            elif p[0] == "vn":
                vn.append([float(x) for x in p[1:4]])
            elif p[0] == "f":
                f.append([int(x.split("/")[0]) - 1 for x in p[1:4]])
        return np.array(v), np.array(vn), np.array(f, np.int64)
    rv, rn, rf = read(tmp_path / "ref.obj")
    mv, mn, mf = read(tmp_path / "mine.obj")
    assert len(rv) == len(mv) > 1000 and len(rv) % 128 == 0 and len(rf) == len(mf) and len(rn) == len(mn) == len(rv)
    used = int(rf.max()) + 1  # the files end with the unused entries of the reference's vertex buffer (all at the origin)
    assert int(mf.max()) + 1 == used and np.array_equal(rv[used:], mv[used:]) and np.array_equal(rn[used:], mn[used:])
    rv, rn, mv, mn = rv[:used], rn[:used], mv[:used], mn[:used]
    # positions are printed with five decimals (vertices next to a lattice point can print alike): every reference vertex is held
    # against the vertices here that print at the nearest position, and takes the one closest in colour and normal
    tree = cKDTree(mv[:, :3])
    dist, _ = tree.query(rv[:, :3])
    assert np.quantile(dist, 0.99) <= 2e-5 and dist.max() <= 2e-3, (dist.max(), np.quantile(dist, 0.99))
    color_err, normal_err = np.zeros(len(rv)), np.zeros(len(rv))
    for k, cand in enumerate(tree.query_ball_point(rv[:, :3], dist + 1e-9)):
        d = np.abs(mv[cand, 3:6] - rv[k, 3:6]).max(1) + np.abs(mn[cand] - rn[k]).max(1)
        j = cand[int(np.argmin(d))]
        color_err[k], normal_err[k] = np.abs(mv[j, 3:6] - rv[k, 3:6]).max(), np.abs(mn[j] - rn[k]).max()
    record("ref_testbed_mesh_export", vertices=len(rv), faces=len(rf), worst_position=float(dist.max()), worst_colour=float(color_err.max()),
           mean_colour=float(color_err.mean()), worst_normal=float(normal_err.max()))
    assert color_err.max() <= 0.02 and color_err.mean() <= 2e-3, "vertex colours (printed with three decimals)"
    assert np.quantile(normal_err, 0.99) <= 0.02
    # the faces by their printed corner positions (nine numbers each), matched by nearest neighbour so that the comparison depends
    # neither on the numbering of the vertices nor on the order of the faces
    corners = lambda v, f: v[f.reshape(-1), :3].reshape(-1, 9)
    face_dist, _ = cKDTree(corners(mv, mf)).query(corners(rv, rf))
    back_dist, _ = cKDTree(corners(rv, rf)).query(corners(mv, mf))
    for d in (face_dist, back_dist):
        assert d.max() <= 4e-3 and np.quantile(d, 0.99) <= 6e-5, "the same faces, corner order included"


def test_reconstruction_accuracy_next_to_the_reference_loop(tmp_path):
    """The surface after 600 steps of the reference's own loop and after 600 steps of this repository's, from the same
    initialisation on the same dataset files: mean distance of the mesh vertices (128^3 lattice) to the analytic sphere.  (The
    kernels under the reference's objects are this repository's layered ones; what differs is everything above them.)"""
    _need_ref()
    import numpy as np
    import torch
    from oracle import extract_mc_table as X
    from oracle import run_ref_testbed as R
    from neus2_b200 import _lib as L
    from neus2_b200 import synthetic as S
    from neus2_b200 import testbed as T
    from util import record
    steps, batch, res = 600, 1 << 16, 128
    scene = S.render_sphere_views(16, 128, 128, fov_deg=40.0, radius=0.3, seed=0, device="cuda")
    S.write_transforms_dataset(scene, str(tmp_path / "data"))
    tb = T.Testbed.from_network_config(R.network_config(), batch_size=batch)
    tb.load_training_data_from_json(str(tmp_path / "data" / "transforms.json"))
    tb.set_params(S.init_params(L.grid_n_params(tb.config.grid), seed=1337))
    np.save(str(tmp_path / "p0.npy"), tb.get_params())
    out = _run_ref(["--data", str(tmp_path / "data"), "--batch", str(batch), "--sdf-res", str(res), "--params", str(tmp_path / "p0.npy"), "--steps", str(steps),
                    "--mesh", str(tmp_path / "ref.obj")])
    assert out["rc"] == 0 and out["training_step"] == steps
    st = tb.train(steps)
    table = X.load()
    tb.compute_and_save_marching_cubes_mesh(str(tmp_path / "mine.obj"), resolution=res, tri_table=torch.from_numpy(table) if table is not None else None)
    tb.close()

    def surface_error(path):
        v, f = [], []
        for line in open(path):
            p = line.split()
            if p and p[0] == "v":
                v.append([float(x) for x in p[1:4]])
            elif p and p[0] == "f":
                f.append([int(x.split("/")[0]) - 1 for x in p[1:4]])
        v = np.array(v)[np.unique(np.array(f).reshape(-1))]  # (the unused tail of the vertex buffer is in the file too)
        r = np.linalg.norm(v - 0.5, axis=1)
        return float(np.abs(r - 0.3).mean()), len(v)
    ref_err, ref_n = surface_error(tmp_path / "ref.obj")
    mine_err, mine_n = surface_error(tmp_path / "mine.obj")
    record("reconstruction_next_to_reference_loop", steps=steps, mean_distance=mine_err, reference_mean_distance=ref_err, vertices=mine_n, reference_vertices=ref_n,
           loss=float(st.loss))
    assert ref_n > 5000 and mine_n > 5000 and ref_err < 0.02 and mine_err < 0.02
    # (either loop's figure moves between 0.008 and 0.011 from run to run: atomics, and the reference's arrival order)
    assert mine_err <= 1.5 * ref_err + 2e-3, (mine_err, ref_err)


def test_config1_long_run_shares_the_fate_of_the_reference_loop(tmp_path):
    """BASELINE config 1 as it is written (learning rate 1e-2, eikonal weight 0.1, all 16 levels open from the first step) for 2000
    steps in both loops, same initialisation, same files.  On the synthetic sphere this combination trains well for 1200-1500
    steps and then falls apart within a few dozen steps -- to a fog (loss 3e-3, the tuner back at its smallest ray counts) or to
    an empty occupancy grid (the tuner at its largest), depending on the run -- in this repository's loop and in the reference's
    own loop alike, which is the point of the test: both are in good shape at step 1000, and at step 2000 they are either both
    still in good shape or both not."""
    _need_ref()
    import numpy as np
    from oracle import run_ref_testbed as R
    from neus2_b200 import _lib as L
    from neus2_b200 import synthetic as S
    from neus2_b200 import testbed as T
    from util import record
    steps = 2000
    scene = S.render_sphere_views(64, 512, 512, fov_deg=40.0, radius=0.3, seed=0, device="cuda")
    S.write_transforms_dataset(scene, str(tmp_path / "data"))
    tb = T.Testbed.from_network_config(R.network_config())
    tb.load_training_data_from_json(str(tmp_path / "data" / "transforms.json"))
    tb.set_params(S.init_params(L.grid_n_params(tb.config.grid), seed=1337))
    np.save(str(tmp_path / "p0.npy"), tb.get_params())
    mine = {}
    for k in range(steps // 100):
        st = tb.train(100)
        mine[int(st.training_step)] = (float(st.loss), int(st.rays_per_batch))
    tb.close()
    out = _run_ref(["--data", str(tmp_path / "data"), "--warmup", "0", "--steps", str(steps), "--params", str(tmp_path / "p0.npy"), "--trace",
                    str(tmp_path / "trace.npz")], timeout=900)
    assert out["rc"] == 0
    t = np.load(str(tmp_path / "trace.npz"))
    ref = {s: (float(t["loss"][(s - 1) // 16 * 16]), int(t["stats"][s - 1][0])) for s in mine}
    best_mine, best_ref = min(v[0] for v in mine.values()), min(v[0] for v in ref.values())
    record("config1_long_run", this_repository={str(k): v for k, v in mine.items()}, reference_loop={str(k): v for k, v in ref.items()})
    assert best_mine < 1e-4 and best_ref < 1e-4, "both reach a sharp surface on the way"
    assert 0.4 * best_ref <= best_mine <= 2.5 * best_ref
    good = lambda v: v[0] < 1.5e-4 and 4096 <= v[1] <= 200000  # a sharp surface: small loss, tens of thousands of rays per batch
    assert good(mine[1000]) and good(ref[1000]), (mine[1000], ref[1000])
    assert good(mine[steps]) == good(ref[steps]), (mine[steps], ref[steps])
