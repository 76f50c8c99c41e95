"""Dynamic sequences through the training loop (BASELINE config 3 in small): a first frame, then frames of the same object moved
rigidly; every later frame first learns its motion with the canonical model frozen, then trains both; a frame switch folds
the learned motion into the accumulated movement of the rays."""
import numpy as np
import pytest
import torch

from util import record

pytestmark = pytest.mark.gpu


def rot_angle_deg(R):
    return float(np.degrees(np.arccos(np.clip((np.trace(R) - 1) / 2, -1, 1))))


@pytest.fixture(scope="module")
def frames():
    from neus2_b200 import synthetic as S
    poses = S.sequence_poses(3, seed=4, bulge=0.0, max_rot_deg=12.0, max_shift=0.05)
    return poses, [S.render_sphere_views(16, 160, 160, device="cuda", seed=1, rotation=R, translation=t, radius=r) for R, t, r in poses]


def host(scene):
    return [scene[k].cpu().numpy() for k in ("pixels", "xforms", "focal", "principal")]


def test_frames_after_the_first_learn_their_motion(frames):
    from neus2_b200 import _lib as L
    from neus2_b200 import ops
    from neus2_b200 import synthetic as S
    from neus2_b200.testbed import Testbed
    poses, scenes = frames
    tb = Testbed(batch_size=1 << 16, predict_global_movement=1, predict_global_movement_training_step=150, finetune_global_movement=1,
                 reset_density_grid_after_global_movement=0, after_learning_rate=1e-3, gm_learning_rate=1e-2, ek_loss_weight=0.01)
    tb.load_training_data(*host(scenes[0]))
    ng = L.grid_n_params(tb.config.grid)
    tb.set_params(S.init_params(ng, seed=1337))
    st = tb.train(600)
    loss0 = float(np.mean([tb.train(1).loss for _ in range(10)]))
    frame, R, t, d = tb.movement()
    assert frame == 0 and np.array_equal(R, np.eye(3)) and not t.any() and np.allclose(d, ops.DELTA_IDENTITY)
    # ---- frame 1: the object has moved
    tb.next_frame(*host(scenes[1]))
    assert tb.movement()[0] == 1
    before = tb.get_params()
    assert np.array_equal(before.astype(np.float16).astype(np.float32), before), "the weights are carried over as fp16 values"
    first = float(np.mean([tb.train(1).loss for _ in range(5)]))
    st = tb.train(145)
    assert st.training_step == 150 and np.isfinite(first) and np.isfinite(st.loss)
    assert np.array_equal(tb.get_params(), before), "the canonical model is frozen while the motion alone is trained"
    frame, R_acc, t_acc, d = tb.movement()
    assert np.array_equal(R_acc, np.eye(3)) and not t_acc.any(), "nothing is accumulated before the frame ends"
    assert not np.allclose(d, ops.DELTA_IDENTITY)
    tb.train(5)
    assert not np.array_equal(tb.get_params(), before), "behind the motion-only phase the canonical model trains again"
    st = tb.train(80)
    assert np.isfinite(st.loss) and st.loss < 3 * loss0 + 1e-4
    # ---- frame 2: the first frame's motion is now part of the rays' movement
    frame, _, _, d1 = tb.movement()
    bits = np.ascontiguousarray(d1.astype(np.float16)).view(np.uint16)
    R_want, t_want = ops.movement_accumulate(bits, np.eye(3, dtype=np.float32), np.zeros(3, np.float32))
    tb.next_frame(*host(scenes[2]))
    frame, R_acc, t_acc, d = tb.movement()
    assert frame == 2 and np.array_equal(R_acc, R_want) and np.array_equal(t_acc, t_want) and np.allclose(d, ops.DELTA_IDENTITY)
    start = float(np.mean([tb.train(1).loss for _ in range(5)]))
    st = tb.train(195)
    assert st.training_step == 200 and np.isfinite(st.loss) and st.loss < 3 * start + 1e-4
    img = tb.render(96, 96)
    assert (img[..., 3] > 0.5).mean() > 0.03, "the renderer sees the object through the accumulated movement and the motion"
    tb.close()


def test_motion_updates_descend_the_training_loss(frames):
    """End to end: the direction the motion's optimizer moves each parameter (sign of the update at a tiny learning rate, over
    20 steps) is the direction in which the step's loss falls, measured by central differences on a frozen copy of the same
    state.  Checked on every parameter whose slope stands clear of the batch-to-batch noise (the optimizer's direction is an
    average over 20 different batches, the slope is measured on one)."""
    import ctypes as C
    from neus2_b200 import _lib as L
    from neus2_b200 import ops
    from neus2_b200 import snapshot as SN
    from neus2_b200 import synthetic as S
    from neus2_b200.testbed import Testbed
    _, scenes = frames
    kw = dict(batch_size=1 << 16, predict_global_movement=1, predict_global_movement_training_step=100000, ek_loss_weight=0.01)
    tb = Testbed(**kw)
    tb.load_training_data(*host(scenes[0]))
    tb.set_params(S.init_params(L.grid_n_params(tb.config.grid), seed=1337))
    tb.train(600)

    def second_frame(gm_lr):
        t = Testbed(gm_learning_rate=gm_lr, **kw)
        t.load_training_data(*host(scenes[0]))
        t.set_params(tb.get_params())
        SN.set_array(t, "density_grid", SN.get_array(tb, "density_grid"))
        t.next_frame(*host(scenes[1]))
        return t
    tg = second_frame(1e-6)
    sign = np.zeros(12)
    for _ in range(20):
        before = tg.movement()[3].astype(np.float64)
        tg.train(1)
        sign += np.sign(tg.movement()[3].astype(np.float64) - before)
    sign /= 20
    tz = second_frame(0.0)
    tz.train(3)  # the frame's occupancy grid
    st0 = SN.get_training_state(tz)
    ident = np.array(ops.DELTA_IDENTITY, np.float32)

    def loss_at(delta, n=8):
        out = []
        for _ in range(n):  # the same step replayed: same rays, same samples
            L.check(L.lib().neus2b_testbed_set_training_state(tz._h, C.byref(st0)))
            tz.set_movement(1, np.eye(3), np.zeros(3), delta)
            out.append(tz.train(1).loss)
        return float(np.mean(out))
    checked = 0
    for k, eps in [(0, 0.004), (1, 0.004), (2, 0.004), (4, 0.01), (5, 0.01), (6, 0.01), (7, 0.01), (8, 0.01), (9, 0.01)]:
        dp, dm = ident.copy(), ident.copy()
        dp[k] += eps
        dm[k] -= eps
        slope = (loss_at(dp) - loss_at(dm)) / (2 * eps)
        print("parameter %d: slope %+.4e, mean sign of the update %+.2f" % (k, slope, sign[k]))
        if abs(slope) > 5e-3:
            checked += 1
            assert sign[k] * slope < 0 and abs(sign[k]) >= 0.8, (k, slope, sign[k])
    assert checked >= 2 and sign[3] == 0 and sign[10] == 0 and sign[11] == 0
    for t in (tb, tg, tz):
        t.close()


def test_sequence_without_motion_prediction_warm_starts_only(frames):
    """predict_global_movement off: a frame switch restarts the optimizer and the schedule, nothing moves the rays or samples."""
    from neus2_b200 import _lib as L
    from neus2_b200 import synthetic as S
    from neus2_b200.testbed import Testbed
    _, scenes = frames
    tb = Testbed(batch_size=1 << 14, after_learning_rate=1e-3)
    tb.load_training_data(*host(scenes[0]))
    tb.set_params(S.init_params(L.grid_n_params(tb.config.grid), seed=1337))
    tb.train(50)
    tb.next_frame(*host(scenes[1]))
    before = tb.get_params()
    st = tb.train(3)
    assert st.training_step == 3 and not np.array_equal(tb.get_params(), before)
    frame, R, t, d = tb.movement()
    assert frame == 1 and np.array_equal(R, np.eye(3)) and not t.any()
    tb.close()


def write_sequence(root, poses, n_views=8, res=96):
    """One transforms file (and its images) per frame, in the reference's dataset format."""
    import json
    from PIL import Image
    from neus2_b200 import loader
    from neus2_b200 import synthetic as S
    for f, (R, t, r) in enumerate(poses):
        sc = S.render_sphere_views(n_views, res, res, device="cuda", seed=1, rotation=R, translation=t, radius=r)
        px = sc["pixels"].cpu().numpy().view(np.uint32)
        frames = []
        for i in range(n_views):
            Image.fromarray(px[i].view(np.uint8).reshape(res, res, 4), "RGBA").save(root / f"f{f:03d}_{i:03d}.png")
            X = sc["xforms"][i].cpu().numpy()
            nerf = loader.ngp_matrix_to_nerf(np.stack([X[0:3], X[3:6], X[6:9], X[9:12]], 1), loader.NERF_SCALE, [0.5, 0.5, 0.5])
            frames.append({"file_path": f"f{f:03d}_{i:03d}", "transform_matrix": np.vstack([nerf, [0, 0, 0, 1]]).tolist()})
        fov = 2.0 * np.arctan(0.5 * res / float(sc["focal"][0, 0]))
        (root / f"frame_{f:03d}.json").write_text(json.dumps({"camera_angle_x": float(fov), "aabb_scale": 1, "frames": frames}))


def test_sequence_from_a_directory_through_frame_and_snapshot(tmp_path):
    """Testbed.frame() on a directory of per-frame transforms files: the first frame trains first_frame_max_training_step steps,
    every later one next_frame_max_training_step, and a snapshot taken mid-sequence restores the movement."""
    from neus2_b200 import _lib as L
    from neus2_b200 import synthetic as S
    from neus2_b200.testbed import Testbed
    poses = S.sequence_poses(3, seed=2)
    write_sequence(tmp_path, poses)
    (tmp_path / "frame_001_downsample.json").write_text("{}")  # ignored by the frame list
    kw = dict(batch_size=1 << 14, predict_global_movement=1, predict_global_movement_training_step=10, after_learning_rate=1e-3,
              reset_density_grid_after_global_movement=0)
    tb = Testbed(**kw)
    tb.first_frame_max_training_step, tb.next_frame_max_training_step = 60, 25
    tb.load_training_data_from_json(tmp_path)
    assert tb.all_training_time_frame == 3 and tb.current_training_time_frame == 0
    tb.set_params(S.init_params(L.grid_n_params(tb.config.grid), seed=1337))
    seen = []
    for _ in range(60 + 25 + 12):
        tb.frame()
        seen.append((tb.current_training_time_frame, tb.training_step))
    assert seen[59] == (0, 60) and seen[60] == (1, 1) and seen[84] == (1, 25) and seen[85] == (2, 1) and seen[-1] == (2, 12)
    frame, R_acc, t_acc, delta = tb.movement()
    assert frame == 2 and not np.array_equal(R_acc, np.eye(3)) and np.isfinite(tb.loss)
    tb.save_snapshot(tmp_path / "mid.msgpack")
    other = Testbed(**kw)
    other.load_training_data_from_json(tmp_path / "frame_002.json")
    other.load_snapshot(tmp_path / "mid.msgpack")
    f2, R2, t2, d2 = other.movement()
    assert f2 == 2 and np.array_equal(R2, R_acc) and np.array_equal(t2, t_acc) and np.array_equal(d2, delta)
    st = other.train(3)
    assert st.training_step == 15 and np.isfinite(st.loss)
    assert not tb.training_network_next_frame(), "no frame behind the last one"
    tb.close()
    other.close()
