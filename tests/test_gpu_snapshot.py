"""Snapshots through the C ABI's state entry points: what is saved comes back bit for bit, a loaded testbed renders the
same image and trains on, files of another architecture are refused."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def make(batch=1 << 16, **kw):
    from neus2_b200 import _lib as L
    from neus2_b200 import synthetic as S
    from neus2_b200.testbed import Testbed
    sc = S.render_sphere_views(12, 128, 128, device="cpu", seed=0)
    tb = Testbed(batch_size=batch, **kw)
    tb.load_training_data(sc["pixels"].numpy(), sc["xforms"].numpy(), sc["focal"].numpy(), sc["principal"].numpy())
    tb.set_params(S.init_params(L.grid_n_params(tb.config.grid), seed=1337))
    X = sc["xforms"][4].numpy()
    tb.camera_matrix = np.stack([X[0:3], X[3:6], X[6:9], X[9:12]], 1)
    tb.fov = 40.0
    tb.snap_to_pixel_centers = True
    return tb


@pytest.fixture(scope="module")
def trained_pair(tmp_path_factory):
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    d = tmp_path_factory.mktemp("snap")
    a = make()
    a.train(300)
    a.save_snapshot(d / "full.msgpack", include_optimizer_state=True)
    a.save_snapshot(d / "small.msgpack")
    yield a, d
    a.close()


def test_full_snapshot_round_trip(trained_pair):
    from neus2_b200 import snapshot as SN
    a, d = trained_pair
    b = make()
    doc = b.load_snapshot(d / "full.msgpack")
    assert doc["encoding"]["n_levels"] == 16 and doc["snapshot"]["density_grid_size"] == 128
    for name in ("master", "adam_m", "adam_v", "ema_master", "params", "params_ema"):
        x, y = SN.get_array(a, name), SN.get_array(b, name)
        assert np.array_equal(x.view(np.uint8), y.view(np.uint8)), name
    ga, gb = SN.get_array(a, "density_grid"), SN.get_array(b, "density_grid")
    np.testing.assert_array_equal(ga.astype(np.float16).astype(np.float32), gb)
    sa, sb = SN.get_training_state(a), SN.get_training_state(b)
    for f, _ in sa._fields_:
        if f in ("rng", "density_rng"):
            assert (getattr(sa, f).state, getattr(sa, f).inc) == (getattr(sb, f).state, getattr(sb, f).inc)
        else:
            assert getattr(sa, f) == getattr(sb, f), f
    assert b.training_step == 300
    # the same picture (the occupancy bits come from the fp16 copy of the grid: a cell at the threshold may flip)
    ia, ib = a.render(96, 96, linear=False), b.render(96, 96, linear=False)
    assert (ia[..., 3] > 0.5).mean() > 0.05
    assert np.abs(ia - ib).mean() < 1e-3
    # both keep training from the same state
    la = a.train(40).loss
    lb = b.train(40).loss
    assert b.training_step == 340 and np.isfinite(lb) and lb < 3 * la + 1e-4 and la < 3 * lb + 1e-4
    b.close()


def test_parameter_only_snapshot(trained_pair):
    from neus2_b200 import snapshot as SN
    a, d = trained_pair
    import msgpack
    doc = msgpack.unpackb((d / "small.msgpack").read_bytes(), raw=False)
    snap = doc["snapshot"]
    assert "optimizer" not in snap and snap["params_type"] == "__half" and len(snap["params_binary"]) == 2 * snap["n_params"]
    assert set(snap["nerf"]["rgb"]) == {"rays_per_batch", "measured_batch_size", "measured_batch_size_before_compaction"}
    assert (d / "small.msgpack").stat().st_size < (d / "full.msgpack").stat().st_size / 4
    b = make()
    b.load_snapshot(d / "small.msgpack")
    saved = np.frombuffer(snap["params_binary"], np.uint16)
    # the stored inference weights become every copy of the weights (Trainer::deserialize)
    for name in ("params", "params_ema"):
        np.testing.assert_array_equal(SN.get_array(b, name), saved)
    np.testing.assert_array_equal(SN.get_array(b, "master"), saved.view(np.float16).astype(np.float32))
    assert not SN.get_array(b, "adam_m").any()
    img = b.render(64, 64)
    assert (img[..., 3] > 0.5).mean() > 0.05
    st = b.train(20)
    assert st.training_step == snap["training_step"] + 20 and np.isfinite(st.loss)
    b.close()


def test_refuses_other_architectures_and_files(trained_pair, tmp_path):
    import msgpack
    a, d = trained_pair
    small = make(n_levels=8)
    with pytest.raises(ValueError):
        small.load_snapshot(d / "full.msgpack")
    small.close()
    (tmp_path / "nosnap.msgpack").write_bytes(msgpack.packb({"encoding": {}}))
    b = make()
    with pytest.raises(ValueError, match="does not contain a snapshot"):
        b.load_snapshot(tmp_path / "nosnap.msgpack")
    b.close()


def test_pregenerated_samples_equal_the_plain_sequence(tmp_path):
    """Drawing the next step's samples between backward and optimizer pass (what data-parallel training overlaps with the
    gradient exchange) leaves the step unchanged: from one saved state, the plain and the reordered sequence generate the
    same rays and samples."""
    a = make()
    a.train(42)
    a.save_snapshot(tmp_path / "s.msgpack", include_optimizer_state=True)
    a.close()

    def run(reordered):
        tb = make()
        tb.load_snapshot(tmp_path / "s.msgpack")
        drew = []
        for _ in range(3):  # steps 42, 43, 44: step 44 starts with an occupancy update, 43 does not
            tb.train_backward()
            if reordered == "between":
                drew.append(tb.train_pregenerate())
                st = tb.optimizer_step()
            elif reordered == "after":  # optimizer pass enqueued, next samples drawn, only then the host waits for the statistics
                tb.optimizer_step_async()
                drew.append(tb.train_pregenerate())
                st = tb.wait_stats()
            else:
                st = tb.optimizer_step()
            out = (st.training_step, st.rays_per_batch, st.n_rays_kept, st.measured_batch_size_before_compaction,
                   st.measured_batch_size, st.loss)
            if st.training_step == 44:
                keep = out
        tb.close()
        return keep, drew
    plain, _ = run(None)
    for mode in ("between", "after"):
        ahead, drew = run(mode)
        assert drew == [True, False, True]
        # ray count, kept rays and generated samples of step 43 do not depend on the (non-deterministic) gradient sums
        assert plain[:4] == ahead[:4], mode
        assert abs(plain[4] - ahead[4]) <= 0.01 * plain[4] and abs(plain[5] - ahead[5]) <= 0.2 * plain[5]
    # a camera update discards samples drawn ahead
    tb = make()
    tb.load_snapshot(tmp_path / "s.msgpack")
    tb.train_backward()
    assert tb.train_pregenerate()
    tb.update_cameras()
    st = tb.optimizer_step()
    tb.train_backward()
    st2 = tb.optimizer_step()
    assert st2.training_step == 44 and (st2.rays_per_batch, st2.n_rays_kept, st2.measured_batch_size_before_compaction) == plain[1:4]
    tb.close()
