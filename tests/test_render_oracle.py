"""CPU checks of the renderer's oracle and host logic: the low-discrepancy jitter (three independent statements agree), the
march of a frame against the round-based frame, compositing of a known scene, accumulate / tone mapping identities."""
import ctypes as C

import numpy as np
import pytest

from test_gpu_raymarch import ball_bitfield, sphere_model


def test_ld_random_val_statements_agree(oracle):
    from neus2_b200 import ops
    O = oracle
    for index, seed in ((0, 0), (1, 0), (5, 12345), (123456, 0xdeadbeef), (2 ** 31 + 7, 99)):
        assert np.float32(O.ld_random_val(index, seed)) == ops.ld_random_val_2d(index, seed)[0]
    vals = np.array([O.ld_random_val(i, 4242) for i in range(4096)])
    assert vals.min() >= 0.0 and vals.max() < 1.0
    # a (0, m, 1)-net in base 2 keeps its stratification under Owen scrambling: one point per interval of length 1/4096
    assert len(np.unique(np.floor(vals * 4096))) == 4096


def test_pixel_offset_host_functions_agree():
    from neus2_b200 import _lib as L
    from neus2_b200 import ops
    for spp in (0, 1, 2, 3, 17, 1000):
        o = (C.c_float * 2)()
        L.lib().neus2b_ld_random_pixel_offset(C.c_uint32(spp), o)
        assert list(o) == ops.ld_random_pixel_offset(spp)
        assert 0.0 <= o[0] < 1.0 and 0.0 <= o[1] < 1.0
    assert ops.ld_random_pixel_offset(0) == [0.5, 0.5]
    pts = np.array([ops.ld_random_val_2d(i, 0xdeadbeef) for i in range(256)])
    # 2-D stratification of the scrambled (0, 2)-sequence: 16 x 16 cells, one point each
    cells = np.floor(pts * 16).astype(int)
    assert len({(a, b) for a, b in cells}) == 256


def make_cfg(O, w=48, h=36, **kw):
    from neus2_b200 import synthetic as S
    X = S.fibonacci_cameras(8, 2.5)[3]
    cam = np.stack([X[0:3], X[3:6], X[6:9], X[9:12]], 1)
    f = 0.5 * h / np.tan(0.5 * np.radians(40.0))
    return O.render_cfg(w, h, (f, f), cam, **kw)


def test_march_covers_the_rounds(oracle):
    O = oracle
    _, bf, _ = ball_bitfield(O)
    d, pb = sphere_model(O)
    cfg = make_cfg(O)
    numsteps, coords, n = O.render_march(cfg, bf)
    frame, depth, n_rounds = O.render_frame(d, pb, cfg, bf)
    assert 0 < n_rounds <= n == numsteps.sum() == coords.shape[0]
    hit = numsteps.reshape(36, 48) > 0
    # pixels whose ray never meets an occupied cell stay untouched
    assert not frame[~hit].any() and np.all(depth[~hit] == np.float32(1e10))
    assert (frame[..., 3] > 0.5).sum() >= 10
    assert frame[..., 3].max() <= 1.0 + 1e-6
    # all coordinates inside the unit cube, direction constant along a ray
    assert coords[:, :3].min() >= 0.0 and coords[:, :3].max() <= 1.0
    first = np.concatenate([[0], np.cumsum(numsteps.astype(np.int64))[:-1]]).astype(np.int64)
    i = int(np.argmax(numsteps))
    seg = coords[int(first[i]):int(first[i]) + int(numsteps[i])]
    assert np.all(seg[:, 4:] == seg[0, 4:]) and np.all(np.diff(seg[:, :3] @ (seg[0, 4:] * 2 - 1)) > 0)
    # the step budget cuts rays
    cut = O.render_march(make_cfg(O, max_steps=5), bf, want_coords=False)[0]
    np.testing.assert_array_equal(cut, np.minimum(numsteps, 5))


def test_jitter_moves_the_first_sample_only_by_less_than_a_step(oracle):
    O = oracle
    _, bf, _ = ball_bitfield(O)
    a = O.render_march(make_cfg(O, sample_index=0), bf)
    b = O.render_march(make_cfg(O, sample_index=1), bf)
    assert np.abs(a[0].astype(int) - b[0].astype(int)).max() <= 2
    assert a[2] != b[2] or not np.array_equal(a[1], b[1])


def test_accumulate_and_tonemap_identities(oracle):
    O = oracle
    rng = np.random.default_rng(1)
    frames = rng.uniform(0, 1, (4, 10, 4)).astype(np.float32)
    acc = np.full((10, 4), 9.0, np.float32)
    for s in range(4):
        O.render_accumulate(frames[s], acc, s)
    np.testing.assert_allclose(acc, frames.mean(0), rtol=1e-6)
    out = O.render_tonemap(acc, 0.0, (0, 0, 0, 0), to_srgb=False)
    np.testing.assert_array_equal(out, acc)
    out = O.render_tonemap(acc, 1.0, (0, 0, 0, 0), to_srgb=False)
    np.testing.assert_allclose(out[:, :3], acc[:, :3] * 2, rtol=1e-6)
    white = O.render_tonemap(np.zeros((3, 4), np.float32), 0.0, (1, 1, 1, 1), to_srgb=True)
    np.testing.assert_allclose(white, 1.0, rtol=1e-5)


def test_snapshot_network_config_uses_reference_keys():
    import ctypes as C
    from neus2_b200 import _lib as L
    from neus2_b200 import snapshot as SN
    cfg = L.TestbedConfig()
    L.lib().neus2b_testbed_default_config(C.byref(cfg))
    doc = SN.network_config(cfg)
    assert doc["encoding"]["otype"] == "HashGrid" and doc["encoding"]["n_levels"] == 16 and doc["encoding"]["log2_hashmap_size"] == 19
    opt = doc["optimizer"]
    assert opt["otype"] == "Ema" and opt["nested"]["otype"] == "ExponentialDecay" and opt["nested"]["nested"]["otype"] == "Adam"
    assert abs(opt["nested"]["nested"]["learning_rate"] - 1e-2) < 1e-9
