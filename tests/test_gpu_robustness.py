"""GPU tests of the guards around the training step: the optimizer's switches and its refusal of non-finite gradients, the
sticky device error word reaching the host through the step statistics, and state changes that must discard samples drawn
ahead.  Nothing here makes a kernel fault, trap or hang: error states are written by the host."""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def adam_reference(cfg, g, w, m, v, flags, n_matrix):
    """numpy restatement of the optimizer pass with its switches (fp32 like the kernel)."""
    f = np.float32
    w, m, v = w.copy(), m.copy(), v.copy()
    lr_t = f(cfg["lr"]) * np.sqrt(f(1) - f(cfg["b2"]) ** f(cfg["step"])) / (f(1) - f(cfg["b1"]) ** f(cfg["step"]))
    bad = ~np.isfinite(g)
    gs = np.where(bad, f(0), g) / f(cfg["ls"])
    is_matrix = np.arange(g.size) < n_matrix
    upd = ~bad & (is_matrix | (gs != 0) | bool(flags & 1))
    decay = is_matrix | bool(flags & 2)
    gs = gs + np.where(decay, f(cfg["l2"]) * w, f(0))
    m2 = f(cfg["b1"]) * m + (f(1) - f(cfg["b1"])) * gs
    v2 = f(cfg["b2"]) * v + (f(1) - f(cfg["b2"])) * gs * gs
    w2 = w - lr_t * m2 / (np.sqrt(v2) + f(cfg["eps"]))
    return np.where(upd, w2, w).astype(f), np.where(upd, m2, m).astype(f), np.where(upd, v2, v).astype(f), int(bad.sum())


@pytest.mark.parametrize("flags", [0, 1, 2, 3, 4])
def test_adam_switches_and_nonfinite_gradients(flags):
    from neus2_b200 import _lib as L
    from neus2_b200 import ops
    rng = np.random.default_rng(5)
    n_matrix, n_grid = 256, 4096
    n = n_matrix + n_grid + 4
    w = rng.normal(0, 0.1, n).astype(np.float32)
    m = rng.normal(0, 1e-3, n).astype(np.float32)
    v = (rng.random(n) * 1e-5).astype(np.float32)
    g = (rng.normal(0, 1, n) * 128).astype(np.float32)
    g[n_matrix:n_matrix + n_grid] = g[n_matrix:n_matrix + n_grid].astype(np.float16).astype(np.float32)
    g[n_matrix:n_matrix + n_grid][rng.random(n_grid) < 0.5] = 0.0
    # what an overflowed fp16 sum or a poisoned exchange buffer looks like
    g[3], g[n_matrix + 10], g[n_matrix + 11], g[n - 4] = np.inf, np.nan, -np.inf, np.nan
    cfg = dict(lr=1e-2, b1=0.9, b2=0.99, eps=1e-15, l2=1e-3, ls=128.0, step=3)
    t = lambda a: torch.from_numpy(a.copy()).cuda()
    gm, gg, gv = t(g[:n_matrix]), t(g[n_matrix:n_matrix + n_grid].astype(np.float16)), t(g[n_matrix + n_grid:])
    W, M, V, E = t(w), t(m), t(v), t(w)
    P = torch.zeros(n, dtype=torch.float16, device="cuda")
    Pe = torch.zeros(n, dtype=torch.float16, device="cuda")
    count = torch.zeros(1, dtype=torch.int32, device="cuda")
    gc = L.AdamCfg(cfg["lr"], cfg["b1"], cfg["b2"], cfg["eps"], cfg["l2"], 0.95, cfg["ls"], cfg["step"], n_matrix, flags, count.data_ptr())
    ops.adam_step(gc, gm, gg, gv, W, M, V, P, Pe, E)
    torch.cuda.synchronize()
    rw, rm, rv, nbad = adam_reference(cfg, g, w, m, v, flags, n_matrix)
    assert int(count.item()) == nbad == 4
    assert np.isfinite(W.cpu().numpy()).all()
    assert np.allclose(W.cpu().numpy(), rw, rtol=2e-5, atol=1e-7)
    assert np.allclose(M.cpu().numpy(), rm, rtol=2e-5, atol=1e-9)
    assert np.allclose(V.cpu().numpy(), rv, rtol=2e-5, atol=1e-12)
    for i in (3, n_matrix + 10, n_matrix + 11, n - 4):  # refused entries: weight and moments untouched, slot cleared
        assert W[i].item() == w[i] and M[i].item() == m[i] and V[i].item() == v[i]
    assert gm.abs().max().item() == 0 and gg.float().abs().max().item() == 0 and gv.abs().max().item() == 0
    # EMA of the new weights: bias-corrected by default, plain with NEUS2B_ADAM_EMA_NO_DEBIAS
    d = np.float32(0.95)
    if flags & 4:
        want = d * w + (1 - d) * rw
    else:
        want = ((1 - d) * rw + d * w * (1 - d ** np.float32(cfg["step"] - 1))) / (1 - d ** np.float32(cfg["step"]))
    assert np.allclose(E.cpu().numpy(), want, rtol=2e-5, atol=1e-7)


@pytest.fixture(scope="module")
def scene():
    from neus2_b200 import synthetic as S
    return S.render_sphere_views(12, 128, 128, device="cpu", seed=1)


def test_device_error_word_reaches_the_step_statistics(scene):
    """A kernel whose bounded wait ran out sets a sticky word; the training loop copies it next to the step statistics and
    the statistics call returns an error instead of numbers computed from garbage.  The word is set by the host here."""
    from neus2_b200 import _lib as L
    from test_gpu_testbed import make_testbed
    tb, _, _ = make_testbed(scene, 1 << 14)
    try:
        st = tb.train(2)
        assert st.device_error == 0 and st.nonfinite_gradients == 0
        L.set_device_error_flags(1)
        assert L.device_error_flags() == 1
        with pytest.raises(L.Neus2bError, match="-7"):
            tb.train(1)
        assert tb.stats.device_error == 1
        with pytest.raises(L.Neus2bError, match="-7"):
            tb.render(16, 16)
        with pytest.raises(L.Neus2bError, match="-7"):
            tb.sdf_grid(8)
    finally:
        L.set_device_error_flags(0)
    st = tb.train(1)
    assert st.device_error == 0 and np.isfinite(st.loss)
    tb.close()


def test_nonfinite_gradient_is_counted_and_does_not_reach_the_weights(scene):
    from neus2_b200 import _lib as L
    from neus2_b200.parallel import device_view
    from test_gpu_testbed import make_testbed
    tb, _, ng = make_testbed(scene, 1 << 14)
    tb.train(3)
    tb.train_backward()
    p = tb.device_ptrs()
    torch.cuda.synchronize()
    gg = device_view(p["grad_grid"], ng * 2, torch.float16)
    gm = device_view(p["grad_mlp"], 12288 * 4, torch.float32)
    gg[:5] = float("inf")  # e.g. an fp16 sum over ranks that overflowed
    gm[7] = float("nan")
    torch.cuda.synchronize()
    st = tb.optimizer_step()
    assert st.nonfinite_gradients == 6
    assert np.isfinite(tb.get_params()).all() and np.isfinite(tb.get_params(ema=True)).all()
    st = tb.train(2)
    assert st.nonfinite_gradients == 6 and np.isfinite(st.loss)
    tb.close()


def test_new_density_grid_discards_samples_drawn_ahead(scene):
    """neus2b_testbed_train_step draws the next step's samples before it returns; a density grid written afterwards (a
    snapshot being loaded) must win over them."""
    from neus2_b200 import snapshot as SN
    from test_gpu_testbed import make_testbed
    tb, _, _ = make_testbed(scene, 1 << 14)
    for _ in range(35):  # past step 32 the occupancy update runs every other step or less often
        st = tb.train_step()
    while (st.training_step % max(1, min(16, st.training_step // 16))) == 0:  # the next step must not begin with an occupancy update
        st = tb.train_step()
    assert st.measured_batch_size_before_compaction > 0
    SN.set_array(tb, "density_grid", np.zeros(128 ** 3, np.float32))  # nothing occupied any more
    st = tb.train_step()
    assert st.measured_batch_size_before_compaction == 0 and st.n_rays_kept == 0
    tb.close()


def test_parameter_only_snapshot_resets_the_optimizer_of_a_trained_testbed(scene, tmp_path):
    from neus2_b200 import snapshot as SN
    from test_gpu_testbed import make_testbed
    a, _, _ = make_testbed(scene, 1 << 14)
    a.train(5)
    a.save_snapshot(tmp_path / "small.msgpack", include_optimizer_state=False)
    b, _, _ = make_testbed(scene, 1 << 14)
    b.train(7)
    assert SN.get_array(b, "adam_m").any() and SN.get_array(b, "adam_v").any()
    b.load_snapshot(tmp_path / "small.msgpack")
    assert not SN.get_array(b, "adam_m").any() and not SN.get_array(b, "adam_v").any()
    assert b.train(1).training_step == 6
    a.close()
    b.close()
