"""The step's network pass in windows of consecutive samples per ray (neus2b_forward_compute_loss): it must leave exactly what
the reference's order leaves -- every sample evaluated, then the loss pass -- while evaluating fewer samples."""
import numpy as np
import pytest
import torch

from test_gpu_raymarch import ball_bitfield, half, scene, sphere_model

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gpu():
    from neus2_b200 import _lib as L
    from neus2_b200 import ops
    L.lib()
    return L, ops


@pytest.mark.parametrize("windows", [(16, 64), (32, 96), (8,), (1, 2, 3, 5, 40, 300), (64, 128, 256), (4096,)])
@pytest.mark.parametrize("variance,target", [(0.8, 1 << 20), (0.5, 1 << 20), (0.3, 1 << 14)])
def test_windowed_pass_equals_the_full_pass(gpu, oracle, windows, variance, target):
    L, ops = gpu
    O = oracle
    _, gds = scene(O, ops)
    _, bf, _ = ball_bitfield(O)
    bf_gpu = torch.from_numpy(bf).cuda()
    d, params = sphere_model(O, variance)
    ld = L.GridDesc(d.n_levels, d.log2_hashmap_size, d.base_resolution, d.per_level_scale, d.n_active_levels)
    P = half(params)
    n_rays, max_samples = 8192, 1 << 20
    cfg = L.train_cfg()
    rng = L.pcg32(99)
    results = []
    for w in ((), windows):
        batch = ops.RayBatch(n_rays, max_samples)
        ops.generate_samples(gds, cfg, n_rays, 777, rng, bf_gpu, batch)
        mlp_out = torch.full((max_samples, 16), float("nan"), dtype=torch.float16, device="cuda")  # unevaluated rows must never be read
        coords_out = torch.zeros((target, 7), dtype=torch.float32, device="cuda")
        dloss = torch.zeros((target, 16), dtype=torch.float16, device="cuda")
        loss, ek = torch.zeros(n_rays, device="cuda"), torch.zeros(n_rays, device="cuda")
        ops.forward_compute_loss(ld, P, gds, cfg, n_rays, 777, rng, target, batch, mlp_out, coords_out, dloss, loss, ek, window_ends=w, rollover=True)
        torch.cuda.synchronize()
        cnt = batch.counters.cpu().numpy().view(np.uint32).copy()
        results.append(dict(cnt=cnt, numsteps=batch.numsteps.cpu().numpy().copy(), coords=coords_out.cpu().numpy().view(np.uint32),
                            dloss=dloss.cpu().view(torch.int16).numpy(), loss=loss.cpu().numpy().view(np.uint32), ek=ek.cpu().numpy().view(np.uint32)))
    full, win = results
    k = int(full["cnt"][0])
    assert k > 0 and win["cnt"][0] == k and win["cnt"][1] == full["cnt"][1]
    assert win["cnt"][2] == full["cnt"][2], "compacted sample count"
    assert np.array_equal(win["numsteps"][:k], full["numsteps"][:k]), "per-ray compacted {count, base}"
    assert np.array_equal(win["coords"], full["coords"]), "compacted coordinates (rolled over to the target batch)"
    if all(w % 32 == 0 for w in windows):
        # window ends on multiples of 32 keep the grouping of the sums along a ray (32 samples per warp step): bit for bit
        assert np.array_equal(win["dloss"], full["dloss"]), "loss gradient bit for bit"
        assert np.array_equal(win["loss"][:k], full["loss"][:k]) and np.array_equal(win["ek"][:k], full["ek"][:k])
    else:
        # other ends regroup the fp32 sums of a ray's colour: last-bit differences in the composited colour and what follows from it
        a, b = win["dloss"].view(np.float16).astype(np.float32), full["dloss"].view(np.float16).astype(np.float32)
        assert np.allclose(a, b, rtol=4e-3, atol=1e-6) and (a == b).mean() > 0.97
        assert np.allclose(win["loss"][:k].view(np.float32), full["loss"][:k].view(np.float32), rtol=1e-4, atol=1e-12)
        assert np.allclose(win["ek"][:k].view(np.float32), full["ek"][:k].view(np.float32), rtol=1e-4, atol=1e-12)
    evaluated, drawn = int(win["cnt"][5]), int(full["cnt"][1])
    assert evaluated <= drawn
    if max(windows) >= 4096:
        assert evaluated == drawn  # one window that covers every ray: the same work as the full pass
    # (this untrained model never turns a ray opaque: what the windows save is shown on a trained one below)


def test_windows_on_a_trained_model(gpu):
    """On a trained model rays turn opaque in front of their last samples: the windowed pass evaluates far fewer samples and still
    leaves the full pass's compacted batch and loss gradient.  The model comes from a testbed; one step's ray pass is replayed by hand."""
    L, ops = gpu
    from neus2_b200 import synthetic as S
    from neus2_b200.parallel import device_view
    from neus2_b200.testbed import Testbed
    sc = S.render_sphere_views(24, 256, 256, device="cuda", seed=2)
    tb = Testbed(batch_size=1 << 16, ek_loss_weight=0.01)
    tb.load_training_data(sc["pixels"].cpu().numpy(), *[sc[k].cpu().numpy() for k in ("xforms", "focal", "principal")])
    ng = L.grid_n_params(tb.config.grid)
    tb.set_params(S.init_params(ng, seed=1337))
    st = tb.train(700)
    assert st.n_samples_evaluated < 0.8 * st.measured_batch_size_before_compaction, "the training loop's own pass saves evaluations too"
    assert st.n_samples_evaluated >= st.measured_batch_size * 0.9
    ptr = tb.device_ptrs()
    P = device_view(ptr["params"], (12288 + ng + 4) * 2, torch.float16)
    bf = device_view(ptr["bitfield"], 128 ** 3, torch.uint8)
    gds = ops.make_dataset(sc["pixels"], sc["xforms"], sc["focal"], sc["principal"])
    cfg, n_rays, max_samples, target = L.train_cfg(ek_loss_weight=0.01), 6000, 1 << 20, 1 << 19
    out = {}
    for w in ((), (32, 96), (16, 64)):
        batch = ops.RayBatch(n_rays, max_samples)
        ops.generate_samples(gds, cfg, n_rays, 4242, L.pcg32(11), bf, batch)
        mlp_out = torch.full((max_samples, 16), float("nan"), dtype=torch.float16, device="cuda")
        coords_out = torch.zeros((target, 7), dtype=torch.float32, device="cuda")
        dloss = torch.zeros((target, 16), dtype=torch.float16, device="cuda")
        loss, ek = torch.zeros(n_rays, device="cuda"), torch.zeros(n_rays, device="cuda")
        ops.forward_compute_loss(tb.config.grid, P, gds, cfg, n_rays, 4242, L.pcg32(11), target, batch, mlp_out, coords_out, dloss, loss, ek, window_ends=w,
                                 rollover=False)
        torch.cuda.synchronize()
        cnt = batch.counters.cpu().numpy().view(np.uint32).copy()
        k = int(cnt[0])
        out[w] = dict(cnt=cnt, numsteps=batch.numsteps.cpu().numpy()[:k].copy(), coords=coords_out.cpu().numpy().view(np.uint32),
                      dloss=dloss.cpu().view(torch.int16).numpy(), loss=loss.cpu().numpy()[:k].copy())
    full = out[()]
    drawn, kept = int(full["cnt"][1]), int(full["cnt"][2])
    assert 0 < kept < 0.7 * drawn and kept <= target, "the scene must have rays that turn opaque"
    for w in ((32, 96), (16, 64)):
        r = out[w]
        assert r["cnt"][2] == kept and np.array_equal(r["numsteps"], full["numsteps"]) and np.array_equal(r["coords"], full["coords"])
        assert kept <= int(r["cnt"][5]) < 0.85 * drawn, "evaluated samples: at least the kept ones, clearly fewer than all"
        assert np.isfinite(r["dloss"].view(np.float16).astype(np.float32)).all() and np.isfinite(r["loss"]).all()  # no unevaluated row was read
    assert np.array_equal(out[(32, 96)]["dloss"], full["dloss"]) and np.array_equal(out[(32, 96)]["loss"], full["loss"])
    a, b = out[(16, 64)]["dloss"].view(np.float16).astype(np.float32), full["dloss"].view(np.float16).astype(np.float32)
    assert np.allclose(a, b, rtol=4e-3, atol=1e-6) and (a == b).mean() > 0.97
    tb.close()


def test_training_with_and_without_windows_agrees(gpu):
    """Same testbed, same seeds: the first steps' statistics are those of the full pass (later steps drift apart only through the
    order of the gradient reductions, which is not fixed in either mode)."""
    from neus2_b200 import synthetic as S
    from test_gpu_testbed import make_testbed
    sc = S.render_sphere_views(12, 128, 128, device="cpu", seed=1)
    stats = []
    for w in ((), (16, 64)):
        tb, _, _ = make_testbed(sc, 1 << 14, forward_windows=w)
        st = tb.train(1)
        first = (st.loss, st.ek_loss, st.measured_batch_size, st.measured_batch_size_before_compaction, st.n_rays_kept)
        st = tb.train(60)
        stats.append((first, st.loss, st.measured_batch_size))
        tb.close()
    assert stats[0][0] == stats[1][0], "the first step is identical"
    assert stats[0][1] < 5e-3 and stats[1][1] < 5e-3  # both runs train (the loss starts near 3e-2)
