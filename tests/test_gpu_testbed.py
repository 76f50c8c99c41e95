"""GPU tests of the training loop (the reference's Testbed::train path) through the C ABI:
one full step against the oracle's composition of the same stages, and convergence on the analytic sphere."""
import numpy as np
import pytest
import torch

from util import check_grad, cosine, record

pytestmark = pytest.mark.gpu


def cuda_view(ptr, nbytes):
    class _V:
        pass
    v = _V()
    v.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}
    return torch.as_tensor(v, device="cuda")


@pytest.fixture(scope="module")
def scene():
    from neus2_b200 import synthetic as S
    return S.render_sphere_views(12, 128, 128, device="cpu", seed=1)


def make_testbed(scene, batch, **kw):
    from neus2_b200 import _lib as L
    from neus2_b200 import synthetic as S
    from neus2_b200.testbed import Testbed
    tb = Testbed(batch_size=batch, **kw)
    tb.load_training_data(scene["pixels"].numpy(), scene["xforms"].numpy(), scene["focal"].numpy(), scene["principal"].numpy())
    ng = L.grid_n_params(tb.config.grid)
    p0 = S.init_params(ng, seed=1337)
    rng = np.random.default_rng(2)
    p0[12288:12288 + ng] = rng.uniform(-1e-2, 1e-2, ng)
    # the geometric init has zero weights on the encoding columns, which makes every grid gradient exactly zero at step 0
    p0[:3072].reshape(64, 48)[:, 3:35] = rng.normal(0, 0.05, (64, 32))
    tb.set_params(p0)
    return tb, p0, ng


def test_first_step_matches_oracle_composition(scene, oracle):
    O = oracle
    target = 1 << 14
    tb, p0, ng = make_testbed(scene, target)
    ptrs = tb.device_ptrs()
    tb.train_backward()
    torch.cuda.synchronize()
    bits_gpu = cuda_view(ptrs["bitfield"], 128 ** 3).cpu().numpy()
    grid_gpu = cuda_view(ptrs["density_grid"], 128 ** 3 * 4).view(torch.float32).cpu().numpy()
    gm = cuda_view(ptrs["grad_mlp"], 12288 * 4).view(torch.float32).cpu().numpy().copy()
    gg = cuda_view(ptrs["grad_grid"], ng * 2).view(torch.float16).float().cpu().numpy().copy()
    gv = cuda_view(ptrs["grad_variance"], 16).view(torch.float32).cpu().numpy().copy()
    # ---- the same step composed from the oracle's stages (rng streams as in reset_network, src/testbed.cu:2077-2091)
    d = O.grid_desc()
    params = O.f16_bits(p0)
    m_rng = O.pcg32(1337)
    dens_rng = O.pcg32(O.pcg32_next_uint(m_rng))
    O.pcg32_next_uint(m_rng)
    n_occ = 128 ** 3
    pos, idx = O.occ_generate_samples(n_occ, dens_rng, 0, np.zeros(n_occ, np.float32), 1, -0.01)
    dens = O.sdf_to_density(O.neus_sdf(d, params, pos), params[O.GRID_OFF + ng])
    grid = O.occ_splat_ema(idx, dens, np.zeros(n_occ, np.float32), 0.95)
    ref_bits, _ = O.occ_bitfield(grid, 1)
    grid_close = np.isclose(grid_gpu, grid, rtol=2e-3, atol=1e-6).mean()
    bit_mismatch = np.unpackbits(bits_gpu ^ ref_bits).mean()
    record("testbed_occupancy_step0", grid_close=float(grid_close), bit_mismatch=float(bit_mismatch))
    assert grid_close > 0.999 and bit_mismatch < 1e-4
    ods = O.make_dataset(scene["pixels"].numpy().view(np.uint32), scene["xforms"].numpy(), scene["focal"].numpy(),
                         scene["principal"].numpy())
    cfg = O.train_cfg(ek_loss_weight=0.1, snap_to_pixel_centers=True)  # the training loop's default (testbed.h:614)
    gen = O.generate_samples(ods, cfg, 4096, 0, target * 16, m_rng, bits_gpu)
    used = int(gen["numsteps"][gen["n_kept"] - 1].sum())
    out = O.neus_forward(d, params, gen["coords"][:used])
    los = O.compute_loss(ods, cfg, gen, 4096, 0, m_rng, target, out)
    nv = min(los["n_compacted"], target)
    coords = O.fill_rollover(los["coords"], nv)
    dloss = O.fill_rollover_and_rescale_half(los["dloss"], nv)
    ref = O.neus_backward(d, params, coords, dloss, indeed_batch_size=target)
    check_grad("testbed_step_grad_mlp", gm, ref[:12288], min_cos=0.995)
    check_grad("testbed_step_grad_grid", gg, ref[O.GRID_OFF:O.GRID_OFF + ng], min_cos=0.995)
    vref = ref[O.GRID_OFF + ng]
    assert abs(gv[0] - vref) <= 2e-2 * abs(vref) + 1e-3
    # ---- optimizer half: Adam from the GPU's gradients must match the oracle's Adam bit-for-bit-ish
    st = tb.optimizer_step()
    assert st.training_step == 1 and st.n_rays_kept == gen["n_kept"]
    assert st.measured_batch_size_before_compaction == gen["n_samples"]
    assert abs(int(st.measured_batch_size) - los["n_compacted"]) <= max(2, los["n_compacted"] // 500)
    assert abs(st.loss - los["loss"].sum() * st.measured_batch_size / target) <= 2e-2 * abs(st.loss) + 1e-6
    grad_all = np.concatenate([gm, gg, gv]).astype(np.float32)
    master, m, v = p0.copy(), np.zeros_like(p0), np.zeros_like(p0)
    pp, pe, em = np.zeros(p0.size, np.uint16), np.zeros(p0.size, np.uint16), p0.copy()
    O.adam_step(O.AdamCfg(1e-2, 0.9, 0.99, 1e-15, 1e-6, 0.95, 128.0, 1, 12288), grad_all, master, m, v, pp, pe, em)
    got = tb.get_params()
    assert np.allclose(got, master, rtol=1e-5, atol=1e-7)
    assert np.allclose(tb.get_params(ema=True), em, rtol=1e-5, atol=1e-7)
    # rays-per-batch re-tune (Counters::update_after_training, src/testbed_nerf.cu:3427-3429)
    want = min((int(np.float32(4096) * np.float32(target) / np.float32(st.measured_batch_size)) + 127) // 128 * 128, 1 << 18)
    assert st.rays_per_batch == max(want, 128)
    tb.close()


def test_training_converges_to_the_sphere(scene):
    tb, p0, ng = make_testbed(scene, 1 << 16)
    first = tb.train(1).loss
    hist = []
    for k in range(12):
        st = tb.train(50)
        hist.append((st.training_step, st.loss, st.ek_loss, st.rays_per_batch, st.measured_batch_size))
    record("testbed_convergence", first_loss=first, history=[list(map(float, h)) for h in hist])
    assert st.overflow == 0
    assert hist[-1][1] < 0.5 * first, hist
    # surface of the learned SDF: zero crossing along rays from the centre should sit at radius 0.3
    res = 96
    sdf = tb.sdf_grid(res, use_ema=False).cpu().numpy()
    zz, yy, xx = np.meshgrid(np.arange(res), np.arange(res), np.arange(res), indexing="ij")
    r = np.sqrt((xx / res - 0.5) ** 2 + (yy / res - 0.5) ** 2 + (zz / res - 0.5) ** 2)
    inside = sdf < 0
    assert inside.any() and (~inside).any()
    r_in, r_out = r[inside].max(), r[~inside].min()
    vol_radius = (inside.mean() * 3 / (4 * np.pi)) ** (1 / 3)
    record("testbed_sphere", r_in_max=float(r_in), r_out_min=float(r_out), volume_radius=float(vol_radius))
    assert abs(vol_radius - 0.3) < 0.03, (vol_radius, r_in, r_out)
    tb.close()
