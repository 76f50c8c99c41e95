"""GPU parity of the ray-march side: sample generation (bit-exact), NeuS compositing / loss / compaction, roll-over,
occupancy grid (bit-exact bits on the same density grid) and the fused optimizer step, each through the C ABI against
the CPU oracle."""
import ctypes as C

import numpy as np
import pytest
import torch

from util import check_fp16, cosine, record

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gpu():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    from neus2_b200 import _lib as L
    from neus2_b200 import ops
    L.lib()
    return L, ops


def half(a_bits):
    return torch.from_numpy(np.ascontiguousarray(a_bits).view(np.int16)).cuda().view(torch.float16)


def bits(t):
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def ball_bitfield(O, radius=0.35):
    """Occupancy bits of a solid ball, built by the oracle from a Morton-ordered density grid."""
    idx = np.arange(128 ** 3, dtype=np.uint32)

    def inv(x):
        x = x & 0x49249249
        x = (x | (x >> 2)) & 0xc30c30c3
        x = (x | (x >> 4)) & 0x0f00f00f
        x = (x | (x >> 8)) & 0xff0000ff
        x = (x | (x >> 16)) & 0x0000ffff
        return x
    c = np.stack([inv(idx), inv(idx >> 1), inv(idx >> 2)], 1).astype(np.float32)
    p = (c + 0.5) / 128.0 - 0.5
    grid = (np.linalg.norm(p, axis=1) < radius).astype(np.float32)
    b, mean = O.occ_bitfield(grid, 1)
    return grid, b, mean


def scene(O, ops, n_views=8, res=96):
    from neus2_b200 import synthetic as S
    sc = S.render_sphere_views(n_views, res, res, device="cpu", seed=3)
    px = sc["pixels"].numpy().view(np.uint32)
    ods = O.make_dataset(px, sc["xforms"].numpy(), sc["focal"].numpy(), sc["principal"].numpy())
    gds = ops.make_dataset(sc["pixels"].cuda(), sc["xforms"].cuda(), sc["focal"].cuda(), sc["principal"].cuda())
    return ods, gds


def sphere_model(O, variance=0.5):
    from neus2_b200 import synthetic as S
    d = O.grid_desc()
    ng = O.grid_n_params(d)
    p = S.init_params(ng, seed=11, variance=variance)
    rng = np.random.default_rng(12)
    p[12288:12288 + ng] = rng.uniform(-2e-2, 2e-2, ng)
    return d, O.f16_bits(p)


@pytest.mark.parametrize("masks", [True, False])
@pytest.mark.parametrize("n_rays,max_samples,snap", [(8192, 1 << 20, False), (4096, 20000, True), (128, 1 << 16, False)])
def test_generate_samples_bit_exact(gpu, oracle, n_rays, max_samples, snap, masks):
    L, ops = gpu
    O = oracle
    ods, gds = scene(O, ops)
    _, bf, _ = ball_bitfield(O)
    ocfg, gcfg = O.train_cfg(snap_to_pixel_centers=snap), L.train_cfg(snap_to_pixel_centers=snap)
    ref = O.generate_samples(ods, ocfg, n_rays, 12345, max_samples, O.pcg32(1337), bf)
    bf_gpu = torch.from_numpy(bf).cuda()
    # with the march masks on, also cull the rays that miss the box of occupied cells: the result must not change
    bounds = ops.occupancy_bounds(bf_gpu) if masks else None
    batch = ops.RayBatch(n_rays, max_samples, march_masks=masks, occupied_bounds=bounds)
    ops.generate_samples(gds, gcfg, n_rays, 12345, L.pcg32(1337), bf_gpu, batch)
    torch.cuda.synchronize()
    cnt = batch.counters.cpu().numpy().view(np.uint32)
    k = ref["n_kept"]
    assert k > 0 and ref["n_samples"] > 0
    assert cnt[0] == k and cnt[1] == ref["n_samples"]
    assert np.array_equal(batch.ray_indices.cpu().numpy().view(np.uint32)[:k], ref["ray_indices"][:k])
    assert np.array_equal(batch.numsteps.cpu().numpy().view(np.uint32)[:k], ref["numsteps"][:k])
    assert np.array_equal(batch.rays.cpu().numpy()[:k].view(np.uint32), ref["rays"][:k].view(np.uint32))
    used = int(ref["numsteps"][k - 1].sum())
    assert cnt[4] == used
    assert np.array_equal(batch.coords.cpu().numpy()[:used].view(np.uint32), ref["coords"][:used].view(np.uint32)), \
        "sample coordinates must be bit-exact"
    if max_samples < ref["n_samples"]:
        assert cnt[3] == 1  # overflow flag: rays were dropped
    record("generate_samples_%d" % n_rays, kept=k, samples=ref["n_samples"])


def test_pcg32_matches_oracle(gpu, oracle):
    L, _ = gpu
    a, b = L.pcg32(42), oracle.pcg32(42)
    assert (a.state, a.inc) == (b.state, b.inc)
    a2, b2 = L.pcg32_advance(a, 123456789), oracle.pcg32_advance(b, 123456789)
    assert (a2.state, a2.inc) == (b2.state, b2.inc)


@pytest.mark.parametrize("n_rays,target,variance", [(8192, 1 << 16, 0.5), (4096, 1 << 15, 0.3), (2048, 4096, 0.5)])
def test_loss_and_compaction(gpu, oracle, n_rays, target, variance):
    L, ops = gpu
    O = oracle
    ods, gds = scene(O, ops)
    _, bf, _ = ball_bitfield(O)
    d, params = sphere_model(O, variance)
    ld = L.GridDesc(d.n_levels, d.log2_hashmap_size, d.base_resolution, d.per_level_scale, d.n_active_levels)
    max_samples = 1 << 20
    ocfg, gcfg = O.train_cfg(), L.train_cfg()
    rng_o, rng_g = O.pcg32(99), L.pcg32(99)
    gen = O.generate_samples(ods, ocfg, n_rays, 777, max_samples, rng_o, bf)
    batch = ops.RayBatch(n_rays, max_samples)
    ops.generate_samples(gds, gcfg, n_rays, 777, rng_g, torch.from_numpy(bf).cuda(), batch)
    mlp_out = ops.neus_forward(ld, half(params), batch.coords, n_dev=batch.counters[4:5])
    torch.cuda.synchronize()
    used = int(batch.counters[4].item())
    # the oracle consumes the GPU's network output so that this test isolates the compositing / loss arithmetic
    ref = O.compute_loss(ods, ocfg, gen, n_rays, 777, rng_o, target, bits(mlp_out))
    coords_out = torch.zeros((target, 7), dtype=torch.float32, device="cuda")
    dloss = torch.zeros((target, 16), dtype=torch.float16, device="cuda")
    loss = torch.zeros(n_rays, dtype=torch.float32, device="cuda")
    ek = torch.zeros(n_rays, dtype=torch.float32, device="cuda")
    ops.compute_loss(gds, gcfg, n_rays, 777, rng_g, target, mlp_out, batch, coords_out, dloss, loss, ek, rollover=False)
    torch.cuda.synchronize()
    k = gen["n_kept"]
    cnt = batch.counters.cpu().numpy().view(np.uint32)
    ns = batch.numsteps.cpu().numpy().view(np.uint32)[:k]
    same = (ns == ref["numsteps"][:k]).all(1)
    record("loss_compaction_%d" % n_rays, rays=k, used=used, compacted=int(cnt[2]), ref_compacted=ref["n_compacted"],
           rays_equal=float(same.mean()))
    assert cnt[2] == ref["n_compacted"], "compacted sample count"
    assert same.all(), "per-ray compacted {count, base}"
    nv = min(ref["n_compacted"], target)
    assert nv > 0
    assert np.array_equal(coords_out.cpu().numpy()[:nv].view(np.uint32), ref["coords"][:nv].view(np.uint32))
    got, want = dloss.float().cpu().numpy()[:nv], O.bits_f32(ref["dloss"])[:nv]
    for name, sl in [("rgb", slice(0, 3)), ("sdf", slice(3, 4)), ("eik", slice(4, 7)), ("var", slice(7, 8)), ("cos", slice(8, 11))]:
        check_fp16("dloss_%s_%d" % (name, n_rays), got[:, sl], want[:, sl], rel=2e-3, min_frac=0.998, min_cos=0.9999)
    assert np.allclose(loss.cpu().numpy()[:k], ref["loss"][:k], rtol=2e-3, atol=1e-9)
    assert np.allclose(ek.cpu().numpy()[:k], ref["ek_loss"][:k], rtol=2e-3, atol=1e-9)
    # roll-over: pad to the target batch by wrap-around and rescale the gradient
    if nv < target:
        ops.compute_loss(gds, gcfg, n_rays, 777, rng_g, target, mlp_out, batch, coords_out, dloss, loss, ek, rollover=True)
        torch.cuda.synchronize()
        rc = O.fill_rollover(ref["coords"].copy(), nv)
        rd = O.fill_rollover_and_rescale_half(ref["dloss"].copy(), nv)
        assert np.array_equal(coords_out.cpu().numpy().view(np.uint32), rc.view(np.uint32))
        check_fp16("rollover_dloss_%d" % n_rays, dloss.float().cpu().numpy(), O.bits_f32(rd), rel=3e-3, min_frac=0.995, min_cos=0.9995)


def test_occupancy_bits_exact_on_same_grid(gpu, oracle):
    """Threshold, Morton bitfield and the 7 max-pool mips are integer work: bit-exact on the same density grid."""
    L, ops = gpu
    O = oracle
    rng = np.random.default_rng(8)
    grid = (rng.random(128 ** 3, dtype=np.float32) ** 8).astype(np.float32)
    grid[rng.random(128 ** 3) < 0.5] = 0.0
    d = O.grid_desc()
    params = torch.zeros(O.model_n_params(d), dtype=torch.float16, device="cuda")
    occ = ops.OccupancyGrid(1)
    occ.grid.copy_(torch.from_numpy(grid))
    ld = L.GridDesc(d.n_levels, d.log2_hashmap_size, d.base_resolution, d.per_level_scale, d.n_active_levels)
    occ.update(ld, params, 0, 0, L.pcg32(1), L.pcg32(2), decay=1.0)
    torch.cuda.synchronize()
    ref_bits, ref_mean = O.occ_bitfield(grid, 1)
    assert np.array_equal(occ.grid.cpu().numpy(), grid)  # decay 1, no samples: grid unchanged
    assert abs(occ.mean.item() - ref_mean) <= 1e-7 * ref_mean
    assert np.array_equal(occ.bitfield.cpu().numpy(), ref_bits)


def test_occupancy_update_matches_oracle(gpu, oracle):
    L, ops = gpu
    O = oracle
    d, params = sphere_model(O, 0.3)
    ld = L.GridDesc(d.n_levels, d.log2_hashmap_size, d.base_resolution, d.per_level_scale, d.n_active_levels)
    n = 128 ** 3 // 4
    occ = ops.OccupancyGrid(1)
    grid = np.zeros(128 ** 3, np.float32)
    for step in range(2):
        ru, rn = 1000 + step, 2000 + step
        occ.update(ld, half(params), n, n, L.pcg32(ru), L.pcg32(rn), decay=0.95)
        torch.cuda.synchronize()
        pu, iu = O.occ_generate_samples(n, O.pcg32(ru), step, grid, 1, -0.01)
        pn, inn = O.occ_generate_samples(n, O.pcg32(rn), step, grid, 1, 0.1)
        pos, idx = np.concatenate([pu, pn]), np.concatenate([iu, inn])
        assert np.array_equal(occ.idx.cpu().numpy().view(np.uint32)[:2 * n], idx)
        assert np.array_equal(occ.pos.cpu().numpy()[:2 * n].view(np.uint32), pos.view(np.uint32))
        # density from the GPU's SDF values: the splat / EMA / threshold chain is what is under test here
        sdf_gpu = bits(occ.sdf[:2 * n])
        sref = O.neus_sdf(d, params, pos)
        check_fp16("occ_sdf_step%d" % step, O.bits_f32(sdf_gpu), O.bits_f32(sref), min_frac=0.9999)
        dens = O.sdf_to_density(sdf_gpu, params[O.GRID_OFF + O.grid_n_params(d)])
        grid = O.occ_splat_ema(idx, dens, grid, 0.95)
        got = occ.grid.cpu().numpy()
        close = np.isclose(got, grid, rtol=2e-3, atol=1e-6).mean()
        record("occ_grid_step%d" % step, close=float(close))
        assert close > 0.9999
        grid = got.copy()  # continue from the GPU's grid so rounding differences do not accumulate
        ref_bits, _ = O.occ_bitfield(grid, 1)
        assert np.array_equal(occ.bitfield.cpu().numpy(), ref_bits)


def test_adam_step(gpu, oracle):
    L, ops = gpu
    O = oracle
    rng = np.random.default_rng(21)
    n_matrix, n_grid = 12288, 100000
    n = n_matrix + n_grid + 4
    master = rng.normal(0, 0.1, n).astype(np.float32)
    m = rng.normal(0, 1e-3, n).astype(np.float32)
    v = (rng.random(n) * 1e-5).astype(np.float32)
    ema = master.copy()
    g = rng.normal(0, 1.0, n).astype(np.float32) * 128
    g[n_matrix:n_matrix + n_grid][rng.random(n_grid) < 0.5] = 0.0  # untouched grid entries
    g_grid_bits = O.f16_bits(g[n_matrix:n_matrix + n_grid])
    g[n_matrix:n_matrix + n_grid] = O.bits_f32(g_grid_bits)
    for step in (1, 7):
        oc = O.AdamCfg(1e-2, 0.9, 0.99, 1e-15, 1e-6, 0.95, 128.0, step, n_matrix)
        gc = L.AdamCfg(1e-2, 0.9, 0.99, 1e-15, 1e-6, 0.95, 128.0, step, n_matrix)
        t = lambda a: torch.from_numpy(a.copy()).cuda()
        gm, gg, gv = t(g[:n_matrix]), half(g_grid_bits), t(g[n_matrix + n_grid:])
        M, Mm, Mv, Me = t(master), t(m), t(v), t(ema)
        P = torch.zeros(n, dtype=torch.float16, device="cuda")
        Pe = torch.zeros(n, dtype=torch.float16, device="cuda")
        ops.adam_step(gc, gm, gg, gv, M, Mm, Mv, P, Pe, Me)
        torch.cuda.synchronize()
        rm, rmm, rv, re = master.copy(), m.copy(), v.copy(), ema.copy()
        rp, rpe = np.zeros(n, np.uint16), np.zeros(n, np.uint16)
        O.adam_step(oc, g, rm, rmm, rv, rp, rpe, re)
        assert np.allclose(M.cpu().numpy(), rm, rtol=1e-5, atol=1e-7)
        assert np.allclose(Mm.cpu().numpy(), rmm, rtol=1e-5, atol=1e-9)
        assert np.allclose(Mv.cpu().numpy(), rv, rtol=1e-5, atol=1e-12)
        assert np.allclose(Me.cpu().numpy(), re, rtol=1e-5, atol=1e-7)
        assert (np.abs(P.float().cpu().numpy() - O.bits_f32(rp)) <= 1e-3 * np.abs(O.bits_f32(rp)) + 1e-7).all()
        assert (np.abs(Pe.float().cpu().numpy() - O.bits_f32(rpe)) <= 1e-3 * np.abs(O.bits_f32(rpe)) + 1e-7).all()
        # gradients are consumed (zeroed) by the step
        assert gm.abs().max().item() == 0 and gg.abs().max().item() == 0 and gv.abs().max().item() == 0
        # zero-gradient grid entries keep their weights and moments
        untouched = np.where(g[n_matrix:n_matrix + n_grid] == 0)[0] + n_matrix
        assert np.array_equal(M.cpu().numpy()[untouched], master[untouched])
