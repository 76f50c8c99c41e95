"""The learned rigid motion of dynamic sequences (the reference's DeltaNetwork) on the GPU against the oracle: the motion alone,
the fused forward and training kernels with the motion applied first, the twelve sums of its backward and the gradients
made from them, its optimizer step, and rays moved by the accumulated motion in the sample generator."""
import numpy as np
import pytest
import torch

from util import check_fp16, check_grad, model, to_lib_desc

pytestmark = pytest.mark.gpu

DELTA = np.array([0.02, -0.01, 0.03, 0.0, 0.98, 0.1, -0.05, 0.07, 1.02, 0.12, 0.0, 0.0], np.float32)


@pytest.fixture(scope="module")
def gpu():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    from neus2_b200 import _lib as L
    from neus2_b200 import ops
    L.lib()
    return L, ops


def half(bits):
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.float16)).cuda()


def test_motion_alone_matches_oracle(gpu, oracle):
    L, ops = gpu
    rng = np.random.default_rng(0)
    coords = rng.random((5000, 7)).astype(np.float32)
    bits = oracle.f16_bits(DELTA)
    for off in ((0.0, 0.0, 0.0), (0.1, -0.2, 0.05)):
        ref = oracle.delta_forward(bits, coords, off)
        got = ops.delta_forward(half(bits), torch.from_numpy(coords).cuda(), off).cpu().numpy()
        assert np.allclose(got, ref, rtol=0, atol=2e-7)
    # identity parameters leave the samples where they are
    ident = oracle.f16_bits(np.array(ops.DELTA_IDENTITY, np.float32))
    same = ops.delta_forward(half(ident), torch.from_numpy(coords).cuda()).cpu().numpy()
    assert np.allclose(same, coords, rtol=0, atol=1e-7)


def test_backward_sums_and_gradients_match_oracle(gpu, oracle):
    L, ops = gpu
    rng = np.random.default_rng(1)
    n = 70001
    coords = rng.random((n, 7)).astype(np.float32)
    dx = rng.normal(0, 1, (n, 3)).astype(np.float32)
    bits = oracle.f16_bits(DELTA)
    ref = oracle.delta_backward(bits, coords, dx)
    sums = ops.delta_backward(half(bits), torch.from_numpy(coords).cuda(), torch.from_numpy(dx).cuda())
    g = ops.delta_gradient(half(bits), sums).cpu().numpy()
    assert float(sums.abs().max()) == 0.0, "the sums are consumed"
    assert ref[3] == 0 and ref[10] == 0 and ref[11] == 0 and g[3] == 0 and g[10] == 0 and g[11] == 0
    check_grad("delta_gradient", g, ref, min_cos=0.999999, max_rel=2e-4)


@pytest.mark.parametrize("n,L_,n_active", [(65536, 16, 16), (3000, 16, 10), (17, 4, 4)])
def test_fused_kernels_with_motion_match_oracle(gpu, oracle, n, L_, n_active):
    L, ops = gpu
    O = oracle
    kw = dict(n_active=n_active) if L_ == 16 else dict(L=L_, log2T=10, base=4, scale=1.7)
    d, params, coords, rng = model(O, seed=3, n=n, **kw)
    coords[:, :3] = 0.2 + 0.6 * coords[:, :3]  # moved samples stay inside the unit cube
    ld = to_lib_desc(L, d)
    bits = O.f16_bits(DELTA)
    moved = O.delta_forward(bits, coords)
    ref = O.bits_f32(O.neus_forward(d, params, moved))
    dev_delta, dev_coords = half(bits), torch.from_numpy(coords).cuda()
    out = ops.neus_forward_moved(ld, half(params), dev_coords, ops.motion(dev_delta)).float().cpu().numpy()
    tag = "delta_fwd_n%d_L%d_a%d" % (n, L_, n_active)
    check_fp16(tag + "_rgb", out[:, 0:3], ref[:, 0:3], min_frac=0.9999, min_cos=0.99999)
    check_fp16(tag + "_sdf", out[:, 3], ref[:, 3], min_frac=0.9999, min_cos=0.99999)
    check_fp16(tag + "_normal", out[:, 4:7], ref[:, 4:7], min_frac=0.9999, min_cos=0.99999)
    assert np.allclose(out[:, 8:11], ref[:, 8:11], atol=1e-3), "the direction handed on is the moved one"
    sdf = ops.neus_sdf(ld, half(params), dev_coords[:, :3].contiguous(), motion=ops.motion(dev_delta)).float().cpu().numpy()
    check_fp16(tag + "_sdf_only", sdf, O.bits_f32(O.neus_sdf(d, params, moved[:, :3])), min_frac=0.9999)
    # ---- training: canonical gradients equal those at the moved samples, the motion's gradients equal the oracle's chain
    dl = (rng.normal(0, 1e-2, (n, 16))).astype(np.float32)
    dl_bits = O.f16_bits(dl)
    gref, dx = O.neus_backward_dx(d, params, moved, dl_bits, indeed_batch_size=n)
    dref = O.delta_backward(bits, coords, dx)
    ng = O.grid_n_params(d)
    gm = torch.zeros(12288, device="cuda")
    gg = torch.zeros(ng, dtype=torch.float16, device="cuda")
    gv = torch.zeros(4, device="cuda")
    sums = torch.zeros(12, device="cuda")
    ops.neus_train_moved(ld, half(params), dev_coords, ops.motion(dev_delta, sums), half(dl_bits), n, gm, gg, gv)
    torch.cuda.synchronize()
    assert L.device_error_flags() == 0
    check_grad(tag + "_mlp", gm.cpu().numpy(), gref[:12288], min_cos=0.9999)
    if n > 100:
        check_grad(tag + "_grid", gg.float().cpu().numpy(), gref[O.GRID_OFF:O.GRID_OFF + ng], min_cos=0.999)
    g = ops.delta_gradient(dev_delta, sums.clone()).cpu().numpy()
    check_grad(tag + "_delta", g, dref, min_cos=0.9999, max_rel=2e-2)
    # the canonical model frozen: only the motion's sums are produced, and they are the same
    sums2 = torch.zeros(12, device="cuda")
    ops.neus_train_moved(ld, half(params), dev_coords, ops.motion(dev_delta, sums2), half(dl_bits), n, None, None, None)
    torch.cuda.synchronize()
    assert np.allclose(sums2.cpu().numpy(), sums.cpu().numpy(), rtol=1e-4, atol=1e-6 * float(sums.abs().max()))
    with pytest.raises(L.Neus2bError):
        ops.neus_train_moved(ld, half(params), dev_coords, None, half(dl_bits), n, None, None, None)


def test_samples_moved_outside_the_unit_cube(gpu, oracle):
    """A motion can carry samples out of the cube the grid was built for: dense levels clamp the cell to the lattice (such
    samples read the edge cells), hashed levels hash whatever coordinate comes; nothing reads outside the tables."""
    L, ops = gpu
    O = oracle
    d, params, coords, rng = model(O, seed=5, n=20000)
    big = DELTA.copy()
    big[:3] = [0.35, -0.3, 0.25]
    bits = O.f16_bits(big)
    moved = O.delta_forward(bits, coords)
    outside = ((moved[:, :3] < 0) | (moved[:, :3] > 1)).any(1)
    assert 0.3 < outside.mean() < 0.95
    ref = O.bits_f32(O.neus_forward(d, params, moved))
    out = ops.neus_forward_moved(to_lib_desc(L, d), half(params), torch.from_numpy(coords).cuda(), ops.motion(half(bits))).float().cpu().numpy()
    torch.cuda.synchronize()
    check_fp16("delta_outside_sdf", out[:, 3], ref[:, 3], min_frac=0.9999, min_cos=0.99999)
    check_fp16("delta_outside_rgb", out[:, 0:3], ref[:, 0:3], min_frac=0.9999, min_cos=0.99999)


def test_motion_optimizer_step(gpu, oracle):
    L, ops = gpu
    bits = oracle.f16_bits(DELTA)
    delta = half(bits)
    master = torch.from_numpy(oracle.bits_f32(bits).astype(np.float32)).cuda()
    m, v, ema = torch.zeros(12, device="cuda"), torch.zeros(12, device="cuda"), master.clone()
    delta_ema = delta.clone()
    rng = np.random.default_rng(3)
    coords = rng.random((4096, 7)).astype(np.float32)
    dx = (rng.normal(0, 1, (4096, 3)) * 128).astype(np.float32)
    sums = ops.delta_backward(delta, torch.from_numpy(coords).cuda(), torch.from_numpy(dx).cuda())
    gref = oracle.delta_backward(bits, coords, dx) / 128.0
    cfg = L.AdamCfg(1e-3, 0.9, 0.99, 1e-10, 1e-10, 0.95, 128.0, 1, 0)
    before = master.cpu().numpy().copy()
    ops.delta_optimizer_step(cfg, sums, master, m, v, delta, delta_ema, ema)
    torch.cuda.synchronize()
    after = master.cpu().numpy()
    # first Adam step: every parameter with a gradient moves by the learning rate against the gradient's sign
    moved = gref != 0
    assert np.allclose(after[moved], before[moved] - 1e-3 * np.sign(gref[moved]), rtol=0, atol=2e-6)
    assert np.array_equal(after[~moved], before[~moved])
    assert np.allclose(delta.float().cpu().numpy(), after, atol=1e-3) and float(sums.abs().max()) == 0.0
    assert np.allclose(ema.cpu().numpy(), after, atol=1e-6)  # bias-corrected EMA after one step = the weights


def test_rays_moved_by_the_accumulated_motion_bit_exact(gpu, oracle):
    """Sample generation of a later frame: every ray goes through the accumulated rotation and transition before the march."""
    L, ops = gpu
    O = oracle
    from test_gpu_raymarch import ball_bitfield, scene
    ods, gds = scene(O, ops)
    _, bf, _ = ball_bitfield(O)
    R, t = np.eye(3, dtype=np.float32), np.zeros(3, np.float32)
    for k in range(3):  # three frames' worth of motion, folded in the way a frame switch does
        dk = DELTA.copy()
        dk[:3] *= (k + 1) * 0.5
        R, t = O.accumulate_global_movement(O.f16_bits(dk), R, t)
    Rg, tg = np.eye(3, dtype=np.float32), np.zeros(3, np.float32)
    for k in range(3):
        dk = DELTA.copy()
        dk[:3] *= (k + 1) * 0.5
        Rg, tg = ops.movement_accumulate(O.f16_bits(dk), Rg, tg)
    assert np.array_equal(Rg, R) and np.array_equal(tg, t), "host accumulation equals the oracle's"
    off = (0.01, 0.0, -0.02)
    n_rays, max_samples = 4096, 1 << 20
    ocfg = O.train_cfg(rotation=R, transition=t, first_frame_offset=off)
    gcfg = L.train_cfg(rotation=R.reshape(9), transition=t, first_frame_offset=off)
    ref = O.generate_samples(ods, ocfg, n_rays, 12345, max_samples, O.pcg32(1337), bf)
    plain = O.generate_samples(ods, O.train_cfg(), n_rays, 12345, max_samples, O.pcg32(1337), bf)
    assert ref["n_samples"] != plain["n_samples"], "the motion must change the march"
    bf_gpu = torch.from_numpy(bf).cuda()
    for masks in (True, False):
        bounds = ops.occupancy_bounds(bf_gpu) if masks else None
        batch = ops.RayBatch(n_rays, max_samples, march_masks=masks, occupied_bounds=bounds)
        ops.generate_samples(gds, gcfg, n_rays, 12345, L.pcg32(1337), bf_gpu, batch)
        torch.cuda.synchronize()
        cnt = batch.counters.cpu().numpy().view(np.uint32)
        k = ref["n_kept"]
        assert k > 0 and cnt[0] == k and cnt[1] == ref["n_samples"]
        assert np.array_equal(batch.numsteps.cpu().numpy().view(np.uint32)[:k], ref["numsteps"][:k])
        assert np.array_equal(batch.rays.cpu().numpy()[:k].view(np.uint32), ref["rays"][:k].view(np.uint32))
        used = int(ref["numsteps"][k - 1].sum())
        assert np.array_equal(batch.coords.cpu().numpy()[:used].view(np.uint32), ref["coords"][:used].view(np.uint32))
