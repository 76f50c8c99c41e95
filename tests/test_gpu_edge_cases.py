"""Edge cases of the path through the C ABI: empty and ragged inputs, a fully occupied and a fully empty occupancy grid
(maximum and zero samples per ray), meshes without a surface, optimizer steps without gradients, the tensor-core path switch."""
import ctypes as C

import numpy as np
import pytest
import torch

from test_gpu_raymarch import ball_bitfield, bits, half, scene, sphere_model

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gpu():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    from neus2_b200 import _lib as L
    from neus2_b200 import ops
    L.lib()
    return L, ops


def compare_batches(ref, batch):
    cnt = batch.counters.cpu().numpy().view(np.uint32)
    k = ref["n_kept"]
    assert cnt[0] == k and cnt[1] == ref["n_samples"]
    if k:
        assert np.array_equal(batch.numsteps.cpu().numpy().view(np.uint32)[:k], ref["numsteps"][:k])
        used = int(ref["numsteps"][k - 1].sum())
        assert np.array_equal(batch.coords.cpu().numpy()[:used].view(np.uint32), ref["coords"][:used].view(np.uint32))
    return cnt


@pytest.mark.parametrize("fill", [0x00, 0xFF])
def test_generate_samples_empty_and_full_grid(gpu, oracle, fill):
    """All cells empty: no ray keeps a sample.  All cells occupied: every ray takes a sample at every step until it leaves
    the box (the most samples a ray can have).  Both bit-exact against the oracle."""
    L, ops = gpu
    O = oracle
    ods, gds = scene(O, ops)
    bf = np.full(128 ** 3 // 8, fill, np.uint8)
    n_rays, max_samples = 2048, 1 << 21
    ref = O.generate_samples(ods, O.train_cfg(), n_rays, 777, max_samples, O.pcg32(5), bf)
    bf_gpu = torch.from_numpy(bf).cuda()
    bounds = ops.occupancy_bounds(bf_gpu)
    b = bounds.cpu().numpy()[:6]
    assert (list(b) == [128, 128, 128, -1, -1, -1]) if fill == 0 else (list(b) == [0, 0, 0, 127, 127, 127])
    for masks in (True, False):
        batch = ops.RayBatch(n_rays, max_samples, march_masks=masks, occupied_bounds=bounds if masks else None)
        ops.generate_samples(gds, L.train_cfg(), n_rays, 777, L.pcg32(5), bf_gpu, batch)
        torch.cuda.synchronize()
        cnt = compare_batches(ref, batch)
        if fill == 0:
            assert cnt[0] == 0 and cnt[1] == 0
        else:
            assert ref["numsteps"][:ref["n_kept"], 0].max() > 500  # rays through the whole cube


def test_generate_samples_ragged_ray_counts(gpu, oracle):
    """Ray counts that are not multiples of the warp / CTA sizes, down to a single ray."""
    L, ops = gpu
    O = oracle
    ods, gds = scene(O, ops)
    _, bf, _ = ball_bitfield(O)
    for n_rays in (1, 31, 33, 1000):
        ref = O.generate_samples(ods, O.train_cfg(), n_rays, 99, 1 << 18, O.pcg32(9), bf)
        batch = ops.RayBatch(n_rays, 1 << 18)
        ops.generate_samples(gds, L.train_cfg(), n_rays, 99, L.pcg32(9), torch.from_numpy(bf).cuda(), batch)
        torch.cuda.synchronize()
        compare_batches(ref, batch)


def test_fused_kernels_accept_empty_batches(gpu):
    """n = 0: both fused kernels return without touching their outputs (both tensor-core paths)."""
    L, ops = gpu
    d = L.grid_desc()
    ng = L.grid_n_params(d)
    params = torch.zeros(12288 + ng + 4, dtype=torch.float16, device="cuda")
    coords = torch.zeros(1, 7, device="cuda")
    out = torch.full((1, 16), 7.0, dtype=torch.float16, device="cuda")
    gm, gg, gv = torch.zeros(12288, device="cuda"), torch.zeros(ng, dtype=torch.float16, device="cuda"), torch.zeros(4, device="cuda")
    dl = torch.zeros(1, 16, dtype=torch.float16, device="cuda")
    for path in (L.MMA_TCGEN05, L.MMA_SYNC):
        L.set_mma_path(path)
        assert L.get_mma_path() == path
        # n = 0 through the host argument and through the device-side count
        L.check(L.lib().neus2b_neus_forward(C.byref(d), L.ptr(params), C.c_float(-0.1), C.c_uint32(0), None, L.ptr(coords), L.ptr(out),
                                            L.cur_stream()))
        ops.neus_forward(d, params, coords, n_dev=torch.zeros(1, dtype=torch.int32, device="cuda"), out=out)
        L.check(L.lib().neus2b_neus_train(C.byref(d), L.ptr(params), C.c_uint32(0), L.ptr(coords), L.ptr(dl), C.c_uint32(1), L.ptr(gm),
                                          L.ptr(gg), L.ptr(gv), L.cur_stream()))
        torch.cuda.synchronize()
        assert float(out[0, 0]) == 7.0 and float(gm.abs().sum()) == 0.0 and float(gg.float().abs().sum()) == 0.0
    L.set_mma_path(L.MMA_TCGEN05)
    assert L.device_error_flags() == 0


def test_marching_cubes_without_surface(gpu):
    """A field that never crosses the threshold gives an empty mesh; a single crossing cell gives its triangles."""
    _, ops = gpu
    sdf = torch.ones(8, 9, 10, device="cuda")
    v, i = ops.marching_cubes(sdf)
    assert v.shape[0] == 0 and i.shape[0] == 0
    sdf[4, 4, 4] = -1.0  # one lattice point inside: an octahedron around it
    v, i = ops.marching_cubes(sdf)
    assert v.shape[0] == 6 and i.shape[0] == 24


def test_adam_without_gradients_leaves_weights(gpu, oracle):
    """Zero gradients: grid entries are skipped (weights, moments untouched), MLP weights only see the L2 term, the EMA moves
    towards the weights; bit-compared with the oracle."""
    L, ops = gpu
    O = oracle
    rng = np.random.default_rng(2)
    n_grid = 4096
    n = 12288 + n_grid + 4
    master = rng.normal(0, 0.1, n).astype(np.float32)
    m = rng.normal(0, 1e-3, n).astype(np.float32)
    v = np.abs(rng.normal(0, 1e-6, n)).astype(np.float32)
    ema = master.copy()
    cfg_o = O.AdamCfg(1e-2, 0.9, 0.99, 1e-15, 1e-6, 0.95, 128.0, 3, 12288)
    cfg_g = L.AdamCfg(1e-2, 0.9, 0.99, 1e-15, 1e-6, 0.95, 128.0, 3, 12288)
    ro = [a.copy() for a in (master, m, v, ema)]
    p_o, pe_o = np.zeros(n, np.uint16), np.zeros(n, np.uint16)
    O.adam_step(cfg_o, np.zeros(n, np.float32), ro[0], ro[1], ro[2], p_o, pe_o, ro[3])
    t = [torch.from_numpy(a.copy()).cuda() for a in (master, m, v, ema)]
    P, Pe = torch.zeros(n, dtype=torch.float16, device="cuda"), torch.zeros(n, dtype=torch.float16, device="cuda")
    gm, gg, gv = torch.zeros(12288, device="cuda"), torch.zeros(n_grid, dtype=torch.float16, device="cuda"), torch.zeros(4, device="cuda")
    ops.adam_step(cfg_g, gm, gg, gv, t[0], t[1], t[2], P, Pe, t[3])
    torch.cuda.synchronize()
    grid = slice(12288, 12288 + n_grid)
    assert np.array_equal(t[0].cpu().numpy()[grid], master[grid]) and np.array_equal(t[1].cpu().numpy()[grid], m[grid])
    for got, want in zip(t, ro):
        assert np.allclose(got.cpu().numpy(), want, rtol=1e-5, atol=1e-7)  # fp32 chains, contraction differs (as in test_adam_step)
    assert (np.abs(P.float().cpu().numpy() - O.bits_f32(p_o)) <= 1e-3 * np.abs(O.bits_f32(p_o)) + 1e-7).all()


def test_occupancy_bounds_of_a_ball(gpu, oracle):
    """The box of occupied cells of a centred ball of radius 0.35 in a 128^3 grid."""
    _, ops = gpu
    _, bf, _ = ball_bitfield(oracle, radius=0.35)
    b = ops.occupancy_bounds(torch.from_numpy(bf).cuda()).cpu().numpy()[:6]
    # cell centres (c + 0.5) / 128 - 0.5 inside the radius: c in [19, 108]
    assert list(b) == [19, 19, 19, 108, 108, 108]
