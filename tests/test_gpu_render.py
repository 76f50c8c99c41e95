"""GPU parity of the inference renderer through the C ABI against the CPU oracle: the rays and sample coordinates of a frame
(bit-exact), the composited frame and depth (tolerance: the network outputs are fp16 and the tensor-core path sums in another
order), windows and bands (bit-identical to a single pass), accumulate / tone mapping, and Testbed.render on a trained
scene."""
import numpy as np
import pytest
import torch

from test_gpu_raymarch import ball_bitfield, half, sphere_model
from util import record

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gpu():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    from neus2_b200 import _lib as L
    from neus2_b200 import ops
    L.lib()
    return L, ops


def camera(view=3, n_views=8):
    from neus2_b200 import synthetic as S
    X = S.fibonacci_cameras(n_views, 2.5)[view]
    return np.stack([X[0:3], X[3:6], X[6:9], X[9:12]], 1)  # 3x4


def cfg_kwargs(w, h, fov=40.0, **kw):
    f = 0.5 * h / np.tan(0.5 * np.radians(fov))
    d = dict(width=w, height=h, focal_length=(f, f), camera=camera())
    d.update(kw)
    return d


def gpu_frame(L, ops, d, params_bits, cfg, bf, max_rays=None, max_samples=1 << 21, bounds=False, masks=False):
    n_pix = cfg.width * cfg.height
    bf_gpu = torch.from_numpy(bf).cuda()
    ob = ops.occupancy_bounds(bf_gpu) if bounds else None
    buf = ops.RenderBuffers(max_rays or n_pix, max_samples, occupied_bounds=ob, masks=masks)
    frame = torch.zeros((cfg.height, cfg.width, 4), dtype=torch.float32, device="cuda")
    depth = torch.zeros((cfg.height, cfg.width), dtype=torch.float32, device="cuda")
    gd = L.GridDesc(d.n_levels, d.log2_hashmap_size, d.base_resolution, d.per_level_scale, d.n_active_levels)
    n = ops.render_frame(gd, half(params_bits), -0.1, cfg, bf_gpu, buf, frame, depth)
    torch.cuda.synchronize()
    return frame.cpu().numpy(), depth.cpu().numpy(), n, buf


@pytest.mark.parametrize("bounds,masks", [(False, False), (True, False), (True, True), (False, True)])
@pytest.mark.parametrize("w,h,offset,spp", [(96, 64, (0.5, 0.5), 0), (61, 47, (0.794, 0.19), 3)])
def test_render_march_bit_exact(gpu, oracle, w, h, offset, spp, bounds, masks):
    L, ops = gpu
    O = oracle
    _, bf, _ = ball_bitfield(O)
    d, pb = sphere_model(O)
    kw = cfg_kwargs(w, h, pixel_offset=offset, sample_index=spp)
    numsteps, coords, n = O.render_march(O.render_cfg(**kw), bf)
    assert n > 1000
    _, _, n_gpu, buf = gpu_frame(L, ops, d, pb, ops.render_cfg(**kw), bf, bounds=bounds, masks=masks)
    assert n_gpu == n
    got_steps = buf.ray_tmp.cpu().numpy().view(np.uint32)[:, 7] & 0x7fffffff
    np.testing.assert_array_equal(got_steps, numsteps)
    np.testing.assert_array_equal(buf.coords.cpu().numpy()[:n].view(np.uint32), coords.view(np.uint32))


@pytest.fixture(scope="module")
def trained(gpu):
    """A briefly trained sphere scene: its weights (EMA, as fp16 bits), occupancy bits and one training camera."""
    L, ops = gpu
    from neus2_b200 import synthetic as S
    from neus2_b200.testbed import Testbed
    from test_gpu_testbed import cuda_view
    res = 128
    sc = S.render_sphere_views(16, res, res, device="cuda", seed=0)
    tb = Testbed(batch_size=1 << 16)
    tb.load_training_data(sc["pixels"].cpu().numpy(), *[sc[k].cpu().numpy() for k in ("xforms", "focal", "principal")])
    tb.set_params(S.init_params(L.grid_n_params(tb.config.grid), seed=1337))
    tb.train(400)
    ptrs = tb.device_ptrs()
    n = tb.n_params
    pb = cuda_view(ptrs["params_ema"], n * 2).cpu().numpy().view(np.uint16).copy()
    bf = cuda_view(ptrs["bitfield"], 128 ** 3 // 8).cpu().numpy().copy()
    yield dict(tb=tb, scene=sc, params_bits=pb, bitfield=bf, res=res)
    tb.close()


def view_camera(sc, view):
    X = sc["xforms"][view].cpu().numpy()
    return np.stack([X[0:3], X[3:6], X[6:9], X[9:12]], 1)


def test_render_frame_matches_oracle(gpu, oracle, trained):
    L, ops = gpu
    O = oracle
    d = O.grid_desc()
    pb, bf = trained["params_bits"], trained["bitfield"]
    w, h = 96, 72
    f = 0.5 * h / np.tan(0.5 * np.radians(40.0))
    kw = dict(width=w, height=h, focal_length=(f, f), camera=view_camera(trained["scene"], 2), pixel_offset=(0.41, 0.77), sample_index=2)
    ref, ref_depth, n_ref = O.render_frame(d, pb, O.render_cfg(**kw), bf)
    got, got_depth, n_gpu, _ = gpu_frame(L, ops, d, pb, ops.render_cfg(**kw), bf, bounds=True)
    assert 0 < n_ref <= n_gpu  # the rounds stop at opaque rays, the single pass evaluates the whole march
    cover = ref[..., 3] > 0.5
    assert cover.sum() > 300, "the test scene must have opaque pixels"
    err = np.abs(got - ref)
    record("render_frame", max_abs_err=float(err.max()), mean_abs_err=float(err.mean()), samples_oracle=n_ref, samples_gpu=n_gpu)
    # fp16 network outputs and another summation order on the tensor cores: a sample near the opacity threshold can fall on
    # the other side, which moves one pixel by up to one sample's weight
    assert err.mean() < 1e-3
    assert np.quantile(err, 0.999) < 2e-2
    wrote = ref_depth < 1e9
    assert ((got_depth < 1e9) == wrote).mean() > 0.995
    both = wrote & (got_depth < 1e9)
    assert np.median(np.abs(got_depth[both] - ref_depth[both])) < 2e-3
    assert np.all(got_depth[got[..., 3] <= 0.2] == np.float32(1e10))


def test_render_windows_and_bands_identical(gpu, oracle):
    L, ops = gpu
    O = oracle
    _, bf, _ = ball_bitfield(O)
    d, pb = sphere_model(O)
    cfg = ops.render_cfg(**cfg_kwargs(72, 56, pixel_offset=(0.3, 0.7), sample_index=1))
    one, one_depth, n, _ = gpu_frame(L, ops, d, pb, cfg, bf)
    win, win_depth, n2, _ = gpu_frame(L, ops, d, pb, cfg, bf, max_samples=4096)       # many windows, rays split across them
    wm, wm_depth, n4, _ = gpu_frame(L, ops, d, pb, cfg, bf, max_samples=4096, masks=True, bounds=True)
    assert n4 == n
    np.testing.assert_array_equal(one.view(np.uint32), wm.view(np.uint32))
    np.testing.assert_array_equal(one_depth.view(np.uint32), wm_depth.view(np.uint32))
    band, band_depth, n3, _ = gpu_frame(L, ops, d, pb, cfg, bf, max_rays=72 * 5 + 10)  # bands of 5 rows
    assert n > 3 * 4096 and n == n2 == n3
    np.testing.assert_array_equal(one.view(np.uint32), win.view(np.uint32))
    np.testing.assert_array_equal(one_depth.view(np.uint32), win_depth.view(np.uint32))
    np.testing.assert_array_equal(one.view(np.uint32), band.view(np.uint32))
    np.testing.assert_array_equal(one_depth.view(np.uint32), band_depth.view(np.uint32))


def test_render_blends_over_existing_frame_and_empty_grid(gpu, oracle):
    L, ops = gpu
    O = oracle
    d, pb = sphere_model(O)
    cfg = ops.render_cfg(**cfg_kwargs(40, 30))
    empty = np.zeros(128 ** 3 * 8 // 8, np.uint8)
    got, depth, n, _ = gpu_frame(L, ops, d, pb, cfg, empty, bounds=True)
    assert n == 0 and not got.any() and np.all(depth == np.float32(1e10))
    # a frame that already holds an opaque colour shows through where the render is transparent (shade_kernel_nerf)
    _, bf, _ = ball_bitfield(O)
    bf_gpu = torch.from_numpy(bf).cuda()
    buf = ops.RenderBuffers(40 * 30, 1 << 20)
    frame = torch.zeros((30, 40, 4), dtype=torch.float32, device="cuda")
    frame[..., 1] = 1.0
    frame[..., 3] = 1.0
    dep = torch.zeros((30, 40), dtype=torch.float32, device="cuda")
    gd = L.GridDesc(d.n_levels, d.log2_hashmap_size, d.base_resolution, d.per_level_scale, d.n_active_levels)
    ops.render_frame(gd, half(pb), -0.1, cfg, bf_gpu, buf, frame, dep)
    f = frame.cpu().numpy()
    ref, _, _ = O.render_frame(d, pb, O.render_cfg(**cfg_kwargs(40, 30)), bf, frame=np.tile(np.float32([0, 1, 0, 1]), (30, 40, 1)))
    assert np.abs(f - ref).max() < 2e-2
    assert np.allclose(f[0, 0], [0, 1, 0, 1])


def test_accumulate_and_tonemap(gpu, oracle):
    L, ops = gpu
    O = oracle
    rng = np.random.default_rng(5)
    frames = rng.uniform(0, 1, (3, 33, 21, 4)).astype(np.float32)
    frames[..., :3] *= frames[..., 3:]
    acc_ref = np.zeros_like(frames[0])
    acc = torch.full((33, 21, 4), 7.0, dtype=torch.float32, device="cuda")  # stale content: sample 0 overwrites
    for s in range(3):
        O.render_accumulate(frames[s], acc_ref, s)
        ops.render_accumulate(torch.from_numpy(frames[s]).cuda(), acc, s)
    np.testing.assert_allclose(acc.cpu().numpy(), acc_ref, rtol=1e-6, atol=1e-7)
    for to_srgb, bg, ex in ((True, (0.2, 0.4, 0.9, 1.0), 0.0), (False, (1.0, 1.0, 1.0, 0.5), 1.5), (True, (0, 0, 0, 0), -1.0)):
        ref = O.render_tonemap(acc_ref, ex, bg, to_srgb)
        got = ops.render_tonemap(acc, ex, bg, to_srgb).cpu().numpy()
        np.testing.assert_allclose(got, ref, rtol=2e-5, atol=2e-6)


def test_testbed_render_after_training(gpu, trained):
    """Render a training view of the briefly trained scene with Testbed.render and compare it with that view's image."""
    tb, sc, res = trained["tb"], trained["scene"], trained["res"]
    view = 5
    tb.camera_matrix = view_camera(sc, view)
    tb.fov = 40.0
    assert abs(tb.fov - 40.0) < 1e-4
    tb.snap_to_pixel_centers = True
    tb.background_color = [0.0, 0.0, 0.0, 0.0]
    img, depth = tb.render(res, res, spp=1, linear=False, return_depth=True)
    px = sc["pixels"][view].cpu().numpy().view(np.uint32)
    gt = np.stack([(px >> s) & 0xFF for s in (0, 8, 16, 24)], -1).astype(np.float32) / 255.0
    inside = gt[..., 3] > 0.5
    agree = ((img[..., 3] > 0.5) == inside).mean()
    assert agree > 0.97
    # colour inside the silhouette (sRGB, both images), away from the rim
    core = inside & (img[..., 3] > 0.99)
    assert core.sum() > 0.8 * inside.sum()
    mse = float(((img[..., :3] - gt[..., :3])[core] ** 2).mean())
    psnr = -10.0 * np.log10(mse)
    record("render_after_400_steps", psnr=float(psnr), silhouette_agreement=float(agree))
    assert psnr > 18.0
    # depth of the sphere's front along the camera axis: between cam_radius - radius and cam_radius
    dd = depth[core]
    assert dd.min() > 2.5 - 0.3 - 0.05 and dd.max() < 2.5 + 0.08  # (a 400-step surface is still a little soft at the rim)
    # two samples per pixel average two jitters; the result stays close to the single-sample image
    tb.snap_to_pixel_centers = False
    img2 = tb.render(res, res, spp=2, linear=False)
    assert np.abs(img2 - img).max() > 0 and np.abs(img2[core] - img[core]).mean() < 0.05
    # linear output: the same image before the sRGB curve
    lin = tb.render(res, res, spp=2, linear=True)
    a = lin[core][:, :3]
    srgb = np.where(a < 0.0031308, 12.92 * a, 1.055 * np.power(np.maximum(a, 1e-12), 0.41666) - 0.055)
    assert np.abs(srgb - img2[core][:, :3]).max() < 1e-4
    # another resolution reallocates the buffers
    small = tb.render(40, 30, spp=1)
    assert small.shape == (30, 40, 4) and small[..., 3].max() > 0.9
