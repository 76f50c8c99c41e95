"""ctypes/numpy front end of the CPU oracle (``neus2_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by ``__graft_entry__.smoke()`` and by the CPU-baseline legs of
``bench.py``.  The product package never imports it.  "Parity unpinned" for the parts whose reference arithmetic
lives in the un-vendored tiny-cuda-nn fork (hash grid, MLPs, SH, Adam, pcg32); see the header of ``neus2_oracle.h``.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libneus2_oracle.so")

MLP_N = 64 * 48 + 16 * 64 + 64 * 48 + 64 * 64 + 16 * 64
SDF_N = 64 * 48 + 16 * 64
GRID_OFF = MLP_N


def build(force=False):
    src = [os.path.join(_HERE, f) for f in ("neus2_oracle.c", "neus2_oracle.h", "Makefile")]
    if force or not os.path.exists(_SO) or any(os.path.getmtime(s) > os.path.getmtime(_SO) for s in src):
        subprocess.run(["make", "-C", _HERE], check=True, capture_output=True)
    return _SO


class GridDesc(C.Structure):
    _fields_ = [("n_levels", C.c_uint32), ("log2_hashmap_size", C.c_uint32), ("base_resolution", C.c_uint32),
                ("per_level_scale", C.c_float), ("n_active_levels", C.c_uint32)]


class GridLevels(C.Structure):
    _fields_ = [("offset", C.c_uint32 * 17), ("res", C.c_uint32 * 16), ("hashed", C.c_uint32 * 16), ("scale", C.c_float * 16)]


class Pcg32(C.Structure):
    _fields_ = [("state", C.c_uint64), ("inc", C.c_uint64)]


class Dataset(C.Structure):
    _fields_ = [("n_images", C.c_uint32), ("width", C.c_uint32), ("height", C.c_uint32), ("pixels", C.c_void_p),
                ("xforms", C.c_void_p), ("focal", C.c_void_p), ("principal", C.c_void_p)]


class TrainCfg(C.Structure):
    _fields_ = [("aabb_min", C.c_float * 3), ("aabb_max", C.c_float * 3), ("cone_angle_constant", C.c_float),
                ("snap_to_pixel_centers", C.c_uint32), ("random_bg_color", C.c_uint32), ("background_color", C.c_float * 3),
                ("loss_scale", C.c_float), ("mask_loss_weight", C.c_float), ("ek_loss_weight", C.c_float),
                ("cos_anneal_ratio", C.c_float), ("ray_index_offset", C.c_uint32), ("ray_count_scale", C.c_uint32),
                ("use_global_movement", C.c_uint32), ("rotation", C.c_float * 9), ("transition", C.c_float * 3),
                ("first_frame_offset", C.c_float * 3)]


class RenderCfg(C.Structure):
    _fields_ = [("width", C.c_uint32), ("height", C.c_uint32), ("focal_length", C.c_float * 2), ("screen_center", C.c_float * 2),
                ("camera", C.c_float * 12), ("pixel_offset", C.c_float * 2), ("sample_index", C.c_uint32),
                ("aabb_min", C.c_float * 3), ("aabb_max", C.c_float * 3), ("cone_angle_constant", C.c_float),
                ("min_transmittance", C.c_float), ("cos_anneal_ratio", C.c_float), ("linear_colors", C.c_uint32),
                ("max_steps", C.c_uint32)]


class AdamCfg(C.Structure):
    _fields_ = [("learning_rate", C.c_float), ("beta1", C.c_float), ("beta2", C.c_float), ("epsilon", C.c_float),
                ("l2_reg", C.c_float), ("ema_decay", C.c_float), ("loss_scale", C.c_float), ("step", C.c_uint32),
                ("n_matrix", C.c_uint32)]


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_SO)
        _lib.n2o_grid_n_params.restype = C.c_uint32
        _lib.n2o_model_n_params.restype = C.c_uint32
        _lib.n2o_generate_samples.restype = C.c_uint32
        _lib.n2o_compute_loss.restype = C.c_uint32
        _lib.n2o_pcg32_next_uint.restype = C.c_uint32
        _lib.n2o_pcg32_next_float.restype = C.c_float
        _lib.n2o_morton3d.restype = C.c_uint32
        _lib.n2o_morton3d_invert.restype = C.c_uint32
        _lib.n2o_ld_random_val.restype = C.c_float
    return _lib


def set_num_threads(n):
    lib().n2o_set_num_threads(C.c_int(int(n)))


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _c(a, dt):
    a = np.ascontiguousarray(a, dtype=dt)
    return a


def grid_desc(n_levels=16, log2_hashmap_size=19, base_resolution=16, per_level_scale=1.447, n_active_levels=None):
    return GridDesc(n_levels, log2_hashmap_size, base_resolution, per_level_scale,
                    n_levels if n_active_levels is None else n_active_levels)


def grid_levels(d):
    lv = GridLevels()
    lib().n2o_grid_make_levels(C.byref(d), C.byref(lv))
    return lv


def grid_n_params(d):
    return int(lib().n2o_grid_n_params(C.byref(d)))


def model_n_params(d):
    return int(lib().n2o_model_n_params(C.byref(d)))


def f16_bits(a):
    """float array -> uint16 bit patterns (round to nearest even)."""
    return np.asarray(a, dtype=np.float32).astype(np.float16).view(np.uint16)


def bits_f32(a):
    return np.asarray(a, dtype=np.uint16).view(np.float16).astype(np.float32)


def grid_forward(d, x, grid, want_dydx=False):
    x = _c(x, np.float32)
    n, W = x.shape[0], 2 * d.n_levels
    enc = np.empty((n, W), np.uint16)
    dydx = np.empty((n, W, 3), np.float32) if want_dydx else None
    lib().n2o_grid_forward(C.byref(d), C.c_uint32(n), _p(x), C.c_uint32(x.shape[1]), _p(grid), _p(enc), _p(dydx))
    return (enc, dydx) if want_dydx else enc


def grid_backward_input(d, x, grid, dL_denc):
    x = _c(x, np.float32)
    out = np.empty((x.shape[0], 3), np.float32)
    lib().n2o_grid_backward_input(C.byref(d), C.c_uint32(x.shape[0]), _p(x), C.c_uint32(x.shape[1]), _p(grid),
                                  _p(_c(dL_denc, np.uint16)), _p(out))
    return out


def grid_backward_params(d, x, dL_denc, grad=None):
    x = _c(x, np.float32)
    if grad is None:
        grad = np.zeros(grid_n_params(d), np.float64)
    lib().n2o_grid_backward_params(C.byref(d), C.c_uint32(x.shape[0]), _p(x), C.c_uint32(x.shape[1]),
                                   _p(_c(dL_denc, np.uint16)), _p(grad))
    return grad


def grid_backward_backward_input(d, x, grid, v, g_e, grad=None):
    x = _c(x, np.float32)
    n, W = x.shape[0], 2 * d.n_levels
    if grad is None:
        grad = np.zeros(grid_n_params(d), np.float64)
    dy = np.empty((n, W), np.uint16)
    lib().n2o_grid_backward_backward_input(C.byref(d), C.c_uint32(n), _p(x), C.c_uint32(x.shape[1]), _p(grid),
                                           _p(_c(v, np.float32)), _p(_c(g_e, np.uint16)), _p(grad), _p(dy))
    return grad, dy


def mlp_forward(in_w, n_hidden, w, inp):
    inp = _c(inp, np.uint16)
    n = inp.shape[0]
    out = np.empty((n, 16), np.uint16)
    hidden = np.empty((n, n_hidden, 64), np.uint16)
    lib().n2o_mlp_forward(C.c_uint32(n), C.c_uint32(in_w), C.c_uint32(n_hidden), _p(_c(w, np.uint16)), _p(inp), _p(out),
                          _p(hidden))
    return out, hidden


def mlp_backward(in_w, n_hidden, w, inp, hidden, dL_dout, want_wgrad=True):
    inp = _c(inp, np.uint16)
    n = inp.shape[0]
    din = np.empty((n, in_w), np.uint16)
    np_ = 64 * in_w + (n_hidden - 1) * 4096 + 1024
    wg = np.zeros(np_, np.float64) if want_wgrad else None
    lib().n2o_mlp_backward(C.c_uint32(n), C.c_uint32(in_w), C.c_uint32(n_hidden), _p(_c(w, np.uint16)), _p(inp),
                           _p(_c(hidden, np.uint16)), _p(_c(dL_dout, np.uint16)), _p(din), _p(wg))
    return din, wg


def mlp_backward_backward_input(in_w, w, hidden, u, dy):
    u = _c(u, np.uint16)
    wg = np.zeros(64 * in_w + 1024, np.float64)
    lib().n2o_mlp_backward_backward_input(C.c_uint32(u.shape[0]), C.c_uint32(in_w), _p(_c(w, np.uint16)),
                                          _p(_c(hidden, np.uint16)), _p(u), _p(_c(dy, np.uint16)), _p(wg))
    return wg


def sh4(dir01):
    dir01 = _c(dir01, np.float32)
    out = np.empty((dir01.shape[0], 16), np.uint16)
    lib().n2o_sh4(C.c_uint32(dir01.shape[0]), _p(dir01), C.c_uint32(dir01.shape[1]), _p(out))
    return out


def neus_forward(d, params, coords, sdf_bias=-0.1):
    coords = _c(coords, np.float32)
    out = np.empty((coords.shape[0], 16), np.uint16)
    lib().n2o_neus_forward(C.byref(d), _p(_c(params, np.uint16)), C.c_float(sdf_bias), C.c_uint32(coords.shape[0]), _p(coords),
                           _p(out))
    return out


def neus_backward(d, params, coords, dL_dout, indeed_batch_size=None, grad=None):
    coords = _c(coords, np.float32)
    n = coords.shape[0]
    if grad is None:
        grad = np.zeros(model_n_params(d), np.float64)
    lib().n2o_neus_backward(C.byref(d), _p(_c(params, np.uint16)), C.c_uint32(n), _p(coords), _p(_c(dL_dout, np.uint16)),
                            C.c_uint32(n if indeed_batch_size is None else indeed_batch_size), _p(grad))
    return grad


def neus_backward_dx(d, params, coords, dL_dout, indeed_batch_size=None, grad=None):
    """neus_backward plus dL/dx [n][3], the gradient handed to the DeltaNetwork."""
    coords = _c(coords, np.float32)
    n = coords.shape[0]
    if grad is None:
        grad = np.zeros(model_n_params(d), np.float64)
    dx = np.zeros((n, 3), np.float32)
    lib().n2o_neus_backward_dx(C.byref(d), _p(_c(params, np.uint16)), C.c_uint32(n), _p(coords), _p(_c(dL_dout, np.uint16)),
                               C.c_uint32(n if indeed_batch_size is None else indeed_batch_size), _p(grad), _p(dx))
    return grad, dx


def rotation_6d_to_matrix(rot6_bits):
    R = np.zeros(9, np.float32)
    lib().n2o_rotation_6d_to_matrix(_p(_c(rot6_bits, np.uint16)), _p(R))
    return R.reshape(3, 3)


def delta_forward(delta_bits, coords, first_frame_offset=(0.0, 0.0, 0.0)):
    coords = _c(coords, np.float32)
    out = np.empty_like(coords)
    lib().n2o_delta_forward(_p(_c(delta_bits, np.uint16)), (C.c_float * 3)(*first_frame_offset), C.c_uint32(coords.shape[0]), _p(coords), _p(out))
    return out


def delta_backward(delta_bits, coords, dL_dx, first_frame_offset=(0.0, 0.0, 0.0)):
    coords, dL_dx = _c(coords, np.float32), _c(dL_dx, np.float32)
    grad = np.zeros(12, np.float64)
    lib().n2o_delta_backward(_p(_c(delta_bits, np.uint16)), (C.c_float * 3)(*first_frame_offset), C.c_uint32(coords.shape[0]), _p(coords),
                             _p(dL_dx), _p(grad))
    return grad


def accumulate_global_movement(delta_bits, acc_rotation, acc_transition):
    R, t = _c(acc_rotation, np.float32).copy().reshape(9), _c(acc_transition, np.float32).copy()
    lib().n2o_accumulate_global_movement(_p(_c(delta_bits, np.uint16)), _p(R), _p(t))
    return R.reshape(3, 3), t


def neus_sdf(d, params, x, sdf_bias=-0.1):
    x = _c(x, np.float32)
    out = np.empty(x.shape[0], np.uint16)
    lib().n2o_neus_sdf(C.byref(d), _p(_c(params, np.uint16)), C.c_float(sdf_bias), C.c_uint32(x.shape[0]), _p(x),
                       C.c_uint32(x.shape[1]), _p(out))
    return out


def pcg32(seed):
    r = Pcg32()
    lib().n2o_pcg32_seed(C.byref(r), C.c_uint64(seed))
    return r


def pcg32_advance(r, delta):
    r2 = Pcg32(r.state, r.inc)
    lib().n2o_pcg32_advance(C.byref(r2), C.c_uint64(delta))
    return r2


def pcg32_next_uint(r):
    """Advances r in place and returns the next 32-bit output."""
    return int(lib().n2o_pcg32_next_uint(C.byref(r)))


def pcg32_floats(r, n):
    r2 = Pcg32(r.state, r.inc)
    return np.array([lib().n2o_pcg32_next_float(C.byref(r2)) for _ in range(n)], np.float32)


def make_dataset(pixels, xforms, focal, principal):
    """pixels uint32 [n][H][W]; xforms float32 [n][12]; focal/principal float32 [n][2]. Keeps references alive."""
    pixels = _c(pixels, np.uint32)
    xforms = _c(xforms, np.float32)
    focal = _c(focal, np.float32)
    principal = _c(principal, np.float32)
    ds = Dataset(pixels.shape[0], pixels.shape[2], pixels.shape[1], _p(pixels), _p(xforms), _p(focal), _p(principal))
    ds._keep = (pixels, xforms, focal, principal)
    return ds


def train_cfg(ek_loss_weight=0.1, mask_loss_weight=0.0, random_bg_color=True, snap_to_pixel_centers=False,
              cos_anneal_ratio=1.0, loss_scale=128.0, background_color=(0.0, 0.0, 0.0), ray_index_offset=0,
              ray_count_scale=1, rotation=None, transition=None, first_frame_offset=(0.0, 0.0, 0.0)):
    c = TrainCfg()
    if rotation is not None:
        c.use_global_movement = 1
        c.rotation[:] = [float(v) for v in np.asarray(rotation, np.float32).reshape(9)]
        c.transition[:] = [float(v) for v in np.asarray(transition, np.float32).reshape(3)]
        c.first_frame_offset[:] = list(first_frame_offset)
    c.aabb_min[:] = [0.0, 0.0, 0.0]
    c.aabb_max[:] = [1.0, 1.0, 1.0]
    c.cone_angle_constant = 0.0
    c.snap_to_pixel_centers = int(snap_to_pixel_centers)
    c.random_bg_color = int(random_bg_color)
    c.background_color[:] = list(background_color)
    c.loss_scale = loss_scale
    c.mask_loss_weight = mask_loss_weight
    c.ek_loss_weight = ek_loss_weight
    c.cos_anneal_ratio = cos_anneal_ratio
    c.ray_index_offset = ray_index_offset
    c.ray_count_scale = ray_count_scale
    return c


def generate_samples(ds, cfg, n_rays, n_rays_total, max_samples, rng, bitfield):
    ray_indices = np.zeros(n_rays, np.uint32)
    rays = np.zeros((n_rays, 6), np.float32)
    numsteps = np.zeros((n_rays, 2), np.uint32)
    coords = np.zeros((max_samples, 7), np.float32)
    ns = C.c_uint32(0)
    kept = lib().n2o_generate_samples(C.byref(ds), C.byref(cfg), C.c_uint32(n_rays), C.c_uint32(n_rays_total),
                                      C.c_uint32(max_samples), rng, _p(_c(bitfield, np.uint8)), _p(ray_indices), _p(rays),
                                      _p(numsteps), _p(coords), C.byref(ns))
    return dict(n_kept=int(kept), n_samples=int(ns.value), ray_indices=ray_indices, rays=rays, numsteps=numsteps,
                coords=coords)


def compute_loss(ds, cfg, gen, n_rays, n_rays_total, rng, max_compacted, mlp_out):
    numsteps = gen["numsteps"].copy()
    coords_out = np.zeros((max_compacted, 7), np.float32)
    dloss = np.zeros((max_compacted, 16), np.uint16)
    loss = np.zeros(max(gen["n_kept"], 1), np.float32)
    ek = np.zeros(max(gen["n_kept"], 1), np.float32)
    total = lib().n2o_compute_loss(C.byref(ds), C.byref(cfg), C.c_uint32(gen["n_kept"]), C.c_uint32(n_rays),
                                   C.c_uint32(n_rays_total), rng, C.c_uint32(max_compacted), _p(_c(mlp_out, np.uint16)),
                                   _p(gen["ray_indices"]), _p(gen["rays"]), _p(numsteps), _p(gen["coords"]), _p(coords_out),
                                   _p(dloss), _p(loss), _p(ek))
    return dict(n_compacted=int(total), numsteps=numsteps, coords=coords_out, dloss=dloss, loss=loss, ek_loss=ek)


def fill_rollover(data, n_valid):
    data = _c(data, np.float32)
    lib().n2o_fill_rollover(C.c_uint32(data.shape[0]), C.c_uint32(data.shape[1]), C.c_uint32(n_valid), _p(data))
    return data


def fill_rollover_and_rescale_half(data, n_valid):
    data = _c(data, np.uint16)
    lib().n2o_fill_rollover_and_rescale_half(C.c_uint32(data.shape[0]), C.c_uint32(data.shape[1]), C.c_uint32(n_valid), _p(data))
    return data


def occ_generate_samples(n, rng, step, grid_in, n_cascades, thresh):
    pos = np.empty((n, 3), np.float32)
    idx = np.empty(n, np.uint32)
    mn = (C.c_float * 3)(0, 0, 0)
    mx = (C.c_float * 3)(1, 1, 1)
    lib().n2o_occ_generate_samples(C.c_uint32(n), rng, C.c_uint32(step), mn, mx, _p(_c(grid_in, np.float32)),
                                   C.c_uint32(n_cascades), C.c_float(thresh), _p(pos), _p(idx))
    return pos, idx


def sdf_to_density(sdf_bits, variance_bits):
    out = _c(sdf_bits, np.uint16).copy()
    lib().n2o_sdf_to_density(C.c_uint32(out.size), C.c_uint16(int(variance_bits)), _p(out))
    return out


def occ_splat_ema(indices, density, grid, decay):
    grid = _c(grid, np.float32)
    tmp = np.empty_like(grid)
    lib().n2o_occ_splat_ema(C.c_uint32(indices.size), _p(_c(indices, np.uint32)), _p(_c(density, np.uint16)),
                            C.c_uint32(grid.size), C.c_float(decay), _p(tmp), _p(grid))
    return grid


def occ_bitfield(grid, n_cascades_used=1):
    bits = np.zeros(128 ** 3 // 8 * 8, np.uint8)
    mean = C.c_float(0)
    lib().n2o_occ_bitfield(C.c_uint32(n_cascades_used), _p(_c(grid, np.float32)), _p(bits), C.byref(mean))
    return bits, float(mean.value)


def adam_step(cfg, grad, master, m, v, params, params_ema=None, ema_master=None):
    lib().n2o_adam_step(C.byref(cfg), C.c_uint32(master.size), _p(_c(grad, np.float32)), _p(master), _p(m), _p(v), _p(params),
                        _p(params_ema), _p(ema_master))


def marching_cubes(sdf, res, tri_table, thresh=0.0, aabb_min=(0, 0, 0), aabb_max=(1, 1, 1)):
    sdf = _c(sdf, np.float32)
    r = (C.c_uint32 * 3)(*res)
    mn = (C.c_float * 3)(*aabb_min)
    mx = (C.c_float * 3)(*aabb_max)
    tt = _c(tri_table, np.int8)
    nv, ni = C.c_uint32(0), C.c_uint32(0)
    lib().n2o_marching_cubes(mn, mx, r, C.c_float(thresh), _p(sdf), _p(tt), None, None, C.byref(nv), C.byref(ni))
    verts = np.zeros((nv.value, 3), np.float32)
    idx = np.zeros(ni.value, np.uint32)
    lib().n2o_marching_cubes(mn, mx, r, C.c_float(thresh), _p(sdf), _p(tt), _p(verts), _p(idx), C.byref(nv), C.byref(ni))
    return verts, idx


def marching_cubes_slab(sdf_slab, res, z0, nz, tri_table, thresh=0.0, aabb_min=(0, 0, 0), aabb_max=(1, 1, 1)):
    """Layers z0 .. z0+nz-1 of a res grid.  Returns (verts, indices, nv_before_last_layer, nv_first_layer)."""
    sdf = _c(sdf_slab, np.float32)
    r = (C.c_uint32 * 3)(*res)
    mn = (C.c_float * 3)(*aabb_min)
    mx = (C.c_float * 3)(*aabb_max)
    tt = _c(tri_table, np.int8)
    cnt = (C.c_uint32 * 4)()
    lib().n2o_marching_cubes_slab(mn, mx, r, C.c_uint32(z0), C.c_uint32(nz), C.c_float(thresh), _p(sdf), _p(tt), None, None, cnt)
    verts = np.zeros((cnt[0], 3), np.float32)
    idx = np.zeros(cnt[1], np.uint32)
    lib().n2o_marching_cubes_slab(mn, mx, r, C.c_uint32(z0), C.c_uint32(nz), C.c_float(thresh), _p(sdf), _p(tt), _p(verts), _p(idx), cnt)
    return verts, idx, int(cnt[2]), int(cnt[3])


def ld_random_val(index, seed):
    return float(lib().n2o_ld_random_val(C.c_uint32(index), C.c_uint32(seed)))


def render_cfg(width, height, focal_length, camera, screen_center=(0.5, 0.5), pixel_offset=(0.5, 0.5), sample_index=0,
               aabb_min=(0.0, 0.0, 0.0), aabb_max=(1.0, 1.0, 1.0), cone_angle_constant=0.0, min_transmittance=0.01,
               cos_anneal_ratio=1.0, linear_colors=False, max_steps=0):
    """camera: 3x4 camera-to-world, camera[i][j] = row i, column j."""
    cam = np.asarray(camera, dtype=np.float32).reshape(3, 4)
    return RenderCfg(width, height, (C.c_float * 2)(*focal_length), (C.c_float * 2)(*screen_center),
                     (C.c_float * 12)(*cam.T.reshape(-1).tolist()), (C.c_float * 2)(*pixel_offset), sample_index,
                     (C.c_float * 3)(*aabb_min), (C.c_float * 3)(*aabb_max), cone_angle_constant, min_transmittance,
                     cos_anneal_ratio, 1 if linear_colors else 0, max_steps)


def render_march(cfg, bitfield, want_coords=True):
    """Every pixel's whole march: (numsteps [h*w], coords [n][7] or None, n)."""
    n_pix = cfg.width * cfg.height
    numsteps = np.zeros(n_pix, np.uint32)
    n = C.c_uint64(0)
    bf = _c(bitfield, np.uint8)
    lib().n2o_render_march(C.byref(cfg), _p(bf), C.c_uint64(0), _p(numsteps), None, C.byref(n))
    if not want_coords:
        return numsteps, None, int(n.value)
    coords = np.zeros((max(int(n.value), 1), 7), np.float32)
    lib().n2o_render_march(C.byref(cfg), _p(bf), C.c_uint64(coords.shape[0]), _p(numsteps), _p(coords), C.byref(n))
    return numsteps, coords[:int(n.value)], int(n.value)


def render_frame(d, params, cfg, bitfield, sdf_bias=-0.1, frame=None):
    """(frame [h][w][4], depth [h][w], samples the rounds evaluated)."""
    h, w = cfg.height, cfg.width
    frame = np.zeros((h, w, 4), np.float32) if frame is None else _c(frame, np.float32)
    depth = np.zeros((h, w), np.float32)
    n = C.c_uint64(0)
    lib().n2o_render_frame(C.byref(d), _p(_c(params, np.uint16)), C.c_float(sdf_bias), C.byref(cfg), _p(_c(bitfield, np.uint8)),
                           _p(frame), _p(depth), C.byref(n))
    return frame, depth, int(n.value)


def render_accumulate(frame, acc, sample_count):
    frame = _c(frame, np.float32)
    lib().n2o_render_accumulate(C.c_uint32(frame.size // 4), _p(frame), _p(acc), C.c_uint32(sample_count))


def render_tonemap(acc, exposure=0.0, background=(0.0, 0.0, 0.0, 0.0), to_srgb=True):
    acc = _c(acc, np.float32)
    out = np.empty_like(acc)
    lib().n2o_render_tonemap(C.c_uint32(acc.size // 4), _p(acc), C.c_float(exposure), (C.c_float * 4)(*background), C.c_int(int(to_srgb)),
                             _p(out))
    return out


def mesh_1ring(verts, indices):
    """(normals [n][3], ring [n][4])"""
    v = _c(verts, np.float32)
    idx = _c(indices, np.uint32)
    normals = np.zeros((v.shape[0], 3), np.float32)
    ring = np.zeros((v.shape[0], 4), np.float32)
    lib().n2o_mesh_1ring(C.c_uint32(v.shape[0]), _p(v), C.c_uint32(idx.size), _p(idx), _p(ring), _p(normals))
    return normals, ring


def mesh_vertex_colors(d, params, verts, sdf_bias=-0.1, linear_colors=False, aabb_min=(0, 0, 0), aabb_max=(1, 1, 1)):
    v = _c(verts, np.float32)
    colors = np.zeros((v.shape[0], 3), np.float32)
    lib().n2o_mesh_vertex_colors(C.byref(d), _p(_c(params, np.uint16)), C.c_float(sdf_bias), C.c_uint32(v.shape[0]), _p(v),
                                 (C.c_float * 3)(*aabb_min), (C.c_float * 3)(*aabb_max), C.c_int(int(linear_colors)), _p(colors))
    return colors


def save_mesh(path, verts, normals, colors, indices, nerf_scale=1.0, nerf_offset=(0.0, 0.0, 0.0), invert_normals=False):
    v, n, c = _c(verts, np.float32), _c(normals, np.float32), _c(colors, np.float32)
    idx = _c(indices, np.uint32)
    rc = lib().n2o_save_mesh(str(path).encode(), C.c_uint32(v.shape[0]), _p(v), _p(n), _p(c), C.c_uint32(idx.size), _p(idx),
                             C.c_float(nerf_scale), (C.c_float * 3)(*nerf_offset), C.c_int(int(invert_normals)))
    if rc != 0:
        raise OSError(f"n2o_save_mesh({path}) failed")
