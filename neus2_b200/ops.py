"""Tensor-level wrappers over the C ABI (torch is only the owner of device memory and streams)."""
import ctypes as C

import torch

from . import _lib as L

u32 = C.c_uint32
_H = torch.float16


def _half(shape, dev):
    return torch.empty(shape, dtype=_H, device=dev)


def grid_forward(d, x, grid, want_dydx=False):
    n, W = x.shape[0], 2 * d.n_levels
    enc = _half((n, W), x.device)
    dydx = torch.empty((n, W, 3), dtype=torch.float32, device=x.device) if want_dydx else None
    L.check(L.lib().neus2b_grid_forward(C.byref(d), u32(n), L.ptr(x), u32(x.shape[1]), L.ptr(grid), L.ptr(enc), L.ptr(dydx),
                                        L.cur_stream()))
    return (enc, dydx) if want_dydx else enc


def grid_backward_input(d, x, grid, dL_denc):
    out = torch.empty((x.shape[0], 3), dtype=torch.float32, device=x.device)
    L.check(L.lib().neus2b_grid_backward_input(C.byref(d), u32(x.shape[0]), L.ptr(x), u32(x.shape[1]), L.ptr(grid),
                                               L.ptr(dL_denc), L.ptr(out), L.cur_stream()))
    return out


def grid_backward_params(d, x, dL_denc, grad, mode=L.GRAD_ACCUMULATE):
    L.check(L.lib().neus2b_grid_backward_params(C.byref(d), u32(x.shape[0]), L.ptr(x), u32(x.shape[1]), L.ptr(dL_denc),
                                                L.ptr(grad), C.c_int(mode), L.cur_stream()))
    return grad


def grid_backward_backward_input(d, x, grid, v, g_e, grad, mode=L.GRAD_ACCUMULATE):
    dy = _half((x.shape[0], 2 * d.n_levels), x.device)
    L.check(L.lib().neus2b_grid_backward_backward_input(C.byref(d), u32(x.shape[0]), L.ptr(x), u32(x.shape[1]), L.ptr(grid),
                                                        L.ptr(v), L.ptr(g_e), L.ptr(dy), L.ptr(grad), C.c_int(mode),
                                                        L.cur_stream()))
    return dy


def mlp_forward(in_w, n_hidden, w, inp):
    n = inp.shape[0]
    out = _half((n, 16), inp.device)
    hidden = _half((n, n_hidden, 64), inp.device)
    L.check(L.lib().neus2b_mlp_forward(u32(n), u32(in_w), u32(n_hidden), L.ptr(w), L.ptr(inp), L.ptr(out), L.ptr(hidden),
                                       L.cur_stream()))
    return out, hidden


def mlp_forward_tcgen05(in_w, n_hidden, w, inp):
    n = inp.shape[0]
    out = _half((n, 16), inp.device)
    hidden = _half((n, n_hidden, 64), inp.device)
    status = torch.zeros(1, dtype=torch.int32, device=inp.device)
    L.check(L.lib().neus2b_mlp_forward_tcgen05(u32(n), u32(in_w), u32(n_hidden), L.ptr(w), L.ptr(inp), L.ptr(out), L.ptr(hidden),
                                               L.ptr(status), L.cur_stream()))
    return out, hidden, status


def mlp_backward(in_w, n_hidden, w, inp, hidden, dL_dout, wgrad=None, mode=L.GRAD_OVERWRITE, want_din=True):
    n = inp.shape[0]
    din = _half((n, in_w), inp.device) if want_din else None
    if wgrad is None and mode != L.GRAD_IGNORE:
        wgrad = torch.zeros(64 * in_w + (n_hidden - 1) * 4096 + 1024, dtype=torch.float32, device=inp.device)
    L.check(L.lib().neus2b_mlp_backward(u32(n), u32(in_w), u32(n_hidden), L.ptr(w), L.ptr(inp), L.ptr(hidden), L.ptr(dL_dout),
                                        L.ptr(din), L.ptr(wgrad), C.c_int(mode), L.cur_stream()))
    return din, wgrad


def mlp_backward_backward_input(in_w, w, hidden, u, dy, wgrad=None, mode=L.GRAD_OVERWRITE):
    if wgrad is None:
        wgrad = torch.zeros(64 * in_w + 1024, dtype=torch.float32, device=u.device)
    L.check(L.lib().neus2b_mlp_backward_backward_input(u32(u.shape[0]), u32(in_w), L.ptr(w), L.ptr(hidden), L.ptr(u), L.ptr(dy),
                                                       L.ptr(wgrad), C.c_int(mode), L.cur_stream()))
    return wgrad


def sh4(dir01):
    out = _half((dir01.shape[0], 16), dir01.device)
    L.check(L.lib().neus2b_sh4_forward(u32(dir01.shape[0]), L.ptr(dir01), u32(dir01.shape[1]), L.ptr(out), L.cur_stream()))
    return out


def neus_forward(d, params, coords, sdf_bias=-0.1, n_dev=None, out=None):
    n = coords.shape[0]
    if out is None:
        out = _half((n, 16), coords.device)
    L.check(L.lib().neus2b_neus_forward(C.byref(d), L.ptr(params), C.c_float(sdf_bias), u32(n), L.ptr(n_dev), L.ptr(coords),
                                        L.ptr(out), L.cur_stream()))
    return out


def neus_train(d, params, coords, dL_dout, indeed_batch_size, grad_mlp, grad_grid, grad_var):
    L.check(L.lib().neus2b_neus_train(C.byref(d), L.ptr(params), u32(coords.shape[0]), L.ptr(coords), L.ptr(dL_dout),
                                      u32(indeed_batch_size), L.ptr(grad_mlp), L.ptr(grad_grid), L.ptr(grad_var), L.cur_stream()))


def neus_sdf(d, params, x, sdf_bias=-0.1, motion=None):
    out = _half((x.shape[0],), x.device)
    L.check(L.lib().neus2b_neus_sdf_moved(C.byref(d), L.ptr(params), C.c_float(sdf_bias), u32(x.shape[0]), L.ptr(x), u32(x.shape[1]),
                                          C.byref(motion) if motion is not None else None, L.ptr(out), L.cur_stream()))
    return out


# ------------------------------------------------------------------------------------------------ dynamic sequences
DELTA_IDENTITY = (0.0, 0.0, 0.0, 0.0, 1.0, 0.0, 0.0, 0.0, 1.0, 0.0, 0.0, 0.0)  # transition (4) | 6-D rotation (8)


def motion(delta, sums=None, first_frame_offset=(0.0, 0.0, 0.0)):
    """neus2b_motion over `delta` (fp16 CUDA tensor [12]) and, for training, the fp32 [12] tensor the backward's sums are added to."""
    m = L.Motion()
    m.d_delta = delta.data_ptr() if hasattr(delta, "data_ptr") else int(delta)
    m.first_frame_offset[:] = list(first_frame_offset)
    m.d_sums = (sums.data_ptr() if hasattr(sums, "data_ptr") else int(sums)) if sums is not None else None
    m._keep = (delta, sums)
    return m


def neus_forward_moved(d, params, coords, mot, sdf_bias=-0.1, n_dev=None, out=None):
    n = coords.shape[0]
    if out is None:
        out = _half((n, 16), coords.device)
    L.check(L.lib().neus2b_neus_forward_moved(C.byref(d), L.ptr(params), C.c_float(sdf_bias), u32(n), L.ptr(n_dev), L.ptr(coords),
                                              C.byref(mot) if mot is not None else None, L.ptr(out), L.cur_stream()))
    return out


def neus_train_moved(d, params, coords, mot, dL_dout, indeed_batch_size, grad_mlp, grad_grid, grad_var):
    L.check(L.lib().neus2b_neus_train_moved(C.byref(d), L.ptr(params), u32(coords.shape[0]), L.ptr(coords),
                                            C.byref(mot) if mot is not None else None, L.ptr(dL_dout), u32(indeed_batch_size),
                                            L.ptr(grad_mlp), L.ptr(grad_grid), L.ptr(grad_var), L.cur_stream()))


def delta_forward(delta, coords, first_frame_offset=(0.0, 0.0, 0.0)):
    out = torch.empty_like(coords)
    L.check(L.lib().neus2b_delta_forward(L.ptr(delta), (C.c_float * 3)(*first_frame_offset), u32(coords.shape[0]), L.ptr(coords), L.ptr(out),
                                         L.cur_stream()))
    return out


def delta_backward(delta, coords, dL_dx, sums=None):
    if sums is None:
        sums = torch.zeros(12, dtype=torch.float32, device=coords.device)
    L.check(L.lib().neus2b_delta_backward(L.ptr(delta), u32(coords.shape[0]), L.ptr(coords), L.ptr(dL_dx), L.ptr(sums), L.cur_stream()))
    return sums


def delta_gradient(delta, sums):
    """The 12 parameters' gradients from the backward's sums (the sums are cleared)."""
    g = torch.zeros(12, dtype=torch.float32, device=sums.device)
    L.check(L.lib().neus2b_delta_optimizer_step(None, L.ptr(sums), None, None, None, L.ptr(delta), None, None, L.ptr(g), L.cur_stream()))
    return g


def delta_optimizer_step(cfg, sums, master, m, v, delta, delta_ema=None, ema_master=None, grad_out=None):
    L.check(L.lib().neus2b_delta_optimizer_step(C.byref(cfg), L.ptr(sums), L.ptr(master), L.ptr(m), L.ptr(v), L.ptr(delta), L.ptr(delta_ema),
                                                L.ptr(ema_master), L.ptr(grad_out), L.cur_stream()))


def movement_accumulate(delta_bits, rotation, transition):
    """Host: (rotation [9] row-major, transition [3]) with the frame's motion (12 fp16 bit patterns) folded in."""
    import numpy as np
    R = (C.c_float * 9)(*[float(v) for v in np.asarray(rotation, np.float32).reshape(9)])
    t = (C.c_float * 3)(*[float(v) for v in np.asarray(transition, np.float32).reshape(3)])
    d = (C.c_uint16 * 12)(*[int(v) for v in np.asarray(delta_bits).reshape(12)])
    L.check(L.lib().neus2b_movement_accumulate(d, R, t))
    return np.array(list(R), np.float32).reshape(3, 3), np.array(list(t), np.float32)


class RayBatch:
    """Device scratch of one ray batch (neus2b_ray_workspace) plus the dataset handle."""

    def __init__(self, max_rays, max_samples, device="cuda", march_masks=True, occupied_bounds=None):
        self.max_rays, self.max_samples = max_rays, max_samples
        i32, f32 = torch.int32, torch.float32
        self.ray_indices = torch.zeros(max_rays, dtype=i32, device=device)
        self.rays = torch.zeros((max_rays, 6), dtype=f32, device=device)
        self.numsteps = torch.zeros((max_rays, 2), dtype=i32, device=device)
        self.coords = torch.zeros((max_samples, 7), dtype=f32, device=device)
        self.counters = torch.zeros(8, dtype=i32, device=device)
        self.scan_tmp = torch.zeros(max_rays + 1024, dtype=torch.int64, device=device)
        self.ray_tmp = torch.zeros((max_rays, 8), dtype=f32, device=device)
        self.march_masks = torch.zeros((max_rays, 64), dtype=i32, device=device) if march_masks else None
        self.window_list = torch.zeros(max_samples, dtype=i32, device=device)
        self.window_lens = torch.zeros(8, dtype=i32, device=device)
        self.ws = L.RayWorkspace(max_rays, max_samples, L.ptr(self.ray_indices), L.ptr(self.rays), L.ptr(self.numsteps),
                                 L.ptr(self.coords), L.ptr(self.counters), L.ptr(self.scan_tmp), L.ptr(self.ray_tmp), None,
                                 L.ptr(self.march_masks), L.ptr(occupied_bounds), L.ptr(self.window_list), L.ptr(self.window_lens))
        self.occupied_bounds = occupied_bounds


def make_dataset(pixels, xforms, focal, principal):
    """pixels int32/uint8x4 [n][H][W] (RGBA8 packed), xforms [n][12], focal/principal [n][2], all CUDA tensors."""
    ds = L.Dataset(pixels.shape[0], pixels.shape[2], pixels.shape[1], L.ptr(pixels), L.ptr(xforms), L.ptr(focal), L.ptr(principal))
    ds._keep = (pixels, xforms, focal, principal)
    return ds


def generate_samples(ds, cfg, n_rays, n_rays_total, rng, bitfield, batch, n_rays_dev=None):
    L.check(L.lib().neus2b_generate_samples(C.byref(ds), C.byref(cfg), u32(n_rays), L.ptr(n_rays_dev), u32(n_rays_total), rng,
                                            L.ptr(bitfield), C.byref(batch.ws), L.cur_stream()))


def generate_samples_static(ds, cfg, n_rays, n_rays_total, rng, bitfield, max_samples, ray_indices, rays, numsteps, coords,
                            counters, n_rays_dev=None):
    """neus2b_generate_samples_static: same outputs, scratch inside the library (no allocation; at most
    NEUS2B_STATIC_MAX_RAYS rays)."""
    L.check(L.lib().neus2b_generate_samples_static(C.byref(ds), C.byref(cfg), u32(n_rays), L.ptr(n_rays_dev), u32(n_rays_total),
                                                   rng, L.ptr(bitfield), u32(max_samples), L.ptr(ray_indices), L.ptr(rays),
                                                   L.ptr(numsteps), L.ptr(coords), L.ptr(counters), L.cur_stream()))


def compute_loss(ds, cfg, n_rays, n_rays_total, rng, max_compacted, mlp_out, batch, coords_out, dloss, loss=None, ek_loss=None,
                 rollover=True, n_rays_dev=None):
    L.check(L.lib().neus2b_compute_loss(C.byref(ds), C.byref(cfg), u32(n_rays), L.ptr(n_rays_dev), u32(n_rays_total), rng,
                                        u32(max_compacted), L.ptr(mlp_out), C.byref(batch.ws), L.ptr(coords_out), L.ptr(dloss),
                                        L.ptr(loss), L.ptr(ek_loss), C.c_int(int(rollover)), L.cur_stream()))


def forward_compute_loss(desc, params, ds, cfg, n_rays, n_rays_total, rng, max_compacted, batch, mlp_out, coords_out, dloss, loss=None,
                         ek_loss=None, window_ends=(32, 96), rollover=True, sdf_bias=-0.1, motion=None, n_rays_dev=None):
    """neus2b_forward_compute_loss: the network pass over the batch's samples in windows per ray plus the loss pass.  window_ends ():
    every sample, like neus_forward followed by compute_loss."""
    ends = (C.c_uint32 * max(1, len(window_ends)))(*window_ends)
    L.check(L.lib().neus2b_forward_compute_loss(C.byref(desc), L.ptr(params), C.c_float(sdf_bias), C.byref(motion) if motion is not None else None,
                                                C.byref(ds), C.byref(cfg), u32(n_rays), L.ptr(n_rays_dev), u32(n_rays_total), rng, u32(max_compacted),
                                                C.byref(batch.ws), ends, u32(len(window_ends)), L.ptr(mlp_out), L.ptr(coords_out), L.ptr(dloss),
                                                L.ptr(loss), L.ptr(ek_loss), C.c_int(int(rollover)), L.cur_stream()))


class OccupancyGrid:
    def __init__(self, n_cascades=1, max_samples=128 ** 3, device="cuda"):
        cells = 128 ** 3
        self.n_cascades = n_cascades
        self.grid = torch.zeros(cells * n_cascades, dtype=torch.float32, device=device)
        self.grid_tmp = torch.zeros_like(self.grid)
        self.bitfield = torch.zeros(cells, dtype=torch.uint8, device=device)
        self.mean = torch.zeros(1, dtype=torch.float32, device=device)
        self.pos = torch.zeros((max_samples, 3), dtype=torch.float32, device=device)
        self.idx = torch.zeros(max_samples, dtype=torch.int32, device=device)
        self.sdf = torch.zeros(max_samples, dtype=_H, device=device)
        self.partial = torch.zeros(1024, dtype=torch.float64, device=device)
        self.ema_step = 0

    def update(self, d, params, n_uniform, n_nonuniform, rng_u, rng_nu, decay=0.95, sdf_bias=-0.1):
        L.check(L.lib().neus2b_occupancy_update(C.byref(d), L.ptr(params), C.c_float(sdf_bias), u32(self.n_cascades),
                                                u32(n_uniform), u32(n_nonuniform), rng_u, rng_nu, u32(self.ema_step),
                                                C.c_float(decay), L.ptr(self.grid), L.ptr(self.grid_tmp), L.ptr(self.bitfield),
                                                L.ptr(self.mean), L.ptr(self.pos), L.ptr(self.idx), L.ptr(self.sdf),
                                                L.ptr(self.partial), L.cur_stream()))
        self.ema_step += 1


def adam_step(cfg, grad_mlp, grad_grid, grad_var, master, m, v, params, params_ema=None, ema_master=None):
    L.check(L.lib().neus2b_adam_step(C.byref(cfg), C.c_uint64(master.numel()), L.ptr(grad_mlp), L.ptr(grad_grid), L.ptr(grad_var),
                                     L.ptr(master), L.ptr(m), L.ptr(v), L.ptr(params), L.ptr(params_ema), L.ptr(ema_master),
                                     L.cur_stream()))


def adam_step_packed(cfg, grad_mlp, grad_grid, grad_var, state, params, params_ema=None):
    """state: float32 [n][4] = {master, m, v, ema master}."""
    L.check(L.lib().neus2b_adam_step_packed(C.byref(cfg), C.c_uint64(state.shape[0]), L.ptr(grad_mlp), L.ptr(grad_grid),
                                            L.ptr(grad_var), L.ptr(state), L.ptr(params), L.ptr(params_ema), L.cur_stream()))


def marching_cubes(sdf, tri_table=None, thresh=0.0, aabb_min=(0.0, 0.0, 0.0), aabb_max=(1.0, 1.0, 1.0)):
    """sdf: float32 CUDA tensor [rz][ry][rx].  Returns (verts [n][3] float32, indices [m] int32) in canonical order.
    tri_table: int8 [256][16] case table (defaults to the generated one of neus2_b200.mc_table)."""
    if tri_table is None:
        from .mc_table import make_table
        tri_table = torch.from_numpy(make_table())
    tt = tri_table.to(device=sdf.device, dtype=torch.int8).contiguous()
    rz, ry, rx = sdf.shape
    res = (C.c_uint32 * 3)(rx, ry, rz)
    mn, mx = (C.c_float * 3)(*aabb_min), (C.c_float * 3)(*aabb_max)
    nb = C.c_uint64(0)
    L.check(L.lib().neus2b_marching_cubes_scratch_bytes(res, C.byref(nb)))
    scratch = torch.empty(nb.value // 8, dtype=torch.int64, device=sdf.device)
    counts = torch.zeros(2, dtype=torch.int32, device=sdf.device)
    L.check(L.lib().neus2b_marching_cubes(mn, mx, res, C.c_float(thresh), L.ptr(sdf), L.ptr(tt), L.ptr(scratch), None, u32(0), None,
                                          u32(0), L.ptr(counts), L.cur_stream()))
    nv, ni = [int(v) for v in counts.cpu()]
    verts = torch.empty((max(nv, 1), 3), dtype=torch.float32, device=sdf.device)
    idx = torch.empty(max(ni, 1), dtype=torch.int32, device=sdf.device)
    L.check(L.lib().neus2b_marching_cubes(mn, mx, res, C.c_float(thresh), L.ptr(sdf), L.ptr(tt), L.ptr(scratch), L.ptr(verts), u32(nv),
                                          L.ptr(idx), u32(ni), L.ptr(counts), L.cur_stream()))
    return verts[:nv], idx[:ni]


def marching_cubes_slab(sdf_slab, res, z0, tri_table=None, thresh=0.0, aabb_min=(0.0, 0.0, 0.0), aabb_max=(1.0, 1.0, 1.0)):
    """One z-slab of a res = (rx, ry, rz) lattice: sdf_slab float32 CUDA tensor [n_layers][ry][rx] = layers z0 .. z0+n_layers-1.
    Returns a part for neus2_b200.mesh_shard.merge_slab_meshes (host arrays)."""
    if tri_table is None:
        from .mc_table import make_table
        tri_table = torch.from_numpy(make_table())
    tt = tri_table.to(device=sdf_slab.device, dtype=torch.int8).contiguous()
    nl = sdf_slab.shape[0]
    r = (C.c_uint32 * 3)(*[int(v) for v in res])
    r_slab = (C.c_uint32 * 3)(int(res[0]), int(res[1]), nl)
    mn, mx = (C.c_float * 3)(*aabb_min), (C.c_float * 3)(*aabb_max)
    nb = C.c_uint64(0)
    L.check(L.lib().neus2b_marching_cubes_scratch_bytes(r_slab, C.byref(nb)))
    scratch = torch.empty(nb.value // 8, dtype=torch.int64, device=sdf_slab.device)
    counts = torch.zeros(4, dtype=torch.int32, device=sdf_slab.device)
    args = (mn, mx, r, u32(z0), u32(nl), C.c_float(thresh), L.ptr(sdf_slab), L.ptr(tt), L.ptr(scratch))
    L.check(L.lib().neus2b_marching_cubes_slab(*args, None, u32(0), None, u32(0), L.ptr(counts), L.cur_stream()))
    nv, ni, nbl, nf = [int(v) for v in counts.cpu()]
    verts = torch.empty((max(nv, 1), 3), dtype=torch.float32, device=sdf_slab.device)
    idx = torch.empty(max(ni, 1), dtype=torch.int32, device=sdf_slab.device)
    L.check(L.lib().neus2b_marching_cubes_slab(*args, L.ptr(verts), u32(nv), L.ptr(idx), u32(ni), L.ptr(counts), L.cur_stream()))
    return dict(verts=verts[:nv].cpu().numpy(), indices=idx[:ni].cpu().numpy().view("uint32"), nv_before_last=nbl, nv_first=nf)


class SlabGlobal:
    """neus2b_marching_cubes_slab_global in its two passes: `count()` -> (ids referred to, indices written, vertices owned) on the
    device, then `emit(vertex_offset)` -> (verts [owned][3], indices [n]) CUDA tensors with global vertex ids."""

    def __init__(self, sdf_slab, res, z0, n_layers, halo, tri_table=None, thresh=0.0, aabb_min=(0.0, 0.0, 0.0), aabb_max=(1.0, 1.0, 1.0)):
        if tri_table is None:
            from .mc_table import make_table
            tri_table = torch.from_numpy(make_table())
        assert sdf_slab.shape[0] == n_layers + halo and sdf_slab.is_contiguous()
        self.dev = sdf_slab.device
        self.sdf, self.tt = sdf_slab, tri_table.to(device=self.dev, dtype=torch.int8).contiguous()
        r_slab = (C.c_uint32 * 3)(int(res[0]), int(res[1]), n_layers + halo)
        nb = C.c_uint64(0)
        L.check(L.lib().neus2b_marching_cubes_scratch_bytes(r_slab, C.byref(nb)))
        self.scratch = torch.empty(nb.value // 8, dtype=torch.int64, device=self.dev)
        self.counts = torch.zeros(4, dtype=torch.int32, device=self.dev)
        self.args = ((C.c_float * 3)(*aabb_min), (C.c_float * 3)(*aabb_max), (C.c_uint32 * 3)(*[int(v) for v in res]), u32(z0),
                     u32(n_layers), u32(halo), C.c_float(thresh), L.ptr(self.sdf), L.ptr(self.tt), L.ptr(self.scratch))

    def count(self):
        L.check(L.lib().neus2b_marching_cubes_slab_global(*self.args, None, u32(0), None, u32(0), u32(0), L.ptr(self.counts), L.cur_stream()))
        return self.counts

    def emit(self, vertex_offset, n_owned, n_indices):
        verts = torch.empty((max(n_owned, 1), 3), dtype=torch.float32, device=self.dev)
        idx = torch.empty(max(n_indices, 1), dtype=torch.int32, device=self.dev)
        L.check(L.lib().neus2b_marching_cubes_slab_global(*self.args, L.ptr(verts), u32(n_owned), L.ptr(idx), u32(n_indices), u32(vertex_offset),
                                                          L.ptr(self.counts), L.cur_stream()))
        return verts[:n_owned], idx[:n_indices]


def occupancy_bounds(bitfield):
    """int32[6] CUDA tensor {min x, y, z, max x, y, z} of the occupied cells of the finest level."""
    out = torch.zeros(8, dtype=torch.int32, device=bitfield.device)
    L.check(L.lib().neus2b_occupancy_bounds(L.ptr(bitfield), L.ptr(out), L.cur_stream()))
    return out


# ------------------------------------------------------------------------------------------------ inference rendering

def _owen_scramble(x, seed):
    def rev(v):
        return int(f"{v & 0xffffffff:032b}"[::-1], 2)
    x = (rev(x) + seed) & 0xffffffff
    for m in (0x6c50b47c, 0xb82f1e52, 0xc7afe638, 0x8d22f6e6):
        x ^= (x * m) & 0xffffffff
    return rev(x)


def _sobol(index, dim):
    """Sobol point (32-bit) of `index` in dimension 0 or 1: direction numbers 2^(31-k) and, for dimension 1 (primitive
    polynomial x + 1), v_k = v_(k-1) xor (v_(k-1) >> 1)."""
    v, x = 0x80000000, 0
    for bit in range(32):
        if (index >> bit) & 1:
            x ^= v
        v = (v >> 1) if dim == 0 else (v ^ (v >> 1))
    return x


def ld_random_val_2d(index, seed):
    """ld_random_val_2d (include/neural-graphics-primitives/random_val.cuh:278-282): a 2-D point of the Owen-scrambled Sobol
    sequence (Burley 2020)."""
    import numpy as np
    index = _owen_scramble(index, seed)
    out = []
    for dim in range(2):
        sd = (seed ^ ((dim + ((seed << 6) & 0xffffffff) + (seed >> 2)) & 0xffffffff)) & 0xffffffff
        out.append(np.float32(_owen_scramble(_sobol(index, dim), sd)) * np.float32(1.0 / 4294967296.0))
    return out


def ld_random_pixel_offset(spp):
    """ld_random_pixel_offset (random_val.cuh:317-322): where inside its pixel the spp-th sample of every pixel lies."""
    import numpy as np
    a, b = ld_random_val_2d(0, 0xdeadbeef), ld_random_val_2d(spp, 0xdeadbeef)
    off = [np.float32(0.5) - a[e] + b[e] for e in range(2)]
    return [float(o - np.floor(o)) for o in off]


class RenderBuffers:
    """Scratch of the renderer for up to max_rays pixels and max_samples samples at a time (neus2b_render_workspace)."""

    def __init__(self, max_rays, max_samples, device="cuda", occupied_bounds=None, masks=False):
        max_samples = (int(max_samples) + 127) // 128 * 128
        self.ray_tmp = torch.empty((max_rays, 8), dtype=torch.float32, device=device)
        self.scan_tmp = torch.zeros(max_rays + 1024, dtype=torch.int64, device=device)
        self.state = torch.empty((max_rays, 8), dtype=torch.float32, device=device)
        self.hit_list = torch.empty(max_rays, dtype=torch.int32, device=device)
        self.coords = torch.empty((max_samples, 7), dtype=torch.float32, device=device)
        self.out = torch.empty((max_samples, 16), dtype=torch.float16, device=device)
        self.counters = torch.zeros(8, dtype=torch.int32, device=device)
        self.occupied_bounds = occupied_bounds
        self.masks = torch.empty((max_rays, 64), dtype=torch.int32, device=device) if masks else None
        self.ws = L.RenderWorkspace(u32(max_rays), u32(max_samples), L.ptr(self.ray_tmp), L.ptr(self.scan_tmp), L.ptr(self.state),
                                    L.ptr(self.hit_list), L.ptr(self.coords), L.ptr(self.out), L.ptr(self.counters),
                                    L.ptr(occupied_bounds), L.ptr(self.masks))


def render_cfg(width, height, focal_length, camera, screen_center=(0.5, 0.5), pixel_offset=(0.5, 0.5), sample_index=0,
               aabb_min=(0.0, 0.0, 0.0), aabb_max=(1.0, 1.0, 1.0), cone_angle_constant=0.0, min_transmittance=0.01,
               cos_anneal_ratio=1.0, linear_colors=False, max_steps=0):
    """camera: 3x4 camera-to-world (array-like, row i column j = camera[i][j])."""
    import numpy as np
    cam = np.asarray(camera, dtype=np.float32).reshape(3, 4)
    return L.RenderCfg(u32(width), u32(height), (C.c_float * 2)(*focal_length), (C.c_float * 2)(*screen_center),
                       (C.c_float * 12)(*cam.T.reshape(-1).tolist()), (C.c_float * 2)(*pixel_offset), u32(sample_index),
                       (C.c_float * 3)(*aabb_min), (C.c_float * 3)(*aabb_max), C.c_float(cone_angle_constant),
                       C.c_float(min_transmittance), C.c_float(cos_anneal_ratio), u32(1 if linear_colors else 0), u32(max_steps))


def render_frame(desc, params, sdf_bias, cfg, bitfield, buffers, frame, depth):
    """neus2b_render_frame: blends one sample per pixel into frame [h][w][4] (float32 CUDA) and writes depth [h][w].
    Returns the number of samples that went through the network."""
    n = C.c_uint64(0)
    L.check(L.lib().neus2b_render_frame(C.byref(desc), L.ptr(params), C.c_float(sdf_bias), C.byref(cfg), L.ptr(bitfield),
                                        C.byref(buffers.ws), L.ptr(frame), L.ptr(depth), C.byref(n), L.cur_stream()))
    return int(n.value)


def render_accumulate(frame, accumulate, sample_count):
    L.check(L.lib().neus2b_render_accumulate(u32(frame.numel() // 4), L.ptr(frame), L.ptr(accumulate), u32(sample_count), L.cur_stream()))


def render_tonemap(accumulate, exposure=0.0, background=(0.0, 0.0, 0.0, 0.0), to_srgb=True):
    out = torch.empty_like(accumulate)
    L.check(L.lib().neus2b_render_tonemap(u32(accumulate.numel() // 4), L.ptr(accumulate), C.c_float(exposure),
                                          (C.c_float * 4)(*background), C.c_int(1 if to_srgb else 0), L.ptr(out), L.cur_stream()))
    return out


# ------------------------------------------------------------------------------------------------ mesh post-processing

def mesh_1ring(verts, indices, want_ring=False):
    """Area-weighted vertex normals [n][3] (not normalised) and, if asked, the homogeneous 1-ring sums [n][4]."""
    n = verts.shape[0]
    normals = torch.empty((n, 3), dtype=torch.float32, device=verts.device)
    ring = torch.empty((n, 4), dtype=torch.float32, device=verts.device) if want_ring else None
    L.check(L.lib().neus2b_mesh_1ring(u32(n), L.ptr(verts), u32(indices.numel()), L.ptr(indices), L.ptr(ring), L.ptr(normals), L.cur_stream()))
    return (normals, ring) if want_ring else normals


def mesh_vertex_colors(desc, params, sdf_bias, verts, linear_colors=False, aabb_min=(0.0, 0.0, 0.0), aabb_max=(1.0, 1.0, 1.0),
                       chunk=1 << 20):
    n = verts.shape[0]
    colors = torch.empty((n, 3), dtype=torch.float32, device=verts.device)
    chunk = max(128, min(chunk, (n + 127) // 128 * 128))
    coords = torch.empty((chunk, 7), dtype=torch.float32, device=verts.device)
    out = torch.empty((chunk, 16), dtype=torch.float16, device=verts.device)
    L.check(L.lib().neus2b_mesh_vertex_colors(C.byref(desc), L.ptr(params), C.c_float(sdf_bias), u32(n), L.ptr(verts), (C.c_float * 3)(*aabb_min),
                                              (C.c_float * 3)(*aabb_max), C.c_int(int(linear_colors)), L.ptr(coords), L.ptr(out), u32(chunk),
                                              L.ptr(colors), L.cur_stream()))
    return colors


def save_mesh(path, verts, normals, colors, indices, nerf_scale=1.0, nerf_offset=(0.0, 0.0, 0.0), invert_normals=False):
    """Host arrays (numpy) to an .obj or .ply file."""
    import numpy as np
    v = np.ascontiguousarray(verts, dtype=np.float32)
    nr = np.ascontiguousarray(normals, dtype=np.float32)
    c = np.ascontiguousarray(colors, dtype=np.float32)
    idx = np.ascontiguousarray(indices).astype(np.uint32, copy=False)
    p = lambda a: a.ctypes.data_as(C.c_void_p)
    L.check(L.lib().neus2b_save_mesh(str(path).encode(), u32(v.shape[0]), p(v), p(nr), p(c), u32(idx.size), p(idx), C.c_float(nerf_scale),
                                     (C.c_float * 3)(*nerf_offset), C.c_int(int(invert_normals))))
