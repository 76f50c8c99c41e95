"""Host-side mirror of the training subset of the reference's ``pyngp.Testbed`` (src/python_api.cu:317-471) over the
C ABI: ``load_training_data`` / ``train`` / ``frame`` / ``training_step`` / ``loss`` / ``ek_loss`` keep their names and
meaning.  All work happens in libneus2b.so; this class owns nothing but the handle."""
import ctypes as C

import numpy as np

from . import _lib as L


class Testbed:
    def __init__(self, config=None, **overrides):
        cfg = L.TestbedConfig()
        L.lib().neus2b_testbed_default_config(C.byref(cfg))
        if config is not None:
            cfg = config
        for k, v in overrides.items():
            if k in ("n_levels", "log2_hashmap_size", "base_resolution", "per_level_scale", "n_active_levels"):
                setattr(cfg.grid, k, v)
            elif k == "first_frame_offset":
                cfg.first_frame_offset[:] = [float(x) for x in v]
            elif k == "forward_windows":  # cumulative window ends of the step's network pass; () = every sample, like the reference
                cfg.n_forward_windows = len(v)
                for i, e in enumerate(v):
                    cfg.forward_window_ends[i] = int(e)
            else:
                if not hasattr(cfg, k):
                    raise AttributeError(k)
                setattr(cfg, k, v)
        if "n_levels" in overrides and "n_active_levels" not in overrides:
            cfg.grid.n_active_levels = cfg.grid.n_levels
        self.config = cfg
        self._h = C.c_void_p()
        L.check(L.lib().neus2b_testbed_create(C.byref(cfg), C.byref(self._h)))
        self.stats = L.TrainStats()
        self.shall_train = True
        # camera and display state of the reference's Testbed (include/neural-graphics-primitives/testbed.h:489-510, 686, 833)
        self.camera_matrix = np.array([[1, 0, 0, 0.5], [0, -1, 0, 0.5], [0, 0, -1, 0.5]], np.float32)
        self.relative_focal_length = np.ones(2, np.float32)
        self.fov_axis = 1
        self.zoom = 1.0
        self.screen_center = np.array([0.5, 0.5], np.float32)
        self.snap_to_pixel_centers = False
        self.exposure = 0.0
        self.background_color = np.array([0.0, 0.0, 0.0, 1.0], np.float32)
        self.rendering_min_transmittance = 0.01

    @classmethod
    def from_network_config(cls, network_config, aabb_scale=1, **overrides):
        """A testbed configured by one of the reference's network configuration files (configs/nerf/*.json) or the parsed
        dict: what ``Testbed.reload_network_from_file`` (src/python_api.cu:339, src/testbed.cu:2093-2339) sets up."""
        from . import config
        if not isinstance(network_config, dict):
            network_config = config.load_json_with_comments(network_config)
        tb = cls(config=config.testbed_config_from_json(network_config, aabb_scale=aabb_scale), **overrides)
        tb.first_frame_max_training_step, tb.next_frame_max_training_step = config.dynamic_schedule(network_config)
        return tb

    def close(self):
        if getattr(self, "_h", None) and self._h.value:
            L.lib().neus2b_testbed_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # --- data / parameters (HOST arrays in, as the reference's loader hands them over)
    def load_training_data(self, pixels, xforms, focal, principal):
        pixels = np.ascontiguousarray(pixels).view(np.uint32)
        self._cams = [np.ascontiguousarray(a, dtype=np.float32) for a in (xforms, focal, principal)]
        n, h, w = pixels.shape
        L.check(L.lib().neus2b_testbed_load_training_data(self._h, C.c_uint32(n), C.c_uint32(w), C.c_uint32(h),
                                                          pixels.ctypes.data_as(C.c_void_p),
                                                          *[a.ctypes.data_as(C.c_void_p) for a in self._cams]))

    def load_training_data_from_json(self, json_paths):
        """``Testbed.load_training_data(path)`` (src/testbed.cu:155, src/testbed_nerf.cu:2957-2996, src/nerf_loader.cu:197): a
        transforms file, a list of them (one scene), or a directory with one transforms file per frame of a dynamic sequence
        (sorted by name; the first is loaded, ``training_network_next_frame`` moves on).  Images and cameras come through
        ``neus2_b200.loader``.  Returns the loaded dataset description."""
        from . import loader
        import os
        if isinstance(json_paths, (str, os.PathLike)) and os.path.isdir(json_paths):
            self.all_json_paths = loader.list_frame_jsons(json_paths)
            json_paths = self.all_json_paths[0]
        else:
            self.all_json_paths = [json_paths]
        self.all_training_time_frame = len(self.all_json_paths)
        self.current_training_time_frame = 0
        ds = loader.load_nerf_dataset(json_paths)
        if ds["aabb_scale"] != 1 << (int(self.config.n_cascades) - 1):
            raise ValueError(f"the dataset's aabb_scale {ds['aabb_scale']} needs n_cascades = {int(ds['aabb_scale']).bit_length()}")
        self.dataset = ds
        self.load_training_data(ds["pixels"], ds["xforms"], ds["focal"], ds["principal"])
        return ds

    def set_nerf_camera_matrix(self, nerf_matrix):
        """``Testbed.set_nerf_camera_matrix`` (src/python_api.cu:430): a camera in the dataset's own convention."""
        from . import loader
        ds = getattr(self, "dataset", None) or dict(scale=loader.NERF_SCALE, offset=[0.5, 0.5, 0.5], from_na=False, from_mitsuba=False)
        self.camera_matrix = loader.nerf_matrix_to_ngp(nerf_matrix, ds["scale"], ds["offset"], ds["from_na"], ds["from_mitsuba"])

    # --- dynamic sequences
    def next_frame(self, pixels, xforms, focal, principal):
        """``Testbed::training_network_next_frame`` (src/testbed.cu:1991-2072): the next frame's images and cameras (same count and
        size), the learned motion folded into the accumulated one, fresh optimizers, the motion-only phase ahead."""
        pixels = np.ascontiguousarray(pixels).view(np.uint32)
        self._cams = [np.ascontiguousarray(a, dtype=np.float32) for a in (xforms, focal, principal)]
        L.check(L.lib().neus2b_testbed_next_frame(self._h, pixels.ctypes.data_as(C.c_void_p), *[a.ctypes.data_as(C.c_void_p) for a in self._cams]))
        self.stats.training_step = 0

    def movement(self):
        """(frame index, accumulated rotation [3][3], accumulated transition [3], the frame's motion parameters [12])."""
        frame = C.c_uint32(0)
        R, t, d = np.zeros(9, np.float32), np.zeros(3, np.float32), np.zeros(12, np.float32)
        L.check(L.lib().neus2b_testbed_get_movement(self._h, C.byref(frame), R.ctypes.data_as(C.c_void_p), t.ctypes.data_as(C.c_void_p),
                                                    d.ctypes.data_as(C.c_void_p)))
        return int(frame.value), R.reshape(3, 3), t, d

    def set_movement(self, frame, rotation, transition, delta=None):
        R = np.ascontiguousarray(rotation, dtype=np.float32).reshape(9)
        t = np.ascontiguousarray(transition, dtype=np.float32).reshape(3)
        d = np.ascontiguousarray(delta, dtype=np.float32).reshape(12) if delta is not None else None
        L.check(L.lib().neus2b_testbed_set_movement(self._h, C.c_uint32(int(frame)), R.ctypes.data_as(C.c_void_p), t.ctypes.data_as(C.c_void_p),
                                                    d.ctypes.data_as(C.c_void_p) if d is not None else None))

    def update_cameras(self, xforms=None, focal=None, principal=None):
        cams = [np.ascontiguousarray(a, dtype=np.float32) if a is not None else b
                for a, b in zip((xforms, focal, principal), self._cams)]
        L.check(L.lib().neus2b_testbed_update_cameras(self._h, *[a.ctypes.data_as(C.c_void_p) for a in cams]))

    @property
    def n_params(self):
        n = C.c_uint64(0)
        L.check(L.lib().neus2b_testbed_n_params(self._h, C.byref(n)))
        return int(n.value)

    def set_params(self, params_fp32):
        p = np.ascontiguousarray(params_fp32, dtype=np.float32)
        L.check(L.lib().neus2b_testbed_set_params(self._h, p.ctypes.data_as(C.c_void_p), C.c_uint64(p.size)))

    def get_params(self, ema=False):
        p = np.empty(self.n_params, np.float32)
        L.check(L.lib().neus2b_testbed_get_params(self._h, p.ctypes.data_as(C.c_void_p), C.c_uint64(p.size), C.c_int(int(ema))))
        return p

    # --- training
    def train(self, n_steps=1, read_stats=True):
        L.check(L.lib().neus2b_testbed_train(self._h, C.c_uint32(n_steps), C.byref(self.stats) if read_stats else None))
        return self.stats

    def frame(self):
        """One training step, like ``Testbed::frame`` with ``shall_train`` set (src/testbed.cu:1712).  On a dynamic sequence the
        frame is switched first when the current one has had its steps (src/testbed.cu:1739-1746)."""
        if self.shall_train:
            n_frames = getattr(self, "all_training_time_frame", 1)
            if n_frames > 1:
                cur = getattr(self, "current_training_time_frame", 0)
                limit = self.first_frame_max_training_step if cur == 0 else self.next_frame_max_training_step
                if self.stats.training_step >= limit:
                    self.training_network_next_frame()
            self.train(1)
        return True

    first_frame_max_training_step = 2000  # hyperparams of the network configuration (src/testbed.cu:2108-2109)
    next_frame_max_training_step = 1000

    def training_network_next_frame(self):
        """``Testbed::training_network_next_frame`` (src/testbed.cu:1991-2072) for a sequence loaded from a directory of per-frame
        transforms files: loads the next frame's images and cameras and switches to it.  False on the last frame."""
        from . import loader
        cur = getattr(self, "current_training_time_frame", 0)
        if cur >= getattr(self, "all_training_time_frame", 1) - 1:
            return False
        ds = loader.load_nerf_dataset(self.all_json_paths[cur + 1])
        self.dataset = ds
        self.next_frame(ds["pixels"], ds["xforms"], ds["focal"], ds["principal"])
        self.current_training_time_frame = cur + 1
        return True

    def train_backward(self):
        L.check(L.lib().neus2b_testbed_train_backward(self._h))

    def train_pregenerate(self):
        """Draws the next step's samples between train_backward and optimizer_step; False if the next step starts with an
        occupancy update and nothing was done."""
        rc = L.lib().neus2b_testbed_train_pregenerate(self._h)
        if rc not in (0, 1):
            L.check(rc)
        return rc == 0

    def train_step(self, next_cameras=None, read_stats=True):
        """One step with the next step's cameras (three float32 arrays, already contiguous) uploaded and its samples drawn
        before the host waits for this step's statistics."""
        keep = [np.ascontiguousarray(a, dtype=np.float32) for a in next_cameras] if next_cameras is not None else None
        cams = [a.ctypes.data_as(C.c_void_p) for a in keep] if keep else [None, None, None]
        L.check(L.lib().neus2b_testbed_train_step(self._h, *cams, C.byref(self.stats) if read_stats else None))
        return self.stats

    def optimizer_step_async(self):
        """Enqueues the optimizer pass and the copy of the step statistics; `wait_stats` returns them."""
        L.check(L.lib().neus2b_testbed_train_optimizer_step_async(self._h))

    def wait_stats(self):
        L.check(L.lib().neus2b_testbed_train_wait_stats(self._h, C.byref(self.stats)))
        return self.stats

    def optimizer_step(self, read_stats=True):
        L.check(L.lib().neus2b_testbed_train_optimizer_step(self._h, C.byref(self.stats) if read_stats else None))
        return self.stats

    @property
    def training_step(self):
        return int(self.stats.training_step)

    @property
    def loss(self):
        return float(self.stats.loss)

    @property
    def ek_loss(self):
        return float(self.stats.ek_loss)

    # --- device views (torch tensors over the library's buffers; for tests and for NCCL)
    def device_ptrs(self):
        names = ("params", "params_ema", "master", "grad_mlp", "grad_grid", "grad_variance", "bitfield", "density_grid")
        ptrs = [C.c_void_p() for _ in names]
        stream = C.c_void_p()
        L.check(L.lib().neus2b_testbed_device_ptrs(self._h, *[C.byref(p) for p in ptrs], C.byref(stream)))
        out = {k: p.value for k, p in zip(names, ptrs)}
        out["stream"] = stream.value
        return out

    def sdf_grid(self, res, z0=0, z1=None, use_ema=True):
        import torch
        res = [int(r) for r in (res if hasattr(res, "__len__") else (res, res, res))]
        z1 = res[2] if z1 is None else z1
        out = torch.empty((z1 - z0, res[1], res[0]), dtype=torch.float32, device="cuda")
        L.check(L.lib().neus2b_testbed_sdf_grid(self._h, (C.c_uint32 * 3)(*res), C.c_uint32(z0), C.c_uint32(z1), C.c_int(int(use_ema)),
                                                C.c_void_p(out.data_ptr())))
        return out

    # --- snapshots
    def save_snapshot(self, path, include_optimizer_state=False):
        """``Testbed.save_snapshot`` (src/python_api.cu:347, src/testbed.cu:3134): msgpack file in the reference's layout."""
        from . import snapshot
        snapshot.save_snapshot(self, path, include_optimizer_state)

    def load_snapshot(self, path):
        """``Testbed.load_snapshot`` (src/testbed.cu:3187)."""
        from . import snapshot
        return snapshot.load_snapshot(self, path)

    # --- rendering
    @property
    def fov(self):
        """Field of view in degrees along fov_axis (Testbed::fov, src/testbed.cu:1820)."""
        return float(2.0 * 180.0 / np.pi * np.arctan(1.0 / (self.relative_focal_length[self.fov_axis] * 2.0)))

    @fov.setter
    def fov(self, degrees):
        self.relative_focal_length[:] = 0.5 / np.tan(0.5 * degrees * np.pi / 180.0)

    def render(self, width, height, spp=1, linear=True, use_ema=True, return_depth=False):
        """``Testbed.render(width, height, spp, linear)`` (src/python_api.cu:123-169, 333) with the camera in
        ``camera_matrix`` (3x4 camera-to-world in the scene's own coordinates, like ``Testbed::m_camera``): float32
        [height][width][4], alpha premultiplied."""
        req = L.RenderRequest()
        req.width, req.height, req.spp = int(width), int(height), int(spp)
        cam = np.asarray(self.camera_matrix, np.float32).reshape(3, 4)
        req.camera = (C.c_float * 12)(*cam.T.reshape(-1).tolist())
        req.relative_focal_length = (C.c_float * 2)(*[float(v) for v in self.relative_focal_length])
        req.fov_axis, req.zoom = int(self.fov_axis), float(self.zoom)
        req.screen_center = (C.c_float * 2)(*[float(v) for v in self.screen_center])
        req.snap_to_pixel_centers = int(bool(self.snap_to_pixel_centers))
        req.exposure = float(self.exposure)
        req.background_color = (C.c_float * 4)(*[float(v) for v in self.background_color])
        req.linear = int(bool(linear))
        req.min_transmittance = float(self.rendering_min_transmittance)
        req.use_ema = int(bool(use_ema))
        out = np.empty((int(height), int(width), 4), np.float32)
        depth = np.empty((int(height), int(width)), np.float32) if return_depth else None
        L.check(L.lib().neus2b_testbed_render(self._h, C.byref(req), out.ctypes.data_as(C.c_void_p),
                                              depth.ctypes.data_as(C.c_void_p) if return_depth else None))
        n, ms = C.c_uint64(0), C.c_float(0.0)
        L.check(L.lib().neus2b_testbed_render_stats(self._h, C.byref(n), C.byref(ms)))
        self.last_render_samples, self.last_render_device_ms = int(n.value), float(ms.value)
        return (out, depth) if return_depth else out

    def profile_train_kernel(self, max_steps=0):
        """Arms timing of the fused forward+backward kernel for the next `max_steps` steps (0 = off) and returns
        (sum of milliseconds, launches) recorded since the previous call."""
        ms, n = C.c_float(0.0), C.c_uint32(0)
        L.check(L.lib().neus2b_testbed_profile(self._h, C.c_uint32(max_steps), C.byref(ms), C.byref(n)))
        return ms.value, n.value

    @staticmethod
    def marching_cubes_resolution(resolution):
        """Testbed::marching_cubes rounds every axis up to a multiple of 16 (src/testbed_nerf.cu:4161-4163)."""
        res = [int(r) for r in (resolution if hasattr(resolution, "__len__") else (resolution,) * 3)]
        return [(r + 15) // 16 * 16 for r in res]

    def compute_marching_cubes_mesh(self, resolution=256, thresh=0.0, tri_table=None, use_ema=True):
        """Testbed::marching_cubes (src/testbed_nerf.cu:4160-4181): SDF on the lattice (every axis rounded up to a multiple of 16)
        with the EMA parameters, marching cubes at `thresh`, and -- on a later frame of a dynamic sequence -- the vertices taken
        from the canonical frame to the current one by the accumulated movement, v <- R_acc^-1 (v - t_acc)
        (transform_mesh_with_6d, src/testbed_nerf.cu:98-128).  Returns (verts, indices) as CUDA tensors."""
        import torch
        from . import ops
        verts, indices = ops.marching_cubes(self.sdf_grid(self.marching_cubes_resolution(resolution), use_ema=use_ema), tri_table=tri_table, thresh=thresh)
        frame, R_acc, t_acc, _ = self.movement()
        if frame >= 1 and (np.any(R_acc != np.eye(3, dtype=np.float32).reshape(R_acc.shape)) or np.any(t_acc != 0)):
            R = torch.from_numpy(np.ascontiguousarray(R_acc, np.float32).reshape(3, 3)).to(verts.device)
            t = torch.from_numpy(np.ascontiguousarray(t_acc, np.float32).reshape(3)).to(verts.device)
            verts = ((verts - t) @ torch.linalg.inv(R).T).contiguous()
        return verts, indices

    def compute_and_save_marching_cubes_mesh(self, filename, resolution=256, thresh=0.0, tri_table=None, use_ema=True,
                                             nerf_scale=None, nerf_offset=None, invert_normals=None):
        """Testbed::compute_and_save_marching_cubes_mesh (src/testbed.cu:298-306; python_api.cu:352): marching cubes on the
        SDF lattice, 1-ring normals, vertex colours from the network, OBJ or PLY file.  Scale, offset and the normals' side default
        to the loaded dataset's `scale`, `offset` and `from_na`, which is what the reference passes to its writer (1, 0 and False
        without a dataset description).  Returns the mesh as host arrays."""
        import torch
        from . import ops
        ds = getattr(self, "dataset", None) or {}
        nerf_scale = float(ds.get("scale", 1.0)) if nerf_scale is None else nerf_scale
        nerf_offset = tuple(ds.get("offset", (0.0, 0.0, 0.0))) if nerf_offset is None else nerf_offset
        invert_normals = bool(ds.get("from_na", False)) if invert_normals is None else invert_normals
        verts, indices = self.compute_marching_cubes_mesh(resolution, thresh, tri_table, use_ema)
        # the reference sizes its vertex buffer up to a multiple of 128 (src/marching_cubes.cu:813) and writes the unused entries
        # too: vertices at the origin that no face refers to.  The file gets them here as well; compute_marching_cubes_mesh does not.
        pad = (-verts.shape[0]) % 128
        if pad:
            verts = torch.cat([verts, torch.zeros((pad, 3), dtype=verts.dtype, device=verts.device)])
        ptrs = self.device_ptrs()
        normals = ops.mesh_1ring(verts, indices)
        colors = ops.mesh_vertex_colors(self.config.grid, ptrs["params_ema" if use_ema else "params"], self.config.sdf_bias, verts)
        torch.cuda.synchronize()
        mesh = dict(verts=verts.cpu().numpy(), normals=normals.cpu().numpy(), colors=colors.cpu().numpy(),
                    indices=indices.cpu().numpy().view(np.uint32))
        ops.save_mesh(filename, mesh["verts"], mesh["normals"], mesh["colors"], mesh["indices"], nerf_scale, nerf_offset, invert_normals)
        return mesh

    def compute_marching_cubes_mesh_sharded(self, resolution, rank, world, thresh=0.0, tri_table=None, use_ema=True, gather=None):
        """The same mesh with the lattice split into z-slabs, one per rank: every rank evaluates the SDF and runs marching cubes
        on its slab only, the parts are gathered and merged on the host (neus2_b200.mesh_shard).  Returns host arrays."""
        from . import mesh_shard, ops
        res = [int(r) for r in (resolution if hasattr(resolution, "__len__") else (resolution,) * 3)]

        def slab(z0, nl):
            return ops.marching_cubes_slab(self.sdf_grid(res, z0, z0 + nl, use_ema=use_ema), res, z0, tri_table=tri_table, thresh=thresh)
        return mesh_shard.extract_mesh_sharded(slab, res, rank, world, gather=gather)

    def compute_marching_cubes_mesh_sharded_device(self, resolution, rank, world, thresh=0.0, tri_table=None, use_ema=True, group=None,
                                                   dst=0):
        """The same mesh with every slab numbered on its own device: SDF of the slab (and of one halo layer when another slab
        follows), count pass, all-gather of the counters over the process group, emit pass at the global offsets, gather of
        the slices into rank `dst` (point-to-point).  No merge or re-indexing on the host.  Returns CUDA tensors
        (verts [n][3] float32, indices [m] int32) on rank `dst`, (None, None) on the others."""
        from . import mesh_shard, ops
        res = [int(r) for r in (resolution if hasattr(resolution, "__len__") else (resolution,) * 3)]

        def slab(z0, nl, halo):
            return ops.SlabGlobal(self.sdf_grid(res, z0, z0 + nl + halo, use_ema=use_ema), res, z0, nl, halo, tri_table=tri_table,
                                  thresh=thresh)
        return mesh_shard.extract_mesh_sharded_device(slab, res, rank, world, group=group, dst=dst)
