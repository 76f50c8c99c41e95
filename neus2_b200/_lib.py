"""ctypes binding of libneus2b.so: one Python function per C entry point of include/neus2b.h.

There is no fallback: if the shared library is missing or a call returns an error, an exception is raised."""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("NEUS2B_LIB", os.path.join(HERE, "_build", "libneus2b.so"))

MLP_N = 12288
GRID_OFF = 12288
GRAD_IGNORE, GRAD_OVERWRITE, GRAD_ACCUMULATE = 0, 1, 2


class GridDesc(C.Structure):
    _fields_ = [("n_levels", C.c_uint32), ("log2_hashmap_size", C.c_uint32), ("base_resolution", C.c_uint32),
                ("per_level_scale", C.c_float), ("n_active_levels", C.c_uint32)]


class Pcg32(C.Structure):
    _fields_ = [("state", C.c_uint64), ("inc", C.c_uint64)]


class Dataset(C.Structure):
    _fields_ = [("n_images", C.c_uint32), ("width", C.c_uint32), ("height", C.c_uint32), ("d_pixels", C.c_void_p),
                ("d_xforms", C.c_void_p), ("d_focal", C.c_void_p), ("d_principal", C.c_void_p)]


class TrainCfg(C.Structure):
    _fields_ = [("aabb_min", C.c_float * 3), ("aabb_max", C.c_float * 3), ("cone_angle_constant", C.c_float),
                ("snap_to_pixel_centers", C.c_uint32), ("random_bg_color", C.c_uint32), ("background_color", C.c_float * 3),
                ("loss_scale", C.c_float), ("mask_loss_weight", C.c_float), ("ek_loss_weight", C.c_float),
                ("cos_anneal_ratio", C.c_float), ("ray_index_offset", C.c_uint32), ("ray_count_scale", C.c_uint32),
                ("use_global_movement", C.c_uint32), ("rotation", C.c_float * 9), ("transition", C.c_float * 3),
                ("first_frame_offset", C.c_float * 3)]


class Motion(C.Structure):
    _fields_ = [("d_delta", C.c_void_p), ("first_frame_offset", C.c_float * 3), ("d_sums", C.c_void_p)]


class RayWorkspace(C.Structure):
    _fields_ = [("max_rays", C.c_uint32), ("max_samples", C.c_uint32), ("d_ray_indices", C.c_void_p), ("d_rays", C.c_void_p),
                ("d_numsteps", C.c_void_p), ("d_coords", C.c_void_p), ("d_counters", C.c_void_p), ("d_scan_tmp", C.c_void_p),
                ("d_ray_tmp", C.c_void_p), ("d_n_rays_total", C.c_void_p), ("d_march_masks", C.c_void_p), ("d_occupied_bounds", C.c_void_p),
                ("d_window_list", C.c_void_p), ("d_window_lens", C.c_void_p), ("d_prev_samples", C.c_void_p)]


class RenderCfg(C.Structure):
    _fields_ = [("width", C.c_uint32), ("height", C.c_uint32), ("focal_length", C.c_float * 2), ("screen_center", C.c_float * 2),
                ("camera", C.c_float * 12), ("pixel_offset", C.c_float * 2), ("sample_index", C.c_uint32),
                ("aabb_min", C.c_float * 3), ("aabb_max", C.c_float * 3), ("cone_angle_constant", C.c_float),
                ("min_transmittance", C.c_float), ("cos_anneal_ratio", C.c_float), ("linear_colors", C.c_uint32),
                ("max_steps", C.c_uint32), ("use_global_movement", C.c_uint32), ("rotation", C.c_float * 9),
                ("transition", C.c_float * 3), ("first_frame_offset", C.c_float * 3), ("d_delta", C.c_void_p)]


class RenderWorkspace(C.Structure):
    _fields_ = [("max_rays", C.c_uint32), ("max_samples", C.c_uint32), ("d_ray_tmp", C.c_void_p), ("d_scan_tmp", C.c_void_p),
                ("d_state", C.c_void_p), ("d_hit_list", C.c_void_p), ("d_coords", C.c_void_p), ("d_out", C.c_void_p),
                ("d_counters", C.c_void_p), ("d_occupied_bounds", C.c_void_p), ("d_march_masks", C.c_void_p)]


class RenderRequest(C.Structure):
    _fields_ = [("width", C.c_uint32), ("height", C.c_uint32), ("spp", C.c_uint32), ("camera", C.c_float * 12),
                ("relative_focal_length", C.c_float * 2), ("fov_axis", C.c_uint32), ("zoom", C.c_float),
                ("screen_center", C.c_float * 2), ("snap_to_pixel_centers", C.c_uint32), ("exposure", C.c_float),
                ("background_color", C.c_float * 4), ("linear", C.c_uint32), ("min_transmittance", C.c_float),
                ("use_ema", C.c_uint32)]


class AdamCfg(C.Structure):
    _fields_ = [("learning_rate", C.c_float), ("beta1", C.c_float), ("beta2", C.c_float), ("epsilon", C.c_float),
                ("l2_reg", C.c_float), ("ema_decay", C.c_float), ("loss_scale", C.c_float), ("step", C.c_uint32),
                ("n_matrix", C.c_uint32), ("flags", C.c_uint32), ("d_nonfinite", C.c_void_p)]


ADAM_UPDATE_UNTOUCHED, ADAM_L2_ALL, ADAM_EMA_NO_DEBIAS = 1, 2, 4


class TestbedConfig(C.Structure):
    _fields_ = [("grid", GridDesc), ("sdf_bias", C.c_float), ("batch_size", C.c_uint32), ("n_cascades", C.c_uint32),
                ("seed", C.c_uint32), ("learning_rate", C.c_float), ("beta1", C.c_float), ("beta2", C.c_float),
                ("epsilon", C.c_float), ("l2_reg", C.c_float), ("ema_decay", C.c_float), ("lr_decay_start", C.c_uint32),
                ("lr_decay_interval", C.c_uint32), ("lr_decay_base", C.c_float), ("ek_loss_weight", C.c_float),
                ("mask_loss_weight", C.c_float), ("anneal_end", C.c_uint32), ("density_grid_decay", C.c_float),
                ("random_bg_color", C.c_uint32), ("snap_to_pixel_centers", C.c_uint32),
                ("progressive_start_levels", C.c_uint32), ("progressive_levels_per_increment", C.c_uint32),
                ("progressive_steps_per_increment", C.c_uint32), ("world_size", C.c_uint32), ("rank", C.c_uint32),
                ("valid_level_scale", C.c_float), ("base_valid_level_scale", C.c_float), ("base_training_step", C.c_uint32),
                ("adam_flags", C.c_uint32), ("loss_scale", C.c_float),
                ("predict_global_movement", C.c_uint32), ("predict_global_movement_training_step", C.c_uint32),
                ("finetune_global_movement", C.c_uint32), ("reset_density_grid_after_global_movement", C.c_uint32),
                ("after_learning_rate", C.c_float), ("gm_learning_rate", C.c_float), ("gm_beta1", C.c_float), ("gm_beta2", C.c_float),
                ("gm_epsilon", C.c_float), ("gm_l2_reg", C.c_float), ("gm_ema_decay", C.c_float), ("gm_lr_decay_start", C.c_uint32),
                ("gm_lr_decay_interval", C.c_uint32), ("gm_lr_decay_base", C.c_float), ("first_frame_offset", C.c_float * 3),
                ("n_forward_windows", C.c_uint32), ("forward_window_ends", C.c_uint32 * 6)]


class TrainingState(C.Structure):
    _fields_ = [("training_step", C.c_uint32), ("density_grid_ema_step", C.c_uint32), ("rays_per_batch", C.c_uint32),
                ("measured_batch_size", C.c_uint32), ("measured_batch_size_before_compaction", C.c_uint32),
                ("n_rays_total", C.c_uint32), ("loss", C.c_float), ("ek_loss", C.c_float), ("rng", Pcg32), ("density_rng", Pcg32)]


class TrainStats(C.Structure):
    _fields_ = [("training_step", C.c_uint32), ("rays_per_batch", C.c_uint32), ("n_rays_kept", C.c_uint32),
                ("measured_batch_size_before_compaction", C.c_uint32), ("measured_batch_size", C.c_uint32),
                ("overflow", C.c_uint32), ("loss", C.c_float), ("ek_loss", C.c_float), ("nonfinite_gradients", C.c_uint32),
                ("device_error", C.c_uint32), ("n_samples_evaluated", C.c_uint32)]


class Neus2bError(RuntimeError):
    pass


_lib = None

# every symbol include/neus2b.h declares
EXPORTS = [
    "neus2b_version", "neus2b_launch_count", "neus2b_error_string", "neus2b_grid_level_table", "neus2b_grid_n_params", "neus2b_model_n_params",
    "neus2b_grid_forward", "neus2b_grid_backward_input", "neus2b_grid_backward_params", "neus2b_grid_backward_backward_input",
    "neus2b_mlp_forward", "neus2b_mlp_forward_tcgen05", "neus2b_mlp_backward", "neus2b_mlp_backward_backward_input", "neus2b_sh4_forward",
    "neus2b_set_mma_path", "neus2b_get_mma_path", "neus2b_device_error_flags", "neus2b_set_device_error_flags",
    "neus2b_per_level_scale_from_top_resolution", "neus2b_testbed_config_active_levels", "neus2b_neus_forward", "neus2b_neus_train", "neus2b_neus_sdf",
    "neus2b_neus_forward_moved", "neus2b_neus_forward_indexed", "neus2b_forward_compute_loss", "neus2b_neus_train_moved", "neus2b_neus_sdf_moved", "neus2b_delta_forward", "neus2b_delta_backward",
    "neus2b_delta_optimizer_step", "neus2b_movement_accumulate", "neus2b_occupancy_update_moved", "neus2b_pcg32_seed", "neus2b_pcg32_advance", "neus2b_abi_struct_sizes",
    "neus2b_generate_samples", "neus2b_generate_samples_static", "neus2b_compute_loss", "neus2b_occupancy_update", "neus2b_occupancy_bounds", "neus2b_adam_step", "neus2b_adam_step_packed",
    "neus2b_testbed_default_config", "neus2b_testbed_create", "neus2b_testbed_destroy", "neus2b_testbed_load_training_data",
    "neus2b_testbed_update_cameras", "neus2b_testbed_set_params", "neus2b_testbed_get_params", "neus2b_testbed_n_params",
    "neus2b_testbed_train", "neus2b_testbed_device_ptrs", "neus2b_testbed_train_backward", "neus2b_testbed_train_pregenerate", "neus2b_testbed_train_optimizer_step_async", "neus2b_testbed_train_wait_stats", "neus2b_testbed_train_step",
    "neus2b_testbed_train_optimizer_step", "neus2b_testbed_sdf_grid", "neus2b_testbed_profile", "neus2b_marching_cubes_scratch_bytes", "neus2b_marching_cubes", "neus2b_marching_cubes_slab", "neus2b_marching_cubes_slab_global",
    "neus2b_render_frame", "neus2b_render_accumulate", "neus2b_render_tonemap", "neus2b_ld_random_pixel_offset", "neus2b_testbed_render", "neus2b_testbed_render_stats",
    "neus2b_mesh_1ring", "neus2b_mesh_vertex_colors", "neus2b_save_mesh", "neus2b_occupancy_mean_and_bitfield",
    "neus2b_testbed_next_frame", "neus2b_testbed_get_movement", "neus2b_testbed_set_movement", "neus2b_testbed_get_training_state", "neus2b_testbed_set_training_state", "neus2b_testbed_get_array", "neus2b_testbed_set_array",
]


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise Neus2bError(f"{LIB_PATH} is missing: run `python -m neus2_b200.build` (there is no CPU fallback)")
        _lib = C.CDLL(LIB_PATH)
        _lib.neus2b_version.restype = C.c_char_p
        _lib.neus2b_error_string.restype = C.c_char_p
        _lib.neus2b_pcg32_seed.restype = None
        _lib.neus2b_pcg32_advance.restype = None
        _lib.neus2b_testbed_default_config.restype = None
        _lib.neus2b_testbed_destroy.restype = None
        _lib.neus2b_ld_random_pixel_offset.restype = None
        _lib.neus2b_testbed_destroy.argtypes = [C.c_void_p]
        _lib.neus2b_per_level_scale_from_top_resolution.restype = C.c_float
        _lib.neus2b_per_level_scale_from_top_resolution.argtypes = [C.c_uint32, C.c_uint32, C.c_float, C.c_uint32]
        _lib.neus2b_testbed_config_active_levels.restype = C.c_uint32
        _lib.neus2b_launch_count.restype = C.c_uint64
        _check_layout(_lib)
    return _lib


def abi_structs():
    """The ctypes mirrors of the header's structures, in the order of neus2b_abi_struct_sizes."""
    return [GridDesc, Motion, Pcg32, Dataset, TrainCfg, RayWorkspace, AdamCfg, TestbedConfig, TrainStats, RenderCfg, RenderWorkspace, RenderRequest,
            TrainingState]


def _check_layout(library):
    """A structure that is laid out differently here than in the loaded library would be read past its end or with shifted
    fields: refuse the library instead."""
    mirrors = abi_structs()
    sizes = (C.c_uint32 * len(mirrors))()
    library.neus2b_abi_struct_sizes.restype = C.c_uint32
    n = library.neus2b_abi_struct_sizes(sizes, C.c_uint32(len(mirrors)))
    bad = [(m.__name__, C.sizeof(m), int(sz)) for m, sz in zip(mirrors, sizes) if C.sizeof(m) != int(sz)]
    if n != len(mirrors) or bad:
        raise Neus2bError(f"{LIB_PATH} and neus2_b200/_lib.py disagree on the C ABI's structures: {n} in the library, {len(mirrors)} here; "
                          f"(name, size here, size there): {bad}; rebuild with `python -m neus2_b200.build`")


MMA_SYNC, MMA_TCGEN05 = 0, 1


def set_mma_path(path):
    check(lib().neus2b_set_mma_path(C.c_int(path)))


def get_mma_path():
    return int(lib().neus2b_get_mma_path())


def device_error_flags():
    v = C.c_uint32(0)
    check(lib().neus2b_device_error_flags(C.byref(v)))
    return int(v.value)


def launch_count():
    return int(lib().neus2b_launch_count())


def set_device_error_flags(flags):
    check(lib().neus2b_set_device_error_flags(C.c_uint32(flags)))


def check(rc):
    if rc != 0:
        raise Neus2bError(f"neus2b error {rc}: {lib().neus2b_error_string(C.c_int(rc)).decode()}")


def ptr(t):
    """Device pointer of a torch tensor (or None)."""
    if t is None:
        return C.c_void_p(0)
    if isinstance(t, int):  # a raw device address, e.g. from Testbed.device_ptrs()
        return C.c_void_p(t)
    assert t.is_cuda and t.is_contiguous(), "neus2b takes contiguous CUDA tensors"
    return C.c_void_p(t.data_ptr())


def cur_stream():
    import torch
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def grid_desc(n_levels=16, log2_hashmap_size=19, base_resolution=16, per_level_scale=1.447, n_active_levels=None):
    return GridDesc(n_levels, log2_hashmap_size, base_resolution, per_level_scale,
                    n_levels if n_active_levels is None else n_active_levels)


def grid_n_params(d):
    n = C.c_uint64(0)
    check(lib().neus2b_grid_n_params(C.byref(d), C.byref(n)))
    return int(n.value)


def model_n_params(d):
    n = C.c_uint64(0)
    check(lib().neus2b_model_n_params(C.byref(d), C.byref(n)))
    return int(n.value)


def grid_level_table(d):
    off = (C.c_uint32 * 17)()
    res = (C.c_uint32 * 16)()
    scale = (C.c_float * 16)()
    hashed = (C.c_uint32 * 16)()
    check(lib().neus2b_grid_level_table(C.byref(d), off, res, scale, hashed))
    return list(off), list(res), list(scale), list(hashed)


def pcg32(seed):
    r = Pcg32()
    lib().neus2b_pcg32_seed(C.byref(r), C.c_uint64(seed))
    return r


def pcg32_advance(r, delta):
    r2 = Pcg32(r.state, r.inc)
    lib().neus2b_pcg32_advance(C.byref(r2), C.c_uint64(delta))
    return r2


def train_cfg(ek_loss_weight=0.1, mask_loss_weight=0.0, random_bg_color=True, snap_to_pixel_centers=False,
              cos_anneal_ratio=1.0, loss_scale=128.0, background_color=(0.0, 0.0, 0.0), ray_index_offset=0,
              ray_count_scale=1, rotation=None, transition=None, first_frame_offset=(0.0, 0.0, 0.0)):
    c = TrainCfg()
    if rotation is not None:
        c.use_global_movement = 1
        c.rotation[:] = [float(v) for v in rotation]
        c.transition[:] = [float(v) for v in transition]
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
