"""Snapshots of a Testbed in the reference's container format (``Testbed::save_snapshot`` / ``load_snapshot``,
src/testbed.cu:3134-3244): one msgpack document = the network configuration plus a ``"snapshot"`` object with the trainer's
serialisation, the occupancy grid as fp16, the training step, the loss and the batch tuner's counters.

The part ``Trainer::serialize`` writes (``n_params``, ``params_type``, ``params_binary`` = the fp16 inference parameters, and
``optimizer`` when the optimizer state is included) lives in the reference's tiny-cuda-nn fork, which is not vendored: the
keys follow the public tiny-cuda-nn trainer, the optimizer object uses this library's own keys.  What this library needs
beyond the reference's fields to continue a run exactly (fp32 master weights, EMA state, random-number streams) sits under
``"neus2b"`` and is ignored by other readers.
"""
import ctypes as C

import numpy as np

from . import _lib as L

GRIDSIZE = 128
ARRAY = dict(master=0, adam_m=1, adam_v=2, ema_master=3, params=4, params_ema=5, density_grid=6)
_DTYPE = dict(master=np.float32, adam_m=np.float32, adam_v=np.float32, ema_master=np.float32, params=np.uint16,
              params_ema=np.uint16, density_grid=np.float32)


def _array_size(tb, name):
    return GRIDSIZE ** 3 * int(tb.config.n_cascades) if name == "density_grid" else tb.n_params


def get_array(tb, name):
    a = np.empty(_array_size(tb, name), _DTYPE[name])
    L.check(L.lib().neus2b_testbed_get_array(tb._h, C.c_int(ARRAY[name]), a.ctypes.data_as(C.c_void_p), C.c_uint64(a.nbytes)))
    return a


def set_array(tb, name, a):
    a = np.ascontiguousarray(a, dtype=_DTYPE[name])
    if a.size != _array_size(tb, name):
        raise ValueError(f"{name}: {a.size} entries, the testbed holds {_array_size(tb, name)}")
    L.check(L.lib().neus2b_testbed_set_array(tb._h, C.c_int(ARRAY[name]), a.ctypes.data_as(C.c_void_p), C.c_uint64(a.nbytes)))


def get_training_state(tb):
    st = L.TrainingState()
    L.check(L.lib().neus2b_testbed_get_training_state(tb._h, C.byref(st)))
    return st


def network_config(cfg):
    """The configuration object the snapshot is embedded in, with the reference's key names (configs/nerf/base.json,
    dtu.json)."""
    g = cfg.grid
    return {
        "encoding": {"otype": "HashGrid", "n_levels": int(g.n_levels), "n_features_per_level": 2,
                     "log2_hashmap_size": int(g.log2_hashmap_size), "base_resolution": int(g.base_resolution),
                     "per_level_scale": float(g.per_level_scale)},
        "network": {"otype": "FullyFusedMLP", "activation": "ReLU", "output_activation": "None", "n_neurons": 64,
                    "n_hidden_layers": 1, "sdf_bias": float(cfg.sdf_bias)},
        "rgb_network": {"otype": "FullyFusedMLP", "activation": "ReLU", "output_activation": "None", "n_neurons": 64,
                        "n_hidden_layers": 2},
        "dir_encoding": {"otype": "SphericalHarmonics", "degree": 4},
        "loss": {"otype": "Huber"},
        "optimizer": {"otype": "Ema", "decay": float(cfg.ema_decay), "nested": {
            "otype": "ExponentialDecay", "decay_start": int(cfg.lr_decay_start), "decay_interval": int(cfg.lr_decay_interval),
            "decay_base": float(cfg.lr_decay_base), "nested": {
                "otype": "Adam", "learning_rate": float(cfg.learning_rate), "beta1": float(cfg.beta1), "beta2": float(cfg.beta2),
                "epsilon": float(cfg.epsilon), "l2_reg": float(cfg.l2_reg)}}},
        "hyperparams": {"batch_size": int(cfg.batch_size), "ek_loss_weight": float(cfg.ek_loss_weight),
                        "mask_loss_weight": float(cfg.mask_loss_weight), "anneal_end": int(cfg.anneal_end)},
    }


def save_snapshot(tb, path, include_optimizer_state=False):
    import msgpack
    st = get_training_state(tb)
    doc = network_config(tb.config)
    snap = {
        "n_params": tb.n_params,
        "params_type": "__half",
        "params_binary": get_array(tb, "params_ema").tobytes(),
        "density_grid_size": GRIDSIZE,
        "density_grid_binary": get_array(tb, "density_grid").astype(np.float16).tobytes(),
        "training_step": int(st.training_step),
        "loss": float(st.loss),
        "nerf": {"aabb_scale": 1 << (int(tb.config.n_cascades) - 1),
                 "rgb": {"rays_per_batch": int(st.rays_per_batch), "measured_batch_size": int(st.measured_batch_size),
                         "measured_batch_size_before_compaction": int(st.measured_batch_size_before_compaction)}},
        "neus2b": {"density_grid_ema_step": int(st.density_grid_ema_step), "n_rays_total": int(st.n_rays_total),
                   "ek_loss": float(st.ek_loss), "rng": [int(st.rng.state), int(st.rng.inc)],
                   "density_rng": [int(st.density_rng.state), int(st.density_rng.inc)]},
    }
    # dynamic sequences (NerfNetwork::save_global_movement / save_local_movement, nerf_network.h:1169-1196, 1231-1235): the
    # accumulated movement as the reference's buffers hold it (rotation: 12 fp16 slots, the matrix row-major in the first nine;
    # transition: 4 slots) and the current frame's motion parameters (8 + 4 fp16 values)
    frame, R_acc, t_acc, delta = tb.movement()
    snap["rotation"] = np.concatenate([R_acc.reshape(9), np.zeros(3)]).astype(np.float16).tobytes()
    snap["transition"] = np.concatenate([t_acc.reshape(3), np.zeros(1)]).astype(np.float16).tobytes()
    snap["local_rotation"] = delta[4:12].astype(np.float16).tobytes()
    snap["local_transition"] = delta[0:4].astype(np.float16).tobytes()
    snap["neus2b"]["frame"] = int(frame)
    snap["neus2b"]["local_movement_fp32"] = delta.astype(np.float32).tobytes()
    if include_optimizer_state:
        snap["optimizer"] = {"otype": "Ema", "ema_master_binary": get_array(tb, "ema_master").tobytes(),
                             "nested": {"otype": "Adam", "current_step": int(st.training_step),
                                        "first_moments_binary": get_array(tb, "adam_m").tobytes(),
                                        "second_moments_binary": get_array(tb, "adam_v").tobytes()}}
        snap["neus2b"]["params_full_precision_binary"] = get_array(tb, "master").tobytes()
        snap["neus2b"]["params_training_binary"] = get_array(tb, "params").tobytes()
    doc["snapshot"] = snap
    with open(path, "wb") as f:
        f.write(msgpack.packb(doc, use_bin_type=True))


def load_snapshot(tb, path):
    """Restores parameters, occupancy grid, step and counters into ``tb`` (which must have the same architecture).  Without
    optimizer state in the file the fp16 inference parameters become every copy of the weights, as in the reference."""
    import msgpack
    with open(path, "rb") as f:
        doc = msgpack.unpackb(f.read(), raw=False, strict_map_key=False)
    if "snapshot" not in doc:
        raise ValueError(f"File '{path}' does not contain a snapshot.")
    snap = doc["snapshot"]
    if snap["density_grid_size"] != GRIDSIZE:
        raise ValueError("Incompatible grid size.")
    if snap["n_params"] != tb.n_params or snap.get("params_type", "__half") != "__half":
        raise ValueError(f"snapshot holds {snap['n_params']} {snap.get('params_type')} parameters, the testbed {tb.n_params} __half")
    half_bits = np.frombuffer(snap["params_binary"], np.uint16)
    extra = snap.get("neus2b", {})
    opt = snap.get("optimizer")
    if opt is not None and "params_full_precision_binary" in extra:
        tb.set_params(np.frombuffer(extra["params_full_precision_binary"], np.float32))
        set_array(tb, "params", np.frombuffer(extra["params_training_binary"], np.uint16))
        set_array(tb, "params_ema", half_bits)
        set_array(tb, "ema_master", np.frombuffer(opt["ema_master_binary"], np.float32))
        set_array(tb, "adam_m", np.frombuffer(opt["nested"]["first_moments_binary"], np.float32))
        set_array(tb, "adam_v", np.frombuffer(opt["nested"]["second_moments_binary"], np.float32))
    else:
        # the reference resets the network before it deserialises (src/testbed.cu:3215): a file without optimizer state
        # leaves a fresh optimizer behind, whatever the testbed had trained before
        tb.set_params(half_bits.view(np.float16).astype(np.float32))
        zeros = np.zeros(tb.n_params, np.float32)
        set_array(tb, "adam_m", zeros)
        set_array(tb, "adam_v", zeros)
    grid = np.frombuffer(snap["density_grid_binary"], np.float16).astype(np.float32)
    if grid.size == GRIDSIZE ** 3 * int(tb.config.n_cascades):
        set_array(tb, "density_grid", grid)
    elif grid.size != 0:  # size 0: a model that was never trained
        raise ValueError("Incompatible number of grid cascades.")
    if "rotation" in snap:  # load_global_movement / load_local_movement (nerf_network.h:1198-1261)
        R_acc = np.frombuffer(snap["rotation"], np.float16).astype(np.float32)[:9]
        t_acc = np.frombuffer(snap["transition"], np.float16).astype(np.float32)[:3]
        if "local_movement_fp32" in extra:
            delta = np.frombuffer(extra["local_movement_fp32"], np.float32)
        else:
            delta = np.concatenate([np.frombuffer(snap["local_transition"], np.float16), np.frombuffer(snap["local_rotation"], np.float16)]).astype(np.float32)
        tb.set_movement(int(extra.get("frame", 0)), R_acc, t_acc, delta)
    st = get_training_state(tb)
    st.training_step = int(snap["training_step"])
    st.loss = float(snap["loss"])
    rgb = snap["nerf"]["rgb"]
    st.rays_per_batch = int(rgb["rays_per_batch"])
    st.measured_batch_size = int(rgb["measured_batch_size"])
    st.measured_batch_size_before_compaction = int(rgb["measured_batch_size_before_compaction"])
    if extra:
        st.density_grid_ema_step = int(extra["density_grid_ema_step"])
        st.n_rays_total = int(extra["n_rays_total"])
        st.ek_loss = float(extra["ek_loss"])
        st.rng.state, st.rng.inc = extra["rng"]
        st.density_rng.state, st.density_rng.inc = extra["density_rng"]
    L.check(L.lib().neus2b_testbed_set_training_state(tb._h, C.byref(st)))
    tb.stats.training_step = st.training_step
    tb.stats.loss, tb.stats.ek_loss = st.loss, st.ek_loss
    tb.stats.rays_per_batch = st.rays_per_batch
    return doc
