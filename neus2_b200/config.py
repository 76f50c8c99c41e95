"""The reference's network configuration files (configs/nerf/*.json) mapped onto ``neus2b_testbed_config``.

``Testbed::reload_network_from_file`` / ``reset_network`` (src/testbed.cu:2093-2339) read these blocks: "optimizer"
(Ema > ExponentialDecay > Adam, nested), "encoding" (hash grid; ``top_resolution`` gives the per-level scale when
``per_level_scale`` is absent, src/testbed.cu:2173-2177; ``base_training_step`` / ``valid_level_scale`` /
``base_valid_level_scale`` drive the progressive level mask), "network" (``sdf_bias``), "hyperparams" (loss weights,
``anneal_end``, ``batch_size``).  Keys this library does not implement are refused rather than ignored when they would
change the result (another encoding or network type, more than one hidden SDF layer, an output activation)."""
import ctypes as C
import json
import re

from . import _lib as L


def load_json_with_comments(path):
    """The shipped files carry // comments (the reference parses them with its JSON library's comment support)."""
    text = open(path).read()
    text = re.sub(r"//[^\n\"]*$", "", text, flags=re.M)
    return json.loads(text)


def _find(opt, otype):
    while opt is not None:
        if str(opt.get("otype", "")).lower() == otype.lower():
            return opt
        opt = opt.get("nested")
    return None


def testbed_config_from_json(cfg, aabb_scale=1, base=None):
    """``cfg``: the parsed file (or its path).  Returns a ``TestbedConfig``; ``base`` (optional) supplies everything the
    file does not name, default ``neus2b_testbed_default_config``."""
    if not isinstance(cfg, dict):
        cfg = load_json_with_comments(cfg)
    out = L.TestbedConfig()
    if base is not None:
        C.memmove(C.byref(out), C.byref(base), C.sizeof(out))
    else:
        L.lib().neus2b_testbed_default_config(C.byref(out))
    enc = cfg.get("encoding", {})
    if str(enc.get("otype", "HashGrid")).lower() not in ("hashgrid", "grid"):
        raise ValueError("encoding.otype %r: only the hash grid is built" % enc.get("otype"))
    if int(enc.get("n_features_per_level", 2)) != 2:
        raise ValueError("n_features_per_level must be 2")
    g = out.grid
    g.n_levels = int(enc.get("n_levels", g.n_levels))
    g.n_active_levels = g.n_levels
    g.log2_hashmap_size = int(enc.get("log2_hashmap_size", g.log2_hashmap_size))
    g.base_resolution = int(enc.get("base_resolution", g.base_resolution))
    scale = float(enc.get("per_level_scale", 0.0))
    if scale <= 0.0 and g.n_levels > 1:  # src/testbed.cu:2173-2177
        scale = float(L.lib().neus2b_per_level_scale_from_top_resolution(g.n_levels, g.base_resolution,
                                                                          C.c_float(float(enc.get("top_resolution", 2048.0))), int(aabb_scale)))
    g.per_level_scale = scale
    out.base_training_step = int(enc.get("base_training_step", 0))
    out.valid_level_scale = float(enc.get("valid_level_scale", 0.0))
    out.base_valid_level_scale = float(enc.get("base_valid_level_scale", 1.0))
    out.progressive_steps_per_increment = 0
    net = cfg.get("network", {})
    if int(net.get("n_neurons", 64)) != 64 or int(net.get("n_hidden_layers", 1)) != 1:
        raise ValueError("the SDF network is 64 neurons, one hidden layer")
    if str(net.get("activation", "ReLU")) != "ReLU" or str(net.get("output_activation", "None")) != "None":
        raise ValueError("the networks are ReLU with no output activation")
    out.sdf_bias = float(net.get("sdf_bias", out.sdf_bias))
    rgb = cfg.get("rgb_network", {})
    if int(rgb.get("n_neurons", 64)) != 64 or int(rgb.get("n_hidden_layers", 2)) != 2:
        raise ValueError("the colour network is 64 neurons, two hidden layers")
    opt = cfg.get("optimizer", {})
    ema, decay, adam = _find(opt, "Ema"), _find(opt, "ExponentialDecay"), _find(opt, "Adam")
    if adam is None:
        raise ValueError("optimizer: an Adam block is required")
    out.learning_rate = float(adam.get("learning_rate", out.learning_rate))
    out.beta1 = float(adam.get("beta1", out.beta1))
    out.beta2 = float(adam.get("beta2", out.beta2))
    out.epsilon = float(adam.get("epsilon", out.epsilon))
    out.l2_reg = float(adam.get("l2_reg", out.l2_reg))
    out.ema_decay = float(ema["decay"]) if ema is not None else 0.0
    if decay is not None:
        out.lr_decay_start = int(decay.get("decay_start", out.lr_decay_start))
        out.lr_decay_interval = int(decay.get("decay_interval", out.lr_decay_interval))
        out.lr_decay_base = float(decay.get("decay_base", out.lr_decay_base))
    else:
        out.lr_decay_interval = 0
    hp = cfg.get("hyperparams", {})
    out.ek_loss_weight = float(hp.get("ek_loss_weight", 0.01))     # src/testbed.cu:2126
    out.mask_loss_weight = float(hp.get("mask_loss_weight", 0.0))  # src/testbed.cu:2125
    out.anneal_end = int(hp.get("anneal_end", 0))
    if "batch_size" in hp:
        out.batch_size = int(hp["batch_size"])
    # dynamic sequences (src/testbed.cu:2108-2122; the frame counts are the caller's loop: dynamic_schedule below)
    out.predict_global_movement = int(bool(hp.get("predict_global_movement", False)))
    out.predict_global_movement_training_step = int(hp.get("predict_global_movement_training_step", 300)) if out.predict_global_movement else 0
    out.finetune_global_movement = int(bool(hp.get("finetune_global_movement", True)))
    out.reset_density_grid_after_global_movement = int(bool(hp.get("reset_density_grid_after_global_movement", True)))
    out.after_learning_rate = float(adam.get("after_learning_rate", 0.0))
    gm = cfg.get("globalmove", {}).get("optimizer", opt)  # src/testbed.cu:2311-2312: the main optimizer's block when absent
    g_ema, g_decay, g_adam = _find(gm, "Ema"), _find(gm, "ExponentialDecay"), _find(gm, "Adam")
    if g_adam is not None:
        out.gm_learning_rate = float(g_adam.get("learning_rate", out.gm_learning_rate))
        out.gm_beta1 = float(g_adam.get("beta1", out.gm_beta1))
        out.gm_beta2 = float(g_adam.get("beta2", out.gm_beta2))
        out.gm_epsilon = float(g_adam.get("epsilon", out.gm_epsilon))
        out.gm_l2_reg = float(g_adam.get("l2_reg", out.gm_l2_reg))
    out.gm_ema_decay = float(g_ema["decay"]) if g_ema is not None else 0.0
    if g_decay is not None:
        out.gm_lr_decay_start = int(g_decay.get("decay_start", out.gm_lr_decay_start))
        out.gm_lr_decay_interval = int(g_decay.get("decay_interval", out.gm_lr_decay_interval))
        out.gm_lr_decay_base = float(g_decay.get("decay_base", out.gm_lr_decay_base))
    else:
        out.gm_lr_decay_interval = 0
    return out


def dynamic_schedule(cfg):
    """(first_frame_max_training_step, next_frame_max_training_step) of a parsed configuration: how long Testbed::frame trains
    the first and every later frame before it switches (src/testbed.cu:1739-1746, 2108-2109)."""
    hp = cfg.get("hyperparams", {})
    return int(hp.get("first_frame_max_training_step", 2000)), int(hp.get("next_frame_max_training_step", 1000))
