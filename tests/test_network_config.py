"""The reference's network configuration blocks mapped onto the testbed configuration (no GPU needed)."""
import ctypes as C
import json

import numpy as np
import pytest

# the values of the reference's configs/nerf/dtu.json (static scenes), restated
DTU = {
    "loss": {"otype": "Huber"},
    "optimizer": {"otype": "Ema", "decay": 0.95, "nested": {
        "otype": "ExponentialDecay", "decay_start": 20000, "decay_interval": 10000, "decay_base": 0.33, "nested": {
            "otype": "Adam", "learning_rate": 1e-2, "beta1": 0.9, "beta2": 0.99, "epsilon": 1e-15, "l2_reg": 1e-6,
            "optimize_delta_params": False, "optimize_canonical_params": True}}},
    "encoding": {"otype": "HashGrid", "n_levels": 14, "n_features_per_level": 2, "log2_hashmap_size": 19, "base_resolution": 16,
                 "top_resolution": 2048, "valid_level_scale": 0.02, "base_valid_level_scale": 0.2, "base_training_step": 200},
    "network": {"otype": "FullyFusedMLP", "activation": "ReLU", "output_activation": "None", "n_neurons": 64, "n_hidden_layers": 1,
                "sdf_bias": -0.1},
    "rgb_network": {"otype": "FullyFusedMLP", "activation": "ReLU", "output_activation": "None", "n_neurons": 64, "n_hidden_layers": 2},
    "hyperparams": {"linear_color": False, "first_frame_max_training_step": 15000, "mask_loss_weight": 0.0, "ek_loss_weight": 0.01},
}


def test_dtu_config_maps_onto_the_testbed_config(tmp_path):
    from neus2_b200 import _lib as L
    from neus2_b200 import config
    c = config.testbed_config_from_json(DTU)
    assert (c.grid.n_levels, c.grid.log2_hashmap_size, c.grid.base_resolution, c.grid.n_active_levels) == (14, 19, 16, 14)
    assert abs(c.grid.per_level_scale - np.exp(np.log(2048 / 16) / 13)) < 1e-6
    assert (c.base_training_step, round(c.valid_level_scale, 6), round(c.base_valid_level_scale, 6)) == (200, 0.02, 0.2)
    assert abs(c.learning_rate - 1e-2) < 1e-9 and abs(c.ek_loss_weight - 0.01) < 1e-9 and c.mask_loss_weight == 0
    assert (c.lr_decay_start, c.lr_decay_interval) == (20000, 10000) and abs(c.lr_decay_base - 0.33) < 1e-7
    assert abs(c.ema_decay - 0.95) < 1e-7 and abs(c.epsilon - 1e-15) < 1e-20 and abs(c.sdf_bias + 0.1) < 1e-7
    act = lambda step: int(L.lib().neus2b_testbed_config_active_levels(C.byref(c), C.c_uint32(step)))
    assert act(0) == 3 and act(4000) == 8 and act(8000) == 14 and act(15000) == 14
    # the same through a file with the // comments the shipped files carry
    p = tmp_path / "cfg.json"
    p.write_text(json.dumps(DTU, indent=1).replace('"learning_rate": 0.01,', '"learning_rate": 0.01, // first frame'))
    c2 = config.testbed_config_from_json(str(p))
    assert bytes(c2) == bytes(c)
    assert L.grid_n_params(c.grid) == L.grid_n_params(L.grid_desc(n_levels=14, per_level_scale=c.grid.per_level_scale))


def test_unbuilt_architectures_are_refused():
    from neus2_b200 import config
    for path, value in ((("network", "n_hidden_layers"), 2), (("encoding", "otype"), "Frequency"), (("rgb_network", "n_neurons"), 128),
                        (("encoding", "n_features_per_level"), 4)):
        bad = json.loads(json.dumps(DTU))
        bad[path[0]][path[1]] = value
        with pytest.raises(ValueError):
            config.testbed_config_from_json(bad)
