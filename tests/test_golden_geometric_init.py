"""The one numeric fixture the reference ships for this path (utils/mlp_weights.txt, sphere-initialised SDF MLP) pins
the weight layout and the SDF-net forward: tests/golden/geometric_init.npz was made from it by
tests/golden/make_geometric_init_golden.py."""
import os

import numpy as np
import pytest

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "geometric_init.npz")


def load():
    g = np.load(GOLD)
    return g, g["sdf_fp16"].view(np.float16).astype(np.float32)


def test_weight_file_layout_is_row_major_out_in():
    g, _ = load()
    # [64][48] first layer: only the xyz columns carry weights; [16][64] last layer: constant sqrt(pi)/sqrt(64)
    assert list(g["nonzero_input_columns"]) == [0, 1, 2]
    assert abs(float(g["w2_min"]) - np.sqrt(np.pi) / 8) < 1e-3 and abs(float(g["w2_max"]) - np.sqrt(np.pi) / 8) < 1e-3
    assert abs(float(g["w1_xyz_std"]) - np.sqrt(2.0) / 8) < 0.02


def test_oracle_reproduces_golden_and_is_sphere_like(oracle):
    O = oracle
    g, sdf = load()
    d = O.grid_desc()
    params = np.zeros(O.model_n_params(d), np.uint16)
    params[:4096] = g["weights_fp16"]
    got = O.neus_sdf(d, params, g["x"], sdf_bias=-0.1)
    assert np.array_equal(got, g["sdf_fp16"])
    # known answer: with a zero grid the net is ~ |x - c| + bias
    r = np.linalg.norm(g["x"] - 0.5, axis=1)
    slope, icpt = np.polyfit(r, sdf, 1)
    assert 0.9 < slope < 1.2 and -0.16 < icpt < -0.05
    # the product's own geometric initialisation follows the same recipe
    from neus2_b200 import synthetic as S
    w = S.geometric_init_sdf_weights()
    W1, W2 = w[:3072].reshape(64, 48), w[3072:].reshape(16, 64)
    assert np.abs(W1[:, 3:]).max() == 0 and np.allclose(W2, np.sqrt(np.pi) / 8)
    assert abs(W1[:, :3].std() - float(g["w1_xyz_std"])) < 0.04


@pytest.mark.gpu
def test_cuda_sdf_net_matches_golden():
    import torch
    from neus2_b200 import _lib as L
    from neus2_b200 import ops
    g, sdf = load()
    d = L.grid_desc()
    params = np.zeros(L.model_n_params(d), np.uint16)
    params[:4096] = g["weights_fp16"]
    P = torch.from_numpy(params.view(np.int16)).cuda().view(torch.float16)
    got = ops.neus_sdf(d, P, torch.from_numpy(g["x"]).cuda(), sdf_bias=-0.1).float().cpu().numpy()
    assert np.abs(got - sdf).max() <= 1e-3 * np.abs(sdf).max() + 1e-3
    # the stand-alone MLP entry point on the same weights: input = [x - 0.5 | zero encoding]
    z = np.zeros((256, 48), np.float32)
    z[:, :3] = g["x"].astype(np.float16).astype(np.float32) - 0.5
    out, _ = ops.mlp_forward(48, 1, P[:4096].contiguous(), torch.from_numpy(z).cuda().half())
    assert np.abs(out[:, 0].float().cpu().numpy() - 0.1 - sdf).max() <= 2e-3
