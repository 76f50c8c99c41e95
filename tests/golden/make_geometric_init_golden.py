"""Generates tests/golden/geometric_init.npz from the only numeric fixture the reference ships for this path:
utils/mlp_weights.txt, the sphere-initialised SDF-MLP weights (64x48 + 16x64 floats, row-major [out][in],
include/neural-graphics-primitives/nerf_network.h:774-823).

Run where a checkout of the reference is at hand:  NEUS2_REFERENCE=<checkout> python tests/golden/make_geometric_init_golden.py

The golden file holds (a) the weights rounded to fp16 (the precision the networks run in), (b) 256 seeded query points,
(c) the SDF-net output of the CPU oracle for them with an all-zero hash grid, and (d) structural facts of the file that
pin the weight layout: only the xyz input columns of the first layer are non-zero and every last-layer weight equals
sqrt(pi)/sqrt(64)."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
REF = os.environ.get("NEUS2_REFERENCE") or (sys.argv[1] if len(sys.argv) > 1 else None)


def main():
    if not REF:
        raise SystemExit("set NEUS2_REFERENCE (or pass the path) to a checkout of 19reborn/NeuS2")
    from oracle import oracle as O
    w = np.loadtxt(os.path.join(REF, "utils", "mlp_weights.txt"), dtype=np.float64)
    assert w.size == 64 * 48 + 16 * 64
    W1, W2 = w[:3072].reshape(64, 48), w[3072:].reshape(16, 64)
    rng = np.random.default_rng(2024)
    x = rng.random((256, 3), dtype=np.float32)
    d = O.grid_desc()
    params = np.zeros(O.model_n_params(d), np.uint16)
    params[:4096] = O.f16_bits(w)
    sdf = O.neus_sdf(d, params, x, sdf_bias=-0.1)
    np.savez_compressed(os.path.join(ROOT, "tests", "golden", "geometric_init.npz"),
                        weights_fp16=O.f16_bits(w), x=x, sdf_fp16=sdf,
                        nonzero_input_columns=np.flatnonzero(np.abs(W1).sum(0) > 0),
                        w2_min=W2.min(), w2_max=W2.max(), w1_xyz_std=W1[:, :3].std())


if __name__ == "__main__":
    main()
