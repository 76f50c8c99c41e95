"""CPU checks of the dynamic-sequence pieces: the oracle's restatement of the DeltaNetwork against torch autograd, and the
library's host-side accumulation of the global movement against the oracle's."""
import numpy as np
import torch

DELTA = np.array([0.02, -0.01, 0.03, 0.0, 0.98, 0.1, -0.05, 0.07, 1.02, 0.12, 0.0, 0.0], np.float32)


def test_oracle_delta_matches_autograd(oracle):
    O = oracle
    rng = np.random.default_rng(0)
    bits = O.f16_bits(DELTA)
    n = 500
    coords = rng.random((n, 7)).astype(np.float32)
    out = O.delta_forward(bits, coords)
    R = O.rotation_6d_to_matrix(bits[4:10])
    assert np.abs(R.T @ R - np.eye(3)).max() < 1e-6 and abs(np.linalg.det(R) - 1) < 1e-6
    d = torch.tensor(O.bits_f32(bits).astype(np.float64), requires_grad=True)
    a1, a2, t = d[4:7], d[7:10], d[0:3]
    b1 = a1 / a1.norm()
    u2 = a2 - (b1 @ a2) * b1
    b2 = u2 / u2.norm()
    Rm = torch.stack([b1, b2, torch.linalg.cross(b1, b2)], 1)
    c = torch.tensor(coords.astype(np.float64))
    pos = (Rm @ (c[:, :3] + t).T).T
    assert np.abs(pos.detach().numpy() - out[:, :3]).max() < 1e-6
    dirs = ((Rm @ (c[:, 4:] * 2 - 1).T).T + 1) / 2
    assert np.abs(dirs.detach().numpy() - out[:, 4:]).max() < 1e-6 and np.array_equal(out[:, 3], coords[:, 3])
    lvec = torch.tensor(rng.normal(size=(n, 3)))
    (pos * lvec).sum().backward()
    g = O.delta_backward(bits, coords, lvec.numpy().astype(np.float32))
    assert np.abs(g - d.grad.numpy()).max() <= 1e-6 * np.abs(d.grad.numpy()).max()


def test_host_accumulation_matches_oracle(oracle):
    from neus2_b200 import ops
    O = oracle
    R, t = np.eye(3, dtype=np.float32), np.zeros(3, np.float32)
    Rg, tg = R.copy(), t.copy()
    for k in range(5):
        dk = DELTA.copy()
        dk[:3] *= 0.3 * (k + 1)
        dk[5] += 0.02 * k
        R, t = O.accumulate_global_movement(O.f16_bits(dk), R, t)
        Rg, tg = ops.movement_accumulate(O.f16_bits(dk), Rg, tg)
        assert np.array_equal(R, Rg) and np.array_equal(t, tg)
    assert np.abs(R @ R.T - np.eye(3)).max() < 5e-3  # a rotation, up to the fp16 storage of the accumulated matrix
    assert np.array_equal(R.astype(np.float16).astype(np.float32), R)
