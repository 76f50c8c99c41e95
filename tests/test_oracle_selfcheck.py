"""Self-validation of the CPU oracle (it has no reference tests to lean on): the hand-derived first- and second-order
backward passes are compared with torch autograd (double backward) on an fp64 dense restatement of the same graph,
and dy/dx with central finite differences."""
import numpy as np
import pytest
import torch

PRIMES = (1, 2654435761, 805459861)


def torch_grid(O, d, x, theta):
    """fp64 differentiable restatement of the multiresolution hash encoding. theta: [n_entries, 2]."""
    lv = O.grid_levels(d)
    feats = []
    for l in range(d.n_levels):
        if l >= d.n_active_levels:
            feats.append(torch.zeros(x.shape[0], 2, dtype=torch.float64))
            continue
        scale = float(np.float32(lv.scale[l]))
        res, n = int(lv.res[l]), int(lv.offset[l + 1] - lv.offset[l])
        pos = x * scale + 0.5
        c0 = torch.floor(pos.detach())
        f = pos - c0
        c0 = c0.to(torch.int64)
        acc = 0
        for k in range(8):
            bits = [(k >> e) & 1 for e in range(3)]
            cc = [c0[:, e] + bits[e] for e in range(3)]
            w = 1.0
            for e in range(3):
                w = w * (f[:, e] if bits[e] else 1.0 - f[:, e])
            if lv.hashed[l]:
                idx = ((cc[0] * PRIMES[0]) & 0xFFFFFFFF) ^ ((cc[1] * PRIMES[1]) & 0xFFFFFFFF) ^ ((cc[2] * PRIMES[2]) & 0xFFFFFFFF)
            else:
                idx = (cc[0] + cc[1] * res + cc[2] * res * res) & 0xFFFFFFFF
            idx = idx % n + int(lv.offset[l])
            acc = acc + w[:, None] * theta[idx]
        feats.append(acc)
    return torch.cat(feats, 1)


def sh4_torch(dir01):
    x, y, z = (dir01 * 2 - 1).unbind(1)
    xy, xz, yz, x2, y2, z2 = x * y, x * z, y * z, x * x, y * y, z * z
    return torch.stack([
        torch.full_like(x, 0.28209479177387814), -0.48860251190291987 * y, 0.48860251190291987 * z, -0.48860251190291987 * x,
        1.0925484305920792 * xy, -1.0925484305920792 * yz, 0.94617469575755997 * z2 - 0.31539156525251999,
        -1.0925484305920792 * xz, 0.54627421529603959 * x2 - 0.54627421529603959 * y2,
        0.59004358992664352 * y * (-3.0 * x2 + y2), 2.8906114426405538 * xy * z, 0.45704579946446572 * y * (1.0 - 5.0 * z2),
        0.3731763325901154 * z * (5.0 * z2 - 3.0), 0.45704579946446572 * x * (1.0 - 5.0 * z2),
        1.4453057213202769 * z * (x2 - y2), 0.59004358992664352 * x * (-x2 + 3.0 * y2)], 1)


def small_model(O, seed=0, n=512, L=4, log2T=8, scale=1.7):
    rng = np.random.default_rng(seed)
    d = O.grid_desc(n_levels=L, log2_hashmap_size=log2T, base_resolution=4, per_level_scale=scale)
    ng = O.grid_n_params(d)
    params = np.zeros(O.model_n_params(d), np.uint16)
    params[:O.MLP_N] = O.f16_bits(rng.uniform(-0.35, 0.35, O.MLP_N))
    params[O.GRID_OFF:O.GRID_OFF + ng] = O.f16_bits(rng.uniform(-0.5, 0.5, ng))
    params[O.GRID_OFF + ng] = O.f16_bits([0.3])[0]
    coords = np.zeros((n, 7), np.float32)
    coords[:, :3] = rng.random((n, 3), dtype=np.float32) * 0.98 + 0.01
    coords[:, 4:] = rng.random((n, 3), dtype=np.float32)
    return d, params, coords, rng


def torch_graph(O, d, params, coords):
    P = torch.tensor(O.bits_f32(params).astype(np.float64), requires_grad=True)
    ng = O.grid_n_params(d)
    W1s = P[0:3072].view(64, 48)
    W2s = P[3072:4096].view(16, 64)
    W1c = P[4096:4096 + 3072].view(64, 48)
    W2c = P[7168:7168 + 4096].view(64, 64)
    W3c = P[11264:12288].view(16, 64)
    theta = P[O.GRID_OFF:O.GRID_OFF + ng].view(-1, 2)
    x = torch.tensor(coords[:, :3].astype(np.float64), requires_grad=True)
    dirs = torch.tensor(coords[:, 4:].astype(np.float64))
    n = x.shape[0]
    enc = torch_grid(O, d, x, theta)
    zs = torch.cat([x - 0.5, enc, torch.zeros(n, 48 - 3 - enc.shape[1], dtype=torch.float64)], 1)
    hs = torch.relu(zs @ W1s.T)
    ys = hs @ W2s.T
    normal, = torch.autograd.grad(ys[:, 0].sum(), x, create_graph=True)
    zc = torch.cat([ys, sh4_torch(dirs), x, normal, torch.zeros(n, 10, dtype=torch.float64)], 1)
    o = torch.relu(torch.relu(zc @ W1c.T) @ W2c.T) @ W3c.T
    return P, x, enc, ys, normal, o


def cosine(a, b):
    a, b = np.asarray(a, np.float64).ravel(), np.asarray(b, np.float64).ravel()
    return float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b) + 1e-300))


def test_forward_matches_dense_restatement(oracle):
    O = oracle
    d, params, coords, _ = small_model(O)
    _, _, enc, ys, normal, o = torch_graph(O, d, params, coords)
    out = O.bits_f32(O.neus_forward(d, params, coords, sdf_bias=-0.1))
    def frac_close(a, b, atol, rtol):  # fp16 rounding can flip a ReLU that sits at zero: allow a few outliers
        return np.isclose(a, b, atol=atol, rtol=rtol).mean()
    assert frac_close(out[:, 0:3], o[:, 0:3].detach().numpy(), 3e-2, 3e-2) > 0.99
    assert np.allclose(out[:, 3], ys[:, 0].detach().numpy() - 0.1, atol=5e-3, rtol=5e-3)
    assert frac_close(out[:, 4:7], normal.detach().numpy(), 3e-2, 2e-2) > 0.99
    assert cosine(out[:, 4:7], normal.detach().numpy()) > 0.9999
    e = O.bits_f32(O.grid_forward(d, coords[:, :3], params[O.GRID_OFF:O.GRID_OFF + O.grid_n_params(d)]))
    assert np.allclose(e, enc.detach().numpy(), atol=1e-3, rtol=1e-3)


def test_backward_first_and_second_order_match_autograd(oracle):
    O = oracle
    d, params, coords, rng = small_model(O, seed=1)
    n = coords.shape[0]
    g = np.zeros((n, 16), np.float32)
    g[:, 0:4] = rng.normal(0, 1, (n, 4))
    g[:, 4:7] = rng.normal(0, 64.0, (n, 3))   # eikonal rows are later divided by the batch size
    g[:, 7] = rng.normal(0, 1, n)
    g[:, 8:11] = rng.normal(0, 0.5, (n, 3))
    gb = O.f16_bits(g)
    gq = O.bits_f32(gb).astype(np.float64)
    P, x, enc, ys, normal, o = torch_graph(O, d, params, coords)
    G = torch.tensor(gq)
    ng = O.grid_n_params(d)
    L = (G[:, 0:3] * o[:, 0:3]).sum() + (G[:, 3] * ys[:, 0]).sum() + ((G[:, 4:7] / n + G[:, 8:11]) * normal).sum() \
        + (G[:, 7]).sum() * P[O.GRID_OFF + ng]
    L.backward()
    ref = P.grad.numpy()
    got = O.neus_backward(d, params, coords, gb, indeed_batch_size=n)
    for name, a, b in [("sdf_w1", 0, 3072), ("sdf_w2", 3072, 4096), ("rgb_w1", 4096, 7168), ("rgb_w2", 7168, 11264),
                       ("rgb_w3", 11264, 12288), ("grid", O.GRID_OFF, O.GRID_OFF + ng)]:
        c = cosine(got[a:b], ref[a:b])
        rel = np.linalg.norm(got[a:b] - ref[a:b]) / np.linalg.norm(ref[a:b])
        assert c > 0.9995 and rel < 3e-2, (name, c, rel)
    assert abs(got[O.GRID_OFF + ng] - ref[O.GRID_OFF + ng]) < 1e-6 * n


def test_second_order_term_alone(oracle):
    """Only the normal feeds the loss: every parameter gradient then comes from the second-order path."""
    O = oracle
    d, params, coords, rng = small_model(O, seed=2)
    params[4096:O.MLP_N] = 0  # colour net off, so its input-gradient rows 35-37 vanish
    n = coords.shape[0]
    g = np.zeros((n, 16), np.float32)
    g[:, 8:11] = rng.normal(0, 1.0, (n, 3))
    gb = O.f16_bits(g)
    P, x, enc, ys, normal, o = torch_graph(O, d, params, coords)
    L = (torch.tensor(O.bits_f32(gb).astype(np.float64))[:, 8:11] * normal).sum()
    L.backward()
    ref = P.grad.numpy()
    got = O.neus_backward(d, params, coords, gb, indeed_batch_size=n)
    ng = O.grid_n_params(d)
    for name, a, b in [("sdf_w1", 0, 3072), ("sdf_w2", 3072, 4096), ("grid", O.GRID_OFF, O.GRID_OFF + ng)]:
        c = cosine(got[a:b], ref[a:b])
        assert c > 0.9995, (name, c)
    assert np.abs(got[4096:O.MLP_N]).max() == 0


def test_dydx_finite_differences(oracle):
    O = oracle
    d, params, coords, _ = small_model(O, seed=3, n=256)
    grid = params[O.GRID_OFF:O.GRID_OFF + O.grid_n_params(d)]
    x = coords[:, :3].astype(np.float64)
    _, J = O.grid_forward(d, coords[:, :3], grid, want_dydx=True)
    P = torch.tensor(O.bits_f32(params).astype(np.float64))
    theta = P[O.GRID_OFF:O.GRID_OFF + O.grid_n_params(d)].view(-1, 2)
    h = 1e-6
    for e in range(3):
        xp, xm = x.copy(), x.copy()
        xp[:, e] += h
        xm[:, e] -= h
        fd = (torch_grid(O, d, torch.tensor(xp), theta) - torch_grid(O, d, torch.tensor(xm), theta)).numpy() / (2 * h)
        ok = np.isfinite(fd).all(1) & (np.abs(fd).max(1) < 1e4)  # skip samples that straddle a cell boundary
        assert ok.mean() > 0.95
        assert np.allclose(J[ok, :, e], fd[ok], atol=2e-3, rtol=2e-3)


def test_component_calls_compose_to_graph(oracle):
    """The component entry points (grid/mlp fwd, bwd, bwd-bwd), wired as nerf_network.h wires them, give the
    same parameter gradient as the fused oracle graph."""
    O = oracle
    d, params, coords, rng = small_model(O, seed=4, n=300)
    n, ng, W = coords.shape[0], O.grid_n_params(d), 2 * d.n_levels
    grid = params[O.GRID_OFF:O.GRID_OFF + ng]
    g = O.f16_bits(rng.normal(0, 1, (n, 16)))
    gf = O.bits_f32(g)
    x = coords[:, :3]
    enc, J = O.grid_forward(d, x, grid, True)
    zs = np.zeros((n, 48), np.uint16)
    zs[:, :3] = O.f16_bits(O.bits_f32(O.f16_bits(x)) - 0.5)
    zs[:, 3:3 + W] = enc
    ws, wc = params[:O.SDF_N], params[O.SDF_N:O.MLP_N]
    ys, hs = O.mlp_forward(48, 1, ws, zs)
    e0 = np.zeros((n, 16), np.float32)
    e0[:, 0] = 1
    gz, _ = O.mlp_backward(48, 1, ws, zs, hs, O.f16_bits(e0), want_wgrad=False)
    nrm = O.grid_backward_input(d, x, grid, gz[:, 3:3 + W]) + O.bits_f32(gz[:, :3])
    zc = np.zeros((n, 48), np.uint16)
    zc[:, :16] = ys
    zc[:, 16:32] = O.sh4(coords[:, 4:])
    zc[:, 32:35] = O.f16_bits(x)
    zc[:, 35:38] = O.f16_bits(nrm)
    o, hc = O.mlp_forward(48, 2, wc, zc)
    out = O.neus_forward(d, params, coords)
    assert np.array_equal(out[:, :3], o[:, :3])
    assert np.array_equal(out[:, 4:7], O.f16_bits(nrm))
    # backward
    d3 = np.zeros((n, 16), np.float32)
    d3[:, :3] = gf[:, :3]
    dzc, wgc = O.mlp_backward(48, 2, wc, zc, hc, O.f16_bits(d3))
    dys = O.bits_f32(dzc[:, :16]).copy()
    dys[:, 0] = O.bits_f32(O.f16_bits(dys[:, 0] + gf[:, 3]))
    dzs, wgs = O.mlp_backward(48, 1, ws, zs, hs, O.f16_bits(dys))
    gg = O.grid_backward_params(d, x, dzs[:, 3:3 + W])
    v = O.bits_f32(dzc[:, 35:38]) + gf[:, 4:7] / np.float32(n) + gf[:, 8:11]
    gg, dyenc = O.grid_backward_backward_input(d, x, grid, v, gz[:, 3:3 + W], grad=gg)
    u = np.zeros((n, 48), np.uint16)
    u[:, :3] = O.f16_bits(v)
    u[:, 3:3 + W] = dyenc
    wgs += O.mlp_backward_backward_input(48, ws, hs, u, O.f16_bits(e0))
    full = O.neus_backward(d, params, coords, g, indeed_batch_size=n)
    assert np.allclose(full[:O.SDF_N], wgs, rtol=1e-9, atol=1e-9)
    assert np.allclose(full[O.SDF_N:O.MLP_N], wgc, rtol=1e-9, atol=1e-9)
    assert np.allclose(full[O.GRID_OFF:O.GRID_OFF + ng], gg, rtol=1e-9, atol=1e-9)
