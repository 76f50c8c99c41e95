"""GPU parity: every C-ABI entry point of libneus2b.so against the CPU oracle on the same seeded inputs.

Tolerances: index / integer work bit-exact; fp16 outputs within 1e-3 relative (see util.fp16_close_fraction);
parameter gradients cosine >= 0.999 against the oracle's fp64 accumulation."""
import numpy as np
import pytest
import torch

from util import check_fp16, check_grad, cosine, model, record, to_lib_desc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gpu():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    from neus2_b200 import _lib as L
    from neus2_b200 import ops
    L.lib()  # raises if the CUDA extension is missing -- there is no fallback
    return L, ops


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.view(dtype) if t.element_size() == torch.empty((), dtype=dtype).element_size() else t.to(dtype)
    return t.cuda()


def half(a_bits):
    return torch.from_numpy(np.ascontiguousarray(a_bits).view(np.int16)).cuda().view(torch.float16)


def bits(t):
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def f32(t_half):
    return t_half.detach().float().cpu().numpy()


GRID_CASES = [
    dict(n=65536, L=16, log2T=19, base=16, scale=1.447),   # BASELINE config 0
    dict(n=1, L=16, log2T=19, base=16, scale=1.447),
    dict(n=129, L=4, log2T=10, base=4, scale=1.7),
    dict(n=4099, L=14, log2T=19, base=16, scale=1.4525),   # shipped 14-level configuration
    dict(n=1000, L=16, log2T=19, base=16, scale=1.447, n_active=8),
]


@pytest.mark.parametrize("case", GRID_CASES)
def test_grid_forward_and_dydx(gpu, oracle, case):
    L, ops = gpu
    O = oracle
    d, params, coords, rng = model(O, seed=1, grid_amp=0.1, **case)
    ng = O.grid_n_params(d)
    assert L.grid_n_params(to_lib_desc(L, d)) == ng
    off, res, scale, hashed = L.grid_level_table(to_lib_desc(L, d))
    lv = O.grid_levels(d)
    nl = d.n_levels
    assert off[:nl + 1] == list(lv.offset)[:nl + 1] and res == list(lv.res) and hashed == list(lv.hashed)
    assert np.array_equal(np.float32(scale), np.float32(list(lv.scale)))
    grid = params[O.GRID_OFF:O.GRID_OFF + ng]
    x = coords[:, :3].copy()
    x[0] = [0.0, 1.0, 0.5]  # cube faces
    enc_ref, J_ref = O.grid_forward(d, x, grid, want_dydx=True)
    enc, J = ops.grid_forward(to_lib_desc(L, d), dev(x), half(grid), want_dydx=True)
    torch.cuda.synchronize()
    assert np.array_equal(bits(enc), enc_ref), "hash-grid features must be bit-exact (same indices, same fp32 order)"
    assert np.allclose(J.cpu().numpy(), J_ref, rtol=1e-6, atol=1e-7)
    if d.n_active_levels < d.n_levels:
        assert not bits(enc)[:, 2 * d.n_active_levels:].any()


@pytest.mark.parametrize("case", GRID_CASES[:4])
def test_grid_backward_paths(gpu, oracle, case):
    L, ops = gpu
    O = oracle
    d, params, coords, rng = model(O, seed=2, grid_amp=0.1, **case)
    ld = to_lib_desc(L, d)
    ng, n, W = O.grid_n_params(d), coords.shape[0], 2 * d.n_levels
    grid = params[O.GRID_OFF:O.GRID_OFF + ng]
    x = coords[:, :3]
    dy = O.f16_bits(rng.normal(0, 1, (n, W)))
    # a2: dL/dx
    ref = O.grid_backward_input(d, x, grid, dy)
    got = ops.grid_backward_input(ld, dev(x), half(grid), half(dy)).cpu().numpy()
    assert np.allclose(got, ref, rtol=1e-5, atol=1e-4 * np.abs(ref).max())
    # a3: parameter gradient (fp16 atomics vs fp64)
    gref = O.grid_backward_params(d, x, dy)
    g = torch.zeros(ng, dtype=torch.float16, device="cuda")
    ops.grid_backward_params(ld, dev(x), half(dy), g, L.GRAD_OVERWRITE)
    check_grad("grid_bwd_params_n%d_L%d" % (n, d.n_levels), f32(g), gref, min_cos=0.999)
    ops.grid_backward_params(ld, dev(x), half(dy), g, L.GRAD_ACCUMULATE)
    check_grad("grid_bwd_params_acc_n%d_L%d" % (n, d.n_levels), f32(g), 2 * gref, min_cos=0.999)
    # a4: second order
    v = rng.normal(0, 1e-2, (n, 3)).astype(np.float32)
    ge = O.f16_bits(rng.normal(0, 1, (n, W)))
    g2ref, dyref = O.grid_backward_backward_input(d, x, grid, v, ge)
    g2 = torch.zeros(ng, dtype=torch.float16, device="cuda")
    dyenc = ops.grid_backward_backward_input(ld, dev(x), half(grid), dev(v), half(ge), g2, L.GRAD_OVERWRITE)
    check_fp16("grid_bwd_bwd_dy_n%d_L%d" % (n, d.n_levels), f32(dyenc), O.bits_f32(dyref), min_frac=0.9999)
    check_grad("grid_bwd_bwd_grad_n%d_L%d" % (n, d.n_levels), f32(g2), g2ref, min_cos=0.999)


@pytest.mark.parametrize("in_w,nh,n", [(48, 1, 65536), (48, 2, 4113), (32, 1, 500), (64, 2, 77), (48, 1, 1)])
def test_mlp_forward_backward(gpu, oracle, in_w, nh, n):
    L, ops = gpu
    O = oracle
    rng = np.random.default_rng(in_w * 7 + nh)
    npar = 64 * in_w + (nh - 1) * 4096 + 1024
    w = O.f16_bits(rng.uniform(-0.3, 0.3, npar))
    inp = O.f16_bits(rng.normal(0, 1, (n, in_w)))
    out_ref, hid_ref = O.mlp_forward(in_w, nh, w, inp)
    out, hid = ops.mlp_forward(in_w, nh, half(w), half(inp))
    check_fp16("mlp_fwd_%d_%d_%d" % (in_w, nh, n), f32(out), O.bits_f32(out_ref))
    check_fp16("mlp_hid_%d_%d_%d" % (in_w, nh, n), f32(hid), O.bits_f32(hid_ref))
    dout = O.f16_bits(rng.normal(0, 1, (n, 16)))
    # backward from the oracle's activations so both sides see identical ReLU masks
    din_ref, wg_ref = O.mlp_backward(in_w, nh, w, inp, hid_ref, dout)
    din, wg = ops.mlp_backward(in_w, nh, half(w), half(inp), half(hid_ref), half(dout))
    check_fp16("mlp_din_%d_%d_%d" % (in_w, nh, n), f32(din), O.bits_f32(din_ref))
    check_grad("mlp_wgrad_%d_%d_%d" % (in_w, nh, n), wg.cpu().numpy(), wg_ref, min_cos=0.9999, max_rel=5e-3)
    din2, none = ops.mlp_backward(in_w, nh, half(w), half(inp), half(hid_ref), half(dout), mode=L.GRAD_IGNORE)
    assert none is None and torch.equal(din2, din)
    if nh == 1:
        u = O.f16_bits(rng.normal(0, 1, (n, in_w)))
        wg2_ref = O.mlp_backward_backward_input(in_w, w, hid_ref, u, dout)
        wg2 = ops.mlp_backward_backward_input(in_w, half(w), half(hid_ref[:, 0].copy()), half(u), half(dout))
        check_grad("mlp_bwd_bwd_%d_%d" % (in_w, n), wg2.cpu().numpy(), wg2_ref, min_cos=0.9999, max_rel=5e-3)


@pytest.mark.parametrize("in_w,nh,n", [(48, 1, 65536), (48, 2, 4113), (64, 2, 129), (48, 1, 1)])
def test_mlp_forward_tcgen05(gpu, oracle, in_w, nh, n):
    """The tcgen05 / TMEM forward against the oracle and against the mma.sync kernel."""
    L, ops = gpu
    O = oracle
    rng = np.random.default_rng(in_w * 11 + nh)
    npar = 64 * in_w + (nh - 1) * 4096 + 1024
    w = O.f16_bits(rng.uniform(-0.3, 0.3, npar))
    inp = O.f16_bits(rng.normal(0, 1, (n, in_w)))
    out_ref, hid_ref = O.mlp_forward(in_w, nh, w, inp)
    out, hid, status = ops.mlp_forward_tcgen05(in_w, nh, half(w), half(inp))
    torch.cuda.synchronize()
    assert status.item() == 0, "a bounded wait inside the tcgen05 kernel ran out"
    check_fp16("mlp_tc_fwd_%d_%d_%d" % (in_w, nh, n), f32(out), O.bits_f32(out_ref))
    check_fp16("mlp_tc_hid_%d_%d_%d" % (in_w, nh, n), f32(hid), O.bits_f32(hid_ref))
    out2, hid2 = ops.mlp_forward(in_w, nh, half(w), half(inp))
    check_fp16("mlp_tc_vs_mma_%d_%d_%d" % (in_w, nh, n), f32(out), f32(out2))


def test_sh4(gpu, oracle):
    L, ops = gpu
    rng = np.random.default_rng(5)
    d = rng.random((1000, 3), dtype=np.float32)
    ref = oracle.sh4(d)
    got = ops.sh4(dev(d))
    assert np.abs(f32(got) - oracle.bits_f32(ref)).max() <= 1e-3


FUSED_CASES = [
    dict(n=65536, L=16, log2T=19, base=16, scale=1.447),  # BASELINE config 0
    dict(n=1, L=16, log2T=19, base=16, scale=1.447),
    dict(n=17, L=4, log2T=10, base=4, scale=1.7),
    dict(n=5003, L=14, log2T=19, base=16, scale=1.4525),
    dict(n=3000, L=16, log2T=19, base=16, scale=1.447, n_active=10),
]


PATHS = [pytest.param(0, id="mma_sync"), pytest.param(1, id="tcgen05")]


@pytest.fixture(autouse=True)
def _default_path():
    yield
    from neus2_b200 import _lib as L
    L.set_mma_path(L.MMA_TCGEN05)


@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("case", FUSED_CASES)
def test_fused_forward(gpu, oracle, case, path):
    L, ops = gpu
    O = oracle
    L.set_mma_path(path)
    d, params, coords, rng = model(O, seed=3, grid_amp=0.05, **case)
    ref = O.bits_f32(O.neus_forward(d, params, coords, sdf_bias=-0.1))
    out = f32(ops.neus_forward(to_lib_desc(L, d), half(params), dev(coords), sdf_bias=-0.1))
    assert L.device_error_flags() == 0
    tag = "fused_fwd_p%d_n%d_L%d_a%d" % (path, coords.shape[0], d.n_levels, d.n_active_levels)
    check_fp16(tag + "_rgb", out[:, 0:3], ref[:, 0:3], min_frac=0.9999, min_cos=0.99999)
    check_fp16(tag + "_sdf", out[:, 3], ref[:, 3], min_frac=0.9999, min_cos=0.99999)
    check_fp16(tag + "_normal", out[:, 4:7], ref[:, 4:7], min_frac=0.9999, min_cos=0.99999)
    assert np.array_equal(out[:, 7:11], ref[:, 7:11])
    sdf = f32(ops.neus_sdf(to_lib_desc(L, d), half(params), dev(coords[:, :3].copy()), sdf_bias=-0.1))
    sref = O.bits_f32(O.neus_sdf(d, params, coords[:, :3]))
    check_fp16(tag + "_sdf_only", sdf, sref, min_frac=0.9999)


def test_fused_forward_device_count(gpu, oracle):
    L, ops = gpu
    O = oracle
    d, params, coords, rng = model(O, seed=4, n=1000, grid_amp=0.05)
    n_dev = torch.tensor([333], dtype=torch.int32, device="cuda")
    out = torch.zeros((1000, 16), dtype=torch.float16, device="cuda")
    ops.neus_forward(to_lib_desc(L, d), half(params), dev(coords), n_dev=n_dev, out=out)
    assert out[333:].abs().max().item() == 0 and out[:333].abs().sum().item() > 0


@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("case", FUSED_CASES)
def test_fused_train_gradients(gpu, oracle, case, path):
    L, ops = gpu
    O = oracle
    L.set_mma_path(path)
    d, params, coords, rng = model(O, seed=5, grid_amp=0.05, **case)
    n, ng = coords.shape[0], O.grid_n_params(d)
    g = np.zeros((n, 16), np.float32)
    g[:, 0:3] = rng.normal(0, 0.5, (n, 3))
    g[:, 3] = rng.normal(0, 0.5, n)
    g[:, 4:7] = rng.normal(0, 10.0, (n, 3))
    g[:, 7] = rng.normal(0, 0.1, n)
    g[:, 8:11] = rng.normal(0, 0.02, (n, 3))
    gb = O.f16_bits(g)
    ref = O.neus_backward(d, params, coords, gb, indeed_batch_size=max(n, 256))
    gm = torch.zeros(12288, dtype=torch.float32, device="cuda")
    gg = torch.zeros(ng, dtype=torch.float16, device="cuda")
    gv = torch.zeros(4, dtype=torch.float32, device="cuda")
    ops.neus_train(to_lib_desc(L, d), half(params), dev(coords), half(gb), max(n, 256), gm, gg, gv)
    torch.cuda.synchronize()
    assert L.device_error_flags() == 0
    tag = "fused_train_p%d_n%d_L%d_a%d_" % (path, n, d.n_levels, d.n_active_levels)
    gm = gm.cpu().numpy()
    for name, a, b in [("sdf_w1", 0, 3072), ("sdf_w2", 3072, 4096), ("rgb_w1", 4096, 7168), ("rgb_w2", 7168, 11264),
                       ("rgb_w3", 11264, 12288)]:
        if np.abs(ref[a:b]).max() > 0:
            check_grad(tag + name, gm[a:b], ref[a:b], min_cos=0.999)
    if n > 1:
        check_grad(tag + "grid", f32(gg), ref[O.GRID_OFF:O.GRID_OFF + ng], min_cos=0.999)
    vref = ref[O.GRID_OFF + ng]
    assert abs(gv[0].item() - vref) <= 1e-3 * max(1.0, abs(vref)) + 1e-3 * np.sqrt(n)
    record(tag + "var", got=gv[0].item(), ref=vref)


def test_fused_train_accumulates(gpu, oracle):
    L, ops = gpu
    O = oracle
    d, params, coords, rng = model(O, seed=6, n=2048, grid_amp=0.05)
    ng = O.grid_n_params(d)
    gb = O.f16_bits(rng.normal(0, 0.3, (2048, 16)))
    gm = torch.zeros(12288, dtype=torch.float32, device="cuda")
    gg = torch.zeros(ng, dtype=torch.float16, device="cuda")
    gv = torch.zeros(4, dtype=torch.float32, device="cuda")
    args = (to_lib_desc(L, d), half(params), dev(coords), half(gb), 2048, gm, gg, gv)
    ops.neus_train(*args)
    one = gm.clone()
    ops.neus_train(*args)
    assert cosine(gm.cpu().numpy(), 2 * one.cpu().numpy()) > 0.99999
