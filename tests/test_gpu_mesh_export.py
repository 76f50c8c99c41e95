"""GPU parity of the mesh post-processing through the C ABI: 1-ring normals and centroids, vertex colours from the
network, and Testbed.compute_and_save_marching_cubes_mesh end to end on a briefly trained scene."""
import numpy as np
import pytest
import torch

from test_gpu_raymarch import half
from test_gpu_render import gpu, trained  # noqa: F401  (fixtures)
from test_mesh_export import icosphere
from util import record

pytestmark = pytest.mark.gpu


def test_1ring_matches_oracle(gpu, oracle):
    L, ops = gpu
    verts, idx = icosphere(4)
    ref_n, ref_r = oracle.mesh_1ring(verts, idx)
    n, r = ops.mesh_1ring(torch.from_numpy(verts).cuda(), torch.from_numpy(idx.view(np.int32)).cuda(), want_ring=True)
    # float atomics add in another order than the oracle's double sums
    np.testing.assert_allclose(n.cpu().numpy(), ref_n, rtol=1e-4, atol=1e-8)
    np.testing.assert_allclose(r.cpu().numpy(), ref_r, rtol=1e-5, atol=1e-6)
    # a second call starts from zero again
    n2 = ops.mesh_1ring(torch.from_numpy(verts).cuda(), torch.from_numpy(idx.view(np.int32)).cuda())
    np.testing.assert_allclose(n2.cpu().numpy(), ref_n, rtol=1e-4, atol=1e-8)
    # no triangles: zeros
    z = ops.mesh_1ring(torch.from_numpy(verts).cuda(), torch.zeros(0, dtype=torch.int32, device="cuda"))
    assert not z.cpu().numpy().any()


@pytest.mark.parametrize("linear_colors", [False, True])
def test_vertex_colors_match_oracle(gpu, oracle, trained, linear_colors):
    L, ops = gpu
    verts, _ = icosphere(3)
    d = oracle.grid_desc()
    ref = oracle.mesh_vertex_colors(d, trained["params_bits"], verts, linear_colors=linear_colors)
    got = ops.mesh_vertex_colors(L.grid_desc(), half(trained["params_bits"]), -0.1, torch.from_numpy(verts).cuda(),
                                 linear_colors=linear_colors, chunk=256).cpu().numpy()  # several network calls
    err = np.abs(got - ref).max()
    record("mesh_vertex_colors_linear" if linear_colors else "mesh_vertex_colors", max_abs_err=float(err))
    assert err < 5e-3
    assert got.min() >= 0.0 and got.max() <= 1.0 and got.std() > 0.01


def test_compute_and_save_mesh(gpu, oracle, trained, tmp_path):
    L, ops = gpu
    tb = trained["tb"]
    for ext in ("obj", "ply"):
        path = tmp_path / f"sphere.{ext}"
        mesh = tb.compute_and_save_marching_cubes_mesh(path, resolution=96)
        nv, nt = len(mesh["verts"]), len(mesh["indices"]) // 3
        assert nv > 2000 and nt > 4000
        # the same arrays through the oracle's writer give the same file
        ref = tmp_path / f"ref.{ext}"
        oracle.save_mesh(ref, mesh["verts"], mesh["normals"], mesh["colors"], mesh["indices"])
        assert path.read_bytes() == ref.read_bytes()
    # the surface is the training sphere: radius 0.3 around the centre, normals all on one side, colours plausible
    rad = np.linalg.norm(mesh["verts"] - 0.5, axis=1)
    assert abs(np.median(rad) - 0.3) < 0.01
    unit = mesh["normals"] / np.maximum(np.linalg.norm(mesh["normals"], axis=1, keepdims=True), 1e-20)
    side = (unit * (mesh["verts"] - 0.5)).sum(1) / rad
    assert np.mean(np.sign(side) == np.sign(np.median(side))) > 0.99 and abs(np.median(side)) > 0.9
    ref_n, _ = oracle.mesh_1ring(mesh["verts"], mesh["indices"])
    np.testing.assert_allclose(mesh["normals"], ref_n, rtol=1e-3, atol=1e-9)
    assert 0.05 < mesh["colors"].mean() < 0.95


def test_mesh_postprocessing_equals_the_reference(gpu, tmp_path):
    """compute_mesh_1ring and save_mesh of the reference (src/marching_cubes.cu:720-738, :824-976, linked unmodified into
    oracle/_ref/libref_testbed.so) on the same mesh: 1-ring sums and normals within the rounding of float atomics in another order,
    and -- given the same normals and colours -- the OBJ and PLY files byte for byte."""
    import ctypes as C
    import os
    L, ops = gpu
    lib_path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "libref_testbed.so")
    if not os.path.exists(lib_path):
        pytest.skip("oracle/_ref/libref_testbed.so was not built: no reference checkout at build time")
    lib = C.CDLL(lib_path)
    verts, idx = icosphere(4)
    verts = np.ascontiguousarray(verts * 0.3 + 0.5, np.float32)
    idx = np.ascontiguousarray(idx).view(np.uint32)
    n = verts.shape[0]
    rng = np.random.default_rng(5)
    colors = rng.uniform(0, 1, (n, 3)).astype(np.float32)
    ring, normals = np.zeros((n, 4), np.float32), np.zeros((n, 3), np.float32)
    mine_n, mine_r = ops.mesh_1ring(torch.from_numpy(verts).cuda(), torch.from_numpy(idx.view(np.int32)).cuda(), want_ring=True)
    mine_n, mine_r = mine_n.cpu().numpy(), mine_r.cpu().numpy()
    ptr = lambda a: a.ctypes.data_as(C.c_void_p)
    offset = np.array([0.5, 0.5, 0.5], np.float32)
    for invert in (0, 1):
        obj, ply = tmp_path / f"ref{invert}.obj", tmp_path / f"ref{invert}.ply"
        rc = lib.ref_mesh_postprocess(C.c_uint32(n), ptr(verts), C.c_uint32(idx.size), ptr(idx), ptr(ring), ptr(normals), ptr(mine_n), ptr(colors),
                                      str(obj).encode(), str(ply).encode(), C.c_float(0.33), ptr(offset), C.c_int(invert))
        assert rc == 0
        np.testing.assert_allclose(mine_n, normals, rtol=1e-4, atol=1e-8)
        np.testing.assert_allclose(mine_r, ring, rtol=1e-5, atol=1e-6)
        for ref_file in (obj, ply):
            mine_file = tmp_path / ("mine%d%s" % (invert, ref_file.suffix))
            ops.save_mesh(mine_file, verts, mine_n, colors, idx, nerf_scale=0.33, nerf_offset=(0.5, 0.5, 0.5), invert_normals=bool(invert))
            a, b = mine_file.read_bytes(), ref_file.read_bytes()
            if a != b:
                la, lb = a.split(b"\n"), b.split(b"\n")
                bad = [(k, x, y) for k, (x, y) in enumerate(zip(la, lb)) if x != y]
                raise AssertionError("%s: %d of %d lines differ, first: line %d %r (this repository) %r (reference)" % (ref_file.name, len(bad), len(lb), *bad[0]))
