"""Mesh export on the host: the library's writer (all host threads, one buffer per thread) against the oracle's serial
restatement of the reference's fprintf calls -- the files must be identical byte for byte -- and the oracle's 1-ring
normals on a closed mesh."""
import numpy as np
import pytest


def icosphere(subdiv=2):
    t = (1.0 + 5.0 ** 0.5) / 2.0
    v = [(-1, t, 0), (1, t, 0), (-1, -t, 0), (1, -t, 0), (0, -1, t), (0, 1, t), (0, -1, -t), (0, 1, -t), (t, 0, -1), (t, 0, 1),
         (-t, 0, -1), (-t, 0, 1)]
    f = [(0, 11, 5), (0, 5, 1), (0, 1, 7), (0, 7, 10), (0, 10, 11), (1, 5, 9), (5, 11, 4), (11, 10, 2), (10, 7, 6), (7, 1, 8),
         (3, 9, 4), (3, 4, 2), (3, 2, 6), (3, 6, 8), (3, 8, 9), (4, 9, 5), (2, 4, 11), (6, 2, 10), (8, 6, 7), (9, 8, 1)]
    v = [np.array(p, np.float64) / np.linalg.norm(p) for p in v]
    for _ in range(subdiv):
        cache, nf = {}, []

        def mid(a, b):
            k = (min(a, b), max(a, b))
            if k not in cache:
                m = v[a] + v[b]
                v.append(m / np.linalg.norm(m))
                cache[k] = len(v) - 1
            return cache[k]
        for a, b, c in f:
            ab, bc, ca = mid(a, b), mid(b, c), mid(c, a)
            nf += [(a, ab, ca), (b, bc, ab), (c, ca, bc), (ab, bc, ca)]
        f = nf
    return (np.array(v) * 0.3 + 0.5).astype(np.float32), np.array(f, np.uint32).reshape(-1)


def test_oracle_1ring_on_a_sphere(oracle):
    verts, idx = icosphere(2)
    normals, ring = oracle.mesh_1ring(verts, idx)
    radial = verts - 0.5
    radial /= np.linalg.norm(radial, axis=1, keepdims=True)
    unit = normals / np.linalg.norm(normals, axis=1, keepdims=True)
    # (pb - pa) x (pa - pc) points inward for counter-clockwise triangles seen from outside
    assert np.all((unit * radial).sum(1) < -0.99)
    # the 1-ring centroid of a vertex of a convex mesh lies inside, close to the vertex; each neighbour is counted twice
    cent = ring[:, :3] / ring[:, 3:]
    assert np.all(np.linalg.norm(cent - 0.5, axis=1) < 0.3) and np.all(np.linalg.norm(cent - verts, axis=1) < 0.05)
    counts = np.bincount(idx, minlength=len(verts))
    np.testing.assert_array_equal(ring[:, 3], 2.0 * counts)


@pytest.mark.parametrize("ext", ["obj", "ply"])
@pytest.mark.parametrize("subdiv,invert", [(1, False), (5, True), (5, False)])
def test_writer_matches_the_serial_restatement(oracle, tmp_path, ext, subdiv, invert):
    from neus2_b200 import ops
    verts, idx = icosphere(subdiv)  # subdiv 5: 10242 vertices, 20480 triangles -> several formatting threads
    rng = np.random.default_rng(subdiv)
    normals, _ = oracle.mesh_1ring(verts, idx)
    normals[3] = 0.0  # a vertex without a normal stays (0, 0, 0)
    colors = rng.uniform(-0.2, 1.2, verts.shape).astype(np.float32)  # out-of-range colours are clamped
    a, b = tmp_path / f"lib.{ext}", tmp_path / f"ref.{ext}"
    kw = dict(nerf_scale=0.33, nerf_offset=(0.5, 0.4, 0.6), invert_normals=invert)
    ops.save_mesh(a, verts, normals, colors, idx, **kw)
    oracle.save_mesh(b, verts, normals, colors, idx, **kw)
    ta, tb = a.read_bytes(), b.read_bytes()
    assert len(ta) > 100 * len(verts) // 4 and ta == tb
    lines = ta.decode().splitlines()
    if ext == "obj":
        assert sum(l.startswith("v ") for l in lines) == len(verts) and sum(l.startswith("vn ") for l in lines) == len(verts)
        faces = [l for l in lines if l.startswith("f ")]
        assert len(faces) == len(idx) // 3
        first = [int(tok.split("//")[0]) - 1 for tok in faces[0].split()[1:]]
        assert first == (list(idx[:3]) if invert else list(idx[:3][::-1]))
    else:
        assert lines[0] == "ply" and f"element vertex {len(verts)}" in lines and f"element face {len(idx) // 3}" in lines
        assert len(lines) == 16 + len(verts) + len(idx) // 3


def test_writer_errors_and_empty_mesh(oracle, tmp_path):
    from neus2_b200 import _lib as L
    from neus2_b200 import ops
    e = np.zeros((0, 3), np.float32)
    ops.save_mesh(tmp_path / "empty.obj", e, e, e, np.zeros(0, np.uint32))
    assert (tmp_path / "empty.obj").read_bytes() == b""
    with pytest.raises(L.Neus2bError):
        ops.save_mesh(tmp_path / "no_such_dir" / "x.obj", e, e, e, np.zeros(0, np.uint32))
    verts, idx = icosphere(0)
    with pytest.raises(L.Neus2bError):
        ops.save_mesh(tmp_path / "bad.obj", verts, verts, verts, idx[:-1])
