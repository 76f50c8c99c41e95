"""Mesh extraction sharded by z-slab (one slab per rank) and the merge that gives back exactly the single-grid mesh.

Rank r runs marching cubes on the lattice layers [z0_r, z1_r] (inclusive: the cells of a slab need the next layer) with
vertex positions in the whole grid's frame.  Vertices and triangles are numbered by cell in z-major order, so the merged
mesh is the concatenation of the slabs in z order, minus each slab's copies of the vertices that lie in its last layer
(edges inside the plane z = z1_r: the next slab owns them as its first layer).  The copies have bit-identical positions,
which is how the indices that referred to them are redirected."""
import numpy as np


def slab_ranges(res_z, world):
    """[(z0, n_layers)] per rank: cells [z0, z0 + n_layers - 1) and the lattice layers they touch.  Ranks beyond the number of
    cell layers get (z0, 0)."""
    cells = res_z - 1
    out = []
    for r in range(world):
        a, b = cells * r // world, cells * (r + 1) // world
        out.append((a, b - a + 1 if b > a else 0))
    return out


def _row_keys(v):
    """One comparable key per vertex row (exact bit pattern of the three floats)."""
    a = np.ascontiguousarray(v, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return (a[:, 0] << np.uint64(42)) ^ (a[:, 1] << np.uint64(21)) ^ a[:, 2], a


def merge_slab_meshes(parts):
    """parts: per rank in z order, dict(verts [n][3] float32, indices [m] uint32, nv_before_last, nv_first) or None for an
    empty slab.  Returns (verts, indices) equal to the mesh of the undivided grid."""
    parts = [p for p in parts if p is not None and p.get("n_layers", 2) > 0]
    out_v, out_i, base = [], [], 0
    for r, p in enumerate(parts):
        v = np.asarray(p["verts"], np.float32).reshape(-1, 3)
        idx = np.asarray(p["indices"]).astype(np.int64)
        last = r + 1 == len(parts)
        n_keep = v.shape[0] if last else int(p["nv_before_last"])
        remap = np.arange(v.shape[0], dtype=np.int64) + base
        if not last and n_keep < v.shape[0]:
            nxt = parts[r + 1]
            cand = np.asarray(nxt["verts"], np.float32).reshape(-1, 3)[:int(nxt["nv_first"])]
            seam = v[n_keep:]
            # exact match of positions (full 96-bit rows; the 64-bit key only orders them)
            ck, ca = _row_keys(cand)
            sk, sa = _row_keys(seam)
            order = np.argsort(ck, kind="stable")
            pos = np.searchsorted(ck[order], sk)
            pos = np.clip(pos, 0, max(len(order) - 1, 0))
            hit = order[pos]
            # key collisions are possible in principle: verify, and fall back to a scan for the few that differ
            bad = ~(ca[hit] == sa).all(axis=1)
            for s in np.nonzero(bad)[0]:
                m = np.nonzero((ca == sa[s]).all(axis=1))[0]
                if len(m) == 0:
                    raise ValueError("slab meshes do not fit together: a seam vertex has no counterpart in the next slab")
                hit[s] = m[0]
            remap[n_keep:] = base + n_keep + hit
        out_v.append(v[:n_keep])
        out_i.append(remap[idx])
        base += n_keep
    if not out_v:
        return np.zeros((0, 3), np.float32), np.zeros(0, np.uint32)
    return np.concatenate(out_v), np.concatenate(out_i).astype(np.uint32)


def extract_mesh_sharded(slab_fn, res, rank, world, gather=None):
    """Runs `slab_fn(z0, n_layers) -> dict` (see merge_slab_meshes) for this rank's slab, gathers the parts with `gather`
    (a callable list_of_parts = gather(part); defaults to torch.distributed.all_gather_object when initialised) and merges.
    Every rank returns the whole mesh."""
    z0, nl = slab_ranges(res[2], world)[rank]
    part = slab_fn(z0, nl) if nl > 1 else None
    if gather is None:
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized() and world > 1:
            def gather(p):
                parts = [None] * world
                dist.all_gather_object(parts, p)
                return parts
        else:
            gather = lambda p: [p]
    return merge_slab_meshes(gather(part))
