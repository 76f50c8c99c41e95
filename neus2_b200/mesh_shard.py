"""Mesh extraction sharded by z-slab (one slab per rank), two ways: slabs numbered locally and merged on the host
(`extract_mesh_sharded`), and slabs numbered globally on the devices after an all-gather of their counters, gathered into
one rank's arrays without a merge (`extract_mesh_sharded_device`).  Both give back exactly the single-grid mesh.

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


# ------------------------------------------------------------------------------------------------ no merge on the host
def global_offsets(all_counts):
    """all_counts [world][>=3] = per slab (ids referred to, indices written, vertices owned), in z order.  Returns
    (vertex_offsets, index_offsets, n_verts, n_indices): exclusive prefix sums over the slabs and the totals."""
    v_off, i_off, nv, ni = [], [], 0, 0
    for c in all_counts:
        v_off.append(nv)
        i_off.append(ni)
        nv += int(c[2])
        ni += int(c[1])
    return v_off, i_off, nv, ni


def extract_mesh_sharded_device(slab_fn, res, rank, world, group=None, dst=0):
    """Mesh extraction sharded by z-slab with the numbering settled on the devices (what the reference does on one GPU with
    two atomic counters, src/marching_cubes.cu:794-822, becomes: count, all-gather of the counters, emit at global offsets,
    gather of the slices).  `slab_fn(z0, n_layers, halo)` returns an object with `count()` -> int32 tensor (ids, indices,
    owned, -) and `emit(vertex_offset, n_owned, n_indices)` -> (verts, indices) tensors (ops.SlabGlobal on CUDA).  The
    counters travel in one all-gather, the slices in point-to-point copies into rank `dst`'s arrays: no host merge, no
    re-indexing.  Returns (verts [n][3] float32, indices [m] int32) on rank `dst` (device tensors), (None, None) elsewhere."""
    import torch
    import torch.distributed as dist
    z0, nl = slab_ranges(res[2], world)[rank]
    halo = 1 if nl > 1 and z0 + nl < res[2] else 0
    slab = slab_fn(z0, nl, halo) if nl > 1 else None
    counts = slab.count() if slab is not None else None
    multi = dist.is_available() and dist.is_initialized() and world > 1
    if counts is None:
        dev = torch.device("cuda") if (multi and dist.get_backend(group) == "nccl") else torch.device("cpu")
        counts = torch.zeros(4, dtype=torch.int32, device=dev)
    if multi:
        allc = torch.empty(world * 4, dtype=torch.int32, device=counts.device)
        dist.all_gather_into_tensor(allc, counts.contiguous(), group=group)
        allc = allc.view(world, 4).cpu().tolist()
    else:
        allc = [counts.cpu().tolist()]
    v_off, i_off, nv, ni = global_offsets(allc)
    mine = allc[rank]
    verts, idx = slab.emit(v_off[rank], int(mine[2]), int(mine[1])) if slab is not None else (None, None)
    if not multi:
        return verts, idx
    if rank == dst:
        out_v = torch.empty((nv, 3), dtype=torch.float32, device=counts.device)
        out_i = torch.empty(ni, dtype=torch.int32, device=counts.device)
        ops_ = []
        for r in range(world):
            n_own, n_idx = int(allc[r][2]), int(allc[r][1])
            if r == rank:
                if n_own:
                    out_v[v_off[r]:v_off[r] + n_own] = verts
                if n_idx:
                    out_i[i_off[r]:i_off[r] + n_idx] = idx
                continue
            if n_own:
                ops_.append(dist.P2POp(dist.irecv, out_v[v_off[r]:v_off[r] + n_own], r, group))
            if n_idx:
                ops_.append(dist.P2POp(dist.irecv, out_i[i_off[r]:i_off[r] + n_idx], r, group))
        if ops_:
            for w in dist.batch_isend_irecv(ops_):
                w.wait()
        return out_v, out_i
    ops_ = []
    if int(mine[2]):
        ops_.append(dist.P2POp(dist.isend, verts.contiguous(), dst, group))
    if int(mine[1]):
        ops_.append(dist.P2POp(dist.isend, idx.contiguous(), dst, group))
    if ops_:
        for w in dist.batch_isend_irecv(ops_):
            w.wait()
    return None, None
