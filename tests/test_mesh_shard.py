"""z-slab sharded mesh extraction: the merged slabs equal the undivided grid's mesh bit for bit (CPU, through the oracle),
and two gloo ranks reach the same mesh through the gather."""
import multiprocessing as mp
import os

import numpy as np
import pytest

from neus2_b200 import mesh_shard as M
from neus2_b200.mc_table import make_table


def field(res, kind="torus"):
    rz, ry, rx = res[2], res[1], res[0]
    z, y, x = np.meshgrid(np.arange(rz), np.arange(ry), np.arange(rx), indexing="ij")
    p = np.stack([x / rx - 0.5, y / ry - 0.52, z / rz - 0.48], -1)
    if kind == "noise":
        return np.random.default_rng(4).normal(0, 1, (rz, ry, rx)).astype(np.float32)
    q = np.stack([np.linalg.norm(p[..., [0, 2]], axis=-1) - 0.25, p[..., 1]], -1)  # torus around the y axis: crosses every slab
    return (np.linalg.norm(q, axis=-1) - 0.08).astype(np.float32)


def slab_part(O, sdf, res, z0, nl, tab):
    v, i, nb, nf = O.marching_cubes_slab(sdf[z0:z0 + nl].ravel(), res, z0, nl, tab)
    return dict(verts=v, indices=i, nv_before_last=nb, nv_first=nf)


@pytest.mark.parametrize("kind,res", [("torus", (24, 20, 33)), ("noise", (9, 11, 10)), ("torus", (16, 16, 2))])
@pytest.mark.parametrize("world", [1, 2, 3, 8])
def test_merged_slabs_equal_the_whole_grid(oracle, kind, res, world):
    tab = make_table()
    sdf = field(res, kind)
    v_ref, i_ref = oracle.marching_cubes(sdf.ravel(), res, tab)
    parts = []
    for z0, nl in M.slab_ranges(res[2], world):
        parts.append(slab_part(oracle, sdf, res, z0, nl, tab) if nl > 1 else None)
    v, i = M.merge_slab_meshes(parts)
    assert v.shape == v_ref.shape and i.shape == i_ref.shape
    assert np.array_equal(v.view(np.uint32), v_ref.view(np.uint32)) and np.array_equal(i, i_ref)


def test_slab_ranges_cover_every_cell_layer_once():
    for res_z, world in ((512, 8), (5, 8), (2, 2), (100, 3)):
        r = M.slab_ranges(res_z, world)
        covered = [z for z0, nl in r for z in range(z0, z0 + max(nl - 1, 0))]
        assert covered == list(range(res_z - 1))


def _rank_main(rank, world, port, res, q):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import oracle as O
    O.set_num_threads(1)
    tab = make_table()
    sdf = field(res)
    v, i = M.extract_mesh_sharded(lambda z0, nl: slab_part(O, sdf, res, z0, nl, tab), res, rank, world)
    q.put((rank, v.tobytes(), i.tobytes()))
    dist.barrier()
    dist.destroy_process_group()


def test_two_gloo_ranks_extract_the_same_mesh(oracle):
    res = (20, 18, 25)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29650 + os.getpid() % 200
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, res, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    v_ref, i_ref = oracle.marching_cubes(field(res).ravel(), res, make_table())
    for _, vb, ib in got:
        assert vb == v_ref.tobytes() and ib == i_ref.tobytes()


# ------------------------------------------------------------------------------------------------ globally numbered slabs
class OracleSlabGlobal:
    """CPU stand-in for ops.SlabGlobal built from the oracle's slab routine: a run over the slab plus its halo layer numbers
    the vertices as the kernel does; the triangles of the slab's own cells are that run's first indices (cell order), as many
    as a run without the halo writes; the vertices it owns are those before its last own layer."""

    def __init__(self, O, sdf, res, z0, nl, halo, tab):
        import torch
        self.torch = torch
        v, i, _, _ = O.marching_cubes_slab(sdf[z0:z0 + nl + halo].ravel(), res, z0, nl + halo, tab)
        _, i_own, nbl, _ = O.marching_cubes_slab(sdf[z0:z0 + nl].ravel(), res, z0, nl, tab)
        self.n_idx = len(i_own)
        self.n_owned = nbl if halo else v.shape[0]
        self.v, self.i = v, i[:self.n_idx]

    def count(self):
        return self.torch.tensor([self.v.shape[0], self.n_idx, self.n_owned, 0], dtype=self.torch.int32)

    def emit(self, vertex_offset, n_owned, n_indices):
        assert n_owned == self.n_owned and n_indices == self.n_idx
        return (self.torch.from_numpy(self.v[:n_owned].copy()),
                self.torch.from_numpy((self.i.astype(np.int64) + vertex_offset).astype(np.int32)))


@pytest.mark.parametrize("kind,res", [("torus", (24, 20, 33)), ("noise", (9, 11, 10))])
@pytest.mark.parametrize("world", [1, 2, 5])
def test_global_offsets_give_the_whole_mesh(oracle, kind, res, world):
    tab = make_table()
    sdf = field(res, kind)
    v_ref, i_ref = oracle.marching_cubes(sdf.ravel(), res, tab)
    slabs = []
    for z0, nl in M.slab_ranges(res[2], world):
        halo = 1 if nl > 1 and z0 + nl < res[2] else 0
        slabs.append(OracleSlabGlobal(oracle, sdf, res, z0, nl, halo, tab) if nl > 1 else None)
    counts = [s.count().tolist() if s else [0, 0, 0, 0] for s in slabs]
    v_off, i_off, nv, ni = M.global_offsets(counts)
    assert (nv, ni) == (v_ref.shape[0], i_ref.shape[0])
    parts = [s.emit(v_off[r], counts[r][2], counts[r][1]) for r, s in enumerate(slabs) if s]
    v = np.concatenate([p[0].numpy() for p in parts])
    i = np.concatenate([p[1].numpy() for p in parts]).view(np.uint32)
    assert np.array_equal(v.view(np.uint32), v_ref.view(np.uint32)) and np.array_equal(i, i_ref)


def _rank_main_device(rank, world, port, res, q):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import oracle as O
    O.set_num_threads(1)
    tab = make_table()
    sdf = field(res)
    v, i = M.extract_mesh_sharded_device(lambda z0, nl, halo: OracleSlabGlobal(O, sdf, res, z0, nl, halo, tab), res, rank, world)
    q.put((rank, None if v is None else v.numpy().tobytes(), None if i is None else i.numpy().tobytes()))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_gloo_ranks_gather_globally_numbered_slices(oracle, world):
    """The exchange of the counters (all-gather) and of the slices (point-to-point into rank 0's arrays) over gloo: rank 0 ends
    up with the undivided mesh, the others with nothing; nothing is pickled or re-indexed."""
    res = (20, 18, 25)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29850 + (os.getpid() + world) % 200
    procs = [ctx.Process(target=_rank_main_device, args=(r, world, port, res, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = dict((r, (v, i)) for r, v, i in [q.get(timeout=120) for _ in procs])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    v_ref, i_ref = oracle.marching_cubes(field(res).ravel(), res, make_table())
    assert got[0][0] == v_ref.tobytes() and got[0][1] == i_ref.tobytes()
    assert all(got[r] == (None, None) for r in range(1, world))
