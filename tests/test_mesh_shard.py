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
