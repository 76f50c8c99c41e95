"""The N > 1 path on CPU: two gloo ranks run the oracle's step on their ray shard, all-reduce the gradients with the same
helper bench.py uses, and must end up with the gradient a single process gets from both shards."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def shard_gradient(rank, world, n_rays=256):
    """Oracle gradient of one rank's shard of the logical batch (ray offset + global normalisation)."""
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from oracle import oracle as O
    from neus2_b200 import parallel as P
    from neus2_b200 import synthetic as S
    sc = S.render_sphere_views(4, 48, 48, device="cpu", seed=2)
    ds = O.make_dataset(sc["pixels"].numpy().view(np.uint32), sc["xforms"].numpy(), sc["focal"].numpy(), sc["principal"].numpy())
    d = O.grid_desc(n_levels=4, log2_hashmap_size=10, base_resolution=4, per_level_scale=1.7)
    ng = O.grid_n_params(d)
    p = S.init_params(ng, seed=3)
    rng = np.random.default_rng(4)
    p[12288:12288 + ng] = rng.uniform(-1e-2, 1e-2, ng)
    p[:3072].reshape(64, 48)[:, 3:11] = rng.normal(0, 0.05, (64, 8))
    params = O.f16_bits(p)
    bits = np.full(128 ** 3, 0xFF, np.uint8)  # everything occupied
    cfg = O.train_cfg(ray_index_offset=P.ray_shard(rank, 1 << 10), ray_count_scale=world)
    rngs = O.pcg32(7)
    gen = O.generate_samples(ds, cfg, n_rays, 0, 1 << 18, rngs, bits)
    used = int(gen["numsteps"][gen["n_kept"] - 1].sum())
    out = O.neus_forward(d, params, gen["coords"][:used])
    target = 1 << 13
    los = O.compute_loss(ds, cfg, gen, n_rays, 0, rngs, target, out)
    nv = min(los["n_compacted"], target)
    grad = O.neus_backward(d, params, los["coords"][:nv], los["dloss"][:nv], indeed_batch_size=target * world)
    return grad, gen["ray_indices"][:gen["n_kept"]] + cfg.ray_index_offset


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sys.path.insert(0, ROOT)
    from neus2_b200 import parallel as P
    grad, rays = shard_gradient(rank, world)
    # the three gradient buffers of the product: grid fp16 is not reducible by gloo on every build, so the CPU test
    # carries it in fp32 -- the helper under test is dtype agnostic
    n = grad.size
    bufs = [torch.from_numpy(grad[12288:n - 4].astype(np.float32)), torch.from_numpy(grad[:12288].astype(np.float32)),
            torch.from_numpy(grad[n - 4:].astype(np.float32))]
    P.allreduce_gradients(bufs)
    q.put((rank, [b.numpy().copy() for b in bufs], rays))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_allreduce_equals_single_process_sum():
    world, port = 2, 29000 + os.getpid() % 2000
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted([q.get(timeout=300) for _ in range(world)], key=lambda x: x[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    g0, _ = shard_gradient(0, world)
    g1, _ = shard_gradient(1, world)
    total = (g0 + g1).astype(np.float32)
    n = total.size
    for rank, bufs, rays in res:
        assert np.allclose(bufs[0], total[12288:n - 4], rtol=1e-6, atol=1e-9)
        assert np.allclose(bufs[1], total[:12288], rtol=1e-6, atol=1e-9)
        assert np.allclose(bufs[2], total[n - 4:], rtol=1e-6, atol=1e-9)
    # shards draw disjoint logical rays
    assert not set(res[0][2].tolist()) & set(res[1][2].tolist())
    assert np.abs(total).max() > 0


def test_ray_shard_offsets():
    sys.path.insert(0, ROOT)
    from neus2_b200 import parallel as P
    assert [P.ray_shard(r) for r in range(4)] == [0, 1 << 18, 2 << 18, 3 << 18]


# ------------------------------------------------------------------------------------------------ failures, made on the host

def _failure_worker(rank, world, port, q, mode):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import datetime
    import time
    store = dist.TCPStore("127.0.0.1", port, world, rank == 0, timeout=datetime.timedelta(seconds=60))
    dist.init_process_group("gloo", store=store, rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    sys.path.insert(0, ROOT)
    from neus2_b200 import parallel as P
    guard = P.StepGuard(store, rank, world, timeout_s=2.0)
    grad = torch.full((1024,), float(rank + 1))
    out = {"rank": rank, "steps_done": 0, "error": None}
    t0 = time.monotonic()
    try:
        for step in range(6):
            if mode == "leaves" and rank == 1 and step == 3:
                guard.leave("done early")  # between steps: nothing of this rank is in flight
                break
            if mode == "never_arrives" and rank == 1 and step == 3:
                time.sleep(6.0)  # stalls on the host past the others' patience, then finds them gone
            if mode != "stalls_in_exchange":
                guard.check(step)
            if mode == "stalls_in_exchange" and rank == 1 and step == 3:
                time.sleep(5.0)
                break
            g = grad.clone()
            P.allreduce_gradients([g], timeout_s=1.5 if mode == "stalls_in_exchange" else None)
            assert float(g[0]) == 3.0
            out["steps_done"] = step + 1
    except P.PeerFailure as e:
        out["error"] = "PeerFailure: " + str(e)
    out["seconds"] = time.monotonic() - t0
    q.put(out)
    q.close()
    q.join_thread()
    os._exit(0)  # the process group may be unusable after a failed collective: leave without its destructor


@pytest.mark.parametrize("mode", ["leaves", "never_arrives", "stalls_in_exchange"])
def test_a_missing_peer_gives_an_error_not_a_hang(mode):
    """One of two ranks leaves between steps, never arrives at a step, or stalls inside the exchange: the other rank's step
    raises PeerFailure within its timeout instead of waiting for ever.  The failure is made on the host (CPU ranks over gloo)."""
    world, port = 2, 31000 + (os.getpid() * 7 + len(mode)) % 2000
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_failure_worker, args=(r, world, port, q, mode)) for r in range(world)]
    for p in procs:
        p.start()
    res = {}
    for _ in range(world):
        o = q.get(timeout=120)
        res[o["rank"]] = o
    for p in procs:
        p.join(timeout=60)
    r0 = res[0]
    assert r0["steps_done"] == 3 and r0["error"] and r0["error"].startswith("PeerFailure"), res
    assert r0["seconds"] < 20, res
    if mode == "leaves":
        assert res[1]["error"] is None and res[1]["steps_done"] == 3
        assert "left" in r0["error"]
    if mode == "never_arrives":
        assert "did not reach step 3" in r0["error"]
