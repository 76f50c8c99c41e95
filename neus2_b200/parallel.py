"""Data-parallel training of the NeuS step: one process per GPU, rays sharded by rank, one gradient all-reduce per step.

The path has exactly one exchange: the sum of the parameter gradients (grid fp16, MLP fp32, variance fp32) between
`Testbed.train_backward()` and `Testbed.optimizer_step()`.  Everything else (parameters, Adam state, occupancy grid) is
replicated and stays bit-identical across ranks because every rank applies the same summed gradient."""
import os

import torch
import torch.distributed as dist


def env_rank_world():
    return int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))


def ray_shard(rank, max_rays=1 << 18):
    """(ray_index_offset, ray_count_scale is the world size): rank r draws the rays [r * max_rays, (r + 1) * max_rays) of the
    logical batch, so no two ranks ever draw the same (pixel, jitter) sequence."""
    return rank * max_rays


class PeerFailure(RuntimeError):
    """Another rank left the job, or did not reach the exchange in time.  The step's collective was not entered (or was
    abandoned): local gradients are intact, parameters have not been updated."""


class StepGuard:
    """Host-side agreement before a step's gradient exchange, through the process group's key-value store (no GPU work, no
    collective): every rank counts itself in for the step; a rank that finds a peer gone, or not there within
    `timeout_s`, raises PeerFailure instead of entering a collective that could never complete.  A rank that stops
    between steps calls `leave()` first, with none of its kernels or collectives in flight.

    One store round trip per checked step: check every `every` steps (1 = every step)."""

    def __init__(self, store, rank, world, timeout_s=30.0, every=1, prefix="neus2b"):
        self.store, self.rank, self.world = store, rank, world
        self.timeout_s, self.every, self.prefix = float(timeout_s), max(1, int(every)), prefix

    def leave(self, reason="left"):
        self.store.add(f"{self.prefix}/left", 1)
        self.store.set(f"{self.prefix}/left_by/{self.rank}", reason)

    def peers_left(self):
        return int(self.store.add(f"{self.prefix}/left", 0))

    def check(self, step):
        """All ranks present for `step`?  Returns once they are; raises PeerFailure otherwise."""
        import time
        if step % self.every:
            return
        key = f"{self.prefix}/step/{step}"
        try:
            self.store.add(key, 1)
            deadline = time.monotonic() + self.timeout_s
            while True:
                if self.peers_left():
                    raise PeerFailure(f"rank {self.rank}: a peer left the job before step {step}")
                if int(self.store.add(key, 0)) >= self.world:
                    return
                if time.monotonic() > deadline:
                    raise PeerFailure(f"rank {self.rank}: {self.world - int(self.store.add(key, 0))} peer(s) did not reach step {step} "
                                      f"within {self.timeout_s:g} s")
                time.sleep(0.0005)
        except PeerFailure:
            raise
        except Exception as e:  # the store's host is gone
            raise PeerFailure(f"rank {self.rank}: the job's store cannot be reached before step {step}: {e}") from e


def allreduce_gradients(tensors, group=None, stream=None, timeout_s=None):
    """Sum every gradient buffer over the ranks, in place.  On CUDA the collectives are enqueued behind `stream` (the
    training stream of the testbed), so they run between the backward kernels and the optimizer pass without a host sync.
    With `timeout_s` the host waits for the collectives and raises PeerFailure if they do not complete in time (a peer
    that stalled or died inside the exchange) instead of waiting for ever."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return
    if timeout_s is not None:
        import datetime
        ctx = torch.cuda.stream(stream) if stream is not None else _null()
        with ctx:
            works = [dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group, async_op=True) for t in tensors]
            try:
                for w in works:
                    if not w.wait(timeout=datetime.timedelta(seconds=float(timeout_s))):
                        raise PeerFailure("gradient all-reduce did not complete")
            except PeerFailure:
                raise
            except Exception as e:  # the backends report a timed-out wait as RuntimeError / DistBackendError
                raise PeerFailure(f"gradient all-reduce failed or timed out after {timeout_s:g} s: {e}") from e
        return
    if stream is not None:
        with torch.cuda.stream(stream):
            for t in tensors:
                dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
    else:
        for t in tensors:
            dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)


class _null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


def device_view(ptr, nbytes, dtype):
    """torch tensor over a raw device pointer owned by libneus2b.so."""
    class _V:
        pass
    v = _V()
    v.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}
    return torch.as_tensor(v, device="cuda").view(dtype)


def gradient_views(testbed, grid_n_params):
    p = testbed.device_ptrs()
    if p["grad_variance"] == p["grad_mlp"] + 12288 * 4:  # adjacent: one fp32 collective for both
        return [device_view(p["grad_grid"], grid_n_params * 2, torch.float16), device_view(p["grad_mlp"], 12288 * 4 + 16, torch.float32)]
    return [device_view(p["grad_grid"], grid_n_params * 2, torch.float16), device_view(p["grad_mlp"], 12288 * 4, torch.float32),
            device_view(p["grad_variance"], 16, torch.float32)]


class DataParallelTrainer:
    """Drives one testbed per process; `step()` = local backward, gradient all-reduce, optimizer.  With `overlap` the next
    step's sample generation runs while the gradients are exchanged."""

    def __init__(self, testbed, grid_n_params, overlap=True, guard=None, exchange_timeout_s=None):
        """`guard` (a StepGuard) makes every rank agree on the host that all peers are present before the step's
        collectives are launched; `exchange_timeout_s` bounds the wait for the collectives themselves.  Both raise
        PeerFailure; both are off by default (one store round trip, one host wait per step)."""
        self.tb = testbed
        self.overlap = overlap
        self.guard, self.exchange_timeout_s, self.steps = guard, exchange_timeout_s, 0
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.grads = gradient_views(testbed, grid_n_params) if self.world > 1 else None
        self.stream = torch.cuda.ExternalStream(testbed.device_ptrs()["stream"])
        # a second communicator for the small fp32 buffer(s): its collective then runs beside the 25 MB one instead of behind it
        # (every rank creates the group here, in the same order)
        self.small_group = dist.new_group() if self.world > 1 and dist.get_backend() == "nccl" else None

    def step(self, read_stats=False, next_cameras=None):
        """`next_cameras` = (xforms, focal, principal) host arrays for the step AFTER this one: uploaded behind this step's
        backward pass so that the samples drawn ahead already use them."""
        if self.world == 1:
            if not self.overlap:
                st = self.tb.train(1, read_stats=read_stats)
                if next_cameras is not None:
                    self.tb.update_cameras(*next_cameras)
                return st
            # the next step's camera upload and sample generation are enqueued before the host waits for this step's
            # statistics, so the GPU has work while the host wakes up and issues the next launches
            return self.tb.train_step(next_cameras, read_stats=read_stats)
        if self.guard is not None:
            self.guard.check(self.steps)  # before anything of this step is launched: a missing peer costs no GPU state
        self.steps += 1
        self.tb.train_backward()
        if not self.overlap or self.exchange_timeout_s is not None:
            allreduce_gradients(self.grads, stream=self.stream, timeout_s=self.exchange_timeout_s)
            if next_cameras is not None:
                self.tb.update_cameras(*next_cameras)
            return self.tb.optimizer_step(read_stats=read_stats)
        # the collectives start behind the backward kernels on NCCL's own stream; the library draws the next step's samples on
        # its second stream meanwhile (and on through the optimizer pass); the training stream waits for the summed gradients
        with torch.cuda.stream(self.stream):
            works = self._start_exchange()
            if next_cameras is not None:
                self.tb.update_cameras(*next_cameras)
            self.tb.train_pregenerate()
            for w in works:
                w.wait()
        return self.tb.optimizer_step(read_stats=read_stats)

    def _start_exchange(self):
        """Enqueues the step's collectives behind the current stream; returns their work handles."""
        works = [dist.all_reduce(self.grads[0], op=dist.ReduceOp.SUM, async_op=True)]
        works += [dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.small_group, async_op=True) for t in self.grads[1:]]
        return works

    def probe_exchange(self, steps=20):
        """Where the gradient exchange sits in a step, by CUDA events on the training stream over `steps` real training steps:
        the all-reduce alone (a step that draws no samples ahead), and the same wait while the library draws the next step's
        samples on its second stream beside it (the optimizer pass follows the wait on the training stream; the generation
        goes on next to both).  Milliseconds per step, maxima over the ranks are the caller's business."""
        assert self.world > 1
        ev = lambda: torch.cuda.Event(enable_timing=True)
        alone, beside = [], []
        for k in range(steps):
            self.tb.train_backward()
            e0, e1 = ev(), ev()
            with torch.cuda.stream(self.stream):
                e0.record()
                if k % 2 == 0:  # exchange with nothing beside it
                    for w in self._start_exchange():
                        w.wait()
                else:
                    works = self._start_exchange()
                    self.tb.train_pregenerate()
                    for w in works:
                        w.wait()
                e1.record()
            self.tb.optimizer_step(read_stats=False)
            torch.cuda.synchronize()
            (alone if k % 2 == 0 else beside).append(e0.elapsed_time(e1))
        med = lambda v: float(sorted(v)[len(v) // 2]) if v else 0.0
        return {"allreduce_ms": med(alone), "allreduce_with_generation_beside_ms": med(beside)}

