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


def allreduce_gradients(tensors, group=None, stream=None):
    """Sum every gradient buffer over the ranks, in place.  On CUDA the collectives are enqueued behind `stream` (the
    training stream of the testbed), so they run between the backward kernels and the optimizer pass without a host sync."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return
    if stream is not None:
        with torch.cuda.stream(stream):
            for t in tensors:
                dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
    else:
        for t in tensors:
            dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)


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

    def __init__(self, testbed, grid_n_params, overlap=True):
        self.tb = testbed
        self.overlap = overlap
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.grads = gradient_views(testbed, grid_n_params) if self.world > 1 else None
        self.stream = torch.cuda.ExternalStream(testbed.device_ptrs()["stream"])

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
        self.tb.train_backward()
        if not self.overlap:
            allreduce_gradients(self.grads, stream=self.stream)
            if next_cameras is not None:
                self.tb.update_cameras(*next_cameras)
            return self.tb.optimizer_step(read_stats=read_stats)
        # the collectives start behind the backward kernels on NCCL's own stream; the training stream meanwhile draws the
        # next step's samples and only then waits for the summed gradients
        with torch.cuda.stream(self.stream):
            works = [dist.all_reduce(t, op=dist.ReduceOp.SUM, async_op=True) for t in self.grads]
            if next_cameras is not None:
                self.tb.update_cameras(*next_cameras)
            self.tb.train_pregenerate()
            for w in works:
                w.wait()
        return self.tb.optimizer_step(read_stats=read_stats)
