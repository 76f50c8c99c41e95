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
    return [device_view(p["grad_grid"], grid_n_params * 2, torch.float16), device_view(p["grad_mlp"], 12288 * 4, torch.float32),
            device_view(p["grad_variance"], 16, torch.float32)]


class DataParallelTrainer:
    """Drives one testbed per process; `step()` = local backward, gradient all-reduce, optimizer."""

    def __init__(self, testbed, grid_n_params):
        self.tb = testbed
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.grads = gradient_views(testbed, grid_n_params) if self.world > 1 else None
        self.stream = torch.cuda.ExternalStream(testbed.device_ptrs()["stream"])

    def step(self, read_stats=False):
        if self.world == 1:
            return self.tb.train(1, read_stats=read_stats)
        self.tb.train_backward()
        allreduce_gradients(self.grads, stream=self.stream)
        return self.tb.optimizer_step(read_stats=read_stats)
