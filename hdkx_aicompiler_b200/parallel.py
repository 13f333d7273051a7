"""Data-parallel plumbing for the operator path: contiguous batch shards and the one exchange step.

Every image is independent through all 49 calls of the graph, so rank r of G simply owns images
[r*N/G, (r+1)*N/G) with replicated weights. The only communication is the reference's
`device.gather_to_worker0`: concatenate the per-worker shards on dim 0, in worker order, into worker 0
(CpuCCLBackend::GatherToWorker0 / ConcatFirstDim, src/base/disco/ccl_cpu.cc:274-294, :134-174).
Works on any torch.distributed backend (NCCL on GPUs, gloo on CPU for the tests).
"""
import torch
import torch.distributed as dist


def shard_range(rank, world, batch):
    """[begin, end) of the images rank `rank` owns; the batch must divide evenly (as in the benchmark)."""
    if batch % world != 0:
        raise ValueError(f"batch {batch} is not divisible by {world} workers")
    per = batch // world
    return rank * per, (rank + 1) * per


class GatherToWorker0:
    """Preallocated gather of equally shaped shards to rank 0."""

    def __init__(self, shard_shape, dtype, device, group=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.buffers = None
        if self.world > 1 and self.rank == 0:
            self.buffers = [torch.empty(shard_shape, dtype=dtype, device=device) for _ in range(self.world)]

    def __call__(self, shard):
        """Rank 0 gets the list of shards in worker order (concatenate on dim 0 for the full tensor); others get None."""
        if self.world == 1:
            return [shard]
        dist.gather(shard, self.buffers, dst=0, group=self.group)
        return self.buffers
