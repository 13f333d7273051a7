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


class PeerStoreToWorker0:
    """The same exchange without a copy: every rank's LAST kernel writes its shard straight into rank 0's gathered
    buffer through a peer-mapped pointer (plain global stores over NVLink; no TMA, no multicast), so "compute the
    logits" and "gather them" are one kernel. The buffers come from torch's symmetric memory; `output()` is the view of
    rank 0's buffer that this rank's shard occupies (rows [rank*rows, (rank+1)*rows), the order of
    ConcatFirstDim, src/base/disco/ccl_cpu.cc:134-174) and is passed as `out=` of CompiledGraph.run; `complete()`
    is a device-side barrier on the current stream after which rank 0 may read `gathered()`.

    NCCL's gather (GatherToWorker0) is the default; this class is checked against it bit for bit on 2 GPUs
    (tests/test_parallel_gpu.py)."""

    def __init__(self, shard_shape, dtype, device, group=None):
        import torch.distributed._symmetric_memory as symm

        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        rows = int(shard_shape[0])
        rest = tuple(int(d) for d in shard_shape[1:])
        per = rows
        for d in rest:
            per *= d
        self.full = symm.empty((self.world * rows,) + rest, dtype=dtype, device=device)
        self.handle = symm.rendezvous(self.full, self.group)
        self.dst = self.handle.get_buffer(0, tuple(shard_shape), dtype, self.rank * per)

    def output(self):
        return self.dst

    def complete(self):
        self.handle.barrier()

    def gathered(self):
        return self.full if self.rank == 0 else None

