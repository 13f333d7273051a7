"""Data-parallel plumbing for the operator path: contiguous batch shards and the one exchange step.

Every image is independent through all 49 calls of the graph, so rank r of G simply owns images
[r*N/G, (r+1)*N/G) with replicated weights. The only communication is the reference's
`device.gather_to_worker0`: concatenate the per-worker shards on dim 0, in worker order, into worker 0
(CpuCCLBackend::GatherToWorker0 / ConcatFirstDim, src/base/disco/ccl_cpu.cc:274-294, :134-174).
Works on any torch.distributed backend (NCCL on GPUs, gloo on CPU for the tests).
"""
import os

import torch
import torch.distributed as dist


def parse_cpu_list(text):
    """'0-3,8,10-11' -> {0, 1, 2, 3, 8, 10, 11} (the format of sysfs cpulist files)."""
    cpus = set()
    for part in text.strip().split(","):
        if not part:
            continue
        lo, _, hi = part.partition("-")
        cpus.update(range(int(lo), int(hi or lo) + 1))
    return cpus


def numa_cpus_of_pci_device(bdf, sysfs_root="/sys"):
    """CPUs of the NUMA node a PCI device ('0000:1b:00.0') is attached to, or None when the kernel does not say."""
    try:
        with open(os.path.join(sysfs_root, "bus/pci/devices", bdf.lower(), "numa_node")) as f:
            node = int(f.read().strip())
        if node < 0:
            return None
        with open(os.path.join(sysfs_root, "devices/system/node", f"node{node}", "cpulist")) as f:
            return parse_cpu_list(f.read()) or None
    except (OSError, ValueError):
        return None


def bind_to_device_numa_node(device_index, sysfs_root="/sys"):
    """Restricts this process to the CPUs next to GPU `device_index`, so that the pinned host buffers it allocates
    afterwards (and the threads that fill them) live on the memory of the socket the GPU's PCIe link hangs off. With one
    process per GPU on a two-socket host, half of the ranks otherwise stage their 600 MB per step through the other
    socket. Returns the CPU set it bound to, or None when the topology is unknown or the binding is not permitted
    (nothing is changed then)."""
    try:
        props = torch.cuda.get_device_properties(device_index)
        bdf = "%04x:%02x:%02x.0" % (props.pci_domain_id, props.pci_bus_id, props.pci_device_id)
    except (AttributeError, RuntimeError, AssertionError):
        return None
    cpus = numa_cpus_of_pci_device(bdf, sysfs_root)
    if not cpus:
        return None
    try:
        allowed = os.sched_getaffinity(0) & cpus
        if not allowed:
            return None
        os.sched_setaffinity(0, allowed)
        return allowed
    except (OSError, AttributeError):
        return None


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

    Checked against NCCL's gather (GatherToWorker0) bit for bit on 2 GPUs (tests/test_parallel_gpu.py)."""

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

