"""world_size-2 gloo test of the data-parallel host logic (shard ranges + gather to worker 0)."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, batch, result_file):
    sys.path.insert(0, ROOT)
    from hdkx_aicompiler_b200.parallel import GatherToWorker0, shard_range
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        full = torch.arange(batch * 5, dtype=torch.float32).reshape(batch, 5)  # stands in for the logits
        b, e = shard_range(rank, world, batch)
        gather = GatherToWorker0((e - b, 5), torch.float32, "cpu")
        for step in range(3):  # repeated use of the preallocated buffers
            parts = gather(full[b:e] + step)
            if rank == 0:
                got = torch.cat(parts, dim=0)
                assert torch.equal(got, full + step), "gathered logits are not the dim-0 concat in worker order"
            else:
                assert parts is None
        if rank == 0:
            with open(result_file, "w") as f:
                f.write("ok")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_gather_to_worker0_gloo(tmp_path, world):
    result = tmp_path / "result.txt"
    mp.spawn(_worker, args=(world, _free_port(), 8, str(result)), nprocs=world, join=True)
    assert result.read_text() == "ok"


def _leaving_worker(rank, world, port, result_dir):
    """Rank 1 takes part in step 0, then leaves BETWEEN steps (nothing of its own in flight). Rank 0's next gather must end
    with an error after the process group's short timeout instead of waiting for ever."""
    import datetime
    sys.path.insert(0, ROOT)
    from hdkx_aicompiler_b200.parallel import GatherToWorker0
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
    gather = GatherToWorker0((2, 5), torch.float32, "cpu")
    shard = torch.full((2, 5), float(rank))
    parts = gather(shard)  # step 0: everyone is there
    if rank == 0:
        assert torch.equal(torch.cat(parts), torch.cat([torch.full((2, 5), float(r)) for r in range(world)]))
    if rank == 1:
        with open(os.path.join(result_dir, "left"), "w") as f:
            f.write("rank 1 left after step 0")
        os._exit(0)  # no destroy_process_group: the rank is simply gone
    try:
        gather(shard)  # step 1: rank 1 never posts
        outcome = "no error"
    except Exception as e:  # noqa: BLE001  (gloo raises RuntimeError / DistBackendError depending on where it notices)
        outcome = "error: " + type(e).__name__
    with open(os.path.join(result_dir, f"rank{rank}"), "w") as f:
        f.write(outcome)
    os._exit(0)  # the group is broken: skip the collective teardown


def test_gather_fails_cleanly_when_a_rank_leaves(tmp_path):
    """Failure detection on the host: a rank that leaves between steps turns the next gather into an error on the ranks
    that are still there (bounded by the group's timeout). No GPU is involved."""
    world = 3
    ctx = mp.spawn(_leaving_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=False)
    import time
    deadline = time.time() + 60
    while time.time() < deadline and not ctx.join(timeout=2):  # join() returns as soon as ONE process has exited
        pass
    for p in ctx.processes:
        if p.is_alive():
            p.terminate()  # the exact processes started above
            pytest.fail("a rank was still waiting after 60 s")
    assert (tmp_path / "left").exists()
    assert (tmp_path / "rank0").read_text().startswith("error: "), (tmp_path / "rank0").read_text()


def test_shard_range():
    from hdkx_aicompiler_b200.parallel import shard_range
    assert [shard_range(r, 4, 1024) for r in range(4)] == [(0, 256), (256, 512), (512, 768), (768, 1024)]
    with pytest.raises(ValueError):
        shard_range(0, 3, 1024)


def test_numa_cpus_of_pci_device_reads_sysfs(tmp_path):
    """The CPU set next to a GPU comes from two sysfs files; unknown topology (-1, missing files) gives None."""
    from hdkx_aicompiler_b200.parallel import numa_cpus_of_pci_device, parse_cpu_list
    assert parse_cpu_list("0-3,8,10-11\n") == {0, 1, 2, 3, 8, 10, 11}
    assert parse_cpu_list("") == set()
    dev = tmp_path / "bus/pci/devices/0000:1b:00.0"
    dev.mkdir(parents=True)
    (dev / "numa_node").write_text("1\n")
    node = tmp_path / "devices/system/node/node1"
    node.mkdir(parents=True)
    (node / "cpulist").write_text("32-63,96-127\n")
    cpus = numa_cpus_of_pci_device("0000:1B:00.0", sysfs_root=str(tmp_path))
    assert cpus == set(range(32, 64)) | set(range(96, 128))
    (dev / "numa_node").write_text("-1\n")
    assert numa_cpus_of_pci_device("0000:1b:00.0", sysfs_root=str(tmp_path)) is None
    assert numa_cpus_of_pci_device("0000:aa:00.0", sysfs_root=str(tmp_path)) is None
