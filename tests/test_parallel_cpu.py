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


def test_shard_range():
    from hdkx_aicompiler_b200.parallel import shard_range
    assert [shard_range(r, 4, 1024) for r in range(4)] == [(0, 256), (256, 512), (512, 768), (768, 1024)]
    with pytest.raises(ValueError):
        shard_range(0, 3, 1024)
