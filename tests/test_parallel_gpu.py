"""Two-GPU check of the peer-store exchange: the dense layer's epilogue writes each rank's logits straight into rank 0's
gathered buffer (PeerStoreToWorker0); the result must equal NCCL's gather (GatherToWorker0) bit for bit.
Runs as two child processes (one per GPU); skipped on boxes with fewer than two GPUs."""
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r'''
import os, sys
sys.path.insert(0, os.environ["KXC_ROOT"])
import numpy as np, torch, torch.distributed as dist
from hdkx_aicompiler_b200 import plan, relay as R, ops
from hdkx_aicompiler_b200.parallel import GatherToWorker0, PeerStoreToWorker0, shard_range
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dev = torch.device("cuda", rank)
dist.init_process_group("nccl", device_id=dev)
rng = np.random.default_rng(0)                      # same weights on every rank
N, C, K = 64, 64, 40
w = torch.from_numpy(rng.normal(0, 0.1, (C, C, 3, 3)).astype(np.float32)).to(dev)
b = torch.from_numpy(rng.normal(0, 0.1, (C,)).astype(np.float32)).to(dev)
fw = torch.from_numpy(rng.normal(0, 0.1, (K, C)).astype(np.float32)).to(dev)
fb = torch.from_numpy(rng.normal(0, 0.1, (K,)).astype(np.float32)).to(dev)
lo, hi = shard_range(rank, world, N)
x = torch.from_numpy(np.random.default_rng(1).normal(0, 1, (N, C, 8, 8)).astype(np.float32)[lo:hi]).to(dev)
xv = R.Var("input", tuple(x.shape))
y = R.Call("nn_relu", [R.Call("nn_conv2d", [xv, R.Constant(w), R.Constant(b)], R.Conv2DAttrs((1, 1), (1, 1, 1, 1), (1, 1), 1))])
y = R.Call("nn_flatten", [R.Call("nn_global_avg_pool2d", [y])])
y = R.Call("nn_gemm", [y, R.Constant(fw), R.Constant(fb)], R.GemmAttrs(1.0, 1.0, 0, 1))
g = plan.CompiledGraph(R.Function([xv], y), "bf16")
s = torch.cuda.Stream(dev)
with torch.cuda.stream(s):
    local = g.run(x)                                                    # ordinary output buffer
    parts = GatherToWorker0(g.out_shape, torch.float32, dev)(local)     # NCCL gather
    peer = PeerStoreToWorker0(g.out_shape, torch.float32, dev)
    for _ in range(3):                                                  # repeated use of the same buffers
        g.run(x, out=peer.output())                                     # last kernel stores into rank 0's memory
        peer.complete()
    s.synchronize()
    assert ops.device_status(dev) == 0
    if rank == 0:
        want = torch.cat(parts, 0)
        got = peer.gathered()
        assert got.shape == want.shape and torch.equal(got, want), "peer-store gather differs from the NCCL gather"
        print("PEER_OK", tuple(got.shape))
dist.barrier()
dist.destroy_process_group()
'''


@pytest.mark.gpu
def test_peer_store_gather_equals_nccl_gather(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "child.py"
    script.write_text(CHILD)
    env = dict(os.environ, KXC_ROOT=ROOT, NCCL_NVLS_ENABLE="0")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                          "--master-port", "29533", str(script)], env=env, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    assert "PEER_OK" in out.stdout
