#!/usr/bin/env python
"""Headline benchmark: ResNet-18 inference throughput (img/s) through the B200 operator path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--batch B]

One "step" = one pass of the whole graph (the stem kernel that reads the fp32 NCHW images and writes the pooled
activation, 19 more convolutions in 16 launches with bias / residual / ReLU fused, global average pool, dense)
over the global batch of 1024 synthetic images, bf16 operands with fp32 accumulation, sharded data-parallel over N GPUs (1024/N images per GPU, weights replicated, logits
gathered to rank 0 inside the step: each rank's last kernel stores its logits into rank 0's buffer over NVLink, or one
NCCL gather where symmetric memory is not available). Prints ONE JSON line on rank 0.

value     device-timed (CUDA events, max over ranks) with the inputs resident in HBM
e2e       the same step through the public API with HOST buffers: pinned-host -> device copy of the
          images and device -> host read of the logits inside the timed region
roofline  the tensor-core launches of a step (20 convolutions in 17 launches + 1 dense): algorithmic FLOPs / their summed
          launch durations, from runs with CUDA events between launches; `frac` is taken against the measured cuBLAS
          bf16 BURST figure (the launches are timed one by one, the whole timed region lasts a tenth of a second),
          `frac_sustained` against the seconds-long figure
hbm_kernels / config1 / config3  (one GPU only) the benchmark's other single-GPU configurations, measured in the same
          run after the headline timing: the memory-bound pool -> add -> relu kernels at 32x64x112x112 against the measured
          copy bandwidth, the single fused convolution, ResNet-18 fp32/tf32 at batch 32 (microbench.py)
cpu_baseline  the reference compiler's own CPU lowering (oracle/_ref) on a bounded sample, rank 0 only

--impl reference times that CPU path alone, on all host cores (independent batch shards per core).
"""
import argparse
import collections
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

GLOBAL_BATCH = 1024
# dram__bytes_read.sum + dram__bytes_write.sum per image of the tensor-core launches of one bf16 plan run, by kernel
# family, from ncu captures of this script at 512 images per GPU (about 2.5 GB on the device; a capture at the full 1024
# would break the size rule for captures). Outputs of 205-411 MB no longer fit the 126 MB L2 at that size, as at 1024.
NCU_TRAFFIC_BATCH = 512
NCU_DRAM_BYTES_PER_IMAGE = {
    "conv_stem_pool_nchw": 0.920e6,   # 1 launch: 308.4 MB read (= the fp32 input, once) + 162.6 MB written
    "conv_rowstack": 3.690e6,         # 4 launches: 1234 MB read + 655 MB written
    "conv_rowstack128": 0.317e6,      # 1 launch: 103.1 MB read + 59.1 MB written
    "conv_igemm": 3.101e6,            # 12 launches (11 at 512 images): 1204 MB read + 384 MB written
    "dense_igemm": 0.003e6,
}

METRIC = "resnet18_inference_throughput"
UNIT = "img/s"


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "tflops_burst": p["bf16_tflops"], "tflops_sustained": p["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops_burst": 1590.0, "tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons while the timed region runs: NVML read-outs from a thread of this process
    every 2 ms (a region of a few milliseconds still gets samples), or, without the NVML module, an nvidia-smi child
    process printing every 20 ms. Read-only: nothing of the GPU's state is changed."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
    NVML_BITS = [0x8, 0x40, 0x20, 0x4]  # nvmlClocksEventReason*: HwSlowdown, HwThermalSlowdown, SwThermalSlowdown, SwPowerCap

    def __init__(self, index):
        self.samples, self.proc, self.thread, self.index = [], None, None, index
        self.nvml, self.handle, self.stop_flag = None, None, threading.Event()

    def _nvml_handle(self):
        import pynvml
        pynvml.nvmlInit()
        try:  # by PCI address: NVML's numbering ignores CUDA_VISIBLE_DEVICES
            import torch
            pr = torch.cuda.get_device_properties(self.index)
            handle = pynvml.nvmlDeviceGetHandleByPciBusId("%08x:%02x:%02x.0" % (pr.pci_domain_id, pr.pci_bus_id, pr.pci_device_id))
        except Exception:  # noqa: BLE001
            handle = pynvml.nvmlDeviceGetHandleByIndex(self.index)
        return pynvml, handle

    def start(self):
        try:
            self.nvml, self.handle = self._nvml_handle()
            self.nvml.nvmlDeviceGetClockInfo(self.handle, self.nvml.NVML_CLOCK_SM)
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
            return
        except Exception:  # noqa: BLE001
            self.nvml = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "20"], stdout=subprocess.PIPE, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()
        t0 = time.time()
        while not self.samples and time.time() - t0 < 3.0:  # the child needs a moment before its first line
            time.sleep(0.01)

    def _poll(self):
        n = self.nvml
        reasons_fn = getattr(n, "nvmlDeviceGetCurrentClocksEventReasons", None) or getattr(n, "nvmlDeviceGetCurrentClocksThrottleReasons")
        mx = n.nvmlDeviceGetMaxClockInfo(self.handle, n.NVML_CLOCK_SM)
        while not self.stop_flag.is_set():
            try:
                mask = int(reasons_fn(self.handle))
                self.samples.append([str(n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM)), str(mx)] +
                                    ["Active" if mask & b else "Not Active" for b in self.NVML_BITS])
            except Exception:  # noqa: BLE001
                pass
            time.sleep(0.002)

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def stop(self):
        if self.nvml is not None:
            self.stop_flag.set()
            self.thread.join(timeout=2)
        elif self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        else:
            self.proc.terminate()  # the exact process started above
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        mhz = sorted(int(s[0]) for s in self.samples if s[0].isdigit())
        mx = [int(s[1]) for s in self.samples if s[1].isdigit()]
        reasons = [n for i, n in enumerate(self.NAMES) if any(s[2 + i].lower().startswith("active") for s in self.samples)]
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(self.samples), "source": "nvml" if self.nvml is not None else "nvidia-smi"}


# ------------------------------------------------------------------------------------------------
# reference arm / cpu baseline
def cpu_reference_throughput(images_per_worker, workers, steps=1, warmup=0):
    """ResNet-18 through the reference compiler's own CPU lowering (oracle/_ref kernels chained per call),
    `workers` independent single-threaded batch shards. Returns (img/s, kind)."""
    import numpy as np
    from concurrent.futures import ThreadPoolExecutor

    from hdkx_aicompiler_b200 import resnet18
    from oracle import graph as ograph
    from oracle import ref as oref
    kind = "reference" if oref.available() else "port"
    backend = oref if kind == "reference" else None
    weights = resnet18.make_weights(seed=0)
    func = resnet18.build(images_per_worker, weights)
    rng = np.random.default_rng(1)
    shards = [rng.normal(0, 1, (images_per_worker, 3, 224, 224)).astype(np.float32) for _ in range(workers)]
    run = lambda x: ograph.run(func, [x], backend=backend)  # noqa: E731
    run(shards[0][:images_per_worker])  # compiles/loads the per-op kernels outside the timed region
    times = []
    for it in range(warmup + steps):
        t0 = time.perf_counter()
        if workers == 1:
            run(shards[0])
        else:
            with ThreadPoolExecutor(workers) as ex:
                list(ex.map(run, shards))
        if it >= warmup:
            times.append(time.perf_counter() - t0)
    return images_per_worker * workers * len(times) / sum(times), kind


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    per_worker = 1
    value, kind = cpu_reference_throughput(per_worker, cores, steps=max(1, args.steps), warmup=min(args.warmup, 1))
    sample = f"{per_worker} image per core x {cores} cores per step (independent single-threaded shards), {max(1, args.steps)} steps"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * per_worker * cores / value, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"resnet18 inference, global batch {GLOBAL_BATCH} (bounded CPU sample)", "global_batch": GLOBAL_BATCH},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--batch", type=int, default=GLOBAL_BATCH, help="global batch (default: the benchmark's 1024)")
    ap.add_argument("--precision", default="bf16", choices=["bf16", "tf32"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-side-configs", action="store_true", help="skip the pool/eltwise, single-conv and batch-32 measurements")
    ap.add_argument("--gather", default="peer", choices=["nccl", "peer"],
                    help="exchange step: the dense layer's epilogue storing the logits into rank 0's buffer over NVLink "
                         "(default; falls back to NCCL when symmetric memory is unavailable) or an NCCL gather")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference_arm(args)

    import numpy as np
    import torch
    import torch.distributed as dist

    from hdkx_aicompiler_b200 import ops, plan, resnet18
    from hdkx_aicompiler_b200.parallel import GatherToWorker0, PeerStoreToWorker0, bind_to_device_numa_node, shard_range

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N")
    assert torch.cuda.is_available(), "bench.py needs a GPU (there is no CPU path)"
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    numa_cpus = bind_to_device_numa_node(local_rank) if world > 1 else None  # before the pinned buffers are allocated
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    shard_begin, shard_end = shard_range(rank, world, args.batch)
    per_gpu = shard_end - shard_begin
    warmup = max(args.warmup, 3)

    weights = resnet18.make_weights(seed=0)
    func = resnet18.build(per_gpu, weights, to_constant=lambda a: torch.from_numpy(a).to(device))
    graph = plan.CompiledGraph(func, args.precision, cuda_graph=True)

    gen = torch.Generator(device="cpu").manual_seed(1234 + rank)
    host_in = torch.empty((per_gpu, 3, 224, 224), dtype=torch.float32).normal_(0, 1, generator=gen).pin_memory()
    # Consecutive steps are pipelined the way a serving loop would run them: two input and two output buffers,
    # the host->device copy of step i+1 (copy stream) and the gather / read-back of step i-1 (gather stream)
    # overlap the kernels of step i (run stream). Every step's copies and its gather are still issued inside
    # the timed region and are complete when it ends.
    xs = [host_in.to(device, non_blocking=True), host_in.to(device, non_blocking=True)]
    x = xs[0]
    logits_buf = [torch.empty(graph.out_shape, dtype=torch.float32, device=device) for _ in range(2)]
    logits = logits_buf[0]
    gathers = [GatherToWorker0(graph.out_shape, torch.float32, device) for _ in range(2)]
    peers = None
    if args.gather == "peer" and world > 1:
        # Measured at 8 GPUs, 30 steps: 0.574 ms per step with peer stores against 0.592 with the NCCL gather, whose kernel
        # holds SMs while the next step's first (persistent) kernel starts. All ranks take the same form: one that
        # cannot set up symmetric memory sends every rank back to NCCL.
        # The set-up is collective, so the ranks first agree that each of them can take part (the module exists and every
        # other GPU of the node is peer-accessible) and only then enter it; a failure inside is agreed on the same way.
        try:
            import torch.distributed._symmetric_memory  # noqa: F401
            able = all(torch.cuda.can_device_access_peer(local_rank, o) for o in range(world) if o != local_rank)
        except Exception:  # noqa: BLE001
            able = False
        ok = torch.tensor([1.0 if able else 0.0], device=device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if ok.item() >= 1:
            try:
                peers = [PeerStoreToWorker0(graph.out_shape, torch.float32, device) for _ in range(2)]
            except Exception:  # noqa: BLE001
                ok.zero_()
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if ok.item() < 1:
                peers = None
    exchange = "peer stores from the last kernel" if peers else ("nccl gather" if world > 1 else "none (one GPU)")
    host_out = torch.empty((args.batch if rank == 0 else per_gpu, graph.out_shape[1]), dtype=torch.float32).pin_memory()

    run_stream = torch.cuda.Stream(device)  # a real stream: the legacy default stream cannot be graph-captured
    copy_stream = torch.cuda.Stream(device)
    gather_stream = torch.cuda.Stream(device)
    run_stream.wait_stream(torch.cuda.current_stream(device))
    copy_stream.wait_stream(torch.cuda.current_stream(device))
    gather_stream.wait_stream(torch.cuda.current_stream(device))
    torch.cuda.set_stream(run_stream)
    x_free = [None, None]      # kernels that read xs[j] have finished
    out_free = [None, None]    # gather / read-back of logits_buf[j] has finished
    counter = [0]

    def step(from_host):
        j = counter[0] & 1
        counter[0] += 1
        if from_host:
            with torch.cuda.stream(copy_stream):
                if x_free[j] is not None:
                    copy_stream.wait_event(x_free[j])
                xs[j].copy_(host_in, non_blocking=True)
                ready = torch.cuda.Event()
                ready.record(copy_stream)
            run_stream.wait_event(ready)
        if out_free[j] is not None:
            run_stream.wait_event(out_free[j])
        graph.run(xs[j], out=peers[j].output() if peers else logits_buf[j])
        done = torch.cuda.Event()
        done.record(run_stream)
        x_free[j] = done
        with torch.cuda.stream(gather_stream):
            gather_stream.wait_event(done)
            if peers:
                peers[j].complete()  # every rank's last kernel has stored its shard into rank 0's buffer
                if from_host and rank == 0:
                    host_out.copy_(peers[j].gathered(), non_blocking=True)
                # a second barrier after rank 0 has read: no rank's stores of a LATER step may land in this buffer before
                peers[j].complete()
            else:
                parts = gathers[j](logits_buf[j])  # GatherToWorker0: shards in rank order on rank 0
                if from_host and rank == 0:
                    for r, part in enumerate(parts):
                        host_out[r * per_gpu:(r + 1) * per_gpu].copy_(part, non_blocking=True)
            fin = torch.cuda.Event()
            fin.record(gather_stream)
        out_free[j] = fin

    def timed(from_host, steps):
        for _ in range(warmup):
            step(from_host)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            step(from_host)
        run_stream.wait_stream(gather_stream)  # the timed region ends when the last gather / read-back has finished
        run_stream.wait_stream(copy_stream)
        e1.record()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        ms = torch.tensor([e0.elapsed_time(e1)], device=device)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    # With more than one GPU: one untimed step through BOTH forms of the exchange, compared bit for bit on rank 0
    # (the dense layer's epilogue storing its logits straight into rank 0's buffer over NVLink vs the NCCL gather).
    peer_check = None
    if world > 1:
        try:
            chk = peers[0] if peers else PeerStoreToWorker0(graph.out_shape, torch.float32, device)
            graph.run(xs[0], out=chk.output())
            chk.complete()
            graph.run(xs[0], out=logits_buf[0])
            parts = gathers[0](logits_buf[0])
            torch.cuda.synchronize()
            if rank == 0:
                peer_check = "ok" if torch.equal(chk.gathered(), torch.cat(parts, 0)) else "failed"
            chk.complete()
        except Exception as e:  # noqa: BLE001  (symmetric memory unavailable on this box: report, do not fail the bench)
            peer_check = f"unavailable: {type(e).__name__}"

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    total_ms = timed(False, args.steps)
    clocks = sampler.stop() if rank == 0 else None
    e2e_ms = timed(True, args.steps)
    ops.device_status(device)

    # per-launch durations (one extra run with an event between launches), rank 0's shard
    _, launch_ms = graph.run_timed(x, out=logits)
    for _ in range(2):
        _, more = graph.run_timed(x, out=logits)
        launch_ms = [min(a, b) for a, b in zip(launch_ms, more)]
    info = graph.launch_info()

    if world > 1:
        dist.barrier()
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks = load_peaks()
    ms_per_step = total_ms / args.steps
    value = args.batch / (ms_per_step / 1e3)
    tc = [(n, f, b, t) for (n, f, b), t in zip(info, launch_ms) if n.startswith(("conv_", "dense_"))]
    tc_flops = sum(f for _, f, _, _ in tc)
    tc_ms = sum(t for _, _, _, t in tc)
    achieved = tc_flops / (tc_ms / 1e3) / 1e12
    layers = [{"launch": n, "ms": round(t, 4), "tflops": round(f / (t / 1e3) / 1e12, 1) if f else None,
               "gbs": round(b / (t / 1e3) / 1e9, 0)} for (n, f, b), t in zip(info, launch_ms)]
    families = collections.Counter(n.split()[0] for n, _, _, _ in tc)
    traffic = None
    if args.precision == "bf16" and all(NCU_DRAM_BYTES_PER_IMAGE.get(k) is not None for k in families):
        traffic = sum(NCU_DRAM_BYTES_PER_IMAGE[k] for k in families) * per_gpu
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16" if args.precision == "bf16" else "tf32", "data": "synthetic",
        "config": {"workload": f"resnet18 inference, global batch {args.batch}, {args.precision} operands / fp32 accumulate, "
                               f"{per_gpu} images per GPU, weights replicated, logits gathered to rank 0"
                               + (" by peer stores from the dense layer's epilogue" if peers else ""),
                   "global_batch": args.batch, "per_gpu_batch": per_gpu, "parallelism": f"dp{world}",
                   "l2": "inputs larger than L2 (616 MB of images and >1 GB of activations per step per GPU at N=1)",
                   "pipelining": "steps overlap: input copy of step i+1 and gather/read-back of step i-1 run beside the kernels of step i",
                   "exchange": exchange,
                   "host_numa_binding": (f"rank 0 bound to {len(numa_cpus)} CPUs next to its GPU" if numa_cpus else "none")},
        "clocks": clocks,
        "e2e": {"value": args.batch / (e2e_ms / args.steps / 1e3), "unit": UNIT,
                "h2d_bytes_per_step": int(host_in.numel() * 4 * world), "d2h_bytes_per_step": int(args.batch * graph.out_shape[1] * 4)},
        "gpu_launches": int(graph.num_launches * args.steps),
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peaks["tflops_burst"], "unit": "TFLOP/s",
                     "frac": achieved / peaks["tflops_burst"],
                     "peak_sustained": peaks["tflops_sustained"], "frac_sustained": achieved / peaks["tflops_sustained"],
                     "peak_note": "frac: cuBLAS bf16 burst figure (each launch is timed alone between CUDA events, best of three; "
                                  "the timed region lasts ~0.1 s); frac_sustained: the seconds-long figure under the power cap",
                     "step_level": {"achieved": tc_flops / (ms_per_step / 1e3) / 1e12,
                                    "frac": tc_flops / (ms_per_step / 1e3) / 1e12 / peaks["tflops_burst"],
                                    "note": "same FLOPs over the whole device-timed step (all launches, gaps and the gather included)"},
                     "traffic": traffic,
                     "traffic_note": f"dram read+write bytes per image by kernel family from ncu captures at {NCU_TRAFFIC_BATCH} images per GPU, "
                                     "summed and scaled by the per-GPU batch; algorithmic bytes: %.2f GB" % (
                                         sum(b for n, f, b in info if n.startswith(("conv_", "dense_"))) / 1e9),
                     "peak_source": peaks["source"],
                     "kernel": "all tensor-core launches of a step: " + ", ".join(f"{c} x {k}" for k, c in sorted(families.items())),
                     "flops_per_step_per_gpu": tc_flops, "ms_per_step_in_kernel": tc_ms},
        "launches": layers,
    }
    if peer_check is not None:
        line["peer_store_check"] = peer_check
    if world == 1 and not args.no_side_configs:
        # the benchmark's other single-GPU configurations, in the same process on the same GPU (after the headline timing)
        import microbench
        microbench.QUIET = True
        del graph, xs, logits_buf
        torch.cuda.empty_cache()
        torch.cuda.set_stream(torch.cuda.default_stream(device))
        flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=device)
        hbm, tf = peaks["hbm_gbs"], peaks["tflops_burst"]
        line["hbm_kernels"] = [{"kernel": r["kernel"], "form": r["form"], "bytes": r["algorithmic_bytes"], "ms": round(r["ms"], 5),
                                "gbs": round(r["gbs"], 1), "frac": round(r["frac_of_hbm_peak"], 4)}
                               for r in microbench.config2(10, flush, hbm, tf, peaks["source"])]
        line["hbm_kernels_note"] = ("max_pool2d 3x3 s2 p1 on 32x64x112x112 fp32 -> add -> relu through the C ABI, L2 flushed between "
                                    f"iterations; frac = algorithmic bytes / time / measured copy bandwidth {hbm} GB/s")
        c1 = microbench.config1_plan(10, flush, hbm, tf, peaks["source"])
        line["config1"] = {"workload": "conv2d 1x64x56x56 (*) 64x64x3x3 + bias + relu, bf16 plan, CUDA-graph replay",
                           "ms": round(c1["ms"], 5), "tflops": round(c1["tflops"], 2), "launch_ms": c1["launch_ms"]}
        line["config3"] = [{"workload": r["kernel"], "ms": round(r["ms"], 4), "img_per_s": round(r["img_per_s"], 1),
                            "tflops": round(r["tflops"], 1)} for r in microbench.config3(5, flush, hbm, tf, peaks["source"])]
    if not args.no_cpu_baseline:
        cpu_value, kind = cpu_reference_throughput(4, 1, steps=1, warmup=0)
        line["cpu_baseline"] = {"value": cpu_value, "unit": UNIT, "cores": 1, "kind": kind,
                                "sample": f"4 images of the same network on one core, {4 / cpu_value:.1f} s timed (the per-operator kernels "
                                          "are compiled and loaded before the timed pass)"}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
