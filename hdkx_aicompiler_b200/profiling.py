"""Profiling events of the operator path in the reference's bundle format.

The reference writes one JSON object per line into <bundle>/events.jsonl (SerializeEventLine, src/base/profiling.cc:741-772)
and its agent reads only that file (python/kxc_agent/services/diagnosis_engine.py): `compiled_module_run` events shorter
than its threshold raise `kernel_launch_overhead`, and `component == "device_api"` events with `event_type == "copy"`
against all device_api events raise `copy_dominance`. This module records the same events for a CompiledGraph:

  component "runtime",    event_type "compiled_module_run"  one per run of the plan (device time of the whole run)
  component "kernel",     event_type "kernel_launch"        one per launch inside the run: kernel_symbol = the launch's
                                                            label, metrics = device time, algorithmic flops and bytes
  component "device_api", event_type "copy"                 host<->device copies made through ProfiledRun.copy_*
  component "device_api", event_type "stream_sync"          the synchronisation that ends a profiled run

Times are device times from CUDA events (`ts_ns` is the host clock at submission). Every key SerializeEventLine writes
is present, so the reference's reader needs no change.
"""
import json
import os
import threading
import time
import uuid

import torch

EVENT_KEYS = ("trace_id", "session_id", "run_id", "span_id", "parent_span_id", "component", "event_type", "phase", "ts_ns",
              "duration_ns", "status", "severity", "device", "worker_id", "op_name", "pass_name", "kernel_symbol",
              "shape_signature", "message", "fields", "metrics")


def make_event(trace_id, session_id, run_id, span_id, parent_span_id, component, event_type, ts_ns, duration_ns, device="",
               worker_id=-1, op_name="", kernel_symbol="", shape_signature="", message="", fields=None, metrics=None,
               status="ok", severity="info"):
    """One events.jsonl record with exactly the reference's keys."""
    f = {str(k): str(v) for k, v in (fields or {}).items()}
    f.setdefault("thread_id", str(threading.get_ident()))
    f["schema_version"] = "1"
    return {"trace_id": trace_id, "session_id": session_id, "run_id": run_id, "span_id": span_id,
            "parent_span_id": parent_span_id, "component": component, "event_type": event_type, "phase": "complete",
            "ts_ns": int(ts_ns), "duration_ns": int(duration_ns), "status": status, "severity": severity, "device": device,
            "worker_id": int(worker_id), "op_name": op_name, "pass_name": "", "kernel_symbol": kernel_symbol,
            "shape_signature": shape_signature, "message": message, "fields": f,
            "metrics": {str(k): float(v) for k, v in (metrics or {}).items()}}


class ProfileBundle:
    """Collects events and writes <bundle_dir>/events.jsonl (the file the reference's agent loads)."""

    def __init__(self, bundle_dir, worker_id=-1, trace_id=None, session_id=None):
        self.bundle_dir = bundle_dir
        self.worker_id = worker_id
        self.trace_id = trace_id or "trace-" + uuid.uuid4().hex[:16]
        self.session_id = session_id or "session-" + uuid.uuid4().hex[:16]
        self.events = []
        self._t0 = time.monotonic_ns()
        self._n = 0

    def now_ns(self):
        return time.monotonic_ns() - self._t0

    def new_id(self, prefix):
        self._n += 1
        return f"{prefix}-{self._n}"

    def add(self, **kw):
        kw.setdefault("worker_id", self.worker_id)
        ev = make_event(self.trace_id, self.session_id, **kw)
        self.events.append(ev)
        return ev

    def write(self):
        """Write the whole bundle the reference's loader asks for (python/kxc_agent/services/bundle_loader.py:14-21):
        manifest.json, events.jsonl, trace.json (Chrome / Perfetto "X" events, SerializePerfettoEvent in
        src/base/profiling.cc:774-798), summary.json, a not-yet-analysed diagnosis.json / diagnosis.md and artifacts/."""
        os.makedirs(os.path.join(self.bundle_dir, "artifacts"), exist_ok=True)

        def dump(name, obj):
            with open(os.path.join(self.bundle_dir, name), "w", encoding="utf-8") as f:
                json.dump(obj, f, separators=(",", ":"))

        dump("manifest.json", {"schema_version": 1, "trace_id": self.trace_id, "session_id": self.session_id,
                               "producer": "hdkx_aicompiler_b200", "enable_nvtx": False, "enable_cupti": False,
                               "event_count": len(self.events)})
        path = os.path.join(self.bundle_dir, "events.jsonl")
        with open(path, "w", encoding="utf-8") as f:
            for ev in self.events:
                f.write(json.dumps(ev, separators=(",", ":")) + "\n")
        trace = [{"name": ev["event_type"] or ev["component"], "cat": ev["component"], "ph": "X" if ev["duration_ns"] > 0 else "i",
                  "ts": ev["ts_ns"] // 1000, "dur": ev["duration_ns"] // 1000, "pid": os.getpid(), "tid": 0, "s": "t",
                  "args": {"status": ev["status"], "severity": ev["severity"], "message": ev["kernel_symbol"] or ev["message"]}}
                 for ev in self.events]
        dump("trace.json", {"traceEvents": trace, "metadata": {"trace_id": self.trace_id, "session_id": self.session_id,
                                                                "start_time_ns": self._t0}})
        counts = {}
        for ev in self.events:
            counts[ev["component"]] = counts.get(ev["component"], 0) + 1
        dump("summary.json", {"trace_id": self.trace_id, "session_id": self.session_id, "event_count": len(self.events),
                              "component_counts": {k: str(v) for k, v in counts.items()}})
        note = {"category": "not_analyzed", "severity": "info", "component": "analysis",
                "summary": "Bundle created. Run the reference's kxc_agent analyze_bundle on this directory to populate diagnostics."}
        dump("diagnosis.json", {"trace_id": self.trace_id, "diagnostics": [note]})
        with open(os.path.join(self.bundle_dir, "diagnosis.md"), "w", encoding="utf-8") as f:
            f.write("# Diagnostics\n\n- [info] not_analyzed (analysis): " + note["summary"] + "\n")
        return path


def launch_events(bundle, run_id, parent_span_id, ts_ns, labels_flops_bytes, launch_ms, device, shape_signature):
    """kernel_launch events of one run from per-launch device times (no GPU needed: used by the CPU tests too)."""
    t = ts_ns
    for (label, flops, nbytes), ms in zip(labels_flops_bytes, launch_ms):
        dur = int(round(ms * 1e6))
        bundle.add(run_id=run_id, span_id=bundle.new_id("span"), parent_span_id=parent_span_id, component="kernel",
                   event_type="kernel_launch", ts_ns=t, duration_ns=dur, device=device, op_name=label.split(" ")[0],
                   kernel_symbol=label, shape_signature=shape_signature,
                   metrics={"device_ms": ms, "algorithmic_flops": flops, "algorithmic_bytes": nbytes})
        t += dur


class ProfiledRun:
    """Runs a CompiledGraph and records the events listed in the module docstring."""

    def __init__(self, graph, bundle):
        self.graph = graph
        self.bundle = bundle
        self.device = f"cuda:{graph.device.index}"
        self._info = graph.launch_info()

    def _timed(self, fn):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ts = self.bundle.now_ns()
        e0.record()
        out = fn()
        e1.record()
        e1.synchronize()
        return out, ts, int(e0.elapsed_time(e1) * 1e6)

    def copy_to_device(self, host, dev, run_id=""):
        _, ts, dur = self._timed(lambda: dev.copy_(host, non_blocking=True))
        self.bundle.add(run_id=run_id, span_id=self.bundle.new_id("span"), parent_span_id="", component="device_api",
                        event_type="copy", ts_ns=ts, duration_ns=dur, device=self.device,
                        fields={"direction": "h2d"}, metrics={"bytes": host.numel() * host.element_size()})
        return dev

    def copy_to_host(self, dev, host, run_id=""):
        _, ts, dur = self._timed(lambda: host.copy_(dev, non_blocking=True))
        self.bundle.add(run_id=run_id, span_id=self.bundle.new_id("span"), parent_span_id="", component="device_api",
                        event_type="copy", ts_ns=ts, duration_ns=dur, device=self.device,
                        fields={"direction": "d2h"}, metrics={"bytes": dev.numel() * dev.element_size()})
        return host

    def run(self, *inputs, out=None):
        run_id = self.bundle.new_id("run")
        span = self.bundle.new_id("span")
        sig = ";".join("x".join(str(int(d)) for d in t.shape) for t in inputs)
        ts = self.bundle.now_ns()
        out, ms = self.graph.run_timed(*inputs, out=out)  # synchronises
        total = int(round(sum(ms) * 1e6))
        self.bundle.add(run_id=run_id, span_id=span, parent_span_id="", component="runtime", event_type="compiled_module_run",
                        ts_ns=ts, duration_ns=total, device=self.device, shape_signature=sig,
                        fields={"precision": self.graph.precision, "launches": len(ms)},
                        metrics={"device_ms": sum(ms)})
        launch_events(self.bundle, run_id, span, ts, self._info, ms, self.device, sig)
        self.bundle.add(run_id=run_id, span_id=self.bundle.new_id("span"), parent_span_id=span, component="device_api",
                        event_type="stream_sync", ts_ns=ts + total, duration_ns=0, device=self.device)
        return out, run_id
