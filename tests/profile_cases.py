"""Synthetic profiling bundles shared by tests/test_profiling.py and tests/golden/make_profile_fixture.py (no GPU)."""
from hdkx_aicompiler_b200 import profiling

CASES = ("large_batch", "tiny_runs_copy_bound")


def build_case(name, bundle_dir):
    b = profiling.ProfileBundle(bundle_dir, worker_id=0, trace_id="trace-fixture", session_id="session-fixture")
    b._t0 = 0
    info = [("stem_pack c3 h224 w224 -> 230x232x4", 0.0, 8.0e8), ("conv_stem_pool c3 h224 w224 -> o64 k7x7 s2 +relu", 2.4e11, 6.0e8),
            ("conv_rowstack c64 h56 w56 -> o64 k3x3 s1 +relu", 2.4e11, 8.2e8), ("gap_nhwc c512 h7 w7", 0.0, 5.2e7),
            ("dense_igemm m1024 k512 -> n1000 bn64", 1.0e9, 6.2e6)]
    if name == "large_batch":
        # one long run per step, copies small against it
        for step in range(3):
            ts = step * 6_000_000
            ms = [0.21, 0.78, 0.21, 0.02, 0.012]
            run_id, span = f"run-{step}", f"span-run-{step}"
            b.add(run_id=run_id, span_id=span, parent_span_id="", component="runtime", event_type="compiled_module_run", ts_ns=ts,
                  duration_ns=int(sum(ms) * 1e6), device="cuda:0", shape_signature="1024x3x224x224",
                  fields={"precision": "bf16", "launches": len(ms)}, metrics={"device_ms": sum(ms)})
            profiling.launch_events(b, run_id, span, ts, info, ms, "cuda:0", "1024x3x224x224")
            b.add(run_id=run_id, span_id=f"span-sync-{step}", parent_span_id=span, component="device_api", event_type="stream_sync",
                  ts_ns=ts + 1_300_000, duration_ns=0, device="cuda:0")
    else:
        # many runs of a tiny batch, each preceded by a host->device copy that takes longer than the run
        for step in range(6):
            ts = step * 400_000
            ms = [0.004, 0.02, 0.01, 0.003, 0.004]
            run_id, span = f"run-{step}", f"span-run-{step}"
            b.add(run_id=run_id, span_id=f"span-copy-{step}", parent_span_id="", component="device_api", event_type="copy", ts_ns=ts,
                  duration_ns=150_000, device="cuda:0", fields={"direction": "h2d"}, metrics={"bytes": 602112.0})
            b.add(run_id=run_id, span_id=span, parent_span_id="", component="runtime", event_type="compiled_module_run",
                  ts_ns=ts + 150_000, duration_ns=int(sum(ms) * 1e6), device="cuda:0", shape_signature="1x3x224x224",
                  fields={"precision": "bf16", "launches": len(ms)}, metrics={"device_ms": sum(ms)})
            profiling.launch_events(b, run_id, span, ts + 150_000, info, ms, "cuda:0", "1x3x224x224")
            b.add(run_id=run_id, span_id=f"span-sync-{step}", parent_span_id=span, component="device_api", event_type="stream_sync",
                  ts_ns=ts + 200_000, duration_ns=1_000, device="cuda:0")
    return b
