"""Generates tests/golden/profile_diagnosis.json.

Builds two synthetic profiling bundles with hdkx_aicompiler_b200.profiling (no GPU: fixed per-launch times), lets the
reference's own agent (python/kxc_agent, imported from a checkout of KDZZZZZZ/hdkx-aicompiler given as argv[1]) analyse
them, and stores the diagnosis categories it reports. tests/test_profiling.py rebuilds the same bundles and checks the
committed result, so the event format stays one the reference's reader accepts.

Usage: python tests/golden/make_profile_fixture.py /path/to/hdkx-aicompiler
"""
import json
import os
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.join(HERE, ".."))

from profile_cases import build_case, CASES  # noqa: E402


def main():
    ref = sys.argv[1]
    sys.path.insert(0, os.path.join(ref, "python"))
    from kxc_agent.services.diagnosis_engine import analyze_bundle
    out = {}
    for name in CASES:
        with tempfile.TemporaryDirectory() as d:
            build_case(name, d).write()
            res = analyze_bundle(d)
            out[name] = {"schema_version": res["schema_version"],
                         "diagnostics": [{"category": x["category"], "severity": x["severity"], "component": x["component"]}
                                         for x in res["diagnostics"]]}
    with open(os.path.join(HERE, "profile_diagnosis.json"), "w") as f:
        json.dump(out, f, indent=2, sort_keys=True)
        f.write("\n")
    print(json.dumps(out, indent=2))


if __name__ == "__main__":
    main()
