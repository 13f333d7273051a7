"""CPU tests of the drop-in boundary: the library loads, exports every symbol the header declares,
and refuses to compute without a GPU (no CPU fallback)."""
import os
import re

import pytest

import hdkx_aicompiler_b200 as kxc
from hdkx_aicompiler_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    names = set()
    inc = os.path.join(ROOT, "include")
    for fn in sorted(os.listdir(inc)):
        if fn.endswith(".h"):
            text = open(os.path.join(inc, fn)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names.update(re.findall(r"\b(kxc_b200_[a-z0-9_]+)\s*\(", text))
    return names


def test_header_symbols_are_exported_and_bound():
    lib = kxc.load()
    declared = _declared_symbols()
    assert declared, "no declarations found in include/*.h"
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} is declared in include/ but not exported by libkxc_b200.so"
    missing_binding = declared - set(_lib.SYMBOLS)
    assert not missing_binding, f"no ctypes binding for {sorted(missing_binding)}"
    assert lib.kxc_b200_abi_version() == 1


def test_no_cpu_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    lib = kxc.load()
    rc = lib.kxc_b200_device_check()
    assert rc == 4, rc
    assert "no CPU fallback" in _lib.last_error()
    # compute entry points refuse as well, before touching any pointer
    rc = lib.kxc_b200_nn_relu(_lib.packed(0, 0), 16, None)
    assert rc == 4
    from hdkx_aicompiler_b200 import ops
    with pytest.raises(ValueError):
        ops.nn_relu(torch.zeros(4))  # CPU tensors are rejected by the host mirror too


def test_product_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, "hdkx_aicompiler_b200")
    for dirpath, _, files in os.walk(pkg):
        for fn in files:
            if fn.endswith((".py", ".cu", ".cuh", ".cc", ".h", ".cpp")):
                text = open(os.path.join(dirpath, fn), errors="replace").read()
                assert "oracle" not in text.replace("no oracle", ""), f"{fn} mentions the oracle"
