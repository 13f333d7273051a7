"""Generates tests/golden/import_block.{json,bin} and import_block_io.npz.

Run in a checkout that has the reference compiler built as the oracle's checker (make -C oracle ref): the graph is
written in the reference's interchange format, read back by the reference's own importer (oracle/_ref/ref_emit
--import) and evaluated with the CPU kernels the reference's compiler generates (oracle backend "ref").
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from hdkx_aicompiler_b200 import onnx_import  # noqa: E402
from oracle import graph as ograph  # noqa: E402
from oracle import importer as oimp  # noqa: E402
from oracle import ref as oref  # noqa: E402
from test_onnx_import import small_block  # noqa: E402

here = os.path.dirname(os.path.abspath(__file__))
rng = np.random.default_rng(2024)
func, out_shape = small_block(rng)
j, p = os.path.join(here, "import_block.json"), os.path.join(here, "import_block.bin")
onnx_import.save_spec(func, out_shape, j, p)
ref_func, ref_shape = oimp.to_relay(oimp.describe(j, p), oimp.read_params(j, p))
x = rng.normal(0, 1, (2, 3, 20, 20)).astype(np.float32)
out = ograph.run(ref_func, [x], backend=oref)
assert tuple(out.shape) == tuple(ref_shape) == tuple(out_shape)
np.savez(os.path.join(here, "import_block_io.npz"), input=x, output=out)
print("wrote", j, p, "output", out.shape, float(np.abs(out).max()))
