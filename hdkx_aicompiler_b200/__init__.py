"""hdkx_aicompiler_b200 — host-side mirror of the hdkx-aicompiler ("kxc") operator API over
libkxc_b200.so, the hand-written sm_100a kernels for the operators its Relay graphs lower into.

The package is named with an underscore because a hyphen cannot appear in a Python module name.

`ops`   per-operator calls named after the Relay ops (nn_conv2d, nn_relu, add, nn_max_pool2d, ...)
`_lib`  the ctypes binding of the C ABI declared in include/kxc_b200.h

There is no CPU implementation here: every call goes to the CUDA library and fails loudly when it or
a Blackwell GPU is missing.
"""
from . import _lib  # noqa: F401
from ._lib import KxcError, library_path, load  # noqa: F401
from . import plan  # noqa: F401,E402  (registers the plan entry points with the binding table)
