"""cuqwen_b200: a B200 (sm_100a) batch-1 Qwen2.5 decode engine behind a C ABI.

The product is ``libcuqwen_b200.so`` (sources in ``csrc/``, interface in
``include/cuqwen_b200.h``).  This package only binds it for tests, benchmarks
and Python hosts; importing the bindings does not load the library until a
function is called, and a missing library raises instead of falling back.
"""
from . import binfmt  # noqa: F401  (pure numpy, usable without the CUDA library)
from ._abi import CuQwenError, Params, lib  # noqa: F401
