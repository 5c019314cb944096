"""Import-path alias: ``import ayla`` resolves to the sm_100a backend.

Code written against the reference imports ``ayla.gemm_jit``, ``ayla.torch_compile``,
``ayla.torch_custom_call`` and ``ayla.jit_compiler`` (README.md:37-45 of the reference).
This package makes those module paths name the modules of :mod:`ayla_b200`, so such code
runs unchanged; it adds no code of its own.  Do not install it next to the reference
itself: both would claim the name ``ayla``.
"""

import sys

import ayla_b200
from ayla_b200 import *  # noqa: F401,F403
from ayla_b200 import (gemm_jit, gemm_schedule_table, jit_compiler, swiglu, torch_compile,  # noqa: F401
                       torch_custom_call)

for _name in ("gemm_jit", "gemm_schedule_table", "jit_compiler", "swiglu", "torch_compile", "torch_custom_call",
              "dynamic_m"):
    _module = __import__(f"ayla_b200.{_name}", fromlist=[_name])
    sys.modules[f"{__name__}.{_name}"] = _module
    globals()[_name] = _module

__all__ = list(getattr(ayla_b200, "__all__", []))
