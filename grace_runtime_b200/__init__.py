"""grace_runtime_b200 - B200-native evaluation backend for GRACE-1L / GRACE-2L models (energy, forces, virial of one
structure or a batch), a drop-in for the GPU plug-in interface of ICAMS/grace-runtime.

`backend` mirrors the reference's plug-in module (Model / System / Batch); `modelgen` and `structures` write the
random-init benchmark models and synthetic structures; `build` compiles libgrace_b200.so for sm_100a.
"""
from . import backend  # noqa: F401
from .backend import ABI, Batch, Model, System, arch, archs, finalize, initialize, initialized, memory_info  # noqa: F401

__all__ = ["ABI", "Batch", "Model", "System", "arch", "archs", "finalize", "initialize", "initialized", "memory_info",
           "backend"]
