"""pssa_b200: B200-native PSSA inference forward path behind the reference's dispatch interface.

`dispatch.B200Dispatch` mirrors the reference's `GpuDispatch` (src/backend.rs:1025-1446); the work
happens in libpssa_b200.so (hand-written sm_100a CUDA), reached through the C ABI of include/pssa_b200.h.
"""
from ._native import B200Error, LIB_PATH, lib  # noqa: F401
from .dispatch import B200Dispatch, Device  # noqa: F401
from .model import PSSAModel  # noqa: F401

__all__ = ["B200Dispatch", "B200Error", "Device", "LIB_PATH", "PSSAModel", "lib"]
