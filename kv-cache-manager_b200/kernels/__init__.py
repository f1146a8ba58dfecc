"""The hand-written CUDA kernels (sm_100a) behind one Python module; see ``library.py``."""
from . import library
from .library import KernelError, launch_count, reset_launch_count

__all__ = ["library", "KernelError", "launch_count", "reset_launch_count"]
