"""B200 (sm_100a) implementation of the tfg_custom_ops hot path of
schellmi42/tensorflow_graphics_point_clouds.

`custom_ops` exposes the reference's op callables; `pc` mirrors the pylib
classes that call them (PointCloud, Grid, Neighborhood, sampling,
PointHierarchy) and `mcconv` the Monte-Carlo convolution layer.  All compute
runs in libtfgpc.so (include/tfgpc.h); nothing falls back to the CPU.
"""
from . import _lib  # noqa: F401
from . import custom_ops  # noqa: F401

__all__ = ["custom_ops", "_lib"]
