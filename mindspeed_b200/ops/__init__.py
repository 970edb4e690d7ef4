"""Op layer: hand-written sm_100a kernels behind small Python functions.

``_lib`` loads the in-tree shared library built by ``mindspeed_b200.ops.build``
(plain ``nvcc -shared``; every kernel launcher is an ``extern "C"`` symbol taking raw
device pointers and a stream, called through ``ctypes``).  On a machine with a GPU a
missing library is an error, never a silent fallback; on a CPU-only machine the
eager PyTorch restatement of each op is used (that is also the numerics oracle in
the tests).
"""
from .loader import lib, have_lib, require_lib, launch_count, reset_launch_count  # noqa: F401
