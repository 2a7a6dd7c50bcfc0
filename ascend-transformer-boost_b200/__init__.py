"""B200-native paged-decode attention (PagedAttention + ReshapeAndCache) behind the ATB operator API.

The product is libatb_b200.so (CUDA kernels for sm_100a, the C ABI of include/atb_b200.h and the
C++ atb:: operator classes of include/atb/).  This package only holds its build recipe, the ctypes
mirror of the C ABI and the seeded synthetic workloads used by tests and the benchmark.

The directory name is not a Python identifier; load it with `__graft_entry__.load_package()`,
which registers it as the module `atb_b200`.
"""
from . import build as _build  # noqa: F401
from . import capi, sharding, torch_atb, workloads  # noqa: F401

build = _build.build
