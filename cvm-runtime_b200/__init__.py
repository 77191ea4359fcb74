"""B200-native operator hot path of the CVM runtime.

`runtime` binds the C-ABI of libcvm_runtime.so (the twelve CVMAPI* entry points of the reference's
kernel/c_api.h); `workloads` builds the seeded synthetic models used for parity and benchmarks;
`build` compiles the library in-tree.  The directory name carries a hyphen, so load the package
with `__graft_entry__.load_package()` (or importlib) rather than a plain import statement.
"""
from . import runtime, sharding, workloads  # noqa: F401
from .build import build, LIB  # noqa: F401
