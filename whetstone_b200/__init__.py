"""B200-native (sm_100a) attention path behind the Whetstone engine's wst_* C ABI.

`decode` and `chunk` mirror the engine's safe wrappers of the same names
(crates/whetstone-kernels/src/decode.rs, src/chunk.rs); `paged` and `sharded`
hold what the engine does not have (a paged batch, a KV sequence split over
GPUs); `workloads` describes the benchmark inputs and needs no GPU.  The first
use of `decode`, `chunk`, `paged` or of anything from `_ffi` loads
libwhetstone_b200.so and fails if it is missing: there is no fallback path.
`workloads` and the partitioning helpers of `sharded` import without it, so a
process that only times a CPU baseline maps no library of this repository.
"""

import importlib

_LAZY_MODULES = ("_ffi", "chunk", "decode", "paged", "sharded", "workloads")
_FFI_NAMES = ("CudaError", "InvalidArg", "OutOfMemory", "ShapeError", "UnsupportedArch",
              "WstError", "version")

__all__ = ["chunk", "decode", "paged", "sharded", "workloads", "version", "WstError",
           "CudaError", "InvalidArg", "UnsupportedArch", "OutOfMemory", "ShapeError"]


def __getattr__(name):
    if name in _LAZY_MODULES:
        return importlib.import_module(f"{__name__}.{name}")
    if name in _FFI_NAMES:
        return getattr(importlib.import_module(f"{__name__}._ffi"), name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
