"""B200-native (sm_100a) attention path behind the Whetstone engine's wst_* C ABI.

`decode` and `chunk` mirror the engine's safe wrappers of the same names
(crates/whetstone-kernels/src/decode.rs, src/chunk.rs); `paged` and `sharded`
hold what the engine does not have (a paged batch, a KV sequence split over
GPUs).  Importing the package loads libwhetstone_b200.so and fails if it is
missing: there is no fallback path.
"""

from . import _ffi  # noqa: F401  (loads the shared library or raises)
from . import chunk, decode, paged  # noqa: F401
from ._ffi import (CudaError, InvalidArg, OutOfMemory, ShapeError, UnsupportedArch, WstError,
                   version)

__all__ = ["chunk", "decode", "paged", "version", "WstError", "CudaError", "InvalidArg",
           "UnsupportedArch", "OutOfMemory", "ShapeError"]
