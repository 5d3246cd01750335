"""ctypes binding of libwhetstone_b200.so -- the raw C ABI of include/whetstone.h
and include/whetstone_b200.h, one Python callable per exported symbol.

This is the Python counterpart of the engine's
crates/whetstone-kernels/src/ffi.rs (raw declarations) plus the status mapping
of crates/whetstone-kernels/src/lib.rs:47-98 (`check`).  There is no fallback:
if the shared library is missing, importing this module raises.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_double, c_float, c_int32, c_int64, c_size_t, c_uint32, c_void_p
from pathlib import Path

_LIB_NAME = "libwhetstone_b200.so"


class WstError(RuntimeError):
    """A non-OK wst_status_t, with the library's thread-local message."""

    code = -1

    def __init__(self, code: int, message: str):
        super().__init__(f"{self.__class__.__name__}({code}): {message}")
        self.code = code
        self.message = message


class CudaError(WstError):
    pass


class InvalidArg(WstError):
    pass


class UnsupportedArch(WstError):
    pass


class OutOfMemory(WstError):
    pass


class ShapeError(WstError):
    pass


_STATUS = {1: CudaError, 2: InvalidArg, 3: UnsupportedArch, 4: OutOfMemory, 5: ShapeError}


def _find_library() -> Path:
    override = os.environ.get("WHETSTONE_B200_LIB")
    here = Path(__file__).resolve().parent
    path = Path(override) if override else here / _LIB_NAME
    if not path.exists():
        raise ImportError(
            f"{path} not found: build it with `make -C {here / 'csrc'}` "
            "(or `python -c 'import __graft_entry__ as g; g.build()'`). "
            "There is no CPU fallback for the attention path.")
    return path


LIB_PATH = _find_library()
lib = ctypes.CDLL(str(LIB_PATH))

P = c_void_p
I = c_int32
F = c_float

# name -> (restype, argtypes).  Kept in one table so that the test which checks
# the exported symbols against the headers can iterate over it.
SIGNATURES: dict[str, tuple] = {
    "wst_last_error": (c_char_p, []),
    "wst_device_count": (I, [ctypes.POINTER(c_int32)]),
    "wst_device_set": (I, [I]),
    "wst_device_synchronize": (I, []),
    "wst_malloc": (I, [ctypes.POINTER(c_void_p), c_size_t]),
    "wst_free": (I, [P]),
    "wst_memset": (I, [P, I, c_size_t]),
    "wst_memcpy_h2d": (I, [P, P, c_size_t]),
    "wst_memcpy_d2h": (I, [P, P, c_size_t]),
    "wst_memcpy_d2d": (I, [P, P, c_size_t]),
    "wst_graph_capture_begin": (I, []),
    "wst_graph_capture_end": (I, [ctypes.POINTER(c_void_p)]),
    "wst_graph_launch": (I, [P]),
    "wst_graph_destroy": (I, [P]),
    "wst_stream_sync": (I, []),
    "wst_event_create": (I, [ctypes.POINTER(c_void_p)]),
    "wst_event_record": (I, [P]),
    "wst_event_elapsed_ms": (I, [P, P, ctypes.POINTER(c_float)]),
    "wst_event_destroy": (I, [P]),
    "wst_advance_pos": (I, [P, I]),
    "wst_rope_cache": (I, [P, P, P, P, P, I, I, I, P, I, P, P, F]),
    "wst_attn_decode": (I, [P, P, P, P, P, I, I, I, P, I, F]),
    "wst_attn_partial_floats": (I, [I, I, I]),
    "wst_rope_cache_chunk": (I, [P, P, P, P, P, I, I, I, I, I, I, P, P, F]),
    "wst_attn_chunk": (I, [P, P, P, P, I, I, I, I, I, I, F]),
    "wst_gemm_fp16": (I, [P, P, P, P, I, I, I, I]),
    "wst_gemm_int4_hier": (I, [P, P, P, P, P, P, I, I, I, I]),
    "wst_chunk_max_tokens": (I, []),
    # extensions (whetstone_b200.h)
    "wst_b200_version": (c_char_p, []),
    "wst_b200_set_stream": (I, [P]),
    "wst_b200_device_error": (I, [ctypes.POINTER(c_uint32)]),
    "wst_b200_set_kernel_choice": (I, [I]),
    "wst_rope_table_host": (I, [P, P, I, I, c_double, I, c_double, c_double, c_double, I]),
    "wst_attn_decode_partial": (I, [P, P, P, P, P, I, I, I, P, I, F]),
    "wst_attn_merge_partials": (I, [P, P, I, I, I]),
    "wst_attn_exchange_merge": (I, [P, P, P, P, I, I, I, I]),
    "wst_attn_decode_sharded": (I, [P, P, P, P, P, I, I, I, P, I, F, P, P, I, I]),
    "wst_b200_set_tuning": (I, [I, I]),
    "wst_b200_set_decode_overlap": (I, [I]),
    "wst_b200_reserve_chunk_workspace": (I, []),
    "wst_b200_enable_peer_access": (I, [I]),
    "wst_b200_ipc_export": (I, [P, P]),
    "wst_b200_ipc_import": (I, [P, ctypes.POINTER(ctypes.c_void_p)]),
    "wst_b200_ipc_close": (I, [P]),
    "wst_attn_decode_noscratch": (I, [P, P, P, P, I, I, I, P, I, F]),
    "wst_rope_cache_chunk_batch": (I, [P, P, P, P, P, P, I, I, I, I, I, I, P, P, F]),
    "wst_attn_chunk_batch": (I, [P, P, P, P, P, I, I, I, I, I, I, F]),
    "wst_b200_qkv_rope_append_batch": (I, [P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, P, P, F]),
    "wst_b200_qkv_int4_rope_append_batch": (I, [P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, P, P, F]),
    "wst_b200_attn_chunk_batch_q16": (I, [P, P, P, P, P, I, I, I, I, I, I, F]),
    "wst_b200_rope_cache_fp8": (I, [P, P, P, P, P, I, I, I, P, I, I, I, P, P, F, F, F]),
    "wst_b200_attn_decode_fp8": (I, [P, P, P, P, P, I, I, I, P, I, F, F, F]),
    "wst_rope_cache_paged": (I, [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, P, P, F]),
    "wst_attn_verify_paged": (I, [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, F]),
    "wst_attn_verify_scratch_floats": (c_int64, [I, I, I, I, I, I]),
    # host-side paged KV-cache manager and scheduler (no GPU work)
    "wst_pkv_create": (I, [I, I, ctypes.POINTER(c_void_p)]),
    "wst_pkv_destroy": (I, [P]),
    "wst_pkv_open": (I, [P, ctypes.POINTER(c_int32)]),
    "wst_pkv_close": (I, [P, I]),
    "wst_pkv_query": (I, [P, I, ctypes.POINTER(c_int32), ctypes.POINTER(c_int32),
                          ctypes.POINTER(c_int32)]),
    "wst_pkv_reserve": (I, [P, I, I]),
    "wst_pkv_commit": (I, [P, I, I]),
    "wst_pkv_rewind": (I, [P, I, I]),
    "wst_pkv_trim": (I, [P, I, I, ctypes.POINTER(c_int32)]),
    "wst_pkv_schedule": (I, [P, P, P, I, I, I, P, ctypes.POINTER(c_int32)]),
    "wst_pkv_build_step": (I, [P, P, P, I, P, P, P, P]),
    "wst_pkv_assign_units": (I, [P, P, I, I, I, P]),
}

for _name, (_res, _args) in SIGNATURES.items():
    _fn = getattr(lib, _name)  # AttributeError here = the library lacks a declared symbol
    _fn.restype = _res
    _fn.argtypes = _args


def last_error() -> str:
    return lib.wst_last_error().decode("utf-8", "replace")


def check(status: int) -> None:
    """Raise the typed error for a non-zero status (lib.rs:88-98)."""
    if status == 0:
        return
    raise _STATUS.get(status, WstError)(status, last_error())


def version() -> str:
    return lib.wst_b200_version().decode()
