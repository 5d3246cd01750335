"""CPU-side checks of the C-ABI library: it loads, it exports every symbol the
headers declare, argument errors come back as status + message with nothing
launched, and the host-side RoPE table equals the oracle's.  No kernel runs."""

import ctypes
import re
import subprocess
from pathlib import Path

import numpy as np
import pytest

from oracle import attention_oracle as orc
from whetstone_b200 import _ffi
from whetstone_b200._ffi import lib

ROOT = Path(__file__).resolve().parent.parent
HEADERS = [ROOT / "include" / "whetstone.h", ROOT / "include" / "whetstone_b200.h"]


def declared_symbols():
    names = []
    for h in HEADERS:
        text = re.sub(r"/\*.*?\*/", "", h.read_text(), flags=re.S)
        names += re.findall(r"\b(wst_[a-z0-9_]+)\s*\(", text)
    return sorted(set(names))


def test_headers_declare_the_dropin_entry_points():
    names = declared_symbols()
    for must in ["wst_rope_cache", "wst_attn_decode", "wst_attn_partial_floats",
                 "wst_rope_cache_chunk", "wst_attn_chunk", "wst_advance_pos", "wst_last_error"]:
        assert must in names


def test_library_exports_every_declared_symbol():
    out = subprocess.run(["nm", "-D", "--defined-only", str(_ffi.LIB_PATH)], check=True,
                         capture_output=True, text=True).stdout
    exported = set(re.findall(r"\sT\s+(wst_[a-z0-9_]+)", out))
    declared = set(declared_symbols())
    assert declared <= exported, f"declared but not exported: {sorted(declared - exported)}"
    assert exported <= declared, f"exported but not declared: {sorted(exported - declared)}"
    assert declared == set(_ffi.SIGNATURES), "ctypes table out of step with the headers"


def test_headers_compile_as_plain_c(tmp_path):
    src = tmp_path / "t.c"
    src.write_text('#include "whetstone_b200.h"\nint main(void){return (int)WST_OK;}\n')
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-I", str(ROOT / "include"), "-c",
                    str(src), "-o", str(tmp_path / "t.o")], check=True)


def test_last_error_is_never_null():
    assert isinstance(_ffi.last_error(), str)


def test_version():
    assert re.fullmatch(r"\d+\.\d+\.\d+", _ffi.version())


NULL = ctypes.c_void_p(0)
ONE = ctypes.c_void_p(0x1000)  # never dereferenced: the checks fail first


def test_null_pointers_are_invalid_arg():
    st = lib.wst_attn_decode(NULL, ONE, ONE, ONE, ONE, 14, 2, 64, ONE, 32, 0.125)
    assert st == 2 and "null pointer" in _ffi.last_error()
    st = lib.wst_rope_cache(ONE, ONE, ONE, ONE, ONE, 14, 2, 64, NULL, 32, NULL, NULL, 0.0)
    assert st == 2 and "wst_rope_cache" in _ffi.last_error()
    st = lib.wst_attn_chunk(ONE, ONE, NULL, ONE, 14, 2, 64, 0, 4, 32, 0.125)
    assert st == 2
    st = lib.wst_advance_pos(NULL, 8)
    assert st == 2


@pytest.mark.parametrize("args,frag", [
    ((14, 3, 64, 32), "multiple of key/value heads"),
    ((14, 2, 48, 32), "multiple of the warp size"),
    ((14, 2, 288, 32), "too large"),
    ((14, 2, 64, 0), "empty cache"),
    ((0, 2, 64, 32), "non-positive"),
])
def test_decode_shape_errors(args, frag):
    n_q, n_kv, hd, max_seq = args
    st = lib.wst_attn_decode(ONE, ONE, ONE, ONE, ONE, n_q, n_kv, hd, ONE, max_seq, 0.125)
    assert st == 2 and frag in _ffi.last_error()


def test_chunk_range_errors():
    st = lib.wst_rope_cache_chunk(ONE, ONE, ONE, ONE, ONE, 14, 2, 64, 30, 4, 32, NULL, NULL, 0.0)
    assert st == 2 and "runs past" in _ffi.last_error()
    st = lib.wst_rope_cache_chunk(ONE, ONE, ONE, ONE, ONE, 14, 2, 64, -1, 4, 32, NULL, NULL, 0.0)
    assert st == 2
    st = lib.wst_attn_chunk(ONE, ONE, ONE, ONE, 14, 2, 64, 29, 4, 32, 0.125)
    assert st == 2 and "runs past" in _ffi.last_error()
    st = lib.wst_rope_cache_chunk(ONE, ONE, ONE, ONE, ONE, 14, 2, 63, 0, 4, 32, NULL, NULL, 0.0)
    assert st == 2 and "even" in _ffi.last_error()


def test_paged_argument_errors():
    st = lib.wst_rope_cache_paged(ONE, ONE, ONE, ONE, ONE, ONE, ONE, ONE, 2, 10, 8, 32, 64, 28,
                                  4, 128, 4096, NULL, NULL, 0.0)
    assert st == 2 and "page_size" in _ffi.last_error()
    st = lib.wst_attn_verify_paged(ONE, ONE, ONE, ONE, ONE, ONE, ONE, ONE, 2, 10, 5, 8, 16, 64,
                                   28, 4, 128, 4096, 0.1)
    assert st == 2 and "page table shorter" in _ffi.last_error()


def test_typed_errors():
    with pytest.raises(_ffi.InvalidArg):
        _ffi.check(2)
    with pytest.raises(_ffi.CudaError):
        _ffi.check(1)
    _ffi.check(0)


def test_partial_floats_is_an_upper_bound_for_any_kv_head_count():
    # n_q * max slices * (head_dim + 4): numerators, max, denominator, 2 floats of padding
    assert lib.wst_attn_partial_floats(28, 128, 32768) == 28 * 64 * 132
    assert lib.wst_attn_partial_floats(14, 64, 1024) == 14 * 16 * 68
    assert lib.wst_attn_partial_floats(14, 64, 8) == 14 * 1 * 68
    assert lib.wst_attn_partial_floats(0, 64, 8) == 0


def test_verify_scratch_floats_positive():
    n = lib.wst_attn_verify_scratch_floats(16, 5, 28, 4, 128, 16389)
    assert n >= 16 * 4 * 35 * 9 * 130


@pytest.mark.parametrize("hd,theta,max_seq", [(64, 1e6, 96), (128, 1e4, 40)])
def test_rope_table_host_matches_oracle(hd, theta, max_seq):
    half = hd // 2
    cos = np.empty((max_seq, half), np.float32)
    sin = np.empty((max_seq, half), np.float32)
    st = lib.wst_rope_table_host(cos.ctypes.data_as(ctypes.c_void_p),
                                 sin.ctypes.data_as(ctypes.c_void_p), max_seq, hd, theta, 0,
                                 1.0, 1.0, 4.0, 8192)
    assert st == 0
    oc, os_ = orc.rope_table(max_seq, hd, theta)
    np.testing.assert_allclose(cos, oc, rtol=0, atol=2e-7)
    np.testing.assert_allclose(sin, os_, rtol=0, atol=2e-7)


def test_rope_table_host_llama3_matches_oracle():
    sc = dict(factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0, original_max_position=8192)
    cos = np.empty((64, 64), np.float32)
    sin = np.empty((64, 64), np.float32)
    st = lib.wst_rope_table_host(cos.ctypes.data_as(ctypes.c_void_p),
                                 sin.ctypes.data_as(ctypes.c_void_p), 64, 128, 5e5, 1, 8.0, 1.0,
                                 4.0, 8192)
    assert st == 0
    oc, os_ = orc.rope_table(64, 128, 5e5, llama3=sc)
    np.testing.assert_allclose(cos, oc, rtol=0, atol=2e-7)
    np.testing.assert_allclose(sin, os_, rtol=0, atol=2e-7)


def test_rope_table_host_rejects_odd_head_dim():
    buf = np.empty(8, np.float32)
    p = buf.ctypes.data_as(ctypes.c_void_p)
    assert lib.wst_rope_table_host(p, p, 2, 7, 1e6, 0, 1.0, 1.0, 4.0, 8192) == 5
    assert "must be even" in _ffi.last_error()
