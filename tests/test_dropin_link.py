"""The integration recipe carried out: all of the engine's own kernel objects with the
entry points this repository replaces weakened, linked with this repository's drop-in archive
(`make -C whetstone_b200/csrc DROPIN=1`) into oracle/_ref/libwhetstone_dropin.so by
`make -C oracle dropin`.  One library must export every symbol the engine's Rust crate
binds (crates/whetstone-kernels/src/ffi.rs:134-473, listed in
tests/golden/ffi_symbols.txt) exactly once, the attention entry points must be this
repository's, and their error text must come back through the ENGINE's
wst_last_error (cuda/runtime.cu:5-7), which is what the Rust side's check() reads
(src/lib.rs:88-98).  The library exists only where the reference checkout was mounted
at build time; it travels to the GPU box prebuilt."""

import ctypes
import subprocess
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
LIB = ROOT / "oracle" / "_ref" / "libwhetstone_dropin.so"
ARCHIVE = ROOT / "whetstone_b200" / "libwhetstone_b200_dropin.a"
ENGINE_RUNTIME = ["wst_last_error", "wst_malloc", "wst_free", "wst_memset", "wst_memcpy_h2d",
                  "wst_memcpy_d2h", "wst_memcpy_d2d", "wst_graph_capture_begin",
                  "wst_graph_capture_end", "wst_graph_launch", "wst_graph_destroy",
                  "wst_stream_sync", "wst_event_create", "wst_event_record",
                  "wst_event_elapsed_ms", "wst_event_destroy", "wst_device_count",
                  "wst_device_set", "wst_device_synchronize", "wst_advance_pos"]

needs_lib = pytest.mark.skipif(not LIB.exists(), reason="drop-in library not built (no reference checkout)")


def defined(path):
    out = subprocess.run(["nm", "-g", "--defined-only", str(path)], check=True, capture_output=True,
                         text=True).stdout
    rows = [line.split() for line in out.splitlines() if len(line.split()) == 3]
    return [(kind, name) for _, kind, name in rows if name.startswith("wst_")]


def test_the_archive_leaves_the_engines_runtime_symbols_out():
    subprocess.run(["make", "-C", str(ROOT / "whetstone_b200" / "csrc"), "DROPIN=1"], check=True,
                   capture_output=True)
    names = {name for _, name in defined(ARCHIVE)}
    assert not names & set(ENGINE_RUNTIME), names & set(ENGINE_RUNTIME)
    for name in ("wst_rope_cache", "wst_attn_decode", "wst_attn_partial_floats",
                 "wst_rope_cache_chunk", "wst_attn_chunk", "wst_gemm_fp16", "wst_gemm_int4_hier",
                 "wst_chunk_max_tokens", "wst_attn_verify_paged", "wst_b200_set_stream"):
        assert name in names


@needs_lib
def test_one_library_every_symbol_once():
    syms = defined(LIB)
    names = [name for _, name in syms]
    assert len(names) == len(set(names)), "a wst_* symbol is defined twice"
    weak = [name for kind, name in syms if kind in "Ww"]
    assert not weak, f"weak definitions won the link: {weak}"
    wanted = (ROOT / "tests" / "golden" / "ffi_symbols.txt").read_text().split()
    assert len(wanted) == 66
    missing = sorted(set(wanted) - set(names))
    assert not missing, f"symbols of ffi.rs that the drop-in library lacks: {missing}"


@needs_lib
def test_attention_entry_points_are_ours_and_report_through_the_engines_buffer():
    lib = ctypes.CDLL(str(LIB))
    lib.wst_last_error.restype = ctypes.c_char_p
    # this repository sizes the split scratch without asking the device: 28 * 64 * (128 + 4)
    lib.wst_attn_partial_floats.argtypes = [ctypes.c_int32] * 3
    assert lib.wst_attn_partial_floats(28, 128, 32768) == 28 * 64 * 132
    # an entry point only this repository has, refused on its arguments alone: the text
    # must arrive in the buffer the ENGINE's wst_last_error returns
    P, I = ctypes.c_void_p, ctypes.c_int32
    lib.wst_attn_decode_noscratch.argtypes = [P, P, P, P, I, I, I, P, I, ctypes.c_float]
    one = P(0x1000)
    assert lib.wst_attn_decode_noscratch(one, one, one, one, 512, 8, 128, one, 32768, 0.1) == 2
    assert b"built-in array holds" in lib.wst_last_error()
    lib.wst_attn_chunk.argtypes = [P, P, P, P, I, I, I, I, I, I, ctypes.c_float]
    assert lib.wst_attn_chunk(one, one, one, one, 14, 2, 64, 30, 4, 32, 0.125) == 2
    assert lib.wst_last_error() == b"wst_attn_chunk: chunk runs past cache"


@needs_lib
@pytest.mark.gpu
def test_decode_and_chunk_through_the_linked_library_match_the_oracle():
    import torch

    from oracle import attention_oracle as orc
    from tests.helpers import assert_close_per_head, dev, host
    from whetstone_b200 import workloads
    from whetstone_b200._ffi import SIGNATURES

    lib = ctypes.CDLL(str(LIB))
    for name in ("wst_last_error", "wst_rope_cache", "wst_attn_decode", "wst_attn_partial_floats",
                 "wst_rope_cache_chunk", "wst_attn_chunk", "wst_device_synchronize", "wst_malloc",
                 "wst_free", "wst_memset"):
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = SIGNATURES[name]

    def ptr(t):
        return ctypes.c_void_p(t.data_ptr())

    n_q, n_kv, hd, theta, n, max_seq = 14, 2, 64, 1e6, 40, 64
    rng = np.random.default_rng(9)
    width = (n_q + 2 * n_kv) * hd
    rows = workloads.f16_values(rng, (n, width))
    cos, sin = orc.rope_table(max_seq, hd, theta)
    cos_d, sin_d = dev(cos.astype(np.float32)), dev(sin.astype(np.float32))
    k = torch.zeros(n_kv, max_seq, hd, dtype=torch.float16, device="cuda")
    v = torch.zeros_like(k)
    torch.cuda.synchronize()
    # the engine's wst_malloc provides the scratch, this repository's kernels use it
    floats = lib.wst_attn_partial_floats(n_q, hd, max_seq)
    scratch = ctypes.c_void_p()
    assert lib.wst_malloc(ctypes.byref(scratch), floats * 4) == 0, lib.wst_last_error()
    rd = dev(rows)
    null = ctypes.c_void_p(0)
    assert lib.wst_rope_cache_chunk(ptr(rd), ptr(k), ptr(v), ptr(cos_d), ptr(sin_d), n_q, n_kv, hd,
                                    0, n - 1, max_seq, null, null, 0.0) == 0, lib.wst_last_error()
    out_c = torch.zeros((n - 1) * n_q * hd, dtype=torch.float16, device="cuda")
    assert lib.wst_attn_chunk(ptr(rd), ptr(k), ptr(v), ptr(out_c), n_q, n_kv, hd, 0, n - 1, max_seq,
                              0.125) == 0, lib.wst_last_error()
    pos = torch.tensor([n - 1], dtype=torch.int32, device="cuda")
    last = rd[n - 1].contiguous()
    assert lib.wst_rope_cache(ptr(last), ptr(k), ptr(v), ptr(cos_d), ptr(sin_d), n_q, n_kv, hd,
                              ptr(pos), max_seq, null, null, 0.0) == 0, lib.wst_last_error()
    out_d = torch.zeros(n_q * hd, dtype=torch.float16, device="cuda")
    assert lib.wst_attn_decode(ptr(last), ptr(k), ptr(v), scratch, ptr(out_d), n_q, n_kv, hd,
                               ptr(pos), max_seq, 0.125) == 0, lib.wst_last_error()
    assert lib.wst_device_synchronize() == 0
    torch.cuda.synchronize()
    qr, kr, vv = orc.rope_append(rows, np.arange(n), n_q, n_kv, hd, theta)
    want = orc.attention_blocked(qr, kr, vv, 1 + np.arange(n))
    assert_close_per_head(host(out_c).astype(np.float64).reshape(n - 1, n_q, hd), want[: n - 1],
                          "chunk through the drop-in library")
    assert_close_per_head(host(out_d).astype(np.float64).reshape(n_q, hd), want[n - 1],
                          "decode through the drop-in library")
    assert lib.wst_free(scratch) == 0
