"""wst_attn_decode_noscratch: the decode entry point for hosts that cannot
allocate the split scratch (their device memory is already committed to a pool,
or they are in a phase where cudaMalloc is not allowed).  It keeps the slices'
partial results in an array built into the library, so every call shares that
array and finds the previous call's leftovers in it.

Checked here through the C ABI: two different calls in a row must each give what
wst_attn_decode gives with a caller-provided buffer, and a shape whose scratch
would not fit in the built-in array must be refused.  This file is collected
last on purpose; it passes on its own in a fresh process as well.
"""

import ctypes

import numpy as np
import pytest
import torch

from tests.helpers import NAN16, assert_close_per_head, dev, fill_bits, host
from whetstone_b200 import decode, workloads
from whetstone_b200._ffi import last_error, lib

pytestmark = pytest.mark.gpu


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def _both_ways(n_q, n_kv, hd, seq, max_seq, seed):
    rng = np.random.default_rng(seed)
    cache = decode.KvCache(n_kv, n_q, hd, max_seq)
    fill_bits(cache.k, NAN16)
    fill_bits(cache.v, NAN16)
    cache.k[:, :seq] = dev(workloads.f16_values(rng, (n_kv, seq, hd), np.float16))
    cache.v[:, :seq] = dev(workloads.f16_values(rng, (n_kv, seq, hd), np.float16))
    q = dev(workloads.f16_values(rng, (n_q, hd)))
    pos = torch.tensor([seq - 1], dtype=torch.int32, device="cuda")
    scale = 1.0 / np.sqrt(hd)
    decode.use_torch_stream()
    with_buffer = torch.zeros(n_q * hd, dtype=torch.float16, device="cuda")
    built_in = torch.zeros(n_q * hd, dtype=torch.float16, device="cuda")
    assert lib.wst_attn_decode(_ptr(q), _ptr(cache.k), _ptr(cache.v), _ptr(cache.partials),
                               _ptr(with_buffer), n_q, n_kv, hd, _ptr(pos), max_seq,
                               scale) == 0, last_error()
    assert lib.wst_attn_decode_noscratch(_ptr(q), _ptr(cache.k), _ptr(cache.v), _ptr(built_in),
                                         n_q, n_kv, hd, _ptr(pos), max_seq,
                                         scale) == 0, last_error()
    torch.cuda.synchronize()
    return host(with_buffer).astype(np.float64).reshape(n_q, hd), \
        host(built_in).astype(np.float64).reshape(n_q, hd)


def test_two_calls_in_a_row_match_the_entry_point_with_a_caller_buffer():
    # first call: many slices; second call: another shape and length, so that it
    # would trip over anything the first one left behind in the shared array
    for n_q, n_kv, hd, seq, max_seq, seed in ((28, 4, 128, 6000, 6100, 1), (14, 2, 64, 777, 1024, 2)):
        want, got = _both_ways(n_q, n_kv, hd, seq, max_seq, seed)
        assert_close_per_head(got, want, f"built-in scratch, {n_q}/{n_kv}/{hd} seq {seq}")
    assert decode.device_error() == 0


def test_a_shape_beyond_the_built_in_array_is_refused():
    one = ctypes.c_void_p(0x1000)  # never dereferenced: the size check comes first
    st = lib.wst_attn_decode_noscratch(one, one, one, one, 512, 8, 128, one, 32768, 0.1)
    assert st == 2
    assert "built-in array holds" in last_error()
