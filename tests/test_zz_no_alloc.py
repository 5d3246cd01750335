"""wst_attn_decode_noscratch: the decode entry point for hosts that cannot
allocate the split scratch (their device memory is already committed to a pool,
or they are in a phase where cudaMalloc is not allowed).  It keeps the slices'
partial results in an array built into the library, so every call shares that
array and finds the previous call's leftovers in it.

Checked here through the C ABI: two different calls in a row must each give what
wst_attn_decode gives with a caller-provided buffer -- and what the numpy oracle
says -- the second call must leave the amount of free device memory where it was,
and a shape whose scratch would not fit in the built-in array must be refused.
This file is collected last on purpose; it passes on its own in a fresh process as
well.
"""

import ctypes

import numpy as np
import pytest
import torch

from oracle import attention_oracle as orc
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
    k = workloads.f16_values(rng, (n_kv, seq, hd), np.float16)
    v = workloads.f16_values(rng, (n_kv, seq, hd), np.float16)
    cache.k[:, :seq] = dev(k)
    cache.v[:, :seq] = dev(v)
    q_host = workloads.f16_values(rng, (n_q, hd))
    q = dev(q_host)
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
        host(built_in).astype(np.float64).reshape(n_q, hd), \
        orc.decode_attention(q_host, k, v, seq)


def test_two_calls_in_a_row_match_the_entry_point_with_a_caller_buffer():
    # first call: many slices; second call: another shape and length, so that it
    # would trip over anything the first one left behind in the shared array
    for n_q, n_kv, hd, seq, max_seq, seed in ((28, 4, 128, 6000, 6100, 1), (14, 2, 64, 777, 1024, 2)):
        want, got, oracle = _both_ways(n_q, n_kv, hd, seq, max_seq, seed)
        assert_close_per_head(got, want, f"built-in scratch, {n_q}/{n_kv}/{hd} seq {seq}")
        assert_close_per_head(got, oracle, f"built-in scratch vs oracle, {n_q}/{n_kv}/{hd} seq {seq}")
    assert decode.device_error() == 0


def test_a_warmed_up_call_takes_no_device_memory():
    """Once the library's device image is in place (any earlier call), a call of this
    entry point must leave the free device memory exactly where it found it."""
    n_q, n_kv, hd, seq, max_seq = 28, 4, 128, 3000, 3072
    rng = np.random.default_rng(5)
    cache = decode.KvCache(n_kv, n_q, hd, max_seq)
    cache.k[:, :seq] = dev(workloads.f16_values(rng, (n_kv, seq, hd), np.float16))
    cache.v[:, :seq] = dev(workloads.f16_values(rng, (n_kv, seq, hd), np.float16))
    q = dev(workloads.f16_values(rng, (n_q, hd)))
    pos = torch.tensor([seq - 1], dtype=torch.int32, device="cuda")
    out = torch.zeros(n_q * hd, dtype=torch.float16, device="cuda")
    decode.use_torch_stream()

    def call():
        assert lib.wst_attn_decode_noscratch(_ptr(q), _ptr(cache.k), _ptr(cache.v), _ptr(out), n_q,
                                             n_kv, hd, _ptr(pos), max_seq,
                                             1.0 / np.sqrt(hd)) == 0, last_error()
        torch.cuda.synchronize()

    call()                                   # warm-up: module load, address look-up
    free_before, _ = torch.cuda.mem_get_info()
    call()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before


def test_a_shape_beyond_the_built_in_array_is_refused():
    one = ctypes.c_void_p(0x1000)  # never dereferenced: the size check comes first
    st = lib.wst_attn_decode_noscratch(one, one, one, one, 512, 8, 128, one, 32768, 0.1)
    assert st == 2
    assert "built-in array holds" in last_error()
