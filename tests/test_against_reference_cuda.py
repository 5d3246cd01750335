"""Second checker: the reference's own CUDA kernels (compiled unmodified for
sm_100a into oracle/_ref/ by oracle/Makefile) run on the same device buffers as
this library's kernels.  Skipped where that file was not built."""

import ctypes
from pathlib import Path

import numpy as np
import pytest
import torch

from tests.helpers import assert_close_per_head, bits16, dev, f16_ulp_distance, host
from whetstone_b200 import chunk, decode, workloads
from whetstone_b200._ffi import SIGNATURES

pytestmark = pytest.mark.gpu

REF_PATH = Path(__file__).resolve().parent.parent / "oracle" / "_ref" / "libwhetstone_ref.so"


@pytest.fixture(scope="module")
def ref():
    if not REF_PATH.exists():
        pytest.skip("oracle/_ref/libwhetstone_ref.so not built")
    lib = ctypes.CDLL(str(REF_PATH))
    for name in ("wst_rope_cache", "wst_attn_decode", "wst_attn_partial_floats",
                 "wst_rope_cache_chunk", "wst_attn_chunk", "wst_last_error",
                 "wst_device_synchronize"):
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = SIGNATURES[name]
    return lib


def P(t):
    return ctypes.c_void_p(t.data_ptr() if t is not None else 0)


@pytest.mark.parametrize("n_q,n_kv,hd,seq", [(14, 2, 64, 513), (28, 4, 128, 3001)])
def test_decode_agrees_with_reference_kernels(ref, n_q, n_kv, hd, seq):
    rng = np.random.default_rng(seq)
    max_seq = seq + 10
    table = decode.RopeTable(max_seq, hd, 1e6)
    mine = decode.KvCache(n_kv, n_q, hd, max_seq)
    k = workloads.f16_values(rng, (n_kv, seq - 1, hd), np.float16)
    v = workloads.f16_values(rng, (n_kv, seq - 1, hd), np.float16)
    mine.k[:, : seq - 1] = dev(k)
    mine.v[:, : seq - 1] = dev(v)
    theirs_k, theirs_v = mine.k.clone(), mine.v.clone()
    theirs_scratch = torch.zeros(max(ref.wst_attn_partial_floats(n_q, hd, max_seq), 1),
                                 dtype=torch.float32, device="cuda")
    qkv = workloads.f16_values(rng, ((n_q + 2 * n_kv) * hd,))
    cur = decode.DeviceCursor(seq - 1)

    q_mine = dev(qkv)
    out_mine = torch.zeros(n_q * hd, dtype=torch.float16, device="cuda")
    decode.rope_cache(q_mine, mine, table, n_q, cur)
    decode.attn_decode(q_mine, mine, out_mine, n_q, cur)

    q_ref = dev(qkv)
    out_ref = torch.zeros(n_q * hd, dtype=torch.float16, device="cuda")
    torch.cuda.synchronize()
    assert ref.wst_rope_cache(P(q_ref), P(theirs_k), P(theirs_v), P(table.cos), P(table.sin),
                              n_q, n_kv, hd, P(cur.buf), max_seq, None, None, 0.0) == 0
    assert ref.wst_attn_decode(P(q_ref), P(theirs_k), P(theirs_v), P(theirs_scratch), P(out_ref),
                               n_q, n_kv, hd, P(cur.buf), max_seq, 1.0 / np.sqrt(hd)) == 0
    assert ref.wst_device_synchronize() == 0

    np.testing.assert_allclose(host(q_mine)[: n_q * hd], host(q_ref)[: n_q * hd], rtol=0, atol=2e-6)
    assert np.array_equal(bits16(mine.v), bits16(theirs_v))
    assert f16_ulp_distance(bits16(mine.k), bits16(theirs_k)).max() <= 1
    assert_close_per_head(host(out_mine).astype(np.float64).reshape(n_q, hd),
                          host(out_ref).astype(np.float64).reshape(n_q, hd), "decode vs reference")


@pytest.mark.parametrize("norm", [False, True])
def test_chunk_agrees_with_reference_kernels(ref, norm):
    n_q, n_kv, hd, pos0, n = 32, 8, 128, 300, 40
    rng = np.random.default_rng(8)
    max_seq = 400
    width = (n_q + 2 * n_kv) * hd
    table = decode.RopeTable(max_seq, hd, 1e6)
    mine = decode.KvCache(n_kv, n_q, hd, max_seq)
    pre = workloads.f16_values(rng, (pos0, width))
    gains = None
    gq = gk = None
    if norm:
        a, b = workloads.qk_gains(rng, hd)
        gq, gk = dev(a), dev(b)
        gains = decode.QkNorm(gq, gk, 1e-6)
    chunk.rope_cache(dev(pre), mine, table, n_q, 0, pos0, gains)
    theirs_k, theirs_v = mine.k.clone(), mine.v.clone()
    qkv = workloads.f16_values(rng, (n, width))

    q_mine = dev(qkv)
    out_mine = torch.zeros(n * n_q * hd, dtype=torch.float16, device="cuda")
    chunk.rope_cache(q_mine, mine, table, n_q, pos0, n, gains)
    chunk.attn(q_mine, mine, out_mine, n_q, pos0, n)

    q_ref = dev(qkv)
    out_ref = torch.zeros(n * n_q * hd, dtype=torch.float16, device="cuda")
    torch.cuda.synchronize()
    assert ref.wst_rope_cache_chunk(P(q_ref), P(theirs_k), P(theirs_v), P(table.cos),
                                    P(table.sin), n_q, n_kv, hd, pos0, n, max_seq, P(gq), P(gk),
                                    1e-6 if norm else 0.0) == 0
    assert ref.wst_attn_chunk(P(q_ref), P(theirs_k), P(theirs_v), P(out_ref), n_q, n_kv, hd,
                              pos0, n, max_seq, 1.0 / np.sqrt(hd)) == 0
    assert ref.wst_device_synchronize() == 0
    assert np.array_equal(bits16(mine.v), bits16(theirs_v))
    assert f16_ulp_distance(bits16(mine.k), bits16(theirs_k)).max() <= 1
    assert_close_per_head(host(out_mine).astype(np.float64).reshape(n, n_q, hd),
                          host(out_ref).astype(np.float64).reshape(n, n_q, hd),
                          "chunk vs reference")
