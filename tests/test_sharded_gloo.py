"""Host logic of the multi-GPU path, on CPU: partitioning, and the all-gather +
merge of per-shard softmax triples over a world_size-2 gloo group."""

import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from oracle import attention_oracle as orc  # noqa: E402
from whetstone_b200 import sharded, workloads  # noqa: E402


def test_partition_units_covers_everything_once_and_balances():
    lengths = workloads.c5_lengths()
    weights = np.repeat(lengths + 5, 4)          # (sequence, KV head) units of config c5
    for world in (1, 2, 4, 8):
        owned = sharded.partition_units(weights, world)
        flat = sorted(i for part in owned for i in part)
        assert flat == list(range(len(weights)))
        loads = [float(weights[p].sum()) for p in owned]
        assert max(loads) <= 1.15 * (sum(loads) / world)


def test_partition_units_is_deterministic_and_handles_more_ranks_than_units():
    a = sharded.partition_units([3, 3, 3], 8)
    assert a == sharded.partition_units([3, 3, 3], 8)
    assert sum(len(x) for x in a) == 3 and all(len(x) <= 1 for x in a)


@pytest.mark.parametrize("rows,world", [(32768, 8), (32769, 4), (5, 8), (0, 2)])
def test_sequence_shard_tiles_the_sequence(rows, world):
    at = 0
    for r in range(world):
        lo, hi = sharded.sequence_shard(rows, world, r)
        assert lo == at and hi >= lo
        at = hi
    assert at == rows


def test_kv_head_units():
    assert sharded.kv_head_units(2, 3) == [(0, 0), (0, 1), (0, 2), (1, 0), (1, 1), (1, 2)]


def oracle_partial(q, k, v, scale):
    """(m, l, acc) of one shard in the wire format of wst_attn_decode_partial:
    natural-log running max, denominator, unnormalised numerators."""
    n_q, hd = q.shape
    n_kv = k.shape[0]
    gqa = n_q // n_kv
    out = np.zeros((n_q, hd + 2), dtype=np.float32)
    for h in range(n_q):
        if k.shape[1] == 0:
            out[h, 0] = -np.inf
            continue
        s = (k[h // gqa].astype(np.float64) @ q[h].astype(np.float64)) * scale
        m = s.max()
        e = np.exp(s - m)
        out[h, 0], out[h, 1] = m, e.sum()
        out[h, 2:] = e @ v[h // gqa].astype(np.float64)
    return out


def oracle_merge(parts):
    """cuda/attention.cu:170-193 across shards."""
    m = parts[:, :, 0]
    big = m.max(axis=0)
    f = np.where(np.isfinite(m), np.exp(m - big[None]), 0.0)
    num = (parts[:, :, 2:] * f[:, :, None]).sum(axis=0)
    den = (parts[:, :, 1] * f).sum(axis=0)
    return num / den[:, None]


def _worker(rank, world, port, seq, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        s = workloads.QWEN25_7B
        rng = np.random.default_rng(1234)           # every rank draws the same tensors
        q = workloads.f16_values(rng, (s.n_q, s.head_dim))
        k = workloads.f16_values(rng, (s.n_kv, seq, s.head_dim), np.float16)
        v = workloads.f16_values(rng, (s.n_kv, seq, s.head_dim), np.float16)
        lo, hi = sharded.sequence_shard(seq, world, rank)
        mine = torch.from_numpy(oracle_partial(q, k[:, lo:hi], v[:, lo:hi], s.scale))
        gathered = sharded.gather_partials(mine)
        assert gathered.shape == (world, s.n_q, s.head_dim + 2)
        # slot r holds rank r's triples
        assert torch.equal(gathered[rank], mine)
        got = oracle_merge(gathered.numpy().astype(np.float64))
        want = orc.decode_attention(q, k, v, seq, s.scale)
        np.save(Path(result_dir) / f"err_{rank}.npy", np.abs(got - want).max())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("seq", [257, 3])
def test_gather_and_merge_over_gloo(tmp_path, seq):
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    world = 2
    mp.spawn(_worker, args=(world, port, seq, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert float(np.load(tmp_path / f"err_{r}.npy")) < 1e-5
