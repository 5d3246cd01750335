"""One process per GPU: how the attention path is partitioned over the GPUs of
one box, and the one real exchange step it has.

The engine itself is single-GPU (crates/whetstone-kernels/src/lib.rs:135-137 picks
device 0 and nothing else ever selects another), so everything here is an
addition.  Two shapes of work:

* independent units -- (sequence, KV head) pairs of a batched prefill or verify
  step.  They are dealt out to ranks (`partition_units`, by bytes for ragged
  lengths) and need NO collective on the data path: each rank appends and
  attends for its own KV heads only.
* one long sequence -- decode at long context.  The KV *sequence* is split: rank
  g holds cache rows [g*S/G, (g+1)*S/G) of every KV head, runs the
  partial-softmax kernel on its shard (wst_attn_decode_partial), the per-head
  (m, l, acc) triples (14.5 KB per rank for 28 heads of 128) are all-gathered
  over NCCL/NVLink into local memory and merged locally
  (wst_attn_merge_partials).  Remote data is only ever read after the
  collective has landed it in this GPU's own memory.

Collectives go through torch.distributed, so the same code runs over gloo on
CPU tensors (the host-logic tests) and over NCCL on device tensors.
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch
import torch.distributed as dist


# ----------------------------------------------------------- partitioning

def partition_units(weights, world: int) -> list[list[int]]:
    """Greedy longest-first assignment of work units to `world` ranks.

    `weights[i]` is the cost of unit i (bytes of KV it streams, or 1 for equal
    units).  Returns, per rank, the sorted list of unit indices it owns.  Every
    unit is assigned exactly once; ties break toward the lower rank so that the
    result is the same on every rank without communication.
    """
    if world <= 0:
        raise ValueError("world must be positive")
    w = np.asarray(weights, dtype=np.float64)
    order = sorted(range(len(w)), key=lambda i: (-w[i], i))
    load = [0.0] * world
    owned: list[list[int]] = [[] for _ in range(world)]
    for i in order:
        r = min(range(world), key=lambda k: (load[k], k))
        owned[r].append(i)
        load[r] += float(w[i])
    return [sorted(x) for x in owned]


def sequence_shard(total_rows: int, world: int, rank: int) -> tuple[int, int]:
    """Rows [lo, hi) of a KV sequence that `rank` holds: equal contiguous slices,
    the remainder spread over the first ranks."""
    base, extra = divmod(total_rows, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def kv_head_units(n_seq: int, n_kv: int):
    """(sequence, KV head) pairs in unit order: unit = seq * n_kv + kv_head."""
    return [(u // n_kv, u % n_kv) for u in range(n_seq * n_kv)]


# ------------------------------------------------------- the exchange step

def gather_partials(mine: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather of this rank's (m, l, acc) triples.

    `mine` is [n_q][head_dim + 2] fp32; returns [world][n_q][head_dim + 2] in rank
    order, resident in this rank's own memory.
    """
    world = dist.get_world_size(group)
    out = torch.empty((world,) + tuple(mine.shape), dtype=mine.dtype, device=mine.device)
    # the collective wants the concatenated (world * n_q, ...) view of the output
    dist.all_gather_into_tensor(out.view((-1,) + tuple(mine.shape[1:])), mine.contiguous(),
                                group=group)
    return out


class PeerExchange:
    """Mailboxes and flags of wst_attn_exchange_merge for the ranks of one box.

    Every rank allocates a mailbox of its own (wst_malloc: 8-byte packets
    [2][world][n_q][head_dim+2]), zeroes it, publishes its CUDA IPC handle to the
    other ranks through the process group (once), imports theirs with its own device
    current, and keeps a small device array with the addresses in rank order -- what
    the kernel takes.  One instance serves any number of layers: calls are told apart
    by the per-head call counters in `state`, and all ranks make the same sequence of
    calls.
    """

    def __init__(self, n_q: int, head_dim: int, group=None):
        import ctypes
        from ._ffi import check, lib

        self._lib, self._check = lib, check
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.n_q, self.head_dim = n_q, head_dim
        dev = torch.device("cuda", torch.cuda.current_device())
        total = 2 * self.world * n_q * (head_dim + 2) * 8
        base = ctypes.c_void_p()
        check(lib.wst_malloc(ctypes.byref(base), total))
        self._base = base.value
        check(lib.wst_memset(ctypes.c_void_p(self._base), 0, total))
        check(lib.wst_device_synchronize())
        handle = ctypes.create_string_buffer(64)
        check(lib.wst_b200_ipc_export(ctypes.c_void_p(self._base), handle))
        handles = [None] * self.world
        dist.all_gather_object(handles, (dev.index, handle.raw), group=group)
        self._imported = []
        bases = []
        for g, (peer_dev, raw) in enumerate(handles):
            if g == self.rank:
                bases.append(self._base)
                continue
            check(lib.wst_b200_enable_peer_access(peer_dev))
            p = ctypes.c_void_p()
            check(lib.wst_b200_ipc_import(ctypes.create_string_buffer(raw, 64), ctypes.byref(p)))
            self._imported.append(p.value)
            bases.append(p.value)
        self.mailboxes_dev = torch.tensor(bases, dtype=torch.int64, device=dev)
        self.state = torch.zeros(n_q, dtype=torch.int32, device=dev)
        torch.cuda.synchronize()
        dist.barrier(group=group)  # nobody launches before everybody has mapped everything

    def merge(self, mine: torch.Tensor, out: torch.Tensor) -> None:
        from . import decode
        decode.attn_exchange_merge(mine, out, self.mailboxes_dev, self.state, self.rank,
                                   self.world, self.n_q, self.head_dim)

    def decode(self, q: torch.Tensor, cache, out: torch.Tensor, length: torch.Tensor) -> None:
        """Attention over this rank's shard and the exchange in one kernel
        (wst_attn_decode_sharded)."""
        from . import decode
        decode.attn_decode_sharded(q, cache, out, self.n_q, length, self.mailboxes_dev,
                                   self.state, self.rank, self.world)

    def close(self, group=None) -> None:
        """Unmaps the other ranks' buffers and frees this rank's (collective: every
        rank calls it, after its last merge has finished)."""
        import ctypes
        torch.cuda.synchronize()
        dist.barrier(group=group)
        for p in self._imported:
            self._check(self._lib.wst_b200_ipc_close(ctypes.c_void_p(p)))
        self._imported = []
        dist.barrier(group=group)
        if self._base:
            self._check(self._lib.wst_free(ctypes.c_void_p(self._base)))
            self._base = 0


@dataclass
class ShardedDecodeLayer:
    """One layer of long-context decode on this rank's slice of the KV sequence."""

    cache: "object"          # whetstone_b200.decode.KvCache holding rows [lo, hi)
    length: torch.Tensor     # device int32[1]: valid rows of the slice
    n_q: int
    exchange: "PeerExchange | None" = None   # None: NCCL all-gather + local merge
    fused: bool = False                      # with an exchange: one kernel per layer

    def __post_init__(self):
        hd = self.cache.head_dim
        world = dist.get_world_size()
        dev = self.cache.k.device
        self.mine = torch.zeros((self.n_q, hd + 2), dtype=torch.float32, device=dev)
        self.gathered = torch.zeros((world, self.n_q, hd + 2), dtype=torch.float32, device=dev)

    def attend(self, q: torch.Tensor, out: torch.Tensor) -> None:
        """q [>= n_q*head_dim] fp32 (replicated on every rank) -> out [n_q*head_dim] fp16
        (identical on every rank)."""
        from . import decode  # the CUDA path; importing it here keeps this module CPU-importable
        if self.exchange is not None and self.fused:
            self.exchange.decode(q, self.cache, out, self.length)
            return
        decode.attn_decode_partial(q, self.cache, self.mine, self.n_q, self.length)
        if self.exchange is not None:
            self.exchange.merge(self.mine, out)
            return
        dist.all_gather_into_tensor(self.gathered.view(-1, self.mine.shape[1]), self.mine)
        decode.attn_merge_partials(self.gathered, out, self.n_q, self.cache.head_dim)


__all__ = ["partition_units", "sequence_shard", "kv_head_units", "gather_partials",
           "PeerExchange", "ShardedDecodeLayer"]
