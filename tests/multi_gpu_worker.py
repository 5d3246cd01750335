"""Worker of tests/test_multi_gpu.py: one process per GPU (torchrun).  Long-context
decode with the KV sequence sharded over the ranks, merged (a) by an NCCL all-gather
and the local merge kernel, (b) through peer memory inside wst_attn_exchange_merge and
(c) through peer memory inside the slice-merge kernel of wst_attn_decode_sharded; all
are compared with the numpy oracle on every rank."""

import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

from oracle import attention_oracle as orc  # noqa: E402  (checker only)
from whetstone_b200 import decode, sharded, workloads  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    n_q, n_kv, hd, ctx, layers = 28, 4, 128, 4096 + 37, 5
    scale = 1.0 / np.sqrt(hd)
    rng = np.random.default_rng(11)                      # same values on every rank
    ks = [workloads.f16_values(rng, (n_kv, ctx, hd), np.float16) for _ in range(layers)]
    vs = [workloads.f16_values(rng, (n_kv, ctx, hd), np.float16) for _ in range(layers)]
    qs = [workloads.f16_values(rng, (n_q * hd,)) for _ in range(layers)]
    lo, hi = sharded.sequence_shard(ctx, world, rank)
    length = torch.tensor([hi - lo], dtype=torch.int32, device="cuda")
    xch = sharded.PeerExchange(n_q, hd)
    lay_nccl, lay_p2p, lay_one, qd = [], [], [], []
    for l in range(layers):
        cache = decode.KvCache(n_kv, n_q, hd, max(hi - lo, 1))
        cache.k.copy_(torch.from_numpy(ks[l][:, lo:hi].copy()).cuda())
        cache.v.copy_(torch.from_numpy(vs[l][:, lo:hi].copy()).cuda())
        lay_nccl.append(sharded.ShardedDecodeLayer(cache, length, n_q))
        lay_p2p.append(sharded.ShardedDecodeLayer(cache, length, n_q, exchange=xch))
        lay_one.append(sharded.ShardedDecodeLayer(cache, length, n_q, exchange=xch, fused=True))
        qd.append(torch.from_numpy(qs[l]).cuda())
    want = []
    for l in range(layers):
        want.append(orc.decode_attention(qs[l].astype(np.float64).reshape(n_q, hd), ks[l], vs[l],
                                         ctx, scale))

    def check(outs, what):
        torch.cuda.synchronize()
        assert decode.device_error() == 0, f"{what}: a kernel gave up a wait"
        for l in range(layers):
            got = outs[l].cpu().numpy().astype(np.float64).reshape(n_q, hd)
            err = np.abs(got - want[l]).max()
            assert err <= 2e-3, f"{what}, rank {rank}, layer {l}: max abs err {err}"

    outs = [torch.zeros(n_q * hd, dtype=torch.float16, device="cuda") for _ in range(layers)]
    for l in range(layers):
        lay_nccl[l].attend(qd[l], outs[l])
    check(outs, "nccl all-gather")

    # peer-memory exchange: eager, three rounds (call counter, both mailbox halves) ...
    for _ in range(3):
        for o in outs:
            o.zero_()
        for l in range(layers):
            lay_p2p[l].attend(qd[l], outs[l])
        check(outs, "peer exchange")
    # the exchange inside the slice-merge kernel, mixed with the two-kernel form on the
    # same mailboxes (every rank makes the same sequence of calls)
    for rnd in range(4):
        for o in outs:
            o.zero_()
        for l in range(layers):
            (lay_one if (rnd + l) % 3 else lay_p2p)[l].attend(qd[l], outs[l])
        check(outs, "exchange in the merge kernel")
    # ... and as a CUDA graph replayed several times
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        for l in range(layers):
            (lay_one if l % 2 else lay_p2p)[l].attend(qd[l], outs[l])
    for _ in range(4):
        for o in outs:
            o.zero_()
        graph.replay()
        check(outs, "peer exchange (graph)")
    xch.close()
    dist.barrier()
    if rank == 0:
        print("MULTI_GPU_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
