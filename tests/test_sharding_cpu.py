"""CPU: the multi-GPU partitioning logic, including a world_size-2 gloo run in which each rank
computes its shard (with the CPU oracle standing in for the kernels) and the gathered result
equals the unsharded one."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flash_attn2_b200 import sharding
from tests._cases import make_qkv


def test_shard_range_covers_everything():
    for n, w in [(256, 8), (16, 3), (5, 8), (32, 4)]:
        seen = [i for r in range(w) for i in sharding.shard_range(n, w, r)]
        assert seen == list(range(n))
        sizes = [len(sharding.shard_range(n, w, r)) for r in range(w)]
        assert max(sizes) - min(sizes) <= 1


def test_shard_heads_keeps_gqa_groups():
    for world in (1, 2, 4, 8):
        qs, ks = zip(*[sharding.shard_heads(32, 8, world, r) for r in range(world)])
        assert sum(s.stop - s.start for s in qs) == 32 and sum(s.stop - s.start for s in ks) == 8
        for q, k in zip(qs, ks):
            assert q.start == 4 * k.start and q.stop == 4 * k.stop
    with pytest.raises(ValueError):
        sharding.shard_heads(30, 8, 2, 0)


def test_sequences_are_balanced_by_quadratic_cost():
    g = torch.Generator().manual_seed(3)
    lengths = torch.randint(128, 4097, (32,), generator=g).tolist()
    for world in (2, 4, 8):
        parts = sharding.shard_sequences_by_cost(lengths, world)
        assert sorted(i for p in parts for i in p) == list(range(32))
        loads = [sum(lengths[i] ** 2 for i in p) for p in parts]
        assert max(loads) <= 1.25 * (sum(loads) / world)


def _worker(rank, world, port, q, k, v, ref):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle.attention_oracle import attention_forward

    try:
        r = sharding.shard_range(q.shape[0], world, rank)
        out, lse = attention_forward(q[r.start:r.stop], k[r.start:r.stop], v[r.start:r.stop], causal=True)
        full = sharding.gather_shards(out, 0)
        torch.testing.assert_close(full, ref)
        hq, hk = sharding.shard_heads(q.shape[2], k.shape[2], world, rank)
        out_h, _ = attention_forward(q[:, :, hq], k[:, :, hk], v[:, :, hk], causal=True)
        torch.testing.assert_close(sharding.gather_shards(out_h, 2), ref)
    finally:
        dist.destroy_process_group()


def test_world_size_2_gloo_shards_reassemble():
    from oracle.attention_oracle import attention_forward

    q, k, v = make_qkv(7, 4, 4, 2, 48, 48, 16, torch.float32)
    ref, _ = attention_forward(q, k, v, causal=True)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, q, k, v, ref), nprocs=2, join=True)
