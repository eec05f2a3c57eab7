"""Host-side multi-rank logic on CPU: world_size-2 (and 3) gloo process groups shard attention units by head and
by batch, compute their shards independently and all-gather the output; the result must equal the single-process
one bit for bit. The per-rank compute here is the CPU oracle standing in for the kernels: the test is about the
partitioning and the collective, not the arithmetic."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from vknn_b200.sharding import gather_dim, shard_dim, shard_range


def test_shard_range_partitions_exactly():
    for n in (0, 1, 7, 16, 33):
        for world in (1, 2, 3, 8):
            spans = [shard_range(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            assert max(hi - lo for lo, hi in spans) - min(hi - lo for lo, hi in spans) <= 1
    with pytest.raises(ValueError):
        shard_range(4, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, dim, q_np, k_np, v_np, ref_np, ret):
    from oracle import vko
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        q, k, v = (torch.from_numpy(a) for a in (q_np, k_np, v_np))
        ql, kl, vl = (shard_dim(t, dim, rank, world).contiguous() for t in (q, k, v))
        if ql.shape[dim] > 0:
            ol = torch.from_numpy(vko.attention(ql.numpy(), kl.numpy(), vl.numpy(), 0.25, threads=1))
        else:
            ol = torch.zeros_like(ql)
        full = gather_dim(ol, dim, q.shape[dim])
        ret[rank] = bool(np.array_equal(full.numpy(), ref_np))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,dim", [(2, 1), (2, 0), (3, 1)])
def test_sharded_attention_matches_single_process(world, dim):
    from oracle import vko
    rng = np.random.default_rng(3)
    q, k, v = (rng.standard_normal((4, 5, 9, 16)).astype(np.float32) for _ in range(3))  # 5 heads: ragged over 2 and 3 ranks
    ref = vko.attention(q, k, v, 0.25, threads=1)
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(world, _free_port(), dim, q, k, v, ref, ret), nprocs=world, join=True)
    assert all(ret[r] for r in range(world)), dict(ret)
