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


def _encoder_worker(rank, world, port, x_np, w, heads, ref_np, ret):
    """One pre-LN block with heads AND tokens sharded, in the order of EncoderLayer.forward_token_sharded: LayerNorm 1 on
    this rank's rows, gathered to all ranks; QKV projection of all tokens for this rank's heads (qkv_head_slice); attention
    on those heads, gathered along the head axis; out-projection, LayerNorm 2 and the MLP on this rank's rows. The two
    gathers stand for the fan-out stores of the GPU kernels."""
    from oracle import vko
    from vknn_b200.sharding import qkv_head_slice
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        T, d = x_np.shape
        D, Hl = d // heads, heads // world
        lo, hi = shard_range(T, rank, world)
        x_loc = x_np[lo:hi]
        h_loc = vko.layernorm(x_loc, w["ln1_g"], w["ln1_b"], 1e-6)
        h_full = gather_dim(torch.from_numpy(h_loc), 0, T).numpy()
        wq, bq = qkv_head_slice(torch.from_numpy(w["wqkv"]), torch.from_numpy(w["bqkv"]), heads, rank, world)
        qkv = vko.matmul(h_full, wq.numpy(), bq.numpy()).reshape(T, 3, Hl, D)
        q, k, v = (np.ascontiguousarray(qkv[:, i].transpose(1, 0, 2))[None] for i in range(3))  # [1,Hl,T,D]
        att = vko.attention(q, k, v, 1.0 / np.sqrt(D), threads=1)[0]                            # [Hl,T,D]
        att_full = gather_dim(torch.from_numpy(att), 0, heads).numpy()                          # [H,T,D]
        att_rows = np.ascontiguousarray(att_full.transpose(1, 0, 2)).reshape(T, d)[lo:hi]       # merged heads, this rank's rows
        x1 = vko.matmul(att_rows, w["wo"], w["bo"]) + x_loc
        h2 = vko.layernorm(x1, w["ln2_g"], w["ln2_b"], 1e-6)
        f = vko.matmul(h2, w["w1"], w["b1"])
        t = vko.binary(f, np.array([np.float32(1.41421356237)], np.float32), 2)
        t = vko.unary(t, 15)
        t = vko.binary(t, np.array([1.0], np.float32), 6)
        f = vko.pw_epilogue(t, [0, 0, 1, 0, 0, 0, 2, 0], [0, 0, 0, 0], [f, np.array([0.5], np.float32)])
        y_loc = vko.matmul(f, w["w2"], w["b2"]) + x1
        y = gather_dim(torch.from_numpy(np.ascontiguousarray(y_loc, dtype=np.float32)), 0, T).numpy()
        ret[rank] = float(np.abs(y - ref_np).max())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,heads,T", [(2, 4, 37), (3, 6, 50)])
def test_token_and_head_sharded_block_matches_single_process(world, heads, T):
    """The partitioning behind the collective-free multi-GPU encoder (ragged row slices, packed QKV head slices, merged-head
    column ranges) reproduces the unsharded block; every element is computed by the same operations in the same order, so
    only the last bits of the fp32 sums may differ."""
    from oracle import vko
    from vknn_b200.synthetic import encoder_weights
    rng = np.random.default_rng(12)
    d = heads * 8
    w = encoder_weights(rng, d, 2 * d, bias_scale=0.05)
    x = rng.standard_normal((T, d)).astype(np.float32)
    ref = vko.encoder_layer(x[None], w, heads, eps=1e-6, threads=1)[0]
    ret = mp.Manager().dict()
    mp.spawn(_encoder_worker, args=(world, _free_port(), x, w, heads, ref, ret), nprocs=world, join=True)
    assert all(ret[r] <= 2e-5 for r in range(world)), dict(ret)
