"""Multi-GPU path on real devices (skipped with fewer than two GPUs): a head-sharded encoder layer must reproduce the
single-GPU layer, both with the NCCL all-gather at the attention-output boundary and with the attention kernel storing its
tiles into every rank's gather buffer over peer memory (no collective, captured as a CUDA graph)."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, ret):
    import torch.distributed as dist
    import vknn_b200
    from vknn_b200.encoder import EncoderLayer
    from vknn_b200.synthetic import encoder_weights
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        ctx = vknn_b200.Context(rank)
        w = encoder_weights(np.random.default_rng(5), 256, 512, bias_scale=0.01)
        x = torch.randn(1, 333, 256, generator=torch.Generator().manual_seed(1)).cuda().half()
        layer = EncoderLayer(ctx, w, 8, device="cuda:%d" % rank)
        ref = layer.forward(x).clone()
        layer.shard_heads(rank, world)
        got = layer.forward_head_sharded(x)
        ctx.sync()
        ret[rank] = float((got.float() - ref.float()).abs().max())
        # the same through peer memory: two layers (the two gather buffers alternate), eager and as a replayed graph
        from vknn_b200.encoder import EncoderStack
        from vknn_b200.sharding import PeerGather
        rng = np.random.default_rng(6)
        x = torch.randn(1, 333, 512, generator=torch.Generator().manual_seed(2)).cuda().half()  # head size 64: the tensor-core kernel
        stack = EncoderStack(ctx, [encoder_weights(rng, 512, 1024, bias_scale=0.01) for _ in range(2)], 8, dtype=torch.float16)
        ref2 = stack.forward(x).clone()
        stack.shard_heads(rank, world)
        gather = PeerGather(ctx, 333, 512, torch.float16)
        got2 = stack.forward_head_sharded_fused(x, gather).clone()
        ctx.sync()
        err = float((got2.float() - ref2.float()).abs().max())
        torch.cuda.synchronize()
        dist.barrier()
        graph, y = stack.capture_head_sharded_fused(x, gather)
        for _ in range(3):
            graph.replay()
        ctx.sync()
        err = max(err, float((y.float() - ref2.float()).abs().max()))
        ret["fused%d" % rank] = err
        dist.barrier()
        # tokens sharded as well: LayerNorm and attention both fan their output out, no collective inside the forward
        from vknn_b200.sharding import gather_dim
        gh = PeerGather(ctx, 333, 512, torch.float16)
        mine = stack.forward_token_sharded(x, gh, gather)
        ctx.sync()
        full = gather_dim(mine.clone(), 0, 333)
        err = float((full.float() - ref2[0].float()).abs().max())
        dist.barrier()
        graph, y = stack.capture_token_sharded(x, gh, gather)
        for _ in range(3):
            graph.replay()
        ctx.sync()
        full = gather_dim(y.clone(), 0, 333)
        ret["tokens%d" % rank] = max(err, float((full.float() - ref2[0].float()).abs().max()))
        dist.barrier()
        gh.close()
        gather.close()
        ctx.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_head_sharded_layer_matches_single_gpu():
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(2, port, ret), nprocs=2, join=True)
    # same kernels on the same values; only the GEMM tile shapes differ between the sharded and the full QKV projection
    assert all(ret[r] <= 2e-3 for r in range(2)), dict(ret)
    assert all(ret["fused%d" % r] <= 4e-3 for r in range(2)), dict(ret)
    assert all(ret["tokens%d" % r] <= 4e-3 for r in range(2)), dict(ret)
