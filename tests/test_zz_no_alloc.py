"""The allocation-free decode entry point (vkc_attn_decode_noalloc) against the regular one.

Hosts that must not allocate device memory when a decode step is due (a fixed start-up memory budget, a device
owned by another allocator, a moment where an allocation would stall the GPU) call this variant: its scratch is a
fixed 16 MiB area inside the library. It has to give the same result as vkc_attn_decode on back-to-back calls,
even though the area still holds the previous call's partial results, and must refuse shapes that do not fit.
This file sorts last on purpose, so a run that stops at the first failure has already run everything else.
"""
import numpy as np
import pytest
import torch

import vknn_b200

pytestmark = pytest.mark.gpu


def _case(seed, B, Hq, Hkv, L, D, dtype):
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = torch.randn(B, Hq, D, generator=g, device="cuda").to(dtype)
    k = torch.randn(B, Hkv, L, D, generator=g, device="cuda").to(dtype)
    v = torch.randn(B, Hkv, L, D, generator=g, device="cuda").to(dtype)
    lens = torch.from_numpy(np.random.default_rng(seed).integers(1, L + 1, B).astype(np.int32)).cuda()
    return q, k, v, lens


def test_noalloc_matches_regular_entry_point_twice(ctx):
    # two calls in a row with different shapes and data: the second one runs over the first one's leftovers
    for seed, (B, Hq, Hkv, L, D, dtype) in enumerate([(4, 32, 8, 2048, 128, torch.float16), (3, 8, 2, 700, 64, torch.bfloat16)]):
        q, k, v, lens = _case(100 + seed, B, Hq, Hkv, L, D, dtype)
        ref = torch.zeros_like(q)
        out = torch.full_like(q, float("nan"))
        ctx.attn_decode(q, k, v, ref, D ** -0.5, kv_len=lens)
        ctx.attn_decode_noalloc(q, k, v, out, D ** -0.5, kv_len=lens)
        ctx.sync()
        a, b = out.float().cpu().numpy(), ref.float().cpu().numpy()
        assert not np.isnan(a).any()
        # same kernels, same split layout: the tolerance of the other 16-bit tests is far more than is needed
        assert np.abs(a - b).max() <= 1e-2
        assert np.array_equal(a, b)


def test_noalloc_refuses_oversized_shapes(ctx):
    limit = int(ctx.lib.vkc_attn_decode_noalloc_max_bytes())
    assert limit == 16 << 20
    B, Hq, Hkv, L, D = 64, 64, 8, 8192, 128  # partials: 64*64*16*130*4 bytes = 34 MB
    assert ctx.attn_decode_workspace_bytes(B, Hq, Hkv, L, D) > limit
    # only shapes are checked before the refusal, so tiny stand-in buffers are enough; nothing is launched
    q = torch.zeros(B, Hq, D, dtype=torch.float16, device="cuda")
    kv = torch.zeros(1, dtype=torch.float16, device="cuda")
    n0 = ctx.launch_count()
    rc = ctx.lib.vkc_attn_decode_noalloc(ctx.h, q.data_ptr(), kv.data_ptr(), kv.data_ptr(), q.data_ptr(), B, Hq, Hkv, L, D, None, 0.1, vknn_b200.F16,
                                         None)
    assert rc == -1 and b"fixed" in ctx.lib.vkc_last_error(ctx.h)
    assert ctx.launch_count() == n0
