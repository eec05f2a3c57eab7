"""GPU parity tests: every kernel, called through the C-ABI, against the CPU oracle on the same seeded inputs.

Tolerances (stated by the task for this path, versus the reference's CPU backend):
  f16 / bf16 storage with fp32 accumulation: max|d| <= 1e-2 and cosine >= 0.9999 (tests.util.assert_low);
  fp32 storage: rel <= 1e-4 (assert_high).
Kernels whose outputs reach magnitudes where half an ulp of the storage type exceeds 1e-2 (GEMM, LayerNorm) are held to
tests.util.assert_storage instead: within 1 ulp of the oracle output rounded to the storage type, and <= 1e-2 from the
unrounded oracle output wherever |y| <= 2.
For 16-bit storage the oracle is fed the inputs already rounded to the storage type.
"""
import numpy as np
import pytest
import torch

import vknn_b200
from oracle import vko
from tests.util import assert_high, assert_low, assert_storage, encoder_weights, metrics, round_to

pytestmark = pytest.mark.gpu

DT = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


def dev(x, dtype):
    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).cuda().to(dtype).contiguous()


def host(t):
    return t.float().cpu().numpy()


# ------------------------------------------------------------------------------------------------ GEMM
@pytest.mark.parametrize("impl", [vknn_b200.IMPL_SIMT, vknn_b200.IMPL_TCGEN05], ids=["simt", "tc"])
@pytest.mark.parametrize("dt", ["f16", "bf16"])
@pytest.mark.parametrize("layout", [vknn_b200.B_KN, vknn_b200.B_NK])
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (197, 192, 72), (300, 520, 264), (64, 40, 128)])
def test_gemm_16bit(ctx, impl, dt, layout, M, N, K):
    rng = np.random.default_rng(M * 7 + N * 3 + K)
    a = round_to(rng.standard_normal((M, K)), DT[dt])
    b = round_to(rng.standard_normal((K, N)) * 0.1, DT[dt])
    bias = rng.standard_normal(N).astype(np.float32)
    ref = vko.matmul(a, b, bias)
    ctx.set_impl(impl)
    try:
        A = dev(a, DT[dt])
        Bm = dev(b if layout == vknn_b200.B_KN else b.T, DT[dt])
        D = torch.zeros(M, N, dtype=DT[dt], device="cuda")
        ctx.gemm(A, Bm, D, bias=torch.from_numpy(bias).cuda(), b_layout=layout)
        ctx.sync()
    finally:
        ctx.set_impl(vknn_b200.IMPL_AUTO)
    assert_storage(host(D), ref, dt, "gemm %s" % dt)


@pytest.mark.parametrize("epi", ["bias", "bias_gelu", "bias_residual"])
@pytest.mark.parametrize("impl", [vknn_b200.IMPL_SIMT, vknn_b200.IMPL_TCGEN05], ids=["simt", "tc"])
def test_gemm_epilogues(ctx, impl, epi):
    rng = np.random.default_rng(11)
    M, N, K = 200, 256, 128
    a = round_to(rng.standard_normal((M, K)), torch.float16)
    b = round_to(0.05 * rng.standard_normal((K, N)), torch.float16)
    bias = (0.1 * rng.standard_normal(N)).astype(np.float32)
    res = round_to(rng.standard_normal((M, N)), torch.float16)
    ref = vko.matmul(a, b, bias)
    flags = vknn_b200.EPI_BIAS
    if epi == "bias_gelu":
        t = vko.binary(ref, np.array([np.float32(1.41421356237)], np.float32), 2)
        t = vko.unary(t, 15)
        t = vko.binary(t, np.array([1.0], np.float32), 6)
        ref = vko.pw_epilogue(t, [0, 0, 1, 0, 0, 0, 2, 0], [0, 0, 0, 0], [ref, np.array([0.5], np.float32)])
        flags |= vknn_b200.EPI_GELU_ERF
    if epi == "bias_residual":
        ref = ref + res
        flags |= vknn_b200.EPI_RESIDUAL
    ctx.set_impl(impl)
    try:
        D = torch.zeros(M, N, dtype=torch.float16, device="cuda")
        ctx.gemm(dev(a, torch.float16), dev(b, torch.float16), D, bias=torch.from_numpy(bias).cuda(),
                 residual=dev(res, torch.float16) if epi == "bias_residual" else None, epilogue=flags)
        ctx.sync()
    finally:
        ctx.set_impl(vknn_b200.IMPL_AUTO)
    assert_low(host(D), ref, epi)


def test_gemm_batched_broadcast(ctx):
    """MatMul batch broadcast [B,M,K] @ [K,N] and [B,M,K] @ [B,K,N], tensor-core path."""
    rng = np.random.default_rng(5)
    Bn, M, N, K = 3, 130, 128, 64
    a = round_to(rng.standard_normal((Bn, M, K)), torch.float16)
    b1 = round_to(0.1 * rng.standard_normal((K, N)), torch.float16)
    b3 = round_to(0.1 * rng.standard_normal((Bn, K, N)), torch.float16)
    for b in (b1, b3):
        D = torch.zeros(Bn, M, N, dtype=torch.float16, device="cuda")
        ctx.gemm(dev(a, torch.float16), dev(b, torch.float16), D)
        ctx.sync()
        assert_low(host(D), vko.matmul(a, b), "batched")


def test_gemm_fp32_high(ctx):
    rng = np.random.default_rng(3)
    a = rng.standard_normal((2, 197, 64)).astype(np.float32)
    b = rng.standard_normal((2, 64, 197)).astype(np.float32)
    D = torch.zeros(2, 197, 197, dtype=torch.float32, device="cuda")
    ctx.gemm(dev(a, torch.float32), dev(b, torch.float32), D)
    ctx.sync()
    assert_high(host(D), vko.matmul(a, b), "gemm fp32")


def test_gemm_known_answer(ctx):
    """Ops.MatMul of the reference's unit tests: [2,3] @ [3,2] -> {4,5,10,11} (tests/test_ops.cpp:309-313)."""
    a = np.array([[1, 2, 3], [4, 5, 6]], np.float32)
    b = np.array([[1, 0], [0, 1], [1, 1]], np.float32)
    D = torch.zeros(2, 2, dtype=torch.float32, device="cuda")
    ctx.gemm(dev(a, torch.float32), dev(b, torch.float32), D)
    ctx.sync()
    np.testing.assert_allclose(host(D).ravel(), [4, 5, 10, 11], atol=1e-4)


# ------------------------------------------------------------------------------------------------ LayerNorm
@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("rows,norm", [(1576, 768), (2738, 1024), (256, 1024), (7, 100), (33, 2056)])
def test_layernorm(ctx, dt, rows, norm):
    rng = np.random.default_rng(rows + norm)
    x = round_to(rng.standard_normal((rows, norm)) * 2 + 0.5, DT[dt])
    g = (1 + 0.1 * rng.standard_normal(norm)).astype(np.float32)
    b = (0.1 * rng.standard_normal(norm)).astype(np.float32)
    ref = vko.layernorm(x, g, b, 1e-6)
    Y = torch.zeros(rows, norm, dtype=DT[dt], device="cuda")
    ctx.layernorm(dev(x, DT[dt]), torch.from_numpy(g).cuda(), torch.from_numpy(b).cuda(), Y, 1e-6)
    ctx.sync()
    if dt == "f32":
        assert_high(host(Y), ref, "layernorm")
    else:
        assert_storage(host(Y), ref, dt, "layernorm %s" % dt)
    # no beta
    ctx.layernorm(dev(x, DT[dt]), torch.from_numpy(g).cuda(), None, Y, 1e-6)
    ctx.sync()
    m = metrics(host(Y), vko.layernorm(x, g, None, 1e-6))
    assert m["cosine"] >= 0.9999, m


# ------------------------------------------------------------------------------------------------ prefill attention
def run_attn(ctx, q, k, v, scale, dt, causal=False, kv_len=None, mask=None, impl=vknn_b200.IMPL_AUTO):
    Q, K, V = dev(q, DT[dt]), dev(k, DT[dt]), dev(v, DT[dt])
    O = torch.zeros_like(Q)
    ctx.set_impl(impl)
    try:
        ctx.attn_prefill(Q, K, V, O, scale, causal=causal, mask=torch.from_numpy(mask).cuda() if mask is not None else None,
                         kv_len=torch.from_numpy(kv_len).cuda() if kv_len is not None else None)
        ctx.sync()
    finally:
        ctx.set_impl(vknn_b200.IMPL_AUTO)
    return host(O)


def test_attention_config1_fp32(ctx):
    """Config 1: Q,K,V fp32 [1,12,197,64] ~ N(0,1), seed 1001, scale 0.125, no mask; 'high' precision."""
    rng = np.random.default_rng(1001)
    q, k, v = (rng.standard_normal((1, 12, 197, 64)).astype(np.float32) for _ in range(3))
    ref = vko.attention(q, k, v, 0.125)
    assert_high(run_attn(ctx, q, k, v, 0.125, "f32"), ref, "config 1 fp32")


@pytest.mark.parametrize("impl", [vknn_b200.IMPL_SIMT, vknn_b200.IMPL_TCGEN05], ids=["simt", "tc"])
@pytest.mark.parametrize("dt", ["f16", "bf16"])
def test_attention_config1_low(ctx, impl, dt):
    rng = np.random.default_rng(1001)
    q, k, v = (round_to(rng.standard_normal((1, 12, 197, 64)), DT[dt]) for _ in range(3))
    ref = vko.attention(q, k, v, 0.125)
    assert_low(run_attn(ctx, q, k, v, 0.125, dt, impl=impl), ref, "config 1 %s" % dt)


@pytest.mark.parametrize("impl", [vknn_b200.IMPL_SIMT, vknn_b200.IMPL_TCGEN05], ids=["simt", "tc"])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("B,Hq,Hkv,Sq,Skv,D", [(2, 4, 4, 256, 256, 128), (1, 4, 2, 200, 333, 128), (1, 2, 1, 1, 130, 64), (2, 2, 2, 7, 65, 64),
                                               (1, 2, 2, 640, 640, 128)])
def test_attention_shapes(ctx, impl, causal, B, Hq, Hkv, Sq, Skv, D):
    """Ragged sizes (not tile multiples), GQA head mapping, Sq != Skv causal offset, multi-tile sequences."""
    rng = np.random.default_rng(B * 1000 + Sq + Skv + D + int(causal))
    q = round_to(rng.standard_normal((B, Hq, Sq, D)), torch.bfloat16)
    k = round_to(rng.standard_normal((B, Hkv, Skv, D)), torch.bfloat16)
    v = round_to(rng.standard_normal((B, Hkv, Skv, D)), torch.bfloat16)
    scale = 1.0 / np.sqrt(D)
    ref = vko.attention(q, k, v, scale, causal=causal)
    assert_low(run_attn(ctx, q, k, v, scale, "bf16", causal=causal, impl=impl), ref, "attn")


@pytest.mark.parametrize("dt", ["f16", "bf16"])
@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("jump", [7.0, 12.0, 30.0, 100.0])
def test_attention_maximum_grows_in_a_late_key_tile(ctx, dt, D, jump):
    """The tensor-core kernel raises its running maximum lazily (only when a key tile exceeds it by more than 2^8) and rescales
    the output accumulator in tensor memory when it does. A key in a later tile whose score exceeds everything before it by
    `jump` nats must still give the oracle's answer, below and above that threshold, with and without the causal mask.
    Different rows meet their dominant key in different tiles, some rows in none. Rows that lock onto one key return that
    key's V row: the comparison is 1e-2 wherever |y| <= 2 and 3 ulps of the rounded oracle output above that (P itself is
    rounded to the storage type)."""
    tdt = DT[dt]
    rng = np.random.default_rng(int(jump) * 10 + D)
    B, H, S = 1, 2, 700
    scale = 1.0 / np.sqrt(D)
    q = rng.standard_normal((B, H, S, D)) * 0.5
    k = rng.standard_normal((B, H, S, D)) * 0.5
    v = rng.standard_normal((B, H, S, D)) * 0.5  # rows torn between two dominant keys see P's own rounding times |v1 - v2|
    # dominant keys at positions 300 (third tile) and 650 (sixth): aligned with the queries of row groups so that the score of
    # (row, key) exceeds the rest by about `jump`
    for pos, rows in ((300, slice(0, 350)), (650, slice(200, 500))):
        direction = rng.standard_normal(D)
        direction /= np.linalg.norm(direction)
        amp = np.sqrt(jump / scale)
        k[:, :, pos] = direction * amp
        q[:, :, rows] += direction * amp
    q, k, v = (round_to(a, tdt) for a in (q, k, v))
    ref = vko.attention(q, k, v, scale)
    got = run_attn(ctx, q, k, v, scale, dt, impl=vknn_b200.IMPL_TCGEN05)
    assert_storage(got, ref, dt, "late dominant key, jump %g" % jump, ulps=3, floor=2.0)
    got = run_attn(ctx, q, k, v, scale, dt, causal=True, impl=vknn_b200.IMPL_TCGEN05)
    assert_storage(got, vko.attention(q, k, v, scale, causal=True), dt, "late dominant key, causal, jump %g" % jump, ulps=3, floor=2.0)


@pytest.mark.parametrize("dt", ["f16", "bf16"])
@pytest.mark.parametrize("B,Hq,Hkv,Sq,Skv", [(1, 2, 2, 1100, 1100), (2, 4, 2, 777, 1303), (1, 16, 16, 300, 2738)])
def test_attention_head64_key_range_split(ctx, dt, B, Hq, Hkv, Sq, Skv):
    """Head size 64, no mask, at least eight key tiles and only a few units: the tensor-core path cuts every unit into pieces
    of its key range, one per CTA, and merges them (ragged last key tile, GQA, ragged query tiles, Sq != Skv)."""
    tdt = torch.float16 if dt == "f16" else torch.bfloat16
    rng = np.random.default_rng(B + Sq + Skv)
    q = round_to(rng.standard_normal((B, Hq, Sq, 64)), tdt)
    k = round_to(rng.standard_normal((B, Hkv, Skv, 64)), tdt)
    v = round_to(rng.standard_normal((B, Hkv, Skv, 64)), tdt)
    ref = vko.attention(q, k, v, 0.125)
    n0 = ctx.launch_count()
    got = run_attn(ctx, q, k, v, 0.125, dt, impl=vknn_b200.IMPL_TCGEN05)
    assert ctx.launch_count() - n0 == 2  # the attention kernel and the merge of the pieces
    assert_low(got, ref, "attn split")


@pytest.mark.parametrize("dt,B,H,Sq,Skv,D,merged", [
    ("f16", 1, 16, 2738, 2738, 64, True),    # more units than SMs: a round of whole units, the left-over ones cut into pieces
    ("f16", 1, 2, 2738, 2738, 64, True),     # a handful of units: every unit cut into pieces, one piece per CTA
    ("bf16", 1, 6, 3072, 3072, 128, True),   # head size 128, units cut in two
    ("bf16", 1, 40, 1200, 1200, 128, True),  # ragged last query group and key tile, a round of whole units plus pieces
    ("bf16", 4, 16, 1024, 1024, 128, False), # two rounds of whole units through persistent CTAs, nothing to merge
])
def test_attention_balanced_forms(ctx, dt, B, H, Sq, Skv, D, merged):
    """Without a mask every (batch, head, query group) unit needs the same number of key tiles and the tensor-core kernel runs
    as persistent CTAs: whole units round-robin, then the left-over units cut into equal pieces whose partial rows a merge
    kernel joins. Every output row is compared with the SIMT kernel (itself checked against the oracle by the other tests),
    and 48 rows of every head — among them the first and last rows of query tiles and of the sequence — with the oracle."""
    tdt = DT[dt]
    rng = np.random.default_rng(B * 100000 + H * 1000 + Sq + D)
    q = round_to(rng.standard_normal((B, H, Sq, D)), tdt)
    k = round_to(rng.standard_normal((B, H, Skv, D)), tdt)
    v = round_to(rng.standard_normal((B, H, Skv, D)), tdt)
    scale = 1.0 / np.sqrt(D)
    n0 = ctx.launch_count()
    got = run_attn(ctx, q, k, v, scale, dt, impl=vknn_b200.IMPL_TCGEN05)
    if ctx.device_info()[1] == 148:  # the plan depends on the number of SMs
        assert ctx.launch_count() - n0 == (2 if merged else 1)
    simt = run_attn(ctx, q, k, v, scale, dt, impl=vknn_b200.IMPL_SIMT)
    assert np.isfinite(got).all()
    assert float(np.abs(got - simt).max()) <= 4e-3, float(np.abs(got - simt).max())
    rows = sorted(set([0, 1, 127, 128, 255, 256, 257, Sq // 2, Sq - 129, Sq - 128, Sq - 2, Sq - 1] + list(rng.integers(0, Sq, 36))))
    ref = vko.attention(np.ascontiguousarray(q[:, :, rows]), k, v, scale)
    assert_low(got[:, :, rows], ref, "balanced attention")


@pytest.mark.parametrize("dt,B,H,S,D", [("bf16", 7, 16, 1536, 128), ("f16", 3, 40, 2048, 64), ("bf16", 5, 64, 512, 128)])
def test_attention_causal_paired_blocks(ctx, dt, B, H, S, D):
    """Causal mask with Sq = Skv a multiple of 256 and enough work for more than two rounds of the SMs: the persistent form
    pairs the query groups (n - 1 - k, k) of a head into blocks of equal length, runs whole blocks round-robin and cuts the
    left-over blocks into pieces (a piece may hold the end of the long group and the start of the short one). Every row is
    compared with the SIMT kernel, 40 rows of every head with the oracle; the output starts as NaN."""
    tdt = DT[dt]
    rng = np.random.default_rng(B * 1000 + H + S + D)
    q = round_to(rng.standard_normal((B, H, S, D)), tdt)
    k = round_to(rng.standard_normal((B, H, S, D)), tdt)
    v = round_to(rng.standard_normal((B, H, S, D)), tdt)
    scale = 1.0 / np.sqrt(D)
    Q, K, V = dev(q, tdt), dev(k, tdt), dev(v, tdt)
    outs = []
    for impl in (vknn_b200.IMPL_TCGEN05, vknn_b200.IMPL_SIMT):
        O = torch.full_like(Q, float("nan"))
        ctx.set_impl(impl)
        try:
            ctx.attn_prefill(Q, K, V, O, scale, causal=True)
            ctx.sync()
        finally:
            ctx.set_impl(vknn_b200.IMPL_AUTO)
        outs.append(host(O))
    assert np.isfinite(outs[0]).all()
    assert float(np.abs(outs[0] - outs[1]).max()) <= (4e-3 if dt == "f16" else 3e-2)
    rows = sorted(set([0, 1, 127, 128, 255, 256, 257, S // 2, S - 257, S - 256, S - 129, S - 128, S - 2, S - 1] + list(rng.integers(0, S, 26))))
    mask = np.zeros((len(rows), S), np.float32)
    for i, r in enumerate(rows):
        mask[i, r + 1:] = -np.inf
    ref = vko.attention(np.ascontiguousarray(q[:, :, rows]), k, v, scale, mask=mask)
    # the first rows see a handful of keys and return (nearly) a V row, |y| up to 4: 1e-2 wherever |y| <= 2, 3 ulps of the rounded
    # oracle output above that (cut units pass through partials in the storage type)
    assert_storage(outs[0][:, :, rows], ref, dt, "causal paired blocks", ulps=3, floor=2.0)


def test_attention_balanced_forms_random_shapes(ctx):
    """Forty random unmasked shapes (1 to 400 units of 1 to 24 key tiles, both head sizes, ragged ends, Sq != Skv), so that the
    work distribution of the persistent form meets many combinations of rounds, left-over units and pieces. The output buffer
    starts as NaN: a row that no item wrote shows. Compared with the SIMT kernel of the same library."""
    rng = np.random.default_rng(4242)
    for case in range(40):
        D = int(rng.choice([64, 128]))
        dt = "f16" if case % 2 else "bf16"
        tdt = DT[dt]
        Sq = int(rng.integers(1, 1400))
        Skv = Sq if case % 3 else int(rng.integers(1, 3000))
        groups = (Sq + 255) // 256
        bh = max(1, int(rng.integers(1, 401)) // groups)
        H = int(rng.choice([h for h in (1, 2, 3, 4, 6, 8, 12, 16) if h <= bh]))
        B = max(1, bh // H)
        q = torch.randn(B, H, Sq, D, device="cuda").to(tdt)
        k = torch.randn(B, H, Skv, D, device="cuda").to(tdt)
        v = torch.randn(B, H, Skv, D, device="cuda").to(tdt)
        outs = []
        for impl in (vknn_b200.IMPL_TCGEN05, vknn_b200.IMPL_SIMT):
            o = torch.full_like(q, float("nan"))
            ctx.set_impl(impl)
            try:
                ctx.attn_prefill(q, k, v, o, D ** -0.5)
                ctx.sync()
            finally:
                ctx.set_impl(vknn_b200.IMPL_AUTO)
            outs.append(o.float())
        what = "case %d: B=%d H=%d Sq=%d Skv=%d D=%d %s" % (case, B, H, Sq, Skv, D, dt)
        assert torch.isfinite(outs[0]).all(), what
        assert float((outs[0] - outs[1]).abs().max()) <= (4e-3 if dt == "f16" else 2e-2), what


def test_captured_graph_survives_scratch_growth():
    """A key-range-split attention keeps its partials in the context's scratch block, whose address a captured CUDA graph
    bakes in. A later, larger call makes the scratch grow; the block the graph points at must stay alive (it is retired,
    not freed), so the replay still matches the oracle. Growth while a caller's stream is being captured is refused with
    an error instead of allocating."""
    c = vknn_b200.Context(0)  # its own context: the scratch starts empty
    try:
        rng = np.random.default_rng(77)
        q, k, v = (round_to(rng.standard_normal((1, 2, 1100, 64)), torch.float16) for _ in range(3))
        ref = vko.attention(q, k, v, 0.125)
        Q, K, V = (dev(a, torch.float16) for a in (q, k, v))
        O = torch.zeros_like(Q)
        st = torch.cuda.Stream()
        with torch.cuda.stream(st):
            small = torch.randn(1, 2, 256, 64, device="cuda").half()
            c.attn_prefill(small, small, small, torch.empty_like(small), 0.125)  # too short to split: no scratch yet
            c.sync()
            # a shape that needs scratch, asked for the first time inside a capture: refused, nothing allocated
            g0 = torch.cuda.CUDAGraph()
            refused = False
            with torch.cuda.graph(g0, stream=st):
                n0 = c.launch_count()
                c.attn_prefill(Q, K, V, O, 0.125)
                refused = c.launch_count() - n0 == 1  # ran unsplit (one launch, no merge) because the scratch could not grow
            assert refused
            n0 = c.launch_count()
            c.attn_prefill(Q, K, V, O, 0.125)  # eager: sizes the scratch
            assert c.launch_count() - n0 == 2
            c.sync()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=st):
                c.attn_prefill(Q, K, V, O, 0.125)
        O.zero_()
        g.replay()
        torch.cuda.synchronize()
        assert_low(host(O), ref, "split attention, graph replay")
        # a much larger user of the scratch: decode partials with no caller workspace, and a bigger split attention
        B, Hq, Hkv, L, D = 16, 32, 8, 4096, 128
        qd = torch.randn(B, Hq, D, device="cuda").half()
        kd, vd = (torch.randn(B, Hkv, L, D, device="cuda").half() for _ in range(2))
        od = torch.empty_like(qd)
        assert c.attn_decode_workspace_bytes(B, Hq, Hkv, L, D) > 4 * 2 * 1100 * (64 * 2 + 8)
        c.attn_decode(qd, kd, vd, od, D ** -0.5)
        Q2, K2, V2 = (torch.randn(1, 8, 2738, 64, device="cuda").half() for _ in range(3))
        c.attn_prefill(Q2, K2, V2, torch.empty_like(Q2), 0.125)
        c.sync()
        junk = [torch.full((1 << 20,), float("nan"), device="cuda") for _ in range(8)]  # reuse whatever the allocator got back
        O.zero_()
        g.replay()
        torch.cuda.synchronize()
        del junk
        assert_low(host(O), ref, "split attention, graph replay after the scratch grew")
    finally:
        c.sync()
        c.close()


@pytest.mark.parametrize("impl", [vknn_b200.IMPL_SIMT, vknn_b200.IMPL_TCGEN05], ids=["simt", "tc"])
def test_attention_kv_len(ctx, impl):
    rng = np.random.default_rng(77)
    B, H, Sq, Skv, D = 3, 2, 130, 300, 64
    q, k, v = (round_to(rng.standard_normal(s), torch.float16) for s in ((B, H, Sq, D), (B, H, Skv, D), (B, H, Skv, D)))
    kv_len = np.array([300, 1, 129], np.int32)
    ref = vko.attention(q, k, v, 0.125, kv_len=kv_len)
    assert_low(run_attn(ctx, q, k, v, 0.125, "f16", kv_len=kv_len, impl=impl), ref, "kv_len")


def test_attention_additive_mask(ctx):
    """FusedPointwise{Mul scale, Add mask} form (the reference's gqa graph), fp32."""
    rng = np.random.default_rng(9)
    q, k, v = (rng.standard_normal((1, 3, 40, 64)).astype(np.float32) for _ in range(3))
    mask = np.where(rng.random((40, 40)) < 0.3, -np.inf, 0.0).astype(np.float32)
    mask[:, 0] = 0
    ref = vko.attention(q, k, v, 0.125, mask=mask)
    assert_high(run_attn(ctx, q, k, v, 0.125, "f32", mask=mask), ref, "mask")


def test_attention_strided_views(ctx):
    """Head split/merge absorbed as strides: Q/K/V are views of a packed [B,T,3,H,D] buffer, O of [B,T,H,D]."""
    rng = np.random.default_rng(21)
    B, T, H, D = 2, 197, 4, 64
    qkv = round_to(rng.standard_normal((B, T, 3, H, D)), torch.float16)
    t = dev(qkv, torch.float16)
    q, k, v = (t[:, :, i].permute(0, 2, 1, 3) for i in range(3))
    o = torch.zeros(B, T, H, D, dtype=torch.float16, device="cuda")
    ctx.attn_prefill(q, k, v, o.permute(0, 2, 1, 3), 0.125)
    ctx.sync()
    qh, kh, vh = (np.ascontiguousarray(qkv[:, :, i].transpose(0, 2, 1, 3)) for i in range(3))
    ref = vko.attention(qh, kh, vh, 0.125).transpose(0, 2, 1, 3)
    assert_low(host(o), ref, "strided")


def test_attention_deterministic(ctx):
    rng = np.random.default_rng(4)
    q, k, v = (round_to(rng.standard_normal((1, 2, 300, 128)), torch.bfloat16) for _ in range(3))
    a = run_attn(ctx, q, k, v, 0.1, "bf16", causal=True)
    b = run_attn(ctx, q, k, v, 0.1, "bf16", causal=True)
    assert np.array_equal(a, b)


# ------------------------------------------------------------------------------------------------ decode attention
@pytest.mark.parametrize("impl", [vknn_b200.IMPL_SIMT, vknn_b200.IMPL_TCGEN05], ids=["simt", "tc"])
@pytest.mark.parametrize("dt", ["f16", "bf16"])
@pytest.mark.parametrize("B,Hq,Hkv,L,D", [(4, 32, 8, 1024, 128), (2, 8, 8, 300, 64), (3, 4, 2, 777, 128), (1, 8, 1, 130, 128), (5, 16, 1, 2100, 128),
                                          (2, 6, 2, 129, 128)])
def test_decode(ctx, impl, dt, B, Hq, Hkv, L, D):
    """Ragged valid lengths (1 .. L), GQA group sizes 1..16, caches that are not tile multiples. Everything past
    kv_len in the cache is NaN: a correct kernel never lets it reach the output."""
    G = Hq // Hkv
    if impl == vknn_b200.IMPL_TCGEN05 and D != 128:
        pytest.skip("the tensor-core decode kernel covers head dim 128")
    if impl == vknn_b200.IMPL_SIMT and G not in (1, 2, 4, 8):
        pytest.skip("the SIMT decode kernel covers group sizes 1, 2, 4, 8")
    rng = np.random.default_rng(B + Hq + L)
    q = round_to(rng.standard_normal((B, Hq, D)), DT[dt])
    k = round_to(rng.standard_normal((B, Hkv, L, D)), DT[dt])
    v = round_to(rng.standard_normal((B, Hkv, L, D)), DT[dt])
    kv_len = rng.integers(1, L + 1, B).astype(np.int32)
    kv_len[0] = L
    if B > 1:
        kv_len[1] = 1
    scale = 1.0 / np.sqrt(D)
    ref = vko.attention(q[:, :, None, :], k, v, scale, kv_len=kv_len)[:, :, 0, :]
    Kd, Vd = dev(k, DT[dt]), dev(v, DT[dt])
    for b in range(B):
        Kd[b, :, int(kv_len[b]):] = float("nan")
        Vd[b, :, int(kv_len[b]):] = float("nan")
    O = torch.zeros(B, Hq, D, dtype=DT[dt], device="cuda")
    lens = torch.from_numpy(kv_len).cuda()
    ctx.set_impl(impl)
    try:
        ctx.attn_decode(dev(q, DT[dt]), Kd, Vd, O, scale, kv_len=lens)
        ctx.sync()
        assert_low(host(O), ref, "decode")
        # caller-provided workspace gives the same bits
        ws = torch.empty(ctx.attn_decode_workspace_bytes(B, Hq, Hkv, L, D), dtype=torch.uint8, device="cuda")
        O2 = torch.zeros_like(O)
        ctx.attn_decode(dev(q, DT[dt]), Kd, Vd, O2, scale, kv_len=lens, workspace=ws)
        ctx.sync()
    finally:
        ctx.set_impl(vknn_b200.IMPL_AUTO)
    assert torch.equal(O, O2)


@pytest.mark.parametrize("case", ["many_short", "zeros_between", "all_empty", "one_long", "tile_edges"])
def test_decode_equal_runs_of_tiles(ctx, case):
    """The tensor-core decode kernel lays the 128-key tiles of all (sequence, kv head) units end to end and gives every CTA an
    equal run of that line. Cases that stress the cuts: many short sequences (a CTA's run spans several units and several
    sequences), empty sequences between full ones (units without a tile; their rows are NaN like the reference's 0/0), a
    batch with nothing in it, a single long unit cut into many pieces, and lengths on both sides of every tile edge."""
    rng = np.random.default_rng(len(case))
    D, dt = 128, "f16"
    if case == "many_short":
        B, Hq, Hkv, L = 40, 16, 4, 640
        kv_len = rng.integers(0, L + 1, B)
    elif case == "zeros_between":
        B, Hq, Hkv, L = 9, 8, 2, 1500
        kv_len = np.array([L, 0, 1, 0, 0, 777, L, 0, 129])
    elif case == "all_empty":
        B, Hq, Hkv, L = 3, 8, 2, 300
        kv_len = np.zeros(B)
    elif case == "one_long":
        B, Hq, Hkv, L = 1, 4, 1, 8192
        kv_len = np.array([8191])
    else:
        B, Hq, Hkv, L = 12, 32, 8, 1024
        kv_len = np.array([127, 128, 129, 255, 256, 257, 511, 512, 513, 1023, 1024, 1])
    kv_len = kv_len.astype(np.int32)
    q = round_to(rng.standard_normal((B, Hq, D)), DT[dt])
    k = round_to(rng.standard_normal((B, Hkv, L, D)), DT[dt])
    v = round_to(rng.standard_normal((B, Hkv, L, D)), DT[dt])
    scale = 1.0 / np.sqrt(D)
    Kd, Vd = dev(k, DT[dt]), dev(v, DT[dt])
    for b in range(B):
        Kd[b, :, int(kv_len[b]):] = float("nan")
        Vd[b, :, int(kv_len[b]):] = float("nan")
    O = torch.full((B, Hq, D), 7.0, dtype=DT[dt], device="cuda")
    ctx.set_impl(vknn_b200.IMPL_TCGEN05)
    try:
        ctx.attn_decode(dev(q, DT[dt]), Kd, Vd, O, scale, kv_len=torch.from_numpy(kv_len).cuda())
        ctx.sync()
    finally:
        ctx.set_impl(vknn_b200.IMPL_AUTO)
    got = host(O)
    full = kv_len > 0
    assert np.isnan(got[~full]).all()  # a sequence without keys: 0/0
    if full.any():
        ref = vko.attention(q[full][:, :, None, :], k[full], v[full], scale, kv_len=kv_len[full])[:, :, 0, :]
        assert_low(got[full], ref, "decode %s" % case)


def test_decode_config5_shape_slice(ctx):
    """Config 5 geometry (32 q / 8 kv heads, D=128, cache 8192, kv_len in [1024, 8192]) on 4 sequences."""
    rng = np.random.default_rng(1005)
    B, Hq, Hkv, L, D = 4, 32, 8, 8192, 128
    q = round_to(rng.standard_normal((B, Hq, D)), torch.float16)
    k = round_to(rng.standard_normal((B, Hkv, L, D)), torch.float16)
    v = round_to(rng.standard_normal((B, Hkv, L, D)), torch.float16)
    kv_len = rng.integers(1024, L + 1, B).astype(np.int32)
    scale = 1.0 / np.sqrt(D)
    ref = vko.attention(q[:, :, None, :], k, v, scale, kv_len=kv_len)[:, :, 0, :]
    O = torch.zeros(B, Hq, D, dtype=torch.float16, device="cuda")
    ctx.attn_decode(dev(q, torch.float16), dev(k, torch.float16), dev(v, torch.float16), O, scale, kv_len=torch.from_numpy(kv_len).cuda())
    ctx.sync()
    assert_low(host(O), ref, "decode config 5")


# ------------------------------------------------------------------------------------------------ pointwise family
def test_pointwise_known_answers(ctx):
    """FusedPwMulAddClip and FusedPwUnaryChannelMul of the reference's tests (tests/test_ops.cpp:502-515)."""
    x = dev(np.array([1, 2, 3, 4], np.float32).reshape(1, 1, 2, 2), torch.float32)
    y = torch.zeros_like(x)
    ops = [dev(np.full((1, 1, 2, 2), 2, np.float32), torch.float32), dev(np.ones((1, 1, 2, 2), np.float32), torch.float32)]
    ctx.pointwise(x, y, [0, 0, 1, 0, 0, 6, 2, 0, 2, 3, -1, 0], [0, 0, 0, 0, 0.0, 10.0], ops)
    ctx.sync()
    np.testing.assert_allclose(host(y).ravel(), [3, 5, 7, 9], atol=1e-5)
    x = dev(np.zeros((1, 3, 1, 2), np.float32), torch.float32)
    y = torch.zeros_like(x)
    ctx.pointwise(x, y, [1, 0, -1, 0, 0, 0, 1, 1], [0, 0, 0, 0], [dev(np.array([10, 20, 30], np.float32).reshape(1, 3, 1, 1), torch.float32)])
    ctx.sync()
    np.testing.assert_allclose(host(y).ravel(), [5, 5, 10, 10, 15, 15], atol=1e-5)


def test_pointwise_gelu_chain_and_softmax(ctx):
    rng = np.random.default_rng(8)
    h = rng.standard_normal((37, 300)).astype(np.float32) * 2
    X = dev(h, torch.float32)
    Y = torch.zeros_like(X)
    # Div(sqrt2) -> Erf -> Add(1) -> Mul(h) -> Mul(0.5) as one step program
    ops = [dev(np.array([np.float32(1.41421356237)]), torch.float32), dev(np.array([1.0], np.float32), torch.float32), X,
           dev(np.array([0.5], np.float32), torch.float32)]
    ctx.pointwise(X, Y, [0, 2, 1, 0, 1, 15, -1, 0, 0, 6, 2, 0, 0, 0, 3, 0, 0, 0, 4, 0], [0] * 10, ops)
    ctx.sync()
    t = vko.unary(vko.binary(h, np.array([np.float32(1.41421356237)]), 2), 15)
    ref = vko.pw_epilogue(vko.binary(t, np.array([1.0], np.float32), 6), [0, 0, 1, 0, 0, 0, 2, 0], [0, 0, 0, 0], [h, np.array([0.5], np.float32)])
    assert_high(host(Y), ref, "gelu chain")
    S = torch.zeros_like(X)
    ctx.softmax(X, S)
    ctx.sync()
    assert_high(host(S), vko.softmax(h), "softmax")


def test_softmax_epilogue_known_answer(ctx):
    """CpuEpilogueHookOnProducer: softmax([1,2,3,4]) * 3 (tests/test_ops.cpp:520-608)."""
    x = dev(np.array([[1, 2, 3, 4]], np.float32), torch.float32)
    s, y = torch.zeros_like(x), torch.zeros_like(x)
    ctx.softmax(x, s)
    ctx.pointwise(s, y, [0, 0, 1, 0], [0, 0], [dev(np.array([3.0], np.float32), torch.float32)])
    ctx.sync()
    e = np.exp(np.array([1, 2, 3, 4], np.float32) - 4)
    np.testing.assert_allclose(host(y).ravel(), e / e.sum() * 3, atol=1e-4)


def test_strided_copy_transpose(ctx):
    rng = np.random.default_rng(2)
    x = rng.standard_normal((2, 5, 3, 4, 6)).astype(np.float32)
    perm = [2, 0, 3, 1, 4]
    ref = vko.transpose(x, perm)
    X = dev(x, torch.float32)
    Y = torch.zeros(ref.shape, dtype=torch.float32, device="cuda")
    ist = [X.stride(p) for p in perm]
    ctx.strided_copy(X, Y, list(ref.shape), ist)
    ctx.sync()
    assert np.array_equal(host(Y), ref)


@pytest.mark.parametrize("dt", [torch.float32, torch.float16])
@pytest.mark.parametrize("inner", [1, 7, 8, 200])
def test_gather_rows_runtime_index(ctx, dt, inner):
    """out[o, k, :] = data[o, idx[k], :] with the index tensor on the device (float, half or int32), rows of odd and
    16-byte-multiple lengths, negative indices counted from the end; numpy indexing is the reference
    (GatherCpu::run src/backend/cpu/ops/gather.cpp:12-99)."""
    rng = np.random.default_rng(40 + inner)
    outer, axis = 3, 19
    data = rng.standard_normal((outer, axis, inner)).astype(np.float16).astype(np.float32)
    idx = np.array([0, 18, -1, 5, 5, -19, 7.9, 3], dtype=np.float32)  # 7.9 truncates to 7 like the reference's cast
    want = data[:, idx.astype(np.int64)]
    D = dev(data, dt)
    for I in (torch.from_numpy(idx).cuda(), torch.from_numpy(idx).cuda().to(torch.float16), torch.from_numpy(idx.astype(np.int32)).cuda()):
        Y = torch.zeros(want.shape, dtype=dt, device="cuda")
        ctx.gather_rows(D, I, Y, outer, axis, inner)
        ctx.sync()
        assert np.array_equal(host(Y), want), str(I.dtype)
    # an index outside the axis is clamped to it, never read from stray memory
    Y = torch.zeros((outer, 2, inner), dtype=dt, device="cuda")
    ctx.gather_rows(D, torch.tensor([1000.0, -1000.0], device="cuda"), Y, outer, axis, inner)
    ctx.sync()
    assert np.array_equal(host(Y), data[:, [axis - 1, 0]])


def test_copy_rows_offset_tables(ctx):
    """Row moves through device offset tables: a gather (source table), a scatter (destination table) and both at once."""
    rng = np.random.default_rng(44)
    src = rng.standard_normal((13, 24)).astype(np.float16).astype(np.float32)
    S = dev(src, torch.float16)
    pick = np.array([12, 0, 5, 5, 3], dtype=np.int64)
    Y = torch.zeros((5, 24), dtype=torch.float16, device="cuda")
    ctx.copy_rows(S, Y, torch.from_numpy(pick * 24).cuda(), None, 24)
    ctx.sync()
    assert np.array_equal(host(Y), src[pick])
    dst_rows = np.array([7, 1, 9], dtype=np.int64)
    Z = torch.zeros((10, 24), dtype=torch.float16, device="cuda")
    ctx.copy_rows(S, Z, None, torch.from_numpy(dst_rows * 24).cuda(), 24)
    ctx.sync()
    want = np.zeros((10, 24), np.float32)
    want[dst_rows] = src[:3]
    assert np.array_equal(host(Z), want)
    # 6-element rows at odd element offsets: the element-wise path
    Z2 = torch.zeros(100, dtype=torch.float16, device="cuda")
    ctx.copy_rows(S, Z2, torch.tensor([3, 51], device="cuda"), torch.tensor([1, 77], device="cuda"), 6)
    ctx.sync()
    want2 = np.zeros(100, np.float32)
    want2[1:7] = src.ravel()[3:9]
    want2[77:83] = src.ravel()[51:57]
    assert np.array_equal(host(Z2), want2)


@pytest.mark.parametrize("H,T,D", [(2, 700, 64), (4, 300, 128), (12, 1500, 64), (2, 2738, 64)])
def test_attention_fanout_stores_and_signals(ctx, H, T, D):
    """vkc_attn_prefill_fanout on one GPU: the same rows as vkc_attn_prefill land in every destination (here two local
    [T, H*D] buffers at a column offset, the merged-head layout a head-sharded encoder gathers into), through the direct
    epilogue (D = 128), the key-range-split merge pass (few heads at D = 64) and the unsplit one-tile form; each call raises
    this rank's flag in every destination by one, and vkc_peer_wait consumes exactly one step per call."""
    g = torch.Generator(device="cuda").manual_seed(70 + H)
    qkv = torch.randn(T, 3, H, D, generator=g, device="cuda").half()
    q, k, v = (qkv[:, i].permute(1, 0, 2).unsqueeze(0) for i in range(3))
    ref = torch.zeros(1, H, T, D, dtype=torch.float16, device="cuda")
    ctx.attn_prefill(q, k, v, ref, scale=D ** -0.5)
    width, off = H * D + 64, 64
    bufs = [torch.zeros(T, width, dtype=torch.float16, device="cuda") for _ in range(2)]
    flags = torch.zeros(2, 4, dtype=torch.int32, device="cuda")  # destination d: this rank owns word 1 of its flag row
    state = torch.zeros(2, dtype=torch.int32, device="cuda")
    expected = torch.zeros(1, dtype=torch.int32, device="cuda")
    for call in (1, 2):
        ctx.attn_prefill_fanout(q, k, v, [b.data_ptr() + off * 2 for b in bufs], [flags[d, 1:].data_ptr() for d in range(2)], state,
                                (T * width, D, width), scale=D ** -0.5)
        ctx.peer_wait(flags[0, 1:].data_ptr(), 1, expected)
        ctx.sync()
        want = ref[0].permute(1, 0, 2).reshape(T, H * D)
        for b in bufs:
            assert torch.equal(b[:, off:], want)
            assert not b[:, :off].any()
        assert flags[:, 1].tolist() == [call, call] and not flags[:, 0].any() and expected.item() == call
        assert state.tolist() == [0, call]


@pytest.mark.parametrize("dt", [torch.float16, torch.float32])
def test_layernorm_fanout_stores_and_signals(ctx, dt):
    """vkc_layernorm_fanout: the rows vkc_layernorm produces, stored at a row offset into two destinations, and the flag raised
    once per call (a grid with idle warps in its last block included)."""
    g = torch.Generator(device="cuda").manual_seed(9)
    rows, norm, at = 1003, 1024, 17
    x = torch.randn(rows, norm, generator=g, device="cuda").to(dt)
    gamma = torch.randn(norm, generator=g, device="cuda")
    beta = torch.randn(norm, generator=g, device="cuda")
    ref = torch.empty_like(x)
    ctx.layernorm(x, gamma, beta, ref, 1e-6)
    bufs = [torch.zeros(rows + 40, norm, dtype=dt, device="cuda") for _ in range(2)]
    flags = torch.zeros(2, dtype=torch.int32, device="cuda")
    state = torch.zeros(2, dtype=torch.int32, device="cuda")
    expected = torch.zeros(1, dtype=torch.int32, device="cuda")
    ctx.layernorm_fanout(x, gamma, beta, [b[at:].data_ptr() for b in bufs], [flags[d:].data_ptr() for d in range(2)], state, 1e-6)
    ctx.peer_wait(flags.data_ptr(), 2, expected)
    ctx.sync()
    for b in bufs:
        assert torch.equal(b[at:at + rows], ref) and not b[:at].any() and not b[at + rows:].any()
    assert flags.tolist() == [1, 1] and state.tolist() == [0, 1] and expected.item() == 1


def test_peer_wait_runs_out_instead_of_hanging(ctx):
    """A flag that nobody raises: the wait kernel gives up after its limit and the next sync reports a device error; the
    context stays usable."""
    import time
    flags = torch.zeros(2, dtype=torch.int32, device="cuda")
    expected = torch.zeros(1, dtype=torch.int32, device="cuda")
    ctx.sync()
    t0 = time.perf_counter()
    ctx.peer_wait(flags.data_ptr(), 2, expected)
    with pytest.raises(vknn_b200.VkcError) as e:
        ctx.sync()
    one = time.perf_counter() - t0
    assert e.value.code == -5
    assert int(expected.item()) == 0, "a wait that ran out must not advance the expected count"
    ctx.sync()
    # once the error word is set, queued waits return at once: eight more cost one limit (the first of them), not eight
    flags2 = torch.zeros(2, dtype=torch.int32, device="cuda")
    t0 = time.perf_counter()
    for _ in range(8):
        ctx.peer_wait(flags2.data_ptr(), 2, expected)
    with pytest.raises(vknn_b200.VkcError):
        ctx.sync()
    assert time.perf_counter() - t0 < 2.5 * one + 0.5
    assert int(expected.item()) == 0
    # a flag that is already there passes and advances the count
    flags.fill_(1)
    ctx.peer_wait(flags.data_ptr(), 2, expected)
    ctx.sync()
    assert int(expected.item()) == 1
    x = torch.randn(64, 256, device="cuda").half()
    y = torch.empty_like(x)
    ctx.layernorm(x, torch.ones(256, device="cuda"), torch.zeros(256, device="cuda"), y, 1e-5)
    ctx.sync()
    assert torch.isfinite(y.float()).all()


def test_gemm_gate_waits_for_flags_inside_the_kernel():
    """A GEMM whose A operand other GPUs produce polls their flags from its own producer warp. With the flags already raised
    the gated kernel equals the plain one and advances the expected count once (every CTA passed); with a flag that nobody
    raises it gives up after its limit, reports a device error through the next sync, leaves the count alone, and the
    context stays usable. Every tensor-core configuration family is covered: one-tile CTAs, split-K clusters, persistent."""
    c = vknn_b200.Context(0)
    try:
        M, N, K = 342, 1024, 1024
        gen = torch.Generator(device="cuda").manual_seed(41)
        a = torch.randn(M, K, device="cuda", generator=gen).half()
        b = (0.05 * torch.randn(K, N, device="cuda", generator=gen)).half()
        want = torch.empty(M, N, device="cuda", dtype=torch.float16)
        c.gemm(a, b, want)
        c.sync()
        flags = torch.zeros(4, dtype=torch.int32, device="cuda")
        state = torch.zeros(2, dtype=torch.int32, device="cuda")
        rounds = 0
        for cfg in [-1] + list(range(c.gemm_config_count())):
            got = torch.zeros_like(want)
            flags.fill_(rounds + 1)
            try:
                c.gemm(a, b, got, config=cfg, gate=(flags.data_ptr(), 4, state))
            except vknn_b200.VkcError as e:
                assert e.code == -2  # a configuration this shape cannot run
                continue
            c.sync()
            rounds += 1
            # split-K sums in another order: one fp16 ulp of outputs that reach |y| < 8
            assert torch.equal(got, want) or float((got.float() - want.float()).abs().max()) <= 2.0 ** -8, cfg
            assert state.tolist() == [rounds, 0], (cfg, state.tolist())
        assert rounds >= 6
        # nobody raises the flags for the next round
        got = torch.full_like(want, 7.0)
        c.gemm(a, b, got, gate=(flags.data_ptr(), 4, state))
        with pytest.raises(vknn_b200.VkcError) as e:
            c.sync()
        assert e.value.code == -5
        assert state.tolist() == [rounds, 0]
        c.gemm(a, b, got)
        c.sync()
        assert torch.equal(got, want)
    finally:
        try:
            c.sync()
        except vknn_b200.VkcError:
            pass
        c.close()


def test_upload_download_roundtrip(ctx):
    rng = np.random.default_rng(1)
    x = rng.standard_normal(10007).astype(np.float32)
    d = torch.zeros(10007, dtype=torch.float16, device="cuda")
    ctx.upload(d, x)
    back = np.zeros(10007, np.float32)
    ctx.download(back, d)
    ctx.sync()
    assert np.array_equal(back, x.astype(np.float16).astype(np.float32))


# ------------------------------------------------------------------------------------------------ encoder block
@pytest.mark.parametrize("B,T,d,H,dm", [(2, 197, 768, 12, 3072), (1, 300, 1024, 16, 4096)])
def test_encoder_layer(ctx, B, T, d, H, dm):
    """A pre-LN block at ViT-B (config 2) and d=1024 (config 3) widths, small batch so the oracle takes seconds."""
    from vknn_b200.encoder import EncoderLayer
    rng = np.random.default_rng(1002)
    w = encoder_weights(rng, d, dm, bias_scale=0.01)
    x = round_to(rng.standard_normal((B, T, d)), torch.float16)
    ref = vko.encoder_layer(x, w, H, eps=1e-6)
    layer = EncoderLayer(ctx, w, H, dtype=torch.float16)
    y = layer.forward(dev(x, torch.float16))
    ctx.sync()
    assert_low(host(y), ref, "encoder layer")


@pytest.mark.parametrize("epi", ["bias", "bias_gelu", "bias_residual"])
@pytest.mark.parametrize("M,N,K", [(300, 520, 1096), (1000, 256, 2048), (130, 200, 96)])
def test_gemm_every_configuration(ctx, epi, M, N, K):
    """Every tile / ring / occupancy / split-K configuration of the tensor-core GEMM (what the autotune chooses from)
    against the oracle, including ragged M, N and K tails; a configuration may refuse a shape, never mis-compute it."""
    rng = np.random.default_rng(21)
    a = round_to(rng.standard_normal((M, K)), torch.float16)
    b = round_to(0.05 * rng.standard_normal((K, N)), torch.float16)
    bias = (0.1 * rng.standard_normal(N)).astype(np.float32)
    res = round_to(rng.standard_normal((M, N)), torch.float16)
    ref = vko.matmul(a, b, bias)
    flags = vknn_b200.EPI_BIAS
    if epi == "bias_gelu":
        t = vko.binary(ref, np.array([np.float32(1.41421356237)], np.float32), 2)
        t = vko.unary(t, 15)
        t = vko.binary(t, np.array([1.0], np.float32), 6)
        ref = vko.pw_epilogue(t, [0, 0, 1, 0, 0, 0, 2, 0], [0, 0, 0, 0], [ref, np.array([0.5], np.float32)])
        flags |= vknn_b200.EPI_GELU_ERF
    if epi == "bias_residual":
        ref = ref + res
        flags |= vknn_b200.EPI_RESIDUAL
    A, Bm, R, bs = dev(a, torch.float16), dev(b, torch.float16), dev(res, torch.float16), torch.from_numpy(bias).cuda()
    ran = 0
    for cfg in range(ctx.gemm_config_count()):
        D = torch.zeros(M, N, dtype=torch.float16, device="cuda")
        try:
            ctx.gemm(A, Bm, D, bias=bs, residual=R if epi == "bias_residual" else None, epilogue=flags, config=cfg)
        except vknn_b200.VkcError as e:
            assert e.code == -2, str(e)  # VKC_ERR_UNSUPPORTED: this configuration does not take the shape
            continue
        ctx.sync()
        assert_low(host(D), ref, "config %d %s" % (cfg, epi))
        ran += 1
    assert ran >= 7
    with pytest.raises(vknn_b200.VkcError):
        ctx.gemm(A, Bm, torch.zeros(M, N, dtype=torch.float16, device="cuda"), bias=bs, epilogue=vknn_b200.EPI_BIAS, config=ctx.gemm_config_count())


def test_encoder_layer_tuned_matches_untuned(ctx):
    """EncoderLayer.tune (the Python mirror of CudaSegment::tuneGemms) only changes which configuration runs."""
    from vknn_b200.encoder import EncoderLayer
    rng = np.random.default_rng(1003)
    w = encoder_weights(rng, 256, 1024, bias_scale=0.01)
    x = round_to(rng.standard_normal((4, 197, 256)), torch.float16)
    ref = vko.encoder_layer(x, w, 4, eps=1e-6)
    layer = EncoderLayer(ctx, w, 4, dtype=torch.float16)
    xd = dev(x, torch.float16)
    layer.forward(xd)
    table = layer.tune(xd)
    assert len(table) == 4 and all(-1 <= v < ctx.gemm_config_count() for v in table.values())
    y = layer.forward(xd)
    ctx.sync()
    assert_low(host(y), ref, "tuned encoder layer")


def test_invalid_arguments(ctx):
    """Error behaviour: bad arguments are refused with a status and a message; nothing is launched."""
    q = torch.zeros(1, 3, 8, 64, dtype=torch.float16, device="cuda")
    k = torch.zeros(1, 2, 8, 64, dtype=torch.float16, device="cuda")
    n0 = ctx.launch_count()
    with pytest.raises(vknn_b200.VkcError) as e:
        ctx.attn_prefill(q, k, k, q, 0.125)
    assert e.value.code == -1 and "multiple" in str(e.value)
    with pytest.raises(vknn_b200.VkcError):
        ctx.attn_decode(torch.zeros(1, 4, 96, dtype=torch.float16, device="cuda"), torch.zeros(1, 4, 8, 96, dtype=torch.float16, device="cuda"),
                        torch.zeros(1, 4, 8, 96, dtype=torch.float16, device="cuda"), torch.zeros(1, 4, 96, dtype=torch.float16, device="cuda"), 1.0)
    assert ctx.launch_count() == n0
