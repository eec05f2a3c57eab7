"""The drop-in boundary end to end: graphs planned by the UNMODIFIED reference engine (its importer-side passes,
Session::plan partitioning, Session::run) with the CUDA backend plug-in selected and no CPU backend active, against
the same engine on its own CPU backend. Both run inside oracle/_ref/vknn_ref_driver(_cuda), which is compiled
from the reference sources plus vknn_b200/backend/cuda_backend.cpp where those sources are present."""
import os

import numpy as np
import pytest

from oracle import vko
from tests.util import assert_high, assert_low
from vknn_b200.synthetic import encoder_weights

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not os.path.exists(vko.REF_DRIVER_CUDA), reason="plug-in driver not built (needs the reference headers)")]

CUDA_KIND = 2


def both(graph_fn, precision, iters=3):
    (ref,), info_cpu = graph_fn().run(backend="cpu")
    (got,), info = graph_fn().run(backend="cuda", precision=precision, iters=iters)
    assert all(n[1] == CUDA_KIND for n in info["nodes"]), info["nodes"]  # every node was assigned to the plug-in
    assert [n[0] for n in info["nodes"]] == [n[0] for n in info_cpu["nodes"]]  # same passes, same node run
    return got, ref, info


def test_config1_attention_high_and_low():
    rng = np.random.default_rng(1001)
    q, k, v = (rng.standard_normal((1, 12, 197, 64)).astype(np.float32) for _ in range(3))
    got, ref, info = both(lambda: vko.attention_graph(q, k, v, 0.125), "high")
    assert [n[0] for n in info["nodes"]] == ["Transpose", "MatMul", "Binary", "Softmax", "MatMul"]
    assert_high(got, ref, "config 1 through the plug-in, fp32")
    got, ref, _ = both(lambda: vko.attention_graph(q, k, v, 0.125), "low")
    assert_low(got, ref, "config 1 through the plug-in, f16 storage")


def test_gqa_decode_graph_with_mask():
    rng = np.random.default_rng(7)
    B, Hkv, G, D, L = 2, 2, 4, 64, 96
    q, k, v = (rng.standard_normal(s).astype(np.float32) for s in ((B, Hkv, G, D), (B, Hkv, L, D), (B, Hkv, L, D)))
    mask = np.zeros((1, 1, G, L), np.float32)
    mask[..., 70:] = -np.inf
    got, ref, info = both(lambda: vko.attention_graph(q, k, v, 0.125, mask=mask), "high")
    assert "FusedPointwise" in [n[0] for n in info["nodes"]]
    assert_high(got, ref, "gqa with mask")


@pytest.mark.parametrize("B,T,d,H,dm", [(2, 130, 256, 4, 512), (1, 197, 768, 12, 3072)])
def test_encoder_layer_graph(B, T, d, H, dm):
    rng = np.random.default_rng(1002)
    w = encoder_weights(rng, d, dm, bias_scale=0.01)
    x = rng.standard_normal((B, T, d)).astype(np.float32)
    got, ref, info = both(lambda: vko.encoder_layer_graph(x, w, H), "low")
    assert_low(got, ref, "encoder layer through the plug-in")
    got, ref, _ = both(lambda: vko.encoder_layer_graph(x, w, H), "high", iters=1)
    assert_high(got, ref, "encoder layer through the plug-in, fp32")


def test_unsupported_node_is_refused_not_run_on_cpu():
    """No CPU backend is active for the CUDA session, so a node the plug-in declines fails the plan."""
    x = np.ones((4, 5), np.float32)
    g = vko.RefGraph()
    g.input("x", x)
    g.output("y", ())
    g.node("Softmax", "sm", ["x"], ["y"], axis=0)
    with pytest.raises(RuntimeError) as e:
        g.run(backend="cuda")
    assert "plan" in str(e.value) or "null" in str(e.value)


def test_fp16_vxm_weights_are_consumed_directly():
    """The on-disk format on the weight side of the path: an encoder layer compiled to a ".vxm" with fp16 initializers
    (what the reference's vknn_compile --fp16 writes) and loaded with Session::createFromVxm on both backends."""
    rng = np.random.default_rng(11)
    w = encoder_weights(rng, 256, 512, bias_scale=0.01)
    x = rng.standard_normal((2, 130, 256)).astype(np.float32)
    (ref,), info_cpu = vko.encoder_layer_graph(x, w, 4).run(backend="cpu", vxm_fp16=True)
    (got,), info = vko.encoder_layer_graph(x, w, 4).run(backend="cuda", precision="low", vxm_fp16=True, iters=2)
    assert all(n[1] == CUDA_KIND for n in info["nodes"])
    assert_low(got, ref, "fp16 .vxm through the plug-in")
    # and the file route gives the CPU backend the same answer as fp16-rounded weights fed directly
    w16 = {k: (v.astype(np.float16).astype(np.float32)) for k, v in w.items()}
    (ref2,), _ = vko.encoder_layer_graph(x, w16, 4).run(backend="cpu")
    assert np.abs(ref - ref2).max() <= 2e-3


def test_device_resident_io_matches_host_io():
    """The CUDA form of the reference's dma-buf I/O: inputs and outputs are caller-owned device buffers named by a
    registered handle that travels through Session::run in IOTensor::dmaBufFd; the segment converts on the device and
    the Session performs no host read-back. Results must be bit-identical to the host-buffer route."""
    rng = np.random.default_rng(12)
    w = encoder_weights(rng, 256, 512, bias_scale=0.01)
    x = rng.standard_normal((2, 130, 256)).astype(np.float32)
    for precision in ("low", "high"):
        (host,), info_h = vko.encoder_layer_graph(x, w, 4).run(backend="cuda", precision=precision, iters=2)
        (dev,), info_d = vko.encoder_layer_graph(x, w, 4).run(backend="cuda", precision=precision, iters=2, device_io=True)
        assert all(n[1] == CUDA_KIND for n in info_d["nodes"])
        assert dev.shape == host.shape
        assert np.array_equal(dev, host), precision
    # attention graph (two MatMuls around a Softmax): same check on the fused attention path
    q, k, v = (rng.standard_normal((1, 4, 100, 64)).astype(np.float32) for _ in range(3))
    (host,), _ = vko.attention_graph(q, k, v, 0.125).run(backend="cuda", precision="low")
    (dev,), _ = vko.attention_graph(q, k, v, 0.125).run(backend="cuda", precision="low", device_io=True)
    assert np.array_equal(dev, host)


def test_gemm_autotune_table_is_cached_and_reused(tmp_path):
    """Hint::Tuning + Config::cacheFile through the plug-in: the first session times the tensor-core GEMM configurations
    per shape and finalize() writes "<cacheFile>.cuda"; a second session loads the table instead of measuring (the
    file stays byte-identical) and produces the same output; with tuning off no file appears."""
    rng = np.random.default_rng(13)
    w = encoder_weights(rng, 256, 1024, bias_scale=0.01)
    x = rng.standard_normal((4, 160, 256)).astype(np.float32)
    cache = str(tmp_path / "model.cache")
    (ref,), _ = vko.encoder_layer_graph(x, w, 4).run(backend="cpu")
    (a,), info = vko.encoder_layer_graph(x, w, 4).run(backend="cuda", precision="low", cache_file=cache, tuning="fast", iters=2)
    assert all(n[1] == CUDA_KIND for n in info["nodes"])
    assert_low(a, ref, "tuned encoder layer")
    table = tmp_path / "model.cache.cuda"
    assert table.exists()
    lines = table.read_text().splitlines()
    assert lines[0] == "VKNNCUDA-TUNE-1" and len(lines) >= 2 + 4, lines     # header, GPU tag, the layer's four GEMM shapes
    assert all(ln.startswith("gemm:") for ln in lines[2:])
    before = table.read_bytes()
    (b,), _ = vko.encoder_layer_graph(x, w, 4).run(backend="cuda", precision="low", cache_file=cache, tuning="fast", iters=2)
    assert table.read_bytes() == before
    assert np.array_equal(a, b)
    cache2 = str(tmp_path / "other.cache")
    (c,), _ = vko.encoder_layer_graph(x, w, 4).run(backend="cuda", precision="low", cache_file=cache2, tuning="off")
    assert not (tmp_path / "other.cache.cuda").exists()
    assert_low(c, ref, "untuned encoder layer")


@pytest.mark.parametrize("precision", ["low", "high"])
def test_vit_frontend_ops_run_on_the_cuda_backend(precision):
    """The graph around the encoder blocks: patch-embedding Conv (as a GEMM over patches), Reshape/Transpose, Expand,
    Concat, Add, Slice (with and without a step), Split, Neg, rotary Mul/Add (FusedPointwise after the passes) and Tile
    all plan into one CUDA segment and match the reference CPU backend."""
    rng = np.random.default_rng(5)
    B, C, H, W, p, O = 2, 3, 64, 48, 16, 64
    N = (H // p) * (W // p)
    img = rng.standard_normal((B, C, H, W)).astype(np.float32)
    args = (img, (0.05 * rng.standard_normal((O, C, p, p))).astype(np.float32), (0.1 * rng.standard_normal(O)).astype(np.float32),
            rng.standard_normal((1, 1, O)).astype(np.float32), rng.standard_normal((1, N + 1, O)).astype(np.float32),
            np.cos(rng.standard_normal((N, O))).astype(np.float32), np.sin(rng.standard_normal((N, O))).astype(np.float32))
    ref, info_cpu = vko.vit_frontend_graph(*args).run(backend="cpu")
    got, info = vko.vit_frontend_graph(*args).run(backend="cuda", precision=precision, iters=2)
    kinds = [n[0] for n in info["nodes"]]
    for op in ("Conv", "Expand", "Concat", "Slice", "Split", "Tile"):
        assert op in kinds, kinds
    assert all(n[1] == CUDA_KIND for n in info["nodes"]), info["nodes"]
    assert len(got) == 3
    for a, b, what in zip(got, ref, ("sequence with class token", "rotary patches", "tile of a strided slice")):
        assert a.shape == b.shape
        if precision == "high":
            assert np.abs(a - b).max() <= 1e-4 * max(1.0, np.abs(b).max()), what
        else:
            assert_low(a, b, what)


@pytest.mark.parametrize("precision", ["low", "high"])
def test_selection_and_reduce_ops_run_on_the_cuda_backend(precision):
    """Greater / GreaterEqual / Equal, Where and the Reduce family (sum, mean, max, min, L2; leading, middle, trailing and
    mixed axes; keepdims on and off) plan into one CUDA segment and match the reference CPU backend. Inputs are exactly
    representable in fp16, so the comparisons see the same values at both storage precisions."""
    rng = np.random.default_rng(7)
    B, T, d = 3, 37, 48
    x = rng.standard_normal((B, T, d)).astype(np.float16).astype(np.float32)
    thr = (0.3 * rng.standard_normal((1, 1, d))).astype(np.float16).astype(np.float32)
    ref, _ = vko.masked_pool_graph(x, thr).run(backend="cpu")
    got, info = vko.masked_pool_graph(x, thr).run(backend="cuda", precision=precision, iters=2)
    kinds = [n[0] for n in info["nodes"]]
    for op in ("Greater", "GreaterEqual", "Equal", "Where", "Reduce"):
        assert op in kinds, kinds
    assert all(n[1] == CUDA_KIND for n in info["nodes"]), info["nodes"]
    names = ("pooled", "count", "argmax_mask_sum", "l2", "minv", "ge_mean")
    for a, b, what in zip(got, ref, names):
        assert a.shape == b.shape, what
        tol = 1e-4 * max(1.0, np.abs(b).max()) if precision == "high" else 1e-2 * max(1.0, np.abs(b).max())
        assert np.abs(a - b).max() <= tol, (what, float(np.abs(a - b).max()))
    # counts and masks are exact integers in either precision
    assert np.array_equal(got[1], ref[1]) and np.array_equal(got[2], ref[2])


@pytest.mark.parametrize("precision", ["low", "high"])
def test_index_driven_ops_run_on_the_cuda_backend(precision):
    """Gather with an index tensor computed at run time and with constant index lists (rank 1 and 2), ScatterND with constant
    indices (duplicates: the later row wins; negative indices) and Where with a broadcasting condition plan into one CUDA
    segment and match the reference CPU backend. Values are exactly representable in fp16 and the only arithmetic is one
    multiplication, so the moved rows are compared exactly against what the multiplication produced."""
    rng = np.random.default_rng(32)
    B, T, d, P = 3, 50, 72, 64
    f16 = lambda a: a.astype(np.float16).astype(np.float32)
    x = f16(rng.standard_normal((B, T, d)))
    table = f16(rng.standard_normal((P, d)))
    pos = rng.integers(0, P, size=T).astype(np.float32)
    keep = np.array([4, 0, -1, 4, 17, 33, 2], dtype=np.int64)
    R = 11
    upd = f16(rng.standard_normal((R, d)))
    scat_idx = np.stack([rng.integers(-B, B, size=R), rng.integers(-T, T, size=R)], axis=1).astype(np.int64)
    scat_idx[5] = scat_idx[1]          # a duplicate destination: row 5 must win over row 1
    scat_idx[9] = [scat_idx[2][0] % B - B, scat_idx[2][1] % T]  # the same destination through a negative batch index
    mask = (rng.random((T, 1)) > 0.5).astype(np.float32)
    graph = lambda: vko.token_lookup_graph(x, table, pos, keep, upd, scat_idx, mask)
    ref, _ = graph().run(backend="cpu")
    got, info = graph().run(backend="cuda", precision=precision, iters=2)
    kinds = [n[0] for n in info["nodes"]]
    for op in ("Gather", "ScatterND", "Where"):
        assert op in kinds, kinds
    assert all(n[1] == CUDA_KIND for n in info["nodes"]), info["nodes"]
    for a, b, what in zip(got, ref, ("rotated_kept", "picked2d", "scattered", "chosen")):
        assert a.shape == b.shape, what
        tol = 1e-4 * max(1.0, np.abs(b).max()) if precision == "high" else 1e-2 * max(1.0, np.abs(b).max())
        assert np.abs(a - b).max() <= tol, (what, float(np.abs(a - b).max()))
    # pure moves of input values are exact at either precision
    assert np.array_equal(got[1], ref[1])
    wrote = np.zeros((B, T), bool)
    for b, t in scat_idx:
        wrote[b, t] = True
    assert np.array_equal(got[2][wrote], ref[2][wrote])


def test_tuning_table_from_another_device_is_ignored(tmp_path):
    """A cache file whose header names another GPU / configuration set must not be trusted: the session measures again and
    rewrites it."""
    rng = np.random.default_rng(14)
    w = encoder_weights(rng, 256, 512, bias_scale=0.01)
    x = rng.standard_normal((2, 130, 256)).astype(np.float32)
    cache = str(tmp_path / "m.cache")
    table = tmp_path / "m.cache.cuda"
    table.write_text("VKNNCUDA-TUNE-1\nsome-other-gpu/configs=3\ngemm:1:260x768x256x1:0:1:111 2\n")
    (ref,), _ = vko.encoder_layer_graph(x, w, 4).run(backend="cpu")
    (got,), _ = vko.encoder_layer_graph(x, w, 4).run(backend="cuda", precision="low", cache_file=cache, tuning="fast")
    assert_low(got, ref, "encoder layer with a foreign tuning table")
    lines = table.read_text().splitlines()
    assert lines[1] != "some-other-gpu/configs=3" and len(lines) >= 2 + 4


@pytest.mark.parametrize("precision", ["low", "high"])
def test_rope_frequency_table_einsum_runs_on_the_cuda_backend(precision):
    """Einsum "i,j->ij" (the rotary frequency tables of the exported encoder; the passes do not lower it) with the Cos / Sin /
    rotation around it plans on the CUDA backend with no CPU backend active and matches the reference CPU backend. Positions
    and inverse frequencies are exactly representable in fp16 and their products stay below 2048, so the table itself is
    compared at storage precision."""
    rng = np.random.default_rng(34)
    B, T, d = 2, 74, 64
    x = rng.standard_normal((B, T, d)).astype(np.float16).astype(np.float32)
    pos = np.arange(T, dtype=np.float32)
    inv_freq = (2.0 ** -np.arange(d // 2, dtype=np.float32) * 4).astype(np.float32)  # powers of two: exact in fp16
    graph = lambda: vko.rope_table_graph(x, pos, inv_freq)
    ref, info_cpu = graph().run(backend="cpu")
    got, info = graph().run(backend="cuda", precision=precision, iters=2)
    assert "Einsum" in [n[0] for n in info["nodes"]]
    assert all(n[1] == CUDA_KIND for n in info["nodes"]), info["nodes"]
    assert got[0].shape == ref[0].shape == (T, d // 2)
    if precision == "high":
        assert np.array_equal(got[0], ref[0])
        assert_high(got[1], ref[1], "rope through the plug-in, fp32")
    else:
        normal = ref[0] >= 2.0 ** -14  # below that fp16 is subnormal
        assert np.array_equal(got[0][normal], ref[0][normal])
        # sin / cos of an argument stored in fp16 differ from fp32 by up to the argument's rounding (ulp/2 of values up to 292)
        small = np.broadcast_to(np.concatenate([ref[0], ref[0]], axis=1) <= 8.0, ref[1].shape)
        assert np.abs(got[1] - ref[1])[small].max() <= 1e-2


def test_profiler_gets_one_record_per_launch():
    """Config::profile: the Session's profiler receives a record per kernel launch of the CUDA segment, tagged with the node
    it was planned for and a device time, like the per-node records of the reference's own backends."""
    rng = np.random.default_rng(35)
    w = encoder_weights(rng, 256, 512, bias_scale=0.01)
    x = rng.standard_normal((2, 130, 256)).astype(np.float32)
    (ref,), _ = vko.encoder_layer_graph(x, w, 4).run(backend="cpu")
    (got,), info = vko.encoder_layer_graph(x, w, 4).run(backend="cuda", precision="low", iters=2, profile=True)
    assert_low(got, ref, "profiled encoder layer")
    recs = info["profile"]
    assert all(r[2] == "CUDA" and r[3] >= 0 for r in recs), recs
    labels = [r[0].split("[")[-1].rstrip("]") for r in recs]
    # LayerNorm, QKV GEMM, attention, out-projection, LayerNorm, fc1 + GELU, fc2 + residual, plus whatever copies the views needed
    assert labels.count("layernorm") == 2 and labels.count("matmul") == 4 and labels.count("attention") == 1, recs
    assert recs[0][0].startswith("ln1 ") and any(r[0].startswith("qk ") for r in recs), recs


def test_runtime_gather_over_a_long_axis_is_left_to_another_backend():
    """An index tensor computed at run time lives in the segment's storage type; fp16 holds integers exactly only up to 2048,
    so with fp16 storage a Gather over a longer axis is declined at plan time (no CPU backend is active here: the plan
    fails) instead of fetching wrong rows. With fp32 storage the same graph runs."""
    rng = np.random.default_rng(36)
    P, T, d = 2738, 40, 8
    table = rng.standard_normal((P, d)).astype(np.float32)
    pos = rng.integers(2049, P, size=T).astype(np.float32)

    def graph():
        g = vko.RefGraph()
        g.input("pos", pos)
        g.input("x", np.ones((T, d), np.float32))
        g.init("table", table)
        g.inter("rows")
        g.output("y", (T, d))
        g.node("Gather", "lookup", ["table", "pos"], ["rows"], axis=0)
        g.node("Binary", "use", ["x", "rows"], ["y"], subop=0)
        return g

    with pytest.raises(RuntimeError) as e:
        graph().run(backend="cuda", precision="low")
    assert "plan" in str(e.value)
    (got,), _ = graph().run(backend="cuda", precision="high")
    assert np.array_equal(got, table[pos.astype(np.int64)])


def test_device_ordinal_from_the_config():
    """The plug-in takes its device from a spare Config::hints slot: the same graph gives the same result on every visible
    GPU, and an ordinal that does not exist is refused when the session is planned."""
    import torch
    rng = np.random.default_rng(37)
    q, k, v = (rng.standard_normal((1, 4, 150, 64)).astype(np.float32) for _ in range(3))
    outs = []
    for dev_i in range(min(torch.cuda.device_count(), 2)):
        (got,), _ = vko.attention_graph(q, k, v, 0.125).run(backend="cuda", precision="low", device=dev_i)
        outs.append(got)
    (ref,), _ = vko.attention_graph(q, k, v, 0.125).run(backend="cpu")
    for got in outs:
        assert_low(got, ref, "attention on a chosen device")
        assert np.array_equal(got, outs[0])
    with pytest.raises(RuntimeError):
        vko.attention_graph(q, k, v, 0.125).run(backend="cuda", precision="low", device=torch.cuda.device_count())
