"""Generates tests/golden/vknn_cpu_golden.npz by running the UNMODIFIED reference engine's CPU backend
(oracle/_ref/vknn_ref_driver, built from the reference sources by oracle/Makefile) on small seeded inputs.

    python tests/golden/make_golden.py

It needs the reference sources to build oracle/_ref and therefore only runs where they are present; the
committed .npz is what the CPU tests read everywhere else. Each case stores its inputs and the reference's
outputs; tests/test_oracle.py requires the C restatement to reproduce every output bit for bit.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import vko  # noqa: E402
from tests.util import encoder_weights  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "vknn_cpu_golden.npz")


def single(op, x, inits=(), subop=0, **attrs):
    g = vko.RefGraph()
    g.input("x", x)
    names = ["x"]
    for i, a in enumerate(inits):
        g.init("i%d" % i, a)
        names.append("i%d" % i)
    g.output("y", ())
    g.node(op, "op", names, ["y"], subop=subop, **attrs)
    (y,), info = g.run()
    return y


def main():
    vko.build()
    rng = np.random.default_rng(20261125)
    G = {}
    f = lambda *s: rng.standard_normal(s).astype(np.float32)  # noqa: E731

    # MatMul: plain, batched with broadcast B, with fusedBias (via MatMul + Add -> fuseMatMulBias)
    a, b = f(2, 3, 7, 5), f(5, 6)
    G["mm_a"], G["mm_b"], G["mm_y"] = a, b, single("MatMul", a, [b])
    a2, b2 = f(3, 1, 4, 8), f(1, 2, 8, 3)
    G["mmb_a"], G["mmb_b"], G["mmb_y"] = a2, b2, single("MatMul", a2, [b2])
    bias = f(6)
    g = vko.RefGraph()
    g.input("x", a)
    g.init("w", b)
    g.init("bias", bias)
    g.inter("t")
    g.output("y", ())
    g.node("MatMul", "mm", ["x", "w"], ["t"])
    g.node("Add", "add", ["t", "bias"], ["y"])
    (y,), info = g.run()
    assert info["nodes"] == [["MatMul", 1, 0, 1]], info["nodes"]  # the bias was fused by the reference's pass
    G["mmbias_bias"], G["mmbias_y"] = bias, y

    # Softmax, LayerNorm (with / without beta), Erf, Binary broadcast
    x = f(6, 33) * 3
    G["sm_x"], G["sm_y"] = x, single("Softmax", x, axis=-1)
    x = f(5, 48) * 2 + 1
    gam, bet = 1 + 0.1 * f(48), 0.1 * f(48)
    G["ln_x"], G["ln_g"], G["ln_b"] = x, gam, bet
    G["ln_y"] = single("LayerNorm", x, [gam, bet], axis=-1, epsilon=1e-6)
    G["ln_y_nobeta_eps5"] = single("LayerNorm", x, [gam], axis=-1)
    x = f(4, 50) * 2
    G["erf_x"], G["erf_y"] = x, single("Unary", x, subop=15)
    x, s = f(2, 3, 4), f(3, 1)
    G["bin_x"], G["bin_s"] = x, s
    for code, name in ((0, "mul"), (1, "sub"), (2, "div"), (3, "max"), (6, "add")):
        G["bin_y_" + name] = single("Binary", x, [s], subop=code)

    # GELU chain as exported: Div -> Erf -> Add -> Mul -> Mul
    h = f(4, 50) * 2
    g = vko.RefGraph()
    g.input("f1", h)
    g.init("sqrt2", np.array([np.float32(1.41421356237)], np.float32))
    g.init("one", np.array([1.0], np.float32))
    g.init("half", np.array([0.5], np.float32))
    for n in ("gd", "ge", "ga", "gm"):
        g.inter(n)
    g.output("gh", ())
    g.node("Binary", "g_div", ["f1", "sqrt2"], ["gd"], subop=2)
    g.node("Unary", "g_erf", ["gd"], ["ge"], subop=15)
    g.node("Add", "g_add", ["ge", "one"], ["ga"])
    g.node("Binary", "g_mul", ["f1", "ga"], ["gm"], subop=0)
    g.node("Binary", "g_half", ["gm", "half"], ["gh"], subop=0)
    (y,), info = g.run()
    G["gelu_x"], G["gelu_y"] = h, y
    G["gelu_nodes"] = np.array([n[0] for n in info["nodes"]])

    # attention, config-1 pattern at a reduced size, and the same with ragged lengths
    q, k, v = f(1, 2, 37, 64), f(1, 2, 37, 64), f(1, 2, 37, 64)
    (o,), info = vko.attention_graph(q, k, v, 0.125).run()
    G["att_q"], G["att_k"], G["att_v"], G["att_o"] = q, k, v, o
    G["att_nodes"] = np.array([n[0] for n in info["nodes"]])

    # GQA decode with an additive -inf valid-length mask (MatMul batch broadcast form)
    B, Hkv, Gq, D, L = 2, 2, 4, 16, 40
    q, k, v = f(B, Hkv, Gq, D), f(B, Hkv, L, D), f(B, Hkv, L, D)
    kv_len = np.array([7, 40], np.int32)
    mask = np.zeros((B, 1, 1, L), np.float32)
    for bi in range(B):
        mask[bi, ..., kv_len[bi]:] = -np.inf
    (o,), info = vko.attention_graph(q, k, v, 0.25, mask=mask).run()
    G["gqa_q"], G["gqa_k"], G["gqa_v"], G["gqa_len"], G["gqa_o"] = q, k, v, kv_len, o
    G["gqa_nodes"] = np.array([n[0] for n in info["nodes"]])

    # causal prefill via an additive mask, Sq != Skv
    q, k, v = f(1, 2, 5, 16), f(1, 2, 9, 16), f(1, 2, 9, 16)
    cm = np.zeros((5, 9), np.float32)
    for i in range(5):
        cm[i, i + 4 + 1:] = -np.inf
    (o,), _ = vko.attention_graph(q, k, v, 0.25, mask=cm).run()
    G["cau_q"], G["cau_k"], G["cau_v"], G["cau_o"] = q, k, v, o

    # one pre-LN encoder block
    B, T, d, H, dm = 2, 9, 32, 2, 64
    w = encoder_weights(rng, d, dm, bias_scale=0.05)
    w["ln1_g"] = (1 + 0.1 * f(d)).astype(np.float32)
    w["ln2_b"] = (0.1 * f(d)).astype(np.float32)
    x = f(B, T, d)
    (y,), info = vko.encoder_layer_graph(x, w, H).run()
    G["enc_x"], G["enc_y"] = x, y
    for kk, vv in w.items():
        G["enc_w_" + kk] = vv
    G["enc_nodes"] = np.array([n[0] for n in info["nodes"]])

    # config 1 at full size (seed 1001): output digest only (the inputs regenerate from the seed)
    r1 = np.random.default_rng(1001)
    q, k, v = (r1.standard_normal((1, 12, 197, 64)).astype(np.float32) for _ in range(3))
    (o,), _ = vko.attention_graph(q, k, v, 0.125).run()
    G["c1_sample"] = o[0, :, ::49, ::8].copy()
    G["c1_sum"] = np.array([o.astype(np.float64).sum(), np.abs(o.astype(np.float64)).sum()])
    G["c1_input_digest"] = np.array([q.astype(np.float64).sum(), k.astype(np.float64).sum(), v.astype(np.float64).sum()])

    np.savez_compressed(OUT, **G)
    print("wrote", OUT, os.path.getsize(OUT), "bytes,", len(G), "arrays")


if __name__ == "__main__":
    main()
