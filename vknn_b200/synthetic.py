"""Seeded synthetic inputs with the shapes and value distributions of the baseline configurations (there are no
model weights or datasets on the machines this runs on)."""
import numpy as np


def encoder_weights(rng, d, dmlp, bias_scale=0.0, round_fp16=True):
    """Pre-LN block weights: matrices ~ N(0, 0.02) rounded to fp16 (as an fp16 .vxm holds them), LN gamma 1 / beta 0,
    biases 0 unless bias_scale is given. Matrices are row-major [K, N] like the reference's MatMul initializers."""
    def w(k, n):
        a = (0.02 * rng.standard_normal((k, n))).astype(np.float32)
        return a.astype(np.float16).astype(np.float32) if round_fp16 else a

    def bvec(n):
        return (bias_scale * rng.standard_normal(n)).astype(np.float32)

    return {
        "ln1_g": np.ones(d, np.float32), "ln1_b": np.zeros(d, np.float32),
        "wqkv": w(d, 3 * d), "bqkv": bvec(3 * d), "wo": w(d, d), "bo": bvec(d),
        "ln2_g": np.ones(d, np.float32), "ln2_b": np.zeros(d, np.float32),
        "w1": w(d, dmlp), "b1": bvec(dmlp), "w2": w(dmlp, d), "b2": bvec(d),
    }
