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


def splat_scene(seed, n, H, W):
    """Seeded synthetic 3D Gaussian-splatting scene (stands in for the encoder's Gaussian outputs; no dataset is used):
    means in front of a camera looking down +z, anisotropic world covariances A A^T, colours in [0, 1], opacities in
    (0, 1), a world-to-camera matrix with a small rotation and pixel intrinsics for an H x W image."""
    rng = np.random.default_rng(seed)
    means = np.stack([rng.uniform(-1.6, 1.6, n), rng.uniform(-1.6, 1.6, n), rng.uniform(-0.3, 5.0, n)], 1).astype(np.float32)
    A = rng.standard_normal((n, 3, 3)) * rng.uniform(0.005, 0.12, (n, 1, 1))
    covs = (A @ A.transpose(0, 2, 1)).astype(np.float32)
    colors = rng.uniform(0.0, 1.0, (n, 3)).astype(np.float32)
    opac = rng.uniform(0.02, 0.98, n).astype(np.float32)
    ang = 0.15
    Ry = np.array([[np.cos(ang), 0, np.sin(ang)], [0, 1, 0], [-np.sin(ang), 0, np.cos(ang)]])
    w2c = np.eye(4)
    w2c[:3, :3] = Ry
    w2c[:3, 3] = [0.05, -0.1, 1.5]
    K = np.array([[0.9 * W, 0, 0.5 * W], [0, 0.9 * H, 0.5 * H], [0, 0, 1.0]])
    return means, covs, colors, opac, w2c, K
