"""Shared helpers of the parity tests: the reference's comparison metrics and seeded input generators."""
import numpy as np


def metrics(got, ref):
    """max|d|, cosine and relL2 exactly as the reference's benchmark tool defines them
    (benchmark/benchmark.cpp:496-525; `ref` plays the role of the golden `b`)."""
    a = np.asarray(got, dtype=np.float64).ravel()
    b = np.asarray(ref, dtype=np.float64).ravel()
    assert a.size == b.size
    nan = int(np.isnan(a).sum())
    keep = ~np.isnan(a)
    a, b = a[keep], b[keep]
    e = a - b
    return {
        "max_abs": float(np.abs(e).max()) if e.size else 0.0,
        "cosine": float(a.dot(b) / (np.sqrt(a.dot(a)) * np.sqrt(b.dot(b)) + 1e-12)),
        "rel_l2": float(np.sqrt(e.dot(e)) / (np.sqrt(b.dot(b)) + 1e-12)),
        "nan": nan,
    }


# Tolerances stated by the task for this path, versus the reference CPU backend on the same seeded inputs.
TOL_LOW = {"max_abs": 1e-2, "cosine": 0.9999}   # f16 / bf16 storage, fp32 accumulation
TOL_HIGH_REL = 1e-4                               # fp32 storage ("high" precision): relL2 and max|d| / max|ref|


def assert_low(got, ref, what=""):
    m = metrics(got, ref)
    assert m["nan"] == 0, (what, m)
    assert m["max_abs"] <= TOL_LOW["max_abs"] and m["cosine"] >= TOL_LOW["cosine"], (what, m)
    return m


def assert_high(got, ref, what=""):
    m = metrics(got, ref)
    scale = float(np.abs(np.asarray(ref)).max()) + 1e-30
    assert m["nan"] == 0, (what, m)
    assert m["rel_l2"] <= TOL_HIGH_REL and m["max_abs"] / scale <= TOL_HIGH_REL, (what, m)
    return m


def round_to(x, dtype):
    """Round fp32 host data to the device storage type and back, so the oracle sees what the GPU sees."""
    import torch
    t = torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32))
    return t.to(dtype).to(torch.float32).numpy()


from vknn_b200.synthetic import encoder_weights  # noqa: E402,F401
