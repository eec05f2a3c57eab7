"""Generates tests/golden/raster_golden.npz: outputs of the reference's own renderer on seeded scenes.

Run where the reference tree is present:  python tests/golden/make_raster_golden.py <path of the reference tree>
It imports scripts/yonosplat/ref_rasterizer.py from that tree (nothing is copied), renders the scenes of
oracle.rasterizer.scene and stores the images; the scene inputs are regenerated from their seeds by the tests."""
import importlib.util
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import rasterizer  # noqa: E402

CASES = [(11, 600, 64, 64), (12, 3000, 96, 80)]  # (seed, gaussians, H, W)


def main(ref_root):
    spec = importlib.util.spec_from_file_location("ref_rasterizer", os.path.join(ref_root, "scripts/yonosplat/ref_rasterizer.py"))
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    out = {}
    for seed, n, H, W in CASES:
        means, covs, colors, opac, w2c, K = rasterizer.scene(seed, n, H, W)
        img, alpha = ref.render_view(*(a.astype(np.float64) for a in (means, covs, colors, opac)), w2c, K, H, W)
        out["rgb_%d" % seed] = img.astype(np.float32)
        out["alpha_%d" % seed] = alpha.astype(np.float32)
        out["case_%d" % seed] = np.array([seed, n, H, W])
    np.savez_compressed(os.path.join(ROOT, "tests/golden/raster_golden.npz"), **out)
    print("wrote", {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_raster_golden.py <path of the reference tree>")
    main(sys.argv[1])
