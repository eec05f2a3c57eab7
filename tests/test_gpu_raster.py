"""3D Gaussian-splatting rasterizer (CUDA) against the CPU restatement of the reference renderer and against images
rendered by the reference's own Python renderer (tests/golden/raster_golden.npz)."""
import os

import numpy as np
import pytest
import torch

import vknn_b200
from oracle import rasterizer

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    c = vknn_b200.Context(0)
    yield c
    c.close()


def render(ctx, scene, H, W, precise):
    means, covs, colors, opac, w2c, K = scene
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()  # noqa: E731
    rgb, alpha = ctx.raster_gaussians(dev(means), dev(covs), dev(colors), dev(opac), w2c, K, H, W, near=rasterizer.NEAR, precise=precise)
    ctx.sync()
    return rgb.cpu().numpy(), alpha.cpu().numpy()


@pytest.mark.parametrize("seed", [11, 12])
def test_matches_the_reference_renderer_images(ctx, seed):
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "raster_golden.npz"))
    _, n, H, W = (int(v) for v in g["case_%d" % seed])
    rgb, alpha = render(ctx, rasterizer.scene(seed, n, H, W), H, W, precise=True)
    assert np.abs(rgb - g["rgb_%d" % seed]).max() <= 1e-6     # double arithmetic: only the fp32 store differs
    assert np.abs(alpha - g["alpha_%d" % seed]).max() <= 1e-6


@pytest.mark.parametrize("n,H,W", [(1, 16, 16), (257, 33, 47), (5000, 128, 160), (100352, 224, 224)])
def test_matches_the_oracle(ctx, n, H, W):
    """Sizes around the chunk (256) and sort-block (2048) boundaries, a ragged image, and the reference's own size
    (100352 gaussians, 224 x 224)."""
    scene = rasterizer.scene(100 + n, n, H, W)
    ref_rgb, ref_alpha = rasterizer.render_view(*scene, H, W)
    rgb, alpha = render(ctx, scene, H, W, precise=True)
    assert np.abs(rgb - ref_rgb).max() <= 1e-6 and np.abs(alpha - ref_alpha).max() <= 1e-6
    # fp32 arithmetic: a gaussian whose alpha sits at the 1/255 gate or whose radius sits at an integer may fall on the
    # other side, which moves a pixel by at most about one gate step times its transmittance
    rgb32, alpha32 = render(ctx, scene, H, W, precise=False)
    assert np.abs(rgb32 - ref_rgb).max() <= 2e-2 and np.mean(np.abs(rgb32 - ref_rgb)) <= 1e-4
    assert np.abs(alpha32 - ref_alpha).max() <= 2e-2


def test_empty_and_culled_scenes(ctx):
    H, W = 32, 48
    means, covs, colors, opac, w2c, K = rasterizer.scene(5, 300, H, W)
    for m in (means[:0], means * 0 - 5.0):  # no gaussians; all behind the near plane
        k = len(m)
        rgb, alpha = render(ctx, (m, covs[:k], colors[:k], opac[:k], w2c, K), H, W, precise=True)
        assert not rgb.any() and not alpha.any()


def test_depth_order_not_input_order(ctx):
    """Shuffling the input must not change the image (ties aside): the compositing order is the depth order."""
    H, W, n = 64, 64, 1500
    means, covs, colors, opac, w2c, K = rasterizer.scene(21, n, H, W)
    perm = np.random.default_rng(3).permutation(n)
    a, _ = render(ctx, (means, covs, colors, opac, w2c, K), H, W, precise=True)
    b, _ = render(ctx, (means[perm], covs[perm], colors[perm], opac[perm], w2c, K), H, W, precise=True)
    assert np.abs(a - b).max() <= 1e-6


def test_bad_arguments_are_refused(ctx):
    means = torch.zeros(4, 3, device="cuda")
    with pytest.raises(vknn_b200.VkcError):
        ctx.raster_gaussians(means, torch.zeros(4, 3, 3, device="cuda"), means, torch.zeros(4, device="cuda"), np.eye(4), np.eye(3), 0, 16)
