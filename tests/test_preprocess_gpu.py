"""GPU Morton reorder against the numpy statement of the same key (adop_b200/synth.py), bit for bit, and the
row permutation against torch indexing."""
import numpy as np
import pytest
import torch

from adop_b200 import preprocess, synth
from adop_b200.raster import PointRasterizer, Scene

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n", [1, 31, 256, 2048, 2049, 70_001, 1_500_000])
def test_morton_order_equals_the_numpy_statement(cuda_lib, n):
    rng = np.random.default_rng(n)
    xyz = rng.normal(0, 2, (n, 3)).astype(np.float32)
    if n > 1000:
        xyz[n // 2: n // 2 + 500] = xyz[7]            # equal keys: the sort must keep their order
        xyz[:200, 2] = xyz[:200, 2].round(1)          # many equal coordinates on one axis
        xyz[5, 0] = 1e6                               # an outlier stretches the bounding box: most keys share high bits
    pos = np.concatenate([xyz, rng.uniform(0, 1, (n, 1)).astype(np.float32)], axis=1)
    want = synth.morton_order(xyz)
    got = preprocess.morton_order(torch.from_numpy(pos).cuda())
    torch.cuda.synchronize()
    assert np.array_equal(got.cpu().numpy().astype(np.int64), want)


def test_morton_order_of_a_degenerate_cloud(cuda_lib):
    """All points equal (zero extent on every axis): every key is 0 and the order is the identity."""
    pos = torch.ones((5000, 4), device="cuda")
    got = preprocess.morton_order(pos)
    assert torch.equal(got.cpu(), torch.arange(5000, dtype=torch.int32))


@pytest.mark.parametrize("shape,dtype", [((1000, 4), torch.float32), ((1000,), torch.int32), ((1000, 3), torch.float32),
                                          ((1000, 2), torch.float32), ((513, 8), torch.float32), ((77, 16), torch.float32)])
def test_permute_rows(cuda_lib, shape, dtype):
    g = torch.Generator(device="cuda")
    g.manual_seed(3)
    t = (torch.randn(shape, device="cuda", generator=g) * 100).to(dtype)
    order = torch.randperm(shape[0], device="cuda", generator=g).to(torch.int32)
    out = preprocess.permute_rows(t, order)
    assert torch.equal(out, t[order.long()])


def test_reordering_a_scene_leaves_the_images_unchanged(cuda_lib):
    """The rasterizer does not depend on the order of the points: depth and weights bit-exact, colours up to the order
    of the float additions; the same holds for the descriptor gradients mapped back through the permutation."""
    dev = torch.device("cuda:0")
    cfg = synth.make_config("c2", n_points=120_000, n_views=2, size=(192, 108))
    a = dict(cfg["arrays"])
    rng = np.random.default_rng(0)
    shuffle = rng.permutation(a["position"].shape[0])
    a["position"] = np.ascontiguousarray(a["position"][shuffle])          # undo the generator's own Morton sort
    a["texture"] = np.ascontiguousarray(a["texture"][:, shuffle])
    scene = Scene(**{k: (torch.from_numpy(v).to(dev) if v is not None else None) for k, v in a.items()})
    sorted_scene, order = preprocess.reorder_scene(scene)
    ras = PointRasterizer(dev)
    f0 = ras.forward(scene, cfg["views"], cfg["params"], 4)
    f1 = ras.forward(sorted_scene, cfg["views"], cfg["params"], 4)
    for l in range(4):
        assert torch.equal(f0.depths[l], f1.depths[l]) and torch.equal(f0.weights[l], f1.weights[l])
        assert torch.allclose(f0.colors[l], f1.colors[l], rtol=1e-4, atol=1e-5)
    grads = [torch.randn_like(c) for c in f0.colors]
    b0 = ras.backward(scene, cfg["params"], f0, grads)
    f1 = ras.forward(sorted_scene, cfg["views"], cfg["params"], 4)
    b1 = ras.backward(sorted_scene, cfg["params"], f1, grads)
    assert torch.allclose(b0["texture"][:, order.long()], b1["texture"], rtol=1e-4, atol=1e-5)
    # the sorted cloud is in curve order: its keys are non-decreasing
    again = preprocess.morton_order(sorted_scene.position)
    assert torch.equal(again.cpu(), torch.arange(order.numel(), dtype=torch.int32))
