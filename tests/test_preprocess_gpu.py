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


def _hash_u32(seed, view, point):
    """numpy statement of hash_u32 (include/adop/adop_math.h)."""
    with np.errstate(over="ignore"):
        seed, view = np.uint32(seed), np.uint32(view)
        h = seed * np.uint32(0x9E3779B1) + view * np.uint32(0x85EBCA77) + np.uint32(0x165667B1)
        h = np.full(point.shape, h, np.uint32)
        h ^= point.astype(np.uint32) + np.uint32(0x7F4A7C15) + (h << np.uint32(6)) + (h >> np.uint32(2))
        h ^= h >> np.uint32(16); h *= np.uint32(0x7FEB352D)
        h ^= h >> np.uint32(15); h *= np.uint32(0x846CA68B)
        h ^= h >> np.uint32(16)
    return h


def test_numpy_hash_is_the_library_hash(oracle):
    pts = np.array([0, 1, 2, 255, 256, 123456789, 2**31 - 1], np.int64)
    for seed in (0, 7, 0xDEADBEEF):
        want = np.array([oracle.lib.adop_oracle_hash(seed, 0, int(p)) for p in pts], np.uint32)
        assert np.array_equal(_hash_u32(seed, 0, pts), want)


@pytest.mark.parametrize("n,block,seed", [(10_000, 256, 0), (256 * 40, 256, 5), (100, 256, 1), (513, 256, 2), (1_000_003, 256, 9), (5000, 100, 3)])
def test_block_shuffle_order(cuda_lib, n, block, seed):
    blocks = n // block
    keys = (_hash_u32(seed, 0, np.arange(blocks)).astype(np.uint64) << np.uint64(32)) | np.arange(blocks, dtype=np.uint64)
    block_order = np.argsort(keys, kind="stable")
    want = np.arange(n)
    if blocks:
        want[: blocks * block] = (block_order[:, None] * block + np.arange(block)[None, :]).reshape(-1)
    got = preprocess.block_shuffle_order(n, "cuda:0", block=block, seed=seed).cpu().numpy()
    assert np.array_equal(got, want)
    assert np.array_equal(np.sort(got), np.arange(n))
    if blocks > 8:
        assert not np.array_equal(got, np.arange(n))


@pytest.mark.parametrize("n", [256, 255, 1000, 256 * 300 + 17])
def test_sort_blocks_by_radius_order(cuda_lib, n):
    rng = np.random.default_rng(n)
    w = rng.uniform(0, 1, n).astype(np.float32)
    w[::7] = w[3]            # equal radii: ordered by index
    w[5::50] = -w[5::50]     # the order is that of the floats, negative values included
    pos = np.zeros((n, 4), np.float32)
    pos[:, 3] = w
    want = np.arange(n)
    for b in range(n // 256):
        sl = slice(b * 256, (b + 1) * 256)
        want[sl] = b * 256 + np.lexsort((np.arange(256), w[sl]))
    got = preprocess.sort_blocks_by_radius_order(torch.from_numpy(pos).cuda()).cpu().numpy()
    assert np.array_equal(got, want)


def _knn_brute_force(xyz, k):
    """The (k+1)-th smallest float32 squared distance per point, square-rooted (all pairs)."""
    x = xyz.astype(np.float32)
    out = np.empty(len(x), np.float32)
    for i in range(len(x)):
        d = x[i] - x
        d2 = (d[:, 0] * d[:, 0] + d[:, 1] * d[:, 1]) + d[:, 2] * d[:, 2]
        out[i] = np.sqrt(np.partition(d2, k)[k]) if len(x) > k else np.inf
    return out


@pytest.mark.parametrize("n,k,shape", [(3000, 4, "ball"), (2500, 1, "ball"), (2000, 7, "sheet"), (1500, 16, "ball"), (3, 4, "ball"),
                                         (4000, 4, "clumps")])
def test_knn_distance_equals_all_pairs(cuda_lib, n, k, shape):
    rng = np.random.default_rng(n + k)
    xyz = rng.normal(0, 1, (n, 3)).astype(np.float32)
    if shape == "sheet":
        xyz[:, 2] = 0.25                                   # a flat cloud: zero extent on one axis
    if shape == "clumps":
        xyz[: n // 2] = xyz[: n // 2] * 0.001 + 5.0         # one dense clump far from a sparse cloud, plus duplicates
        xyz[10:20] = xyz[9]
    pos = np.concatenate([xyz, np.zeros((n, 1), np.float32)], axis=1)
    got = preprocess.knn_distance(torch.from_numpy(pos).cuda(), k=k).cpu().numpy()
    assert np.array_equal(got, _knn_brute_force(xyz, k))


def test_knn_distance_against_a_kd_tree(cuda_lib):
    """300 k points on surfaces (the benchmark's scene generator): scipy's KD-tree in float64 as the second opinion."""
    from scipy.spatial import cKDTree
    cfg = synth.make_config("c2", n_points=300_000, n_views=1, size=(64, 36))
    pos = cfg["arrays"]["position"]
    got = preprocess.knn_distance(torch.from_numpy(pos).cuda(), k=4).cpu().numpy()
    want = cKDTree(pos[:, :3].astype(np.float64)).query(pos[:, :3].astype(np.float64), k=5)[0][:, 4]
    assert np.allclose(got, want, rtol=2e-5, atol=1e-7)


def test_radius_sample(cuda_lib):
    n = 100_000
    dist = np.random.default_rng(1).uniform(0.001, 0.1, n).astype(np.float32)
    u = ((_hash_u32(3, 1, np.arange(n)) >> np.uint32(8)).astype(np.float32) + np.float32(1)) * np.float32(1.0 / 16777216.0)
    want = dist * np.sqrt(np.float32(1.0) / u)
    got = preprocess.radius_sample(torch.from_numpy(dist).cuda(), seed=3).cpu().numpy()
    assert np.array_equal(got, want.astype(np.float32))
    assert np.all(got >= dist)


def test_knn_gives_up_on_a_cloud_of_coincident_points(cuda_lib):
    """A quarter of a million points in one place: every query would have to walk all of them. The kernel gives up after
    a bounded number of visited points, the rest of the grid drains, and the call reports the size limit in seconds, not
    hours."""
    import time
    from adop_b200 import capi
    rng = np.random.default_rng(0)
    n_same, n_other = 250_000, 2_000
    pos = np.ones((n_same + n_other, 4), np.float32)
    pos[:n_same, :3] = [0.25, -0.5, 1.0]
    pos[n_same:, :3] = rng.uniform(-1, 1, (n_other, 3))
    t0 = time.time()
    with pytest.raises(capi.AdopError, match="size beyond the supported maximum"):
        preprocess.knn_distance(torch.from_numpy(pos).cuda(), k=4)
    torch.cuda.synchronize()
    assert time.time() - t0 < 20.0
    assert b"65536" in cuda_lib.adop_last_error()
    # an ordinary cloud right afterwards: the status word does not stick
    ok = rng.uniform(-1, 1, (5000, 4)).astype(np.float32)
    d = preprocess.knn_distance(torch.from_numpy(ok).cuda(), k=4)
    assert bool(torch.isfinite(d).all())


def test_scene_directory_preprocessed_and_rendered(cuda_lib, tmp_path):
    """A scene written in ADOP's directory layout, read back (scene_io), preprocessed on the GPU as the reference does once per
    scene (Morton reorder, drop-out radius from the 4 nearest neighbours: SceneData.cpp:100-103) and rendered: the images
    agree with those of the arrays the directory was written from (the poses went through text and two inversions, so
    depth agrees to rounding, not bit for bit)."""
    from adop_b200 import scene_io
    from adop_b200.raster import PointRasterizer, Scene
    dev = torch.device("cuda:0")
    cfg = synth.make_config("c2", n_points=60_000, n_views=3, size=(160, 90), sort=False)
    a = cfg["arrays"]
    q_cw, t_cw = scene_io.invert_poses(a["poses"][:, :4], a["poses"][:, 4:7])
    cams = [dict(w=160, h=90, K=a["intrinsics"][0, :5], distortion=a["intrinsics"][0, 5:13])]
    scene_io.save_scene_directory(str(tmp_path), a["position"][:, :3], np.concatenate([q_cw, t_cw], axis=1), cams)
    sc = scene_io.load_scene_directory(str(tmp_path))
    pos = torch.from_numpy(sc["arrays"]["position"]).to(dev)
    order = preprocess.morton_order(pos)
    pos = preprocess.permute_rows(pos, order)
    dist = preprocess.knn_distance(pos, k=4)
    assert bool(torch.isfinite(dist).all()) and float(dist.min()) > 0
    pos[:, 3] = dist
    tex = torch.from_numpy(a["texture"]).to(dev)
    tex_sorted = tex[:, order.long()].contiguous()      # descriptor i belongs to point i of the file's order
    common = dict(background=torch.from_numpy(a["background"]).to(dev), env_map=torch.from_numpy(a["env_map"]).to(dev))
    loaded = Scene(position=pos, texture=tex_sorted, poses=torch.from_numpy(sc["arrays"]["poses"]).to(dev),
                   intrinsics=torch.from_numpy(sc["arrays"]["intrinsics"]).to(dev), **common)
    source = Scene(position=torch.from_numpy(a["position"]).to(dev), texture=tex, poses=torch.from_numpy(a["poses"]).to(dev),
                   intrinsics=torch.from_numpy(a["intrinsics"]).to(dev), **common)
    ras = PointRasterizer(dev)
    f1 = ras.forward(loaded, sc["views"], cfg["params"], 4)
    f2 = PointRasterizer(dev).forward(source, cfg["views"], cfg["params"], 4)
    torch.cuda.synchronize()
    for l in range(4):
        same_depth = torch.isclose(f1.depths[l], f2.depths[l], rtol=1e-5, atol=1e-5)
        assert float(same_depth.float().mean()) > 0.999
        assert float((f1.weights[l] == f2.weights[l]).float().mean()) > 0.995
        ok = same_depth.expand_as(f1.colors[l]) & (f1.weights[l] == f2.weights[l]).expand_as(f1.colors[l])
        assert torch.allclose(f1.colors[l][ok], f2.colors[l][ok], rtol=1e-3, atol=1e-4)
