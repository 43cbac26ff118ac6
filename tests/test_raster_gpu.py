"""GPU parity of the rasterizer against the CPU checker, through the C ABI.

Bar: depth, weight and mask buffers bit-exact (integer-like data); colours of pixels that hold exactly one splat
bit-exact (nothing is summed); everything that the GPU sums with float atomics in an order of its own (colours of
multi-splat pixels, all gradients) per element within |a - b| <= 1e-4 |b| + 1e-5 max|b|: 1e-4 relative where atomic
ordering differs, and a floor of 1e-5 of the tensor's largest magnitude for elements whose terms cancel. Results that
involve no atomics are held to 1e-5 relative (RTOL_EXACT_ORDER).
"""
import numpy as np
import pytest
import torch

from adop_b200 import capi, synth
from adop_b200.raster import PointRasterizer, Scene

pytestmark = pytest.mark.gpu

RTOL = 1e-4              # sums formed by float atomics in GPU order
RTOL_EXACT_ORDER = 1e-5  # no atomics involved
FLOOR = 1e-5             # of the tensor's largest magnitude: the cancellation floor
floor_report = {}        # name -> (elements that needed the floor, elements): printed at the end of the session


def to_scene(arrays, dev="cuda:0"):
    return Scene(**{k: (torch.from_numpy(v).to(dev) if v is not None else None) for k, v in arrays.items()})


def close(a, b, rtol=RTOL, name="", floor=FLOOR):
    """Per element: |a - b| <= rtol |b| + floor max|b|. Records how many elements passed only thanks to the floor."""
    a = a.detach().cpu().numpy() if isinstance(a, torch.Tensor) else a
    a64, b64 = a.astype(np.float64), np.asarray(b).astype(np.float64)
    scale = max(float(np.abs(b64).max()), 1e-30) if b64.size else 1.0
    err = np.abs(a64 - b64)
    rel_ok = err <= rtol * np.abs(b64)
    ok = err <= rtol * np.abs(b64) + floor * scale
    needed = int((ok & ~rel_ok).sum())
    seen = floor_report.get(name, (0, 0))
    floor_report[name] = (seen[0] + needed, seen[1] + int(b64.size))
    if not ok.all():
        worst = int(np.argmax(err - rtol * np.abs(b64)))
        raise AssertionError(f"{name}: {int((~ok).sum())} of {b64.size} elements off; worst |a-b| = {err.flat[worst]:.3e} at "
                             f"b = {b64.flat[worst]:.3e} (max|b| = {scale:.3e})")


@pytest.fixture(scope="module", autouse=True)
def _print_floor_report():
    yield
    if floor_report:
        print("\nelements that needed the cancellation floor (1e-5 of the tensor's maximum):")
        for name, (needed, total) in sorted(floor_report.items()):
            if total:
                print(f"  {name:24s} {needed:>10d} of {total:>12d} ({100.0 * needed / total:.4f} %)")


def run_both(oracle, cfg, want_env=False, dropout_mask=None, record_visible=True, interleave=True, **bw):
    arrays, views, params, L = cfg["arrays"], cfg["views"], cfg["params"], cfg["num_layers"]
    grads = synth.upstream_gradients(cfg["meta"], batch=len(views))
    ref = oracle.forward(arrays, views, params, L, dropout_mask=dropout_mask)
    ref_b = oracle.backward(arrays, views, params, L, ref, grads, want_env=want_env, dropout_mask=dropout_mask, **bw)
    scene = to_scene(arrays)
    r = PointRasterizer("cuda:0", interleave_descriptors=interleave)
    dm = torch.from_numpy(dropout_mask).cuda() if dropout_mask is not None else None
    fwd = r.forward(scene, views, params, L, dropout_mask=dm, record_visible=record_visible)
    bwd = r.backward(scene, params, fwd, [torch.from_numpy(g).cuda() for g in grads], want_env=want_env,
                     dropout_mask=dm, **bw)
    torch.cuda.synchronize()
    return ref, ref_b, fwd, bwd


def check_forward(ref, fwd, L, masks=False):
    for l in range(L):
        d = fwd.depths[l].cpu().numpy()
        assert np.array_equal(d.view(np.uint32), ref["depths"][l].view(np.uint32)), f"depth layer {l} not bit-exact"
        w = fwd.weights[l].cpu().numpy()
        assert np.array_equal(w, ref["weights"][l]), f"weight layer {l}"
        c = fwd.colors[l].cpu().numpy()
        close(c, ref["colors"][l], name=f"colour layer {l}")
        # a pixel with at most one splat sums nothing: its colour is the descriptor (or the background / environment
        # map) itself, whatever the order of the atomics
        single = np.broadcast_to(w <= 1, c.shape)
        close(c[single], ref["colors"][l][single], rtol=RTOL_EXACT_ORDER, floor=0.0, name=f"colour layer {l}, <= 1 splat")
        if masks:
            assert np.array_equal(fwd.masks[l].cpu().numpy(), ref["masks"][l])


def check_backward(ref_b, bwd):
    for k in ("texture", "background", "points", "pose", "intrinsics", "env_map"):
        if ref_b.get(k) is None:
            assert bwd.get(k) is None
            continue
        close(bwd[k], ref_b[k], name=f"grad {k}")
    for k in ("count_pose", "count_intrinsics"):
        if ref_b.get(k) is not None:
            close(bwd[k], ref_b[k], rtol=1e-6, name=k)


@pytest.mark.parametrize("seed", [0, 1])
def test_c1_small_cloud(oracle, cuda_lib, seed):
    cfg = synth.make_config("c1", n_points=1 << 17, size=(256, 256), seed=seed)
    ref, ref_b, fwd, bwd = run_both(oracle, cfg)
    check_forward(ref, fwd, cfg["num_layers"])
    check_backward(ref_b, bwd)
    assert ref["weights"][0].sum() > 1000


def test_c1_full_size(oracle, cuda_lib):
    cfg = synth.make_config("c1")
    ref, ref_b, fwd, bwd = run_both(oracle, cfg)
    check_forward(ref, fwd, 4)
    check_backward(ref_b, bwd)


@pytest.mark.parametrize("listed", [True, False])
def test_c2_distortion_env_map_pose_grads(oracle, cuda_lib, listed):
    """listed: the backward pass walks the visible list the forward pass recorded; else it walks all points."""
    cfg = synth.make_config("c2", n_points=400_000, n_views=3, size=(480, 270))
    ref, ref_b, fwd, bwd = run_both(oracle, cfg, want_env=True, record_visible=listed)
    assert (fwd.visible is not None) == listed
    check_forward(ref, fwd, 4, masks=True)
    check_backward(ref_b, bwd)
    assert np.abs(ref_b["pose"]).max() > 0 and np.abs(ref_b["env_map"]).max() > 0


@pytest.mark.parametrize("listed", [True, False])
def test_c3_ocam(oracle, cuda_lib, listed):
    cfg = synth.make_config("c3", n_points=500_000, size=(480, 270))
    ref, ref_b, fwd, bwd = run_both(oracle, cfg, record_visible=listed)
    check_forward(ref, fwd, 4)
    check_backward(ref_b, bwd)
    assert ref["weights"][0].sum() > 1000


def test_visible_list_is_used_on_a_dense_cloud(oracle, cuda_lib):
    """Many points per pixel (the normal case): the list holds at least one point per covered pixel of the finest layer
    and at most one entry per accepted (point, layer) pair."""
    cfg = synth.make_config("c2", n_points=600_000, n_views=2, size=(160, 90))
    ref, ref_b, fwd, bwd = run_both(oracle, cfg, want_env=True)
    assert not bool(fwd.list_unusable().any())
    covered = [int((ref["weights"][0][b] > 0).sum()) for b in range(2)]
    accepted = [sum(int(ref["weights"][l][b].sum()) for l in range(4)) for b in range(2)]
    counts = fwd.entry_counts().cpu().numpy()
    assert all(p <= c <= a for c, p, a in zip(counts, covered, accepted))
    check_forward(ref, fwd, 4, masks=True)
    check_backward(ref_b, bwd)


def test_c5_eight_channels_six_layers(oracle, cuda_lib):
    cfg = synth.make_config("c5", n_points=300_000, n_views=2, size=(384, 216))
    ref, ref_b, fwd, bwd = run_both(oracle, cfg, want_env=True)
    check_forward(ref, fwd, 6, masks=True)
    check_backward(ref_b, bwd)


@pytest.mark.parametrize("interleave", [True, False])
@pytest.mark.parametrize("channels", [3, 16])
def test_other_channel_counts(oracle, cuda_lib, channels, interleave):
    """interleave: descriptors and their gradient go through the [T,C] working copies; else straight to the [C,T] planes."""
    cfg = synth.make_config("c1", n_points=50_000, size=(96, 64), channels=channels, layers=3)
    ref, ref_b, fwd, bwd = run_both(oracle, cfg, interleave=interleave)
    check_forward(ref, fwd, 3)
    check_backward(ref_b, bwd)


@pytest.mark.parametrize("layers,size", [(8, (512, 384)), (5, (200, 120)), (7, (320, 192))])
def test_deep_pyramids(oracle, cuda_lib, layers, size):
    """The largest layer count the header allows (8: the coarsest layer of a 512 x 384 view is 4 x 3 pixels) and two counts
    in between: the backward pass's staged-tile kernel has a variant of its own for more than four layers."""
    cfg = synth.make_config("c2", n_points=120_000, n_views=2, size=size, layers=layers)
    ref, ref_b, fwd, bwd = run_both(oracle, cfg, want_env=True)
    check_forward(ref, fwd, layers)
    check_backward(ref_b, bwd)
    assert not bool(fwd.list_unusable().any())


def test_odd_sizes_and_ragged_point_count(oracle, cuda_lib):
    # 135 -> 67 -> 33 by integer halving; N not a multiple of 32
    cfg = synth.make_config("c1", n_points=10_007, size=(135, 77), layers=3)
    ref, ref_b, fwd, bwd = run_both(oracle, cfg)
    check_forward(ref, fwd, 3)
    check_backward(ref_b, bwd)


@pytest.mark.parametrize("listed", [True, False])
@pytest.mark.parametrize("ghost", [0, 1])
def test_dropout_hash_and_ghost_gradients(oracle, cuda_lib, ghost, listed):
    cfg = synth.make_config("c1", n_points=80_000, size=(128, 128))
    cfg["params"].dropout = 0.25
    cfg["params"].dropout_seed = 7
    cfg["params"].ghost_gradients = ghost
    ref, ref_b, fwd, bwd = run_both(oracle, cfg, record_visible=listed)
    check_forward(ref, fwd, 4)
    check_backward(ref_b, bwd)
    assert np.abs(ref_b["points"]).max() > 0


def test_dropout_mask_all_and_none(oracle, cuda_lib):
    cfg = synth.make_config("c1", n_points=20_000, size=(64, 64))
    n = cfg["meta"]["n_points"]
    for value in (0, 1):
        mask = np.full((1, n), value, np.uint8)
        ref, ref_b, fwd, bwd = run_both(oracle, cfg, dropout_mask=mask)
        check_forward(ref, fwd, 4)
        check_backward(ref_b, bwd)
        if value == 1:  # everything dropped: depth still written (dropped points occlude), nothing blended
            assert ref["weights"][0].sum() == 0 and (ref["depths"][0] < 100000).any()


def test_planar_descriptor_path_without_list(oracle, cuda_lib):
    cfg = synth.make_config("c2", n_points=200_000, n_views=2, size=(240, 136))
    ref, ref_b, fwd, bwd = run_both(oracle, cfg, want_env=True, interleave=False, record_visible=False)
    check_forward(ref, fwd, 4, masks=True)
    check_backward(ref_b, bwd)


def test_normals_radius_dropout_and_index(oracle, cuda_lib):
    cfg = synth.make_config("c1", n_points=60_000, size=(128, 96))
    rng = np.random.default_rng(3)
    n = cfg["meta"]["n_points"]
    nrm = rng.normal(size=(n, 3))
    nrm /= np.linalg.norm(nrm, axis=1, keepdims=True)
    q = np.round((nrm + 1) * 0.5 * 1023).astype(np.uint32)
    cfg["arrays"]["normal"] = (q[:, 0] | (q[:, 1] << 10) | (q[:, 2] << 20)).astype(np.int32)
    cfg["arrays"]["index"] = rng.permutation(n).astype(np.int32)
    cfg["arrays"]["position"][:, 3] = rng.uniform(0.001, 0.02, n).astype(np.float32)
    cfg["params"].check_normal = 1
    cfg["params"].drop_out_points_by_radius = 1
    ref, ref_b, fwd, bwd = run_both(oracle, cfg)
    check_forward(ref, fwd, 4)
    check_backward(ref_b, bwd)
    assert 0 < ref["weights"][0].sum() < n


@pytest.mark.parametrize("normals,listed", [(False, True), (True, True), (False, False)])
def test_outlier_cloud(oracle, cuda_lib, normals, listed):
    """The optional second cloud (the reference's outlier cloud, PointRenderer.cu:1402-1441): rendered into the same depth,
    weight and colour buffers by the forward pass, ignored by the backward pass. Depth and weights bit-exact against the
    checker, colours and the main cloud's gradients within tolerance, with and without a visible list; with normals on both
    clouds the normal test applies to both; a drop-out mask is shared index by index."""
    cfg = synth.make_config("c2", n_points=300_000, n_views=3, size=(320, 180), seed=6)
    a, params = cfg["arrays"], cfg["params"]
    n = len(a["position"])
    rng = np.random.default_rng(8)
    # a sphere INSIDE the scene's bounding sphere, so that outliers land in front of and between the surfaces
    a.update(synth.outlier_cloud(a, 40_000, seed=2, distance=-0.55, with_normals=normals))
    if normals:
        nrm = rng.normal(size=(n, 3))
        a["normal"] = synth.pack_normals(nrm / np.linalg.norm(nrm, axis=1, keepdims=True))
        params.check_normal = 1
    mask = (rng.uniform(size=(len(cfg["views"]), n)) < 0.2).astype(np.uint8)
    plain = oracle.forward({k: v for k, v in a.items() if not k.startswith("outlier")}, cfg["views"], params, 4, dropout_mask=mask)
    ref, ref_b, fwd, bwd = run_both(oracle, cfg, want_env=True, dropout_mask=mask, record_visible=listed)
    assert (ref["weights"][0] != plain["weights"][0]).sum() > 1000 and (ref["depths"][0] < plain["depths"][0]).sum() > 1000
    check_forward(ref, fwd, 4)
    check_backward(ref_b, bwd)


def test_outlier_cloud_argument_checks(cuda_lib):
    cfg = synth.make_config("c1", n_points=1000, size=(64, 64))
    a = cfg["arrays"]
    a.update(synth.outlier_cloud(a, 500, seed=1))
    scene = to_scene(a)
    r = PointRasterizer("cuda:0")
    r.forward(scene, cfg["views"], cfg["params"], 4)
    # more outliers than main points: they would index the drop-out decisions out of range
    scene.outlier_position = torch.zeros((1001, 4), device="cuda:0")
    scene.outlier_index, scene.outlier_normal = None, None
    with pytest.raises(capi.AdopError, match="invalid argument"):
        r.forward(scene, cfg["views"], cfg["params"], 4)


@pytest.mark.parametrize("with_index", [False, True])
def test_touched_flags_cover_every_chunk_that_gets_a_gradient(cuda_lib, with_index):
    """The forward pass can flag the chunks of 256 consecutive points in which it listed a point for the backward pass. Every
    chunk in which the backward pass of the same views then adds a point or descriptor gradient must carry its flag (the
    multi-GPU exchange does not read unflagged chunks), chunks the views cannot see stay unflagged, and with an index
    array (descriptor columns in another order than the points) every texel chunk counts as touched."""
    cfg = synth.make_config("c2", n_points=400_000, n_views=2, size=(320, 180), seed=12)
    a = cfg["arrays"]
    n = len(a["position"])
    if with_index:
        a["index"] = np.random.default_rng(0).permutation(n).astype(np.int32)
    scene = to_scene(a)
    chunks = (n + 255) // 256
    flags_p = torch.full((chunks,), 7, dtype=torch.uint8, device="cuda:0")
    flags_t = torch.full((chunks,), 7, dtype=torch.uint8, device="cuda:0")
    r = PointRasterizer("cuda:0")
    fwd = r.forward(scene, cfg["views"], cfg["params"], 4, touched=(flags_p, flags_t))
    grads = [torch.from_numpy(g).cuda() for g in synth.upstream_gradients(cfg["meta"])]
    bwd = r.backward(scene, cfg["params"], fwd, grads, normalize=False)
    torch.cuda.synchronize()
    assert set(flags_p.unique().tolist()) <= {0, 1}
    pad = chunks * 256 - n
    got_p = torch.nn.functional.pad(bwd["points"][:, 3] > 0, (0, pad)).view(chunks, 256).any(dim=1)
    got_t = torch.nn.functional.pad((bwd["texture"] != 0).any(dim=0), (0, pad)).view(chunks, 256).any(dim=1)
    assert int(got_p.sum()) > 100 and int(got_t.sum()) > 100
    assert not bool((got_p & (flags_p == 0)).any()), "a chunk with point gradients is not flagged"
    assert not bool((got_t & (flags_t == 0)).any()), "a chunk with descriptor gradients is not flagged"
    assert 0.05 < float((flags_p != 0).float().mean()) < 0.95     # two views of an orbit do not see everything
    if with_index:
        assert bool((flags_t == 1).all())
    else:
        assert torch.equal(flags_t, flags_p)


def test_unusable_list_falls_back_to_all_points(oracle, cuda_lib):
    """A list whose header says that it is not usable: the backward pass finds the mark on the device (no host round
    trip), its tile kernels return at once and the all-points kernels behind them do the work, with the same result."""
    cfg = synth.make_config("c2", n_points=150_000, n_views=2, size=(240, 136))
    arrays, views, params, L = cfg["arrays"], cfg["views"], cfg["params"], cfg["num_layers"]
    grads = synth.upstream_gradients(cfg["meta"], batch=len(views))
    ref = oracle.forward(arrays, views, params, L)
    ref_b = oracle.backward(arrays, views, params, L, ref, grads, want_env=True)
    scene = to_scene(arrays)
    r = PointRasterizer("cuda:0")
    fwd = r.forward(scene, views, params, L)
    fwd.visible[:, 2048 + 2] = 1
    assert bool(fwd.list_unusable().all())
    bwd = r.backward(scene, params, fwd, [torch.from_numpy(g).cuda() for g in grads], want_env=True)
    torch.cuda.synchronize()
    check_forward(ref, fwd, L, masks=True)
    check_backward(ref_b, bwd)


def test_overflowing_tile_bucket_marks_the_list_unusable(oracle, cuda_lib):
    """A cluster of coplanar points that all pass the depth test inside one screen tile: more visible points than a tile's
    bucket holds (2048 here). The forward pass marks the list unusable and the backward pass walks all points."""
    cfg = synth.make_config("c1", n_points=6000, size=(64, 64), layers=2)
    rng = np.random.default_rng(5)
    pos = cfg["arrays"]["position"]
    pos[:, 0] = rng.uniform(-0.1, -0.02, pos.shape[0])  # image x in 7 .. 27, y in 37 .. 47: one 32 x 16 tile
    pos[:, 1] = rng.uniform(0.02, 0.1, pos.shape[0])
    pos[:, 2] = 3.0
    ref, ref_b, fwd, bwd = run_both(oracle, cfg)
    assert bool(fwd.list_unusable().all())
    assert ref["weights"][0].sum() > 2048
    check_forward(ref, fwd, 2)
    check_backward(ref_b, bwd)


def test_second_backward_on_the_same_list(oracle, cuda_lib):
    """The backward pass turns the list's entries into work items, so the list serves one backward call; it is marked
    consumed and a second call on the same forward result walks all points: same gradients."""
    cfg = synth.make_config("c2", n_points=150_000, n_views=2, size=(240, 136))
    arrays, views, params, L = cfg["arrays"], cfg["views"], cfg["params"], cfg["num_layers"]
    grads = [torch.from_numpy(g).cuda() for g in synth.upstream_gradients(cfg["meta"], batch=len(views))]
    scene = to_scene(arrays)
    r = PointRasterizer("cuda:0")
    fwd = r.forward(scene, views, params, L)
    first = {k: (v.clone() if v is not None else None) for k, v in r.backward(scene, params, fwd, grads, want_env=True).items()}
    assert bool((fwd.visible[:, 2048 + 3] == 1).all())
    second = r.backward(scene, params, fwd, grads, want_env=True)
    torch.cuda.synchronize()
    for k in ("texture", "background", "points", "pose", "intrinsics", "env_map"):
        close(second[k], first[k].cpu().numpy(), name=f"second backward {k}")


def test_small_workspace_matches_full_workspace(cuda_lib):
    """With the full workspace the depth prepass hands projected points to the blend kernel; with the small one the blend
    kernel projects again. Same depth and weight bits, colours and gradients within the atomic-order tolerance."""
    cfg = synth.make_config("c2", n_points=300_000, n_views=5, size=(320, 180))
    scene = to_scene(cfg["arrays"])
    grads = [torch.from_numpy(g).cuda() for g in synth.upstream_gradients(cfg["meta"])]
    out = []
    for full in (False, True):
        r = PointRasterizer("cuda:0", full_workspace=full)
        fwd = r.forward(scene, cfg["views"], cfg["params"], 4)
        bwd = r.backward(scene, cfg["params"], fwd, grads, want_env=True)
        out.append((fwd, bwd))
    torch.cuda.synchronize()
    (fa, ba), (fb, bb) = out
    for l in range(4):
        assert torch.equal(fa.depths[l], fb.depths[l]) and torch.equal(fa.weights[l], fb.weights[l])
        close(fa.colors[l], fb.colors[l].cpu().numpy(), name=f"small vs full colour {l}")
    for k in ("texture", "background", "points", "pose", "intrinsics", "env_map"):
        close(ba[k], bb[k].cpu().numpy(), name=f"small vs full grad {k}")


def test_backward_mode_4(oracle, cuda_lib):
    cfg = synth.make_config("c1", n_points=40_000, size=(96, 96))
    cfg["params"].test_backward_mode = 4
    ref, ref_b, fwd, bwd = run_both(oracle, cfg)
    check_backward(ref_b, bwd)


def test_no_visible_points(oracle, cuda_lib):
    cfg = synth.make_config("c1", n_points=1000, size=(64, 64))
    cfg["arrays"]["position"][:, 2] = -5.0  # everything behind the camera
    cfg["arrays"]["background"][:] = [0.1, 0.2, 0.3, 0.4]
    ref, ref_b, fwd, bwd = run_both(oracle, cfg)
    check_forward(ref, fwd, 4)
    assert float(fwd.weights[0].sum()) == 0
    assert torch.allclose(fwd.colors[0][0, :, 5, 5].cpu(), torch.tensor([0.1, 0.2, 0.3, 0.4]))
    close(bwd["background"], ref_b["background"], name="background gradient")


def test_empty_cloud(oracle, cuda_lib):
    """No points at all: every pixel takes the background (and the environment map), the descriptor gradient is zero and the
    background gradient is the sum of the upstream gradient over all pixels."""
    cfg = synth.make_config("c2", n_points=1000, n_views=2, size=(96, 54))
    a = cfg["arrays"]
    a["position"] = np.zeros((0, 4), np.float32)
    ref, ref_b, fwd, bwd = run_both(oracle, cfg, want_env=True)
    check_forward(ref, fwd, 4)
    check_backward(ref_b, bwd)
    assert float(fwd.weights[0].sum()) == 0 and not bool(bwd["texture"].any())


def test_thousands_of_points_on_one_pixel(oracle, cuda_lib):
    """Collisions: 60 000 points at one position (one pixel per layer holds them all, its tile's bucket of the visible list
    overflows and the backward pass takes the all-points kernels) among a normal cloud. Depth and the counts stay exact."""
    cfg = synth.make_config("c1", n_points=100_000, size=(128, 128))
    a = cfg["arrays"]
    a["position"][:60_000, :3] = np.array([0.1, -0.05, 3.0], np.float32)
    ref, ref_b, fwd, bwd = run_both(oracle, cfg)
    check_forward(ref, fwd, 4)
    check_backward(ref_b, bwd)
    assert float(ref["weights"][0].max()) >= 60_000 and bool(fwd.list_unusable().all())


def test_points_that_are_not_finite(oracle, cuda_lib):
    """NaN, infinite and absurdly distant coordinates: such points take part in nothing, on either side, and their
    neighbours in memory are not disturbed."""
    cfg = synth.make_config("c2", n_points=80_000, n_views=2, size=(160, 90))
    a = cfg["arrays"]
    rng = np.random.default_rng(5)
    idx = rng.choice(80_000, 900, replace=False)
    a["position"][idx[:300], 0] = np.nan
    a["position"][idx[300:600], 1] = np.inf
    a["position"][idx[600:], 2] = -3e38
    ref, ref_b, fwd, bwd = run_both(oracle, cfg, want_env=True)
    check_forward(ref, fwd, 4)
    check_backward(ref_b, bwd)
    assert not bool(torch.isnan(bwd["points"]).any()) and not bool(bwd["points"][torch.from_numpy(idx).cuda()].any())


def test_unnormalized_then_normalize_matches(oracle, cuda_lib):
    cfg = synth.make_config("c1", n_points=50_000, size=(128, 128))
    ref, ref_b, fwd, bwd = run_both(oracle, cfg, normalize=False)
    check_backward(ref_b, bwd)
    r = PointRasterizer("cuda:0")
    r.normalize_gradients(bwd)
    ref_n = oracle.backward(cfg["arrays"], cfg["views"], cfg["params"], 4, ref,
                            synth.upstream_gradients(cfg["meta"], batch=1))
    check_backward(ref_n, bwd)


def test_descriptor_gradient_is_exact_adjoint(cuda_lib):
    """The op is linear in the descriptors: <G, forward(T)> == <backward(G), T> when the background is 0. One layer,
    because with more the backward pass stops at a point's first depth failure while the forward pass goes on
    (PointRenderer.cu:380 vs :462), so their accept sets differ on purpose."""
    cfg = synth.make_config("c1", n_points=100_000, size=(128, 128), layers=1)
    scene = to_scene(cfg["arrays"])
    r = PointRasterizer("cuda:0")
    fwd = r.forward(scene, cfg["views"], cfg["params"], 1)
    grads = [torch.from_numpy(g).cuda() for g in synth.upstream_gradients(cfg["meta"], batch=1)]
    bwd = r.backward(scene, cfg["params"], fwd, grads, want_points=False, want_pose=False, want_intrinsics=False)
    lhs = sum(float((g.double() * c.double()).sum()) for g, c in zip(grads, fwd.colors))
    rhs = float((bwd["texture"].double() * scene.texture.double()).sum())
    assert abs(lhs - rhs) <= 1e-4 * max(abs(lhs), 1.0)


def test_point_order_invariance(cuda_lib):
    cfg = synth.make_config("c1", n_points=60_000, size=(128, 128))
    scene = to_scene(cfg["arrays"])
    r = PointRasterizer("cuda:0")
    a = r.forward(scene, cfg["views"], cfg["params"], 4)
    perm = torch.randperm(scene.position.shape[0], device="cuda")
    scene2 = Scene(scene.position[perm].contiguous(), scene.texture[:, perm].contiguous(), scene.background,
                   scene.poses, scene.intrinsics)
    r2 = PointRasterizer("cuda:0")
    b = r2.forward(scene2, cfg["views"], cfg["params"], 4)
    for l in range(4):
        assert torch.equal(a.depths[l], b.depths[l]) and torch.equal(a.weights[l], b.weights[l])
        assert torch.allclose(a.colors[l], b.colors[l], rtol=1e-4, atol=1e-5)


def test_workspace_is_clean_across_calls(cuda_lib):
    cfg = synth.make_config("c2", n_points=100_000, n_views=2, size=(320, 180))
    scene = to_scene(cfg["arrays"])
    r = PointRasterizer("cuda:0")
    a = r.forward(scene, cfg["views"], cfg["params"], 4)
    first = [c.clone() for c in a.colors]
    b = r.forward(scene, cfg["views"], cfg["params"], 4, out=a)
    for x, y in zip(first, b.colors):
        assert torch.allclose(x, y, rtol=1e-4, atol=1e-5)


def test_argument_errors(cuda_lib):
    cfg = synth.make_config("c1", n_points=1000, size=(64, 64))
    scene = to_scene(cfg["arrays"])
    r = PointRasterizer("cuda:0")
    bad = [dict(cfg["views"][0], image_index=5)]
    with pytest.raises(capi.AdopError, match="invalid argument"):
        r.forward(scene, bad, cfg["params"], 4)
    with pytest.raises((capi.AdopError, ValueError)):
        r.forward(scene, cfg["views"], cfg["params"], 9)
    with pytest.raises(capi.AdopError):
        r.forward(Scene(**{k: (v.cpu() if v is not None else None) for k, v in scene.tensors().items()}),
                  cfg["views"], cfg["params"], 4)
    # five descriptor channels: inside the header's bound, but no kernels are built for it
    five = synth.make_config("c1", n_points=1000, size=(64, 64), channels=5)
    with pytest.raises(capi.AdopError, match="built for 3, 4, 8 and 16"):
        PointRasterizer("cuda:0").forward(to_scene(five["arrays"]), five["views"], five["params"], 4)


def test_c2_full_size_one_view_against_checker(oracle, cuda_lib):
    """The benchmark's own size (10 M points, 1920x1080, 4 layers) for one view: depth and weight bit-exact, colours and all
    gradients within tolerance. The checker runs with its OpenMP point loops (depth / weight do not depend on the order)."""
    cfg = synth.make_config("c2", n_views=1)
    arrays, views, params, L = cfg["arrays"], cfg["views"], cfg["params"], cfg["num_layers"]
    grads = synth.upstream_gradients(cfg["meta"], batch=1)
    ref = oracle.forward(arrays, views, params, L, threads=16)
    ref_b = oracle.backward(arrays, views, params, L, ref, grads, want_env=True, threads=16)
    scene = to_scene(arrays)
    r = PointRasterizer("cuda:0")
    fwd = r.forward(scene, views, params, L)
    bwd = r.backward(scene, params, fwd, [torch.from_numpy(g).cuda() for g in grads], want_env=True)
    torch.cuda.synchronize()
    assert not bool(fwd.list_unusable().any())
    check_forward(ref, fwd, L, masks=True)
    check_backward(ref_b, bwd)


def _full_size_case(oracle, cfg, want_env):
    arrays, views, params, L = cfg["arrays"], cfg["views"], cfg["params"], cfg["num_layers"]
    grads = synth.upstream_gradients(cfg["meta"], batch=len(views))
    ref = oracle.forward(arrays, views, params, L, threads=16)
    ref_b = oracle.backward(arrays, views, params, L, ref, grads, want_env=want_env, threads=16)
    scene = to_scene(arrays)
    r = PointRasterizer("cuda:0")
    fwd = r.forward(scene, views, params, L)
    bwd = r.backward(scene, params, fwd, [torch.from_numpy(g).cuda() for g in grads], want_env=want_env)
    torch.cuda.synchronize()
    assert not bool(fwd.list_unusable().any())
    check_forward(ref, fwd, L, masks=bool(params.output_background_mask))
    check_backward(ref_b, bwd)
    return ref


def test_c3_omnidirectional_10m_points_full_hd_against_checker(oracle, cuda_lib):
    """The viewer configuration's camera and image size (omnidirectional model, 1920x1080, 4 layers) on 10 M of its points,
    forward and backward."""
    ref = _full_size_case(oracle, synth.make_config("c3", n_points=10_000_000), want_env=False)
    assert ref["weights"][0].sum() > 100_000


def test_c4_30m_points_one_view_against_checker(oracle, cuda_lib):
    """The multi-GPU configuration's cloud (30 M points on surfaces) for one 1080p view."""
    _full_size_case(oracle, synth.make_config("c4", n_views=1), want_env=True)


def test_c5_one_4k_view_8_channels_6_layers_against_checker(oracle, cuda_lib):
    """The HDR configuration's image size, channel and layer count (3840x2160, 8 channels, 6 layers, 2048x1024 environment
    map) for one view on 6 M points."""
    _full_size_case(oracle, synth.make_config("c5", n_points=6_000_000, n_views=1), want_env=True)


def test_full_size_properties_16_views(cuda_lib):
    """Size-independent properties on the full benchmark batch (10 M points x 16 views), no checker involved:
    every listed point has at least one accepted layer, so the list length lies between the points accepted on the
    finest layer and the sum of all weights; the background mask is the indicator of weight > 0; depth is 100000 exactly
    where nothing landed on the finest layer; a second forward pass reproduces depth and weight bit for bit."""
    cfg = synth.make_config("c2")
    scene = to_scene(cfg["arrays"])
    r = PointRasterizer("cuda:0")
    fwd = r.forward(scene, cfg["views"], cfg["params"], 4)
    torch.cuda.synchronize()
    assert not bool(fwd.list_unusable().any())
    splats = fwd.entry_counts().double()
    w_all = sum(w.double().sum(dim=(1, 2, 3)) for w in fwd.weights)
    w0 = fwd.weights[0].double().sum(dim=(1, 2, 3))
    assert bool((splats <= w_all).all()) and bool((splats >= w0).all())
    for l in range(4):
        assert torch.equal(fwd.masks[l], (fwd.weights[l] > 0).float())
        assert bool(((fwd.depths[l] < 100000) | (fwd.weights[l] == 0)).all())
    d0, w0t = [d.clone() for d in fwd.depths], [w.clone() for w in fwd.weights]
    fwd = r.forward(scene, cfg["views"], cfg["params"], 4, out=fwd)
    for l in range(4):
        assert torch.equal(fwd.depths[l], d0[l]) and torch.equal(fwd.weights[l], w0t[l])


def test_forward_backward_replay_from_a_cuda_graph(oracle, cuda_lib):
    """After one warm-up call nothing in the library synchronises or allocates, so a whole forward + backward step can be
    captured into a CUDA graph and replayed (what a launch-bound small workload wants)."""
    cfg = synth.make_config("c1", n_points=50_000, size=(128, 128))
    arrays, views, params, L = cfg["arrays"], cfg["views"], cfg["params"], cfg["num_layers"]
    grads = synth.upstream_gradients(cfg["meta"], batch=1)
    ref = oracle.forward(arrays, views, params, L)
    ref_b = oracle.backward(arrays, views, params, L, ref, grads)
    scene = to_scene(arrays)
    r = PointRasterizer("cuda:0")
    g = [torch.from_numpy(x).cuda() for x in grads]
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        fwd = r.forward(scene, views, params, L)
        bwd = r.backward(scene, params, fwd, g)
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            r.forward(scene, views, params, L, out=fwd)
            r.backward(scene, params, fwd, g, out=bwd)
    for t in fwd.colors + fwd.depths + fwd.weights + [bwd["texture"], bwd["points"], bwd["pose"]]:
        t.zero_()
    graph.replay()
    torch.cuda.synchronize()
    check_forward(ref, fwd, L)
    check_backward(ref_b, bwd)


def test_many_views_crops_two_cameras_shared_texels(oracle, cuda_lib):
    """70 views (more than one camera-record chunk of 64), each with its own crop transform (zoom + shift + skew, as the
    training crops of Dataset.cpp:140-171 produce), two cameras with different intrinsics, views that repeat an image
    index (their pose gradients add up), and an index tensor in which pairs of points share a descriptor."""
    rng = np.random.default_rng(11)
    cfg = synth.make_config("c2", n_points=60_000, n_views=8, size=(96, 64))
    a = cfg["arrays"]
    n = cfg["meta"]["n_points"]
    a["index"] = (np.arange(n) // 2).astype(np.int32)           # two points per texel
    a["texture"] = np.ascontiguousarray(a["texture"][:, : (n + 1) // 2])
    intr2 = a["intrinsics"].copy()
    intr2[0, :4] *= 1.1
    # the second camera has all eight distortion coefficients (the first one only k1, k2: the shorter radial-only form)
    intr2[0, 5:13] = [-0.05, 0.01, 0.002, 0.01, -0.003, 0.001, 0.0005, -0.0004]
    a["intrinsics"] = np.ascontiguousarray(np.concatenate([a["intrinsics"], intr2]))
    views = []
    for k in range(70):
        zoom = rng.uniform(0.8, 1.6)
        views.append(dict(w=96, h=64, image_index=int(rng.integers(0, 8)), camera_index=int(k % 2), camera_model=0,
                          crop=(zoom, zoom * rng.uniform(0.95, 1.05), rng.uniform(-20, 5), rng.uniform(-12, 4), rng.uniform(-0.02, 0.02))))
    cfg["views"] = views
    ref, ref_b, fwd, bwd = run_both(oracle, cfg, want_env=True)
    check_forward(ref, fwd, 4, masks=True)
    check_backward(ref_b, bwd)
    assert (ref_b["count_pose"] > 0).sum() >= 6 and np.all(ref_b["count_intrinsics"] > 0)


def test_accumulate_adds_to_existing_gradients(cuda_lib):
    """accumulate = 1 adds this call's sums to what the buffers hold (two half-batches = one full batch)."""
    import ctypes as C
    from adop_b200.raster import fill_scene_struct
    cfg = synth.make_config("c2", n_points=80_000, n_views=4, size=(128, 72))
    scene = to_scene(cfg["arrays"])
    r = PointRasterizer("cuda:0", interleave_descriptors=False)
    grads = [torch.from_numpy(g).cuda() for g in synth.upstream_gradients(cfg["meta"])]
    fwd = r.forward(scene, cfg["views"], cfg["params"], 4)
    full = r.backward(scene, cfg["params"], fwd, grads, want_env=True, normalize=False)
    full = {k: (v.clone() if v is not None else None) for k, v in full.items()}
    acc = None
    lib = r.lib
    for half in (slice(0, 2), slice(2, 4)):
        views = cfg["views"][half]
        f2 = r.forward(scene, views, cfg["params"], 4)
        g2 = [g[half].contiguous() for g in grads]
        if acc is None:
            acc = r.backward(scene, cfg["params"], f2, g2, want_env=True, normalize=False)
            continue
        # second half: same buffers, accumulate = 1, straight through the C ABI
        va = capi.make_views(views)
        sc = fill_scene_struct(scene.tensors(), lambda t: t.data_ptr())
        io = capi.AdopBackwardIO()
        for l in range(4):
            io.layers[l].color, io.layers[l].depth = f2.colors[l].data_ptr(), f2.depths[l].data_ptr()
            io.layers[l].weight = f2.weights[l].data_ptr()
            io.grad_color[l] = g2[l].data_ptr()
        io.grad_texture, io.grad_background, io.grad_points = acc["texture"].data_ptr(), acc["background"].data_ptr(), acc["points"].data_ptr()
        io.grad_pose, io.count_pose = acc["pose"].data_ptr(), acc["count_pose"].data_ptr()
        io.grad_intrinsics, io.count_intrinsics = acc["intrinsics"].data_ptr(), acc["count_intrinsics"].data_ptr()
        io.grad_env_map = acc["env_map"].data_ptr()
        io.accumulate, io.normalize = 1, 0
        ws = r._workspace(128, 72, 4, 4, scene.position.shape[0], 2)
        io.workspace, io.workspace_bytes = ws.data_ptr(), ws.numel()
        io.visible_list = f2.visible.data_ptr()
        st = lib.adop_raster_backward(C.byref(sc), va, 2, C.byref(cfg["params"]), 4, C.byref(io), None)
        assert st == 0, lib.adop_last_error()
    torch.cuda.synchronize()
    for k in ("texture", "background", "points", "pose", "count_pose", "intrinsics", "count_intrinsics", "env_map"):
        close(acc[k], full[k].cpu().numpy(), name=k)


@pytest.mark.gpu
def test_packed_depth_index_word_matches_the_cpu_checker(oracle, cuda_lib):
    """Optional packed depth|index planes: bit-exact against the CPU checker (the word does not depend on the order in
    which the GPU visits the points), high word identical to the depth buffer, everything else unchanged."""
    cfg = synth.make_config("c2", n_points=80_000, n_views=5, size=(160, 90))
    ref = oracle.forward(cfg["arrays"], cfg["views"], cfg["params"], 4, packed_depth=True)
    dev = torch.device("cuda:0")
    scene = Scene(**{k: (torch.from_numpy(v).to(dev) if v is not None else None) for k, v in cfg["arrays"].items()})
    ras = PointRasterizer(dev)
    fwd = ras.forward(scene, cfg["views"], cfg["params"], 4, packed_depth=True)
    plain = ras.forward(scene, cfg["views"], cfg["params"], 4)
    torch.cuda.synchronize()
    for l in range(4):
        got = fwd.packed[l].cpu().numpy().view(np.uint64)
        assert np.array_equal(got, ref["packed"][l])
        assert np.array_equal((got >> np.uint64(32)).astype(np.uint32), fwd.depths[l].cpu().numpy().view(np.uint32))
        assert torch.equal(fwd.depths[l], plain.depths[l]) and torch.equal(fwd.weights[l], plain.weights[l])
