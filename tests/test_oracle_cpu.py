"""CPU tests (no GPU): the CPU checker against independent pins, and the C-ABI library's exported symbols.

The reference has no tests or golden vectors for this path, so the checker is pinned by things that do not share its
code: a float64 numpy restatement of the published camera models (tests/f64_model.py), central finite differences for
every Jacobian chain, torch's CPU grid_sample for the environment map and the tonemapper, and invariants of the
rasterization itself.
"""
import ctypes
import os

import numpy as np
import pytest
import torch

from adop_b200 import capi, synth
from tests import f64_model as fm

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


# ---------------------------------------------------------------------------------------------- arithmetic
def test_own_atan_family_matches_libm(oracle):
    lib = oracle.lib
    ts = np.concatenate([np.linspace(-50, 50, 4001), np.linspace(-1.2, 1.2, 4001), [0.0, 1e-8, -1e-8, 1e6, -1e6]])
    for t in ts:
        assert abs(lib.adop_oracle_atan(float(t)) - np.arctan(t)) < 3e-7
    rng = np.random.default_rng(0)
    for y, x in rng.normal(size=(4000, 2)):
        assert abs(lib.adop_oracle_atan2(float(y), float(x)) - np.arctan2(y, x)) < 5e-7
    for y, x in [(0, 1), (0, -1), (1, 0), (-1, 0), (0, 0)]:
        assert abs(lib.adop_oracle_atan2(float(y), float(x)) - np.arctan2(y, x)) < 5e-7
    for c in np.linspace(-1, 1, 2001):
        assert abs(lib.adop_oracle_acos(float(c)) - np.arccos(c)) < 1e-6


def test_round_half_even(oracle):
    lib = oracle.lib
    cases = {0.5: 0, 1.5: 2, 2.5: 2, -0.5: 0, -1.5: -2, 3.4999: 3, 1e20: 1000000000, -1e20: -1000000000}
    for x, want in cases.items():
        assert lib.adop_oracle_round(x) == want
    assert lib.adop_oracle_round(float("nan")) == -1000000000  # lands outside every image


def test_normal_packing_roundtrip(oracle):
    rng = np.random.default_rng(1)
    out = np.zeros(3, np.float32)
    for n in rng.normal(size=(200, 3)):
        n /= np.linalg.norm(n)
        e = oracle.lib.adop_oracle_pack_normal(*map(float, n))
        oracle.lib.adop_oracle_unpack_normal(e, out.ctypes.data)
        assert np.abs(out - n).max() < 1.1e-3


def test_dropout_hash_rate_and_determinism(oracle):
    lib = oracle.lib
    n = 200000
    d = np.array([lib.adop_oracle_dropout(0.25, 3, 1, i) for i in range(0, n, 7)])
    assert abs(d.mean() - 0.25) < 0.01
    assert lib.adop_oracle_dropout(0.0, 3, 1, 5) == 0
    assert lib.adop_oracle_hash(1, 2, 3) == lib.adop_oracle_hash(1, 2, 3) != lib.adop_oracle_hash(1, 3, 2)


def _pinhole_case(seed=0, n=300):
    rng = np.random.default_rng(seed)
    pts = np.stack([rng.normal(0, 1, n), rng.normal(0, 1, n), rng.uniform(2, 6, n), np.full(n, 0.01)], 1).astype(np.float32)
    pose = synth.look_at_pose((0.5, -0.3, -1.0), (0.1, 0.2, 4.0))
    intr = np.array([[420.0, 410.0, 250.0, 190.0, 0.7, -0.12, 0.03, 0.004, 0.01, -0.005, 0.002, 0.003, -0.002]], np.float32)
    arrays = dict(position=pts, normal=None, index=None, texture=np.zeros((4, n), np.float32),
                  background=np.zeros(4, np.float32), poses=pose[None].copy(), intrinsics=intr, env_map=None)
    view = dict(w=512, h=384, image_index=0, camera_index=0, camera_model=capi.CAMERA_PINHOLE_DISTORTION,
                crop=(0.9, 1.1, 12.0, -7.0, 0.05))
    return arrays, view


def _ocam_case(seed=0, n=300):
    rng = np.random.default_rng(seed)
    pts = np.stack([rng.uniform(-6, 6, n), rng.uniform(-6, 6, n), rng.uniform(0.5, 4, n), np.full(n, 0.01)], 1).astype(np.float32)
    pose = synth.look_at_pose((0.2, 0.1, -0.5), (0.0, 0.0, 3.0))
    coef, theta_max = synth.ocam_world2cam_poly()
    intr = np.concatenate([[1.01, 0.002, -0.003, 960.0, 540.0], coef]).astype(np.float32)[None]
    arrays = dict(position=pts, normal=None, index=None, texture=np.zeros((4, n), np.float32),
                  background=np.zeros(4, np.float32), poses=pose[None].copy(), intrinsics=intr, env_map=None)
    view = dict(w=1920, h=1080, image_index=0, camera_index=0, camera_model=capi.CAMERA_OCAM,
                crop=(1.0, 1.0, 0.0, 0.0, 0.0))
    return arrays, view, float(np.tan(theta_max))


def test_pinhole_projection_matches_float64_model(oracle):
    arrays, view = _pinhole_case()
    params = capi.default_render_params()
    params.check_normal = 0
    params.dist_cutoff = 10.0
    got = oracle.project(arrays, view, params)
    T = fm.pose_matrix(arrays["poses"][0])
    K, dist = arrays["intrinsics"][0, :5].astype(np.float64), arrays["intrinsics"][0, 5:].astype(np.float64)
    checked = 0
    for i, p in enumerate(arrays["position"]):
        ip, z = fm.project_pinhole(T, K, dist, np.array(view["crop"], np.float64), p[:3].astype(np.float64))
        if z <= 0:
            assert got[i, 2] == 0
            continue
        assert abs(got[i, 2] - z) < 1e-5 * z
        assert np.abs(got[i, :2] - ip).max() < 2e-3, (i, got[i], ip)
        focal = float(np.float32(K[0]) * np.float32(view["crop"][0]))
        assert abs(got[i, 3] - focal * 0.01 / z) < 1e-4
        checked += 1
    assert checked > 250


def test_distortion_cutoff_rejects(oracle):
    arrays, view = _pinhole_case()
    params = capi.default_render_params()
    params.check_normal = 0
    params.dist_cutoff = 0.2
    got = oracle.project(arrays, view, params)
    T = fm.pose_matrix(arrays["poses"][0])
    for i, p in enumerate(arrays["position"]):
        v = T[:3, :3] @ p[:3].astype(np.float64) + T[:3, 3]
        if v[2] > 0:
            r2 = (v[0] / v[2]) ** 2 + (v[1] / v[2]) ** 2
            if abs(r2 - 0.04) > 1e-4:
                assert (got[i, 2] == 0) == (r2 > 0.04)


def test_ocam_projection_matches_float64_model(oracle):
    arrays, view, tmax = _ocam_case()
    params = capi.default_render_params()
    params.check_normal = 0
    params.dist_cutoff = tmax
    got = oracle.project(arrays, view, params)
    T = fm.pose_matrix(arrays["poses"][0])
    aff, poly = arrays["intrinsics"][0, :5].astype(np.float64), arrays["intrinsics"][0, 5:].astype(np.float64)
    for i, p in enumerate(arrays["position"]):
        ip, z = fm.project_ocam(T, aff, poly, np.array(view["crop"], np.float64), p[:3].astype(np.float64))
        assert abs(got[i, 2] - z) < 1e-5 * z
        assert np.abs(got[i, :2] - ip).max() < 0.05, (i, got[i], ip)  # rho is ~1e3 px and a degree-10 polynomial in f32


def test_ocam_inverse_polynomial_roundtrip():
    """The fitted world->cam polynomial inverts the cam->world one of the configuration within a fraction of a pixel."""
    c2w = (-300.0, 0.0, 5e-4, -1e-7)
    coef, _ = synth.ocam_world2cam_poly(c2w)
    for rho in np.linspace(5, 1100, 50):
        f = sum(c * rho ** i for i, c in enumerate(c2w))
        theta = np.arctan2(f, rho)
        assert abs(sum(a * theta ** i for i, a in enumerate(coef)) - rho) < 0.05


def test_pinhole_backward_chain_matches_finite_differences(oracle):
    arrays, view = _pinhole_case(seed=2, n=40)
    params = capi.default_render_params()
    params.check_normal = 0
    params.dist_cutoff = 10.0
    T = fm.pose_matrix(arrays["poses"][0])
    K, dist = arrays["intrinsics"][0, :5].astype(np.float64), arrays["intrinsics"][0, 5:].astype(np.float64)
    crop = np.array(view["crop"], np.float64)
    g = np.array([0.7, -1.3])
    done = 0
    for i, p in enumerate(arrays["position"]):
        p3 = p[:3].astype(np.float64)
        ok, out = oracle.project_backward(arrays, view, params, i, float(g[0]), float(g[1]))
        if not ok:
            continue
        gp = fm.numeric_grad(lambda q: fm.project_pinhole(T, K, dist, crop, q)[0], p3, g)
        gxi = fm.numeric_grad(lambda xi: fm.project_pinhole(fm.se3_exp_matrix(xi) @ T, K, dist, crop, p3)[0], np.zeros(6), g)
        gk = fm.numeric_grad(lambda k: fm.project_pinhole(T, k, dist, crop, p3)[0], K, g)
        gd = fm.numeric_grad(lambda d: fm.project_pinhole(T, K, d, crop, p3)[0], dist, g)
        for got, want, name in ((out[0:3], gp, "point"), (out[3:9], gxi, "pose"), (out[9:14], gk, "K"), (out[14:22], gd, "dist")):
            scale = max(np.abs(want).max(), 1e-3)
            assert np.abs(got - want).max() < 2e-3 * scale, (name, i, got, want)
        done += 1
    assert done > 20


def test_ocam_backward_chain_matches_finite_differences(oracle):
    arrays, view, tmax = _ocam_case(seed=4, n=40)
    params = capi.default_render_params()
    params.check_normal = 0
    params.dist_cutoff = tmax
    T = fm.pose_matrix(arrays["poses"][0])
    aff, poly = arrays["intrinsics"][0, :5].astype(np.float64), arrays["intrinsics"][0, 5:].astype(np.float64)
    crop = np.array(view["crop"], np.float64)
    g = np.array([-0.4, 0.9])
    for i, p in enumerate(arrays["position"]):
        p3 = p[:3].astype(np.float64)
        ok, out = oracle.project_backward(arrays, view, params, i, float(g[0]), float(g[1]))
        assert ok
        gp = fm.numeric_grad(lambda q: fm.project_ocam(T, aff, poly, crop, q)[0], p3, g)
        gxi = fm.numeric_grad(lambda xi: fm.project_ocam(fm.se3_exp_matrix(xi) @ T, aff, poly, crop, p3)[0], np.zeros(6), g)
        ga = fm.numeric_grad(lambda a: fm.project_ocam(T, a, poly, crop, p3)[0], aff, g)
        for got, want, name in ((out[0:3], gp, "point"), (out[3:9], gxi, "pose"), (out[9:14], ga, "affine")):
            scale = max(np.abs(want).max(), 1e-3)
            assert np.abs(got - want).max() < 5e-3 * scale, (name, i, got, want)


def test_apply_tangent_matches_matrix_exponential(oracle):
    rng = np.random.default_rng(5)
    n = 20
    poses = np.stack([synth.look_at_pose(rng.normal(size=3) * 3, rng.normal(size=3)) for _ in range(n)])
    tangents = rng.normal(size=(n, 6)) * 0.2
    tangents[0] = 0
    tangents[1] *= 1e-10
    want = [fm.se3_exp_matrix(tangents[i]) @ fm.pose_matrix(poses[i]) for i in range(n)]
    t, p = tangents.copy(), poses.copy()
    oracle.apply_tangent(t, p)
    assert np.all(t == 0)
    for i in range(n):
        assert np.abs(fm.pose_matrix(p[i]) - want[i]).max() < 1e-12
        assert abs(np.linalg.norm(p[i, :4]) - 1) < 1e-14 and p[i, 7] == 0


# ---------------------------------------------------------------------------------------------- golden fixtures
def test_golden_projection_fixture(oracle):
    """tests/golden/projection_f64.npz was written by tests/golden/make_golden.py from the float64 model."""
    g = np.load(os.path.join(ROOT, "tests", "golden", "projection_f64.npz"))
    params = capi.default_render_params()
    params.check_normal = 0
    params.dist_cutoff = 10.0
    for tag, model in (("pinhole", capi.CAMERA_PINHOLE_DISTORTION), ("ocam", capi.CAMERA_OCAM)):
        pts = g[f"{tag}_points"]
        arrays = dict(position=pts, normal=None, index=None, texture=np.zeros((4, len(pts)), np.float32),
                      background=np.zeros(4, np.float32), poses=g[f"{tag}_pose"], intrinsics=g[f"{tag}_intrinsics"], env_map=None)
        view = dict(w=int(g[f"{tag}_wh"][0]), h=int(g[f"{tag}_wh"][1]), image_index=0, camera_index=0, camera_model=model,
                    crop=tuple(g[f"{tag}_crop"]))
        got = oracle.project(arrays, view, params)
        want = g[f"{tag}_expected"]
        tol = 2e-3 if tag == "pinhole" else 0.05
        assert np.abs(got[:, :2] - want[:, :2]).max() < tol
        assert np.abs(got[:, 2] - want[:, 2]).max() < 1e-4


# ---------------------------------------------------------------------------------------------- rasterizer invariants
def _small(seed=0, **kw):
    return synth.make_config("c1", n_points=20000, size=(96, 80), seed=seed, **kw)


def test_depth_is_min_and_weight_counts_accepted_points(oracle):
    cfg = _small()
    params = cfg["params"]
    out = oracle.forward(cfg["arrays"], cfg["views"], params, 4)
    proj = oracle.project(cfg["arrays"], cfg["views"][0], params)
    for l, (w, h) in enumerate(capi.layer_sizes(96, 80, 4)):
        depth = np.full((h, w), 100000.0, np.float32)
        s = np.float32(0.5) ** l
        px = np.rint(proj[:, 0] * s).astype(np.int64)  # numpy rint = ties to even
        py = np.rint(proj[:, 1] * s).astype(np.int64)
        ok = (proj[:, 2] > 0) & (px >= 0) & (py >= 0) & (px < w) & (py < h)
        np.minimum.at(depth, (py[ok], px[ok]), proj[ok, 2])
        assert np.array_equal(depth, out["depths"][l][0, 0])
        thr = depth[py[ok], px[ok]] * (np.float32(params.depth_accept) + np.float32(1))
        acc = proj[ok, 2] <= thr
        wgt = np.zeros((h, w), np.float32)
        np.add.at(wgt, (py[ok][acc], px[ok][acc]), 1)
        assert np.array_equal(wgt, out["weights"][l][0, 0])
        # every covered pixel is the mean of its accepted descriptors; uncovered ones are the background
        col = np.zeros((4, h, w), np.float64)
        tex = cfg["arrays"]["texture"][:, ok][:, acc]
        for c in range(4):
            np.add.at(col[c], (py[ok][acc], px[ok][acc]), tex[c])
        cov = wgt > 0
        assert np.allclose(out["colors"][l][0][:, cov], (col[:, cov] / wgt[cov]), rtol=1e-5, atol=1e-6)
        assert np.all(out["colors"][l][0][:, ~cov] == 0)


def test_point_order_does_not_change_depth_or_weight(oracle):
    cfg = _small(seed=3)
    a = oracle.forward(cfg["arrays"], cfg["views"], cfg["params"], 4)
    perm = np.random.default_rng(0).permutation(cfg["meta"]["n_points"])
    arr = dict(cfg["arrays"])
    arr["position"] = np.ascontiguousarray(arr["position"][perm])
    arr["texture"] = np.ascontiguousarray(arr["texture"][:, perm])
    b = oracle.forward(arr, cfg["views"], cfg["params"], 4)
    for l in range(4):
        assert np.array_equal(a["depths"][l], b["depths"][l]) and np.array_equal(a["weights"][l], b["weights"][l])
        assert np.allclose(a["colors"][l], b["colors"][l], rtol=1e-5, atol=1e-6)


def test_parallel_oracle_equals_scalar_oracle(oracle):
    cfg = synth.make_config("c2", n_points=30000, n_views=2, size=(160, 90))
    grads = synth.upstream_gradients(cfg["meta"])
    a = oracle.forward(cfg["arrays"], cfg["views"], cfg["params"], 4)
    b = oracle.forward(cfg["arrays"], cfg["views"], cfg["params"], 4, threads=4)
    for l in range(4):
        assert np.array_equal(a["depths"][l], b["depths"][l]) and np.array_equal(a["weights"][l], b["weights"][l])
        assert np.allclose(a["colors"][l], b["colors"][l], rtol=1e-5, atol=1e-6)
    ga = oracle.backward(cfg["arrays"], cfg["views"], cfg["params"], 4, a, grads)
    gb = oracle.backward(cfg["arrays"], cfg["views"], cfg["params"], 4, a, grads, threads=4)
    for k in ("texture", "points", "pose", "intrinsics"):
        assert np.allclose(ga[k], gb[k], rtol=1e-4, atol=1e-5 * np.abs(ga[k]).max())


def test_descriptor_gradient_is_the_adjoint_single_layer(oracle):
    """With one layer the forward's accept set equals the backward's, and the op is linear in the descriptors."""
    cfg = _small(layers=1)
    arrays = cfg["arrays"]
    fwd = oracle.forward(arrays, cfg["views"], cfg["params"], 1)
    g = synth.upstream_gradients(cfg["meta"], batch=1)
    bwd = oracle.backward(arrays, cfg["views"], cfg["params"], 1, fwd, g, want_points=False, want_pose=False,
                          want_intrinsics=False)
    lhs = float((g[0].astype(np.float64) * fwd["colors"][0]).sum())
    rhs = float((bwd["texture"].astype(np.float64) * arrays["texture"]).sum())
    assert abs(lhs - rhs) < 1e-4 * max(abs(lhs), 1)


def test_background_gradient_is_sum_over_uncovered_pixels(oracle):
    cfg = _small()
    fwd = oracle.forward(cfg["arrays"], cfg["views"], cfg["params"], 4)
    g = synth.upstream_gradients(cfg["meta"], batch=1)
    bwd = oracle.backward(cfg["arrays"], cfg["views"], cfg["params"], 4, fwd, g)
    want = sum((g[l][0] * (fwd["weights"][l][0] == 0)).sum(axis=(1, 2)) for l in range(4))
    assert np.allclose(bwd["background"], want, rtol=1e-4, atol=1e-4)


def test_forward_continues_but_backward_stops_at_first_depth_failure(oracle):
    """Two points: A (near) and B (far) share a layer-0 pixel, so B fails the fuzzy depth test there, but they round to
    different layer-1 pixels. Forward: B is skipped on layer 0 and still blended on layer 1 (continue,
    PointRenderer.cu:380). Backward: B stops at its first failure and gets no gradient at all (break, :462)."""
    # cx = 32.6: A lands at u = 32.6 (pixel 33, layer 1: 16.3 -> 16); B at u = 33.4 (pixel 33, layer 1: 16.7 -> 17)
    pos = np.array([[0.0, 0.0, 2.0, 0.01], [0.0064, 0.0, 4.0, 0.01]], np.float32)
    arrays = dict(position=pos, normal=None, index=None, texture=np.array([[1.0, 3.0]], np.float32).repeat(4, 0).copy(),
                  background=np.zeros(4, np.float32), poses=np.array([[0, 0, 0, 1, 0, 0, 0, 0.0]]),
                  intrinsics=np.array([[500, 500, 32.6, 32.4, 0, 0, 0, 0, 0, 0, 0, 0, 0]], np.float32), env_map=None)
    views = [dict(w=64, h=64, image_index=0, camera_index=0)]
    params = capi.default_render_params()
    params.dropout = 0
    params.check_normal = 0
    params.drop_out_points_by_radius = 0
    fwd = oracle.forward(arrays, views, params, 2)
    assert fwd["weights"][0].sum() == 1 and fwd["weights"][0][0, 0, 32, 33] == 1
    assert fwd["weights"][1].sum() == 2 and fwd["weights"][1][0, 0, 16, 16] == 1 and fwd["weights"][1][0, 0, 16, 17] == 1
    assert np.all(fwd["colors"][1][0, :, 16, 17] == 3.0)
    g = [np.ones((1, 4, 64, 64), np.float32), np.ones((1, 4, 32, 32), np.float32)]
    bwd = oracle.backward(arrays, views, params, 2, fwd, g, want_points=False, want_pose=False, want_intrinsics=False)
    assert np.allclose(bwd["texture"][:, 0], 2.0) and np.all(bwd["texture"][:, 1] == 0.0)


def test_ghost_gradient_stencil_by_hand(oracle):
    """One dropped point next to a covered pixel: the image-space gradient is the central difference of
    (T_p - I_x) * G_x averaged over the channels (PointRenderer.cu:588-611)."""
    pos = np.array([[0.0, 0.0, 2.0, 0.01], [0.004 * 2, 0.0, 2.0, 0.01]], np.float32)  # pixels (16,16) and (18,16)
    tex = np.array([[0.8, 0.2]], np.float32).repeat(4, 0).copy()
    arrays = dict(position=pos, normal=None, index=None, texture=tex, background=np.full(4, 0.1, np.float32),
                  poses=np.array([[0, 0, 0, 1, 0, 0, 0, 0.0]]),
                  intrinsics=np.array([[500, 500, 16, 16, 0, 0, 0, 0, 0, 0, 0, 0, 0]], np.float32), env_map=None)
    views = [dict(w=32, h=32, image_index=0, camera_index=0)]
    params = capi.default_render_params()
    params.check_normal = 0
    params.drop_out_points_by_radius = 0
    params.ghost_gradients = 1
    mask = np.array([[1, 0]], np.uint8)  # point 0 is dropped (a ghost); point 1 renders
    fwd = oracle.forward(arrays, views, params, 1, dropout_mask=mask)
    assert fwd["weights"][0][0, 0, 16, 18] == 1 and fwd["weights"][0][0, 0, 16, 16] == 0
    rng = np.random.default_rng(0)
    G = rng.normal(size=(1, 4, 32, 32)).astype(np.float32)
    bwd = oracle.backward(arrays, views, params, 1, fwd, [G], dropout_mask=mask, normalize=False)
    I = fwd["colors"][0][0]
    d = lambda x, y: sum((0.8 - I[c, y, x]) * G[0, c, y, x] for c in range(4))
    gx = 0.5 * (-d(15, 16) + d(17, 16)) / 4
    gy = 0.5 * (-d(16, 15) + d(16, 17)) / 4
    # pinhole without distortion at the optical axis: d(pixel)/d(point) = (fx / z, 0), so g_point = (gx fx/z, gy fy/z, 0)
    want = np.array([gx * 500 / 2, gy * 500 / 2, 0.0])
    assert np.allclose(bwd["points"][0, :3], want, rtol=1e-4, atol=1e-6)
    assert bwd["points"][0, 3] == 1 and np.all(bwd["points"][1] == 0)
    assert bwd["count_pose"][0] == 1 and abs(bwd["count_intrinsics"][0] - 1 / 1024) < 1e-9
    assert np.allclose(bwd["pose"][0, :3], [gx * 250, gy * 250, 0], rtol=1e-4, atol=1e-6)


def test_environment_map_lookup_matches_float64_and_grid_sample(oracle):
    cfg = synth.make_config("c2", n_points=2000, n_views=2, size=(64, 36))
    arrays = cfg["arrays"]
    view = cfg["views"][1]
    uv = oracle.env_uv(arrays, view, 1)
    T = fm.pose_matrix(arrays["poses"][1])
    K, dist = arrays["intrinsics"][0, :5].astype(np.float64), arrays["intrinsics"][0, 5:].astype(np.float64)
    for (gy, gx) in [(0, 0), (5, 7), (17, 31), (9, 20)]:
        ip = np.array([gx, gy], np.float64) / 0.5  # undo the layer-1 crop (identity * 0.5)
        m = fm.undistort([(ip[0] - K[2] - K[4] * (ip[1] - K[3]) / K[1]) / K[0], (ip[1] - K[3]) / K[1]], dist)
        d = T[:3, :3].T @ np.array([m[0], m[1], 1.0])
        want = fm.spherical_uv(d / np.linalg.norm(d))
        assert np.abs(uv[gy, gx] - want).max() < 1e-4
    # the composite: out = background + (1 - mask) * grid_sample(env, uv) on uncovered pixels
    cfg["params"].output_background_mask = 1
    fwd = oracle.forward(arrays, cfg["views"], cfg["params"], 2)
    env = torch.from_numpy(arrays["env_map"])[None]
    for b in range(2):
        uvb = torch.from_numpy(oracle.env_uv(arrays, cfg["views"][b], 0))[None]
        samp = torch.nn.functional.grid_sample(env, uvb, mode="bilinear", padding_mode="border", align_corners=True)[0].numpy()
        bgm = fwd["weights"][0][b, 0] == 0
        assert bgm.any()
        assert np.allclose(fwd["colors"][0][b][:, bgm], samp[:, bgm], rtol=1e-4, atol=1e-5)
        assert np.array_equal(fwd["masks"][0][b, 0], (~bgm).astype(np.float32))


def test_environment_map_gradient_matches_grid_sample_autograd(oracle):
    cfg = synth.make_config("c2", n_points=2000, n_views=1, size=(64, 36))
    arrays = cfg["arrays"]
    fwd = oracle.forward(arrays, cfg["views"], cfg["params"], 1)
    g = synth.upstream_gradients(cfg["meta"], batch=1)[:1]
    bwd = oracle.backward(arrays, cfg["views"], cfg["params"], 1, fwd, g, want_env=True)
    env = torch.from_numpy(arrays["env_map"])[None].clone().requires_grad_(True)
    uv = torch.from_numpy(oracle.env_uv(arrays, cfg["views"][0], 0))[None]
    samp = torch.nn.functional.grid_sample(env, uv, mode="bilinear", padding_mode="border", align_corners=True)
    bgm = torch.from_numpy((fwd["weights"][0] == 0).astype(np.float32))
    (samp * bgm * torch.from_numpy(g[0])).sum().backward()
    assert np.allclose(bwd["env_map"], env.grad[0].numpy(), rtol=1e-4, atol=1e-5)


# ---------------------------------------------------------------------------------------------- tonemapper
def _torch_tonemap(x, frame_index, exposure, wb, vig, uv, response, leak, image_size):
    """The reference's sequence of libtorch operations (NeuralCamera.cpp:22-42, 87-135, 258-335) in torch."""
    e = exposure[frame_index.long()].view(-1, 1, 1, 1)
    x = x * (1.0 / torch.exp2(e))
    x = wb[frame_index.long()].view(-1, 3, 1, 1) * x
    aspect = image_size[0] / image_size[1]
    t = uv - vig[3:5].view(1, 2, 1, 1)
    t = torch.cat([t[:, :1] * aspect, t[:, 1:]], 1)
    r2 = (t * t).sum(1, keepdim=True)
    x = (1.0 + vig[0] * r2 + vig[1] * r2 * r2 + vig[2] * r2 * r2 * r2) * x
    leak_add = 0
    if leak > 0:
        leak_add = (x * leak) * (x < 0) + (-leak / ((x.abs() + 1e-4).sqrt()) + leak) * (x > 1)
    B, C = x.shape[:2]
    grid = x * 2.0 - 1.0
    res = torch.ones_like(x)
    for c in range(C):
        sl = torch.stack([grid[:, c], torch.zeros_like(grid[:, c])], dim=3)
        lut = response[c].view(1, 1, 1, -1).repeat(B, 1, 1, 1)
        res[:, c:c + 1] = torch.nn.functional.grid_sample(lut, sl, mode="bilinear", padding_mode="border", align_corners=True)
    return res + leak_add


@pytest.mark.parametrize("leak", [0.0, 0.01])
def test_tonemapper_matches_reference_op_sequence(oracle, leak):
    rng = np.random.default_rng(0)
    B, H, W, K, n = 2, 18, 24, 25, 5
    x = rng.uniform(-0.2, 2.5, (B, 3, H, W)).astype(np.float32)
    fi = np.array([3, 1], np.int32)
    exposure = rng.uniform(-1, 1, n).astype(np.float32)
    wb = rng.normal(1, 0.05, (n, 3)).astype(np.float32)
    vig = np.array([0.1, -0.05, 0.01, 0.02, -0.03], np.float32)
    ys, xs = np.meshgrid(np.arange(H), np.arange(W), indexing="ij")
    uv = np.stack([2 * xs / (W - 1) - 1, 2 * ys / (H - 1) - 1])[None].repeat(B, 0).astype(np.float32)
    uv += rng.normal(0, 0.01, uv.shape).astype(np.float32)
    response = np.sort(rng.uniform(0, 1, (3, K)), axis=1).astype(np.float32)
    kw = dict(image_size=(W, H), frame_index=fi, exposure=exposure, white_balance=wb, vignette=vig, uv=uv,
              response=response, leak=leak)
    got = oracle.tonemap_forward(x, **kw)
    tx = torch.from_numpy(x).requires_grad_(True)
    te, twb = torch.from_numpy(exposure).requires_grad_(True), torch.from_numpy(wb).requires_grad_(True)
    tv, tr = torch.from_numpy(vig).requires_grad_(True), torch.from_numpy(response).requires_grad_(True)
    want = _torch_tonemap(tx, torch.from_numpy(fi), te, twb, tv, torch.from_numpy(uv), tr, leak, (W, H))
    assert np.allclose(got, want.detach().numpy(), rtol=1e-5, atol=2e-6)
    go = rng.normal(size=x.shape).astype(np.float32)
    want.backward(torch.from_numpy(go))
    g = oracle.tonemap_backward(x, go, **kw)
    assert np.allclose(g["x"], tx.grad.numpy(), rtol=1e-4, atol=1e-5)
    assert np.allclose(g["exposure"], te.grad.numpy(), rtol=1e-4, atol=1e-4)
    assert np.allclose(g["white_balance"], twb.grad.numpy(), rtol=1e-4, atol=1e-4)
    assert np.allclose(g["vignette"], tv.grad.numpy(), rtol=1e-4, atol=1e-4)
    assert np.allclose(g["response"], tr.grad.numpy(), rtol=1e-4, atol=1e-4)


def test_tonemapper_default_uv_and_plain_clamp(oracle):
    rng = np.random.default_rng(1)
    x = rng.uniform(-0.5, 1.5, (1, 3, 9, 16)).astype(np.float32)
    out = oracle.tonemap_forward(x, image_size=(16, 9))
    assert np.array_equal(out, np.clip(x, 0, 1))
    vig = np.array([0.3, 0, 0, 0, 0], np.float32)
    out = oracle.tonemap_forward(x, image_size=(16, 9), vignette=vig)
    r2 = (-1 * 16 / 9) ** 2 + 1  # corner pixel (0,0): uv = (-1,-1)
    assert abs(out[0, 0, 0, 0] - np.clip(x[0, 0, 0, 0] * (1 + 0.3 * r2), 0, 1)) < 1e-6


# ---------------------------------------------------------------------------------------------- C ABI
def test_c_abi_library_exports_every_declared_symbol():
    """Loads libadop_raster.so without a GPU and resolves each entry point of include/adop/adop_raster.h."""
    from adop_b200 import build
    build.build_library()
    lib = ctypes.CDLL(capi.LIB_PATH)
    header = open(os.path.join(ROOT, "include", "adop", "adop_raster.h")).read()
    import re
    declared = set(re.findall(r"\b(adop_[a-z_]+)\s*\(", header))
    assert declared == set(capi.EXPORTED_SYMBOLS), declared ^ set(capi.EXPORTED_SYMBOLS)
    for name in declared:
        assert getattr(lib, name) is not None
    lib.adop_status_string.restype = ctypes.c_char_p
    assert lib.adop_status_string(0) == b"ok" and lib.adop_status_string(4) == b"workspace too small"
    p = capi.AdopRenderParams()
    lib.adop_render_params_default(ctypes.byref(p))
    d = capi.default_render_params()
    for f, _ in capi.AdopRenderParams._fields_:
        assert getattr(p, f) == getattr(d, f), f
    lib.adop_raster_workspace_bytes.restype = ctypes.c_size_t
    assert lib.adop_raster_workspace_bytes(1920, 1080, 4, 4) == 32768 + 2754000 * 8 * 4 + 256
    assert lib.adop_raster_workspace_bytes(0, 1080, 4, 4) == 0


def test_struct_sizes_match_the_header():
    """ctypes mirrors must have the C layout (compiled probe with the system compiler)."""
    import subprocess
    import tempfile
    src = '#include <stdio.h>\n#include "adop/adop_raster.h"\nint main(){printf("%zu %zu %zu %zu %zu %zu %zu %zu %zu %zu %zu %zu\\n",' \
          'sizeof(adop_view),sizeof(adop_render_params),sizeof(adop_scene),sizeof(adop_layer_buffers),' \
          'sizeof(adop_forward_io),sizeof(adop_backward_io),sizeof(adop_tonemap_params),sizeof(adop_tonemap_grads),' \
          'sizeof(adop_peer_layout),sizeof(adop_peer_reduce_out),sizeof(adop_peer_param_layout),sizeof(adop_peer_update));return 0;}'
    with tempfile.TemporaryDirectory() as d:
        open(os.path.join(d, "p.c"), "w").write(src)
        subprocess.run(["/usr/bin/gcc", "-I", os.path.join(ROOT, "include"), os.path.join(d, "p.c"), "-o", os.path.join(d, "p")], check=True)
        sizes = list(map(int, subprocess.run([os.path.join(d, "p")], capture_output=True, text=True).stdout.split()))
    mirrors = [capi.AdopView, capi.AdopRenderParams, capi.AdopScene, capi.AdopLayerBuffers, capi.AdopForwardIO,
               capi.AdopBackwardIO, capi.AdopTonemapParams, capi.AdopTonemapGrads, capi.AdopPeerLayout, capi.AdopPeerReduceOut,
               capi.AdopPeerParamLayout, capi.AdopPeerUpdate]
    assert sizes == [ctypes.sizeof(m) for m in mirrors]


def test_missing_library_fails_loudly(monkeypatch):
    monkeypatch.setattr(capi, "_lib", None)
    monkeypatch.setattr(capi, "LIB_PATH", "/nonexistent/libadop_raster.so")
    with pytest.raises(capi.AdopError, match="no CPU fallback"):
        capi.load_library()


def test_libtorch_operator_builds_and_registers():
    """The C++ autograd operator links against the C-ABI library and registers the reference's entry points."""
    from adop_b200 import build
    build.build_torch_op()
    torch.ops.load_library(build.TORCH_OP_LIB)
    assert hasattr(torch.ops.adop, "blend_point_cloud") and hasattr(torch.ops.adop, "apply_tangent_to_pose")
    info = torch.classes.adop.RenderInfo()
    info.set_num_layers(4)
    info.set_param("depth_accept", 0.01)
    with pytest.raises(RuntimeError, match="unknown render parameter"):
        info.set_param("no_such_field", 1.0)


def test_packed_depth_index_word(oracle):
    """The packed depth|index by-product: high word = the depth buffer's bits, low word = the lowest index among the points
    that have that depth in the pixel (checked against a direct search), empty pixels hold (100000.0, 0xFFFFFFFF)."""
    cfg = synth.make_config("c2", n_points=20000, n_views=2, size=(64, 36))
    fwd = oracle.forward(cfg["arrays"], cfg["views"], cfg["params"], 3, packed_depth=True)
    for l in range(3):
        packed = fwd["packed"][l]
        depth_bits = fwd["depths"][l].view(np.uint32)
        assert np.array_equal((packed >> np.uint64(32)).astype(np.uint32), depth_bits)
        idx = (packed & np.uint64(0xFFFFFFFF)).astype(np.uint32)
        empty = fwd["depths"][l] == np.float32(100000.0)
        assert np.all(idx[empty] == 0xFFFFFFFF) and np.all(idx[~empty] < 20000)
    # direct search on layer 0 of view 0: the winner is the lowest index among the nearest points of the pixel
    q = oracle.project(cfg["arrays"], cfg["views"][0], cfg["params"])
    px, py = np.rint(q[:, 0]).astype(int), np.rint(q[:, 1]).astype(int)
    ok = (q[:, 2] > 0) & (px >= 0) & (px < 64) & (py >= 0) & (py < 36)
    idx0 = (fwd["packed"][0][0, 0] & np.uint64(0xFFFFFFFF)).astype(np.int64)
    d0 = fwd["depths"][0][0, 0]
    for y, x in zip(*np.nonzero(d0 < 100000.0)):
        cand = np.nonzero(ok & (px == x) & (py == y) & (q[:, 2] == d0[y, x]))[0]
        assert idx0[y, x] == cand.min()


def test_five_vector_projection_has_the_same_bits_as_the_general_one(oracle):
    """project_for_raster_hot (what the GPU's plain kernels use for pinhole cameras with k1, k2 only) against
    project_for_raster, bit for bit, on points in front of, behind and far outside the camera; cameras with more
    coefficients or the omnidirectional model do not offer the short form."""
    cfg = synth.make_config("c2", n_points=200_000, n_views=3, size=(320, 180))
    a = cfg["arrays"]
    rng = np.random.default_rng(5)
    a["position"][:5000, :3] *= 40.0                      # far outside: distortion cut-off and the range check
    a["position"][5000:6000, :3] = rng.normal(0, 1e-3, (1000, 3)).astype(np.float32)
    for view in cfg["views"]:
        view = dict(view, crop=(1.3, 0.9, -20.5, 7.25, 0.01))
        general = oracle.project(a, view, cfg["params"])
        hot = oracle.project_hot(a, view, cfg["params"])
        assert hot is not None
        accepted = hot[:, 3] == 1
        assert np.array_equal(accepted, general[:, 2] > 0)
        assert np.array_equal(hot[:, :3].view(np.uint32), general[:, :3].view(np.uint32))
        assert 0.2 < accepted.mean() < 1.0
    full = dict(a)
    full["intrinsics"] = a["intrinsics"].copy()
    full["intrinsics"][0, 7] = 0.001                      # k3
    assert oracle.project_hot(full, cfg["views"][0], cfg["params"]) is None
    c3 = synth.make_config("c3", n_points=1000, size=(64, 36))
    assert oracle.project_hot(c3["arrays"], c3["views"][0], c3["params"]) is None


def test_outlier_cloud_takes_part_in_the_forward_pass_only(oracle):
    """The second cloud of a scene (PointRenderer.cu:1402-1441) goes into the same depth, weight and colour buffers: the
    depth of a pixel is the minimum over both clouds, the weights count both, and the result equals that of ONE cloud
    that holds the points of both. The backward pass walks the main cloud only (:1588-1600): descriptor columns that only
    outliers use get no gradient, and the main points' gradients are those of the merged render restricted to them."""
    cfg = synth.make_config("c1", n_points=30_000, size=(96, 96))
    a, views, params, L = cfg["arrays"], cfg["views"], cfg["params"], cfg["num_layers"]
    n = len(a["position"])
    # extra descriptor columns that only the outliers use
    rng = np.random.default_rng(2)
    a["texture"] = np.ascontiguousarray(np.concatenate([a["texture"], rng.uniform(0, 1, (4, 500)).astype(np.float32)], axis=1))
    out = synth.outlier_cloud(a, 4000, seed=1, with_normals=False)
    # pull the sphere in so that a good share of the outliers lies between the camera and the cloud
    out["outlier_position"][:, :3] = (out["outlier_position"][:, :3] * 0.25 + np.array([0, 0, 2.5], np.float32)).astype(np.float32)
    out["outlier_index"] = (n + rng.integers(0, 500, 4000)).astype(np.int32)
    both = dict(a, **out)
    plain = oracle.forward(a, views, params, L)
    ref = oracle.forward(both, views, params, L)
    merged = dict(a)
    merged["position"] = np.ascontiguousarray(np.concatenate([a["position"], out["outlier_position"]]))
    merged["index"] = np.concatenate([np.arange(n, dtype=np.int32), out["outlier_index"]])
    one = oracle.forward(merged, views, params, L)
    changed = 0
    for l in range(L):
        assert np.array_equal(ref["depths"][l], one["depths"][l]) and np.array_equal(ref["weights"][l], one["weights"][l])
        assert np.allclose(ref["colors"][l], one["colors"][l], rtol=1e-6, atol=1e-7)
        assert (ref["depths"][l] <= plain["depths"][l]).all()
        changed += int((ref["depths"][l] < plain["depths"][l]).sum())
    assert changed > 100
    grads = synth.upstream_gradients(cfg["meta"], batch=len(views))
    gb = oracle.backward(both, views, params, L, ref, grads)
    gm = oracle.backward(merged, views, params, L, one, grads, normalize=False)
    assert not gb["texture"][:, n:].any()
    assert gm["texture"][:, n:].any()
    g1 = oracle.backward(both, views, params, L, ref, grads, normalize=False)
    assert np.allclose(g1["texture"][:, :n], gm["texture"][:, :n], rtol=1e-5, atol=1e-7)
    assert np.allclose(g1["points"], gm["points"][:n], rtol=1e-5, atol=1e-7)
