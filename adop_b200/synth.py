"""Seeded synthetic workloads with the shapes, sizes and value distributions of the benchmark configurations.

They stand in for the reference's real scenes (Tanks & Temples / boat scenes, README.md:73-88), which are not
available offline. Everything is numpy on the host; callers upload the arrays. Point clouds are Morton-sorted
once, as the reference's scene preprocessing does (SceneData.cpp:96-118); that sort is not part of any timing.
"""
import math

import numpy as np

from . import capi


def morton_order(xyz):
    """Permutation that sorts points along a 3-D Morton curve (21 bits per axis)."""
    lo = xyz.min(axis=0)
    span = np.maximum(xyz.max(axis=0) - lo, 1e-12)
    q = np.minimum(((xyz - lo) / span * 2097151.0).astype(np.uint64), np.uint64(2097151))

    def spread(v):
        v = v & np.uint64(0x1FFFFF)
        v = (v | (v << np.uint64(32))) & np.uint64(0x1F00000000FFFF)
        v = (v | (v << np.uint64(16))) & np.uint64(0x1F0000FF0000FF)
        v = (v | (v << np.uint64(8))) & np.uint64(0x100F00F00F00F00F)
        v = (v | (v << np.uint64(4))) & np.uint64(0x10C30C30C30C30C3)
        v = (v | (v << np.uint64(2))) & np.uint64(0x1249249249249249)
        return v

    code = spread(q[:, 0]) | (spread(q[:, 1]) << np.uint64(1)) | (spread(q[:, 2]) << np.uint64(2))
    return np.argsort(code, kind="stable")


def quat_from_matrix(R):
    """Unit quaternion (x, y, z, w) of a rotation matrix."""
    t = np.trace(R)
    if t > 0:
        s = math.sqrt(t + 1.0) * 2
        w = 0.25 * s
        x = (R[2, 1] - R[1, 2]) / s
        y = (R[0, 2] - R[2, 0]) / s
        z = (R[1, 0] - R[0, 1]) / s
    else:
        i = int(np.argmax(np.diag(R)))
        j, k = (i + 1) % 3, (i + 2) % 3
        s = math.sqrt(1.0 + R[i, i] - R[j, j] - R[k, k]) * 2
        q = [0.0, 0.0, 0.0]
        q[i] = 0.25 * s
        q[j] = (R[j, i] + R[i, j]) / s
        q[k] = (R[k, i] + R[i, k]) / s
        w = (R[k, j] - R[j, k]) / s
        x, y, z = q
    q = np.array([x, y, z, w], dtype=np.float64)
    return q / np.linalg.norm(q)


def look_at_pose(eye, target=(0, 0, 0), up=(0, -1, 0)):
    """World->camera pose record [8] (quaternion xyzw, translation, pad) of a camera at `eye` looking at `target`
    along its +z axis."""
    eye, target, up = (np.asarray(v, dtype=np.float64) for v in (eye, target, up))
    zc = target - eye
    zc /= np.linalg.norm(zc)
    xc = np.cross(up, zc)
    xc /= np.linalg.norm(xc)
    yc = np.cross(zc, xc)
    R = np.stack([xc, yc, zc])  # rows = camera axes in world coordinates
    t = -R @ eye
    return np.concatenate([quat_from_matrix(R), t, [0.0]])


def orbit_poses(n, radius=4.0):
    return np.stack([look_at_pose((radius * math.cos(2 * math.pi * i / n), 0.3 * math.sin(4 * math.pi * i / n),
                                   radius * math.sin(2 * math.pi * i / n))) for i in range(n)])


def surface_points(rng, n, primitives=64, jitter=0.005):
    """n points on the surfaces of random spheres and square plane patches (radii / half sizes U[0.2,2], centres
    U[-1.5,1.5]^3), plus N(0, jitter) noise. float32 [n,3]."""
    kinds = rng.integers(0, 2, primitives)
    radii = rng.uniform(0.2, 2.0, primitives)
    centres = rng.uniform(-1.5, 1.5, (primitives, 3))
    frames = []
    for _ in range(primitives):
        a = rng.normal(size=3)
        a /= np.linalg.norm(a)
        b = np.cross(a, rng.normal(size=3))
        b /= np.linalg.norm(b)
        frames.append((a, b))
    area = np.where(kinds == 0, 4 * math.pi * radii ** 2, 4 * radii ** 2)
    counts = np.floor(area / area.sum() * n).astype(np.int64)
    counts[0] += n - counts.sum()
    out = np.empty((n, 3), dtype=np.float32)
    o = 0
    for k in range(primitives):
        m = int(counts[k])
        if m == 0:
            continue
        if kinds[k] == 0:
            d = rng.normal(size=(m, 3)).astype(np.float32)
            d /= np.linalg.norm(d, axis=1, keepdims=True)
            p = centres[k].astype(np.float32) + np.float32(radii[k]) * d
        else:
            uv = rng.uniform(-radii[k], radii[k], (m, 2)).astype(np.float32)
            a, b = frames[k]
            p = centres[k].astype(np.float32) + uv[:, :1] * a.astype(np.float32) + uv[:, 1:] * b.astype(np.float32)
        p += rng.normal(0, jitter, (m, 3)).astype(np.float32)
        out[o:o + m] = p
        o += m
    return out


def ocam_world2cam_poly(cam2world=(-300.0, 0.0, 5e-4, -1e-7), rho_max=1150.0, degree=10):
    """Least-squares inversion (float64) of a cam->world polynomial z = f(rho) into the world->cam polynomial
    rho(theta), theta = atan(f(rho) / rho), which is what the projection evaluates (NeuralStructure.h:57).
    Returns (coefficients a_0..a_degree, largest theta covered)."""
    rho = np.linspace(1e-3, rho_max, 20000)
    f = sum(c * rho ** i for i, c in enumerate(cam2world))
    theta = np.arctan2(f, rho)
    V = np.vander(theta, degree + 1, increasing=True)
    coef, *_ = np.linalg.lstsq(V, rho, rcond=None)
    return coef, float(theta.max())


def _finish_cloud(xyz, rng, radius=0.01, sort=True):
    if sort:
        xyz = xyz[morton_order(xyz)]
    pos = np.empty((xyz.shape[0], 4), dtype=np.float32)
    pos[:, :3] = xyz
    pos[:, 3] = radius
    return pos


def make_config(name, n_points=None, n_views=None, size=None, seed=0, channels=None, layers=None, sort=True):
    """Returns dict(arrays=..., views=[...], params=AdopRenderParams, num_layers=L, meta=...).

    name: 'c1' small cloud / 'c2' training scene / 'c3' viewer (OCam) / 'c4' = c2 with 30 M points / 'c5' HDR 4K.
    n_points / n_views / size=(w,h) / channels / layers override the configuration's own values (for tests)."""
    rng = np.random.default_rng(seed)
    params = capi.default_render_params()
    params.dropout = 0.0
    params.drop_out_points_by_radius = 0
    params.check_normal = 0
    params.depth_accept = 0.01
    meta = dict(name=name, seed=seed)
    env = None
    if name == "c1":
        n = n_points or (1 << 20)
        w, h = size or (512, 512)
        C, L = channels or 4, layers or 4
        xyz = np.stack([rng.normal(0, 1, n), rng.normal(0, 1, n), rng.uniform(2, 6, n)], axis=1).astype(np.float32)
        tex = rng.uniform(0, 1, (C, n)).astype(np.float32)
        poses = np.array([[0, 0, 0, 1, 0, 0, 0, 0]], dtype=np.float64)
        s = w / 512.0
        intr = np.array([[500 * s, 500 * s, 256 * s, 256 * s * h / w, 0, 0, 0, 0, 0, 0, 0, 0, 0]], dtype=np.float32)
        views = [dict(w=w, h=h, image_index=0, camera_index=0, camera_model=capi.CAMERA_PINHOLE_DISTORTION)]
    elif name in ("c2", "c4", "c5"):
        defaults = dict(c2=(10_000_000, 16, (1920, 1080), 4, 4), c4=(30_000_000, 8, (1920, 1080), 4, 4),
                        c5=(50_000_000, 4, (3840, 2160), 8, 6))[name]
        n = n_points or defaults[0]
        nv = n_views or defaults[1]
        w, h = size or defaults[2]
        C, L = channels or defaults[3], layers or defaults[4]
        xyz = surface_points(rng, n)
        if name == "c5":
            tex = rng.uniform(0, 1, (C, n)).astype(np.float32)
            eh, ew = 1024, 2048
        else:
            tex = rng.normal(0.5, 0.1, (C, n)).astype(np.float32)
            eh, ew = 512, 1024
        if size is not None:  # shrink the environment map with the image in tests
            ew = max(8, ew * w // defaults[2][0])
            eh = max(4, eh * h // defaults[2][1])
        env = rng.uniform(0, 1, (C, eh, ew)).astype(np.float32)
        poses = orbit_poses(nv)
        f = 1400.0 * w / 1920.0
        intr = np.array([[f, f, w / 2, h / 2, 0, -0.1, 0.02, 0, 0, 0, 0, 0, 0]], dtype=np.float32)
        views = [dict(w=w, h=h, image_index=i, camera_index=0, camera_model=capi.CAMERA_PINHOLE_DISTORTION)
                 for i in range(nv)]
        params.output_background_mask = 1
        params.composite_environment_map = 1
    elif name == "c3":
        n = n_points or 100_000_000
        w, h = size or (1920, 1080)
        C, L = channels or 4, layers or 4
        xyz = np.empty((n, 3), dtype=np.float32)
        xyz[:, 0] = rng.uniform(-10, 10, n)
        xyz[:, 1] = rng.uniform(-10, 10, n)
        xyz[:, 2] = rng.uniform(-2.5, 2.5, n)
        tex = rng.uniform(0, 1, (C, n)).astype(np.float16).astype(np.float32)  # fp16-storable values
        poses = np.array([[0, 0, 0, 1, 0, 0, 0, 0]], dtype=np.float64)
        s = w / 1920.0
        c2w = (-300.0 * s, 0.0, 5e-4 / s, -1e-7 / (s * s))
        coef, theta_max = ocam_world2cam_poly(c2w, rho_max=1150.0 * s)
        intr = np.concatenate([[1, 0, 0, w / 2, h / 2], coef]).astype(np.float32)[None]
        views = [dict(w=w, h=h, image_index=0, camera_index=0, camera_model=capi.CAMERA_OCAM)]
        params.dist_cutoff = float(math.tan(theta_max) * 0.98)
        meta.update(cam2world=c2w, world2cam=coef.tolist(), theta_max=theta_max)
    else:
        raise ValueError(name)
    pos = _finish_cloud(xyz, rng, sort=sort)
    bg = np.zeros(C, dtype=np.float32)
    arrays = dict(position=pos, normal=None, index=None, texture=np.ascontiguousarray(tex), background=bg,
                  poses=np.ascontiguousarray(poses), intrinsics=np.ascontiguousarray(intr), env_map=env)
    meta.update(n_points=int(pos.shape[0]), channels=C, layers=L, w=w, h=h, n_views=len(views))
    return dict(arrays=arrays, views=views, params=params, num_layers=L, meta=meta)


def pack_normals(n):
    """[M,3] unit vectors -> the library's 10-bit packing x | y<<10 | z<<20 (components mapped from [-1,1] to 0..1023)."""
    q = np.round((np.asarray(n, np.float64) + 1) * 0.5 * 1023).astype(np.uint32)
    return (q[:, 0] | (q[:, 1] << 10) | (q[:, 2] << 20)).astype(np.int32)


def outlier_cloud(arrays, count, seed=0, distance=0.1, with_normals=True):
    """The reference's outlier cloud for a scene (SceneData.cpp:419-439, NeuralScene.cpp:248-252): `count` points (at most
    as many as the main cloud has) on the sphere around the cloud's bounding box, radius grown by `distance`, normals
    towards the centre, descriptor columns drawn uniformly from the scene's texture. Returns the three outlier_* arrays."""
    rng = np.random.default_rng(seed)
    xyz = arrays["position"][:, :3]
    count = min(int(count), len(xyz))
    lo, hi = xyz.min(axis=0).astype(np.float64), xyz.max(axis=0).astype(np.float64)
    centre = 0.5 * (lo + hi)
    radius = 0.5 * np.linalg.norm(hi - lo) * (1.0 + distance)
    d = rng.normal(size=(count, 3))
    d /= np.linalg.norm(d, axis=1, keepdims=True)
    pos = np.zeros((count, 4), np.float32)
    pos[:, :3] = (centre + radius * d).astype(np.float32)
    T = arrays["texture"].shape[1]
    out = dict(outlier_position=pos, outlier_normal=pack_normals(-d) if with_normals else None,
               outlier_index=rng.integers(0, max(T - 1, 1), count).astype(np.int32))
    return out


def upstream_gradients(meta, seed=1, batch=None):
    """N(0,1) upstream gradients, one [B,C,h_l,w_l] float32 array per layer."""
    rng = np.random.default_rng(seed)
    B = batch or meta["n_views"]
    return [rng.standard_normal((B, meta["channels"], hh, ww), dtype=np.float32)
            for ww, hh in capi.layer_sizes(meta["w"], meta["h"], meta["layers"])]
