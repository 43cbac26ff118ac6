"""Independent float64 numpy statement of the camera models, written from the published model definitions
(rigid transform by rotation matrix, OpenCV rational distortion, Scaramuzza omnidirectional model), not from the
shared arithmetic header. Used to pin the CPU checker: values within float32 rounding, Jacobians by central differences.
"""
import numpy as np


def quat_to_matrix(q):
    x, y, z, w = q
    return np.array([[1 - 2 * (y * y + z * z), 2 * (x * y - z * w), 2 * (x * z + y * w)],
                     [2 * (x * y + z * w), 1 - 2 * (x * x + z * z), 2 * (y * z - x * w)],
                     [2 * (x * z - y * w), 2 * (y * z + x * w), 1 - 2 * (x * x + y * y)]], dtype=np.float64)


def hat(w):
    return np.array([[0, -w[2], w[1]], [w[2], 0, -w[0]], [-w[1], w[0], 0]], dtype=np.float64)


def se3_exp_matrix(xi):
    """4x4 matrix exponential of the twist (translation part first) by its power series."""
    A = np.zeros((4, 4))
    A[:3, :3] = hat(xi[3:])
    A[:3, 3] = xi[:3]
    out = np.eye(4)
    term = np.eye(4)
    for k in range(1, 30):
        term = term @ A / k
        out = out + term
    return out


def pose_matrix(p8):
    T = np.eye(4)
    T[:3, :3] = quat_to_matrix(p8[:4])
    T[:3, 3] = p8[4:7]
    return T


def distort(m, d):
    k1, k2, k3, k4, k5, k6, p1, p2 = d
    x, y = m
    r2 = x * x + y * y
    rad = (1 + k1 * r2 + k2 * r2 ** 2 + k3 * r2 ** 3) / (1 + k4 * r2 + k5 * r2 ** 2 + k6 * r2 ** 3)
    return np.array([x * rad + 2 * p1 * x * y + p2 * (r2 + 2 * x * x),
                     y * rad + p1 * (r2 + 2 * y * y) + 2 * p2 * x * y])


def apply_k(K, p):
    fx, fy, cx, cy, s = K
    return np.array([fx * p[0] + s * p[1] + cx, fy * p[1] + cy])


def project_pinhole(T, K, dist, crop, p):
    """-> (cropped image position, depth)"""
    v = T[:3, :3] @ p + T[:3, 3]
    m = v[:2] / v[2]
    return apply_k(crop, apply_k(K, distort(m, dist))), v[2]


def project_ocam(T, aff, poly, crop, p):
    v = T[:3, :3] @ p + T[:3, 3]
    c, d, e, cx, cy = aff
    l = np.hypot(v[0], v[1])
    theta = np.arctan(-v[2] / l)
    rho = sum(a * theta ** i for i, a in enumerate(poly))
    xp, yp = v[0] * rho / l, v[1] * rho / l
    ip = np.array([c * xp + d * yp + cx, e * xp + yp + cy])
    return apply_k(crop, ip), np.linalg.norm(v)


def numeric_grad(f, x0, g, eps=1e-6):
    """g^T d f / d x by central differences; f returns a 2-vector."""
    x0 = np.asarray(x0, dtype=np.float64)
    out = np.zeros_like(x0)
    for i in range(x0.size):
        d = np.zeros_like(x0)
        d[i] = eps * max(1.0, abs(x0[i]))
        out[i] = g @ (f(x0 + d) - f(x0 - d)) / (2 * d[i])
    return out


def spherical_uv(dirw):
    phi = np.arctan2(-dirw[2], dirw[0])
    x = phi / (2 * np.pi)
    x = x - np.floor(x)
    y = 1 - np.arccos(np.clip(dirw[1], -1, 1)) / np.pi
    return np.array([2 * x - 1, 2 * y - 1])


def undistort(dp, dist, iters=50):
    k1, k2, k3, k4, k5, k6, p1, p2 = dist
    m = np.array(dp, dtype=np.float64)
    for _ in range(iters):
        x, y = m
        r2 = x * x + y * y
        rad = (1 + k1 * r2 + k2 * r2 ** 2 + k3 * r2 ** 3) / (1 + k4 * r2 + k5 * r2 ** 2 + k6 * r2 ** 3)
        tx = 2 * p1 * x * y + p2 * (r2 + 2 * x * x)
        ty = p1 * (r2 + 2 * y * y) + 2 * p2 * x * y
        m = np.array([(dp[0] - tx) / rad, (dp[1] - ty) / rad])
    return m
