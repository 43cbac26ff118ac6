"""Writes tests/golden/projection_f64.npz: known-answer vectors for the two camera models.

The reference ships no golden vectors for this path, and its camera arithmetic (saiga) is not available to run. These
vectors come from the independent float64 model in tests/f64_model.py (published pinhole + OpenCV rational distortion
and Scaramuzza omnidirectional models); the CPU checker must reproduce them within float32 rounding.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from adop_b200 import synth  # noqa: E402
from tests import f64_model as fm  # noqa: E402


def main():
    rng = np.random.default_rng(1234)
    out = {}
    n = 64
    # pinhole + 8-coefficient distortion, skew, non-trivial crop
    pts = np.stack([rng.normal(0, 1, n), rng.normal(0, 1, n), rng.uniform(2, 6, n), np.full(n, 0.01)], 1).astype(np.float32)
    pose = synth.look_at_pose((0.4, -0.2, -1.5), (0.0, 0.1, 4.0))[None]
    intr = np.array([[430.0, 415.0, 255.0, 200.0, 0.5, -0.1, 0.02, 0.003, 0.008, -0.004, 0.001, 0.002, -0.001]], np.float32)
    crop = np.array([0.8, 1.2, 10.0, -5.0, 0.02], np.float32)
    T = fm.pose_matrix(pose[0])
    exp = np.zeros((n, 3))
    for i, p in enumerate(pts):
        ip, z = fm.project_pinhole(T, intr[0, :5].astype(np.float64), intr[0, 5:].astype(np.float64), crop.astype(np.float64),
                                   p[:3].astype(np.float64))
        exp[i] = [ip[0], ip[1], z] if z > 0 else [0, 0, 0]
    out.update(pinhole_points=pts, pinhole_pose=pose, pinhole_intrinsics=intr, pinhole_crop=crop,
               pinhole_wh=np.array([512, 384]), pinhole_expected=exp.astype(np.float32))
    # omnidirectional
    pts = np.stack([rng.uniform(-6, 6, n), rng.uniform(-6, 6, n), rng.uniform(0.5, 4, n), np.full(n, 0.01)], 1).astype(np.float32)
    pose = synth.look_at_pose((0.1, 0.2, -0.4), (0.0, 0.0, 3.0))[None]
    coef, _ = synth.ocam_world2cam_poly()
    intr = np.concatenate([[1.01, 0.002, -0.003, 960.0, 540.0], coef]).astype(np.float32)[None]
    crop = np.array([1.0, 1.0, 0.0, 0.0, 0.0], np.float32)
    T = fm.pose_matrix(pose[0])
    exp = np.zeros((n, 3))
    for i, p in enumerate(pts):
        ip, z = fm.project_ocam(T, intr[0, :5].astype(np.float64), intr[0, 5:].astype(np.float64), crop.astype(np.float64),
                                p[:3].astype(np.float64))
        exp[i] = [ip[0], ip[1], z]
    out.update(ocam_points=pts, ocam_pose=pose, ocam_intrinsics=intr, ocam_crop=crop, ocam_wh=np.array([1920, 1080]),
               ocam_expected=exp.astype(np.float32))
    np.savez(os.path.join(ROOT, "tests", "golden", "projection_f64.npz"), **out)
    print("wrote projection_f64.npz")


if __name__ == "__main__":
    main()
