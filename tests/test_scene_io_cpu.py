"""The scene directory reader (adop_b200/scene_io.py) against hand-written files in the layout of scenes/README.md:59-95 and
against a write -> read round trip; pose inversion against the float64 camera model. No GPU."""
import os

import numpy as np
import pytest

from adop_b200 import capi, scene_io, synth


def _write(path, text):
    with open(path, "w") as f:
        f.write(text)


def test_hand_written_scene_directory(tmp_path):
    d = str(tmp_path)
    _write(os.path.join(d, "dataset.ini"), "[SceneDatasetParams]\nimage_dir = images/\ncamera_files = camera0.ini camera1.ini\n"
                                           "file_point_cloud = cloud.ply\ncamera_type_int = 0\nznear = 0.1\n")
    _write(os.path.join(d, "camera0.ini"), "[SceneCameraParams]\nw = 640\nh = 480\nK = 500 501 320 240 0.5 # fx fy cx cy s\n"
                                           "distortion = -0.1 0.02 0 0 0 0 0.001 -0.002 # 8 paramter distortion model\n")
    _write(os.path.join(d, "camera1.ini"), "[SceneCameraParams]\nw = 320\nh = 200\nK = 250 250 160 100 0\ndistortion = 0 0 0 0 0 0 0 0\n")
    # image 0: identity; image 1: camera at (1, 2, 3) rotated by 90 degrees about z
    s = np.sqrt(0.5)
    _write(os.path.join(d, "poses.txt"), f"0 0 0 1 0 0 0\n0 0 {s} {s} 1 2 3\n")
    _write(os.path.join(d, "camera_indices.txt"), "0\n1\n")
    _write(os.path.join(d, "exposure.txt"), "13.1\n14\n")
    _write(os.path.join(d, "white_balance.txt"), "1 1 1\n1.1 1 0.9\n")
    _write(os.path.join(d, "images.txt"), "0000.jpg\n0001.jpg\n")
    _write(os.path.join(d, "cloud.ply"), "ply\nformat ascii 1.0\nelement vertex 3\nproperty float x\nproperty float y\nproperty float z\n"
                                         "property float nx\nproperty float ny\nproperty float nz\nproperty uchar red\nproperty uchar green\n"
                                         "property uchar blue\nelement face 0\nend_header\n0 0 5 0 0 -1 255 0 0\n1 2 3 0 1 0 0 255 0\n-1 -2 7 1 0 0 0 0 255\n")
    sc = scene_io.load_scene_directory(d)
    a = sc["arrays"]
    assert a["intrinsics"].shape == (2, 13)
    assert np.allclose(a["intrinsics"][0], [500, 501, 320, 240, 0.5, -0.1, 0.02, 0, 0, 0, 0, 0.001, -0.002])
    assert [(v["w"], v["h"], v["image_index"], v["camera_index"], v["camera_model"]) for v in sc["views"]] == [(640, 480, 0, 0, 0), (320, 200, 1, 1, 0)]
    assert np.allclose(a["position"], [[0, 0, 5, 0], [1, 2, 3, 0], [-1, -2, 7, 0]])
    assert a["normal"].tolist() == synth.pack_normals(np.array([[0, 0, -1], [0, 1, 0], [1, 0, 0]], float)).tolist()
    assert sc["color"].tolist() == [[255, 0, 0], [0, 255, 0], [0, 0, 255]]
    assert np.allclose(sc["exposure"], [13.1, 14]) and np.allclose(sc["white_balance"][1], [1.1, 1, 0.9])
    assert sc["images"] == ["0000.jpg", "0001.jpg"] and sc["masks"] == []
    # world -> camera: the camera centre (1, 2, 3) of image 1 maps to the origin of its camera frame
    assert np.allclose(a["poses"][0], [0, 0, 0, 1, 0, 0, 0, 0])
    q, t = a["poses"][1, :4], a["poses"][1, 4:7]
    assert np.allclose(q, [0, 0, -s, s]) and a["poses"][1, 7] == 0
    # the inverse rotation turns (1, 2, 3) into (2, -1, 3): the translation is its negative
    assert np.allclose(t, [-2, 1, -3], atol=1e-12)


def test_round_trip_of_a_synthetic_scene(tmp_path):
    cfg = synth.make_config("c2", n_points=5000, n_views=5, size=(64, 36))
    a = cfg["arrays"]
    rng = np.random.default_rng(0)
    normals = rng.normal(size=(5000, 3))
    normals /= np.linalg.norm(normals, axis=1, keepdims=True)
    colors = rng.integers(0, 256, (5000, 3)).astype(np.uint8)
    # the generator's poses are world -> camera; the files hold camera -> world
    q_cw, t_cw = scene_io.invert_poses(a["poses"][:, :4], a["poses"][:, 4:7])
    cams = [dict(w=64, h=36, K=a["intrinsics"][0, :5], distortion=a["intrinsics"][0, 5:13])]
    scene_io.save_scene_directory(str(tmp_path), a["position"][:, :3], np.concatenate([q_cw, t_cw], axis=1), cams, normals=normals,
                                  colors=colors, exposure=np.linspace(10, 14, 5), white_balance=np.ones((5, 3)),
                                  images=[f"{i:04d}.jpg" for i in range(5)])
    sc = scene_io.load_scene_directory(str(tmp_path))
    b = sc["arrays"]
    assert np.array_equal(b["position"][:, :3], a["position"][:, :3]) and not b["position"][:, 3].any()
    assert np.allclose(b["intrinsics"], a["intrinsics"][:1], rtol=1e-7)
    # quaternions up to sign, translations to rounding
    same = np.minimum(np.abs(b["poses"][:, :4] - a["poses"][:, :4]).max(axis=1), np.abs(b["poses"][:, :4] + a["poses"][:, :4]).max(axis=1))
    assert same.max() < 1e-12 and np.allclose(b["poses"][:, 4:7], a["poses"][:, 4:7], atol=1e-12)
    assert np.array_equal(b["normal"], synth.pack_normals(normals.astype(np.float32)))
    assert np.array_equal(sc["color"], colors) and len(sc["views"]) == 5 and sc["views"][3]["image_index"] == 3


def test_omnidirectional_scene_and_bad_directories(tmp_path):
    c3 = synth.make_config("c3", n_points=100, size=(64, 36))
    intr = c3["arrays"]["intrinsics"][0]
    d = str(tmp_path / "ocam")
    scene_io.save_scene_directory(d, c3["arrays"]["position"][:, :3], [[0, 0, 0, 1, 0, 0, 0]],
                                  [dict(w=64, h=36, op=intr[:5], poly_world2cam=intr[5:])], camera_model=capi.CAMERA_OCAM)
    sc = scene_io.load_scene_directory(d)
    assert sc["views"][0]["camera_model"] == capi.CAMERA_OCAM and np.allclose(sc["arrays"]["intrinsics"][0], intr, rtol=1e-7)
    assert sc["arrays"]["normal"] is None and sc["color"] is None and sc["exposure"] is None
    # more exposure values than poses: the reference asserts (SceneData.cpp:233-238), the reader raises
    _write(os.path.join(d, "exposure.txt"), "1\n2\n")
    with pytest.raises(ValueError, match="exposure"):
        scene_io.load_scene_directory(d)
    os.remove(os.path.join(d, "exposure.txt"))
    os.remove(os.path.join(d, "poses.txt"))
    with pytest.raises(ValueError, match="pose file is required"):
        scene_io.load_scene_directory(d)
