"""Reads and writes an ADOP scene directory (scenes/README.md:59-95; SceneData::SceneData, SceneData.cpp:36-263) as the arrays
the rasterizer takes.

    dataset.ini          [SceneDatasetParams]: image_dir, mask_dir, camera_files, file_point_cloud, camera_type_int, ...
    camera*.ini          [SceneCameraParams]: w, h, K = fx fy cx cy s, distortion = k1 .. k6 p1 p2,
                         op = c d e cx cy, poly_world2cam, poly_cam2world (omnidirectional model)
    poses.txt            per image: qx qy qz qw tx ty tz, camera -> world
    camera_indices.txt   per image: index into camera_files        (optional: all 0)
    exposure.txt         per image: EV                             (optional)
    white_balance.txt    per image: r g b                          (optional)
    images.txt, masks.txt  file names                              (kept as lists)
    point_cloud.ply      positions, optional normals and colours (ASCII or binary little-endian PLY)

The operator wants world -> camera poses (PoseModuleImpl stores pose.inverse(), NeuralStructure.cpp:13-27), 10-bit packed
normals and one intrinsics row per camera: those conversions happen here. The reference's cached `point_cloud.bin` is a
saiga format that is not part of the reference tree and is not read; the preprocessing that produces it from the PLY file
(SceneData.cpp:96-118) is adop_b200.preprocess on the GPU. Host-side file handling: numpy only, no GPU needed.
"""
import configparser
import os

import numpy as np

from . import capi


def _read_ini(path, section):
    cp = configparser.ConfigParser(inline_comment_prefixes=("#", ";"), strict=False)
    cp.optionxform = str
    with open(path) as f:
        text = f.read()
    if not text.lstrip().startswith("["):
        text = f"[{section}]\n" + text
    cp.read_string(text)
    sec = section if cp.has_section(section) else cp.sections()[0]
    return dict(cp[sec])


def _numbers(text):
    return [float(t) for t in text.replace(",", " ").split()]


def _lines(path):
    if not os.path.exists(path):
        return []
    with open(path) as f:
        return [ln.strip() for ln in f if ln.strip()]


def invert_poses(q_xyzw, t):
    """camera -> world (unit quaternion xyzw, translation) to world -> camera, in float64: q' = conj(q), t' = -R(q') t."""
    q = np.asarray(q_xyzw, np.float64)
    q = q / np.linalg.norm(q, axis=1, keepdims=True)
    qi = q * np.array([-1.0, -1.0, -1.0, 1.0])
    x, y, z, w = qi[:, 0], qi[:, 1], qi[:, 2], qi[:, 3]
    R = np.stack([1 - 2 * (y * y + z * z), 2 * (x * y - z * w), 2 * (x * z + y * w),
                  2 * (x * y + z * w), 1 - 2 * (x * x + z * z), 2 * (y * z - x * w),
                  2 * (x * z - y * w), 2 * (y * z + x * w), 1 - 2 * (x * x + y * y)], axis=1).reshape(-1, 3, 3)
    ti = -np.einsum("nij,nj->ni", R, np.asarray(t, np.float64))
    return qi, ti


_PLY_TYPES = {"char": "i1", "uchar": "u1", "short": "i2", "ushort": "u2", "int": "i4", "uint": "u4", "float": "f4", "double": "f8",
              "int8": "i1", "uint8": "u1", "int16": "i2", "uint16": "u2", "int32": "i4", "uint32": "u4", "float32": "f4", "float64": "f8"}


def read_ply_vertices(path):
    """-> dict of per-vertex columns (x, y, z, optionally nx ny nz, red green blue alpha) of an ASCII or binary
    little-endian PLY file; other elements (faces) are ignored, list properties on the vertex element are not supported."""
    with open(path, "rb") as f:
        if f.readline().strip() != b"ply":
            raise ValueError("not a PLY file")
        fmt, n_vertex, props, in_vertex = None, 0, [], False
        while True:
            line = f.readline()
            if not line:
                raise ValueError("PLY header without end_header")
            tok = line.decode("ascii", "replace").split()
            if not tok:
                continue
            if tok[0] == "format":
                fmt = tok[1]
            elif tok[0] == "element":
                in_vertex = tok[1] == "vertex"
                if in_vertex:
                    n_vertex = int(tok[2])
            elif tok[0] == "property" and in_vertex:
                if tok[1] == "list":
                    raise ValueError("list properties on the vertex element are not supported")
                props.append((tok[2], _PLY_TYPES[tok[1]]))
            elif tok[0] == "end_header":
                break
        if fmt == "ascii":
            rows = np.loadtxt(f, max_rows=n_vertex, ndmin=2, dtype=np.float64) if n_vertex else np.zeros((0, len(props)))
            return {name: rows[:, k].astype(dt) for k, (name, dt) in enumerate(props)}
        if fmt != "binary_little_endian":
            raise ValueError(f"PLY format {fmt} is not supported")
        dtype = np.dtype([(name, "<" + dt) for name, dt in props])
        data = np.frombuffer(f.read(n_vertex * dtype.itemsize), dtype=dtype, count=n_vertex)
        return {name: np.ascontiguousarray(data[name]) for name, _ in props}


def write_ply_vertices(path, xyz, normals=None, colors=None):
    """Binary little-endian PLY with float positions, optional float normals and uchar rgb colours."""
    n = len(xyz)
    fields, cols = [("x", "<f4"), ("y", "<f4"), ("z", "<f4")], [xyz[:, 0], xyz[:, 1], xyz[:, 2]]
    if normals is not None:
        fields += [("nx", "<f4"), ("ny", "<f4"), ("nz", "<f4")]
        cols += [normals[:, 0], normals[:, 1], normals[:, 2]]
    if colors is not None:
        fields += [("red", "u1"), ("green", "u1"), ("blue", "u1")]
        cols += [colors[:, 0], colors[:, 1], colors[:, 2]]
    data = np.zeros(n, dtype=np.dtype(fields))
    for (name, _), c in zip(fields, cols):
        data[name] = c
    names = {"<f4": "float", "u1": "uchar"}
    with open(path, "wb") as f:
        f.write(b"ply\nformat binary_little_endian 1.0\n")
        f.write(f"element vertex {n}\n".encode())
        for name, dt in fields:
            f.write(f"property {names[dt]} {name}\n".encode())
        f.write(b"end_header\n")
        f.write(data.tobytes())


def pack_normals(n):
    """[M,3] vectors -> the library's 10-bit packing x | y<<10 | z<<20 of the normalised vector."""
    n = np.asarray(n, np.float64)
    n = n / np.maximum(np.linalg.norm(n, axis=1, keepdims=True), 1e-30)
    q = np.round((n + 1) * 0.5 * 1023).astype(np.uint32)
    return (q[:, 0] | (q[:, 1] << 10) | (q[:, 2] << 20)).astype(np.int32)


def load_scene_directory(path):
    """-> dict with
         arrays   position [N,4] f32 (w = 0: the drop-out radius comes from the preprocessing), normal [N] i32 or None,
                  poses [I,8] f64 world -> camera, intrinsics [K,13] f32 (pinhole) or [K,5+m] (omnidirectional)
         views    one dict per image: w, h, image_index, camera_index, camera_model (what PointRasterizer.forward takes)
         color [N,3] u8 or None, exposure [I] f32 or None, white_balance [I,3] f32 or None, images, masks (file names),
         dataset (the dataset.ini entries as strings)"""
    ds = _read_ini(os.path.join(path, "dataset.ini"), "SceneDatasetParams")
    model = int(ds.get("camera_type_int", "0"))
    cam_files = ds.get("camera_files", "camera.ini").split()
    cams = [_read_ini(os.path.join(path, f), "SceneCameraParams") for f in cam_files]
    if not cams:
        raise ValueError("a scene needs at least one camera file")
    if model == capi.CAMERA_OCAM:
        rows = [_numbers(c["op"]) + _numbers(c["poly_world2cam"]) for c in cams]
        if len({len(r) for r in rows}) != 1:
            raise ValueError("all omnidirectional cameras of a scene need polynomials of one length")
    else:
        rows = [_numbers(c["K"]) + _numbers(c.get("distortion", "0 0 0 0 0 0 0 0")) for c in cams]
        if any(len(r) != 13 for r in rows):
            raise ValueError("K has 5 entries (fx fy cx cy s) and distortion 8 (k1 .. k6 p1 p2)")
    intrinsics = np.asarray(rows, np.float32)
    pose_rows = np.asarray([_numbers(ln)[:7] for ln in _lines(os.path.join(path, "poses.txt"))], np.float64)
    if pose_rows.size == 0:
        raise ValueError("the pose file is required")   # SceneData.cpp:143
    q, t = invert_poses(pose_rows[:, :4], pose_rows[:, 4:7])
    poses = np.zeros((len(q), 8), np.float64)
    poses[:, :4], poses[:, 4:7] = q, t
    n_img = len(poses)
    idx = [int(ln) for ln in _lines(os.path.join(path, "camera_indices.txt"))] or [0] * n_img
    exposure = np.asarray([_numbers(ln)[0] for ln in _lines(os.path.join(path, "exposure.txt"))], np.float32)
    wb = np.asarray([_numbers(ln)[:3] for ln in _lines(os.path.join(path, "white_balance.txt"))], np.float32)
    images, masks = _lines(os.path.join(path, "images.txt")), _lines(os.path.join(path, "masks.txt"))
    for name, count in (("camera_indices", len(idx)), ("exposure", len(exposure) or n_img), ("white_balance", len(wb) or n_img),
                        ("images", len(images) or n_img), ("masks", len(masks) or n_img)):
        if count != n_img:
            raise ValueError(f"{name}: {count} entries for {n_img} poses")   # the asserts of SceneData.cpp:233-238
    if max(idx) >= len(cams) or min(idx) < 0:
        raise ValueError("camera_indices.txt names a camera that has no file")
    views = [dict(w=int(cams[c]["w"]), h=int(cams[c]["h"]), image_index=i, camera_index=c, camera_model=model)
             for i, c in enumerate(idx)]
    v = read_ply_vertices(os.path.join(path, ds.get("file_point_cloud", "point_cloud.ply")))
    n = len(v["x"])
    position = np.zeros((n, 4), np.float32)
    position[:, 0], position[:, 1], position[:, 2] = v["x"], v["y"], v["z"]
    normal = pack_normals(np.stack([v["nx"], v["ny"], v["nz"]], axis=1)) if all(k in v for k in ("nx", "ny", "nz")) else None
    color = np.stack([v["red"], v["green"], v["blue"]], axis=1).astype(np.uint8) if all(k in v for k in ("red", "green", "blue")) else None
    return dict(arrays=dict(position=position, normal=normal, poses=poses, intrinsics=intrinsics), views=views, color=color,
                exposure=exposure if len(exposure) else None, white_balance=wb if len(wb) else None, images=images, masks=masks,
                dataset=ds)


def save_scene_directory(path, xyz, poses_camera_to_world, cameras, camera_indices=None, normals=None, colors=None,
                         exposure=None, white_balance=None, images=None, camera_model=capi.CAMERA_PINHOLE_DISTORTION):
    """Writes the files load_scene_directory reads. poses_camera_to_world [I,7] = qx qy qz qw tx ty tz; cameras: list of
    dicts with w, h and K [5] + distortion [8] (pinhole) or op [5] + poly_world2cam (omnidirectional)."""
    os.makedirs(path, exist_ok=True)
    names = [f"camera{k}.ini" for k in range(len(cameras))]
    with open(os.path.join(path, "dataset.ini"), "w") as f:
        f.write("[SceneDatasetParams]\nimage_dir = color/\nmask_dir = not set\n")
        f.write("camera_files = " + " ".join(names) + "\n")
        f.write(f"file_point_cloud = point_cloud.ply\nfile_point_cloud_compressed = point_cloud.bin\ncamera_type_int = {int(camera_model)}\n")

    def fmt(vals):
        return " ".join(f"{float(x):.15e}" for x in vals)

    for name, c in zip(names, cameras):
        with open(os.path.join(path, name), "w") as f:
            f.write(f"[SceneCameraParams]\nw = {int(c['w'])}\nh = {int(c['h'])}\n")
            if camera_model == capi.CAMERA_OCAM:
                f.write(f"op = {fmt(c['op'])} # c d e cx cy\npoly_world2cam = {fmt(c['poly_world2cam'])}\n")
            else:
                f.write(f"K = {fmt(c['K'])} # fx fy cx cy s\ndistortion = {fmt(c.get('distortion', [0] * 8))}\n")
    with open(os.path.join(path, "poses.txt"), "w") as f:
        for row in np.asarray(poses_camera_to_world, np.float64):
            f.write(" ".join(f"{x:.17g}" for x in row[:7]) + "\n")
    n_img = len(poses_camera_to_world)
    with open(os.path.join(path, "camera_indices.txt"), "w") as f:
        f.write("\n".join(str(int(i)) for i in (camera_indices if camera_indices is not None else [0] * n_img)) + "\n")
    if exposure is not None:
        with open(os.path.join(path, "exposure.txt"), "w") as f:
            f.write("\n".join(f"{float(e):.9g}" for e in exposure) + "\n")
    if white_balance is not None:
        with open(os.path.join(path, "white_balance.txt"), "w") as f:
            f.write("\n".join(" ".join(f"{float(x):.9g}" for x in row) for row in white_balance) + "\n")
    if images is not None:
        with open(os.path.join(path, "images.txt"), "w") as f:
            f.write("\n".join(images) + "\n")
    write_ply_vertices(os.path.join(path, "point_cloud.ply"), np.asarray(xyz, np.float32),
                       None if normals is None else np.asarray(normals, np.float32), colors)
