"""Point-cloud preprocessing on the GPU (host mirror of the adop_points_* entry points).

The reference reorders a scene's cloud once, when the scene is first loaded (SceneData.cpp:96-118: ReorderMorton64,
RandomBlockShuffle, ComputeRadius, SortBlocksByRadius); the Morton reorder is the part the rasterizer's memory behaviour
depends on and the one implemented here. torch is used for device memory and the stream only."""
import ctypes as C

import torch

from . import capi


def morton_order(position):
    """position: [N,4] float32 CUDA tensor -> [N] int32 CUDA tensor, order[i] = index of the point that comes i-th
    along the 21-bit-per-axis Morton curve over the cloud's bounding box (ties keep their order)."""
    if not (position.is_cuda and position.dtype == torch.float32 and position.dim() == 2 and position.shape[1] == 4
            and position.is_contiguous()):
        raise ValueError("position must be a contiguous [N,4] float32 CUDA tensor")
    lib = capi.load_library()
    n = position.shape[0]
    with torch.cuda.device(position.device):
        order = torch.empty(n, dtype=torch.int32, device=position.device)
        ws = torch.empty(lib.adop_points_morton_workspace_bytes(n), dtype=torch.uint8, device=position.device)
        stream = torch.cuda.current_stream(position.device).cuda_stream
        capi.check(lib.adop_points_morton_order(position.data_ptr(), n, order.data_ptr(), ws.data_ptr(), ws.numel(),
                                                C.c_void_p(stream)), "adop_points_morton_order")
    return order


def block_shuffle_order(num_points, device, block=256, seed=0):
    """RandomBlockShuffle(256): [N] int32 order that moves whole blocks of `block` points into a seeded pseudo-random order."""
    lib = capi.load_library()
    device = torch.device(device)
    with torch.cuda.device(device):
        order = torch.empty(num_points, dtype=torch.int32, device=device)
        ws = torch.empty(max(lib.adop_points_morton_workspace_bytes(num_points), 4096), dtype=torch.uint8, device=device)
        stream = torch.cuda.current_stream(device).cuda_stream
        capi.check(lib.adop_points_block_shuffle_order(num_points, block, seed, order.data_ptr(), ws.data_ptr(), ws.numel(),
                                                       C.c_void_p(stream)), "adop_points_block_shuffle_order")
    return order


def sort_blocks_by_radius_order(position):
    """SortBlocksByRadius(256): [N] int32 order that sorts every full block of 256 points by position[:, 3] (then index)."""
    lib = capi.load_library()
    with torch.cuda.device(position.device):
        order = torch.empty(position.shape[0], dtype=torch.int32, device=position.device)
        stream = torch.cuda.current_stream(position.device).cuda_stream
        capi.check(lib.adop_points_sort_blocks_by_radius_order(position.data_ptr(), position.shape[0], order.data_ptr(),
                                                               C.c_void_p(stream)), "adop_points_sort_blocks_by_radius_order")
    return order


def knn_distance(position, k=4):
    """ComputeRadius' first half: [N] float32 distance of every point to its k-th nearest other point (exact)."""
    lib = capi.load_library()
    n = position.shape[0]
    with torch.cuda.device(position.device):
        out = torch.empty(n, dtype=torch.float32, device=position.device)
        ws = torch.empty(lib.adop_points_knn_workspace_bytes(n), dtype=torch.uint8, device=position.device)
        stream = torch.cuda.current_stream(position.device).cuda_stream
        capi.check(lib.adop_points_knn_distance(position.data_ptr(), n, k, out.data_ptr(), ws.data_ptr(), ws.numel(),
                                                C.c_void_p(stream)), "adop_points_knn_distance")
    return out


def radius_sample(distance, seed=0):
    """ComputeRadius' second half: drop-out radius = distance * sqrt(1 / u), u in (0,1] from the counter hash."""
    lib = capi.load_library()
    with torch.cuda.device(distance.device):
        out = torch.empty_like(distance)
        stream = torch.cuda.current_stream(distance.device).cuda_stream
        capi.check(lib.adop_points_radius_sample(distance.data_ptr(), distance.numel(), seed, out.data_ptr(), C.c_void_p(stream)),
                   "adop_points_radius_sample")
    return out


def permute_rows(t, order):
    """out[i] = t[order[i]] along the first dimension; rows of 4, 8, 12, 16, 32 or 64 bytes."""
    if not (t.is_cuda and t.is_contiguous() and order.is_cuda and order.dtype == torch.int32):
        raise ValueError("contiguous CUDA tensors, int32 order")
    n = t.shape[0]
    row_bytes = t[0].numel() * t.element_size() if t.dim() > 1 else t.element_size()
    lib = capi.load_library()
    out = torch.empty_like(t)
    with torch.cuda.device(t.device):
        stream = torch.cuda.current_stream(t.device).cuda_stream
        capi.check(lib.adop_points_permute(t.data_ptr(), out.data_ptr(), order.data_ptr(), n, row_bytes, C.c_void_p(stream)),
                   "adop_points_permute")
    return out


def reorder_scene(scene):
    """A Scene (raster.py) with its points in Morton order: positions, normals, index; with the identity index the
    descriptor planes move with the points, otherwise the index keeps pointing at the unmoved descriptors."""
    from .raster import Scene
    order = morton_order(scene.position)
    fields = {k: getattr(scene, k) for k in ("position", "normal", "index", "texture", "background", "poses", "intrinsics", "env_map")}
    fields["position"] = permute_rows(scene.position, order)
    if scene.normal is not None:
        fields["normal"] = permute_rows(scene.normal, order)
    if scene.index is not None:
        fields["index"] = permute_rows(scene.index, order)
    else:
        fields["texture"] = torch.stack([permute_rows(plane.contiguous(), order) for plane in scene.texture])
    return Scene(**fields), order
