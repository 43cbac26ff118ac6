"""ctypes mirror of include/adop/adop_raster.h.

The same structures serve two libraries with the same call shapes: the CUDA product
(`adop_b200/libadop_raster.so`, device pointers) and — in tests and the CPU-baseline leg of the
benchmark only — the CPU checker (`oracle/libadop_oracle.so`, host pointers).
"""
import ctypes as C
import os

MAX_LAYERS = 8
MAX_CHANNELS = 32

ADOP_OK = 0
CAMERA_PINHOLE_DISTORTION = 0
CAMERA_OCAM = 1

_c_float_p = C.c_void_p  # all data pointers travel as raw addresses


class AdopView(C.Structure):
    """ReducedImageInfo (src/lib/data/SceneData.h:37-47)."""
    _fields_ = [("w", C.c_int32), ("h", C.c_int32), ("image_index", C.c_int32), ("camera_index", C.c_int32),
                ("camera_model", C.c_int32), ("crop", C.c_float * 5)]


class AdopRenderParams(C.Structure):
    """RenderParams (src/lib/data/Settings.h:16-52), compute-relevant fields."""
    _fields_ = [("test_backward_mode", C.c_int32), ("check_normal", C.c_int32), ("dropout", C.c_float),
                ("dropout_seed", C.c_uint32), ("depth_accept", C.c_float), ("ghost_gradients", C.c_int32),
                ("drop_out_radius_threshold", C.c_float), ("drop_out_points_by_radius", C.c_int32),
                ("distortion_gradient_factor", C.c_float), ("K_gradient_factor", C.c_float),
                ("dist_cutoff", C.c_float), ("output_background_mask", C.c_int32),
                ("output_background_mask_value", C.c_float), ("composite_environment_map", C.c_int32)]


class AdopScene(C.Structure):
    _fields_ = [("num_points", C.c_int32), ("num_texels", C.c_int32), ("channels", C.c_int32),
                ("num_images", C.c_int32), ("num_cameras", C.c_int32), ("intrinsics_cols", C.c_int32),
                ("env_h", C.c_int32), ("env_w", C.c_int32),
                ("position", C.c_void_p), ("normal", C.c_void_p), ("index", C.c_void_p), ("texture", C.c_void_p),
                ("background", C.c_void_p), ("poses", C.c_void_p), ("intrinsics", C.c_void_p),
                ("env_map", C.c_void_p), ("texture_interleaved", C.c_void_p),
                ("outlier_position", C.c_void_p), ("outlier_normal", C.c_void_p), ("outlier_index", C.c_void_p),
                ("num_outliers", C.c_int32), ("reserved_", C.c_int32)]


class AdopLayerBuffers(C.Structure):
    _fields_ = [("color", C.c_void_p), ("depth", C.c_void_p), ("weight", C.c_void_p), ("mask", C.c_void_p)]


class AdopForwardIO(C.Structure):
    _fields_ = [("layers", AdopLayerBuffers * MAX_LAYERS), ("dropout_mask", C.c_void_p),
                ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("visible_list", C.c_void_p),
                ("packed_depth", C.c_void_p * MAX_LAYERS), ("touched_points", C.c_void_p), ("touched_texels", C.c_void_p)]


class AdopBackwardIO(C.Structure):
    _fields_ = [("layers", AdopLayerBuffers * MAX_LAYERS), ("grad_color", C.c_void_p * MAX_LAYERS),
                ("dropout_mask", C.c_void_p), ("grad_texture", C.c_void_p), ("grad_background", C.c_void_p),
                ("grad_points", C.c_void_p), ("grad_pose", C.c_void_p), ("count_pose", C.c_void_p),
                ("grad_intrinsics", C.c_void_p), ("count_intrinsics", C.c_void_p), ("grad_env_map", C.c_void_p),
                ("accumulate", C.c_int32), ("normalize", C.c_int32),
                ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("visible_list", C.c_void_p),
                ("grad_texture_interleaved", C.c_void_p), ("grad_env_map_interleaved", C.c_void_p)]


class AdopTonemapParams(C.Structure):
    _fields_ = [("batch", C.c_int32), ("height", C.c_int32), ("width", C.c_int32), ("response_bins", C.c_int32),
                ("vignette_image_w", C.c_int32), ("vignette_image_h", C.c_int32), ("leak", C.c_float),
                ("frame_index", C.c_void_p), ("exposure", C.c_void_p), ("white_balance", C.c_void_p),
                ("vignette", C.c_void_p), ("uv", C.c_void_p), ("response", C.c_void_p)]


class AdopTonemapGrads(C.Structure):
    _fields_ = [("grad_x", C.c_void_p), ("grad_exposure", C.c_void_p), ("grad_white_balance", C.c_void_p),
                ("grad_vignette", C.c_void_p), ("grad_response", C.c_void_p), ("num_frames", C.c_int32),
                ("accumulate", C.c_int32)]


class AdopPeerHandle(C.Structure):
    _fields_ = [("bytes", C.c_ubyte * 64)]


class AdopPeerLayout(C.Structure):
    _fields_ = [("channels", C.c_int32), ("num_texels", C.c_int32), ("num_points", C.c_int32), ("num_images", C.c_int32),
                ("num_cameras", C.c_int32), ("intrinsics_cols", C.c_int32), ("env_h", C.c_int32), ("env_w", C.c_int32),
                ("background", C.c_int32), ("touched", C.c_int32),
                ("off_texture", C.c_size_t), ("off_points", C.c_size_t), ("off_pose", C.c_size_t),
                ("off_count_pose", C.c_size_t), ("off_intrinsics", C.c_size_t), ("off_count_intrinsics", C.c_size_t),
                ("off_background", C.c_size_t), ("off_env_map", C.c_size_t), ("off_touched_texels", C.c_size_t),
                ("off_touched_points", C.c_size_t), ("off_gathered", C.c_size_t), ("total_bytes", C.c_size_t)]


class AdopPeerReduceOut(C.Structure):
    _fields_ = [("grad_texture_shard", C.c_void_p), ("grad_points_shard", C.c_void_p), ("grad_pose", C.c_void_p),
                ("count_pose", C.c_void_p), ("grad_intrinsics", C.c_void_p), ("count_intrinsics", C.c_void_p),
                ("grad_background", C.c_void_p), ("grad_env_map", C.c_void_p), ("normalize", C.c_int32)]


class AdopPeerParamLayout(C.Structure):
    _fields_ = [("channels", C.c_int32), ("num_texels", C.c_int32), ("num_points", C.c_int32), ("reserved", C.c_int32),
                ("off_texture", C.c_size_t), ("off_points", C.c_size_t), ("total_bytes", C.c_size_t)]


class AdopPeerUpdate(C.Structure):
    _fields_ = [("grad_texture_shard", C.c_void_p), ("adam_m", C.c_void_p), ("adam_v", C.c_void_p),
                ("grad_points_shard", C.c_void_p), ("lr_texture", C.c_float), ("beta1", C.c_float), ("beta2", C.c_float),
                ("eps", C.c_float), ("step", C.c_int32), ("lr_points", C.c_float)]


class AdopKernelTime(C.Structure):
    _fields_ = [("name", C.c_char * 48), ("launches", C.c_int32), ("total_ms", C.c_float)]


# every symbol include/adop/adop_raster.h declares
EXPORTED_SYMBOLS = [
    "adop_status_string", "adop_last_error", "adop_render_params_default", "adop_raster_workspace_bytes",
    "adop_raster_workspace_bytes_full",
    "adop_raster_forward", "adop_raster_backward", "adop_raster_normalize_gradients", "adop_apply_tangent",
    "adop_tonemap_forward", "adop_tonemap_backward", "adop_profile_enable", "adop_profile_collect",
    "adop_raster_static_scratch_bytes", "adop_raster_forward_static", "adop_raster_visible_list_ints",
    "adop_texture_interleave", "adop_texture_deinterleave",
    "adop_peer_alloc", "adop_peer_free", "adop_peer_open", "adop_peer_close", "adop_peer_layout_fill",
    "adop_peer_shard_range", "adop_peer_reduce_gradients", "adop_peer_param_layout_fill", "adop_peer_apply_update",
    "adop_points_morton_workspace_bytes", "adop_points_morton_order", "adop_points_permute",
    "adop_points_block_shuffle_order", "adop_points_sort_blocks_by_radius_order",
    "adop_points_knn_workspace_bytes", "adop_points_knn_distance", "adop_points_radius_sample",
]

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG_DIR, "libadop_raster.so")
_lib = None


class AdopError(RuntimeError):
    pass


def load_library():
    """Load the CUDA library. There is no fallback: a missing build is an error."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise AdopError(f"{LIB_PATH} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
                        "(there is no CPU fallback)")
    lib = C.CDLL(LIB_PATH)
    lib.adop_status_string.restype = C.c_char_p
    lib.adop_status_string.argtypes = [C.c_int]
    lib.adop_last_error.restype = C.c_char_p
    lib.adop_render_params_default.argtypes = [C.POINTER(AdopRenderParams)]
    lib.adop_render_params_default.restype = None
    lib.adop_raster_workspace_bytes.restype = C.c_size_t
    lib.adop_raster_workspace_bytes.argtypes = [C.c_int32] * 4
    lib.adop_raster_workspace_bytes_full.restype = C.c_size_t
    lib.adop_raster_workspace_bytes_full.argtypes = [C.c_int32] * 6
    lib.adop_raster_forward.argtypes = [C.POINTER(AdopScene), C.POINTER(AdopView), C.c_int32,
                                        C.POINTER(AdopRenderParams), C.c_int32, C.POINTER(AdopForwardIO), C.c_void_p]
    lib.adop_raster_forward_static.argtypes = lib.adop_raster_forward.argtypes
    lib.adop_raster_forward_static.restype = C.c_int
    lib.adop_raster_static_scratch_bytes.argtypes = []
    lib.adop_raster_static_scratch_bytes.restype = C.c_size_t
    lib.adop_texture_interleave.argtypes = [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p]
    lib.adop_texture_interleave.restype = C.c_int
    lib.adop_texture_deinterleave.argtypes = [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p]
    lib.adop_texture_deinterleave.restype = C.c_int
    lib.adop_raster_visible_list_ints.argtypes = [C.c_int32] * 4
    lib.adop_raster_visible_list_ints.restype = C.c_size_t
    lib.adop_raster_backward.argtypes = [C.POINTER(AdopScene), C.POINTER(AdopView), C.c_int32,
                                         C.POINTER(AdopRenderParams), C.c_int32, C.POINTER(AdopBackwardIO), C.c_void_p]
    lib.adop_raster_normalize_gradients.argtypes = [C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p, C.c_int32,
                                                    C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p]
    lib.adop_apply_tangent.argtypes = [C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p]
    lib.adop_tonemap_forward.argtypes = [C.POINTER(AdopTonemapParams), C.c_void_p, C.c_void_p, C.c_void_p]
    lib.adop_tonemap_backward.argtypes = [C.POINTER(AdopTonemapParams), C.c_void_p, C.c_void_p,
                                          C.POINTER(AdopTonemapGrads), C.c_void_p]
    lib.adop_peer_alloc.argtypes = [C.c_size_t, C.POINTER(C.c_void_p), C.POINTER(AdopPeerHandle)]
    lib.adop_peer_free.argtypes = [C.c_void_p]
    lib.adop_peer_open.argtypes = [C.POINTER(AdopPeerHandle), C.POINTER(C.c_void_p)]
    lib.adop_peer_close.argtypes = [C.c_void_p]
    lib.adop_peer_layout_fill.argtypes = [C.POINTER(AdopPeerLayout)]
    lib.adop_peer_shard_range.argtypes = [C.c_int32, C.c_int32, C.c_int32, C.POINTER(C.c_int32), C.POINTER(C.c_int32)]
    lib.adop_peer_shard_range.restype = None
    lib.adop_peer_reduce_gradients.argtypes = [C.POINTER(C.c_void_p), C.c_int32, C.c_int32, C.POINTER(AdopPeerLayout),
                                               C.POINTER(AdopPeerReduceOut), C.c_void_p]
    lib.adop_peer_param_layout_fill.argtypes = [C.POINTER(AdopPeerParamLayout)]
    lib.adop_peer_apply_update.argtypes = [C.POINTER(C.c_void_p), C.c_int32, C.c_int32, C.POINTER(AdopPeerParamLayout),
                                           C.POINTER(AdopPeerUpdate), C.c_void_p]
    for name in ("adop_peer_alloc", "adop_peer_free", "adop_peer_open", "adop_peer_close", "adop_peer_layout_fill",
                 "adop_peer_reduce_gradients", "adop_peer_param_layout_fill", "adop_peer_apply_update"):
        getattr(lib, name).restype = C.c_int
    lib.adop_points_morton_workspace_bytes.argtypes = [C.c_int32]
    lib.adop_points_morton_workspace_bytes.restype = C.c_size_t
    lib.adop_points_morton_order.argtypes = [C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]
    lib.adop_points_morton_order.restype = C.c_int
    lib.adop_points_block_shuffle_order.argtypes = [C.c_int32, C.c_int32, C.c_uint32, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]
    lib.adop_points_block_shuffle_order.restype = C.c_int
    lib.adop_points_sort_blocks_by_radius_order.argtypes = [C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p]
    lib.adop_points_sort_blocks_by_radius_order.restype = C.c_int
    lib.adop_points_knn_workspace_bytes.argtypes = [C.c_int32]
    lib.adop_points_knn_workspace_bytes.restype = C.c_size_t
    lib.adop_points_knn_distance.argtypes = [C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]
    lib.adop_points_knn_distance.restype = C.c_int
    lib.adop_points_radius_sample.argtypes = [C.c_void_p, C.c_int32, C.c_uint32, C.c_void_p, C.c_void_p]
    lib.adop_points_radius_sample.restype = C.c_int
    lib.adop_points_permute.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p]
    lib.adop_points_permute.restype = C.c_int
    lib.adop_profile_enable.argtypes = [C.c_int32]
    lib.adop_profile_enable.restype = C.c_int
    lib.adop_profile_collect.argtypes = [C.POINTER(AdopKernelTime), C.c_int32]
    lib.adop_profile_collect.restype = C.c_int32
    for name in ("adop_raster_forward", "adop_raster_backward", "adop_raster_normalize_gradients",
                 "adop_apply_tangent", "adop_tonemap_forward", "adop_tonemap_backward"):
        getattr(lib, name).restype = C.c_int
    _lib = lib
    return lib


def check(status, what):
    if status != ADOP_OK:
        lib = load_library()
        raise AdopError(f"{what}: {lib.adop_status_string(status).decode()} ({status}) "
                        f"{lib.adop_last_error().decode()}")


def profile_enable(on=True):
    """Bracket every kernel launch of the library with CUDA events (the CudaTimerSystem scopes of the reference)."""
    load_library().adop_profile_enable(1 if on else 0)


def profile_collect():
    """-> {kernel name: (launches, total ms)}; synchronises the recorded events and resets the collection."""
    lib = load_library()
    buf = (AdopKernelTime * 64)()
    n = lib.adop_profile_collect(buf, 64)
    if n < 0:
        raise AdopError("adop_profile_collect: CUDA error while reading events")
    return {buf[i].name.decode(): (buf[i].launches, buf[i].total_ms) for i in range(min(n, 64))}


def default_render_params():
    """RenderParams defaults of Settings.h:22-52 (does not need the CUDA library)."""
    p = AdopRenderParams()
    p.test_backward_mode = 0
    p.check_normal = 1
    p.dropout = 0.25
    p.dropout_seed = 0
    p.depth_accept = 0.01
    p.ghost_gradients = 0
    p.drop_out_radius_threshold = 0.6
    p.drop_out_points_by_radius = 1
    p.distortion_gradient_factor = 0.005
    p.K_gradient_factor = 0.5
    p.dist_cutoff = 2.0
    p.output_background_mask = 0
    p.output_background_mask_value = 0.0
    p.composite_environment_map = 0
    return p


def layer_sizes(w, h, num_layers):
    """Integer halving per layer (PointRenderer.cu:1015-1016)."""
    out = []
    for _ in range(num_layers):
        out.append((w, h))
        w //= 2
        h //= 2
    return out


def make_views(view_dicts):
    arr = (AdopView * len(view_dicts))()
    for a, v in zip(arr, view_dicts):
        a.w, a.h = int(v["w"]), int(v["h"])
        a.image_index = int(v["image_index"])
        a.camera_index = int(v.get("camera_index", 0))
        a.camera_model = int(v.get("camera_model", CAMERA_PINHOLE_DISTORTION))
        crop = v.get("crop", (1.0, 1.0, 0.0, 0.0, 0.0))
        for i in range(5):
            a.crop[i] = float(crop[i])
    return arr
