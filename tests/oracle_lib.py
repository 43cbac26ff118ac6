"""ctypes binding of the CPU checker (oracle/libadop_oracle.so). Test infrastructure only."""
import ctypes as C
import os
import subprocess

import numpy as np

from adop_b200 import capi
from adop_b200.raster import fill_scene_struct

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
ORACLE_LIB = os.path.join(ORACLE_DIR, "libadop_oracle.so")


def _nptr(a):
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data


class Oracle:
    def __init__(self):
        if not os.path.exists(ORACLE_LIB):
            subprocess.run(["make", "-C", ORACLE_DIR], check=True, capture_output=True)
        lib = C.CDLL(ORACLE_LIB)
        lib.adop_oracle_forward.argtypes = [C.POINTER(capi.AdopScene), C.POINTER(capi.AdopView), C.c_int,
                                            C.POINTER(capi.AdopRenderParams), C.c_int, C.POINTER(capi.AdopForwardIO), C.c_int]
        lib.adop_oracle_backward.argtypes = [C.POINTER(capi.AdopScene), C.POINTER(capi.AdopView), C.c_int,
                                             C.POINTER(capi.AdopRenderParams), C.c_int, C.POINTER(capi.AdopBackwardIO), C.c_int]
        lib.adop_oracle_apply_tangent.argtypes = [C.c_void_p, C.c_void_p, C.c_int]
        lib.adop_oracle_tonemap_forward.argtypes = [C.POINTER(capi.AdopTonemapParams), C.c_void_p, C.c_void_p]
        lib.adop_oracle_tonemap_backward.argtypes = [C.POINTER(capi.AdopTonemapParams), C.c_void_p, C.c_void_p,
                                                     C.POINTER(capi.AdopTonemapGrads)]
        for f, r, a in (("adop_oracle_atan", C.c_float, [C.c_float]), ("adop_oracle_atan2", C.c_float, [C.c_float, C.c_float]),
                        ("adop_oracle_acos", C.c_float, [C.c_float]), ("adop_oracle_round", C.c_int, [C.c_float]),
                        ("adop_oracle_hash", C.c_uint32, [C.c_uint32] * 3),
                        ("adop_oracle_dropout", C.c_int, [C.c_float, C.c_uint32, C.c_uint32, C.c_uint32]),
                        ("adop_oracle_pack_normal", C.c_int32, [C.c_float] * 3),
                        ("adop_oracle_unpack_normal", None, [C.c_int32, C.c_void_p]),
                        ("adop_oracle_project", None, [C.POINTER(capi.AdopScene), C.POINTER(capi.AdopView),
                                                       C.POINTER(capi.AdopRenderParams), C.c_void_p]),
                        ("adop_oracle_project_hot", C.c_int, [C.POINTER(capi.AdopScene), C.POINTER(capi.AdopView),
                                                              C.POINTER(capi.AdopRenderParams), C.c_void_p]),
                        ("adop_oracle_project_backward", C.c_int, [C.POINTER(capi.AdopScene), C.POINTER(capi.AdopView),
                                                                  C.POINTER(capi.AdopRenderParams), C.c_int, C.c_float,
                                                                  C.c_float, C.c_void_p]),
                        ("adop_oracle_env_uv", None, [C.POINTER(capi.AdopScene), C.POINTER(capi.AdopView), C.c_int, C.c_void_p]),
                        ("adop_oracle_max_threads", C.c_int, [])):
            getattr(lib, f).restype = r
            getattr(lib, f).argtypes = a
        self.lib = lib

    # -- rasterizer ----------------------------------------------------------------------------------
    def forward(self, arrays, views, params, num_layers, dropout_mask=None, threads=1, packed_depth=False):
        va = views if isinstance(views, C.Array) else capi.make_views(views)
        B = len(va)
        sc = fill_scene_struct(arrays, _nptr)
        ch = sc.channels
        sizes = capi.layer_sizes(va[0].w, va[0].h, num_layers)
        out = dict(colors=[np.zeros((B, ch, h, w), np.float32) for w, h in sizes],
                   depths=[np.zeros((B, 1, h, w), np.float32) for w, h in sizes],
                   weights=[np.zeros((B, 1, h, w), np.float32) for w, h in sizes],
                   masks=[np.zeros((B, 1, h, w), np.float32) for w, h in sizes] if params.output_background_mask else [])
        io = capi.AdopForwardIO()
        for l in range(num_layers):
            io.layers[l].color = _nptr(out["colors"][l])
            io.layers[l].depth = _nptr(out["depths"][l])
            io.layers[l].weight = _nptr(out["weights"][l])
            io.layers[l].mask = _nptr(out["masks"][l]) if out["masks"] else None
        io.dropout_mask = _nptr(dropout_mask) if dropout_mask is not None else None
        if packed_depth:
            out["packed"] = [np.zeros((B, 1, h, w), np.uint64) for w, h in sizes]
            for l in range(num_layers):
                io.packed_depth[l] = _nptr(out["packed"][l])
        st = self.lib.adop_oracle_forward(C.byref(sc), va, B, C.byref(params), num_layers, C.byref(io), threads)
        assert st == 0, st
        out["views"] = va
        return out

    def backward(self, arrays, views, params, num_layers, fwd, grad_colors, want_points=True, want_pose=True,
                 want_intrinsics=True, want_env=False, dropout_mask=None, normalize=True, threads=1):
        va = views if isinstance(views, C.Array) else capi.make_views(views)
        B = len(va)
        sc = fill_scene_struct(arrays, _nptr)
        out = dict(texture=np.zeros_like(arrays["texture"]), background=np.zeros_like(arrays["background"]),
                   points=np.zeros_like(arrays["position"]) if want_points else None,
                   pose=np.zeros((sc.num_images, 6), np.float64) if want_pose else None,
                   count_pose=np.zeros(sc.num_images, np.float32) if want_pose else None,
                   intrinsics=np.zeros_like(arrays["intrinsics"]) if want_intrinsics else None,
                   count_intrinsics=np.zeros(sc.num_cameras, np.float32) if want_intrinsics else None,
                   env_map=np.zeros_like(arrays["env_map"]) if (want_env and arrays.get("env_map") is not None) else None)
        io = capi.AdopBackwardIO()
        for l in range(num_layers):
            io.layers[l].color = _nptr(fwd["colors"][l])
            io.layers[l].depth = _nptr(fwd["depths"][l])
            io.layers[l].weight = _nptr(fwd["weights"][l])
            io.grad_color[l] = _nptr(grad_colors[l])
        io.dropout_mask = _nptr(dropout_mask) if dropout_mask is not None else None

        def p(name):
            return _nptr(out[name]) if out[name] is not None else None

        io.grad_texture, io.grad_background, io.grad_points = p("texture"), p("background"), p("points")
        io.grad_pose, io.count_pose = p("pose"), p("count_pose")
        io.grad_intrinsics, io.count_intrinsics = p("intrinsics"), p("count_intrinsics")
        io.grad_env_map = p("env_map")
        io.accumulate = 0
        io.normalize = 1 if normalize else 0
        st = self.lib.adop_oracle_backward(C.byref(sc), va, B, C.byref(params), num_layers, C.byref(io), threads)
        assert st == 0, st
        return out

    def project(self, arrays, view, params):
        va = capi.make_views([view])
        sc = fill_scene_struct(arrays, _nptr)
        out = np.zeros((sc.num_points, 4), np.float32)
        self.lib.adop_oracle_project(C.byref(sc), va, C.byref(params), _nptr(out))
        return out

    def project_hot(self, arrays, view, params):
        """The five-vector form of the projection; None when the view's camera does not allow it."""
        va = capi.make_views([view])
        sc = fill_scene_struct(arrays, _nptr)
        out = np.zeros((sc.num_points, 4), np.float32)
        ok = self.lib.adop_oracle_project_hot(C.byref(sc), va, C.byref(params), _nptr(out))
        return out if ok else None

    def project_backward(self, arrays, view, params, point, gx, gy):
        va = capi.make_views([view])
        sc = fill_scene_struct(arrays, _nptr)
        out = np.zeros(22, np.float32)
        ok = self.lib.adop_oracle_project_backward(C.byref(sc), va, C.byref(params), point, gx, gy, _nptr(out))
        return ok, out

    def env_uv(self, arrays, view, layer):
        va = capi.make_views([view])
        sc = fill_scene_struct(arrays, _nptr)
        w, h = capi.layer_sizes(view["w"], view["h"], layer + 1)[layer]
        out = np.zeros((h, w, 2), np.float32)
        self.lib.adop_oracle_env_uv(C.byref(sc), va, layer, _nptr(out))
        return out

    def apply_tangent(self, tangent, pose):
        self.lib.adop_oracle_apply_tangent(_nptr(tangent), _nptr(pose), tangent.shape[0])

    # -- tonemapper ----------------------------------------------------------------------------------
    @staticmethod
    def tonemap_params(x, image_size, frame_index=None, exposure=None, white_balance=None, vignette=None, uv=None,
                       response=None, leak=0.0):
        p = capi.AdopTonemapParams()
        p.batch, _, p.height, p.width = x.shape
        p.response_bins = response.shape[1] if response is not None else 0
        p.vignette_image_w, p.vignette_image_h = image_size
        p.leak = leak
        for name, a in (("frame_index", frame_index), ("exposure", exposure), ("white_balance", white_balance),
                        ("vignette", vignette), ("uv", uv), ("response", response)):
            setattr(p, name, _nptr(a) if a is not None else None)
        return p

    def tonemap_forward(self, x, **kw):
        p = self.tonemap_params(x, **kw)
        out = np.zeros_like(x)
        assert self.lib.adop_oracle_tonemap_forward(C.byref(p), _nptr(x), _nptr(out)) == 0
        return out

    def tonemap_backward(self, x, grad_out, **kw):
        p = self.tonemap_params(x, **kw)
        g = capi.AdopTonemapGrads()
        res = dict(x=np.zeros_like(x))
        g.grad_x = _nptr(res["x"])
        for name in ("exposure", "white_balance", "vignette", "response"):
            a = kw.get(name)
            res[name] = np.zeros_like(a) if a is not None else None
            setattr(g, "grad_" + name, _nptr(res[name]) if a is not None else None)
        g.num_frames = kw["exposure"].shape[0] if kw.get("exposure") is not None else (
            kw["white_balance"].shape[0] if kw.get("white_balance") is not None else 0)
        g.accumulate = 0
        assert self.lib.adop_oracle_tonemap_backward(C.byref(p), _nptr(x), _nptr(grad_out), C.byref(g)) == 0
        return res
