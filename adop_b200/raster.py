"""Host-side mirror of the reference's operator for the rasterizer path, over the C ABI.

`PointRasterizer.forward/backward` take what `torch::autograd::PointRender::forward/backward`
(src/lib/rendering/RenderInfo.cpp:34-58) take — descriptors [C,T], background [C], points [N,4], pose tangents,
intrinsics, plus the non-differentiable scene tensors and the batch of `ReducedImageInfo` — and return the layer
pyramid (then the masks) and the gradients in the reference's order. torch is used for device memory and streams
only; every computation happens in `libadop_raster.so`.
"""
import ctypes as C

import torch

from . import capi


class Scene:
    """The tensors the operator reads from the scene modules (PointRenderer.cu:1146-1155).

    position [N,4] f32, normal [N] i32 or None, index [N] i32 or None (identity), texture [C,T] f32,
    background [C] f32, poses [I,8] f64, intrinsics [K,cols] f32, env_map [C,eh,ew] f32 or None.
    Optional second cloud (the reference's outlier cloud, PointRenderer.cu:1402-1441; forward pass only):
    outlier_position [M,4] f32, outlier_normal [M] i32 or None, outlier_index [M] i32 or None, M <= N.
    """

    def __init__(self, position, texture, background, poses, intrinsics, normal=None, index=None, env_map=None,
                 outlier_position=None, outlier_normal=None, outlier_index=None):
        self.position, self.texture, self.background = position, texture, background
        self.poses, self.intrinsics = poses, intrinsics
        self.normal, self.index, self.env_map = normal, index, env_map
        self.outlier_position, self.outlier_normal, self.outlier_index = outlier_position, outlier_normal, outlier_index

    def tensors(self):
        return dict(position=self.position, normal=self.normal, index=self.index, texture=self.texture,
                    background=self.background, poses=self.poses, intrinsics=self.intrinsics, env_map=self.env_map,
                    outlier_position=self.outlier_position, outlier_normal=self.outlier_normal,
                    outlier_index=self.outlier_index)

    def to(self, device):
        return Scene(**{k: (v.to(device) if v is not None else None) for k, v in self.tensors().items()})


_DTYPES = dict(position="float32", normal="int32", index="int32", texture="float32", background="float32",
               poses="float64", intrinsics="float32", env_map="float32", outlier_position="float32",
               outlier_normal="int32", outlier_index="int32")


def fill_scene_struct(tensors, ptr):
    """Build an AdopScene from a dict of arrays (torch or numpy); `ptr` maps an array to its address."""
    s = capi.AdopScene()
    pos, tex = tensors["position"], tensors["texture"]
    for name, a in tensors.items():
        if a is None:
            continue
        dt = str(a.dtype).replace("torch.", "")
        if dt != _DTYPES[name]:
            raise TypeError(f"{name}: expected {_DTYPES[name]}, got {dt}")
    if pos.ndim != 2 or pos.shape[1] != 4:
        raise ValueError("position must be [N,4]")
    if tex.ndim != 2:
        raise ValueError("texture must be [C,T]")
    s.num_points = int(pos.shape[0])
    s.channels = int(tex.shape[0])
    s.num_texels = int(tex.shape[1])
    s.num_images = int(tensors["poses"].shape[0])
    if tensors["poses"].shape[1] != 8:
        raise ValueError("poses must be [I,8]")
    s.num_cameras = int(tensors["intrinsics"].shape[0])
    s.intrinsics_cols = int(tensors["intrinsics"].shape[1])
    env = tensors.get("env_map")
    if env is not None:
        if env.ndim == 4:
            env = env[0]
        if env.shape[0] != s.channels:
            raise ValueError("env_map must be [C,eh,ew]")
        s.env_h, s.env_w = int(env.shape[1]), int(env.shape[2])
    for name in ("position", "normal", "index", "texture", "background", "poses", "intrinsics", "env_map",
                 "outlier_position", "outlier_normal", "outlier_index"):
        a = tensors.get(name)
        setattr(s, name, ptr(a) if a is not None else None)
    out = tensors.get("outlier_position")
    if out is not None:
        if out.ndim != 2 or out.shape[1] != 4:
            raise ValueError("outlier_position must be [M,4]")
        s.num_outliers = int(out.shape[0])
    return s


def _tptr(t):
    if not t.is_cuda:
        raise capi.AdopError("the rasterizer takes CUDA tensors only (there is no CPU path)")
    if not t.is_contiguous():
        raise ValueError("tensors must be contiguous")
    return t.data_ptr()


class ForwardResult:
    """Outputs of the forward pass plus what the backward pass needs again (the reference's saved variables,
    PointRenderer.cu:1514-1527): depth, weight and colour per layer, and the per-view list of points that passed the
    depth test (in place of the saved [B,N] drop-out tensor)."""

    def __init__(self, colors, masks, depths, weights, views, num_layers, visible=None, packed=None):
        self.colors, self.masks, self.depths, self.weights = colors, masks, depths, weights
        self.views, self.num_layers = views, num_layers
        self.visible = visible
        self.packed = packed  # optional per layer [B,1,h,w] int64: depth bits << 32 | index of the nearest point

    def _tiles(self):
        w, h = self.views[0].w, self.views[0].h
        return ((w + 31) // 32) * ((h + 15) // 16)

    def entry_counts(self):
        """Listed points per view (points with at least one accepted layer), as recorded in `visible`."""
        header, t = 2048 + 8, self._tiles()
        return self.visible[:, header: header + t].sum(dim=1)

    def list_unusable(self):
        """True for views whose list is marked as not usable (the backward pass then walks all points)."""
        return self.visible[:, 2048 + 2] != 0


class PointRasterizer:
    """Owns the reusable scratch (the role of PointRendererCache, PointRenderer.h:96-157)."""

    def __init__(self, device="cuda:0", interleave_descriptors=True, full_workspace=None):
        """full_workspace: True sizes the forward scratch with adop_raster_workspace_bytes_full (16 bytes per point and view
        of a group more), which lets the depth prepass hand the projected in-image points to the blend kernel instead of the
        blend kernel reading the cloud and projecting again; False keeps the small workspace. None (default) decides per
        call: on for views of the omnidirectional model, whose projection is expensive and whose image holds a small part
        of the cloud (forward pass of the 100 M point viewer configuration: a third faster), off for pinhole views, where the
        extra stream costs more than it saves (measured on the training configuration)."""
        self.lib = capi.load_library()
        self.device = torch.device(device)
        self._ws = None
        self.interleave_descriptors = interleave_descriptors
        self.full_workspace = full_workspace
        self._tex_i = None    # [T,C] working copy of the descriptors, refreshed by every forward call
        self._gtex_i = None   # [T,C] scratch for the descriptor gradient

    def _scene_struct(self, scene, refresh):
        """AdopScene of `scene`; with interleave_descriptors also keeps the [T,C] working copy up to date."""
        sc = fill_scene_struct(scene.tensors(), _tptr)
        if self.interleave_descriptors:
            shape = (sc.num_texels, sc.channels)
            if self._tex_i is None or tuple(self._tex_i.shape) != shape:
                self._tex_i = torch.empty(shape, dtype=torch.float32, device=self.device)
                refresh = True
            if refresh:
                stream = torch.cuda.current_stream(self.device).cuda_stream
                capi.check(self.lib.adop_texture_interleave(scene.texture.data_ptr(), self._tex_i.data_ptr(), sc.channels,
                                                            sc.num_texels, C.c_void_p(stream)), "adop_texture_interleave")
            sc.texture_interleaved = self._tex_i.data_ptr()
        return sc

    def _workspace(self, w, h, layers, channels, num_points=0, num_views=1, full=False):
        if full:
            need = self.lib.adop_raster_workspace_bytes_full(num_points, num_views, w, h, layers, channels)
        else:
            need = self.lib.adop_raster_workspace_bytes(w, h, layers, channels)
        if need == 0:
            raise ValueError("invalid size")
        if self._ws is None or self._ws.numel() < need:
            self._ws = torch.empty(need, dtype=torch.uint8, device=self.device)
        # the library picks its kernels by the size it is told: it is told the size asked for, not what an earlier, larger
        # call left behind
        self._ws_bytes = need
        return self._ws

    def forward(self, scene, views, params, num_layers, dropout_mask=None, out=None, record_visible=True,
                refresh_descriptors=True, packed_depth=False, touched=None):
        """BlendPointCloudForward (PointRenderer.cu:1389-1531). `views`: list of dicts or an AdopView array.

        Returns a ForwardResult; result.colors + result.masks is the reference's return list.
        `out`: a previous ForwardResult whose tensors are reused (no allocation in steady state).
        `touched`: optional (points, texels) uint8 tensors of ceil(N / 256) and ceil(T / 256) flags that the call fills: 1
        where the backward pass of these views can add a gradient (dist.PeerGradientExchange.touched_flags())."""
        va = views if isinstance(views, C.Array) else capi.make_views(views)
        B = len(va)
        w, h = va[0].w, va[0].h
        with torch.cuda.device(self.device):
            # refresh_descriptors=False: the caller vouches that scene.texture has not changed since the last call (a viewer
            # rendering frame after frame), so the [T,C] working copy is reused as it is
            sc = self._scene_struct(scene, refresh=refresh_descriptors)
            ch = sc.channels
            full = self.full_workspace
            if full is None:
                full = any(v.camera_model == capi.CAMERA_OCAM for v in va)
            ws = self._workspace(w, h, num_layers, ch, sc.num_points, B, full=bool(full))
            sizes = capi.layer_sizes(w, h, num_layers)
            if out is None:
                f32 = dict(dtype=torch.float32, device=self.device)
                colors = [torch.empty((B, ch, hh, ww), **f32) for ww, hh in sizes]
                depths = [torch.empty((B, 1, hh, ww), **f32) for ww, hh in sizes]
                weights = [torch.empty((B, 1, hh, ww), **f32) for ww, hh in sizes]
                masks = [torch.empty((B, 1, hh, ww), **f32) for ww, hh in sizes] if params.output_background_mask else []
                visible = None
                if record_visible:
                    ints = self.lib.adop_raster_visible_list_ints(sc.num_points, w, h, num_layers)
                    visible = torch.empty((B, ints), dtype=torch.int32, device=self.device)
                packed = [torch.empty((B, 1, hh, ww), dtype=torch.int64, device=self.device) for ww, hh in sizes] \
                    if packed_depth else None
                out = ForwardResult(colors, masks, depths, weights, va, num_layers, visible, packed)
            else:
                out.views = va
            io = capi.AdopForwardIO()
            for l in range(num_layers):
                io.layers[l].color = out.colors[l].data_ptr()
                io.layers[l].depth = out.depths[l].data_ptr()
                io.layers[l].weight = out.weights[l].data_ptr()
                io.layers[l].mask = out.masks[l].data_ptr() if out.masks else None
            io.dropout_mask = _tptr(dropout_mask) if dropout_mask is not None else None
            io.workspace = ws.data_ptr()
            io.workspace_bytes = self._ws_bytes
            io.visible_list = out.visible.data_ptr() if out.visible is not None else None
            if touched is not None:
                io.touched_points, io.touched_texels = _tptr(touched[0]), _tptr(touched[1])
            if out.packed is not None:
                for l in range(num_layers):
                    io.packed_depth[l] = out.packed[l].data_ptr()
            stream = torch.cuda.current_stream(self.device).cuda_stream
            st = self.lib.adop_raster_forward(C.byref(sc), va, B, C.byref(params), num_layers, C.byref(io),
                                              C.c_void_p(stream))
            capi.check(st, "adop_raster_forward")
        return out

    def backward(self, scene, params, fwd, grad_colors, want_points=True, want_pose=True, want_intrinsics=True,
                 want_env=False, dropout_mask=None, normalize=True, out=None):
        """BlendPointCloudBackward (PointRenderer.cu:1549-1644).

        Returns a dict: texture, background, points, pose, intrinsics (the reference's order), plus count_pose /
        count_intrinsics and env_map when asked for."""
        va, L = fwd.views, fwd.num_layers
        B = len(va)
        with torch.cuda.device(self.device):
            sc = self._scene_struct(scene, refresh=False)  # the forward call of this step refreshed the copy
            dev = self.device
            if out is None:
                out = dict(texture=torch.empty_like(scene.texture), background=torch.empty_like(scene.background))
                out["points"] = torch.empty_like(scene.position) if want_points else None
                if want_pose:
                    out["pose"] = torch.empty((sc.num_images, 6), dtype=torch.float64, device=dev)
                    out["count_pose"] = torch.empty((sc.num_images,), dtype=torch.float32, device=dev)
                else:
                    out["pose"] = out["count_pose"] = None
                if want_intrinsics:
                    out["intrinsics"] = torch.empty_like(scene.intrinsics)
                    out["count_intrinsics"] = torch.empty((sc.num_cameras,), dtype=torch.float32, device=dev)
                else:
                    out["intrinsics"] = out["count_intrinsics"] = None
                out["env_map"] = torch.empty_like(scene.env_map) if (want_env and scene.env_map is not None) else None
            io = capi.AdopBackwardIO()
            for l in range(L):
                io.layers[l].color = fwd.colors[l].data_ptr()
                io.layers[l].depth = fwd.depths[l].data_ptr()
                io.layers[l].weight = fwd.weights[l].data_ptr()
                g = grad_colors[l]
                if g.dtype != torch.float32 or tuple(g.shape) != tuple(fwd.colors[l].shape):
                    raise ValueError("image gradients must be float32 and shaped like the layers")  # :1553-1556
                io.grad_color[l] = _tptr(g)
            io.dropout_mask = _tptr(dropout_mask) if dropout_mask is not None else None

            def p(name):
                t = out.get(name)
                return t.data_ptr() if t is not None else None

            io.grad_texture, io.grad_background, io.grad_points = p("texture"), p("background"), p("points")
            io.grad_pose, io.count_pose = p("pose"), p("count_pose")
            io.grad_intrinsics, io.count_intrinsics = p("intrinsics"), p("count_intrinsics")
            io.grad_env_map = p("env_map")
            io.accumulate = 0
            io.normalize = 1 if normalize else 0
            ws = self._workspace(va[0].w, va[0].h, L, sc.channels, sc.num_points, B)
            io.workspace = ws.data_ptr()
            io.workspace_bytes = self._ws_bytes
            io.visible_list = fwd.visible.data_ptr() if fwd.visible is not None else None
            if out.get("texture_interleaved") is not None:
                # the caller keeps the descriptor gradients in [T,C] layout (the block the GPUs exchange, dist.py)
                if out.get("texture") is not None:
                    raise ValueError("give either texture [C,T] or texture_interleaved [T,C] as the output, not both")
                io.grad_texture_interleaved = out["texture_interleaved"].data_ptr()
            elif self.interleave_descriptors:
                if self._gtex_i is None or self._gtex_i.shape != self._tex_i.shape:
                    self._gtex_i = torch.empty_like(self._tex_i)
                io.grad_texture_interleaved = self._gtex_i.data_ptr()
            if out.get("env_map") is not None and sc.channels % 4 == 0:
                # [eh,ew,C] scratch for the environment-map gradient (vector atomics), kept between calls
                if getattr(self, "_genv_i", None) is None or self._genv_i.numel() != out["env_map"].numel():
                    self._genv_i = torch.empty(out["env_map"].numel(), dtype=torch.float32, device=dev)
                io.grad_env_map_interleaved = self._genv_i.data_ptr()
            stream = torch.cuda.current_stream(self.device).cuda_stream
            st = self.lib.adop_raster_backward(C.byref(sc), va, B, C.byref(params), L, C.byref(io), C.c_void_p(stream))
            capi.check(st, "adop_raster_backward")
        return out

    def normalize_gradients(self, grads):
        """NormalizeGradient (PointRenderer.cu:1609-1637) as its own step, after gradients of several GPUs were summed."""
        with torch.cuda.device(self.device):
            pts, pose, intr = grads.get("points"), grads.get("pose"), grads.get("intrinsics")
            stream = torch.cuda.current_stream(self.device).cuda_stream
            st = self.lib.adop_raster_normalize_gradients(
                pts.data_ptr() if pts is not None else None, pts.shape[0] if pts is not None else 0,
                pose.data_ptr() if pose is not None else None,
                grads["count_pose"].data_ptr() if pose is not None else None, pose.shape[0] if pose is not None else 0,
                intr.data_ptr() if intr is not None else None,
                grads["count_intrinsics"].data_ptr() if intr is not None else None,
                intr.shape[0] if intr is not None else 0, intr.shape[1] if intr is not None else 0, C.c_void_p(stream))
            capi.check(st, "adop_raster_normalize_gradients")


def apply_tangent_to_pose(tangent, pose):
    """ApplyTangentToPose (PointRenderer.cu:1659-1665): pose <- exp(tangent) * pose; tangent <- 0 (in place)."""
    lib = capi.load_library()
    if tangent.dtype != torch.float64 or pose.dtype != torch.float64:
        raise TypeError("tangent and pose are float64")
    if not (tangent.is_contiguous() and pose.is_contiguous()):
        raise ValueError("tangent and pose must be contiguous")  # SAIGA_ASSERT at :1661
    with torch.cuda.device(tangent.device):
        stream = torch.cuda.current_stream(tangent.device).cuda_stream
        capi.check(lib.adop_apply_tangent(_tptr(tangent), _tptr(pose), tangent.shape[0], C.c_void_p(stream)),
                   "adop_apply_tangent")


class Tonemapper:
    """NeuralCameraImpl::forward (NeuralCamera.cpp:258-335) as one fused kernel each way.

    exposure [n] (exposures_values), white_balance [n,3], vignette [5] = 3 coefficients + centre, response [3,K]."""

    def __init__(self, image_size, exposure=None, white_balance=None, vignette=None, response=None, leak=0.0):
        self.lib = capi.load_library()
        self.image_w, self.image_h = image_size
        self.exposure, self.white_balance, self.vignette, self.response = exposure, white_balance, vignette, response
        self.leak = float(leak)

    def _params(self, x, frame_index, uv):
        p = capi.AdopTonemapParams()
        p.batch, _, p.height, p.width = x.shape
        if x.shape[1] != 3:
            raise ValueError("the tonemapper works on RGB images")  # SAIGA_ASSERT(x.size(1) == 3), :263
        p.response_bins = self.response.shape[1] if self.response is not None else 0
        p.vignette_image_w, p.vignette_image_h = self.image_w, self.image_h
        p.leak = self.leak
        p.frame_index = _tptr(frame_index) if frame_index is not None else None
        for name in ("exposure", "white_balance", "vignette", "response"):
            t = getattr(self, name)
            setattr(p, name, _tptr(t) if t is not None else None)
        p.uv = _tptr(uv) if uv is not None else None
        return p

    def forward(self, x, frame_index=None, uv=None):
        p = self._params(x, frame_index, uv)
        out = torch.empty_like(x)
        with torch.cuda.device(x.device):
            stream = torch.cuda.current_stream(x.device).cuda_stream
            capi.check(self.lib.adop_tonemap_forward(C.byref(p), _tptr(x), out.data_ptr(), C.c_void_p(stream)),
                       "adop_tonemap_forward")
        return out

    def backward(self, x, grad_out, frame_index=None, uv=None, want_response=True):
        """Gradients for x and for every parameter tensor the tonemapper has; want_response=False leaves the response curve's
        out (a fixed curve: the backward pass then has no histogram to build)."""
        p = self._params(x, frame_index, uv)
        g = capi.AdopTonemapGrads()
        res = dict(x=torch.empty_like(x))
        g.grad_x = res["x"].data_ptr()
        for name in ("exposure", "white_balance", "vignette", "response"):
            t = getattr(self, name)
            if name == "response" and not want_response:
                t = None
            res[name] = torch.empty_like(t) if t is not None else None
            setattr(g, "grad_" + name, res[name].data_ptr() if t is not None else None)
        g.num_frames = self.exposure.shape[0] if self.exposure is not None else (
            self.white_balance.shape[0] if self.white_balance is not None else 0)
        g.accumulate = 0
        with torch.cuda.device(x.device):
            stream = torch.cuda.current_stream(x.device).cuda_stream
            capi.check(self.lib.adop_tonemap_backward(C.byref(p), _tptr(x), _tptr(grad_out), C.byref(g),
                                                      C.c_void_p(stream)), "adop_tonemap_backward")
        return res
