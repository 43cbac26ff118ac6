"""The workspace-free forward entry point against the regular one, through the C ABI.

Some hosts of the library cannot allocate device memory when they render: a callback that runs while the allocator is
locked, a plugin that only gets input and output buffers from its host application, a process whose memory budget was
fixed at start-up. `adop_raster_forward_static` serves them with a built-in 32 MiB device array instead of a
caller-owned workspace. Its results must equal `adop_raster_forward`'s: depth and weight buffers bit for bit, colours
within the float-atomic tolerance the other GPU tests use (1e-4 of the tensor's magnitude). Two calls in a row, of
different sizes, check that the array's leftover contents do not leak into the next call. This file is collected last so
that a run that stops at the first failure has already run everything else.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from adop_b200 import capi, synth
from adop_b200.raster import Scene, fill_scene_struct

pytestmark = pytest.mark.gpu

RTOL = 1e-4


def _forward(lib, entry, scene, views, params, L, workspace):
    """Call one of the two forward entry points on freshly allocated outputs; returns (colors, depths, weights, masks)."""
    dev = scene.position.device
    va = capi.make_views(views)
    B = len(va)
    sc = fill_scene_struct(scene.tensors(), lambda t: t.data_ptr())
    sizes = capi.layer_sizes(va[0].w, va[0].h, L)
    f32 = dict(dtype=torch.float32, device=dev)
    colors = [torch.full((B, sc.channels, h, w), float("nan"), **f32) for w, h in sizes]
    depths = [torch.full((B, 1, h, w), float("nan"), **f32) for w, h in sizes]
    weights = [torch.full((B, 1, h, w), float("nan"), **f32) for w, h in sizes]
    masks = [torch.full((B, 1, h, w), float("nan"), **f32) for w, h in sizes]
    io = capi.AdopForwardIO()
    for l in range(L):
        io.layers[l].color, io.layers[l].depth = colors[l].data_ptr(), depths[l].data_ptr()
        io.layers[l].weight, io.layers[l].mask = weights[l].data_ptr(), masks[l].data_ptr()
    if workspace is not None:
        io.workspace, io.workspace_bytes = workspace.data_ptr(), workspace.numel()
    stream = torch.cuda.current_stream(dev).cuda_stream
    st = getattr(lib, entry)(C.byref(sc), va, B, C.byref(params), L, C.byref(io), C.c_void_p(stream))
    torch.cuda.synchronize(dev)
    return st, colors, depths, weights, masks


def _compare(lib, cfg):
    dev = torch.device("cuda:0")
    scene = Scene(**{k: (torch.from_numpy(v).to(dev) if v is not None else None) for k, v in cfg["arrays"].items()})
    views, params, L = cfg["views"], cfg["params"], cfg["num_layers"]
    need = lib.adop_raster_workspace_bytes(views[0]["w"], views[0]["h"], L, cfg["meta"]["channels"])
    assert 0 < need <= lib.adop_raster_static_scratch_bytes()
    ws = torch.empty(need, dtype=torch.uint8, device=dev)
    st, c_ref, d_ref, w_ref, m_ref = _forward(lib, "adop_raster_forward", scene, views, params, L, ws)
    assert st == capi.ADOP_OK
    st, c_new, d_new, w_new, m_new = _forward(lib, "adop_raster_forward_static", scene, views, params, L, None)
    assert st == capi.ADOP_OK, lib.adop_last_error()
    for l in range(L):
        assert torch.equal(d_new[l], d_ref[l]), f"depth layer {l}"
        assert torch.equal(w_new[l], w_ref[l]), f"weight layer {l}"
        assert torch.equal(m_new[l], m_ref[l]), f"mask layer {l}"
        scale = max(float(c_ref[l].abs().max()), 1e-12)
        assert float((c_new[l] - c_ref[l]).abs().max()) <= RTOL * scale, f"colour layer {l}"
        assert float(w_ref[l].sum()) > 0


def test_static_scratch_forward_matches_workspace_forward_twice(cuda_lib):
    lib = cuda_lib
    assert lib.adop_raster_static_scratch_bytes() == 32 << 20
    # first call: a larger pyramid; second call: a smaller one with another channel count, reusing the same array
    _compare(lib, synth.make_config("c2", n_points=300_000, n_views=3, size=(640, 360)))
    _compare(lib, synth.make_config("c5", n_points=150_000, n_views=2, size=(384, 216)))
    # and the first size again, now on top of the second call's leftovers
    _compare(lib, synth.make_config("c2", n_points=300_000, n_views=3, size=(640, 360), seed=5))


def test_static_scratch_forward_leaves_device_memory_in_use_unchanged(cuda_lib):
    """The entry point's contract is that it allocates nothing. After one warm-up call (the first call on a device loads
    the module with its 32 MiB array and looks up the array's address), the driver's free-memory figure must be the same
    before and after a call, outputs and inputs being allocated beforehand."""
    lib = cuda_lib
    dev = torch.device("cuda:0")
    cfg = synth.make_config("c2", n_points=100_000, n_views=2, size=(320, 180))
    scene = Scene(**{k: (torch.from_numpy(v).to(dev) if v is not None else None) for k, v in cfg["arrays"].items()})
    views, params, L = cfg["views"], cfg["params"], cfg["num_layers"]
    st, *_ = _forward(lib, "adop_raster_forward_static", scene, views, params, L, None)  # warm-up: module load, address
    assert st == capi.ADOP_OK, lib.adop_last_error()
    # everything the measured call touches exists before the first reading
    va = capi.make_views(views)
    B = len(va)
    sc = fill_scene_struct(scene.tensors(), lambda t: t.data_ptr())
    sizes = capi.layer_sizes(va[0].w, va[0].h, L)
    f32 = dict(dtype=torch.float32, device=dev)
    bufs = [[torch.empty((B, ch, h, w), **f32) for w, h in sizes] for ch in (sc.channels, 1, 1, 1)]
    io = capi.AdopForwardIO()
    for l in range(L):
        io.layers[l].color, io.layers[l].depth = bufs[0][l].data_ptr(), bufs[1][l].data_ptr()
        io.layers[l].weight, io.layers[l].mask = bufs[2][l].data_ptr(), bufs[3][l].data_ptr()
    stream = torch.cuda.current_stream(dev).cuda_stream
    torch.cuda.synchronize(dev)
    free_before, _ = torch.cuda.mem_get_info(dev)
    st = lib.adop_raster_forward_static(C.byref(sc), va, B, C.byref(params), L, C.byref(io), C.c_void_p(stream))
    torch.cuda.synchronize(dev)
    free_after, _ = torch.cuda.mem_get_info(dev)
    assert st == capi.ADOP_OK, lib.adop_last_error()
    assert free_after == free_before, f"device memory in use changed by {free_before - free_after} bytes across the call"
    assert float(bufs[2][0].sum()) > 0


def test_static_scratch_rejects_views_beyond_its_size(cuda_lib):
    lib = cuda_lib
    cfg = synth.make_config("c2", n_points=1000, n_views=1, size=(1920, 1080))
    dev = torch.device("cuda:0")
    scene = Scene(**{k: (torch.from_numpy(v).to(dev) if v is not None else None) for k, v in cfg["arrays"].items()})
    assert lib.adop_raster_workspace_bytes(1920, 1080, 4, 4) > lib.adop_raster_static_scratch_bytes()
    st, *_ = _forward(lib, "adop_raster_forward_static", scene, cfg["views"], cfg["params"], 4, None)
    assert st == 5  # ADOP_ERR_SIZE_LIMIT
    msg = lib.adop_last_error().decode()
    assert "bytes of scratch" in msg and "adop_raster_forward" in msg
