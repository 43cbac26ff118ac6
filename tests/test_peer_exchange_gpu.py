"""The gradient exchange over peer memory (adop_peer_reduce_gradients).

* On one GPU the kernel is checked with `world` blocks that all live on that GPU: it only takes base pointers, so the
  arithmetic, the shard ranges and the layouts are covered without a second device.
* With two or more GPUs a two-process run (one rank per GPU, CUDA IPC mappings, NCCL for the barriers) renders a
  small scene view-sharded and compares the exchanged gradients with a single-GPU run over all views and with the
  NCCL exchange.
"""
import ctypes as C
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from adop_b200 import capi
from adop_b200 import dist as adist

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _fill_block(lay, dev, gen):
    """A rank's block with random gradient sums and integer counts; returns (raw byte tensor, dict of views)."""
    raw = torch.zeros(lay.total_bytes, dtype=torch.uint8, device=dev)
    assert raw.data_ptr() % 256 == 0

    def view(off, shape, dtype):
        n = int(np.prod(shape))
        if n == 0:
            return None
        size = n * torch.empty((), dtype=dtype).element_size()
        return raw[off:off + size].view(dtype).view(*shape)

    t = {"texture": view(lay.off_texture, (lay.num_texels, lay.channels), torch.float32),
         "points": view(lay.off_points, (lay.num_points, 4), torch.float32),
         "pose": view(lay.off_pose, (lay.num_images, 6), torch.float64),
         "count_pose": view(lay.off_count_pose, (lay.num_images,), torch.float32),
         "intrinsics": view(lay.off_intrinsics, (lay.num_cameras, lay.intrinsics_cols), torch.float32),
         "count_intrinsics": view(lay.off_count_intrinsics, (lay.num_cameras,), torch.float32),
         "background": view(lay.off_background, (lay.channels if lay.background else 0,), torch.float32),
         "env_map": view(lay.off_env_map, (lay.channels, lay.env_h, lay.env_w), torch.float32)}
    for k, v in t.items():
        if v is None:
            continue
        if k.startswith("count"):
            v.copy_(torch.randint(0, 3, v.shape, device=dev, generator=gen).to(v.dtype))
        else:
            v.copy_(torch.randn(v.shape, device=dev, generator=gen, dtype=torch.float32).to(v.dtype))
    if t["points"] is not None:
        t["points"][:, 3] = torch.randint(0, 3, (lay.num_points,), device=dev, generator=gen).float()
    return raw, t


@pytest.mark.parametrize("channels,world,texels,points", [(4, 3, 1001, 777), (3, 2, 500, 0), (8, 8, 4099, 4099), (16, 1, 64, 64)])
def test_reduce_kernel_with_all_blocks_on_one_gpu(cuda_lib, channels, world, texels, points):
    dev = torch.device("cuda:0")
    gen = torch.Generator(device=dev)
    gen.manual_seed(channels * 100 + world)
    lay = adist.peer_layout(channels, texels, points, num_images=5, num_cameras=2, intrinsics_cols=13, env_hw=(6, 10))
    blocks = [_fill_block(lay, dev, gen) for _ in range(world)]
    ptrs = (C.c_void_p * world)(*[b[0].data_ptr() for b in blocks])

    def total(name):
        acc = torch.zeros_like(blocks[0][1][name])
        for _, t in blocks:  # rank order, as the kernel sums
            acc = acc + t[name]
        return acc

    tex_sum = total("texture").t().contiguous()  # [C,T]
    pts_sum = total("points") if points else None
    for rank in range(world):
        t_lo, t_hi = adist.peer_shard_range(texels, rank, world)
        p_lo, p_hi = adist.peer_shard_range(points, rank, world)
        out = capi.AdopPeerReduceOut()
        res_tex = torch.full((channels, t_hi - t_lo), float("nan"), device=dev)
        res_pts = torch.full((max(p_hi - p_lo, 1), 4), float("nan"), device=dev)
        res_pose = torch.empty((5, 6), dtype=torch.float64, device=dev)
        res_cp = torch.empty((5,), device=dev)
        res_intr = torch.empty((2, 13), device=dev)
        res_ci = torch.empty((2,), device=dev)
        res_bg = torch.empty((channels,), device=dev)
        res_env = torch.empty((channels, 6, 10), device=dev)
        out.grad_texture_shard = res_tex.data_ptr() if t_hi > t_lo else None
        out.grad_points_shard = res_pts.data_ptr() if p_hi > p_lo else None
        out.grad_pose, out.count_pose = res_pose.data_ptr(), res_cp.data_ptr()
        out.grad_intrinsics, out.count_intrinsics = res_intr.data_ptr(), res_ci.data_ptr()
        out.grad_background, out.grad_env_map = res_bg.data_ptr(), res_env.data_ptr()
        out.normalize = 1
        st = cuda_lib.adop_peer_reduce_gradients(ptrs, world, rank, C.byref(lay), C.byref(out), None)
        capi.check(st, "adop_peer_reduce_gradients")
        torch.cuda.synchronize()
        assert torch.equal(res_tex, tex_sum[:, t_lo:t_hi])
        if p_hi > p_lo:
            s = pts_sum[p_lo:p_hi]
            want = s.clone()
            nz = s[:, 3] > 0
            want[nz, :3] = s[nz, :3] / s[nz, 3:4]
            want[:, 3] = 0
            assert torch.equal(res_pts, want)
        cp, ci = total("count_pose"), total("count_intrinsics")
        pose = total("pose")
        pose = torch.where(cp[:, None] > 0, pose / cp[:, None].double().clamp(min=1), pose)
        intr = total("intrinsics")
        intr = torch.where(ci[:, None] > 0, intr / ci[:, None].clamp(min=1), intr)
        assert torch.equal(res_cp, cp) and torch.equal(res_ci, ci)
        assert torch.equal(res_pose, pose)
        assert torch.equal(res_intr, intr)
        assert torch.equal(res_bg, total("background"))
        assert torch.equal(res_env, total("env_map"))


@pytest.mark.parametrize("channels,world,texels,points", [(4, 3, 5000, 3333), (3, 2, 1000, 0), (8, 8, 40_000, 20_001)])
def test_reduce_kernel_skips_what_a_rank_did_not_touch(cuda_lib, channels, world, texels, points):
    """Blocks with touched flags: every rank has gradients only in some chunks of 256 texels / points (zeros elsewhere, as
    the backward pass leaves them) and flags exactly those chunks. The sums must equal the plain sums of all blocks. To
    show that unflagged chunks are really not read, a second run poisons them with NaN: the result must not change."""
    dev = torch.device("cuda:0")
    gen = torch.Generator(device=dev)
    gen.manual_seed(channels * 7 + world)
    lay = adist.peer_layout(channels, texels, points, num_images=2, num_cameras=1, intrinsics_cols=13, touched=True)
    chunk = 256
    blocks = [_fill_block(lay, dev, gen) for _ in range(world)]
    flags = []
    for raw, t in blocks:
        tc, pc = (texels + chunk - 1) // chunk, (points + chunk - 1) // chunk
        ft = torch.rand(tc, device=dev, generator=gen) < 0.5
        fp = torch.rand(max(pc, 1), device=dev, generator=gen)[:pc] < 0.4
        t["texture"][~ft.repeat_interleave(chunk)[:texels]] = 0
        if points:
            t["points"][~fp.repeat_interleave(chunk)[:points]] = 0
        raw[lay.off_touched_texels:lay.off_touched_texels + tc] = ft.to(torch.uint8)
        if points:
            raw[lay.off_touched_points:lay.off_touched_points + pc] = fp.to(torch.uint8)
        flags.append((ft, fp))
    ptrs = (C.c_void_p * world)(*[b[0].data_ptr() for b in blocks])
    tex_sum = sum(t["texture"] for _, t in blocks).t().contiguous()
    pts_sum = sum(t["points"] for _, t in blocks) if points else None

    def run_all():
        res = []
        for rank in range(world):
            t_lo, t_hi = adist.peer_shard_range(texels, rank, world)
            p_lo, p_hi = adist.peer_shard_range(points, rank, world)
            out = capi.AdopPeerReduceOut()
            r_tex = torch.full((channels, t_hi - t_lo), float("nan"), device=dev)
            r_pts = torch.full((max(p_hi - p_lo, 1), 4), float("nan"), device=dev)
            out.grad_texture_shard = r_tex.data_ptr()
            out.grad_points_shard = r_pts.data_ptr() if p_hi > p_lo else None
            out.normalize = 0
            capi.check(cuda_lib.adop_peer_reduce_gradients(ptrs, world, rank, C.byref(lay), C.byref(out), None), "reduce")
            torch.cuda.synchronize()
            res.append((r_tex, r_pts[:p_hi - p_lo], (t_lo, t_hi), (p_lo, p_hi)))
        return res

    first = run_all()
    for r_tex, r_pts, (t_lo, t_hi), (p_lo, p_hi) in first:
        assert torch.allclose(r_tex, tex_sum[:, t_lo:t_hi], rtol=1e-6, atol=1e-6)
        if points:
            assert torch.allclose(r_pts, pts_sum[p_lo:p_hi], rtol=1e-6, atol=1e-6)
    for (raw, t), (ft, fp) in zip(blocks, flags):
        t["texture"][~ft.repeat_interleave(chunk)[:texels]] = float("nan")
        if points:
            t["points"][~fp.repeat_interleave(chunk)[:points]] = float("nan")
    second = run_all()
    for a, b in zip(first, second):
        assert torch.equal(a[0], b[0]) and (not points or torch.equal(a[1], b[1]))


@pytest.mark.parametrize("channels,env_hw", [(3, (1, 1)), (3, (1, 2)), (4, (1, 1))])
def test_reduce_kernel_with_only_a_tiny_environment_map(cuda_lib, channels, env_hw):
    """The only work is an environment-map gradient of one to three floats (fewer than one 16-byte vector): the launch
    must not come out empty."""
    dev = torch.device("cuda:0")
    gen = torch.Generator(device=dev)
    gen.manual_seed(17)
    lay = adist.peer_layout(channels, 0, 0, num_images=0, num_cameras=0, intrinsics_cols=0, env_hw=env_hw, background=False)
    blocks = [_fill_block(lay, dev, gen) for _ in range(2)]
    ptrs = (C.c_void_p * 2)(*[b[0].data_ptr() for b in blocks])
    out = capi.AdopPeerReduceOut()
    res_env = torch.full((channels,) + env_hw, float("nan"), device=dev)
    out.grad_env_map = res_env.data_ptr()
    out.normalize = 1
    capi.check(cuda_lib.adop_peer_reduce_gradients(ptrs, 2, 0, C.byref(lay), C.byref(out), None), "adop_peer_reduce_gradients")
    torch.cuda.synchronize()
    assert torch.equal(res_env, blocks[0][1]["env_map"] + blocks[1][1]["env_map"])


def test_reduce_rejects_bad_arguments(cuda_lib):
    lay = adist.peer_layout(4, 16, 16)
    out = capi.AdopPeerReduceOut()
    ptrs = (C.c_void_p * 1)(None)
    assert cuda_lib.adop_peer_reduce_gradients(ptrs, 1, 0, C.byref(lay), C.byref(out), None) != capi.ADOP_OK  # null block
    buf = torch.zeros(lay.total_bytes, dtype=torch.uint8, device="cuda:0")
    ptrs = (C.c_void_p * 1)(buf.data_ptr())
    assert cuda_lib.adop_peer_reduce_gradients(ptrs, 9, 0, C.byref(lay), C.byref(out), None) != capi.ADOP_OK  # world > 8
    assert cuda_lib.adop_peer_reduce_gradients(ptrs, 1, 1, C.byref(lay), C.byref(out), None) != capi.ADOP_OK  # rank >= world
    lay.total_bytes += 256  # a layout that adop_peer_layout_fill did not produce
    assert cuda_lib.adop_peer_reduce_gradients(ptrs, 1, 0, C.byref(lay), C.byref(out), None) != capi.ADOP_OK


def test_backward_leaves_descriptor_gradients_interleaved(cuda_lib):
    """grad_texture == NULL with a [T,C] buffer: the gradients stay there and equal the [C,T] result transposed."""
    from adop_b200 import synth
    from adop_b200.raster import PointRasterizer, Scene
    dev = torch.device("cuda:0")
    cfg = synth.make_config("c2", n_points=30000, n_views=2, size=(128, 72))
    scene = Scene(**{k: (torch.from_numpy(v).to(dev) if v is not None else None) for k, v in cfg["arrays"].items()})
    ras = PointRasterizer(dev)
    fwd = ras.forward(scene, cfg["views"], cfg["params"], cfg["num_layers"])
    grads = [torch.randn_like(c) for c in fwd.colors]
    ref = ras.backward(scene, cfg["params"], fwd, grads, normalize=False)
    fwd = ras.forward(scene, cfg["views"], cfg["params"], cfg["num_layers"])
    out = {k: (torch.empty_like(v) if v is not None else None) for k, v in ref.items()}
    out["texture"] = None
    out["texture_interleaved"] = torch.full((scene.texture.shape[1], scene.texture.shape[0]), float("nan"), device=dev)
    ras.backward(scene, cfg["params"], fwd, grads, normalize=False, out=out)
    torch.cuda.synchronize()
    assert torch.allclose(out["texture_interleaved"].t(), ref["texture"], rtol=1e-5, atol=1e-6)
    assert torch.allclose(out["points"], ref["points"], rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("channels,world,texels,points", [(4, 3, 1001, 777), (4, 4, 4096, 0), (8, 8, 40_000, 4099), (16, 1, 64, 64)])
def test_update_kernel_with_all_replicas_on_one_gpu(cuda_lib, channels, world, texels, points):
    """adop_peer_apply_update with `world` parameter blocks that all live on one GPU (the kernel only takes base pointers):
    after every rank's launch of a step all replicas hold the same tensors, and after three steps those equal what
    torch.optim.Adam (descriptors) and torch.optim.SGD (points) make of the full tensors and the full gradients. Covers
    the vector path (shares that are multiples of four texels) and the element path (ragged shares)."""
    dev = torch.device("cuda:0")
    gen = torch.Generator(device=dev)
    gen.manual_seed(channels + world)
    lay = adist.peer_param_layout(channels, texels, points)
    raws = [torch.zeros(lay.total_bytes, dtype=torch.uint8, device=dev) for _ in range(world)]
    ptrs = (C.c_void_p * world)(*[r.data_ptr() for r in raws])

    def views(raw):
        tex = raw[lay.off_texture:lay.off_texture + channels * texels * 4].view(torch.float32).view(channels, texels)
        pts = raw[lay.off_points:lay.off_points + points * 16].view(torch.float32).view(points, 4) if points else None
        return tex, pts

    tex0 = torch.randn((channels, texels), device=dev, generator=gen)
    pts0 = torch.randn((points, 4), device=dev, generator=gen) if points else None
    for raw in raws:
        t, p = views(raw)
        t.copy_(tex0)
        if points:
            p.copy_(pts0)
    ref_tex = tex0.clone().requires_grad_(True)
    adam = torch.optim.Adam([ref_tex], lr=0.08)
    ref_pts = pts0[:, :3].clone().requires_grad_(True) if points else None
    sgd = torch.optim.SGD([ref_pts], lr=0.005) if points else None
    m = [torch.zeros((channels, adist.peer_shard_range(texels, r, world)[1] - adist.peer_shard_range(texels, r, world)[0]), device=dev)
         for r in range(world)]
    v = [torch.zeros_like(x) for x in m]
    for step in range(1, 4):
        g_tex = torch.randn((channels, texels), device=dev, generator=gen) * (10.0 ** (step - 2))
        g_pts = torch.randn((points, 4), device=dev, generator=gen) if points else None
        for rank in range(world):
            t_lo, t_hi = adist.peer_shard_range(texels, rank, world)
            p_lo, p_hi = adist.peer_shard_range(points, rank, world)
            u = capi.AdopPeerUpdate()
            shard = g_tex[:, t_lo:t_hi].contiguous()
            pshard = g_pts[p_lo:p_hi].contiguous() if points and p_hi > p_lo else None
            u.grad_texture_shard = shard.data_ptr() if t_hi > t_lo else None
            u.adam_m, u.adam_v = m[rank].data_ptr(), v[rank].data_ptr()
            u.grad_points_shard = pshard.data_ptr() if pshard is not None else None
            u.lr_texture, u.beta1, u.beta2, u.eps, u.step, u.lr_points = 0.08, 0.9, 0.999, 1e-8, step, 0.005
            capi.check(cuda_lib.adop_peer_apply_update(ptrs, world, rank, C.byref(lay), C.byref(u), None), "adop_peer_apply_update")
        torch.cuda.synchronize()
        ref_tex.grad = g_tex.clone()
        adam.step()
        if points:
            ref_pts.grad = g_pts[:, :3].clone()
            sgd.step()
        t_first, p_first = views(raws[0])
        for raw in raws[1:]:
            t, p = views(raw)
            assert torch.equal(t, t_first) and (not points or torch.equal(p, p_first))
        assert torch.allclose(t_first, ref_tex.detach(), rtol=2e-6, atol=1e-7), float((t_first - ref_tex.detach()).abs().max())
        if points:
            assert torch.allclose(p_first[:, :3], ref_pts.detach(), rtol=1e-6, atol=1e-7)
            assert torch.equal(p_first[:, 3], pts0[:, 3])  # the drop-out radius is not a parameter


def test_update_kernel_argument_checks(cuda_lib):
    dev = torch.device("cuda:0")
    lay = adist.peer_param_layout(4, 64, 0)
    raw = torch.zeros(lay.total_bytes, dtype=torch.uint8, device=dev)
    ptrs = (C.c_void_p * 1)(raw.data_ptr())
    g = torch.zeros((4, 64), device=dev)
    u = capi.AdopPeerUpdate()
    u.grad_texture_shard, u.adam_m, u.adam_v = g.data_ptr(), g.data_ptr(), g.data_ptr()
    u.lr_texture, u.beta1, u.beta2, u.eps, u.step = 0.1, 0.9, 0.999, 1e-8, 0   # steps count from 1
    assert cuda_lib.adop_peer_apply_update(ptrs, 1, 0, C.byref(lay), C.byref(u), None) == 1  # ADOP_ERR_INVALID_ARGUMENT
    u.step, u.adam_v = 1, None
    assert cuda_lib.adop_peer_apply_update(ptrs, 1, 0, C.byref(lay), C.byref(u), None) == 1  # ADOP_ERR_INVALID_ARGUMENT
    assert cuda_lib.adop_peer_apply_update(ptrs, 9, 0, C.byref(lay), C.byref(u), None) == 1  # ADOP_ERR_INVALID_ARGUMENT


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_exchange_matches_single_gpu_and_nccl(cuda_lib, tmp_path):
    port = 29600 + (os.getpid() % 1000)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(ROOT, "tests", "peer_exchange_worker.py"), str(tmp_path)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert (tmp_path / "ok_0").exists() and (tmp_path / "ok_1").exists(), r.stdout[-3000:] + r.stderr[-3000:]


def test_one_rank_runs_the_whole_sharded_step(cuda_lib, tmp_path):
    """The worker of the two-GPU test with a single rank on one GPU: gradient blocks, touched flags, reduce kernel, optimiser
    kernel and the scene optimiser's training steps all run (a world of one shards nothing, but every code path between the
    backward pass and the next forward pass is the one the multi-GPU job takes), against the plain single-GPU results."""
    port = 29700 + (os.getpid() % 1000)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT, CUDA_VISIBLE_DEVICES="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "1", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(ROOT, "tests", "peer_exchange_worker.py"), str(tmp_path)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert (tmp_path / "ok_0").exists(), r.stdout[-3000:] + r.stderr[-3000:]
