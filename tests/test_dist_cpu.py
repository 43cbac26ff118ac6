"""World-size-2 gloo test of the view-sharded gradient exchange (host logic only, no GPU).

Each rank computes un-normalised gradients of its own views with the CPU checker, the exchange sums and shards them, the
shards are normalised, and the result must equal the single-process gradient over all views."""
import os

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from adop_b200 import synth
from adop_b200 import dist as adist


def _normalize_points(flat):
    p = flat.reshape(-1, 4).copy()
    c = p[:, 3:4]
    p[:, :3] = np.where(c > 0, p[:, :3] / np.maximum(c, 1e-30), p[:, :3])
    p[:, 3] = 0
    return p


def _worker(rank, world, port, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from tests.oracle_lib import Oracle
    ora = Oracle()
    cfg = synth.make_config("c2", n_points=20000, n_views=4, size=(96, 54))
    grads_up = synth.upstream_gradients(cfg["meta"])
    mine = adist.shard_views(list(range(4)), rank, world)
    views = [cfg["views"][i] for i in mine]
    g_mine = [np.ascontiguousarray(g[mine]) for g in grads_up]
    fwd = ora.forward(cfg["arrays"], views, cfg["params"], 4)
    bwd = ora.backward(cfg["arrays"], views, cfg["params"], 4, fwd, g_mine, want_env=True, normalize=False)
    t = {k: (torch.from_numpy(v) if v is not None else None) for k, v in bwd.items()}
    ex = adist.exchange_gradients(t)
    np.save(os.path.join(result_dir, f"tex_{rank}.npy"), ex["texture_shard"].numpy())
    np.save(os.path.join(result_dir, f"pts_{rank}.npy"), ex["points_shard"].numpy())
    if rank == 0:
        np.save(os.path.join(result_dir, "pose.npy"), ex["pose"].numpy())
        np.save(os.path.join(result_dir, "count_pose.npy"), ex["count_pose"].numpy())
        np.save(os.path.join(result_dir, "intr.npy"), ex["intrinsics"].numpy())
        np.save(os.path.join(result_dir, "count_intr.npy"), ex["count_intrinsics"].numpy())
        np.save(os.path.join(result_dir, "bg.npy"), ex["background"].numpy())
        np.save(os.path.join(result_dir, "env.npy"), ex["env_map"].numpy())
    dist.destroy_process_group()


def test_view_sharded_gradient_exchange_world_size_2(oracle, tmp_path):
    world = 2
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    cfg = synth.make_config("c2", n_points=20000, n_views=4, size=(96, 54))
    grads_up = synth.upstream_gradients(cfg["meta"])
    fwd = oracle.forward(cfg["arrays"], cfg["views"], cfg["params"], 4)
    ref = oracle.backward(cfg["arrays"], cfg["views"], cfg["params"], 4, fwd, grads_up, want_env=True, normalize=True)
    tex = np.concatenate([np.load(tmp_path / f"tex_{r}.npy") for r in range(world)])
    assert np.allclose(tex.reshape(ref["texture"].shape), ref["texture"], rtol=1e-5, atol=1e-6)
    pts = np.concatenate([np.load(tmp_path / f"pts_{r}.npy") for r in range(world)])
    assert adist.points_shard_is_aligned(20000, world)
    assert np.allclose(_normalize_points(pts), ref["points"], rtol=1e-5, atol=1e-6)
    pose, cp = np.load(tmp_path / "pose.npy"), np.load(tmp_path / "count_pose.npy")
    assert np.allclose(pose / np.maximum(cp, 1)[:, None], ref["pose"], rtol=1e-9, atol=1e-12)
    intr, ci = np.load(tmp_path / "intr.npy"), np.load(tmp_path / "count_intr.npy")
    assert np.allclose(intr / ci[:, None], ref["intrinsics"], rtol=1e-4, atol=1e-5)
    assert np.allclose(np.load(tmp_path / "bg.npy"), ref["background"], rtol=1e-4, atol=1e-4)
    assert np.allclose(np.load(tmp_path / "env.npy"), ref["env_map"], rtol=1e-4, atol=1e-5)


def _update_worker(rank, world, port, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    g = torch.Generator().manual_seed(3)
    C_, T, N = 4, 1001, 600
    texture = torch.randn((C_, T), generator=g)
    points = torch.randn((N, 4), generator=g)
    upd = adist.ShardedParameterUpdate(texture, points)
    for step in range(3):
        gr = torch.Generator().manual_seed(100 * step + rank)   # every rank has gradients of its own views
        grads = {"texture": torch.randn((C_, T), generator=gr), "points": torch.randn((N, 4), generator=gr)}
        grads["points"][:, 3] = torch.randint(0, 3, (N,), generator=gr).float()
        upd.step(adist.exchange_gradients(grads), lr_texture=0.05, lr_points=0.01)
    np.save(os.path.join(result_dir, f"texture_{rank}.npy"), texture.numpy())
    np.save(os.path.join(result_dir, f"points_{rank}.npy"), points.numpy())
    dist.destroy_process_group()


def test_sharded_optimiser_step_and_all_gather_world_size_2(tmp_path):
    """ShardedParameterUpdate under gloo: after three steps every rank's replicas equal what torch.optim.Adam (descriptors)
    and SGD on the normalised point gradients make of the full tensors with the gradients summed over the ranks."""
    world = 2
    port = 29500 + ((os.getpid() + 7) % 2000)
    mp.spawn(_update_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    g = torch.Generator().manual_seed(3)
    C_, T, N = 4, 1001, 600
    texture = torch.randn((C_, T), generator=g).requires_grad_(True)
    points = torch.randn((N, 4), generator=g)
    adam = torch.optim.Adam([texture], lr=0.05)
    for step in range(3):
        tg, pg = torch.zeros((C_, T)), torch.zeros((N, 4))
        for rank in range(world):
            gr = torch.Generator().manual_seed(100 * step + rank)
            tg += torch.randn((C_, T), generator=gr)
            p = torch.randn((N, 4), generator=gr)
            p[:, 3] = torch.randint(0, 3, (N,), generator=gr).float()
            pg += p
        texture.grad = tg
        adam.step()
        cnt = pg[:, 3:4]
        points[:, :3] -= 0.01 * torch.where(cnt > 0, pg[:, :3] / cnt.clamp(min=1e-30), pg[:, :3])
    for rank in range(world):
        assert np.allclose(np.load(tmp_path / f"texture_{rank}.npy"), texture.detach().numpy(), rtol=1e-5, atol=1e-6)
        assert np.allclose(np.load(tmp_path / f"points_{rank}.npy"), points.numpy(), rtol=1e-5, atol=1e-6)
    assert np.array_equal(np.load(tmp_path / "texture_0.npy"), np.load(tmp_path / "texture_1.npy"))


def test_shard_helpers():
    assert adist.shard_views(list(range(10)), 0, 4) == [0, 1, 2]
    assert adist.shard_views(list(range(10)), 3, 4) == [8, 9]
    assert sum(len(adist.shard_views(list(range(10)), r, 4)) for r in range(4)) == 10
    assert adist.shard_range(10, 3, 4) == (9, 10)
    assert adist.shard_range(8, 1, 4) == (2, 4)


def test_peer_layout_and_shard_ranges():
    """Host-side pieces of the peer-memory exchange: block layout and ownership ranges (no GPU needed)."""
    import ctypes as C
    from adop_b200 import capi
    lib = capi.load_library()
    lay = adist.peer_layout(4, 1000, 333, num_images=7, num_cameras=2, intrinsics_cols=13, env_hw=(8, 16))
    offs = [lay.off_texture, lay.off_points, lay.off_pose, lay.off_count_pose, lay.off_intrinsics,
            lay.off_count_intrinsics, lay.off_background, lay.off_env_map, lay.total_bytes]
    sizes = [1000 * 4 * 4, 333 * 16, 7 * 6 * 8, 7 * 4, 2 * 13 * 4, 2 * 4, 4 * 4, 4 * 8 * 16 * 4]
    assert all(o % 256 == 0 for o in offs)
    for a, b, size in zip(offs[:-1], offs[1:], sizes):
        assert b - a >= size and b - a < size + 256
    empty = adist.peer_layout(3, 10, 0, background=False)
    assert empty.off_points == empty.off_pose == empty.off_env_map and empty.total_bytes == 256
    for count in (0, 1, 7, 8, 1000, 10_000_019):
        for world in (1, 2, 3, 8):
            covered = 0
            for rank in range(world):
                lo, hi = C.c_int32(), C.c_int32()
                lib.adop_peer_shard_range(count, world, rank, C.byref(lo), C.byref(hi))
                assert (lo.value, hi.value) == adist.peer_shard_range(count, rank, world)
                assert lo.value == covered and hi.value >= lo.value
                covered = hi.value
            assert covered == count
    bad = capi.AdopPeerLayout()
    bad.channels = 0
    assert lib.adop_peer_layout_fill(C.byref(bad)) != capi.ADOP_OK


def test_touched_and_parameter_layouts():
    """Host-side layouts of the flags inside a gradient block and of a parameter block (no GPU needed)."""
    import ctypes as C
    from adop_b200 import capi
    lib = capi.load_library()
    plain = adist.peer_layout(4, 100_000, 70_001, num_images=3, num_cameras=1, intrinsics_cols=13, env_hw=(4, 8))
    flagged = adist.peer_layout(4, 100_000, 70_001, num_images=3, num_cameras=1, intrinsics_cols=13, env_hw=(4, 8), touched=True)
    # the gradient tensors sit where they sit without flags; the flags and the gather scratch follow them
    for name in ("off_texture", "off_points", "off_pose", "off_count_pose", "off_intrinsics", "off_count_intrinsics", "off_background", "off_env_map"):
        assert getattr(plain, name) == getattr(flagged, name)
    t_chunks, p_chunks = (100_000 + 255) // 256, (70_001 + 255) // 256
    assert plain.off_touched_texels == plain.off_touched_points == plain.off_gathered
    assert flagged.off_touched_texels >= flagged.off_env_map + 4 * 4 * 8 * 4
    assert flagged.off_touched_points - flagged.off_touched_texels >= t_chunks
    assert flagged.off_gathered - flagged.off_touched_points >= p_chunks
    assert flagged.total_bytes - flagged.off_gathered >= t_chunks + p_chunks and flagged.total_bytes > plain.total_bytes
    assert all(getattr(flagged, n) % 256 == 0 for n in ("off_touched_texels", "off_touched_points", "off_gathered", "total_bytes"))
    pl = adist.peer_param_layout(8, 1001, 77)
    assert pl.off_texture == 0 and pl.off_points >= 8 * 1001 * 4 and pl.off_points % 256 == 0
    assert pl.total_bytes >= pl.off_points + 77 * 16 and pl.total_bytes % 256 == 0
    bad = capi.AdopPeerParamLayout()
    bad.channels, bad.num_texels = 4, 0
    assert lib.adop_peer_param_layout_fill(C.byref(bad)) != capi.ADOP_OK
