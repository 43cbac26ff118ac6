"""One rank of the two-GPU exchange test (started by test_peer_exchange_gpu.py through torch.distributed.run).

Renders its share of the views of a small scene, exchanges the gradients over peer memory, and compares the result
with (a) a single-GPU run over all views on this rank's GPU and (b) the NCCL exchange of the same gradients."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from adop_b200 import dist as adist  # noqa: E402
from adop_b200 import synth  # noqa: E402
from adop_b200.raster import PointRasterizer, Scene  # noqa: E402


def close(a, b, what, rtol=1e-4, atol=1e-5):
    scale = float(b.abs().max()) if b.numel() else 1.0
    if not torch.allclose(a, b, rtol=rtol, atol=atol * max(scale, 1.0)):
        raise AssertionError(f"{what}: max abs diff {float((a - b).abs().max())} at scale {scale}")


def train_steps(ras, scene, cfg, views, mine, ex, dev, rank, world):
    """Four training steps of the whole scene through train.ViewShardedSceneOptimizer (descriptors and points sharded over
    the ranks, the small tensors stepped on every rank), fitting the pyramid to that of a scene with other descriptors,
    against the same steps in one process over all views with torch's optimisers on every tensor."""
    from adop_b200.train import SceneLearningRates, ViewShardedSceneOptimizer
    from adop_b200.raster import apply_tangent_to_pose
    params, L = cfg["params"], cfg["num_layers"]
    gen = torch.Generator(device=dev)
    gen.manual_seed(11)
    target_scene = Scene(**dict(scene.tensors(), texture=scene.texture + 0.3 * torch.randn(scene.texture.shape, device=dev, generator=gen)))
    targets = [c.clone() for c in ras.forward(target_scene, cfg["views"], params, L).colors]
    rates = SceneLearningRates(lr_texture=0.02, lr_background_color=0.004, lr_environment_map=0.02, lr_points=1e-4,
                               lr_poses=1e-5, lr_intrinsics=1e-4, lock_structure_params_epochs=0)
    C_, T = scene.texture.shape
    n_img = scene.poses.shape[0]

    def copies():
        t = {k: (v.clone() if v is not None else None) for k, v in scene.tensors().items()}
        return t, torch.zeros((n_img, 6), dtype=torch.float64, device=dev)

    # the sharded job
    t_a, tan_a = copies()
    pp = adist.PeerParameters(adist.peer_param_layout(C_, T, scene.position.shape[0]), dev)
    pp.texture.copy_(scene.texture)
    pp.points.copy_(scene.position)
    t_a["texture"], t_a["position"] = pp.texture, pp.points
    live = Scene(**t_a)
    opt = ViewShardedSceneOptimizer(pp, live.background, live.env_map, tan_a, live.poses, live.intrinsics, rates)
    # one process, all views, torch's optimisers
    t_b, tan_b = copies()
    ref = Scene(**t_b)
    xyz = ref.position[:, :3].clone().requires_grad_(True)
    for p in (ref.texture, ref.background, ref.env_map, tan_b, ref.intrinsics):
        p.requires_grad_(True)
    adam = torch.optim.Adam([{"params": [ref.texture], "lr": rates.lr_texture}, {"params": [ref.background], "lr": rates.lr_background_color},
                             {"params": [ref.env_map], "lr": rates.lr_environment_map}], lr=1.0)
    sgd = torch.optim.SGD([{"params": [xyz], "lr": rates.lr_points}, {"params": [tan_b], "lr": rates.lr_poses},
                           {"params": [ref.intrinsics], "lr": rates.lr_intrinsics}], lr=1e-10)
    losses = []
    for step in range(4):
        fwd = ras.forward(live, views, params, L, touched=ex.touched_flags())
        g = [(c - t[mine[0]:mine[-1] + 1]).contiguous() for c, t in zip(fwd.colors, targets)]
        loss = torch.stack([0.5 * (x * x).sum() for x in g]).sum()
        dist.all_reduce(loss)
        losses.append(float(loss))
        ex.release()
        ras.backward(live, params, fwd, g, want_env=True, normalize=False, out=ex.backward_outputs())
        opt.step(ex.reduce(), epoch_id=1)
        with torch.no_grad():
            ref.position[:, :3] = xyz
            f_all = ras.forward(ref, cfg["views"], params, L)
            g_all = [(c - t).contiguous() for c, t in zip(f_all.colors, targets)]
            b_all = ras.backward(ref, params, f_all, g_all, want_env=True, normalize=True)
        ref.texture.grad, ref.background.grad, ref.env_map.grad = b_all["texture"], b_all["background"], b_all["env_map"]
        xyz.grad, tan_b.grad, ref.intrinsics.grad = b_all["points"][:, :3].contiguous(), b_all["pose"], b_all["intrinsics"]
        adam.step()
        sgd.step()
        with torch.no_grad():
            apply_tangent_to_pose(tan_b.detach(), ref.poses)
        torch.cuda.synchronize()
        close(pp.texture, ref.texture.detach(), f"descriptors after training step {step}", rtol=1e-3, atol=1e-4)
        close(pp.points[:, :3], xyz.detach(), f"points after training step {step}", rtol=1e-5, atol=1e-6)
        close(live.background.detach(), ref.background.detach(), "background colour", rtol=1e-3, atol=1e-4)
        close(live.env_map.detach(), ref.env_map.detach(), "environment map", rtol=1e-3, atol=1e-4)
        close(live.poses, ref.poses, "poses", rtol=1e-9, atol=1e-9)
        close(live.intrinsics.detach(), ref.intrinsics.detach(), "intrinsics", rtol=1e-4, atol=1e-5)
    assert losses[-1] < 0.8 * losses[0], losses
    same = pp.texture.clone()
    dist.broadcast(same, src=0)
    assert torch.equal(same, pp.texture), "descriptor replicas differ between ranks after training"
    small = torch.cat([live.background.detach().double().flatten(), live.poses.flatten(), live.intrinsics.detach().double().flatten()])
    other = small.clone()
    dist.broadcast(other, src=0)
    assert torch.equal(other, small), "small-tensor replicas differ between ranks after training"
    pp.close()


def main():
    out_dir = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    n_views = 2 * world
    cfg = synth.make_config("c2", n_points=50000, n_views=n_views, size=(192, 108))
    L, params = cfg["num_layers"], cfg["params"]
    scene = Scene(**{k: (torch.from_numpy(v).to(dev) if v is not None else None) for k, v in cfg["arrays"].items()})
    ras = PointRasterizer(dev)
    gen = torch.Generator(device=dev)
    gen.manual_seed(7)  # the same upstream gradients on every rank
    fwd_all = ras.forward(scene, cfg["views"], params, L)
    grads_all = [torch.randn(c.shape, device=dev, generator=gen) for c in fwd_all.colors]
    ref = ras.backward(scene, params, fwd_all, grads_all, want_env=True, normalize=True)

    mine = adist.shard_views(list(range(n_views)), rank, world)
    views = [cfg["views"][i] for i in mine]
    grads = [g[mine[0]:mine[-1] + 1].contiguous() for g in grads_all]
    C_, T = scene.texture.shape
    lay = adist.peer_layout(C_, T, scene.position.shape[0], num_images=ref["pose"].shape[0],
                            num_cameras=ref["intrinsics"].shape[0], intrinsics_cols=ref["intrinsics"].shape[1],
                            env_hw=tuple(scene.env_map.shape[1:]), touched=True)
    ex = adist.PeerGradientExchange(lay, dev)
    for step in range(2):  # the second pass re-uses the blocks: covers the barrier after the kernel
        fwd = ras.forward(scene, views, params, L, touched=ex.touched_flags())
        ex.release()  # the barrier that the first pass deferred
        ras.backward(scene, params, fwd, grads, want_env=True, normalize=False, out=ex.backward_outputs())
        res = ex.reduce(defer_release=(step == 0))
        torch.cuda.synchronize()
        t_lo, t_hi = res["texel_range"]
        p_lo, p_hi = res["point_range"]
        close(res["texture_shard"], ref["texture"][:, t_lo:t_hi], f"texture shard (pass {step})")
        close(res["points_shard"], ref["points"][p_lo:p_hi], f"points shard (pass {step})")
        close(res["pose"], ref["pose"], "pose")
        close(res["intrinsics"], ref["intrinsics"], "intrinsics")
        close(res["count_pose"], ref["count_pose"], "pose counts", 0, 0)
        close(res["background"], ref["background"], "background")
        close(res["env_map"], ref["env_map"], "environment map")
    # every rank computed the same bits for the tensors that all ranks get
    check = res["pose"].clone()
    dist.broadcast(check, src=0)
    assert torch.equal(check, res["pose"]), "pose gradients differ between ranks"

    # the NCCL exchange of the same per-rank gradients
    fwd = ras.forward(scene, views, params, L)
    plain = ras.backward(scene, params, fwd, grads, want_env=True, normalize=False)
    nccl = adist.exchange_gradients(plain)
    tex_all = torch.empty_like(ref["texture"])
    tex_all[:, t_lo:t_hi] = res["texture_shard"]
    flat_lo, flat_hi = adist.shard_range(C_ * T, rank, world)
    # the NCCL path shards the flattened [C,T] tensor; compare on the overlap of the two ownership rules
    nccl_flat = torch.zeros(C_ * T, device=dev)
    nccl_flat[flat_lo:flat_hi] = nccl["texture_shard"]
    nccl_ct = nccl_flat.view(C_, T)
    own = torch.zeros(C_ * T, dtype=torch.bool, device=dev)
    own[flat_lo:flat_hi] = True
    both = own.view(C_, T)[:, t_lo:t_hi]
    close(res["texture_shard"][both], nccl_ct[:, t_lo:t_hi][both], "texture shard against the NCCL exchange")
    close(nccl["pose"] / nccl["count_pose"].clamp(min=1)[:, None].double(), ref["pose"], "NCCL pose")
    # optimiser step on the owned shard + all-gather of the updated parameters (one kernel), three training steps on
    # parameter replicas in peer-mapped blocks, against torch.optim on the full tensors with the single-GPU gradients
    play = adist.peer_param_layout(C_, T, scene.position.shape[0])
    pp = adist.PeerParameters(play, dev)
    pp.texture.copy_(scene.texture)
    pp.points.copy_(scene.position)
    live = Scene(**dict(scene.tensors(), texture=pp.texture, position=pp.points))
    ref_scene = Scene(**dict(scene.tensors(), texture=scene.texture.clone(), position=scene.position.clone()))
    ref_tex = ref_scene.texture.requires_grad_(True)
    ref_xyz = ref_scene.position[:, :3].clone().requires_grad_(True)
    adam, sgd = torch.optim.Adam([ref_tex], lr=0.02), torch.optim.SGD([ref_xyz], lr=1e-4)
    for step in range(3):
        fwd = ras.forward(live, views, params, L, touched=ex.touched_flags())
        ras.backward(live, params, fwd, grads, want_env=True, normalize=False, out=ex.backward_outputs())
        res = ex.reduce()
        pp.step(res, lr_texture=0.02, lr_points=1e-4)
        with torch.no_grad():
            ref_scene.position[:, :3] = ref_xyz
        f_all = ras.forward(ref_scene, cfg["views"], params, L)
        g_all = ras.backward(ref_scene, params, f_all, grads_all, want_env=True, normalize=True)
        ref_tex.grad, ref_xyz.grad = g_all["texture"].clone(), g_all["points"][:, :3].clone()
        adam.step()
        sgd.step()
        torch.cuda.synchronize()
        close(pp.texture, ref_tex.detach(), f"descriptors after step {step}", rtol=1e-4, atol=1e-5)
        close(pp.points[:, :3], ref_xyz.detach(), f"points after step {step}", rtol=1e-5, atol=1e-6)
    gathered = pp.texture.clone()
    dist.broadcast(gathered, src=0)
    assert torch.equal(gathered, pp.texture), "parameter replicas differ between ranks"
    pp.close()
    train_steps(ras, scene, cfg, views, mine, ex, dev, rank, world)
    ex.close()
    dist.barrier()
    with open(os.path.join(out_dir, f"ok_{rank}"), "w") as f:
        f.write("ok\n")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
