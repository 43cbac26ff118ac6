"""The libTorch autograd operator (adop_b200/libadop_torch.so, C++) against the CPU checker: the reference's call shape
`BlendPointCloud(info)` -> `PointRender::apply(texture, background, points, pose_tangents, intrinsics, info)`
(RenderInfo.cpp:19-58), driven through torch autograd."""
import numpy as np
import pytest
import torch

from adop_b200 import build, synth

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def op():
    torch.ops.load_library(build.TORCH_OP_LIB)
    return torch.ops.adop


def _info(cfg, dev):
    a = cfg["arrays"]
    info = torch.classes.adop.RenderInfo()
    t = lambda v: torch.from_numpy(v).to(dev) if v is not None else None
    info.set_scene(t(a["poses"]), t(a["normal"]), t(a["index"]), t(a["env_map"]))
    v = cfg["views"]
    views = torch.tensor([[x["w"], x["h"], x["image_index"], x["camera_index"], x.get("camera_model", 0)] for x in v])
    crops = torch.tensor([list(x.get("crop", (1.0, 1.0, 0.0, 0.0, 0.0))) for x in v], dtype=torch.float32)
    info.set_views(views, crops)
    info.set_num_layers(cfg["num_layers"])
    p = cfg["params"]
    for name, _ in type(p)._fields_:
        info.set_param(name, float(getattr(p, name)))
    return info


def _close(a, b, name, rtol=1e-4):
    a = a.detach().cpu().numpy()
    scale = max(float(np.abs(b).max()), 1e-12)
    assert float(np.abs(a.astype(np.float64) - b).max()) <= rtol * scale, name


@pytest.mark.parametrize("name,kw", [("c2", dict(n_points=300_000, n_views=2, size=(320, 180))),
                                      ("c3", dict(n_points=300_000, size=(320, 180)))])
def test_point_render_autograd_matches_checker(oracle, cuda_lib, op, name, kw):
    cfg = synth.make_config(name, **kw)
    a, L = cfg["arrays"], cfg["num_layers"]
    dev = torch.device("cuda:0")
    grads_up = synth.upstream_gradients(cfg["meta"], batch=len(cfg["views"]))
    ref = oracle.forward(a, cfg["views"], cfg["params"], L)
    ref_b = oracle.backward(a, cfg["views"], cfg["params"], L, ref, grads_up)
    texture = torch.from_numpy(a["texture"]).to(dev).requires_grad_(True)
    background = torch.from_numpy(a["background"]).to(dev).requires_grad_(True)
    points = torch.from_numpy(a["position"]).to(dev).requires_grad_(True)
    tangents = torch.zeros((a["poses"].shape[0], 6), dtype=torch.float64, device=dev, requires_grad=True)
    intrinsics = torch.from_numpy(a["intrinsics"]).to(dev).requires_grad_(True)
    info = _info(cfg, dev)
    out = op.blend_point_cloud(texture, background, points, tangents, intrinsics, info)
    n_masks = L if cfg["params"].output_background_mask else 0
    assert len(out) == L + n_masks
    for l in range(L):
        _close(out[l], ref["colors"][l], f"colour {l}")
        if n_masks:
            assert np.array_equal(out[L + l].cpu().numpy(), ref["masks"][l]) and not out[L + l].requires_grad
    loss = sum((o * torch.from_numpy(g).to(dev)).sum() for o, g in zip(out[:L], grads_up))
    loss.backward()
    _close(texture.grad, ref_b["texture"], "grad texture")
    _close(background.grad, ref_b["background"], "grad background")
    _close(points.grad, ref_b["points"], "grad points")
    _close(tangents.grad, ref_b["pose"], "grad pose")
    _close(intrinsics.grad, ref_b["intrinsics"], "grad intrinsics")


def test_only_requested_gradients_are_returned(cuda_lib, op):
    cfg = synth.make_config("c1", n_points=20_000, size=(64, 64))
    a = cfg["arrays"]
    dev = torch.device("cuda:0")
    texture = torch.from_numpy(a["texture"]).to(dev).requires_grad_(True)
    background = torch.from_numpy(a["background"]).to(dev)
    points = torch.from_numpy(a["position"]).to(dev)
    tangents = torch.zeros((1, 6), dtype=torch.float64, device=dev)
    intrinsics = torch.from_numpy(a["intrinsics"]).to(dev)
    out = op.blend_point_cloud(texture, background, points, tangents, intrinsics, _info(cfg, dev))
    sum(o.sum() for o in out).backward()
    assert texture.grad is not None and points.grad is None and tangents.grad is None


def test_apply_tangent_to_pose_op(oracle, cuda_lib, op):
    rng = np.random.default_rng(0)
    poses = np.stack([synth.look_at_pose(rng.normal(size=3) * 3 + 0.2, rng.normal(size=3)) for _ in range(10)])
    tang = rng.normal(size=(10, 6)) * 0.1
    t_ref, p_ref = tang.copy(), poses.copy()
    oracle.apply_tangent(t_ref, p_ref)
    t, p = torch.from_numpy(tang).cuda(), torch.from_numpy(poses).cuda()
    op.apply_tangent_to_pose(t, p)
    assert float(t.abs().max()) == 0 and np.abs(p.cpu().numpy() - p_ref).max() < 1e-12
    with pytest.raises(RuntimeError):
        op.apply_tangent_to_pose(t.float(), p)
